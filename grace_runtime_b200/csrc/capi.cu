// extern "C" entry points declared in include/grace_b200.h: exceptions of the C++ layer become status codes and a
// thread-local message, as the reference's Python binding turns them into ValueError / RuntimeError
// (python/kk/kk_module.cpp:202-208).
#include "../../include/grace_b200.h"

#include "engine.h"
#include "peaks.h"

#include <cstring>
#include <mutex>
#include <set>

using namespace gb;

struct grace_model {
  std::shared_ptr<ModelObj> m;
};
struct grace_system {
  std::unique_ptr<SystemObj> s;
};
struct grace_batch {
  std::unique_ptr<BatchObj> b;
};
struct grace_engine {
  std::unique_ptr<EngineRunObj> e;
};

namespace {

thread_local std::string g_error;
std::recursive_mutex g_device_mu;    // all device work of the process is serialised (kk_core.cpp:58-63)
std::set<grace_system *> g_systems;
std::set<grace_batch *> g_batches;
std::set<grace_engine *> g_engines;

template<class F> int guarded(F &&f)
{
  try {
    std::lock_guard<std::recursive_mutex> lk(g_device_mu);
    // the current device is a per-thread setting of the CUDA runtime: a host thread other than the one that called
    // grace_initialize would otherwise allocate and launch on device 0
    if (dev().initialized) GB_CUDA(cudaSetDevice(dev().device));
    f();
    return GRACE_OK;
  } catch (const InvalidArgument &e) {
    g_error = e.what();
    return GRACE_INVALID_ARGUMENT;
  } catch (const std::invalid_argument &e) {
    g_error = e.what();
    return GRACE_INVALID_ARGUMENT;
  } catch (const ModelError &e) {    // a file that is no usable model: the reference raises ValueError
    g_error = e.what();
    return GRACE_INVALID_ARGUMENT;
  } catch (const Unsupported &e) {
    g_error = e.what();
    return GRACE_UNSUPPORTED;
  } catch (const OutOfMemory &e) {
    g_error = e.what();
    return GRACE_OUT_OF_MEMORY;
  } catch (const std::bad_alloc &) {
    g_error = "out of host memory";
    return GRACE_OUT_OF_MEMORY;
  } catch (const std::exception &e) {
    g_error = e.what();
    return GRACE_RUNTIME_ERROR;
  } catch (...) {
    g_error = "unknown error";
    return GRACE_RUNTIME_ERROR;
  }
}

std::vector<std::string> names(const char *const *species, int n)
{
  if (n < 0 || (n > 0 && !species)) throw InvalidArgument("species must be given");
  std::vector<std::string> v;
  for (int i = 0; i < n; i++) {
    if (!species[i]) throw InvalidArgument("species must be given");
    v.emplace_back(species[i]);
  }
  return v;
}

}    // namespace

extern "C" {

int grace_initialize(int device)
{
  return guarded([&] {
    DeviceState &d = dev();
    if (d.initialized) {
      if (d.device != device) throw DeviceError("the backend is already initialised on another device (one GPU per process)");
      return;
    }
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
      (void) cudaGetLastError();
      throw DeviceError("no CUDA device available: this backend has no CPU path");
    }
    if (device < 0 || device >= count) throw InvalidArgument("no such CUDA device");
    GB_CUDA(cudaSetDevice(device));
    cudaDeviceProp p{};
    GB_CUDA(cudaGetDeviceProperties(&p, device));
    if (p.major < 10) throw DeviceError(std::string("this backend is built for sm_100a only; device is ") + p.name);
    d.sm_count = p.multiProcessorCount;
    GB_CUDA(cudaStreamCreateWithFlags(&d.stream, cudaStreamNonBlocking));
    d.device = device;
    d.initialized = true;
  });
}

int grace_finalize(void)
{
  return guarded([&] {
    DeviceState &d = dev();
    if (!d.initialized) return;
    for (auto *s : g_systems)
      if (s->s) s->s->release();
    for (auto *b : g_batches)
      if (b->b) b->b->release();
    for (auto *e : g_engines)
      if (e->e) e->e->release();
    comm_finalize();
    cudaStreamSynchronize(d.stream);
    cudaStreamDestroy(d.stream);
    d.stream = nullptr;
    d.initialized = false;
  });
}

int grace_initialized(void) { return dev().initialized ? 1 : 0; }
int grace_device(void) { return dev().device; }
const char *grace_arch(void) { return "sm100"; }
const char *grace_platform(void) { return "cuda"; }
const char *grace_blas(void) { return ""; }
int grace_abi(void) { return GRACE_B200_ABI; }
const char *grace_last_error(void) { return g_error.c_str(); }
uint64_t grace_kernel_launches(void) { return dev().launches; }

int grace_profile_enable(int on)
{
  return guarded([&] {
    require_initialized();
    profile_enable(on != 0);
  });
}

int grace_profile_report(char *buf, size_t len)
{
  return guarded([&] {
    if (!buf || len == 0) throw InvalidArgument("buf must be given");
    const std::string r = profile_report();
    const size_t n = std::min(len - 1, r.size());
    std::memcpy(buf, r.data(), n);
    buf[n] = 0;
  });
}

int grace_memory_info(size_t *free_bytes, size_t *total_bytes)
{
  return guarded([&] {
    require_initialized();
    size_t f = 0, t = 0;
    GB_CUDA(cudaMemGetInfo(&f, &t));
    if (free_bytes) *free_bytes = f;
    if (total_bytes) *total_bytes = t;
  });
}

int grace_debug_fail_alloc(const char *label, int nth)
{
  return guarded([&] {
    dev().fail_label = label ? label : "";
    dev().fail_alloc_nth = nth > 0 ? nth : 0;
  });
}

int grace_debug_fail_launch(int nth)
{
  return guarded([&] { dev().fail_launch_nth = nth > 0 ? nth : 0; });
}

int grace_measure_peak(int kind, double *tflops)
{
  return guarded([&] {
    if (!tflops) throw InvalidArgument("tflops must be given");
    if (kind == 0) *tflops = measure_peak_fp32_tflops();
    else if (kind == 1) *tflops = measure_peak_tf32_tflops();
    else if (kind == 2) *tflops = measure_peak_fp32_tflops(true);
    else if (kind >= 16) *tflops = measure_peak_tf32_tflops(kind);    // the same with N = kind instead of 256
    else throw InvalidArgument("kind must be 0 (fp32 FMA), 1 (tf32 tensor cores, N = 256), 2 (fp32 packed FMA) or N (a multiple of 16 up to 256)");
  });
}

int grace_debug_track_alloc(int on)
{
  return guarded([&] { track_alloc(on != 0); });
}

uint64_t grace_debug_peak_alloc(void)
{
  std::lock_guard<std::recursive_mutex> lk(g_device_mu);
  return (uint64_t) tracked_peak_bytes();
}

int grace_debug_live_alloc(char *buf, size_t len)
{
  return guarded([&] {
    if (!buf || len == 0) throw InvalidArgument("buf must be given");
    std::string r;
    for (const auto &kv : tracked_live()) r += kv.first + "\t" + std::to_string(kv.second) + "\n";
    const size_t n = std::min(len - 1, r.size());
    std::memcpy(buf, r.data(), n);
    buf[n] = 0;
  });
}

int grace_model_load(const char *path, int spline, grace_model **out)
{
  return guarded([&] {
    if (!path || !out) throw InvalidArgument("path and out must be given");
    if (spline != 0 && spline < 16) throw InvalidArgument("spline N must be >= 16 (or 0: exact radial MLP)");
    auto m = std::make_shared<ModelObj>();
    m->model = GraceModel::load(path);
    m->path = path;
    m->spline = spline;
    *out = new grace_model{m};
  });
}

int grace_model_layers(const grace_model *m) { return m ? m->m->model.layers : 0; }
int grace_model_has_uq(const grace_model *m) { return m && m->m->model.has_uq ? 1 : 0; }
int grace_model_validate_uq(const grace_model *m)
{
  return guarded([&] {
    if (!m) throw InvalidArgument("model must be given");
    try {
      m->m->model.validate_uq();
    } catch (const ModelError &e) {
      throw InvalidArgument(e.what());
    }
  });
}
int grace_model_n_elements(const grace_model *m) { return m ? (int) m->m->model.element_names.size() : 0; }
const char *grace_model_element_name(const grace_model *m, int i)
{
  if (!m || i < 0 || i >= (int) m->m->model.element_names.size()) return "";
  return m->m->model.element_names[i].c_str();
}
int64_t grace_model_engine_setups(const grace_model *m) { return m ? m->m->setups : 0; }
double grace_model_dense_flops(const grace_model *m)
{
  if (!m) return 0.0;
  std::lock_guard<std::mutex> lk(m->m->mu);
  return m->m->engines.empty() ? 0.0 : m->m->engines.begin()->second->plan().dense_flops_per_atom;
}
int grace_model_dense_stats(const grace_model *m, double *out6)
{
  return guarded([&] {
    if (!m || !out6) throw InvalidArgument("model and output must be given");
    std::lock_guard<std::mutex> lk(m->m->mu);
    if (m->m->engines.empty()) throw InvalidArgument("the model has no engine yet: create a System or Batch first");
    m->m->engines.begin()->second->dense_stats(out6);
  });
}

int grace_model_radial_mlp_device(grace_model *m, int layer, int64_t nb, const float *d_x, float *d_R, float *d_dR)
{
  return guarded([&] {
    if (!m) throw InvalidArgument("model must be given");
    m->m->radial_exact(layer, d_x, (long long) nb, d_R, d_dR);
  });
}
int grace_model_radial_mlp_width(const grace_model *m, int layer)
{
  if (!m || layer < 1 || layer > m->m->model.layers) return 0;
  const auto &L = layer == 1 ? m->m->model.rad1 : m->m->model.rad2;
  return L.empty() ? 0 : L.back().n_out;
}
void grace_model_free(grace_model *m)
{
  std::lock_guard<std::recursive_mutex> lk(g_device_mu);
  delete m;
}

int grace_system_create(const grace_model *m, const char *const *species, int n_species, double skin, int spline,
                        int chunksize, grace_system **out)
{
  return guarded([&] {
    if (!m || !out) throw InvalidArgument("model and out must be given");
    auto s = std::make_unique<SystemObj>(m->m, names(species, n_species), skin, spline, chunksize);
    *out = new grace_system{std::move(s)};
    g_systems.insert(*out);
  });
}

double grace_system_cutoff(const grace_system *s) { return s ? s->s->cutoff() : 0.0; }

int grace_system_compute(grace_system *s, int n, const int32_t *types, const double *pos, const double *cell,
                         const uint8_t *pbc, int flags, double *energy, double *virial6, double *forces,
                         double *energies)
{
  return guarded([&] {
    if (!s) throw InvalidArgument("system must be given");
    s->s->compute(n, types, pos, false, cell, pbc, flags, energy, virial6, forces, energies, false);
  });
}

int grace_system_compute_device(grace_system *s, int n, const int32_t *d_types, const double *d_pos,
                                const double *cell, const uint8_t *pbc, int flags, double *d_energy,
                                double *d_virial6, double *d_forces, double *d_energies)
{
  return guarded([&] {
    if (!s) throw InvalidArgument("system must be given");
    if (!d_energy) throw InvalidArgument("the energy output must be given");
    s->s->compute(n, d_types, d_pos, true, cell, pbc, flags, d_energy, d_virial6, d_forces, d_energies, true);
  });
}

int grace_system_set_uq_outputs(grace_system *s, double *gamma, double *sigma, double *cluster)
{
  return guarded([&] {
    if (!s) throw InvalidArgument("system must be given");
    s->s->uq_out = UqOutputs{gamma, sigma, cluster};
  });
}

int grace_sum_rows_static(const double *d_values, int64_t n, int k, double *d_out)
{
  return guarded([&] { static_sum(d_values, (long long) n, k, d_out); });
}

int grace_comm_unique_id(void *id128)
{
  return guarded([&] { comm_unique_id(id128); });
}

int grace_comm_init(const void *id128, int rank, int world)
{
  return guarded([&] { comm_init(id128, rank, world); });
}

int grace_comm_finalize(void)
{
  return guarded([&] { comm_finalize(); });
}

int grace_comm_rank(void) { return comm_rank(); }
int grace_comm_size(void) { return comm_size(); }

int grace_system_set_exchange(grace_system *s, int n, int nlocal, int ninner, const int32_t *send_counts,
                              const int32_t *send_index, const int32_t *recv_counts, const int32_t *recv_index)
{
  return guarded([&] {
    if (!s) throw InvalidArgument("system must be given");
    std::lock_guard<std::mutex> lk(s->s->mu);
    s->s->set_exchange(n, nlocal, ninner, send_counts, send_index, recv_counts, recv_index);
  });
}

int grace_system_set_owned(grace_system *s, int nlocal, int ninner)
{
  return guarded([&] {
    if (!s) throw InvalidArgument("system must be given");
    std::lock_guard<std::mutex> lk(s->s->mu);
    s->s->set_owned(nlocal, ninner);
  });
}

int grace_system_neighbor_list(grace_system *s, int64_t capacity, int32_t *bi, int32_t *bj, int32_t *bS, int64_t *count)
{
  return guarded([&] {
    if (!s || !count) throw InvalidArgument("system and count must be given");
    if (!s->s->has_list()) throw InvalidArgument("the system has no neighbour list yet: call compute first");
    std::vector<int> i, j, S;
    s->s->neighbor_list().export_host(i, j, S);
    *count = (int64_t) i.size();
    if (capacity < (int64_t) i.size()) return;    // the caller asks again with room for `count` bonds
    if (!i.empty() && (!bi || !bj || !bS)) throw InvalidArgument("output arrays must be given");
    std::memcpy(bi, i.data(), sizeof(int) * i.size());
    std::memcpy(bj, j.data(), sizeof(int) * j.size());
    std::memcpy(bS, S.data(), sizeof(int) * S.size());
  });
}

int64_t grace_system_rebuilds(const grace_system *s) { return s ? s->s->rebuilds : 0; }
int grace_system_chunksize(const grace_system *s) { return s ? s->s->last_chunk : 0; }
int grace_system_release_buffers(grace_system *s)
{
  return guarded([&] {
    if (!s) throw InvalidArgument("system must be given");
    s->s->release();
  });
}
int grace_system_stage_ms(const grace_system *s, double *ms5)
{
  if (!s || !ms5) return GRACE_INVALID_ARGUMENT;
  for (int k = 0; k < 5; k++) ms5[k] = s->s->stage_ms[k];
  return GRACE_OK;
}
void grace_system_free(grace_system *s)
{
  std::lock_guard<std::recursive_mutex> lk(g_device_mu);
  if (!s) return;
  g_systems.erase(s);
  delete s;
}

int grace_engine_create(const grace_model *m, const char *const *species, int n_species, int spline, int chunksize,
                        grace_engine **out)
{
  return guarded([&] {
    if (!m || !out) throw InvalidArgument("model and out must be given");
    auto e = std::make_unique<EngineRunObj>(m->m, names(species, n_species), spline, chunksize);
    *out = new grace_engine{std::move(e)};
    g_engines.insert(*out);
  });
}

double grace_engine_cutoff(const grace_engine *e) { return e ? e->e->cutoff() : 0.0; }
int grace_engine_comm_width(const grace_engine *e) { return e ? e->e->comm_width() : 0; }

int grace_engine_run(grace_engine *e, const grace_run_input *in, double *energy, double *virial6, double *d_f, double *d_eatom)
{
  return guarded([&] {
    if (!e || !in) throw InvalidArgument("engine and input must be given");
    ExchangeHooks h;
    h.forward = in->forward;
    h.reverse = in->reverse;
    h.user = in->user;
    e->e->run(in->nlocal, in->nall, in->d_type, in->d_x, in->d_numneigh, in->d_neighbors, in->maxneigh, in->flags, h, energy,
              virial6, d_f, d_eatom);
  });
}

void grace_engine_free(grace_engine *e)
{
  std::lock_guard<std::recursive_mutex> lk(g_device_mu);
  if (!e) return;
  g_engines.erase(e);
  delete e;
}

int grace_batch_create(const grace_model *m, const char *const *species, int n_species, int spline, int chunksize,
                       grace_batch **out)
{
  return guarded([&] {
    if (!m || !out) throw InvalidArgument("model and out must be given");
    auto b = std::make_unique<BatchObj>(m->m, names(species, n_species), spline, chunksize);
    *out = new grace_batch{std::move(b)};
    g_batches.insert(*out);
  });
}

double grace_batch_cutoff(const grace_batch *b) { return b ? b->b->cutoff() : 0.0; }

int grace_batch_compute(grace_batch *b, int nsys, const int32_t *natoms, int64_t ntot, const int32_t *types,
                        const double *pos, const double *cell, const uint8_t *pbc, int flags, int64_t max_nall,
                        double *energy, double *virial, double *forces, double *energies)
{
  return guarded([&] {
    if (!b) throw InvalidArgument("batch must be given");
    b->b->compute(nsys, natoms, ntot, types, pos, false, cell, pbc, flags, max_nall, energy, virial, forces, energies);
  });
}

int grace_batch_compute_device(grace_batch *b, int nsys, const int32_t *natoms, int64_t ntot, const int32_t *d_types,
                               const double *d_pos, const double *cell, const uint8_t *pbc, int flags,
                               int64_t max_nall, double *d_energy, double *d_virial, double *d_forces,
                               double *d_energies)
{
  return guarded([&] {
    if (!b) throw InvalidArgument("batch must be given");
    if (!d_energy) throw InvalidArgument("the energy output must be given");
    b->b->compute(nsys, natoms, ntot, d_types, d_pos, true, cell, pbc, flags, max_nall, d_energy, d_virial, d_forces,
                  d_energies);
  });
}

int grace_batch_set_uq_outputs(grace_batch *b, double *gamma, double *sigma, double *cluster)
{
  return guarded([&] {
    if (!b) throw InvalidArgument("batch must be given");
    b->b->uq_out = UqOutputs{gamma, sigma, cluster};
  });
}

int grace_batch_passes(const grace_batch *b) { return b ? b->b->passes : 0; }
double grace_batch_host_seconds(const grace_batch *b) { return b ? b->b->host_seconds : 0.0; }
int grace_batch_set_keep_buffers(grace_batch *b, int on)
{
  if (!b) return GRACE_INVALID_ARGUMENT;
  b->b->keep_buffers = on != 0;
  return GRACE_OK;
}
int grace_batch_release_buffers(grace_batch *b)
{
  return guarded([&] {
    if (!b) throw InvalidArgument("batch must be given");
    b->b->release();
  });
}
void grace_batch_free(grace_batch *b)
{
  std::lock_guard<std::recursive_mutex> lk(g_device_mu);
  if (!b) return;
  g_batches.erase(b);
  delete b;
}

}    // extern "C"
