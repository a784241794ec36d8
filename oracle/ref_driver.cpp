// TEST INFRASTRUCTURE ONLY. C entry points over the unmodified reference CPU drivers
// (Grace1LFused / Grace2LFused / Grace3LFused::compute<CsrBonds>, libgrace/src/fused_{1l,2l,3l}.cpp) and the
// reference cell-list neighbour search (python/src/neighbors.cpp:15-95). Built by oracle/Makefile into
// oracle/_ref/libgrace_ref.so from the reference sources where they lie; nothing of the product links or loads it.
// The call sequence follows the reference's own Python module (python/src/core.cpp:292-396): neighbour search,
// positions and types permuted into the list order, compute on the CSR, results scattered back.
#include "grace/fused_1l.h"
#include "grace/fused_2l.h"
#include "grace/fused_3l.h"
#include "grace/model_kind.h"
#include "neighbors.h"

#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace {

struct RefModel {
  grace::ModelKind kind;
  std::shared_ptr<grace::GRACE1LModel> m1;
  std::shared_ptr<grace::GRACE2LModel> m2;
  std::shared_ptr<grace::GRACE3LModel> m3;
  std::unique_ptr<grace::Grace1LFused> d1;
  std::unique_ptr<grace::Grace2LFused> d2;
  std::unique_ptr<grace::Grace3LFused> d3;
  std::vector<std::string> names;
  int ntypes = 0;
};

thread_local std::string g_err;

double now_s()
{
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

}    // namespace

extern "C" {

const char *ref_last_error() { return g_err.c_str(); }

// spline_n: table intervals of the radial functions (reference default 1024)
void *ref_model_load(const char *path, int spline_n)
{
  try {
    auto r = std::make_unique<RefModel>();
    r->kind = grace::model_kind(path);
    grace::FusedSettings fs;
    if (spline_n > 0) fs.spline_n = spline_n;
    if (r->kind == grace::ModelKind::Grace1L) {
      r->m1 = std::make_shared<grace::GRACE1LModel>();
      r->m1->load(path);
      r->names = r->m1->element_names;
      r->d1 = std::make_unique<grace::Grace1LFused>(r->m1, fs, grace::Logger{});
    } else if (r->kind == grace::ModelKind::Grace2L) {
      r->m2 = std::make_shared<grace::GRACE2LModel>();
      r->m2->load(path);
      r->names = r->m2->element_names;
      r->d2 = std::make_unique<grace::Grace2LFused>(r->m2, fs, grace::Logger{});
    } else if (r->kind == grace::ModelKind::Grace3L) {
      r->m3 = std::make_shared<grace::GRACE3LModel>();
      r->m3->load(path);
      r->names = r->m3->element_names;
      r->d3 = std::make_unique<grace::Grace3LFused>(r->m3, fs, grace::Logger{});
    } else {
      g_err = "not a GRACE model";
      return nullptr;
    }
    return r.release();
  } catch (const std::exception &e) {
    g_err = e.what();
    return nullptr;
  }
}

void ref_model_free(void *h) { delete static_cast<RefModel *>(h); }

int ref_model_layers(void *h)
{
  auto *r = static_cast<RefModel *>(h);
  return r->d1 ? 1 : r->d2 ? 2 : 3;
}

// species: element names of the atom types 1..ns
int ref_set_species(void *h, int ns, const char *const *species)
{
  auto *r = static_cast<RefModel *>(h);
  try {
    std::vector<int> t2m(ns + 1, -1);
    for (int t = 0; t < ns; t++) {
      auto it = std::find(r->names.begin(), r->names.end(), std::string(species[t]));
      if (it == r->names.end()) {
        g_err = std::string("element not in the model: ") + species[t];
        return 1;
      }
      t2m[t + 1] = (int) (it - r->names.begin());
    }
    r->ntypes = ns;
    if (r->d1) r->d1->setup_types(ns, t2m);
    if (r->d2) r->d2->setup_types(ns, t2m);
    if (r->d3) r->d3->setup_types(ns, t2m);
    return 0;
  } catch (const std::exception &e) {
    g_err = e.what();
    return 1;
  }
}

double ref_cutoff(void *h)
{
  auto *r = static_cast<RefModel *>(h);
  double c = 0.0;
  for (int a = 1; a <= r->ntypes; a++)
    for (int b = 1; b <= r->ntypes; b++)
      c = std::max(c, r->d1 ? r->d1->cutoff(a, b) : r->d2 ? r->d2->cutoff(a, b) : r->d3->cutoff(a, b));
  return c;
}

// energy, forces [n][3], virial [6] (xx yy zz xy xz yz), eatom [n] (may be null) of one structure, caller's atom
// order. repeats >= 1 computes: seconds[0] = neighbour search, seconds[1] = best compute time, seconds[2] = median.
// gamma, sigma, cluster [n] (all three or none): the UQ outputs of the drivers (ComputeFlags::uq after enable_uq(),
// libgrace/src/fused_1l.cpp:584-638, libgrace/src/fused_2l.cpp:1101-1187)
static int compute_impl(void *h, int n, const int32_t *types, const double *pos, const double *cell, const uint8_t *pbc8,
                        int nthreads, int energy_only, int repeats, double *energy, double *forces, double *virial,
                        double *eatom, double *seconds, double *gamma, double *sigma, double *cluster)
{
  auto *r = static_cast<RefModel *>(h);
  try {
    const bool uq = gamma && sigma && cluster;
    if (uq) {
      if (r->d1 && !r->d1->uq_enabled()) r->d1->enable_uq();
      if (r->d2 && !r->d2->uq_enabled()) r->d2->enable_uq();
      if (r->d3) throw std::runtime_error("UQ of GRACE-3L is not driven here");
    }
    const bool pbc[3] = {pbc8[0] != 0, pbc8[1] != 0, pbc8[2] != 0};
    const double rc = ref_cutoff(h);
    double t0 = now_s();
    auto nl = grace_runtime::neighbor_search(pos, n, cell, pbc, rc, nthreads);
    const double t_nl = now_s() - t0;
    std::vector<double> x(3 * (size_t) n);
    std::vector<int> ty(n);
    for (int q = 0; q < n; q++) {
      const int64_t a = nl.perm[q];
      for (int d = 0; d < 3; d++) x[3 * (size_t) q + d] = pos[3 * a + d];
      ty[q] = types[a];
    }
    grace::CsrBonds src{ty.data(), nl.offset.data(), nl.j.data(), nullptr, x.data(), nl.image.data(), nl.shifts.data()};
    std::vector<double> f(3 * (size_t) n), ea(n), times, ug(uq ? n : 0), us(uq ? n : 0), uc(uq ? n : 0);
    double e = 0.0, v[6];
    for (int rep = 0; rep < std::max(1, repeats); rep++) {
      std::fill(f.begin(), f.end(), 0.0);
      std::fill(ea.begin(), ea.end(), 0.0);
      grace::Outputs out;
      out.f = f.data();
      out.eatom = ea.data();
      grace::ComputeFlags fl;
      fl.eflag_atom = eatom != nullptr;
      fl.virial = !energy_only;
      fl.energy_only = energy_only != 0;
      if (uq) {
        fl.uq = true;
        out.gamma = ug.data();
        out.atomic_sigma = us.data();
        out.gmm_cluster = uc.data();
      }
      grace::NoExchange ex;
      t0 = now_s();
      if (r->d1) r->d1->compute(n, nullptr, n, n, src, out, fl, nthreads);
      else if (r->d2) r->d2->compute(n, nullptr, n, n, src, ex, out, fl, nthreads);
      else r->d3->compute(n, nullptr, n, n, src, ex, out, fl, nthreads);
      times.push_back(now_s() - t0);
      e = out.energy;
      std::copy(out.virial, out.virial + 6, v);
    }
    *energy = e;
    if (virial) std::copy(v, v + 6, virial);
    for (int q = 0; q < n; q++) {
      const int64_t a = nl.perm[q];
      if (forces)
        for (int d = 0; d < 3; d++) forces[3 * a + d] = f[3 * (size_t) q + d];
      if (eatom) eatom[a] = ea[q];
      if (uq) {
        gamma[a] = ug[q];
        sigma[a] = us[q];
        cluster[a] = uc[q];
      }
    }
    if (seconds) {
      std::sort(times.begin(), times.end());
      seconds[0] = t_nl;
      seconds[1] = times.front();
      seconds[2] = times[times.size() / 2];
    }
    return 0;
  } catch (const std::exception &e) {
    g_err = e.what();
    return 1;
  }
}

int ref_compute(void *h, int n, const int32_t *types, const double *pos, const double *cell, const uint8_t *pbc8,
                int nthreads, int energy_only, int repeats, double *energy, double *forces, double *virial,
                double *eatom, double *seconds)
{
  return compute_impl(h, n, types, pos, cell, pbc8, nthreads, energy_only, repeats, energy, forces, virial, eatom,
                      seconds, nullptr, nullptr, nullptr);
}

int ref_compute_uq(void *h, int n, const int32_t *types, const double *pos, const double *cell, const uint8_t *pbc8,
                   int nthreads, int energy_only, double *energy, double *forces, double *virial, double *eatom,
                   double *gamma, double *sigma, double *cluster)
{
  return compute_impl(h, n, types, pos, cell, pbc8, nthreads, energy_only, 1, energy, forces, virial, eatom, nullptr,
                      gamma, sigma, cluster);
}

// the reference neighbour list of one structure as bond triples in the caller's frame, for the device-list parity
// test: returns the bond count; bi, bj (caller's atom indices) and bs [nb][3] (integer lattice translation S of
// r_ij = x_j - x_i + S cell, recovered from the shift vector) are filled up to cap bonds
int64_t ref_neighbors(int n, const double *pos, const double *cell, const uint8_t *pbc8, double cutoff, int nthreads,
                      int64_t cap, int32_t *bi, int32_t *bj, int32_t *bs)
{
  try {
    const bool pbc[3] = {pbc8[0] != 0, pbc8[1] != 0, pbc8[2] != 0};
    auto nl = grace_runtime::neighbor_search(pos, n, cell, pbc, cutoff, nthreads);
    const double *a = cell;
    const double det = a[0] * (a[4] * a[8] - a[5] * a[7]) - a[1] * (a[3] * a[8] - a[5] * a[6]) +
                       a[2] * (a[3] * a[7] - a[4] * a[6]);
    const double d = 1.0 / det;
    const double inv[9] = {(a[4] * a[8] - a[5] * a[7]) * d, (a[2] * a[7] - a[1] * a[8]) * d,
                           (a[1] * a[5] - a[2] * a[4]) * d, (a[5] * a[6] - a[3] * a[8]) * d,
                           (a[0] * a[8] - a[2] * a[6]) * d, (a[2] * a[3] - a[0] * a[5]) * d,
                           (a[3] * a[7] - a[4] * a[6]) * d, (a[1] * a[6] - a[0] * a[7]) * d,
                           (a[0] * a[4] - a[1] * a[3]) * d};
    const int64_t nb = nl.offset[n];
    for (int q = 0; q < n; q++)
      for (int64_t b = nl.offset[q]; b < nl.offset[q + 1] && b < cap; b++) {
        bi[b] = (int32_t) nl.perm[q];
        bj[b] = (int32_t) nl.perm[nl.j[b]];
        const double *s = &nl.shifts[3 * (size_t) nl.image[b]];
        for (int k = 0; k < 3; k++)
          bs[3 * b + k] = (int32_t) std::lround(s[0] * inv[k] + s[1] * inv[3 + k] + s[2] * inv[6 + k]);
      }
    return nb;
  } catch (const std::exception &e) {
    g_err = e.what();
    return -1;
  }
}

}    // extern "C"
