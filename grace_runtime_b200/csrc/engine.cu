#include "engine.h"

#include <climits>
#include <cstdio>

#include "bond_common.cuh"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>

namespace gb {

// ---- tables ----------------------------------------------------------------------------------------------------
const SHTable &sh_table_host()
{
  static SHTable t = [] {
    SHTable s{};
    for (int l = 2; l <= 4; l++) {
      for (int mm = 0; mm < l - 1; mm++) {
        const double l2 = l * l, m2 = mm * mm, lm1 = l - 1;
        s.a[l * (l + 1) / 2 + mm] = (float) std::sqrt((4.0 * l2 - 1.0) / (l2 - m2));
        s.b[l * (l + 1) / 2 + mm] = (float) -std::sqrt((lm1 * lm1 - m2) / (4.0 * lm1 * lm1 - 1.0));
      }
      s.c[l] = (float) -std::sqrt(1.0 + 0.5 / l);
      s.d[l] = (float) std::sqrt(2.0 * l + 1.0);
    }
    return s;
  }();
  return t;
}

std::vector<int> species_to_elements(const GraceModel &m, const std::vector<std::string> &species)
{
  if (species.empty()) throw InvalidArgument("species must name at least one element");
  std::vector<int> t2m;
  for (const auto &s : species) {
    const int mu = m.element_index(s);
    if (mu < 0) throw InvalidArgument("element " + s + " is not in the model");
    t2m.push_back(mu);
  }
  return t2m;
}

// ---- engine ----------------------------------------------------------------------------------------------------
namespace {

__global__ void __launch_bounds__(256) types_to_mu(const int *__restrict__ types, const int *__restrict__ t2m, int ns,
                                                   int *mu, int *flag, long long n)
{
  const long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int t = types[i];
  if (t < 1 || t > ns) {
    atomicOr(flag, 1);
    mu[i] = 0;
  } else {
    mu[i] = t2m[t - 1];
  }
}

__global__ void __launch_bounds__(256) types_differ(const int *__restrict__ a, const int *__restrict__ b, int *flag,
                                                    long long n)
{
  const long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && a[i] != b[i]) atomicOr(flag, 2);
}

unsigned nblocks(long long n, int per) { return (unsigned) ((n + per - 1) / per); }

}    // namespace

void Engine::setup_layer(LayerEngine &E, const LayerPlan &P)
{
  E.plan = &P;
  E.tab.set_label("engine:radial_table");
  E.z.set_label("engine:chemical_weights");
  E.tab.upload(P.radial.tab);
  E.z.upload(P.z);
  // all index tables of the layer in one buffer each (the fused kernel copies them to shared memory as a whole)
  std::vector<int> itab;
  std::vector<MVItem> items;
  std::vector<ProdTerm> terms;
  std::vector<size_t> mv_row, mv_off, mv_item, mv_ud, mv_so, mv_ue, pr_row, pr_off, pr_term, pr_first;
  auto put = [&](const std::vector<int> &v) {
    const size_t at = itab.size();
    itab.insert(itab.end(), v.begin(), v.end());
    return at;
  };
  for (const MVOp &o : P.mv) {
    mv_row.push_back(put(o.row_out));
    mv_off.push_back(put(o.item_off));
    mv_item.push_back(items.size());
    items.insert(items.end(), o.items.begin(), o.items.end());
    mv_ud.push_back(put(o.unit_desc));
    mv_so.push_back(put(o.slot_off));
    mv_ue.push_back(items.size());
    items.insert(items.end(), o.unit_ent.begin(), o.unit_ent.end());
  }
  for (const ProdOp &o : P.prod) {
    pr_row.push_back(put(o.row_out));
    pr_off.push_back(put(o.term_off));
    pr_first.push_back(put(o.row_first));
    pr_term.push_back(terms.size());
    terms.insert(terms.end(), o.terms.begin(), o.terms.end());
  }
  E.itab.set_label("engine:tables"); E.items.set_label("engine:tables"); E.terms.set_label("engine:tables");
  E.itab.upload(itab);
  E.items.upload(items);
  E.terms.upload(terms);
  E.n_itab = (int) itab.size(); E.n_items = (int) items.size(); E.n_terms = (int) terms.size();
  for (size_t q = 0; q < P.mv.size(); q++) {
    const MVOp &o = P.mv[q];
    MVDev d{};
    d.row_out = E.itab.get() + mv_row[q];
    d.item_off = E.itab.get() + mv_off[q];
    d.items = E.items.get() + mv_item[q];
    d.unit_desc = E.itab.get() + mv_ud[q];
    d.slot_off = E.itab.get() + mv_so[q];
    d.unit_ent = E.items.get() + mv_ue[q];
    d.nslots = o.slot_off.empty() ? 0 : (int) o.slot_off.size() - 1;
    d.unit_nmax = 0;
    d.n_uniform = o.items.empty() ? 0 : o.items[0].n_in;
    for (const MVItem &it : o.items)
      if (it.n_in != d.n_uniform) d.n_uniform = 0;
    bool same = true;
    for (const MVItem &it : o.items) {
      d.unit_nmax = std::max(d.unit_nmax, it.n_in);
      same = same && it.n_in == o.n_out && P.tensors[it.src].channels == o.n_out;
    }
    same = same && P.tensors[o.dst].channels == o.n_out && (o.n_out == 32 || o.n_out == 64);
    d.unit_exact = same ? o.n_out : 0;
    E.fbufs.emplace_back("engine:weights");
    E.fbufs.back().upload(o.W);
    d.W = E.fbufs.back().get();
    d.ty_stride = o.ty_stride;
    d.n_out = o.n_out;
    d.ldw = o.ldw;
    d.nrows = (int) o.row_out.size();
    d.accumulate = o.accumulate;
    d.elem = o.elem;
    d.dst = o.dst;
    d.dst_C = P.tensors[o.dst].channels;
    d.max_row_items = 0;
    for (size_t r = 0; r + 1 < o.item_off.size(); r++) d.max_row_items = std::max(d.max_row_items, o.item_off[r + 1] - o.item_off[r]);
    E.mv.push_back(d);
  }
  for (size_t q = 0; q < P.prod.size(); q++) {
    const ProdOp &o = P.prod[q];
    ProdDev d{};
    d.row_out = E.itab.get() + pr_row[q];
    d.term_off = E.itab.get() + pr_off[q];
    d.terms = E.terms.get() + pr_term[q];
    d.row_first = o.row_first.empty() ? nullptr : E.itab.get() + pr_first[q];
    d.nrows = (int) o.row_out.size();
    d.accumulate = o.accumulate;
    d.dst = o.dst;
    d.srcA = o.srcA;
    d.srcB = o.srcB;
    E.prod.push_back(d);
  }
  // tensor-core form of the operations with shared weights
  {
    double covered = 0.0, all = 0.0;
    E.mv_tc.clear();
    E.mv_tc.resize(P.mv.size());
    for (size_t q = 0; q < P.mv.size(); q++) {
      const double fl = (int) q == P.uq_mv ? 0.0 : P.mv[q].flops_per_atom();    // the UQ projection is not part of a step
      all += fl;
      if (MVTensorCore::eligible(P.mv[q], P.tensors)) {
        E.mv_tc[q].setup(P.mv[q]);
        covered += fl;
      }
    }
    E.tc_flop_share = all > 0.0 ? covered / all : 0.0;
  }
  // tensors: values first, then the gradients that are zeroed per chunk (one contiguous range)
  E.toff.assign(P.tensors.size(), 0);
  long long at = 0;
  for (int pass = 0; pass < 2; pass++) {
    if (pass == 1) E.grad_begin = at;
    for (size_t t = 0; t < P.tensors.size(); t++)
      if ((int) P.tensors[t].grad == pass) {
        E.toff[t] = at;
        at += (long long) P.tensors[t].nfuncs * P.tensors[t].channels;
      }
  }
  E.grad_end = at;
  E.per_atom = at;
  E.tensors.set_label("engine:tensor_table");
  E.tensors_host.assign(P.tensors.size(), TensorDev{nullptr, 0});
}

Engine::Engine(const GraceModel &m, int spline_n) : plan_(build_plan(m, spline_n > 0 ? spline_n : 1024))
{
  if (spline_n == 0 && m.layers == 3) throw Unsupported("GRACE-3L: the exact radial MLP (spline 0) is not supported");
  if (spline_n == 0) {    // exact radial MLP (what the reference's generic engine evaluates), tensor-core kernel
    exact_ = true;
    rad1_.setup(m, m.rad1, m.chain1.c0);
    if (m.layers == 2) rad2_.setup(m, m.rad2, m.cr);
    xs_.set_label("work:radial"); R1_.set_label("work:radial"); dR1_.set_label("work:radial");
    R2_.set_label("work:radial"); dR2_.set_label("work:radial");
  }
  require_initialized();
  const ModelPlan &P = plan_;
  if (P.lmax < 1 || P.lmax > 4) throw Unsupported("models with lmax outside 1..4 are not supported");
  if (P.e_nin.size() > 4) throw Unsupported("energy MLPs with more than 4 layers are not supported");
  for (size_t L = 0; L < P.e_nin.size(); L++)
    if (P.e_nin[L] > 128 || P.e_nout[L] > 128) throw Unsupported("energy MLP widths above 128 are not supported");
  if (P.nrho > 128) throw Unsupported("rho_n_out above 128 is not supported");
  l1_saved_.set_label("work:layer1_tensors");
  if (getenv("GRACE_B200_RECOMPUTE_L1")) keep_l1_ = false;
  rcsq_.set_label("engine:cutoffs"); eW_.set_label("engine:energy_mlp"); shift_.set_label("engine:shift");
  lnI_.set_label("engine:norm_scale"); ln0_.set_label("engine:norm_scale"); rcf_.set_label("engine:cutoffs");
  arena_.set_label("work:chunk_tensors"); arena1_.set_label("work:layer1_tensors"); fv_.set_label("work:bond_forces"); I_rows_.set_label("work:messages");
  gmsg_slot_.set_label("work:message_gradient_shares");
  gI_rows_.set_label("work:message_gradients"); rho_rows_.set_label("work:rho"); e_atom_.set_label("work:atom_energy");
  vir_atom_.set_label("work:atom_virial"); sum_scratch_.set_label("work:sums"); grho_rows_.set_label("work:rho_gradients");
  rcsq_.upload(P.rcsq);
  std::vector<float> rcf(P.rc.begin(), P.rc.end());
  rcf_.upload(rcf);
  if (P.layers == 3) {    // its own set-up and drivers (engine3l.cu); none of the GRACE-1L / 2L paths below applies
    if (exact_) throw Unsupported("GRACE-3L: the exact radial MLP (spline 0) is not supported");
    shift_.upload(P.shift);
    if (const char *env = getenv("GRACE_B200_DENSE")) {
      const std::string v = env;
      dense_ = v == "fused" ? Dense::Fused : v == "tc" ? Dense::Tc : v == "ops" ? Dense::Ops : Dense::Auto;
    }
    if (const char *env = getenv("GRACE_B200_TC_MIN_ATOMS")) tc_min_atoms_ = std::max(1, atoi(env));
    tc_error_.set_label("engine:flag");
    tc_error_.ensure(1);
    GB_CUDA(cudaMemsetAsync(tc_error_.get(), 0, sizeof(int), dev().stream));
    setup_3l();
    return;
  }
  eW_.upload(P.eW);
  {    // transposed copies of the energy MLP layers for the reverse pass of the warp readout
    std::vector<double> wt(P.eW.size());
    size_t at = 0;
    for (size_t L = 0; L < P.e_nin.size(); L++) {
      const int ni = P.e_nin[L], no = P.e_nout[L];
      for (int a = 0; a < ni; a++)
        for (int c = 0; c < no; c++) wt[at + (size_t) c * ni + a] = P.eW[at + (size_t) a * no + c];
      at += (size_t) ni * no;
    }
    eWT_.set_label("engine:energy_mlp");
    eWT_.upload(wt);
  }
  shift_.upload(P.shift);
  setup_layer(L1_, P.L1);
  setup_fused(L1_, P.L1);
  fused_ = L1_.fused_TA > 0;
  if (P.layers == 2) {
    setup_layer(L2_, P.L2);
    setup_fused(L2_, P.L2);
    fused_ = fused_ && L2_.fused_TA > 0;
    lnI_.upload(P.lnI);
    ln0_.upload(P.ln0);
  }
  if (P.uq.ready) {
    uq_cen_.set_label("engine:uq"); uq_icov_.set_label("engine:uq"); uq_thr_.set_label("engine:uq"); uq_ncl_.set_label("engine:uq");
    uq_out_.set_label("work:uq"); uq_n2a_.set_label("work:uq"); uq_n2b_.set_label("work:uq"); uq_z1_.set_label("work:uq");
    uq_cen_.upload(P.uq.centroids);
    uq_icov_.upload(P.uq.inv_cov);
    uq_thr_.upload(P.uq.thresholds);
    uq_ncl_.upload(P.uq.n_clusters);
    uq_dev_ = UqDev{uq_cen_.get(), uq_icov_.get(), uq_thr_.get(), uq_ncl_.get(), P.uq.rp_dim, P.uq.feature_dim,
                    P.uq.max_clusters, P.uq.n_density, P.uq.density_scale};
  }
  ReadoutDev &r = readout_;
  r.W = eW_.get();
  r.WT = eWT_.get();
  r.shift = shift_.get();
  r.lnI = lnI_.get();
  r.ln0 = ln0_.get();
  r.nlay = (int) P.e_nin.size();
  for (int L = 0; L < r.nlay; L++) {
    r.n_in[L] = P.e_nin[L];
    r.n_out[L] = P.e_nout[L];
    r.norm[L] = P.e_norm[L];
  }
  r.act = P.e_act;
  r.ln = P.e_ln;
  r.rms = P.rms;
  r.nrho = P.nrho;
  r.out_scale = P.out_scale;
  if (getenv("GRACE_B200_NO_FUSED")) fused_ = false;    // the per-operation kernels, for comparison
  if (const char *env = getenv("GRACE_B200_DENSE")) {
    const std::string v = env;
    dense_ = v == "fused" ? Dense::Fused : v == "tc" ? Dense::Tc : v == "ops" ? Dense::Ops : Dense::Auto;
  }
  if (const char *env = getenv("GRACE_B200_TC_MIN_ATOMS")) tc_min_atoms_ = std::max(1, atoi(env));
  // the tensor-core path pays when it covers most of the MV work of every layer
  tc_ready_ = L1_.tc_flop_share > 0.5 && (P.layers == 1 || L2_.tc_flop_share > 0.5);
  tc_error_.set_label("engine:flag");
  tc_error_.ensure(1);
  GB_CUDA(cudaMemsetAsync(tc_error_.get(), 0, sizeof(int), dev().stream));
  GB_CUDA(cudaStreamSynchronize(dev().stream));    // the uploads read host vectors of this scope
}

Engine::~Engine() = default;

void Engine::dense_stats(double *o) const
{
  if (plan_.layers == 3) {
    for (int q = 0; q < 6; q++) o[q] = 0.0;
    return;
  }
  for (int k = 0; k < 6; k++) o[k] = 0.0;
  for (const LayerEngine *E : {&L1_, &L2_}) {
    if (!E->plan) continue;
    const LayerPlan &P = *E->plan;
    for (size_t q = 0; q < P.mv.size(); q++) {
      if ((int) q == P.uq_mv) continue;
      const MVOp &m = P.mv[q];
      double fl = 0.0, by = 0.0;
      for (const MVItem &it : m.items) {
        fl += 2.0 * it.n_in * m.n_out;
        by += 4.0 * it.n_in;
      }
      by += 4.0 * m.n_out * (double) m.row_out.size() * (m.accumulate ? 2.0 : 1.0);
      const int k = E->mv_tc[q].ready() ? 0 : 4;
      o[k] += fl;
      o[k + 1] += by;
    }
    for (const ProdOp &pr : P.prod) {
      const int C = P.tensors[pr.dst].channels;
      o[2] += 3.0 * (double) pr.terms.size() * C;
      double rows = P.tensors[pr.srcA].nfuncs;
      if (pr.srcB >= 0 && pr.srcB != pr.srcA) rows += P.tensors[pr.srcB].nfuncs;
      rows += (double) pr.row_out.size() * (pr.accumulate ? 2.0 : 1.0);
      o[3] += 4.0 * C * rows;
    }
  }
}

bool Engine::use_tc(int64_t n_eval) const
{
  if (!tc_ready_ || dense_ == Dense::Fused || dense_ == Dense::Ops) return false;
  if (dense_ == Dense::Tc) return true;
  return n_eval >= tc_min_atoms_ || !fused_;
}

bool Engine::use_fused(int64_t n_eval) const
{
  if (!fused_ || dense_ == Dense::Ops) return false;
  return !use_tc(n_eval);
}

double Engine::per_atom_bytes(int64_t n_eval) const
{
  if (use_fused(n_eval)) return 8.0 * (double) std::max(L1_.q_floats, L2_.q_floats);
  return 4.0 * (double) std::max(L1_.per_atom, L2_.per_atom);
}

int Engine::auto_chunk(int64_t n) const
{
  if (plan_.layers == 3) return (int) std::max<int64_t>(n, 1);    // one pass
  size_t free_b = 0, total_b = 0;
  if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) free_b = (size_t) 8 << 30;
  const double budget = 0.35 * (double) free_b + 4.0 * (double) arena_.capacity();
  int64_t c = (int64_t) (budget / per_atom_bytes(n));
  // per-operation passes: large enough that the atom tiles of a pass fill the GPU, small enough to bound the work memory
  c = std::min<int64_t>(c, use_fused(n) ? ((int64_t) 1 << 22) : (use_tc(n) ? 524288 : 32768));
  c = std::max<int64_t>(c, 512);
  return (int) std::min<int64_t>(c, std::max<int64_t>(n, 1));
}

void Engine::release_work()
{
  arena_.release(); fv_.release(); I_rows_.release(); gI_rows_.release(); rho_rows_.release();
  e_atom_.release(); vir_atom_.release(); grho_rows_.release(); sum_scratch_.release();
  xs_.release(); R1_.release(); dR1_.release(); R2_.release(); dR2_.release(); l1_saved_.release(); gmsg_slot_.release();
  uq_out_.release(); uq_n2a_.release(); uq_n2b_.release(); uq_z1_.release();
  arena1_.release();
  arena1_bound_ = nullptr;
  arena1_NA_ = 0;
  arena_NA_ = 0;
}

void Engine::bind_arena(LayerEngine &E, float *base, int NA)
{
  if (!E.plan) return;
  for (size_t t = 0; t < E.tensors_host.size(); t++)
    E.tensors_host[t] = TensorDev{base + E.toff[t] * NA, E.plan->tensors[t].channels};
  E.tensors.upload(E.tensors_host);
}

LayerDev Engine::layer_dev(const LayerEngine &E) const
{
  LayerDev L{};
  L.tab = E.tab.get();
  L.z = E.z.get();
  L.rc = rcf_.get();
  L.msg = nullptr;
  L.gmsg = nullptr;
  L.gmsg_slot = nullptr;
  L.N = E.plan->radial.N;
  L.C = E.plan->C;
  L.n_msg = E.plan->n_msg;
  L.n_elements = plan_.n_elements;
  L.Rex = exact_ ? (&E == &L1_ ? R1_.get() : R2_.get()) : nullptr;
  L.dRex = exact_ ? (&E == &L1_ ? dR1_.get() : dR2_.get()) : nullptr;
  return L;
}

namespace {
struct TagScope {
  bool on;
  TagScope(const char *t) : on(getenv("GRACE_B200_PROFILE_OPS") != nullptr) { if (on) launch_tag(t); }
  ~TagScope() { if (on) launch_tag(nullptr); }
};
}    // namespace

// Buffer for the per-bond shares of dE/dmsg (one row of n_msg x C floats per list slot), when it can be had: the
// reverse bond kernel of layer 2 then stores instead of adding atomically and gather_message_gradients() sums the shares
// per neighbour in list order.  Null (the buffer does not fit): fp32 atomics into the zeroed rows, as the reference does.
float *Engine::message_gradient_slots(NeighborList &nl)
{
  const size_t need = (size_t) std::max<int64_t>(nl.nslots(), 1) * plan_.nI * plan_.cr;
  cudaStream_t st = dev().stream;
  float *p = nullptr;
  if (!getenv("GRACE_B200_MSG_ATOMICS") && !nl.external()) {
    try {
      p = gmsg_slot_.ensure(need);
    } catch (const OutOfMemory &) {
      p = nullptr;
    }
  }
  if (!p) launch_fill_zero(gI_rows_.get(), sizeof(float) * (size_t) nl.n() * plan_.nI * plan_.cr);
  return p;
}

void Engine::gather_message_gradients(NeighborList &nl, const float *slots, const ActiveRanges &R)
{
  if (!slots) return;
  launch_msg_grad_gather(nl.bonds(), nl.rev(), slots, gI_rows_.get(), plan_.nI * plan_.cr, nullptr, (long long) nl.n(),
                         R.nlocal >= 0 ? nl.perm() : nullptr, R.nlocal);
}

void Engine::run(LayerEngine &E, const Program &prog, const int *mu, int NA, int stride)
{
  // NA here is the number of atoms in use; stride: the atom stride of the layer's chunk tensors
  const int arena_NA_ = stride;
  static const bool tag_ops = getenv("GRACE_B200_PROFILE_OPS") != nullptr;
  for (const Op &o : prog.ops) {
    if (tag_ops) launch_tag(o.kind == Op::MV ? E.plan->mv[o.index].name.c_str() : E.plan->prod[o.index].name.c_str());
    if (o.kind == Op::MV) {
      if (tc_now_ && E.mv_tc[o.index].ready())
        E.mv_tc[o.index].launch(E.mv[o.index], E.tensors.get(), (int) E.tensors_host.size(), arena_NA_, NA, tc_error_.get());
      else launch_mv(E.mv[o.index], E.tensors.get(), mu, arena_NA_, NA);
    } else {
      const ProdDev &pd = E.prod[o.index];
      const auto &ts = E.plan->tensors;
      const int C = ts[pd.dst].channels;
      const bool same = ts[pd.srcA].channels == C && (pd.srcB < 0 || ts[pd.srcB].channels == C);
      launch_prod(pd, E.tensors.get(), arena_NA_, NA, C, same ? ts[pd.srcA].nfuncs : 0,
                  pd.srcB >= 0 ? ts[pd.srcB].nfuncs : 0, (int) E.plan->prod[o.index].terms.size());
    }
  }
  if (tag_ops) launch_tag(nullptr);
}

// UQ of GRACE-2L, layer 1 (after the forward program of a chunk of layer 1): projection of the rho block, kept per atom
// with its squared norm until layer 2 adds its own (libgrace/src/fused_2l.cpp:1116-1170)
void Engine::uq_layer1(const int *mu, int64_t a0, int na, int stride)
{
  const LayerPlan &P = *L1_.plan;
  const int q = P.uq_mv;
  if (tc_now_ && L1_.mv_tc[q].ready())
    L1_.mv_tc[q].launch(L1_.mv[q], L1_.tensors.get(), (int) L1_.tensors_host.size(), stride, na, tc_error_.get());
  else launch_mv(L1_.mv[q], L1_.tensors.get(), mu, stride, na);
  launch_uq_norm(L1_.mv[q], L1_.tensors.get(), stride, na, uq_n2b_.get() + a0);
  launch_rows_from_chunk(L1_.tensors_host[P.tUQ].p, uq_z1_.get(), 1, plan_.uq.rp_dim, stride, na, (int) a0);
}

// UQ after the forward program of a chunk of the last layer E: its projection and norm, then the mixture model
void Engine::uq_last(LayerEngine &E, const int *mu, int64_t a0, int na, int stride, int64_t n)
{
  const LayerPlan &P = *E.plan;
  const int q = P.uq_mv;
  if (tc_now_ && E.mv_tc[q].ready())
    E.mv_tc[q].launch(E.mv[q], E.tensors.get(), (int) E.tensors_host.size(), stride, na, tc_error_.get());
  else launch_mv(E.mv[q], E.tensors.get(), mu + a0, stride, na);
  launch_uq_norm(E.mv[q], E.tensors.get(), stride, na, uq_n2a_.get() + a0);
  const bool two = plan_.layers == 2;
  double *o = uq_out_.get();
  launch_uq_gmm(uq_dev_, E.tensors_host[P.tUQ].p, two ? uq_z1_.get() : nullptr, uq_n2a_.get(), two ? uq_n2b_.get() : nullptr, mu,
                na, (long long) a0, o, o + n, o + 2 * n);
}

// shared-memory layout of the tensors of an atom tile: every tensor padded to 4 floats per atom; a gradient that may
// alias a forward tensor shares its offset; TA = the largest atom tile that fits the 227 KB of an SM
void Engine::setup_fused(LayerEngine &E, const LayerPlan &P)
{
  const size_t nt = P.tensors.size();
  std::vector<int> soff(nt, 0), tch(nt, 0);
  std::vector<int2> zero, ops;
  long long at = 0;
  auto size_of = [&](size_t t) { return ((long long) P.tensors[t].nfuncs * P.tensors[t].channels + 3) / 4 * 4; };
  for (size_t t = 0; t < nt; t++) {
    tch[t] = P.tensors[t].channels;
    if (P.tensors[t].alias >= 0 || (int) t == P.tUQ) continue;    // the UQ projection runs on the per-operation path only
    soff[t] = (int) at;
    at += size_of(t);
  }
  for (size_t t = 0; t < nt; t++) {
    if (P.tensors[t].alias >= 0) soff[t] = soff[P.tensors[t].alias];
    if (P.tensors[t].grad) zero.push_back(make_int2(soff[t], (int) size_of(t)));
  }
  for (const Op &o : P.fwd.ops) ops.push_back(make_int2(o.kind == Op::MV ? 0 : 1, o.index));
  for (const Op &o : P.bwd.ops) ops.push_back(make_int2(o.kind == Op::MV ? 0 : 1, o.index));
  if (getenv("GRACE_B200_PRINT_PLAN")) {    // diagnostics: the operation list of the layer
    int k = 0;
    for (const Program *prog : {&P.fwd, &P.bwd})
      for (const Op &o : prog->ops) {
        if (o.kind == Op::MV) {
          const MVOp &m = P.mv[o.index];
          int nmin = 1 << 30, nmax = 0;
          for (const MVItem &it : m.items) { nmin = std::min(nmin, it.n_in); nmax = std::max(nmax, it.n_in); }
          fprintf(stderr, "op %2d MV   %-18s rows %4zu n_out %3d items %4zu n_in %d..%d elem %d slots %zu units %zu\n", k,
                  m.name.c_str(), m.row_out.size(), m.n_out, m.items.size(), nmin, nmax, (int) m.elem,
                  m.slot_off.empty() ? (size_t) 0 : m.slot_off.size() - 1, m.unit_desc.size() / 5);
        } else {
          const ProdOp &q = P.prod[o.index];
          fprintf(stderr, "op %2d PROD %-18s rows %4zu terms %5zu channels %d\n", k, q.name.c_str(), q.row_out.size(),
                  q.terms.size(), P.tensors[q.dst].channels);
        }
        k++;
      }
  }
  E.f_mv.set_label("engine:tables"); E.f_prod.set_label("engine:tables"); E.f_ops.set_label("engine:tables");
  E.f_zero.set_label("engine:tables"); E.f_soff.set_label("engine:tables"); E.f_tch.set_label("engine:tables");
  E.f_mv.upload(E.mv);
  E.f_prod.upload(E.prod);
  E.f_ops.upload(ops);
  E.f_zero.upload(zero);
  // forward tensors some reverse operation reads (operands of product adjoints, inputs of reduces over them)
  std::vector<int4> save;
  long long save_floats = 0;
  {
    std::vector<char> read(nt, 0);
    for (const Op &o : P.bwd.ops) {
      if (o.kind == Op::MV) {
        for (const MVItem &it : P.mv[o.index].items) read[it.src] = 1;
      } else {
        const ProdOp &q = P.prod[o.index];
        read[q.srcA] = 1;
        if (q.srcB >= 0) read[q.srcB] = 1;
      }
    }
    for (size_t t = 0; t < nt; t++)
      if (read[t] && !P.tensors[t].grad) {
        save.push_back(make_int4(soff[t], P.tensors[t].nfuncs, P.tensors[t].channels, (int) save_floats));
        save_floats += size_of(t);
      }
  }
  E.f_save.set_label("engine:tables");
  E.f_save.upload(save);
  E.f_soff.upload(soff);
  E.f_tch.upload(tch);
  FusedLayerDev &F = E.fused;
  F.mv = E.f_mv.get();
  F.prod = E.f_prod.get();
  F.ops = E.f_ops.get();
  F.nfwd = (int) P.fwd.ops.size();
  F.nbwd = (int) P.bwd.ops.size();
  F.soff = E.f_soff.get();
  F.tch = E.f_tch.get();
  F.zero = E.f_zero.get();
  F.nzero = (int) zero.size();
  F.save = E.f_save.get();
  F.nsave = (int) save.size();
  F.save_floats = (int) save_floats;
  F.per_atom = (int) at;
  E.q_floats = (long long) P.tensors[P.tQ].nfuncs * P.tensors[P.tQ].channels;
  F.nmv = (int) E.mv.size();
  F.nprod = (int) E.prod.size();
  F.ntensors = (int) nt;
  F.itab = E.itab.get();
  F.items = E.items.get();
  F.terms = E.terms.get();
  F.n_itab = E.n_itab;
  F.n_items = E.n_items;
  F.n_terms = E.n_terms;
  // shared memory: the tables, then TA atoms of tensors; the product terms are staged only if a tile still fits
  const long long limit = 227 * 1024 - 1024;
  auto tab_bytes = [&](bool with_terms) {
    long long b = (long long) sizeof(MVDev) * F.nmv + sizeof(ProdDev) * F.nprod + sizeof(int2) * (ops.size() + zero.size()) +
                  sizeof(int) * (2 * nt + E.n_itab) + sizeof(MVItem) * E.n_items + (with_terms ? sizeof(ProdTerm) * E.n_terms : 0);
    return (b + 15) / 16 * 16;
  };
  // two warp groups per CTA (each on its own tile) unless they would get one atom each while a single group of all
  // warps gets a tile of two or more: then the atoms of the tile share every weight fetched (GRACE_B200_GROUPS
  // overrides)
  auto tile_for = [&](long long tbytes, int ng) {
    for (int ta : {8, 6, 5, 4, 3, 2, 1})
      if (tbytes + at * 4 * ta * ng <= limit) return ta;
    return 0;
  };
  int ng = 2;
  {
    const long long t2 = tab_bytes(tab_bytes(true) + at * 4 * 2 <= limit), t1 = tab_bytes(tab_bytes(true) + at * 4 <= limit);
    if (tile_for(t2, 2) <= 1 && tile_for(t1, 1) >= 2) ng = 1;
    if (const char *env = getenv("GRACE_B200_GROUPS")) {
      const int g = atoi(env);
      if (g == 1 || g == 2) ng = g;
    }
  }
  E.fused_NG = ng;
  F.stage_terms = tab_bytes(true) + at * 4 * ng <= limit;
  long long tb = tab_bytes(F.stage_terms);
  // a small energy MLP goes to shared memory too (its rows are read one after the other by the warp readout: from
  // global memory every row is an L2 round trip), unless that would cost an atom of the tile
  F.stage_ro = 0;
  F.ro_offset = 0;
  {
    const long long nd = (long long) plan_.eW.size(), extra = (2 * nd * 8 + 15) / 16 * 16;
    if (nd > 0 && extra <= 16384 && tile_for(tb, ng) > 0 && tile_for(tb + extra, ng) == tile_for(tb, ng)) {
      F.stage_ro = (int) nd;
      F.ro_offset = (int) tb;
      tb += extra;
    }
  }
  F.tab_floats = (int) (tb / 4);
  E.fused_TA = tile_for(tb, ng);
  if (const char *env = getenv("GRACE_B200_TILE_ATOMS")) {
    const int ta = atoi(env);
    if (ta >= 1 && ta <= 8 && ta != 7 && tb + at * 4 * ta * ng <= limit) E.fused_TA = ta;
  }
  if (getenv("GRACE_B200_PRINT_PLAN"))
    fprintf(stderr, "fused layer: %lld floats per atom, tables %lld bytes, tile atoms %d x %d groups\n", at, tb, E.fused_TA, ng);
  GB_CUDA(cudaStreamSynchronize(dev().stream));
}

void Engine::run_fused(LayerEngine &E, int mode, int NA, int a0, int na, const int *mu, const int *ilist, float *saved)
{
  const ModelPlan &P = plan_;
  const LayerPlan &LP = *E.plan;
  FusedIO io{};
  io.mode = mode;
  io.tQ = LP.tQ;
  io.tGQ = LP.tGQ;
  io.nQ = LP.tensors[LP.tQ].nfuncs;
  io.CQ = LP.tensors[LP.tQ].channels;
  io.Q = arena_.get();
  io.gQ = arena_.get() + (size_t) E.q_floats * NA;
  io.NA = NA;
  io.nrho = P.nrho;
  io.nI = P.nI;
  io.CR = P.cr;
  if (&E == &L1_) {
    io.t_rho = P.t1_rho; io.t_grho = P.t1_grho; io.t_I = P.t1_I; io.t_gI = P.t1_gI;
  } else {
    io.t_I2 = P.t2_I2; io.t_gI2 = P.t2_gI2;
  }
  io.I_rows = I_rows_.get();
  io.rho_rows = rho_rows_.get();
  io.gI_rows = gI_rows_.get();
  io.grho_rows = grho_rows_.get();
  io.ro = readout_;
  io.mu = mu;
  io.e_atom = e_atom_.get();
  io.a0 = a0;
  io.na = na;
  io.ilist = ilist;
  io.saved = saved;
  const int TA = E.fused_TA;
  const int ntiles = (na + TA - 1) / TA, nctas = (ntiles + E.fused_NG - 1) / E.fused_NG;
  if (E.fused_NG == 1) launch_chain_fused_g1(TA, E.fused, io, std::min(nctas, dev().sm_count));
  else launch_chain_fused(TA, E.fused, io, std::min(nctas, dev().sm_count));
}

// bond sums -> fused dense network (forward, readout, reverse in one kernel) -> bond forces; only the bond-sum tensor
// and its gradient live in global memory, so a pass can hold every atom of most structures
void Engine::evaluate_fused(NeighborList &nl, bool energy_only, int NA, StageTimer *tm, const ActiveRanges &R)
{
  const int64_t n = nl.n();
  cudaStream_t st = dev().stream;
  const ModelPlan &P = plan_;
  const long long qf = std::max(L1_.q_floats, L2_.q_floats);
  arena_.ensure((size_t) 2 * qf * NA);
  arena_NA_ = 0;    // the chunked layout, if it was bound, no longer is
  const int *mu = nl.mu_sorted();
  float *fv = fv_.get();
  float *Q = arena_.get();
  const int bwd = energy_only ? 0 : FUSED_BWD;
  // atoms evaluated per layer: all of the list, or the exact sets of a domain-decomposed caller (positions a0 .. of
  // the set are the chunk's atoms)
  BondsDev b0 = nl.bonds(), b1 = nl.bonds();
  b0.ilist = R.list0;
  b1.ilist = R.list1;
  const int64_t n0 = R.list0 ? R.n0 : n, n1 = R.list1 ? R.n1 : n;
  if (P.layers == 1) {
    const LayerDev L = layer_dev(L1_);
    const float *gQ = arena_.get() + (size_t) L1_.q_floats * NA;
    for (int64_t a0 = 0; a0 < n0; a0 += NA) {
      const int na = (int) std::min<int64_t>(NA, n0 - a0);
      if (tm) tm->begin(StageTimer::FWD);
      launch_bond_fwd(P.lmax, b0, L, Q, NA, (int) a0, na);
      run_fused(L1_, FUSED_READOUT_1L | bwd, NA, (int) a0, na, mu, R.list0);
      if (tm) tm->end(StageTimer::FWD);
      if (energy_only) continue;
      if (tm) tm->begin(StageTimer::BWD);
      launch_bond_bwd(P.lmax, b0, L, gQ, NA, (int) a0, na, fv, vir_atom_.get(), 0);
      if (tm) tm->end(StageTimer::BWD);
    }
    return;
  }
  const int nI = P.nI, CR = P.cr, nrho = P.nrho;
  I_rows_.ensure((size_t) n * nI * CR);
  rho_rows_.ensure((size_t) n * nrho);
  float *gslots = nullptr;
  if (!energy_only) {
    gI_rows_.ensure((size_t) n * nI * CR);
    grho_rows_.ensure((size_t) n * nrho);
    gslots = message_gradient_slots(nl);
  }
  const LayerDev La = layer_dev(L1_);
  LayerDev Lb = layer_dev(L2_);
  Lb.msg = I_rows_.get();
  Lb.gmsg = gI_rows_.get();
  Lb.gmsg_slot = gslots;
  const float *gQ1 = arena_.get() + (size_t) L1_.q_floats * NA, *gQ2 = arena_.get() + (size_t) L2_.q_floats * NA;
  if (tm) tm->begin(StageTimer::FWD);
  // the layer-1 tensors its reverse pass reads are kept in global memory between the passes when they fit (else layer
  // 1 is evaluated a second time)
  float *saved = nullptr;
  if (!energy_only && keep_l1_ && L1_.fused.save_floats > 0) {
    try {
      saved = l1_saved_.ensure((size_t) L1_.fused.save_floats * (size_t) n1);
    } catch (const OutOfMemory &) {
      keep_l1_ = false;
    }
  }
  for (int64_t a0 = 0; a0 < n1; a0 += NA) {    // layer 1 forward: messages and rho of the atoms layer 2 reads
    const int na = (int) std::min<int64_t>(NA, n1 - a0);
    launch_bond_fwd(P.lmax, b1, La, Q, NA, (int) a0, na);
    run_fused(L1_, FUSED_STORE_MSG | (saved ? FUSED_SAVE : 0), NA, (int) a0, na, mu, R.list1, saved);
  }
  call_hook(true);
  for (int64_t a0 = 0; a0 < n0; a0 += NA) {    // layer 2, energy, layer-2 reverse
    const int na = (int) std::min<int64_t>(NA, n0 - a0);
    launch_bond_fwd(P.lmax, b0, Lb, Q, NA, (int) a0, na);
    run_fused(L2_, FUSED_READOUT_2L | bwd, NA, (int) a0, na, mu, R.list0);
    if (!energy_only) launch_bond_bwd(P.lmax, b0, Lb, gQ2, NA, (int) a0, na, fv, vir_atom_.get(), 0);
  }
  if (tm) tm->end(StageTimer::FWD);
  if (energy_only) return;
  if (tm) tm->begin(StageTimer::BWD);
  gather_message_gradients(nl, gslots, R);
  call_hook(false);
  for (int64_t a0 = 0; a0 < n1; a0 += NA) {    // layer 1 recomputed and reversed from dE/dI, dE/drho
    const int na = (int) std::min<int64_t>(NA, n1 - a0);
    if (!saved) launch_bond_fwd(P.lmax, b1, La, Q, NA, (int) a0, na);
    run_fused(L1_, FUSED_LOAD_SEED | FUSED_BWD | (saved ? FUSED_RESTORE : 0), NA, (int) a0, na, mu, R.list1, saved);
    launch_bond_bwd(P.lmax, b1, La, gQ1, NA, (int) a0, na, fv, vir_atom_.get(), 1);
  }
  if (tm) tm->end(StageTimer::BWD);
}

// the dense network as one kernel launch per operation on chunk tensors in global memory: the path for layers whose
// tensors of a single atom do not fit the shared memory of an SM
void Engine::evaluate_chunked(NeighborList &nl, bool energy_only, int NA, StageTimer *tm, const ActiveRanges &R)
{
  const int64_t n = nl.n();
  cudaStream_t st = dev().stream;
  const ModelPlan &P = plan_;
  const long long per_atom = std::max(L1_.per_atom, L2_.per_atom);
  // Atoms of a pass: positions lo .. hi of the list order, or - for a domain-decomposed caller - of the exact lists of
  // the atoms each layer needs (position p then stands for atom ilist[p]); mu: the elements by position
  struct Span {
    int64_t lo, hi;
    const int *ilist, *mu;
  };
  Span s0{R.lo0, R.hi0, nullptr, nl.mu_sorted()}, s1{R.lo1, R.hi1, nullptr, nl.mu_sorted()};
  if (R.list0 && R.list1) {
    launch_gather_int(nl.mu_sorted(), R.list0, mu_l0_.ensure((size_t) std::max<int64_t>(R.n0, 1)), R.n0);
    launch_gather_int(nl.mu_sorted(), R.list1, mu_l1_.ensure((size_t) std::max<int64_t>(R.n1, 1)), R.n1);
    s0 = Span{0, R.n0, R.list0, mu_l0_.get()};
    s1 = Span{0, R.n1, R.list1, mu_l1_.get()};
  }
  // GRACE-2L with forces: layer 1 gets tensors of its own for all of its atoms in one pass when they fit, so that its
  // reverse pass finds the forward tensors where they were left instead of evaluating the layer a second time
  float *base1 = nullptr;
  int NA1 = 0;
  if (P.layers == 2 && !energy_only && keep_l1_ && s1.hi > s1.lo) {
    const int64_t w1 = (s1.hi - s1.lo + 3) / 4 * 4;
    size_t free_b = 0, total_b = 0;
    const size_t need = (size_t) L1_.per_atom * (size_t) w1 * sizeof(float);
    if (w1 < ((int64_t) 1 << 30) && cudaMemGetInfo(&free_b, &total_b) == cudaSuccess &&
        need <= (size_t) (0.45 * (double) free_b) + arena1_.capacity() * sizeof(float)) {
      try {
        base1 = arena1_.ensure((size_t) L1_.per_atom * (size_t) w1);
        NA1 = (int) w1;
      } catch (const OutOfMemory &) {
        base1 = nullptr;
      }
    }
  }
  const float *arena_before = arena_.get();
  arena_.ensure((size_t) (base1 ? L2_.per_atom : per_atom) * NA);
  if (arena_.get() != arena_before || arena_NA_ != NA || arena1_bound_ != base1 || arena1_NA_ != NA1) {
    arena_NA_ = NA;
    arena1_bound_ = base1;
    arena1_NA_ = NA1;
    bind_arena(L1_, base1 ? base1 : arena_.get(), base1 ? NA1 : NA);
    bind_arena(L2_, arena_.get(), NA);
  }
  BondsDev bonds0 = nl.bonds(), bonds1 = nl.bonds();
  bonds0.ilist = s0.ilist;
  bonds1.ilist = s1.ilist;
  const int *mu = nl.mu_sorted();
  float *fv = fv_.get();
  auto zero_grads = [&](LayerEngine &E, float *base, int stride) {
    if (!E.plan->zero_grads) return;    // every gradient row is written before it is added to
    launch_fill_zero(base + E.grad_begin * stride, sizeof(float) * (size_t) (E.grad_end - E.grad_begin) * stride);
  };
  const int S1 = base1 ? NA1 : NA;                   // atom stride of the layer-1 tensors
  const int64_t step1 = base1 ? (int64_t) NA1 : NA;    // atoms per layer-1 pass
  float *const abase1 = base1 ? base1 : arena_.get();
  auto T1 = [&](int t) { return L1_.tensors_host[t].p; };
  auto T2 = [&](int t) { return L2_.tensors_host[t].p; };

  if (P.layers == 1) {
    const LayerDev L = layer_dev(L1_);
    for (int64_t a0 = s0.lo; a0 < s0.hi; a0 += NA) {
      const int na = (int) std::min<int64_t>(NA, s0.hi - a0);
      if (tm) tm->begin(StageTimer::FWD);
      launch_bond_fwd(P.lmax, bonds0, L, T1(P.L1.tQ), NA, (int) a0, na);
      run(L1_, P.L1.fwd, s0.mu + a0, na, NA);
      if (uq_now_) uq_last(L1_, mu, a0, na, NA, n);
      launch_readout_1l(readout_, T1(P.t1_rho), T1(P.t1_grho), mu, e_atom_.get(), NA, na, (int) a0, !energy_only, s0.ilist);
      if (tm) tm->end(StageTimer::FWD);
      if (energy_only) continue;
      if (tm) tm->begin(StageTimer::BWD);
      zero_grads(L1_, arena_.get(), NA);
      run(L1_, P.L1.bwd, s0.mu + a0, na, NA);
      launch_bond_bwd(P.lmax, bonds0, L, T1(P.L1.tGQ), NA, (int) a0, na, fv, vir_atom_.get(), 0);
      if (tm) tm->end(StageTimer::BWD);
    }
  } else {
    const int nI = P.nI, CR = P.cr, nrho = P.nrho;
    I_rows_.ensure((size_t) n * nI * CR);
    rho_rows_.ensure((size_t) n * nrho);
    float *gslots = nullptr;
    if (!energy_only) {
      gI_rows_.ensure((size_t) n * nI * CR);
      grho_rows_.ensure((size_t) n * nrho);
      gslots = message_gradient_slots(nl);
    }
    const LayerDev La = layer_dev(L1_);
    LayerDev Lb = layer_dev(L2_);
    Lb.msg = I_rows_.get();
    Lb.gmsg = gI_rows_.get();
    Lb.gmsg_slot = gslots;
    // layer 1 forward of every chunk: messages I and rho of all atoms
    if (tm) tm->begin(StageTimer::FWD);
    for (int64_t a0 = s1.lo; a0 < s1.hi; a0 += step1) {
      const int na = (int) std::min<int64_t>(step1, s1.hi - a0);
      { TagScope tg("layer1"); launch_bond_fwd(P.lmax, bonds1, La, T1(P.L1.tQ), S1, (int) a0, na); }
      run(L1_, P.L1.fwd, s1.mu + a0, na, S1);
      if (uq_now_) uq_layer1(mu + a0, a0, na, S1);
      launch_rows_from_chunk(T1(P.t1_I), I_rows_.get(), nI, CR, S1, na, (int) a0, s1.ilist);
      launch_rows_from_chunk(T1(P.t1_rho), rho_rows_.get(), 1, nrho, S1, na, (int) a0, s1.ilist);
    }
    if (tm) tm->end(StageTimer::FWD);
    call_hook(true);
    // layer 2 forward, energy and layer-2 reverse per chunk
    for (int64_t a0 = s0.lo; a0 < s0.hi; a0 += NA) {
      const int na = (int) std::min<int64_t>(NA, s0.hi - a0);
      if (tm) tm->begin(StageTimer::FWD);
      { TagScope tg("layer2"); launch_bond_fwd(P.lmax, bonds0, Lb, T2(P.L2.tQ), NA, (int) a0, na); }
      run(L2_, P.L2.fwd, s0.mu + a0, na, NA);
      if (uq_now_) uq_last(L2_, mu, a0, na, NA, n);
      launch_readout_2l(readout_, rho_rows_.get(), T2(P.t2_I2), grho_rows_.get(), T2(P.t2_gI2), mu, e_atom_.get(), NA,
                        na, (int) a0, !energy_only, s0.ilist);
      if (tm) tm->end(StageTimer::FWD);
      if (energy_only) continue;
      if (tm) tm->begin(StageTimer::BWD);
      zero_grads(L2_, arena_.get(), NA);
      run(L2_, P.L2.bwd, s0.mu + a0, na, NA);
      { TagScope tg("layer2"); launch_bond_bwd(P.lmax, bonds0, Lb, T2(P.L2.tGQ), NA, (int) a0, na, fv, vir_atom_.get(), 0); }
      if (tm) tm->end(StageTimer::BWD);
    }
    // layer 1 again (recomputed) and its reverse, seeded with dE/dI and dE/drho of each atom
    if (!energy_only) {
      if (tm) tm->begin(StageTimer::BWD);
      gather_message_gradients(nl, gslots, R);
      call_hook(false);
      for (int64_t a0 = s1.lo; a0 < s1.hi; a0 += step1) {
        const int na = (int) std::min<int64_t>(step1, s1.hi - a0);
        if (!base1) {    // the tensors of layer 1 were overwritten by layer 2: evaluate it again
          launch_bond_fwd(P.lmax, bonds1, La, T1(P.L1.tQ), S1, (int) a0, na);
          run(L1_, P.L1.fwd, s1.mu + a0, na, S1);
        }
        zero_grads(L1_, abase1, S1);
        launch_chunk_from_rows(T1(P.t1_gI), gI_rows_.get(), nI, CR, S1, na, (int) a0, s1.ilist);
        launch_chunk_from_rows_f64(T1(P.t1_grho), grho_rows_.get(), 1, nrho, S1, na, (int) a0, s1.ilist);
        run(L1_, P.L1.bwd, s1.mu + a0, na, S1);
        { TagScope tg("layer1"); launch_bond_bwd(P.lmax, bonds1, La, T1(P.L1.tGQ), S1, (int) a0, na, fv, vir_atom_.get(), 1); }
      }
      if (tm) tm->end(StageTimer::BWD);
    }
  }
}

ActiveRanges Engine::active_ranges(NeighborList &nl, int nlocal, int ninner, DBuf<int> &list0, DBuf<int> &list1)
{
  ActiveRanges R;
  const int64_t n = nl.n();
  R.hi0 = R.hi1 = R.n0 = R.n1 = n;
  if (nlocal < 0 || n == 0) return R;
  R.nlocal = nlocal;
  // once per list build: the order of the list on the host, the two sets in that order back to the device
  std::vector<int> perm((size_t) n), l0, l1;
  cudaStream_t st = dev().stream;
  GB_CUDA(cudaMemcpyAsync(perm.data(), nl.perm(), sizeof(int) * (size_t) n, cudaMemcpyDeviceToHost, st));
  GB_CUDA(cudaStreamSynchronize(st));
  const int ni = ninner < 0 ? INT_MAX : std::max(ninner, nlocal);
  for (int64_t i = 0; i < n; i++) {
    if (perm[(size_t) i] < nlocal) l0.push_back((int) i);
    if (perm[(size_t) i] < ni) l1.push_back((int) i);
  }
  R.n0 = (int64_t) l0.size();
  R.n1 = (int64_t) l1.size();
  R.lo0 = l0.empty() ? 0 : l0.front(); R.hi0 = l0.empty() ? 0 : l0.back() + 1;
  R.lo1 = l1.empty() ? 0 : l1.front(); R.hi1 = l1.empty() ? 0 : l1.back() + 1;
  list0.set_label("work:active_atoms");
  list1.set_label("work:active_atoms");
  list0.ensure(std::max<size_t>(l0.size(), 1));
  list1.ensure(std::max<size_t>(l1.size(), 1));
  if (!l0.empty()) GB_CUDA(cudaMemcpyAsync(list0.get(), l0.data(), sizeof(int) * l0.size(), cudaMemcpyHostToDevice, st));
  if (!l1.empty()) GB_CUDA(cudaMemcpyAsync(list1.get(), l1.data(), sizeof(int) * l1.size(), cudaMemcpyHostToDevice, st));
  GB_CUDA(cudaStreamSynchronize(st));    // the host vectors go out of scope
  R.list0 = list0.get();
  R.list1 = list1.get();
  return R;
}

void Engine::call_hook(bool forward)
{
  if (!hooks_) return;
  auto fn = forward ? hooks_->forward : hooks_->reverse;
  if (!fn) return;
  cudaStream_t st = dev().stream;
  GB_CUDA(cudaStreamSynchronize(st));
  fn(hooks_->user, forward ? I_rows_.get() : gI_rows_.get(), plan_.nI * plan_.cr, (void *) st);
}

void Engine::evaluate(NeighborList &nl, bool energy_only, const OutputsDev &out, int chunk, StageTimer *tm,
                      const ActiveRanges *act, const ExchangeHooks *hooks)
{
  hooks_ = plan_.layers == 2 ? hooks : nullptr;
  const int64_t n = nl.n();
  const int nsys = nl.nsys();
  ActiveRanges R;
  if (act && act->nlocal >= 0) R = *act;
  else R.hi0 = R.hi1 = n;
  readout_.perm = R.nlocal >= 0 ? nl.perm() : nullptr;
  readout_.nlocal = R.nlocal;
  cudaStream_t st = dev().stream;
  if (n == 0) {
    if (out.energy) GB_CUDA(cudaMemsetAsync(out.energy, 0, sizeof(double) * nsys, st));
    if (out.virial && !energy_only) GB_CUDA(cudaMemsetAsync(out.virial, 0, sizeof(double) * 6 * nsys, st));
    return;
  }
  if (plan_.layers == 3) {
    if (R.nlocal >= 0) throw Unsupported("GRACE-3L: domain-decomposed callers are not supported");
    if (out.gamma) throw InvalidArgument("the model has no usable UQ head");
    e_atom_.ensure(n);
    if (!energy_only) vir_atom_.ensure(6 * n);
    evaluate_3l(nl, energy_only, tm);
    write_outputs(nl, energy_only, out);
    return;
  }
  const int64_t n_eval = R.list0 ? std::max(R.n0, R.n1) : std::max(R.hi0 - R.lo0, R.hi1 - R.lo1);
  uq_now_ = out.gamma != nullptr;
  if (uq_now_) {
    if (!plan_.uq.ready) throw InvalidArgument("the model has no usable UQ head");
    if (!out.sigma || !out.cluster) throw InvalidArgument("uq needs the gamma, sigma and cluster outputs");
    // results per atom in list order (zero for atoms the call does not own); layer-1 rows of GRACE-2L
    GB_CUDA(cudaMemsetAsync(uq_out_.ensure(3 * (size_t) n), 0, sizeof(double) * 3 * (size_t) n, st));
    uq_n2a_.ensure(n);
    if (plan_.layers == 2) {
      uq_n2b_.ensure(n);
      uq_z1_.ensure((size_t) n * plan_.uq.rp_dim);
    }
  }
  // the UQ projection reads the chunk tensors of the per-operation path
  const bool fused_now = !uq_now_ && use_fused(n_eval);
  tc_now_ = !fused_now && use_tc(n_eval);
  if (uq_now_) R.list0 = R.list1 = nullptr;    // the UQ arrays are indexed by list position: the enclosing ranges
  const bool partial = R.list0 ? (R.n0 < n || R.n1 < n) : (R.lo0 > 0 || R.hi0 < n || R.lo1 > 0 || R.hi1 < n);
  const int64_t widest = std::max<int64_t>(1, R.list0 ? std::max(R.n0, R.n1) : std::max(R.hi0 - R.lo0, R.hi1 - R.lo1));
  // atoms per pass, rounded up to a multiple of 4: it is the atom stride of the chunk tensors, whose rows the vector
  // loads of the kernels want 16-byte aligned whatever the channel counts are
  const int NA = (int) ((std::min<int64_t>(widest, chunk > 0 ? chunk : n) + 3) / 4 * 4);
  e_atom_.ensure(n);
  if (!energy_only) vir_atom_.ensure(6 * n);
  if (partial) {    // what the skipped atoms would have written is read below or by the active atoms: zeros
    launch_fill_zero(e_atom_.get(), sizeof(double) * n);
    if (!energy_only) {
      launch_fill_zero(vir_atom_.get(), sizeof(double) * 6 * n);
      launch_fill_zero(fv_.get(), sizeof(float) * 3 * (size_t) nl.nslots());
    }
    if (plan_.layers == 2) {
      I_rows_.ensure((size_t) n * plan_.nI * plan_.cr);
      launch_fill_zero(I_rows_.get(), sizeof(float) * (size_t) n * plan_.nI * plan_.cr);
      if (!energy_only) {
        grho_rows_.ensure((size_t) n * plan_.nrho);
        launch_fill_zero(grho_rows_.get(), sizeof(double) * (size_t) n * plan_.nrho);
      }
    }
  }
  if (exact_) {    // R and dR/dx of every list slot by the tensor-core MLP (memory: slots x outputs x 8 bytes per layer)
    const long long ns = nl.nslots();
    if (tm) tm->begin(StageTimer::FWD);
    launch_bond_x(nl.bonds(), rcf_.get(), plan_.n_elements, xs_.ensure((size_t) std::max<long long>(ns, 1)), (long long) n);
    const size_t w1 = (size_t) rad1_.n_out();
    R1_.ensure(w1 * (size_t) std::max<long long>(ns, 1));
    dR1_.ensure(w1 * (size_t) std::max<long long>(ns, 1));
    rad1_.run(xs_.get(), ns, R1_.get(), dR1_.get());
    if (plan_.layers == 2) {
      const size_t w2 = (size_t) rad2_.n_out();
      R2_.ensure(w2 * (size_t) std::max<long long>(ns, 1));
      dR2_.ensure(w2 * (size_t) std::max<long long>(ns, 1));
      rad2_.run(xs_.get(), ns, R2_.get(), dR2_.get());
    }
    if (tm) tm->end(StageTimer::FWD);
  }
  if (fused_now) evaluate_fused(nl, energy_only, NA, tm, R);
  else evaluate_chunked(nl, energy_only, NA, tm, R);
  if (tc_now_) {
    int e = 0;
    GB_CUDA(cudaMemcpyAsync(&e, tc_error_.get(), sizeof(int), cudaMemcpyDeviceToHost, st));
    GB_CUDA(cudaStreamSynchronize(st));
    if (e) {
      GB_CUDA(cudaMemsetAsync(tc_error_.get(), 0, sizeof(int), st));
      throw DeviceError("the tensor-core FC kernel gave up waiting for its matrix instructions");
    }
  }
  if (exact_) {
    rad1_.check();
    if (plan_.layers == 2) rad2_.check();
  }
  write_outputs(nl, energy_only, out);
}

// sums and gathers that leave the engine
void Engine::write_outputs(NeighborList &nl, bool energy_only, const OutputsDev &out)
{
  const int64_t n = nl.n();
  const int nsys = nl.nsys();
  float *fv = fv_.get();
  // one or a few large structures: partial sums by 64 blocks per structure and component
  const int nb = (nsys <= 8 && n > 16384) ? 64 : 1;
  double *scr = nb > 1 ? sum_scratch_.ensure((size_t) nsys * 6 * nb) : nullptr;
  if (out.energy) launch_segment_sum(e_atom_.get(), 1, nl.seg(), nsys, out.energy, scr, nb);
  if (out.energies) launch_scatter_f64(e_atom_.get(), nl.perm(), out.energies, (int) n);
  if (uq_now_) {
    launch_scatter_f64(uq_out_.get(), nl.perm(), out.gamma, (int) n);
    launch_scatter_f64(uq_out_.get() + n, nl.perm(), out.sigma, (int) n);
    launch_scatter_f64(uq_out_.get() + 2 * n, nl.perm(), out.cluster, (int) n);
  }
  if (!energy_only) {
    if (out.virial) launch_segment_sum(vir_atom_.get(), 6, nl.seg(), nsys, out.virial, scr, nb);
    if (out.forces) {
      if (nl.external()) launch_force_scatter(nl.bonds(), fv, out.forces, (long long) n);    // accumulates
      else launch_force_gather(nl.off(), nl.rev(), fv, nl.perm(), out.forces, (int) n);
    }
  }
}

// ---- model -----------------------------------------------------------------------------------------------------
void ModelObj::radial_exact(int layer, const float *d_x, long long nb, float *d_R, float *d_dR)
{
  require_initialized();
  if (layer < 1 || layer > model.layers) throw InvalidArgument("layer must be 1 .. layers of the model");
  if (nb < 0 || (nb > 0 && (!d_x || !d_R || !d_dR))) throw InvalidArgument("distances and outputs must be given");
  std::lock_guard<std::mutex> lk(mu);
  RadialMlpTC &r = radial_tc[layer - 1];
  if (!r.ready()) {
    if (layer == 1) r.setup(model, model.rad1, model.chain1.c0);
    else r.setup(model, model.rad2, model.cr);
  }
  r.run(d_x, nb, d_R, d_dR);
  r.check();
}

std::shared_ptr<Engine> ModelObj::get_engine(int spline_n)
{
  std::lock_guard<std::mutex> lk(mu);
  if (spline_n != 0 && spline_n < 16) throw InvalidArgument("spline N must be >= 16 (or 0: exact radial MLP)");
  std::shared_ptr<Engine> &e = engines[spline_n];
  if (!e) {
    try {
      e = std::make_shared<Engine>(model, spline_n);
    } catch (...) {
      engines.erase(spline_n);
      throw;
    }
    setups++;
  }
  return e;
}

// ---- system ----------------------------------------------------------------------------------------------------
namespace {

void label_ws(Workspace &w)
{
  w.pos.set_label("system:positions"); w.energy.set_label("system:energy"); w.virial.set_label("system:virial");
  w.forces.set_label("system:forces"); w.energies.set_label("system:energies"); w.types.set_label("system:types");
  w.mu.set_label("system:elements"); w.t2m.set_label("system:type_map"); w.flag.set_label("system:flag");
  w.types_prev.set_label("system:types");
}

int read_int(const int *d)
{
  int h = 0;
  GB_CUDA(cudaMemcpyAsync(&h, d, sizeof(int), cudaMemcpyDeviceToHost, dev().stream));
  GB_CUDA(cudaStreamSynchronize(dev().stream));
  return h;
}

// flag 4 (UQ): the engine must have a usable head and the caller must have named the three outputs
// (python/kk/kk_core.cpp:826-827, 1284-1286)
void check_flags(int flags, const Engine &e, const UqOutputs &uq)
{
  if (flags & ~7) throw InvalidArgument("unknown compute flag");
  if (!(flags & 4)) return;
  if (!e.uq_available()) throw InvalidArgument("the model has no usable UQ head (schema 6, gamma only)");
  if (!uq.gamma || !uq.sigma || !uq.cluster) throw InvalidArgument("uq needs the gamma, sigma and cluster outputs");
}

}    // namespace

SystemObj::SystemObj(std::shared_ptr<ModelObj> m, const std::vector<std::string> &species, double skin, int spline,
                     int chunk)
    : model_(std::move(m)), skin_(skin), chunk_req_(chunk)
{
  require_initialized();
  if (!(skin >= 0.0) || !std::isfinite(skin)) throw InvalidArgument("skin must be >= 0");
  t2m_ = species_to_elements(model_->model, species);
  engine_ = model_->get_engine(model_->effective_spline(spline));
  engine_->prepare_species(t2m_);
  cutoff_ = 0.0;
  for (int a : t2m_)
    for (int b : t2m_) cutoff_ = std::max(cutoff_, model_->model.pair_cutoff(a, b));
  label_ws(ws_);
}

void SystemObj::release()
{
  nl_.release();
  ws_ = Workspace{};
  label_ws(ws_);
  have_list_ = false;
  engine_->release_work();
}

void SystemObj::set_owned(int nlocal_, int ninner_)
{
  nlocal = nlocal_ < 0 ? -1 : nlocal_;
  ninner = ninner_ < 0 ? -1 : std::max(ninner_, nlocal);
  have_list_ = false;    // the active ranges belong to the list: rebuilt by the next compute
}

void SystemObj::set_exchange(int n, int nlocal_, int ninner_, const int32_t *send_counts, const int32_t *send_index,
                             const int32_t *recv_counts, const int32_t *recv_index)
{
  exchange.setup(n, nlocal_, send_counts, send_index, recv_counts, recv_index);
  set_owned(nlocal_, ninner_);
}

void SystemObj::compute(int n, const int *types, const double *pos, bool device_in, const double *cell,
                        const unsigned char *pbc, int flags, double *energy, double *virial, double *forces,
                        double *energies, bool device_out)
{
  require_initialized();
  check_flags(flags, *engine_, uq_out);
  if (n < 0) throw InvalidArgument("negative atom count");
  if (n > 0 && (!types || !pos)) throw InvalidArgument("types and positions must be given");
  if (!cell || !pbc) throw InvalidArgument("cell and pbc must be given");
  for (int k = 0; k < 9; k++)
    if (!std::isfinite(cell[k])) throw InvalidArgument("the cell must be finite");
  std::lock_guard<std::mutex> lk(engine_->mu);
  int chunk = chunk_req_ < 0 ? engine_->auto_chunk(n) : chunk_req_;
  for (;;) {
    try {
      compute_once(n, types, pos, device_in, cell, pbc, flags, energy, virial, forces, energies, device_out, chunk);
      last_chunk = (chunk > 0 && chunk < n) ? chunk : 0;
      return;
    } catch (const OutOfMemory &e) {
      // what was half grown is dropped, so the next call starts clean.  A fixed chunksize reports the failure; the
      // automatic one retries with half the pass (from one pass: the power of two below n / 2) down to 512 atoms
      // (python/kk/kk_core.cpp:451-497)
      nl_.release();
      have_list_ = false;
      engine_->release_work();
      if (chunk_req_ >= 0)
        throw OutOfMemory(std::string("failed to allocate device memory with chunksize ") + std::to_string(chunk_req_) +
                          " (chunksize -1 tries smaller ones): " + e.what());
      int next;
      if (chunk > 0 && chunk < n) next = chunk / 2;
      else for (next = 1; (int64_t) next * 2 <= n / 2; next *= 2) {}
      if (next < 512)
        throw OutOfMemory("the structure (" + std::to_string(n) + " atoms) does not fit the GPU memory even with smaller "
                          "chunks (down to 512 atoms): " + e.what());
      chunk = next;
    }
  }
}

void SystemObj::compute_once(int n, const int *types, const double *pos, bool device_in, const double *cell,
                             const unsigned char *pbc, int flags, double *energy, double *virial, double *forces,
                             double *energies, bool device_out, int chunk)
{
  cudaStream_t st = dev().stream;
  const bool eonly = flags & 2, want_e = flags & 1, want_uq = flags & 4;
  timer_.reset();
  timer_.begin(StageTimer::TOTAL);
  const int ns = (int) t2m_.size();
  const int *d_types = types;
  const double *d_pos = pos;
  ws_.flag.ensure(1);
  GB_CUDA(cudaMemsetAsync(ws_.flag.get(), 0, sizeof(int), st));
  if (n > 0) {
    if (!device_in) {
      ws_.types.ensure(n);
      ws_.pos.ensure(3 * (size_t) n);
      GB_CUDA(cudaMemcpyAsync(ws_.types.get(), types, sizeof(int) * n, cudaMemcpyHostToDevice, st));
      GB_CUDA(cudaMemcpyAsync(ws_.pos.get(), pos, sizeof(double) * 3 * n, cudaMemcpyHostToDevice, st));
      d_types = ws_.types.get();
      d_pos = ws_.pos.get();
    }
    ws_.mu.ensure(n);
    ws_.t2m.upload(t2m_);
    GB_LAUNCH(types_to_mu, nblocks(n, 256), 256, 0, d_types, ws_.t2m.get(), ns, ws_.mu.get(), ws_.flag.get(), (long long) n);
  }
  // rebuild when the atoms, cell or pbc changed or an atom moved more than half the skin (kk_core.cpp:691-708); the
  // three device-side checks (types in range, types unchanged, displacements) set bits of one flag, read back once
  bool need = !have_list_ || list_n_ != n || ws_.h_cell.size() != 9 || std::memcmp(ws_.h_cell.data(), cell, 72) != 0 ||
              std::memcmp(ws_.h_pbc.data(), pbc, 3) != 0;
  if (n > 0) {
    if (!need) {
      GB_LAUNCH(types_differ, nblocks(n, 256), 256, 0, d_types, ws_.types_prev.get(), ws_.flag.get(), (long long) n);
      nl_.moved_launch(d_pos, 0.5 * skin_, ws_.flag.get(), 4);
    }
    const int fl = read_int(ws_.flag.get());
    if (fl & 1) throw InvalidArgument("types must be 1 .. len(species)");
    if (fl & 6) need = true;
  }
  if (need) {
    timer_.begin(StageTimer::NL);
    have_list_ = false;
    nl_.build(1, &n, n, d_pos, ws_.mu.get(), cell, pbc, cutoff_ + skin_);
    ws_.h_cell.assign(cell, cell + 9);
    ws_.h_pbc.assign(pbc, pbc + 3);
    if (n > 0) {
      ws_.types_prev.ensure(n);
      GB_CUDA(cudaMemcpyAsync(ws_.types_prev.get(), d_types, sizeof(int) * n, cudaMemcpyDeviceToDevice, st));
    }
    list_n_ = n;
    have_list_ = true;
    rebuilds++;
    if (nlocal >= 0) ranges = engine_->active_ranges(nl_, std::min(nlocal, n), ninner < 0 ? n : std::min(ninner, n), list0_, list1_);
    timer_.end(StageTimer::NL);
  }
  timer_.begin(StageTimer::GEOM);
  float *fv = engine_->bond_forces(nl_.nslots());
  nl_.prepare(d_pos, engine_->rcsq(), model_->model.n_elements, fv);
  timer_.end(StageTimer::GEOM);
  OutputsDev o;
  if (device_out) {
    o.energy = energy;
    o.virial = eonly ? nullptr : virial;
    o.forces = eonly ? nullptr : forces;
    o.energies = want_e ? energies : nullptr;
    if (want_uq) { o.gamma = uq_out.gamma; o.sigma = uq_out.sigma; o.cluster = uq_out.cluster; }
  } else {
    o.energy = ws_.energy.ensure(1);
    if (!eonly && virial) o.virial = ws_.virial.ensure(6);
    if (!eonly && forces) o.forces = ws_.forces.ensure(3 * (size_t) std::max(n, 1));
    if (want_e && energies) o.energies = ws_.energies.ensure(std::max(n, 1));
    if (want_uq) {
      o.gamma = ws_.uq.ensure(3 * (size_t) std::max(n, 1));
      o.sigma = o.gamma + n;
      o.cluster = o.gamma + 2 * (size_t) n;
    }
  }
  engine_->evaluate(nl_, eonly, o, chunk, &timer_, nlocal >= 0 ? &ranges : nullptr);
  if (exchange.active()) {
    if (n != exchange.n()) throw InvalidArgument("the atom count differs from the one the exchange plan was made for");
    exchange.run(eonly ? nullptr : o.forces, o.energy, eonly ? nullptr : o.virial);
  }
  if (!device_out) {
    if (energy) GB_CUDA(cudaMemcpyAsync(energy, o.energy, sizeof(double), cudaMemcpyDeviceToHost, st));
    if (o.virial) GB_CUDA(cudaMemcpyAsync(virial, o.virial, sizeof(double) * 6, cudaMemcpyDeviceToHost, st));
    if (o.forces && n > 0) GB_CUDA(cudaMemcpyAsync(forces, o.forces, sizeof(double) * 3 * n, cudaMemcpyDeviceToHost, st));
    if (o.energies && n > 0) GB_CUDA(cudaMemcpyAsync(energies, o.energies, sizeof(double) * n, cudaMemcpyDeviceToHost, st));
    if (want_uq && n > 0) {
      GB_CUDA(cudaMemcpyAsync(uq_out.gamma, o.gamma, sizeof(double) * n, cudaMemcpyDeviceToHost, st));
      GB_CUDA(cudaMemcpyAsync(uq_out.sigma, o.sigma, sizeof(double) * n, cudaMemcpyDeviceToHost, st));
      GB_CUDA(cudaMemcpyAsync(uq_out.cluster, o.cluster, sizeof(double) * n, cudaMemcpyDeviceToHost, st));
    }
  }
  timer_.end(StageTimer::TOTAL);
  const int fl = n > 0 ? nl_.take_flag() : 0;    // synchronises the stream
  GB_CUDA(cudaStreamSynchronize(st));
  timer_.collect(stage_ms);
  if (fl & 2) {
    have_list_ = false;
    throw InvalidArgument("two atoms at the same position (a bond of length 0): not a physical structure");
  }
}

// ---- engine interface with the caller's list -------------------------------------------------------------------
EngineRunObj::EngineRunObj(std::shared_ptr<ModelObj> m, const std::vector<std::string> &species, int spline, int chunk)
    : model_(std::move(m)), chunk_req_(chunk)
{
  require_initialized();
  t2m_ = species_to_elements(model_->model, species);
  if (model_->model.layers == 3) throw Unsupported("GRACE-3L: the engine interface for callers with their own neighbour lists is not supported");
  engine_ = model_->get_engine(model_->effective_spline(spline));
  engine_->prepare_species(t2m_);
  cutoff_ = 0.0;
  for (int a : t2m_)
    for (int b : t2m_) cutoff_ = std::max(cutoff_, model_->model.pair_cutoff(a, b));
  label_ws(ws_);
}

int EngineRunObj::comm_width() const { return engine_->plan().layers == 2 ? engine_->plan().nI * engine_->plan().cr : 0; }

void EngineRunObj::release()
{
  nl_.release();
  ws_ = Workspace{};
  label_ws(ws_);
  engine_->release_work();
}

void EngineRunObj::run(int nlocal, int nall, const int *d_type, const double *d_x, const int *d_numneigh,
                       const int *d_neighbors, int maxneigh, int flags, const ExchangeHooks &hooks, double *energy,
                       double *virial6, double *d_f, double *d_eatom)
{
  require_initialized();
  if (flags & 4) throw Unsupported("UQ outputs are not provided through the engine interface");
  if (flags & ~7) throw InvalidArgument("unknown compute flag");
  if (nlocal < 0 || nall < nlocal) throw InvalidArgument("nlocal must be in 0 .. nall");
  if (nall > 0 && (!d_type || !d_x)) throw InvalidArgument("types and positions must be given");
  const bool eonly = flags & 2;
  if (!eonly && nall > 0 && !d_f) throw InvalidArgument("the force array must be given");
  std::lock_guard<std::mutex> lk(engine_->mu);
  cudaStream_t st = dev().stream;
  const int n = nall, ns = (int) t2m_.size();
  ws_.flag.ensure(1);
  GB_CUDA(cudaMemsetAsync(ws_.flag.get(), 0, sizeof(int), st));
  ws_.energy.ensure(1);
  ws_.virial.ensure(6);
  OutputsDev o;
  o.energy = ws_.energy.get();
  if (!eonly) {
    o.virial = ws_.virial.get();
    o.forces = d_f;
  }
  if (d_eatom) o.energies = ws_.energies.ensure(std::max(n, 1));
  if (n > 0) {
    ws_.mu.ensure(n);
    ws_.t2m.upload(t2m_);
    GB_LAUNCH(types_to_mu, nblocks(n, 256), 256, 0, d_type, ws_.t2m.get(), ns, ws_.mu.get(), ws_.flag.get(), (long long) n);
    if (read_int(ws_.flag.get()) & 1) throw InvalidArgument("types must be 1 .. len(species)");
  }
  nl_.adopt(nlocal, nall, ws_.mu.get(), d_numneigh, d_neighbors, maxneigh);
  ActiveRanges ranges = engine_->active_ranges(nl_, nlocal, nlocal, list0_, list1_);
  float *fv = engine_->bond_forces(nl_.nslots());
  nl_.prepare(d_x, engine_->rcsq(), model_->model.n_elements, fv);
  const int chunk = chunk_req_ < 0 ? engine_->auto_chunk(std::max(nlocal, 1)) : chunk_req_;
  engine_->evaluate(nl_, eonly, o, chunk, nullptr, &ranges, &hooks);
  if (d_eatom && nlocal > 0) launch_add_f64(o.energies, d_eatom, nlocal);
  if (energy) GB_CUDA(cudaMemcpyAsync(energy, o.energy, sizeof(double), cudaMemcpyDeviceToHost, st));
  if (virial6 && !eonly) GB_CUDA(cudaMemcpyAsync(virial6, o.virial, sizeof(double) * 6, cudaMemcpyDeviceToHost, st));
  const int fl = n > 0 ? nl_.take_flag() : 0;    // synchronises the stream
  GB_CUDA(cudaStreamSynchronize(st));
  if (fl & 2) throw InvalidArgument("two atoms at the same position (a bond of length 0): not a physical structure");
}

// ---- batch -----------------------------------------------------------------------------------------------------
BatchObj::BatchObj(std::shared_ptr<ModelObj> m, const std::vector<std::string> &species, int spline, int chunk)
    : model_(std::move(m)), chunk_req_(chunk)
{
  require_initialized();
  t2m_ = species_to_elements(model_->model, species);
  engine_ = model_->get_engine(model_->effective_spline(spline));
  engine_->prepare_species(t2m_);
  cutoff_ = 0.0;
  for (int a : t2m_)
    for (int b : t2m_) cutoff_ = std::max(cutoff_, model_->model.pair_cutoff(a, b));
  label_ws(ws_);
}

void BatchObj::release()
{
  nl_.release();
  ws_ = Workspace{};
  label_ws(ws_);
  engine_->release_work();
}

void BatchObj::compute(int nsys, const int *natoms, int64_t ntot, const int *types, const double *pos, bool device_io,
                       const double *cell, const unsigned char *pbc, int flags, int64_t max_nall, double *energy,
                       double *virial, double *forces, double *energies)
{
  require_initialized();
  check_flags(flags, *engine_, uq_out);
  if (nsys < 0 || ntot < 0) throw InvalidArgument("negative structure or atom count");
  if (nsys > 0 && (!natoms || !cell || !pbc)) throw InvalidArgument("natoms, cell and pbc must be given");
  if (ntot > 0 && (!types || !pos)) throw InvalidArgument("types and positions must be given");
  int64_t sum = 0;
  for (int s = 0; s < nsys; s++) {
    if (natoms[s] < 0) throw InvalidArgument("negative atom count");
    sum += natoms[s];
  }
  if (sum != ntot) throw InvalidArgument("natoms must sum to the atom count");
  for (int64_t k = 0; k < 9 * (int64_t) nsys; k++)
    if (!std::isfinite(cell[k])) throw InvalidArgument("the cells must be finite");
  if (max_nall <= 0) max_nall = (int64_t) 1 << 21;
  std::lock_guard<std::mutex> lk(engine_->mu);
  int chunk = chunk_req_;
  for (;;) {
    try {
      const int c = chunk < 0 ? engine_->auto_chunk(std::min<int64_t>(ntot, max_nall)) : chunk;
      compute_once(nsys, natoms, ntot, types, pos, device_io, cell, pbc, flags, max_nall, energy, virial, forces,
                   energies, c);
      last_chunk = c;
      if (!keep_buffers) {
        nl_.release();
        engine_->release_work();
      }
      return;
    } catch (const OutOfMemory &e) {
      // smaller passes: max_nall halved down to 16384 atoms, then give up (kk_core.cpp:1456-1483)
      nl_.release();
      engine_->release_work();
      if (max_nall <= 16384) throw OutOfMemory(std::string("the batch does not fit the device memory: ") + e.what());
      max_nall = std::max<int64_t>(16384, max_nall / 2);
      if (chunk > 0) chunk = std::max(512, chunk / 2);
    }
  }
}

void BatchObj::compute_once(int nsys, const int *natoms, int64_t ntot, const int *types, const double *pos,
                            bool device_io, const double *cell, const unsigned char *pbc, int flags, int64_t max_nall,
                            double *energy, double *virial, double *forces, double *energies, int chunk)
{
  cudaStream_t st = dev().stream;
  const bool eonly = flags & 2, want_e = flags & 1, want_uq = flags & 4;
  const int ns = (int) t2m_.size();
  passes = 0;
  host_seconds = 0.0;
  const int *d_types = types;
  const double *d_pos = pos;
  ws_.flag.ensure(1);
  GB_CUDA(cudaMemsetAsync(ws_.flag.get(), 0, sizeof(int), st));
  if (ntot > 0) {
    if (!device_io) {
      ws_.types.ensure(ntot);
      ws_.pos.ensure(3 * (size_t) ntot);
      GB_CUDA(cudaMemcpyAsync(ws_.types.get(), types, sizeof(int) * ntot, cudaMemcpyHostToDevice, st));
      GB_CUDA(cudaMemcpyAsync(ws_.pos.get(), pos, sizeof(double) * 3 * ntot, cudaMemcpyHostToDevice, st));
      d_types = ws_.types.get();
      d_pos = ws_.pos.get();
    }
    ws_.mu.ensure(ntot);
    ws_.t2m.upload(t2m_);
    GB_LAUNCH(types_to_mu, nblocks(ntot, 256), 256, 0, d_types, ws_.t2m.get(), ns, ws_.mu.get(), ws_.flag.get(), (long long) ntot);
    if (read_int(ws_.flag.get()) & 1) throw InvalidArgument("types must be 1 .. len(species)");
  }
  OutputsDev all;
  if (device_io) {
    all.energy = energy;
    all.virial = eonly ? nullptr : virial;
    all.forces = eonly ? nullptr : forces;
    all.energies = want_e ? energies : nullptr;
    if (want_uq) { all.gamma = uq_out.gamma; all.sigma = uq_out.sigma; all.cluster = uq_out.cluster; }
  } else {
    all.energy = ws_.energy.ensure(std::max(nsys, 1));
    if (!eonly && virial) all.virial = ws_.virial.ensure(6 * (size_t) std::max(nsys, 1));
    if (!eonly && forces) all.forces = ws_.forces.ensure(3 * (size_t) std::max<int64_t>(ntot, 1));
    if (want_e && energies) all.energies = ws_.energies.ensure(std::max<int64_t>(ntot, 1));
    if (want_uq) {
      const size_t m = (size_t) std::max<int64_t>(ntot, 1);
      all.gamma = ws_.uq.ensure(3 * m);
      all.sigma = all.gamma + m;
      all.cluster = all.gamma + 2 * m;
    }
  }
  // passes of whole structures with at most max_nall atoms (a single larger structure gets a pass of its own)
  int s0 = 0;
  int64_t a0 = 0;
  bool zero_bond = false;
  while (s0 < nsys) {
    int s1 = s0;
    int64_t na = 0;
    while (s1 < nsys && (s1 == s0 || na + natoms[s1] <= max_nall)) na += natoms[s1++];
    const auto t0 = std::chrono::steady_clock::now();
    nl_.build(s1 - s0, natoms + s0, na, d_pos + 3 * a0, ws_.mu.get() + a0, cell + 9 * (size_t) s0, pbc + 3 * (size_t) s0,
              cutoff_);
    float *fv = engine_->bond_forces(nl_.nslots());
    nl_.prepare(d_pos + 3 * a0, engine_->rcsq(), model_->model.n_elements, fv);
    GB_CUDA(cudaStreamSynchronize(st));
    host_seconds += std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    OutputsDev o;
    o.energy = all.energy ? all.energy + s0 : nullptr;
    o.virial = all.virial ? all.virial + 6 * (size_t) s0 : nullptr;
    o.forces = all.forces ? all.forces + 3 * a0 : nullptr;
    o.energies = all.energies ? all.energies + a0 : nullptr;
    if (want_uq) { o.gamma = all.gamma + a0; o.sigma = all.sigma + a0; o.cluster = all.cluster + a0; }
    engine_->evaluate(nl_, eonly, o, chunk, nullptr);
    if (na > 0 && (nl_.take_flag() & 2)) zero_bond = true;
    passes++;
    s0 = s1;
    a0 += na;
  }
  if (!device_io) {
    if (energy && nsys > 0) GB_CUDA(cudaMemcpyAsync(energy, all.energy, sizeof(double) * nsys, cudaMemcpyDeviceToHost, st));
    if (all.virial && nsys > 0) GB_CUDA(cudaMemcpyAsync(virial, all.virial, sizeof(double) * 6 * nsys, cudaMemcpyDeviceToHost, st));
    if (all.forces && ntot > 0) GB_CUDA(cudaMemcpyAsync(forces, all.forces, sizeof(double) * 3 * ntot, cudaMemcpyDeviceToHost, st));
    if (all.energies && ntot > 0) GB_CUDA(cudaMemcpyAsync(energies, all.energies, sizeof(double) * ntot, cudaMemcpyDeviceToHost, st));
    if (want_uq && ntot > 0) {
      GB_CUDA(cudaMemcpyAsync(uq_out.gamma, all.gamma, sizeof(double) * ntot, cudaMemcpyDeviceToHost, st));
      GB_CUDA(cudaMemcpyAsync(uq_out.sigma, all.sigma, sizeof(double) * ntot, cudaMemcpyDeviceToHost, st));
      GB_CUDA(cudaMemcpyAsync(uq_out.cluster, all.cluster, sizeof(double) * ntot, cudaMemcpyDeviceToHost, st));
    }
  }
  GB_CUDA(cudaStreamSynchronize(st));
  if (zero_bond) throw InvalidArgument("two atoms at the same position (a bond of length 0): not a physical structure");
}

}    // namespace gb
