// Model / System / Batch objects behind the C ABI: the device engine of a model (weights and tables, shared by the
// Systems and Batches of the model as in python/kk/kk_core.cpp:199-221, 555-588) and the evaluation drivers
// (System::compute python/kk/kk_core.cpp:802-958, Batch::compute :1276-1504; layer order of GRACE-2L as
// libgrace/src/fused_2l.cpp:988-1091).
#pragma once

#include "comm.h"
#include "kernels.h"
#include "mv_tc.h"
#include "nlist.h"
#include "plan.h"
#include "radial_mlp_tc.h"

#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace gb {

struct State3L;    // device state of a GRACE-3L model (engine3l.cu)

struct LayerEngine {
  const LayerPlan *plan = nullptr;
  DBuf<float> tab, z;
  DBuf<int> itab;            // row / offset tables of every operation
  DBuf<MVItem> items;
  DBuf<ProdTerm> terms;
  int n_itab = 0, n_items = 0, n_terms = 0;
  std::vector<DBuf<float>> fbufs;
  std::vector<MVDev> mv;
  std::vector<ProdDev> prod;
  std::vector<long long> toff;    // offset of each tensor in floats per atom
  long long per_atom = 0, grad_begin = 0, grad_end = 0;
  DBuf<TensorDev> tensors;
  std::vector<TensorDev> tensors_host;
  // the same operations on shared-memory tensors of an atom tile (chain_fused.cu)
  DBuf<MVDev> f_mv;
  DBuf<ProdDev> f_prod;
  DBuf<int2> f_ops, f_zero;
  DBuf<int4> f_save;
  DBuf<int> f_soff, f_tch;
  FusedLayerDev fused{};
  int fused_TA = 0;           // atoms per tile that fit the shared memory (0: the layer does not fit)
  int fused_NG = 2;           // warp groups per CTA the layer runs with (2, or 1 when two would get one atom each)
  long long q_floats = 0;     // floats per atom of the bond-sum tensor
  // tensor-core form of each MV operation on chunk tensors (mv_tc.cu); not ready: the operation runs as mv_kernel
  std::vector<MVTensorCore> mv_tc;
  double tc_flop_share = 0.0;    // share of the layer's MV flops the tensor-core kernel covers
};

// Atoms a domain-decomposed caller wants evaluated, as ranges of the list order: [lo0, hi0) covers the owned atoms
// (energy, last layer), [lo1, hi1) the atoms whose layer-1 outputs the owned atoms read (GRACE-2L); everything else
// is only a neighbour.  nlocal < 0: every atom is owned and the ranges are the whole list.
struct ActiveRanges {
  int nlocal = -1;
  int64_t lo0 = 0, hi0 = 0, lo1 = 0, hi1 = 0;
  // the same sets exactly, as lists of list positions in increasing order (device; the fused path evaluates these,
  // the per-operation path the enclosing ranges)
  const int *list0 = nullptr, *list1 = nullptr;
  int64_t n0 = 0, n1 = 0;
};

// Message exchange of a caller with ghost atoms that are images of its local atoms (GRACE-2L): forward copies the
// message rows of the owners to their ghosts after layer 1, reverse adds the dE/dmsg rows of the ghosts into their
// owners before layer 1 is reversed (Exchange::forward / reverse of the reference's engine interface,
// libgrace/include/grace/kk/grace_2l_kk.h:92-96, libgrace/include/grace/system.h:53-64).  rows: device, [atoms][width]
// fp32; stream: the library's stream, already synchronised when the hook is called - work enqueued on it, or finished
// before the hook returns, is ordered before the library's next kernel.
struct ExchangeHooks {
  void (*forward)(void *user, float *d_rows, int width, void *stream) = nullptr;
  void (*reverse)(void *user, float *d_rows, int width, void *stream) = nullptr;
  void *user = nullptr;
};

// outputs of one evaluation, device pointers (null: not wanted)
struct OutputsDev {
  double *energy = nullptr;      // [nsys]
  double *virial = nullptr;      // [nsys][6]
  double *forces = nullptr;      // [n][3] caller's order
  double *energies = nullptr;    // [n] caller's order
  // UQ (all three or none): extrapolation grade, Mahalanobis distance and cluster per atom, [n] caller's order
  double *gamma = nullptr, *sigma = nullptr, *cluster = nullptr;
};

class Engine {
 public:
  Engine(const GraceModel &m, int spline_n);
  ~Engine();
  const ModelPlan &plan() const { return plan_; }
  bool uq_available() const { return plan_.uq.ready; }
  // Per atom and evaluation (forward and reverse programs of every layer, each once), on the per-operation path:
  // [0] useful flops and [1] algorithmic bytes of the MV operations that run on the tensor cores, [2] / [3] of the
  // products, [4] / [5] of the remaining (per-element) MV operations.  Bytes: every input row once per item or tensor,
  // every output row once (twice when the operation accumulates).
  void dense_stats(double *out6) const;
  // evaluates the structures of the neighbour list nl (positions prepared by nl.prepare); chunk: atoms per pass
  // act (optional): owned atoms and active ranges of a domain-decomposed caller
  void evaluate(NeighborList &nl, bool energy_only, const OutputsDev &out, int chunk, StageTimer *tm,
                const ActiveRanges *act = nullptr, const ExchangeHooks *hooks = nullptr);
  // ranges of the list order that hold the atoms with caller index < nlocal / < ninner (reads back 4 integers)
  ActiveRanges active_ranges(NeighborList &nl, int nlocal, int ninner, DBuf<int> &list0, DBuf<int> &list1);
  // bond-force slots [3 * nslots] the list zeroes for bonds outside the cutoff (grown here)
  float *bond_forces(int64_t nslots) { return fv_.ensure(3 * (size_t) std::max<int64_t>(nslots, 1)); }
  const double *rcsq() const { return rcsq_.get(); }
  // GRACE-3L: builds the radial tables of every pair of these model elements (the species of a System or Batch) once
  void prepare_species(const std::vector<int> &elements);
  int auto_chunk(int64_t n) const;
  void release_work();
  double per_atom_bytes(int64_t n_eval) const;
  std::mutex mu;    // one evaluation at a time per engine

 private:
  ModelPlan plan_;
  LayerEngine L1_, L2_;
  DBuf<double> rcsq_, eW_, eWT_, shift_, lnI_, ln0_;
  DBuf<float> rcf_;
  ReadoutDev readout_{};
  // work buffers
  DBuf<float> arena_, fv_, I_rows_, gI_rows_, rho_rows_, gmsg_slot_;
  float *message_gradient_slots(NeighborList &nl);
  void gather_message_gradients(NeighborList &nl, const float *slots, const ActiveRanges &R);
  DBuf<double> e_atom_, vir_atom_, grho_rows_, sum_scratch_;
  // UQ head: tables, per-atom results in list order, and (GRACE-2L) the layer-1 projection rows and squared norms
  DBuf<double> uq_cen_, uq_icov_, uq_thr_, uq_out_, uq_n2a_, uq_n2b_;
  DBuf<int> uq_ncl_;
  DBuf<int> mu_l0_, mu_l1_;    // elements of the atoms of a domain-decomposed caller's exact lists, by list position
  DBuf<float> uq_z1_;
  UqDev uq_dev_{};
  bool uq_now_ = false;    // the evaluation in progress computes the UQ outputs
  void uq_layer1(const int *mu, int64_t a0, int na, int stride);
  void uq_last(LayerEngine &E, const int *mu, int64_t a0, int na, int stride, int64_t n);
  int arena_NA_ = 0;
  void setup_layer(LayerEngine &E, const LayerPlan &P);
  void setup_fused(LayerEngine &E, const LayerPlan &P);
  bool fused_ = false;        // both layers fit the fused shared-memory kernel
  // Dense-network path of an evaluation.  Large evaluations stream the network operation by operation over chunk
  // tensors in global memory with the FC layers on the tensor cores (atoms are the long GEMM dimension: 128-atom
  // tiles fill an MMA); small ones (too few atom tiles to fill the GPU) and shapes the tensor-core kernel does not
  // cover run as the fused shared-memory kernel.  GRACE_B200_DENSE = fused | tc | ops overrides (ops: every operation
  // as its SIMT kernel).
  enum class Dense { Auto, Fused, Tc, Ops };
  Dense dense_ = Dense::Auto;
  bool tc_ready_ = false;
  int64_t tc_min_atoms_ = 16384;
  DBuf<int> tc_error_;
  bool use_fused(int64_t n_eval) const;
  bool use_tc(int64_t n_eval) const;
  bool tc_now_ = false;       // the evaluation in progress runs eligible MV operations on the tensor cores
  const ExchangeHooks *hooks_ = nullptr;    // of the evaluation in progress
  void call_hook(bool forward);
  // exact radial MLP per bond on the tensor cores instead of the tables (spline N = 0)
  bool exact_ = false;
  RadialMlpTC rad1_, rad2_;
  DBuf<float> xs_, R1_, dR1_, R2_, dR2_;
  // GRACE-2L: forward tensors of layer 1 its reverse pass reads, kept between the passes instead of recomputed
  DBuf<float> l1_saved_;
  bool keep_l1_ = true;
  void evaluate_fused(NeighborList &nl, bool energy_only, int NA, StageTimer *tm, const ActiveRanges &R);
  void evaluate_chunked(NeighborList &nl, bool energy_only, int NA, StageTimer *tm, const ActiveRanges &R);
  void run_fused(LayerEngine &E, int mode, int NA, int a0, int na, const int *mu, const int *ilist, float *saved = nullptr);
  void bind_arena(LayerEngine &E, float *base, int NA);
  void run(LayerEngine &E, const Program &prog, const int *mu, int NA, int stride);
  DBuf<float> arena1_;               // chunk tensors of layer 1 for all of its atoms (GRACE-2L on the per-operation path)
  const float *arena1_bound_ = nullptr;
  int arena1_NA_ = 0;
  LayerDev layer_dev(const LayerEngine &E) const;
  // GRACE-3L (engine3l.cu)
  std::shared_ptr<State3L> s3_;
  void setup_3l();
  void evaluate_3l(NeighborList &nl, bool energy_only, StageTimer *tm);
  void write_outputs(NeighborList &nl, bool energy_only, const OutputsDev &out);
};

struct ModelObj {
  GraceModel model;
  std::string path;
  int spline = 1024;
  std::mutex mu;
  // one engine per radial mode (table intervals, or 0: exact radial MLP), created by the first System / Batch that
  // asks for it and shared by all of them (python/kk/kk_core.cpp:232,268-300 keeps one per (spline, chunksize); the
  // pass size is an argument of every evaluation here, so the key is the spline alone)
  std::map<int, std::shared_ptr<Engine>> engines;
  int64_t setups = 0;
  std::shared_ptr<Engine> get_engine(int spline_n);
  // spline argument of a System / Batch: > 0 table intervals, 0 exact radial MLP, < 0 the value the model was loaded with
  int effective_spline(int spline_arg) const { return spline_arg >= 0 ? spline_arg : spline; }
  // exact radial MLP of layer 1 or 2 on the tensor cores (set up by the first call)
  RadialMlpTC radial_tc[2];
  void radial_exact(int layer, const float *d_x, long long nb, float *d_R, float *d_dR);
};

// where a compute call with the UQ flag leaves gamma, sigma and cluster [atoms] (host or device as the call's other
// outputs); set by the caller before the call
struct UqOutputs {
  double *gamma = nullptr, *sigma = nullptr, *cluster = nullptr;
};

struct Workspace {
  DBuf<double> pos, energy, virial, forces, energies, uq;
  DBuf<int> types, mu, t2m, flag, types_prev;
  std::vector<double> h_cell;
  std::vector<unsigned char> h_pbc;
  std::vector<int> h_natoms;
};

class SystemObj {
 public:
  SystemObj(std::shared_ptr<ModelObj> m, const std::vector<std::string> &species, double skin, int spline, int chunk);
  double cutoff() const { return cutoff_; }
  void compute(int n, const int *types, const double *pos, bool device_in, const double *cell,
               const unsigned char *pbc, int flags, double *energy, double *virial, double *forces, double *energies,
               bool device_out);
  int64_t rebuilds = 0;
  int last_chunk = 0;
  UqOutputs uq_out;
  int nlocal = -1, ninner = -1;    // owned atoms / atoms with layer-1 outputs of a domain-decomposed caller (-1: all)
  ActiveRanges ranges;
  DBuf<int> list0_, list1_;
  void set_owned(int nlocal_, int ninner_);
  // domain decomposition over the library's communicator: as set_owned, and after every evaluation the ghost force rows
  // go back to their owners and energy and virial are summed over the ranks (comm.h)
  void set_exchange(int n, int nlocal_, int ninner_, const int32_t *send_counts, const int32_t *send_index,
                    const int32_t *recv_counts, const int32_t *recv_index);
  Exchange exchange;
  double stage_ms[StageTimer::NSTAGE] = {0, 0, 0, 0, 0};
  void release();
  std::mutex mu;
  const NeighborList &neighbor_list() const { return nl_; }
  bool has_list() const { return have_list_; }

 private:
  void compute_once(int n, const int *types, const double *pos, bool device_in, const double *cell,
                    const unsigned char *pbc, int flags, double *energy, double *virial, double *forces,
                    double *energies, bool device_out, int chunk);
  std::shared_ptr<ModelObj> model_;
  std::shared_ptr<Engine> engine_;
  std::vector<int> t2m_;
  double skin_, cutoff_;
  int chunk_req_;
  NeighborList nl_;
  Workspace ws_;
  StageTimer timer_;
  bool have_list_ = false;
  int64_t list_n_ = -1;
};

class BatchObj {
 public:
  BatchObj(std::shared_ptr<ModelObj> m, const std::vector<std::string> &species, int spline, int chunk);
  double cutoff() const { return cutoff_; }
  void compute(int nsys, const int *natoms, int64_t ntot, const int *types, const double *pos, bool device_io,
               const double *cell, const unsigned char *pbc, int flags, int64_t max_nall, double *energy,
               double *virial, double *forces, double *energies);
  int passes = 0;
  int last_chunk = 0;
  UqOutputs uq_out;
  double host_seconds = 0.0;
  bool keep_buffers = false;
  void release();
  std::mutex mu;

 private:
  void compute_once(int nsys, const int *natoms, int64_t ntot, const int *types, const double *pos, bool device_io,
                    const double *cell, const unsigned char *pbc, int flags, int64_t max_nall, double *energy,
                    double *virial, double *forces, double *energies, int chunk);
  std::shared_ptr<ModelObj> model_;
  std::shared_ptr<Engine> engine_;
  std::vector<int> t2m_;
  double cutoff_;
  int chunk_req_;
  NeighborList nl_;
  Workspace ws_;
};

// The engine interface of MD codes that bring their own neighbour list and ghost atoms (the LAMMPS glue of the
// reference: RunInput / RunOutput / Exchange, libgrace/include/grace/kk/grace_2l_kk.h:87-119): local atoms first, then
// ghosts; a padded neighbour table of the local atoms over all atoms; forces are ADDED to f [nall][3] (ghost rows too:
// the caller returns them to their owners), per-atom energies to eatom [nlocal]; energy and virial of the local atoms
// are returned.  GRACE-2L exchanges its message rows through the caller's hooks.
class EngineRunObj {
 public:
  EngineRunObj(std::shared_ptr<ModelObj> m, const std::vector<std::string> &species, int spline, int chunk);
  double cutoff() const { return cutoff_; }
  int comm_width() const;    // floats per atom the hooks move (0: one-layer model, no exchange)
  void run(int nlocal, int nall, const int *d_type, const double *d_x, const int *d_numneigh, const int *d_neighbors,
           int maxneigh, int flags, const ExchangeHooks &hooks, double *energy, double *virial6, double *d_f,
           double *d_eatom);
  void release();
  std::mutex mu;

 private:
  std::shared_ptr<ModelObj> model_;
  std::shared_ptr<Engine> engine_;
  std::vector<int> t2m_;
  double cutoff_;
  int chunk_req_;
  NeighborList nl_;
  Workspace ws_;
  DBuf<int> list0_, list1_;
};

std::vector<int> species_to_elements(const GraceModel &m, const std::vector<std::string> &species);

}    // namespace gb
