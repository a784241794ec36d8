// Device-side descriptors and host launchers of the CUDA kernels.  Tensors of the dense network are
// [function][atom of the chunk][channel] fp32; geometry and all sums leaving the network are fp64.
#pragma once

#include "device.h"
#include "plan.h"

namespace gb {

struct TensorDev {
  float *p;
  int C;
};

struct MVDev {
  const int *row_out;
  const int *item_off;
  const MVItem *items;
  const float *W;
  long long ty_stride;
  int n_out, ldw, nrows, accumulate, elem, dst;
  // matrix-major work list (plan.h MVOp::unit_desc); nslots == 0: none
  const int *unit_desc;
  const int *slot_off;
  const MVItem *unit_ent;
  int nslots;
  int n_uniform;     // n_in of the items when they all agree, else 0
  int unit_nmax;     // largest n_in of the units
  int unit_exact;    // 32 or 64 when every n_in, n_out and channel stride of the operation equals it, else 0
  int dst_C;         // channels (row stride) of the output tensor
  int max_row_items; // most items of one output row
};

struct ProdDev {
  const int *row_out;
  const int *term_off;
  const ProdTerm *terms;
  int nrows, accumulate, dst, srcA, srcB;
  const int *row_first;    // accumulating operation: rows flagged 1 are written instead of added to (null: none); the
                           // fused kernel clears its gradients beforehand and may ignore it
};

// the neighbour list of one pass and this call's bond records
struct BondsDev {
  const long long *off;    // [n + 1] slots of the list (built with cutoff + skin)
  const int *cnt;          // [n] bonds inside the cutoff this call, compacted to the front of the atom's slots
  const float4 *rec;       // per slot: bond vector x_j - x_i + S cell (fp32 of the fp64 difference), j in .w
  const int *cslot;        // per compacted bond: the slot it came from
  const int *mu;           // [n] model element of each atom (list order)
  const int *ilist;        // atoms to evaluate, in list order (null: all): position a0 + a of it is chunk atom a
};

// per layer: radial table, chemical weights, messages
struct LayerDev {
  const float *tab;        // [N][nl][C][4]: cubic Hermite coefficients
  const float *z;          // [n_elements][C]
  const float *rc;         // [n_elements][n_elements] pair cutoffs
  const float *msg;        // [n][n_msg][C] message rows of all atoms (layer 2) or null
  float *gmsg;             // [n][n_msg][C] dE/dmsg rows, added to atomically by the reverse bond kernel when gmsg_slot is null
  float *gmsg_slot;        // [list slots][n_msg][C]: each bond's share of dE/dmsg of its neighbour, stored at the bond's slot
                           // and summed per neighbour afterwards through the reverse-bond index (no atomics)
  int N, C, n_msg, n_elements;
  // exact radial MLP instead of the tables: value and d/dx per list slot, [slot][l][C] (null: tables)
  const float *Rex, *dRex;
};

// element of a tensor: p[(f * NA + a) * C + c]; NA: atom stride of the chunk tensors, na <= NA: atoms in use
void launch_mv(const MVDev &op, const TensorDev *tensors, const int *mu, int NA, int na);
// nfA, nfB: functions of the source tensors; nterms: terms of the operation (all staged in shared memory per atom tile)
void launch_prod(const ProdDev &op, const TensorDev *tensors, int NA, int na, int C, int nfA, int nfB, int nterms);

// x[slot] = r / r_cut of the bond compacted into the slot (0.5 for slots without a bond): input of the exact radial MLP
void launch_bond_x(const BondsDev &b, const float *rc, int n_elements, float *x, long long n);

// Q[(I, lm)][a][n] = sum over the bonds of atom a0 + a of Y_lm R[n, l] msg_I[n]
void launch_bond_fwd(int lmax, const BondsDev &b, const LayerDev &L, float *Q, int NA, int a0, int na);
// reverse: per bond dE/dx and dE/dY from gQ -> bond force (written or added at the bond's slot), per-atom virial,
// dE/dmsg rows of the neighbours
void launch_bond_bwd(int lmax, const BondsDev &b, const LayerDev &L, const float *gQ, int NA, int a0, int na,
                     float *fv, double *vir_atom, int add);

struct ReadoutDev {
  const double *W;        // layers concatenated, [n_in][n_out] each
  const double *WT;       // the same layers transposed, [n_out][n_in] each
  const double *shift;    // [n_elements]
  const double *lnI, *ln0;
  int nlay, n_in[4], n_out[4];
  double norm[4];
  int act, ln, rms, nrho;
  double out_scale;
  // owned atoms of a domain-decomposed caller: atoms whose caller index perm[i] is >= nlocal are ghosts, which
  // take part in every neighbour sum but whose own energy (and its gradient seed) is left out (the nlocal / ghost
  // convention of the reference's engine interface, libgrace/include/grace/kk/grace_2l_kk.h:87-107).  perm null: all owned
  const int *perm;
  int nlocal;
  __host__ __device__ bool owned(long long i) const { return perm == nullptr || perm[i] < nlocal; }
};
// GRACE-1L: E_i = (MLP(rho[1:]) + rho[0]) scale + shift, dE/drho
// ilist (optional, here and below): chunk position a0 + a stands for atom ilist[a0 + a] instead of atom a0 + a
void launch_readout_1l(const ReadoutDev &r, const float *rho, float *grho, const int *mu, double *e_atom, int NA,
                       int na, int a0, int want_grad, const int *ilist = nullptr);
// GRACE-2L: rho from the per-atom rows, I2 of the chunk; dE/drho to the per-atom rows, dE/dI2 to the chunk
void launch_readout_2l(const ReadoutDev &r, const float *rho_rows, const float *I2, double *grho_rows, float *gI2,
                       const int *mu, double *e_atom, int NA, int na, int a0, int want_grad, const int *ilist = nullptr);

// ---- UQ head (uq.cu) ----
struct UqDev {
  const double *centroids;     // [n_elements][max_clusters][feature_dim]
  const double *inv_cov;       // [n_elements][max_clusters][feature_dim][feature_dim]
  const double *thresholds;    // [n_elements][max_clusters]
  const int *n_clusters;       // [n_elements]
  int rp_dim, feature_dim, max_clusters, n_density;
  double density_scale;
};
// n2[a] = |B_a|^2 (fp64) over the inputs of the projection operation `op`, a < na atoms of the chunk
void launch_uq_norm(const MVDev &op, const TensorDev *tensors, int NA, int na, double *n2);
// gamma / sigma / cluster of the atoms a0 .. a0 + na (list order) from the projection z [na][rp_dim] of the last layer,
// the rows z_prev [n][rp_dim] and squared norms n2_prev [n] of the layer before (null: one layer) and n2_last [n]
void launch_uq_gmm(const UqDev &u, const float *z, const float *z_prev, const double *n2_last, const double *n2_prev,
                   const int *mu, int na, long long a0, double *gamma, double *sigma, double *cluster);

// ---- the dense network of a layer as one kernel on shared-memory tensors (chain_fused.cu) ----
// FUSED_SAVE: after the forward operations, the tensors the reverse operations read go to global memory;
// FUSED_RESTORE: they come back from there instead of the bond sums and the forward operations being run again
enum { FUSED_STORE_MSG = 1, FUSED_READOUT_1L = 2, FUSED_READOUT_2L = 4, FUSED_BWD = 8, FUSED_LOAD_SEED = 16, FUSED_SAVE = 32,
       FUSED_RESTORE = 64 };

struct FusedLayerDev {
  const MVDev *mv;
  const ProdDev *prod;
  const int2 *ops;      // (kind: 0 MV, 1 PROD; index), forward operations then reverse operations
  int nfwd, nbwd;
  const int *soff;      // per tensor: offset in floats per atom of the tile
  const int *tch;       // per tensor: channels
  const int2 *zero;     // (offset, length) in floats per atom of the gradients cleared before the reverse operations
  int nzero;
  int per_atom;         // shared-memory floats per atom
  // the tables every operation reads (copied to shared memory once per CTA: reading them from global memory is a chain
  // of dependent L2 round trips per operation and tile)
  int nmv, nprod, ntensors;
  const int *itab;      // row_out / item_off / term_off arrays of all operations, contiguous
  const MVItem *items;
  const ProdTerm *terms;
  int n_itab, n_items, n_terms;
  int stage_terms;      // the product terms fit the shared memory next to the tile
  // forward tensors that reverse operations read: (shared-memory offset in floats per atom, functions, channels,
  // offset in the per-atom record), and the floats of a record
  const int4 *save;
  int nsave, save_floats;
  int tab_floats;       // shared-memory floats in front of the tile's tensors that hold the tables
  int stage_ro;         // doubles of the energy MLP (layers concatenated) staged behind the tables, twice (W, WT); 0: none
  int ro_offset;        // byte offset of that copy in the dynamic shared memory
};

struct FusedIO {
  int mode;
  int tQ, tGQ, nQ, CQ;              // bond-sum tensor and its gradient: ids, rows, channels
  const float *Q;                   // global [nQ][NA][CQ]
  float *gQ;
  long long NA;
  int t_rho, t_grho, nrho, t_I, t_gI, nI, CR, t_I2, t_gI2;
  float *I_rows, *rho_rows;         // GRACE-2L per-atom rows [n][nI][CR], [n][nrho]
  const float *gI_rows;
  double *grho_rows;
  ReadoutDev ro;
  const int *mu;                    // [n] elements in list order
  double *e_atom;
  int a0, na;                       // first atom of the chunk in list order (or position in ilist), atoms of the chunk
  const int *ilist;                 // atoms to evaluate (null: all)
  float *saved;                     // [atoms of the evaluation][save_floats]: FUSED_SAVE / FUSED_RESTORE, by position a0 + a
};

// TA: atoms per tile (1, 2, 3, 4, 6, 8); grid CTAs loop over the tiles
void launch_chain_fused(int TA, const FusedLayerDev &L, const FusedIO &io, int grid);       // two groups per CTA
void launch_chain_fused_g1(int TA, const FusedLayerDev &L, const FusedIO &io, int grid);    // one group per CTA

// chunk tensor [nf][NA][C] <-> per-atom rows [n][nf][C] (message I, its gradient) and [n][C] (rho)
void launch_rows_from_chunk(const float *t, float *rows, int nf, int C, int NA, int na, int a0, const int *ilist = nullptr);
void launch_chunk_from_rows(float *t, const float *rows, int nf, int C, int NA, int na, int a0, const int *ilist = nullptr);
void launch_chunk_from_rows_f64(float *t, const double *rows, int nf, int C, int NA, int na, int a0, const int *ilist = nullptr);
// out[a] = v[list[a]], a < n
void launch_gather_int(const int *v, const int *list, int *out, long long n);

// gmsg[j] = sum over the bonds e of atom j inside the cutoff of gslot[rev[slot of e]]: the shares the bonds i -> j stored,
// added in the order of j's own list (bit-reproducible).  width = n_msg * C floats per row.  perm / nlocal (optional):
// bonds whose other atom is a ghost (perm[i] >= nlocal) are left out - its layer was not evaluated, its slots hold nothing
void launch_msg_grad_gather(const BondsDev &b, const int *rev, const float *gslot, float *gmsg, int width, const int *ilist,
                            long long n, const int *perm, int nlocal);
// F_i = sum over the slots q of atom i of fv[q] - fv[rev[q]], written at the caller's index of atom i
void launch_force_gather(const long long *off, const int *rev, const float *fv, const int *perm, double *forces,
                         int n);
// lists without a reverse-bond index (a caller's own list with ghost atoms): forces[i] += sum of the atom's bond forces,
// forces[j] -= each bond force, with fp64 atomic adds (forces is accumulated into, indexed like the list's atoms)
void launch_force_scatter(const BondsDev &b, const float *fv, double *forces, long long n);
// zero fill on the library's stream (a kernel for large aligned buffers, the driver's memset otherwise)
void launch_fill_zero(void *p, size_t bytes);
// out[i] += v[i]
void launch_add_f64(const double *v, double *out, long long n);
// per-structure sums of per-atom values: out[s][k] = sum_{i in [seg[s], seg[s+1])} v[i][k]
// column sums of values[n][K] into out[K] with the partial sums in a static device array: no allocation
// (static_sum.cu); throws InvalidArgument beyond static_sum_max_rows() / static_sum_max_cols()
void static_sum(const double *d_values, long long n, int K, double *d_out);
long long static_sum_max_rows();
int static_sum_max_cols();
// scratch (nseg * K * nb doubles) with nb > 1: two launches with nb partial sums per (segment, component), for few long
// segments
void launch_segment_sum(const double *v, int K, const int *seg, int nseg, double *out, double *scratch = nullptr,
                        int nb = 1);
// out[perm[i]] = v[i]
void launch_scatter_f64(const double *v, const int *perm, double *out, int n);

}    // namespace gb
