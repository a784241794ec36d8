// Execution plan of a model: the dense per-atom network of each layer as a list of two kinds of table-driven
// operations on [function][atom][channel] tensors, with the pruning of outputs nothing reads that the reference
// drivers apply (libgrace/src/fused_1l.cpp:176-214, libgrace/src/fused_2l.cpp:292-351), plus the radial tables.
//
//   MV   out[row] (+)= sum_items scale * M_item^T x[item.src][item.irow]        (FC, reduce and their adjoints)
//   PROD out[row] (+)= sum_terms coef * A[term.a] * B[term.b]  (channel-wise)    (CG products, YI, their adjoints)
//
// Weights are fp32 with the norms folded in (as the reference packs them: libgrace/include/grace/fused_cpu.h:1131-1142,
// 1229-1243).
#pragma once

#include "model.h"

#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace gb {

struct TensorSpec {
  std::string name;
  int nfuncs = 0, channels = 0;
  bool grad = false;    // zeroed before the reverse pass of a chunk
  int alias = -1;       // gradient only: a value tensor of the same shape that no reverse operation reads, whose
                        // storage the gradient may take over once the forward pass is done
  bool external = false;    // written or read outside the program (bond kernels, readout): every row is kept
};

struct MVItem {
  int mat;      // offset (floats) of the [n_in][n_out] matrix in the weight buffer (within the element's block)
  int src;      // tensor id of the input
  int irow;     // function of the input
  int n_in;
  float scale;
};

struct MVOp {
  std::string name;
  int dst = -1;
  int n_out = 0;
  int ldw = 0;                 // row stride of the weight matrices: n_out rounded up to a multiple of 4
  bool accumulate = false;
  bool elem = false;           // weights per central element: matrix at mu * ty_stride + item.mat
  int64_t ty_stride = 0;
  std::vector<int> row_out;    // output function of each row
  std::vector<int> item_off;   // rows + 1
  std::vector<MVItem> items;
  std::vector<float> W;
  // the same work ordered by weight matrix for the fused kernel: a unit is one matrix (a block of 32 of its output
  // channels) applied to up to a few input rows; units of one slot never write the same output row, slots run one
  // after the other (slot = position of an item in its row).  Per unit 5 ints: mat, n_in, k0, first entry, end entry;
  // an entry is an MVItem whose `mat` field holds the OUTPUT row.  Empty for per-element weights or n_in > 64.
  std::vector<int> unit_desc, slot_off;
  std::vector<MVItem> unit_ent;
  double flops_per_atom() const;
};

struct ProdTerm {
  int a, b;
  float coef;
};

struct ProdOp {
  std::string name;
  int dst = -1, srcA = -1, srcB = -1;    // srcB < 0: out = sum coef * A[a]
  bool accumulate = false;
  std::vector<int> row_out;
  std::vector<int> term_off;
  std::vector<ProdTerm> terms;
  std::vector<int> row_first;    // accumulating operation: 1 for the rows it is the first to touch (written, not added to); empty: none
};

struct Op {
  enum Kind { MV, PROD } kind;
  int index;    // into mv / prod
};

// one direction (forward or reverse) of the dense network of a layer
struct Program {
  std::vector<Op> ops;
};

struct RadialTable {
  int N = 0, nl = 0, C = 0;
  std::vector<float> tab;    // [N][nl][C][4]: cubic Hermite coefficients per interval
};

struct LayerPlan {
  std::vector<TensorSpec> tensors;
  std::vector<MVOp> mv;
  std::vector<ProdOp> prod;
  Program fwd, bwd;
  bool zero_grads = true;   // some gradient row has no writing operation: the drivers clear the gradients before the
                            // reverse pass (otherwise the first operation on a row writes it: plan.cpp first_writers)
  int tQ = -1, tGQ = -1;    // the bond-sum tensor written by the forward bond kernel and its gradient
  int n_msg = 0;            // message functions of the neighbours coupled in (layer 2: I_n_funcs; layer 1: 0)
  int C = 0;                // channels of the bond sum
  RadialTable radial;
  std::vector<float> z;     // [n_elements][C] chemical weight of the neighbour (the virtual message function)
  // UQ: index in `mv` of the projection of the layer's invariant basis (the collected inputs of its scalar reduce)
  // onto the rows of the projection matrix that belong to it, and the [1][rp_dim] tensor it writes; -1: no UQ head.
  // The operation is not part of `fwd`: the drivers run it after the forward program when UQ is asked for.
  int uq_mv = -1, tUQ = -1;
};

// Gaussian-mixture part of the UQ head as the device kernels read it (fp64, libgrace/include/grace/fused_cpu.h:1378-1412)
struct UqPlan {
  bool ready = false;
  int rp_dim = 0, feature_dim = 0, n_density = 0, max_clusters = 0;
  double density_scale = 1.0;
  std::vector<double> centroids, inv_cov, thresholds;
  std::vector<int> n_clusters;
};

// One layer of GRACE-3L (libgrace/src/fused_3l.cpp:439-873): the single-particle basis A[f] = sum_q cg[q, f] P[q],
// P[(ly, li)] = sum_j Y_ly R_l(ly) (msg_j[li] + mask[li] zproj[mu_j])  (layer 1: li = 0 only, msg = 0, mask = zproj = 1,
// cg the identity), the dense chain as a LayerPlan (cp_l projections and reduces as MV operations, the couples as
// products, the FCs with an identity on their left input), and the two norms behind its reduces.
struct Layer3Plan {
  LayerPlan dense;
  int C = 0, nfA = 0, nlmi = 1;       // channels, functions of A, message functions coupled in
  int tA = -1, tGA = -1;              // A and its gradient (written / read by the bond kernels)
  int tEQ = -1, tGEQ = -1;            // input of the EquivariantRMSNorm (layers 1, 2) and its gradient
  int tRHO = -1, tGRHO = -1;          // input of the RMSNorm and its gradient
  int nfEQ = 0, cEQ = 0, wr = 0;      // message functions and channels, density width
  std::vector<int> lt;                // l of each lm (selects the radial function)
  std::vector<int> cg_off, cg_p, cgt_off, cgt_f;    // the couple by output function f, and by pair q = ly nlmi + li
  std::vector<float> cg_v, cgt_v;
  std::vector<float> l0mask;          // [nlmi]
  std::vector<float> zproj;           // [n_elements][C]
  std::vector<float> eq_dw, eq_mask, eq_aff;    // [nfEQ], [nfEQ], [groups][cEQ]
  std::vector<int> eq_e;              // [nfEQ] group of each function
  double eq_eps = 0.0;
  int eq_center = 1;
  std::vector<float> rho_scale;       // [wr - n0]
  int rho_n0 = 0;                     // 1: channel 0 passes the norm unchanged
};

struct Plan3L {
  std::shared_ptr<const Grace3LModel> model;    // radial MLPs and embeddings, for the per-pair tables
  Layer3Plan L[3];
  int spline_n = 1024;
  std::vector<double> eW0, eW1;       // energy MLP [wr - 1][nh], [nh]
  double en0 = 1.0, en1 = 1.0;
  int e_nin = 0, e_nh = 0, e_act = 0;
};

// cubic Hermite coefficients [N][nl][C][4] of the radial functions of layer k for the element pair (centre, neighbour)
// (libgrace/src/fused_3l.cpp:307-351, 488-533)
std::vector<float> radial_table_3l(const Grace3LModel &m, int k, int mu_i, int mu_j, int N);

struct ModelPlan {
  int layers = 0, lmax = 0, nlm = 0, n_elements = 0;
  std::vector<double> rcsq;     // [n_elements][n_elements] squared pair cutoffs
  std::vector<double> rc;       // [n_elements][n_elements]
  double rc_max = 0.0;
  LayerPlan L1, L2;
  // tensors of the plans the drivers address by name
  int t1_rho = -1, t1_grho = -1, t1_I = -1, t1_gI = -1;
  int t2_I2 = -1, t2_gI2 = -1;
  int nrho = 0, nI = 0, cr = 0;
  // readout
  std::vector<double> eW;       // energy MLP weights, layers concatenated, [n_in][n_out] each
  std::vector<int> e_nin, e_nout;
  std::vector<double> e_norm;
  int e_act = 0;
  bool e_ln = false, rms = true;
  double out_scale = 1.0;
  std::vector<double> shift;    // [n_elements]
  std::vector<double> lnI, ln0;
  UqPlan uq;
  std::shared_ptr<Plan3L> p3;   // GRACE-3L
  double dense_flops_per_atom = 0.0;    // FC / reduce / product flops of the forward and reverse programs (diagnostics)
};

ModelPlan build_plan(const GraceModel &m, int spline_n);

}    // namespace gb
