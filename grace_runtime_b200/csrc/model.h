// Host-side (fp64) container of a GRACE-1L / GRACE-2L model read from a kokkos.npz file.
// Mirrors what the reference loaders GRACE1LModel::load_arrays (libgrace/src/model_1l.cpp:18-273) and
// GRACE2LModel::load_arrays (libgrace/src/model_2l.cpp:28-400) read and check; a file with max_order 3 simply has no
// fourth-order stage here (the reference adds a dead one, libgrace/src/max_order3.h:122-134, with identical results).
#pragma once

#include "model3l.h"
#include "npz.h"

#include <memory>
#include <string>
#include <vector>

namespace gb {

struct MlpLayer {
  std::vector<double> W;    // [n_in][n_out]
  double norm = 1.0;
  int n_in = 0, n_out = 0;
};

// out[f] = nof[f] (norm_l W_l[:, :, tile_l[f]] . Xl[f] + sum_{c: to[c] = f} norm_r W_r[:, :, tile_r[c]] . Xr[from[c]])
struct FCWeights {
  bool present = false;
  std::vector<double> w_left, w_right;    // [n_out][n_in][tiles]
  std::vector<int> tile_left, tile_right, collect_to, collect_from;
  std::vector<double> nof;
  double norm_left = 1.0, norm_right = 1.0;
  int n_out = 0, n_in_left = 0, n_in_right = 0, tiles_left = 0, tiles_right = 0, n_funcs = 0;
};

// out[m_sum[t]] += cg[t] L[left[t]] R[right[t]] (channel-wise)
struct CGProduct {
  bool present = false;
  std::vector<int> left, right, m_sum;
  std::vector<double> cg;
  int n_out = 0;
};

// out[fo[c]] += norm W[mu?][:, :, tile[c]] . X[collect[c]]
struct ReduceWeights {
  bool present = false;
  std::vector<double> W;    // [n_elements?][n_out][n_in][w_shape]
  double norm = 1.0;
  int n_in = 0, w_shape = 0, n_out = 0;
  bool elem = false;
  std::vector<int> collect, tile, fo;
};

// X0 -> X1 = FC(X0, X0) -> XX = X1 x X1 -> XX1 = FC(XX, X0) -> XXX = XX1 x (X0 | X1) -> XX2 = FC(XX, X0)
// -> XXXX = XX2 x XX2; the chain of layer 1 (A ...) and of layer 2 (B ...)
struct Chain {
  int n0 = 0;          // functions of X0
  int c0 = 0, cf = 0;  // channels of X0 and of the FC outputs
  FCWeights fc1, fcXX1, fcXX2;
  CGProduct pXX, pXXX, pXXXX;
  bool xxx_right_x0 = true;    // XXX = XX1 x X0 (false: x X1, the current GRACE-1L models)
  bool order4 = false;
};

struct YICoupling {
  std::vector<int> y, i, m_sum;
  std::vector<double> cg;
  int n_out = 0;
  double inv_avg = 1.0;
};

// UQ head of schema 6 (libgrace/include/grace/uq_head.h:16-33): the Gaussian-mixture feature of an atom is
// phi = concat((B / |B|) R, log-norm density channels), B the collected inputs of the model's scalar reduces.
// A head that fails its checks leaves the model usable without UQ: the message is kept and raised when UQ is asked for
// (libgrace/src/model_1l.cpp:216-272).
struct UqHead {
  bool present = false;      // uq_schema_version != 0
  int schema = 0;
  std::string error;         // why the head cannot be evaluated (empty: it can)
  int rp_dim = 0, feature_dim = 0, n_density = 0, max_clusters = 0, d_basis = 0;
  double density_scale = 1.0;
  std::vector<double> R;              // [d_basis][rp_dim]
  std::vector<double> centroids;      // [n_elements][max_clusters][feature_dim]
  std::vector<double> inv_cov;        // [n_elements][max_clusters][feature_dim][feature_dim]
  std::vector<double> thresholds;     // [n_elements][max_clusters]
  std::vector<int> n_clusters;        // [n_elements]
};

struct GraceModel {
  int layers = 0;
  int n_elements = 0, embedding = 0, lmax = 0, nradbase = 0, p = 0, max_order = 4;
  double rcut = 0.0;
  bool bond_specific = false;
  std::vector<double> bond_cutoff;    // [n_elements][n_elements]
  std::vector<std::string> element_names;
  std::vector<double> chem;           // [n_elements][embedding]
  int radial_activation = 0, energy_activation = 0;
  bool energy_ln = false;
  std::vector<MlpLayer> energy_mlp;
  double output_scale = 1.0;
  std::vector<double> shift;
  bool has_uq = false;
  UqHead uq;
  // throws ModelError unless the UQ head is there and can be evaluated (GRACE1LModel::validate_uq,
  // libgrace/src/model_1l.cpp:275-285; GRACE2LModel::validate_uq, libgrace/src/model_2l.cpp:464-478)
  void validate_uq() const;
  int uq_basis_width() const;    // rows the projection matrix must have: the collected inputs of the scalar reduces

  // layer 1 (GRACE-1L: the only layer)
  std::vector<MlpLayer> rad1;
  std::vector<double> zA;             // [n_elements][c1], the folded chemical weight of the neighbour
  Chain chain1;
  int rho_n_out = 0;
  ReduceWeights rho[4];               // sources X0, XX, XXX, XXXX of chain1

  // GRACE-2L
  std::vector<MlpLayer> rad2;
  std::vector<double> zB0;            // [n_elements][cr]
  int cr = 0, nI1 = 0, nI = 0, i1_out = 0, nB = 0, nI2 = 0;
  ReduceWeights I1[4], I_from_I1, B_from_YI, B_from_B0, I2[4];
  YICoupling yi;
  Chain chain2;
  bool rms = true;
  std::vector<double> lnI, ln0;

  // GRACE-3L: the whole model (the fields above hold only what Systems and the neighbour list read)
  std::shared_ptr<Grace3LModel> m3;

  double pair_cutoff(int mu_i, int mu_j) const
  {
    return bond_specific ? bond_cutoff[(size_t) mu_i * n_elements + mu_j] : rcut;
  }
  int element_index(const std::string &name) const;
  static GraceModel load(const std::string &path);
};

// kind of the file: 1, 2 or 3 layers (grace_model_kind, else by member names: libgrace/src/model_kind.cpp:111-134)
int model_layers_of_file(const Npz &z);

}    // namespace gb
