// GRACE-3L model container: every array of a GRACE-3L kokkos.npz, read and checked as the reference loader does
// (libgrace/src/model_3l.cpp:165-464 for the keys and shapes, :36-154 for the layer graph; container
// libgrace/include/grace/model_3l.h).  The components are name-list driven: spbf_names [A1, A2, A3], prod_names (cp_l
// products), reduce_names, fc_names, eqnorm_names, rmsnorm_names, out1_origins.  Weights stay raw (fp64) next to their
// scalar norm = 1 / sqrt(fan-in), to be folded once by whoever evaluates them.
#pragma once

#include "npz.h"

#include <string>
#include <vector>

namespace gb {

struct Grace3LModel {
  struct Mlp {
    int n_layers = 0;
    bool has_bias = false;
    std::vector<std::vector<double>> W, b;    // [layer][n_in * n_out], [layer][n_out] (empty: no bias)
    std::vector<double> norm;
    std::vector<int> n_in, n_out;
  };
  struct Spbf {    // single-particle basis of a layer: A1 scalar, A2 / A3 couple the message of the layer before
    std::string name;
    bool equivariant = false;
    int n_rad_max = 0, n_rad_basis = 0, lmax = 0, Lmax = 0, p = 0, nfunc = 0, n_lm_ind = 0;
    double rcut = 0.0, inv_avg_n_neigh = 1.0, lin_transform_norm = 1.0, chem_linear_norm = 1.0;
    std::vector<int> l_tile;
    Mlp mlp;
    std::vector<double> lin_transform_W, chem_linear_W, chem_l0_mask, cg_W;
  };
  struct Cpl {     // low-rank product: projections U, V per lm group, then a sparse Clebsch-Gordan couple
    std::string name;
    int rank = 0, nfunc = 0, n_left = 0, n_right = 0, n_groups_left = 0, n_groups_right = 0, n_cg = 0;
    double norm_u = 1.0, norm_v = 1.0;
    std::vector<double> U, V, cg;
    std::vector<int> group_left, group_right, left_ind, right_ind, m_sum_ind, out_l;
  };
  struct ReduceInstr {
    std::string name;
    std::vector<double> W;
    double norm = 1.0;
    int n_in = 0, w_shape = 0, n_conn = 0;
    std::vector<int> collect_ind, w_l_tile, total_sum_ind;
  };
  struct Reduce {
    std::string name;
    int n_out = 0, n_funcs = 0;
    bool only_invar = false, elem_dep = false, has_norm_map = false;
    std::vector<ReduceInstr> instr;
    std::vector<double> norm_map;
  };
  struct Fc {
    std::string name;
    int n_out = 0, n_funcs_left = 0, n_funcs_right = 0, n_in_left = 0, n_in_right = 0, w_shape_left = 0, w_shape_right = 0;
    bool left_coefs = false;
    double norm_left = 1.0, norm_right = 1.0;
    std::vector<double> w_left, w_right, norm_out_factor;
    std::vector<int> w_tile_left, w_tile_right, collect_to, collect_from;
  };
  struct EqNorm {
    std::string name;
    int center_l0 = 0, n_groups = 0, n_out = 0, M = 0;
    double eps = 0.0;
    std::vector<double> affine_weight, degree_weights, l0_mask;
    std::vector<int> expand_index;
  };
  struct RmsNorm {
    std::string name;
    int type = 0, n_out = 0;    // type 1: channel 0 passes, scale has n_out - 1 values
    std::vector<double> scale;
  };

  int n_elements = 0, embedding_size = 0, lmax = 0, nradbase = 0, radial_basis_p = 0;
  double rcut = 0.0, output_scale = 1.0;
  bool has_bond_specific_cutoff = false;
  std::vector<double> bond_cutoff_map, chem_embedding, shift_values;
  std::vector<std::string> element_names, out1_origins;
  std::vector<Spbf> spbf;
  std::vector<Cpl> prod;
  std::vector<Reduce> reduce;
  std::vector<Fc> fc;
  std::vector<EqNorm> eqnorm;
  std::vector<RmsNorm> rmsnorm;
  Mlp energy_mlp;
  int energy_mlp_activation = 0, energy_mlp_origin_n_out = 0, energy_mlp_n_origins = 0;
  int readout_width = 0;    // channels of the densities the readout sums

  // throws ModelError naming the offending array
  static Grace3LModel load(const Npz &z);
  // floats of tensors a layer keeps per atom (X, the products' projections, reduces, message), for memory estimates
  std::string summary() const;
};

}    // namespace gb
