// Host-side container of a GRACE-3L model as read from its kokkos.npz file, in this library's own terms.  A 3L file
// is a set of named components listed by kind (spbf_names, prod_names, reduce_names, fc_names, eqnorm_names,
// rmsnorm_names, out1_origins) which the reader resolves into the fixed three-layer graph and checks array by array, as
// the reference loader does (libgrace/src/model_3l.cpp:36-154 graph, :165-464 arrays).  Every weight array is kept as
// stored (fp64) beside its scalar factor 1 / sqrt(fan-in); whoever evaluates the model folds the factor in once.
//
// Kinds of component and what they compute on [function][channel] tensors of an atom:
//   BondBasis    bond sums of a layer: A1 plain (Y_lm R_l z), A2 / A3 coupling the message of the layer before
//   LowRank      cp_l product: both inputs projected to `rank` channels by a matrix per lm group, then a sparse couple
//   Collect      weighted collection of functions of one or several inputs into output functions (optionally per element)
//   Mix          out = factor (left + W right): the "FC" steps between the products
//   MessageNorm  equivariant RMS norm of a layer's message;  DensityNorm  RMS norm of a layer's density
#pragma once

#include "npz.h"

#include <string>
#include <vector>

namespace gb {

struct Grace3LModel {
  // chain of dense layers h -> scale (W^T h + b), SiLU between them (radial MLPs: with biases; readout: without)
  struct DenseStack {
    int depth = 0;
    bool biased = false;
    std::vector<std::vector<double>> weight, bias;    // per layer [fan_in * fan_out], [fan_out] (empty: none)
    std::vector<double> scale;
    std::vector<int> fan_in, fan_out;
  };

  struct BondBasis {
    std::string name;
    bool coupled = false;                  // couples the message of the layer before (A2, A3)
    int channels = 0, nbasis = 0, lmax = 0, Lmax = 0, env_p = 0;
    int n_coupled = 0, n_msg = 0;          // coupled output functions, message functions read (coupled layers)
    double cutoff = 0.0, inv_neigh = 1.0;
    double z_scale = 1.0, zc_scale = 1.0;
    std::vector<int> l_of_lm;              // radial function of each Y lm
    DenseStack radial;                     // [Chebyshev basis, embedding of the centre, of the neighbour] -> channels (lmax + 1)
    std::vector<double> z_weight;          // plain layer: [embedding][channels], species weight of the neighbour
    std::vector<double> zc_weight;         // coupled layers: [embedding][channels], species term of the message ...
    std::vector<double> msg_mask;          // ... applied to the message functions flagged here [n_msg]
    std::vector<double> couple;            // [(Y lm, message function)][n_coupled] dense coupling matrix
  };

  struct LowRank {
    std::string name;
    int rank = 0, n_out = 0, width_l = 0, width_r = 0, groups_l = 0, groups_r = 0, nterms = 0;
    double scale_u = 1.0, scale_v = 1.0;
    std::vector<double> U, V;              // [groups][rank][width]
    std::vector<double> coef;              // [nterms]
    std::vector<int> group_l, group_r;     // projection group of each input function
    std::vector<int> term_l, term_r, term_out;
    std::vector<int> l_of_out;
  };

  struct Source {                          // one input of a Collect
    std::string from;
    std::vector<double> weight;            // [elements?][width out][width][tiles]
    double scale = 1.0;
    int width = 0, tiles = 0, nconn = 0;
    std::vector<int> pick, tile_of, into;  // per connection: input function, weight tile, output function
  };

  struct Collect {
    std::string name;
    int width = 0, nfuncs = 0;
    bool invariant = false, per_element = false, row_scaled = false;
    std::vector<Source> sources;
    std::vector<double> row_scale;         // factor per output function (when row_scaled)
  };

  struct Mix {
    std::string name;
    int width = 0, nf_left = 0, nf_right = 0, in_left = 0, in_right = 0, tiles_left = 0, tiles_right = 0;
    bool weighted_left = false;
    double scale_left = 1.0, scale_right = 1.0;
    std::vector<double> w_left, w_right, out_factor;
    std::vector<int> tile_left, tile_right, to, from;
  };

  struct MessageNorm {
    std::string name;
    int centred = 0, groups = 0, width = 0, nfuncs = 0;
    double eps = 0.0;
    std::vector<double> gain;              // [groups][width]
    std::vector<double> degree_weight, centre_mask;    // [nfuncs]
    std::vector<int> group_of;             // [nfuncs]
  };

  struct DensityNorm {
    std::string name;
    int skip_first = 0, width = 0;         // skip_first 1: channel 0 passes unchanged, gain has width - 1 values
    std::vector<double> gain;
  };

  int n_elements = 0, embedding = 0, lmax = 0, nbasis = 0, env_p = 0;
  double cutoff = 0.0, energy_scale = 1.0;
  bool pair_cutoffs_given = false;
  std::vector<double> pair_cutoff, embedding_table, energy_shift;
  std::vector<std::string> elements, readout_inputs;
  std::vector<BondBasis> bases;
  std::vector<LowRank> products;
  std::vector<Collect> collects;
  std::vector<Mix> mixes;
  std::vector<MessageNorm> message_norms;
  std::vector<DensityNorm> density_norms;
  DenseStack readout;
  int readout_act = 0, readout_origin_width = 0, readout_n_origins = 0;
  int readout_width = 0;    // channels of the densities the readout sums

  // throws ModelError naming the offending array
  static Grace3LModel load(const Npz &z);
  std::string summary() const;
};

}    // namespace gb
