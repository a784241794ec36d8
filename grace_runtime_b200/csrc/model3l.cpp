// Reader of GRACE-3L kokkos.npz files.  Same keys, shapes, index ranges and layer graph as the reference loader
// (libgrace/src/model_3l.cpp:165-464, graph :36-154): a malformed file fails here with the name of the array.
#include "model3l.h"

#include <algorithm>
#include <map>
#include <set>

namespace gb {

namespace {

constexpr int kMaxDim = 1 << 16;
constexpr int kMaxL = 8, kMaxP = 64;
constexpr int kFormatVersion = 2;

std::string num(int64_t v) { return std::to_string(v); }

void want_count(const std::string &key, size_t got, size_t want)
{
  if (got != want) throw bad_array(key, "has " + num((int64_t) got) + " values, expected " + num((int64_t) want));
}

void want_below(const std::string &key, const std::vector<int> &v, int64_t n)
{
  for (size_t q = 0; q < v.size(); q++)
    if (v[q] < 0 || v[q] >= n) throw bad_array(key, "has " + num(v[q]) + " at " + num((int64_t) q) + ", outside [0, " + num(n) + ")");
}

void want_equal(const std::string &key, int64_t got, int64_t want, const std::string &why)
{
  if (got != want) throw bad_array(key, "is " + num(got) + ", expected " + num(want) + " (" + why + ")");
}

std::vector<int64_t> shape_of_rank(const Npz &z, const std::string &key, size_t rank)
{
  const auto s = z.shape(key);
  if (s.size() != rank) throw bad_array(key, "has " + num((int64_t) s.size()) + " dimensions, expected " + num((int64_t) rank));
  for (int64_t d : s)
    if (d < 1 || d > kMaxDim) throw bad_array(key, "has an extent outside [1, " + num(kMaxDim) + "]");
  return s;
}

bool flag(const Npz &z, const std::string &key, int def) { return z.int_in(key, def, 0, 1) != 0; }

int size_key(const Npz &z, const std::string &key) { return z.int_in(key, 0, 1, kMaxDim); }    // required, in [1, kMaxDim]

double cutoff_scalar(const Npz &z, const std::string &key, double def)
{
  if (!z.has(key)) return def;
  const double v = z.real_scalar(key, def);
  if (!(v > 0.0)) throw bad_array(key, "is not a positive cutoff");
  return v;
}

// prefix_n_layers layers prefix_W{i} [n_in, n_out] chained from n_in to n_out, scalar norms prefix_norm{i}, optional
// biases prefix_b{i}
void read_mlp(const Npz &z, const std::string &prefix, Grace3LModel::DenseStack &m, int64_t n_in, int64_t n_out, const std::string &in_why,
              const std::string &out_why)
{
  m.depth = size_key(z, prefix + "_n_layers");
  if (z.has(prefix + "_W" + num(m.depth)))
    throw bad_array(prefix + "_n_layers", "is " + num(m.depth) + ", but the file has " + prefix + "_W" + num(m.depth));
  int64_t prev = n_in;
  for (int i = 0; i < m.depth; i++) {
    const std::string wk = prefix + "_W" + num(i), bk = prefix + "_b" + num(i);
    const auto s = shape_of_rank(z, wk, 2);
    want_equal(wk, s[0], prev, i ? "the columns of " + prefix + "_W" + num(i - 1) : in_why);
    m.weight.push_back(z.reals(wk));
    m.bias.push_back(z.reals(bk, false));
    if (z.has(bk)) {
      want_count(bk, m.bias.back().size(), (size_t) s[1]);
      m.biased = true;
    }
    m.scale.push_back(z.real_scalar(prefix + "_norm" + num(i), 1.0));
    m.fan_in.push_back((int) s[0]);
    m.fan_out.push_back((int) s[1]);
    prev = s[1];
  }
  want_equal(prefix + "_W" + num(m.depth - 1), prev, n_out, out_why);
}

Grace3LModel::BondBasis read_spbf(const Npz &z, const std::string &nm, const Grace3LModel &m)
{
  Grace3LModel::BondBasis s;
  const int nl = m.lmax + 1, nlm = nl * nl;
  s.name = nm;
  s.coupled = flag(z, nm + "_equivariant", 0);
  s.channels = size_key(z, nm + "_n_rad_max");
  s.nbasis = z.int_scalar(nm + "_n_rad_basis", m.nbasis);
  want_equal(nm + "_n_rad_basis", s.nbasis, m.nbasis, "nradbase, the Chebyshev inputs of the radial MLP");
  s.lmax = z.int_scalar(nm + "_lmax", 4);
  want_equal(nm + "_lmax", s.lmax, m.lmax, "the model's lmax");
  s.Lmax = z.int_in(nm + "_Lmax", 4, 0, kMaxL);
  s.env_p = z.int_in(nm + "_p", 5, 1, kMaxP);
  s.cutoff = cutoff_scalar(z, nm + "_rcut", m.cutoff);
  s.inv_neigh = z.real_scalar(nm + "_inv_avg_n_neigh", 1.0);
  s.l_of_lm = z.ints(nm + "_l_tile");
  want_count(nm + "_l_tile", s.l_of_lm.size(), (size_t) nlm);
  want_below(nm + "_l_tile", s.l_of_lm, nl);
  read_mlp(z, nm + "_mlp", s.radial, m.nbasis + 2 * m.embedding, (int64_t) s.channels * nl, "nradbase + 2 embedding_size",
           "n_rad_max (lmax + 1)");
  if (!s.coupled) {
    s.z_weight = z.reals(nm + "_lin_transform_W");
    z.require_shape(nm + "_lin_transform_W", {m.embedding, s.channels});
    s.z_scale = z.real_scalar(nm + "_lin_transform_norm", 1.0);
  } else {
    s.n_coupled = size_key(z, nm + "_nfunc");
    s.n_msg = size_key(z, nm + "_n_lm_ind");
    s.zc_weight = z.reals(nm + "_chem_linear_W");
    z.require_shape(nm + "_chem_linear_W", {m.embedding, s.channels});
    s.zc_scale = z.real_scalar(nm + "_chem_linear_norm", 1.0);
    s.msg_mask = z.reals(nm + "_chem_l0_mask");
    want_count(nm + "_chem_l0_mask", s.msg_mask.size(), (size_t) s.n_msg);
    s.couple = z.reals(nm + "_cg_W");
    z.require_shape(nm + "_cg_W", {(int64_t) nlm * s.n_msg, s.n_coupled});
  }
  return s;
}

Grace3LModel::LowRank read_cpl(const Npz &z, const std::string &nm)
{
  Grace3LModel::LowRank c;
  c.name = nm;
  c.rank = size_key(z, nm + "_rank");
  c.n_out = size_key(z, nm + "_nfunc");
  c.width_l = size_key(z, nm + "_n_left");
  c.width_r = size_key(z, nm + "_n_right");
  c.groups_l = size_key(z, nm + "_n_groups_left");
  c.groups_r = size_key(z, nm + "_n_groups_right");
  c.scale_u = z.real_scalar(nm + "_norm_u", 1.0);
  c.scale_v = z.real_scalar(nm + "_norm_v", 1.0);
  c.U = z.reals(nm + "_U");
  z.require_shape(nm + "_U", {c.groups_l, c.rank, c.width_l});
  c.V = z.reals(nm + "_V");
  z.require_shape(nm + "_V", {c.groups_r, c.rank, c.width_r});
  c.coef = z.reals(nm + "_cg");
  c.nterms = (int) c.coef.size();
  c.group_l = z.ints(nm + "_group_left");
  want_below(nm + "_group_left", c.group_l, c.groups_l);
  c.group_r = z.ints(nm + "_group_right");
  want_below(nm + "_group_right", c.group_r, c.groups_r);
  const struct {
    const char *key;
    std::vector<int> *v;
    int64_t bound;
  } terms[] = {{"_left_ind", &c.term_l, (int64_t) c.group_l.size()},
               {"_right_ind", &c.term_r, (int64_t) c.group_r.size()},
               {"_m_sum_ind", &c.term_out, c.n_out}};
  for (const auto &t : terms) {
    *t.v = z.ints(nm + t.key);
    want_count(nm + t.key, t.v->size(), (size_t) c.nterms);
    want_below(nm + t.key, *t.v, t.bound);
  }
  c.l_of_out = z.ints(nm + "_out_l");
  want_count(nm + "_out_l", c.l_of_out.size(), (size_t) c.n_out);
  want_below(nm + "_out_l", c.l_of_out, kMaxL + 1);
  return c;
}

Grace3LModel::Collect read_reduce(const Npz &z, const std::string &nm, int n_elements)
{
  Grace3LModel::Collect r;
  r.name = nm;
  r.width = size_key(z, nm + "_n_out");
  r.nfuncs = size_key(z, nm + "_n_funcs");
  r.invariant = flag(z, nm + "_only_invar", 0);
  r.per_element = flag(z, nm + "_is_central_atom_type_dependent", 0);
  const int nfo = r.invariant ? 1 : r.nfuncs;
  for (const std::string &src : z.names(nm + "_instruction_names")) {
    Grace3LModel::Source in;
    in.from = src;
    in.width = size_key(z, nm + "_n_in_" + src);
    in.tiles = size_key(z, nm + "_w_shape_" + src);
    const std::string wk = nm + "_reduce_" + src + "_W";
    in.weight = z.reals(wk);
    if (r.per_element) z.require_shape(wk, {n_elements, r.width, in.width, in.tiles});
    else z.require_shape(wk, {r.width, in.width, in.tiles});
    in.scale = z.real_scalar(nm + "_reduce_" + src + "_norm", 1.0);
    in.pick = z.ints(nm + "_collect_ind_" + src);    // range checked against the producer in the graph walk
    in.nconn = (int) in.pick.size();
    in.tile_of = z.ints(nm + "_w_l_tile_" + src);
    want_count(nm + "_w_l_tile_" + src, in.tile_of.size(), (size_t) in.nconn);
    want_below(nm + "_w_l_tile_" + src, in.tile_of, in.tiles);
    in.into = z.ints(nm + "_total_sum_ind_" + src);
    want_count(nm + "_total_sum_ind_" + src, in.into.size(), (size_t) in.nconn);
    want_below(nm + "_total_sum_ind_" + src, in.into, nfo);
    r.sources.push_back(std::move(in));
  }
  r.row_scaled = z.has(nm + "_norm_map");    // the reduce's own key, not the `<name>_norm_*` keys of an RMS norm
  r.row_scale = z.reals(nm + "_norm_map", false);
  if (r.row_scaled) want_count(nm + "_norm_map", r.row_scale.size(), (size_t) nfo);
  return r;
}

Grace3LModel::Mix read_fc(const Npz &z, const std::string &nm)
{
  Grace3LModel::Mix f;
  f.name = nm;
  const std::string p = "fc_" + nm;
  f.width = size_key(z, p + "_n_out");
  f.weighted_left = flag(z, p + "_left_coefs", 0);
  f.w_right = z.reals(p + "_w_right");
  const auto wr = shape_of_rank(z, p + "_w_right", 3);    // [n_out, n_in_right, tiles]
  want_equal(p + "_w_right", wr[0], f.width, p + "_n_out");
  f.in_right = (int) wr[1];
  f.tiles_right = (int) wr[2];
  f.scale_right = z.real_scalar(p + "_norm_right", 1.0);
  f.nf_left = (int) shape_of_rank(z, p + "_w_tile_left", 1)[0];
  f.out_factor = z.reals(p + "_norm_out_factor");
  want_count(p + "_norm_out_factor", f.out_factor.size(), (size_t) f.nf_left);
  f.from = z.ints(p + "_collect_from");
  f.nf_right = (int) f.from.size();
  f.to = z.ints(p + "_collect_to");
  want_count(p + "_collect_to", f.to.size(), (size_t) f.nf_right);
  want_below(p + "_collect_to", f.to, f.nf_left);
  f.tile_right = z.ints(p + "_w_tile_right");
  want_count(p + "_w_tile_right", f.tile_right.size(), (size_t) f.nf_right);
  want_below(p + "_w_tile_right", f.tile_right, f.tiles_right);
  if (f.weighted_left) {
    f.tile_left = z.ints(p + "_w_tile_left");
    f.w_left = z.reals(p + "_w_left");
    const auto wl = shape_of_rank(z, p + "_w_left", 3);
    want_equal(p + "_w_left", wl[0], f.width, p + "_n_out");
    f.in_left = (int) wl[1];
    f.tiles_left = (int) wl[2];
    f.scale_left = z.real_scalar(p + "_norm_left", 1.0);
    want_below(p + "_w_tile_left", f.tile_left, f.tiles_left);
  }
  return f;
}

Grace3LModel::MessageNorm read_eqnorm(const Npz &z, const std::string &nm)
{
  Grace3LModel::MessageNorm e;
  e.name = nm;
  e.gain = z.reals(nm + "_affine_weight");
  const auto aw = shape_of_rank(z, nm + "_affine_weight", 2);
  e.groups = (int) aw[0];
  e.width = (int) aw[1];
  e.degree_weight = z.reals(nm + "_degree_weights");
  e.nfuncs = (int) e.degree_weight.size();
  e.centre_mask = z.reals(nm + "_l0_mask");
  want_count(nm + "_l0_mask", e.centre_mask.size(), (size_t) e.nfuncs);
  e.group_of = z.ints(nm + "_expand_index");
  want_count(nm + "_expand_index", e.group_of.size(), (size_t) e.nfuncs);
  want_below(nm + "_expand_index", e.group_of, e.groups);
  e.eps = z.real_scalar(nm + "_eps", 1e-8);
  if (e.eps < 0.0) throw bad_array(nm + "_eps", "is negative");
  e.centred = flag(z, nm + "_center_l0", 1);
  return e;
}

Grace3LModel::DensityNorm read_rmsnorm(const Npz &z, const std::string &nm)
{
  Grace3LModel::DensityNorm r;
  r.name = nm;
  r.gain = z.reals(nm + "_scale");
  r.skip_first = flag(z, nm + "_type", 0);
  r.width = z.int_in(nm + "_n_out", (int) std::min<size_t>(r.gain.size() + r.skip_first, kMaxDim), 1, kMaxDim);
  want_count(nm + "_scale", r.gain.size(), (size_t) (r.width - r.skip_first));
  return r;
}

// The layer graph, resolved by name.  Every component is looked up once, checked against the functions and channels
// of its inputs, and marked; a component missing from its name list, listed twice or left over is an error.
class Graph {
 public:
  explicit Graph(Grace3LModel &m) : m_(m) {}

 private:
  struct Shape {
    int nf, nc;
  };

  template<class V> auto &take(V &vec, const char *list, const std::string &name)
  {
    int at = -1;
    for (size_t i = 0; i < vec.size(); i++)
      if (vec[i].name == name) {
        if (at >= 0) throw bad_array(list, "lists '" + name + "' twice");
        at = (int) i;
      }
    if (at < 0) throw bad_array(list, "has no '" + name + "', a part of the GRACE-3L architecture");
    used_.insert(std::string(list) + "/" + name);
    return vec[at];
  }

  template<class V> void leftovers(const V &vec, const char *list) const
  {
    for (const auto &c : vec)
      if (!used_.count(std::string(list) + "/" + c.name))
        throw bad_array(list, "lists '" + c.name + "', not a part of the GRACE-3L architecture");
  }

 public:
  int walk(bool has_origin_n_out)
  {
    if (m_.bases.size() != 3) throw bad_array("spbf_names", "has " + num((int64_t) m_.bases.size()) + " names, expected 3 (A1, A2, A3)");
    const int nlm = (m_.lmax + 1) * (m_.lmax + 1);
    for (int k = 1; k <= 3; k++) {
      const std::string ks = num(k), K = "A" + ks;
      auto &s = take(m_.bases, "spbf_names", K);
      if (m_.bases[k - 1].name != K) throw bad_array("spbf_names", "lists '" + K + "' out of order");
      std::string X = K;
      if (k == 1) {
        if (s.coupled) throw bad_array(K + "_equivariant", "is 1, expected 0 (the first layer has no message to couple)");
        shape_[K] = {nlm, s.channels};
      } else {
        if (!s.coupled) throw bad_array(K + "_equivariant", "is 0, expected 1 (the layer couples the message of the one before)");
        const std::string msg = "eq" + num(k - 1) + "_norm";
        want_equal(K + "_n_lm_ind", s.n_msg, shape_.at(msg).nf, "the functions of the message " + msg);
        want_equal(K + "_n_rad_max", s.channels, shape_.at(msg).nc, "the channels of the message " + msg);
        shape_[K] = {s.n_coupled, s.channels};
        reduce(K + "_red", {K});
        X = K + "_red";
      }
      product(K + "_2", X, X);
      reduce(K + "_2_red", {K + "_2"});
      dense(K + "_2a", K + "_2_red", X);
      product(K + "_3", K + "_2a", X);
      reduce(K + "_3_red", {K + "_3"});
      dense(K + "_2b", K + "_2_red", X);
      product(K + "_4", K + "_2b", K + "_2b");
      reduce(K + "_4_red", {K + "_4"});
      const std::vector<std::string> collected = {X, K + "_2_red", K + "_3_red", K + "_4_red"};
      if (k < 3) {
        reduce("eq" + ks, collected);
        auto &e = take(m_.message_norms, "eqnorm_names", "eq" + ks + "_norm");
        const Shape in = shape_.at("eq" + ks);
        want_equal(e.name + "_degree_weights", e.nfuncs, in.nf, "the functions of eq" + ks);
        want_equal(e.name + "_affine_weight", e.width, in.nc, "the channels of eq" + ks);
        shape_[e.name] = {e.nfuncs, e.width};
      }
      reduce("rho" + ks, collected);
      auto &n = take(m_.density_norms, "rmsnorm_names", "rho" + ks + "_norm");
      const Shape in = shape_.at("rho" + ks);
      want_equal(n.name + "_n_out", n.width, in.nc, "the channels of rho" + ks);
      shape_[n.name] = {in.nf, n.width};
    }
    leftovers(m_.bases, "spbf_names");
    leftovers(m_.products, "prod_names");
    leftovers(m_.collects, "reduce_names");
    leftovers(m_.mixes, "fc_names");
    leftovers(m_.message_norms, "eqnorm_names");
    leftovers(m_.density_norms, "rmsnorm_names");

    const std::vector<std::string> origins = {"rho1_norm", "rho2_norm", "rho3_norm"};
    same_names("out1_origins", m_.readout_inputs, origins);
    const int w = shape_.at(origins[0]).nc;
    for (const auto &o : origins) want_equal(o + "_n_out", shape_.at(o).nc, w, "the channels of " + origins[0]);
    if (has_origin_n_out) want_equal("energy_mlp_origin_n_out", m_.readout_origin_width, w, "the channels of out1_origins");
    return w;
  }

 private:
  static void same_names(const std::string &key, std::vector<std::string> got, std::vector<std::string> want)
  {
    std::sort(got.begin(), got.end());
    std::sort(want.begin(), want.end());
    if (got != want) {
      std::string w;
      for (const auto &s : want) w += (w.empty() ? "" : ", ") + s;
      throw bad_array(key, "must name exactly: " + w);
    }
  }

  void reduce(const std::string &name, const std::vector<std::string> &inputs)
  {
    auto &r = take(m_.collects, "reduce_names", name);
    std::vector<std::string> got;
    for (const auto &in : r.sources) got.push_back(in.from);
    same_names(name + "_instruction_names", got, inputs);
    for (const auto &in : r.sources) {
      const Shape src = shape_.at(in.from);
      want_equal(name + "_n_in_" + in.from, in.width, src.nc, "the channels of " + in.from);
      want_below(name + "_collect_ind_" + in.from, in.pick, src.nf);
    }
    shape_[name] = {r.invariant ? 1 : r.nfuncs, r.width};
  }

  void product(const std::string &name, const std::string &left, const std::string &right)
  {
    auto &c = take(m_.products, "prod_names", name);
    const Shape l = shape_.at(left), r = shape_.at(right);
    want_equal(name + "_group_left", (int64_t) c.group_l.size(), l.nf, "the functions of " + left);
    want_equal(name + "_n_left", c.width_l, l.nc, "the channels of " + left);
    want_equal(name + "_group_right", (int64_t) c.group_r.size(), r.nf, "the functions of " + right);
    want_equal(name + "_n_right", c.width_r, r.nc, "the channels of " + right);
    shape_[name] = {c.n_out, c.rank};
  }

  void dense(const std::string &name, const std::string &left, const std::string &right)
  {
    auto &f = take(m_.mixes, "fc_names", name);
    const std::string p = "fc_" + name;
    const Shape l = shape_.at(left), r = shape_.at(right);
    want_equal(p + "_w_tile_left", f.nf_left, l.nf, "the functions of " + left);
    if (f.weighted_left) want_equal(p + "_w_left", f.in_left, l.nc, "the channels of " + left);
    else want_equal(p + "_n_out", f.width, l.nc, "the channels of " + left + ", which pass unweighted");
    want_equal(p + "_w_right", f.in_right, r.nc, "the channels of " + right);
    want_below(p + "_collect_from", f.from, r.nf);
    shape_[name] = {f.nf_left, f.width};
  }

  Grace3LModel &m_;
  std::map<std::string, Shape> shape_;
  std::set<std::string> used_;
};

}    // namespace

Grace3LModel Grace3LModel::load(const Npz &z)
{
  Grace3LModel m;
  if (z.has("grace_model_kind")) {
    const auto k = z.names("grace_model_kind");
    if (k.size() != 1) throw bad_array("grace_model_kind", "must hold one name");
    if (k[0] != "GRACE-3L") throw ModelError("GRACE-3L: the file holds a " + k[0] + " model");
    if (z.int_scalar("grace_format_version", 0) < 1)
      throw bad_array("grace_format_version", "is missing or below 1 next to grace_model_kind");
  }
  if (z.int_scalar("grace_format_version", 0) > kFormatVersion)
    throw ModelError("GRACE-3L: kokkos.npz format " + num(z.int_scalar("grace_format_version", 0)) + ", this library reads up to " +
                     num(kFormatVersion));
  for (const char *k : {"energy_mlp_scale", "radial_activation", "energy_rms_norm", "AAA_right_A"})
    if (z.has(k)) throw bad_array(k, "is a legacy GRACE-1L/2L key, not supported in GRACE-3L");

  m.n_elements = size_key(z, "n_elements");
  m.embedding = z.int_in("embedding_size", 64, 1, kMaxDim);
  m.nbasis = z.int_in("nradbase", 10, 1, kMaxDim);
  m.lmax = z.int_in("lmax", z.int_in("A1_lmax", 4, 0, kMaxL), 0, kMaxL);    // no bare lmax key in an export: A1_lmax
  m.cutoff = cutoff_scalar(z, "rcut", 6.0);
  m.pair_cutoffs_given = flag(z, "has_bond_specific_cutoff", 0);
  m.embedding_table = z.reals("chem_embedding");
  z.require_shape("chem_embedding", {m.n_elements, m.embedding});
  m.energy_shift = z.reals("shift_values");
  want_count("shift_values", m.energy_shift.size(), (size_t) m.n_elements);
  m.energy_scale = z.real_scalar("output_scale", 1.0);
  m.elements = z.names("element_names");
  want_count("element_names", m.elements.size(), (size_t) m.n_elements);
  m.pair_cutoff = z.reals("bond_cutoff_map", false);
  for (double c : m.pair_cutoff)
    if (c < 0.0) throw bad_array("bond_cutoff_map", "holds a negative cutoff");
  z.require_shape("bond_cutoff_map", {m.n_elements, m.n_elements});
  if (m.pair_cutoff.empty()) m.pair_cutoff.assign((size_t) m.n_elements * m.n_elements, m.cutoff);

  for (const auto &nm : z.names("spbf_names")) m.bases.push_back(read_spbf(z, nm, m));
  if (!m.bases.empty()) m.env_p = m.bases[0].env_p;
  for (const auto &s : m.bases)    // one envelope order for all layers
    if (s.env_p != m.env_p)
      throw bad_array(s.name + "_p", "is " + num(s.env_p) + ", the envelope order of " + m.bases[0].name + " is " + num(m.env_p) +
                                         "; layers with different orders are not supported");
  for (const auto &nm : z.names("prod_names")) m.products.push_back(read_cpl(z, nm));
  for (const auto &nm : z.names("reduce_names")) m.collects.push_back(read_reduce(z, nm, m.n_elements));
  for (const auto &nm : z.names("fc_names")) m.mixes.push_back(read_fc(z, nm));
  for (const auto &nm : z.names("eqnorm_names")) m.message_norms.push_back(read_eqnorm(z, nm));
  for (const auto &nm : z.names("rmsnorm_names")) m.density_norms.push_back(read_rmsnorm(z, nm));

  m.readout_inputs = z.names("out1_origins");
  m.readout_origin_width = z.int_scalar("energy_mlp_origin_n_out", 0);
  m.readout_n_origins = z.int_scalar("energy_mlp_n_origins", (int) m.readout_inputs.size());
  want_equal("energy_mlp_n_origins", m.readout_n_origins, (int64_t) m.readout_inputs.size(), "the names in out1_origins");

  m.readout_width = Graph(m).walk(z.has("energy_mlp_origin_n_out"));
  read_mlp(z, "energy_mlp", m.readout, m.readout_width - 1, 1, "the channels of out1_origins but the linear channel 0",
           "one energy per atom");
  m.readout_act = z.int_in("energy_mlp_activation", 0, 0, 1);
  return m;
}

std::string Grace3LModel::summary() const
{
  std::string s = "GRACE-3L: " + num(n_elements) + " elements, lmax " + num(lmax) + ", channels";
  for (const auto &b : bases) s += " " + num(b.channels);
  s += ", message functions";
  for (const auto &e : message_norms) s += " " + num(e.nfuncs);
  s += ", coupled functions";
  for (const auto &b : bases)
    if (b.coupled) s += " " + num(b.n_coupled);
  s += ", cp_l terms";
  for (const auto &c : products) s += " " + num(c.nterms);
  s += ", readout width " + num(readout_width);
  return s;
}

}    // namespace gb
