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
void read_mlp(const Npz &z, const std::string &prefix, Grace3LModel::Mlp &m, int64_t n_in, int64_t n_out, const std::string &in_why,
              const std::string &out_why)
{
  m.n_layers = size_key(z, prefix + "_n_layers");
  if (z.has(prefix + "_W" + num(m.n_layers)))
    throw bad_array(prefix + "_n_layers", "is " + num(m.n_layers) + ", but the file has " + prefix + "_W" + num(m.n_layers));
  int64_t prev = n_in;
  for (int i = 0; i < m.n_layers; i++) {
    const std::string wk = prefix + "_W" + num(i), bk = prefix + "_b" + num(i);
    const auto s = shape_of_rank(z, wk, 2);
    want_equal(wk, s[0], prev, i ? "the columns of " + prefix + "_W" + num(i - 1) : in_why);
    m.W.push_back(z.reals(wk));
    m.b.push_back(z.reals(bk, false));
    if (z.has(bk)) {
      want_count(bk, m.b.back().size(), (size_t) s[1]);
      m.has_bias = true;
    }
    m.norm.push_back(z.real_scalar(prefix + "_norm" + num(i), 1.0));
    m.n_in.push_back((int) s[0]);
    m.n_out.push_back((int) s[1]);
    prev = s[1];
  }
  want_equal(prefix + "_W" + num(m.n_layers - 1), prev, n_out, out_why);
}

Grace3LModel::Spbf read_spbf(const Npz &z, const std::string &nm, const Grace3LModel &m)
{
  Grace3LModel::Spbf s;
  const int nl = m.lmax + 1, nlm = nl * nl;
  s.name = nm;
  s.equivariant = flag(z, nm + "_equivariant", 0);
  s.n_rad_max = size_key(z, nm + "_n_rad_max");
  s.n_rad_basis = z.int_scalar(nm + "_n_rad_basis", m.nradbase);
  want_equal(nm + "_n_rad_basis", s.n_rad_basis, m.nradbase, "nradbase, the Chebyshev inputs of the radial MLP");
  s.lmax = z.int_scalar(nm + "_lmax", 4);
  want_equal(nm + "_lmax", s.lmax, m.lmax, "the model's lmax");
  s.Lmax = z.int_in(nm + "_Lmax", 4, 0, kMaxL);
  s.p = z.int_in(nm + "_p", 5, 1, kMaxP);
  s.rcut = cutoff_scalar(z, nm + "_rcut", m.rcut);
  s.inv_avg_n_neigh = z.real_scalar(nm + "_inv_avg_n_neigh", 1.0);
  s.l_tile = z.ints(nm + "_l_tile");
  want_count(nm + "_l_tile", s.l_tile.size(), (size_t) nlm);
  want_below(nm + "_l_tile", s.l_tile, nl);
  read_mlp(z, nm + "_mlp", s.mlp, m.nradbase + 2 * m.embedding_size, (int64_t) s.n_rad_max * nl, "nradbase + 2 embedding_size",
           "n_rad_max (lmax + 1)");
  if (!s.equivariant) {
    s.lin_transform_W = z.reals(nm + "_lin_transform_W");
    z.require_shape(nm + "_lin_transform_W", {m.embedding_size, s.n_rad_max});
    s.lin_transform_norm = z.real_scalar(nm + "_lin_transform_norm", 1.0);
  } else {
    s.nfunc = size_key(z, nm + "_nfunc");
    s.n_lm_ind = size_key(z, nm + "_n_lm_ind");
    s.chem_linear_W = z.reals(nm + "_chem_linear_W");
    z.require_shape(nm + "_chem_linear_W", {m.embedding_size, s.n_rad_max});
    s.chem_linear_norm = z.real_scalar(nm + "_chem_linear_norm", 1.0);
    s.chem_l0_mask = z.reals(nm + "_chem_l0_mask");
    want_count(nm + "_chem_l0_mask", s.chem_l0_mask.size(), (size_t) s.n_lm_ind);
    s.cg_W = z.reals(nm + "_cg_W");
    z.require_shape(nm + "_cg_W", {(int64_t) nlm * s.n_lm_ind, s.nfunc});
  }
  return s;
}

Grace3LModel::Cpl read_cpl(const Npz &z, const std::string &nm)
{
  Grace3LModel::Cpl c;
  c.name = nm;
  c.rank = size_key(z, nm + "_rank");
  c.nfunc = size_key(z, nm + "_nfunc");
  c.n_left = size_key(z, nm + "_n_left");
  c.n_right = size_key(z, nm + "_n_right");
  c.n_groups_left = size_key(z, nm + "_n_groups_left");
  c.n_groups_right = size_key(z, nm + "_n_groups_right");
  c.norm_u = z.real_scalar(nm + "_norm_u", 1.0);
  c.norm_v = z.real_scalar(nm + "_norm_v", 1.0);
  c.U = z.reals(nm + "_U");
  z.require_shape(nm + "_U", {c.n_groups_left, c.rank, c.n_left});
  c.V = z.reals(nm + "_V");
  z.require_shape(nm + "_V", {c.n_groups_right, c.rank, c.n_right});
  c.cg = z.reals(nm + "_cg");
  c.n_cg = (int) c.cg.size();
  c.group_left = z.ints(nm + "_group_left");
  want_below(nm + "_group_left", c.group_left, c.n_groups_left);
  c.group_right = z.ints(nm + "_group_right");
  want_below(nm + "_group_right", c.group_right, c.n_groups_right);
  const struct {
    const char *key;
    std::vector<int> *v;
    int64_t bound;
  } terms[] = {{"_left_ind", &c.left_ind, (int64_t) c.group_left.size()},
               {"_right_ind", &c.right_ind, (int64_t) c.group_right.size()},
               {"_m_sum_ind", &c.m_sum_ind, c.nfunc}};
  for (const auto &t : terms) {
    *t.v = z.ints(nm + t.key);
    want_count(nm + t.key, t.v->size(), (size_t) c.n_cg);
    want_below(nm + t.key, *t.v, t.bound);
  }
  c.out_l = z.ints(nm + "_out_l");
  want_count(nm + "_out_l", c.out_l.size(), (size_t) c.nfunc);
  want_below(nm + "_out_l", c.out_l, kMaxL + 1);
  return c;
}

Grace3LModel::Reduce read_reduce(const Npz &z, const std::string &nm, int n_elements)
{
  Grace3LModel::Reduce r;
  r.name = nm;
  r.n_out = size_key(z, nm + "_n_out");
  r.n_funcs = size_key(z, nm + "_n_funcs");
  r.only_invar = flag(z, nm + "_only_invar", 0);
  r.elem_dep = flag(z, nm + "_is_central_atom_type_dependent", 0);
  const int nfo = r.only_invar ? 1 : r.n_funcs;
  for (const std::string &src : z.names(nm + "_instruction_names")) {
    Grace3LModel::ReduceInstr in;
    in.name = src;
    in.n_in = size_key(z, nm + "_n_in_" + src);
    in.w_shape = size_key(z, nm + "_w_shape_" + src);
    const std::string wk = nm + "_reduce_" + src + "_W";
    in.W = z.reals(wk);
    if (r.elem_dep) z.require_shape(wk, {n_elements, r.n_out, in.n_in, in.w_shape});
    else z.require_shape(wk, {r.n_out, in.n_in, in.w_shape});
    in.norm = z.real_scalar(nm + "_reduce_" + src + "_norm", 1.0);
    in.collect_ind = z.ints(nm + "_collect_ind_" + src);    // range checked against the producer in the graph walk
    in.n_conn = (int) in.collect_ind.size();
    in.w_l_tile = z.ints(nm + "_w_l_tile_" + src);
    want_count(nm + "_w_l_tile_" + src, in.w_l_tile.size(), (size_t) in.n_conn);
    want_below(nm + "_w_l_tile_" + src, in.w_l_tile, in.w_shape);
    in.total_sum_ind = z.ints(nm + "_total_sum_ind_" + src);
    want_count(nm + "_total_sum_ind_" + src, in.total_sum_ind.size(), (size_t) in.n_conn);
    want_below(nm + "_total_sum_ind_" + src, in.total_sum_ind, nfo);
    r.instr.push_back(std::move(in));
  }
  r.has_norm_map = z.has(nm + "_norm_map");    // the reduce's own key, not the `<name>_norm_*` keys of an RMS norm
  r.norm_map = z.reals(nm + "_norm_map", false);
  if (r.has_norm_map) want_count(nm + "_norm_map", r.norm_map.size(), (size_t) nfo);
  return r;
}

Grace3LModel::Fc read_fc(const Npz &z, const std::string &nm)
{
  Grace3LModel::Fc f;
  f.name = nm;
  const std::string p = "fc_" + nm;
  f.n_out = size_key(z, p + "_n_out");
  f.left_coefs = flag(z, p + "_left_coefs", 0);
  f.w_right = z.reals(p + "_w_right");
  const auto wr = shape_of_rank(z, p + "_w_right", 3);    // [n_out, n_in_right, tiles]
  want_equal(p + "_w_right", wr[0], f.n_out, p + "_n_out");
  f.n_in_right = (int) wr[1];
  f.w_shape_right = (int) wr[2];
  f.norm_right = z.real_scalar(p + "_norm_right", 1.0);
  f.n_funcs_left = (int) shape_of_rank(z, p + "_w_tile_left", 1)[0];
  f.norm_out_factor = z.reals(p + "_norm_out_factor");
  want_count(p + "_norm_out_factor", f.norm_out_factor.size(), (size_t) f.n_funcs_left);
  f.collect_from = z.ints(p + "_collect_from");
  f.n_funcs_right = (int) f.collect_from.size();
  f.collect_to = z.ints(p + "_collect_to");
  want_count(p + "_collect_to", f.collect_to.size(), (size_t) f.n_funcs_right);
  want_below(p + "_collect_to", f.collect_to, f.n_funcs_left);
  f.w_tile_right = z.ints(p + "_w_tile_right");
  want_count(p + "_w_tile_right", f.w_tile_right.size(), (size_t) f.n_funcs_right);
  want_below(p + "_w_tile_right", f.w_tile_right, f.w_shape_right);
  if (f.left_coefs) {
    f.w_tile_left = z.ints(p + "_w_tile_left");
    f.w_left = z.reals(p + "_w_left");
    const auto wl = shape_of_rank(z, p + "_w_left", 3);
    want_equal(p + "_w_left", wl[0], f.n_out, p + "_n_out");
    f.n_in_left = (int) wl[1];
    f.w_shape_left = (int) wl[2];
    f.norm_left = z.real_scalar(p + "_norm_left", 1.0);
    want_below(p + "_w_tile_left", f.w_tile_left, f.w_shape_left);
  }
  return f;
}

Grace3LModel::EqNorm read_eqnorm(const Npz &z, const std::string &nm)
{
  Grace3LModel::EqNorm e;
  e.name = nm;
  e.affine_weight = z.reals(nm + "_affine_weight");
  const auto aw = shape_of_rank(z, nm + "_affine_weight", 2);
  e.n_groups = (int) aw[0];
  e.n_out = (int) aw[1];
  e.degree_weights = z.reals(nm + "_degree_weights");
  e.M = (int) e.degree_weights.size();
  e.l0_mask = z.reals(nm + "_l0_mask");
  want_count(nm + "_l0_mask", e.l0_mask.size(), (size_t) e.M);
  e.expand_index = z.ints(nm + "_expand_index");
  want_count(nm + "_expand_index", e.expand_index.size(), (size_t) e.M);
  want_below(nm + "_expand_index", e.expand_index, e.n_groups);
  e.eps = z.real_scalar(nm + "_eps", 1e-8);
  if (e.eps < 0.0) throw bad_array(nm + "_eps", "is negative");
  e.center_l0 = flag(z, nm + "_center_l0", 1);
  return e;
}

Grace3LModel::RmsNorm read_rmsnorm(const Npz &z, const std::string &nm)
{
  Grace3LModel::RmsNorm r;
  r.name = nm;
  r.scale = z.reals(nm + "_scale");
  r.type = flag(z, nm + "_type", 0);
  r.n_out = z.int_in(nm + "_n_out", (int) std::min<size_t>(r.scale.size() + r.type, kMaxDim), 1, kMaxDim);
  want_count(nm + "_scale", r.scale.size(), (size_t) (r.n_out - r.type));
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
    if (m_.spbf.size() != 3) throw bad_array("spbf_names", "has " + num((int64_t) m_.spbf.size()) + " names, expected 3 (A1, A2, A3)");
    const int nlm = (m_.lmax + 1) * (m_.lmax + 1);
    for (int k = 1; k <= 3; k++) {
      const std::string ks = num(k), K = "A" + ks;
      auto &s = take(m_.spbf, "spbf_names", K);
      if (m_.spbf[k - 1].name != K) throw bad_array("spbf_names", "lists '" + K + "' out of order");
      std::string X = K;
      if (k == 1) {
        if (s.equivariant) throw bad_array(K + "_equivariant", "is 1, expected 0 (the first layer has no message to couple)");
        shape_[K] = {nlm, s.n_rad_max};
      } else {
        if (!s.equivariant) throw bad_array(K + "_equivariant", "is 0, expected 1 (the layer couples the message of the one before)");
        const std::string msg = "eq" + num(k - 1) + "_norm";
        want_equal(K + "_n_lm_ind", s.n_lm_ind, shape_.at(msg).nf, "the functions of the message " + msg);
        want_equal(K + "_n_rad_max", s.n_rad_max, shape_.at(msg).nc, "the channels of the message " + msg);
        shape_[K] = {s.nfunc, s.n_rad_max};
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
        auto &e = take(m_.eqnorm, "eqnorm_names", "eq" + ks + "_norm");
        const Shape in = shape_.at("eq" + ks);
        want_equal(e.name + "_degree_weights", e.M, in.nf, "the functions of eq" + ks);
        want_equal(e.name + "_affine_weight", e.n_out, in.nc, "the channels of eq" + ks);
        shape_[e.name] = {e.M, e.n_out};
      }
      reduce("rho" + ks, collected);
      auto &n = take(m_.rmsnorm, "rmsnorm_names", "rho" + ks + "_norm");
      const Shape in = shape_.at("rho" + ks);
      want_equal(n.name + "_n_out", n.n_out, in.nc, "the channels of rho" + ks);
      shape_[n.name] = {in.nf, n.n_out};
    }
    leftovers(m_.spbf, "spbf_names");
    leftovers(m_.prod, "prod_names");
    leftovers(m_.reduce, "reduce_names");
    leftovers(m_.fc, "fc_names");
    leftovers(m_.eqnorm, "eqnorm_names");
    leftovers(m_.rmsnorm, "rmsnorm_names");

    const std::vector<std::string> origins = {"rho1_norm", "rho2_norm", "rho3_norm"};
    same_names("out1_origins", m_.out1_origins, origins);
    const int w = shape_.at(origins[0]).nc;
    for (const auto &o : origins) want_equal(o + "_n_out", shape_.at(o).nc, w, "the channels of " + origins[0]);
    if (has_origin_n_out) want_equal("energy_mlp_origin_n_out", m_.energy_mlp_origin_n_out, w, "the channels of out1_origins");
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
    auto &r = take(m_.reduce, "reduce_names", name);
    std::vector<std::string> got;
    for (const auto &in : r.instr) got.push_back(in.name);
    same_names(name + "_instruction_names", got, inputs);
    for (const auto &in : r.instr) {
      const Shape src = shape_.at(in.name);
      want_equal(name + "_n_in_" + in.name, in.n_in, src.nc, "the channels of " + in.name);
      want_below(name + "_collect_ind_" + in.name, in.collect_ind, src.nf);
    }
    shape_[name] = {r.only_invar ? 1 : r.n_funcs, r.n_out};
  }

  void product(const std::string &name, const std::string &left, const std::string &right)
  {
    auto &c = take(m_.prod, "prod_names", name);
    const Shape l = shape_.at(left), r = shape_.at(right);
    want_equal(name + "_group_left", (int64_t) c.group_left.size(), l.nf, "the functions of " + left);
    want_equal(name + "_n_left", c.n_left, l.nc, "the channels of " + left);
    want_equal(name + "_group_right", (int64_t) c.group_right.size(), r.nf, "the functions of " + right);
    want_equal(name + "_n_right", c.n_right, r.nc, "the channels of " + right);
    shape_[name] = {c.nfunc, c.rank};
  }

  void dense(const std::string &name, const std::string &left, const std::string &right)
  {
    auto &f = take(m_.fc, "fc_names", name);
    const std::string p = "fc_" + name;
    const Shape l = shape_.at(left), r = shape_.at(right);
    want_equal(p + "_w_tile_left", f.n_funcs_left, l.nf, "the functions of " + left);
    if (f.left_coefs) want_equal(p + "_w_left", f.n_in_left, l.nc, "the channels of " + left);
    else want_equal(p + "_n_out", f.n_out, l.nc, "the channels of " + left + ", which pass unweighted");
    want_equal(p + "_w_right", f.n_in_right, r.nc, "the channels of " + right);
    want_below(p + "_collect_from", f.collect_from, r.nf);
    shape_[name] = {f.n_funcs_left, f.n_out};
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
  m.embedding_size = z.int_in("embedding_size", 64, 1, kMaxDim);
  m.nradbase = z.int_in("nradbase", 10, 1, kMaxDim);
  m.lmax = z.int_in("lmax", z.int_in("A1_lmax", 4, 0, kMaxL), 0, kMaxL);    // no bare lmax key in an export: A1_lmax
  m.rcut = cutoff_scalar(z, "rcut", 6.0);
  m.has_bond_specific_cutoff = flag(z, "has_bond_specific_cutoff", 0);
  m.chem_embedding = z.reals("chem_embedding");
  z.require_shape("chem_embedding", {m.n_elements, m.embedding_size});
  m.shift_values = z.reals("shift_values");
  want_count("shift_values", m.shift_values.size(), (size_t) m.n_elements);
  m.output_scale = z.real_scalar("output_scale", 1.0);
  m.element_names = z.names("element_names");
  want_count("element_names", m.element_names.size(), (size_t) m.n_elements);
  m.bond_cutoff_map = z.reals("bond_cutoff_map", false);
  for (double c : m.bond_cutoff_map)
    if (c < 0.0) throw bad_array("bond_cutoff_map", "holds a negative cutoff");
  z.require_shape("bond_cutoff_map", {m.n_elements, m.n_elements});
  if (m.bond_cutoff_map.empty()) m.bond_cutoff_map.assign((size_t) m.n_elements * m.n_elements, m.rcut);

  for (const auto &nm : z.names("spbf_names")) m.spbf.push_back(read_spbf(z, nm, m));
  if (!m.spbf.empty()) m.radial_basis_p = m.spbf[0].p;
  for (const auto &s : m.spbf)    // one envelope order for all layers
    if (s.p != m.radial_basis_p)
      throw bad_array(s.name + "_p", "is " + num(s.p) + ", the envelope order of " + m.spbf[0].name + " is " + num(m.radial_basis_p) +
                                         "; layers with different orders are not supported");
  for (const auto &nm : z.names("prod_names")) m.prod.push_back(read_cpl(z, nm));
  for (const auto &nm : z.names("reduce_names")) m.reduce.push_back(read_reduce(z, nm, m.n_elements));
  for (const auto &nm : z.names("fc_names")) m.fc.push_back(read_fc(z, nm));
  for (const auto &nm : z.names("eqnorm_names")) m.eqnorm.push_back(read_eqnorm(z, nm));
  for (const auto &nm : z.names("rmsnorm_names")) m.rmsnorm.push_back(read_rmsnorm(z, nm));

  m.out1_origins = z.names("out1_origins");
  m.energy_mlp_origin_n_out = z.int_scalar("energy_mlp_origin_n_out", 0);
  m.energy_mlp_n_origins = z.int_scalar("energy_mlp_n_origins", (int) m.out1_origins.size());
  want_equal("energy_mlp_n_origins", m.energy_mlp_n_origins, (int64_t) m.out1_origins.size(), "the names in out1_origins");

  m.readout_width = Graph(m).walk(z.has("energy_mlp_origin_n_out"));
  read_mlp(z, "energy_mlp", m.energy_mlp, m.readout_width - 1, 1, "the channels of out1_origins but the linear channel 0",
           "one energy per atom");
  m.energy_mlp_activation = z.int_in("energy_mlp_activation", 0, 0, 1);
  return m;
}

std::string Grace3LModel::summary() const
{
  std::string s = "GRACE-3L: " + num(n_elements) + " elements, lmax " + num(lmax) + ", channels";
  for (const auto &b : spbf) s += " " + num(b.n_rad_max);
  s += ", message functions";
  for (const auto &e : eqnorm) s += " " + num(e.M);
  s += ", coupled functions";
  for (const auto &b : spbf)
    if (b.equivariant) s += " " + num(b.nfunc);
  s += ", cp_l terms";
  for (const auto &c : prod) s += " " + num(c.n_cg);
  s += ", readout width " + num(readout_width);
  return s;
}

}    // namespace gb
