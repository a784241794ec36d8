#include "model.h"

#include <algorithm>
#include <cmath>

namespace gb {

namespace {

constexpr int kMaxDim = 1 << 16;
constexpr int kFormatVersion = 2;

void require_size(const std::string &key, size_t got, size_t want)
{
  if (got != want) throw bad_array(key, "has " + std::to_string(got) + " values, expected " + std::to_string(want));
}

void require_index(const std::string &key, const std::vector<int> &v, int64_t n)
{
  for (size_t q = 0; q < v.size(); q++)
    if (v[q] < 0 || v[q] >= n)
      throw bad_array(key, "has " + std::to_string(v[q]) + " at " + std::to_string(q) + ", outside [0, " + std::to_string(n) + ")");
}

void require_eq(const std::string &key, int64_t got, int64_t want, const std::string &why)
{
  if (got != want) throw bad_array(key, "is " + std::to_string(got) + ", expected " + std::to_string(want) + " (" + why + ")");
}

int extent(const std::vector<int> &v)
{
  int m = 0;
  for (int x : v) m = std::max(m, x + 1);
  return m;
}

std::vector<MlpLayer> load_mlp(const Npz &z, const std::string &prefix, int n_layers, int n_in, int n_out)
{
  std::vector<MlpLayer> layers;
  int prev = n_in;
  for (int i = 0; i < n_layers; i++) {
    const std::string k = prefix + "_W" + std::to_string(i);
    MlpLayer L;
    L.W = z.reals(k);
    const auto sh = z.shape(k);
    if (sh.size() != 2) throw bad_array(k, "must be a matrix");
    if (sh[0] != prev) throw bad_array(k, "has " + std::to_string(sh[0]) + " rows, expected " + std::to_string(prev));
    if (sh[1] < 1 || sh[1] > kMaxDim) throw bad_array(k, "has an unsupported width");
    L.n_in = (int) sh[0];
    L.n_out = (int) sh[1];
    L.norm = z.real_scalar(prefix + "_norm" + std::to_string(i), 1.0);
    prev = L.n_out;
    layers.push_back(std::move(L));
  }
  if (prev != n_out) throw bad_array(prefix + "_W" + std::to_string(n_layers - 1), "has " + std::to_string(prev) + " outputs, expected " + std::to_string(n_out));
  return layers;
}

FCWeights load_fc(const Npz &z, const std::string &p, int n_funcs, int ch_l, int ch_r, int nf_r, int ch_out, const char *kind)
{
  FCWeights f;
  if (!z.has(p + "_w_left")) return f;
  f.present = true;
  f.w_left = z.reals(p + "_w_left");
  f.w_right = z.reals(p + "_w_right");
  f.tile_left = z.ints(p + "_w_tile_left");
  f.tile_right = z.ints(p + "_w_tile_right");
  f.collect_to = z.ints(p + "_collect_to");
  f.collect_from = z.ints(p + "_collect_from");
  f.nof = z.reals(p + "_norm_out_factor");
  f.norm_left = z.real_scalar(p + "_norm_left", 1.0);
  f.norm_right = z.real_scalar(p + "_norm_right", 1.0);
  f.n_out = z.int_in(p + "_n_out", 64, 1, kMaxDim);
  require_eq(p + "_left_coefs", z.int_scalar(p + "_left_coefs", 1), 1, std::string("the ") + kind + " engines apply left weights in every FC");
  const auto sl = z.shape(p + "_w_left"), sr = z.shape(p + "_w_right");
  if (sl.size() != 3 || sr.size() != 3) throw bad_array(p + "_w_left", "must have three dimensions");
  f.tiles_left = (int) sl[2];
  f.tiles_right = (int) sr[2];
  require_eq(p + "_n_out", f.n_out, ch_out, "the channels of the stage");
  z.require_shape(p + "_w_left", {f.n_out, ch_l, f.tiles_left});
  z.require_shape(p + "_w_right", {f.n_out, ch_r, f.tiles_right});
  f.n_in_left = ch_l;
  f.n_in_right = ch_r;
  f.n_funcs = n_funcs;
  require_size(p + "_w_tile_left", f.tile_left.size(), n_funcs);
  require_size(p + "_norm_out_factor", f.nof.size(), n_funcs);
  require_index(p + "_w_tile_left", f.tile_left, f.tiles_left);
  const size_t nc = f.collect_from.size();
  require_size(p + "_collect_to", f.collect_to.size(), nc);
  require_size(p + "_w_tile_right", f.tile_right.size(), nc);
  require_index(p + "_collect_from", f.collect_from, nf_r);
  require_index(p + "_collect_to", f.collect_to, n_funcs);
  require_index(p + "_w_tile_right", f.tile_right, f.tiles_right);
  return f;
}

CGProduct load_prod(const Npz &z, const std::string &p, int n_left, int n_right)
{
  CGProduct c;
  if (!z.has(p + "_n_cg_terms")) return c;
  c.present = true;
  c.left = z.ints(p + "_left_ind");
  c.right = z.ints(p + "_right_ind");
  c.m_sum = z.ints(p + "_m_sum_ind");
  c.cg = z.reals(p + "_cg_coeff");
  c.n_out = z.int_in(p + "_n_output_funcs", 0, 1, kMaxDim);
  const size_t nt = z.int_in(p + "_n_cg_terms", 0, 1, kMaxDim);
  require_size(p + "_left_ind", c.left.size(), nt);
  require_size(p + "_right_ind", c.right.size(), nt);
  require_size(p + "_m_sum_ind", c.m_sum.size(), nt);
  require_size(p + "_cg_coeff", c.cg.size(), nt);
  require_index(p + "_left_ind", c.left, n_left);
  require_index(p + "_right_ind", c.right, n_right);
  require_index(p + "_m_sum_ind", c.m_sum, c.n_out);
  require_eq(p + "_n_output_funcs", c.n_out, extent(c.m_sum), "1 + the largest " + p + "_m_sum_ind");
  return c;
}

// scalar: every connection goes to output function 0 (rho, I2)
ReduceWeights load_reduce(const Npz &z, const std::string &r, const std::string &s, bool elem, int n_el, int n_out,
                          int n_in, int n_funcs_in, int nfo, bool scalar)
{
  ReduceWeights w;
  const std::string wkey = r + "_reduce_" + s + "_W";
  if (!z.has(wkey)) return w;
  w.present = true;
  w.W = z.reals(wkey);
  w.norm = z.real_scalar(r + "_reduce_" + s + "_norm", 1.0);
  w.collect = z.ints(r + "_collect_ind_" + s);
  w.tile = z.ints(r + "_w_l_tile_" + s);
  w.n_in = z.int_scalar(r + "_n_in_" + s, 0);
  w.w_shape = z.int_in(r + "_w_shape_" + s, 0, 1, kMaxDim);
  w.n_out = n_out;
  w.elem = elem;
  require_eq(r + "_n_in_" + s, w.n_in, n_in, "the channels of " + s);
  if (elem) z.require_shape(wkey, {n_el, n_out, n_in, w.w_shape});
  else z.require_shape(wkey, {n_out, n_in, w.w_shape});
  require_size(r + "_w_l_tile_" + s, w.tile.size(), w.collect.size());
  require_index(r + "_collect_ind_" + s, w.collect, n_funcs_in);
  require_index(r + "_w_l_tile_" + s, w.tile, w.w_shape);
  if (scalar) {
    w.fo.assign(w.collect.size(), 0);
  } else {
    w.fo = z.ints(r + "_total_sum_ind_" + s);
    require_size(r + "_total_sum_ind_" + s, w.fo.size(), w.collect.size());
    require_index(r + "_total_sum_ind_" + s, w.fo, nfo);
  }
  return w;
}

void check_format(const Npz &z, const char *kind)
{
  const bool described = z.has("grace_model_kind");
  if (described) {
    const auto k = z.names("grace_model_kind");
    if (k.size() != 1) throw bad_array("grace_model_kind", "must hold one name");
    if (k[0] != kind) throw ModelError(std::string(kind) + ": the file holds a " + k[0] + " model");
  }
  const int v = z.int_scalar("grace_format_version", 0);
  if (described && v < 1) throw bad_array("grace_format_version", "is missing or below 1 next to grace_model_kind");
  if (v > kFormatVersion)
    throw ModelError(std::string(kind) + ": kokkos.npz format " + std::to_string(v) + ", this backend reads up to " + std::to_string(kFormatVersion));
}

// legacy models: RMS layer norm of the energy-MLP input, its scale folded into the first layer
// (libgrace/src/npz3.h:330-338)
bool fold_ln_scale(const Npz &z, MlpLayer &L)
{
  const auto s = z.reals("energy_mlp_scale", false);
  if (s.empty()) return false;
  require_size("energy_mlp_scale", s.size(), L.n_in);
  for (int k = 0; k < L.n_in; k++)
    for (int j = 0; j < L.n_out; j++) L.W[(size_t) k * L.n_out + j] *= s[k];
  return true;
}

std::vector<double> fold_z(const GraceModel &m, const std::vector<double> &W, int c, double norm, double inv_avg)
{
  std::vector<double> zt((size_t) m.n_elements * c);
  for (int mu = 0; mu < m.n_elements; mu++)
    for (int n = 0; n < c; n++) {
      double v = 0.0;
      for (int e = 0; e < m.embedding; e++) v += W[(size_t) e * c + n] * m.chem[(size_t) mu * m.embedding + e];
      zt[(size_t) mu * c + n] = v * norm * inv_avg;
    }
  return zt;
}

void load_common(const Npz &z, GraceModel &m, const char *kind)
{
  m.n_elements = z.int_in("n_elements", 89, 1, kMaxDim);
  m.embedding = z.int_in("embedding_size", 128, 1, kMaxDim);
  m.lmax = z.int_in("lmax", 4, 0, 255);
  if (m.lmax > 4) throw ModelError(std::string(kind) + ": lmax > 4 not supported");
  m.nradbase = z.int_in("nradbase", 10, 1, kMaxDim);
  m.p = z.int_in("radial_basis_p", 16, 1, 46339);
  m.rcut = z.real_scalar("rcut", 6.0);
  if (!(m.rcut > 0.0)) throw bad_array("rcut", "must be positive");
  m.bond_specific = z.int_in("has_bond_specific_cutoff", 0, 0, 1) != 0;
  m.element_names = z.names("element_names");
  m.chem = z.reals("chem_embedding");
  if (!m.element_names.empty()) require_size("element_names", m.element_names.size(), m.n_elements);
  z.require_shape("chem_embedding", {m.n_elements, m.embedding});
  m.bond_cutoff = z.reals("bond_cutoff_map", false);
  if (!m.bond_cutoff.empty()) {
    z.require_shape("bond_cutoff_map", {m.n_elements, m.n_elements});
    for (double c : m.bond_cutoff)
      if (!(c > 0.0)) throw bad_array("bond_cutoff_map", "must be positive");
  } else {
    m.bond_cutoff.assign((size_t) m.n_elements * m.n_elements, m.rcut);
  }
  m.radial_activation = z.int_in("radial_activation", 0, 0, 1);
  m.output_scale = z.real_scalar("output_scale", 1.0);
  m.shift = z.reals("shift_values", false);
  if (z.has("shift_values")) require_size("shift_values", m.shift.size(), m.n_elements);
  else m.shift.assign(m.n_elements, 0.0);
  m.has_uq = z.int_scalar("uq_schema_version", 0) != 0;
}

void load_energy_mlp(const Npz &z, GraceModel &m, int def_act)
{
  const int n = z.int_in("energy_mlp_n_layers", 2, 1, 7);
  m.energy_mlp = load_mlp(z, "energy_mlp", n, m.rho_n_out - 1, 1);
  for (auto &L : m.energy_mlp)
    if (L.n_in > 256 || L.n_out > 256) throw ModelError("energy MLP widths above 256 are not supported");
  m.energy_activation = z.int_in("energy_mlp_activation", def_act, 0, 1);
  m.energy_ln = fold_ln_scale(z, m.energy_mlp[0]);
}

void load_chain(const Npz &z, Chain &c, const char *x0, int n0, int c0, int cf, const char *kind)
{
  // names: x0 = "A": fc_A1, prod_AA, fc_AA1, prod_AAA, fc_AA2, prod_AAAA
  const std::string X(x0), XX = X + X, XXX = XX + X, XXXX = XXX + X;
  c.n0 = n0;
  c.c0 = c0;
  c.cf = cf;
  c.pXX = load_prod(z, "prod_" + XX, n0, n0);
  if (!c.pXX.present) throw bad_array("prod_" + XX + "_n_cg_terms", "is missing from the .npz file");
  const int nXX = c.pXX.n_out;
  c.fc1 = load_fc(z, "fc_" + X + "1", n0, c0, c0, n0, cf, kind);
  c.fcXX1 = load_fc(z, "fc_" + XX + "1", nXX, cf, c0, n0, cf, kind);
  if (!c.fc1.present || !c.fcXX1.present) throw bad_array("fc_" + X + "1_w_left", "is missing from the .npz file");
  c.pXXX = load_prod(z, "prod_" + XXX, nXX, n0);
  if (!c.pXXX.present) throw bad_array("prod_" + XXX + "_n_cg_terms", "is missing from the .npz file");
  c.pXXXX = load_prod(z, "prod_" + XXXX, nXX, nXX);
  c.order4 = c.pXXXX.present;
  if (c.order4) {
    c.fcXX2 = load_fc(z, "fc_" + XX + "2", nXX, cf, c0, n0, cf, kind);
    if (!c.fcXX2.present) throw bad_array("fc_" + XX + "2_w_left", "is missing although prod_" + XXXX + " is present");
  } else {
    for (const auto &k : z.keys())
      if (k.find(XXXX) != std::string::npos || k.rfind("fc_" + XX + "2_", 0) == 0)
        throw bad_array(k, "is present, but prod_" + XXXX + "_n_cg_terms is not: the " + XXXX + " stage is incomplete");
  }
}

void load_reduce4(const Npz &z, ReduceWeights *out, const std::string &r, const Chain &c, const char *x0, bool elem,
                  int n_el, int n_out, int nfo, bool scalar)
{
  const std::string X(x0), XX = X + X, XXX = XX + X, XXXX = XXX + X;
  out[0] = load_reduce(z, r, X, elem, n_el, n_out, c.c0, c.n0, nfo, scalar);
  out[1] = load_reduce(z, r, XX, elem, n_el, n_out, c.cf, c.pXX.n_out, nfo, scalar);
  out[2] = load_reduce(z, r, XXX, elem, n_el, n_out, c.cf, c.pXXX.n_out, nfo, scalar);
  if (c.order4) out[3] = load_reduce(z, r, XXXX, elem, n_el, n_out, c.cf, c.pXXXX.n_out, nfo, scalar);
  for (int s = 0; s < (c.order4 ? 4 : 3); s++)
    if (!out[s].present) throw bad_array(r + "_reduce_" + (s == 0 ? X : s == 1 ? XX : s == 2 ? XXX : XXXX) + "_W", "is missing from the .npz file");
}

void require_elem_dep(const Npz &z, const std::string &prefix, int fixed, const char *kind)
{
  const std::string key = prefix + "_is_central_atom_type_dependent";
  require_eq(key, z.int_scalar(key, fixed), fixed, std::string("the ") + kind + " engines implement this layout only");
}

void load_1l(const Npz &z, GraceModel &m)
{
  check_format(z, "GRACE-1L");
  load_common(z, m, "GRACE-1L");
  const int nl = m.lmax + 1, nlm = nl * nl;
  const int c1 = z.int_in("nradmax", 32, 1, kMaxDim);
  require_eq("mlp_rad_has_chem_emb", z.int_scalar("mlp_rad_has_chem_emb", 0), 0, "chem-embedded radial MLPs are not supported");
  const auto W = z.reals("A_lin_transform_W");
  z.require_shape("A_lin_transform_W", {m.embedding, c1});
  m.zA = fold_z(m, W, c1, z.real_scalar("A_lin_transform_norm", 1.0), z.real_scalar("A_inv_avg_n_neigh", 1.0));
  m.rad1 = load_mlp(z, "mlp_rad", z.int_in("mlp_rad_n_layers", 3, 1, 16), m.nradbase, c1 * nl);
  const int cf = z.int_in("fc_A1_n_out", 64, 1, kMaxDim);
  load_chain(z, m.chain1, "A", nlm, c1, cf, "GRACE-1L");
  m.chain1.xxx_right_x0 = z.int_in("AAA_right_A", 0, 0, 1) != 0;
  if (m.chain1.xxx_right_x0) require_eq("fc_AA1_n_out", cf, c1, "nradmax (AAA = AA1 x A)");
  m.max_order = m.chain1.order4 ? 4 : 3;
  m.rho_n_out = z.int_in("rho_n_out", 17, 2, kMaxDim);
  require_elem_dep(z, "rho", 1, "GRACE-1L");
  load_reduce4(z, m.rho, "rho", m.chain1, "A", true, m.n_elements, m.rho_n_out, 1, true);
  load_energy_mlp(z, m, 0);
}

void load_2l(const Npz &z, GraceModel &m)
{
  check_format(z, "GRACE-2L");
  load_common(z, m, "GRACE-2L");
  const int nl = m.lmax + 1, nlm = nl * nl;
  auto rad = [&](const std::string &p, int &nrad) {
    require_eq(p + "_has_chem_emb", z.int_scalar(p + "_has_chem_emb", 0), 0, "chem-embedded radial MLPs are not supported");
    nrad = z.int_in(p + "_n_rad_max", 32, 1, kMaxDim);
    return load_mlp(z, p, z.int_in(p + "_n_layers", 3, 1, 16), m.nradbase, nrad * nl);
  };
  int c1 = 0;
  m.rad1 = rad("mlp_rad_R", c1);
  m.rad2 = rad("mlp_rad_R1", m.cr);
  {
    const auto W = z.reals("A_lin_transform_W");
    z.require_shape("A_lin_transform_W", {m.embedding, c1});
    m.zA = fold_z(m, W, c1, z.real_scalar("A_lin_transform_norm", 1.0), z.real_scalar("A_inv_avg_n_neigh", 1.0));
    const auto WB = z.reals("B0_lin_transform_W");
    z.require_shape("B0_lin_transform_W", {m.embedding, m.cr});
    m.zB0 = fold_z(m, WB, m.cr, z.real_scalar("B0_lin_transform_norm", 1.0), z.real_scalar("B0_inv_avg_n_neigh", 1.0));
  }
  load_chain(z, m.chain1, "A", nlm, c1, c1, "GRACE-2L");
  m.chain1.xxx_right_x0 = true;
  m.i1_out = z.int_in("I1_n_out", 12, 1, kMaxDim);
  m.nI1 = z.int_in("I1_n_funcs", 4, 1, kMaxDim);
  require_elem_dep(z, "I1", 1, "GRACE-2L");
  load_reduce4(z, m.I1, "I1", m.chain1, "A", true, m.n_elements, m.i1_out, m.nI1, false);
  const int I_n_out = z.int_in("I_n_out", 32, 1, kMaxDim);
  m.nI = z.int_in("I_n_funcs", 4, 1, kMaxDim);
  require_elem_dep(z, "I", 0, "GRACE-2L");
  m.I_from_I1 = load_reduce(z, "I", "I1", false, m.n_elements, I_n_out, m.i1_out, m.nI1, m.nI, false);
  if (!m.I_from_I1.present) throw bad_array("I_reduce_I1_W", "is missing from the .npz file");
  require_eq("I_n_out", I_n_out, m.cr, "YI couples I with the layer-2 radial channels mlp_rad_R1_n_rad_max");
  m.rho_n_out = z.int_in("rho_n_out", 17, 2, kMaxDim);
  require_elem_dep(z, "rho", 1, "GRACE-2L");
  load_reduce4(z, m.rho, "rho", m.chain1, "A", true, m.n_elements, m.rho_n_out, 1, true);
  m.rms = z.int_in("energy_rms_norm", 1, 0, 1) != 0;
  if (m.rms) {
    m.lnI = z.reals("I_nl_LN_scale");
    require_eq("I_nl_LN_type", z.int_scalar("I_nl_LN_type", 1), 1, "the GRACE-2L engines implement the only_nonlin RMSNorm here");
    require_eq("I_nl_LN_n_out", z.int_scalar("I_nl_LN_n_out", 17), m.rho_n_out, "rho_n_out");
    require_size("I_nl_LN_scale", m.lnI.size(), m.rho_n_out - 1);
  } else {
    m.lnI.assign(m.rho_n_out - 1, 1.0);
  }
  // YI coupling
  {
    const auto lr = z.ints("YI_lr_inds");
    m.yi.m_sum = z.ints("YI_m_sum_ind");
    m.yi.cg = z.reals("YI_cg_coeff");
    const int nt = z.int_in("YI_n_cg_terms", 0, 1, kMaxDim);
    m.yi.n_out = z.int_in("YI_n_output_funcs", 0, 1, kMaxDim);
    require_eq("YI_n_rad_max", z.int_scalar("YI_n_rad_max", 32), m.cr, "the layer-2 radial channels mlp_rad_R1_n_rad_max");
    m.yi.inv_avg = z.real_scalar("YI_inv_avg_n_neigh", 1.0);
    z.require_shape("YI_lr_inds", {nt, 2});
    require_size("YI_m_sum_ind", m.yi.m_sum.size(), nt);
    require_size("YI_cg_coeff", m.yi.cg.size(), nt);
    for (int t = 0; t < nt; t++) {
      const int y = lr[2 * t], i = lr[2 * t + 1];
      if (y < 0 || y >= nlm || i < 0 || i >= m.nI) throw bad_array("YI_lr_inds", "has an index pair outside [0, nlm) x [0, I_n_funcs)");
      m.yi.y.push_back(y);
      m.yi.i.push_back(i);
    }
    require_index("YI_m_sum_ind", m.yi.m_sum, m.yi.n_out);
    require_eq("YI_n_output_funcs", m.yi.n_out, extent(m.yi.m_sum), "1 + the largest YI_m_sum_ind");
  }
  const int c2 = z.int_in("B_n_out", 64, 1, kMaxDim);
  m.nB = z.int_in("B_n_funcs", 31, 1, kMaxDim);
  require_elem_dep(z, "B", 0, "GRACE-2L");
  m.B_from_YI = load_reduce(z, "B", "YI", false, m.n_elements, c2, m.cr, m.yi.n_out, m.nB, false);
  m.B_from_B0 = load_reduce(z, "B", "B0", false, m.n_elements, c2, m.cr, nlm, m.nB, false);
  if (!m.B_from_YI.present || !m.B_from_B0.present) throw bad_array("B_reduce_YI_W", "is missing from the .npz file");
  require_eq("B_n_funcs", m.nB, std::max(extent(m.B_from_YI.fo), extent(m.B_from_B0.fo)), "1 + the largest B_total_sum_ind_*");
  load_chain(z, m.chain2, "B", m.nB, c2, c2, "GRACE-2L");
  m.chain2.xxx_right_x0 = true;
  if (m.chain1.order4 != m.chain2.order4)
    throw ModelError("the file has one of the stages AAAA, BBBB but not the other (a GRACE model has all or none of them)");
  m.max_order = m.chain1.order4 ? 4 : 3;
  m.nI2 = z.int_in("I2_n_out", 17, 1, kMaxDim);
  require_elem_dep(z, "I2", 1, "GRACE-2L");
  load_reduce4(z, m.I2, "I2", m.chain2, "B", true, m.n_elements, m.nI2, 1, true);
  require_eq("I2_n_out", m.nI2, m.rho_n_out, "the energy adds rho and I2 function by function: rho_n_out");
  if (m.rms) {
    m.ln0 = z.reals("I_0_LN_scale");
    require_eq("I_0_LN_type", z.int_scalar("I_0_LN_type", 0), 0, "the GRACE-2L engines implement the full RMSNorm here");
    require_eq("I_0_LN_n_out", z.int_scalar("I_0_LN_n_out", 17), m.nI2, "I2_n_out");
    require_size("I_0_LN_scale", m.ln0.size(), m.nI2);
  } else {
    m.ln0.assign(m.nI2, 1.0);
  }
  load_energy_mlp(z, m, 1);
}

}    // namespace

int model_layers_of_file(const Npz &z)
{
  if (z.has("grace_model_kind")) {
    const auto k = z.names("grace_model_kind");
    if (k.size() == 1) {
      if (k[0] == "GRACE-1L") return 1;
      if (k[0] == "GRACE-2L") return 2;
      if (k[0] == "GRACE-3L") return 3;
    }
    throw bad_array("grace_model_kind", "names no GRACE-1L / 2L / 3L model");
  }
  if (z.has("mlp_rad_W0")) return 1;
  if (z.has("B0_lin_transform_W")) return 2;
  if (z.has("prod_names")) return 3;
  throw ModelError("the file is no GRACE kokkos.npz model");
}

namespace {

// the arrays of a schema-6 head with the size checks of libgrace/src/uq_head.cpp:12-78 (every array is indexed flat by
// the kernels, so a mismatched export has to fail here)
void load_uq_arrays(const Npz &z, const GraceModel &m, UqHead &h)
{
  require_eq("uq_n_elements", z.int_scalar("uq_n_elements", m.n_elements), m.n_elements, "n_elements");
  h.max_clusters = z.int_in("uq_max_clusters", 0, 1, kMaxDim);
  h.rp_dim = z.int_in("uq_rp_dim", 0, 1, kMaxDim);
  h.feature_dim = z.int_in("uq_feature_dim", 0, h.rp_dim, kMaxDim);
  const int normalize = z.int_scalar("uq_rp_normalize", 0), add_density = z.int_scalar("uq_rp_add_density_channel", 0);
  const int transform = z.int_scalar("uq_feature_transform", 0);
  h.density_scale = z.real_scalar("uq_rp_density_scale", 1.0);
  h.centroids = z.reals("uq_centroids");
  h.inv_cov = z.reals("uq_inv_cov");
  h.n_clusters = z.ints("uq_n_clusters");
  h.thresholds = z.reals("uq_interp_thresholds");
  h.R = z.reals("uq_rp_matrix");
  if (normalize != 1 || add_density != 1 || transform != 0)
    throw ModelError("schema 6 means normalize = 1, add_density_channel = 1, feature_transform = 0; the file has " +
                     std::to_string(normalize) + ", " + std::to_string(add_density) + ", " + std::to_string(transform));
  h.n_density = h.feature_dim - h.rp_dim;
  const auto rs = z.shape("uq_rp_matrix");
  if (rs.size() != 2) throw bad_array("uq_rp_matrix", "must be a matrix");
  require_eq("uq_rp_matrix", rs[1], h.rp_dim, "uq_rp_dim columns");
  h.d_basis = (int) rs[0];
  const size_t E = m.n_elements, K = h.max_clusters, D = h.feature_dim;
  require_size("uq_centroids", h.centroids.size(), E * K * D);
  require_size("uq_inv_cov", h.inv_cov.size(), E * K * D * D);
  require_size("uq_n_clusters", h.n_clusters.size(), E);
  require_size("uq_interp_thresholds", h.thresholds.size(), E * K);
  for (size_t e = 0; e < E; e++) {
    if (h.n_clusters[e] <= 0) throw ModelError("element index " + std::to_string(e) + " has no clusters");
    if (h.n_clusters[e] > h.max_clusters)
      throw ModelError("element index " + std::to_string(e) + " has more clusters than uq_max_clusters");
  }
}

void load_uq(const Npz &z, GraceModel &m)
{
  UqHead &h = m.uq;
  h.schema = z.int_scalar("uq_schema_version", 0);
  h.present = h.schema != 0;
  m.has_uq = h.present;
  if (!h.present) return;
  if (h.schema != 6) {
    h.error = "UQ schema " + std::to_string(h.schema) + " is not supported (schema 6 only); re-export the UQ artifacts";
    return;
  }
  try {
    load_uq_arrays(z, m, h);
  } catch (const std::exception &e) {
    h.error = std::string("UQ head: ") + e.what();
  }
}

}    // namespace

int GraceModel::uq_basis_width() const
{
  int w = 0;
  if (layers == 2)
    for (const ReduceWeights &r : I2) w += r.present ? r.n_in * (int) r.collect.size() : 0;
  for (const ReduceWeights &r : rho) w += r.present ? r.n_in * (int) r.collect.size() : 0;
  return w;
}

void GraceModel::validate_uq() const
{
  if (!uq.present) throw ModelError("the model has no UQ head");
  if (max_order == 3) throw ModelError("UQ is not supported for max_order 3 models");
  if (!uq.error.empty()) throw ModelError(uq.error);
  if (uq.d_basis != uq_basis_width())
    throw ModelError("UQ head: uq_rp_matrix has " + std::to_string(uq.d_basis) + " rows, the model's invariant basis has " +
                     std::to_string(uq_basis_width()) + "; re-export the UQ artifacts for this model");
  if (uq.n_density != 1 + layers)
    throw ModelError("UQ head: " + std::to_string(uq.n_density) + " density channels, expected " + std::to_string(1 + layers));
  if (uq.rp_dim > 128) throw ModelError("UQ head: projections wider than 128 are not supported");
}

int GraceModel::element_index(const std::string &name) const
{
  for (size_t i = 0; i < element_names.size(); i++)
    if (element_names[i] == name) return (int) i;
  return -1;
}

GraceModel GraceModel::load(const std::string &path)
{
  Npz z(path);
  GraceModel m;
  m.layers = model_layers_of_file(z);
  if (m.layers == 1) load_1l(z, m);
  else if (m.layers == 2) load_2l(z, m);
  else {
    // the whole model lives in m3; the common fields are what Systems, Batches and the neighbour list read
    m.m3 = std::make_shared<Grace3LModel>(Grace3LModel::load(z));
    const Grace3LModel &t = *m.m3;
    m.n_elements = t.n_elements;
    m.embedding = t.embedding;
    m.lmax = t.lmax;
    m.nradbase = t.nbasis;
    m.p = t.env_p;
    m.rcut = t.cutoff;
    m.bond_specific = t.pair_cutoffs_given;
    m.bond_cutoff = t.pair_cutoff;
    m.element_names = t.elements;
    m.chem = t.embedding_table;
    m.output_scale = t.energy_scale;
    m.shift = t.energy_shift;
    if (z.has("uq_schema_version")) throw ModelError("GRACE-3L: the UQ head of GRACE-3L models is not supported");
    return m;
  }
  load_uq(z, m);
  return m;
}

}    // namespace gb
