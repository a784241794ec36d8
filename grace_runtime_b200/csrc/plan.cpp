#include "plan.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <map>
#include <memory>

namespace gb {

double MVOp::flops_per_atom() const
{
  double f = 0.0;
  for (const auto &it : items) f += 2.0 * it.n_in * n_out;
  return f;
}

namespace {

// ---- radial tables -------------------------------------------------------------------------------------------

// g_k = T_k(2x - 1) fc_p(x), k = 1..nrb, and d/dx (libgrace/include/grace/radial_x.h:11-26)
void radial_basis_x(double x, int p, int nrb, std::vector<double> &g, std::vector<double> &dg)
{
  const double xp = std::pow(x, p), xp1 = xp * x, xp2 = xp1 * x;
  const double fc = 1.0 - 0.5 * (p + 1) * (p + 2) * xp + p * (p + 2) * xp1 - 0.5 * p * (p + 1) * xp2;
  const double dfc = 0.5 * p * (p + 1) * (p + 2) * (-std::pow(x, p - 1) + 2.0 * xp - xp1);
  const double t = 2.0 * x - 1.0;
  double Tp = 1.0, Tc = t, dTp = 0.0, dTc = 2.0;
  g.resize(nrb);
  dg.resize(nrb);
  for (int k = 0; k < nrb; k++) {
    g[k] = Tc * fc;
    dg[k] = dTc * fc + Tc * dfc;
    const double Tn = 2.0 * t * Tc - Tp, dTn = 2.0 * (2.0 * Tc + t * dTc) - dTp;
    Tp = Tc; dTp = dTc; Tc = Tn; dTc = dTn;
  }
}

// value and d/dx of the radial MLP in forward mode (libgrace/include/grace/radial_x.h:30-60)
void mlp_x(const std::vector<MlpLayer> &layers, std::vector<double> h, std::vector<double> dh, std::vector<double> &out,
           std::vector<double> &dout, int act)
{
  const int n = (int) layers.size();
  for (int il = 0; il < n; il++) {
    const MlpLayer &L = layers[il];
    std::vector<double> s(L.n_out, 0.0), ds(L.n_out, 0.0);
    for (int k = 0; k < L.n_in; k++)
      for (int j = 0; j < L.n_out; j++) {
        const double w = L.W[(size_t) k * L.n_out + j];
        s[j] += w * h[k];
        ds[j] += w * dh[k];
      }
    for (int j = 0; j < L.n_out; j++) {
      s[j] *= L.norm;
      ds[j] *= L.norm;
      if (il < n - 1 && act == 1) {
        s[j] = std::tanh(s[j]);
        ds[j] *= 1.0 - s[j] * s[j];
      } else if (il < n - 1) {
        const double sg = 1.0 / (1.0 + std::exp(-s[j]));
        ds[j] = sg * (1.0 + s[j] * (1.0 - sg)) * ds[j];
        s[j] = s[j] * sg;
      }
    }
    h.swap(s);
    dh.swap(ds);
  }
  out.swap(h);
  dout.swap(dh);
}

// cubic Hermite coefficients of R[n][l](x) on N intervals of [0, 1], [N][nl][C][4] in fp32 (the four coefficients of a
// channel side by side: one 16-byte load per lane and l)
// (libgrace/src/fused_1l.cpp:102-129)
RadialTable build_radial(const GraceModel &m, const std::vector<MlpLayer> &layers, int C, int N)
{
  RadialTable T;
  T.N = N;
  T.nl = m.lmax + 1;
  T.C = C;
  const int nl = T.nl, nout = layers.back().n_out;
  if (nout != C * nl) throw ModelError("radial MLP output width mismatch");
  const double h = 1.0 / N;
  std::vector<double> fv((size_t) (N + 1) * nout), dv((size_t) (N + 1) * nout), g, dg, out, dout;
  for (int k = 0; k <= N; k++) {
    radial_basis_x(k * h, m.p, m.nradbase, g, dg);
    mlp_x(layers, g, dg, out, dout, m.radial_activation);
    for (int o = 0; o < nout; o++) {
      fv[(size_t) k * nout + o] = out[o];
      dv[(size_t) k * nout + o] = h * dout[o];
    }
  }
  T.tab.assign((size_t) N * 4 * nl * C, 0.0f);
  for (int k = 0; k < N; k++)
    for (int n = 0; n < C; n++)
      for (int l = 0; l < nl; l++) {
        const int o = n * nl + l;
        const double f0 = fv[(size_t) k * nout + o], f1 = fv[(size_t) (k + 1) * nout + o];
        const double d0 = dv[(size_t) k * nout + o], d1 = dv[(size_t) (k + 1) * nout + o];
        const double c[4] = {f0, d0, -3.0 * f0 - 2.0 * d0 + 3.0 * f1 - d1, 2.0 * f0 + d0 - 2.0 * f1 + d1};
        for (int q = 0; q < 4; q++) T.tab[((((size_t) k * nl + l) * C + n) << 2) + q] = (float) c[q];
      }
  return T;
}

// ---- dense network -------------------------------------------------------------------------------------------

inline int pad4(int n) { return (n + 3) / 4 * 4; }

struct ReduceGroup {
  std::string name;
  std::vector<const ReduceWeights *> src;    // per source (nullptr: absent)
  std::vector<int> src_tensor, src_grad, src_row0;
  int n_out = 0, nfo = 0;
  bool elem = false;
  int t_out = -1, t_gout = -1;
};

struct LayerBuilder {
  LayerPlan &P;
  const GraceModel &m;
  std::vector<std::vector<Op>> adj;    // adjoint ops of each forward op, in forward order

  int tensor(const std::string &name, int nf, int ch, bool grad = false)
  {
    P.tensors.push_back({name, nf, ch, grad});
    return (int) P.tensors.size() - 1;
  }
  Op add(MVOp &&o)
  {
    o.item_off.push_back((int) o.items.size());    // closes the last row (rows push their start)
    P.mv.push_back(std::move(o));
    return {Op::MV, (int) P.mv.size() - 1};
  }
  Op add(ProdOp &&o)
  {
    o.term_off.push_back((int) o.terms.size());
    P.prod.push_back(std::move(o));
    return {Op::PROD, (int) P.prod.size() - 1};
  }
  void emit(Op fwd, std::vector<Op> adjoint)
  {
    P.fwd.ops.push_back(fwd);
    adj.push_back(std::move(adjoint));
  }
  void finish()
  {
    for (size_t q = adj.size(); q-- > 0;)
      for (const Op &o : adj[q]) P.bwd.ops.push_back(o);
    first_writers();
  }

  // rows `sel` (positions in row_out) of an operation as an operation of its own
  static MVOp subset(const MVOp &o, const std::vector<int> &sel, const std::string &suffix)
  {
    MVOp s;
    s.name = o.name + suffix; s.dst = o.dst; s.n_out = o.n_out; s.ldw = o.ldw; s.accumulate = o.accumulate; s.elem = o.elem;
    s.ty_stride = o.ty_stride; s.W = o.W;
    for (int r : sel) {
      s.row_out.push_back(o.row_out[r]);
      s.item_off.push_back((int) s.items.size());
      s.items.insert(s.items.end(), o.items.begin() + o.item_off[r], o.items.begin() + o.item_off[r + 1]);
    }
    s.item_off.push_back((int) s.items.size());
    return s;
  }

  // The reverse operations add into gradient tensors.  The first operation that touches a row may as well write it:
  // then nothing has to clear the gradients before the reverse pass (half of a layer's tensors per pass) and the first
  // writers do not read zeros back.  An MV operation whose rows are partly new is split in two; a product keeps adding and
  // is told which of its rows are new (row_first).  zero_grads stays set if some gradient row has no writer at all.
  void first_writers()
  {
    std::vector<std::vector<char>> written(P.tensors.size());
    for (size_t t = 0; t < P.tensors.size(); t++) written[t].assign(P.tensors[t].nfuncs, 0);
    std::vector<Op> out;
    for (const Op &o : P.bwd.ops) {
      const bool mv = o.kind == Op::MV;
      const int dst = mv ? P.mv[o.index].dst : P.prod[o.index].dst;
      const bool acc = mv ? P.mv[o.index].accumulate : P.prod[o.index].accumulate;
      const std::vector<int> rows = mv ? P.mv[o.index].row_out : P.prod[o.index].row_out;
      std::vector<int> fresh, old;
      for (size_t r = 0; r < rows.size(); r++) (written[dst][rows[r]] ? old : fresh).push_back((int) r);
      for (int r : rows) written[dst][r] = 1;
      if (!P.tensors[dst].grad || !acc || fresh.empty()) {
        out.push_back(o);
        continue;
      }
      if (old.empty()) {
        if (mv) P.mv[o.index].accumulate = false;
        else P.prod[o.index].accumulate = false;
        out.push_back(o);
        continue;
      }
      if (mv) {
        MVOp a = subset(P.mv[o.index], fresh, ":first"), b = subset(P.mv[o.index], old, "");
        a.accumulate = false;
        P.mv[o.index] = std::move(b);
        P.mv.push_back(std::move(a));
        out.push_back({Op::MV, (int) P.mv.size() - 1});
      } else {
        // a product stages all rows of its inputs per launch, so it is not split: it is told which rows to write
        P.prod[o.index].row_first.assign(rows.size(), 0);
        for (int r : fresh) P.prod[o.index].row_first[r] = 1;
      }
      out.push_back(o);
    }
    P.bwd.ops = out;
  }

  // FC: dst = nof (Wl Xl + sum Wr Xr) on the live outputs, and its two adjoints
  void fc(const std::string &name, const FCWeights &w, const std::vector<char> &live, int tL, int tR, int tD, int gL,
          int gR, int gD)
  {
    const int no = w.n_out, nil = w.n_in_left, nir = w.n_in_right;
    // weight rows are padded to a multiple of 4 outputs (16-byte loads of 4 output channels)
    const int ldo = pad4(no), ldl = pad4(nil), ldr = pad4(nir);
    MVOp F, BL, BR;
    F.name = name + ":fwd"; BL.name = name + ":adj_left"; BR.name = name + ":adj_right";
    F.dst = tD; F.n_out = no; F.ldw = ldo;
    BL.dst = gL; BL.n_out = nil; BL.ldw = ldl; BL.accumulate = true;
    BR.dst = gR; BR.n_out = nir; BR.ldw = ldr; BR.accumulate = true;
    const int base_r = w.tiles_left * nil * ldo;
    F.W.assign((size_t) base_r + (size_t) w.tiles_right * nir * ldo, 0.0f);
    BL.W.assign((size_t) w.tiles_left * no * ldl, 0.0f);
    BR.W.assign((size_t) w.tiles_right * no * ldr, 0.0f);
    for (int k = 0; k < no; k++) {
      for (int n = 0; n < nil; n++)
        for (int t = 0; t < w.tiles_left; t++) {
          const float v = (float) (w.norm_left * w.w_left[((size_t) k * nil + n) * w.tiles_left + t]);
          F.W[((size_t) t * nil + n) * ldo + k] = v;
          BL.W[((size_t) t * no + k) * ldl + n] = v;
        }
      for (int n = 0; n < nir; n++)
        for (int t = 0; t < w.tiles_right; t++) {
          const float v = (float) (w.norm_right * w.w_right[((size_t) k * nir + n) * w.tiles_right + t]);
          F.W[(size_t) base_r + ((size_t) t * nir + n) * ldo + k] = v;
          BR.W[((size_t) t * no + k) * ldr + n] = v;
        }
    }
    std::map<int, std::vector<int>> by_to, by_from;
    for (size_t c = 0; c < w.collect_to.size(); c++)
      if (live[w.collect_to[c]]) {
        by_to[w.collect_to[c]].push_back((int) c);
        by_from[w.collect_from[c]].push_back((int) c);
      }
    for (int f = 0; f < w.n_funcs; f++) {
      if (!live[f]) continue;
      const float nof = (float) w.nof[f];
      F.row_out.push_back(f);
      F.item_off.push_back((int) F.items.size());
      F.items.push_back({w.tile_left[f] * nil * ldo, tL, f, nil, nof});
      for (int c : by_to[f]) F.items.push_back({base_r + w.tile_right[c] * nir * ldo, tR, w.collect_from[c], nir, nof});
      BL.row_out.push_back(f);
      BL.item_off.push_back((int) BL.items.size());
      BL.items.push_back({w.tile_left[f] * no * ldl, gD, f, no, nof});
    }
    for (auto &kv : by_from) {
      BR.row_out.push_back(kv.first);
      BR.item_off.push_back((int) BR.items.size());
      for (int c : kv.second)
        BR.items.push_back({w.tile_right[c] * no * ldr, gD, w.collect_to[c], no, (float) w.nof[w.collect_to[c]]});
    }
    const Op f = add(std::move(F));
    std::vector<Op> a;
    if (gL == gR && nil == nir) {
      // both inputs are the same tensor (fc(X, X)): one adjoint operation, every row of the gradient written once with
      // the left item first and the right items behind it
      MVOp B;
      B.name = name + ":adj";
      B.dst = gL; B.n_out = nil; B.ldw = ldl; B.accumulate = true;
      const int base = (int) BL.W.size();
      B.W = BL.W;
      B.W.insert(B.W.end(), BR.W.begin(), BR.W.end());
      std::map<int, std::vector<MVItem>> rows;
      for (size_t r = 0; r < BL.row_out.size(); r++)
        for (int q = BL.item_off[r]; q < (r + 1 < BL.row_out.size() ? BL.item_off[r + 1] : (int) BL.items.size()); q++)
          rows[BL.row_out[r]].push_back(BL.items[q]);
      for (size_t r = 0; r < BR.row_out.size(); r++)
        for (int q = BR.item_off[r]; q < (r + 1 < BR.row_out.size() ? BR.item_off[r + 1] : (int) BR.items.size()); q++) {
          MVItem it = BR.items[q];
          it.mat += base;
          rows[BR.row_out[r]].push_back(it);
        }
      for (auto &kv : rows) {
        B.row_out.push_back(kv.first);
        B.item_off.push_back((int) B.items.size());
        B.items.insert(B.items.end(), kv.second.begin(), kv.second.end());
      }
      a.push_back(add(std::move(B)));
    } else {
      a.push_back(add(std::move(BL)));
      a.push_back(add(std::move(BR)));
    }
    emit(f, a);
  }

  // CG product with pruned terms: dst[o] = sum c L[l] R[r]
  void prod(const std::string &name, const CGProduct &p, const std::vector<char> &need, int tL, int tR, int tD, int gL,
            int gR, int gD)
  {
    ProdOp F, BL, BR;
    F.name = name + ":fwd"; BL.name = name + ":adj_left"; BR.name = name + ":adj_right";
    F.dst = tD; F.srcA = tL; F.srcB = tR;
    BL.dst = gL; BL.srcA = gD; BL.srcB = tR; BL.accumulate = true;
    BR.dst = gR; BR.srcA = gD; BR.srcB = tL; BR.accumulate = true;
    std::map<int, std::vector<int>> by_o, by_l, by_r;
    for (size_t t = 0; t < p.cg.size(); t++)
      if (need[p.m_sum[t]]) {
        by_o[p.m_sum[t]].push_back((int) t);
        by_l[p.left[t]].push_back((int) t);
        by_r[p.right[t]].push_back((int) t);
      }
    for (auto &kv : by_o) {
      F.row_out.push_back(kv.first);
      F.term_off.push_back((int) F.terms.size());
      for (int t : kv.second) F.terms.push_back({p.left[t], p.right[t], (float) p.cg[t]});
    }
    for (auto &kv : by_l) {
      BL.row_out.push_back(kv.first);
      BL.term_off.push_back((int) BL.terms.size());
      for (int t : kv.second) BL.terms.push_back({p.m_sum[t], p.right[t], (float) p.cg[t]});
    }
    for (auto &kv : by_r) {
      BR.row_out.push_back(kv.first);
      BR.term_off.push_back((int) BR.terms.size());
      for (int t : kv.second) BR.terms.push_back({p.m_sum[t], p.left[t], (float) p.cg[t]});
    }
    const Op f = add(std::move(F));
    std::vector<Op> a;
    if (tL == tR && gL == gR) {
      // product of a tensor with itself: one adjoint operation over the union of the terms (left terms of a row first)
      ProdOp B;
      B.name = name + ":adj";
      B.dst = gL; B.srcA = gD; B.srcB = tL; B.accumulate = true;
      std::map<int, std::vector<ProdTerm>> rows;
      for (auto &kv : by_l)
        for (int t : kv.second) rows[kv.first].push_back({p.m_sum[t], p.right[t], (float) p.cg[t]});
      for (auto &kv : by_r)
        for (int t : kv.second) rows[kv.first].push_back({p.m_sum[t], p.left[t], (float) p.cg[t]});
      for (auto &kv : rows) {
        B.row_out.push_back(kv.first);
        B.term_off.push_back((int) B.terms.size());
        B.terms.insert(B.terms.end(), kv.second.begin(), kv.second.end());
      }
      a.push_back(add(std::move(B)));
    } else {
      a.push_back(add(std::move(BL)));
      a.push_back(add(std::move(BR)));
    }
    emit(f, a);
  }

  // reduce of several sources into one tensor, and one adjoint per source
  void reduce(const ReduceGroup &R)
  {
    MVOp F;
    F.name = R.name + ":fwd";
    F.dst = R.t_out;
    F.n_out = R.n_out;
    F.ldw = pad4(R.n_out);
    F.elem = R.elem;
    const int nty = R.elem ? m.n_elements : 1;
    std::vector<int64_t> base(R.src.size(), 0);
    int64_t per_type = 0;
    for (size_t s = 0; s < R.src.size(); s++)
      if (R.src[s]) {
        base[s] = per_type;
        per_type += (int64_t) R.src[s]->w_shape * R.src[s]->n_in * pad4(R.n_out);
      }
    F.ty_stride = R.elem ? per_type : 0;
    F.W.assign((size_t) per_type * nty, 0.0f);
    std::vector<Op> adjoint;
    for (size_t s = 0; s < R.src.size(); s++) {
      if (!R.src[s]) continue;
      const ReduceWeights &w = *R.src[s];
      const int nin = w.n_in, ws = w.w_shape, no = R.n_out, ldf = pad4(no), ldb = pad4(nin);
      MVOp B;
      B.name = R.name + ":adj_src" + std::to_string(s);
      B.dst = R.src_grad[s];
      B.n_out = nin;
      B.ldw = ldb;
      B.accumulate = true;
      B.elem = R.elem;
      B.ty_stride = R.elem ? (int64_t) ws * no * ldb : 0;
      B.W.assign((size_t) ws * no * ldb * nty, 0.0f);
      for (int ty = 0; ty < nty; ty++)
        for (int k = 0; k < no; k++)
          for (int n = 0; n < nin; n++)
            for (int t = 0; t < ws; t++) {
              const size_t off = R.elem ? ((((size_t) ty * no + k) * nin + n) * ws + t) : (((size_t) k * nin + n) * ws + t);
              const float v = (float) (w.norm * w.W[off]);
              F.W[(size_t) ty * per_type + base[s] + ((size_t) t * nin + n) * ldf + k] = v;
              B.W[(size_t) ty * ws * no * ldb + ((size_t) t * no + k) * ldb + n] = v;
            }
      std::map<int, std::vector<int>> by_ci;
      for (size_t c = 0; c < w.collect.size(); c++) by_ci[w.collect[c]].push_back((int) c);
      for (auto &kv : by_ci) {
        B.row_out.push_back(R.src_row0[s] + kv.first);
        B.item_off.push_back((int) B.items.size());
        for (int c : kv.second) B.items.push_back({w.tile[c] * no * ldb, R.t_gout, w.fo[c], no, 1.0f});
      }
      adjoint.push_back(add(std::move(B)));
    }
    for (int fo = 0; fo < R.nfo; fo++) {
      bool any = false;
      for (size_t s = 0; s < R.src.size(); s++) {
        if (!R.src[s]) continue;
        const ReduceWeights &w = *R.src[s];
        for (size_t c = 0; c < w.collect.size(); c++)
          if (w.fo[c] == fo) {
            if (!any) {
              F.row_out.push_back(fo);
              F.item_off.push_back((int) F.items.size());
              any = true;
            }
            F.items.push_back({(int) (base[s] + (int64_t) w.tile[c] * w.n_in * pad4(R.n_out)), R.src_tensor[s],
                               R.src_row0[s] + w.collect[c], w.n_in, 1.0f});
          }
      }
    }
    const Op f = add(std::move(F));
    emit(f, adjoint);
  }

  // UQ: z[d] = sum over the collected inputs b of the reduce R of x_b Rp[row0 + b][d]; the inputs of a source are
  // numbered channel-major (b = n * collected + c: libgrace/include/grace/fused_cpu.h:1291-1305), so the matrix of the
  // collected function c takes every collected-th row of the source's block.  Returns the rows used.
  int uq_projection(const ReduceGroup &R, const UqHead &h, int row0)
  {
    const int RP = h.rp_dim, ldw = pad4(RP);
    MVOp F;
    F.name = "uq:" + R.name;
    P.tUQ = tensor("uq_" + R.name, 1, RP);
    P.tensors[P.tUQ].external = true;
    F.dst = P.tUQ; F.n_out = RP; F.ldw = ldw;
    F.row_out.push_back(0);
    F.item_off.push_back(0);
    int row = row0;
    for (size_t s = 0; s < R.src.size(); s++) {
      const ReduceWeights *w = R.src[s];
      if (!w || !w->present) continue;
      const int nc = (int) w->collect.size(), nin = w->n_in;
      for (int c = 0; c < nc; c++) {
        const int mat = (int) F.W.size();
        F.W.resize(F.W.size() + (size_t) nin * ldw, 0.0f);
        for (int n = 0; n < nin; n++)
          for (int d = 0; d < RP; d++)
            F.W[(size_t) mat + (size_t) n * ldw + d] = (float) h.R[((size_t) row + (size_t) n * nc + c) * RP + d];
        F.items.push_back({mat, R.src_tensor[s], R.src_row0[s] + w->collect[c], nin, 1.0f});
      }
      row += nin * nc;
    }
    P.uq_mv = add(std::move(F)).index;
    return row - row0;
  }

  struct ChainTensors {
    int X0, X1, XX, XX1, XX2, XXX, XXXX;
    int gX0, gX1, gXX, gXX1, gXX2, gXXX, gXXXX;
  };

  // the chain X1 .. XXXX of one layer; readers: the reduces that read (X0, XX, XXX, XXXX)
  ChainTensors chain(const std::string &x, const Chain &c, int tX0, int gX0,
                     const std::vector<const ReduceWeights *> &readers_XX,
                     const std::vector<const ReduceWeights *> &readers_XXX,
                     const std::vector<const ReduceWeights *> &readers_XXXX)
  {
    const int n0 = c.n0, nXX = c.pXX.n_out, nXXX = c.pXXX.n_out, nXXXX = c.order4 ? c.pXXXX.n_out : 0;
    ChainTensors T{};
    T.X0 = tX0;
    T.gX0 = gX0;
    const std::string xx = x + x, xxx = xx + x, xxxx = xxx + x;
    T.X1 = tensor(x + "1", n0, c.cf);
    T.XX = tensor(xx, nXX, c.cf);
    T.XX1 = tensor(xx + "1", nXX, c.cf);
    T.XXX = tensor(xxx, nXXX, c.cf);
    T.gX1 = tensor("g" + x + "1", n0, c.cf, true);
    T.gXX = tensor("g" + xx, nXX, c.cf, true);
    T.gXX1 = tensor("g" + xx + "1", nXX, c.cf, true);
    T.gXXX = tensor("g" + xxx, nXXX, c.cf, true);
    T.XX2 = T.XXXX = T.gXX2 = T.gXXXX = -1;
    if (c.order4) {
      T.XX2 = tensor(xx + "2", nXX, c.cf);
      T.XXXX = tensor(xxxx, nXXXX, c.cf);
      T.gXX2 = tensor("g" + xx + "2", nXX, c.cf, true);
      T.gXXXX = tensor("g" + xxxx, nXXXX, c.cf, true);
      P.tensors[T.gXXXX].alias = T.XXXX;
    }
    // XX, XXX, XXXX are read by forward operations only (the adjoints need X0, X1, XX1, XX2): libgrace/src/
    // fused_1l.cpp:309-310 keeps their gradients in the same buffers
    P.tensors[T.gXX].alias = T.XX;
    P.tensors[T.gXXX].alias = T.XXX;
    // liveness, backwards from the reduces
    auto mark = [](const std::vector<const ReduceWeights *> &rs, std::vector<char> &need) {
      for (auto *r : rs)
        if (r)
          for (int ci : r->collect) need[ci] = 1;
    };
    std::vector<char> needXXX(nXXX, 0), needXXXX(std::max(nXXXX, 1), 0), needXX(nXX, 0);
    mark(readers_XXX, needXXX);
    mark(readers_XXXX, needXXXX);
    std::vector<char> liveXX1(nXX, 0), liveXX2(nXX, 0), liveX1(n0, 0);
    for (size_t t = 0; t < c.pXXX.cg.size(); t++)
      if (needXXX[c.pXXX.m_sum[t]]) {
        liveXX1[c.pXXX.left[t]] = 1;
        if (!c.xxx_right_x0) liveX1[c.pXXX.right[t]] = 1;
      }
    if (c.order4)
      for (size_t t = 0; t < c.pXXXX.cg.size(); t++)
        if (needXXXX[c.pXXXX.m_sum[t]]) liveXX2[c.pXXXX.left[t]] = liveXX2[c.pXXXX.right[t]] = 1;
    for (int q = 0; q < nXX; q++) needXX[q] = liveXX1[q] || liveXX2[q];
    mark(readers_XX, needXX);
    for (size_t t = 0; t < c.pXX.cg.size(); t++)
      if (needXX[c.pXX.m_sum[t]]) liveX1[c.pXX.left[t]] = liveX1[c.pXX.right[t]] = 1;

    fc("fc_" + x + "1", c.fc1, liveX1, T.X0, T.X0, T.X1, T.gX0, T.gX0, T.gX1);
    prod("prod_" + xx, c.pXX, needXX, T.X1, T.X1, T.XX, T.gX1, T.gX1, T.gXX);
    fc("fc_" + xx + "1", c.fcXX1, liveXX1, T.XX, T.X0, T.XX1, T.gXX, T.gX0, T.gXX1);
    if (c.order4) fc("fc_" + xx + "2", c.fcXX2, liveXX2, T.XX, T.X0, T.XX2, T.gXX, T.gX0, T.gXX2);
    const int tR = c.xxx_right_x0 ? T.X0 : T.X1, gR = c.xxx_right_x0 ? T.gX0 : T.gX1;
    prod("prod_" + xxx, c.pXXX, needXXX, T.XX1, tR, T.XXX, T.gXX1, gR, T.gXXX);
    if (c.order4) prod("prod_" + xxxx, c.pXXXX, needXXXX, T.XX2, T.XX2, T.XXXX, T.gXX2, T.gXX2, T.gXXXX);
    return T;
  }

  ReduceGroup reduce4(const std::string &name, const ReduceWeights *w, const ChainTensors &T, bool order4, int n_out,
                      int nfo, bool elem, int t_out, int t_gout)
  {
    ReduceGroup R;
    R.name = name;
    R.src = {&w[0], &w[1], &w[2], order4 ? &w[3] : nullptr};
    R.src_tensor = {T.X0, T.XX, T.XXX, T.XXXX};
    R.src_grad = {T.gX0, T.gXX, T.gXXX, T.gXXXX};
    R.src_row0 = {0, 0, 0, 0};
    R.n_out = n_out; R.nfo = nfo; R.elem = elem; R.t_out = t_out; R.t_gout = t_gout;
    return R;
  }
};

// Rows (functions) of the internal tensors that no operation touches are dropped and the rest renumbered: the pruned
// outputs take no memory.  A gradient and the value tensor it may alias keep the same rows.
void compact_rows(LayerPlan &P)
{
  const size_t nt = P.tensors.size();
  std::vector<std::vector<char>> used(nt);
  for (size_t t = 0; t < nt; t++) used[t].assign(P.tensors[t].nfuncs, P.tensors[t].external ? 1 : 0);
  for (const MVOp &o : P.mv) {
    for (int r : o.row_out) used[o.dst][r] = 1;
    for (const MVItem &it : o.items) used[it.src][it.irow] = 1;
  }
  for (const ProdOp &o : P.prod) {
    for (int r : o.row_out) used[o.dst][r] = 1;
    for (const ProdTerm &tm : o.terms) {
      used[o.srcA][tm.a] = 1;
      if (o.srcB >= 0) used[o.srcB][tm.b] = 1;
    }
  }
  for (size_t t = 0; t < nt; t++)
    if (P.tensors[t].alias >= 0) {
      const int v = P.tensors[t].alias;
      for (size_t r = 0; r < used[t].size(); r++) used[t][r] = used[v][r] = (used[t][r] || used[v][r]);
    }
  std::vector<std::vector<int>> map(nt);
  for (size_t t = 0; t < nt; t++) {
    map[t].assign(used[t].size(), -1);
    int k = 0;
    for (size_t r = 0; r < used[t].size(); r++)
      if (used[t][r]) map[t][r] = k++;
    P.tensors[t].nfuncs = k;
  }
  for (MVOp &o : P.mv) {
    for (int &r : o.row_out) r = map[o.dst][r];
    for (MVItem &it : o.items) it.irow = map[it.src][it.irow];
  }
  for (ProdOp &o : P.prod) {
    for (int &r : o.row_out) r = map[o.dst][r];
    for (ProdTerm &tm : o.terms) {
      tm.a = map[o.srcA][tm.a];
      if (o.srcB >= 0) tm.b = map[o.srcB][tm.b];
    }
  }
}

// after compact_rows: the gradients still have to be cleared before the reverse pass if some row of a gradient tensor
// that survived the pruning has no writing operation at all
void check_gradient_writers(LayerPlan &P)
{
  std::vector<std::vector<char>> written(P.tensors.size());
  for (size_t t = 0; t < P.tensors.size(); t++) written[t].assign(P.tensors[t].nfuncs, 0);
  for (const Op &o : P.bwd.ops) {
    const int dst = o.kind == Op::MV ? P.mv[o.index].dst : P.prod[o.index].dst;
    for (int r : (o.kind == Op::MV ? P.mv[o.index].row_out : P.prod[o.index].row_out)) written[dst][r] = 1;
  }
  P.zero_grads = false;
  for (size_t t = 0; t < P.tensors.size(); t++)
    if (P.tensors[t].grad)
      for (char w : written[t])
        if (!w) P.zero_grads = true;
}

// matrix-major work list of an operation with shared weights (see MVOp::unit_desc)
void build_units(MVOp &o)
{
  o.unit_desc.clear();
  o.slot_off.clear();
  o.unit_ent.clear();
  if (o.elem) return;
  for (const MVItem &it : o.items)
    if (it.n_in > 64) return;
  // input rows per unit: enough units per slot to occupy the warps of a CTA (GRACE_B200_UNIT_ROWS overrides, for tuning)
  int RMAX = 4;
  if (const char *env = getenv("GRACE_B200_UNIT_ROWS")) RMAX = std::max(1, atoi(env));
  int nslots = 0;
  for (size_t r = 0; r + 1 < o.item_off.size(); r++) nslots = std::max(nslots, o.item_off[r + 1] - o.item_off[r]);
  o.slot_off.push_back(0);
  for (int slot = 0; slot < nslots; slot++) {
    std::map<std::pair<int, int>, std::vector<MVItem>> by_mat;    // (mat, n_in) -> entries
    for (size_t r = 0; r + 1 < o.item_off.size(); r++) {
      const int i = o.item_off[r] + slot;
      if (i >= o.item_off[r + 1]) continue;
      MVItem e = o.items[i];
      const int mat = e.mat;
      e.mat = o.row_out[r];
      by_mat[{mat, e.n_in}].push_back(e);
    }
    for (auto &kv : by_mat)
      for (size_t c0 = 0; c0 < kv.second.size(); c0 += RMAX)
        for (int k0 = 0; k0 < o.n_out; k0 += 32) {
          const int e0 = (int) o.unit_ent.size();
          for (size_t c = c0; c < std::min(kv.second.size(), c0 + RMAX); c++) o.unit_ent.push_back(kv.second[c]);
          const int d[5] = {kv.first.first, kv.first.second, k0, e0, (int) o.unit_ent.size()};
          o.unit_desc.insert(o.unit_desc.end(), d, d + 5);
        }
    o.slot_off.push_back((int) o.unit_desc.size() / 5);
  }
}

}    // namespace

// ---- GRACE-3L ----------------------------------------------------------------------------------------------------
namespace {

// the dense chain of layer k as MV / PROD operations with their adjoints
void build_layer_3l(const GraceModel &gm, const Grace3LModel &m, int k, Layer3Plan &L)
{
  const std::string K = "A" + std::to_string(k + 1), ks = std::to_string(k + 1);
  const Grace3LModel::BondBasis &sp = m.bases[k];
  const int nl = m.lmax + 1, nlm = nl * nl, C = sp.channels;
  L.C = C;
  L.lt = sp.l_of_lm;
  auto find = [](const auto &v, const std::string &name) -> const auto & {
    for (const auto &c : v)
      if (c.name == name) return c;
    throw ModelError("GRACE-3L: component " + name + " is missing");
  };
  LayerBuilder B{L.dense, gm, {}};
  std::map<std::string, std::pair<int, int>> T;    // component -> (tensor, gradient)
  auto tensors = [&](const std::string &name, int nf, int ch) {
    const int t = B.tensor(name, nf, ch), g = B.tensor("g" + name, nf, ch, true);
    T[name] = {t, g};
    return std::make_pair(t, g);
  };
  // keep the reduce weights alive until the plan is finished (the builder reads them through pointers)
  std::vector<std::unique_ptr<ReduceWeights>> keep;
  auto reduce = [&](const std::string &name, const std::string &out_name, bool external) {
    const Grace3LModel::Collect &r = find(m.collects, name);
    const int nfo = r.invariant ? 1 : r.nfuncs;
    double scale = 1.0;
    if (r.row_scaled) {
      scale = r.row_scale[0];
      for (double v : r.row_scale)
        if (v != scale) throw ModelError("GRACE-3L: reduce " + name + " scales its output functions differently (norm_map)");
    }
    const auto out = tensors(out_name, nfo, r.width);
    if (external) L.dense.tensors[out.first].external = L.dense.tensors[out.second].external = true;
    ReduceGroup G;
    G.name = name;
    G.n_out = r.width;
    G.nfo = nfo;
    G.elem = r.per_element;
    G.t_out = out.first;
    G.t_gout = out.second;
    for (const auto &in : r.sources) {
      auto w = std::make_unique<ReduceWeights>();
      w->present = true;
      w->W = in.weight;
      w->norm = in.scale * scale;
      w->n_in = in.width;
      w->w_shape = in.tiles;
      w->n_out = r.width;
      w->elem = r.per_element;
      w->collect = in.pick;
      w->tile = in.tile_of;
      w->fo = in.into;
      if (r.invariant) w->fo.assign(in.pick.size(), 0);
      G.src.push_back(w.get());
      G.src_tensor.push_back(T.at(in.from).first);
      G.src_grad.push_back(T.at(in.from).second);
      G.src_row0.push_back(0);
      keep.push_back(std::move(w));
    }
    B.reduce(G);
    return out;
  };
  // projection of the functions of `src` by the matrix of their group: out[w] = norm M[group[w]] src[w]
  auto project = [&](const std::string &name, const std::string &src, const std::vector<double> &M, double norm,
                     const std::vector<int> &group, int ngroups, int rank, int n_in) {
    const int nf = (int) group.size();
    const auto out = tensors(name, nf, rank);
    auto w = std::make_unique<ReduceWeights>();
    w->present = true;
    w->W.assign((size_t) rank * n_in * ngroups, 0.0);    // [rank][n_in][group] from [group][rank][n_in]
    for (int g = 0; g < ngroups; g++)
      for (int r = 0; r < rank; r++)
        for (int n = 0; n < n_in; n++) w->W[((size_t) r * n_in + n) * ngroups + g] = M[((size_t) g * rank + r) * n_in + n];
    w->norm = norm;
    w->n_in = n_in;
    w->w_shape = ngroups;
    w->n_out = rank;
    w->tile = group;
    for (int f = 0; f < nf; f++) {
      w->collect.push_back(f);
      w->fo.push_back(f);
    }
    ReduceGroup G;
    G.name = name;
    G.n_out = rank;
    G.nfo = nf;
    G.t_out = out.first;
    G.t_gout = out.second;
    G.src.push_back(w.get());
    G.src_tensor.push_back(T.at(src).first);
    G.src_grad.push_back(T.at(src).second);
    G.src_row0.push_back(0);
    keep.push_back(std::move(w));
    B.reduce(G);
  };
  auto product = [&](const std::string &name, const std::string &left, const std::string &right) {
    const Grace3LModel::LowRank &c = find(m.products, name);
    project(name + "_lp", left, c.U, c.scale_u, c.group_l, c.groups_l, c.rank, c.width_l);
    project(name + "_rp", right, c.V, c.scale_v, c.group_r, c.groups_r, c.rank, c.width_r);
    const auto out = tensors(name, c.n_out, c.rank);
    CGProduct p;
    p.present = true;
    p.left = c.term_l;
    p.right = c.term_r;
    p.m_sum = c.term_out;
    p.cg = c.coef;
    p.n_out = c.n_out;
    const std::vector<char> need(c.n_out, 1);
    B.prod(name, p, need, T.at(name + "_lp").first, T.at(name + "_rp").first, out.first, T.at(name + "_lp").second,
           T.at(name + "_rp").second, out.second);
  };
  // out = nof (left + W right): the left input passes through an identity
  auto dense = [&](const std::string &name, const std::string &left, const std::string &right) {
    const Grace3LModel::Mix &f = find(m.mixes, name);
    if (f.weighted_left) throw ModelError("GRACE-3L: FC " + name + " with weights on its left input");
    FCWeights w;
    w.present = true;
    w.n_out = f.width;
    w.n_in_left = f.width;
    w.n_in_right = f.in_right;
    w.tiles_left = 1;
    w.tiles_right = f.tiles_right;
    w.n_funcs = f.nf_left;
    w.w_left.assign((size_t) f.width * f.width, 0.0);
    for (int q = 0; q < f.width; q++) w.w_left[(size_t) q * f.width + q] = 1.0;
    w.w_right = f.w_right;
    w.norm_right = f.scale_right;
    w.tile_left.assign(f.nf_left, 0);
    w.tile_right = f.tile_right;
    w.collect_to = f.to;
    w.collect_from = f.from;
    w.nof = f.out_factor;
    const auto out = tensors(name, f.nf_left, f.width);
    const std::vector<char> live(f.nf_left, 1);
    B.fc(name, w, live, T.at(left).first, T.at(right).first, out.first, T.at(left).second, T.at(right).second, out.second);
  };

  std::string X = K;
  if (!sp.coupled) {
    L.nfA = nlm;
    L.nlmi = 1;
  } else {
    L.nfA = sp.n_coupled;
    L.nlmi = sp.n_msg;
  }
  const auto A = tensors(K, L.nfA, C);
  L.tA = A.first;
  L.tGA = A.second;
  L.dense.tensors[L.tA].external = L.dense.tensors[L.tGA].external = true;
  if (sp.coupled) {
    reduce(K + "_red", K + "_red", false);
    X = K + "_red";
  }
  product(K + "_2", X, X);
  reduce(K + "_2_red", K + "_2_red", false);
  dense(K + "_2a", K + "_2_red", X);
  product(K + "_3", K + "_2a", X);
  reduce(K + "_3_red", K + "_3_red", false);
  dense(K + "_2b", K + "_2_red", X);
  product(K + "_4", K + "_2b", K + "_2b");
  reduce(K + "_4_red", K + "_4_red", false);
  if (k < 2) {
    const auto eq = reduce("eq" + ks, "eq" + ks, true);
    L.tEQ = eq.first;
    L.tGEQ = eq.second;
    const Grace3LModel::MessageNorm &e = find(m.message_norms, "eq" + ks + "_norm");
    L.nfEQ = e.nfuncs;
    L.cEQ = e.width;
    L.eq_dw.assign(e.degree_weight.begin(), e.degree_weight.end());
    L.eq_mask.assign(e.centre_mask.begin(), e.centre_mask.end());
    L.eq_aff.assign(e.gain.begin(), e.gain.end());
    L.eq_e = e.group_of;
    L.eq_eps = e.eps;
    L.eq_center = e.centred;
  }
  const auto rho = reduce("rho" + ks, "rho" + ks, true);
  L.tRHO = rho.first;
  L.tGRHO = rho.second;
  const Grace3LModel::DensityNorm &rn = find(m.density_norms, "rho" + ks + "_norm");
  L.wr = rn.width;
  L.rho_n0 = rn.skip_first;
  L.rho_scale.assign(rn.gain.begin(), rn.gain.end());
  if (L.dense.tensors[L.tRHO].nfuncs != 1) throw ModelError("GRACE-3L: rho" + ks + " must be an invariant reduce");
  B.finish();
  compact_rows(L.dense);
  check_gradient_writers(L.dense);
  for (MVOp &o : L.dense.mv) build_units(o);
  L.dense.C = C;

  // the couple of the bond sums: by output function and by pair
  const int np = nlm * L.nlmi;
  L.cg_off.assign(L.nfA + 1, 0);
  L.cgt_off.assign(np + 1, 0);
  if (!sp.coupled) {
    for (int f = 0; f < nlm; f++) {
      L.cg_off[f + 1] = L.cgt_off[f + 1] = f + 1;
      L.cg_p.push_back(f);
      L.cgt_f.push_back(f);
      L.cg_v.push_back(1.0f);
      L.cgt_v.push_back(1.0f);
    }
    L.l0mask.assign(1, 1.0f);
    L.zproj.assign((size_t) m.n_elements * C, 1.0f);
  } else {
    std::vector<std::vector<std::pair<int, float>>> by_f(L.nfA), by_q(np);
    for (int q = 0; q < np; q++)
      for (int f = 0; f < L.nfA; f++) {
        const double v = sp.couple[(size_t) q * L.nfA + f];
        if (v != 0.0) {
          by_f[f].push_back({q, (float) v});
          by_q[q].push_back({f, (float) v});
        }
      }
    for (int f = 0; f < L.nfA; f++) {
      for (auto &e : by_f[f]) {
        L.cg_p.push_back(e.first);
        L.cg_v.push_back(e.second);
      }
      L.cg_off[f + 1] = (int) L.cg_p.size();
    }
    for (int q = 0; q < np; q++) {
      for (auto &e : by_q[q]) {
        L.cgt_f.push_back(e.first);
        L.cgt_v.push_back(e.second);
      }
      L.cgt_off[q + 1] = (int) L.cgt_f.size();
    }
    L.l0mask.assign(sp.msg_mask.begin(), sp.msg_mask.end());
    L.zproj.assign((size_t) m.n_elements * C, 0.0f);
    for (int e = 0; e < m.n_elements; e++)
      for (int c = 0; c < C; c++) {
        double v = 0.0;
        for (int q = 0; q < m.embedding; q++)
          v += m.embedding_table[(size_t) e * m.embedding + q] * sp.zc_weight[(size_t) q * C + c];
        L.zproj[(size_t) e * C + c] = (float) (v * sp.zc_scale);
      }
  }
}

}    // namespace

std::vector<float> radial_table_3l(const Grace3LModel &m, int k, int mu_i, int mu_j, int N)
{
  const Grace3LModel::BondBasis &sp = m.bases[k];
  const Grace3LModel::DenseStack &mlp = sp.radial;
  const int nl = m.lmax + 1, C = sp.channels, ne = m.embedding, nrb = m.nbasis, p = sp.env_p;
  const double *zi = m.embedding_table.data() + (size_t) mu_i * ne, *zj = m.embedding_table.data() + (size_t) mu_j * ne;
  // layer 1: the species weight of the neighbour is part of the table
  std::vector<double> fac(C, sp.inv_neigh);
  if (!sp.coupled)
    for (int c = 0; c < C; c++) {
      double v = 0.0;
      for (int e = 0; e < ne; e++) v += zj[e] * sp.z_weight[(size_t) e * C + c];
      fac[c] *= v * sp.z_scale;
    }
  std::vector<double> fv((size_t) (N + 1) * nl * C), dv(fv.size());
  const double h = 1.0 / N;
  for (int q = 0; q <= N; q++) {
    const double x = q * h, t = 2.0 * x - 1.0;
    std::vector<double> a(nrb + 2 * ne, 0.0), da(a.size(), 0.0);
    double Tp = 1.0, Tc = t, dTp = 0.0, dTc = 2.0;
    for (int b = 0; b < nrb; b++) {
      a[b] = Tc;
      da[b] = dTc;
      const double Tn = 2.0 * t * Tc - Tp, dTn = 2.0 * (2.0 * Tc + t * dTc) - dTp;
      Tp = Tc; dTp = dTc; Tc = Tn; dTc = dTn;
    }
    for (int e = 0; e < ne; e++) {
      a[nrb + e] = zi[e];
      a[nrb + ne + e] = zj[e];
    }
    for (int il = 0; il < mlp.depth; il++) {
      const int ni = mlp.fan_in[il], no = mlp.fan_out[il];
      std::vector<double> s(no, 0.0), ds(no, 0.0);
      for (int i = 0; i < ni; i++) {
        const double *w = mlp.weight[il].data() + (size_t) i * no;
        for (int j = 0; j < no; j++) {
          s[j] += w[j] * a[i];
          ds[j] += w[j] * da[i];
        }
      }
      for (int j = 0; j < no; j++) {
        s[j] *= mlp.scale[il];
        ds[j] *= mlp.scale[il];
        if (il < mlp.depth - 1) {
          if (!mlp.bias[il].empty()) s[j] += mlp.scale[il] * mlp.bias[il][j];
          const double sg = 1.0 / (1.0 + std::exp(-s[j]));
          ds[j] *= sg * (1.0 + s[j] * (1.0 - sg));
          s[j] *= sg;
        }
      }
      a.swap(s);
      da.swap(ds);
    }
    const double xp = std::pow(x, p), xp1 = xp * x, xp2 = xp1 * x;
    const double env = 1.0 - 0.5 * (p + 1) * (p + 2) * xp + p * (p + 2) * xp1 - 0.5 * p * (p + 1) * xp2;
    const double denv = 0.5 * p * (p + 1) * (p + 2) * (-std::pow(x, p - 1) + 2.0 * xp - xp1);
    for (int c = 0; c < C; c++)
      for (int l = 0; l < nl; l++) {
        const int o = c * nl + l;
        fv[((size_t) q * nl + l) * C + c] = a[o] * env * fac[c];
        dv[((size_t) q * nl + l) * C + c] = h * (da[o] * env + a[o] * denv) * fac[c];
      }
  }
  std::vector<float> tab((size_t) N * nl * C * 4);
  for (int q = 0; q < N; q++)
    for (int l = 0; l < nl; l++)
      for (int c = 0; c < C; c++) {
        const size_t i0 = ((size_t) q * nl + l) * C + c, i1 = ((size_t) (q + 1) * nl + l) * C + c;
        const double f0 = fv[i0], f1 = fv[i1], d0 = dv[i0], d1 = dv[i1];
        float *o = tab.data() + i0 * 4;
        o[0] = (float) f0;
        o[1] = (float) d0;
        o[2] = (float) (-3.0 * f0 - 2.0 * d0 + 3.0 * f1 - d1);
        o[3] = (float) (2.0 * f0 + d0 - 2.0 * f1 + d1);
      }
  return tab;
}

static ModelPlan build_plan_3l(const GraceModel &gm, int spline_n)
{
  const Grace3LModel &m = *gm.m3;
  ModelPlan P;
  P.layers = 3;
  P.lmax = m.lmax;
  P.nlm = (m.lmax + 1) * (m.lmax + 1);
  P.n_elements = m.n_elements;
  P.rcsq.resize((size_t) m.n_elements * m.n_elements);
  P.rc.resize(P.rcsq.size());
  for (int a = 0; a < m.n_elements; a++)
    for (int b = 0; b < m.n_elements; b++) {
      const double rc = gm.pair_cutoff(a, b);
      P.rc[(size_t) a * m.n_elements + b] = rc;
      P.rcsq[(size_t) a * m.n_elements + b] = rc * rc;
      P.rc_max = std::max(P.rc_max, rc);
    }
  P.out_scale = m.energy_scale;
  P.shift = m.energy_shift;
  P.p3 = std::make_shared<Plan3L>();
  Plan3L &Q = *P.p3;
  Q.model = gm.m3;
  Q.spline_n = spline_n;
  for (int k = 0; k < 3; k++) build_layer_3l(gm, m, k, Q.L[k]);
  for (int k = 0; k < 2; k++)
    if (Q.L[k].nfEQ != Q.L[k + 1].nlmi || Q.L[k].cEQ != Q.L[k + 1].C)
      throw ModelError("GRACE-3L: the message of layer " + std::to_string(k + 1) + " does not fit the next layer");
  if (Q.L[0].wr != Q.L[1].wr || Q.L[0].wr != Q.L[2].wr) throw ModelError("GRACE-3L: densities of different widths");
  const Grace3LModel::DenseStack &e = m.readout;
  if (e.depth != 2 || e.fan_out[1] != 1 || e.fan_in[0] != Q.L[0].wr - 1 || e.fan_out[0] > 256 || e.fan_in[0] > 128)
    throw ModelError("GRACE-3L: the energy MLP must have two layers of at most 128 inputs and 256 hidden units");
  Q.eW0 = e.weight[0];
  Q.eW1 = e.weight[1];
  Q.en0 = e.scale[0];
  Q.en1 = e.scale[1];
  Q.e_nin = e.fan_in[0];
  Q.e_nh = e.fan_out[0];
  Q.e_act = m.readout_act;
  return P;
}

ModelPlan build_plan(const GraceModel &m, int spline_n)
{
  if (spline_n < 16) throw std::invalid_argument("spline N must be >= 16");
  ModelPlan P;
  if (m.layers == 3) return build_plan_3l(m, spline_n);
  // (P is filled below for GRACE-1L / GRACE-2L)
  P.layers = m.layers;
  P.lmax = m.lmax;
  const int nl = m.lmax + 1, nlm = nl * nl;
  P.nlm = nlm;
  P.n_elements = m.n_elements;
  P.rcsq.resize((size_t) m.n_elements * m.n_elements);
  P.rc.resize(P.rcsq.size());
  for (int a = 0; a < m.n_elements; a++)
    for (int b = 0; b < m.n_elements; b++) {
      const double rc = m.pair_cutoff(a, b);
      P.rc[(size_t) a * m.n_elements + b] = rc;
      P.rcsq[(size_t) a * m.n_elements + b] = rc * rc;
      P.rc_max = std::max(P.rc_max, rc);
    }
  P.nrho = m.rho_n_out;
  // UQ head: evaluated only if it passes the checks (the message is raised when a caller asks for UQ)
  bool uq_ok = m.uq.present;
  if (uq_ok) {
    try {
      m.validate_uq();
    } catch (const std::exception &) {
      uq_ok = false;
    }
  }
  int uq_rows_l2 = 0;    // GRACE-2L: the I2 block comes first in the projection matrix (libgrace/src/model_2l.cpp:520-535)
  if (uq_ok && m.layers == 2)
    for (const ReduceWeights &r : m.I2) uq_rows_l2 += r.present ? r.n_in * (int) r.collect.size() : 0;

  {    // layer 1
    LayerPlan &L = P.L1;
    LayerBuilder B{L, m, {}};
    const Chain &c = m.chain1;
    L.C = c.c0;
    L.n_msg = 0;
    L.radial = build_radial(m, m.rad1, c.c0, spline_n);
    L.z.assign(m.zA.begin(), m.zA.end());
    L.tQ = B.tensor("A", nlm, c.c0);
    L.tGQ = B.tensor("gA", nlm, c.c0, true);
    L.tensors[L.tQ].external = L.tensors[L.tGQ].external = true;
    // with AAA = AA1 x A1 no adjoint reads A itself, so its gradient may take over its storage
    if (!c.xxx_right_x0) L.tensors[L.tGQ].alias = L.tQ;
    std::vector<const ReduceWeights *> rXX{&m.rho[1]}, rXXX{&m.rho[2]}, rXXXX{c.order4 ? &m.rho[3] : nullptr};
    if (m.layers == 2) {
      rXX.push_back(&m.I1[1]);
      rXXX.push_back(&m.I1[2]);
      rXXXX.push_back(c.order4 ? &m.I1[3] : nullptr);
    }
    const auto T = B.chain("A", c, L.tQ, L.tGQ, rXX, rXXX, rXXXX);
    P.t1_rho = B.tensor("rho", 1, m.rho_n_out);
    P.t1_grho = B.tensor("grho", 1, m.rho_n_out);    // written by the readout, not zeroed
    L.tensors[P.t1_rho].external = L.tensors[P.t1_grho].external = true;
    if (m.layers == 2) {
      const int tI1 = B.tensor("I1", m.nI1, m.i1_out), gI1 = B.tensor("gI1", m.nI1, m.i1_out, true);
      P.t1_I = B.tensor("I", m.nI, m.cr);
      P.t1_gI = B.tensor("gI", m.nI, m.cr);    // copied from the per-atom dE/dI rows, not zeroed
      L.tensors[P.t1_I].external = L.tensors[P.t1_gI].external = true;
      B.reduce(B.reduce4("I1", m.I1, T, c.order4, m.i1_out, m.nI1, true, tI1, gI1));
      B.reduce(B.reduce4("rho", m.rho, T, c.order4, m.rho_n_out, 1, true, P.t1_rho, P.t1_grho));
      if (uq_ok) B.uq_projection(B.reduce4("rho", m.rho, T, c.order4, m.rho_n_out, 1, true, P.t1_rho, P.t1_grho), m.uq, uq_rows_l2);
      ReduceGroup R;
      R.name = "I";
      R.src = {&m.I_from_I1};
      R.src_tensor = {tI1};
      R.src_grad = {gI1};
      R.src_row0 = {0};
      R.n_out = m.cr; R.nfo = m.nI; R.elem = false; R.t_out = P.t1_I; R.t_gout = P.t1_gI;
      B.reduce(R);
    } else {
      B.reduce(B.reduce4("rho", m.rho, T, c.order4, m.rho_n_out, 1, true, P.t1_rho, P.t1_grho));
      if (uq_ok) B.uq_projection(B.reduce4("rho", m.rho, T, c.order4, m.rho_n_out, 1, true, P.t1_rho, P.t1_grho), m.uq, 0);
    }
    B.finish();
  }
  if (m.layers == 2) {
    LayerPlan &L = P.L2;
    LayerBuilder B{L, m, {}};
    const Chain &c = m.chain2;
    P.nI = m.nI;
    P.cr = m.cr;
    L.C = m.cr;
    L.n_msg = m.nI;
    L.radial = build_radial(m, m.rad2, m.cr, spline_n);
    L.z.assign(m.zB0.begin(), m.zB0.end());
    // bond sum Q[(I, lm)] = sum_j Y_lm R1[l] msg_I, I < nI the neighbour's message functions, I = nI the chemical
    // weight (B0): the dense form of the YI pairs (libgrace/src/fused_2l.cpp:229-276)
    const int nq = (m.nI + 1) * nlm;
    L.tQ = B.tensor("Q", nq, m.cr);
    L.tGQ = B.tensor("gQ", nq, m.cr, true);
    L.tensors[L.tQ].external = L.tensors[L.tGQ].external = true;
    L.tensors[L.tGQ].alias = L.tQ;    // Q is read by the forward YI / B operations only
    const int tYI = B.tensor("YI", m.yi.n_out, m.cr), gYI = B.tensor("gYI", m.yi.n_out, m.cr, true);
    L.tensors[gYI].alias = tYI;
    {
      CGProduct y;    // YI[o] = inv_avg sum_t cg_t Q[I_t nlm + y_t]
      y.present = true;
      y.n_out = m.yi.n_out;
      for (size_t t = 0; t < m.yi.cg.size(); t++) {
        y.left.push_back(m.yi.i[t] * nlm + m.yi.y[t]);
        y.right.push_back(0);
        y.m_sum.push_back(m.yi.m_sum[t]);
        y.cg.push_back(m.yi.cg[t] * m.yi.inv_avg);
      }
      ProdOp F, A;
      F.name = "YI:fwd"; A.name = "YI:adj";
      F.dst = tYI; F.srcA = L.tQ; F.srcB = -1;
      A.dst = L.tGQ; A.srcA = gYI; A.srcB = -1; A.accumulate = true;
      std::map<int, std::vector<int>> by_o, by_l;
      for (size_t t = 0; t < y.cg.size(); t++) {
        by_o[y.m_sum[t]].push_back((int) t);
        by_l[y.left[t]].push_back((int) t);
      }
      for (auto &kv : by_o) {
        F.row_out.push_back(kv.first);
        F.term_off.push_back((int) F.terms.size());
        for (int t : kv.second) F.terms.push_back({y.left[t], 0, (float) y.cg[t]});
      }
      for (auto &kv : by_l) {
        A.row_out.push_back(kv.first);
        A.term_off.push_back((int) A.terms.size());
        for (int t : kv.second) A.terms.push_back({y.m_sum[t], 0, (float) y.cg[t]});
      }
      const Op f = B.add(std::move(F));
      B.emit(f, {B.add(std::move(A))});
    }
    const int tB = B.tensor("B", m.nB, c.c0), gB = B.tensor("gB", m.nB, c.c0, true);
    {
      ReduceGroup R;
      R.name = "B";
      R.src = {&m.B_from_YI, &m.B_from_B0};
      R.src_tensor = {tYI, L.tQ};
      R.src_grad = {gYI, L.tGQ};
      R.src_row0 = {0, m.nI * nlm};
      R.n_out = c.c0; R.nfo = m.nB; R.elem = false; R.t_out = tB; R.t_gout = gB;
      B.reduce(R);
    }
    const auto T = B.chain("B", c, tB, gB, {&m.I2[1]}, {&m.I2[2]}, {c.order4 ? &m.I2[3] : nullptr});
    P.t2_I2 = B.tensor("I2", 1, m.nI2);
    P.t2_gI2 = B.tensor("gI2", 1, m.nI2);
    L.tensors[P.t2_I2].external = L.tensors[P.t2_gI2].external = true;
    B.reduce(B.reduce4("I2", m.I2, T, c.order4, m.nI2, 1, true, P.t2_I2, P.t2_gI2));
    if (uq_ok) B.uq_projection(B.reduce4("I2", m.I2, T, c.order4, m.nI2, 1, true, P.t2_I2, P.t2_gI2), m.uq, 0);
    B.finish();
  }
  compact_rows(P.L1);
  check_gradient_writers(P.L1);
  if (m.layers == 2) {
    compact_rows(P.L2);
    check_gradient_writers(P.L2);
  }
  for (LayerPlan *L : {&P.L1, &P.L2})
    for (MVOp &o : L->mv) build_units(o);
  // readout
  for (const auto &Lr : m.energy_mlp) {
    P.eW.insert(P.eW.end(), Lr.W.begin(), Lr.W.end());
    P.e_nin.push_back(Lr.n_in);
    P.e_nout.push_back(Lr.n_out);
    P.e_norm.push_back(Lr.norm);
  }
  P.e_act = m.energy_activation;
  P.e_ln = m.energy_ln;
  P.rms = m.rms;
  P.out_scale = m.output_scale;
  P.shift = m.shift;
  P.lnI = m.lnI;
  P.ln0 = m.ln0;
  if (uq_ok) {
    UqPlan &u = P.uq;
    u.ready = true;
    u.rp_dim = m.uq.rp_dim; u.feature_dim = m.uq.feature_dim; u.n_density = m.uq.n_density;
    u.max_clusters = m.uq.max_clusters; u.density_scale = m.uq.density_scale;
    u.centroids = m.uq.centroids; u.inv_cov = m.uq.inv_cov; u.thresholds = m.uq.thresholds; u.n_clusters = m.uq.n_clusters;
  }
  for (const LayerPlan *L : {&P.L1, &P.L2}) {
    for (size_t q = 0; q < L->mv.size(); q++)
      if ((int) q != L->uq_mv) P.dense_flops_per_atom += L->mv[q].flops_per_atom();
    for (const auto &o : L->prod)    // 3 flop per (term, channel): libgrace/include/grace/fused_cpu.h:411-429
      P.dense_flops_per_atom += 3.0 * (double) o.terms.size() * L->tensors[o.dst].channels;
  }
  return P;
}

}    // namespace gb
