// fp64 readout shared by the per-chunk readout kernels and the fused dense-network kernel
// (libgrace/src/fused_1l.cpp:378-427, libgrace/src/fused_2l.cpp:548-615).
#pragma once

#include "kernels.h"

namespace gb {

// ---- readouts (fp64, one thread per atom) ---------------------------------------------------------------------
constexpr int RW = 128;    // largest width of the energy MLP (checked on the host)

// value of the MLP on x[0..nin) and, with g_out, its gradient dvalue/dx scaled by out_scale
__device__ inline double energy_mlp(const ReadoutDev &r, double *x, int nin, double *g_out)
{
  double x0[RW], pre[3][RW], h[RW];
  double q = 0.0;
  if (r.ln) {    // legacy: RMS layer norm of the input (libgrace/include/grace/fused_cpu.h:664-681)
    double ms = 0.0;
    for (int k = 0; k < nin; k++) { x0[k] = x[k]; ms += x[k] * x[k]; }
    q = 1.0 / sqrt(ms / nin + 1e-16);
    for (int k = 0; k < nin; k++) x[k] *= q;
  }
  for (int k = 0; k < nin; k++) h[k] = x[k];
  const double *W = r.W;
  for (int L = 0; L < r.nlay; L++) {
    double v[RW];
    for (int c = 0; c < r.n_out[L]; c++) v[c] = 0.0;
    for (int a = 0; a < r.n_in[L]; a++) {
      const double xa = h[a];
      const double *Wr = W + (size_t) a * r.n_out[L];
      for (int c = 0; c < r.n_out[L]; c++) v[c] += xa * Wr[c];
    }
    for (int c = 0; c < r.n_out[L]; c++) {
      v[c] *= r.norm[L];
      if (L < r.nlay - 1) {
        pre[L][c] = v[c];
        h[c] = (r.act == 1) ? tanh(v[c]) : v[c] / (1.0 + exp(-v[c]));
      } else {
        h[c] = v[c];
      }
    }
    W += (size_t) r.n_in[L] * r.n_out[L];
  }
  const double val = h[0];
  if (!g_out) return val;
  double g[RW], gn[RW];
  g[0] = r.out_scale;
  for (int L = r.nlay - 1; L >= 0; L--) {
    W -= (size_t) r.n_in[L] * r.n_out[L];
    if (L < r.nlay - 1)
      for (int c = 0; c < r.n_out[L]; c++) {
        const double v = pre[L][c];
        if (r.act == 1) {
          const double t = tanh(v);
          g[c] *= 1.0 - t * t;
        } else {
          const double sg = 1.0 / (1.0 + exp(-v));
          g[c] *= sg * (1.0 + v * (1.0 - sg));
        }
      }
    for (int a = 0; a < r.n_in[L]; a++) {
      const double *Wr = W + (size_t) a * r.n_out[L];
      double s = 0.0;
      for (int c = 0; c < r.n_out[L]; c++) s += g[c] * Wr[c];
      gn[a] = s * r.norm[L];
    }
    for (int a = 0; a < r.n_in[L]; a++) g[a] = gn[a];
  }
  if (r.ln) {
    double t = 0.0;
    for (int k = 0; k < nin; k++) t += g[k] * x0[k];
    for (int k = 0; k < nin; k++) g[k] = q * (g[k] - x0[k] * t * q * q / nin);
  }
  for (int k = 0; k < nin; k++) g_out[k] = g[k];
  return val;
}


// GRACE-2L: RMSNorms of rho[1:] and I2, MLP on their sum, and the reverse; returns E_i (without writing it)
__device__ inline double readout_2l_atom(const ReadoutDev &r, const float *rho, const float *i2, int mu, double *gr,
                                         float *go, bool want_grad, bool owned = true)
{
  const int nr = r.nrho;
  if (!owned) {    // a ghost atom: no energy of its own, no gradient seed
    if (want_grad)
      for (int k = 0; k < nr; k++) { gr[k] = 0.0; go[k] = 0.0f; }
    return 0.0;
  }
  double ms1 = 0.0, ms0 = 0.0;
  for (int k = 1; k < nr; k++) ms1 += (double) rho[k] * rho[k];
  for (int k = 0; k < nr; k++) ms0 += (double) i2[k] * i2[k];
  const double eps = 1e-10;
  const double s1 = r.rms ? sqrt(ms1 / (nr - 1) + eps) : 1.0, s0 = r.rms ? sqrt(ms0 / nr + eps) : 1.0;
  double x[RW], g[RW];
  for (int k = 1; k < nr; k++) x[k - 1] = rho[k] / s1 * r.lnI[k - 1] + i2[k] / s0 * r.ln0[k];
  const double val = energy_mlp(r, x, nr - 1, want_grad ? g : nullptr);
  const double e = (val + (double) rho[0] + (double) i2[0] / s0 * r.ln0[0]) * r.out_scale + r.shift[mu];
  if (!want_grad) return e;
  gr[0] = r.out_scale;
  double t1 = 0.0;
  if (r.rms)
    for (int k = 1; k < nr; k++) t1 += g[k - 1] * r.lnI[k - 1] * rho[k];
  for (int k = 1; k < nr; k++) gr[k] = g[k - 1] * r.lnI[k - 1] / s1 - rho[k] * t1 / ((nr - 1) * s1 * s1 * s1);
  double t0 = 0.0;
  if (r.rms) {
    t0 = r.out_scale * r.ln0[0] * i2[0];
    for (int k = 1; k < nr; k++) t0 += g[k - 1] * r.ln0[k] * i2[k];
  }
  for (int k = 0; k < nr; k++) {
    const double gy = k == 0 ? r.out_scale : g[k - 1];
    go[k] = (float) (gy * r.ln0[k] / s0 - i2[k] * t0 / (nr * s0 * s0 * s0));
  }
  return e;
}

// GRACE-1L: E_i = (MLP(rho[1:]) + rho[0]) scale + shift and dE/drho
__device__ inline double readout_1l_atom(const ReadoutDev &r, const float *ra, int mu, float *ga, bool want_grad,
                                         bool owned = true)
{
  const int nr = r.nrho;
  if (!owned) {
    if (want_grad)
      for (int k = 0; k < nr; k++) ga[k] = 0.0f;
    return 0.0;
  }
  double x[RW], g[RW];
  for (int k = 1; k < nr; k++) x[k - 1] = ra[k];
  const double val = energy_mlp(r, x, nr - 1, want_grad ? g : nullptr);
  if (want_grad) {
    ga[0] = (float) r.out_scale;
    for (int k = 1; k < nr; k++) ga[k] = (float) g[k - 1];
  }
  return (val + (double) ra[0]) * r.out_scale + r.shift[mu];
}

}    // namespace gb
