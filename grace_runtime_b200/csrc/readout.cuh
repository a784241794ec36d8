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

// ---- the same readouts by one warp per atom: lane l owns the channels l, l + 32, l + 64, l + 96 of every vector, a
// matrix-vector product broadcasts one input channel at a time by shuffle and reads a coalesced weight row; the
// reverse uses the transposed copies of the weights (WT) the same way.  fp64 throughout, same formulas as above.
constexpr int RJ = RW / 32;

__device__ inline double warp_sum(double v)
{
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}

__device__ inline double act_value(int act, double v) { return act == 1 ? tanh(v) : v / (1.0 + exp(-v)); }
__device__ inline double act_slope(int act, double v)
{
  if (act == 1) {
    const double t = tanh(v);
    return 1.0 - t * t;
  }
  const double sg = 1.0 / (1.0 + exp(-v));
  return sg * (1.0 + v * (1.0 - sg));
}

// x, g: this lane's channels; returns the value (all lanes); g = dvalue/dx scaled by out_scale when want_grad
__device__ inline double energy_mlp_warp(const ReadoutDev &r, double (&x)[RJ], int nin, double (&g)[RJ], bool want_grad)
{
  const int lane = threadIdx.x & 31;
  double x0[RJ], pre[3][RJ], h[RJ];
  double q = 0.0;
#pragma unroll
  for (int j = 0; j < RJ; j++) {
    if (lane + 32 * j >= nin) x[j] = 0.0;
    x0[j] = x[j];
  }
  if (r.ln) {
    double ms = 0.0;
#pragma unroll
    for (int j = 0; j < RJ; j++) ms += x[j] * x[j];
    ms = warp_sum(ms);
    q = 1.0 / sqrt(ms / nin + 1e-16);
#pragma unroll
    for (int j = 0; j < RJ; j++) x[j] *= q;
  }
#pragma unroll
  for (int j = 0; j < RJ; j++) h[j] = x[j];
  const double *W = r.W;
  for (int L = 0; L < r.nlay; L++) {
    const int n_in = r.n_in[L], n_out = r.n_out[L];
    double v[RJ];
#pragma unroll
    for (int j = 0; j < RJ; j++) v[j] = 0.0;
#pragma unroll
    for (int ja = 0; ja < RJ; ja++) {
      if (ja * 32 >= n_in) break;
      const int la = min(32, n_in - ja * 32);
      for (int l = 0; l < la; l++) {
        const double ha = __shfl_sync(0xffffffffu, h[ja], l);
        const double *Wr = W + (size_t) (ja * 32 + l) * n_out + lane;
#pragma unroll
        for (int j = 0; j < RJ; j++)
          if (lane + 32 * j < n_out) v[j] += ha * Wr[32 * j];
      }
    }
#pragma unroll
    for (int j = 0; j < RJ; j++) {
      v[j] *= r.norm[L];
      if (L < r.nlay - 1) {
        if (L < 3) pre[L][j] = v[j];
        h[j] = lane + 32 * j < n_out ? act_value(r.act, v[j]) : 0.0;
      } else {
        h[j] = v[j];
      }
    }
    W += (size_t) n_in * n_out;
  }
  const double val = __shfl_sync(0xffffffffu, h[0], 0);
  if (!want_grad) return val;
#pragma unroll
  for (int j = 0; j < RJ; j++) g[j] = 0.0;
  if (lane == 0) g[0] = r.out_scale;
  const double *WT = r.WT + (W - r.W);
  for (int L = r.nlay - 1; L >= 0; L--) {
    const int n_in = r.n_in[L], n_out = r.n_out[L];
    WT -= (size_t) n_in * n_out;
    if (L < r.nlay - 1) {
#pragma unroll
      for (int j = 0; j < RJ; j++) g[j] = lane + 32 * j < n_out ? g[j] * act_slope(r.act, pre[L][j]) : 0.0;
    }
    double gn[RJ];
#pragma unroll
    for (int j = 0; j < RJ; j++) gn[j] = 0.0;
#pragma unroll
    for (int jc = 0; jc < RJ; jc++) {
      if (jc * 32 >= n_out) break;
      const int lc = min(32, n_out - jc * 32);
      for (int l = 0; l < lc; l++) {
        const double gc = __shfl_sync(0xffffffffu, g[jc], l);
        const double *Wr = WT + (size_t) (jc * 32 + l) * n_in + lane;
#pragma unroll
        for (int j = 0; j < RJ; j++)
          if (lane + 32 * j < n_in) gn[j] += gc * Wr[32 * j];
      }
    }
#pragma unroll
    for (int j = 0; j < RJ; j++) g[j] = gn[j] * r.norm[L];
  }
  if (r.ln) {
    double t = 0.0;
#pragma unroll
    for (int j = 0; j < RJ; j++) t += g[j] * x0[j];
    t = warp_sum(t);
#pragma unroll
    for (int j = 0; j < RJ; j++) g[j] = q * (g[j] - x0[j] * t * q * q / nin);
  }
  return val;
}

// GRACE-1L, one warp: lane 0 holds the returned energy; ga (dE/drho of the atom) is written by the lanes
__device__ inline double readout_1l_warp(const ReadoutDev &r, const float *ra, int mu, float *ga, bool want_grad, bool owned)
{
  const int lane = threadIdx.x & 31, nr = r.nrho;
  if (!owned) {
    if (want_grad)
      for (int k = lane; k < nr; k += 32) ga[k] = 0.0f;
    return 0.0;
  }
  double x[RJ], g[RJ];
#pragma unroll
  for (int j = 0; j < RJ; j++) x[j] = lane + 32 * j < nr - 1 ? (double) ra[lane + 32 * j + 1] : 0.0;
  const double val = energy_mlp_warp(r, x, nr - 1, g, want_grad);
  if (want_grad) {
    if (lane == 0) ga[0] = (float) r.out_scale;
#pragma unroll
    for (int j = 0; j < RJ; j++)
      if (lane + 32 * j < nr - 1) ga[lane + 32 * j + 1] = (float) g[j];
  }
  return (val + (double) ra[0]) * r.out_scale + r.shift[mu];
}

// GRACE-2L, one warp
__device__ inline double readout_2l_warp(const ReadoutDev &r, const float *rho, const float *i2, int mu, double *gr,
                                         float *go, bool want_grad, bool owned)
{
  const int lane = threadIdx.x & 31, nr = r.nrho;
  if (!owned) {
    if (want_grad)
      for (int k = lane; k < nr; k += 32) { gr[k] = 0.0; go[k] = 0.0f; }
    return 0.0;
  }
  // this lane's channels c = lane + 32 j of x[0 .. nr - 1) are rho[c + 1], i2[c + 1]
  double rh[RJ], iv[RJ], ms1 = 0.0, ms0 = 0.0;
#pragma unroll
  for (int j = 0; j < RJ; j++) {
    const int c = lane + 32 * j;
    rh[j] = c < nr - 1 ? (double) rho[c + 1] : 0.0;
    iv[j] = c < nr - 1 ? (double) i2[c + 1] : 0.0;
    ms1 += rh[j] * rh[j];
    ms0 += iv[j] * iv[j];
  }
  const double i20 = (double) i2[0], rho0 = (double) rho[0];
  ms1 = warp_sum(ms1);
  ms0 = warp_sum(ms0) + i20 * i20;
  const double eps = 1e-10;
  const double s1 = r.rms ? sqrt(ms1 / (nr - 1) + eps) : 1.0, s0 = r.rms ? sqrt(ms0 / nr + eps) : 1.0;
  double x[RJ], g[RJ], lI[RJ], l0[RJ];
#pragma unroll
  for (int j = 0; j < RJ; j++) {
    const int c = lane + 32 * j;
    lI[j] = c < nr - 1 ? r.lnI[c] : 0.0;
    l0[j] = c < nr - 1 ? r.ln0[c + 1] : 0.0;
    x[j] = rh[j] / s1 * lI[j] + iv[j] / s0 * l0[j];
  }
  const double val = energy_mlp_warp(r, x, nr - 1, g, want_grad);
  const double e = (val + rho0 + i20 / s0 * r.ln0[0]) * r.out_scale + r.shift[mu];
  if (!want_grad) return e;
  double t1 = 0.0, t0 = 0.0;
  if (r.rms) {
#pragma unroll
    for (int j = 0; j < RJ; j++) {
      t1 += g[j] * lI[j] * rh[j];
      t0 += g[j] * l0[j] * iv[j];
    }
    t1 = warp_sum(t1);
    t0 = warp_sum(t0) + r.out_scale * r.ln0[0] * i20;
  }
  if (lane == 0) {
    gr[0] = r.out_scale;
    go[0] = (float) (r.out_scale * r.ln0[0] / s0 - i20 * t0 / (nr * s0 * s0 * s0));
  }
#pragma unroll
  for (int j = 0; j < RJ; j++) {
    const int c = lane + 32 * j;
    if (c < nr - 1) {
      gr[c + 1] = g[j] * lI[j] / s1 - rh[j] * t1 / ((nr - 1) * s1 * s1 * s1);
      go[c + 1] = (float) (g[j] * l0[j] / s0 - iv[j] * t0 / (nr * s0 * s0 * s0));
    }
  }
  return e;
}

}    // namespace gb
