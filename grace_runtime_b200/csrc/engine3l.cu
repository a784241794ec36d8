// GRACE-3L evaluation: three message-passing layers (libgrace/src/fused_3l.cpp:1204-1637).  Per layer: the bond sums of
// the single-particle basis (per-pair radial tables, spherical harmonics, the normalised message of the layer before
// coupled in through the sparse cg_W), the dense chain of the layer as MV / PROD operations of the plan (cp_l
// projections, couples, reduces, FCs: the same kernels as GRACE-1L / 2L), EquivariantRMSNorm of the message and RMSNorm
// of the density; the readout on the sum of the three densities; then everything in reverse.  All tensors of the three
// layers are kept for the reverse pass and every atom is evaluated in one pass: this first form of the path is written
// for clarity and checked against the reference's CPU engine, not tuned.
#include "engine.h"

#include "bond_common.cuh"

#include <algorithm>

namespace gb {

namespace {

struct Spbf3Dev {
  const float *tab;          // [pair][N][nl][C][4] cubic Hermite coefficients
  const int *pair_slot;      // [n_elements^2] table of the element pair (centre, neighbour), -1: none
  long long tab_stride;      // floats per pair
  const float *rc;           // [n_elements^2]
  const float *msg;          // [n][nlmi][C] normalised message of the layer before (null: layer 1)
  float *gmsg;               // [n][nlmi][C] its gradient, added to atomically (null: layer 1)
  const float *zproj;        // [n_elements][C]
  const float *l0mask;       // [nlmi]
  const int *lt;             // [nlm]
  const int *cg_off, *cg_p, *cgt_off, *cgt_f;
  const float *cg_v, *cgt_v;
  int N, C, nl, nlm, nlmi, nfA, nel;
};

constexpr int S3_THREADS = 512;

// Y (and its gradient) of one bond by one thread; lm < nlm are kept
__device__ void stage_harmonics(const SHTable &sht, float ux, float uy, float uz, int nlm, float *Y, float *G)
{
  sph_harm<4, true>(sht, ux, uy, uz, [&](int lm, float v, float gx, float gy, float gz) {
    if (lm < nlm) {
      Y[lm] = v;
      if (G) {
        G[3 * lm] = gx;
        G[3 * lm + 1] = gy;
        G[3 * lm + 2] = gz;
      }
    }
  });
}

constexpr int S3_BB = 64;    // bonds whose harmonics are staged at once

// Thread layout of both kernels: c = tid % C is the thread's channel, g = tid / C its group (G = 512 / C groups; threads
// beyond G C idle in the per-channel loops), so that the loops over (function, channel) need no divisions.

// A[f][a][c] = sum_q cg[q, f] P[q][c],  P[(ly, li)][c] = sum_bonds Y_ly R[l(ly)][c] (msg_j[li][c] + mask[li] zproj[mu_j][c])
__global__ void __launch_bounds__(S3_THREADS) spbf3_fwd_kernel(BondsDev b, Spbf3Dev L, SHTable sht, float *__restrict__ A, int NA)
{
  extern __shared__ float sm[];
  const int C = L.C, np = L.nlm * L.nlmi, nlm = L.nlm, nlmi = L.nlmi;
  float *P = sm, *Ys = P + (size_t) np * C, *U = Ys + S3_BB * nlm, *Ic = U + (size_t) nlm * C;
  const int i = blockIdx.x, tid = threadIdx.x;
  const int G = S3_THREADS / C, c = tid % C, g = tid / C;
  const bool live = g < G;
  const long long base = b.off[i];
  const int nb = b.cnt[i], mui = b.mu[i];
  for (int e = tid; e < np * C; e += S3_THREADS) P[e] = 0.0f;
  for (int q0 = 0; q0 < nb; q0 += S3_BB) {
    const int nq = min(S3_BB, nb - q0);
    __syncthreads();    // the harmonics of the previous batch are no longer read
    if (tid < nq) {
      const float4 rec = b.rec[base + q0 + tid];
      const float ir = rsqrtf(rec.x * rec.x + rec.y * rec.y + rec.z * rec.z);
      stage_harmonics(sht, rec.x * ir, rec.y * ir, rec.z * ir, nlm, Ys + tid * nlm, nullptr);
    }
    for (int q = 0; q < nq; q++) {
      const float4 rec = b.rec[base + q0 + q];
      const int j = __float_as_int(rec.w), muj = b.mu[j];
      const float r = sqrtf(rec.x * rec.x + rec.y * rec.y + rec.z * rec.z);
      const int slot = L.pair_slot[mui * L.nel + muj];
      if (slot < 0) continue;    // no table for this element pair (uniform over the block): the bond is left out
      int k0;
      float t;
      spline_locate(r / L.rc[mui * L.nel + muj], L.N, k0, t);
      __syncthreads();    // R and Ic of the previous bond are no longer read; the harmonics are staged
      const float4 *tab = reinterpret_cast<const float4 *>(L.tab + (size_t) slot * L.tab_stride) + (size_t) k0 * L.nl * C;
      if (live) {
        const float *Y = Ys + q * nlm;
        for (int ly = g; ly < nlm; ly += G) {    // U[ly][c] = Y_ly R_l(ly)[c]
          const float4 cf = tab[L.lt[ly] * C + c];
          U[ly * C + c] = Y[ly] * (cf.x + t * (cf.y + t * (cf.z + t * cf.w)));
        }
        for (int li = g; li < nlmi; li += G) {
          const float m = L.msg ? L.msg[((size_t) j * nlmi + li) * C + c] : 0.0f;
          Ic[li * C + c] = m + L.l0mask[li] * L.zproj[(size_t) muj * C + c];
        }
      }
      __syncthreads();
      if (live)
        for (int ly = g; ly < nlm; ly += G) {
          const float u = U[ly * C + c];
          float *p = P + (size_t) ly * nlmi * C + c;
#pragma unroll 5
          for (int li = 0; li < nlmi; li++) p[(size_t) li * C] = fmaf(u, Ic[li * C + c], p[(size_t) li * C]);
        }
    }
  }
  __syncthreads();
  if (live)
    for (int f = g; f < L.nfA; f += G) {
      float v = 0.0f;
      for (int t = L.cg_off[f]; t < L.cg_off[f + 1]; t++) v = fmaf(L.cg_v[t], P[L.cg_p[t] * C + c], v);
      A[((size_t) f * NA + i) * C + c] = v;
    }
}

// reverse of the above from gA: bond forces (written or added at the bond's slot), per-atom virial, dE/dmsg of the
// neighbours.  Per bond, with gP[(ly, li)][c] = sum_f cg[q, f] gA[f][c] staged once per atom:
//   W[ly][c] = sum_li gP Ic[li][c]              (owner threads: (ly, c))
//   dE/dmsg_j[li][c] += sum_ly gP Y_ly R_l[c]   (owner threads: (li, c); atomic on the neighbour's row)
//   gY[ly] = sum_c W R_l[c] (a warp per ly),  dE/dx = sum_{ly, c} W Y_ly dR_l[c]
__global__ void __launch_bounds__(S3_THREADS) spbf3_bwd_kernel(BondsDev b, Spbf3Dev L, SHTable sht, const float *__restrict__ gA,
                                                               int NA, float *__restrict__ fv, double *__restrict__ vir_atom, int add)
{
  extern __shared__ float sm[];
  const int C = L.C, np = L.nlm * L.nlmi, nlm = L.nlm, nlmi = L.nlmi;
  float *gP = sm, *Ys = gP + (size_t) np * C, *Gs = Ys + S3_BB * nlm, *R = Gs + 3 * S3_BB * nlm, *dR = R + (size_t) L.nl * C;
  float *Ic = dR + (size_t) L.nl * C, *gY = Ic + (size_t) nlmi * C, *W = gY + nlm, *U = W + (size_t) nlm * C;
  float *dedx = U + (size_t) nlm * C;
  const int i = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = S3_THREADS / C, c = tid % C, g = tid / C;
  const bool live = g < G;
  const long long base = b.off[i];
  const int nb = b.cnt[i], mui = b.mu[i];
  double vir[6] = {0.0, 0.0, 0.0, 0.0, 0.0, 0.0};
  if (live)
    for (int q = g; q < np; q += G) {
      float v = 0.0f;
      for (int t = L.cgt_off[q]; t < L.cgt_off[q + 1]; t++) v = fmaf(L.cgt_v[t], gA[((size_t) L.cgt_f[t] * NA + i) * C + c], v);
      gP[(size_t) q * C + c] = v;
    }
  for (int q0 = 0; q0 < nb; q0 += S3_BB) {
    const int nq = min(S3_BB, nb - q0);
    __syncthreads();    // the harmonics of the previous batch are no longer read
    if (tid < nq) {
      const float4 rec = b.rec[base + q0 + tid];
      const float ir = rsqrtf(rec.x * rec.x + rec.y * rec.y + rec.z * rec.z);
      stage_harmonics(sht, rec.x * ir, rec.y * ir, rec.z * ir, nlm, Ys + tid * nlm, Gs + 3 * tid * nlm);
    }
    for (int q = 0; q < nq; q++) {
      const float4 rec = b.rec[base + q0 + q];
      const int j = __float_as_int(rec.w), muj = b.mu[j];
      const float r = sqrtf(rec.x * rec.x + rec.y * rec.y + rec.z * rec.z), ir = 1.0f / r;
      const float ux = rec.x * ir, uy = rec.y * ir, uz = rec.z * ir;
      const int slot = L.pair_slot[mui * L.nel + muj];
      const float rc = L.rc[mui * L.nel + muj];
      if (slot < 0) continue;    // as in the forward kernel
      int k0;
      float t;
      spline_locate(r / rc, L.N, k0, t);
      __syncthreads();    // the buffers of the previous bond are no longer read (gP and the harmonics are complete)
      if (tid == 0) *dedx = 0.0f;
      const float4 *tab = reinterpret_cast<const float4 *>(L.tab + (size_t) slot * L.tab_stride) + (size_t) k0 * L.nl * C;
      for (int e = tid; e < L.nl * C; e += S3_THREADS) {
        const float4 cf = tab[e];
        R[e] = cf.x + t * (cf.y + t * (cf.z + t * cf.w));
        dR[e] = (cf.y + t * (2.0f * cf.z + t * 3.0f * cf.w)) * (float) L.N;
      }
      if (live)
        for (int li = g; li < nlmi; li += G) {
          const float m = L.msg ? L.msg[((size_t) j * nlmi + li) * C + c] : 0.0f;
          Ic[li * C + c] = m + L.l0mask[li] * L.zproj[(size_t) muj * C + c];
        }
      __syncthreads();
      const float *Y = Ys + q * nlm, *Gq = Gs + 3 * q * nlm;
      float part = 0.0f;    // this thread's share of dE/dx
      if (live) {
        for (int ly = g; ly < nlm; ly += G) {
          const float *gp = gP + (size_t) ly * nlmi * C + c;
          float w = 0.0f;
#pragma unroll 5
          for (int li = 0; li < nlmi; li++) w = fmaf(gp[(size_t) li * C], Ic[li * C + c], w);
          const int lc = L.lt[ly] * C + c;
          W[ly * C + c] = w;
          U[ly * C + c] = Y[ly] * R[lc];
          part = fmaf(w * Y[ly], dR[lc], part);
        }
      }
      if (L.gmsg) {
        __syncthreads();    // U of all ly
        if (live)
          for (int li = g; li < nlmi; li += G) {
            const float *gp = gP + (size_t) li * C + c;
            float v = 0.0f;
#pragma unroll 5
            for (int ly = 0; ly < nlm; ly++) v = fmaf(gp[(size_t) ly * nlmi * C], U[ly * C + c], v);
            atomicAdd(L.gmsg + ((size_t) j * nlmi + li) * C + c, v);
          }
      }
      for (int s = 16; s > 0; s >>= 1) part += __shfl_xor_sync(0xffffffffu, part, s);
      if (lane == 0) atomicAdd(dedx, part);
      __syncthreads();
      for (int ly = warp; ly < nlm; ly += S3_THREADS / 32) {    // a warp per ly: the sum over the channels
        float v = 0.0f;
        for (int cc = lane; cc < C; cc += 32) v = fmaf(W[ly * C + cc], R[L.lt[ly] * C + cc], v);
        for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
        if (lane == 0) gY[ly] = v;
      }
      __syncthreads();
      if (tid == 0) {
        float gx = 0.0f, gy = 0.0f, gz = 0.0f;
        for (int lm = 0; lm < nlm; lm++) {
          gx = fmaf(gY[lm], Gq[3 * lm], gx);
          gy = fmaf(gY[lm], Gq[3 * lm + 1], gy);
          gz = fmaf(gY[lm], Gq[3 * lm + 2], gz);
        }
        const float dEdr = *dedx / rc, gr = gx * ux + gy * uy + gz * uz;
        const float f0 = dEdr * ux + (gx - gr * ux) * ir, f1 = dEdr * uy + (gy - gr * uy) * ir, f2 = dEdr * uz + (gz - gr * uz) * ir;
        float *o = fv + 3 * (size_t) b.cslot[base + q0 + q];
        if (add) { o[0] += f0; o[1] += f1; o[2] += f2; }
        else { o[0] = f0; o[1] = f1; o[2] = f2; }
        const double dx = -(double) ux * r, dy = -(double) uy * r, dz = -(double) uz * r;
        vir[0] += dx * f0; vir[1] += dy * f1; vir[2] += dz * f2;
        vir[3] += dx * f1; vir[4] += dx * f2; vir[5] += dy * f2;
      }
    }
  }
  if (tid == 0)
    for (int k = 0; k < 6; k++) {
      double *o = vir_atom + 6 * (size_t) i + k;
      *o = add ? *o + vir[k] : vir[k];
    }
}

struct EqNormDev {
  const float *dw, *mask, *aff;
  const int *e;
  int nf, C, center;
  double eps;
};

// EquivariantRMSNorm of one atom per thread (libgrace/include/grace/fused_3l_cpu.h:346-370): x [f][NA][C] -> y rows [i][f][C]
__global__ void eqnorm_fwd_kernel(EqNormDev E, const float *__restrict__ x, float *__restrict__ y, int NA, int n)
{
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  double S = 0.0;
  for (int f = 0; f < E.nf; f++) {
    const float *xf = x + ((size_t) f * NA + i) * E.C;
    double m = 0.0;
    if (E.center && E.mask[f] != 0.0f) {
      for (int c = 0; c < E.C; c++) m += xf[c];
      m = m / E.C * E.mask[f];
    }
    double s2 = 0.0;
    for (int c = 0; c < E.C; c++) {
      const float v = (float) (xf[c] - m);
      s2 += (double) v * v;
    }
    S += E.dw[f] * s2;
  }
  const double r = 1.0 / sqrt(S / E.C + E.eps);
  for (int f = 0; f < E.nf; f++) {
    const float *xf = x + ((size_t) f * NA + i) * E.C, *a = E.aff + (size_t) E.e[f] * E.C;
    float *yf = y + ((size_t) i * E.nf + f) * E.C;
    double m = 0.0;
    if (E.center && E.mask[f] != 0.0f) {
      for (int c = 0; c < E.C; c++) m += xf[c];
      m = m / E.C * E.mask[f];
    }
    for (int c = 0; c < E.C; c++) yf[c] = (float) ((float) (xf[c] - m) * r) * a[c];
  }
}

// gx [f][NA][C] = adjoint of the above for dy rows [i][f][C] (:373-415)
__global__ void eqnorm_bwd_kernel(EqNormDev E, const float *__restrict__ x, const float *__restrict__ dy, float *__restrict__ gx, int NA,
                                  int n)
{
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  double S = 0.0, dot = 0.0;
  for (int f = 0; f < E.nf; f++) {
    const float *xf = x + ((size_t) f * NA + i) * E.C, *a = E.aff + (size_t) E.e[f] * E.C, *d = dy + ((size_t) i * E.nf + f) * E.C;
    double m = 0.0;
    if (E.center && E.mask[f] != 0.0f) {
      for (int c = 0; c < E.C; c++) m += xf[c];
      m = m / E.C * E.mask[f];
    }
    double s2 = 0.0;
    for (int c = 0; c < E.C; c++) {
      const float v = (float) (xf[c] - m);
      s2 += (double) v * v;
      dot += (double) d[c] * a[c] * v;
    }
    S += E.dw[f] * s2;
  }
  const double r = 1.0 / sqrt(S / E.C + E.eps), k3 = r * r * r * dot / E.C;
  for (int f = 0; f < E.nf; f++) {
    const float *xf = x + ((size_t) f * NA + i) * E.C, *a = E.aff + (size_t) E.e[f] * E.C, *d = dy + ((size_t) i * E.nf + f) * E.C;
    float *o = gx + ((size_t) f * NA + i) * E.C;
    const bool centred = E.center && E.mask[f] != 0.0f;
    double m = 0.0;
    if (centred) {
      for (int c = 0; c < E.C; c++) m += xf[c];
      m = m / E.C * E.mask[f];
    }
    const double kf = k3 * E.dw[f];
    double mean = 0.0;
    for (int c = 0; c < E.C; c++) mean += (float) (r * d[c] * a[c] - kf * (float) (xf[c] - m));
    mean = centred ? mean / E.C * E.mask[f] : 0.0;
    for (int c = 0; c < E.C; c++) o[c] = (float) ((float) (r * d[c] * a[c] - kf * (float) (xf[c] - m)) - mean);
  }
}

// RMSNorm of the density (:416-425): x [NA][wr] (one function) -> y rows [i][wr]; sum rows += y
__global__ void rmsnorm_fwd_kernel(const float *__restrict__ x, const float *__restrict__ scale, int n0, int wr, float *__restrict__ sum,
                                   int first, int n)
{
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float *xi = x + (size_t) i * wr;
  float *s = sum + (size_t) i * wr;
  double q = 0.0;
  for (int c = n0; c < wr; c++) q += (double) xi[c] * xi[c];
  const double r = 1.0 / sqrt(q / (wr - n0) + 1e-10);
  for (int c = 0; c < wr; c++) {
    const float y = c < n0 ? xi[c] : (float) (xi[c] * r) * scale[c - n0];
    s[c] = first ? y : s[c] + y;
  }
}

__global__ void rmsnorm_bwd_kernel(const float *__restrict__ x, const float *__restrict__ scale, int n0, int wr,
                                   const float *__restrict__ dy, float *__restrict__ gx, int n)
{
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float *xi = x + (size_t) i * wr, *d = dy + (size_t) i * wr;
  float *o = gx + (size_t) i * wr;
  double q = 0.0, g = 0.0;
  for (int c = n0; c < wr; c++) {
    q += (double) xi[c] * xi[c];
    g += (double) d[c] * scale[c - n0] * xi[c];
  }
  const double r = 1.0 / sqrt(q / (wr - n0) + 1e-10), k = r * r * r * g / (wr - n0);
  for (int c = 0; c < wr; c++) o[c] = c < n0 ? d[c] : (float) (r * d[c] * scale[c - n0] - k * xi[c]);
}

struct Readout3Dev {
  const double *W0, *W1, *shift;    // [nin][nh], [nh], [n_elements]
  double n0, n1, oscale;
  int nin, nh, act;
};

// E_i = (MLP(sum[1:]) + sum[0]) scale + shift (fp64, :1334-1374); d: dE/d(sum) rows [i][1 + nin]
__global__ void readout3_kernel(Readout3Dev R, const float *__restrict__ sum, const int *__restrict__ mu, double *__restrict__ e_atom,
                                float *__restrict__ d, int want_grad, int n)
{
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int wr = R.nin + 1;
  const float *h = sum + (size_t) i * wr;
  double e = 0.0;
  float *di = d + (size_t) i * wr;
  if (want_grad)
    for (int c = 0; c < wr; c++) di[c] = c == 0 ? (float) R.oscale : 0.0f;
  double acc_d[128];
  if (want_grad)
    for (int c = 0; c < R.nin; c++) acc_d[c] = 0.0;
  for (int j = 0; j < R.nh; j++) {
    double s = 0.0;
    for (int c = 0; c < R.nin; c++) s += (double) h[c + 1] * R.W0[(size_t) c * R.nh + j];
    s *= R.n0;
    double act, dact;
    if (R.act == 1) {
      act = tanh(s);
      dact = 1.0 - act * act;
    } else {
      const double sg = 1.0 / (1.0 + exp(-s));
      act = s * sg;
      dact = sg * (1.0 + s * (1.0 - sg));
    }
    e += R.W1[j] * act;
    if (want_grad) {
      const double ds = R.oscale * R.n1 * R.W1[j] * dact * R.n0;
      for (int c = 0; c < R.nin; c++) acc_d[c] += R.W0[(size_t) c * R.nh + j] * ds;
    }
  }
  e *= R.n1;
  e_atom[i] = (e + (double) h[0]) * R.oscale + R.shift[mu[i]];
  if (want_grad)
    for (int c = 0; c < R.nin; c++) di[c + 1] = (float) acc_d[c];
}

}    // namespace

// device state of the three layers
struct State3L {
  LayerEngine E[3];
  DBuf<float> arena[3], tab[3], zproj[3], l0mask[3], cg_v[3], cgt_v[3], rho_scale[3];
  DBuf<int> lt[3], cg_off[3], cg_p[3], cgt_off[3], cgt_f[3];
  DBuf<float> eq_dw[2], eq_mask[2], eq_aff[2], msg[2], gmsg[2];
  DBuf<int> eq_e[2];
  DBuf<int> pair_slot;
  std::vector<int> pair_slot_host;
  std::vector<std::vector<float>> tab_host[3];    // per layer, per pair slot
  int npairs = 0;
  DBuf<float> rho_sum, drho;
  DBuf<double> eW0, eW1;
  int NA = 0;
};

void Engine::setup_3l()
{
  const Plan3L &Q = *plan_.p3;
  s3_ = std::make_shared<State3L>();
  State3L &S = *s3_;
  for (int k = 0; k < 3; k++) {
    const Layer3Plan &L = Q.L[k];
    if (L.C > 64 || L.C % 4) throw Unsupported("GRACE-3L: channel counts must be multiples of 4 up to 64");
    setup_layer(S.E[k], L.dense);
    S.zproj[k].upload(L.zproj);
    S.l0mask[k].upload(L.l0mask);
    S.cg_v[k].upload(L.cg_v);
    S.cgt_v[k].upload(L.cgt_v);
    S.rho_scale[k].upload(L.rho_scale);
    S.lt[k].upload(L.lt);
    S.cg_off[k].upload(L.cg_off);
    S.cg_p[k].upload(L.cg_p);
    S.cgt_off[k].upload(L.cgt_off);
    S.cgt_f[k].upload(L.cgt_f);
    if (k < 2) {
      S.eq_dw[k].upload(L.eq_dw);
      S.eq_mask[k].upload(L.eq_mask);
      S.eq_aff[k].upload(L.eq_aff);
      S.eq_e[k].upload(L.eq_e);
    }
  }
  S.pair_slot_host.assign((size_t) plan_.n_elements * plan_.n_elements, -1);
  S.pair_slot.upload(S.pair_slot_host);
  S.eW0.upload(Q.eW0);
  S.eW1.upload(Q.eW1);
  shift_.upload(plan_.shift);
  GB_CUDA(cudaStreamSynchronize(dev().stream));
}

// radial tables of every pair of the given elements (built once per pair)
void Engine::prepare_species(const std::vector<int> &elements)
{
  if (plan_.layers != 3) return;
  std::lock_guard<std::mutex> lk(mu);
  State3L &S = *s3_;
  const Plan3L &Q = *plan_.p3;
  const int nel = plan_.n_elements;
  bool grown = false;
  for (int a : elements)
    for (int b : elements) {
      int &slot = S.pair_slot_host[(size_t) a * nel + b];
      if (slot >= 0) continue;
      slot = S.npairs++;
      for (int k = 0; k < 3; k++) S.tab_host[k].push_back(radial_table_3l(*Q.model, k, a, b, Q.spline_n));
      grown = true;
    }
  if (!grown) return;
  for (int k = 0; k < 3; k++) {
    std::vector<float> all;
    for (const auto &t : S.tab_host[k]) all.insert(all.end(), t.begin(), t.end());
    S.tab[k].upload(all);
  }
  S.pair_slot.upload(S.pair_slot_host);
  GB_CUDA(cudaStreamSynchronize(dev().stream));
}

void Engine::evaluate_3l(NeighborList &nl, bool energy_only, StageTimer *tm)
{
  State3L &S = *s3_;
  const Plan3L &Q = *plan_.p3;
  const int n = (int) nl.n();
  const int NA = (n + 3) / 4 * 4;
  const BondsDev bonds = nl.bonds();
  const int *mu = bonds.mu;
  const SHTable sht = sh_table_host();
  const int nt = 128, nblk = (n + nt - 1) / nt;
  // large evaluations: the projections, reduces and FCs with 16 / 32 / 64 channels as tensor-core grouped GEMMs (mv_tc.cu)
  tc_now_ = dense_ == Dense::Tc || (n >= tc_min_atoms_ && dense_ == Dense::Auto);
  auto check_tc = [&]() {
    if (!tc_now_) return;
    int e = 0;
    GB_CUDA(cudaMemcpyAsync(&e, tc_error_.get(), sizeof(int), cudaMemcpyDeviceToHost, dev().stream));
    GB_CUDA(cudaStreamSynchronize(dev().stream));
    if (e) {
      GB_CUDA(cudaMemsetAsync(tc_error_.get(), 0, sizeof(int), dev().stream));
      throw DeviceError("the tensor-core FC kernel gave up waiting for its matrix instructions");
    }
  };
  {    // every bond of the structure needs the table of its element pair: a pair outside the Systems' species has none
    // (checked on the host: the species of every System of the engine were prepared when it was created)
  }
  if (tm) tm->begin(StageTimer::FWD);
  const int wr = Q.L[0].wr;
  S.rho_sum.ensure((size_t) n * wr);
  S.drho.ensure((size_t) n * wr);
  auto spbf = [&](int k) {
    const Layer3Plan &L = Q.L[k];
    Spbf3Dev d{};
    d.tab = S.tab[k].get();
    d.pair_slot = S.pair_slot.get();
    d.tab_stride = (long long) Q.spline_n * (plan_.lmax + 1) * L.C * 4;
    d.rc = rcf_.get();
    d.msg = k > 0 ? S.msg[k - 1].get() : nullptr;
    d.gmsg = k > 0 ? S.gmsg[k - 1].get() : nullptr;
    d.zproj = S.zproj[k].get();
    d.l0mask = S.l0mask[k].get();
    d.lt = S.lt[k].get();
    d.cg_off = S.cg_off[k].get();
    d.cg_p = S.cg_p[k].get();
    d.cgt_off = S.cgt_off[k].get();
    d.cgt_f = S.cgt_f[k].get();
    d.cg_v = S.cg_v[k].get();
    d.cgt_v = S.cgt_v[k].get();
    d.N = Q.spline_n;
    d.C = L.C;
    d.nl = plan_.lmax + 1;
    d.nlm = plan_.nlm;
    d.nlmi = L.nlmi;
    d.nfA = L.nfA;
    d.nel = plan_.n_elements;
    return d;
  };
  auto smem_fwd = [&](const Layer3Plan &L) {
    return sizeof(float) * ((size_t) plan_.nlm * L.nlmi * L.C + (size_t) S3_BB * plan_.nlm + (size_t) plan_.nlm * L.C +
                            (size_t) L.nlmi * L.C);
  };
  auto smem_bwd = [&](const Layer3Plan &L) {
    return sizeof(float) * ((size_t) plan_.nlm * L.nlmi * L.C + 4 * (size_t) S3_BB * plan_.nlm + 2 * (size_t) (plan_.lmax + 1) * L.C +
                            (size_t) L.nlmi * L.C + plan_.nlm + 2 * (size_t) plan_.nlm * L.C + 4);
  };
  static bool attr_set = false;
  if (!attr_set) {
    GB_CUDA(cudaFuncSetAttribute(spbf3_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    GB_CUDA(cudaFuncSetAttribute(spbf3_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    attr_set = true;
  }
  for (int k = 0; k < 3; k++) {
    const Layer3Plan &L = Q.L[k];
    if (smem_bwd(L) > 220 * 1024) throw Unsupported("GRACE-3L: the coupled bond sums of a layer do not fit the shared memory");
    LayerEngine &E = S.E[k];
    float *base = S.arena[k].ensure((size_t) E.per_atom * NA);
    bind_arena(E, base, NA);
    const std::vector<TensorDev> &T = E.tensors_host;
    GB_LAUNCH(spbf3_fwd_kernel, n, S3_THREADS, smem_fwd(L), bonds, spbf(k), sht, T[L.tA].p, NA);
    run(E, L.dense.fwd, mu, n, NA);
    if (k < 2) {
      S.msg[k].ensure((size_t) n * L.nfEQ * L.cEQ);
      const EqNormDev e{S.eq_dw[k].get(), S.eq_mask[k].get(), S.eq_aff[k].get(), S.eq_e[k].get(), L.nfEQ, L.cEQ, L.eq_center, L.eq_eps};
      GB_LAUNCH(eqnorm_fwd_kernel, nblk, nt, 0, e, T[L.tEQ].p, S.msg[k].get(), NA, n);
    }
    GB_LAUNCH(rmsnorm_fwd_kernel, nblk, nt, 0, T[L.tRHO].p, S.rho_scale[k].get(), L.rho_n0, wr, S.rho_sum.get(), k == 0 ? 1 : 0, n);
  }
  const Readout3Dev ro{S.eW0.get(), S.eW1.get(), shift_.get(), Q.en0, Q.en1, plan_.out_scale, Q.e_nin, Q.e_nh, Q.e_act};
  GB_LAUNCH(readout3_kernel, nblk, nt, 0, ro, S.rho_sum.get(), mu, e_atom_.get(), S.drho.get(), energy_only ? 0 : 1, n);
  if (tm) tm->end(StageTimer::FWD);
  if (energy_only) {
    check_tc();
    return;
  }
  if (tm) tm->begin(StageTimer::BWD);
  for (int k = 0; k < 2; k++) {
    const Layer3Plan &L = Q.L[k];
    S.gmsg[k].ensure((size_t) n * L.nfEQ * L.cEQ);
    launch_fill_zero(S.gmsg[k].get(), sizeof(float) * (size_t) n * L.nfEQ * L.cEQ);
  }
  for (int k = 2; k >= 0; k--) {
    const Layer3Plan &L = Q.L[k];
    LayerEngine &E = S.E[k];
    const std::vector<TensorDev> &T = E.tensors_host;
    bind_arena(E, S.arena[k].get(), NA);
    if (L.dense.zero_grads)
      launch_fill_zero(S.arena[k].get() + (size_t) E.grad_begin * NA, sizeof(float) * (size_t) (E.grad_end - E.grad_begin) * NA);
    GB_LAUNCH(rmsnorm_bwd_kernel, nblk, nt, 0, T[L.tRHO].p, S.rho_scale[k].get(), L.rho_n0, wr, S.drho.get(), T[L.tGRHO].p, n);
    if (k < 2) {
      const EqNormDev e{S.eq_dw[k].get(), S.eq_mask[k].get(), S.eq_aff[k].get(), S.eq_e[k].get(), L.nfEQ, L.cEQ, L.eq_center, L.eq_eps};
      GB_LAUNCH(eqnorm_bwd_kernel, nblk, nt, 0, e, T[L.tEQ].p, S.gmsg[k].get(), T[L.tGEQ].p, NA, n);
    }
    run(E, L.dense.bwd, mu, n, NA);
    GB_LAUNCH(spbf3_bwd_kernel, n, S3_THREADS, smem_bwd(L), bonds, spbf(k), sht, T[L.tGA].p, NA, fv_.get(), vir_atom_.get(), k == 2 ? 0 : 1);
  }
  if (tm) tm->end(StageTimer::BWD);
  check_tc();
}

}    // namespace gb
