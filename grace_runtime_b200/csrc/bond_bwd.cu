// Reverse bond kernel: from gQ = dE/dQ of the central atom, per bond
//   S[I, l]   = sum_{m} Y_lm gQ[(I, lm)]                      dE/dR[l] = sum_I S[I, l] msg_I,  dE/dmsg_I = sum_l S[I, l] R[l]
//   dE/dx     = sum_{l, n} dE/dR[n, l] dR[n, l]/dx
//   g         = sum_{I, lm, n} gQ[(I, lm)][n] R[n, l] msg_I[n] grad Y_lm
//   f         = (dE/dx / rcut) rhat + (g - (g . rhat) rhat) / r          (force on i; -f on j)
// as bond_scatter_bwd_t / bond_yi_bwd_g / bond_dEdx_t / bond_force of the reference
// (libgrace/include/grace/fused_cpu.h:836-942, 1027-1050) and add_bond_virial (libgrace/src/fused_1l.cpp:45-51).
//
// One block of 4 warps per atom; a lane owns channel n and keeps gQ of its channel in registers; warps (half-warps
// for C <= 16) take the bonds in turn and reduce the four bond scalars over the channels by shuffles.  The bond force
// is stored at the bond's slot of the neighbour list (no atomics; forces are gathered afterwards through the
// reverse-bond index), the virial as one fp64 row per atom.  A bond's share of dE/dmsg of its neighbour goes to the
// bond's slot too and is summed per neighbour by msg_grad_gather_kernel (chain.cu); only when that buffer could not be
// allocated the shares are added with fp32 atomics, as the reference does.
#include "bond_common.cuh"

#include <cstdlib>

namespace gb {

namespace {

constexpr int EBB = 96;    // bonds staged per round: most atoms in one round, every thread of the block staging one bond

template<int LMAX, int NIT, int NCH, int LPE, bool EXACT>
__global__ void __launch_bounds__(128) bond_bwd_kernel(BondsDev b, LayerDev L, SHTable sht,
                                                       const float *__restrict__ gQ, int NA, int a0,
                                                       float *__restrict__ fv, double *__restrict__ vir_atom, int add)
{
  constexpr int NL = LMAX + 1, NLM = NL * NL, EPW = 32 / LPE;
  __shared__ float4 YG[EBB][NLM];
  __shared__ float su[EBB][4];     // rhat, r
  __shared__ float srci[EBB], st[EBB];
  __shared__ int sk[EBB], smu[EBB], sj[EBB], scs[EBB];
  __shared__ float fe[EBB][4];     // g (3), dE/dx
  __shared__ double vred[4][6];

  const int a = blockIdx.x, i = b.ilist ? b.ilist[a0 + a] : a0 + a, tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
  const int ln = lane % LPE, esub = lane / LPE;
  const long long base = b.off[i];
  const int nb = b.cnt[i];
  const int mui = b.mu[i];
  const int C = L.C, nel = L.n_elements;
  const int tiles = (L.n_msg + 1 + NIT - 1) / NIT;
  const float fN = (float) L.N;
  double vir[6] = {0.0, 0.0, 0.0, 0.0, 0.0, 0.0};

  for (int b0 = 0; b0 < nb; b0 += EBB) {
    const int nbat = min(EBB, nb - b0);
    for (int e = tid; e < nbat; e += 128) {
      const float4 rec = b.rec[base + b0 + e];
      const float r = sqrtf(rec.x * rec.x + rec.y * rec.y + rec.z * rec.z), ir = 1.0f / r;
      const int j = __float_as_int(rec.w);
      const int muj = b.mu[j];
      const float rc = L.rc[mui * nel + muj];
      int k;
      float t;
      spline_locate(r / rc, L.N, k, t);
      sk[e] = k; st[e] = t; smu[e] = muj; sj[e] = j;
      scs[e] = b.cslot[base + b0 + e];
      srci[e] = 1.0f / rc;
      su[e][0] = rec.x * ir; su[e][1] = rec.y * ir; su[e][2] = rec.z * ir; su[e][3] = r;
      float4 *yg = YG[e];
      sph_harm<LMAX, true>(sht, rec.x * ir, rec.y * ir, rec.z * ir,
                           [&](int lm, float v, float gx, float gy, float gz) { yg[lm] = make_float4(v, gx, gy, gz); });
      fe[e][0] = fe[e][1] = fe[e][2] = fe[e][3] = 0.0f;
    }
    __syncthreads();
    for (int tile = 0; tile < tiles; tile++) {
      const int Ibase = tile * NIT;
      float g[NIT][NLM][NCH];
#pragma unroll
      for (int I = 0; I < NIT; I++)
#pragma unroll
        for (int q = 0; q < NLM; q++)
#pragma unroll
          for (int ch = 0; ch < NCH; ch++) {
            const int n = ln + ch * LPE;
            g[I][q][ch] = (n < C && Ibase + I <= L.n_msg)
                              ? __ldg(gQ + ((size_t) ((Ibase + I) * NLM + q) * NA + a) * C + n) : 0.0f;
          }
      for (int e0 = w * EPW; e0 < nbat; e0 += 4 * EPW) {
        const int e = e0 + esub;
        const bool valid = e < nbat;
        float gx = 0.0f, gy = 0.0f, gz = 0.0f, dedx = 0.0f;
        if (valid) {
          const int k = sk[e], muj = smu[e], j = sj[e];
          const float t = st[e];
          const float4 *yg = YG[e];
#pragma unroll
          for (int ch = 0; ch < NCH; ch++) {
            const int n = ln + ch * LPE;
            if (n < C) {
              float R[NL], dR[NL];
              if (EXACT) {    // exact radial MLP, evaluated per slot beforehand
                const size_t ro = (size_t) (base + b0 + e) * (NL * C) + n;
#pragma unroll
                for (int l = 0; l < NL; l++) {
                  R[l] = __ldg(L.Rex + ro + l * C);
                  dR[l] = __ldg(L.dRex + ro + l * C);
                }
              } else {
                const float4 *cf = reinterpret_cast<const float4 *>(L.tab) + (size_t) k * NL * C + n;
#pragma unroll
                for (int l = 0; l < NL; l++) {
                  const float4 c = __ldg(cf + l * C);
                  R[l] = c.x + t * (c.y + t * (c.z + t * c.w));
                  dR[l] = (c.y + t * (2.0f * c.z + t * 3.0f * c.w)) * fN;
                }
              }
              if constexpr (NIT == 1) {    // one message function per pass: nothing to contract first
                const int Ig = Ibase;
                float m = 0.0f;
                if (Ig < L.n_msg) m = __ldg(L.msg + ((size_t) j * L.n_msg + Ig) * C + n);
                else if (Ig == L.n_msg) m = __ldg(L.z + (size_t) muj * C + n);
                float gm = 0.0f;
#pragma unroll
                for (int l = 0; l < NL; l++) {
                  const float rm = R[l] * m;
                  float S = 0.0f;
#pragma unroll
                  for (int q = l * l; q < (l + 1) * (l + 1); q++) {
                    const float4 y4 = yg[q];
                    const float gq = g[0][q][ch];
                    S = fmaf(y4.x, gq, S);
                    const float p = gq * rm;
                    gx = fmaf(p, y4.y, gx);
                    gy = fmaf(p, y4.z, gy);
                    gz = fmaf(p, y4.w, gz);
                  }
                  dedx = fmaf(S * m, dR[l], dedx);
                  gm = fmaf(S, R[l], gm);
                }
                if (Ig < L.n_msg) {
                  if (L.gmsg_slot) L.gmsg_slot[((size_t) scs[e] * L.n_msg + Ig) * C + n] = gm;
                  else atomicAdd(L.gmsg + ((size_t) j * L.n_msg + Ig) * C + n, gm);
                }
              } else {
                // messages of this tile first, then one contraction over them per lm: h[q] = sum_I msg_I gQ[I][q] carries
                // everything dE/dx and the direction gradient need, so the harmonics are applied once per bond and
                // channel instead of once per message function
                float m[NIT];
  #pragma unroll
                for (int I = 0; I < NIT; I++) {
                  const int Ig = Ibase + I;
                  m[I] = 0.0f;
                  if (Ig < L.n_msg) m[I] = __ldg(L.msg + ((size_t) j * L.n_msg + Ig) * C + n);
                  else if (Ig == L.n_msg) m[I] = __ldg(L.z + (size_t) muj * C + n);
                }
  #pragma unroll
                for (int l = 0; l < NL; l++) {
                  float T = 0.0f, vx = 0.0f, vy = 0.0f, vz = 0.0f;
  #pragma unroll
                  for (int q = l * l; q < (l + 1) * (l + 1); q++) {
                    float h = 0.0f;
  #pragma unroll
                    for (int I = 0; I < NIT; I++) h = fmaf(m[I], g[I][q][ch], h);
                    const float4 y4 = yg[q];
                    T = fmaf(y4.x, h, T);
                    vx = fmaf(h, y4.y, vx);
                    vy = fmaf(h, y4.z, vy);
                    vz = fmaf(h, y4.w, vz);
                  }
                  dedx = fmaf(T, dR[l], dedx);
                  gx = fmaf(R[l], vx, gx);
                  gy = fmaf(R[l], vy, gy);
                  gz = fmaf(R[l], vz, gz);
                }
  #pragma unroll
                for (int I = 0; I < NIT; I++) {    // dE/dmsg_I = sum_l R_l sum_{m} Y_lm gQ[I][lm]
                  const int Ig = Ibase + I;
                  if (Ig < L.n_msg) {
                    float gm = 0.0f;
  #pragma unroll
                    for (int l = 0; l < NL; l++) {
                      float S = 0.0f;
  #pragma unroll
                      for (int q = l * l; q < (l + 1) * (l + 1); q++) S = fmaf(yg[q].x, g[I][q][ch], S);
                      gm = fmaf(S, R[l], gm);
                    }
                    if (L.gmsg_slot) L.gmsg_slot[((size_t) scs[e] * L.n_msg + Ig) * C + n] = gm;
                    else atomicAdd(L.gmsg + ((size_t) j * L.n_msg + Ig) * C + n, gm);
                  }
                }
              }
            }
          }
        }
        const float tot = group_sum4<LPE>(gx, gy, gz, dedx, ln);
        if (valid && (ln & (LPE / 4 - 1)) == 0) fe[e][ln / (LPE / 4)] += tot;    // one owner per bond, tile and component: no race
      }
      __syncthreads();
    }
    for (int e = tid; e < nbat; e += 128) {
      const float ux = su[e][0], uy = su[e][1], uz = su[e][2], r = su[e][3];
      const float gxx = fe[e][0], gyy = fe[e][1], gzz = fe[e][2];
      const float dEdr = fe[e][3] * srci[e];
      const float gr = gxx * ux + gyy * uy + gzz * uz, ir = 1.0f / r;
      const float f0 = dEdr * ux + (gxx - gr * ux) * ir;
      const float f1 = dEdr * uy + (gyy - gr * uy) * ir;
      const float f2 = dEdr * uz + (gzz - gr * uz) * ir;
      float *o = fv + 3 * (size_t) scs[e];
      if (add) { o[0] += f0; o[1] += f1; o[2] += f2; }
      else { o[0] = f0; o[1] = f1; o[2] = f2; }
      const double dx = -(double) ux * r, dy = -(double) uy * r, dz = -(double) uz * r;
      vir[0] += dx * f0; vir[1] += dy * f1; vir[2] += dz * f2;
      vir[3] += dx * f1; vir[4] += dx * f2; vir[5] += dy * f2;
    }
    __syncthreads();
  }
#pragma unroll
  for (int k = 0; k < 6; k++) {
    for (int s = 16; s > 0; s >>= 1) vir[k] += __shfl_xor_sync(0xffffffffu, vir[k], s);
    if (lane == 0) vred[w][k] = vir[k];
  }
  __syncthreads();
  if (tid < 6) {
    const double v = vred[0][tid] + vred[1][tid] + vred[2][tid] + vred[3][tid];
    double *o = vir_atom + 6 * (size_t) i + tid;
    *o = add ? *o + v : v;
  }
}

// The same for layers that couple message functions in (NIT > 1) with at most 16 channels: a whole warp per bond, lane
// = (channel n, half h) with the lm of the bond sums split between the halves (lm = 2 k + h), so that a lane keeps
// NIT x NLM / 2 gradients in registers instead of NIT x NLM (twice the resident warps) and the two halves share the
// work of a bond.  Per lm the lane forms h = sum_I msg_I gQ[I][lm] once; with R and dR/dx of the lm's degree
// (selected per lm) everything is linear in h:
//   dE/dx += dR_l Y_lm h,   g += R_l h grad Y_lm,   dE/dmsg_I += R_l Y_lm gQ[I][lm].
template<int LMAX, int NIT>
__global__ void __launch_bounds__(128) bond_bwd_split_kernel(BondsDev b, LayerDev L, SHTable sht, const float *__restrict__ gQ,
                                                             int NA, int a0, float *__restrict__ fv,
                                                             double *__restrict__ vir_atom, int add)
{
  constexpr int NL = LMAX + 1, NLM = NL * NL, NK = (NLM + 1) / 2;
  __shared__ float4 YG[EBB][NLM];
  __shared__ float su[EBB][4];     // rhat, r
  __shared__ float srci[EBB], st[EBB];
  __shared__ int sk[EBB], smu[EBB], sj[EBB], scs[EBB];
  __shared__ float fe[EBB][4];     // g (3), dE/dx
  __shared__ double vred[4][6];

  const int a = blockIdx.x, i = b.ilist ? b.ilist[a0 + a] : a0 + a, tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
  const int n = lane & 15, h = lane >> 4;
  const long long base = b.off[i];
  const int nb = b.cnt[i];
  const int mui = b.mu[i];
  const int C = L.C, nel = L.n_elements;
  const float fN = (float) L.N;
  double vir[6] = {0.0, 0.0, 0.0, 0.0, 0.0, 0.0};
  // gradients of this lane's channel and lm's: g[I][k] = gQ[(I, 2 k + h)][n]
  float g[NIT][NK];
#pragma unroll
  for (int I = 0; I < NIT; I++)
#pragma unroll
    for (int k = 0; k < NK; k++) {
      const int q = 2 * k + h;
      g[I][k] = (n < C && q < NLM && I <= L.n_msg) ? __ldg(gQ + ((size_t) (I * NLM + q) * NA + a) * C + n) : 0.0f;
    }

  for (int b0 = 0; b0 < nb; b0 += EBB) {
    const int nbat = min(EBB, nb - b0);
    for (int e = tid; e < nbat; e += 128) {
      const float4 rec = b.rec[base + b0 + e];
      const float r = sqrtf(rec.x * rec.x + rec.y * rec.y + rec.z * rec.z), ir = 1.0f / r;
      const int j = __float_as_int(rec.w);
      const int muj = b.mu[j];
      const float rc = L.rc[mui * nel + muj];
      int k;
      float t;
      spline_locate(r / rc, L.N, k, t);
      sk[e] = k; st[e] = t; smu[e] = muj; sj[e] = j;
      scs[e] = b.cslot[base + b0 + e];
      srci[e] = 1.0f / rc;
      su[e][0] = rec.x * ir; su[e][1] = rec.y * ir; su[e][2] = rec.z * ir; su[e][3] = r;
      float4 *yg = YG[e];
      sph_harm<LMAX, true>(sht, rec.x * ir, rec.y * ir, rec.z * ir,
                           [&](int lm, float v, float gx, float gy, float gz) { yg[lm] = make_float4(v, gx, gy, gz); });
    }
    __syncthreads();
    for (int e = w; e < nbat; e += 4) {    // a warp per bond
      float gx = 0.0f, gy = 0.0f, gz = 0.0f, dedx = 0.0f;
      float gm[NIT];
#pragma unroll
      for (int I = 0; I < NIT; I++) gm[I] = 0.0f;
      if (n < C) {
        const int k0 = sk[e], muj = smu[e], j = sj[e];
        const float t = st[e];
        const float4 *yg = YG[e];
        float R[NL], dR[NL];
        const float4 *cf = reinterpret_cast<const float4 *>(L.tab) + (size_t) k0 * NL * C + n;
#pragma unroll
        for (int l = 0; l < NL; l++) {
          const float4 c = __ldg(cf + l * C);
          R[l] = c.x + t * (c.y + t * (c.z + t * c.w));
          dR[l] = (c.y + t * (2.0f * c.z + t * 3.0f * c.w)) * fN;
        }
        float m[NIT];
#pragma unroll
        for (int I = 0; I < NIT; I++) {
          m[I] = 0.0f;
          if (I < L.n_msg) m[I] = __ldg(L.msg + ((size_t) j * L.n_msg + I) * C + n);
          else if (I == L.n_msg) m[I] = __ldg(L.z + (size_t) muj * C + n);
        }
#pragma unroll
        for (int k = 0; k < NK; k++) {
          // degree of lm = 2 k (h = 0) and lm = 2 k + 1 (h = 1): compile-time constants, selected per lane
          constexpr auto deg = [](int q) { int l = 0; while ((l + 1) * (l + 1) <= q) l++; return l; };
          const int q = 2 * k + h;
          const int l0 = deg(2 * k), l1 = deg(2 * k + 1 < NLM ? 2 * k + 1 : NLM - 1);
          const float Rl = h ? R[l1] : R[l0], dRl = h ? dR[l1] : dR[l0];
          if (q < NLM) {
            const float4 y4 = yg[q];
            float hq = 0.0f;
#pragma unroll
            for (int I = 0; I < NIT; I++) hq = fmaf(m[I], g[I][k], hq);
            dedx = fmaf(dRl * y4.x, hq, dedx);
            const float p = Rl * hq;
            gx = fmaf(p, y4.y, gx);
            gy = fmaf(p, y4.z, gy);
            gz = fmaf(p, y4.w, gz);
            const float ry = Rl * y4.x;
#pragma unroll
            for (int I = 0; I < NIT; I++) gm[I] = fmaf(ry, g[I][k], gm[I]);
          }
        }
      }
      // dE/dmsg: the two halves of a channel add up; force terms: all lanes
#pragma unroll
      for (int I = 0; I < NIT; I++) gm[I] += __shfl_xor_sync(0xffffffffu, gm[I], 16);
      if (h == 0 && n < C) {
#pragma unroll
        for (int I = 0; I < NIT; I++)
          if (I < L.n_msg) {
            if (L.gmsg_slot) L.gmsg_slot[((size_t) scs[e] * L.n_msg + I) * C + n] = gm[I];
            else atomicAdd(L.gmsg + ((size_t) sj[e] * L.n_msg + I) * C + n, gm[I]);
          }
      }
      const float tot = group_sum4<32>(gx, gy, gz, dedx, lane);
      if ((lane & 7) == 0) fe[e][lane >> 3] = tot;
    }
    __syncthreads();
    for (int e = tid; e < nbat; e += 128) {
      const float ux = su[e][0], uy = su[e][1], uz = su[e][2], r = su[e][3];
      const float gxx = fe[e][0], gyy = fe[e][1], gzz = fe[e][2];
      const float dEdr = fe[e][3] * srci[e];
      const float gr = gxx * ux + gyy * uy + gzz * uz, ir = 1.0f / r;
      const float f0 = dEdr * ux + (gxx - gr * ux) * ir;
      const float f1 = dEdr * uy + (gyy - gr * uy) * ir;
      const float f2 = dEdr * uz + (gzz - gr * uz) * ir;
      float *o = fv + 3 * (size_t) scs[e];
      if (add) { o[0] += f0; o[1] += f1; o[2] += f2; }
      else { o[0] = f0; o[1] = f1; o[2] = f2; }
      const double dx = -(double) ux * r, dy = -(double) uy * r, dz = -(double) uz * r;
      vir[0] += dx * f0; vir[1] += dy * f1; vir[2] += dz * f2;
      vir[3] += dx * f1; vir[4] += dx * f2; vir[5] += dy * f2;
    }
    __syncthreads();
  }
#pragma unroll
  for (int k = 0; k < 6; k++) {
    for (int s = 16; s > 0; s >>= 1) vir[k] += __shfl_xor_sync(0xffffffffu, vir[k], s);
    if (lane == 0) vred[w][k] = vir[k];
  }
  __syncthreads();
  if (tid < 6) {
    const double v = vred[0][tid] + vred[1][tid] + vred[2][tid] + vred[3][tid];
    double *o = vir_atom + 6 * (size_t) i + tid;
    *o = add ? *o + v : v;
  }
}

template<int LMAX, int NIT, int NCH, int LPE>
void launch_t(const BondsDev &b, const LayerDev &L, const float *gQ, int NA, int a0, int na, float *fv,
              double *vir_atom, int add)
{
  if (L.Rex) GB_LAUNCH((bond_bwd_kernel<LMAX, NIT, NCH, LPE, true>), na, 128, 0, b, L, sh_table_host(), gQ, NA, a0, fv, vir_atom, add);
  else GB_LAUNCH((bond_bwd_kernel<LMAX, NIT, NCH, LPE, false>), na, 128, 0, b, L, sh_table_host(), gQ, NA, a0, fv, vir_atom, add);
}

template<int LMAX>
void launch_l(const BondsDev &b, const LayerDev &L, const float *gQ, int NA, int a0, int na, float *fv,
              double *vir_atom, int add)
{
  const int C = L.C, nI = L.n_msg + 1;
  if (C > 64) throw Unsupported("bond sums with more than 64 channels are not supported");
  if (C > 32) launch_t<LMAX, 1, 2, 32>(b, L, gQ, NA, a0, na, fv, vir_atom, add);
  else if (C > 16) { if (nI == 5) launch_t<LMAX, 5, 1, 32>(b, L, gQ, NA, a0, na, fv, vir_atom, add); else launch_t<LMAX, 1, 1, 32>(b, L, gQ, NA, a0, na, fv, vir_atom, add); }
  else if (nI == 5 && !L.Rex && !getenv("GRACE_B200_BOND_NOSPLIT"))
    GB_LAUNCH((bond_bwd_split_kernel<LMAX, 5>), na, 128, 0, b, L, sh_table_host(), gQ, NA, a0, fv, vir_atom, add);
  else { if (nI == 5) launch_t<LMAX, 5, 1, 16>(b, L, gQ, NA, a0, na, fv, vir_atom, add); else launch_t<LMAX, 1, 1, 16>(b, L, gQ, NA, a0, na, fv, vir_atom, add); }
}

}    // namespace

void launch_bond_bwd(int lmax, const BondsDev &b, const LayerDev &L, const float *gQ, int NA, int a0, int na,
                     float *fv, double *vir_atom, int add)
{
  if (na == 0) return;
  switch (lmax) {
    case 1: launch_l<1>(b, L, gQ, NA, a0, na, fv, vir_atom, add); break;
    case 2: launch_l<2>(b, L, gQ, NA, a0, na, fv, vir_atom, add); break;
    case 3: launch_l<3>(b, L, gQ, NA, a0, na, fv, vir_atom, add); break;
    case 4: launch_l<4>(b, L, gQ, NA, a0, na, fv, vir_atom, add); break;
    default: throw Unsupported("lmax must be 1..4");
  }
}

}    // namespace gb
