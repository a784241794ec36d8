// Forward bond kernel: the neighbour sums of a layer,
//   Q[(I, lm)][a][n] = sum_j Y_lm(rhat_ij) R[n, l](r_ij / rcut) msg_I(j)[n]
// with msg_I the message functions of the neighbour (layer 2: I < n_msg) and, as the last I, its chemical weight
// z[mu_j][n] (layer 1: A; layer 2: B0).  This is atom_scatter + atom_yi of the reference CPU driver
// (libgrace/include/grace/fused_cpu.h:947-1025) in the dense (I, lm) form of its GPU kernels
// (libgrace/include/grace/kk/grace_2l_fused_kk_impl.h:858-1070).
//
// One block of 4 warps per atom.  A lane owns channel n (NCH channels for C > 32); the 4 warps (and with C <= 16 the
// two half-warps) take the atom's bonds in turn, every thread keeping all NIT x NLM partial sums of its channel in
// registers; the partial sums of the warps are added in shared memory in a fixed order and written once, coalesced
// over n: no global atomics, bit-reproducible.
#include "bond_common.cuh"

#include <cstdlib>

namespace gb {

namespace {

constexpr int EB = 96;    // bonds staged per round: most atoms in one round

template<int LMAX, int NIT, int NCH, int LPE, bool EXACT>
__global__ void __launch_bounds__(128) bond_fwd_kernel(BondsDev b, LayerDev L, SHTable sht, float *__restrict__ Q,
                                                       int NA, int a0)
{
  // rows of the staged harmonics: a multiple of 4 floats (the lanes of a bond read them as broadcast 16-byte loads, a
  // quarter of the shared-memory transactions of scalar reads) plus 4, which spreads the rows over the banks
  constexpr int NL = LMAX + 1, NLM = NL * NL, NLM4 = (NLM + 3) / 4, NLMP = 4 * NLM4 + ((4 * NLM4 + 4) % 32 ? 4 : 8), NQ = NIT * NLM, CP = LPE * NCH, EPW = 32 / LPE;
  __shared__ __align__(16) float Ys[EB][NLMP];
  __shared__ float st[EB];
  __shared__ int sk[EB], smu[EB], sj[EB];
  __shared__ float red[NQ][CP];

  const int a = blockIdx.x, i = b.ilist ? b.ilist[a0 + a] : a0 + a, tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
  const int ln = lane % LPE, esub = lane / LPE;
  const int Ibase = blockIdx.y * NIT;
  const long long base = b.off[i];
  const int nb = b.cnt[i];
  const int mui = b.mu[i];
  const int C = L.C, nel = L.n_elements;

  float acc[NIT][NLM][NCH];
#pragma unroll
  for (int I = 0; I < NIT; I++)
#pragma unroll
    for (int q = 0; q < NLM; q++)
#pragma unroll
      for (int ch = 0; ch < NCH; ch++) acc[I][q][ch] = 0.0f;

  for (int b0 = 0; b0 < nb; b0 += EB) {
    const int nbat = min(EB, nb - b0);
    for (int e = tid; e < nbat; e += 128) {
      const float4 rec = b.rec[base + b0 + e];
      const float r = sqrtf(rec.x * rec.x + rec.y * rec.y + rec.z * rec.z), ir = 1.0f / r;
      const int j = __float_as_int(rec.w);
      const int muj = b.mu[j];
      int k;
      float t;
      spline_locate(r / L.rc[mui * nel + muj], L.N, k, t);
      sk[e] = k; st[e] = t; smu[e] = muj; sj[e] = j;
      float *y = Ys[e];
      sph_harm<LMAX, false>(sht, rec.x * ir, rec.y * ir, rec.z * ir,
                            [&](int lm, float v, float, float, float) { y[lm] = v; });
    }
    __syncthreads();
    for (int e0 = w * EPW; e0 < nbat; e0 += 4 * EPW) {
      const int e = e0 + esub;
      if (e < nbat) {
        const int k = sk[e], muj = smu[e], j = sj[e];
        const float t = st[e];
        float y[4 * NLM4];
#pragma unroll
        for (int q4 = 0; q4 < NLM4; q4++) {
          const float4 v = reinterpret_cast<const float4 *>(Ys[e])[q4];
          y[4 * q4] = v.x; y[4 * q4 + 1] = v.y; y[4 * q4 + 2] = v.z; y[4 * q4 + 3] = v.w;
        }
#pragma unroll
        for (int ch = 0; ch < NCH; ch++) {
          const int n = ln + ch * LPE;
          if (n < C) {
            float R[NL];
            if (EXACT) {    // exact radial MLP, evaluated per slot beforehand
              const float *rr = L.Rex + (size_t) (base + b0 + e) * (NL * C) + n;
#pragma unroll
              for (int l = 0; l < NL; l++) R[l] = __ldg(rr + l * C);
            } else {
              const float4 *cf = reinterpret_cast<const float4 *>(L.tab) + (size_t) k * NL * C + n;
#pragma unroll
              for (int l = 0; l < NL; l++) {
                const float4 c = __ldg(cf + l * C);
                R[l] = c.x + t * (c.y + t * (c.z + t * c.w));
              }
            }
#pragma unroll
            for (int I = 0; I < NIT; I++) {
              const int Ig = Ibase + I;
              float m = 0.0f;
              if (Ig < L.n_msg) m = __ldg(L.msg + ((size_t) j * L.n_msg + Ig) * C + n);
              else if (Ig == L.n_msg) m = __ldg(L.z + (size_t) muj * C + n);
#pragma unroll
              for (int l = 0; l < NL; l++) {
                const float rm = R[l] * m;
#pragma unroll
                for (int q = l * l; q < (l + 1) * (l + 1); q++) acc[I][q][ch] = fmaf(y[q], rm, acc[I][q][ch]);
              }
            }
          }
        }
      }
    }
    __syncthreads();
  }

  if (EPW == 2) {    // the two half-warps worked on different bonds: add them
#pragma unroll
    for (int I = 0; I < NIT; I++)
#pragma unroll
      for (int q = 0; q < NLM; q++) acc[I][q][0] += __shfl_xor_sync(0xffffffffu, acc[I][q][0], 16);
  }
  for (int ww = 0; ww < 4; ww++) {
    if (w == ww && esub == 0) {
#pragma unroll
      for (int I = 0; I < NIT; I++)
#pragma unroll
        for (int q = 0; q < NLM; q++)
#pragma unroll
          for (int ch = 0; ch < NCH; ch++) {
            float *r = &red[I * NLM + q][ln + ch * LPE];
            *r = (ww == 0) ? acc[I][q][ch] : *r + acc[I][q][ch];
          }
    }
    __syncthreads();
  }
  for (int idx = tid; idx < NQ * C; idx += 128) {
    const int q = idx / C, n = idx - q * C;
    if (Ibase + q / NLM <= L.n_msg) Q[((size_t) (Ibase * NLM + q) * NA + a) * C + n] = red[q][n];
  }
}

// The same for layers that couple message functions in (NIT > 1) with at most 16 channels: a whole warp per bond, lane
// = (channel n, half h) with the lm split between the halves (lm = h NK + k), so that a lane keeps NIT x NLM / 2 partial
// sums in registers instead of NIT x NLM (twice the resident warps) and the two halves share the work of a bond:
//   Q[(I, lm)][n] += (Y_lm R_l) msg_I      with R of the lm's degree selected per lm.
template<int LMAX, int NIT>
__global__ void __launch_bounds__(128) bond_fwd_split_kernel(BondsDev b, LayerDev L, SHTable sht, float *__restrict__ Q, int NA,
                                                             int a0)
{
  // half h of a bond's lanes takes lm = h NK .. h NK + NK - 1: contiguous, so that its harmonics come as broadcast
  // 16-byte loads (rows of NK4 float4 per half)
  constexpr int NL = LMAX + 1, NLM = NL * NL, NQ = NIT * NLM, NK = (NLM + 1) / 2, NK4 = (NK + 3) / 4, NLMP = 8 * NK4 + 4;
  __shared__ __align__(16) float Ys[EB][NLMP];
  __shared__ float st[EB];
  __shared__ int sk[EB], smu[EB], sj[EB];
  __shared__ float red[NQ][16];

  const int a = blockIdx.x, i = b.ilist ? b.ilist[a0 + a] : a0 + a, tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
  const int n = lane & 15, h = lane >> 4;
  const long long base = b.off[i];
  const int nb = b.cnt[i];
  const int mui = b.mu[i];
  const int C = L.C, nel = L.n_elements;

  float acc[NIT][NK];
#pragma unroll
  for (int I = 0; I < NIT; I++)
#pragma unroll
    for (int k = 0; k < NK; k++) acc[I][k] = 0.0f;

  for (int b0 = 0; b0 < nb; b0 += EB) {
    const int nbat = min(EB, nb - b0);
    for (int e = tid; e < nbat; e += 128) {
      const float4 rec = b.rec[base + b0 + e];
      const float r = sqrtf(rec.x * rec.x + rec.y * rec.y + rec.z * rec.z), ir = 1.0f / r;
      const int j = __float_as_int(rec.w);
      const int muj = b.mu[j];
      int k;
      float t;
      spline_locate(r / L.rc[mui * nel + muj], L.N, k, t);
      sk[e] = k; st[e] = t; smu[e] = muj; sj[e] = j;
      float *y = Ys[e];
      sph_harm<LMAX, false>(sht, rec.x * ir, rec.y * ir, rec.z * ir,
                            [&](int lm, float v, float, float, float) { y[lm < NK ? lm : 4 * NK4 + lm - NK] = v; });
    }
    __syncthreads();
    for (int e = w; e < nbat; e += 4) {    // a warp per bond
      if (n < C) {
        const int k0 = sk[e], muj = smu[e], j = sj[e];
        const float t = st[e];
        float y[4 * NK4];
#pragma unroll
        for (int q4 = 0; q4 < NK4; q4++) {
          const float4 v = reinterpret_cast<const float4 *>(Ys[e])[h * NK4 + q4];
          y[4 * q4] = v.x; y[4 * q4 + 1] = v.y; y[4 * q4 + 2] = v.z; y[4 * q4 + 3] = v.w;
        }
        float R[NL];
        const float4 *cf = reinterpret_cast<const float4 *>(L.tab) + (size_t) k0 * NL * C + n;
#pragma unroll
        for (int l = 0; l < NL; l++) {
          const float4 c = __ldg(cf + l * C);
          R[l] = c.x + t * (c.y + t * (c.z + t * c.w));
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
          constexpr auto deg = [](int q) { int l = 0; while ((l + 1) * (l + 1) <= q) l++; return l; };
          const int q = h * NK + k;
          const int l0 = deg(k), l1 = deg(NK + k < NLM ? NK + k : NLM - 1);
          if (q < NLM) {
            const float yr = y[k] * (h ? R[l1] : R[l0]);
#pragma unroll
            for (int I = 0; I < NIT; I++) acc[I][k] = fmaf(yr, m[I], acc[I][k]);
          }
        }
      }
    }
    __syncthreads();
  }

  for (int ww = 0; ww < 4; ww++) {    // the partial sums of the warps, added in warp order
    if (w == ww && n < C) {
#pragma unroll
      for (int I = 0; I < NIT; I++)
#pragma unroll
        for (int k = 0; k < NK; k++) {
          const int q = h * NK + k;
          if (q < NLM) {
            float *r = &red[I * NLM + q][n];
            *r = (ww == 0) ? acc[I][k] : *r + acc[I][k];
          }
        }
    }
    __syncthreads();
  }
  for (int idx = tid; idx < NQ * C; idx += 128) {
    const int q = idx / C, nn = idx - q * C;
    if (q / NLM <= L.n_msg) Q[((size_t) q * NA + a) * C + nn] = red[q][nn];
  }
}

template<int LMAX, int NIT, int NCH, int LPE>
void launch_t(const BondsDev &b, const LayerDev &L, float *Q, int NA, int a0, int na)
{
  const int tiles = (L.n_msg + 1 + NIT - 1) / NIT;
  if (L.Rex) GB_LAUNCH((bond_fwd_kernel<LMAX, NIT, NCH, LPE, true>), dim3(na, tiles), 128, 0, b, L, sh_table_host(), Q, NA, a0);
  else GB_LAUNCH((bond_fwd_kernel<LMAX, NIT, NCH, LPE, false>), dim3(na, tiles), 128, 0, b, L, sh_table_host(), Q, NA, a0);
}

template<int LMAX> void launch_l(const BondsDev &b, const LayerDev &L, float *Q, int NA, int a0, int na)
{
  const int C = L.C, nI = L.n_msg + 1;
  if (C > 64) throw Unsupported("bond sums with more than 64 channels are not supported");
  if (C > 32) launch_t<LMAX, 1, 2, 32>(b, L, Q, NA, a0, na);
  else if (C > 16) { if (nI == 5) launch_t<LMAX, 5, 1, 32>(b, L, Q, NA, a0, na); else launch_t<LMAX, 1, 1, 32>(b, L, Q, NA, a0, na); }
  else if (nI == 5 && !L.Rex && !getenv("GRACE_B200_BOND_NOSPLIT"))
    GB_LAUNCH((bond_fwd_split_kernel<LMAX, 5>), na, 128, 0, b, L, sh_table_host(), Q, NA, a0);
  else { if (nI == 5) launch_t<LMAX, 5, 1, 16>(b, L, Q, NA, a0, na); else launch_t<LMAX, 1, 1, 16>(b, L, Q, NA, a0, na); }
}

}    // namespace

__global__ void __launch_bounds__(128) bond_x_kernel(BondsDev b, const float *__restrict__ rc, int nel, float *x)
{
  const int i = blockIdx.x;
  const long long base = b.off[i];
  const int ns = (int) (b.off[i + 1] - base), nb = b.cnt[i], mui = b.mu[i];
  for (int s = threadIdx.x; s < ns; s += 128) {
    float v = 0.5f;
    if (s < nb) {
      const float4 rec = b.rec[base + s];
      const int j = __float_as_int(rec.w);
      v = sqrtf(rec.x * rec.x + rec.y * rec.y + rec.z * rec.z) / rc[mui * nel + b.mu[j]];
    }
    x[base + s] = v;
  }
}

void launch_bond_x(const BondsDev &b, const float *rc, int n_elements, float *x, long long n)
{
  if (n == 0) return;
  GB_LAUNCH(bond_x_kernel, (unsigned) n, 128, 0, b, rc, n_elements, x);
}

void launch_bond_fwd(int lmax, const BondsDev &b, const LayerDev &L, float *Q, int NA, int a0, int na)
{
  if (na == 0) return;
  switch (lmax) {
    case 1: launch_l<1>(b, L, Q, NA, a0, na); break;
    case 2: launch_l<2>(b, L, Q, NA, a0, na); break;
    case 3: launch_l<3>(b, L, Q, NA, a0, na); break;
    case 4: launch_l<4>(b, L, Q, NA, a0, na); break;
    default: throw Unsupported("lmax must be 1..4");
  }
}

}    // namespace gb
