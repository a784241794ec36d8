// GRACE-3L evaluation: three message-passing layers (libgrace/src/fused_3l.cpp:1204-1637).  Per layer: the bond sums of
// the single-particle basis (per-pair radial tables, spherical harmonics, the normalised message of the layer before
// coupled in through the sparse cg_W), the dense chain of the layer as MV / PROD operations of the plan (cp_l
// projections, couples, reduces, FCs: the same kernels as GRACE-1L / 2L), EquivariantRMSNorm of the message and RMSNorm
// of the density; the readout on the sum of the three densities; then everything in reverse.  While they fit, the
// tensors of the three layers of all atoms are kept for the reverse pass; larger structures run every layer in passes
// over atom chunks and recompute a chunk's forward tensors when it is reversed.  A first form of the path, checked
// against the reference's CPU engine; its bond kernels are bound by instruction issue and not tuned.
#include "engine.h"

#include "bond_common.cuh"

#include <algorithm>
#include <cstdlib>

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
constexpr int S3_T = 5;      // a thread keeps a tile of S3_T x S3_T (Y lm, message function) pairs of one channel in registers

// Thread layout of both kernels.  A CTA works on one atom and a slice of CC = 2^cshift channels (blockIdx.y); thread
// tid has the channel c = tid % CC of the slice and the tile g = tid / CC of the (ly, li) plane: ly in [5 tl, 5 tl + 5),
// li in [5 ti, 5 ti + 5) with tl = g / nTI, ti = g % nTI.  The 25 products of a tile and a bond need 5 + 5 shared-memory
// reads, and the bond sums P (or their gradients) never leave the registers.

__device__ __forceinline__ void s3_cp16(void *dst_smem, const void *src)
{
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned) __cvta_generic_to_shared(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void s3_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void s3_cp_wait() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// geometry of a bond: neighbour, its element, table of the element pair, table row and offset, distance and cutoff.
// Worked out once per batch of bonds by one thread per bond (a chain of dependent global loads: record -> element of the
// neighbour -> table of the pair) and kept in shared memory, 8 words per bond.
struct S3Bond {
  int j, muj, slot, k0;
  float t, r, rc;
};
__device__ __forceinline__ void s3_bond_store(const BondsDev &b, const Spbf3Dev &L, long long at, int mui, float *meta)
{
  const float4 rec = b.rec[at];
  const int j = __float_as_int(rec.w), muj = b.mu[j];
  const float r = sqrtf(rec.x * rec.x + rec.y * rec.y + rec.z * rec.z), rc = L.rc[mui * L.nel + muj];
  int k0;
  float t;
  spline_locate(r / rc, L.N, k0, t);
  meta[0] = __int_as_float(j);
  meta[1] = __int_as_float(muj);
  meta[2] = __int_as_float(L.pair_slot[mui * L.nel + muj]);    // < 0: no table for this element pair, the bond is left out
  meta[3] = __int_as_float(k0);
  meta[4] = t;
  meta[5] = r;
  meta[6] = rc;
}
__device__ __forceinline__ S3Bond s3_bond(const float *meta)
{
  S3Bond o;
  o.j = __float_as_int(meta[0]);
  o.muj = __float_as_int(meta[1]);
  o.slot = __float_as_int(meta[2]);
  o.k0 = __float_as_int(meta[3]);
  o.t = meta[4];
  o.r = meta[5];
  o.rc = meta[6];
  return o;
}

// asynchronous copies of what the bonds [at, at + ns) of an atom read from global memory, for the channel slice c0 ..
// c0 + CC: the table rows [nl][CC] float4 of each bond to craw, the message rows [nlmi][CC] of its neighbour to mraw,
// the chemical weights [CC] of the neighbour's element to zraw
__device__ __forceinline__ void s3_issue(const Spbf3Dev &L, const float *meta, int ns, int c0, int cshift, float4 *craw, float *mraw,
                                         float *zraw, int tid, int nth)
{
  const int CC = 1 << cshift, nT = L.nl * CC, nM4 = L.nlmi * CC / 4;
  for (int s = 0; s < ns; s++) {
    const S3Bond B = s3_bond(meta + 8 * s);
    if (tid < CC / 4) s3_cp16(zraw + s * CC + 4 * tid, L.zproj + (size_t) B.muj * L.C + c0 + 4 * tid);
    const float4 *tab = reinterpret_cast<const float4 *>(L.tab + (size_t) max(B.slot, 0) * L.tab_stride) + (size_t) B.k0 * L.nl * L.C + c0;
    for (int e = tid; e < nT; e += nth) s3_cp16(craw + s * nT + e, tab + (e >> cshift) * L.C + (e & (CC - 1)));
    if (L.msg) {
      const float *m = L.msg + (size_t) B.j * L.nlmi * L.C + c0;
      for (int e = tid; e < nM4; e += nth) {
        const int li = (4 * e) >> cshift, cc = (4 * e) & (CC - 1);
        s3_cp16(mraw + s * L.nlmi * CC + 4 * e, m + (size_t) li * L.C + cc);
      }
    }
  }
  s3_cp_commit();
}

// ---- forward bond sums on the tensor cores --------------------------------------------------------------------------
// For one atom and one channel c the bond sums are a small matrix product over the bonds j:
//     P[ly][li] = sum_j U[j][ly] Ic[j][li],   U[j][ly] = Y_ly(j) R_l(ly)(j)[c],  Ic[j][li] = msg_j[li][c] + mask[li] z[mu_j][c]
// with M = (lmax + 1)^2 <= 32 rows, N = message functions <= 32 columns, K = bonds.  A warp owns a channel and keeps the
// 32 x 32 accumulators in registers (mma.sync m16n8k8 tf32, 2 x 4 tiles); every product is three instructions on hi / lo
// splits (a_lo b_hi + a_hi b_lo + a_hi b_hi), which keeps fp32-level accuracy.  A CTA works on one atom and a slice of
// 16 channels; the operands of 16 bonds at a time are staged in shared memory with a row stride of 40 floats, which
// makes the fragment reads of a warp conflict-free.
constexpr int S3M_CH = 16, S3M_GB = 16, S3M_LD = 40, S3M_CS = S3M_GB * S3M_LD + 1;    // CS: floats per channel block (odd: the
                                                                                        // channel-major stores of the staging spread over the banks)

__device__ __forceinline__ void s3_split(float x, unsigned &hi, unsigned &lo)
{
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(x));
  const float r = x - __uint_as_float(hi);
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(r));
}
__device__ __forceinline__ void s3_mma(float (&d)[4], const unsigned (&a)[4], const unsigned (&b)[2])
{
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__global__ void __launch_bounds__(32 * S3M_CH) spbf3_fwd_mma_kernel(BondsDev b, Spbf3Dev L, SHTable sht, float *__restrict__ A, int NA, int a0)
{
  extern __shared__ __align__(16) float sm[];
  const int C = L.C, nlm = L.nlm, nlmi = L.nlmi, nth = blockDim.x;
  float *Us = sm, *Is = Us + S3M_CH * S3M_CS, *meta = Is + S3M_CH * S3M_CS + 3, *Ys = meta + 8 * S3_BB;
  float *mask = Ys + S3_BB * nlm;
  int *lts = reinterpret_cast<int *>(mask + 32);
  const int a = blockIdx.x, i = a0 + a, c0 = blockIdx.y * S3M_CH, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const long long base = b.off[i];
  const int nb = b.cnt[i], mui = b.mu[i];
  float acc[2][4][4];
#pragma unroll
  for (int mt = 0; mt < 2; mt++)
#pragma unroll
    for (int nt = 0; nt < 4; nt++)
#pragma unroll
      for (int r = 0; r < 4; r++) acc[mt][nt][r] = 0.0f;
  for (int e = tid; e < nlm; e += nth) lts[e] = L.lt[e];
  for (int e = tid; e < 32; e += nth) mask[e] = e < nlmi ? L.l0mask[e] : 0.0f;
  for (int q0 = 0; q0 < nb; q0 += S3_BB) {
    const int nq = min(S3_BB, nb - q0);
    __syncthreads();    // harmonics and geometry of the previous batch are no longer read
    for (int e = tid; e < nq; e += nth) {
      const float4 rec = b.rec[base + q0 + e];
      const float ir = rsqrtf(rec.x * rec.x + rec.y * rec.y + rec.z * rec.z);
      stage_harmonics(sht, rec.x * ir, rec.y * ir, rec.z * ir, nlm, Ys + e * nlm, nullptr);
      s3_bond_store(b, L, base + q0 + e, mui, meta + 8 * e);
    }
    for (int q = 0; q < nq; q += S3M_GB) {
      const int ns = min(S3M_GB, nq - q);
      __syncthreads();    // the operands of the previous group are no longer read; harmonics and geometry are staged
      // operands of the group: rows (channel, bond), the function index runs along the lanes; rows of bonds beyond the
      // group and functions beyond the model's are zero
      for (int e = tid; e < S3M_CH * S3M_GB * 32; e += nth) {    // U: a warp per (channel, bond) row, the lanes along ly
        const int f = e & 31, row = e >> 5, s = row % S3M_GB, ch = row / S3M_GB;
        float u = 0.0f;
        if (s < ns && f < nlm) {
          const S3Bond B = s3_bond(meta + 8 * (q + s));
          if (B.slot >= 0) {
            const float4 cf = reinterpret_cast<const float4 *>(L.tab + (size_t) B.slot * L.tab_stride)[((size_t) B.k0 * L.nl + lts[f]) * C + c0 + ch];
            u = Ys[(q + s) * nlm + f] * (cf.x + B.t * (cf.y + B.t * (cf.z + B.t * cf.w)));
          }
        }
        Us[ch * S3M_CS + s * S3M_LD + f] = u;
      }
      for (int e = tid; e < S3M_GB * 32 * S3M_CH; e += nth) {    // Ic: the lanes along the channels (whole 64-byte pieces of a row)
        const int ch = e % S3M_CH, f = (e / S3M_CH) & 31, s = e / (S3M_CH * 32);
        float ic = 0.0f;
        if (s < ns && f < nlmi) {
          const S3Bond B = s3_bond(meta + 8 * (q + s));
          ic = (L.msg ? L.msg[((size_t) B.j * nlmi + f) * C + c0 + ch] : 0.0f) + mask[f] * L.zproj[(size_t) B.muj * C + c0 + ch];
        }
        Is[ch * S3M_CS + s * S3M_LD + f] = ic;
      }
      __syncthreads();
      const float *Uw = Us + warp * S3M_CS, *Iw = Is + warp * S3M_CS;
#pragma unroll
      for (int k8 = 0; k8 < S3M_GB; k8 += 8) {
        if (k8 >= ns) break;
        // A[m = ly][k = bond] = U[bond][ly], B[k = bond][n = li] = Ic[bond][li]
        unsigned ah[2][4], al[2][4], bh[4][2], bl[4][2];
#pragma unroll
        for (int mt = 0; mt < 2; mt++) {
          s3_split(Uw[(k8 + t) * S3M_LD + 16 * mt + g], ah[mt][0], al[mt][0]);
          s3_split(Uw[(k8 + t) * S3M_LD + 16 * mt + g + 8], ah[mt][1], al[mt][1]);
          s3_split(Uw[(k8 + t + 4) * S3M_LD + 16 * mt + g], ah[mt][2], al[mt][2]);
          s3_split(Uw[(k8 + t + 4) * S3M_LD + 16 * mt + g + 8], ah[mt][3], al[mt][3]);
        }
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
          s3_split(Iw[(k8 + t) * S3M_LD + 8 * nt + g], bh[nt][0], bl[nt][0]);
          s3_split(Iw[(k8 + t + 4) * S3M_LD + 8 * nt + g], bh[nt][1], bl[nt][1]);
        }
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
          for (int nt = 0; nt < 4; nt++) {
            s3_mma(acc[mt][nt], al[mt], bh[nt]);
            s3_mma(acc[mt][nt], ah[mt], bl[nt]);
            s3_mma(acc[mt][nt], ah[mt], bh[nt]);
          }
      }
    }
  }
  // P of the 16 channels to shared memory [channel][ly][li] (32 x 33), then the couple: one thread per (function, channel)
  __syncthreads();
  float *Ps = sm;
  {
    float *Pw = Ps + warp * 32 * 33;
#pragma unroll
    for (int mt = 0; mt < 2; mt++)
#pragma unroll
      for (int nt = 0; nt < 4; nt++) {
        Pw[(16 * mt + g) * 33 + 8 * nt + 2 * t] = acc[mt][nt][0];
        Pw[(16 * mt + g) * 33 + 8 * nt + 2 * t + 1] = acc[mt][nt][1];
        Pw[(16 * mt + g + 8) * 33 + 8 * nt + 2 * t] = acc[mt][nt][2];
        Pw[(16 * mt + g + 8) * 33 + 8 * nt + 2 * t + 1] = acc[mt][nt][3];
      }
  }
  __syncthreads();
  for (int e = tid; e < L.nfA * S3M_CH; e += nth) {
    const int f = e / S3M_CH, ch = e - f * S3M_CH;
    const float *Pc = Ps + ch * 32 * 33;
    float v = 0.0f;
    for (int k = L.cg_off[f]; k < L.cg_off[f + 1]; k++) {
      const int q = L.cg_p[k], ly = q / nlmi, li = q - ly * nlmi;
      v = fmaf(L.cg_v[k], Pc[ly * 33 + li], v);
    }
    A[((size_t) f * NA + a) * C + c0 + ch] = v;
  }
}

constexpr int S3_NBS = 4;    // bonds staged and worked on together: one pair of barriers and one round of global loads for all

// A[f][a][c] = sum_q cg[q, f] P[q][c],  P[(ly, li)][c] = sum_bonds Y_ly R[l(ly)][c] (msg_j[li][c] + mask[li] zproj[mu_j][c])
__global__ void __launch_bounds__(832) spbf3_fwd_kernel(BondsDev b, Spbf3Dev L, SHTable sht, float *__restrict__ A, int NA, int cshift,
                                                        int nTI, int a0)
{
  extern __shared__ __align__(16) float sm[];
  const int C = L.C, nlm = L.nlm, nlmi = L.nlmi, CC = 1 << cshift, nth = blockDim.x;
  const int nU = nlm * CC, nI = nlmi * CC;
  const int nT = L.nl * CC;
  float4 *craw = reinterpret_cast<float4 *>(sm);                      // [2][NBS][nl][CC] table rows
  float *mraw = reinterpret_cast<float *>(craw + 2 * S3_NBS * nT);    // [2][NBS][nlmi][CC] message rows
  float *zraw = mraw + 2 * (size_t) S3_NBS * nI;                      // [2][NBS][CC] chemical weights of the neighbours' elements
  float *meta = zraw + 2 * S3_NBS * CC, *Ys = meta + 8 * S3_BB, *U = Ys + S3_BB * nlm, *Ic = U + (size_t) S3_NBS * nU,
        *As = Ic + (size_t) S3_NBS * nI, *mask = As + (size_t) L.nfA * CC;
  int *lts = reinterpret_cast<int *>(mask + nlmi);                    // l of each lm, and the mask of the message functions above
  const int ap = blockIdx.x, i = a0 + ap, c0 = blockIdx.y * CC, tid = threadIdx.x;
  const int c = tid & (CC - 1), g = tid >> cshift, tl = g / nTI, ti = g - tl * nTI, ly0 = S3_T * tl, li0 = S3_T * ti;
  const long long base = b.off[i];
  const int nb = b.cnt[i], mui = b.mu[i];
  float acc[S3_T][S3_T];
#pragma unroll
  for (int a = 0; a < S3_T; a++)
#pragma unroll
    for (int q = 0; q < S3_T; q++) acc[a][q] = 0.0f;
  for (int e = tid; e < nlm; e += nth) lts[e] = L.lt[e];
  for (int e = tid; e < nlmi; e += nth) mask[e] = L.l0mask[e];
  for (int q0 = 0; q0 < nb; q0 += S3_BB) {
    const int nq = min(S3_BB, nb - q0);
    __syncthreads();    // the harmonics of the previous batch are no longer read
    for (int e = tid; e < nq; e += nth) {
      const float4 rec = b.rec[base + q0 + e];
      const float ir = rsqrtf(rec.x * rec.x + rec.y * rec.y + rec.z * rec.z);
      stage_harmonics(sht, rec.x * ir, rec.y * ir, rec.z * ir, nlm, Ys + e * nlm, nullptr);
      s3_bond_store(b, L, base + q0 + e, mui, meta + 8 * e);
    }
    __syncthreads();
    s3_issue(L, meta, min(S3_NBS, nq), c0, cshift, craw, mraw, zraw, tid, nth);    // the first group of the batch
    for (int q = 0, k = 0; q < nq; q += S3_NBS, k ^= 1) {
      const int ns = min(S3_NBS, nq - q);
      s3_cp_wait();
      __syncthreads();    // this group's rows have arrived; U and Ic of the previous group are no longer read
      if (q + S3_NBS < nq)    // the next group's rows travel while this group is worked on
        s3_issue(L, meta + 8 * (q + S3_NBS), min(S3_NBS, nq - q - S3_NBS), c0, cshift, craw + (k ^ 1) * S3_NBS * nT,
                 mraw + (size_t) (k ^ 1) * S3_NBS * nI, zraw + (k ^ 1) * S3_NBS * CC, tid, nth);
      for (int s = 0; s < ns; s++) {
        const S3Bond B = s3_bond(meta + 8 * (q + s));
        const float4 *cr = craw + (k * S3_NBS + s) * nT;
        const float *mr = mraw + (size_t) (k * S3_NBS + s) * nI, *Y = Ys + (q + s) * nlm;
        const float t = B.t;
        for (int e = tid; e < nU; e += nth) {    // U[ly][c] = Y_ly R_l(ly)[c]
          const int ly = e >> cshift, cc = e & (CC - 1);
          const float4 cf = cr[lts[ly] * CC + cc];
          U[s * nU + e] = B.slot < 0 ? 0.0f : Y[ly] * (cf.x + t * (cf.y + t * (cf.z + t * cf.w)));
        }
        for (int e = tid; e < nI; e += nth) {
          const int li = e >> cshift, cc = e & (CC - 1);
          Ic[s * nI + e] = (L.msg ? mr[e] : 0.0f) + mask[li] * zraw[(k * S3_NBS + s) * CC + cc];
        }
      }
      __syncthreads();
      for (int s = 0; s < ns; s++) {
        float u[S3_T], ic[S3_T];
#pragma unroll
        for (int a = 0; a < S3_T; a++) u[a] = ly0 + a < nlm ? U[s * nU + (ly0 + a) * CC + c] : 0.0f;
#pragma unroll
        for (int q2 = 0; q2 < S3_T; q2++) ic[q2] = li0 + q2 < nlmi ? Ic[s * nI + (li0 + q2) * CC + c] : 0.0f;
#pragma unroll
        for (int a = 0; a < S3_T; a++)
#pragma unroll
          for (int q2 = 0; q2 < S3_T; q2++) acc[a][q2] = fmaf(u[a], ic[q2], acc[a][q2]);
      }
    }
  }
  // the couple: every pair's sum goes to the functions it feeds (shared-memory adds), then the slice is written
  __syncthreads();
  for (int e = tid; e < L.nfA * CC; e += nth) As[e] = 0.0f;
  __syncthreads();
#pragma unroll
  for (int a = 0; a < S3_T; a++)
#pragma unroll
    for (int q2 = 0; q2 < S3_T; q2++) {
      if (ly0 + a >= nlm || li0 + q2 >= nlmi) continue;
      const int q = (ly0 + a) * nlmi + li0 + q2;
      for (int t = L.cgt_off[q]; t < L.cgt_off[q + 1]; t++) atomicAdd(&As[L.cgt_f[t] * CC + c], L.cgt_v[t] * acc[a][q2]);
    }
  __syncthreads();
  for (int e = tid; e < L.nfA * CC; e += nth) {
    const int f = e >> cshift, cc = e & (CC - 1);
    A[((size_t) f * NA + ap) * C + c0 + cc] = As[e];
  }
}

// Reverse of the above from gA: bond forces and per-atom virial (added: the caller clears them before the first layer
// is reversed), dE/dmsg of the neighbours.  The thread's tile of gP[(ly, li)][c] = sum_f cg[q, f] gA[f][c] stays in
// registers; per bond
//   W[ly][c] = sum_li gP Ic[li][c],   dE/dmsg_j[li][c] += sum_ly gP Y_ly R_l[c]      (tiles add their shares in shared memory)
//   gY[ly] = sum_c W R_l[c] (a warp per ly),  dE/dx = sum_{ly, c} W Y_ly dR_l[c]
// and the bond force is linear in (gY, dE/dx), so every channel slice adds its own share.
__global__ void __launch_bounds__(832) spbf3_bwd_kernel(BondsDev b, Spbf3Dev L, SHTable sht, const float *__restrict__ gA, int NA,
                                                        float *__restrict__ fv, double *__restrict__ vir_atom, int cshift, int nTI,
                                                        int a0)
{
  extern __shared__ __align__(16) float sm[];
  const int C = L.C, nlm = L.nlm, nlmi = L.nlmi, CC = 1 << cshift, nth = blockDim.x;
  const int nU = nlm * CC, nI = nlmi * CC;
  const int nT = L.nl * CC;
  float4 *craw = reinterpret_cast<float4 *>(sm);                      // [2][NBS][nl][CC] table rows
  float *mraw = reinterpret_cast<float *>(craw + 2 * S3_NBS * nT);    // [2][NBS][nlmi][CC] message rows
  float *zraw = mraw + 2 * (size_t) S3_NBS * nI;                      // [2][NBS][CC] chemical weights of the neighbours' elements
  float *meta = zraw + 2 * S3_NBS * CC, *Ys = meta + 8 * S3_BB, *Gs = Ys + S3_BB * nlm, *Rl = Gs + 3 * S3_BB * nlm, *dRl = Rl + (size_t) S3_NBS * nU,
        *W = dRl + (size_t) S3_NBS * nU;
  float *Ic = W + (size_t) S3_NBS * nU, *gI = Ic + (size_t) S3_NBS * nI, *gY = gI + (size_t) S3_NBS * nI, *dedx = gY + S3_NBS * nlm;
  float *mask = dedx + 8;
  int *lts = reinterpret_cast<int *>(mask + nlmi);
  const int ap = blockIdx.x, i = a0 + ap, c0 = blockIdx.y * CC, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = tid & (CC - 1), g = tid >> cshift, tl = g / nTI, ti = g - tl * nTI, ly0 = S3_T * tl, li0 = S3_T * ti;
  const long long base = b.off[i];
  const int nb = b.cnt[i], mui = b.mu[i];
  double vir[6] = {0.0, 0.0, 0.0, 0.0, 0.0, 0.0};
  float gp[S3_T][S3_T];
#pragma unroll
  for (int a = 0; a < S3_T; a++)
#pragma unroll
    for (int q2 = 0; q2 < S3_T; q2++) {
      float v = 0.0f;
      if (ly0 + a < nlm && li0 + q2 < nlmi) {
        const int q = (ly0 + a) * nlmi + li0 + q2;
        for (int t = L.cgt_off[q]; t < L.cgt_off[q + 1]; t++) v = fmaf(L.cgt_v[t], gA[((size_t) L.cgt_f[t] * NA + ap) * C + c0 + c], v);
      }
      gp[a][q2] = v;
    }
  for (int e = tid; e < nlm; e += nth) lts[e] = L.lt[e];
  for (int e = tid; e < nlmi; e += nth) mask[e] = L.l0mask[e];
  for (int q0 = 0; q0 < nb; q0 += S3_BB) {
    const int nq = min(S3_BB, nb - q0);
    __syncthreads();    // the harmonics of the previous batch are no longer read
    for (int e = tid; e < nq; e += nth) {
      const float4 rec = b.rec[base + q0 + e];
      const float ir = rsqrtf(rec.x * rec.x + rec.y * rec.y + rec.z * rec.z);
      stage_harmonics(sht, rec.x * ir, rec.y * ir, rec.z * ir, nlm, Ys + e * nlm, Gs + 3 * e * nlm);
      s3_bond_store(b, L, base + q0 + e, mui, meta + 8 * e);
    }
    __syncthreads();
    s3_issue(L, meta, min(S3_NBS, nq), c0, cshift, craw, mraw, zraw, tid, nth);    // the first group of the batch
    for (int q = 0, k = 0; q < nq; q += S3_NBS, k ^= 1) {
      const int ns = min(S3_NBS, nq - q);
      s3_cp_wait();
      __syncthreads();    // this group's rows have arrived; the buffers of the previous group are no longer read
      if (q + S3_NBS < nq)    // the next group's rows travel while this group is worked on
        s3_issue(L, meta + 8 * (q + S3_NBS), min(S3_NBS, nq - q - S3_NBS), c0, cshift, craw + (k ^ 1) * S3_NBS * nT,
                 mraw + (size_t) (k ^ 1) * S3_NBS * nI, zraw + (k ^ 1) * S3_NBS * CC, tid, nth);
      if (tid < S3_NBS) dedx[tid] = 0.0f;
      for (int s = 0; s < ns; s++) {
        const S3Bond B = s3_bond(meta + 8 * (q + s));
        const float4 *cr = craw + (k * S3_NBS + s) * nT;
        const float *mr = mraw + (size_t) (k * S3_NBS + s) * nI;
        const float t = B.t;
        for (int e = tid; e < nU; e += nth) {
          const int ly = e >> cshift, cc = e & (CC - 1);
          const float4 cf = cr[lts[ly] * CC + cc];
          Rl[s * nU + e] = B.slot < 0 ? 0.0f : cf.x + t * (cf.y + t * (cf.z + t * cf.w));
          dRl[s * nU + e] = B.slot < 0 ? 0.0f : (cf.y + t * (2.0f * cf.z + t * 3.0f * cf.w)) * (float) L.N;
          W[s * nU + e] = 0.0f;
        }
        for (int e = tid; e < nI; e += nth) {
          const int li = e >> cshift, cc = e & (CC - 1);
          Ic[s * nI + e] = (L.msg ? mr[e] : 0.0f) + mask[li] * zraw[(k * S3_NBS + s) * CC + cc];
          gI[s * nI + e] = 0.0f;
        }
      }
      __syncthreads();
#pragma unroll
      for (int s = 0; s < S3_NBS; s++) {    // unrolled: the bonds of the group are independent work for the scheduler
        if (s >= ns) break;
        const float *Y = Ys + (q + s) * nlm;
        float u[S3_T], ic[S3_T];
#pragma unroll
        for (int a = 0; a < S3_T; a++) u[a] = ly0 + a < nlm ? Y[ly0 + a] * Rl[s * nU + (ly0 + a) * CC + c] : 0.0f;
#pragma unroll
        for (int q2 = 0; q2 < S3_T; q2++) ic[q2] = li0 + q2 < nlmi ? Ic[s * nI + (li0 + q2) * CC + c] : 0.0f;
        float w[S3_T], v[S3_T];
#pragma unroll
        for (int a = 0; a < S3_T; a++) w[a] = 0.0f;
#pragma unroll
        for (int q2 = 0; q2 < S3_T; q2++) v[q2] = 0.0f;
#pragma unroll
        for (int a = 0; a < S3_T; a++)
#pragma unroll
          for (int q2 = 0; q2 < S3_T; q2++) {
            w[a] = fmaf(gp[a][q2], ic[q2], w[a]);
            v[q2] = fmaf(gp[a][q2], u[a], v[q2]);
          }
#pragma unroll
        for (int a = 0; a < S3_T; a++)
          if (ly0 + a < nlm) atomicAdd(&W[s * nU + (ly0 + a) * CC + c], w[a]);
        if (L.gmsg) {
#pragma unroll
          for (int q2 = 0; q2 < S3_T; q2++)
            if (li0 + q2 < nlmi) atomicAdd(&gI[s * nI + (li0 + q2) * CC + c], v[q2]);
        }
      }
      __syncthreads();
      for (int s = 0; s < ns; s++) {
        const float *Y = Ys + (q + s) * nlm;
        float part = 0.0f;    // this thread's share of dE/dx
        for (int e = tid; e < nU; e += nth) part = fmaf(W[s * nU + e] * Y[e >> cshift], dRl[s * nU + e], part);
        for (int sh = 16; sh > 0; sh >>= 1) part += __shfl_xor_sync(0xffffffffu, part, sh);
        if (lane == 0 && part != 0.0f) atomicAdd(&dedx[s], part);
        if (L.gmsg) {
          const int j = __float_as_int(meta[8 * (q + s)]);
          for (int e = tid; e < nI / 4; e += nth) {    // four channels per atomic (16-byte vector add)
            const int li = (4 * e) >> cshift, cc = (4 * e) & (CC - 1);
            atomicAdd(reinterpret_cast<float4 *>(L.gmsg + ((size_t) j * nlmi + li) * C + c0 + cc),
                      *reinterpret_cast<const float4 *>(gI + s * nI + 4 * e));
          }
        }
        for (int ly = warp; ly < nlm; ly += nth / 32) {    // a warp per ly: the sum over the channels of the slice
          float v = 0.0f;
          for (int cc = lane; cc < CC; cc += 32) v = fmaf(W[s * nU + ly * CC + cc], Rl[s * nU + ly * CC + cc], v);
          for (int sh = 16; sh > 0; sh >>= 1) v += __shfl_xor_sync(0xffffffffu, v, sh);
          if (lane == 0) gY[s * nlm + ly] = v;
        }
      }
      __syncthreads();
      if (tid < ns) {    // one thread per bond of the group
        const int s = tid;
        const float4 rec = b.rec[base + q0 + q + s];
        const S3Bond B = s3_bond(meta + 8 * (q + s));
        const float r = B.r, ir = 1.0f / r, rc = B.rc;
        const float ux = rec.x * ir, uy = rec.y * ir, uz = rec.z * ir;
        const float *Gq = Gs + 3 * (q + s) * nlm;
        float gx = 0.0f, gy = 0.0f, gz = 0.0f;
        for (int lm = 0; lm < nlm; lm++) {
          const float w = gY[s * nlm + lm];
          gx = fmaf(w, Gq[3 * lm], gx);
          gy = fmaf(w, Gq[3 * lm + 1], gy);
          gz = fmaf(w, Gq[3 * lm + 2], gz);
        }
        const float dEdr = dedx[s] / rc, gr = gx * ux + gy * uy + gz * uz;
        const float f0 = dEdr * ux + (gx - gr * ux) * ir, f1 = dEdr * uy + (gy - gr * uy) * ir, f2 = dEdr * uz + (gz - gr * uz) * ir;
        float *o = fv + 3 * (size_t) b.cslot[base + q0 + q + s];
        atomicAdd(o, f0);
        atomicAdd(o + 1, f1);
        atomicAdd(o + 2, f2);
        const double dx = -(double) ux * r, dy = -(double) uy * r, dz = -(double) uz * r;
        vir[0] += dx * f0; vir[1] += dy * f1; vir[2] += dz * f2;
        vir[3] += dx * f1; vir[4] += dx * f2; vir[5] += dy * f2;
      }
    }
  }
  if (tid < S3_NBS)
    for (int k = 0; k < 6; k++)
      if (vir[k] != 0.0) atomicAdd(vir_atom + 6 * (size_t) i + k, vir[k]);
}

struct EqNormDev {
  const float *dw, *mask, *aff;
  const int *e;
  int nf, C, center;
  double eps;
};

// EquivariantRMSNorm of one atom per thread (libgrace/include/grace/fused_3l_cpu.h:346-370): x [f][NA][C] -> y rows [i][f][C]
__global__ void eqnorm_fwd_kernel(EqNormDev E, const float *__restrict__ x, float *__restrict__ y, int NA, int n, int a0)
{
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  y += (size_t) a0 * E.nf * E.C;    // rows of the atoms of the pass
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
                                  int n, int a0)
{
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  dy += (size_t) a0 * E.nf * E.C;
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
                                   int first, int n, int a0)
{
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float *xi = x + (size_t) i * wr;
  float *s = sum + (size_t) (a0 + i) * wr;
  double q = 0.0;
  for (int c = n0; c < wr; c++) q += (double) xi[c] * xi[c];
  const double r = 1.0 / sqrt(q / (wr - n0) + 1e-10);
  for (int c = 0; c < wr; c++) {
    const float y = c < n0 ? xi[c] : (float) (xi[c] * r) * scale[c - n0];
    s[c] = first ? y : s[c] + y;
  }
}

__global__ void rmsnorm_bwd_kernel(const float *__restrict__ x, const float *__restrict__ scale, int n0, int wr,
                                   const float *__restrict__ dy, float *__restrict__ gx, int n, int a0)
{
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float *xi = x + (size_t) i * wr, *d = dy + (size_t) (a0 + i) * wr;
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
    // (the reference's CPU engine asks for multiples of 16 as well: libgrace/src/fused_3l.cpp:433)
    if (L.C > 64 || L.C % 16) throw Unsupported("GRACE-3L: channel counts must be multiples of 16 up to 64");
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
  // every bond needs the radial table of its element pair: the species of every System / Batch of this engine were
  // prepared when it was created (prepare_species); a bond of a pair without a table is left out by the kernels
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
  // launch shape of the bond kernels of a layer: channel slice, tiles of the (ly, li) plane, threads, shared memory
  struct Shape {
    int cshift, nTI, threads, slices;
    size_t smem_fwd, smem_bwd;
  };
  auto shape = [&](const Layer3Plan &L) {
    const int nTL = (plan_.nlm + S3_T - 1) / S3_T, nTI = (L.nlmi + S3_T - 1) / S3_T, groups = nTL * nTI;
    int cshift = 5;
    while (cshift > 2 && (L.C % (1 << cshift) != 0 || groups * (1 << cshift) > 832)) cshift--;
    const int CC = 1 << cshift;
    if (L.C % CC != 0 || groups * CC > 832) throw Unsupported("GRACE-3L: the coupled bond sums of a layer do not fit a thread block");
    Shape s{};
    s.cshift = cshift;
    s.nTI = nTI;
    s.threads = (groups * CC + 31) / 32 * 32;
    s.slices = L.C / CC;
    const size_t raw = 2 * (size_t) S3_NBS * (4 * (size_t) (plan_.lmax + 1) * CC + (size_t) L.nlmi * CC + CC) + plan_.nlm + L.nlmi + 8;    // the two staging buffers
    s.smem_fwd = sizeof(float) * (raw + 8 * S3_BB + (size_t) S3_BB * plan_.nlm + S3_NBS * ((size_t) plan_.nlm * CC + (size_t) L.nlmi * CC) + (size_t) L.nfA * CC);
    s.smem_bwd = sizeof(float) * (raw + 8 * S3_BB + 4 * (size_t) S3_BB * plan_.nlm +
                                  S3_NBS * (3 * (size_t) plan_.nlm * CC + 2 * (size_t) L.nlmi * CC + plan_.nlm) + 8);
    if (std::max(s.smem_fwd, s.smem_bwd) > 200 * 1024) throw Unsupported("GRACE-3L: the bond sums of a layer do not fit the shared memory");
    return s;
  };
  static bool attr_set = false;
  if (!attr_set) {
    GB_CUDA(cudaFuncSetAttribute(spbf3_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    GB_CUDA(cudaFuncSetAttribute(spbf3_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_set = true;
  }
  // Passes.  When the tensors of all three layers of all atoms fit the memory they are kept from the forward to the
  // reverse pass (arena k holds layer k).  Otherwise every layer runs in passes over atom chunks through one arena, and
  // the reverse pass of a layer evaluates the forward operations of a chunk again before it reverses them: the messages,
  // their gradients and the densities live in per-atom rows outside the arenas either way.
  long long per_all = 0, per_max = 0;
  for (int k = 0; k < 3; k++) {
    per_all += S.E[k].per_atom;
    per_max = std::max(per_max, S.E[k].per_atom);
  }
  size_t free_b = 0, total_b = 0;
  if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) free_b = (size_t) 8 << 30;
  double budget = 0.7 * (double) free_b;
  for (int k = 0; k < 3; k++) budget += 4.0 * (double) S.arena[k].capacity();
  if (const char *env = getenv("GRACE_B200_3L_CHUNK")) budget = std::min(budget, 4.0 * per_all * std::max(4, atoi(env)) - 1.0);
  const bool keep = 4.0 * (double) per_all * NA <= budget;
  int NC = NA;    // atoms per pass (a multiple of 4: the atom stride of the arena)
  if (!keep) {
    NC = (int) std::min<double>(NA, std::max(512.0, budget / (4.0 * per_max)));
    if (const char *env = getenv("GRACE_B200_3L_CHUNK")) NC = std::min(NC, std::max(4, atoi(env)));
    NC = std::max(4, NC / 4 * 4);
    for (int k = 1; k < 3; k++) S.arena[k].release();
  }
  const bool simt_only = getenv("GRACE_B200_3L_MMA") == nullptr;    // read per evaluation
  // GRACE_B200_3L_MMA=1: the forward bond sums as small matrix products on the tensor cores where the shape allows.  Same
  // results; measured slower than the register-tile kernel so far (its operand staging, not the matrix instructions),
  // so it is not the default
  const size_t smem_mma = sizeof(float) * std::max<size_t>(2 * S3M_CH * S3M_CS + 3 + 8 * S3_BB + (size_t) S3_BB * plan_.nlm + 32 + 32,
                                                            (size_t) S3M_CH * 32 * 33);
  static bool mma_attr = false;
  if (!simt_only && !mma_attr) {
    GB_CUDA(cudaFuncSetAttribute(spbf3_fwd_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    mma_attr = true;
  }
  // the arena of layer k bound for passes of NC atoms
  auto bind = [&](int k) {
    LayerEngine &E = S.E[k];
    DBuf<float> &ar = S.arena[keep ? k : 0];
    float *base = ar.ensure((size_t) (keep ? E.per_atom : per_max) * NC);
    bind_arena(E, base, NC);
    return base;
  };
  // forward operations of layer k for the atoms [a0, a0 + na); outputs: the message rows and the density sums
  auto forward = [&](int k, int a0, int na, bool outputs) {
    const Layer3Plan &L = Q.L[k];
    const Shape sh = shape(L);
    LayerEngine &E = S.E[k];
    const std::vector<TensorDev> &T = E.tensors_host;
    const int nbk = (na + nt - 1) / nt;
    if (!simt_only && plan_.nlm <= 32 && L.nlmi <= 32 && L.C % S3M_CH == 0)
      GB_LAUNCH(spbf3_fwd_mma_kernel, dim3(na, L.C / S3M_CH), 32 * S3M_CH, smem_mma, bonds, spbf(k), sht, T[L.tA].p, NC, a0);
    else
      GB_LAUNCH(spbf3_fwd_kernel, dim3(na, sh.slices), sh.threads, sh.smem_fwd, bonds, spbf(k), sht, T[L.tA].p, NC, sh.cshift, sh.nTI, a0);
    run(E, L.dense.fwd, mu + a0, na, NC);
    if (!outputs) return;
    if (k < 2) {
      const EqNormDev e{S.eq_dw[k].get(), S.eq_mask[k].get(), S.eq_aff[k].get(), S.eq_e[k].get(), L.nfEQ, L.cEQ, L.eq_center, L.eq_eps};
      GB_LAUNCH(eqnorm_fwd_kernel, nbk, nt, 0, e, T[L.tEQ].p, S.msg[k].get(), NC, na, a0);
    }
    GB_LAUNCH(rmsnorm_fwd_kernel, nbk, nt, 0, T[L.tRHO].p, S.rho_scale[k].get(), L.rho_n0, wr, S.rho_sum.get(), k == 0 ? 1 : 0, na, a0);
  };
  // reverse operations of layer k for the atoms [a0, a0 + na), whose forward tensors are in the bound arena
  auto reverse = [&](int k, int a0, int na, float *base) {
    const Layer3Plan &L = Q.L[k];
    const Shape sh = shape(L);
    LayerEngine &E = S.E[k];
    const std::vector<TensorDev> &T = E.tensors_host;
    const int nbk = (na + nt - 1) / nt;
    if (L.dense.zero_grads)
      launch_fill_zero(base + (size_t) E.grad_begin * NC, sizeof(float) * (size_t) (E.grad_end - E.grad_begin) * NC);
    GB_LAUNCH(rmsnorm_bwd_kernel, nbk, nt, 0, T[L.tRHO].p, S.rho_scale[k].get(), L.rho_n0, wr, S.drho.get(), T[L.tGRHO].p, na, a0);
    if (k < 2) {
      const EqNormDev e{S.eq_dw[k].get(), S.eq_mask[k].get(), S.eq_aff[k].get(), S.eq_e[k].get(), L.nfEQ, L.cEQ, L.eq_center, L.eq_eps};
      GB_LAUNCH(eqnorm_bwd_kernel, nbk, nt, 0, e, T[L.tEQ].p, S.gmsg[k].get(), T[L.tGEQ].p, NC, na, a0);
    }
    run(E, L.dense.bwd, mu + a0, na, NC);
    GB_LAUNCH(spbf3_bwd_kernel, dim3(na, sh.slices), sh.threads, sh.smem_bwd, bonds, spbf(k), sht, T[L.tGA].p, NC, fv_.get(), vir_atom_.get(),
              sh.cshift, sh.nTI, a0);
  };
  for (int k = 0; k < 2; k++) S.msg[k].ensure((size_t) n * Q.L[k].nfEQ * Q.L[k].cEQ);
  for (int k = 0; k < 3; k++) {
    bind(k);
    for (int a0 = 0; a0 < n; a0 += NC) forward(k, a0, std::min(NC, n - a0), true);
  }
  const Readout3Dev ro{S.eW0.get(), S.eW1.get(), shift_.get(), Q.en0, Q.en1, plan_.out_scale, Q.e_nin, Q.e_nh, Q.e_act};
  GB_LAUNCH(readout3_kernel, nblk, nt, 0, ro, S.rho_sum.get(), mu, e_atom_.get(), S.drho.get(), energy_only ? 0 : 1, n);
  if (tm) tm->end(StageTimer::FWD);
  if (energy_only) {
    check_tc();
    return;
  }
  if (tm) tm->begin(StageTimer::BWD);
  // the reverse bond kernels add their shares (three layers, channel slices) to the bond forces and the virial
  launch_fill_zero(fv_.get(), sizeof(float) * 3 * (size_t) std::max<int64_t>(nl.nslots(), 1));
  launch_fill_zero(vir_atom_.get(), sizeof(double) * 6 * (size_t) n);
  for (int k = 0; k < 2; k++) {
    const Layer3Plan &L = Q.L[k];
    S.gmsg[k].ensure((size_t) n * L.nfEQ * L.cEQ);
    launch_fill_zero(S.gmsg[k].get(), sizeof(float) * (size_t) n * L.nfEQ * L.cEQ);
  }
  for (int k = 2; k >= 0; k--) {
    float *base = bind(k);
    for (int a0 = 0; a0 < n; a0 += NC) {
      const int na = std::min(NC, n - a0);
      if (!keep) forward(k, a0, na, false);    // the chunk's forward tensors again
      reverse(k, a0, na, base);
    }
  }
  if (tm) tm->end(StageTimer::BWD);
  check_tc();
}

}    // namespace gb
