// The dense per-atom network of a layer as ONE kernel: a CTA takes tiles of TA atoms and runs the whole operation
// list (FC, Clebsch-Gordan products, reduces, the fp64 readout, and all adjoints) on tensors that never leave shared
// memory.  Only the bond sums Q come in and their gradient gQ goes out (plus the message / rho rows of GRACE-2L), so
// the HBM traffic of the dense network is 2 x nlm x C floats per atom instead of every intermediate twice.
// Same operation tables as the per-chunk kernels (plan.h); same arithmetic (fp32 FMA, fp64 readout).
// Reference counterpart: the thread-private batch workspace of the CPU driver (libgrace/src/fused_1l.cpp:54-77,
// 260-372), which keeps the tensors of NB atoms in cache for the same reason.
#include "kernels.h"
#include "readout.cuh"

namespace gb {

namespace {

#ifndef GB_FUSED_THREADS
#define GB_FUSED_THREADS 512
#endif
constexpr int NTB = GB_FUSED_THREADS;    // threads of the CTA
#ifndef GB_FUSED_GROUPS
#define GB_FUSED_GROUPS 2
#endif
constexpr int NG = GB_FUSED_GROUPS;       // independent groups of warps, each on its own atom tile (this file is
                                          // compiled once more with one group of all warps: chain_fused_g1.cu)
constexpr int NT = NTB / NG;              // threads of a group

// barrier of the calling thread's group (named barrier 1 + group)
__device__ __forceinline__ void group_sync()
{
  asm volatile("bar.sync %0, %1;" ::"r"(1 + (int) threadIdx.x / NT), "r"(NT) : "memory");
}
__device__ __forceinline__ int gtid() { return (int) threadIdx.x % NT; }

// Matrix-major form of an operation with shared weights: a warp takes one unit = one weight matrix (32 of its output
// channels, lane = channel) and keeps that matrix column in registers, one 128-byte coalesced load per input channel,
// all in flight at once; it then applies it to the unit's few input rows for all TA atoms with the activations
// broadcast from shared memory.  A weight is fetched once per tile and unit instead of once per row, and the only
// global-memory latency is one round trip per unit.  Units of a slot write disjoint output rows; slots are separated
// by a CTA barrier (an output row gets its left and right terms in consecutive slots), so the sums are ordered and
// bit-reproducible.
template<int TA, int NMAX, bool EXACT>
__device__ __forceinline__ void mv_units(const MVDev &op, float *sm, const int *__restrict__ soff,
                                         const int *__restrict__ tch)
{
  const int warp = gtid() >> 5, lane = gtid() & 31, nwarp = NT / 32;
  // EXACT: every width of the operation (inputs, outputs, channel strides) equals NMAX, the usual case of equal
  // radial and FC channel counts: no bounds predicates, constant address strides
  const int Cd = EXACT ? NMAX : tch[op.dst];
  float *dst = sm + (size_t) soff[op.dst] * TA;
  for (int slot = 0; slot < op.nslots; slot++) {
    for (int u = op.slot_off[slot] + warp; u < op.slot_off[slot + 1]; u += nwarp) {
      const int *d = op.unit_desc + 5 * u;
      const int n_in = EXACT ? NMAX : d[1], k = d[2] + lane;
      const bool kv = EXACT || k < op.n_out;
      const float *M = op.W + d[0] + (kv ? k : 0);
      float w[NMAX];
#pragma unroll
      for (int n = 0; n < NMAX; n++) w[n] = (n < n_in && kv) ? __ldg(M + (size_t) n * op.ldw) : 0.0f;
      for (int e = d[3]; e < d[4]; e++) {
        const MVItem ent = op.unit_ent[e];
        const int Cs = EXACT ? NMAX : tch[ent.src];
        const float *x = sm + (size_t) soff[ent.src] * TA + (size_t) ent.irow * TA * Cs;
        float *o = dst + (size_t) ent.mat * TA * Cd + k;
        // TA independent sums, input channels outermost: the activation loads of all atoms for 4 channels are in
        // flight together and the FMA chains of the atoms interleave
        float sum[TA];
#pragma unroll
        for (int a = 0; a < TA; a++) sum[a] = 0.0f;
        if ((Cs & 3) == 0) {
#pragma unroll
          for (int n = 0; n < NMAX; n += 4) {
            if (n < n_in) {
              float4 x4[TA];
#pragma unroll
              for (int a = 0; a < TA; a++) x4[a] = *reinterpret_cast<const float4 *>(x + a * Cs + n);
#pragma unroll
              for (int a = 0; a < TA; a++) {
                sum[a] = fmaf(x4[a].x, w[n], sum[a]);
                sum[a] = fmaf(x4[a].y, w[n + 1], sum[a]);
                sum[a] = fmaf(x4[a].z, w[n + 2], sum[a]);
                sum[a] = fmaf(x4[a].w, w[n + 3], sum[a]);
              }
            }
          }
        } else {
#pragma unroll
          for (int n = 0; n < NMAX; n++) {
            if (n < n_in) {
#pragma unroll
              for (int a = 0; a < TA; a++) sum[a] = fmaf(x[a * Cs + n], w[n], sum[a]);
            }
          }
        }
        if (kv) {
#pragma unroll
          for (int a = 0; a < TA; a++)
            o[a * Cd] = (slot > 0 || op.accumulate) ? fmaf(ent.scale, sum[a], o[a * Cd]) : ent.scale * sum[a];
        }
      }
    }
    group_sync();
  }
}

// One (row, channel quad, atom) unit of an operation with per-element weights whose items all have PI x S input
// channels: lane s takes the channels s, s + S, ... of every item, and the weight loads of NE / PI items (every one an
// L2 round trip) are in flight together.
template<int TA, int PI>
__device__ __forceinline__ void elem_items(const MVDev &op, const float *sm, const int *__restrict__ soff,
                                           const int *__restrict__ tch, const float *Wa, int i0, int i1, int a, int s,
                                           int S, float4 &acc)
{
  constexpr int NE = 8, IB = NE / PI;
  const int ld = op.ldw;
  for (int it0 = i0; it0 < i1; it0 += IB) {
    float4 w[NE];
    float xv[NE];
#pragma unroll
    for (int jj = 0; jj < IB; jj++) {
      const bool in = it0 + jj < i1;
      const MVItem &item = op.items[in ? it0 + jj : i0];
      const float *x = sm + (size_t) soff[item.src] * TA + ((size_t) item.irow * TA + a) * tch[item.src];
      const float *M = Wa + item.mat;
#pragma unroll
      for (int q = 0; q < PI; q++) {
        const int n = s + S * q;
        w[jj * PI + q] = in ? __ldg(reinterpret_cast<const float4 *>(M + (size_t) n * ld)) : make_float4(0.f, 0.f, 0.f, 0.f);
        xv[jj * PI + q] = in ? x[n] * item.scale : 0.0f;
      }
    }
#pragma unroll
    for (int j = 0; j < NE; j++) {
      acc.x = fmaf(xv[j], w[j].x, acc.x); acc.y = fmaf(xv[j], w[j].y, acc.y);
      acc.z = fmaf(xv[j], w[j].z, acc.z); acc.w = fmaf(xv[j], w[j].w, acc.w);
    }
  }
}

// out[row][a][k] (+)= sum_items scale * sum_n M[n][k] x[item][a][n] on the tile's shared-memory tensors.
// A thread owns 4 consecutive output channels of one row for all TA atoms: a 16-byte weight load (rows of the weight
// matrices are padded to 4 outputs) feeds 4 TA FMAs, a 16-byte activation load (broadcast in the warp) 16.  The weight
// loads of a batch of input channels are issued before the first FMA needs one, because the L1 left beside the tile's
// shared memory is small and every load is an L2 round trip.  When an operation has fewer (row, channel quad) pairs
// than the CTA has threads, S lanes share the items of a pair and add their partial sums by shuffles.
template<int TA>
__device__ __forceinline__ void mv_tile(const MVDev &op, float *sm, const int *__restrict__ soff,
                                        const int *__restrict__ tch, const int *s_mu)
{
  const int tid = gtid();
  const int Cd = tch[op.dst], ld = op.ldw;
  float *dst = sm + (size_t) soff[op.dst] * TA;
  const int KQ = ld >> 2;
  int KQP = 1;
  while (KQP < KQ) KQP <<= 1;
  if (op.elem) {
    // weights of each atom's own element: nothing is shared between the atoms of the tile, so the unit of work is
    // (row, channel quad, atom) and S lanes split the (item, input channel) pairs of the row.  Every weight is an L2
    // round trip (the matrices of one element exceed the L1 left beside the tile), so the pairs of ALL items are one
    // flat index space and NE independent 16-byte weight loads are in flight per lane before the first FMA.
    const int total_e = op.nrows * KQ * TA;
    int S = 1;
    while (S < 32 && total_e * S * 2 <= NT) S <<= 1;
    const int s = tid & (S - 1), per_pass = NT / S;
    for (int base = 0; base < total_e; base += per_pass) {
      const int u = base + tid / S, a = u % TA, rk = u / TA, row = rk / KQ, kq = rk - row * KQ;
      const bool valid = u < total_e;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      if (valid) {
        const float *Wa = op.W + (size_t) s_mu[a] * op.ty_stride + 4 * kq;
        const int i0 = op.item_off[row], i1 = op.item_off[row + 1];
        constexpr int NE = 8;
        const int per_item = op.n_uniform > 0 && op.n_uniform % S == 0 ? op.n_uniform / S : 0;
        if (per_item == 1) elem_items<TA, 1>(op, sm, soff, tch, Wa, i0, i1, a, s, S, acc);
        else if (per_item == 2) elem_items<TA, 2>(op, sm, soff, tch, Wa, i0, i1, a, s, S, acc);
        else if (per_item == 4) elem_items<TA, 4>(op, sm, soff, tch, Wa, i0, i1, a, s, S, acc);
        else {
          for (int it = i0; it < i1; it++) {
            const MVItem item = op.items[it];
            const int Cs = tch[item.src];
            const float *x = sm + (size_t) soff[item.src] * TA + ((size_t) item.irow * TA + a) * Cs;
            const float *M = Wa + item.mat;
            for (int n0 = s; n0 < item.n_in; n0 += NE * S) {
              float4 w[NE];
              float xv[NE];
#pragma unroll
              for (int j = 0; j < NE; j++) {
                const int n = n0 + j * S;
                const bool in = n < item.n_in;
                w[j] = in ? __ldg(reinterpret_cast<const float4 *>(M + (size_t) n * ld)) : make_float4(0.f, 0.f, 0.f, 0.f);
                xv[j] = in ? x[n] * item.scale : 0.0f;
              }
#pragma unroll
              for (int j = 0; j < NE; j++) {
                acc.x = fmaf(xv[j], w[j].x, acc.x); acc.y = fmaf(xv[j], w[j].y, acc.y);
                acc.z = fmaf(xv[j], w[j].z, acc.z); acc.w = fmaf(xv[j], w[j].w, acc.w);
              }
            }
          }
        }
      }
      for (int d = S >> 1; d > 0; d >>= 1) {
        acc.x += __shfl_xor_sync(0xffffffffu, acc.x, d); acc.y += __shfl_xor_sync(0xffffffffu, acc.y, d);
        acc.z += __shfl_xor_sync(0xffffffffu, acc.z, d); acc.w += __shfl_xor_sync(0xffffffffu, acc.w, d);
      }
      if (!valid || s != 0) continue;
      float *o = dst + ((size_t) op.row_out[row] * TA + a) * Cd + 4 * kq;
      const float v[4] = {acc.x, acc.y, acc.z, acc.w};
      const int nk = min(4, op.n_out - 4 * kq);
      for (int q = 0; q < nk; q++) o[q] = op.accumulate ? o[q] + v[q] : v[q];
    }
    return;
  }
  const int total = op.nrows * KQP;
  int S = 1;
  while (S < 32 && total * S * 2 <= NT) S <<= 1;
  const int s = tid & (S - 1), per_pass = NT / S;
  for (int base = 0; base < total; base += per_pass) {
    const int rk = base + tid / S, row = rk / KQP, kq = rk - row * KQP;
    const bool valid = rk < total && kq < KQ;
    float4 acc[TA];
#pragma unroll
    for (int a = 0; a < TA; a++) acc[a] = make_float4(0.f, 0.f, 0.f, 0.f);
    const int i0 = valid ? op.item_off[row] + s : 0, i1 = valid ? op.item_off[row + 1] : 0;
    for (int it = i0; it < i1; it += S) {
      const MVItem item = op.items[it];
      const int Cs = tch[item.src];
      const float *x = sm + (size_t) soff[item.src] * TA + (size_t) item.irow * TA * Cs;
      const float *M = op.W + item.mat + 4 * kq;
      const float sc = item.scale;
      if (((item.n_in | Cs) & 3) == 0) {
        constexpr int NB = 16;
        for (int n0 = 0; n0 < item.n_in; n0 += NB) {
          float4 w[NB];
#pragma unroll
          for (int j = 0; j < NB; j++)
            w[j] = (n0 + j < item.n_in) ? __ldg(reinterpret_cast<const float4 *>(M + (size_t) (n0 + j) * ld))
                                        : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int j = 0; j < NB; j += 4) {
            if (n0 + j < item.n_in) {
#pragma unroll
              for (int a = 0; a < TA; a++) {
                float4 x4 = *reinterpret_cast<const float4 *>(x + a * Cs + n0 + j);
                x4.x *= sc; x4.y *= sc; x4.z *= sc; x4.w *= sc;
                acc[a].x = fmaf(x4.x, w[j].x, acc[a].x); acc[a].y = fmaf(x4.x, w[j].y, acc[a].y);
                acc[a].z = fmaf(x4.x, w[j].z, acc[a].z); acc[a].w = fmaf(x4.x, w[j].w, acc[a].w);
                acc[a].x = fmaf(x4.y, w[j + 1].x, acc[a].x); acc[a].y = fmaf(x4.y, w[j + 1].y, acc[a].y);
                acc[a].z = fmaf(x4.y, w[j + 1].z, acc[a].z); acc[a].w = fmaf(x4.y, w[j + 1].w, acc[a].w);
                acc[a].x = fmaf(x4.z, w[j + 2].x, acc[a].x); acc[a].y = fmaf(x4.z, w[j + 2].y, acc[a].y);
                acc[a].z = fmaf(x4.z, w[j + 2].z, acc[a].z); acc[a].w = fmaf(x4.z, w[j + 2].w, acc[a].w);
                acc[a].x = fmaf(x4.w, w[j + 3].x, acc[a].x); acc[a].y = fmaf(x4.w, w[j + 3].y, acc[a].y);
                acc[a].z = fmaf(x4.w, w[j + 3].z, acc[a].z); acc[a].w = fmaf(x4.w, w[j + 3].w, acc[a].w);
              }
            }
          }
        }
      } else {    // input widths that are no multiples of 4: scalar activation loads
        constexpr int NB = 8;
        for (int n0 = 0; n0 < item.n_in; n0 += NB) {
          float4 w[NB];
#pragma unroll
          for (int j = 0; j < NB; j++)
            w[j] = (n0 + j < item.n_in) ? __ldg(reinterpret_cast<const float4 *>(M + (size_t) (n0 + j) * ld))
                                        : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int j = 0; j < NB; j++) {
            if (n0 + j < item.n_in) {
#pragma unroll
              for (int a = 0; a < TA; a++) {
                const float xv = x[a * Cs + n0 + j] * sc;
                acc[a].x = fmaf(xv, w[j].x, acc[a].x); acc[a].y = fmaf(xv, w[j].y, acc[a].y);
                acc[a].z = fmaf(xv, w[j].z, acc[a].z); acc[a].w = fmaf(xv, w[j].w, acc[a].w);
              }
            }
          }
        }
      }
    }
    for (int d = S >> 1; d > 0; d >>= 1) {
#pragma unroll
      for (int a = 0; a < TA; a++) {
        acc[a].x += __shfl_xor_sync(0xffffffffu, acc[a].x, d); acc[a].y += __shfl_xor_sync(0xffffffffu, acc[a].y, d);
        acc[a].z += __shfl_xor_sync(0xffffffffu, acc[a].z, d); acc[a].w += __shfl_xor_sync(0xffffffffu, acc[a].w, d);
      }
    }
    if (!valid || s != 0) continue;
    float *o = dst + (size_t) op.row_out[row] * TA * Cd + 4 * kq;
    if (((Cd | op.n_out) & 3) == 0) {
#pragma unroll
      for (int a = 0; a < TA; a++) {
        float4 *p = reinterpret_cast<float4 *>(o + a * Cd);
        if (op.accumulate) {
          const float4 old = *p;
          acc[a].x += old.x; acc[a].y += old.y; acc[a].z += old.z; acc[a].w += old.w;
        }
        *p = acc[a];
      }
    } else {
      const int nk = min(4, op.n_out - 4 * kq);
#pragma unroll
      for (int a = 0; a < TA; a++) {
        const float v[4] = {acc[a].x, acc[a].y, acc[a].z, acc[a].w};
        for (int q = 0; q < nk; q++) o[a * Cd + q] = op.accumulate ? o[a * Cd + q] + v[q] : v[q];
      }
    }
  }
}

template<int TA>
__device__ __forceinline__ void mv_any(const MVDev &op, float *sm, const int *__restrict__ soff,
                                       const int *__restrict__ tch, const int *s_mu)
{
  if (op.nslots > 0) {
    if (op.unit_exact == 32) mv_units<TA, 32, true>(op, sm, soff, tch);
    else if (op.unit_exact == 64) mv_units<TA, 64, true>(op, sm, soff, tch);
    else if (op.unit_nmax <= 32) mv_units<TA, 32, false>(op, sm, soff, tch);
    else mv_units<TA, 64, false>(op, sm, soff, tch);
  } else {
    mv_tile<TA>(op, sm, soff, tch, s_mu);
  }
}

// out[row][i] (+)= sum_terms coef A[a][i] B[b][i] over the TA * C values of a row, four channels per thread
template<int TA>
__device__ __forceinline__ void prod_tile(const ProdDev &op, float *sm, const int *__restrict__ soff,
                                          const int *__restrict__ tch)
{
  const int TAC = TA * tch[op.dst];
  const float *A = sm + (size_t) soff[op.srcA] * TA;
  const float *B = op.srcB >= 0 ? sm + (size_t) soff[op.srcB] * TA : nullptr;
  float *D = sm + (size_t) soff[op.dst] * TA;
  if ((tch[op.dst] & 3) == 0) {
    const int Q = TAC >> 2, total = op.nrows * Q;
    for (int idx = gtid(); idx < total; idx += NT) {
      const int row = idx / Q, i = (idx - row * Q) * 4;
      const int t0 = op.term_off[row], t1 = op.term_off[row + 1];
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int t = t0; t < t1; t++) {
        const ProdTerm tm = op.terms[t];
        const float4 av = *reinterpret_cast<const float4 *>(A + tm.a * TAC + i);
        if (B) {
          const float4 bv = *reinterpret_cast<const float4 *>(B + tm.b * TAC + i);
          acc.x = fmaf(tm.coef * av.x, bv.x, acc.x); acc.y = fmaf(tm.coef * av.y, bv.y, acc.y);
          acc.z = fmaf(tm.coef * av.z, bv.z, acc.z); acc.w = fmaf(tm.coef * av.w, bv.w, acc.w);
        } else {
          acc.x = fmaf(tm.coef, av.x, acc.x); acc.y = fmaf(tm.coef, av.y, acc.y);
          acc.z = fmaf(tm.coef, av.z, acc.z); acc.w = fmaf(tm.coef, av.w, acc.w);
        }
      }
      float4 *o = reinterpret_cast<float4 *>(D + op.row_out[row] * TAC + i);
      if (op.accumulate) {
        const float4 old = *o;
        acc.x += old.x; acc.y += old.y; acc.z += old.z; acc.w += old.w;
      }
      *o = acc;
    }
    return;
  }
  const int total = op.nrows * TAC;
  for (int idx = gtid(); idx < total; idx += NT) {
    const int row = idx / TAC, i = idx - row * TAC;
    const int t0 = op.term_off[row], t1 = op.term_off[row + 1];
    float acc = 0.0f;
    for (int t = t0; t < t1; t++) {
      const ProdTerm tm = op.terms[t];
      acc = fmaf(tm.coef * A[tm.a * TAC + i], B ? B[tm.b * TAC + i] : 1.0f, acc);
    }
    float *o = D + op.row_out[row] * TAC + i;
    *o = op.accumulate ? *o + acc : acc;
  }
}

// The forward tensors a later reverse pass reads (L.save: shared-memory offset, functions, channels and offset in the
// per-atom record of each) to or from global memory, [position of the atom in the evaluation][save_floats]; a tensor
// is [f][TA][C] in shared memory and [f][C] in the record.
template<int TA, bool SAVE>
__device__ __forceinline__ void move_saved(const FusedLayerDev &L, const FusedIO &io, float *sm, int al0, int nta, int tid)
{
  for (int z = 0; z < L.nsave; z++) {
    const int4 sv = L.save[z];
    float *t = sm + (size_t) sv.x * TA;
    const int nf = sv.y, C = sv.z;
    float *g0 = io.saved + (size_t) (io.a0 + al0) * L.save_floats + sv.w;
    if ((C & 3) == 0 && (L.save_floats & 3) == 0 && (sv.w & 3) == 0) {
      const int C4 = C >> 2, total = nf * nta * C4;
      for (int idx = tid; idx < total; idx += NT) {
        const int c = idx % C4, fa = idx / C4, a = fa % nta, f = fa / nta;
        float4 *g = reinterpret_cast<float4 *>(g0 + (size_t) a * L.save_floats + f * C) + c;
        float4 *p = reinterpret_cast<float4 *>(t + (size_t) (f * TA + a) * C) + c;
        if (SAVE) *g = *p;
        else *p = *g;
      }
    } else {
      const int total = nf * nta * C;
      for (int idx = tid; idx < total; idx += NT) {
        const int c = idx % C, fa = idx / C, a = fa % nta, f = fa / nta;
        float *g = g0 + (size_t) a * L.save_floats + f * C + c;
        float *p = t + (size_t) (f * TA + a) * C + c;
        if (SAVE) *g = *p;
        else *p = *g;
      }
    }
  }
}

template<int TA>
__global__ void __launch_bounds__(NTB) chain_fused_kernel(FusedLayerDev L, FusedIO io)
{
  GB_DYN_SMEM(float4, smem4);
  __shared__ int s_mu_all[NG][TA], s_at_all[NG][TA];
  const int btid = threadIdx.x, grp = btid / NT, tid = btid % NT;
  int *s_mu = s_mu_all[grp], *s_at = s_at_all[grp];    // element and list index of the tile's atoms
  const int ntiles = (io.na + TA - 1) / TA;
  // tables first, the tile's tensors behind them
  char *tp = reinterpret_cast<char *>(smem4);
  MVDev *s_mv = reinterpret_cast<MVDev *>(tp);            tp += sizeof(MVDev) * L.nmv;
  ProdDev *s_prod = reinterpret_cast<ProdDev *>(tp);      tp += sizeof(ProdDev) * L.nprod;
  int2 *s_ops = reinterpret_cast<int2 *>(tp);             tp += sizeof(int2) * (L.nfwd + L.nbwd);
  int2 *s_zero = reinterpret_cast<int2 *>(tp);            tp += sizeof(int2) * L.nzero;
  int *s_soff = reinterpret_cast<int *>(tp);              tp += sizeof(int) * L.ntensors;
  int *s_tch = reinterpret_cast<int *>(tp);               tp += sizeof(int) * L.ntensors;
  int *s_itab = reinterpret_cast<int *>(tp);              tp += sizeof(int) * L.n_itab;
  MVItem *s_items = reinterpret_cast<MVItem *>(tp);       tp += sizeof(MVItem) * L.n_items;
  ProdTerm *s_terms = reinterpret_cast<ProdTerm *>(tp);
  float *sm = reinterpret_cast<float *>(smem4) + L.tab_floats + (size_t) grp * L.per_atom * TA;
  for (int q = btid; q < L.nmv; q += NTB) {
    MVDev d = L.mv[q];
    d.row_out = s_itab + (d.row_out - L.itab);
    d.item_off = s_itab + (d.item_off - L.itab);
    d.items = s_items + (d.items - L.items);
    d.unit_desc = s_itab + (d.unit_desc - L.itab);
    d.slot_off = s_itab + (d.slot_off - L.itab);
    d.unit_ent = s_items + (d.unit_ent - L.items);
    s_mv[q] = d;
  }
  for (int q = btid; q < L.nprod; q += NTB) {
    ProdDev d = L.prod[q];
    d.row_out = s_itab + (d.row_out - L.itab);
    d.term_off = s_itab + (d.term_off - L.itab);
    if (L.stage_terms) d.terms = s_terms + (d.terms - L.terms);
    s_prod[q] = d;
  }
  for (int q = btid; q < L.nfwd + L.nbwd; q += NTB) s_ops[q] = L.ops[q];
  for (int q = btid; q < L.nzero; q += NTB) s_zero[q] = L.zero[q];
  for (int q = btid; q < L.ntensors; q += NTB) { s_soff[q] = L.soff[q]; s_tch[q] = L.tch[q]; }
  for (int q = btid; q < L.n_itab; q += NTB) s_itab[q] = L.itab[q];
  for (int q = btid; q < L.n_items; q += NTB) s_items[q] = L.items[q];
  if (L.stage_terms)
    for (int q = btid; q < L.n_terms; q += NTB) s_terms[q] = L.terms[q];
  ReadoutDev ro = io.ro;
  if (L.stage_ro > 0) {    // the energy MLP and its transpose, read row by row by the warp readout
    double *s_ro = reinterpret_cast<double *>(reinterpret_cast<char *>(smem4) + L.ro_offset);
    for (int q = btid; q < L.stage_ro; q += NTB) {
      s_ro[q] = io.ro.W[q];
      s_ro[L.stage_ro + q] = io.ro.WT[q];
    }
    ro.W = s_ro;
    ro.WT = s_ro + L.stage_ro;
  }
  __syncthreads();
  for (int tile = blockIdx.x * NG + grp; tile < ntiles; tile += gridDim.x * NG) {
    const int al0 = tile * TA;                      // first atom of the tile, chunk-local
    const int nta = min(TA, io.na - al0);
    if (tid < TA) {
      const int q = io.a0 + al0 + min(tid, nta - 1), i = io.ilist ? io.ilist[q] : q;
      s_at[tid] = i;
      s_mu[tid] = io.mu[i];
    }
    if (io.mode & FUSED_RESTORE) {    // forward tensors kept by an earlier FUSED_SAVE launch instead of a second evaluation
      move_saved<TA, false>(L, io, sm, al0, nta, tid);
      group_sync();
    } else {
      {    // bond sums of the tile: global [f][NA][C] -> shared [f][TA][C]; atoms past the end are zero
        const int C = io.CQ;
        float *q = sm + (size_t) s_soff[io.tQ] * TA;
        if ((C & 3) == 0) {
          const int C4 = C >> 2, total = io.nQ * TA * C4;
          for (int idx = tid; idx < total; idx += NT) {
            const int c = idx % C4, a = (idx / C4) % TA, f = idx / (C4 * TA);
            reinterpret_cast<float4 *>(q)[idx] =
                a < nta ? __ldg(reinterpret_cast<const float4 *>(io.Q + ((size_t) f * io.NA + al0 + a) * C) + c)
                        : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        } else {
          const int total = io.nQ * TA * C;
          for (int idx = tid; idx < total; idx += NT) {
            const int c = idx % C, a = (idx / C) % TA, f = idx / (C * TA);
            q[idx] = a < nta ? __ldg(io.Q + ((size_t) f * io.NA + al0 + a) * C + c) : 0.0f;
          }
        }
      }
      group_sync();
      for (int o = 0; o < L.nfwd; o++) {
        const int2 op = s_ops[o];
        if (op.x == 0) mv_any<TA>(s_mv[op.y], sm, s_soff, s_tch, s_mu);
        else prod_tile<TA>(s_prod[op.y], sm, s_soff, s_tch);
        group_sync();
      }
    }
    if (io.mode & FUSED_SAVE) move_saved<TA, true>(L, io, sm, al0, nta, tid);
    if (io.mode & FUSED_STORE_MSG) {    // GRACE-2L layer 1: message rows [n][nI][CR] and rho rows [n][nrho]
      const int CR = io.CR, nI = io.nI, total = nta * nI * CR;
      const float *I = sm + (size_t) s_soff[io.t_I] * TA;
      for (int idx = tid; idx < total; idx += NT) {
        const int c = idx % CR, f = (idx / CR) % nI, a = idx / (CR * nI);
        io.I_rows[((size_t) s_at[a] * nI + f) * CR + c] = I[(f * TA + a) * CR + c];
      }
      const float *rho = sm + (size_t) s_soff[io.t_rho] * TA;
      for (int idx = tid; idx < nta * io.nrho; idx += NT)
        io.rho_rows[(size_t) s_at[idx / io.nrho] * io.nrho + idx % io.nrho] = rho[idx];
    }
    const bool bwd = io.mode & FUSED_BWD;
    if (bwd) {    // gradients start at zero; those that alias forward tensors take their storage over now
      for (int z = 0; z < L.nzero; z++) {
        const int2 zr = s_zero[z];
        float4 *p = reinterpret_cast<float4 *>(sm + (size_t) zr.x * TA);
        for (int idx = tid; idx < zr.y * TA / 4; idx += NT) p[idx] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    if (io.mode & FUSED_READOUT_1L) {    // one warp per atom
      const int w = tid >> 5, ln = tid & 31;
      if (w < nta) {
        const float *rho = sm + (size_t) s_soff[io.t_rho] * TA + w * io.nrho;
        float *grho = sm + (size_t) s_soff[io.t_grho] * TA + w * io.nrho;
        const size_t i = s_at[w];
        const double e = readout_1l_warp(ro, rho, s_mu[w], grho, bwd, ro.owned(i));
        if (ln == 0) io.e_atom[i] = e;
      } else if (w < TA && bwd) {
        float *grho = sm + (size_t) s_soff[io.t_grho] * TA + w * io.nrho;
        for (int k = ln; k < io.nrho; k += 32) grho[k] = 0.0f;
      }
    }
    if (io.mode & FUSED_READOUT_2L) {
      const int w = tid >> 5, ln = tid & 31;
      if (w < nta) {
        const size_t i = s_at[w];
        const float *I2 = sm + (size_t) s_soff[io.t_I2] * TA + w * io.nrho;
        float *gI2 = sm + (size_t) s_soff[io.t_gI2] * TA + w * io.nrho;
        const double e = readout_2l_warp(ro, io.rho_rows + i * io.nrho, I2, s_mu[w], io.grho_rows + i * io.nrho, gI2,
                                         bwd, ro.owned(i));
        if (ln == 0) io.e_atom[i] = e;
      } else if (w < TA && bwd) {
        float *gI2 = sm + (size_t) s_soff[io.t_gI2] * TA + w * io.nrho;
        for (int k = ln; k < io.nrho; k += 32) gI2[k] = 0.0f;
      }
    }
    if (io.mode & FUSED_LOAD_SEED) {    // GRACE-2L layer 1 reverse: dE/dI and dE/drho of each atom
      const int CR = io.CR, nI = io.nI, total = TA * nI * CR;
      float *gI = sm + (size_t) s_soff[io.t_gI] * TA;
      for (int idx = tid; idx < total; idx += NT) {
        const int c = idx % CR, a = (idx / CR) % TA, f = idx / (CR * TA);
        gI[idx] = a < nta ? io.gI_rows[((size_t) s_at[a] * nI + f) * CR + c] : 0.0f;
      }
      float *grho = sm + (size_t) s_soff[io.t_grho] * TA;
      for (int idx = tid; idx < TA * io.nrho; idx += NT)
        grho[idx] = idx < nta * io.nrho ? (float) io.grho_rows[(size_t) s_at[idx / io.nrho] * io.nrho + idx % io.nrho] : 0.0f;
    }
    group_sync();
    if (bwd) {
      for (int o = L.nfwd; o < L.nfwd + L.nbwd; o++) {
        const int2 op = s_ops[o];
        if (op.x == 0) mv_any<TA>(s_mv[op.y], sm, s_soff, s_tch, s_mu);
        else prod_tile<TA>(s_prod[op.y], sm, s_soff, s_tch);
        group_sync();
      }
      const int C = io.CQ;
      const float *g = sm + (size_t) s_soff[io.tGQ] * TA;
      if ((C & 3) == 0) {
        const int C4 = C >> 2, total = io.nQ * TA * C4;
        for (int idx = tid; idx < total; idx += NT) {
          const int c = idx % C4, a = (idx / C4) % TA, f = idx / (C4 * TA);
          if (a < nta)
            reinterpret_cast<float4 *>(io.gQ + ((size_t) f * io.NA + al0 + a) * C)[c] = reinterpret_cast<const float4 *>(g)[idx];
        }
      } else {
        const int total = io.nQ * TA * C;
        for (int idx = tid; idx < total; idx += NT) {
          const int c = idx % C, a = (idx / C) % TA, f = idx / (C * TA);
          if (a < nta) io.gQ[((size_t) f * io.NA + al0 + a) * C + c] = g[idx];
        }
      }
      group_sync();
    }
  }
}

template<int TA> void launch_ta(const FusedLayerDev &L, const FusedIO &io, int grid, size_t smem)
{
  static size_t attr_smem = 48 * 1024;    // dynamic shared memory this instantiation may use so far
  if (smem > attr_smem) {
    GB_CUDA(cudaFuncSetAttribute(chain_fused_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    attr_smem = smem;
  }
  GB_LAUNCH((chain_fused_kernel<TA>), grid, NTB, smem, L, io);
}

}    // namespace

#if GB_FUSED_GROUPS == 2
void launch_chain_fused(int TA, const FusedLayerDev &L, const FusedIO &io, int grid)
#else
void launch_chain_fused_g1(int TA, const FusedLayerDev &L, const FusedIO &io, int grid)
#endif
{
  if (io.na == 0) return;
  const size_t smem = ((size_t) L.tab_floats + (size_t) L.per_atom * TA * NG) * sizeof(float);
  switch (TA) {
    case 1: launch_ta<1>(L, io, grid, smem); break;
    case 2: launch_ta<2>(L, io, grid, smem); break;
    case 3: launch_ta<3>(L, io, grid, smem); break;
    case 4: launch_ta<4>(L, io, grid, smem); break;
    case 5: launch_ta<5>(L, io, grid, smem); break;
    case 6: launch_ta<6>(L, io, grid, smem); break;
    case 8: launch_ta<8>(L, io, grid, smem); break;
    default: throw DeviceError("fused dense network: unsupported atom tile");
  }
}

}    // namespace gb
