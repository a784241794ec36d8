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

constexpr int NT = 256;

template<int TA>
__device__ __forceinline__ void mv_tile(const MVDev &op, float *sm, const int *__restrict__ soff,
                                        const int *__restrict__ tch, const int *s_mu)
{
  int KP = 8;
  while (KP < op.n_out) KP <<= 1;
  const int tid = threadIdx.x, k = tid & (KP - 1), rstep = NT / KP;
  const int Cd = tch[op.dst];
  float *dst = sm + (size_t) soff[op.dst] * TA;
  if (k >= op.n_out) return;
  for (int row = tid / KP; row < op.nrows; row += rstep) {
    float acc[TA];
#pragma unroll
    for (int a = 0; a < TA; a++) acc[a] = 0.0f;
    const int i0 = op.item_off[row], i1 = op.item_off[row + 1];
    for (int it = i0; it < i1; it++) {
      const MVItem item = op.items[it];
      const int Cs = tch[item.src];
      const float *x = sm + (size_t) soff[item.src] * TA + (size_t) item.irow * TA * Cs;
      float part[TA];
#pragma unroll
      for (int a = 0; a < TA; a++) part[a] = 0.0f;
      if (!op.elem) {
        const float *M = op.W + item.mat + k;
        if (((item.n_in | Cs) & 3) == 0) {
          for (int n = 0; n < item.n_in; n += 4) {
            const float w0 = __ldg(M + (size_t) n * op.n_out), w1 = __ldg(M + (size_t) (n + 1) * op.n_out);
            const float w2 = __ldg(M + (size_t) (n + 2) * op.n_out), w3 = __ldg(M + (size_t) (n + 3) * op.n_out);
#pragma unroll
            for (int a = 0; a < TA; a++) {
              const float4 x4 = *reinterpret_cast<const float4 *>(x + a * Cs + n);
              part[a] = fmaf(x4.x, w0, part[a]);
              part[a] = fmaf(x4.y, w1, part[a]);
              part[a] = fmaf(x4.z, w2, part[a]);
              part[a] = fmaf(x4.w, w3, part[a]);
            }
          }
        } else {
          for (int n = 0; n < item.n_in; n++) {
            const float w = __ldg(M + (size_t) n * op.n_out);
#pragma unroll
            for (int a = 0; a < TA; a++) part[a] = fmaf(x[a * Cs + n], w, part[a]);
          }
        }
      } else {
        const float *M[TA];
#pragma unroll
        for (int a = 0; a < TA; a++) M[a] = op.W + (size_t) s_mu[a] * op.ty_stride + item.mat + k;
        for (int n = 0; n < item.n_in; n++) {
#pragma unroll
          for (int a = 0; a < TA; a++) part[a] = fmaf(x[a * Cs + n], __ldg(M[a] + (size_t) n * op.n_out), part[a]);
        }
      }
#pragma unroll
      for (int a = 0; a < TA; a++) acc[a] = fmaf(item.scale, part[a], acc[a]);
    }
    float *o = dst + (size_t) op.row_out[row] * TA * Cd + k;
#pragma unroll
    for (int a = 0; a < TA; a++) o[a * Cd] = op.accumulate ? o[a * Cd] + acc[a] : acc[a];
  }
}

template<int TA>
__device__ __forceinline__ void prod_tile(const ProdDev &op, float *sm, const int *__restrict__ soff,
                                          const int *__restrict__ tch)
{
  const int TAC = TA * tch[op.dst];
  const float *A = sm + (size_t) soff[op.srcA] * TA;
  const float *B = op.srcB >= 0 ? sm + (size_t) soff[op.srcB] * TA : nullptr;
  float *D = sm + (size_t) soff[op.dst] * TA;
  const int total = op.nrows * TAC;
  for (int idx = threadIdx.x; idx < total; idx += NT) {
    const int row = idx / TAC, i = idx - row * TAC;
    const int t0 = op.term_off[row], t1 = op.term_off[row + 1];
    float acc = 0.0f;
    if (B) {
      for (int t = t0; t < t1; t++) {
        const ProdTerm tm = op.terms[t];
        acc = fmaf(tm.coef * A[tm.a * TAC + i], B[tm.b * TAC + i], acc);
      }
    } else {
      for (int t = t0; t < t1; t++) {
        const ProdTerm tm = op.terms[t];
        acc = fmaf(tm.coef, A[tm.a * TAC + i], acc);
      }
    }
    float *o = D + op.row_out[row] * TAC + i;
    *o = op.accumulate ? *o + acc : acc;
  }
}

template<int TA>
__global__ void __launch_bounds__(NT) chain_fused_kernel(FusedLayerDev L, FusedIO io)
{
  GB_DYN_SMEM(float4, smem4);
  float *sm = reinterpret_cast<float *>(smem4);
  __shared__ int s_mu[TA];
  const int tid = threadIdx.x;
  const int ntiles = (io.na + TA - 1) / TA;
  for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const int al0 = tile * TA;                      // first atom of the tile, chunk-local
    const int nta = min(TA, io.na - al0);
    if (tid < TA) s_mu[tid] = io.mu[io.a0 + al0 + min(tid, nta - 1)];
    {    // bond sums of the tile: global [f][NA][C] -> shared [f][TA][C]; atoms past the end are zero
      const int C = io.CQ, total = io.nQ * TA * C;
      float *q = sm + (size_t) L.soff[io.tQ] * TA;
      for (int idx = tid; idx < total; idx += NT) {
        const int c = idx % C, a = (idx / C) % TA, f = idx / (C * TA);
        q[idx] = a < nta ? __ldg(io.Q + ((size_t) f * io.NA + al0 + a) * C + c) : 0.0f;
      }
    }
    __syncthreads();
    for (int o = 0; o < L.nfwd; o++) {
      const int2 op = L.ops[o];
      if (op.x == 0) mv_tile<TA>(L.mv[op.y], sm, L.soff, L.tch, s_mu);
      else prod_tile<TA>(L.prod[op.y], sm, L.soff, L.tch);
      __syncthreads();
    }
    if (io.mode & FUSED_STORE_MSG) {    // GRACE-2L layer 1: message rows [n][nI][CR] and rho rows [n][nrho]
      const int CR = io.CR, nI = io.nI, total = nta * nI * CR;
      const float *I = sm + (size_t) L.soff[io.t_I] * TA;
      for (int idx = tid; idx < total; idx += NT) {
        const int c = idx % CR, f = (idx / CR) % nI, a = idx / (CR * nI);
        io.I_rows[((size_t) (io.a0 + al0 + a) * nI + f) * CR + c] = I[(f * TA + a) * CR + c];
      }
      const float *rho = sm + (size_t) L.soff[io.t_rho] * TA;
      for (int idx = tid; idx < nta * io.nrho; idx += NT)
        io.rho_rows[(size_t) (io.a0 + al0) * io.nrho + idx] = rho[idx];
    }
    const bool bwd = io.mode & FUSED_BWD;
    if (bwd) {    // gradients start at zero; those that alias forward tensors take their storage over now
      for (int z = 0; z < L.nzero; z++) {
        const int2 zr = L.zero[z];
        float4 *p = reinterpret_cast<float4 *>(sm + (size_t) zr.x * TA);
        for (int idx = tid; idx < zr.y * TA / 4; idx += NT) p[idx] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    if (io.mode & FUSED_READOUT_1L) {
      if (tid < nta) {
        const float *rho = sm + (size_t) L.soff[io.t_rho] * TA + tid * io.nrho;
        float *grho = sm + (size_t) L.soff[io.t_grho] * TA + tid * io.nrho;
        io.e_atom[io.a0 + al0 + tid] = readout_1l_atom(io.ro, rho, s_mu[tid], grho, bwd);
      } else if (tid < TA && bwd) {
        float *grho = sm + (size_t) L.soff[io.t_grho] * TA + tid * io.nrho;
        for (int k = 0; k < io.nrho; k++) grho[k] = 0.0f;
      }
    }
    if (io.mode & FUSED_READOUT_2L) {
      if (tid < nta) {
        const size_t i = io.a0 + al0 + tid;
        const float *I2 = sm + (size_t) L.soff[io.t_I2] * TA + tid * io.nrho;
        float *gI2 = sm + (size_t) L.soff[io.t_gI2] * TA + tid * io.nrho;
        io.e_atom[i] = readout_2l_atom(io.ro, io.rho_rows + i * io.nrho, I2, s_mu[tid], io.grho_rows + i * io.nrho,
                                       gI2, bwd);
      } else if (tid < TA && bwd) {
        float *gI2 = sm + (size_t) L.soff[io.t_gI2] * TA + tid * io.nrho;
        for (int k = 0; k < io.nrho; k++) gI2[k] = 0.0f;
      }
    }
    if (io.mode & FUSED_LOAD_SEED) {    // GRACE-2L layer 1 reverse: dE/dI and dE/drho of each atom
      const int CR = io.CR, nI = io.nI, total = TA * nI * CR;
      float *gI = sm + (size_t) L.soff[io.t_gI] * TA;
      for (int idx = tid; idx < total; idx += NT) {
        const int c = idx % CR, a = (idx / CR) % TA, f = idx / (CR * TA);
        gI[idx] = a < nta ? io.gI_rows[((size_t) (io.a0 + al0 + a) * nI + f) * CR + c] : 0.0f;
      }
      float *grho = sm + (size_t) L.soff[io.t_grho] * TA;
      for (int idx = tid; idx < TA * io.nrho; idx += NT)
        grho[idx] = idx < nta * io.nrho ? (float) io.grho_rows[(size_t) (io.a0 + al0) * io.nrho + idx] : 0.0f;
    }
    __syncthreads();
    if (bwd) {
      for (int o = L.nfwd; o < L.nfwd + L.nbwd; o++) {
        const int2 op = L.ops[o];
        if (op.x == 0) mv_tile<TA>(L.mv[op.y], sm, L.soff, L.tch, s_mu);
        else prod_tile<TA>(L.prod[op.y], sm, L.soff, L.tch);
        __syncthreads();
      }
      const int C = io.CQ, total = io.nQ * TA * C;
      const float *g = sm + (size_t) L.soff[io.tGQ] * TA;
      for (int idx = tid; idx < total; idx += NT) {
        const int c = idx % C, a = (idx / C) % TA, f = idx / (C * TA);
        if (a < nta) io.gQ[((size_t) f * io.NA + al0 + a) * C + c] = g[idx];
      }
      __syncthreads();
    }
  }
}

template<int TA> void launch_ta(const FusedLayerDev &L, const FusedIO &io, int grid, size_t smem)
{
#ifndef GB_CPU_EMU
  static bool attr_set = false;
  if (!attr_set) {
    GB_CUDA(cudaFuncSetAttribute(chain_fused_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_set = true;
  }
#endif
  GB_LAUNCH((chain_fused_kernel<TA>), grid, NT, smem, L, io);
}

}    // namespace

void launch_chain_fused(int TA, const FusedLayerDev &L, const FusedIO &io, int grid)
{
  if (io.na == 0) return;
  const size_t smem = (size_t) L.per_atom * TA * sizeof(float);
  switch (TA) {
    case 1: launch_ta<1>(L, io, grid, smem); break;
    case 2: launch_ta<2>(L, io, grid, smem); break;
    case 3: launch_ta<3>(L, io, grid, smem); break;
    case 4: launch_ta<4>(L, io, grid, smem); break;
    case 6: launch_ta<6>(L, io, grid, smem); break;
    case 8: launch_ta<8>(L, io, grid, smem); break;
    default: throw DeviceError("fused dense network: unsupported atom tile");
  }
}

}    // namespace gb
