// Kernels of the dense per-atom network (FC, Clebsch-Gordan products, reduces and their adjoints as two table-driven
// kernels), the fp64 readouts, and the per-atom gathers and sums that leave the network.
// Mathematics: libgrace/include/grace/fused_cpu.h:349-364 (FC), 411-453 (products), 637-649 (reduces);
// libgrace/src/fused_1l.cpp:378-427 and libgrace/src/fused_2l.cpp:548-615 (readouts).
#include "kernels.h"
#include "readout.cuh"

namespace gb {

// ---- MV: out[row][a][k] (+)= sum_items scale * sum_n M[n][k] x[item][a][n] ----------------------------------
// block (KP, 128 / KP): threadIdx.x = output channel k, threadIdx.y = atom group; AT atoms per thread share each
// weight load.  grid (rows, atom blocks).
template<int AT, bool ELEM>
__global__ void __launch_bounds__(128) mv_kernel(MVDev op, const TensorDev *__restrict__ T, const int *__restrict__ mu,
                                                 int NA, int na)
{
  const int row = blockIdx.x;
  const int k = threadIdx.x;
  const int a_first = (blockIdx.y * blockDim.y + threadIdx.y) * AT;
  if (k >= op.n_out || a_first >= na) return;
  float acc[AT];
  long long tyo[AT];
#pragma unroll
  for (int i = 0; i < AT; i++) {
    acc[i] = 0.0f;
    const int a = min(a_first + i, na - 1);
    tyo[i] = ELEM ? (long long) mu[a] * op.ty_stride : 0;
  }
  const int i0 = op.item_off[row], i1 = op.item_off[row + 1];
  for (int it = i0; it < i1; it++) {
    const MVItem item = op.items[it];
    const TensorDev src = T[item.src];
    const float *x[AT];
#pragma unroll
    for (int i = 0; i < AT; i++) x[i] = src.p + ((size_t) item.irow * NA + min(a_first + i, na - 1)) * src.C;
    float part[AT];
#pragma unroll
    for (int i = 0; i < AT; i++) part[i] = 0.0f;
    if (ELEM) {
      for (int n = 0; n < item.n_in; n++) {
#pragma unroll
        for (int i = 0; i < AT; i++)
          part[i] = fmaf(__ldg(x[i] + n), __ldg(op.W + tyo[i] + item.mat + (size_t) n * op.ldw + k), part[i]);
      }
    } else {
      const float *M = op.W + item.mat + k;
#pragma unroll 4
      for (int n = 0; n < item.n_in; n++) {
        const float w = __ldg(M + (size_t) n * op.ldw);
#pragma unroll
        for (int i = 0; i < AT; i++) part[i] = fmaf(__ldg(x[i] + n), w, part[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < AT; i++) acc[i] = fmaf(item.scale, part[i], acc[i]);
  }
  const TensorDev dst = T[op.dst];
  const int orow = op.row_out[row];
#pragma unroll
  for (int i = 0; i < AT; i++) {
    const int a = a_first + i;
    if (a < na) {
      float *o = dst.p + ((size_t) orow * NA + a) * dst.C + k;
      *o = op.accumulate ? *o + acc[i] : acc[i];
    }
  }
}

void launch_mv(const MVDev &op, const TensorDev *tensors, const int *mu, int NA, int na)
{
  if (op.nrows == 0 || na == 0) return;
  int KP = 8;
  while (KP < op.n_out) KP *= 2;
  if (KP > 128) throw Unsupported("dense network: more than 128 channels are not supported");
  constexpr int AT = 4;
  const dim3 block(KP, 128 / KP);
  const dim3 grid(op.nrows, (na + block.y * AT - 1) / (block.y * AT));
  if (op.elem) GB_LAUNCH((mv_kernel<AT, true>), grid, block, 0, op, tensors, mu, NA, na);
  else GB_LAUNCH((mv_kernel<AT, false>), grid, block, 0, op, tensors, mu, NA, na);
}

// ---- PROD: out[row][i] (+)= sum_terms coef A[a][i] B[b][i], i over the NA * C values of a function row ---------
__global__ void __launch_bounds__(256) prod_kernel(ProdDev op, const TensorDev *__restrict__ T, long long row_len,
                                                   long long act_len)
{
  const int row = blockIdx.x;
  const long long i = (long long) blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= act_len) return;
  const float *A = T[op.srcA].p + i;
  const float *B = op.srcB >= 0 ? T[op.srcB].p + i : nullptr;
  const int t0 = op.term_off[row], t1 = op.term_off[row + 1];
  float acc = 0.0f;
  if (B) {
    for (int t = t0; t < t1; t++) {
      const ProdTerm tm = op.terms[t];
      acc = fmaf(tm.coef * __ldg(A + tm.a * row_len), __ldg(B + tm.b * row_len), acc);
    }
  } else {
    for (int t = t0; t < t1; t++) {
      const ProdTerm tm = op.terms[t];
      acc = fmaf(tm.coef, __ldg(A + tm.a * row_len), acc);
    }
  }
  float *o = T[op.dst].p + (long long) op.row_out[row] * row_len + i;
  *o = op.accumulate ? *o + acc : acc;
}

void launch_prod(const ProdDev &op, const TensorDev *tensors, int NA, int na, int C)
{
  if (op.nrows == 0 || na == 0) return;
  const long long row_len = (long long) NA * C, act_len = (long long) na * C;
  const dim3 grid(op.nrows, (unsigned) ((act_len + 255) / 256));
  GB_LAUNCH(prod_kernel, grid, 256, 0, op, tensors, row_len, act_len);
}

// ---- readouts (fp64, one thread per atom) ---------------------------------------------------------------------
__global__ void __launch_bounds__(64) readout_1l_kernel(ReadoutDev r, const float *__restrict__ rho, float *grho,
                                                        const int *__restrict__ mu, double *e_atom, int NA, int na,
                                                        int a0, int want_grad)
{
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= na) return;
  e_atom[a0 + a] = readout_1l_atom(r, rho + (size_t) a * r.nrho, mu[a0 + a], grho + (size_t) a * r.nrho, want_grad,
                                   r.owned(a0 + a));
}

void launch_readout_1l(const ReadoutDev &r, const float *rho, float *grho, const int *mu, double *e_atom, int NA,
                       int na, int a0, int want_grad)
{
  if (na == 0) return;
  GB_LAUNCH(readout_1l_kernel, (na + 63) / 64, 64, 0, r, rho, grho, mu, e_atom, NA, na, a0, want_grad);
}

__global__ void __launch_bounds__(64) readout_2l_kernel(ReadoutDev r, const float *__restrict__ rho_rows,
                                                        const float *__restrict__ I2, double *grho_rows, float *gI2,
                                                        const int *__restrict__ mu, double *e_atom, int NA, int na,
                                                        int a0, int want_grad)
{
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= na) return;
  const int nr = r.nrho;
  e_atom[a0 + a] = readout_2l_atom(r, rho_rows + (size_t) (a0 + a) * nr, I2 + (size_t) a * nr, mu[a0 + a],
                                   grho_rows + (size_t) (a0 + a) * nr, gI2 + (size_t) a * nr, want_grad, r.owned(a0 + a));
}

void launch_readout_2l(const ReadoutDev &r, const float *rho_rows, const float *I2, double *grho_rows, float *gI2,
                       const int *mu, double *e_atom, int NA, int na, int a0, int want_grad)
{
  if (na == 0) return;
  GB_LAUNCH(readout_2l_kernel, (na + 63) / 64, 64, 0, r, rho_rows, I2, grho_rows, gI2, mu, e_atom, NA, na, a0,
            want_grad);
}

// ---- chunk tensor <-> per-atom rows ----------------------------------------------------------------------------
template<class TR, bool TO_ROWS>
__global__ void __launch_bounds__(256) rows_kernel(float *t, TR *rows, int nf, int C, int NA, int na, int a0)
{
  const long long idx = (long long) blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long) na * nf * C;
  if (idx >= total) return;
  const int c = (int) (idx % C);
  const int f = (int) ((idx / C) % nf);
  const int a = (int) (idx / ((long long) C * nf));
  float *tp = t + ((size_t) f * NA + a) * C + c;
  TR *rp = rows + ((size_t) (a0 + a) * nf + f) * C + c;
  if (TO_ROWS) *rp = (TR) *tp;
  else *tp = (float) *rp;
}

void launch_rows_from_chunk(const float *t, float *rows, int nf, int C, int NA, int na, int a0)
{
  const long long total = (long long) na * nf * C;
  if (total == 0) return;
  GB_LAUNCH((rows_kernel<float, true>), (unsigned) ((total + 255) / 256), 256, 0, const_cast<float *>(t), rows, nf, C,
            NA, na, a0);
}
void launch_chunk_from_rows(float *t, const float *rows, int nf, int C, int NA, int na, int a0)
{
  const long long total = (long long) na * nf * C;
  if (total == 0) return;
  GB_LAUNCH((rows_kernel<float, false>), (unsigned) ((total + 255) / 256), 256, 0, t, const_cast<float *>(rows), nf, C,
            NA, na, a0);
}
void launch_chunk_from_rows_f64(float *t, const double *rows, int nf, int C, int NA, int na, int a0)
{
  const long long total = (long long) na * nf * C;
  if (total == 0) return;
  GB_LAUNCH((rows_kernel<double, false>), (unsigned) ((total + 255) / 256), 256, 0, t, const_cast<double *>(rows), nf,
            C, NA, na, a0);
}

// ---- forces: gather of the bond forces of an atom and of their reverse bonds, no atomics ------------------------
// one warp per atom: F_i = sum_q fv[q] - fv[rev[q]] over the slots q of atom i (fp64 sum of the fp32 bond forces)
__global__ void __launch_bounds__(128) force_gather_kernel(const long long *__restrict__ off,
                                                           const int *__restrict__ rev, const float *__restrict__ fv,
                                                           const int *__restrict__ perm, double *forces, int n)
{
  const int i = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  const int lane = threadIdx.x & 31;
  if (i >= n) return;    // whole warps leave together
  double f0 = 0.0, f1 = 0.0, f2 = 0.0;
  for (long long q = off[i] + lane; q < off[i + 1]; q += 32) {
    const long long p = rev[q];
    f0 += (double) fv[3 * q] - (double) fv[3 * p];
    f1 += (double) fv[3 * q + 1] - (double) fv[3 * p + 1];
    f2 += (double) fv[3 * q + 2] - (double) fv[3 * p + 2];
  }
  for (int s = 16; s > 0; s >>= 1) {
    f0 += __shfl_xor_sync(0xffffffffu, f0, s);
    f1 += __shfl_xor_sync(0xffffffffu, f1, s);
    f2 += __shfl_xor_sync(0xffffffffu, f2, s);
  }
  if (lane == 0) {
    double *o = forces + 3 * (size_t) perm[i];
    o[0] = f0; o[1] = f1; o[2] = f2;
  }
}

void launch_force_gather(const long long *off, const int *rev, const float *fv, const int *perm, double *forces, int n)
{
  if (n == 0) return;
  GB_LAUNCH(force_gather_kernel, (n + 3) / 4, 128, 0, off, rev, fv, perm, forces, n);
}

// ---- per-structure sums (deterministic: fixed tree per segment) ------------------------------------------------
// one block per (segment, component)
__global__ void __launch_bounds__(256) segment_sum_kernel(const double *__restrict__ v, int K,
                                                          const int *__restrict__ seg, double *out)
{
  __shared__ double sh[256];
  const int s = blockIdx.x, k = blockIdx.y;
  double acc = 0.0;
  for (int i = seg[s] + threadIdx.x; i < seg[s + 1]; i += blockDim.x) acc += v[(size_t) i * K + k];
  sh[threadIdx.x] = acc;
  __syncthreads();
  for (int st = 128; st > 0; st >>= 1) {
    if ((int) threadIdx.x < st) sh[threadIdx.x] += sh[threadIdx.x + st];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[(size_t) s * K + k] = sh[0];
}

// few long segments (one large structure): NB blocks per (segment, component) write partial sums over equal slices
// of the segment, a second launch adds them in slice order - still a fixed tree
__global__ void __launch_bounds__(256) segment_partial_kernel(const double *__restrict__ v, int K,
                                                              const int *__restrict__ seg, double *partial)
{
  __shared__ double sh[256];
  const int s = blockIdx.x, k = blockIdx.y, b = blockIdx.z, NB = gridDim.z;
  const long long s0 = seg[s], len = seg[s + 1] - s0, per = (len + NB - 1) / NB;
  const long long lo = s0 + b * per, hi = min(s0 + len, lo + per);
  double acc = 0.0;
  for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) acc += v[(size_t) i * K + k];
  sh[threadIdx.x] = acc;
  __syncthreads();
  for (int st = 128; st > 0; st >>= 1) {
    if ((int) threadIdx.x < st) sh[threadIdx.x] += sh[threadIdx.x + st];
    __syncthreads();
  }
  if (threadIdx.x == 0) partial[((size_t) s * K + k) * NB + b] = sh[0];
}

__global__ void __launch_bounds__(32) segment_final_kernel(const double *__restrict__ partial, int NB, double *out)
{
  const int sk = blockIdx.x;    // segment * K + component
  if (threadIdx.x != 0) return;
  double acc = 0.0;
  for (int b = 0; b < NB; b++) acc += partial[(size_t) sk * NB + b];
  out[sk] = acc;
}

void launch_segment_sum(const double *v, int K, const int *seg, int nseg, double *out, double *scratch, int nb)
{
  if (nseg == 0) return;
  if (scratch && nb > 1) {
    GB_LAUNCH(segment_partial_kernel, dim3(nseg, K, nb), 256, 0, v, K, seg, scratch);
    GB_LAUNCH(segment_final_kernel, nseg * K, 32, 0, scratch, nb, out);
    return;
  }
  GB_LAUNCH(segment_sum_kernel, dim3(nseg, K), 256, 0, v, K, seg, out);
}

__global__ void __launch_bounds__(256) scatter_f64_kernel(const double *__restrict__ v, const int *__restrict__ perm,
                                                          double *out, int n)
{
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[perm[i]] = v[i];
}

void launch_scatter_f64(const double *v, const int *perm, double *out, int n)
{
  if (n == 0) return;
  GB_LAUNCH(scatter_f64_kernel, (n + 255) / 256, 256, 0, v, perm, out, n);
}

}    // namespace gb
