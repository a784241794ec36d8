// Kernels of the dense per-atom network (FC, Clebsch-Gordan products, reduces and their adjoints as two table-driven
// kernels), the fp64 readouts, and the per-atom gathers and sums that leave the network.
// Mathematics: libgrace/include/grace/fused_cpu.h:349-364 (FC), 411-453 (products), 637-649 (reduces);
// libgrace/src/fused_1l.cpp:378-427 and libgrace/src/fused_2l.cpp:548-615 (readouts).
#include "kernels.h"

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
          part[i] = fmaf(__ldg(x[i] + n), __ldg(op.W + tyo[i] + item.mat + (size_t) n * op.n_out + k), part[i]);
      }
    } else {
      const float *M = op.W + item.mat + k;
#pragma unroll 4
      for (int n = 0; n < item.n_in; n++) {
        const float w = __ldg(M + (size_t) n * op.n_out);
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
constexpr int RW = 128;    // largest width of the energy MLP (checked on the host)

// value of the MLP on x[0..nin) and, with g_out, its gradient dvalue/dx scaled by out_scale
__device__ double energy_mlp(const ReadoutDev &r, double *x, int nin, double *g_out)
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

__global__ void __launch_bounds__(64) readout_1l_kernel(ReadoutDev r, const float *__restrict__ rho, float *grho,
                                                        const int *__restrict__ mu, double *e_atom, int NA, int na,
                                                        int a0, int want_grad)
{
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= na) return;
  const int nr = r.nrho;
  double x[RW], g[RW];
  const float *ra = rho + (size_t) a * nr;
  for (int k = 1; k < nr; k++) x[k - 1] = ra[k];
  const double val = energy_mlp(r, x, nr - 1, want_grad ? g : nullptr);
  e_atom[a0 + a] = (val + (double) ra[0]) * r.out_scale + r.shift[mu[a0 + a]];
  if (want_grad) {
    float *ga = grho + (size_t) a * nr;
    ga[0] = (float) r.out_scale;
    for (int k = 1; k < nr; k++) ga[k] = (float) g[k - 1];
  }
}

void launch_readout_1l(const ReadoutDev &r, const float *rho, float *grho, const int *mu, double *e_atom, int NA,
                       int na, int a0, int want_grad)
{
  if (na == 0) return;
  GB_LAUNCH(readout_1l_kernel, (na + 63) / 64, 64, 0, r, rho, grho, mu, e_atom, NA, na, a0, want_grad);
}

// RMSNorms of rho[1:] and I2, MLP on their sum, and the reverse (libgrace/src/fused_2l.cpp:548-615)
__global__ void __launch_bounds__(64) readout_2l_kernel(ReadoutDev r, const float *__restrict__ rho_rows,
                                                        const float *__restrict__ I2, double *grho_rows, float *gI2,
                                                        const int *__restrict__ mu, double *e_atom, int NA, int na,
                                                        int a0, int want_grad)
{
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= na) return;
  const int nr = r.nrho;
  const float *rho = rho_rows + (size_t) (a0 + a) * nr;
  const float *i2 = I2 + (size_t) a * nr;
  double ms1 = 0.0, ms0 = 0.0;
  for (int k = 1; k < nr; k++) ms1 += (double) rho[k] * rho[k];
  for (int k = 0; k < nr; k++) ms0 += (double) i2[k] * i2[k];
  const double eps = 1e-10;
  const double s1 = r.rms ? sqrt(ms1 / (nr - 1) + eps) : 1.0, s0 = r.rms ? sqrt(ms0 / nr + eps) : 1.0;
  double x[RW], g[RW];
  for (int k = 1; k < nr; k++) x[k - 1] = rho[k] / s1 * r.lnI[k - 1] + i2[k] / s0 * r.ln0[k];
  const double val = energy_mlp(r, x, nr - 1, want_grad ? g : nullptr);
  e_atom[a0 + a] = (val + (double) rho[0] + (double) i2[0] / s0 * r.ln0[0]) * r.out_scale + r.shift[mu[a0 + a]];
  if (!want_grad) return;
  double *gr = grho_rows + (size_t) (a0 + a) * nr;
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
  float *go = gI2 + (size_t) a * nr;
  for (int k = 0; k < nr; k++) {
    const double gy = k == 0 ? r.out_scale : g[k - 1];
    go[k] = (float) (gy * r.ln0[k] / s0 - i2[k] * t0 / (nr * s0 * s0 * s0));
  }
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

void launch_segment_sum(const double *v, int K, const int *seg, int nseg, double *out)
{
  if (nseg == 0) return;
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
