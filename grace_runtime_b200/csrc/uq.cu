// UQ head (extrapolation grade) of GRACE-1L / GRACE-2L, forward only: after the projection z = B R of an atom's
// invariant basis B (an MV operation of the plan: plan.h LayerPlan::uq_mv), these two kernels give |B|^2 in fp64 and
// the Gaussian-mixture part: normalisation, log-norm density channels, nearest centroid of the atom's element,
// Mahalanobis distance -> sigma, gamma = sigma / threshold, cluster (libgrace/include/grace/fused_cpu.h:1291-1305,
// 1378-1412; libgrace/src/fused_1l.cpp:616-637; libgrace/src/fused_2l.cpp:1156-1187).  One warp per atom.
#include "kernels.h"

namespace gb {

namespace {

constexpr int UQ_WARPS = 4;

__device__ __forceinline__ double warp_sum(double v)
{
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// n2[a] = sum over the inputs of the projection operation of x^2, accumulated in fp64
__global__ void __launch_bounds__(32 * UQ_WARPS) uq_norm_kernel(MVDev op, const TensorDev *__restrict__ T, int NA, int na,
                                                                 double *__restrict__ n2)
{
  const int lane = threadIdx.x & 31, a = blockIdx.x * UQ_WARPS + (threadIdx.x >> 5);
  if (a >= na) return;
  const int i0 = op.item_off[0], i1 = op.item_off[op.nrows];
  double s = 0.0;
  for (int i = i0; i < i1; i++) {
    const MVItem it = op.items[i];
    const TensorDev t = T[it.src];
    const float *x = t.p + ((long long) it.irow * NA + a) * t.C;
    for (int n = lane; n < it.n_in; n += 32) {
      const double v = (double) x[n];
      s += v * v;
    }
  }
  s = warp_sum(s);
  if (lane == 0) n2[a] = s;
}

// z: projection of the last layer for the atoms of the chunk [na][RP]; z_prev / n2_prev: rows and squared norms of
// the earlier layer for all atoms (null: one-layer model); i = a0 + a indexes the per-atom arrays
__global__ void __launch_bounds__(32 * UQ_WARPS) uq_gmm_kernel(UqDev u, const float *__restrict__ z,
                                                                const float *__restrict__ z_prev,
                                                                const double *__restrict__ n2_last,
                                                                const double *__restrict__ n2_prev,
                                                                const int *__restrict__ mu, int na, long long a0,
                                                                double *__restrict__ gamma, double *__restrict__ sigma,
                                                                double *__restrict__ cluster)
{
  extern __shared__ double uq_sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, a = blockIdx.x * UQ_WARPS + warp;
  if (a >= na) return;
  const int RP = u.rp_dim, D = u.feature_dim, K = u.max_clusters;
  double *f = uq_sm + (size_t) warp * 2 * D, *delta = f + D;
  const long long i = a0 + a;
  const double s_last = n2_last[i], s_prev = n2_prev ? n2_prev[i] : 0.0;
  const double nrm = sqrt(s_prev + s_last);
  for (int d = lane; d < RP; d += 32) {
    double v = (double) z[(long long) a * RP + d];
    if (z_prev) v = (double) z_prev[i * RP + d] + v;
    f[d] = v / (nrm + 1.0e-12);
  }
  if (lane < u.n_density) {
    const double dens = lane == 0 ? nrm : lane == 1 ? sqrt(s_last) : sqrt(s_prev);
    f[RP + lane] = log(dens + 1.0e-12) * u.density_scale;
  }
  __syncwarp();
  const int m = mu[i];
  int kstar = 0;
  double best = 1.0e300;
  const int nq = u.n_clusters[m];
  for (int q = 0; q < nq; q++) {
    const double *cen = u.centroids + ((size_t) m * K + q) * D;
    double d2 = 0.0;
    for (int p = lane; p < D; p += 32) {
      const double t = f[p] - cen[p];
      d2 += t * t;
    }
    d2 = warp_sum(d2);
    if (d2 < best) {
      best = d2;
      kstar = q;
    }
  }
  const double *cen = u.centroids + ((size_t) m * K + kstar) * D;
  for (int p = lane; p < D; p += 32) delta[p] = f[p] - cen[p];
  __syncwarp();
  // sig2 = delta^T S delta with y = S^T delta formed column by column (lanes over the columns: coalesced rows of S)
  const double *S = u.inv_cov + ((size_t) m * K + kstar) * D * D;
  double sig2 = 0.0;
  for (int q = lane; q < D; q += 32) {
    double y = 0.0;
    for (int p = 0; p < D; p++) y += delta[p] * S[(size_t) p * D + q];
    sig2 += delta[q] * y;
  }
  sig2 = warp_sum(sig2);
  if (lane == 0) {
    const double sg = sqrt(sig2 + 1.0e-8);
    sigma[i] = sg;
    gamma[i] = sg / fmax(u.thresholds[(size_t) m * K + kstar], 1.0e-10);
    cluster[i] = (double) kstar;
  }
}

}    // namespace

void launch_uq_norm(const MVDev &op, const TensorDev *tensors, int NA, int na, double *n2)
{
  if (na <= 0) return;
  GB_LAUNCH(uq_norm_kernel, dim3((na + UQ_WARPS - 1) / UQ_WARPS), dim3(32 * UQ_WARPS), 0, op, tensors, NA, na, n2);
}

void launch_uq_gmm(const UqDev &u, const float *z, const float *z_prev, const double *n2_last, const double *n2_prev,
                   const int *mu, int na, long long a0, double *gamma, double *sigma, double *cluster)
{
  if (na <= 0) return;
  const size_t smem = sizeof(double) * 2 * (size_t) u.feature_dim * UQ_WARPS;
  GB_LAUNCH(uq_gmm_kernel, dim3((na + UQ_WARPS - 1) / UQ_WARPS), dim3(32 * UQ_WARPS), smem, u, z, z_prev, n2_last, n2_prev,
            mu, na, a0, gamma, sigma, cluster);
}

}    // namespace gb
