#include "nlist.h"

#include <algorithm>
#include <cmath>
#include <cstring>

namespace gb {

// ---- exclusive scan int32 -> int64 -----------------------------------------------------------------------------
namespace {

constexpr int SCAN_T = 256, SCAN_I = 8, SCAN_TILE = SCAN_T * SCAN_I;

__global__ void __launch_bounds__(SCAN_T) scan_tile_sums(const int *__restrict__ in, long long *tmp, long long n)
{
  __shared__ long long sh[SCAN_T];
  const long long t0 = (long long) blockIdx.x * SCAN_TILE + (long long) threadIdx.x * SCAN_I;
  long long s = 0;
  for (int k = 0; k < SCAN_I; k++)
    if (t0 + k < n) s += in[t0 + k];
  sh[threadIdx.x] = s;
  __syncthreads();
  for (int st = SCAN_T / 2; st > 0; st >>= 1) {
    if ((int) threadIdx.x < st) sh[threadIdx.x] += sh[threadIdx.x + st];
    __syncthreads();
  }
  if (threadIdx.x == 0) tmp[blockIdx.x] = sh[0];
}

// exclusive scan of the tile sums in place by one block: 1024 tile sums at a time (Hillis-Steele in shared memory) with
// a running carry, so that tens of millions of atoms cost a few passes instead of one thread walking every tile
__global__ void __launch_bounds__(1024) scan_partials(long long *tmp, long long ntiles, long long *out, long long n)
{
  __shared__ long long sh[1024];
  __shared__ long long carry;
  const int t = threadIdx.x;
  if (t == 0) carry = 0;
  __syncthreads();
  for (long long b0 = 0; b0 < ntiles; b0 += 1024) {
    const long long b = b0 + t;
    const long long v = b < ntiles ? tmp[b] : 0;
    sh[t] = v;
    __syncthreads();
    for (int st = 1; st < 1024; st <<= 1) {
      const long long add = t >= st ? sh[t - st] : 0;
      __syncthreads();
      sh[t] += add;
      __syncthreads();
    }
    if (b < ntiles) tmp[b] = carry + sh[t] - v;
    __syncthreads();
    if (t == 1023) carry += sh[1023];
    __syncthreads();
  }
  if (t == 0) out[n] = carry;
}

__global__ void __launch_bounds__(SCAN_T) scan_tile_final(const int *__restrict__ in, const long long *__restrict__ tmp,
                                                          long long *out, long long n)
{
  __shared__ long long sh[SCAN_T];
  const long long t0 = (long long) blockIdx.x * SCAN_TILE + (long long) threadIdx.x * SCAN_I;
  int v[SCAN_I];
  long long s = 0;
  for (int k = 0; k < SCAN_I; k++) {
    v[k] = (t0 + k < n) ? in[t0 + k] : 0;
    s += v[k];
  }
  sh[threadIdx.x] = s;
  __syncthreads();
  // inclusive Hillis-Steele scan of the thread sums
  for (int st = 1; st < SCAN_T; st <<= 1) {
    const long long add = ((int) threadIdx.x >= st) ? sh[threadIdx.x - st] : 0;
    __syncthreads();
    sh[threadIdx.x] += add;
    __syncthreads();
  }
  long long run = tmp[blockIdx.x] + sh[threadIdx.x] - s;
  for (int k = 0; k < SCAN_I; k++) {
    if (t0 + k < n) out[t0 + k] = run;
    run += v[k];
  }
}

}    // namespace

void launch_scan(const int *in, long long *out, long long *tmp, int64_t n)
{
  const long long ntiles = (n + SCAN_TILE - 1) / SCAN_TILE;
  if (ntiles > 0) GB_LAUNCH(scan_tile_sums, (unsigned) ntiles, SCAN_T, 0, in, tmp, (long long) n);
  GB_LAUNCH(scan_partials, 1, 1024, 0, tmp, ntiles, out, (long long) n);
  if (ntiles > 0) GB_LAUNCH(scan_tile_final, (unsigned) ntiles, SCAN_T, 0, in, tmp, out, (long long) n);
}

// ---- list build ------------------------------------------------------------------------------------------------
namespace {

__device__ __forceinline__ int floordiv(int a, int b) { return a >= 0 ? a / b : -((-a + b - 1) / b); }
__device__ __forceinline__ int pack_S(int s0, int s1, int s2)
{
  return (s0 & 0xff) | ((s1 & 0xff) << 8) | ((s2 & 0xff) << 16);
}
__device__ __forceinline__ void unpack_S(int p, int &s0, int &s1, int &s2)
{
  s0 = (int) (signed char) (p & 0xff);
  s1 = (int) (signed char) ((p >> 8) & 0xff);
  s2 = (int) (signed char) ((p >> 16) & 0xff);
}

// fractional coordinates, wrapped in periodic directions, and the integer image removed by the wrap
__global__ void __launch_bounds__(256) nl_frac(const double *__restrict__ pos, const int *__restrict__ sid,
                                               const NLStructHost *__restrict__ S, double *frac, int *img,
                                               double *xbuild, int *flag, long long n)
{
  const long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const NLStructHost &s = S[sid[i]];
  const double x = pos[3 * i], y = pos[3 * i + 1], z = pos[3 * i + 2];
  xbuild[3 * i] = x; xbuild[3 * i + 1] = y; xbuild[3 * i + 2] = z;
  for (int k = 0; k < 3; k++) {
    const double f = x * s.inv[k] + y * s.inv[3 + k] + z * s.inv[6 + k];
    if (!isfinite(f)) atomicOr(flag, 1);
    const double fl = s.pbc[k] ? floor(f) : 0.0;
    if (fabs(fl) > 1.0e9) atomicOr(flag, 1);
    img[3 * i + k] = (int) fl;
    frac[3 * i + k] = f - fl;
  }
}

// occupied range of the fractional coordinates of each structure (open directions): one block per structure
__global__ void __launch_bounds__(256) nl_minmax(const double *__restrict__ frac, const NLStructHost *__restrict__ S,
                                                 double *lohi)
{
  __shared__ double smin[3][256], smax[3][256];
  const int s = blockIdx.x;
  double mn[3] = {1e300, 1e300, 1e300}, mx[3] = {-1e300, -1e300, -1e300};
  for (int i = S[s].atom0 + threadIdx.x; i < S[s].atom1; i += blockDim.x)
    for (int k = 0; k < 3; k++) {
      const double f = frac[3 * (size_t) i + k];
      mn[k] = fmin(mn[k], f);
      mx[k] = fmax(mx[k], f);
    }
  for (int k = 0; k < 3; k++) { smin[k][threadIdx.x] = mn[k]; smax[k][threadIdx.x] = mx[k]; }
  __syncthreads();
  for (int st = 128; st > 0; st >>= 1) {
    if ((int) threadIdx.x < st)
      for (int k = 0; k < 3; k++) {
        smin[k][threadIdx.x] = fmin(smin[k][threadIdx.x], smin[k][threadIdx.x + st]);
        smax[k][threadIdx.x] = fmax(smax[k][threadIdx.x], smax[k][threadIdx.x + st]);
      }
    __syncthreads();
  }
  if (threadIdx.x < 3) {
    lohi[6 * s + threadIdx.x] = smin[threadIdx.x][0];
    lohi[6 * s + 3 + threadIdx.x] = smax[threadIdx.x][0];
  }
}

__global__ void __launch_bounds__(256) nl_bin(const double *__restrict__ frac, const int *__restrict__ sid,
                                              const NLStructHost *__restrict__ S, int *binid, int *count, long long n)
{
  const long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const NLStructHost &s = S[sid[i]];
  int b[3];
  for (int k = 0; k < 3; k++) {
    const int v = (int) floor((frac[3 * i + k] - s.lo[k]) / s.span[k] * (double) s.nbin[k]);
    b[k] = min(max(v, 0), s.nbin[k] - 1);
  }
  const int bin = s.bin_base + (b[0] * s.nbin[1] + b[1]) * s.nbin[2] + b[2];
  binid[i] = bin;
  atomicAdd(&count[bin], 1);
}

__global__ void __launch_bounds__(256) nl_place(const int *__restrict__ binid, const long long *__restrict__ start,
                                                int *fill, int *members, long long n)
{
  const long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int bin = binid[i];
  members[start[bin] + atomicAdd(&fill[bin], 1)] = (int) i;
}

// stable order inside each bin: rank of an atom = atoms of its bin with a smaller caller index
__global__ void __launch_bounds__(256) nl_order(const int *__restrict__ binid, const long long *__restrict__ start,
                                                const int *__restrict__ members, int *perm, long long n)
{
  const long long p = (long long) blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n) return;
  const int i = members[p], bin = binid[i];
  int rank = 0;
  for (long long q = start[bin]; q < start[bin + 1]; q++) rank += members[q] < i;
  perm[start[bin] + rank] = i;
}

// per atom in list order: wrapped position, element, structure, bin coordinates, image
__global__ void __launch_bounds__(256) nl_sorted(const int *__restrict__ perm, const double *__restrict__ frac,
                                                 const int *__restrict__ sid, const int *__restrict__ mu,
                                                 const int *__restrict__ img, const NLStructHost *__restrict__ S,
                                                 double *xs, int *mu_s, int *sid_s, int *b3_s, int *img_s, long long n)
{
  const long long q = (long long) blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= n) return;
  const int i = perm[q];
  const NLStructHost &s = S[sid[i]];
  const double f0 = frac[3 * (size_t) i], f1 = frac[3 * (size_t) i + 1], f2 = frac[3 * (size_t) i + 2];
  for (int d = 0; d < 3; d++) xs[3 * q + d] = f0 * s.cell[d] + f1 * s.cell[3 + d] + f2 * s.cell[6 + d];
  const double f[3] = {f0, f1, f2};
  for (int k = 0; k < 3; k++) {
    const int v = (int) floor((f[k] - s.lo[k]) / s.span[k] * (double) s.nbin[k]);
    b3_s[3 * q + k] = min(max(v, 0), s.nbin[k] - 1);
    img_s[3 * q + k] = img[3 * (size_t) i + k];
  }
  mu_s[q] = mu[i];
  sid_s[q] = sid[i];
}

// neighbours of atom q within the radius: FILL false counts them, FILL true writes j and the lattice translation
template<bool FILL>
__global__ void __launch_bounds__(128) nl_neigh(const double *__restrict__ xs, const int *__restrict__ sid_s,
                                                const int *__restrict__ b3_s, const NLStructHost *__restrict__ S,
                                                const long long *__restrict__ start, double rad2, int *cnt,
                                                const long long *__restrict__ off, int *nbr_j, int *nbr_S, int *flag,
                                                long long n)
{
  const long long q = (long long) blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= n) return;
  const NLStructHost &s = S[sid_s[q]];
  const double xq = xs[3 * q], yq = xs[3 * q + 1], zq = xs[3 * q + 2];
  const int bq0 = b3_s[3 * q], bq1 = b3_s[3 * q + 1], bq2 = b3_s[3 * q + 2];
  int c = 0;
  long long w = FILL ? off[q] : 0;
  for (int o0 = -s.reach[0]; o0 <= s.reach[0]; o0++) {
    int c0 = bq0 + o0, s0 = 0;
    if (s.pbc[0]) { s0 = floordiv(c0, s.nbin[0]); c0 -= s0 * s.nbin[0]; }
    else if (c0 < 0 || c0 >= s.nbin[0]) continue;
    for (int o1 = -s.reach[1]; o1 <= s.reach[1]; o1++) {
      int c1 = bq1 + o1, s1 = 0;
      if (s.pbc[1]) { s1 = floordiv(c1, s.nbin[1]); c1 -= s1 * s.nbin[1]; }
      else if (c1 < 0 || c1 >= s.nbin[1]) continue;
      for (int o2 = -s.reach[2]; o2 <= s.reach[2]; o2++) {
        int c2 = bq2 + o2, s2 = 0;
        if (s.pbc[2]) { s2 = floordiv(c2, s.nbin[2]); c2 -= s2 * s.nbin[2]; }
        else if (c2 < 0 || c2 >= s.nbin[2]) continue;
        const int bin = s.bin_base + (c0 * s.nbin[1] + c1) * s.nbin[2] + c2;
        const double sx = s0 * s.cell[0] + s1 * s.cell[3] + s2 * s.cell[6];
        const double sy = s0 * s.cell[1] + s1 * s.cell[4] + s2 * s.cell[7];
        const double sz = s0 * s.cell[2] + s1 * s.cell[5] + s2 * s.cell[8];
        const bool own = s0 == 0 && s1 == 0 && s2 == 0;
        for (long long p = start[bin]; p < start[bin + 1]; p++) {
          if (own && p == q) continue;
          const double dx = (xs[3 * p] - xq) + sx, dy = (xs[3 * p + 1] - yq) + sy, dz = (xs[3 * p + 2] - zq) + sz;
          const double r2 = dx * dx + dy * dy + dz * dz;
          if (r2 < rad2) {
            if (r2 == 0.0) atomicOr(flag, 2);
            if (FILL) {
              nbr_j[w] = (int) p;
              nbr_S[w] = pack_S(s0, s1, s2);
              w++;
            }
            c++;
          }
        }
      }
    }
  }
  if (!FILL) cnt[q] = c;
}

// reverse bond of every slot: the slot of atom j that points back at i with the opposite translation
__global__ void __launch_bounds__(128) nl_reverse(const long long *__restrict__ off, const int *__restrict__ nbr_j,
                                                  const int *__restrict__ nbr_S, int *rev, int *flag, long long n)
{
  const long long i = (long long) blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  const int lane = threadIdx.x & 31;
  if (i >= n) return;
  for (long long e = off[i] + lane; e < off[i + 1]; e += 32) {
    const int j = nbr_j[e];
    int s0, s1, s2;
    unpack_S(nbr_S[e], s0, s1, s2);
    const int want = pack_S(-s0, -s1, -s2);
    long long found = -1;
    for (long long p = off[j]; p < off[j + 1]; p++)
      if (nbr_j[p] == (int) i && nbr_S[p] == want) { found = p; break; }
    if (found < 0) { atomicOr(flag, 4); found = e; }
    rev[e] = (int) found;
  }
}

__global__ void __launch_bounds__(256) nl_moved(const double *__restrict__ pos, const double *__restrict__ xbuild,
                                                double lim2, int *flag, int bit, long long n)
{
  const long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const double dx = pos[3 * i] - xbuild[3 * i], dy = pos[3 * i + 1] - xbuild[3 * i + 1],
               dz = pos[3 * i + 2] - xbuild[3 * i + 2];
  if (!(dx * dx + dy * dy + dz * dz <= lim2)) atomicOr(flag, bit);    // NaN counts as moved
}

// this call's positions in list order, shifted by the images of the build
__global__ void __launch_bounds__(256) nl_positions(const double *__restrict__ pos, const int *__restrict__ perm,
                                                    const int *__restrict__ img_s, const int *__restrict__ sid_s,
                                                    const NLStructHost *__restrict__ S, double *xs, long long n)
{
  const long long q = (long long) blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= n) return;
  const NLStructHost &s = S[sid_s[q]];
  const size_t i = perm[q];
  const int m0 = img_s[3 * q], m1 = img_s[3 * q + 1], m2 = img_s[3 * q + 2];
  for (int d = 0; d < 3; d++) xs[3 * q + d] = pos[3 * i + d] - (m0 * s.cell[d] + m1 * s.cell[3 + d] + m2 * s.cell[6 + d]);
}

// one warp per atom: bonds inside the pair cutoff compacted to the front of the atom's slots
__global__ void __launch_bounds__(128) nl_compact(const double *__restrict__ xs, const int *__restrict__ mu_s,
                                                  const int *__restrict__ sid_s, const NLStructHost *__restrict__ S,
                                                  const long long *__restrict__ off, const int *__restrict__ nbr_j,
                                                  const int *__restrict__ nbr_S, const double *__restrict__ rcsq,
                                                  int nel, float4 *rec, int *cslot, int *cnt, float *fv, int *flag,
                                                  long long n)
{
  const long long i = (long long) blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  const int lane = threadIdx.x & 31;
  if (i >= n) return;
  const NLStructHost &s = S[sid_s[i]];
  const double xi = xs[3 * i], yi = xs[3 * i + 1], zi = xs[3 * i + 2];
  const int mui = mu_s[i];
  const long long base = off[i];
  const int cntf = (int) (off[i + 1] - base);
  int nact = 0;
  for (int q0 = 0; q0 < cntf; q0 += 32) {
    const int q = q0 + lane;
    const bool valid = q < cntf;
    bool act = false;
    float4 r4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (valid) {
      const int j = nbr_j[base + q];
      int s0, s1, s2;
      unpack_S(nbr_S[base + q], s0, s1, s2);
      const double dx = (xs[3 * (size_t) j] - xi) + (s0 * s.cell[0] + s1 * s.cell[3] + s2 * s.cell[6]);
      const double dy = (xs[3 * (size_t) j + 1] - yi) + (s0 * s.cell[1] + s1 * s.cell[4] + s2 * s.cell[7]);
      const double dz = (xs[3 * (size_t) j + 2] - zi) + (s0 * s.cell[2] + s1 * s.cell[5] + s2 * s.cell[8]);
      const double r2 = dx * dx + dy * dy + dz * dz;
      act = r2 < rcsq[(size_t) mui * nel + mu_s[j]];
      if (act && r2 == 0.0) { atomicOr(flag, 2); act = false; }
      r4 = make_float4((float) dx, (float) dy, (float) dz, __int_as_float(j));
    }
    const unsigned m = __ballot_sync(0xffffffffu, act);
    if (act) {
      const int pos = nact + __popc(m & ((1u << lane) - 1u));
      rec[base + pos] = r4;
      cslot[base + pos] = (int) (base + q);
    } else if (valid) {
      fv[3 * (base + q)] = 0.0f; fv[3 * (base + q) + 1] = 0.0f; fv[3 * (base + q) + 2] = 0.0f;
    }
    nact += __popc(m);
  }
  if (lane == 0) cnt[i] = nact;
}

__global__ void __launch_bounds__(256) nl_fill_sid(int *sid, const NLStructHost *__restrict__ S, int nsys)
{
  const int s = blockIdx.x;
  for (int i = S[s].atom0 + threadIdx.x; i < S[s].atom1; i += blockDim.x) sid[i] = s;
}

void invert3(const double *a, double *inv, double &det)
{
  det = a[0] * (a[4] * a[8] - a[5] * a[7]) - a[1] * (a[3] * a[8] - a[5] * a[6]) + a[2] * (a[3] * a[7] - a[4] * a[6]);
  const double d = 1.0 / det;
  const double r[9] = {(a[4] * a[8] - a[5] * a[7]) * d, (a[2] * a[7] - a[1] * a[8]) * d, (a[1] * a[5] - a[2] * a[4]) * d,
                       (a[5] * a[6] - a[3] * a[8]) * d, (a[0] * a[8] - a[2] * a[6]) * d, (a[2] * a[3] - a[0] * a[5]) * d,
                       (a[3] * a[7] - a[4] * a[6]) * d, (a[1] * a[6] - a[0] * a[7]) * d, (a[0] * a[4] - a[1] * a[3]) * d};
  std::memcpy(inv, r, sizeof(r));
}

int read_flag(int *d_flag)
{
  int h = 0;
  GB_CUDA(cudaMemcpyAsync(&h, d_flag, sizeof(int), cudaMemcpyDeviceToHost, dev().stream));
  GB_CUDA(cudaStreamSynchronize(dev().stream));
  return h;
}

unsigned blocks(long long n, int per) { return (unsigned) ((n + per - 1) / per); }

}    // namespace

NeighborList::NeighborList()
{
  frac_.set_label("nlist:frac"); xs_.set_label("nlist:positions"); xbuild_.set_label("nlist:positions_build");
  lohi_.set_label("nlist:range"); img_.set_label("nlist:image"); img_s_.set_label("nlist:image");
  sid_.set_label("nlist:structure"); sid_s_.set_label("nlist:structure"); binid_.set_label("nlist:bin");
  b3_s_.set_label("nlist:bin"); count_.set_label("nlist:bin_count"); fill_.set_label("nlist:bin_count");
  members_.set_label("nlist:members"); perm_.set_label("nlist:perm"); mu_s_.set_label("nlist:element");
  cnt_full_.set_label("nlist:count"); cnt_.set_label("nlist:count"); nbr_j_.set_label("nlist:neighbors");
  nbr_S_.set_label("nlist:neighbors"); rev_.set_label("nlist:reverse"); cslot_.set_label("nlist:bond_slot");
  seg_.set_label("nlist:segments"); flag_.set_label("nlist:flag"); start_.set_label("nlist:bin_start");
  off_.set_label("nlist:offset"); scan_tmp_.set_label("nlist:scan"); rec_.set_label("nlist:bonds");
  d_st_.set_label("nlist:cells");
}

void NeighborList::build(int nsys, const int *natoms, int64_t n, const double *d_pos, const int *d_mu,
                         const double *cells, const unsigned char *pbc, double radius)
{
  if (!(radius > 0.0) || !std::isfinite(radius)) throw InvalidArgument("cutoff must be positive");
  if (n >= (int64_t) 1 << 31) throw InvalidArgument("atom count out of range");
  n_ = 0;
  nslots_ = 0;
  nsys_ = nsys;
  st_.assign(nsys, NLStructHost{});
  std::vector<double> heights(3 * (size_t) nsys);
  int64_t at = 0;
  for (int s = 0; s < nsys; s++) {
    NLStructHost &S = st_[s];
    std::memcpy(S.cell, cells + 9 * (size_t) s, sizeof(S.cell));
    double det;
    invert3(S.cell, S.inv, det);
    const double *a = S.cell;
    const double na = std::sqrt(a[0] * a[0] + a[1] * a[1] + a[2] * a[2]), nb = std::sqrt(a[3] * a[3] + a[4] * a[4] + a[5] * a[5]),
                 nc = std::sqrt(a[6] * a[6] + a[7] * a[7] + a[8] * a[8]);
    if (!std::isfinite(det) || !(std::fabs(det) > 1e-12 * na * nb * nc)) throw InvalidArgument("neighbour search needs a full-rank cell");
    for (int k = 0; k < 3; k++) {
      S.pbc[k] = pbc[3 * (size_t) s + k] != 0;
      heights[3 * (size_t) s + k] = 1.0 / std::sqrt(S.inv[k] * S.inv[k] + S.inv[3 + k] * S.inv[3 + k] + S.inv[6 + k] * S.inv[6 + k]);
      S.lo[k] = 0.0; S.span[k] = 1.0; S.nbin[k] = 1; S.reach[k] = 0; S.width[k] = 1.0;
    }
    if (natoms[s] < 0) throw InvalidArgument("negative atom count");
    S.atom0 = (int) at;
    at += natoms[s];
    S.atom1 = (int) at;
  }
  if (at != n) throw InvalidArgument("natoms does not sum to the atom count");
  {
    std::vector<int> seg(nsys + 1);
    for (int s = 0; s < nsys; s++) seg[s] = st_[s].atom0;
    seg[nsys] = (int) n;
    seg_.upload(seg);
  }
  flag_.ensure(1);
  GB_CUDA(cudaMemsetAsync(flag_.get(), 0, sizeof(int), dev().stream));
  off_.ensure(n + 1);
  cnt_.ensure(n + 1);
  if (n == 0) {
    GB_CUDA(cudaMemsetAsync(off_.get(), 0, sizeof(long long), dev().stream));
    n_ = 0;
    return;
  }
  d_st_.upload(st_);
  sid_.ensure(n);
  GB_LAUNCH(nl_fill_sid, nsys, 256, 0, sid_.get(), d_st_.get(), nsys);
  frac_.ensure(3 * n); img_.ensure(3 * n); xbuild_.ensure(3 * n);
  GB_LAUNCH(nl_frac, blocks(n, 256), 256, 0, d_pos, sid_.get(), d_st_.get(), frac_.get(), img_.get(), xbuild_.get(),
            flag_.get(), (long long) n);
  bool any_open = false;
  for (auto &S : st_) any_open = any_open || !S.pbc[0] || !S.pbc[1] || !S.pbc[2];
  std::vector<double> lohi;
  if (any_open) {
    lohi_.ensure(6 * (size_t) nsys);
    GB_LAUNCH(nl_minmax, nsys, 256, 0, frac_.get(), d_st_.get(), lohi_.get());
    lohi.resize(6 * (size_t) nsys);
    GB_CUDA(cudaMemcpyAsync(lohi.data(), lohi_.get(), lohi.size() * sizeof(double), cudaMemcpyDeviceToHost, dev().stream));
    GB_CUDA(cudaStreamSynchronize(dev().stream));
  }
  // bins of edge >= radius / 2 along each height (libgrace/include/grace/cell_list.h:96-105)
  const double bin_size = 0.5 * radius;
  int64_t nbins_total = 0;
  for (int s = 0; s < nsys; s++) {
    NLStructHost &S = st_[s];
    const int64_t ns = S.atom1 - S.atom0;
    for (int k = 0; k < 3; k++)
      if (!S.pbc[k] && ns > 0) {
        S.lo[k] = lohi[6 * (size_t) s + k];
        S.span[k] = std::max(lohi[6 * (size_t) s + 3 + k] - S.lo[k], 1e-12);
        if (!std::isfinite(S.span[k])) throw InvalidArgument("positions must be finite");
      }
    const int64_t max_bins = 8 * ns + 64;
    int64_t nb[3];
    for (int k = 0; k < 3; k++) {
      const double v = std::floor(S.span[k] * heights[3 * (size_t) s + k] / bin_size);
      nb[k] = (int64_t) std::min<double>(std::max(v, 1.0), (double) max_bins);
    }
    while ((double) nb[0] * (double) nb[1] * (double) nb[2] > (double) max_bins) {
      const int k = (int) (std::max_element(nb, nb + 3) - nb);
      nb[k] = std::max<int64_t>(1, nb[k] / 2);
    }
    for (int k = 0; k < 3; k++) {
      S.nbin[k] = (int) nb[k];
      S.width[k] = S.span[k] * heights[3 * (size_t) s + k] / (double) nb[k];
      const int64_t r = (int64_t) std::ceil(radius / S.width[k] - 1e-12);
      const int64_t rr = S.pbc[k] ? r : std::min<int64_t>(r, nb[k] - 1);
      if (rr > 120) throw InvalidArgument("the cell is too small for the cutoff (more than 120 periodic images per direction)");
      S.reach[k] = (int) rr;
    }
    if (nbins_total + nb[0] * nb[1] * nb[2] >= ((int64_t) 1 << 31)) throw InvalidArgument("too many neighbour-list bins");
    S.bin_base = (int) nbins_total;
    nbins_total += nb[0] * nb[1] * nb[2];
  }
  d_st_.upload(st_);
  binid_.ensure(n); count_.ensure(nbins_total); fill_.ensure(nbins_total);
  GB_CUDA(cudaMemsetAsync(count_.get(), 0, nbins_total * sizeof(int), dev().stream));
  GB_CUDA(cudaMemsetAsync(fill_.get(), 0, nbins_total * sizeof(int), dev().stream));
  GB_LAUNCH(nl_bin, blocks(n, 256), 256, 0, frac_.get(), sid_.get(), d_st_.get(), binid_.get(), count_.get(), (long long) n);
  start_.ensure(nbins_total + 1);
  scan_tmp_.ensure(std::max<int64_t>(nbins_total, n) / SCAN_TILE + 2);
  launch_scan(count_.get(), start_.get(), scan_tmp_.get(), nbins_total);
  members_.ensure(n); perm_.ensure(n);
  GB_LAUNCH(nl_place, blocks(n, 256), 256, 0, binid_.get(), start_.get(), fill_.get(), members_.get(), (long long) n);
  GB_LAUNCH(nl_order, blocks(n, 256), 256, 0, binid_.get(), start_.get(), members_.get(), perm_.get(), (long long) n);
  xs_.ensure(3 * n); mu_s_.ensure(n); sid_s_.ensure(n); b3_s_.ensure(3 * n); img_s_.ensure(3 * n);
  GB_LAUNCH(nl_sorted, blocks(n, 256), 256, 0, perm_.get(), frac_.get(), sid_.get(), d_mu, img_.get(), d_st_.get(),
            xs_.get(), mu_s_.get(), sid_s_.get(), b3_s_.get(), img_s_.get(), (long long) n);
  cnt_full_.ensure(n);
  const double rad2 = radius * radius;
  GB_LAUNCH((nl_neigh<false>), blocks(n, 128), 128, 0, xs_.get(), sid_s_.get(), b3_s_.get(), d_st_.get(), start_.get(),
            rad2, cnt_full_.get(), (const long long *) nullptr, (int *) nullptr, (int *) nullptr, flag_.get(), (long long) n);
  launch_scan(cnt_full_.get(), off_.get(), scan_tmp_.get(), n);
  long long total = 0;
  GB_CUDA(cudaMemcpyAsync(&total, off_.get() + n, sizeof(long long), cudaMemcpyDeviceToHost, dev().stream));
  GB_CUDA(cudaStreamSynchronize(dev().stream));
  if (total >= ((long long) 1 << 31)) throw Unsupported("more than 2^31 neighbour-list entries in one pass: use a smaller pass");
  nbr_j_.ensure(total); nbr_S_.ensure(total); rev_.ensure(total); cslot_.ensure(total); rec_.ensure(total);
  GB_LAUNCH((nl_neigh<true>), blocks(n, 128), 128, 0, xs_.get(), sid_s_.get(), b3_s_.get(), d_st_.get(), start_.get(),
            rad2, (int *) nullptr, (const long long *) off_.get(), nbr_j_.get(), nbr_S_.get(), flag_.get(), (long long) n);
  GB_LAUNCH(nl_reverse, blocks(n, 4), 128, 0, off_.get(), nbr_j_.get(), nbr_S_.get(), rev_.get(), flag_.get(), (long long) n);
  const int fl = read_flag(flag_.get());
  if (fl & 1) throw InvalidArgument("positions must be finite");
  if (fl & 2) throw InvalidArgument("two atoms at the same position (a bond of length 0): not a physical structure");
  if (fl & 4) throw DeviceError("neighbour list: a bond without its reverse bond");
  n_ = n;
  nslots_ = total;
}

namespace {

// a caller's padded neighbour table [nlocal][maxneigh] -> CSR slots; ghosts (i >= nlocal) have none
__global__ void __launch_bounds__(256) nl_adopt_counts(const int *__restrict__ numneigh, int nlocal, int maxneigh, int *cnt,
                                                       int *flag, long long nall)
{
  const long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nall) return;
  int c = 0;
  if (i < nlocal) {
    c = numneigh[i];
    if (c < 0 || c > maxneigh) { atomicOr(flag, 8); c = 0; }
  }
  cnt[i] = c;
}

__global__ void __launch_bounds__(128) nl_adopt_fill(const int *__restrict__ neighbors, int maxneigh,
                                                     const long long *__restrict__ off, int *nbr_j, int *nbr_S, int *rev,
                                                     int *flag, long long nlocal, long long nall)
{
  const long long i = (long long) blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  const int lane = threadIdx.x & 31;
  if (i >= nlocal) return;
  const long long base = off[i];
  const int c = (int) (off[i + 1] - base);
  for (int q = lane; q < c; q += 32) {
    int j = neighbors[i * maxneigh + q];
    if (j < 0 || j >= nall) { atomicOr(flag, 8); j = (int) i; }
    nbr_j[base + q] = j;
    nbr_S[base + q] = 0;      // ghosts are atoms of their own: no cell shift
    rev[base + q] = -1;       // no reverse bond: a ghost has no list
  }
}

__global__ void __launch_bounds__(256) nl_identity(int *perm, int *sid, int *img, long long n)
{
  const long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  perm[i] = (int) i;
  sid[i] = 0;
  img[3 * i] = img[3 * i + 1] = img[3 * i + 2] = 0;
}

}    // namespace

void NeighborList::adopt(int nlocal, int nall, const int *d_mu, const int *d_numneigh, const int *d_neighbors, int maxneigh)
{
  if (nlocal < 0 || nall < nlocal) throw InvalidArgument("nlocal must be in 0 .. nall");
  if (maxneigh < 0 || (nlocal > 0 && (!d_numneigh || (maxneigh > 0 && !d_neighbors)))) throw InvalidArgument("the neighbour table must be given");
  cudaStream_t st = dev().stream;
  const int64_t n = nall;
  nsys_ = 1;
  external_ = true;
  st_.assign(1, NLStructHost{});
  NLStructHost &S = st_[0];
  const double eye[9] = {1, 0, 0, 0, 1, 0, 0, 0, 1};
  std::memcpy(S.cell, eye, sizeof(eye));
  std::memcpy(S.inv, eye, sizeof(eye));
  for (int k = 0; k < 3; k++) { S.pbc[k] = 0; S.lo[k] = 0.0; S.span[k] = 1.0; S.nbin[k] = 1; S.reach[k] = 0; S.width[k] = 1.0; }
  S.bin_base = 0; S.atom0 = 0; S.atom1 = (int) n;
  d_st_.upload(st_);
  std::vector<int> seg = {0, (int) n};
  seg_.upload(seg);
  flag_.ensure(1);
  GB_CUDA(cudaMemsetAsync(flag_.get(), 0, sizeof(int), st));
  off_.ensure(n + 1);
  cnt_.ensure(n + 1);
  if (n == 0) {
    GB_CUDA(cudaMemsetAsync(off_.get(), 0, sizeof(long long), st));
    GB_CUDA(cudaStreamSynchronize(st));
    n_ = 0;
    nslots_ = 0;
    return;
  }
  perm_.ensure(n); sid_s_.ensure(n); img_s_.ensure(3 * n); mu_s_.ensure(n); xs_.ensure(3 * n); cnt_full_.ensure(n);
  scan_tmp_.ensure(n / 1024 + 64);
  GB_LAUNCH(nl_identity, blocks(n, 256), 256, 0, perm_.get(), sid_s_.get(), img_s_.get(), (long long) n);
  GB_CUDA(cudaMemcpyAsync(mu_s_.get(), d_mu, sizeof(int) * (size_t) n, cudaMemcpyDeviceToDevice, st));
  GB_LAUNCH(nl_adopt_counts, blocks(n, 256), 256, 0, d_numneigh, nlocal, maxneigh, cnt_full_.get(), flag_.get(), (long long) n);
  launch_scan(cnt_full_.get(), off_.get(), scan_tmp_.get(), n);
  long long total = 0;
  GB_CUDA(cudaMemcpyAsync(&total, off_.get() + n, sizeof(long long), cudaMemcpyDeviceToHost, st));
  GB_CUDA(cudaStreamSynchronize(st));    // also: the host vectors uploaded above
  if (total >= ((long long) 1 << 31)) throw Unsupported("more than 2^31 neighbour-list entries in one pass");
  const long long cap = std::max<long long>(total, 1);
  nbr_j_.ensure(cap); nbr_S_.ensure(cap); rev_.ensure(cap); cslot_.ensure(cap); rec_.ensure(cap);
  if (nlocal > 0)
    GB_LAUNCH(nl_adopt_fill, blocks(nlocal, 4), 128, 0, d_neighbors, maxneigh, off_.get(), nbr_j_.get(), nbr_S_.get(), rev_.get(),
              flag_.get(), (long long) nlocal, (long long) n);
  if (read_flag(flag_.get()) & 8) throw InvalidArgument("neighbour table: a count beyond maxneigh or an index outside the atoms");
  n_ = n;
  nslots_ = total;
}

bool NeighborList::moved_beyond(const double *d_pos, double half_skin)
{
  if (n_ == 0) return false;
  GB_CUDA(cudaMemsetAsync(flag_.get(), 0, sizeof(int), dev().stream));
  GB_LAUNCH(nl_moved, blocks(n_, 256), 256, 0, d_pos, xbuild_.get(), half_skin * half_skin, flag_.get(), 1, (long long) n_);
  return read_flag(flag_.get()) != 0;
}

void NeighborList::moved_launch(const double *d_pos, double half_skin, int *d_flag, int bit)
{
  if (n_ == 0) return;
  GB_LAUNCH(nl_moved, blocks(n_, 256), 256, 0, d_pos, xbuild_.get(), half_skin * half_skin, d_flag, bit, (long long) n_);
}

void NeighborList::prepare(const double *d_pos, const double *d_rcsq, int n_elements, float *fv)
{
  if (n_ == 0) return;
  GB_CUDA(cudaMemsetAsync(flag_.get(), 0, sizeof(int), dev().stream));
  GB_LAUNCH(nl_positions, blocks(n_, 256), 256, 0, d_pos, perm_.get(), img_s_.get(), sid_s_.get(), d_st_.get(), xs_.get(),
            (long long) n_);
  GB_LAUNCH(nl_compact, blocks(n_, 4), 128, 0, xs_.get(), mu_s_.get(), sid_s_.get(), d_st_.get(), off_.get(),
            nbr_j_.get(), nbr_S_.get(), d_rcsq, n_elements, rec_.get(), cslot_.get(), cnt_.get(), fv, flag_.get(),
            (long long) n_);
}

int NeighborList::take_flag() { return n_ > 0 ? read_flag(flag_.get()) : 0; }

BondsDev NeighborList::bonds() const
{
  BondsDev b;
  b.off = off_.get();
  b.cnt = cnt_.get();
  b.rec = rec_.get();
  b.cslot = cslot_.get();
  b.mu = mu_s_.get();
  b.ilist = nullptr;
  return b;
}

void NeighborList::export_host(std::vector<int> &bi, std::vector<int> &bj, std::vector<int> &bS) const
{
  bi.clear(); bj.clear(); bS.clear();
  if (n_ == 0 || nslots_ == 0) return;
  cudaStream_t st = dev().stream;
  std::vector<long long> off((size_t) n_ + 1);
  std::vector<int> j((size_t) nslots_), S((size_t) nslots_), perm((size_t) n_), img(3 * (size_t) n_);
  GB_CUDA(cudaMemcpyAsync(off.data(), off_.get(), sizeof(long long) * off.size(), cudaMemcpyDeviceToHost, st));
  GB_CUDA(cudaMemcpyAsync(j.data(), nbr_j_.get(), sizeof(int) * j.size(), cudaMemcpyDeviceToHost, st));
  GB_CUDA(cudaMemcpyAsync(S.data(), nbr_S_.get(), sizeof(int) * S.size(), cudaMemcpyDeviceToHost, st));
  GB_CUDA(cudaMemcpyAsync(perm.data(), perm_.get(), sizeof(int) * perm.size(), cudaMemcpyDeviceToHost, st));
  GB_CUDA(cudaMemcpyAsync(img.data(), img_s_.get(), sizeof(int) * img.size(), cudaMemcpyDeviceToHost, st));
  GB_CUDA(cudaStreamSynchronize(st));
  bi.reserve((size_t) nslots_); bj.reserve((size_t) nslots_); bS.reserve(3 * (size_t) nslots_);
  for (int64_t q = 0; q < n_; q++)
    for (long long e = off[(size_t) q]; e < off[(size_t) q + 1]; e++) {
      const int p = j[(size_t) e];
      bi.push_back(perm[(size_t) q]);
      bj.push_back(perm[(size_t) p]);
      // the list holds wrapped positions x - img cell: back in the caller's frame the shift is S - img_j + img_i
      for (int k = 0; k < 3; k++) {
        const int sk = (int) (signed char) ((S[(size_t) e] >> (8 * k)) & 0xff);
        bS.push_back(sk - img[3 * (size_t) p + k] + img[3 * (size_t) q + k]);
      }
    }
}

void NeighborList::release()
{
  frac_.release(); xs_.release(); xbuild_.release(); lohi_.release(); img_.release(); img_s_.release();
  sid_.release(); sid_s_.release(); binid_.release(); b3_s_.release(); count_.release(); fill_.release();
  members_.release(); perm_.release(); mu_s_.release(); cnt_full_.release(); cnt_.release(); nbr_j_.release();
  nbr_S_.release(); rev_.release(); cslot_.release(); seg_.release(); start_.release(); off_.release();
  scan_tmp_.release(); rec_.release(); d_st_.release(); flag_.release();
  n_ = 0;
  nslots_ = 0;
  external_ = false;
}

size_t NeighborList::bytes() const
{
  return (size_t) nslots_ * (4 * sizeof(int) + sizeof(float4)) + (size_t) n_ * 200;
}

}    // namespace gb
