// Shared device code of the bond kernels: real spherical harmonics with the gradient of their polynomial extension,
// and the cubic Hermite evaluation of the radial functions.
#pragma once

#include "kernels.h"

namespace gb {

// recurrence coefficients of the real spherical harmonics for l <= 4, set once per process by
// bond_tables_init(): a, b indexed l (l + 1) / 2 + m, c and d indexed l (libgrace/include/grace/fused_cpu.h:686-702)
struct SHTable {
  float a[15], b[15], c[5], d[5];
};
const SHTable &sh_table_host();

// Y[lm] (and G[lm] = dY/d(x, y, z) of the polynomial extension) of the unit vector (rx, ry, rz); Y00 = 1,
// lm = l (l + 1) + m (libgrace/include/grace/fused_cpu.h:711-798).  Out: a functor out(lm, y, gx, gy, gz).
template<int LMAX, bool GRAD, class Out>
__device__ __forceinline__ void sph_harm(const SHTable &t, float rx, float ry, float rz, Out out)
{
  constexpr int NP = (LMAX + 1) * (LMAX + 2) / 2;
  float plm[NP], dplm[NP];
  plm[0] = 1.0f;
  dplm[0] = 0.0f;
  if (LMAX > 0) {
    plm[1] = 1.7320508075688772f * rz;
    dplm[1] = 1.7320508075688772f;
    plm[2] = -1.224744871391589f;
    dplm[2] = 0.0f;
  }
#pragma unroll
  for (int l = 2; l <= LMAX; l++) {
#pragma unroll
    for (int mm = 0; mm < l - 1; mm++) {
      const int id = l * (l + 1) / 2 + mm, i1 = (l - 1) * l / 2 + mm, i2 = (l - 2) * (l - 1) / 2 + mm;
      plm[id] = t.a[id] * (rz * plm[i1] + t.b[id] * plm[i2]);
      dplm[id] = t.a[id] * (plm[i1] + rz * dplm[i1] + t.b[id] * dplm[i2]);
    }
    const int prev = (l - 1) * l / 2 + l - 1, i0 = l * (l + 1) / 2 + l - 1, i1 = l * (l + 1) / 2 + l;
    plm[i0] = t.d[l] * plm[prev] * rz;
    plm[i1] = t.c[l] * plm[prev];
    dplm[i0] = t.d[l] * (dplm[prev] * rz + plm[prev]);
    dplm[i1] = t.c[l] * dplm[prev];
  }
  const float sq2 = 1.4142135623730951f;
#pragma unroll
  for (int l = 0; l <= LMAX; l++) {
    const int c = l * (l + 1), p0 = l * (l + 1) / 2;
    out(c, plm[p0], 0.0f, 0.0f, dplm[p0]);
    float pr = rx, pi = ry, prx = 1.0f, pry = 0.0f, pix = 0.0f, piy = 1.0f;
#pragma unroll
    for (int mm = 1; mm <= l; mm++) {
      const float sg = (mm % 2 == 0) ? sq2 : -sq2;
      const float pv = plm[p0 + mm], dpv = dplm[p0 + mm];
      out(c + mm, sg * pr * pv, sg * prx * pv, sg * pry * pv, sg * pr * dpv);
      out(c - mm, sg * pi * pv, sg * pix * pv, sg * piy * pv, sg * pi * dpv);
      if (GRAD) {
        const float nrx = prx * rx + pr - pix * ry, nry = pry * rx - piy * ry - pi;
        const float nix = prx * ry + pix * rx + pi, niy = pry * ry + pr + piy * rx;
        prx = nrx; pry = nry; pix = nix; piy = niy;
      }
      const float nr = pr * rx - pi * ry, ni = pr * ry + pi * rx;
      pr = nr; pi = ni;
    }
  }
}

// Sums of four per-lane values over the groups of G consecutive lanes of a warp (G = 8, 16 or 32) with 1 + log2(G)
// shuffles instead of 4 log2(G): the halves of a group first trade two of the values, the quarters one, and from then
// on every lane carries a single value.  Afterwards lane q G / 4 of a group (q = 0 .. 3) holds the sum of value q in
// `out`; the additions pair the same lanes as a butterfly per value, so the sums are bit-identical to it.
template<int G>
__device__ __forceinline__ float group_sum4(float v0, float v1, float v2, float v3, int lane_in_group)
{
  const bool up = lane_in_group & (G / 2), odd = lane_in_group & (G / 4);
  const float r0 = __shfl_xor_sync(0xffffffffu, up ? v0 : v2, G / 2), r1 = __shfl_xor_sync(0xffffffffu, up ? v1 : v3, G / 2);
  const float k0 = (up ? v2 : v0) + r0, k1 = (up ? v3 : v1) + r1;
  float v = (odd ? k1 : k0) + __shfl_xor_sync(0xffffffffu, odd ? k0 : k1, G / 4);
#pragma unroll
  for (int s = G / 8; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  return v;
}

// interval k and offset t of x = r / rcut in a table of N intervals (libgrace/include/grace/fused_cpu.h:1052-1058)
__device__ __forceinline__ void spline_locate(float x, int N, int &k, float &t)
{
  const float s = x * (float) N;
  k = (int) s;
  if (k > N - 1) k = N - 1;
  if (k < 0) k = 0;
  t = s - (float) k;
}

}    // namespace gb
