// Kernels of the dense per-atom network (FC, Clebsch-Gordan products, reduces and their adjoints as two table-driven
// kernels), the fp64 readouts, and the per-atom gathers and sums that leave the network.
// Mathematics: libgrace/include/grace/fused_cpu.h:349-364 (FC), 411-453 (products), 637-649 (reduces);
// libgrace/src/fused_1l.cpp:378-427 and libgrace/src/fused_2l.cpp:548-615 (readouts).
#include "kernels.h"
#include "readout.cuh"

#include <algorithm>
#include <cstdint>
#include <cstdlib>

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

// Per-element weights (reduces over the central atom's element and their adjoints) for a tile of 128 atoms, one thread
// per atom with all NQ x 4 output channels of a row in registers.  The atoms of the tile are taken in order of their
// element, so the lanes of a warp mostly read the same weights (one broadcast shared-memory read serves them).  A CTA
// walks the (row, item) pairs of its rows in groups of G items; the weight matrices of a group, for the elements
// present in the tile, are staged in shared memory together - a weight is fetched from global memory once per tile and
// element - through asynchronous copies into the half of a double buffer that the group before is not reading: the
// fetch of a group runs under the arithmetic of the previous one and a group costs one barrier.  Same summation order
// as mv_kernel.
constexpr int ELEM_MAXS = 4;    // elements staged at a time (tiles with more walk the items once more per group of elements)
constexpr int ELEM_GROUP = 4;   // most items whose weights are staged together
constexpr int ELEM_TA = 128;

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gmem_src)
{
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned) __cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

template<int NQ>
__global__ void __launch_bounds__(ELEM_TA) mv_elem_tile_kernel(MVDev op, const TensorDev *__restrict__ T,
                                                               const int *__restrict__ mu, int NA, int na, int n_in_max,
                                                               int rows_per_cta, int G)
{
  extern __shared__ __align__(16) float wsm[];    // [2][G][ELEM_MAXS][n_in_max][NQ * 4]
  __shared__ int s_slot[ELEM_TA], s_el[ELEM_TA], s_mu[ELEM_TA], s_order[ELEM_TA], s_cnt[ELEM_TA + 1], s_nsp;
  const int a0 = blockIdx.x * ELEM_TA, nta = min(ELEM_TA, na - a0), t = threadIdx.x;
  const int row_lo = blockIdx.y * rows_per_cta, row_hi = min(op.nrows, row_lo + rows_per_cta);
  if (t < nta) s_mu[t] = mu[a0 + t];
  __syncthreads();
  if (t == 0) {    // distinct elements of the tile in order of first appearance, and the atoms grouped by them
    int ns = 0;
    for (int a = 0; a < nta; a++) {
      const int e = s_mu[a];
      int s = 0;
      while (s < ns && s_el[s] != e) s++;
      if (s == ns) { s_el[ns] = e; s_cnt[ns++] = 0; }
      s_slot[a] = s;
      s_cnt[s]++;
    }
    int at = 0;
    for (int s = 0; s < ns; s++) { const int c = s_cnt[s]; s_cnt[s] = at; at += c; }
    for (int a = 0; a < nta; a++) s_order[s_cnt[s_slot[a]]++] = a;
    s_nsp = ns;
  }
  __syncthreads();
  const bool active = t < nta;
  const int p = active ? s_order[t] : 0;    // this thread's atom of the tile
  const int nsp = s_nsp, slot = active ? s_slot[p] : -1;
  const int i_lo = op.item_off[row_lo], i_hi = op.item_off[row_hi];
  const int wstride = n_in_max * NQ;                      // float4 per (item of the group, element)
  const int bstride = G * ELEM_MAXS * wstride;            // float4 per buffer
  float4 *const w4 = reinterpret_cast<float4 *>(wsm);
  const TensorDev dst = T[op.dst];
  for (int s0 = 0; s0 < nsp; s0 += ELEM_MAXS) {
    const int ng = min(ELEM_MAXS, nsp - s0);
    const bool mine = slot >= s0 && slot < s0 + ng;
    int row = row_lo;
    float4 acc[NQ];
#pragma unroll
    for (int k = 0; k < NQ; k++) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    auto flush = [&]() {    // the sums of `row` are complete
      if (mine) {
        float *o = dst.p + ((size_t) op.row_out[row] * NA + a0 + p) * dst.C;
        if ((dst.C & 3) == 0 && op.n_out == 4 * NQ) {
#pragma unroll
          for (int k = 0; k < NQ; k++) {
            float4 v = acc[k];
            if (op.accumulate) {
              const float4 old = reinterpret_cast<const float4 *>(o)[k];
              v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
            }
            reinterpret_cast<float4 *>(o)[k] = v;
          }
        } else {
#pragma unroll
          for (int k = 0; k < NQ; k++) {
            const float v[4] = {acc[k].x, acc[k].y, acc[k].z, acc[k].w};
            for (int q = 0; q < 4; q++)
              if (4 * k + q < op.n_out) o[4 * k + q] = op.accumulate ? o[4 * k + q] + v[q] : v[q];
          }
        }
      }
#pragma unroll
      for (int k = 0; k < NQ; k++) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      row++;
    };
    // asynchronous copies of the weights of the items it0 .. it0 + G of the elements s0 .. s0 + ng into buffer `buf`
    auto stage = [&](int it0, int buf) {
      const int nit = min(G, i_hi - it0);
      for (int g = 0; g < nit; g++) {
        const MVItem item = op.items[it0 + g];
        const int per = item.n_in * NQ;
        for (int q = t; q < ng * per; q += ELEM_TA) {
          const int s = q / per, r = q - s * per;
          cp_async16(w4 + (size_t) buf * bstride + (size_t) (g * ELEM_MAXS + s) * wstride + r,
                     reinterpret_cast<const float4 *>(op.W + (size_t) s_el[s0 + s] * op.ty_stride + item.mat) + r);
        }
      }
      cp_async_commit();
    };
    __syncthreads();    // the buffers of the previous group of elements are no longer read
    if (i_lo < i_hi) stage(i_lo, 0);
    int buf = 0;
    for (int it0 = i_lo; it0 < i_hi; it0 += G, buf ^= 1) {
      const int nit = min(G, i_hi - it0);
      cp_async_wait_all();
      __syncthreads();    // this group's weights are in place; the other buffer's readers are done
      if (it0 + G < i_hi) stage(it0 + G, buf ^ 1);
      for (int g = 0; g < nit; g++) {
        while (it0 + g >= op.item_off[row + 1]) flush();
        if (!mine) continue;
        const MVItem item = op.items[it0 + g];
        const TensorDev src = T[item.src];
        const float *x = src.p + ((size_t) item.irow * NA + a0 + p) * src.C;
        const float4 *w = w4 + (size_t) buf * bstride + (size_t) (g * ELEM_MAXS + slot - s0) * wstride;
        float4 part[NQ];
#pragma unroll
        for (int k = 0; k < NQ; k++) part[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        auto one = [&](float xv, int n) {
#pragma unroll
          for (int k = 0; k < NQ; k++) {
            const float4 wv = w[(size_t) n * NQ + k];
            part[k].x = fmaf(xv, wv.x, part[k].x); part[k].y = fmaf(xv, wv.y, part[k].y);
            part[k].z = fmaf(xv, wv.z, part[k].z); part[k].w = fmaf(xv, wv.w, part[k].w);
          }
        };
        if (((src.C | item.n_in) & 3) == 0) {    // 16-byte activation loads, eight of them in flight
          for (int n0 = 0; n0 < item.n_in; n0 += 32) {
            float4 xv[8];
#pragma unroll
            for (int j = 0; j < 8; j++)
              xv[j] = n0 + 4 * j < item.n_in ? __ldg(reinterpret_cast<const float4 *>(x + n0) + j) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 8; j++) {
              if (n0 + 4 * j < item.n_in) {
                one(xv[j].x, n0 + 4 * j); one(xv[j].y, n0 + 4 * j + 1); one(xv[j].z, n0 + 4 * j + 2); one(xv[j].w, n0 + 4 * j + 3);
              }
            }
          }
        } else {
          for (int n = 0; n < item.n_in; n++) one(__ldg(x + n), n);
        }
#pragma unroll
        for (int k = 0; k < NQ; k++) {
          acc[k].x = fmaf(item.scale, part[k].x, acc[k].x); acc[k].y = fmaf(item.scale, part[k].y, acc[k].y);
          acc[k].z = fmaf(item.scale, part[k].z, acc[k].z); acc[k].w = fmaf(item.scale, part[k].w, acc[k].w);
        }
      }
    }
    while (row < row_hi) flush();    // the last row, and rows without items
  }
}

template<int NQ> void launch_elem(const MVDev &op, const TensorDev *tensors, const int *mu, int NA, int na)
{
  // items per group: both halves of the double buffer within ~56 KB, so that several CTAs share an SM
  const size_t per_item = (size_t) ELEM_MAXS * op.unit_nmax * op.ldw * sizeof(float);
  int G = ELEM_GROUP;
  while (G > 1 && 2 * G * per_item > 56 * 1024) G--;
  const size_t smem = 2 * G * per_item;
  static size_t attr = 32 * 1024;    // static shared memory counts against the 48 KB a kernel gets without the attribute
  if (smem > attr) {
    GB_CUDA(cudaFuncSetAttribute(mv_elem_tile_kernel<NQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr = 200 * 1024;
  }
  // rows of a tile go to one CTA unless the tiles alone cannot fill the GPU
  const int tiles = (na + ELEM_TA - 1) / ELEM_TA, want = 16 * dev().sm_count;
  const int gy = std::max(1, std::min(op.nrows, (want + tiles - 1) / tiles));
  const int rows_per_cta = (op.nrows + gy - 1) / gy;
  GB_LAUNCH((mv_elem_tile_kernel<NQ>), dim3(tiles, (op.nrows + rows_per_cta - 1) / rows_per_cta), ELEM_TA, smem, op, tensors, mu,
            NA, na, op.unit_nmax, rows_per_cta, G);
}

// Per-element weights with wide outputs (the adjoints of the reduces: 9 - 17 inputs, 32 or 64 outputs per row): LPA =
// n_out / 4 lanes per atom, each with one float4 of the output row, so that a row of an atom is written (and, when the
// operation accumulates, read) as whole 128-byte lines; 32 / LPA atoms per warp, 8 warps per CTA, tiles of 128 atoms.
// The weights of a group of output rows, for the elements present in the tile, are staged in shared memory; the inputs
// of an atom are broadcast loads shared by its lanes.  Same summation order as mv_kernel.
template<int LPA>
__global__ void __launch_bounds__(256) mv_elem_wide_kernel(MVDev op, const TensorDev *__restrict__ T,
                                                           const int *__restrict__ mu, int NA, int na, int n_in_max,
                                                           int rows_per_cta, int G)
{
  constexpr int APW = 32 / LPA, APP = 8 * APW;    // atoms per warp and per pass of the CTA
  extern __shared__ __align__(16) float wsm[];    // [G][ELEM_MAXS][n_in_max][LPA * 4]
  __shared__ int s_slot[ELEM_TA], s_el[ELEM_TA], s_mu[ELEM_TA], s_nsp;
  const int a0 = blockIdx.x * ELEM_TA, nta = min(ELEM_TA, na - a0), t = threadIdx.x;
  const int row_lo = blockIdx.y * rows_per_cta, row_hi = min(op.nrows, row_lo + rows_per_cta);
  if (t < nta) s_mu[t] = mu[a0 + t];
  __syncthreads();
  if (t == 0) {    // distinct elements of the tile in order of first appearance
    int ns = 0;
    for (int a = 0; a < nta; a++) {
      const int e = s_mu[a];
      int s = 0;
      while (s < ns && s_el[s] != e) s++;
      if (s == ns) s_el[ns++] = e;
      s_slot[a] = s;
    }
    s_nsp = ns;
  }
  __syncthreads();
  const int lane = t & 31, warp = t >> 5, kq = lane % LPA, asub = lane / LPA;
  const int nsp = s_nsp, wstride = n_in_max * LPA;    // float4 per (item of the group, element)
  float4 *const w4 = reinterpret_cast<float4 *>(wsm);
  const TensorDev dst = T[op.dst];
  for (int s0 = 0; s0 < nsp; s0 += ELEM_MAXS) {
    const int ng = min(ELEM_MAXS, nsp - s0);
    for (int r0 = row_lo; r0 < row_hi;) {
      const int i_first = op.item_off[r0];
      int r1 = r0 + 1;    // rows of the group: at most G items (a single row never has more: checked by the launcher)
      while (r1 < row_hi && op.item_off[r1 + 1] - i_first <= G) r1++;
      const int nit = op.item_off[r1] - i_first;
      __syncthreads();    // the weights of the previous group are no longer read
      for (int g = 0; g < nit; g++) {
        const MVItem item = op.items[i_first + g];
        const int per = item.n_in * LPA;
        for (int q = t; q < ng * per; q += 256) {
          const int s = q / per, r = q - s * per;
          w4[(size_t) (g * ELEM_MAXS + s) * wstride + r] =
              __ldg(reinterpret_cast<const float4 *>(op.W + (size_t) s_el[s0 + s] * op.ty_stride + item.mat) + r);
        }
      }
      __syncthreads();
      for (int ab = 0; ab < nta; ab += APP) {
        const int ai = ab + warp * APW + asub;
        if (ai >= nta) continue;
        const int slot = s_slot[ai];
        if (slot < s0 || slot >= s0 + ng) continue;
        for (int row = r0; row < r1; row++) {
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int it = op.item_off[row]; it < op.item_off[row + 1]; it++) {
            const MVItem item = op.items[it];
            const TensorDev src = T[item.src];
            const float *x = src.p + ((size_t) item.irow * NA + a0 + ai) * src.C;
            const float4 *w = w4 + (size_t) ((it - i_first) * ELEM_MAXS + slot - s0) * wstride + kq;
            float4 part = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int n = 0; n < item.n_in; n++) {
              const float xv = __ldg(x + n);
              const float4 wv = w[(size_t) n * LPA];
              part.x = fmaf(xv, wv.x, part.x); part.y = fmaf(xv, wv.y, part.y);
              part.z = fmaf(xv, wv.z, part.z); part.w = fmaf(xv, wv.w, part.w);
            }
            acc.x = fmaf(item.scale, part.x, acc.x); acc.y = fmaf(item.scale, part.y, acc.y);
            acc.z = fmaf(item.scale, part.z, acc.z); acc.w = fmaf(item.scale, part.w, acc.w);
          }
          float4 *o = reinterpret_cast<float4 *>(dst.p + ((size_t) op.row_out[row] * NA + a0 + ai) * dst.C) + kq;
          if (op.accumulate) {
            const float4 old = *o;
            acc.x += old.x; acc.y += old.y; acc.z += old.z; acc.w += old.w;
          }
          *o = acc;
        }
      }
      r0 = r1;
    }
  }
}

template<int LPA> bool launch_elem_wide(const MVDev &op, const TensorDev *tensors, const int *mu, int NA, int na)
{
  const size_t per_item = (size_t) ELEM_MAXS * op.unit_nmax * op.ldw * sizeof(float);
  const int G = (int) std::min<size_t>(16, (40 * 1024) / per_item);
  if (G < 1 || op.max_row_items > G) return false;
  const size_t smem = G * per_item;
  const int tiles = (na + ELEM_TA - 1) / ELEM_TA, want = 8 * dev().sm_count;
  const int gy = std::max(1, std::min(op.nrows, (want + tiles - 1) / tiles));
  const int rows_per_cta = (op.nrows + gy - 1) / gy;
  GB_LAUNCH((mv_elem_wide_kernel<LPA>), dim3(tiles, (op.nrows + rows_per_cta - 1) / rows_per_cta), 256, smem, op, tensors, mu, NA,
            na, op.unit_nmax, rows_per_cta, G);
  return true;
}

void launch_mv(const MVDev &op, const TensorDev *tensors, const int *mu, int NA, int na)
{
  if (op.nrows == 0 || na == 0) return;
  // wide per-element operations (adjoints of the reduces): channel-parallel form with whole-line stores
  static const bool nowide = getenv("GRACE_B200_ELEM_NOWIDE") != nullptr;
  if (!nowide && op.elem && op.ldw == op.n_out && op.dst_C == op.n_out && (op.ty_stride & 3) == 0 && op.unit_nmax > 0 &&
      op.unit_nmax <= 20) {
    if (op.n_out == 32 && launch_elem_wide<8>(op, tensors, mu, NA, na)) return;
    if (op.n_out == 64 && launch_elem_wide<16>(op, tensors, mu, NA, na)) return;
  }
  if (op.elem && (op.ldw & 3) == 0 && (op.ty_stride & 3) == 0 && op.unit_nmax > 0 &&
      (size_t) 2 * ELEM_MAXS * op.unit_nmax * op.ldw * sizeof(float) <= 192 * 1024) {
    switch (op.ldw >> 2) {
      case 1: launch_elem<1>(op, tensors, mu, NA, na); return;
      case 2: launch_elem<2>(op, tensors, mu, NA, na); return;
      case 3: launch_elem<3>(op, tensors, mu, NA, na); return;
      case 4: launch_elem<4>(op, tensors, mu, NA, na); return;
      case 5: launch_elem<5>(op, tensors, mu, NA, na); return;
      case 8: launch_elem<8>(op, tensors, mu, NA, na); return;
      case 12: launch_elem<12>(op, tensors, mu, NA, na); return;
      case 16: launch_elem<16>(op, tensors, mu, NA, na); return;
      default: break;    // other widths: the per-atom kernel below
    }
  }
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
  *o = (op.accumulate && !(op.row_first && op.row_first[row])) ? *o + acc : acc;
}

// The same for a tile of TA atoms with the input rows staged in shared memory: every input value comes from global
// memory once (coalesced, TA x C contiguous floats per function) however many terms read it, and the term loop runs on
// shared memory.  srcB == srcA or srcB < 0: one staged tensor.
__global__ void __launch_bounds__(256) prod_tile_kernel(ProdDev op, const TensorDev *__restrict__ T, int NA, int na, int TA,
                                                        int nfA, int nfB, int C, int nterms)
{
  extern __shared__ __align__(16) float psm[];
  const int C4 = C >> 2, TAC4 = TA * C4, t = threadIdx.x;
  const int a0 = blockIdx.x * TA, nta = min(TA, na - a0);
  float4 *sA = reinterpret_cast<float4 *>(psm);
  float4 *sB = sA + (size_t) nfA * TAC4;
  int4 *sT = reinterpret_cast<int4 *>(sB + (size_t) nfB * TAC4);    // per term: row offsets of both operands, coefficient
  const bool two = op.srcB >= 0 && op.srcB != op.srcA;
  {
    // eight independent 16-byte loads per thread in flight: the tile's rows come from nf separate regions of the
    // tensor, and a CTA has nothing else to do until they are there
    auto stage = [&](const float *G, float4 *S, int nf) {
      const int total = nf * TAC4;
      for (int base = 0; base < total; base += 256 * 8) {
        float4 v[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const int idx = base + j * 256 + t, f = idx / TAC4, r = idx - f * TAC4;
          v[j] = (idx < total && r / C4 < nta) ? __ldg(reinterpret_cast<const float4 *>(G + ((size_t) f * NA + a0) * C) + r)
                                               : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const int idx = base + j * 256 + t;
          if (idx < total) S[idx] = v[j];
        }
      }
    };
    stage(T[op.srcA].p, sA, nfA);
    if (two) stage(T[op.srcB].p, sB, nfB);
    for (int idx = t; idx < nterms; idx += 256) {
      const ProdTerm tm = op.terms[idx];
      sT[idx] = make_int4(tm.a * TAC4, tm.b * TAC4, __float_as_int(tm.coef), 0);
    }
  }
  __syncthreads();
  const float4 *Bs = op.srcB < 0 ? nullptr : (two ? sB : sA);
  float *D = T[op.dst].p;
  const int nvalid = nta * C4, warp = t >> 5, lane = t & 31;
  // a warp takes an output row and walks its TA x C values 64 float4 at a time, two per lane, so that a term (one
  // broadcast 16-byte read) serves two positions; the products are packed two-wide FMAs (the same roundings as
  // fmaf(coef * a, b, acc) per channel)
  auto f2 = [](float x, float y) { return make_float2(x, y); };
  for (int row = warp; row < op.nrows; row += 8) {
    const int t0 = op.term_off[row], t1 = op.term_off[row + 1];
    const bool add = op.accumulate && !(op.row_first && op.row_first[row]);
    float4 *orow = reinterpret_cast<float4 *>(D + ((size_t) op.row_out[row] * NA + a0) * C);
    for (int r = lane; r < nvalid; r += 64) {
      const bool has1 = r + 32 < nvalid;
      const int r1 = has1 ? r + 32 : r;
      float2 a0l = f2(0.f, 0.f), a0h = a0l, a1l = a0l, a1h = a0l;
      if (Bs) {
        for (int q = t0; q < t1; q++) {
          const int4 tm = sT[q];
          const float cf = __int_as_float(tm.z);
          const float2 c2 = f2(cf, cf);
          const float4 av0 = sA[tm.x + r], bv0 = Bs[tm.y + r], av1 = sA[tm.x + r1], bv1 = Bs[tm.y + r1];
          a0l = __ffma2_rn(__fmul2_rn(c2, f2(av0.x, av0.y)), f2(bv0.x, bv0.y), a0l);
          a0h = __ffma2_rn(__fmul2_rn(c2, f2(av0.z, av0.w)), f2(bv0.z, bv0.w), a0h);
          a1l = __ffma2_rn(__fmul2_rn(c2, f2(av1.x, av1.y)), f2(bv1.x, bv1.y), a1l);
          a1h = __ffma2_rn(__fmul2_rn(c2, f2(av1.z, av1.w)), f2(bv1.z, bv1.w), a1h);
        }
      } else {
        for (int q = t0; q < t1; q++) {
          const int4 tm = sT[q];
          const float cf = __int_as_float(tm.z);
          const float2 c2 = f2(cf, cf);
          const float4 av0 = sA[tm.x + r], av1 = sA[tm.x + r1];
          a0l = __ffma2_rn(c2, f2(av0.x, av0.y), a0l);
          a0h = __ffma2_rn(c2, f2(av0.z, av0.w), a0h);
          a1l = __ffma2_rn(c2, f2(av1.x, av1.y), a1l);
          a1h = __ffma2_rn(c2, f2(av1.z, av1.w), a1h);
        }
      }
      float4 o0 = make_float4(a0l.x, a0l.y, a0h.x, a0h.y), o1 = make_float4(a1l.x, a1l.y, a1h.x, a1h.y);
      if (add) {
        const float4 old0 = orow[r], old1 = orow[r1];
        o0.x += old0.x; o0.y += old0.y; o0.z += old0.z; o0.w += old0.w;
        o1.x += old1.x; o1.y += old1.y; o1.z += old1.z; o1.w += old1.w;
      }
      orow[r] = o0;
      if (has1) orow[r1] = o1;
    }
  }
}

void launch_prod(const ProdDev &op, const TensorDev *tensors, int NA, int na, int C, int nfA, int nfB, int nterms)
{
  if (op.nrows == 0 || na == 0) return;
  // tiled form: channels a multiple of 4 and at least one atom of input rows in shared memory
  if ((C & 3) == 0 && nfA > 0) {
    const bool two = op.srcB >= 0 && op.srcB != op.srcA;
    const size_t per_atom = (size_t) (nfA + (two ? nfB : 0)) * C * 4, fixed = (size_t) nterms * sizeof(int4) + 64;
    // several CTAs per SM (the load, compute and store phases of a tile overlap only across CTAs): a quarter of the
    // shared memory when that holds 4+ atoms, else half, else all of it
    static const size_t first = getenv("GRACE_B200_PROD_KB") ? (size_t) atoi(getenv("GRACE_B200_PROD_KB")) * 1024 : 54 * 1024;
    const size_t quarter = first, half = 110 * 1024, large = 200 * 1024;
    size_t budget = quarter;
    if (fixed + 4 * per_atom > quarter) budget = half;
    if (fixed + 4 * per_atom > half) budget = large;
    int TA = fixed < budget ? (int) std::min<size_t>(32, (budget - fixed) / per_atom) : 0;
    {    // a warp walks a row 64 float4 at a time: tiles whose rows are a multiple of that leave no lane idle
      const int unit = std::max(1, 64 / (C >> 2));
      if (TA > unit) TA = TA / unit * unit;
    }
    if (TA >= 1) {
      const size_t smem = fixed + (size_t) TA * per_atom;
      static size_t attr = 48 * 1024;
      if (smem > attr) {
        GB_CUDA(cudaFuncSetAttribute(prod_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) large));
        attr = large;
      }
      GB_LAUNCH(prod_tile_kernel, (na + TA - 1) / TA, 256, smem, op, tensors, NA, na, TA, nfA, two ? nfB : 0, C, nterms);
      return;
    }
  }
  const long long row_len = (long long) NA * C, act_len = (long long) na * C;
  const dim3 grid(op.nrows, (unsigned) ((act_len + 255) / 256));
  GB_LAUNCH(prod_kernel, grid, 256, 0, op, tensors, row_len, act_len);
}

// ---- readouts (fp64, one thread per atom) ---------------------------------------------------------------------
__global__ void __launch_bounds__(64) readout_1l_kernel(ReadoutDev r, const float *__restrict__ rho, float *grho,
                                                        const int *__restrict__ mu, double *e_atom, int NA, int na,
                                                        int a0, int want_grad, const int *__restrict__ ilist)
{
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= na) return;
  const int i = ilist ? ilist[a0 + a] : a0 + a;    // the atom of chunk position a
  e_atom[i] = readout_1l_atom(r, rho + (size_t) a * r.nrho, mu[i], grho + (size_t) a * r.nrho, want_grad, r.owned(i));
}

void launch_readout_1l(const ReadoutDev &r, const float *rho, float *grho, const int *mu, double *e_atom, int NA,
                       int na, int a0, int want_grad, const int *ilist)
{
  if (na == 0) return;
  GB_LAUNCH(readout_1l_kernel, (na + 63) / 64, 64, 0, r, rho, grho, mu, e_atom, NA, na, a0, want_grad, ilist);
}

__global__ void __launch_bounds__(64) readout_2l_kernel(ReadoutDev r, const float *__restrict__ rho_rows,
                                                        const float *__restrict__ I2, double *grho_rows, float *gI2,
                                                        const int *__restrict__ mu, double *e_atom, int NA, int na,
                                                        int a0, int want_grad, const int *__restrict__ ilist)
{
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= na) return;
  const int nr = r.nrho;
  const size_t i = ilist ? (size_t) ilist[a0 + a] : (size_t) (a0 + a);    // the atom of chunk position a
  e_atom[i] = readout_2l_atom(r, rho_rows + i * nr, I2 + (size_t) a * nr, mu[i], grho_rows + i * nr, gI2 + (size_t) a * nr,
                              want_grad, r.owned((long long) i));
}

void launch_readout_2l(const ReadoutDev &r, const float *rho_rows, const float *I2, double *grho_rows, float *gI2,
                       const int *mu, double *e_atom, int NA, int na, int a0, int want_grad, const int *ilist)
{
  if (na == 0) return;
  GB_LAUNCH(readout_2l_kernel, (na + 63) / 64, 64, 0, r, rho_rows, I2, grho_rows, gI2, mu, e_atom, NA, na, a0,
            want_grad, ilist);
}

// out[a] = v[list[a]]
__global__ void __launch_bounds__(256) gather_int_kernel(const int *__restrict__ v, const int *__restrict__ list, int *out, long long n)
{
  const long long a = (long long) blockIdx.x * blockDim.x + threadIdx.x;
  if (a < n) out[a] = v[list[a]];
}

void launch_gather_int(const int *v, const int *list, int *out, long long n)
{
  if (n == 0) return;
  GB_LAUNCH(gather_int_kernel, (unsigned) ((n + 255) / 256), 256, 0, v, list, out, n);
}

// ---- chunk tensor <-> per-atom rows ----------------------------------------------------------------------------
template<class TR, bool TO_ROWS>
__global__ void __launch_bounds__(256) rows_kernel(float *t, TR *rows, int nf, int C, int NA, int na, int a0,
                                                   const int *__restrict__ ilist)
{
  const long long idx = (long long) blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long) na * nf * C;
  if (idx >= total) return;
  const int c = (int) (idx % C);
  const int f = (int) ((idx / C) % nf);
  const int a = (int) (idx / ((long long) C * nf));
  float *tp = t + ((size_t) f * NA + a) * C + c;
  const size_t i = ilist ? (size_t) ilist[a0 + a] : (size_t) (a0 + a);    // the atom of chunk position a
  TR *rp = rows + (i * nf + f) * C + c;
  if (TO_ROWS) *rp = (TR) *tp;
  else *tp = (float) *rp;
}

void launch_rows_from_chunk(const float *t, float *rows, int nf, int C, int NA, int na, int a0, const int *ilist)
{
  const long long total = (long long) na * nf * C;
  if (total == 0) return;
  GB_LAUNCH((rows_kernel<float, true>), (unsigned) ((total + 255) / 256), 256, 0, const_cast<float *>(t), rows, nf, C,
            NA, na, a0, ilist);
}
void launch_chunk_from_rows(float *t, const float *rows, int nf, int C, int NA, int na, int a0, const int *ilist)
{
  const long long total = (long long) na * nf * C;
  if (total == 0) return;
  GB_LAUNCH((rows_kernel<float, false>), (unsigned) ((total + 255) / 256), 256, 0, t, const_cast<float *>(rows), nf, C,
            NA, na, a0, ilist);
}
void launch_chunk_from_rows_f64(float *t, const double *rows, int nf, int C, int NA, int na, int a0, const int *ilist)
{
  const long long total = (long long) na * nf * C;
  if (total == 0) return;
  GB_LAUNCH((rows_kernel<double, false>), (unsigned) ((total + 255) / 256), 256, 0, t, const_cast<double *>(rows), nf,
            C, NA, na, a0, ilist);
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

// one warp per atom j: lanes over the `width` floats of a row, the atom's bonds one after the other
__global__ void __launch_bounds__(128) msg_grad_gather_kernel(BondsDev b, const int *__restrict__ rev,
                                                              const float *__restrict__ gslot, float *gmsg, int width,
                                                              const int *__restrict__ ilist, long long n,
                                                              const int *__restrict__ perm, int nlocal)
{
  const long long a = (long long) blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  const int lane = threadIdx.x & 31;
  if (a >= n) return;
  const long long j = ilist ? ilist[a] : a;
  const long long base = b.off[j];
  const int nb = b.cnt[j];
  for (int c0 = 0; c0 < width; c0 += 128) {    // 4 floats per lane and pass
    const int c = c0 + 4 * lane;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < width) {
      for (int e = 0; e < nb; e++) {
        if (perm && perm[__float_as_int(b.rec[base + e].w)] >= nlocal) continue;
        const size_t p = (size_t) rev[b.cslot[base + e]];
        const float4 v = __ldg(reinterpret_cast<const float4 *>(gslot + p * width + c));
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      *reinterpret_cast<float4 *>(gmsg + (size_t) j * width + c) = acc;
    }
  }
}

void launch_msg_grad_gather(const BondsDev &b, const int *rev, const float *gslot, float *gmsg, int width, const int *ilist,
                            long long n, const int *perm, int nlocal)
{
  if (n == 0) return;
  GB_LAUNCH(msg_grad_gather_kernel, (unsigned) ((n + 3) / 4), 128, 0, b, rev, gslot, gmsg, width, ilist, n, perm, nlocal);
}

// one warp per atom with bonds: own sum by shuffles, neighbours by atomics
__global__ void __launch_bounds__(128) force_scatter_kernel(BondsDev b, const float *__restrict__ fv, double *forces, long long n)
{
  const long long i = (long long) blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  const int lane = threadIdx.x & 31;
  if (i >= n) return;
  const long long base = b.off[i];
  const int nb = b.cnt[i];
  double f0 = 0.0, f1 = 0.0, f2 = 0.0;
  for (int e = lane; e < nb; e += 32) {
    const size_t q = (size_t) b.cslot[base + e];
    const size_t j = (size_t) __float_as_int(b.rec[base + e].w);
    const double x = fv[3 * q], y = fv[3 * q + 1], z = fv[3 * q + 2];
    f0 += x; f1 += y; f2 += z;
    atomicAdd(forces + 3 * j, -x);
    atomicAdd(forces + 3 * j + 1, -y);
    atomicAdd(forces + 3 * j + 2, -z);
  }
  for (int s = 16; s > 0; s >>= 1) {
    f0 += __shfl_xor_sync(0xffffffffu, f0, s);
    f1 += __shfl_xor_sync(0xffffffffu, f1, s);
    f2 += __shfl_xor_sync(0xffffffffu, f2, s);
  }
  if (lane == 0 && nb > 0) {
    atomicAdd(forces + 3 * (size_t) i, f0);
    atomicAdd(forces + 3 * (size_t) i + 1, f1);
    atomicAdd(forces + 3 * (size_t) i + 2, f2);
  }
}

void launch_force_scatter(const BondsDev &b, const float *fv, double *forces, long long n)
{
  if (n == 0) return;
  GB_LAUNCH(force_scatter_kernel, (unsigned) ((n + 3) / 4), 128, 0, b, fv, forces, n);
}

// Zero fill of a 16-byte aligned buffer whose size is a multiple of 4 bytes: 16-byte stores, a grid-stride loop over a
// grid that fills the GPU.  For buffers of hundreds of megabytes this is several times faster than the driver's memset.
__global__ void __launch_bounds__(256) fill_zero_kernel(float4 *__restrict__ p4, long long n4, float *__restrict__ tail, int ntail)
{
  const long long stride = (long long) gridDim.x * blockDim.x;
  for (long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) p4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  if (blockIdx.x == 0 && (int) threadIdx.x < ntail) tail[threadIdx.x] = 0.0f;
}

void launch_fill_zero(void *p, size_t bytes)
{
  if (bytes == 0) return;
  if ((reinterpret_cast<uintptr_t>(p) & 15) != 0 || (bytes & 3) != 0 || bytes < (1u << 20)) {
    GB_CUDA(cudaMemsetAsync(p, 0, bytes, dev().stream));
    return;
  }
  const long long n4 = (long long) (bytes / 16);
  const int ntail = (int) ((bytes % 16) / 4);
  const unsigned grid = (unsigned) std::min<long long>((n4 + 255) / 256, (long long) dev().sm_count * 16);
  GB_LAUNCH(fill_zero_kernel, grid, 256, 0, reinterpret_cast<float4 *>(p), n4, reinterpret_cast<float *>(p) + 4 * n4, ntail);
}

__global__ void __launch_bounds__(256) add_f64_kernel(const double *__restrict__ v, double *out, long long n)
{
  const long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] += v[i];
}

void launch_add_f64(const double *v, double *out, long long n)
{
  if (n == 0) return;
  GB_LAUNCH(add_f64_kernel, (unsigned) ((n + 255) / 256), 256, 0, v, out, n);
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
