// The exact radial MLP of a layer over a batch of bonds on the 5th-generation tensor cores: value and d/dx of
// R[o](x) = W3' act(W2' act(W1' g(x))) for every bond, the three layers as tcgen05.mma (kind::tf32, M = 128, fp32
// accumulators in tensor memory) with the activation, its slope and the 3 x tf32 operand split fused into the epilogues
// between them.  Counterpart of the reference's generic GPU engine, which runs the same chain as six cuBLAS SGEMMs with
// every intermediate in global memory (libgrace/include/grace/kk/grace_1l_kk_impl.h:1592-1751); forward-mode
// derivative as libgrace/include/grace/radial_x.h:30-60.
//
// One CTA of 256 threads per SM loops over tiles of 64 bonds.  A tile is a 128-row operand: rows 0-63 carry the values
// (g, h1, h2), rows 64-127 the derivatives (dg, dh1, dh2), so one MMA chain propagates both; threads t and t + 128 own
// row t = tensor-memory lane t and take 32 of its columns each.  Operands live in shared memory in the canonical K-major layout without swizzle (8-row x
// 16-byte core matrices); the weights are converted to that layout, transposed, scaled and split into tf32 hi + lo on
// the host once.  fp32-level accuracy comes from the split: a b ~ a_lo b_hi + a_hi b_lo + a_hi b_hi.
//
// Every wait on the tensor cores is bounded: a wait that runs out sets the error flag, the CTA frees its tensor memory
// and returns, and the host reports the failure.
#include "radial_mlp_tc.h"

#include <cmath>
#include <cstring>

namespace gb {

namespace {

constexpr int TM = 128;         // rows of a tile = tensor-memory lanes
constexpr int NTH = 256;        // threads: two per row
constexpr int TB = 64;          // bonds of a tile
constexpr int KH = 64;          // hidden width (both hidden layers)
constexpr int KG = 8;           // padded width of the radial basis
constexpr int TMEM_COLS = 512;
constexpr long long WAIT_CYCLES = 40000000LL;    // ~20 ms: far beyond any tile, far below a watchdog

// byte offset of element (r, k) of a K-major operand tile with K columns (canonical layout, no swizzle)
__host__ __device__ inline int tile_off(int r, int k, int K) { return (r >> 3) * (K >> 2) * 128 + (k >> 2) * 128 + (r & 7) * 16 + (k & 3) * 4; }

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned) __cvta_generic_to_shared(p); }

// shared-memory matrix descriptor: start address, leading (K direction) and stride (8-row group) byte offsets in
// 16-byte units, descriptor version 1, no swizzle
__device__ __forceinline__ unsigned long long make_desc(unsigned addr, int K)
{
  const unsigned long long lbo = 128 >> 4, sbo = ((K >> 2) * 128) >> 4;
  return (unsigned long long) ((addr & 0x3ffff) >> 4) | (lbo << 16) | (sbo << 32) | (1ull << 46);
}

// instruction descriptor: fp32 accumulate, tf32 x tf32, both operands K-major, M = 128, N = n
__device__ __forceinline__ unsigned make_idesc(int n) { return (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned) (n >> 3) << 17) | ((unsigned) (TM >> 4) << 24); }

__device__ __forceinline__ void mma_tf32_ss(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned idesc, bool accumulate)
{
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"((unsigned) accumulate) : "memory");
}

__device__ __forceinline__ void split_tf32(float x, float &hi, float &lo)
{
  unsigned h, l;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
  hi = __uint_as_float(h);
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(x - hi));
  lo = __uint_as_float(l);
}

// 32 consecutive columns of this thread's tensor-memory lane
__device__ __forceinline__ void tmem_ld32(unsigned taddr, float (&v)[32])
{
  unsigned r[32];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
               "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

// waits for the phase `parity` of the barrier; false when the limit ran out
__device__ __forceinline__ bool mbar_wait(unsigned mbar, unsigned parity)
{
  const long long t0 = clock64();
  for (;;) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(mbar), "r"(parity) : "memory");
    if (ok) return true;
    if (clock64() - t0 > WAIT_CYCLES) return false;
  }
}

struct Act {
  int kind;    // 0 SiLU, 1 tanh
  __device__ __forceinline__ void operator()(float s, float &h, float &slope) const
  {
    if (kind == 1) {
      h = tanhf(s);
      slope = 1.0f - h * h;
    } else {
      const float sg = __frcp_rn(1.0f + __expf(-s));
      h = s * sg;
      slope = sg * (1.0f + s * (1.0f - sg));
    }
  }
};

// value rows: h = act(pre), slope kept for the derivative rows; derivative rows: dh = slope dpre.  Both as hi / lo
// operand rows of the next layer.
__device__ __forceinline__ void hidden_epilogue(unsigned tmem_row, int col0, int r, int half, Act act,
                                                float *slope /* [TB][KH + 1] */, char *Hhi, char *Hlo)
{
  float pre[32];
  tmem_ld32(tmem_row + col0 + 32 * half, pre);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  if (r < TB) {
#pragma unroll
    for (int c4 = 0; c4 < 8; c4++) {
      float hi[4], lo[4];
#pragma unroll
      for (int q = 0; q < 4; q++) {
        float h, sl;
        act(pre[4 * c4 + q], h, sl);
        slope[r * (KH + 1) + 32 * half + 4 * c4 + q] = sl;
        split_tf32(h, hi[q], lo[q]);
      }
      const int off = tile_off(r, 32 * half + 4 * c4, KH);
      *reinterpret_cast<float4 *>(Hhi + off) = make_float4(hi[0], hi[1], hi[2], hi[3]);
      *reinterpret_cast<float4 *>(Hlo + off) = make_float4(lo[0], lo[1], lo[2], lo[3]);
    }
  }
  __syncthreads();
  if (r >= TB) {
#pragma unroll
    for (int c4 = 0; c4 < 8; c4++) {
      float hi[4], lo[4];
#pragma unroll
      for (int q = 0; q < 4; q++)
        split_tf32(slope[(r - TB) * (KH + 1) + 32 * half + 4 * c4 + q] * pre[4 * c4 + q], hi[q], lo[q]);
      const int off = tile_off(r, 32 * half + 4 * c4, KH);
      *reinterpret_cast<float4 *>(Hhi + off) = make_float4(hi[0], hi[1], hi[2], hi[3]);
      *reinterpret_cast<float4 *>(Hlo + off) = make_float4(lo[0], lo[1], lo[2], lo[3]);
    }
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
}

// the 3 x tf32 product of an operand pair over K (steps of 8 columns = 256 bytes of either tile)
__device__ __forceinline__ void issue_layer(unsigned tmem_d, unsigned a_hi, unsigned a_lo, int Ka, unsigned b_hi, unsigned b_lo,
                                            int n)
{
  const unsigned idesc = make_idesc(n);
  bool acc = false;
  for (int pass = 0; pass < 3; pass++) {    // small terms first
    const unsigned a = pass == 0 ? a_lo : a_hi, b = pass == 1 ? b_lo : b_hi;
    for (int ks = 0; ks < Ka / 8; ks++) {
      mma_tf32_ss(tmem_d, make_desc(a + ks * 256, Ka), make_desc(b + ks * 256, Ka), idesc, acc);
      acc = true;
    }
  }
}

__global__ void __launch_bounds__(NTH, 1) radial_mlp_tc_kernel(RadialMlpTCDev m, const float *__restrict__ x, long long nb,
                                                              float *__restrict__ R, float *__restrict__ dR, int *error)
{
  extern __shared__ __align__(1024) char smem[];
  __shared__ unsigned long long s_mbar;
  __shared__ unsigned s_tmem;
  const int t = threadIdx.x, warp = t >> 5, r = t & (TM - 1), half = t >> 7;    // row and column half of this thread
  const int NO = m.n_out;
  // shared memory: operand tiles of the activations, then the weights
  char *Ghi = smem, *Glo = Ghi + TM * KG * 4, *Hhi = Glo + TM * KG * 4, *Hlo = Hhi + TM * KH * 4;
  char *W1hi = Hlo + TM * KH * 4, *W1lo = W1hi + KH * KG * 4, *W2hi = W1lo + KH * KG * 4, *W2lo = W2hi + KH * KH * 4;
  char *W3hi = W2lo + KH * KH * 4, *W3lo = W3hi + NO * KH * 4;
  float *slope = reinterpret_cast<float *>(W3lo + NO * KH * 4);
  {    // the weight images are byte-for-byte the shared-memory layout
    const int4 *src = reinterpret_cast<const int4 *>(m.weights);
    int4 *dst = reinterpret_cast<int4 *>(W1hi);
    for (int i = t; i < m.weight_bytes / 16; i += NTH) dst[i] = src[i];
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (t == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s_mbar)) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem = s_tmem, mbar = smem_u32(&s_mbar);
  const unsigned tmem_row = tmem + ((unsigned) ((warp & 3) * 32) << 16);    // this warp's lanes
  const Act act{m.act};
  unsigned phase = 0;
  bool ok = true;
  const long long ntiles = (nb + TB - 1) / TB;
  for (long long tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
    const long long b0 = tile * TB;
    if (t < TB) {    // radial basis and its derivative: rows t (values) and t + 64 (derivatives) of the first operand
      const long long b = b0 + t;
      const float xb = b < nb ? x[b] : 0.5f;
      const int p = m.p;
      float xp = 1.0f;
      for (int q = 0; q < p - 1; q++) xp *= xb;
      const float xpm1 = xp;    // x^(p-1)
      xp *= xb;
      const float xp1 = xp * xb, xp2 = xp1 * xb;
      const float fc = 1.0f - 0.5f * (p + 1) * (p + 2) * xp + (float) (p * (p + 2)) * xp1 - 0.5f * p * (p + 1) * xp2;
      const float dfc = 0.5f * p * (p + 1) * (p + 2) * (-xpm1 + 2.0f * xp - xp1);
      const float tt = 2.0f * xb - 1.0f;
      float Tp = 1.0f, Tc = tt, dTp = 0.0f, dTc = 2.0f;
      float g[KG], dg[KG];
#pragma unroll
      for (int k = 0; k < KG; k++) {
        const bool in = k < m.nrb;
        g[k] = in ? Tc * fc : 0.0f;
        dg[k] = in ? dTc * fc + Tc * dfc : 0.0f;
        const float Tn = 2.0f * tt * Tc - Tp, dTn = 2.0f * (2.0f * Tc + tt * dTc) - dTp;
        Tp = Tc; dTp = dTc; Tc = Tn; dTc = dTn;
      }
#pragma unroll
      for (int c4 = 0; c4 < 2; c4++) {
        float hi[4], lo[4];
#pragma unroll
        for (int q = 0; q < 4; q++) split_tf32(g[4 * c4 + q], hi[q], lo[q]);
        *reinterpret_cast<float4 *>(Ghi + tile_off(t, 4 * c4, KG)) = make_float4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<float4 *>(Glo + tile_off(t, 4 * c4, KG)) = make_float4(lo[0], lo[1], lo[2], lo[3]);
#pragma unroll
        for (int q = 0; q < 4; q++) split_tf32(dg[4 * c4 + q], hi[q], lo[q]);
        *reinterpret_cast<float4 *>(Ghi + tile_off(t + TB, 4 * c4, KG)) = make_float4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<float4 *>(Glo + tile_off(t + TB, 4 * c4, KG)) = make_float4(lo[0], lo[1], lo[2], lo[3]);
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    // layer 1
    if (t == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      issue_layer(tmem + 0, smem_u32(Ghi), smem_u32(Glo), KG, smem_u32(W1hi), smem_u32(W1lo), KH);
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
    }
    ok = __syncthreads_and(mbar_wait(mbar, phase));    // all threads leave together if any wait ran out
    phase ^= 1;
    if (!ok) break;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    hidden_epilogue(tmem_row, 0, r, half, act, slope, Hhi, Hlo);
    // layer 2
    if (t == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      issue_layer(tmem + KH, smem_u32(Hhi), smem_u32(Hlo), KH, smem_u32(W2hi), smem_u32(W2lo), KH);
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
    }
    ok = __syncthreads_and(mbar_wait(mbar, phase));    // all threads leave together if any wait ran out
    phase ^= 1;
    if (!ok) break;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    hidden_epilogue(tmem_row, KH, r, half, act, slope, Hhi, Hlo);
    // output layer
    if (t == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      issue_layer(tmem + 2 * KH, smem_u32(Hhi), smem_u32(Hlo), KH, smem_u32(W3hi), smem_u32(W3lo), NO);
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
    }
    ok = __syncthreads_and(mbar_wait(mbar, phase));    // all threads leave together if any wait ran out
    phase ^= 1;
    if (!ok) break;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    {    // rows 0-63 -> R, rows 64-127 -> dR of bond b0 + (row mod 64); the two threads of a row alternate 32-column blocks
      const long long b = b0 + (r & (TB - 1));
      float *dst = (r < TB ? R : dR) + (size_t) b * NO;
      for (int c0 = 32 * half; c0 < NO; c0 += 64) {
        float v[32];
        tmem_ld32(tmem_row + 2 * KH + c0, v);
        if (b < nb) {
#pragma unroll
          for (int q = 0; q < 32; q += 4) *reinterpret_cast<float4 *>(dst + c0 + q) = make_float4(v[q], v[q + 1], v[q + 2], v[q + 3]);
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
  }
  if (!ok && t == 0) atomicExch(error, 1);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

}    // namespace

bool RadialMlpTC::supported(const GraceModel &m, const std::vector<MlpLayer> &layers)
{
  if (layers.size() != 3 || m.nradbase > KG) return false;
  if (layers[0].n_out != KH || layers[1].n_in != KH || layers[1].n_out != KH || layers[2].n_in != KH) return false;
  const int no = layers[2].n_out;
  if (no % 32 != 0 || no < 32 || no > 256 || 2 * KH + no > TMEM_COLS) return false;
  return smem_bytes(no) <= 227 * 1024;
}

size_t RadialMlpTC::smem_bytes(int n_out)
{
  return (size_t) 2 * TM * KG * 4 + 2 * TM * KH * 4 + 2 * KH * KG * 4 + 2 * KH * KH * 4 + 2 * (size_t) n_out * KH * 4 +
         (size_t) TB * (KH + 1) * 4;
}

// B operand image of a layer: W'[n][k] = norm W[k][perm(n)] split into tf32 hi and lo, canonical layout with K columns
static void weight_image(const MlpLayer &L, int K, const std::vector<int> &col, std::vector<char> &out)
{
  const int N = (int) col.size();
  std::vector<char> hi((size_t) N * K * 4, 0), lo((size_t) N * K * 4, 0);
  for (int n = 0; n < N; n++)
    for (int k = 0; k < K; k++) {
      const float w = k < L.n_in ? (float) (L.W[(size_t) k * L.n_out + col[n]] * L.norm) : 0.0f;
      unsigned u;
      std::memcpy(&u, &w, 4);
      u = (u + 0x1000u) & 0xffffe000u;    // round to nearest tf32 (10-bit mantissa)
      float h;
      std::memcpy(&h, &u, 4);
      const float r = w - h;
      unsigned v;
      std::memcpy(&v, &r, 4);
      v = (v + 0x1000u) & 0xffffe000u;
      std::memcpy(hi.data() + tile_off(n, k, K), &u, 4);
      std::memcpy(lo.data() + tile_off(n, k, K), &v, 4);
    }
  out.insert(out.end(), hi.begin(), hi.end());
  out.insert(out.end(), lo.begin(), lo.end());
}

void RadialMlpTC::setup(const GraceModel &m, const std::vector<MlpLayer> &layers, int C)
{
  if (!supported(m, layers)) throw Unsupported("radial MLP shape outside the tensor-core kernel (8 -> 64 -> 64 -> n)");
  const int nl = m.lmax + 1, no = layers[2].n_out;
  if (no != C * nl) throw ModelError("radial MLP output width mismatch");
  std::vector<char> img;
  std::vector<int> id(KH);
  for (int i = 0; i < KH; i++) id[i] = i;
  weight_image(layers[0], KG, id, img);
  weight_image(layers[1], KH, id, img);
  std::vector<int> col(no);    // outputs in the order of the radial tables: o' = l C + n from the model's o = n nl + l
  for (int n = 0; n < C; n++)
    for (int l = 0; l < nl; l++) col[l * C + n] = n * nl + l;
  weight_image(layers[2], KH, col, img);
  weights_.set_label("engine:radial_mlp");
  weights_.ensure(img.size());
  GB_CUDA(cudaMemcpyAsync(weights_.get(), img.data(), img.size(), cudaMemcpyHostToDevice, dev().stream));
  GB_CUDA(cudaStreamSynchronize(dev().stream));
  error_.set_label("engine:radial_mlp");
  error_.ensure(1);
  GB_CUDA(cudaMemsetAsync(error_.get(), 0, sizeof(int), dev().stream));
  d_.weights = weights_.get();
  d_.weight_bytes = (int) img.size();
  d_.n_out = no;
  d_.nrb = m.nradbase;
  d_.p = m.p;
  d_.act = m.radial_activation;
  ready_ = true;
}

void RadialMlpTC::run(const float *d_x, long long nb, float *d_R, float *d_dR)
{
  if (!ready_) throw DeviceError("radial MLP kernel used before its set-up");
  if (nb <= 0) return;
  const size_t smem = smem_bytes(d_.n_out);
  GB_CUDA(cudaFuncSetAttribute(radial_mlp_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
  const long long ntiles = (nb + TB - 1) / TB;
  const int grid = (int) std::min<long long>(ntiles, dev().sm_count);
  GB_LAUNCH(radial_mlp_tc_kernel, grid, NTH, smem, d_, d_x, nb, d_R, d_dR, error_.get());
}

void RadialMlpTC::check()
{
  int e = 0;
  GB_CUDA(cudaMemcpyAsync(&e, error_.get(), sizeof(int), cudaMemcpyDeviceToHost, dev().stream));
  GB_CUDA(cudaStreamSynchronize(dev().stream));
  if (e) {
    GB_CUDA(cudaMemsetAsync(error_.get(), 0, sizeof(int), dev().stream));
    throw DeviceError("the tensor-core radial MLP kernel gave up waiting for its matrix instructions");
  }
}

}    // namespace gb
