// Two microbenchmarks that give the denominators of the compute-bound rooflines on the device the library runs on:
// the fp32 FMA rate of the SIMT lanes (a register-only FFMA loop at full occupancy) and the tf32 rate of the 5th
// generation tensor cores (tcgen05.mma kind::tf32, M = 128, N = 256, both operands in shared memory, accumulators in
// tensor memory).  Timed with CUDA events on the library's stream.  No counterpart in the reference.
#include "peaks.h"

#include <algorithm>

namespace gb {

namespace {

constexpr int FMA_THREADS = 1024, FMA_CHAINS = 8, FMA_UNROLL = 16;

__global__ void __launch_bounds__(FMA_THREADS) peak_fma_kernel(float *out, int iters, float a, float b)
{
  float x[FMA_CHAINS];
#pragma unroll
  for (int c = 0; c < FMA_CHAINS; c++) x[c] = (float) (threadIdx.x + c) * 1.0e-3f;
  for (int it = 0; it < iters; it++) {
#pragma unroll
    for (int u = 0; u < FMA_UNROLL; u++) {
#pragma unroll
      for (int c = 0; c < FMA_CHAINS; c++) x[c] = fmaf(x[c], a, b);
    }
  }
  float s = 0.0f;
#pragma unroll
  for (int c = 0; c < FMA_CHAINS; c++) s += x[c];
  if (s == 123.456f) out[0] = s;    // never true for the arguments used: keeps the loop alive
}

// the same chains with packed two-wide FMAs (fma.rn.f32x2): half the instructions for the same flops
__global__ void __launch_bounds__(FMA_THREADS) peak_fma2_kernel(float *out, int iters, float a, float b)
{
  float2 x[FMA_CHAINS / 2];
#pragma unroll
  for (int c = 0; c < FMA_CHAINS / 2; c++) x[c] = make_float2((float) (threadIdx.x + c) * 1.0e-3f, (float) (threadIdx.x - c) * 1.0e-3f);
  const float2 a2 = make_float2(a, a), b2 = make_float2(b, b);
  for (int it = 0; it < iters; it++) {
#pragma unroll
    for (int u = 0; u < FMA_UNROLL; u++) {
#pragma unroll
      for (int c = 0; c < FMA_CHAINS / 2; c++) x[c] = __ffma2_rn(x[c], a2, b2);
    }
  }
  float s = 0.0f;
#pragma unroll
  for (int c = 0; c < FMA_CHAINS / 2; c++) s += x[c].x + x[c].y;
  if (s == 123.456f) out[0] = s;
}

constexpr int TM = 128, TN = 256, TK = 32;
constexpr long long WAIT_CYCLES = 40000000LL;

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned) __cvta_generic_to_shared(p); }

// K-major operand tile with TK columns in the canonical layout without swizzle (8-row x 16-byte core matrices)
__device__ __forceinline__ unsigned long long make_desc(unsigned addr)
{
  const unsigned long long lbo = 128 >> 4, sbo = ((TK >> 2) * 128) >> 4;
  return (unsigned long long) ((addr & 0x3ffff) >> 4) | (lbo << 16) | (sbo << 32) | (1ull << 46);
}

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

// one warp per CTA, one CTA per SM: lane 0 issues `iters` x 4 MMAs (K = 32 in steps of 8) into two accumulators in
// turn, with a commit and a bounded wait every 32 iterations so that the issue queue stays short
__global__ void __launch_bounds__(32, 1) peak_tf32_kernel(int iters, int n, int *error)
{
  extern __shared__ __align__(1024) char smem[];
  __shared__ unsigned long long s_mbar;
  __shared__ unsigned s_tmem;
  const int lane = threadIdx.x;
  float *A = reinterpret_cast<float *>(smem), *B = A + TM * TK;
  for (int i = lane; i < (TM + n) * TK; i += 32) A[i] = 1.0f + (float) ((i * 2654435761u) >> 20) * 1.0e-4f;
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(512) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  if (lane == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s_mbar)) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncwarp();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem = s_tmem, mbar = smem_u32(&s_mbar);
  // fp32 accumulate, tf32 x tf32, both operands K-major, M = 128, N = n
  const unsigned idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned) (n >> 3) << 17) | ((unsigned) (TM >> 4) << 24);
  const unsigned a0 = smem_u32(A), b0 = smem_u32(B);
  unsigned phase = 0;
  bool ok = true;
  for (int it0 = 0; it0 < iters && ok; it0 += 32) {
    if (lane == 0) {
      for (int it = it0; it < min(iters, it0 + 32); it++) {
        const unsigned d = tmem + (unsigned) (it & 1) * TN;
        for (int ks = 0; ks < TK / 8; ks++) {
          const unsigned acc = (it >= 2 || ks > 0) ? 1u : 0u;
          asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                       "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                       ::"r"(d), "l"(make_desc(a0 + ks * 256)), "l"(make_desc(b0 + ks * 256)), "r"(idesc), "r"(acc) : "memory");
        }
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
    }
    __syncwarp();
    ok = __all_sync(0xffffffffu, mbar_wait(mbar, phase));
    phase ^= 1;
  }
  if (!ok && lane == 0) atomicExch(error, 1);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncwarp();
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
}

double time_ms(cudaEvent_t a, cudaEvent_t b)
{
  float ms = 0.0f;
  GB_CUDA(cudaEventElapsedTime(&ms, a, b));
  return ms;
}

}    // namespace

double measure_peak_fp32_tflops(bool packed)
{
  require_initialized();
  cudaStream_t st = dev().stream;
  DBuf<float> out("peaks:sink");
  out.ensure(4);
  cudaEvent_t a, b;
  GB_CUDA(cudaEventCreate(&a));
  GB_CUDA(cudaEventCreate(&b));
  const int grid = 2 * dev().sm_count, iters = 4096;
  double best = 0.0;
  for (int rep = 0; rep < 4; rep++) {    // the first repetition warms up
    GB_CUDA(cudaEventRecord(a, st));
    if (packed) peak_fma2_kernel<<<grid, FMA_THREADS, 0, st>>>(out.get(), iters, 0.999f, 1.0e-3f);
    else peak_fma_kernel<<<grid, FMA_THREADS, 0, st>>>(out.get(), iters, 0.999f, 1.0e-3f);
    GB_CUDA(cudaGetLastError());
    GB_CUDA(cudaEventRecord(b, st));
    GB_CUDA(cudaEventSynchronize(b));
    dev().launches++;
    const double flop = 2.0 * (double) grid * FMA_THREADS * FMA_CHAINS * FMA_UNROLL * iters;
    if (rep > 0) best = std::max(best, flop / (time_ms(a, b) * 1e-3) / 1e12);
  }
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  return best;
}

double measure_peak_tf32_tflops(int n)
{
  if (n < 16 || n > TN || n % 16 != 0) throw InvalidArgument("N of the tensor-core microbenchmark must be a multiple of 16 up to 256");
  require_initialized();
  cudaStream_t st = dev().stream;
  DBuf<int> err("peaks:flag");
  err.ensure(1);
  GB_CUDA(cudaMemsetAsync(err.get(), 0, sizeof(int), st));
  const size_t smem = (size_t) (TM + TN) * TK * 4;
  GB_CUDA(cudaFuncSetAttribute(peak_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
  cudaEvent_t a, b;
  GB_CUDA(cudaEventCreate(&a));
  GB_CUDA(cudaEventCreate(&b));
  const int grid = dev().sm_count, iters = 4096;
  double best = 0.0;
  for (int rep = 0; rep < 4; rep++) {
    GB_CUDA(cudaEventRecord(a, st));
    peak_tf32_kernel<<<grid, 32, smem, st>>>(iters, n, err.get());
    GB_CUDA(cudaGetLastError());
    GB_CUDA(cudaEventRecord(b, st));
    GB_CUDA(cudaEventSynchronize(b));
    dev().launches++;
    const double flop = 2.0 * TM * n * TK * (double) iters * grid;
    if (rep > 0) best = std::max(best, flop / (time_ms(a, b) * 1e-3) / 1e12);
  }
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  int e = 0;
  GB_CUDA(cudaMemcpyAsync(&e, err.get(), sizeof(int), cudaMemcpyDeviceToHost, st));
  GB_CUDA(cudaStreamSynchronize(st));
  if (e) throw DeviceError("the tensor-core microbenchmark gave up waiting for its matrix instructions");
  return best;
}

}    // namespace gb
