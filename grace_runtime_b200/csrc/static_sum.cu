// Column sums of a device matrix of doubles (per-atom energies or virial rows -> totals) without any device
// allocation: the two-level variant of segment_sum_kernel (chain.cu) whose per-block partial sums live in a
// file-scope device array instead of a buffer obtained from the allocator.  No counterpart in the reference.
//
// The array is one per device and shared by every call: the first 256 bytes hold the arrival counter of the blocks
// (must be zero when a launch starts: cleared by a memset on the stream before each launch, and left at zero by the
// kernel), the rest the partial sums (fully overwritten before they are read).  Calls that overlap in time on one
// device would race on the array: the C ABI serialises its calls under the library's lock and waits for the stream
// before it returns, and a caller that launches from several contexts or libraries must keep that order itself.
// The first call on a device looks the array's address up (cudaGetSymbolAddress, which may load the module's device
// code): make one call before any stream capture starts.
#include "device.h"

#include <algorithm>
#include <string>

namespace gb {

namespace {

constexpr int SS_THREADS = 256;
constexpr int SS_MAX_BLOCKS = 1024;         // partial sums kept: SS_MAX_BLOCKS x SS_MAX_COLS doubles
constexpr int SS_MAX_COLS = 8;
constexpr int SS_ROWS_PER_THREAD = 64;      // a block never walks more than SS_THREADS x this many rows
constexpr int SS_HEADER = 256;              // bytes in front of the partial sums (arrival counter)
constexpr size_t SS_BYTES = SS_HEADER + sizeof(double) * SS_MAX_BLOCKS * SS_MAX_COLS;    // 65,792 bytes

static __device__ __align__(256) unsigned char g_static_scratch[SS_BYTES];

__global__ void __launch_bounds__(SS_THREADS) static_sum_kernel(const double *__restrict__ v, long long n, int K,
                                                                unsigned char *scratch, double *out)
{
  __shared__ double sh[SS_THREADS];
  __shared__ bool last;
  unsigned int *arrived = reinterpret_cast<unsigned int *>(scratch);
  double *partial = reinterpret_cast<double *>(scratch + SS_HEADER);
  const int t = threadIdx.x, B = gridDim.x;
  double acc[SS_MAX_COLS];
#pragma unroll
  for (int k = 0; k < SS_MAX_COLS; k++) acc[k] = 0.0;
  for (long long i = (long long) blockIdx.x * SS_THREADS + t; i < n; i += (long long) B * SS_THREADS) {
#pragma unroll
    for (int k = 0; k < SS_MAX_COLS; k++)
      if (k < K) acc[k] += v[i * K + k];
  }
  // fixed tree per block and column
#pragma unroll
  for (int k = 0; k < SS_MAX_COLS; k++) {
    if (k >= K) break;
    sh[t] = acc[k];
    __syncthreads();
    for (int st = SS_THREADS / 2; st > 0; st >>= 1) {
      if (t < st) sh[t] += sh[t + st];
      __syncthreads();
    }
    if (t == 0) partial[(size_t) blockIdx.x * SS_MAX_COLS + k] = sh[0];
    __syncthreads();
  }
  // the block that arrives last adds the partial sums in block order, whichever block it is
  if (t == 0) {
    __threadfence();
    last = atomicAdd(arrived, 1u) == (unsigned int) (B - 1);
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  for (int k = 0; k < K; k++) {
    double s = 0.0;
    for (int b = t; b < B; b += SS_THREADS) s += __ldcg(partial + (size_t) b * SS_MAX_COLS + k);    // written by other blocks: read past L1
    sh[t] = s;
    __syncthreads();
    for (int st = SS_THREADS / 2; st > 0; st >>= 1) {
      if (t < st) sh[t] += sh[t + st];
      __syncthreads();
    }
    if (t == 0) out[k] = sh[0];
    __syncthreads();
  }
  if (t == 0) *arrived = 0u;
}

// address of the array on each device, looked up once per device
constexpr int SS_MAX_DEVICES = 64;
unsigned char *g_scratch_addr[SS_MAX_DEVICES] = {nullptr};

}    // namespace

long long static_sum_max_rows() { return (long long) SS_MAX_BLOCKS * SS_THREADS * SS_ROWS_PER_THREAD; }
int static_sum_max_cols() { return SS_MAX_COLS; }

void static_sum(const double *d_values, long long n, int K, double *d_out)
{
  require_initialized();
  if (n < 0) throw InvalidArgument("negative row count");
  if (K < 1 || K > SS_MAX_COLS)
    throw InvalidArgument("the static scratch holds partial sums of at most " + std::to_string(SS_MAX_COLS) +
                          " columns; got " + std::to_string(K));
  if (n > static_sum_max_rows())
    throw InvalidArgument("the static scratch covers at most " + std::to_string(static_sum_max_rows()) +
                          " rows; got " + std::to_string(n));
  if (!d_out || (n > 0 && !d_values)) throw InvalidArgument("values and output must be given");
  const int device = dev().device;
  if (device < 0 || device >= SS_MAX_DEVICES) throw InvalidArgument("device ordinal outside 0..63");
  if (!g_scratch_addr[device]) {
    unsigned char *p = nullptr;
    GB_CUDA(cudaGetSymbolAddress((void **) &p, g_static_scratch));
    if (!p) throw DeviceError("cudaGetSymbolAddress returned no address for the static scratch");
    g_scratch_addr[device] = p;
  }
  unsigned char *scratch = g_scratch_addr[device];
  cudaStream_t st = dev().stream;
  int blocks = (int) ((n + (long long) SS_THREADS * SS_ROWS_PER_THREAD - 1) / ((long long) SS_THREADS * SS_ROWS_PER_THREAD));
  // enough blocks to fill the device for mid-sized inputs, never more than the partial sums kept
  const long long by_rows = (n + SS_THREADS - 1) / SS_THREADS;
  blocks = (int) std::max<long long>(blocks, std::min<long long>(by_rows, 4LL * dev().sm_count));
  blocks = std::max(1, std::min(blocks, SS_MAX_BLOCKS));
  GB_CUDA(cudaMemsetAsync(scratch, 0, SS_HEADER, st));
  static_sum_kernel<<<blocks, SS_THREADS, 0, st>>>(d_values, n, K, scratch, d_out);
  GB_CUDA(cudaGetLastError());
  dev().launches++;
  GB_CUDA(cudaStreamSynchronize(st));
}

}    // namespace gb
