// Device plumbing of the backend: error classes, labelled device buffers with the allocation-failure hook of the
// reference's test interface (python/kk/kk_core.cpp:128-141,187-195: debug_fail_alloc / debug_fail_launch), the
// kernel launch macro with launch counting, and a stream-ordered event timer.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace gb {

struct InvalidArgument : std::invalid_argument {
  using std::invalid_argument::invalid_argument;
};
struct DeviceError : std::runtime_error {
  using std::runtime_error::runtime_error;
};
struct OutOfMemory : std::runtime_error {
  using std::runtime_error::runtime_error;
};
struct Unsupported : std::runtime_error {
  using std::runtime_error::runtime_error;
};

void cuda_check(cudaError_t e, const char *what);
#define GB_CUDA(call) ::gb::cuda_check((call), #call)

// process-wide device state
struct DeviceState {
  bool initialized = false;
  int device = -1;
  cudaStream_t stream = nullptr;
  uint64_t launches = 0;
  // fault injection (host side only; nothing here makes a GPU fault)
  std::string fail_label;
  int fail_alloc_nth = 0;
  int fail_launch_nth = 0;
  int sm_count = 148;
};
DeviceState &dev();
void require_initialized();

// around every kernel launch: count it, report launch errors, apply debug_fail_launch; with the kernel profile on,
// a pair of CUDA events on the launch stream per launch
void before_launch(const char *name);
void after_launch(const char *name);
// label appended to the kernel name of the launches that follow in the kernel profile (null: none); the engine tags
// the operations of the dense network with their names when GRACE_B200_PROFILE_OPS is set
void launch_tag(const char *tag);
// per-kernel device time (CUDA events around every launch while on)
void profile_enable(bool on);
// "name launches total_ms" lines of the launches since profile_enable(true); synchronises the stream
std::string profile_report();

// dynamic shared memory of a kernel as an array of T
#define GB_DYN_SMEM(T, name) extern __shared__ T name[]
#define GB_LAUNCH(kernel, grid, block, smem, ...)                                   \
  do {                                                                              \
    ::gb::before_launch(#kernel);                                                   \
    kernel<<<(grid), (block), (smem), ::gb::dev().stream>>>(__VA_ARGS__);           \
    ::gb::after_launch(#kernel);                                                    \
  } while (0)

void *device_alloc(size_t bytes, const char *label);
void device_free(void *p);

// a device array that grows on demand (contents are not kept across a grow)
template<class T> class DBuf {
 public:
  DBuf() = default;
  explicit DBuf(const char *label) : label_(label) {}
  DBuf(const DBuf &) = delete;
  DBuf &operator=(const DBuf &) = delete;
  DBuf(DBuf &&o) noexcept { *this = std::move(o); }
  DBuf &operator=(DBuf &&o) noexcept
  {
    if (this != &o) {
      release();
      p_ = o.p_; cap_ = o.cap_; label_ = o.label_;
      o.p_ = nullptr; o.cap_ = 0;
    }
    return *this;
  }
  ~DBuf() { release(); }
  void set_label(const char *l) { label_ = l; }
  // at least n elements; grows with 12.5 % headroom
  T *ensure(size_t n)
  {
    if (n > cap_) {
      release();
      const size_t want = n + n / 8 + 16;
      p_ = static_cast<T *>(device_alloc(want * sizeof(T), label_));
      cap_ = want;
    }
    return p_;
  }
  void release()
  {
    if (p_) device_free(p_);
    p_ = nullptr;
    cap_ = 0;
  }
  T *get() const { return p_; }
  size_t capacity() const { return cap_; }
  void upload(const std::vector<T> &h)
  {
    ensure(h.size());
    if (!h.empty()) GB_CUDA(cudaMemcpyAsync(p_, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice, dev().stream));
  }

 private:
  T *p_ = nullptr;
  size_t cap_ = 0;
  const char *label_ = "buffer";
};

// bytes currently allocated through device_alloc (diagnostics)
size_t device_bytes_live();
// allocation tracking of the reference's test interface (python/kk/kk_core.cpp:143-184): from track_alloc(true) on,
// every device_alloc is recorded by label; live bytes by label (largest first) and their high-water mark
void track_alloc(bool on);
size_t tracked_peak_bytes();
std::vector<std::pair<std::string, size_t>> tracked_live();

// device time per stage of one compute call: pairs of CUDA events on the launch stream, summed per stage after the
// call's synchronize (a stage may be entered once per chunk)
class StageTimer {
 public:
  enum { NL = 0, GEOM, FWD, BWD, TOTAL, NSTAGE };
  StageTimer() = default;
  ~StageTimer();
  StageTimer(const StageTimer &) = delete;
  StageTimer &operator=(const StageTimer &) = delete;
  void reset();
  void begin(int stage);
  void end(int stage);
  void collect(double *ms);    // after a stream synchronize

 private:
  struct Span { int stage; cudaEvent_t a, b; };
  std::vector<Span> spans_;
  std::vector<cudaEvent_t> pool_;
  size_t used_ = 0;
  int open_[NSTAGE] = {-1, -1, -1, -1, -1};
  cudaEvent_t take();
};

}    // namespace gb
