#include "device.h"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>

namespace gb {

namespace {
DeviceState g_dev;
std::map<void *, size_t> g_live;
size_t g_live_bytes = 0;
// allocations made since track_alloc(true), by label, with their high-water mark: the reference's
// _debug_track_alloc / _debug_live_alloc / _debug_peak_alloc (python/kk/kk_core.cpp:143-184)
bool g_track = false;
std::map<void *, std::pair<std::string, size_t>> g_tracked;
size_t g_tracked_bytes = 0, g_tracked_peak = 0;
}    // namespace

void track_alloc(bool on)
{
  g_tracked.clear();
  g_tracked_bytes = g_tracked_peak = 0;
  g_track = on;
}

size_t tracked_peak_bytes() { return g_tracked_peak; }

std::vector<std::pair<std::string, size_t>> tracked_live()
{
  std::map<std::string, size_t> by;
  for (const auto &kv : g_tracked) by[kv.second.first] += kv.second.second;
  std::vector<std::pair<std::string, size_t>> v(by.begin(), by.end());
  std::sort(v.begin(), v.end(), [](const auto &a, const auto &b) { return a.second > b.second; });
  return v;
}

DeviceState &dev() { return g_dev; }

void require_initialized()
{
  if (!g_dev.initialized) throw DeviceError("the GPU backend is not initialised (call grace_initialize first) or was finalised");
}

void cuda_check(cudaError_t e, const char *what)
{
  if (e == cudaSuccess) return;
  const std::string msg = std::string("CUDA error: ") + cudaGetErrorString(e) + " in " + what;
  if (e == cudaErrorMemoryAllocation) {
    (void) cudaGetLastError();    // the allocation error is not sticky: clear it so the context stays usable
    throw OutOfMemory(msg);
  }
  throw DeviceError(msg);
}

namespace {
struct ProfSpan { std::string name; cudaEvent_t a, b; };
const char *g_tag = nullptr;
bool g_prof_on = false;
std::vector<ProfSpan> g_prof;
std::vector<cudaEvent_t> g_prof_pool;
size_t g_prof_used = 0;
cudaEvent_t prof_event()
{
  if (g_prof_used == g_prof_pool.size()) {
    cudaEvent_t e;
    GB_CUDA(cudaEventCreate(&e));
    g_prof_pool.push_back(e);
  }
  return g_prof_pool[g_prof_used++];
}
}    // namespace

void launch_tag(const char *tag) { g_tag = tag; }

void profile_enable(bool on)
{
  g_prof_on = on;
  g_prof.clear();
  g_prof_used = 0;
}

std::string profile_report()
{
  if (g_dev.initialized) cudaStreamSynchronize(g_dev.stream);
  std::map<std::string, std::pair<long long, double>> acc;
  for (const auto &s : g_prof) {
    float ms = 0.0f;
    if (cudaEventElapsedTime(&ms, s.a, s.b) != cudaSuccess) continue;
    auto &e = acc[s.name];
    e.first++;
    e.second += ms;
  }
  std::string out;
  for (const auto &kv : acc) out += kv.first + " " + std::to_string(kv.second.first) + " " + std::to_string(kv.second.second) + "\n";
  return out;
}

void before_launch(const char *name)
{
  if (!g_prof_on) return;
  ProfSpan s{g_tag ? std::string(name) + ":" + g_tag : std::string(name), prof_event(), prof_event()};
  cudaEventRecord(s.a, g_dev.stream);
  g_prof.push_back(s);
}

void after_launch(const char *name)
{
  if (g_prof_on && !g_prof.empty()) cudaEventRecord(g_prof.back().b, g_dev.stream);
  g_dev.launches++;
  if (g_dev.fail_launch_nth > 0 && --g_dev.fail_launch_nth == 0)
    throw OutOfMemory(std::string("kernel launch ran out of device memory (injected) in ") + name);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) cuda_check(e, name);
}

void *device_alloc(size_t bytes, const char *label)
{
  require_initialized();
  if (bytes == 0) bytes = 16;
  void *p = nullptr;
  GB_CUDA(cudaMalloc(&p, bytes));
  // the injected failure comes after the allocation, as the reference's hook does (kk_core.cpp:128-141): the buffer is
  // returned to the device before the error is raised
  if (g_dev.fail_alloc_nth > 0 && label && std::strstr(label, g_dev.fail_label.c_str()) != nullptr &&
      --g_dev.fail_alloc_nth == 0) {
    cudaFree(p);
    throw OutOfMemory(std::string("out of device memory (injected) allocating '") + label + "'");
  }
  g_live[p] = bytes;
  g_live_bytes += bytes;
  if (g_track) {
    g_tracked[p] = {label ? label : "buffer", bytes};
    g_tracked_bytes += bytes;
    g_tracked_peak = std::max(g_tracked_peak, g_tracked_bytes);
  }
  return p;
}

void device_free(void *p)
{
  if (!p) return;
  auto it = g_live.find(p);
  if (it != g_live.end()) {
    g_live_bytes -= it->second;
    g_live.erase(it);
  }
  auto tr = g_tracked.find(p);
  if (tr != g_tracked.end()) {    // allocated before tracking started: not counted
    g_tracked_bytes -= tr->second.second;
    g_tracked.erase(tr);
  }
  if (g_dev.initialized) cudaFree(p);
}

size_t device_bytes_live() { return g_live_bytes; }

StageTimer::~StageTimer()
{
  if (!g_dev.initialized) return;
  for (auto e : pool_) cudaEventDestroy(e);
}

cudaEvent_t StageTimer::take()
{
  if (used_ == pool_.size()) {
    cudaEvent_t e;
    GB_CUDA(cudaEventCreate(&e));
    pool_.push_back(e);
  }
  return pool_[used_++];
}

void StageTimer::reset()
{
  spans_.clear();
  used_ = 0;
  for (int s = 0; s < NSTAGE; s++) open_[s] = -1;
}

void StageTimer::begin(int stage)
{
  Span sp{stage, take(), take()};
  GB_CUDA(cudaEventRecord(sp.a, g_dev.stream));
  open_[stage] = (int) spans_.size();
  spans_.push_back(sp);
}

void StageTimer::end(int stage)
{
  if (open_[stage] < 0) return;
  GB_CUDA(cudaEventRecord(spans_[open_[stage]].b, g_dev.stream));
  open_[stage] = -1;
}

void StageTimer::collect(double *ms)
{
  for (int s = 0; s < NSTAGE; s++) ms[s] = 0.0;
  for (size_t q = 0; q < spans_.size(); q++) {
    bool closed = true;
    for (int s = 0; s < NSTAGE; s++) closed = closed && open_[s] != (int) q;
    if (!closed) continue;
    float t = 0.0f;
    if (cudaEventElapsedTime(&t, spans_[q].a, spans_[q].b) == cudaSuccess) ms[spans_[q].stage] += t;
  }
}

}    // namespace gb
