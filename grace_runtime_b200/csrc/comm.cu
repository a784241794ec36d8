#include "comm.h"

#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <map>
#include <string>

namespace gb {

namespace {

// the NCCL entry points the exchange uses, resolved from libnccl.so.2 on first use (a process that already loaded
// NCCL, e.g. through PyTorch, gets that copy: same soname)
struct Nccl {
  void *lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*Send)(const void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

Nccl &nccl()
{
  static Nccl n;
  if (n.lib) return n;
  void *lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) throw DeviceError(std::string("NCCL is not available (libnccl.so.2): ") + dlerror());
  auto sym = [&](const char *name) {
    void *p = dlsym(lib, name);
    if (!p) throw DeviceError(std::string("libnccl has no symbol ") + name);
    return p;
  };
  n.GetUniqueId = reinterpret_cast<decltype(n.GetUniqueId)>(sym("ncclGetUniqueId"));
  n.CommInitRank = reinterpret_cast<decltype(n.CommInitRank)>(sym("ncclCommInitRank"));
  n.CommDestroy = reinterpret_cast<decltype(n.CommDestroy)>(sym("ncclCommDestroy"));
  n.Send = reinterpret_cast<decltype(n.Send)>(sym("ncclSend"));
  n.Recv = reinterpret_cast<decltype(n.Recv)>(sym("ncclRecv"));
  n.AllReduce = reinterpret_cast<decltype(n.AllReduce)>(sym("ncclAllReduce"));
  n.GroupStart = reinterpret_cast<decltype(n.GroupStart)>(sym("ncclGroupStart"));
  n.GroupEnd = reinterpret_cast<decltype(n.GroupEnd)>(sym("ncclGroupEnd"));
  n.GetErrorString = reinterpret_cast<decltype(n.GetErrorString)>(sym("ncclGetErrorString"));
  n.lib = lib;
  return n;
}

void nccl_check(ncclResult_t r, const char *what)
{
  if (r == ncclSuccess) return;
  throw DeviceError(std::string("NCCL error: ") + nccl().GetErrorString(r) + " in " + what);
}
#define GB_NCCL(call) nccl_check((call), #call)

ncclComm_t g_comm = nullptr;
int g_rank = -1, g_world = 0;

// send rows: buf[q] = f[index[q]]
__global__ void __launch_bounds__(256) pack_rows_kernel(const double *__restrict__ f, const int *__restrict__ index,
                                                        double *buf, long long n)
{
  const long long q = (long long) blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= n) return;
  const size_t i = index[q];
  buf[3 * q] = f[3 * i];
  buf[3 * q + 1] = f[3 * i + 1];
  buf[3 * q + 2] = f[3 * i + 2];
}

// owned atom target[k] receives the rows rows[off[k] .. off[k + 1]) of the receive buffer, added in that order
__global__ void __launch_bounds__(256) add_rows_kernel(double *f, const int *__restrict__ target, const int *__restrict__ off,
                                                       const int *__restrict__ rows, const double *__restrict__ buf, long long nt)
{
  const long long k = (long long) blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= nt) return;
  const size_t i = target[k];
  double a = f[3 * i], b = f[3 * i + 1], c = f[3 * i + 2];
  for (int q = off[k]; q < off[k + 1]; q++) {
    const size_t r = rows[q];
    a += buf[3 * r];
    b += buf[3 * r + 1];
    c += buf[3 * r + 2];
  }
  f[3 * i] = a;
  f[3 * i + 1] = b;
  f[3 * i + 2] = c;
}

__global__ void totals_kernel(double *t, double *energy, double *virial, int to_buffer)
{
  const int k = threadIdx.x;
  if (k >= 7) return;
  double *p = k == 0 ? energy : (virial ? virial + (k - 1) : nullptr);
  if (to_buffer) t[k] = p ? *p : 0.0;
  else if (p) *p = t[k];
}

unsigned nblocks(long long n) { return (unsigned) ((n + 255) / 256); }

}    // namespace

void comm_unique_id(void *id128)
{
  if (!id128) throw InvalidArgument("id buffer must be given");
  ncclUniqueId id;
  GB_NCCL(nccl().GetUniqueId(&id));
  static_assert(sizeof(id) == 128, "NCCL unique id size");
  memcpy(id128, &id, sizeof(id));
}

void comm_init(const void *id128, int rank, int world)
{
  require_initialized();
  if (!id128) throw InvalidArgument("id must be given");
  if (world < 1 || rank < 0 || rank >= world) throw InvalidArgument("rank must be in 0 .. world - 1");
  if (g_comm) throw DeviceError("the library already has a communicator (one per process)");
  ncclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  GB_NCCL(nccl().CommInitRank(&g_comm, world, id, rank));
  g_rank = rank;
  g_world = world;
}

void comm_finalize()
{
  if (!g_comm) return;
  if (dev().initialized) cudaStreamSynchronize(dev().stream);
  nccl().CommDestroy(g_comm);
  g_comm = nullptr;
  g_rank = -1;
  g_world = 0;
}

int comm_rank() { return g_rank; }
int comm_size() { return g_world; }

void Exchange::setup(int n, int nlocal, const int32_t *send_counts, const int32_t *send_index, const int32_t *recv_counts,
                     const int32_t *recv_index)
{
  if (!g_comm) throw DeviceError("no communicator: call grace_comm_init first");
  if (n < 0 || nlocal < 0 || nlocal > n) throw InvalidArgument("nlocal must be in 0 .. n");
  if (!send_counts || !recv_counts) throw InvalidArgument("send and receive counts must be given");
  world_ = g_world;
  n_ = n;
  nlocal_ = nlocal;
  send_counts_.assign(send_counts, send_counts + world_);
  recv_counts_.assign(recv_counts, recv_counts + world_);
  nsend_ = nrecv_ = 0;
  for (int r = 0; r < world_; r++) {
    if (send_counts_[r] < 0 || recv_counts_[r] < 0) throw InvalidArgument("negative row count");
    nsend_ += send_counts_[r];
    nrecv_ += recv_counts_[r];
  }
  if ((nsend_ > 0 && !send_index) || (nrecv_ > 0 && !recv_index)) throw InvalidArgument("row indices must be given");
  std::vector<int> sidx((size_t) nsend_);
  for (int64_t q = 0; q < nsend_; q++) {
    if (send_index[q] < 0 || send_index[q] >= n) throw InvalidArgument("send index outside the sub-system");
    sidx[(size_t) q] = send_index[q];
  }
  // rows received per owned atom, in arrival order: the sums do not depend on timing
  std::map<int, std::vector<int>> by_atom;
  for (int64_t q = 0; q < nrecv_; q++) {
    if (recv_index[q] < 0 || recv_index[q] >= nlocal) throw InvalidArgument("receive index outside the owned atoms");
    by_atom[recv_index[q]].push_back((int) q);
  }
  std::vector<int> target, off(1, 0), rows;
  for (const auto &kv : by_atom) {
    target.push_back(kv.first);
    rows.insert(rows.end(), kv.second.begin(), kv.second.end());
    off.push_back((int) rows.size());
  }
  ntarget_ = (int64_t) target.size();
  send_index_.set_label("exchange:index"); target_.set_label("exchange:index"); target_off_.set_label("exchange:index");
  target_rows_.set_label("exchange:index"); send_buf_.set_label("exchange:rows"); recv_buf_.set_label("exchange:rows");
  totals_.set_label("exchange:totals");
  send_index_.upload(sidx);
  target_.upload(target);
  target_off_.upload(off);
  target_rows_.upload(rows);
  send_buf_.ensure(3 * (size_t) std::max<int64_t>(nsend_, 1));
  recv_buf_.ensure(3 * (size_t) std::max<int64_t>(nrecv_, 1));
  totals_.ensure(8);
  GB_CUDA(cudaStreamSynchronize(dev().stream));    // the uploads read host vectors of this scope
  active_ = true;
}

void Exchange::run(double *d_forces, double *d_energy, double *d_virial)
{
  if (!active_) return;
  if (!g_comm || g_world != world_) throw DeviceError("the communicator of this exchange plan is gone");
  cudaStream_t st = dev().stream;
  Nccl &N = nccl();
  if (d_forces && nsend_ > 0) {
    pack_rows_kernel<<<nblocks(nsend_), 256, 0, st>>>(d_forces, send_index_.get(), send_buf_.get(), (long long) nsend_);
    GB_CUDA(cudaGetLastError());
    dev().launches++;
  }
  totals_kernel<<<1, 32, 0, st>>>(totals_.get(), d_energy, d_virial, 1);
  GB_CUDA(cudaGetLastError());
  dev().launches++;
  GB_NCCL(N.GroupStart());
  if (d_forces) {
    int64_t so = 0, ro = 0;
    for (int r = 0; r < world_; r++) {
      if (send_counts_[r] > 0) GB_NCCL(N.Send(send_buf_.get() + 3 * so, 3 * (size_t) send_counts_[r], ncclDouble, r, g_comm, st));
      if (recv_counts_[r] > 0) GB_NCCL(N.Recv(recv_buf_.get() + 3 * ro, 3 * (size_t) recv_counts_[r], ncclDouble, r, g_comm, st));
      so += send_counts_[r];
      ro += recv_counts_[r];
    }
  }
  GB_NCCL(N.AllReduce(totals_.get(), totals_.get(), 7, ncclDouble, ncclSum, g_comm, st));
  GB_NCCL(N.GroupEnd());
  if (d_forces && ntarget_ > 0) {
    add_rows_kernel<<<nblocks(ntarget_), 256, 0, st>>>(d_forces, target_.get(), target_off_.get(), target_rows_.get(), recv_buf_.get(),
                                                       (long long) ntarget_);
    GB_CUDA(cudaGetLastError());
    dev().launches++;
  }
  totals_kernel<<<1, 32, 0, st>>>(totals_.get(), d_energy, d_virial, 0);
  GB_CUDA(cudaGetLastError());
  dev().launches++;
}

}    // namespace gb
