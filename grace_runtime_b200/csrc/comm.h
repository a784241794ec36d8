// Multi-GPU plumbing of the library: one process per GPU, an NCCL communicator between the processes, and the
// per-step exchange of a domain-decomposed System (ghost force rows back to their owners, energy and virial summed
// over the ranks) on the library's own stream.  NCCL is loaded at run time (libnccl.so.2): single-GPU users need no
// NCCL at all.  The reference's counterpart is the engine interface LAMMPS drives with ghost atoms and forward /
// reverse communication (libgrace/include/grace/system.h:53-64, libgrace/include/grace/kk/grace_2l_kk.h:136-153).
#pragma once

#include "device.h"

#include <cstdint>
#include <vector>

namespace gb {

// process-wide communicator
void comm_unique_id(void *id128);
void comm_init(const void *id128, int rank, int world);
void comm_finalize();
int comm_rank();     // -1 without a communicator
int comm_size();     // 0 without a communicator

// exchange plan of one System: set once per decomposition, run after every evaluation
class Exchange {
 public:
  // send_index: sub-system indices of this rank's ghost atoms grouped by owner rank (send_counts[r] rows go to r);
  // recv_index: for the rows arriving from rank 0, 1, ... in that order, the owned atom each one adds to
  void setup(int n, int nlocal, const int32_t *send_counts, const int32_t *send_index, const int32_t *recv_counts,
             const int32_t *recv_index);
  bool active() const { return active_; }
  int n() const { return n_; }
  // forces [n][3] of the sub-system (device): ghost rows leave, the rows received are added to the owned rows in a
  // fixed order; energy [1] and virial [6] (device, null: skipped) become the sums over the ranks
  void run(double *d_forces, double *d_energy, double *d_virial);

 private:
  bool active_ = false;
  int n_ = 0, nlocal_ = 0, world_ = 0;
  std::vector<int> send_counts_, recv_counts_;
  int64_t nsend_ = 0, nrecv_ = 0, ntarget_ = 0;
  DBuf<int> send_index_, target_, target_off_, target_rows_;
  DBuf<double> send_buf_, recv_buf_, totals_;
};

}    // namespace gb
