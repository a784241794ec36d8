// Device neighbour list of one structure or of a batch of structures (one concatenated CSR), and the per-call bond
// records.  The bond set equals the reference's cell-list search (python/src/neighbors.cpp:15-95,
// libgrace/include/grace/cell_list.h:39-152): bins in fractional coordinates of edge >= (cutoff + skin) / 2, wrapped
// in periodic directions, over the occupied range in open ones; atoms in stable bin order; every neighbour within the
// radius including periodic images and self-images; two atoms at distance zero are an error.
// Its device counterpart in the reference is NeighborListKK / BatchNeighborListKK
// (libgrace/include/grace/kk/neighbors_kk.h:118-294, 422-...).
#pragma once

#include "device.h"
#include "kernels.h"

#include <vector>

namespace gb {

struct NLStructHost {
  double cell[9], inv[9], lo[3], span[3], width[3];
  int nbin[3], reach[3], pbc[3];
  int bin_base, atom0, atom1;
};

class NeighborList {
 public:
  NeighborList();
  // (re)build for n atoms in nsys structures: d_pos [n][3] and d_mu [n] in the caller's order (device), natoms [nsys],
  // cells [nsys][9], pbc [nsys][3] on the host; radius = cutoff + skin
  void build(int nsys, const int *natoms, int64_t n, const double *d_pos, const int *d_mu, const double *cells,
             const unsigned char *pbc, double radius);
  // A caller's own list instead of a search (the engine interface of MD codes with ghost atoms,
  // libgrace/include/grace/kk/grace_2l_kk.h:97-119): nall atoms, local ones first; d_numneigh [nlocal] and the padded table
  // d_neighbors [nlocal][maxneigh] of indices into the nall atoms (device).  Ghosts are atoms of their own (no cell
  // shifts, no lists), so the list has no reverse-bond index: external() tells the engine to scatter bond forces with
  // atomic adds and to add the neighbours' message gradients atomically, as the reference's engines do.
  void adopt(int nlocal, int nall, const int *d_mu, const int *d_numneigh, const int *d_neighbors, int maxneigh);
  bool external() const { return external_; }
  // true when an atom moved more than half the skin since the build (device max-reduce, one int read back)
  bool moved_beyond(const double *d_pos, double half_skin);
  // the same check without the read-back: sets `bit` of the caller's device flag
  void moved_launch(const double *d_pos, double half_skin, int *d_flag, int bit);
  // positions of this call into list order (wrapped with the images of the build) and the bonds inside the pair
  // cutoffs rcsq [n_elements][n_elements]: records compacted to the front of each atom's slots; bond forces of the
  // slots left out are zeroed in fv
  void prepare(const double *d_pos, const double *d_rcsq, int n_elements, float *fv);

  int64_t n() const { return n_; }
  int64_t nslots() const { return nslots_; }
  int nsys() const { return nsys_; }
  BondsDev bonds() const;
  const int *perm() const { return perm_.get(); }         // list order -> caller index
  const int *mu_sorted() const { return mu_s_.get(); }
  const int *rev() const { return rev_.get(); }
  const long long *off() const { return off_.get(); }
  const int *seg() const { return seg_.get(); }            // [nsys + 1] atom ranges of the structures in list order
  // error bits raised by prepare() since it was called (2: a bond of length 0); synchronises the stream
  int take_flag();
  void release();
  size_t bytes() const;
  // diagnostics: the list of the last build (radius cutoff + skin) on the host, in the caller's atom order and frame:
  // per slot the atoms i, j and the integer cell shift S [3] with bond vector x_j - x_i + S cell
  void export_host(std::vector<int> &bi, std::vector<int> &bj, std::vector<int> &bS) const;

 private:
  int64_t n_ = 0, nslots_ = 0;
  int nsys_ = 0;
  bool external_ = false;
  std::vector<NLStructHost> st_;
  DBuf<NLStructHost> d_st_;
  DBuf<double> frac_, xs_, xbuild_, lohi_;
  DBuf<int> img_, img_s_, sid_, sid_s_, binid_, b3_s_, count_, fill_, members_, perm_, mu_s_, cnt_full_, cnt_, nbr_j_,
      nbr_S_, rev_, cslot_, seg_, flag_;
  DBuf<long long> start_, off_, scan_tmp_;
  DBuf<float4> rec_;
};

// exclusive scan of n int32 counts into n + 1 int64 offsets (tmp: scratch of at least n / 2048 + 2 values)
void launch_scan(const int *in, long long *out, long long *tmp, int64_t n);

}    // namespace gb
