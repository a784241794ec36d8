// Tensor-core form of the MV operations with shared weights (FC layers, non-element reduces, their adjoints) on chunk
// tensors in global memory: see mv_tc.cu.
#pragma once

#include "kernels.h"

namespace gb {

struct MVTCDev {
  const int *row_out;      // output function of each row
  const int *item_off;     // rows + 1
  const MVItem *items;     // as MVDev::items with `mat` = index of the matrix's operand image
  const char *images;      // per matrix: [n_out][K] tf32 hi image, then the lo image (canonical K-major layout)
  int n_out, nrows, nitems, accumulate, dst;
};

class MVTensorCore {
 public:
  // shapes the kernel covers: shared weights, every item with the same input width K in {8, 16, 32, 64}, n_out a
  // multiple of 16 up to 256, channel strides that keep rows 16-byte aligned, every row with at least one item
  static bool eligible(const MVOp &o, const std::vector<TensorSpec> &tensors);
  void setup(const MVOp &o);
  bool ready() const { return ready_; }
  // d: the operation's device tables (rows, offsets); tensors: device table of the chunk tensors; error: device flag
  // set when a bounded wait ran out
  void launch(const MVDev &d, const TensorDev *tensors, int ntensors, int NA, int na, int *error) const;

 private:
  bool ready_ = false;
  int K_ = 0, nitems_ = 0;
  DBuf<char> images_;
  DBuf<MVItem> items_;
};

}    // namespace gb
