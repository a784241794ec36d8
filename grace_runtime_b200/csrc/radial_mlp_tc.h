// Exact radial MLP of a layer on the tensor cores (tcgen05): see radial_mlp_tc.cu.
#pragma once

#include "device.h"
#include "model.h"

#include <vector>

namespace gb {

struct RadialMlpTCDev {
  const char *weights;    // W1 hi, W1 lo, W2 hi, W2 lo, W3 hi, W3 lo operand images (shared-memory layout)
  int weight_bytes;
  int n_out;              // outputs per bond, ordered [l][channel] like the radial tables
  int nrb, p, act;        // radial basis functions, envelope power, activation (0 SiLU, 1 tanh)
};

class RadialMlpTC {
 public:
  // shapes the kernel covers: up to 8 basis functions, two hidden layers of 64, a multiple of 32 outputs that fits
  static bool supported(const GraceModel &m, const std::vector<MlpLayer> &layers);
  static size_t smem_bytes(int n_out);
  void setup(const GraceModel &m, const std::vector<MlpLayer> &layers, int C);
  bool ready() const { return ready_; }
  int n_out() const { return d_.n_out; }
  // R[b][o], dR[b][o] = value and d/dx of the MLP at the scaled distances x[b] in (0, 1); device pointers, stream-ordered
  void run(const float *d_x, long long nb, float *d_R, float *d_dR);
  // raises DeviceError if a launch since the last check gave up waiting (synchronises the stream)
  void check();

 private:
  DBuf<char> weights_;
  DBuf<int> error_;
  RadialMlpTCDev d_{};
  bool ready_ = false;
};

}    // namespace gb
