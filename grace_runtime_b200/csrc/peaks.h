// Measured compute peaks of the device (microbenchmarks, peaks.cu): the denominators of the compute-bound rooflines.
#pragma once

#include "device.h"

namespace gb {

// fp32 FMA rate of the SIMT lanes in TFLOP/s (2 flop per FMA), best of 3 launches after a warm-up launch;
// packed: the same arithmetic as two-wide fma.rn.f32x2 instructions
double measure_peak_fp32_tflops(bool packed = false);
// tf32 tensor-core rate in TFLOP/s: tcgen05.mma kind::tf32 M = 128, N = n (256: the peak; smaller N shows the
// instruction-rate limit of narrow tiles), operands in shared memory
double measure_peak_tf32_tflops(int n = 256);

}    // namespace gb
