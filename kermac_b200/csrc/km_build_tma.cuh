// Kernel-matrix build, TMA staged (declarations; implementation in km_build_tma.cu).
#pragma once

#include "km_build_params.cuh"

namespace km {

// True when the operands of `p` satisfy what a tiled TMA copy needs (both operands
// contiguous along their tile dimension, 16-byte aligned base, pitches and batch
// strides that are multiples of 16 bytes) and the inner step has a TMA kernel.
bool tma_supported(const BuildParams& p);

// True when the TMA variant is expected to be the faster one for this problem.
bool tma_preferred(const BuildParams& p);

int launch_build_tma(const BuildParams& p, cudaStream_t stream);

}  // namespace km
