// Kernel-matrix build, TMA staged (declarations; implementation in km_build_tma.cu).
#pragma once

#include <cuda.h>

#include "km_build_params.cuh"

namespace km {

// True when the operands of `p` satisfy what a tiled TMA copy needs (both operands
// contiguous along their tile dimension, 16-byte aligned base, pitches and batch
// strides that are multiples of 16 bytes) and the inner step has a TMA kernel.
bool tma_supported(const BuildParams& p);

// True when the TMA variant is expected to be the faster one for this problem.
bool tma_preferred(const BuildParams& p);

int launch_build_tma(const BuildParams& p, cudaStream_t stream);

// Describes one fp32 operand as a rank-3 tensor (tile dimension, k, batch) with a box of
// 128 x box_k x 1 elements.  `map` is a CUtensorMap.  Returns 0 or a KM_ERR_* code.
int encode_tma_operand(CUtensorMap* map, const float* base, int extent, int K, int L, long long s_k, long long s_l,
                       int box_k);
// Describes an fp32 matrix (inner extent contiguous, `outer` rows s_outer elements apart, L batch entries
// s_l apart, s_l == 0 for a broadcast one) as a rank-3 tensor with a box of box_inner x box_outer x 1.
// The base must be 16-byte aligned, s_outer and s_l multiples of 4 elements, box_inner * 4 a multiple of 16.
int encode_tma_box(CUtensorMap* map, const float* base, int inner, int outer, int L, long long s_outer, long long s_l,
                   int box_inner, int box_outer);
// True when an operand with these strides can be described that way.
bool tma_operand_ok(const float* base, long long s_t, long long s_k, long long s_l, int K, int L);

}  // namespace km
