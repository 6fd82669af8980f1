// Host-side helpers shared by the C-ABI translation units.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/kermac_b200.h"

namespace km {

// Stores a formatted message for kermac_b200_last_error() on this thread and
// returns `code`, so call sites can `return fail(KM_ERR_..., "...")`.
int fail(int code, const char* fmt, ...);

// Turns a cudaError_t into a return code (0 on success), recording the message.
int cuda_status(cudaError_t e, const char* what);

// True when the current device is compute capability 10.x; records an error otherwise.
int require_sm100();

// Number of SMs of the current device (cached per device).
int sm_count();

// Reads back and clears the wait-ran-out flag of the tensor-core matvec kernel
// (km_matvec.cu); the device must already be synchronised.  0 / 1, or -1 on error.
int matvec_take_wait_flag();

// Tensor-core form of the gradient contraction (km_grad_tensor.cu): tile extents the planner
// needs, the kernel's parameter block and its launcher.  norm_kind is a KmNormType or
// GT_NORM_SQRT (|x|^(1/2), chosen by the caller for a host scalar p = 1.5).
constexpr int GT_TM = 32;          // m per thread block
constexpr int GT_BK = 32;          // k rows per staged slab; k ranges of a split are multiples of it
// Channels per thread block: 16, 32 or 64, the smallest that holds them all (an MMA of up to 64 output
// columns holds the tensor pipe as long as one of 16, one of 128 only 1.4 times as long); n rows per thread
// block that go with it (tensor memory holds four row groups of 128 pairs at 16 and 32 channels, two at 64).
inline int gt_ot_for(int o) { return o > 32 ? 64 : (o > 16 ? 32 : 16); }
int gt_rg_for(int ot);                                 // row groups of 128 pairs per thread block
inline int gt_tn_for(int ot) { return 4 * gt_rg_for(ot); }
int gt_blocks_per_sm(int ot);
constexpr int GT_NORM_SQRT = 3;
struct GradTensorParams {
    int M, N, O, K, L;
    const float* A; long long lda, a_sl;
    const float* B; long long ldb, b_sl;
    const float* C; long long ldc, c_sl;
    const float* D; long long ldd, d_sl;
    float*       E; long long e_sn, e_so, e_sl;   // destination (out, or scratch when split)
    KmHyper p;
    int ot;                                         // channels per thread block: 16, 32 or 64
    int rg;                                         // row groups per thread block
    int tiles_m, tiles_n, o_chunks, splits;
    int k_per_split;
    long long split_stride;
    int c_vec;                                      // c rows can be read 16 bytes at a time
};
int grad_tensor_launch(const GradTensorParams& p, int norm_kind, cudaStream_t st);
// Reads back and clears the wait-ran-out flag of the tensor-core gradient kernel; the device
// must already be synchronised.  0 / 1, or -1 on error.
int grad_tensor_take_wait_flag();

inline long long ceil_div_ll(long long a, long long b) { return (a + b - 1) / b; }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Checks a KmHyper that is in use: a device vector needs a non-negative stride.
inline bool hyper_ok(const KmHyper& h) { return h.ptr == nullptr || h.batch_stride >= 0; }

}  // namespace km
