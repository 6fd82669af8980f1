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

inline long long ceil_div_ll(long long a, long long b) { return (a + b - 1) / b; }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Checks a KmHyper that is in use: a device vector needs a non-negative stride.
inline bool hyper_ok(const KmHyper& h) { return h.ptr == nullptr || h.batch_stride >= 0; }

}  // namespace km
