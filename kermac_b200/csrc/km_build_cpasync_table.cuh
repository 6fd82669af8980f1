// Lookup of the cp.async build-kernel instantiations.  The instantiations are
// spread over two translation units (difference and product inner steps) so they
// compile in parallel.
#pragma once

#include "km_build_params.cuh"

namespace km {

typedef void (*BuildKernelFn)(const BuildParams);

// `avec` / `bvec`: the operand may be staged with 16-byte copies.
BuildKernelFn cpasync_kernel_diff(int inner, bool avec, bool bvec);
BuildKernelFn cpasync_kernel_dot(int inner, bool avec, bool bvec);

}  // namespace km
