// Lookup of the cp.async build-kernel instantiations.  The instantiations are
// spread over two translation units (difference and product inner steps) so they
// compile in parallel.
#pragma once

#include "km_build_params.cuh"

namespace km {

typedef void (*BuildKernelFn)(const BuildParams);

// `avec` / `bvec`: the operand may be staged with 16-byte copies.  `symmetric`: the
// one-triangle variant (a and b are the same matrix, so avec == bvec); nullptr for the
// inner steps that are not even in the difference.
BuildKernelFn cpasync_kernel_diff(int inner, bool avec, bool bvec, bool symmetric);
BuildKernelFn cpasync_kernel_dot(int inner, bool avec, bool bvec, bool symmetric);

}  // namespace km
