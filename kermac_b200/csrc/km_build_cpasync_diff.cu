// cp.async build kernels for the difference inner steps (b - a).
#include "km_build_cpasync.cuh"
#include "km_build_cpasync_table.cuh"

namespace km {
namespace {
template <int INNER>
BuildKernelFn pick(bool avec, bool bvec) {
    if (avec && bvec) return build_cpasync_kernel<INNER, true, true>;
    if (avec) return build_cpasync_kernel<INNER, true, false>;
    if (bvec) return build_cpasync_kernel<INNER, false, true>;
    return build_cpasync_kernel<INNER, false, false>;
}
}  // namespace

BuildKernelFn cpasync_kernel_diff(int inner, bool avec, bool bvec) {
    switch (inner) {
        case IN_DIFF_ABS: return pick<IN_DIFF_ABS>(avec, bvec);
        case IN_DIFF_SQUARE: return pick<IN_DIFF_SQUARE>(avec, bvec);
        case IN_DIFF_POW: return pick<IN_DIFF_POW>(avec, bvec);
        case IN_DIFF_NOOP: return pick<IN_DIFF_NOOP>(avec, bvec);
        case IN_DIFF_SQRT: return pick<IN_DIFF_SQRT>(avec, bvec);
    }
    return nullptr;
}
}  // namespace km
