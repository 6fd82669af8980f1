// cp.async build kernels for the difference inner steps (b - a).
#include "km_build_cpasync.cuh"
#include "km_build_cpasync_table.cuh"

namespace km {
namespace {
template <int INNER>
BuildKernelFn pick(bool avec, bool bvec) {
    if (avec && bvec) return build_cpasync_kernel<INNER, true, true, false>;
    if (avec) return build_cpasync_kernel<INNER, true, false, false>;
    if (bvec) return build_cpasync_kernel<INNER, false, true, false>;
    return build_cpasync_kernel<INNER, false, false, false>;
}
template <int INNER>
BuildKernelFn pick_symmetric(bool vec) {
    return vec ? build_cpasync_kernel<INNER, true, true, true> : build_cpasync_kernel<INNER, false, false, true>;
}
}  // namespace

BuildKernelFn cpasync_kernel_diff(int inner, bool avec, bool bvec, bool symmetric) {
    switch (inner) {
        case IN_DIFF_ABS: return symmetric ? pick_symmetric<IN_DIFF_ABS>(avec && bvec) : pick<IN_DIFF_ABS>(avec, bvec);
        case IN_DIFF_SQUARE: return symmetric ? pick_symmetric<IN_DIFF_SQUARE>(avec && bvec) : pick<IN_DIFF_SQUARE>(avec, bvec);
        case IN_DIFF_POW: return symmetric ? pick_symmetric<IN_DIFF_POW>(avec && bvec) : pick<IN_DIFF_POW>(avec, bvec);
        case IN_DIFF_NOOP: return symmetric ? nullptr : pick<IN_DIFF_NOOP>(avec, bvec);
        case IN_DIFF_SQRT: return symmetric ? nullptr : pick<IN_DIFF_SQRT>(avec, bvec);
    }
    return nullptr;
}
}  // namespace km
