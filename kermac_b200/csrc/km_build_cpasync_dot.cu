// cp.async build kernels for the product inner steps (b * a).
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

BuildKernelFn cpasync_kernel_dot(int inner, bool avec, bool bvec, bool symmetric) {
    switch (inner) {
        case IN_DOT_NOOP: return symmetric ? pick_symmetric<IN_DOT_NOOP>(avec && bvec) : pick<IN_DOT_NOOP>(avec, bvec);
        case IN_DOT_ABS: return symmetric ? pick_symmetric<IN_DOT_ABS>(avec && bvec) : pick<IN_DOT_ABS>(avec, bvec);
        case IN_DOT_SQUARE: return symmetric ? pick_symmetric<IN_DOT_SQUARE>(avec && bvec) : pick<IN_DOT_SQUARE>(avec, bvec);
        case IN_DOT_SQRT: return symmetric ? pick_symmetric<IN_DOT_SQRT>(avec && bvec) : pick<IN_DOT_SQRT>(avec, bvec);
        case IN_DOT_POW: return symmetric ? pick_symmetric<IN_DOT_POW>(avec && bvec) : pick<IN_DOT_POW>(avec, bvec);
    }
    return nullptr;
}
}  // namespace km
