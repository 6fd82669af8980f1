// cp.async build kernels for the product inner steps (b * a).
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

BuildKernelFn cpasync_kernel_dot(int inner, bool avec, bool bvec) {
    switch (inner) {
        case IN_DOT_NOOP: return pick<IN_DOT_NOOP>(avec, bvec);
        case IN_DOT_ABS: return pick<IN_DOT_ABS>(avec, bvec);
        case IN_DOT_SQUARE: return pick<IN_DOT_SQUARE>(avec, bvec);
        case IN_DOT_SQRT: return pick<IN_DOT_SQRT>(avec, bvec);
        case IN_DOT_POW: return pick<IN_DOT_POW>(avec, bvec);
    }
    return nullptr;
}
}  // namespace km
