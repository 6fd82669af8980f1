// kermac_b200_build_kernel: validation, operand exchange for n-contiguous outputs,
// variant choice and launch.  Host-side counterpart of the second half of the
// reference's run_kernel (src/kermac/build_a_kernel.py:237-392).
#include <cstring>

#include "km_build_cpasync_table.cuh"
#include "km_build_tma.cuh"
#include "km_host.h"

namespace km {

namespace {

BuildKernelFn cpasync_kernel(int inner, bool avec, bool bvec, bool symmetric) {
    return inner < IN_DOT_NOOP ? cpasync_kernel_diff(inner, avec, bvec, symmetric)
                               : cpasync_kernel_dot(inner, avec, bvec, symmetric);
}

// One of the two layouts TensorStats accepts (src/kermac/common.py:96-102):
// the stride along `rows` or along `cols` is 1 and the other spans the unit one.
bool layout_ok(long long rows, long long cols, long long s_row, long long s_col) {
    if (rows <= 0 || cols <= 0) return true;
    if (s_col == 1 && s_row >= cols) return true;
    if (s_row == 1 && s_col >= rows) return true;
    return false;
}

struct BuildPlan {
    BuildParams p;
    bool avec, bvec;
    bool swapped;
    int  variant;
};

int make_plan(const KmBuildArgs* a, BuildPlan* plan) {
    if (!a) return fail(KM_ERR_NULL_POINTER, "args is NULL");
    if (a->m < 0 || a->n < 0 || a->k < 0 || a->l < 1)
        return fail(KM_ERR_BAD_SHAPE, "bad extents m=%d n=%d k=%d l=%d", a->m, a->n, a->k, a->l);
    const bool empty = (a->m == 0 || a->n == 0);
    if (!empty && (!a->out || ((!a->a || !a->b) && a->k > 0)))
        return fail(KM_ERR_NULL_POINTER, "a, b and out must be device pointers");
    if (a->inner_operator < 0 || a->inner_operator > KM_INNER_DOT)
        return fail(KM_ERR_BAD_ENUM, "inner_operator %d is not a KmInnerOperator", a->inner_operator);
    if (a->inner_power < 0 || a->inner_power > KM_POW_POW)
        return fail(KM_ERR_BAD_ENUM, "inner_power %d is not a KmPowerType", a->inner_power);
    if (a->outer_power < 0 || a->outer_power > KM_POW_POW)
        return fail(KM_ERR_BAD_ENUM, "outer_power %d is not a KmPowerType", a->outer_power);
    if (a->kernel_type < 0 || a->kernel_type > KM_KERNEL_GAUSSIAN)
        return fail(KM_ERR_BAD_ENUM, "kernel_type %d is not a KmKernelType", a->kernel_type);
    if (a->variant < KM_VARIANT_AUTO || a->variant > KM_VARIANT_TMA)
        return fail(KM_ERR_BAD_ENUM, "variant %d is not a KM_VARIANT_*", a->variant);
    if (!layout_ok(a->m, a->k, a->a_stride_m, a->a_stride_k))
        return fail(KM_ERR_BAD_STRIDE, "a has a non-standard memory layout: strides (%lld, %lld) for shape (%d, %d)",
                    (long long)a->a_stride_m, (long long)a->a_stride_k, a->m, a->k);
    if (!layout_ok(a->n, a->k, a->b_stride_n, a->b_stride_k))
        return fail(KM_ERR_BAD_STRIDE, "b has a non-standard memory layout: strides (%lld, %lld) for shape (%d, %d)",
                    (long long)a->b_stride_n, (long long)a->b_stride_k, a->n, a->k);
    if (!layout_ok(a->m, a->n, a->out_stride_m, a->out_stride_n))
        return fail(KM_ERR_BAD_STRIDE, "out has a non-standard memory layout: strides (%lld, %lld) for shape (%d, %d)",
                    (long long)a->out_stride_m, (long long)a->out_stride_n, a->m, a->n);
    if (a->a_stride_l < 0 || a->b_stride_l < 0 || a->out_stride_l < 0)
        return fail(KM_ERR_BAD_STRIDE, "batch strides must be non-negative");
    if (a->l > 1 && a->out_stride_l == 0)
        return fail(KM_ERR_BAD_STRIDE, "out cannot be broadcast over the batch");
    if (!hyper_ok(a->p_inner) || !hyper_ok(a->p_outer) || !hyper_ok(a->bandwidth) || !hyper_ok(a->regularization))
        return fail(KM_ERR_BAD_HYPERPARAM, "hyper-parameter vectors need a non-negative batch stride");

    BuildParams& p = plan->p;
    std::memset(&p, 0, sizeof(p));
    // An out whose n stride is 1 is written by the same kernel after exchanging the
    // roles of a and b (the kernel always writes its first tile dimension contiguously).
    const bool out_m_contig = (a->out_stride_m == 1 && (a->out_stride_n >= a->m || a->n <= 1));
    plan->swapped           = !out_m_contig;
    p.K = a->k;
    p.L = a->l;
    if (!plan->swapped) {
        p.M = a->m; p.N = a->n;
        p.A = a->a; p.a_sm = a->a_stride_m; p.a_sk = a->a_stride_k; p.a_sl = a->a_stride_l;
        p.B = a->b; p.b_sn = a->b_stride_n; p.b_sk = a->b_stride_k; p.b_sl = a->b_stride_l;
        p.c_ld = a->out_stride_n;
        p.reg_off_m = a->reg_off_x; p.reg_off_n = a->reg_off_y;
        p.sgn = 1.0f;
    } else {
        p.M = a->n; p.N = a->m;
        p.A = a->b; p.a_sm = a->b_stride_n; p.a_sk = a->b_stride_k; p.a_sl = a->b_stride_l;
        p.B = a->a; p.b_sn = a->a_stride_m; p.b_sk = a->a_stride_k; p.b_sl = a->a_stride_l;
        p.c_ld = a->out_stride_m;
        p.reg_off_m = a->reg_off_y; p.reg_off_n = a->reg_off_x;
        p.sgn = -1.0f;
    }
    p.C    = a->out;
    p.c_sl = a->out_stride_l;
    p.inner_id = inner_id(a->inner_operator, a->inner_power);
    if (p.inner_id < 0) return fail(KM_ERR_BAD_ENUM, "unsupported inner operator / power pair");
    p.outer_power    = a->outer_power;
    p.kernel_type    = a->kernel_type;
    p.p_inner        = a->p_inner;
    p.p_outer        = a->p_outer;
    p.bandwidth      = a->bandwidth;
    p.regularization = a->regularization;
    p.epsilon        = a->epsilon;
    p.tiles_m        = (int)ceil_div_ll(p.M, BUILD_TILE);
    p.tiles_n        = (int)ceil_div_ll(p.N, BUILD_TILE);
    p.panel          = 16;
    if ((long long)p.tiles_m * p.tiles_n > 0x7fffffffLL) return fail(KM_ERR_TOO_LARGE, "too many output tiles");
    p.c_vec4 = aligned16(p.C) && (p.c_ld % 4 == 0) && (p.c_sl % 4 == 0);
    if (a->out_multicast != 0 && a->out_multicast != 1)
        return fail(KM_ERR_BAD_ENUM, "out_multicast must be 0 or 1");
    p.c_multicast = a->out_multicast;
    const int total_tiles = p.tiles_m * p.tiles_n;
    if (a->tile_first < 0 || a->tile_count < 0 || a->tile_first > total_tiles ||
        (long long)a->tile_first + a->tile_count > total_tiles)
        return fail(KM_ERR_BAD_SHAPE, "tile range [%d, %d + %d) is outside the %d tiles of this problem", a->tile_first,
                    a->tile_first, a->tile_count, total_tiles);
    p.tile_first = a->tile_first;
    p.tile_count = a->tile_count > 0 ? a->tile_count : total_tiles - a->tile_first;
    const bool all_tiles = (p.tile_first == 0 && p.tile_count == total_tiles);

    // a and b the same matrix, a chain that does not change when m and n trade places (the
    // diagonal rule included): compute the tiles on and above the diagonal and mirror them.
    // The mirrored values are the same bits the skipped tiles would have produced: the sum
    // over k runs in the same order over the same terms.
    if (a->symmetry < KM_SYMMETRY_AUTO || a->symmetry > KM_SYMMETRY_OFF)
        return fail(KM_ERR_BAD_ENUM, "symmetry must be KM_SYMMETRY_AUTO or KM_SYMMETRY_OFF");
    const bool even_chain = (p.inner_id == IN_DIFF_ABS || p.inner_id == IN_DIFF_SQUARE || p.inner_id == IN_DIFF_POW ||
                             p.inner_id >= IN_DOT_NOOP);
    p.symmetric = (a->symmetry == KM_SYMMETRY_AUTO) && even_chain && p.M == p.N && p.tiles_m > 1 && p.A == p.B &&
                  p.a_sm == p.b_sn && p.a_sk == p.b_sk && p.a_sl == p.b_sl && p.reg_off_m == p.reg_off_n &&
                  !p.c_multicast && all_tiles;

    plan->avec = (p.a_sm == 1) && aligned16(p.A) && (p.a_sk % 4 == 0 || p.K <= 1) && (p.a_sl % 4 == 0);
    plan->bvec = (p.b_sn == 1) && aligned16(p.B) && (p.b_sk % 4 == 0 || p.K <= 1) && (p.b_sl % 4 == 0);

    const bool tma_ok = plan->avec && plan->bvec && tma_supported(p);
    int variant       = a->variant;
    if (variant == KM_VARIANT_TMA && !tma_ok)
        return fail(KM_ERR_BAD_STRIDE, "the TMA variant needs m-contiguous, 16-byte aligned a and b with 16-byte pitches");
    if (variant == KM_VARIANT_AUTO) variant = (tma_ok && tma_preferred(p)) ? KM_VARIANT_TMA : KM_VARIANT_CPASYNC;
    plan->variant = variant;
    return 0;
}

const char* const kInnerNames[IN_COUNT] = {"diff_abs", "diff_square", "diff_pow", "diff_noop", "diff_sqrt",
                                           "dot_noop", "dot_abs",     "dot_square", "dot_sqrt", "dot_pow"};

}  // namespace
}  // namespace km

extern "C" int kermac_b200_build_kernel(const KmBuildArgs* args, void* stream) {
    using namespace km;
    BuildPlan plan;
    if (int rc = make_plan(args, &plan)) return rc;
    BuildParams& p = plan.p;
    if (p.M == 0 || p.N == 0 || p.tile_count == 0) return 0;
    if (int rc = require_sm100()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    if (plan.variant == KM_VARIANT_TMA) return launch_build_tma(p, st);

    BuildKernelFn fn = cpasync_kernel(p.inner_id, plan.avec, plan.bvec, p.symmetric != 0);
    if (!fn) return fail(KM_ERR_INTERNAL, "no kernel for inner id %d", p.inner_id);
    if (int rc = cuda_status(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, BUILD_CPA_SMEM_BYTES),
                             "cudaFuncSetAttribute(build_cpasync_kernel)"))
        return rc;
    const int total_l = p.L;
    for (int l0 = 0; l0 < total_l; l0 += 65535) {
        BuildParams q = p;
        q.L           = (total_l - l0 < 65535) ? (total_l - l0) : 65535;
        q.A += (long long)l0 * p.a_sl;
        q.B += (long long)l0 * p.b_sl;
        q.C += (long long)l0 * p.c_sl;
        if (q.p_inner.ptr) q.p_inner.ptr += (long long)l0 * q.p_inner.batch_stride;
        if (q.p_outer.ptr) q.p_outer.ptr += (long long)l0 * q.p_outer.batch_stride;
        if (q.bandwidth.ptr) q.bandwidth.ptr += (long long)l0 * q.bandwidth.batch_stride;
        if (q.regularization.ptr) q.regularization.ptr += (long long)l0 * q.regularization.batch_stride;
        dim3 grid((unsigned)q.tile_count, (unsigned)q.L, 1);
        fn<<<grid, BUILD_CPA_THREADS, BUILD_CPA_SMEM_BYTES, st>>>(q);
        if (int rc = cuda_status(cudaGetLastError(), "launch of build_cpasync_kernel")) return rc;
    }
    return 0;
}

extern "C" int64_t kermac_b200_build_tile_count(const KmBuildArgs* args) {
    using namespace km;
    if (!args) return fail(KM_ERR_NULL_POINTER, "args is NULL");
    KmBuildArgs whole = *args;
    whole.tile_first = whole.tile_count = 0;
    BuildPlan plan;
    if (int rc = make_plan(&whole, &plan)) return rc;
    return (int64_t)plan.p.tiles_m * plan.p.tiles_n;
}

extern "C" int kermac_b200_describe_variant(const KmBuildArgs* args, char* buf, int32_t buf_len) {
    using namespace km;
    if (!buf || buf_len <= 0) return fail(KM_ERR_NULL_POINTER, "buf is NULL or empty");
    BuildPlan plan;
    if (int rc = make_plan(args, &plan)) return rc;
    const BuildParams& p = plan.p;
    snprintf(buf, (size_t)buf_len,
             "build_kernel variant=%s inner=%s outer_power=%d kernel_type=%d exchanged=%d a_vec16=%d b_vec16=%d "
             "out_vec16=%d tiles=%dx%d batches=%d symmetric=%d tile_range=%d+%d",
             plan.variant == KM_VARIANT_TMA ? "tma" : "cpasync", kInnerNames[p.inner_id], p.outer_power, p.kernel_type,
             plan.swapped ? 1 : 0, plan.avec ? 1 : 0, plan.bvec ? 1 : 0, p.c_vec4, p.tiles_m, p.tiles_n, p.L, p.symmetric,
             p.tile_first, p.tile_count);
    return 0;
}
