/*
 * kermac_b200 C-ABI: the drop-in boundary for kermac's fused distance hot path
 * on NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain pointers, sizes and element strides; there are no
 * torch types in any signature.  All device pointers must belong to the CUDA
 * device that is current when the call is made, and `stream` is a cudaStream_t
 * (pass NULL for the legacy default stream).  Calls are asynchronous with respect
 * to the host: they enqueue work on `stream` and return.
 *
 * Return value convention (all `int` functions unless stated otherwise):
 *     0   success, work enqueued
 *   < 0   a precondition was rejected, nothing was launched (KM_ERR_*)
 *   > 0   a CUDA runtime error code (cudaError_t) from the launch
 * `kermac_b200_last_error()` returns a thread-local human readable message for the
 * last non-zero return on the calling thread.
 *
 * Reference interfaces replaced (paths inside the kermac project):
 *   - kermac_b200_build_kernel   <- the launch of `cute_build_kernel<...>` made by
 *                                   src/kermac/build_a_kernel.py:342-392 (21 kernel
 *                                   arguments packed at :378-390), kernel entry
 *                                   include/build_a_kernel.cuh:541-623
 *   - kermac_b200_cdist_grad     <- the launch of `cute_norm_kernel_gradient<...>`
 *                                   made by src/kermac/cdist_grad.py:181-237
 *                                   (arguments packed at :226-235), kernel entry
 *                                   include/p_norm_gradient.cuh:407-497
 *   - kermac_b200_kernel_matvec  <- no single reference call; it fuses
 *                                   run_kernel(...) (build_a_kernel.py:158-394)
 *                                   with the coefficient product that callers do
 *                                   afterwards (examples/linalg.py:55-119)
 *   - kermac_b200_describe_variant <- the `debug=True` print of the chosen
 *                                   instantiation, build_a_kernel.py:345-346
 *   - kermac_b200_abi_version / kermac_b200_build_id <- the version part of the
 *                                   JIT cache key, module_cache/function_db_key.py:19-28
 */
#ifndef KERMAC_B200_H
#define KERMAC_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KERMAC_B200_ABI_VERSION 6

/* Rejected preconditions (negative return codes). */
#define KM_ERR_NULL_POINTER   (-1)
#define KM_ERR_BAD_SHAPE      (-2)
#define KM_ERR_BAD_STRIDE     (-3)
#define KM_ERR_BAD_ENUM       (-4)
#define KM_ERR_BAD_HYPERPARAM (-5)
#define KM_ERR_TOO_LARGE      (-6)
#define KM_ERR_NOT_SM100      (-7)
#define KM_ERR_INTERNAL       (-8)

/* Mirrors InnerOperator, src/kermac/build_a_kernel.py:15-17 */
enum KmInnerOperator { KM_INNER_DIFF = 0, KM_INNER_DOT = 1 };
/* Mirrors PowerType, src/kermac/build_a_kernel.py:21-26 */
enum KmPowerType { KM_POW_NOOP = 0, KM_POW_ABS = 1, KM_POW_SQUARE = 2, KM_POW_SQRT = 3, KM_POW_POW = 4 };
/* Mirrors KernelType, src/kermac/build_a_kernel.py:30-33 */
enum KmKernelType { KM_KERNEL_NONE = 0, KM_KERNEL_LAPLACE = 1, KM_KERNEL_GAUSSIAN = 2 };
/* Mirrors NormType, include/kermac_internal_common.cuh:41-45 */
enum KmNormType { KM_NORM_L1 = 0, KM_NORM_L2 = 1, KM_NORM_P = 2 };

/*
 * A hyper-parameter that is either one host scalar (ptr == NULL, `value` used for
 * every batch entry) or a device vector read as ptr[l * batch_stride] for batch
 * entry l (batch_stride 0 = one device scalar broadcast over the batch).
 * Replaces the 0-dim / 1-dim device tensors of build_a_kernel.py:263-310,364-373;
 * a host scalar costs no allocation and no copy.
 */
typedef struct KmHyper {
    const float* ptr;
    float        value;
    int64_t      batch_stride;
} KmHyper;

/*
 * out[l, m, n] = Kfn( outer( sum_k inner( b[l, n, k] (-|*) a[l, m, k] ) ) )
 *
 * Strides are in elements and may describe either majorness of each operand
 * (one of the two matrix strides must be 1, the other >= the extent it spans;
 * the rule of TensorStats, src/kermac/common.py:96-102).  A batch stride of 0
 * broadcasts the operand over the batch.  The difference is always b - a,
 * whatever the output layout, and the diagonal rule is
 * reg_off_x + m == reg_off_y + n.
 */
typedef struct KmBuildArgs {
    int32_t m, n, k, l;
    const float* a; int64_t a_stride_m, a_stride_k, a_stride_l;
    const float* b; int64_t b_stride_n, b_stride_k, b_stride_l;
    float*       out; int64_t out_stride_m, out_stride_n, out_stride_l;
    int32_t inner_operator;   /* KmInnerOperator */
    int32_t inner_power;      /* KmPowerType */
    int32_t outer_power;      /* KmPowerType */
    int32_t kernel_type;      /* KmKernelType */
    KmHyper p_inner;          /* used when inner_power == KM_POW_POW */
    KmHyper p_outer;          /* used when outer_power == KM_POW_POW */
    KmHyper bandwidth;        /* used when kernel_type != KM_KERNEL_NONE */
    KmHyper regularization;   /* used when kernel_type != KM_KERNEL_NONE */
    int32_t reg_off_x, reg_off_y;
    float   epsilon;          /* used when kernel_type != KM_KERNEL_NONE */
    int32_t variant;          /* 0 = automatic; otherwise force a kernel variant (KM_VARIANT_*) */
    int32_t out_multicast;    /* 0: `out` is ordinary device memory.  1: `out` is the multicast address of an
                                 NVSwitch multicast object that every GPU of the group has bound to its own result
                                 buffer (e.g. torch symmetric memory's multicast_ptr): results are written with
                                 multimem.st, so each GPU's buffer receives them while the kernel computes.  The
                                 caller synchronises the GPUs afterwards.  No reference counterpart. */
    int32_t symmetry;         /* KM_SYMMETRY_AUTO: when a and b are the same matrix (same pointer, strides and
                                 extent), reg_off_x == reg_off_y and the chain is even in the difference (|.|,
                                 square, |.|^p, or any product), only the tiles on and above the diagonal are
                                 computed and each is also written transposed: half the arithmetic, bit-identical
                                 results (equal to rounding for |.|^p, whose exp2 takes one of two routes).  KM_SYMMETRY_OFF computes every tile.  The reference declares a Symmetry
                                 enum (src/kermac/build_a_kernel.py:35-37) that nothing uses. */
    int32_t tile_first;       /* This call computes only the output tiles [tile_first, tile_first + tile_count) of */
    int32_t tile_count;       /* the launcher's linear order of 128 x 128 tiles (kermac_b200_build_tile_count gives
                                 the total); tile_count 0 = every tile from tile_first on.  Calls whose ranges
                                 partition [0, total) together write every element of `out` exactly once, which
                                 is how several GPUs share one problem in equal parts whatever its shape (with
                                 out_multicast each GPU's tiles land in every GPU's buffer).  A partial range
                                 switches the symmetric plan off.  The reference always launches the full grid
                                 (src/kermac/build_a_kernel.py:348-353). */
} KmBuildArgs;

#define KM_SYMMETRY_AUTO 0
#define KM_SYMMETRY_OFF  1

/* Kernel variants of kermac_b200_build_kernel (for benchmarks and tests). */
#define KM_VARIANT_AUTO     0
#define KM_VARIANT_CPASYNC  1   /* cp.async staged, any layout */
#define KM_VARIANT_TMA      2   /* TMA + mbarrier, needs m-contiguous 16-byte aligned a and b */

int kermac_b200_build_kernel(const KmBuildArgs* args, void* stream);

/* Number of 128 x 128 output tiles of one batch entry of this problem: the extent of the
 * linear tile order that tile_first / tile_count index.  Negative KM_ERR_* code when the
 * arguments are rejected.  Counterpart of the grid computation at
 * src/kermac/build_a_kernel.py:348-353. */
int64_t kermac_b200_build_tile_count(const KmBuildArgs* args);

/*
 * out[l, o, n, m] = sum_k c[l, o, k] * a[l, k, m] * g(d[l, n, m] - b[l, n, k])
 *   g(x) = copysign(1, x)                       (KM_NORM_L1)
 *   g(x) = x                                    (KM_NORM_L2)
 *   g(x) = copysign(1, x) * |x|^(p - 1)         (KM_NORM_P, p read per batch entry)
 * a, d and out are m-contiguous, b and c are k-contiguous (last stride 1, as
 * src/kermac/cdist_grad.py:156-166 demands); ld* are the row pitches in elements.
 * `scratch` may be NULL; when given it must hold `scratch_bytes` bytes of device
 * memory, which lets the launcher split the contracted k range over several
 * thread blocks (see kermac_b200_cdist_grad_scratch_bytes).
 * `contraction` (KM_CONTRACT_*, defined below with kermac_b200_kernel_matvec) selects where the
 * products with c run: KM_CONTRACT_FP32 as packed FP32 FMAs; KM_CONTRACT_TENSOR on the tcgen05
 * tensor cores, up to 64 channels at a time, as three tf32 products per term (weights and
 * coefficients split into a tf32 head and an fp32 remainder, accumulation chains of 128 k added up
 * in fp32: fp32-level accuracy, not the FP32 kernel's bits); KM_CONTRACT_AUTO takes the tensor
 * cores from 17 channels and 256 k on.  The weights a * g(d - b) are computed in FP32 either way.  A bounded
 * wait inside the tensor-core kernel that runs out raises kermac_b200_device_error_flag().
 */
typedef struct KmGradArgs {
    int32_t m, n, o, k, l;
    const float* a; int64_t lda, a_stride_l;      /* a[l][k][m] */
    const float* b; int64_t ldb, b_stride_l;      /* b[l][n][k] */
    const float* c; int64_t ldc, c_stride_l;      /* c[l][o][k] */
    const float* d; int64_t ldd, d_stride_l;      /* d[l][n][m] */
    float*       out; int64_t out_stride_n, out_stride_o, out_stride_l;  /* out[l][o][n][m] */
    int32_t norm_type;        /* KmNormType */
    KmHyper p;                /* used when norm_type == KM_NORM_P */
    void*   scratch; int64_t scratch_bytes;
    int32_t split_k;          /* 0 = automatic (1 when scratch is NULL) */
    int32_t contraction;      /* KM_CONTRACT_*: where the channel products run (see below) */
} KmGradArgs;

int kermac_b200_cdist_grad(const KmGradArgs* args, void* stream);

/* Bytes of scratch that let kermac_b200_cdist_grad use its preferred k split for
 * this problem (0 when no split is useful). */
int64_t kermac_b200_cdist_grad_scratch_bytes(const KmGradArgs* args);

/*
 * Same computation and arguments as kermac_b200_cdist_grad, for callers that cannot
 * allocate device memory where they call it (a plugin inside another runtime's fixed
 * memory pool, a latency-bound loop that must not enter an allocator, a foreign-function
 * layer that can only forward the pointers it was given).  The partial sums of the k
 * split go to an array that is part of the library image, KM_GRAD_STATIC_SCRATCH_BYTES
 * large, which every GPU that loads the library holds until the process exits.
 * args->scratch and args->scratch_bytes are ignored.  The library makes no allocator call;
 * the array itself is placed by the CUDA runtime when it loads the module on a device, which
 * happens at the latest during the first call there, so make one warm-up call per device
 * outside any region that must not reserve device memory.
 *   - An explicit args->split_k > 1 whose partial sums need more than
 *     KM_GRAD_STATIC_SCRATCH_BYTES is rejected with KM_ERR_TOO_LARGE.  With split_k = 0 the
 *     automatic split is reduced to the largest one that fits, down to a single pass (the same
 *     thing kermac_b200_cdist_grad does when the caller's scratch is too small); split_k = 1
 *     always fits (single pass, no scratch).
 *   - All calls share the one array and it keeps the previous call's contents.  Nothing
 *     in it needs clearing (each call writes every partial it later reads), but calls that
 *     overlap on the GPU race on it: order them on one stream or with events.
 *   - The first call on each device looks up the array's device address with the CUDA
 *     runtime; make that first call outside any stream capture.  The address is kept for the
 *     life of the process and does not survive cudaDeviceReset() or a teardown of the
 *     device's primary context.
 * It has no counterpart in the reference.
 */
#define KM_GRAD_STATIC_SCRATCH_BYTES (64LL << 20)
int kermac_b200_cdist_grad_static(const KmGradArgs* args, void* stream);

/*
 * y[l, n, o] = sum_m Kfn( outer( sum_k inner( b[l, n, k] (-|*) a[l, m, k] ) ) ) * c[l, o, m]
 * with the same inner / outer / kernel-function chain (epsilon mask included) as
 * kermac_b200_build_kernel, but the (m, n) kernel matrix is never stored.
 * c is m-contiguous: c[l][o][m] = c[l * c_stride_l + o * ldc + m].
 * y[l][n][o] = y[l * y_stride_l + n * y_stride_n + o * y_stride_o].
 * The diagonal rule of kermac_b200_build_kernel applies to the kernel-matrix values
 * before the product (only with a kernel function): where reg_off_x + m == reg_off_y + n
 * and regularization != 0 the value is 1 + regularization, which gives
 * y = (K + lambda I) c for a square K(X, X) without a second pass.
 *
 * contraction selects where the coefficient product runs: KM_CONTRACT_TENSOR (and
 * KM_CONTRACT_AUTO) on the tcgen05 tensor cores as three tf32 products per term
 * (operands split into a tf32 head and an fp32 remainder, fp32 accumulation: fp32-level
 * accuracy), KM_CONTRACT_FP32 as packed FP32 FMAs.  The kernel-matrix values are
 * computed in FP32 either way.
 */
#define KM_CONTRACT_AUTO   0
#define KM_CONTRACT_FP32   1
#define KM_CONTRACT_TENSOR 2
typedef struct KmMatvecArgs {
    int32_t m, n, k, o, l;
    const float* a; int64_t a_stride_m, a_stride_k, a_stride_l;
    const float* b; int64_t b_stride_n, b_stride_k, b_stride_l;
    const float* c; int64_t ldc, c_stride_l;
    float*       y; int64_t y_stride_n, y_stride_o, y_stride_l;
    int32_t inner_operator, inner_power, outer_power, kernel_type;
    KmHyper p_inner, p_outer, bandwidth;
    float   epsilon;
    void*   scratch; int64_t scratch_bytes;
    int32_t split_m;          /* 0 = automatic (1 when scratch is NULL) */
    int32_t contraction;      /* KM_CONTRACT_* */
    KmHyper regularization;
    int32_t reg_off_x, reg_off_y;
} KmMatvecArgs;

int kermac_b200_kernel_matvec(const KmMatvecArgs* args, void* stream);
int64_t kermac_b200_kernel_matvec_scratch_bytes(const KmMatvecArgs* args);

/* Writes a description of the kernel variant and grid that kermac_b200_build_kernel
 * would launch for `args` into buf (NUL terminated, truncated to buf_len). */
int kermac_b200_describe_variant(const KmBuildArgs* args, char* buf, int32_t buf_len);

/*
 * Measures an arithmetic pipe of the current device with a register-only kernel:
 *   kind 0: scalar fma.rn.f32        -> result in FP32 lane-operations per second
 *   kind 1: packed fma.rn.f32x2      -> result in FP32 lane-operations per second
 *   kind 2: MUFU (lg2.approx + ex2.approx) -> result in MUFU operations per second
 *   kind 3: scalar add.f32 (sub then add-abs chain, the p=1 inner step)
 *   kind 4: the cdist p=2 inner loop (shared-memory operand loads, duplicate moves, packed
 *           sub + fma) with no global staging -> FP32 lane-operations per second
 *   kind 5: the same for the p=1 inner loop (packed sub + add|.|)
 *   kind 6: the gradient's k step for p = 1 and four channels in registers only (packed subtract,
 *           sign flip, four packed FMAs with three different register-pair sources per (m, n) pair)
 *           -> FP32 lane-operations per second (1 + 4 per (m, n, k))
 *   kind 7: the same with the channel FMAs as scalar instructions
 *   kind 8 .. 11: tcgen05.mma kind::tf32 of 128 rows x N columns x 8 k with the A operand in tensor
 *           memory, N = 32, 64, 128, 256, issued back to back by one thread per SM (8 per iteration)
 *           -> MMAs per second over all SMs (the narrow ones of the tensor-core gradient kernel hold
 *           the pipe ~45 cycles whatever N up to 64)
 * Synchronises the device.  Returns 0 and stores the rate in *ops_per_second.
 */
int kermac_b200_measure_pipe(int32_t kind, int32_t iterations, double* ops_per_second, double* milliseconds);

/* Reads back and clears the device-side flag that a bounded wait inside a kernel sets
 * when it runs out (the kernel then skips its stores and still terminates).
 * Synchronises the current device.  Returns 0 (clear), 1 (a wait ran out) or a
 * negative code if the device could not be queried.  No reference counterpart. */
int kermac_b200_device_error_flag(void);

/* Test hook for the report path above: launches one block that waits `tries` (1 .. 2^20)
 * attempts on an mbarrier nothing ever arrives at, gives up, raises the device error flag
 * and ends.  The wait is bounded by construction; nothing faults or hangs.  After it,
 * kermac_b200_device_error_flag() returns 1 once and then 0.  No reference counterpart
 * (the reference's kernels have no waits on asynchronous units). */
int kermac_b200_selftest_wait_expiry(int32_t tries, void* stream);

/*
 * Asynchronous copy of `rows` runs of `row_bytes` bytes between host and device memory, the runs
 * `src_pitch_bytes` apart in the source and `dst_pitch_bytes` apart in the destination (a strided
 * 2-D block: cudaMemcpy2DAsync on `stream`).  direction: 0 host -> device, 1 device -> host.  Host
 * memory should be pinned, otherwise the copy does not overlap with anything.  It lets a caller
 * whose operands live in host memory send b[K, n0:n1], a column block of the storage layout,
 * without a staging copy, so the first rows can be computed while the rest of b is still on its way
 * (kermac_b200.host.HostCdist).  The reference takes device tensors only
 * (src/kermac/cdist.py:9-83); no reference counterpart.
 */
int kermac_b200_copy_2d_async(void* dst, int64_t dst_pitch_bytes, const void* src, int64_t src_pitch_bytes,
                              int64_t row_bytes, int64_t rows, int32_t direction, void* stream);

const char* kermac_b200_last_error(void);
int kermac_b200_abi_version(void);
const char* kermac_b200_build_id(void);

#ifdef __cplusplus
}
#endif
#endif /* KERMAC_B200_H */
