// Kernel-matrix build, TMA staged: the fast path for operands that are contiguous
// along their tile dimension and 16-byte aligned (the a[K, M] / b[K, N] storage of
// the headline cdist configurations).
//
// One thread block (256 threads, two resident per SM) owns a 128 x 128 output tile.
// Slabs of BK k-rows of both operands are brought in by tiled TMA copies
// (cp.async.bulk.tensor, no multicast) into a ring of STAGES shared-memory stages;
// each stage has a "full" mbarrier armed with the slab's byte count and an "empty"
// mbarrier on which every warp arrives once it has read the slab.  The arrival that
// completes a stage's empty phase (exactly one lane sees a pending count of 1) hands
// the next slab for that stage to the TMA engine on the spot: nobody waits for a stage
// to be released, and there is no block-wide barrier in the main loop.  TMA zero-fills rows and columns outside the tensor,
// and the last slab only consumes the k-rows that exist.
//
// Every mbarrier wait is bounded: if it runs out, the thread records the fact in a
// device-global flag, stops waiting and skips its stores, and the block still
// terminates.  kermac_b200_device_error_flag() reads the flag back.
//
// Computes what the reference's kernel_cute_build_kernel computes
// (include/build_a_kernel.cuh:19-463) for its COL_MAJOR / ALIGN_4 instantiations.
#include <cuda.h>

#include <mutex>

#include "km_build_cpasync.cuh"
#include "km_build_tma.cuh"
#include "km_mbar.cuh"
#include "km_host.h"

namespace km {

__device__ int g_tma_wait_expired = 0;

namespace {

constexpr int TMA_TILE    = 128;
constexpr int TMA_THREADS = 256;
constexpr int TMA_WARPS   = TMA_THREADS / 32;

template <int INNER, int BK, int STAGES, bool SYM>
__global__ void __launch_bounds__(TMA_THREADS, 2)
build_tma_kernel(const __grid_constant__ BuildParams p, const __grid_constant__ CUtensorMap map_a,
                 const __grid_constant__ CUtensorMap map_b) {
    constexpr int STAGE_FLOATS = 2 * BK * TMA_TILE;
    constexpr int STAGE_BYTES  = STAGE_FLOATS * 4;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * STAGES];

    float* smem = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~static_cast<uintptr_t>(127));
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base  = smem_u32(bars);
    auto full_bar  = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };

    const int tid  = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int l    = blockIdx.y;

    int tm, tn;
    tile_coords(p.tile_first + blockIdx.x, p.tiles_m, p.tiles_n, p.panel, tm, tn);
    if (SYM && tn < tm) return;   // the tile's mirror image (tn, tm) writes this part of C
    const int m0 = tm * TMA_TILE;
    const int n0 = tn * TMA_TILE;
    const int K  = p.K;
    const int ktiles = (K + BK - 1) / BK;
    const int la = (p.a_sl == 0) ? 0 : l;   // broadcast operands have a single batch slice in their map
    const int lb = (p.b_sl == 0) ? 0 : l;

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), TMA_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    auto issue = [&](int slab) {
        const int s        = slab % STAGES;
        const uint32_t dst = smem_base + s * STAGE_BYTES;
        mbar_expect_tx(full_bar(s), STAGE_BYTES);
        tma_load_3d(dst, &map_a, m0, slab * BK, la, full_bar(s));
        tma_load_3d(dst + BK * TMA_TILE * 4, &map_b, n0, slab * BK, lb, full_bar(s));
    };

    if (tid == 0) {
        const int first = ktiles < STAGES ? ktiles : STAGES;
        for (int s = 0; s < first; ++s) issue(s);
    }

    const float p_inner = (INNER == IN_DIFF_POW || INNER == IN_DOT_POW) ? read_hyper(p.p_inner, l) : 0.0f;

    const int lm = lane & 7, ln = lane >> 3;
    const int wm = warp & 1, wn = warp >> 1;
    const int tm_off = wm * 64 + lm * 4;
    const int tn_off = wn * 32 + ln * 4;

    u64 acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0ull;

    bool alive = true;
    int fail_kt = -1;   // first slab whose wait ran out on this thread

    // Refill by the last arriver: every warp arrives on a stage's empty barrier when it has read the
    // slab, and the one arrival that completes the phase (it sees a pending count of 1) hands the
    // next slab for that stage to the TMA engine on the spot.  Nobody waits for a stage to be
    // released, and a stage is refilled the moment it is free.
    for (int kt = 0; kt < ktiles; ++kt) {
        const int s = kt % STAGES;
        if (alive && !mbar_wait_bounded(full_bar(s), (kt / STAGES) & 1)) alive = false;

        const float* sa = smem + s * STAGE_FLOATS + tm_off;
        const float* sb = smem + s * STAGE_FLOATS + BK * TMA_TILE + tn_off;
        consume_slab<INNER, BK, TMA_TILE>(acc, sa, sb, K - kt * BK, p_inner, p.sgn);
        __syncwarp();
        if (lane == 0 && mbar_arrive_pending(empty_bar(s)) == 1 && kt + STAGES < ktiles && alive) {
            mbar_try_wait(empty_bar(s), (kt / STAGES) & 1);   // completed by this very arrival: the acquire side of the hand-over
            issue(kt + STAGES);
        }
        if (!alive && fail_kt < 0) fail_kt = kt;
    }

    if (!alive) {
        atomicExch(&g_tma_wait_expired, 1);
        if (tid == 0) {
            // Give copies that were already handed to the TMA engine a bounded chance
            // to land before this block's shared memory is released.
            // any warp may have requested the slabs from the failing one on; those that were never
            // requested simply run the short limit out
            const int first = fail_kt < 0 ? 0 : fail_kt;
            const int last  = first + STAGES < ktiles ? first + STAGES : ktiles;
            for (int slab = first; slab < last; ++slab)
                for (int i = 0; i < (1 << 16); ++i)
                    if (mbar_try_wait(full_bar(slab % STAGES), (slab / STAGES) & 1)) break;
        }
        return;
    }
    finish_block<INNER, SYM>(p, l, acc, m0 + tm_off, n0 + tn_off, SYM && tm != tn);
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

// Describes one operand as a rank-3 tensor (tile dimension, k, batch) of fp32 with a
// box of 128 x box_k x 1 elements.
int encode_operand(CUtensorMap* map, const float* base, int extent, int K, int L, long long s_k, long long s_l,
                   int box_k) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(KM_ERR_INTERNAL, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t row_bytes = (static_cast<cuuint64_t>(extent) * 4 + 15) & ~static_cast<cuuint64_t>(15);
    const int        kk        = K > 0 ? K : 1;
    const int        ll        = (s_l == 0) ? 1 : L;
    cuuint64_t stride_k        = (kk > 1) ? static_cast<cuuint64_t>(s_k) * 4 : row_bytes;
    cuuint64_t stride_l        = (ll > 1) ? static_cast<cuuint64_t>(s_l) * 4 : stride_k * kk;
    cuuint64_t dims[3]         = {static_cast<cuuint64_t>(extent), static_cast<cuuint64_t>(kk), static_cast<cuuint64_t>(ll)};
    cuuint64_t strides[2]      = {stride_k, stride_l};
    cuuint32_t box[3]          = {TMA_TILE, static_cast<cuuint32_t>(box_k), 1};
    cuuint32_t estr[3]         = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(KM_ERR_INTERNAL, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return 0;
}

int encode_box(CUtensorMap* map, const float* base, int inner, int outer, int L, long long s_outer, long long s_l,
               int box_inner, int box_outer) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(KM_ERR_INTERNAL, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t row_bytes = (static_cast<cuuint64_t>(inner) * 4 + 15) & ~static_cast<cuuint64_t>(15);
    const int        oo        = outer > 0 ? outer : 1;
    const int        ll        = (s_l == 0) ? 1 : L;
    cuuint64_t stride_o        = (oo > 1) ? static_cast<cuuint64_t>(s_outer) * 4 : row_bytes;
    cuuint64_t stride_l        = (ll > 1) ? static_cast<cuuint64_t>(s_l) * 4 : stride_o * oo;
    cuuint64_t dims[3]         = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(oo), static_cast<cuuint64_t>(ll)};
    cuuint64_t strides[2]      = {stride_o, stride_l};
    cuuint32_t box[3]          = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_outer), 1};
    cuuint32_t estr[3]         = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(KM_ERR_INTERNAL, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return 0;
}

bool operand_tma_ok(const float* base, long long s_t, long long s_k, long long s_l, int K, int L) {
    if (s_t != 1 || !aligned16(base)) return false;
    if (K > 1 && (s_k % 4 != 0 || s_k <= 0 || s_k >= (1LL << 36))) return false;
    if (L > 1 && s_l != 0 && (s_l % 4 != 0 || s_l >= (1LL << 36))) return false;
    return true;
}

typedef void (*TmaKernelFn)(const BuildParams, const CUtensorMap, const CUtensorMap);

// Pipeline shape per inner step: k rows per TMA box / stage and ring depth.  Measured on B200 at
// 30000 x 30000 x 1024: for the square and product steps 32-row slabs (3 stages) run 2 %
// faster than 16-row slabs (6 stages) because fewer slab boundaries interrupt the load
// scheduling; the |.| and |.|^p steps are slower with deep slabs.  Refill by the last arriver
// took the square step from 54.9 ms (thread 0 waiting for each stage's release) to 53.6; with it
// 32 x 3 is still the best shape (16 x 6: 56.4, 24 x 4: 54.5, 32 x 2: 54.1, 48 x 2: 54.1 ms).
template <int INNER>
struct TmaShape {
    static constexpr bool deep = (INNER == IN_DIFF_SQUARE || INNER == IN_DOT_NOOP);
    static constexpr int BK     = deep ? 32 : 16;
    static constexpr int STAGES = deep ? 3 : 6;
    static constexpr int SMEM   = STAGES * 2 * BK * TMA_TILE * 4 + 128;
};

struct TmaChoice {
    TmaKernelFn fn, fn_symmetric;
    int bk, smem;
};

template <int INNER>
TmaChoice tma_choice() {
    typedef TmaShape<INNER> S;
    return {build_tma_kernel<INNER, S::BK, S::STAGES, false>, build_tma_kernel<INNER, S::BK, S::STAGES, true>,
            S::BK, S::SMEM};
}

TmaChoice tma_kernel(int inner) {
    switch (inner) {
        case IN_DIFF_ABS: return tma_choice<IN_DIFF_ABS>();
        case IN_DIFF_SQUARE: return tma_choice<IN_DIFF_SQUARE>();
        case IN_DIFF_POW: return tma_choice<IN_DIFF_POW>();
        case IN_DOT_NOOP: return tma_choice<IN_DOT_NOOP>();
    }
    return {nullptr, nullptr, 0, 0};
}

}  // namespace

int encode_tma_operand(CUtensorMap* map, const float* base, int extent, int K, int L, long long s_k, long long s_l,
                       int box_k) {
    return encode_operand(map, base, extent, K, L, s_k, s_l, box_k);
}
int encode_tma_box(CUtensorMap* map, const float* base, int inner, int outer, int L, long long s_outer, long long s_l,
                   int box_inner, int box_outer) {
    return encode_box(map, base, inner, outer, L, s_outer, s_l, box_inner, box_outer);
}
bool tma_operand_ok(const float* base, long long s_t, long long s_k, long long s_l, int K, int L) {
    return operand_tma_ok(base, s_t, s_k, s_l, K, L);
}

bool tma_supported(const BuildParams& p) {
    if (!tma_kernel(p.inner_id).fn) return false;
    if (p.K < 1) return false;
    return operand_tma_ok(p.A, p.a_sm, p.a_sk, p.a_sl, p.K, p.L) && operand_tma_ok(p.B, p.b_sn, p.b_sk, p.b_sl, p.K, p.L);
}

// Measured on B200 at 30000 x 30000 x 1024: the TMA kernel wins for the square and
// product steps (53.6 vs 57.0 ms); for |.| and |.|^p the cp.async kernel is ahead
// (59.6 vs 64.2 ms, 331 vs 356 ms), so those keep it.
bool tma_preferred(const BuildParams& p) {
    return p.K >= 64 && (p.inner_id == IN_DIFF_SQUARE || p.inner_id == IN_DOT_NOOP);
}

int launch_build_tma(const BuildParams& p, cudaStream_t stream) {
    const TmaChoice choice = tma_kernel(p.inner_id);
    TmaKernelFn fn         = p.symmetric ? choice.fn_symmetric : choice.fn;
    if (!fn) return fail(KM_ERR_INTERNAL, "no TMA kernel for inner id %d", p.inner_id);
    const int kBK = choice.bk, kSmemBytes = choice.smem;
    if (int rc = cuda_status(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes),
                             "cudaFuncSetAttribute(build_tma_kernel)"))
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
        CUtensorMap map_a, map_b;
        if (int rc = encode_operand(&map_a, q.A, q.M, q.K, q.L, q.a_sk, q.a_sl, kBK)) return rc;
        if (int rc = encode_operand(&map_b, q.B, q.N, q.K, q.L, q.b_sk, q.b_sl, kBK)) return rc;
        dim3 grid((unsigned)q.tile_count, (unsigned)q.L, 1);
        fn<<<grid, TMA_THREADS, kSmemBytes, stream>>>(q, map_a, map_b);
        if (int rc = cuda_status(cudaGetLastError(), "launch of build_tma_kernel")) return rc;
    }
    return 0;
}

}  // namespace km

// The path a kernel takes when one of its bounded waits runs out, exercised on purpose and
// safely: one block initialises an mbarrier that expects one arrival, nobody ever arrives,
// thread 0 waits for `tries` attempts, gives up, records the fact in the same device flag the
// build kernels use and the block ends.  Nothing faults or hangs: the loop is bounded by
// construction and the barrier lives in the block's own shared memory.
namespace km {
namespace {
__global__ void wait_expiry_selftest_kernel(int tries, int* gave_up) {
    __shared__ __align__(8) unsigned long long bar;
    const uint32_t bar_addr = smem_u32(&bar);
    if (threadIdx.x == 0) {
        mbar_init(bar_addr, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0 && !mbar_wait_bounded(bar_addr, 0, tries)) {
        atomicExch(&g_tma_wait_expired, 1);
        if (gave_up) *gave_up = 1;
    }
}
}  // namespace
}  // namespace km

extern "C" int kermac_b200_selftest_wait_expiry(int32_t tries, void* stream) {
    using namespace km;
    if (tries < 1 || tries > (1 << 20)) return fail(KM_ERR_BAD_SHAPE, "tries must be in [1, 2^20]");
    if (int rc = require_sm100()) return rc;
    wait_expiry_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(tries, nullptr);
    return cuda_status(cudaGetLastError(), "launch of wait_expiry_selftest_kernel");
}

// Reads back (and clears) the flag that a bounded mbarrier wait sets when it runs
// out.  Synchronises the device.  Returns 0 / 1, or a negative / CUDA error code.
extern "C" int kermac_b200_device_error_flag(void) {
    int v = 0, zero = 0;
    if (int rc = km::cuda_status(cudaDeviceSynchronize(), "cudaDeviceSynchronize")) return rc < 0 ? rc : -rc;
    if (km::cuda_status(cudaMemcpyFromSymbol(&v, km::g_tma_wait_expired, sizeof(int)), "cudaMemcpyFromSymbol")) return KM_ERR_INTERNAL;
    if (v) cudaMemcpyToSymbol(km::g_tma_wait_expired, &zero, sizeof(int));
    const int mv = km::matvec_take_wait_flag();
    const int gv = km::grad_tensor_take_wait_flag();
    if (mv < 0 || gv < 0) return KM_ERR_INTERNAL;
    return (v || mv || gv) ? 1 : 0;
}
