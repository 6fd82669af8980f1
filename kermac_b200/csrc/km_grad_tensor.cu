// Tensor-core form of the p-norm gradient contraction
//   out[l, o, n, m] = sum_k c[l, o, k] * a[l, k, m] * g(d[l, n, m] - b[l, n, k])
// (what the reference's kernel_cute_p_norm_kernel_gradient computes, include/p_norm_gradient.cuh:22-405).
//
// For a fixed (n, m) the weights w[k] = a[k, m] * g(d[n, m] - b[n, k]) form one row of a matrix
// W[(n, m), k], and the result is the product W * c^T: 128 (n, m) pairs x OT channels per
// tcgen05.mma.  The FP32 pipe only forms the weights (a subtract, the norm's g, one multiply, the
// split below); the channel products run on the tensor cores.
//
// The weights never touch shared memory.  A thread owns one (n, m) pair, computes 16 consecutive k
// of its row in registers and writes them with tcgen05.st straight into tensor memory, where the
// MMA reads its A operand (row = tensor-memory lane, k = column).  Only the coefficients c go
// through shared memory, as the B operand.
//
// fp32 accuracy from tf32 products: every weight is split into hi (13 low mantissa bits cleared,
// exact in tf32) and lo = w - hi, every coefficient likewise, and three products are taken,
//   W_hi * [c_hi | c_lo]   one MMA with 2 OT output columns (OT "main" + OT "correction")
//   W_lo * c_hi            one MMA into the OT correction columns
// (W_lo * c_lo is below 2^-22 of the product and is dropped).
//
// The tensor core truncates when it adds into its fp32 accumulator, so a long chain of MMAs
// drifts low.  Chains are therefore cut every 128 k: two sets of accumulator columns alternate,
// and the finished set is added, rounding to nearest, to running sums in the owning thread's
// registers while the next chain is already being issued.
//
// Work decomposition: a thread block owns 32 (m) x 4 RG (n) pairs = RG row groups of 128 pairs and
// up to OT channels.  4 RG warps generate weights (4 per row group, one per quarter of the tensor-memory
// lanes), two warps issue the MMAs (half of the row groups each), one or two warps split and park the
// coefficients.  Per row group tensor memory holds two A buffers of 16 k (hi and lo: 2 x 32 columns)
// and the accumulators (2 OT columns per set); the block allocates all 512 columns of its SM and runs
// alone there: OT = 16 with 4 row groups (16 n) and two accumulator sets; OT = 32 with 4 row groups and
// OT = 64 with 2 (8 n), one accumulator set each (the next chain's MMAs wait until the generating warps
// have read the finished one).
//
// What bounds it (B200, K = 30000, M = 4096, N = 256, p = 1: 19.1 ms at 16 channels, 22.0 at 32, 29.6
// at 64, against 20.4 / 40.4 / 80.7 ms of the FP32 kernel): a tcgen05.mma kind::tf32 of 128 rows x 8 k
// holds the tensor pipe for max(45, N / 2) cycles whatever its width N, so the narrow MMAs of this product
// run the pipe at a quarter (N = 32) or half (N = 64) of its rate: 9.5 ms of MMAs per pass alone.  The
// weight generation, the tensor-memory stores and the MMAs of a step hang on one another (with the copy
// staging at 16 channels: 11 ms for the generation alone, +5 to 8 with the stores, +4 to 7 with the MMAs)
// and overlap only in part: tensor memory has room for two A buffers per row group, and the registers for
// no more than ~20 warps.  The automatic choice takes the tensor cores from 17 channels on, where the FP32
// kernel needs a second pass.
//
// Hand-over between the warps is by mbarriers; every wait is bounded, and a wait that runs out sets a
// flag (kermac_b200_device_error_flag) and lets the block run to its end without its results.  (Spinning
// on the non-blocking mbarrier test instead of the suspending try_wait measured 1 % slower and tripled
// the instructions executed.)
#include <cstring>

#include "km_build_tma.cuh"
#include "km_common.cuh"
#include "km_host.h"
#include "km_mbar.cuh"
#include "km_tcgen05.cuh"

namespace km {
namespace {

constexpr int GT_STAGES  = 3;               // staged slabs of GT_BK k rows (five are no faster)
constexpr int GT_PA      = GT_BK + 4;       // floats per staged row of a (transposed: [m][k])
constexpr int GT_PB      = GT_BK + 8;       // floats per staged row of b ([n][k])
constexpr int GT_KA      = 16;              // k per tensor-memory A buffer
constexpr int GT_C_SLOTS = 4;               // ring of coefficient tiles, one per slab
constexpr int GT_A_COLS  = 2 * GT_KA;       // one A buffer: hi, lo
constexpr int gt_pow2_cols(int cols) { return cols <= 32 ? 32 : cols <= 64 ? 64 : cols <= 128 ? 128 : cols <= 256 ? 256 : 512; }
static_assert(GT_BK == 2 * GT_KA, "a slab is two A buffers");

// OT channels per block, RG row groups of 128 (n, m) pairs per block.
template <int OT, int RG>
struct GtShape {
    static constexpr int GEN_WARPS    = 4 * RG;
    static constexpr int GEN_THREADS  = 32 * GEN_WARPS;
    static constexpr int ISSUERS      = RG >= 2 ? 2 : 1;           // warps that issue MMAs, RG / ISSUERS row groups each
    // warps that park the coefficients: at 64 channels one was the slowest warp of the block (48.3 ms with one,
    // 36.7 with two; four cost registers the generating warps need: 40.6); at 32 channels on four row groups
    // one is enough and a second only competes with the generating warps (22.0 against 23.0 ms)
    static constexpr int C_WARPS      = OT >= 64 ? 2 : 1;
    static constexpr int THREADS      = GEN_THREADS + 32 * (ISSUERS + C_WARPS);   // + the MMA warps and the coefficient warps
    static constexpr int TN           = 4 * RG;                    // n rows of the tile
    static constexpr int STAGE_FLOATS = GT_TM * GT_PA + TN * GT_PB;
    static constexpr int C_BYTES      = 2 * OT * 128;              // 2 OT rows (c_hi, c_lo) of 32 k
    static constexpr int D_COLS       = 2 * OT;                    // one accumulator set: main, correction
    // Accumulator sets per row group.  Two alternate, so that a finished chain is added up while the next one
    // runs, where tensor memory has room for them (16 channels); otherwise there is one, and the MMAs of the
    // next chain wait for the generating warps to have read the finished one.  (32 channels with two row groups
    // and two sets: 26.9 ms; with four row groups and one set, i.e. twice the generating warps: 23.1.)
    static constexpr int SETS         = RG * (2 * GT_A_COLS + 2 * D_COLS) <= 512 ? 2 : 1;
    // A buffers per accumulator chain (128 k).  Twice as long saves 5 % at 64 channels (34.6 against 36.5 ms) and
    // doubles the drift of same-sign sums (2.0e-6 against 1.1e-6 of the result over 20000 terms).
    static constexpr int CHAIN        = 8;
    // A buffers of 16 k per row group.  Four of them (at two row groups) are no faster than two: 28.0 against
    // 27.5 ms at 32 channels, 32.3 against 33.1 at 64.
    static constexpr int A_BUFS       = 2;
    static constexpr int D_OFF        = A_BUFS * GT_A_COLS;        // accumulator sets start after the A buffers
    static constexpr int RG_COLS      = D_OFF + SETS * D_COLS;     // tensor-memory columns per row group
    static constexpr int TMEM_COLS    = gt_pow2_cols(RG * RG_COLS);  // allocated (a power of two)
    static constexpr int BLOCKS_PER_SM = 512 / TMEM_COLS;          // as many blocks as tensor memory holds
    // Shared memory asked for: more than 1 / (BLOCKS_PER_SM + 1) of an SM's, so that no more blocks become
    // resident than tensor memory has room for (a block waits inside tcgen05.alloc otherwise).
    static constexpr int SMEM_BYTES   = BLOCKS_PER_SM == 1 ? 117 * 1024 : 78 * 1024;
    static_assert(RG * RG_COLS <= 512 && BLOCKS_PER_SM <= 2, "tensor memory");
    static_assert(1024 + GT_C_SLOTS * C_BYTES + GT_STAGES * STAGE_FLOATS * 4 <= SMEM_BYTES, "shared memory");
    static_assert(GT_TM == 32, "a row group is 32 m x 4 n");
};

__device__ int g_grad_tensor_wait_expired = 0;

template <int THREADS>
__device__ __forceinline__ void generators_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory"); }


// 16 weights of one (n, m) row: k = 0..15 of arow (a transposed) and brow, split into hi / lo.
// A_STRIDE: floats between consecutive k of the a operand (1: staged transposed, read 16 bytes at a time).
template <int NORM, bool TAIL, int A_STRIDE>
__device__ __forceinline__ void weights16(uint32_t (&hi)[16], uint32_t (&lo)[16], const float* arow, const float* brow,
                                          u64 dd, float pm1, int kvalid) {
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
        ulonglong2 a4;
        if constexpr (A_STRIDE == 1) {
            a4 = *reinterpret_cast<const ulonglong2*>(arow + 4 * q4);
        } else {
            a4.x = pack2(arow[(4 * q4) * A_STRIDE], arow[(4 * q4 + 1) * A_STRIDE]);
            a4.y = pack2(arow[(4 * q4 + 2) * A_STRIDE], arow[(4 * q4 + 3) * A_STRIDE]);
        }
        const ulonglong2 b4 = *reinterpret_cast<const ulonglong2*>(brow + 4 * q4);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const u64 a2   = h ? a4.y : a4.x;
            const u64 b2   = h ? b4.y : b4.x;
            const u64 diff = sub2(dd, b2);
            u64 w;
            if constexpr (NORM == KM_NORM_L1) {
                w = a2 ^ (diff & 0x8000000080000000ull);
            } else if constexpr (NORM == KM_NORM_L2) {
                w = mul2(a2, diff);
            } else if constexpr (NORM == GT_NORM_SQRT) {
                float d0, d1;
                unpack2(diff, d0, d1);
                w = mul2(a2, pack2(sqrt_approx(fabsf(d0)), sqrt_approx(fabsf(d1)))) ^ (diff & 0x8000000080000000ull);
            } else {
                float d0, d1;
                unpack2(diff, d0, d1);
                w = mul2(a2, pack2(copysignf(pow_approx(fabsf(d0), pm1), d0), copysignf(pow_approx(fabsf(d1), pm1), d1)));
            }
            if constexpr (TAIL) {
                // rows of k past the end of the range: a is staged as 0 there, but 0 * g(.) can be NaN
                const int k = 4 * q4 + 2 * h;
                if (k >= kvalid) w &= 0xFFFFFFFF00000000ull;
                if (k + 1 >= kvalid) w &= 0x00000000FFFFFFFFull;
            }
            const u64 whi = w & 0xFFFFE000FFFFE000ull;
            const u64 wlo = sub2(w, whi);
            hi[4 * q4 + 2 * h]     = static_cast<uint32_t>(whi);
            hi[4 * q4 + 2 * h + 1] = static_cast<uint32_t>(whi >> 32);
            lo[4 * q4 + 2 * h]     = static_cast<uint32_t>(wlo);
            lo[4 * q4 + 2 * h + 1] = static_cast<uint32_t>(wlo >> 32);
        }
    }
}

// TMA: a and b staged by tiled TMA copies (no multicast) into a ring with a full and an empty mbarrier per
// stage, each stage refilled by the warp whose arrival completes its empty phase: no per-thread copies, no
// block barrier, the warps drift apart freely.  a then sits in shared memory as it does in global memory
// ([k][m]) and is read one float at a time.  Otherwise: 4-byte cp.async copies (any alignment), a transposed.
template <int NORM, int OT, int RG, bool TMA>
__global__ void __launch_bounds__(GtShape<OT, RG>::THREADS, GtShape<OT, RG>::BLOCKS_PER_SM)
grad_tensor_kernel(const __grid_constant__ GradTensorParams p, const __grid_constant__ CUtensorMap map_a,
                   const __grid_constant__ CUtensorMap map_b) {
    using S = GtShape<OT, RG>;
    extern __shared__ unsigned char smem_raw[];
    // afull[rg][buf] (one arrival per generating warp of the row group), aempty[buf], dfull[set], cfree[slot]
    // (tcgen05.commit), cfull[slot] (the coefficient warp)
    __shared__ __align__(8) unsigned long long s_bars[S::ISSUERS * S::A_BUFS + S::A_BUFS + 2 + 2 * GT_C_SLOTS + S::ISSUERS];
    __shared__ __align__(8) unsigned long long s_ring[2 * GT_STAGES];   // full[stage], empty[stage] (TMA staging)
    __shared__ uint32_t s_tmem;

    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t c_addr   = (raw_addr + 1023u) & ~1023u;           // coefficient tiles, 1024-byte aligned
    unsigned char* c_tiles  = smem_raw + (c_addr - raw_addr);
    float* stages           = reinterpret_cast<float*>(c_tiles + GT_C_SLOTS * S::C_BYTES);

    const int tid  = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;

    // n-tiles fastest: the blocks that read the same (k range, m-column) tile of a run together
    int bx          = blockIdx.x;
    const int tn    = bx % p.tiles_n; bx /= p.tiles_n;
    const int split = bx % p.splits;  bx /= p.splits;
    const int tm    = bx;
    const int oc    = blockIdx.y;
    const int l     = blockIdx.z;
    const int m0 = tm * GT_TM, n0 = tn * S::TN, o0 = oc * OT;

    const int k_begin = split * p.k_per_split;
    const int k_end   = min(p.K, k_begin + p.k_per_split);
    const int nslabs  = (k_end > k_begin) ? (k_end - k_begin + GT_BK - 1) / GT_BK : 0;
    const int T       = 2 * nslabs;                                   // A buffers in all
    const int chains  = (T + S::CHAIN - 1) / S::CHAIN;

    const uint32_t bars = smem_u32(s_bars);
    constexpr int NI    = S::ISSUERS;
    constexpr int RG_PER = RG / NI;                                   // row groups per issuing warp
    constexpr int NB    = S::A_BUFS;
    auto afull  = [&](int is, int b) { return bars + 8u * (is * NB + b); };
    auto aempty = [&](int b) { return bars + 8u * (NI * NB + b); };
    auto dfull  = [&](int set) { return bars + 8u * (NI * NB + NB + set); };
    auto cfull  = [&](int slot) { return bars + 8u * (NI * NB + NB + 2 + slot); };
    auto cfree  = [&](int slot) { return bars + 8u * (NI * NB + NB + 2 + GT_C_SLOTS + slot); };
    auto dfree  = [&](int is) { return bars + 8u * (NI * NB + NB + 2 + 2 * GT_C_SLOTS + is); };   // single accumulator set only
    constexpr int SETS = S::SETS;
    constexpr int GT_CHAIN = S::CHAIN;

    if (tid == 0) {
        for (int is = 0; is < NI; ++is)
            for (int b = 0; b < NB; ++b) mbar_init(afull(is, b), 4 * RG_PER);  // the generating warps of its row groups
        for (int b = 0; b < NB; ++b) mbar_init(aempty(b), NI);                  // one tcgen05.commit per issuer
        for (int b = 0; b < 2; ++b) mbar_init(dfull(b), NI);
        for (int is = 0; is < NI; ++is) mbar_init(dfree(is), 4 * RG_PER);
        for (int sl = 0; sl < GT_C_SLOTS; ++sl) {
            mbar_init(cfull(sl), S::C_WARPS);
            mbar_init(cfree(sl), NI);
        }
        if constexpr (TMA) {
            for (int st = 0; st < GT_STAGES; ++st) {
                mbar_init(smem_u32(s_ring) + 8u * st, 1);
                mbar_init(smem_u32(s_ring) + 8u * (GT_STAGES + st), S::GEN_WARPS);
            }
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        tc::fence_smem_to_async();
    }
    if (warp == S::GEN_WARPS) tc::tmem_alloc(smem_u32(&s_tmem), S::TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = s_tmem;
    bool expired = false;

    if (warp < S::GEN_WARPS) {
        // ------------------------------------------------------------------ weight generators
        const int rg = warp >> 2, q = warp & 3;
        const int mm = 8 * q + (lane & 7);          // pair of this thread inside the tile
        const int nn = 4 * rg + (lane >> 3);
        const int m = m0 + mm, n = n0 + nn;
        const float* A = p.A + (long long)l * p.a_sl + m0;
        const float* B = p.B + (long long)l * p.b_sl + (long long)n0 * p.ldb;
        const float* D = p.D + (long long)l * p.d_sl;
        const float dval = (n < p.N && m < p.M) ? D[(long long)n * p.ldd + m] : 0.0f;
        const u64 dd     = pack2(dval, dval);
        float pm1 = 0.0f;
        if (NORM == KM_NORM_P) pm1 = read_hyper(p.p, l) - 1.0f;
        // this thread's tensor-memory lane (its row of the row group) and the row group's columns
        const uint32_t t_row = tmem + (static_cast<uint32_t>(32 * q) << 16) + rg * S::RG_COLS;

        float run[OT];
#pragma unroll
        for (int i = 0; i < OT; ++i) run[i] = 0.0f;

        // Staging roles, fixed for the whole walk.
        // a: a warp copies 8 consecutive m of 4 k rows: 32-byte runs in global memory, and on the shared
        // side (transposed, pitch 36) banks 4 * mi + ki, all different.  b: a warp copies 8 consecutive k
        // of 4 rows n; pitch 40 puts them on banks 8 * ni + ki.
        constexpr int A_COPIES = (GT_TM * GT_BK) / S::GEN_THREADS;
        static_assert(S::TN * GT_BK == S::GEN_THREADS, "one element of b per thread and slab");
        const float* a_src[A_COPIES];
        uint32_t a_dst[A_COPIES];
        int a_kk[A_COPIES];
        bool a_ok[A_COPIES];
#pragma unroll
        for (int i = 0; i < A_COPIES; ++i) {
            const int idx = tid + i * S::GEN_THREADS;
            const int mi = (idx & 7) + ((idx >> 5) & 3) * 8;
            a_kk[i]  = ((idx >> 3) & 3) + (idx >> 7) * 4;
            a_ok[i]  = (m0 + mi) < p.M;
            a_src[i] = A + (long long)(k_begin + a_kk[i]) * p.lda + mi;
            a_dst[i] = (mi * GT_PA + a_kk[i]) * 4;
        }
        const int b_kk = (tid & 7) + ((tid >> 5) & 3) * 8;
        const int b_ni = ((tid >> 3) & 3) + (tid >> 7) * 4;
        const bool b_ok = (n0 + b_ni) < p.N;
        const float* b_src   = B + (long long)b_ni * p.ldb + k_begin + b_kk;
        const uint32_t b_dst = (GT_TM * GT_PA + b_ni * GT_PB + b_kk) * 4;
        const uint32_t stages_addr = smem_u32(stages);

        auto stage = [&](int s) {
            if constexpr (TMA) return;
            const uint32_t base = stages_addr + (s % GT_STAGES) * (S::STAGE_FLOATS * 4);
            const int krem      = k_end - (k_begin + s * GT_BK);        // k rows of this slab that exist
            const long long ks  = (long long)s * GT_BK;
#pragma unroll
            for (int i = 0; i < A_COPIES; ++i) {
                const bool ok = a_ok[i] && a_kk[i] < krem;
                cp_async_4(base + a_dst[i], ok ? a_src[i] + ks * p.lda : p.A, ok ? 4 : 0);
            }
            const bool ok = b_ok && b_kk < krem;
            cp_async_4(base + b_dst, ok ? b_src + ks : p.B, ok ? 4 : 0);
        };
        // TMA staging: one thread asks for a slab's two boxes; the stage's full barrier receives the bytes
        const uint32_t ring = smem_u32(s_ring);
        auto full_bar  = [&](int st) { return ring + 8u * st; };
        auto empty_bar = [&](int st) { return ring + 8u * (GT_STAGES + st); };
        const int la = (p.a_sl == 0) ? 0 : l, lb = (p.b_sl == 0) ? 0 : l;   // a broadcast operand has one batch slice
        auto issue = [&](int s) {
            const int st       = s % GT_STAGES;
            const uint32_t dst = stages_addr + st * (S::STAGE_FLOATS * 4);
            mbar_expect_tx(full_bar(st), (GT_TM + S::TN) * GT_BK * 4);
            tma_load_3d(dst, &map_a, m0, k_begin + s * GT_BK, la, full_bar(st));
            tma_load_3d(dst + GT_TM * GT_BK * 4, &map_b, k_begin + s * GT_BK, n0, lb, full_bar(st));
        };
        int fail_s = -1;                               // first slab whose wait ran out on this thread
        auto drain = [&](int c) {
            const int set = SETS == 2 ? (c & 1) : 0;
            if (!expired && !mbar_wait_bounded(dfull(set), (SETS == 2 ? (c >> 1) : c) & 1)) expired = true;
            __syncwarp();
            tc::fence_after_sync();
#pragma unroll
            for (int part = 0; part < OT / 16; ++part) {
                uint32_t r0[16], r1[16];
                tc::ld_32x32b_x16(t_row + S::D_OFF + set * S::D_COLS + part * 16, r0);
                tc::ld_32x32b_x16(t_row + S::D_OFF + set * S::D_COLS + OT + part * 16, r1);
#pragma unroll
                for (int i = 0; i < 16; ++i) run[part * 16 + i] += __uint_as_float(r0[i]) + __uint_as_float(r1[i]);
            }
            tc::fence_before_sync();
            if constexpr (SETS == 1) {
                // the one accumulator set may be started over
                __syncwarp();
                if (lane == 0) mbar_arrive(dfree(rg / RG_PER));
            }
        };
        // hands the A buffer of step t to the MMA warp, once its tensor-memory stores have landed (putting the
        // next step's weights between the stores and this wait measured slower: 20.6 against 19.1 ms at 16 channels)
        auto publish = [&](int t) {
            tc::wait_st();
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(afull(rg / RG_PER, t % NB));
        };

        if constexpr (TMA) {
            if (tid == 0)
                for (int s = 0; s < GT_STAGES && s < nslabs; ++s) issue(s);
        } else {
#pragma unroll
            for (int s = 0; s < GT_STAGES - 1; ++s) {
                if (s < nslabs) stage(s);
                cp_async_commit();
            }
        }
        int next_drain = 0;
        for (int s = 0; s < nslabs; ++s) {
            if constexpr (TMA) {
                if (!expired && !mbar_wait_bounded(full_bar(s % GT_STAGES), (s / GT_STAGES) & 1)) {
                    expired = true;
                    fail_s  = s;
                }
            } else {
                cp_async_wait<GT_STAGES - 2>();
                generators_barrier<S::GEN_THREADS>();
                if (s + GT_STAGES - 1 < nslabs) stage(s + GT_STAGES - 1);
                cp_async_commit();
            }
            constexpr int A_STRIDE = TMA ? GT_TM : 1;
            const float* sa  = stages + (s % GT_STAGES) * S::STAGE_FLOATS + (TMA ? mm : mm * GT_PA);
            const float* sb  = stages + (s % GT_STAGES) * S::STAGE_FLOATS + (TMA ? GT_TM * GT_BK + nn * GT_BK : GT_TM * GT_PA + nn * GT_PB);
            const int kvalid = k_end - (k_begin + s * GT_BK);
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int t = 2 * s + hf;
                uint32_t hi[16], lo[16];
                if (kvalid >= GT_BK)
                    weights16<NORM, false, A_STRIDE>(hi, lo, sa + hf * GT_KA * A_STRIDE, sb + hf * GT_KA, dd, pm1, GT_KA);
                else
                    weights16<NORM, true, A_STRIDE>(hi, lo, sa + hf * GT_KA * A_STRIDE, sb + hf * GT_KA, dd, pm1, kvalid - hf * GT_KA);
                if constexpr (TMA) {
                    if (hf == 1) {
                        // the slab is in registers: the arrival that completes the stage's empty phase refills it
                        __syncwarp();
                        if (lane == 0 && mbar_arrive_pending(empty_bar(s % GT_STAGES)) == 1 && s + GT_STAGES < nslabs && !expired) {
                            mbar_try_wait(empty_bar(s % GT_STAGES), (s / GT_STAGES) & 1);   // the acquire side of the hand-over
                            issue(s + GT_STAGES);
                        }
                    }
                }
                // the chain before the running one finished a buffer ago: add it to the running sums
                // (with a single accumulator set: at the first step of the next chain, which cannot start before)
                if (t == GT_CHAIN * next_drain + GT_CHAIN + (SETS == 2 ? 1 : 0)) {
                    drain(next_drain);
                    ++next_drain;
                }
                // the MMAs that read this buffer NB steps ago must be done before it is overwritten
                if (t >= NB && !expired && !mbar_wait_bounded(aempty(t % NB), (t / NB - 1) & 1)) expired = true;
                __syncwarp();
                tc::fence_after_sync();
                tc::st_32x32b_x16(t_row + (t % NB) * GT_A_COLS, hi);
                tc::st_32x32b_x16(t_row + (t % NB) * GT_A_COLS + GT_KA, lo);
                publish(t);
            }
        }
        cp_async_wait<0>();
        if constexpr (TMA) {
            // give copies already handed to the TMA engine a bounded chance to land before the block's shared
            // memory is released
            if (expired && lane == 0) {
                const int first = fail_s < 0 ? 0 : fail_s;
                const int last  = first + GT_STAGES < nslabs ? first + GT_STAGES : nslabs;
                for (int slab = first; slab < last; ++slab)
                    for (int i = 0; i < (1 << 16); ++i)
                        if (mbar_try_wait(full_bar(slab % GT_STAGES), (slab / GT_STAGES) & 1)) break;
            }
        }
        while (next_drain < chains) {
            drain(next_drain);
            ++next_drain;
        }

        if (!expired && n < p.N && m < p.M) {
            float* E = p.E + (long long)split * p.split_stride + (long long)l * p.e_sl + (long long)n * p.e_sn + m;
#pragma unroll
            for (int o = 0; o < OT; ++o)
                if (o0 + o < p.O) E[(long long)(o0 + o) * p.e_so] = run[o];
        }
    } else if (warp < S::GEN_WARPS + NI) {
        // ------------------------------------------------------------------ MMA issue (one lane per issuing warp)
        const int is = warp - S::GEN_WARPS;
        constexpr uint32_t idesc_main = tc::instr_desc_tf32(128, 2 * OT);
        constexpr uint32_t idesc_corr = tc::instr_desc_tf32(128, OT);
        if (lane == 0) {
            for (int s = 0; s < nslabs; ++s) {
                const int slot           = s % GT_C_SLOTS;
                const uint32_t slot_addr = c_addr + slot * S::C_BYTES;
                if (!expired && !mbar_wait_bounded(cfull(slot), (s / GT_C_SLOTS) & 1)) expired = true;
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    const int t     = 2 * s + hf;
                    const int set   = SETS == 2 ? (t / GT_CHAIN) & 1 : 0;
                    const bool head = (t % GT_CHAIN) == 0;
                    const bool tail = (t % GT_CHAIN) == GT_CHAIN - 1 || t == T - 1;
                    const uint64_t db0 = tc::smem_desc_k_major_sw128(slot_addr + (hf * 2) * 32);
                    const uint64_t db1 = tc::smem_desc_k_major_sw128(slot_addr + (hf * 2 + 1) * 32);
                    const uint32_t d0  = tmem + is * RG_PER * S::RG_COLS + S::D_OFF + set * S::D_COLS;
                    const uint32_t a0  = tmem + is * RG_PER * S::RG_COLS + (t % NB) * GT_A_COLS;
                    if (!expired && !mbar_wait_bounded(afull(is, t % NB), (t / NB) & 1)) expired = true;
                    // one accumulator set: the generating warps must have read the finished chain
                    if (SETS == 1 && head && t > 0 && !expired && !mbar_wait_bounded(dfree(is), (t / GT_CHAIN - 1) & 1)) expired = true;
                    tc::fence_after_sync();
                    {
                        // Every MMA of this shape holds the tensor pipe for the same ~45 cycles whatever its width
                        // up to 64 columns (64 cycles at 128); consecutive ones go to different accumulator columns.
#pragma unroll
                        for (int rg = 0; rg < RG_PER; ++rg)
                            tc::mma_tf32_a_tmem(d0 + rg * S::RG_COLS, a0 + rg * S::RG_COLS, db0, idesc_main, !head);
#pragma unroll
                        for (int rg = 0; rg < RG_PER; ++rg)
                            tc::mma_tf32_a_tmem(d0 + rg * S::RG_COLS + OT, a0 + rg * S::RG_COLS + GT_KA, db0, idesc_corr, true);
#pragma unroll
                        for (int rg = 0; rg < RG_PER; ++rg)
                            tc::mma_tf32_a_tmem(d0 + rg * S::RG_COLS, a0 + rg * S::RG_COLS + 8, db1, idesc_main, true);
#pragma unroll
                        for (int rg = 0; rg < RG_PER; ++rg)
                            tc::mma_tf32_a_tmem(d0 + rg * S::RG_COLS + OT, a0 + rg * S::RG_COLS + GT_KA + 8, db1, idesc_corr, true);
                    }
                    tc::commit(aempty(t % NB));
                    if (tail) tc::commit(dfull(set));
                    if (hf == 1) tc::commit(cfree(slot));
                }
            }
        }
        __syncwarp();
        expired = __any_sync(0xFFFFFFFFu, expired);
    } else {
        // ------------------------------------------------------------------ coefficient warp
        // A slab's OT x 32 coefficients, split into hi / lo and parked as the MMA's B operand: K-major rows
        // of 128 bytes with the 128-byte swizzle, rows 0..OT-1 c_hi, rows OT..2 OT-1 c_lo.
        constexpr int CPW    = OT / S::C_WARPS;        // channels this warp parks
        constexpr int CHUNKS = CPW / 4;                // 16-byte chunks per lane and slab
        const int cw0        = (warp - S::GEN_WARPS - NI) * CPW;
        const float* C = p.C + (long long)l * p.c_sl;
        float cv[CHUNKS][4];
        auto load_c = [&](int s, float (&v)[CHUNKS][4]) {
            const int k0 = k_begin + s * GT_BK;
#pragma unroll
            for (int i = 0; i < CHUNKS; ++i) {
                const int id = lane + 32 * i;
                const int o = cw0 + (id >> 3), ck = id & 7;
                const int gk = k0 + 4 * ck;
                const bool o_ok = (o0 + o) < p.O;
                const float* src = C + (long long)(o0 + o) * p.ldc + gk;
                if (p.c_vec && o_ok && gk + 3 < k_end) {
                    const float4 x = *reinterpret_cast<const float4*>(src);
                    v[i][0] = x.x; v[i][1] = x.y; v[i][2] = x.z; v[i][3] = x.w;
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e) v[i][e] = (o_ok && gk + e < k_end) ? src[e] : 0.0f;
                }
            }
        };
        if (nslabs > 0) load_c(0, cv);
        for (int s = 0; s < nslabs; ++s) {
            const int slot = s % GT_C_SLOTS;
            float nx[CHUNKS][4];
            if (s + 1 < nslabs) load_c(s + 1, nx);
            // the MMAs that read this slot four slabs ago must be done
            if (s >= GT_C_SLOTS && !expired && !mbar_wait_bounded(cfree(slot), ((s / GT_C_SLOTS) - 1) & 1)) expired = true;
            __syncwarp();
            unsigned char* dst = c_tiles + slot * S::C_BYTES;
#pragma unroll
            for (int i = 0; i < CHUNKS; ++i) {
                const int id = lane + 32 * i;
                const int o = cw0 + (id >> 3), ck = id & 7;
                float hi[4], lo[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    hi[e] = __uint_as_float(__float_as_uint(cv[i][e]) & 0xFFFFE000u);
                    lo[e] = cv[i][e] - hi[e];
                }
                const int off = o * 128 + ((ck ^ (o & 7)) << 4);
                *reinterpret_cast<float4*>(dst + off)            = make_float4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<float4*>(dst + OT * 128 + off) = make_float4(lo[0], lo[1], lo[2], lo[3]);
            }
            tc::fence_smem_to_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(cfull(slot));
            if (s + 1 < nslabs) {
#pragma unroll
                for (int i = 0; i < CHUNKS; ++i)
#pragma unroll
                    for (int e = 0; e < 4; ++e) cv[i][e] = nx[i][e];
            }
        }
        expired = __any_sync(0xFFFFFFFFu, expired);
    }

    if (expired) atomicExch(&g_grad_tensor_wait_expired, 1);
    tc::fence_before_sync();
    __syncthreads();
    if (warp == S::GEN_WARPS) tc::tmem_dealloc(tmem, S::TMEM_COLS);
}

typedef void (*GradTensorFn)(const GradTensorParams, const CUtensorMap, const CUtensorMap);

template <int OT, int RG, bool TMA>
GradTensorFn grad_tensor_fn(int norm_kind) {
    switch (norm_kind) {
        case KM_NORM_L1: return grad_tensor_kernel<KM_NORM_L1, OT, RG, TMA>;
        case KM_NORM_L2: return grad_tensor_kernel<KM_NORM_L2, OT, RG, TMA>;
        case KM_NORM_P: return grad_tensor_kernel<KM_NORM_P, OT, RG, TMA>;
        case GT_NORM_SQRT: return grad_tensor_kernel<GT_NORM_SQRT, OT, RG, TMA>;
    }
    return nullptr;
}

template <int OT, int RG>
int grad_tensor_launch_shape(const GradTensorParams& p, int norm_kind, cudaStream_t st) {
    using S = GtShape<OT, RG>;
    // tiled TMA copies need 16-byte aligned bases and pitches that are multiples of 16 bytes
#ifndef GT_NO_TMA
    const bool tma = tma_operand_ok(p.A, 1, p.lda, p.a_sl, p.K, p.L) && tma_operand_ok(p.B, 1, p.ldb, p.b_sl, p.N, p.L);
#else
    const bool tma = false;
#endif
    GradTensorFn fn = tma ? grad_tensor_fn<OT, RG, true>(norm_kind) : grad_tensor_fn<OT, RG, false>(norm_kind);
    CUtensorMap map_a, map_b;
    memset(&map_a, 0, sizeof(map_a));
    memset(&map_b, 0, sizeof(map_b));
    if (tma) {
        if (int rc = encode_tma_box(&map_a, p.A, p.M, p.K, p.L, p.lda, p.a_sl, GT_TM, GT_BK)) return rc;
        if (int rc = encode_tma_box(&map_b, p.B, p.K, p.N, p.L, p.ldb, p.b_sl, GT_BK, S::TN)) return rc;
    }
    if (!fn) return fail(KM_ERR_INTERNAL, "no tensor-core gradient kernel for norm kind %d", norm_kind);
    if (int rc = cuda_status(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM_BYTES),
                             "cudaFuncSetAttribute(grad_tensor_kernel)"))
        return rc;
    dim3 grid((unsigned)((long long)p.tiles_m * p.tiles_n * p.splits), (unsigned)p.o_chunks, (unsigned)p.L);
    fn<<<grid, S::THREADS, S::SMEM_BYTES, st>>>(p, map_a, map_b);
    return cuda_status(cudaGetLastError(), "launch of grad_tensor_kernel");
}

}  // namespace

int grad_tensor_launch(const GradTensorParams& p, int norm_kind, cudaStream_t st) {
    if (p.ot == 16 && p.rg == 4) return grad_tensor_launch_shape<16, 4>(p, norm_kind, st);
    if (p.ot == 32 && p.rg == 4) return grad_tensor_launch_shape<32, 4>(p, norm_kind, st);
    if (p.ot == 64 && p.rg == 2) return grad_tensor_launch_shape<64, 2>(p, norm_kind, st);
    return fail(KM_ERR_INTERNAL, "no tensor-core gradient kernel for %d channels x %d row groups per block", p.ot, p.rg);
}

// Row groups per block: as many as tensor memory holds (two A buffers of 32 columns and two accumulator
// sets of 2 OT columns per row group).
int gt_rg_for(int ot) { return ot == 64 ? 2 : 4; }
int gt_blocks_per_sm(int ot) { return ot == 64 ? GtShape<64, 2>::BLOCKS_PER_SM : ot == 32 ? GtShape<32, 4>::BLOCKS_PER_SM : GtShape<16, 4>::BLOCKS_PER_SM; }

int grad_tensor_take_wait_flag() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_grad_tensor_wait_expired, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_grad_tensor_wait_expired, &zero, sizeof(int));
    return v ? 1 : 0;
}

}  // namespace km
