// kermac_b200_kernel_matvec: y[l, n, o] = sum_m Kmat[l, m, n] * c[l, o, m] where
// Kmat is the kernel matrix kermac_b200_build_kernel would produce, which is never
// written to global memory.
//
// A thread block owns 128 rows n and walks m in chunks of 128.  For each chunk it
// builds the 128 x 128 kernel-matrix tile exactly as the build kernel does (same
// staging, same packed 8 x 8 register blocks, same outer chain and epsilon mask),
// parks the tile in shared memory, and contracts it with the chunk's coefficients
// c[o, m] into per-thread accumulators y[n, o..] that live in registers for the
// whole walk.  The sum over m is therefore taken in a fixed order inside one block.
// With split_m > 1 the m range is divided over several blocks whose partial sums go
// to caller-provided scratch and are added in a fixed order by a second kernel.
//
// The reference has no such kernel: callers materialise run_kernel(...)
// (src/kermac/build_a_kernel.py:158-394) and multiply afterwards.
#include <cstring>

#include "km_build_cpasync.cuh"
#include "km_build_tma.cuh"
#include "km_host.h"
#include "km_mbar.cuh"
#include "km_tcgen05.cuh"

namespace km {
namespace {

constexpr int MV_THREADS = 256;
constexpr int MV_TILE    = 128;
constexpr int MV_BK      = 16;
constexpr int MV_STAGES  = 2;
constexpr int MV_PITCH   = CPA_PITCH;
constexpr int MV_STAGE_FLOATS = 2 * MV_BK * MV_PITCH;
constexpr int MV_KT_PITCH     = MV_TILE + 4;   // kernel-matrix tile rows [n][m]

struct MatvecParams {
    int M, N, K, O, L;
    const float* A; long long a_sm, a_sk, a_sl;
    const float* B; long long b_sn, b_sk, b_sl;
    const float* C; long long ldc, c_sl;
    float*       Y; long long y_sn, y_so, y_sl;     // destination (y, or scratch when split)
    int inner_id, outer_power, kernel_type;
    KmHyper p_inner, p_outer, bandwidth, regularization;
    int   reg_off_m, reg_off_n;                       // diagonal rule: reg_off_m + m == reg_off_n + n
    float epsilon;
    int tiles_n, splits, o_chunks;
    int m_per_split;                                  // multiple of MV_TILE
    long long split_stride;
};

template <int OT>
constexpr int mv_smem_bytes() {
    return (MV_STAGES * MV_STAGE_FLOATS + MV_TILE * MV_KT_PITCH + MV_TILE * OT) * 4;
}

template <int INNER, int OT, bool AVEC, bool BVEC>
__global__ void __launch_bounds__(MV_THREADS, 2) matvec_kernel(const __grid_constant__ MatvecParams p) {
    constexpr int OH = OT / 2;   // outputs per thread: one row n, OH channels
    extern __shared__ __align__(16) float smem[];
    float* s_kt = smem + MV_STAGES * MV_STAGE_FLOATS;     // [128 n][MV_KT_PITCH]
    float* s_c  = s_kt + MV_TILE * MV_KT_PITCH;           // [128 m][OT]

    const int tid  = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int tn    = blockIdx.x % p.tiles_n;
    const int split = blockIdx.x / p.tiles_n;
    const int oc    = blockIdx.y;
    const int l     = blockIdx.z;
    const int n0 = tn * MV_TILE;
    const int o0 = oc * OT;
    const int m_begin = split * p.m_per_split;
    const int m_end   = min(p.M, m_begin + p.m_per_split);
    const int chunks  = (m_end > m_begin) ? (m_end - m_begin + MV_TILE - 1) / MV_TILE : 0;

    const float* A = p.A + (long long)l * p.a_sl;
    const float* B = p.B + (long long)l * p.b_sl + (long long)n0 * p.b_sn;
    const float* C = p.C + (long long)l * p.c_sl;
    const int rem_n = p.N - n0;
    const int K = p.K;
    const int ktiles = K > 0 ? (K + MV_BK - 1) / MV_BK : 1;   // K = 0 still runs the outer chain on a zero sum
    const int total  = chunks * ktiles;

    const float p_inner = (INNER == IN_DIFF_POW || INNER == IN_DOT_POW) ? read_hyper(p.p_inner, l) : 0.0f;
    const Epilogue epi  = make_epilogue(p.outer_power, p.kernel_type, p.p_outer, p.bandwidth, p.epsilon, l);

    const int lm = lane & 7, ln = lane >> 3;
    const int wm = warp & 1, wn = warp >> 1;
    const int tm_off = wm * 64 + lm * 4;
    const int tn_off = wn * 32 + ln * 4;

    // contraction role of this thread
    const int cn = tid & (MV_TILE - 1);
    const int ch = tid >> 7;
    u64 yacc[OH / 2 > 0 ? OH / 2 : 1];
#pragma unroll
    for (int i = 0; i < (OH / 2 > 0 ? OH / 2 : 1); ++i) yacc[i] = 0ull;

    u64 acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0ull;

    auto stage = [&](int it) {
        const int chunk = it / ktiles, kt = it - chunk * ktiles;
        const int mc0   = m_begin + chunk * MV_TILE;
        float* st       = smem + (it % MV_STAGES) * MV_STAGE_FLOATS;
        stage_operand<AVEC, MV_BK>(st, A + (long long)mc0 * p.a_sm, p.a_sm, p.a_sk, m_end - mc0, K, kt, tid);
        stage_operand<BVEC, MV_BK>(st + MV_BK * MV_PITCH, B, p.b_sn, p.b_sk, rem_n, K, kt, tid);
    };

    if (total > 0) stage(0);
    cp_async_commit();

    for (int it = 0; it < total; ++it) {
        const int chunk = it / ktiles, kt = it - chunk * ktiles;
        cp_async_wait<0>();
        __syncthreads();
        if (it + 1 < total) stage(it + 1);
        cp_async_commit();

        const float* sa = smem + (it % MV_STAGES) * MV_STAGE_FLOATS + tm_off;
        const float* sb = smem + (it % MV_STAGES) * MV_STAGE_FLOATS + MV_BK * MV_PITCH + tn_off;
        consume_slab<INNER, MV_BK, MV_PITCH>(acc, sa, sb, K - kt * MV_BK, p_inner, 1.0f);

        if (kt == ktiles - 1) {
            const int mc0 = m_begin + chunk * MV_TILE;
            // kernel-matrix values of this chunk -> shared memory, [n][m]; columns of
            // m outside the range are zeroed so they add nothing.
            apply_epilogue(epi, acc, 0, 4);
            const bool partial = (mc0 + MV_TILE > m_end);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int nn = tn_off + (j >> 2) * 16 + (j & 3);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int mm = tm_off + h * 32;
                    float v[4];
                    unpack2(acc[j][2 * h], v[0], v[1]);
                    unpack2(acc[j][2 * h + 1], v[2], v[3]);
                    if (partial) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) v[e] = (mc0 + mm + e < m_end) ? v[e] : 0.0f;
                    }
                    *reinterpret_cast<float4*>(s_kt + nn * MV_KT_PITCH + mm) = make_float4(v[0], v[1], v[2], v[3]);
                    acc[j][2 * h] = acc[j][2 * h + 1] = 0ull;
                }
            }
            // coefficients of this chunk -> shared memory, [m][o]
            for (int idx = tid; idx < MV_TILE * OT; idx += MV_THREADS) {
                const int mm = idx & (MV_TILE - 1), o = idx >> 7;
                const bool ok = (mc0 + mm < m_end) && (o0 + o < p.O);
                s_c[mm * OT + o] = ok ? C[(long long)(o0 + o) * p.ldc + mc0 + mm] : 0.0f;
            }
            {
                // Diagonal rule, applied to the parked tile: row n holds 1 + reg at m = n + delta.
                // Read once per tile, so nothing of it stays live through the k loop.
                const float reg       = (p.kernel_type != KM_KERNEL_NONE) ? read_hyper(p.regularization, l) : 0.0f;
                const long long delta = (long long)p.reg_off_n - (long long)p.reg_off_m;
                if (reg != 0.0f && mc0 + MV_TILE > n0 + delta && mc0 < n0 + delta + MV_TILE) {
                    __syncthreads();
                    const long long m_want = n0 + cn + delta;
                    if (ch == 0 && m_want >= mc0 && m_want < mc0 + MV_TILE && m_want < m_end)
                        s_kt[cn * MV_KT_PITCH + (int)(m_want - mc0)] = 1.0f + reg;
                }
            }
            __syncthreads();
            if constexpr (OT >= 4) {
#pragma unroll 2
                for (int mm = 0; mm < MV_TILE; mm += 4) {
                    const float4 k4  = *reinterpret_cast<const float4*>(s_kt + cn * MV_KT_PITCH + mm);
                    const float kv[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const u64 kd  = pack2(kv[e], kv[e]);
                        const u64* cp = reinterpret_cast<const u64*>(s_c + (mm + e) * OT + ch * OH);
#pragma unroll
                        for (int i = 0; i < OH / 2; ++i) yacc[i] = fma2(kd, cp[i], yacc[i]);
                    }
                }
            } else {
                // OT == 2: one channel per thread half
                float y0, y1;
                unpack2(yacc[0], y0, y1);
#pragma unroll 8
                for (int mm = 0; mm < MV_TILE; ++mm) y0 = fmaf(s_kt[cn * MV_KT_PITCH + mm], s_c[mm * OT + ch], y0);
                yacc[0] = pack2(y0, y1);
            }
            // the next chunk's epilogue overwrites s_kt / s_c only after the barrier at
            // the top of a later iteration, which every thread passes after this point
        }
    }
    cp_async_wait<0>();

    const int n = n0 + cn;
    if (n < p.N) {
        float* yrow = p.Y + (long long)split * p.split_stride + (long long)l * p.y_sl + (long long)n * p.y_sn;
        if constexpr (OT >= 4) {
#pragma unroll
            for (int i = 0; i < OH / 2; ++i) {
                float v0, v1;
                unpack2(yacc[i], v0, v1);
                const int o = o0 + ch * OH + 2 * i;
                if (o < p.O) yrow[(long long)o * p.y_so] = v0;
                if (o + 1 < p.O) yrow[(long long)(o + 1) * p.y_so] = v1;
            }
        } else {
            float v0, v1;
            unpack2(yacc[0], v0, v1);
            const int o = o0 + ch;
            if (o < p.O) yrow[(long long)o * p.y_so] = v0;
        }
    }
}

// ---------------------------------------------------------------------------
// Tensor-core contraction.  Same walk as matvec_kernel, but the coefficient product
// of each 128 (n) x 128 (m) kernel-matrix tile runs on the 5th-generation tensor
// cores: D[n, o] (128 x 16, fp32, in tensor memory) += Ktile[n, m] * c[o, m]^T with
// tcgen05.mma kind::tf32 reading both operands from shared memory.
//
// fp32 accuracy is kept by splitting every operand value x into hi = x with the 13
// low mantissa bits cleared (exactly representable in tf32) and lo = x - hi, and
// issuing three products per k-block: hi*c_hi + lo*c_hi + hi*c_lo (the dropped
// lo*c_lo term is below 2^-22 of the product).
//
// A tile is contracted in two rounds of 64 m-columns (the columns a thread holds in
// its accumulator halves h = 0, 1), so that hi and lo of a round fit in 64 KiB.
// Operand tiles use the K-major 128-byte-swizzle layout (see km_tcgen05.cuh): 32
// floats per 128-byte row, one slab of rows per 32 m-columns.
//
// The tensor core truncates when it adds into its fp32 accumulator, so a long chain
// of MMAs drifts low (measured: 5e-6 relative after 48 steps on same-sign data).
// Chains are therefore kept short: per tile, each round's hi*c_hi products (8 MMAs)
// have their own 16-column accumulator and the two correction products share a third,
// whose truncation is relative to sums 2^-11 smaller.  The three partial sums are
// added, rounding to nearest, to the thread's fp32 running sums one tile later, when
// the tile's MMAs are known to be complete (two sets of accumulators alternate).
// One mbarrier tracks MMA completion (tcgen05.commit); every wait on it is bounded.
constexpr int MT_OT         = 16;
constexpr int MT_SLAB_A     = 128 * 128;              // bytes: 128 rows (n) of 32 floats
constexpr int MT_SLAB_B     = MT_OT * 128;            // bytes: 16 rows (o) of 32 floats
constexpr int MT_A_BYTES    = 2 * MT_SLAB_A;          // one round: 64 m-columns
constexpr int MT_B_BYTES    = 2 * MT_SLAB_B;
constexpr int MT_OFF_A_HI   = 0;
constexpr int MT_OFF_A_LO   = MT_A_BYTES;
constexpr int MT_OFF_B_HI   = 2 * MT_A_BYTES;
constexpr int MT_OFF_B_LO   = 2 * MT_A_BYTES + MT_B_BYTES;
constexpr int MT_TILE_BYTES = 2 * MT_A_BYTES + 2 * MT_B_BYTES;
constexpr int MT_SMEM_BYTES = 1024 + MT_TILE_BYTES + MV_STAGES * MV_STAGE_FLOATS * 4;
constexpr int MT_TMEM_SET   = 64;                     // columns per tile: main h=0, main h=1, corrections, (unused)
constexpr int MT_TMEM_COLS  = 2 * MT_TMEM_SET;
static_assert(MT_TILE_BYTES % 1024 == 0 && MT_SLAB_B % 1024 == 0, "operand slabs must stay 1024-byte aligned");

__device__ int g_matvec_wait_expired = 0;

__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); }

//
// Operand staging comes in two forms.  TMA = false: the 2-stage cp.async pipeline of
// matvec_kernel (any layout).  TMA = true (operands contiguous along m / n, 16-byte
// aligned): tiled TMA copies (no multicast) into a 2-stage ring with a full and an empty
// mbarrier per stage, each stage refilled by the arrival that completes its empty phase, so
// the k loop has no block-wide barrier, no per-thread copy instructions and no wait for a
// stage's release.
template <int INNER, bool AVEC, bool BVEC, bool TMA>
__global__ void __launch_bounds__(MV_THREADS, 2)
matvec_tensor_kernel(const __grid_constant__ MatvecParams p, const __grid_constant__ CUtensorMap map_a,
                     const __grid_constant__ CUtensorMap map_b) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long s_bar;
    __shared__ __align__(8) unsigned long long s_ring[2 * MV_STAGES];   // full[0..], empty[0..]
    __shared__ uint32_t s_tmem;

    const uint32_t raw_addr  = smem_u32(smem_raw);
    const uint32_t tile_addr = (raw_addr + 1023u) & ~1023u;          // operand tiles, 1024-byte aligned
    unsigned char* tiles     = smem_raw + (tile_addr - raw_addr);
    float* stages            = reinterpret_cast<float*>(tiles + MT_TILE_BYTES);
    const uint32_t bar       = smem_u32(&s_bar);

    const int tid  = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int tn    = blockIdx.x % p.tiles_n;
    const int split = blockIdx.x / p.tiles_n;
    const int oc    = blockIdx.y;
    const int l     = blockIdx.z;
    const int n0 = tn * MV_TILE;
    const int o0 = oc * MT_OT;
    const int m_begin = split * p.m_per_split;
    const int m_end   = min(p.M, m_begin + p.m_per_split);
    const int chunks  = (m_end > m_begin) ? (m_end - m_begin + MV_TILE - 1) / MV_TILE : 0;

    const float* A = p.A + (long long)l * p.a_sl;
    const float* B = p.B + (long long)l * p.b_sl + (long long)n0 * p.b_sn;
    const float* C = p.C + (long long)l * p.c_sl;
    const int rem_n = p.N - n0;
    const int K = p.K;
    const int ktiles = K > 0 ? (K + MV_BK - 1) / MV_BK : 1;
    const int total  = chunks * ktiles;

    const float p_inner = (INNER == IN_DIFF_POW || INNER == IN_DOT_POW) ? read_hyper(p.p_inner, l) : 0.0f;
    const Epilogue epi  = make_epilogue(p.outer_power, p.kernel_type, p.p_outer, p.bandwidth, p.epsilon, l);

    const uint32_t ring = smem_u32(s_ring);
    auto full_bar  = [&](int s) { return ring + 8u * s; };
    auto empty_bar = [&](int s) { return ring + 8u * (MV_STAGES + s); };
    if (tid == 0) {
        mbar_init(bar, 1);
        if constexpr (TMA) {
#pragma unroll
            for (int s = 0; s < MV_STAGES; ++s) {
                mbar_init(full_bar(s), 1);
                mbar_init(empty_bar(s), MV_THREADS / 32);
            }
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        tc::fence_smem_to_async();
    }
    if (warp == 0) tc::tmem_alloc(smem_u32(&s_tmem), MT_TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = s_tmem;

    const int lm = lane & 7, ln = lane >> 3;
    const int wm = warp & 1, wn = warp >> 1;
    const int tm_off = wm * 64 + lm * 4;
    const int tn_off = wn * 32 + ln * 4;

    // read-back role: row cn of the tile, channels ch * 8 .. ch * 8 + 7
    const int cn = tid & (MV_TILE - 1);
    const int ch = tid >> 7;
    const uint32_t tmem_mine = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + ch * 8;
    float yacc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) yacc[i] = 0.0f;

    // coefficient staging role: channel co, 16-byte chunk cq of the round's 64 columns
    const int co = tid >> 4;
    const int cq = tid & 15;

    u64 acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0ull;

    bool pending = false;   // a commit has been issued that nobody has waited for yet
    int  parity  = 0;
    bool expired = false;
    auto wait_mma = [&]() {
        if (pending) {
            // once a wait has run out this thread stops waiting, so a stuck barrier costs one limit, not one per tile
            if (!expired && !mbar_wait_bounded(bar, parity)) expired = true;
            parity ^= 1;
            pending = false;
        }
    };
    auto drain = [&](int buffer) {
        tc::fence_after_sync();
#pragma unroll
        for (int part = 0; part < 3; ++part) {
            uint32_t r[8];
            tc::ld_32x32b_x8(tmem_mine + buffer * MT_TMEM_SET + part * MT_OT, r);
#pragma unroll
            for (int i = 0; i < 8; ++i) yacc[i] += __uint_as_float(r[i]);
        }
        tc::fence_before_sync();
    };

    constexpr int PITCH        = TMA ? MV_TILE : MV_PITCH;               // floats per staged k row
    constexpr int STAGE_FLOATS = 2 * MV_BK * PITCH;
    const int la = (p.a_sl == 0) ? 0 : l;   // broadcast operands have a single batch slice in their map
    const int lb = (p.b_sl == 0) ? 0 : l;
    int fail_it = -1;                       // first slab whose wait ran out on this thread

    auto stage = [&](int it) {
        const int chunk = it / ktiles, kt = it - chunk * ktiles;
        const int mc0   = m_begin + chunk * MV_TILE;
        float* st       = stages + (it % MV_STAGES) * STAGE_FLOATS;
        if constexpr (TMA) {
            const int s        = it % MV_STAGES;
            const uint32_t dst = smem_u32(st);
            mbar_expect_tx(full_bar(s), STAGE_FLOATS * 4);
            tma_load_3d(dst, &map_a, mc0, kt * MV_BK, la, full_bar(s));
            tma_load_3d(dst + MV_BK * PITCH * 4, &map_b, n0, kt * MV_BK, lb, full_bar(s));
        } else {
            stage_operand<AVEC, MV_BK>(st, A + (long long)mc0 * p.a_sm, p.a_sm, p.a_sk, m_end - mc0, K, kt, tid);
            stage_operand<BVEC, MV_BK>(st + MV_BK * MV_PITCH, B, p.b_sn, p.b_sk, rem_n, K, kt, tid);
        }
    };

    if constexpr (TMA) {
        if (tid == 0)
            for (int it = 0; it < MV_STAGES && it < total; ++it) stage(it);
    } else {
        if (total > 0) stage(0);
        cp_async_commit();
    }

    for (int it = 0; it < total; ++it) {
        const int chunk = it / ktiles, kt = it - chunk * ktiles;
        const int s     = it % MV_STAGES;
        if constexpr (TMA) {
            if (!expired && !mbar_wait_bounded(full_bar(s), (it / MV_STAGES) & 1)) {
                expired = true;
                fail_it = it;
            }
        } else {
            cp_async_wait<0>();
            __syncthreads();
            if (it + 1 < total) stage(it + 1);
            cp_async_commit();
        }

        const float* sa = stages + s * STAGE_FLOATS + tm_off;
        const float* sb = stages + s * STAGE_FLOATS + MV_BK * PITCH + tn_off;
        consume_slab<INNER, MV_BK, PITCH>(acc, sa, sb, K - kt * MV_BK, p_inner, 1.0f);
        if constexpr (TMA) {
            // the arrival that completes the stage's empty phase refills it on the spot: nobody
            // waits for a stage to be released
            __syncwarp();
            if (lane == 0 && mbar_arrive_pending(empty_bar(s)) == 1 && it + MV_STAGES < total && !expired) {
                mbar_try_wait(empty_bar(s), (it / MV_STAGES) & 1);   // the acquire side of the hand-over
                stage(it + MV_STAGES);
            }
        }

        if (kt == ktiles - 1) {
            const int mc0 = m_begin + chunk * MV_TILE;
            const uint32_t d_set = tmem + (chunk & 1) * MT_TMEM_SET;
            // diagonal rule; read here, once per tile, so nothing of it stays live through the k loop
            const float reg       = (p.kernel_type != KM_KERNEL_NONE) ? read_hyper(p.regularization, l) : 0.0f;
            const long long delta = (long long)p.reg_off_n - (long long)p.reg_off_m;   // diagonal: m == n + delta
            const bool on_diagonal = (reg != 0.0f && mc0 + MV_TILE > n0 + delta && mc0 < n0 + delta + MV_TILE);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                // outer chain of this round's 32 values, in place; in the last, partial tile of the m
                // range the columns outside it become 0
                apply_epilogue(epi, acc, 2 * h, 2);
                if (mc0 + MV_TILE > m_end) {
                    const int mcol = mc0 + tm_off + h * 32;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float v[4];
                        unpack2(acc[j][2 * h], v[0], v[1]);
                        unpack2(acc[j][2 * h + 1], v[2], v[3]);
#pragma unroll
                        for (int e = 0; e < 4; ++e) v[e] = (mcol + e < m_end) ? v[e] : 0.0f;
                        acc[j][2 * h]     = pack2(v[0], v[1]);
                        acc[j][2 * h + 1] = pack2(v[2], v[3]);
                    }
                }
                // this thread's four coefficients of the round: local column q <-> m = mc0 + (q / 32) * 64 + h * 32 + q % 32
                float cv[4];
                {
                    const int q  = cq * 4;
                    const int mg = mc0 + (q >> 5) * 64 + h * 32 + (q & 31);
                    const bool o_ok = (o0 + co < p.O);
                    const float* crow = C + (long long)(o0 + co) * p.ldc;
#pragma unroll
                    for (int e = 0; e < 4; ++e) cv[e] = (o_ok && mg + e < m_end) ? crow[mg + e] : 0.0f;
                }
                // the previous round's MMAs must have finished reading the operand tiles
                wait_mma();
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int r = tn_off + (j >> 2) * 16 + (j & 3);
                    float v[4];
                    unpack2(acc[j][2 * h], v[0], v[1]);
                    unpack2(acc[j][2 * h + 1], v[2], v[3]);
                    float hi[4], lo[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) { hi[e] = tf32_hi(v[e]); lo[e] = v[e] - hi[e]; }
                    const int off = wm * MT_SLAB_A + r * 128 + ((lm ^ (r & 7)) << 4);
                    *reinterpret_cast<float4*>(tiles + MT_OFF_A_HI + off) = make_float4(hi[0], hi[1], hi[2], hi[3]);
                    *reinterpret_cast<float4*>(tiles + MT_OFF_A_LO + off) = make_float4(lo[0], lo[1], lo[2], lo[3]);
                    acc[j][2 * h] = acc[j][2 * h + 1] = 0ull;
                }
                {
                    float hi[4], lo[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) { hi[e] = tf32_hi(cv[e]); lo[e] = cv[e] - hi[e]; }
                    const int off = (cq >> 3) * MT_SLAB_B + co * 128 + (((cq & 7) ^ (co & 7)) << 4);
                    *reinterpret_cast<float4*>(tiles + MT_OFF_B_HI + off) = make_float4(hi[0], hi[1], hi[2], hi[3]);
                    *reinterpret_cast<float4*>(tiles + MT_OFF_B_LO + off) = make_float4(lo[0], lo[1], lo[2], lo[3]);
                }
                if (on_diagonal) {
                    // diagonal rule on the parked tile: row n holds 1 + reg at m = n + delta
                    __syncthreads();
                    const long long m_want = n0 + cn + delta;
                    const int ml           = (int)(m_want - mc0);          // column inside the 128-wide tile
                    if (ch == 0 && m_want >= mc0 && ml < MV_TILE && m_want < m_end && ((ml >> 5) & 1) == h) {
                        const int q     = (ml >> 6) * 32 + (ml & 31);      // column inside this round
                        const int off   = (q >> 5) * MT_SLAB_A + cn * 128 + ((((q & 31) >> 2) ^ (cn & 7)) << 4) + (q & 3) * 4;
                        const float one = 1.0f + reg;
                        const float hi  = tf32_hi(one);
                        *reinterpret_cast<float*>(tiles + MT_OFF_A_HI + off) = hi;
                        *reinterpret_cast<float*>(tiles + MT_OFF_A_LO + off) = one - hi;
                    }
                }
                tc::fence_smem_to_async();
                tc::fence_before_sync();
                __syncthreads();
                if (tid == 0) {
                    tc::fence_after_sync();
                    constexpr uint32_t idesc = tc::instr_desc_tf32(MV_TILE, MT_OT);
#pragma unroll
                    for (int pass = 0; pass < 3; ++pass) {
                        const uint32_t a_base = tile_addr + (pass == 1 ? MT_OFF_A_LO : MT_OFF_A_HI);
                        const uint32_t b_base = tile_addr + (pass == 2 ? MT_OFF_B_LO : MT_OFF_B_HI);
#pragma unroll
                        for (int kb = 0; kb < 8; ++kb) {
                            const uint64_t da = tc::smem_desc_k_major_sw128(a_base + (kb >> 2) * MT_SLAB_A + (kb & 3) * 32);
                            const uint64_t db = tc::smem_desc_k_major_sw128(b_base + (kb >> 2) * MT_SLAB_B + (kb & 3) * 32);
                            if (pass == 0) tc::mma_tf32(d_set + h * MT_OT, da, db, idesc, kb != 0);
                            else           tc::mma_tf32(d_set + 2 * MT_OT, da, db, idesc, !(h == 0 && pass == 1 && kb == 0));
                        }
                    }
                    tc::commit(bar);
                }
                pending = true;
            }
            // the tile before this one finished before this tile's first round started
            if (chunk > 0) drain((chunk - 1) & 1);
        }
    }
    cp_async_wait<0>();

    wait_mma();
    if (chunks > 0) drain((chunks - 1) & 1);
    if (expired) {
        atomicExch(&g_matvec_wait_expired, 1);
        if constexpr (TMA) {
            // give copies already handed to the TMA engine a bounded chance to land before
            // this block's shared memory is released
            // (any warp may have requested the slabs from the failing one on; those never requested
            // simply run the short limit out)
            if (tid == 0) {
                const int first = fail_it < 0 ? 0 : fail_it;
                const int last  = first + MV_STAGES < total ? first + MV_STAGES : total;
                for (int slab = first; slab < last; ++slab)
                    for (int i = 0; i < (1 << 16); ++i)
                        if (mbar_try_wait(full_bar(slab % MV_STAGES), (slab / MV_STAGES) & 1)) break;
            }
        }
    }

    const int n = n0 + cn;
    if (n < p.N && !expired) {
        float* yrow = p.Y + (long long)split * p.split_stride + (long long)l * p.y_sl + (long long)n * p.y_sn;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int o = o0 + ch * 8 + i;
            if (o < p.O) yrow[(long long)o * p.y_so] = yacc[i];
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem, MT_TMEM_COLS);
}

__global__ void __launch_bounds__(256) matvec_reduce_kernel(const float* __restrict__ partial, float* __restrict__ y,
                                                            int N, int O, int L, int splits, long long split_stride,
                                                            long long y_sn, long long y_so, long long y_sl) {
    const long long total = (long long)L * N * O;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        float s = 0.0f;
        for (int sp = 0; sp < splits; ++sp) s += partial[sp * split_stride + i];
        long long r = i;
        const int o = (int)(r % O); r /= O;
        const int n = (int)(r % N); r /= N;
        const int l = (int)r;
        y[l * y_sl + n * y_sn + o * y_so] = s;
    }
}

typedef void (*MatvecFn)(const MatvecParams);

template <int INNER, int OT>
MatvecFn mv_pick_layout(bool avec, bool bvec) {
    if (avec && bvec) return matvec_kernel<INNER, OT, true, true>;
    if (avec) return matvec_kernel<INNER, OT, true, false>;
    if (bvec) return matvec_kernel<INNER, OT, false, true>;
    return matvec_kernel<INNER, OT, false, false>;
}
template <int INNER>
MatvecFn mv_pick_ot(int ot, bool avec, bool bvec) {
    switch (ot) {
        case 2: return mv_pick_layout<INNER, 2>(avec, bvec);
        case 4: return mv_pick_layout<INNER, 4>(avec, bvec);
        case 8: return mv_pick_layout<INNER, 8>(avec, bvec);
        default: return mv_pick_layout<INNER, 16>(avec, bvec);
    }
}
MatvecFn mv_pick(int inner, int ot, bool avec, bool bvec) {
    switch (inner) {
        case IN_DIFF_ABS: return mv_pick_ot<IN_DIFF_ABS>(ot, avec, bvec);
        case IN_DIFF_SQUARE: return mv_pick_ot<IN_DIFF_SQUARE>(ot, avec, bvec);
        case IN_DIFF_POW: return mv_pick_ot<IN_DIFF_POW>(ot, avec, bvec);
        case IN_DOT_NOOP: return mv_pick_ot<IN_DOT_NOOP>(ot, avec, bvec);
    }
    return nullptr;
}
typedef void (*MatvecTensorFn)(const MatvecParams, const CUtensorMap, const CUtensorMap);

template <int INNER>
MatvecTensorFn mv_pick_tensor_layout(bool avec, bool bvec, bool tma) {
    if (tma) return matvec_tensor_kernel<INNER, true, true, true>;
    if (avec && bvec) return matvec_tensor_kernel<INNER, true, true, false>;
    if (avec) return matvec_tensor_kernel<INNER, true, false, false>;
    if (bvec) return matvec_tensor_kernel<INNER, false, true, false>;
    return matvec_tensor_kernel<INNER, false, false, false>;
}
MatvecTensorFn mv_pick_tensor(int inner, bool avec, bool bvec, bool tma) {
    switch (inner) {
        case IN_DIFF_ABS: return mv_pick_tensor_layout<IN_DIFF_ABS>(avec, bvec, tma);
        case IN_DIFF_SQUARE: return mv_pick_tensor_layout<IN_DIFF_SQUARE>(avec, bvec, tma);
        case IN_DIFF_POW: return mv_pick_tensor_layout<IN_DIFF_POW>(avec, bvec, tma);
        case IN_DOT_NOOP: return mv_pick_tensor_layout<IN_DOT_NOOP>(avec, bvec, tma);
    }
    return nullptr;
}
int mv_smem_for(int ot) {
    switch (ot) {
        case 2: return mv_smem_bytes<2>();
        case 4: return mv_smem_bytes<4>();
        case 8: return mv_smem_bytes<8>();
        default: return mv_smem_bytes<16>();
    }
}

bool mv_layout_ok(long long rows, long long cols, long long s_row, long long s_col) {
    if (rows <= 0 || cols <= 0) return true;
    return (s_col == 1 && s_row >= cols) || (s_row == 1 && s_col >= rows);
}

struct MatvecPlan {
    MatvecParams p;
    int ot;
    bool avec, bvec;
    bool tensor;              // contraction on the tensor cores (3 x tf32) instead of packed FP32
    bool tma;                 // tensor kernel with TMA operand staging
    int splits_wanted;
    long long partial_elems;
};

int make_matvec_plan(const KmMatvecArgs* a, MatvecPlan* plan) {
    if (!a) return fail(KM_ERR_NULL_POINTER, "args is NULL");
    if (a->m < 0 || a->n < 0 || a->k < 0 || a->o < 0 || a->l < 1)
        return fail(KM_ERR_BAD_SHAPE, "bad extents m=%d n=%d k=%d o=%d l=%d", a->m, a->n, a->k, a->o, a->l);
    if (a->l > 65535) return fail(KM_ERR_TOO_LARGE, "at most 65535 batch entries per call");
    const bool empty = (a->n == 0 || a->o == 0);
    if (!empty && (!a->y || (a->m > 0 && (!a->c || (a->k > 0 && (!a->a || !a->b))))))
        return fail(KM_ERR_NULL_POINTER, "a, b, c and y must be device pointers");
    if (a->inner_operator < 0 || a->inner_operator > KM_INNER_DOT || a->inner_power < 0 || a->inner_power > KM_POW_POW ||
        a->outer_power < 0 || a->outer_power > KM_POW_POW || a->kernel_type < 0 || a->kernel_type > KM_KERNEL_GAUSSIAN)
        return fail(KM_ERR_BAD_ENUM, "descriptor enums out of range");
    if (!mv_layout_ok(a->m, a->k, a->a_stride_m, a->a_stride_k))
        return fail(KM_ERR_BAD_STRIDE, "a has a non-standard memory layout");
    if (!mv_layout_ok(a->n, a->k, a->b_stride_n, a->b_stride_k))
        return fail(KM_ERR_BAD_STRIDE, "b has a non-standard memory layout");
    if (a->o > 1 && a->ldc < a->m) return fail(KM_ERR_BAD_STRIDE, "ldc is smaller than m");
    if (a->a_stride_l < 0 || a->b_stride_l < 0 || a->c_stride_l < 0 || a->y_stride_l < 0 || a->y_stride_n < 0 ||
        a->y_stride_o < 0)
        return fail(KM_ERR_BAD_STRIDE, "strides must be non-negative");
    if (!hyper_ok(a->p_inner) || !hyper_ok(a->p_outer) || !hyper_ok(a->bandwidth) || !hyper_ok(a->regularization))
        return fail(KM_ERR_BAD_HYPERPARAM, "hyper-parameter vectors need a non-negative batch stride");
    if (a->split_m < 0) return fail(KM_ERR_BAD_SHAPE, "split_m must be >= 0");
    if (a->contraction < KM_CONTRACT_AUTO || a->contraction > KM_CONTRACT_TENSOR)
        return fail(KM_ERR_BAD_ENUM, "contraction must be KM_CONTRACT_AUTO, _FP32 or _TENSOR");

    MatvecParams& p = plan->p;
    p.M = a->m; p.N = a->n; p.K = a->k; p.O = a->o; p.L = a->l;
    p.A = a->a; p.a_sm = a->a_stride_m; p.a_sk = a->a_stride_k; p.a_sl = a->a_stride_l;
    p.B = a->b; p.b_sn = a->b_stride_n; p.b_sk = a->b_stride_k; p.b_sl = a->b_stride_l;
    p.C = a->c; p.ldc = a->ldc; p.c_sl = a->c_stride_l;
    p.inner_id = inner_id(a->inner_operator, a->inner_power);
    if (!mv_pick(p.inner_id, 16, false, false))
        return fail(KM_ERR_BAD_ENUM, "kernel_matvec supports the inner steps |b-a|, (b-a)^2, |b-a|^p and b*a");
    p.outer_power = a->outer_power;
    p.kernel_type = a->kernel_type;
    p.p_inner = a->p_inner; p.p_outer = a->p_outer; p.bandwidth = a->bandwidth;
    p.regularization = a->regularization;
    p.reg_off_m = a->reg_off_x; p.reg_off_n = a->reg_off_y;
    p.epsilon = a->epsilon;
    plan->tensor = (a->contraction != KM_CONTRACT_FP32);
    int ot = 2;
    while (ot < a->o && ot < 16) ot *= 2;
    if (plan->tensor) ot = MT_OT;
    plan->ot   = ot;
    p.tiles_n  = (int)ceil_div_ll(p.N, MV_TILE);
    p.o_chunks = (int)ceil_div_ll(p.O > 0 ? p.O : 1, ot);
    if (p.o_chunks > 65535) return fail(KM_ERR_TOO_LARGE, "too many output channels");
    plan->avec = (p.a_sm == 1) && aligned16(p.A) && (p.a_sk % 4 == 0 || p.K <= 1) && (p.a_sl % 4 == 0);
    plan->bvec = (p.b_sn == 1) && aligned16(p.B) && (p.b_sk % 4 == 0 || p.K <= 1) && (p.b_sl % 4 == 0);
    // Measured on B200 (K=64, M=N=131072, O=16): TMA staging takes the (b-a)^2 walk from 345 to
    // 323 ms per 262144^2 pairs; for |b-a| and |b-a|^p it changes nothing (90.9 vs 90.9 ms,
    // 448 vs 450 ms), so those keep the cp.async pipeline, which accepts every layout.
    const bool tma_inner = (p.inner_id == IN_DIFF_SQUARE || p.inner_id == IN_DOT_NOOP);
    plan->tma = plan->tensor && tma_inner && p.K >= 1 && p.M > 0 && p.N > 0 &&
                tma_operand_ok(p.A, p.a_sm, p.a_sk, p.a_sl, p.K, p.L) &&
                tma_operand_ok(p.B, p.b_sn, p.b_sk, p.b_sl, p.K, p.L);

    // Preferred m split: fill whole waves of 2 blocks per SM when the row tiles alone
    // leave more than ~10 % of a wave idle.
    const long long blocks = (long long)p.tiles_n * p.o_chunks * p.L;
    const long long slots  = 2LL * sm_count();
    int want = 1;
    if (blocks > 0) {
        const double waves = (double)blocks / (double)slots;
        const double eff   = waves / (double)ceil_div_ll(blocks, slots);
        if (eff < 0.9) {
            // smallest split that brings the efficiency above 0.95, capped by chunk count
            const int max_split = (int)ceil_div_ll(p.M > 0 ? p.M : 1, 8 * MV_TILE);
            for (int s = 2; s <= 32 && s <= max_split; ++s) {
                const double w = (double)(blocks * s) / (double)slots;
                if (w / (double)ceil_div_ll(blocks * s, slots) >= 0.95) { want = s; break; }
                want = s;
            }
        }
    }
    plan->splits_wanted = want;
    plan->partial_elems = (long long)p.L * p.N * p.O;
    return 0;
}

}  // namespace
}  // namespace km

namespace km {
// Reads back and clears the flag a bounded wait of matvec_tensor_kernel sets (device already synchronised).
int matvec_take_wait_flag() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_matvec_wait_expired, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_matvec_wait_expired, &zero, sizeof(int));
    return v ? 1 : 0;
}
}  // namespace km

extern "C" int64_t kermac_b200_kernel_matvec_scratch_bytes(const KmMatvecArgs* args) {
    using namespace km;
    MatvecPlan plan;
    if (make_matvec_plan(args, &plan)) return 0;
    int splits = args->split_m > 0 ? args->split_m : plan.splits_wanted;
    if (splits <= 1) return 0;
    return (int64_t)splits * plan.partial_elems * 4;
}

extern "C" int kermac_b200_kernel_matvec(const KmMatvecArgs* args, void* stream) {
    using namespace km;
    MatvecPlan plan;
    if (int rc = make_matvec_plan(args, &plan)) return rc;
    MatvecParams& p = plan.p;
    if (p.N == 0 || p.O == 0) return 0;
    if (int rc = require_sm100()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    int splits = args->split_m > 0 ? args->split_m : plan.splits_wanted;
    if (splits > 1) {
        const int64_t need = (int64_t)splits * plan.partial_elems * 4;
        if (!args->scratch || args->scratch_bytes < need) {
            if (args->split_m > 1)
                return fail(KM_ERR_BAD_SHAPE, "split_m=%d needs %lld bytes of scratch, got %lld", splits, (long long)need,
                            (long long)(args->scratch ? args->scratch_bytes : 0));
            splits = 1;
        }
    }
    const int chunks = (int)ceil_div_ll(p.M > 0 ? p.M : 1, MV_TILE);
    p.m_per_split    = (int)ceil_div_ll(chunks, splits) * MV_TILE;
    splits           = (int)ceil_div_ll(p.M > 0 ? p.M : 1, p.m_per_split);
    p.splits         = splits;
    if (splits > 1) {
        p.Y = static_cast<float*>(args->scratch);
        p.y_so = 1; p.y_sn = p.O; p.y_sl = (long long)p.N * p.O;
        p.split_stride = plan.partial_elems;
    } else {
        p.Y = args->y;
        p.y_sn = args->y_stride_n; p.y_so = args->y_stride_o; p.y_sl = args->y_stride_l;
        p.split_stride = 0;
    }
    dim3 grid((unsigned)((long long)p.tiles_n * splits), (unsigned)p.o_chunks, (unsigned)p.L);
    if (plan.tensor) {
        MatvecTensorFn fn = mv_pick_tensor(p.inner_id, plan.avec, plan.bvec, plan.tma);
        if (!fn) return fail(KM_ERR_INTERNAL, "no matvec kernel for inner id %d", p.inner_id);
        if (int rc = cuda_status(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, MT_SMEM_BYTES),
                                 "cudaFuncSetAttribute(matvec_tensor_kernel)"))
            return rc;
        CUtensorMap map_a, map_b;
        memset(&map_a, 0, sizeof(map_a));
        memset(&map_b, 0, sizeof(map_b));
        if (plan.tma) {
            if (int rc = encode_tma_operand(&map_a, p.A, p.M, p.K, p.L, p.a_sk, p.a_sl, MV_BK)) return rc;
            if (int rc = encode_tma_operand(&map_b, p.B, p.N, p.K, p.L, p.b_sk, p.b_sl, MV_BK)) return rc;
        }
        fn<<<grid, MV_THREADS, MT_SMEM_BYTES, st>>>(p, map_a, map_b);
        if (int rc = cuda_status(cudaGetLastError(), "launch of matvec_tensor_kernel")) return rc;
    } else {
        MatvecFn fn = mv_pick(p.inner_id, plan.ot, plan.avec, plan.bvec);
        if (!fn) return fail(KM_ERR_INTERNAL, "no matvec kernel for inner id %d", p.inner_id);
        const int smem_bytes = mv_smem_for(plan.ot);
        if (int rc = cuda_status(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes),
                                 "cudaFuncSetAttribute(matvec_kernel)"))
            return rc;
        fn<<<grid, MV_THREADS, smem_bytes, st>>>(p);
        if (int rc = cuda_status(cudaGetLastError(), "launch of matvec_kernel")) return rc;
    }
    if (splits > 1) {
        const long long total = plan.partial_elems;
        int blocks = (int)(ceil_div_ll(total, 256) < 4LL * sm_count() ? ceil_div_ll(total, 256) : 4LL * sm_count());
        matvec_reduce_kernel<<<blocks, 256, 0, st>>>(p.Y, args->y, p.N, p.O, p.L, splits, plan.partial_elems,
                                                     args->y_stride_n, args->y_stride_o, args->y_stride_l);
        if (int rc = cuda_status(cudaGetLastError(), "launch of matvec_reduce_kernel")) return rc;
    }
    return 0;
}
