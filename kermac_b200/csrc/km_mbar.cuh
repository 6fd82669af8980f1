// mbarrier helpers shared by the kernels that wait on asynchronous units (TMA copies,
// tensor-core commits).  Every wait is bounded.
#pragma once

#include <cuda.h>

#include <cstdint>

namespace km {

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrives and returns how many arrivals the current phase was still waiting for BEFORE this
// one: 1 means this arrival completed the phase (exactly one arriving thread sees 1).
__device__ __forceinline__ uint32_t mbar_arrive_pending(uint32_t bar) {
    uint32_t count;
    asm volatile(
        "{\n\t.reg .b64 state;\n\t"
        "mbarrier.arrive.shared::cta.b64 state, [%1];\n\t"
        "mbarrier.pending_count.b64 %0, state;\n\t}"
        : "=r"(count)
        : "r"(bar)
        : "memory");
    return count;
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, int parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
// Waits for the phase of `bar` with the given parity; gives up after `tries` attempts
// (the default amounts to seconds at most) and returns false.
constexpr int MBAR_WAIT_TRIES = 1 << 22;
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, int parity, int tries = MBAR_WAIT_TRIES) {
    for (int i = 0; i < tries; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// Tiled TMA copy (no multicast) of one box of a rank-3 tensor into shared memory; the
// mbarrier receives the byte count.  x is the innermost coordinate: x * 4 bytes must be a
// multiple of 16.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}

}  // namespace km
