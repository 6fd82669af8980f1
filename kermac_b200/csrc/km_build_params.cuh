// Device-side parameter block of the kernel-matrix build kernels, filled by the
// launcher in km_build_launch.cu after validation and the operand exchange for
// n-contiguous outputs (the role of src/kermac/build_a_kernel.py:323-390 in the
// reference).
#pragma once

#include "km_common.cuh"

namespace km {

// Geometry shared by the launcher and the build kernels.
constexpr int BUILD_TILE           = 128;   // output tile edge (m and n)
constexpr int BUILD_CPA_THREADS    = 256;
#ifndef KM_CPA_BK
#define KM_CPA_BK 32
#endif
constexpr int BUILD_CPA_BK         = KM_CPA_BK;   // k rows per staged slab
constexpr int BUILD_CPA_STAGES     = 3;
constexpr int BUILD_CPA_PITCH      = 132;   // floats per staged k row; 528 bytes keeps rows 16-byte aligned
constexpr int BUILD_CPA_SMEM_BYTES = BUILD_CPA_STAGES * 2 * BUILD_CPA_BK * BUILD_CPA_PITCH * 4;

struct BuildParams {
    int M, N, K, L;                 // kernel-side extents: C is (M, N) with M contiguous
    const float* A; long long a_sm, a_sk, a_sl;
    const float* B; long long b_sn, b_sk, b_sl;
    float*       C; long long c_ld, c_sl;   // C[l][n][m] = C[l * c_sl + n * c_ld + m]
    int inner_id, outer_power, kernel_type;
    KmHyper p_inner, p_outer, bandwidth, regularization;
    int   reg_off_m, reg_off_n;     // diagonal rule in kernel coordinates: reg_off_m + m == reg_off_n + n
    float epsilon;
    float sgn;                      // -1 when A and B were exchanged, else +1
    int   tiles_m, tiles_n;         // 128 x 128 output tiles
    int   panel;                    // rasterisation: n-tiles per panel
    int   tile_count;               // thread blocks (tiles) of this launch per batch entry
    int   tile_first;               // linear index of the tile that block 0 computes (a launch may cover a sub-range)
    int   c_vec4;                   // C rows may be written with 16-byte stores
    int   c_multicast;              // C is an NVSwitch multicast address: write with multimem.st
    int   symmetric;                // A and B are the same matrix and the chain is symmetric in (m, n):
                                    // tiles with tile_n < tile_m are skipped, the others also write their mirror image
};

// Maps a linear tile index to (tile_m, tile_n) so that thread blocks that run at
// the same time cover a compact patch of the output and share A and B tiles in L2.
// Panels of `panel` tile-columns are walked row by row.
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int panel, int& tm, int& tn) {
    const int per_panel = panel * tiles_m;
    const int pidx      = t / per_panel;
    const int r         = t - pidx * per_panel;
    const int n0        = pidx * panel;
    const int width     = min(panel, tiles_n - n0);
    tm                  = r / width;
    tn                  = n0 + (r - tm * width);
}

}  // namespace km
