// Argument block shared by every matrix-product kernel of the engine.
//
//   C[c_row(i), n] (=|+=) epilogue( sum_k A[a_row(i), k] * W[g(i)][n, k] )      i in [0, M)
//
// A is [rows, K] with leading dimension lda; W is [groups][N (or 2N), K], row-major
// ("out, in"), groups `w_group_stride` elements apart.  Logical rows are split
// among the groups by `group_offsets[0..n_groups]` (ascending; rows of group g are
// [off[g], off[g+1])); with no offsets there is one group.  `a_rows` gathers the
// rows of A, `c_rows` scatters the rows of C; either may be null (identity).
// `row_scale`, if given, is indexed by a_row(i) when `scale_by_a_row` else by i.
#pragma once
#include "common.cuh"

enum GemmEpilogue {
    EPI_STORE = 0,        // C (activation type) = acc * scale
    EPI_STORE_F32 = 1,    // C (float32) = acc * scale
    EPI_ADD_F32 = 2,      // C (float32) += acc * scale          (residual stream)
    EPI_SWIGLU = 3        // C (activation type) = silu(s*gate) * (s*up); W rows [0,N) gate, [N,2N) up
};

struct GemmParams {
    const void* A;
    const void* W;
    void* C;
    const int* a_rows;
    const int* c_rows;
    const int* group_offsets;
    const float* row_scale;
    long long lda, ldc, w_group_stride;
    int n_groups, M, N, K;
    int epilogue;
    int scale_by_a_row;
};

__device__ __forceinline__ float silu_f32(float g) { return g / (1.0f + expf(-g)); }

// Finds the (group, first row, row count) of the `tile`-th row tile when every
// group is cut into tiles of `bm` rows of its own.  Returns false past the end.
__device__ __forceinline__ bool locate_row_tile(const GemmParams& p, int tile, int bm,
                                                int& group, int& row0, int& rows) {
    if (!p.group_offsets) {
        group = 0; row0 = tile * bm; rows = min(bm, p.M - row0);
        return row0 < p.M;
    }
    for (int g = 0; g < p.n_groups; ++g) {
        const int lo = p.group_offsets[g], hi = p.group_offsets[g + 1];
        const int tiles = (hi - lo + bm - 1) / bm;
        if (tile < tiles) { group = g; row0 = lo + tile * bm; rows = min(bm, hi - row0); return true; }
        tile -= tiles;
    }
    return false;
}
