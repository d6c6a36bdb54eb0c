// What the tcgen05 product kernels share: the epilogue that moves one row of an accumulator from
// tensor memory to the output, and the host-side tensor maps and tile-width choice.
#pragma once
#include "gemm.cuh"
#include "tcgen05.cuh"

namespace tc {

// One thread, one accumulator row: logical row `li` of the product (row `li` of the sorted order in
// a grouped product), output columns n0 .. n0 + cols_per_tile - 1, read 32 columns at a time from
// tensor memory at `lane_addr` (the SwiGLU form reads the gate columns there and the up columns
// `bnh` columns on).  Warp-collective: every lane calls it, `row_ok` says whether its row exists.
template <int EPI>
__device__ __forceinline__ void drain_accumulator_row(const GemmParams& p, int li, bool row_ok, int n0,
                                                      int cols_per_tile, int bnh, unsigned lane_addr) {
    constexpr bool DUAL = (EPI == EPI_SWIGLU);
    int crow = li, srow = li;
    float sc = 1.f;
    if (row_ok) {
        if (p.c_rows) crow = p.c_rows[li];
        if (p.row_scale) {
            if (p.scale_by_a_row && p.a_rows) srow = p.a_rows[li];
            sc = p.row_scale[srow];
        }
    }
#pragma unroll 1
    for (int c0 = 0; c0 < cols_per_tile; c0 += 32) {
        float v[32];
        ld32(v, lane_addr + c0);                    // warp-collective: every lane takes part
        float u[32];
        if (DUAL) ld32(u, lane_addr + bnh + c0);
        const int n = n0 + c0;
        if (!row_ok || n >= p.N) continue;
        const size_t o = (size_t)crow * p.ldc + n;
        const bool full = (n + 32 <= p.N);
        if (EPI == EPI_STORE || EPI == EPI_SWIGLU) {
            __nv_bfloat16* dst = (__nv_bfloat16*)p.C + o;
            float y[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) y[i] = DUAL ? silu_f32(v[i] * sc) * (u[i] * sc) : v[i] * sc;
            if (full && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 q;
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(y[i], y[i + 1]), h1 = __floats2bfloat162_rn(y[i + 2], y[i + 3]);
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(y[i + 4], y[i + 5]), h3 = __floats2bfloat162_rn(y[i + 6], y[i + 7]);
                    q.x = *(unsigned*)&h0; q.y = *(unsigned*)&h1; q.z = *(unsigned*)&h2; q.w = *(unsigned*)&h3;
                    *(uint4*)(dst + i) = q;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (n + i < p.N) dst[i] = __float2bfloat16_rn(y[i]);
            }
        } else {
            float* dst = (float*)p.C + o;
            if (full && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    float4 q = make_float4(v[i] * sc, v[i + 1] * sc, v[i + 2] * sc, v[i + 3] * sc);
                    if (EPI == EPI_ADD_F32) {
                        const float4 old = *(const float4*)(dst + i);
                        q.x += old.x; q.y += old.y; q.z += old.z; q.w += old.w;
                    }
                    *(float4*)(dst + i) = q;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (n + i < p.N) dst[i] = (EPI == EPI_ADD_F32 ? dst[i] : 0.f) + v[i] * sc;
            }
        }
    }
}

// A row-major [rows, cols] bfloat16 matrix with leading dimension ld; boxes of 64 columns x box_rows rows.
static inline bool make_matrix_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld,
                                   int box_rows) {
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    return make_map(map, base, 2, dims, strides, box);
}

}  // namespace tc
