// Matrix product for few tokens (decode): y[M, N] = x[M, K] W[N, K]^T with M <= 64
// rows per group, bfloat16 inputs, float32 sums.
//
// With few tokens the product is bound by reading W once from HBM.  The weight
// rows are the 16-row operand of mma.sync.m16n8k16 and the tokens its 8 columns,
// so 8 tokens cost one instruction per 16x16 weight tile.  Each lane fetches 16
// contiguous bytes of a weight row straight into its fragment registers: the k
// index inside a 32-wide step is permuted, identically for W and x, which leaves
// every dot product unchanged.  A block of 8 warps owns 32 weight rows (or 16 gate
// and 16 up rows for the SwiGLU epilogue) and splits K among its warps; the partial
// sums meet in shared memory, where the epilogue runs.  An output element is summed
// in an order fixed by K alone, whatever else is in the batch.
//
// Grouped form (experts): blockIdx.y is the group; its tokens are
// rows [off[g], off[g+1]) of the sorted order, gathered through a_rows.
#include "gemm.cuh"

namespace {

constexpr int WARPS = 8;
constexpr int NFRAG = 2;          // 16-row weight fragments per warp

__device__ __forceinline__ void mma16816(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream(const void* p) {     // read once: do not keep in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

template <int NT, int U, int EPI>
__global__ void __launch_bounds__(WARPS * 32) gemm_skinny_kernel(const GemmParams p) {
    constexpr bool DUAL = (EPI == EPI_SWIGLU);
    constexpr int ROWS = DUAL ? 16 : 32;                         // output columns (weight rows) per block
    constexpr int TOK = NT * 8;
    extern __shared__ float red[];                               // [WARPS][NFRAG*16][TOK]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int group = blockIdx.y;
    int row_lo = 0, m = p.M;
    if (p.group_offsets) {
        row_lo = p.group_offsets[group];
        m = p.group_offsets[group + 1] - row_lo;
    }
    if (m <= 0) return;
    const int n0 = blockIdx.x * ROWS;
    const __nv_bfloat16* W = (const __nv_bfloat16*)p.W + (size_t)group * p.w_group_stride;
    const __nv_bfloat16* X = (const __nv_bfloat16*)p.A;

    // weight row pointers of this lane: fragment f, rows g and g+8
    const __nv_bfloat16* wrow[NFRAG][2];
#pragma unroll
    for (int f = 0; f < NFRAG; ++f)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            int r = DUAL ? (n0 + g + 8 * h + (f ? p.N : 0)) : (n0 + 16 * f + g + 8 * h);
            const int last = DUAL ? (f ? 2 * p.N - 1 : p.N - 1) : p.N - 1;
            wrow[f][h] = W + (size_t)min(r, last) * p.K + 8 * c;
        }

    const int steps = p.K >> 5;
    const int s_begin = (int)((long long)steps * warp / WARPS), s_end = (int)((long long)steps * (warp + 1) / WARPS);

    for (int t0 = 0; t0 < m; t0 += TOK) {                        // one pass unless a group has more than TOK tokens
        const __nv_bfloat16* xrow[NT];
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int t = t0 + 8 * j + g;
            if (t < m) {
                const int li = row_lo + t;
                xrow[j] = X + (size_t)(p.a_rows ? p.a_rows[li] : li) * p.lda + 8 * c;
            } else {
                xrow[j] = nullptr;
            }
        }
        float acc[NFRAG][NT][4];
#pragma unroll
        for (int f = 0; f < NFRAG; ++f)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[f][j][e] = 0.f;

        uint4 wbuf[U][NFRAG][2];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int s = min(s_begin + u, steps - 1);
#pragma unroll
            for (int f = 0; f < NFRAG; ++f)
#pragma unroll
                for (int h = 0; h < 2; ++h) wbuf[u][f][h] = ld_stream(wrow[f][h] + (size_t)s * 32);
        }
        for (int s0 = s_begin; s0 < s_end; s0 += U) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int s = s0 + u;
                if (s < s_end) {
                    uint4 xv[NT];
#pragma unroll
                    for (int j = 0; j < NT; ++j)
                        xv[j] = xrow[j] ? *(const uint4*)(xrow[j] + (size_t)s * 32) : make_uint4(0, 0, 0, 0);
                    uint4 w[NFRAG][2];
#pragma unroll
                    for (int f = 0; f < NFRAG; ++f) { w[f][0] = wbuf[u][f][0]; w[f][1] = wbuf[u][f][1]; }
                    const int sn = min(s + U, steps - 1);
#pragma unroll
                    for (int f = 0; f < NFRAG; ++f)
#pragma unroll
                        for (int h = 0; h < 2; ++h) wbuf[u][f][h] = ld_stream(wrow[f][h] + (size_t)sn * 32);
#pragma unroll
                    for (int f = 0; f < NFRAG; ++f)
#pragma unroll
                        for (int j = 0; j < NT; ++j) {
                            mma16816(acc[f][j], w[f][0].x, w[f][1].x, w[f][0].y, w[f][1].y, xv[j].x, xv[j].y);
                            mma16816(acc[f][j], w[f][0].z, w[f][1].z, w[f][0].w, w[f][1].w, xv[j].z, xv[j].w);
                        }
                }
            }
        }
        // partial sums of this warp: red[warp][fragment row][token]
        __syncthreads();
#pragma unroll
        for (int f = 0; f < NFRAG; ++f)
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                float* base = red + ((size_t)warp * NFRAG * 16 + f * 16) * TOK + 8 * j + 2 * c;
                base[(size_t)g * TOK] = acc[f][j][0];
                base[(size_t)g * TOK + 1] = acc[f][j][1];
                base[(size_t)(g + 8) * TOK] = acc[f][j][2];
                base[(size_t)(g + 8) * TOK + 1] = acc[f][j][3];
            }
        __syncthreads();
        // epilogue: one output element per thread and round, weight rows fastest
        const int n_tok = min(TOK, m - t0);
        for (int idx = threadIdx.x; idx < ROWS * n_tok; idx += WARPS * 32) {
            const int r = idx % ROWS, t = idx / ROWS;
            const int n = n0 + r;
            if (n >= p.N) continue;
            float v = 0.f, v2 = 0.f;
#pragma unroll
            for (int w8 = 0; w8 < WARPS; ++w8) {
                v += red[((size_t)w8 * NFRAG * 16 + r) * TOK + t];
                if (DUAL) v2 += red[((size_t)w8 * NFRAG * 16 + 16 + r) * TOK + t];
            }
            const int li = row_lo + t0 + t;
            const int arow = p.a_rows ? p.a_rows[li] : li;
            const int crow = p.c_rows ? p.c_rows[li] : li;
            const float sc = p.row_scale ? p.row_scale[p.scale_by_a_row ? arow : li] : 1.f;
            const size_t o = (size_t)crow * p.ldc + n;
            if (EPI == EPI_STORE) ((__nv_bfloat16*)p.C)[o] = __float2bfloat16_rn(v * sc);
            else if (EPI == EPI_STORE_F32) ((float*)p.C)[o] = v * sc;
            else if (EPI == EPI_ADD_F32) ((float*)p.C)[o] += v * sc;
            else ((__nv_bfloat16*)p.C)[o] = __float2bfloat16_rn(silu_f32(v * sc) * (v2 * sc));
        }
    }
}

template <int NT, int U>
int launch_nt(const GemmParams& p, cudaStream_t st) {
    const int rows = p.epilogue == EPI_SWIGLU ? 16 : 32;
    dim3 grid((p.N + rows - 1) / rows, p.group_offsets ? p.n_groups : 1);
    if (grid.y > 65535) return SPITE_UNSUPPORTED;
    const size_t smem = (size_t)WARPS * NFRAG * 16 * NT * 8 * sizeof(float);
#define SPITE_SKINNY_CASE(E)                                                                              \
    case E: {                                                                                             \
        auto k = gemm_skinny_kernel<NT, U, E>;                                                            \
        if (smem > 48 * 1024 &&                                                                           \
            cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
            return SPITE_LAUNCH_FAILED;                                                                   \
        k<<<grid, WARPS * 32, smem, st>>>(p);                                                             \
        break;                                                                                            \
    }
    switch (p.epilogue) {
        SPITE_SKINNY_CASE(EPI_STORE)
        SPITE_SKINNY_CASE(EPI_STORE_F32)
        SPITE_SKINNY_CASE(EPI_ADD_F32)
        SPITE_SKINNY_CASE(EPI_SWIGLU)
        default: return SPITE_BAD_ARG;
    }
#undef SPITE_SKINNY_CASE
    return spite_launch_status();
}

}  // namespace

int gemm_check(const GemmParams* p);

// `max_rows_per_group`: an upper bound on the tokens of any group (M for one group).
SPITE_API int spite_gemm_skinny(const GemmParams* p, int max_rows_per_group, void* stream) {
    if (!p || !p->A || !p->W || !p->C) return SPITE_BAD_ARG;
    if (p->M < 0 || p->N <= 0 || p->K <= 0 || p->lda < p->K || p->ldc < p->N) return SPITE_BAD_ARG;
    if (p->group_offsets ? p->n_groups < 1 : p->n_groups != 1) return SPITE_BAD_ARG;
    if (p->K % 32 || p->lda % 8) return SPITE_UNSUPPORTED;                 // 16-byte loads, 32-wide steps
    if (((uintptr_t)p->A | (uintptr_t)p->W) & 15) return SPITE_UNSUPPORTED;
    if (max_rows_per_group < 1 || max_rows_per_group > 64) return SPITE_UNSUPPORTED;
    if (p->M == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (max_rows_per_group <= 8) return launch_nt<1, 4>(*p, st);
    if (max_rows_per_group <= 16) return launch_nt<2, 4>(*p, st);
    if (max_rows_per_group <= 32) return launch_nt<4, 2>(*p, st);
    return launch_nt<8, 2>(*p, st);
}
