// Matrix product for few tokens (decode): y[M, N] = x[M, K] W[N, K]^T with at most 64
// rows per group, bfloat16 inputs, float32 sums.
//
// With few tokens the product is bound by reading W once from HBM.  The weight rows are
// the 16-row operand of mma.sync.m16n8k16 and the tokens its 8 columns, so 8 tokens cost
// one instruction per 16x16 weight tile.  Each lane fetches 16 contiguous bytes of a
// weight row straight into its fragment registers: the k index inside a 32-wide step is
// permuted, identically for W and x, which leaves every dot product unchanged.
//
// The kernel is persistent: a fixed number of blocks walk the work items (group, tile of
// 32 weight rows; 16 gate + 16 up rows for the SwiGLU epilogue) with a stride of the grid
// size.  A block's 8 warps split K; each warp keeps a ring of U steps of weight and token
// fragments in flight, and the first steps of the next item are requested before the
// current item's partial sums meet in shared memory, so the stream from HBM keeps
// flowing through the epilogue.
// An output element is summed in an order fixed by K alone, whatever else is in the batch.
//
// Grouped form (experts): the tokens of group g are rows [off[g], off[g+1]) of the sorted
// order, gathered through a_rows; groups without tokens are skipped on the device.
#include "gemm.cuh"

namespace {

constexpr int WARPS = 8;
constexpr int MAX_GROUPS = 1024;
constexpr int MAX_ACTIVE = MAX_GROUPS + 64;   // (group, token chunk) pairs of one call

__device__ __forceinline__ void mma16816(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream(const void* p) {     // read once: do not keep in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::256B.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

struct Item {                     // one work item of a block
    int group, row_lo, m, tile;
};

// NFRAG: 16-row weight fragments per warp (2, or 1 for narrow matrices, which then have twice
// as many items to spread over the multiprocessors; the SwiGLU form needs 2: gate and up).
template <int NT, int U, int EPI, int NFRAG>
__global__ void __launch_bounds__(WARPS * 32, (NT <= 1 ? 2 : 1)) gemm_skinny_kernel(const GemmParams p) {
    constexpr bool DUAL = (EPI == EPI_SWIGLU);
    static_assert(!DUAL || NFRAG == 2, "the SwiGLU epilogue pairs a gate and an up fragment");
    constexpr int ROWS = DUAL ? 16 : 16 * NFRAG;                 // output columns (weight rows) per item
    constexpr int TOK = NT * 8;
    extern __shared__ float red[];                               // [WARPS][NFRAG*16][TOK]
    __shared__ int active_s[MAX_ACTIVE];
    __shared__ int n_active_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int n_tiles = (p.N + ROWS - 1) / ROWS;
    // Routed calls read the group sizes, which the step's router wrote: wait for it first.
    // One-group calls know their items without any earlier kernel's data: they start their
    // first weight loads and wait only before they touch the tokens.
    if (p.group_offsets) { pdl_wait(); pdl_launch_dependents(); }

    // (group, chunk of TOK tokens) pairs that have tokens: a group with more than TOK tokens
    // streams its weights once per chunk
    if (warp == 0) {
        // lanes read the group sizes side by side (one round trip to memory for 32 groups),
        // then the list is written in group order
        int n = 0;
        const int groups = p.group_offsets ? p.n_groups : 1;
        for (int e0 = 0; e0 < groups; e0 += 32) {
            const int e = e0 + lane;
            int m = 0;
            if (e < groups) m = p.group_offsets ? p.group_offsets[e + 1] - p.group_offsets[e] : p.M;
            const int chunks = (m + TOK - 1) / TOK;
            int before = chunks;                                 // inclusive scan of the chunk counts
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, before, o);
                if (lane >= o) before += v;
            }
            const int start = n + before - chunks;
            for (int ch = 0; ch < chunks; ++ch)
                if (start + ch < MAX_ACTIVE) active_s[start + ch] = e | (ch << 16);
            n += __shfl_sync(0xffffffffu, before, 31);
        }
        if (lane == 0) n_active_s = min(n, MAX_ACTIVE);
    }
    __syncthreads();
    const int total = n_active_s * n_tiles;

    auto item_at = [&](int i) {
        Item it;
        const int a = active_s[i / n_tiles];
        it.group = a & 0xffff;
        it.tile = i % n_tiles;
        const int lo = p.group_offsets ? p.group_offsets[it.group] : 0;
        const int m = p.group_offsets ? p.group_offsets[it.group + 1] - lo : p.M;
        it.row_lo = lo + (a >> 16) * TOK;
        it.m = min(TOK, m - (a >> 16) * TOK);
        return it;
    };
    const __nv_bfloat16* X = (const __nv_bfloat16*)p.A;
    auto weight_rows = [&](const Item& it, const __nv_bfloat16* (&wrow)[NFRAG][2]) {
        const __nv_bfloat16* W = (const __nv_bfloat16*)p.W + (size_t)it.group * p.w_group_stride;
        const int n0 = it.tile * ROWS;
#pragma unroll
        for (int f = 0; f < NFRAG; ++f)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int r = DUAL ? (n0 + g + 8 * h + (f ? p.N : 0)) : (n0 + 16 * f + g + 8 * h);
                const int last = DUAL ? (f ? 2 * p.N - 1 : p.N - 1) : p.N - 1;
                wrow[f][h] = W + (size_t)min(r, last) * p.K + 8 * c;
            }
    };
    auto token_rows = [&](const Item& it, const __nv_bfloat16* (&xrow)[NT]) {
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int t = 8 * j + g;
            if (t < it.m) {
                const int li = it.row_lo + t;
                xrow[j] = X + (size_t)(p.a_rows ? p.a_rows[li] : li) * p.lda + 8 * c;
            } else {
                xrow[j] = nullptr;
            }
        }
    };

    // this warp's share of the 32-wide k steps
    const int steps = p.K >> 5;
    const int s_begin = (int)((long long)steps * warp / WARPS), s_end = (int)((long long)steps * (warp + 1) / WARPS);
    const int n_my = s_end - s_begin;

    int i_cur = blockIdx.x;
    if (i_cur >= total) return;
    Item cur = item_at(i_cur);
    const __nv_bfloat16* wrow[NFRAG][2];
    const __nv_bfloat16* xrow[NT];
    uint4 wbuf[U][NFRAG][2];
    uint4 xbuf[U][NT];

    // first U steps of an item into the ring
    auto fill_ring = [&](bool with_weights) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (u < n_my) {
                const size_t off = (size_t)(s_begin + u) * 32;
                if (with_weights) {
#pragma unroll
                    for (int f = 0; f < NFRAG; ++f)
#pragma unroll
                        for (int h = 0; h < 2; ++h) wbuf[u][f][h] = ld_stream(wrow[f][h] + off);
                }
#pragma unroll
                for (int j = 0; j < NT; ++j)
                    xbuf[u][j] = xrow[j] ? *(const uint4*)(xrow[j] + off) : make_uint4(0, 0, 0, 0);
            }
        }
    };
    weight_rows(cur, wrow);
    if (!p.group_offsets) {
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (u < n_my) {
#pragma unroll
                for (int f = 0; f < NFRAG; ++f)
#pragma unroll
                    for (int h = 0; h < 2; ++h) wbuf[u][f][h] = ld_stream(wrow[f][h] + (size_t)(s_begin + u) * 32);
            }
        pdl_wait();
        pdl_launch_dependents();
    }
    token_rows(cur, xrow);
    fill_ring(p.group_offsets != nullptr);          // one-group calls have their weights on the way already

    for (; i_cur < total; i_cur += gridDim.x) {
        float acc[NFRAG][NT][4];
#pragma unroll
        for (int f = 0; f < NFRAG; ++f)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[f][j][e] = 0.f;

        for (int i0 = 0; i0 < n_my; i0 += U) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int i = i0 + u;
                if (i < n_my) {
                    uint4 w[NFRAG][2], xv[NT];
#pragma unroll
                    for (int f = 0; f < NFRAG; ++f) { w[f][0] = wbuf[u][f][0]; w[f][1] = wbuf[u][f][1]; }
#pragma unroll
                    for (int j = 0; j < NT; ++j) xv[j] = xbuf[u][j];
                    if (i + U < n_my) {                          // refill this ring slot, U steps ahead
                        const size_t off = (size_t)(s_begin + i + U) * 32;
#pragma unroll
                        for (int f = 0; f < NFRAG; ++f)
#pragma unroll
                            for (int h = 0; h < 2; ++h) wbuf[u][f][h] = ld_stream(wrow[f][h] + off);
#pragma unroll
                        for (int j = 0; j < NT; ++j)
                            xbuf[u][j] = xrow[j] ? *(const uint4*)(xrow[j] + off) : make_uint4(0, 0, 0, 0);
                    }
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
        // the next item's first steps go out now and travel while this item's sums are reduced
        const Item done = cur;
        if (i_cur + gridDim.x < total) {
            cur = item_at(i_cur + gridDim.x);
            weight_rows(cur, wrow);
            token_rows(cur, xrow);
            fill_ring(true);
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
        const int n0 = done.tile * ROWS;
        const int n_tok = min(TOK, done.m);
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
            const int li = done.row_lo + t;
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

template <int NT, int U, int NFRAG>
int launch_nf(const GemmParams& p, int n_blocks, cudaStream_t st) {
    const int rows = p.epilogue == EPI_SWIGLU ? 16 : 16 * NFRAG;
    const long long tiles = (long long)((p.N + rows - 1) / rows) * (p.group_offsets ? p.n_groups : 1);
    const int grid = (int)(tiles < n_blocks ? tiles : n_blocks);
    const size_t smem = (size_t)WARPS * NFRAG * 16 * NT * 8 * sizeof(float);
#define SPITE_SKINNY_CASE(E, NF)                                                                          \
    case E: {                                                                                             \
        auto k = gemm_skinny_kernel<NT, U, E, NF>;                                                        \
        if (smem > 44 * 1024 &&                                                                           \
            cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
            return SPITE_LAUNCH_FAILED;                                                                   \
        SPITE_LAUNCH(k, grid, WARPS * 32, smem, st, p);                                                   \
        break;                                                                                            \
    }
    switch (p.epilogue) {
        SPITE_SKINNY_CASE(EPI_STORE, NFRAG)
        SPITE_SKINNY_CASE(EPI_STORE_F32, NFRAG)
        SPITE_SKINNY_CASE(EPI_ADD_F32, NFRAG)
        SPITE_SKINNY_CASE(EPI_SWIGLU, 2)
        default: return SPITE_BAD_ARG;
    }
#undef SPITE_SKINNY_CASE
    return spite_launch_status();
}

// 32-row items throughout.  16-row items for narrow matrices (twice the items to spread) were
// measured slower on B200 at 5120 x 5120 .. 7168 x 5120: the per-item reduction costs more than
// the extra parallelism gains, so the one-fragment instantiation is not used.  Runs of 8 to 32 rows
// cut so that every resident block gets one equal item made each such product 3-9 % faster alone
// and the decode step slower (batch 1: 223 against 238 tokens/s): with fewer items than resident
// blocks the next kernel's blocks start on the free slots and fetch their first weights early.
template <int NT, int U>
int launch_nt(const GemmParams& p, int n_blocks, cudaStream_t st) {
    return launch_nf<NT, U, 2>(p, n_blocks, st);
}

}  // namespace

// `max_rows_per_group`: an upper bound on the tokens of any group (M for one group).
// `n_blocks`: twice the number of multiprocessors; the launch uses as many blocks as stay resident
// (two per multiprocessor up to 8 tokens, one above), fewer if there is less work.
SPITE_API int spite_gemm_skinny(const GemmParams* p, int max_rows_per_group, int n_blocks, void* stream) {
    if (!p || !p->A || !p->W || !p->C) return SPITE_BAD_ARG;
    if (p->M < 0 || p->N <= 0 || p->K <= 0 || p->lda < p->K || p->ldc < p->N || n_blocks < 1) return SPITE_BAD_ARG;
    if (p->group_offsets ? p->n_groups < 1 : p->n_groups != 1) return SPITE_BAD_ARG;
    if (p->epilogue < 0 || p->epilogue > EPI_SWIGLU) return SPITE_BAD_ARG;
    if (p->K % 32 || p->lda % 8) return SPITE_UNSUPPORTED;                 // 16-byte loads, 32-wide steps
    if (((uintptr_t)p->A | (uintptr_t)p->W) & 15) return SPITE_UNSUPPORTED;
    if (max_rows_per_group < 1 || p->n_groups > MAX_GROUPS || p->M > 64 * 8) return SPITE_UNSUPPORTED;
    if (p->M == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const int half = (n_blocks + 1) / 2;                                   // kernels that fit once per multiprocessor
    // Tokens per pass: a group with more tokens than one pass holds streams its weights again
    // for the next chunk.  Groups of a routed batch are small, so 16 tokens a pass serve them;
    // one dense group of up to 64 tokens is held whole.
    if (max_rows_per_group <= 8) return launch_nt<1, 4>(*p, n_blocks, st);
    if (max_rows_per_group <= 16 || p->group_offsets) return launch_nt<2, 4>(*p, half, st);
    if (max_rows_per_group <= 32) return launch_nt<4, 2>(*p, half, st);
    if (max_rows_per_group <= 64) return launch_nt<8, 2>(*p, half, st);
    return SPITE_UNSUPPORTED;
}
