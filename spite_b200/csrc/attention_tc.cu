// Attention over the paged cache for prompt portions on the fifth-generation tensor cores
// (bfloat16, head size 64 or 128, pages of a multiple of 64 keys, up to 128 query heads per kv head).
//
// A block owns 128 rows of the score matrix: (token, query head of one kv group) pairs of
// consecutive tokens of one request, row = token * group + head.  It walks the visible keys in
// tiles of 64 (one TMA box, never across a page).  Roles:
//   warp 0    one lane loads the rows of q once (a three-dimensional TMA box: 64 elements x
//             the group's heads x the tokens, which lands row by row in the 128-byte-swizzled
//             K-major layout) and then the K and V tiles into two rings of two stages each;
//   warp 1    allocates tensor memory (two score tiles of 64 columns and the output tile of
//             head-size columns); one lane issues  S = Q K^T  (128 x 64 x head size) and
//             O += P V  (128 x head size x 64; V is used as it lies in the cache, as an
//             MN-major operand), two score tiles ahead of the softmax;
//   warps 2-5 one thread per row: read a score tile with tcgen05.ld, scale and mask it, keep the
//             running maximum and sum in float32, write P as bfloat16 into shared memory in
//             the K-major operand layout, and at the end divide the output by the sum.
// The output accumulates in tensor memory.  A row's reference maximum moves only when the
// tile's maximum exceeds it by more than 8 (in log2 units): then the row's part of O and its
// sum are multiplied by 2^(old - new) before the next product is added.  P stays below 2^8, and
// the result is the same softmax(S) V up to rounding, since sum and output share the reference.
// Two blocks fit a multiprocessor (112 KiB of shared memory and 256 tensor-memory columns
// each), so one block's softmax overlaps the other's products.
//
// Score, mask and softmax: crates/spite-compute/src/flash_attn.rs:111-156; window rules in
// attention.cuh.  Every wait is bounded (see tcgen05.cuh); spite_attention_tc_error() returns
// and clears the code of a wait that gave up: 1 loader, 2 tensor-core issue, 3 softmax.
#include "attention.cuh"
#include "tcgen05.cuh"

namespace {
using namespace tc;

constexpr int BM = 128;                 // rows a block owns
constexpr int BN = 64;                  // keys per tile
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 256;
constexpr float RESCALE_STEP = 8.f;     // log2 units
constexpr float LOG2E = 1.4426950408889634f;

__device__ int g_attn_tc_error = 0;

struct Barriers {
    unsigned long long q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], s_free[2], p_ready, pv_done;
    unsigned tmem_base;
    int abort_flag;
};

__device__ __forceinline__ unsigned pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *(unsigned*)&v;
}

// NKB = head_dim / 64.  grid (blocks over (request, token tile), kv heads).
template <int NKB>
__global__ void __launch_bounds__(THREADS, 2)
attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, const AttentionParams p, const StepTokens b,
               const PagedCache c, const AttnMmaExtra x, const int q_box_tokens) {
    constexpr int HD = 64 * NKB;
    constexpr int Q_BYTES = NKB * BM * 128;
    constexpr int KT_BYTES = NKB * BN * 128;             // one K tile, one V tile
    extern __shared__ __align__(1024) unsigned char smem[];   // [Q][K0][K1][V0][V1][P], each 1024-byte aligned
    __shared__ Barriers bars;
    pdl_wait();
    pdl_launch_dependents();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nq = p.num_heads, nkv = c.num_kv_heads, G = nq / nkv;
    const int kvh = blockIdx.y;

    // which request and which of its tokens; the blocks with the most keys start first
    int idx = gridDim.x - 1 - blockIdx.x, seg = -1, t0 = 0, nt = 0;
    for (int s = 0; s < x.n_segments; ++s) {
        const int lo = x.cu_seqlens[s], n = x.cu_seqlens[s + 1] - lo;
        if (n < x.seg_min_tokens || n > x.seg_max_tokens) continue;   // another kernel serves this segment
        const int blocks = (n + x.tokens_per_block - 1) / x.tokens_per_block;
        if (idx < blocks) { seg = s; t0 = lo + idx * x.tokens_per_block; nt = min(x.tokens_per_block, lo + n - t0); break; }
        idx -= blocks;
    }
    if (seg < 0) return;                                  // before any barrier or allocation: the whole block leaves
    const int n_rows = nt * G;
    const int* table = b.block_table + (size_t)seg * b.table_width;
    const int p_first = b.positions[t0], p_last = b.positions[t0 + nt - 1];
    const int lo_first = window_lowest(p.window_kind, p.window_size, p_first);
    const int lo_last = window_lowest(p.window_kind, p.window_size, p_last);
    const int k_begin = (lo_first / BN) * BN;
    const int n_tiles = (p_last - k_begin) / BN + 1;

    unsigned char* q_s = smem;
    unsigned char* k_s = q_s + Q_BYTES;
    unsigned char* v_s = k_s + 2 * KT_BYTES;
    unsigned char* p_s = v_s + 2 * KT_BYTES;
    volatile int* abort_flag = &bars.abort_flag;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bars.q_full), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&bars.k_full[s]), 1); mbar_init(smem_u32(&bars.k_empty[s]), 1);
            mbar_init(smem_u32(&bars.v_full[s]), 1); mbar_init(smem_u32(&bars.v_empty[s]), 1);
            mbar_init(smem_u32(&bars.s_full[s]), 1); mbar_init(smem_u32(&bars.s_free[s]), BM);
        }
        mbar_init(smem_u32(&bars.p_ready), BM);
        mbar_init(smem_u32(&bars.pv_done), 1);
        bars.abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc(&bars.tmem_base, TMEM_COLS);
    if (warp >= 2) {
        // rows of the q tile that the TMA box does not write: zero, so that their scores are plain numbers
        const int r = (warp & 3) * 32 + lane;
        if (r >= q_box_tokens * G) {
#pragma unroll
            for (int kb = 0; kb < NKB; ++kb)
#pragma unroll
                for (int ch = 0; ch < 8; ++ch) *(uint4*)(q_s + kb * BM * 128 + r * 128 + ch * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();
    }
    fence_before();
    __syncthreads();
    fence_after();
    const unsigned tmem = bars.tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            // ---- loader
            const unsigned q_bar = smem_u32(&bars.q_full);
            mbar_expect_tx(q_bar, (unsigned)(NKB * q_box_tokens * G * 128));
#pragma unroll
            for (int kb = 0; kb < NKB; ++kb) tma_load_3d(smem_u32(q_s + kb * BM * 128), &map_q, kb * 64, kvh * G, t0, q_bar);
            int issued_k = 0, issued_v = 0;
            for (int i = 0; i < n_tiles; ++i) {
                const int s = i & 1;
                const unsigned ph = (i >> 1) & 1;
                const int j0 = k_begin + i * BN;
                int page = table[j0 / c.page_size];
                if (page < 0 || page >= c.n_pages) page = 0;   // a page behind every row's window: its keys are masked
                const int y = (page * nkv + kvh) * c.page_size + j0 % c.page_size;
                if (!mbar_wait(smem_u32(&bars.k_empty[s]), ph ^ 1, abort_flag, &g_attn_tc_error, 1)) break;
                mbar_expect_tx(smem_u32(&bars.k_full[s]), KT_BYTES);
#pragma unroll
                for (int kb = 0; kb < NKB; ++kb)
                    tma_load_2d(smem_u32(k_s + s * KT_BYTES + kb * BN * 128), &map_k, kb * 64, y, smem_u32(&bars.k_full[s]));
                ++issued_k;
                if (!mbar_wait(smem_u32(&bars.v_empty[s]), ph ^ 1, abort_flag, &g_attn_tc_error, 1)) break;
                mbar_expect_tx(smem_u32(&bars.v_full[s]), KT_BYTES);
#pragma unroll
                for (int kb = 0; kb < NKB; ++kb)
                    tma_load_2d(smem_u32(v_s + s * KT_BYTES + kb * BN * 128), &map_v, kb * 64, y, smem_u32(&bars.v_full[s]));
                ++issued_v;
            }
            if (*abort_flag) {
                // copies in flight must land before the block gives its shared memory back
                mbar_drain(q_bar, 0);
                for (int j = max(0, issued_k - 2); j < issued_k; ++j) mbar_drain(smem_u32(&bars.k_full[j & 1]), (j >> 1) & 1);
                for (int j = max(0, issued_v - 2); j < issued_v; ++j) mbar_drain(smem_u32(&bars.v_full[j & 1]), (j >> 1) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- tensor-core issue
            const unsigned idesc_s = make_idesc(BM, BN), idesc_pv = make_idesc(BM, HD, true);
            bool ok = mbar_wait(smem_u32(&bars.q_full), 0, abort_flag, &g_attn_tc_error, 2);
            auto issue_scores = [&](int j) {
                const int s = j & 1;
                const unsigned ph = (j >> 1) & 1;
                if (!mbar_wait(smem_u32(&bars.k_full[s]), ph, abort_flag, &g_attn_tc_error, 2)) return false;
                if (!mbar_wait(smem_u32(&bars.s_free[s]), ph ^ 1, abort_flag, &g_attn_tc_error, 2)) return false;
                fence_after();
                const unsigned qa = smem_u32(q_s), ka = smem_u32(k_s + s * KT_BYTES);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)
                    mma(tmem + s * BN, smem_desc_k_major(qa + (ks / 4) * BM * 128 + (ks % 4) * 32),
                        smem_desc_k_major(ka + (ks / 4) * BN * 128 + (ks % 4) * 32), idesc_s, ks > 0 ? 1u : 0u);
                commit(smem_u32(&bars.s_full[s]));
                commit(smem_u32(&bars.k_empty[s]));
                return true;
            };
            ok = ok && issue_scores(0);
            if (ok && n_tiles > 1) ok = issue_scores(1);
            for (int i = 0; i < n_tiles && ok; ++i) {
                const int s = i & 1;
                ok = mbar_wait(smem_u32(&bars.p_ready), i & 1, abort_flag, &g_attn_tc_error, 2) &&
                     mbar_wait(smem_u32(&bars.v_full[s]), (i >> 1) & 1, abort_flag, &g_attn_tc_error, 2);
                if (!ok) break;
                fence_after();
                const unsigned pa = smem_u32(p_s), va = smem_u32(v_s + s * KT_BYTES);
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks)
                    mma(tmem + 2 * BN, smem_desc_k_major(pa + ks * 32), smem_desc(va + ks * 16 * 128, BN * 128, 1024),
                        idesc_pv, (i > 0 || ks > 0) ? 1u : 0u);
                commit(smem_u32(&bars.pv_done));
                commit(smem_u32(&bars.v_empty[s]));
                if (i + 2 < n_tiles) ok = issue_scores(i + 2);
            }
        }
    } else {
        // ---- softmax: one thread per row; warp w may read tensor-memory lanes [32 (w % 4), + 32)
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const bool row_ok = r < n_rows;
        const int tok = t0 + (row_ok ? r / G : 0), head = kvh * G + (row_ok ? r % G : 0);
        const int pos = row_ok ? b.positions[tok] : -1;       // a row without a token sees no key
        const int lo = window_lowest(p.window_kind, p.window_size, max(pos, 0));
        const float scale = p.softmax_scale * LOG2E;
        const unsigned lane_base = tmem + ((unsigned)(quarter * 32) << 16);
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int i = 0; i < n_tiles; ++i) {
            const int sb = i & 1;
            ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.s_full[sb]), (i >> 1) & 1, abort_flag, &g_attn_tc_error, 3));
            if (!ok) break;
            fence_after();
            float s[BN];
            {
                float t[32];
                ld32(t, lane_base + sb * BN);
#pragma unroll
                for (int e = 0; e < 32; ++e) s[e] = t[e];
                ld32(t, lane_base + sb * BN + 32);
#pragma unroll
                for (int e = 0; e < 32; ++e) s[32 + e] = t[e];
            }
            fence_before();
            mbar_arrive(smem_u32(&bars.s_free[sb]));          // the tensor cores may overwrite this score tile
            const int j0 = k_begin + i * BN;
            const bool open = j0 >= lo_last && j0 + BN - 1 <= p_first;   // every key visible to every row with a token
            float mx = -INFINITY;
#pragma unroll
            for (int e = 0; e < BN; ++e) {
                float v = s[e] * scale;
                if (!open) { const int j = j0 + e; v = (j >= lo && j <= pos) ? v : -INFINITY; }
                s[e] = v;
                mx = fmaxf(mx, v);
            }
            const bool need = mx > m_ref + RESCALE_STEP;
            float corr = 1.f;
            if (need) { corr = exp2f(m_ref - mx); l *= corr; m_ref = mx; }
            const float m_safe = (m_ref == -INFINITY) ? 0.f : m_ref;
            unsigned packed[BN / 2];
            float sum = 0.f;
#pragma unroll
            for (int e = 0; e < BN; e += 2) {
                const float a = exp2f(s[e] - m_safe), bb = exp2f(s[e + 1] - m_safe);
                sum += a + bb;
                packed[e / 2] = pack_bf16(a, bb);
            }
            l += sum;
            if (i > 0) {
                // the product of the tile before must have read P and left O before either changes
                ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.pv_done), (i - 1) & 1, abort_flag, &g_attn_tc_error, 3));
                if (!ok) break;
                fence_after();
                if (__any_sync(0xffffffffu, need)) {
#pragma unroll 1
                    for (int c0 = 0; c0 < HD; c0 += 32) {
                        float o[32];
                        ld32(o, lane_base + 2 * BN + c0);
#pragma unroll
                        for (int e = 0; e < 32; ++e) o[e] *= corr;
                        st32(lane_base + 2 * BN + c0, o);
                    }
                }
            }
#pragma unroll
            for (int ch = 0; ch < 8; ++ch)
                *(uint4*)(p_s + r * 128 + ((ch ^ (r & 7)) << 4)) =
                    make_uint4(packed[4 * ch], packed[4 * ch + 1], packed[4 * ch + 2], packed[4 * ch + 3]);
            fence_proxy_async();
            fence_before();
            mbar_arrive(smem_u32(&bars.p_ready));
        }
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.pv_done), (n_tiles - 1) & 1, abort_flag, &g_attn_tc_error, 3));
        if (ok) {
            fence_after();
            const float inv = 1.0f / fmaxf(l, 1e-30f);
            __nv_bfloat16* dst = (__nv_bfloat16*)p.out + ((size_t)tok * nq + head) * HD;
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 32) {
                float o[32];
                ld32(o, lane_base + 2 * BN + c0);              // warp-collective: every lane takes part
                if (!row_ok) continue;
#pragma unroll
                for (int e = 0; e < 32; e += 8)
                    *(uint4*)(dst + c0 + e) = make_uint4(pack_bf16(o[e] * inv, o[e + 1] * inv), pack_bf16(o[e + 2] * inv, o[e + 3] * inv),
                                                         pack_bf16(o[e + 4] * inv, o[e + 5] * inv), pack_bf16(o[e + 6] * inv, o[e + 7] * inv));
            }
        }
    }
    fence_before();
    __syncthreads();
    if (warp == 1) {
        fence_after();
        tmem_free(tmem, TMEM_COLS);
    }
}

template <int NKB>
int launch(const AttentionParams& p, const StepTokens& b, const PagedCache& c, const AttnMmaExtra& x, int n_blocks,
           cudaStream_t st) {
    const int hd = 64 * NKB, nq = p.num_heads, nkv = c.num_kv_heads, G = nq / nkv;
    const int box_tokens = x.tokens_per_block < b.n_tokens ? x.tokens_per_block : b.n_tokens;
    CUtensorMap mq, mk, mv;
    {
        cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)nq, (cuuint64_t)b.n_tokens};
        cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)nq * hd * 2};
        cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)box_tokens};
        if (!make_map(&mq, p.q, 3, dims, strides, box)) return SPITE_LAUNCH_FAILED;
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)c.n_pages * nkv * c.page_size};
        cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)BN};
        if (!make_map(&mk, c.kv, 2, dims, strides, box)) return SPITE_LAUNCH_FAILED;
        if (!make_map(&mv, (const __nv_bfloat16*)c.kv + c.v_offset, 2, dims, strides, box)) return SPITE_LAUNCH_FAILED;
    }
    const size_t smem = (size_t)NKB * BM * 128 + 4 * (size_t)NKB * BN * 128 + (size_t)BM * 128;
    auto k = attn_tc_kernel<NKB>;
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return SPITE_LAUNCH_FAILED;
    dim3 grid(n_blocks, nkv);
    SPITE_LAUNCH(k, grid, THREADS, smem, st, mq, mk, mv, p, b, c, x, box_tokens);
    return spite_launch_status();
}

}  // namespace

// `n_blocks` = sum over the served segments of ceil(tokens / tokens_per_block), computed by the caller;
// tokens_per_block * (query heads per kv head) <= 128.
SPITE_API int spite_paged_attention_tc(const AttentionParams* p, const StepTokens* b, const PagedCache* c,
                                       const AttnMmaExtra* x, int n_blocks, void* stream) {
    if (!p || !b || !c || !x || !p->q || !p->out || !x->cu_seqlens || !c->kv) return SPITE_BAD_ARG;
    if (!b->positions || !b->block_table || b->n_tokens < 0 || b->table_width < 1) return SPITE_BAD_ARG;
    if (p->num_heads < 1 || c->num_kv_heads < 1 || p->num_heads % c->num_kv_heads) return SPITE_BAD_ARG;
    if (p->window_kind < 0 || p->window_kind > 2) return SPITE_BAD_ARG;
    if (p->window_kind != SPITE_WINDOW_FULL && p->window_size < 1) return SPITE_BAD_ARG;
    if (x->n_segments < 1 || x->tokens_per_block < 1 || n_blocks < 0 || c->n_pages < 1 || c->page_size < 1) return SPITE_BAD_ARG;
    const int G = p->num_heads / c->num_kv_heads;
    if ((c->head_dim != 64 && c->head_dim != 128) || G > BM || c->page_size % BN) return SPITE_UNSUPPORTED;
    if (x->tokens_per_block * G > BM) return SPITE_BAD_ARG;
    if (c->num_kv_heads > 65535 || p->num_heads > 256 * c->num_kv_heads) return SPITE_UNSUPPORTED;
    if ((long long)c->n_pages * c->num_kv_heads * c->page_size > 0x7fffffffll) return SPITE_UNSUPPORTED;   // TMA coordinates are int32
    if ((((uintptr_t)p->q | (uintptr_t)p->out | (uintptr_t)c->kv) & 15) || (c->v_offset & 7)) return SPITE_UNSUPPORTED;
    if (b->n_tokens == 0 || n_blocks == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    return c->head_dim == 64 ? launch<1>(*p, *b, *c, *x, n_blocks, st) : launch<2>(*p, *b, *c, *x, n_blocks, st);
}

// Error code recorded by a block that gave up waiting (0: none); reading it clears it.
SPITE_API int spite_attention_tc_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_attn_tc_error, &zero, sizeof(int));
    return v;
}
