// Attention over the paged cache for prompt portions on the fifth-generation tensor cores
// (bfloat16, head size 64 or 128, pages of a multiple of 64 keys, up to 128 query heads per kv head).
//
// A block owns two tiles of 128 rows of the score matrix: (token, query head of one kv group)
// pairs of consecutive tokens of one request, row = token * group + head; the second tile holds
// the tokens after the first's.  Both walk the same visible keys in tiles of 64 (one TMA box, never
// across a page), so a key or value tile is fetched once for 256 rows.  Roles:
//   warp 0     one lane loads the rows of q of both tiles once (three-dimensional TMA boxes: 64
//              elements x the group's heads x the tokens, which land row by row in the
//              128-byte-swizzled K-major layout) and then the K and V tiles into two rings of
//              four stages each;
//   warps 1-2  warp 1 allocates tensor memory (per row tile two score tiles of 64 columns and
//              the output tile of head-size columns); one lane of each issues, for its row
//              tile,  S = Q K^T  (128 x 64 x head size) and  O += P V  (128 x head size x 64; P
//              is read from tensor memory, V is used as it lies in the cache, as an MN-major
//              operand), two score tiles ahead of the softmax;
//   warps 3-10 four warps per row tile, one thread per row: read a score tile with tcgen05.ld,
//              scale and mask it, keep the running maximum and sum in float32, write P as
//              bfloat16 pairs over the first 32 columns of the score tile it came from
//              (tcgen05.st), and at the end divide the output by the sum.
// P never passes through shared memory: the tensor cores' operand reads from shared memory
// (q and the K tile for the scores, the V tile for the output) are what bounds the kernel, and P
// through shared memory would add a third to them.  A score tile's columns are written again
// (scores of the tile after next) only after the product that read P from them has completed.
// While one row tile's threads compute a softmax, the tensor cores work on the other tile's
// products.  (A kernel that allocates tensor memory gets one block per multiprocessor, so the
// overlap has to come from within the block.)  Blocks are persistent, one per multiprocessor:
// the work items (pair of row tiles, kv head) are dealt out round by round in alternating
// direction, heaviest first, and between items the block renews its barriers.
// The output accumulates in tensor memory.  A row's reference maximum moves only when the
// tile's maximum exceeds it by more than 8 (in log2 units): then the row's part of O and its
// sum are multiplied by 2^(old - new) before the next product is added.  P stays below 2^8, and
// the result is the same softmax(S) V up to rounding, since sum and output share the reference.
// A masked key has probability exactly 0, but 0 x (a value that is not a number) is not 0: the
// cache must hold finite values everywhere (it starts zeroed and only finite rows are appended).
//
// Score, mask and softmax: crates/spite-compute/src/flash_attn.rs:111-156; window rules in
// attention.cuh.  Every wait is bounded (see tcgen05.cuh); spite_attention_tc_error() returns
// and clears the code of a wait that gave up: 1 loader, 2 tensor-core issue, 3 softmax.
#include "attention.cuh"
#include "tcgen05.cuh"

namespace {
using namespace tc;

constexpr int BM = 128;                 // rows of one row tile
constexpr int BN = 64;                  // keys per tile (the softmax reads a score tile with one 64-column load)
constexpr int ST = 4;                   // stages of the K ring and of the V ring
constexpr int THREADS = 11 * 32;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_COLS = 256;         // tensor-memory columns of one row tile: S0, S1 (64 each), O
constexpr float RESCALE_STEP = 8.f;     // log2 units
constexpr float LOG2E = 1.4426950408889634f;

__device__ int g_attn_tc_error = 0;
}  // namespace
// 1: the loader waited for a free stage, 2: the tensor-core issuer waited, 3: a softmax warp waited.
// (`extra_tx` is not used here.)
SPITE_WAIT_CONTROLS(attention_tc, g_attn_tc_error)
namespace {

struct GroupBarriers {
    unsigned long long s_full[2], p_ready, pv_done, exp_done;
};
struct Barriers {
    unsigned long long q_full, k_full[ST], k_empty[ST], v_full[ST], v_empty[ST];
    GroupBarriers g[2];
    unsigned tmem_base;
    int abort_flag;
};

// 2^x by the special-function unit (relative error about 2^-22; 2^-inf = 0)
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *(unsigned*)&v;
}

// NKB = head_dim / 64.  grid (blocks over (request, pair of token tiles), kv heads).
template <int NKB>
__global__ void __launch_bounds__(THREADS, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, const AttentionParams p, const StepTokens b,
               const PagedCache c, const AttnMmaExtra x, const int q_box_tokens, const int n_tile_pairs,
               const WaitControl waits) {
    constexpr int HD = 64 * NKB;
    constexpr int Q_BYTES = NKB * BM * 128;              // q of one row tile
    constexpr int KT_BYTES = NKB * BN * 128;             // one K tile, one V tile
    extern __shared__ __align__(1024) unsigned char smem[];   // [Q0][Q1][K ring][V ring], each 1024-byte aligned
    __shared__ Barriers bars;
    pdl_wait();
    pdl_launch_dependents();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nq = p.num_heads, nkv = c.num_kv_heads, G = nq / nkv;
    const int tpt = x.tokens_per_block;                   // tokens of one row tile

    unsigned char* q_s = smem;
    unsigned char* k_s = q_s + 2 * Q_BYTES;
    unsigned char* v_s = k_s + ST * KT_BYTES;
    volatile int* abort_flag = &bars.abort_flag;
    int* const err_word = waits.error_word ? waits.error_word : &g_attn_tc_error;
    const long long wait_limit = waits.limit_cycles;

    auto init_barriers = [&](bool renew) {
        auto one = [&](unsigned long long* bar, unsigned count) {
            if (renew) mbar_inval(smem_u32(bar));
            mbar_init(smem_u32(bar), count);
        };
        one(&bars.q_full, 1);
        for (int s = 0; s < ST; ++s) {
            one(&bars.k_full[s], 1); one(&bars.k_empty[s], 2);     // both row tiles release a stage
            one(&bars.v_full[s], 1); one(&bars.v_empty[s], 2);
        }
        for (int g = 0; g < 2; ++g) {
            for (int s = 0; s < 2; ++s) one(&bars.g[g].s_full[s], 1);
            one(&bars.g[g].p_ready, 4);                            // one arrival per softmax warp
            one(&bars.g[g].pv_done, 1);
            one(&bars.g[g].exp_done, 4);
        }
        mbar_init_fence();
    };
    if (threadIdx.x == 0) {
        bars.abort_flag = 0;
        init_barriers(false);
    }
    if (warp == 1) tmem_alloc(&bars.tmem_base, TMEM_COLS);
    if (warp >= 3) {
        // rows of a q tile that the TMA box does not write: zero, so that their scores are plain numbers
        const int g = (warp - 3) >> 2, r = (warp & 3) * 32 + lane;
        if (r >= q_box_tokens * G) {
#pragma unroll
            for (int kb = 0; kb < NKB; ++kb)
#pragma unroll
                for (int ch = 0; ch < 8; ++ch)
                    *(uint4*)(q_s + g * Q_BYTES + kb * BM * 128 + r * 128 + ch * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();
    }
    fence_before();
    __syncthreads();
    fence_after();
    const unsigned tmem = bars.tmem_base;

    // Work items: (pair of row tiles of a request, kv head), numbered so that the work falls with the
    // number (later tokens see more keys).  Blocks are persistent; round r deals items r * blocks ..
    // (r + 1) * blocks - 1 to the blocks, in alternating direction, so that the shares come out alike.
    const int n_items = n_tile_pairs * nkv;
    for (int round = 0;; ++round) {
        const int item = round * gridDim.x + ((round & 1) ? gridDim.x - 1 - blockIdx.x : blockIdx.x);
        if (item >= n_items) break;
        const int kvh = item % nkv;
        int idx = n_tile_pairs - 1 - item / nkv, seg = -1, t0 = 0, nt = 0;
        for (int s = 0; s < x.n_segments; ++s) {
            const int lo = x.cu_seqlens[s], n = x.cu_seqlens[s + 1] - lo;
            if (n < x.seg_min_tokens || n > x.seg_max_tokens) continue;   // another kernel serves this segment
            const int blocks = (n + 2 * tpt - 1) / (2 * tpt);
            if (idx < blocks) { seg = s; t0 = lo + idx * 2 * tpt; nt = min(2 * tpt, lo + n - t0); break; }
            idx -= blocks;
        }
        if (seg < 0) break;                                   // the caller counted more tile pairs than there are
        const int* table = b.block_table + (size_t)seg * b.table_width;
        // key tiles of the item: from the first key the first token sees to the last token's own
        const int k_begin = (window_lowest(p.window_kind, p.window_size, b.positions[t0]) / BN) * BN;
        const int n_tiles = (b.positions[t0 + nt - 1] - k_begin) / BN + 1;

        if (warp == 0) {
            if (lane == 0) {
                // ---- loader
                const unsigned q_bar = smem_u32(&bars.q_full);
                mbar_expect_tx(q_bar, (unsigned)(2 * NKB * q_box_tokens * G * 128));
#pragma unroll
                for (int g = 0; g < 2; ++g)
#pragma unroll
                    for (int kb = 0; kb < NKB; ++kb)
                        tma_load_3d(smem_u32(q_s + g * Q_BYTES + kb * BM * 128), &map_q, kb * 64, kvh * G, t0 + g * tpt, q_bar);
                int issued_k = 0, issued_v = 0;
                for (int i = 0; i < n_tiles; ++i) {
                    const int s = i % ST;
                    const unsigned ph = (i / ST) & 1;
                    const int j0 = k_begin + i * BN;
                    int page = table[j0 / c.page_size];
                    if (page < 0 || page >= c.n_pages) page = 0;   // a page behind every row's window: its keys are masked
                    const int y = (page * nkv + kvh) * c.page_size + j0 % c.page_size;
                    if (!mbar_wait(smem_u32(&bars.k_empty[s]), ph ^ 1, abort_flag, err_word, 1, wait_limit)) break;
                    mbar_expect_tx(smem_u32(&bars.k_full[s]), KT_BYTES);
#pragma unroll
                    for (int kb = 0; kb < NKB; ++kb)
                        tma_load_2d(smem_u32(k_s + s * KT_BYTES + kb * BN * 128), &map_k, kb * 64, y, smem_u32(&bars.k_full[s]));
                    ++issued_k;
                    if (!mbar_wait(smem_u32(&bars.v_empty[s]), ph ^ 1, abort_flag, err_word, 1, wait_limit)) break;
                    mbar_expect_tx(smem_u32(&bars.v_full[s]), KT_BYTES);
#pragma unroll
                    for (int kb = 0; kb < NKB; ++kb)
                        tma_load_2d(smem_u32(v_s + s * KT_BYTES + kb * BN * 128), &map_v, kb * 64, y, smem_u32(&bars.v_full[s]));
                    ++issued_v;
                }
                // the last releases of the stages must have arrived before the barriers are renewed for the next item
                for (int j = max(0, n_tiles - ST); j < n_tiles && !*abort_flag; ++j) {
                    if (!mbar_wait(smem_u32(&bars.k_empty[j % ST]), (j / ST) & 1, abort_flag, err_word, 1, wait_limit)) break;
                    if (!mbar_wait(smem_u32(&bars.v_empty[j % ST]), (j / ST) & 1, abort_flag, err_word, 1, wait_limit)) break;
                }
                if (*abort_flag) {
                    // copies in flight must land before the block gives its shared memory back
                    mbar_drain(q_bar, 0, wait_limit);
                    for (int j = max(0, issued_k - ST); j < issued_k; ++j) mbar_drain(smem_u32(&bars.k_full[j % ST]), (j / ST) & 1, wait_limit);
                    for (int j = max(0, issued_v - ST); j < issued_v; ++j) mbar_drain(smem_u32(&bars.v_full[j % ST]), (j / ST) & 1, wait_limit);
                }
            }
        } else {
            // ---- one of the two row tiles
            const int g = warp < 3 ? warp - 1 : (warp - 3) >> 2;
            GroupBarriers& gb = bars.g[g];
            const int tg0 = t0 + g * tpt;
            const int ntg = max(0, min(tpt, nt - g * tpt));
            // this row tile's own key tiles, [first, last] among the block's; the second tile of a block may hold no token
            int first = 0, last = -1, p_first = 0, lo_last = 0;
            if (ntg > 0) {
                p_first = b.positions[tg0];
                const int p_last = b.positions[tg0 + ntg - 1];
                lo_last = window_lowest(p.window_kind, p.window_size, p_last);
                first = (window_lowest(p.window_kind, p.window_size, p_first) / BN * BN - k_begin) / BN;
                last = (p_last - k_begin) / BN;
            }
            const int n_own = last - first + 1;
            // the key tiles that both row tiles own, [shared_lo, shared_hi] among the block's: there the two take
            // turns at the exponentials
            int shared_lo = 0, shared_hi = -1;
            {
                const int og = g ^ 1, otg0 = t0 + og * tpt, ontg = max(0, min(tpt, nt - og * tpt));
                if (ontg > 0 && ntg > 0) {
                    const int op_first = b.positions[otg0], op_last = b.positions[otg0 + ontg - 1];
                    shared_lo = max(first, (window_lowest(p.window_kind, p.window_size, op_first) / BN * BN - k_begin) / BN);
                    shared_hi = min(last, (op_last - k_begin) / BN);
                }
            }
            const unsigned tmem_g = tmem + g * GROUP_COLS;
            unsigned char* q_g = q_s + g * Q_BYTES;

            if (warp < 3) {
                if (lane == 0) {
                    // ---- tensor-core issue for this row tile
                    const unsigned idesc_s = make_idesc(BM, BN), idesc_pv = make_idesc(BM, HD, true);
                    bool ok = mbar_wait(smem_u32(&bars.q_full), 0, abort_flag, err_word, 2, wait_limit);
                    // a key tile that this row tile does not need: wait until it has landed (so that the two
                    // row tiles never drift apart by more than the ring) and hand the stage back unread
                    auto pass_tile = [&](int i) {
                        const int s = i % ST;
                        const unsigned ph = (i / ST) & 1;
                        if (!mbar_wait(smem_u32(&bars.k_full[s]), ph, abort_flag, err_word, 2, wait_limit)) return false;
                        mbar_arrive(smem_u32(&bars.k_empty[s]));
                        if (!mbar_wait(smem_u32(&bars.v_full[s]), ph, abort_flag, err_word, 2, wait_limit)) return false;
                        mbar_arrive(smem_u32(&bars.v_empty[s]));
                        return true;
                    };
                    // scores of own tile li (key tile first + li) into score buffer li & 1, whose columns held
                    // P of tile li - 2: the product that read it must have completed
                    auto issue_scores = [&](int li) {
                        const int i = first + li, s = i % ST, sb = li & 1;
                        if (!mbar_wait(smem_u32(&bars.k_full[s]), (i / ST) & 1, abort_flag, err_word, 2, wait_limit)) return false;
                        if (li >= 2 && !mbar_wait(smem_u32(&gb.pv_done), li & 1, abort_flag, err_word, 2, wait_limit)) return false;
                        fence_after();
                        const unsigned qa = smem_u32(q_g), ka = smem_u32(k_s + s * KT_BYTES);
#pragma unroll
                        for (int ks = 0; ks < HD / 16; ++ks)
                            mma(tmem_g + sb * BN, smem_desc_k_major(qa + (ks / 4) * BM * 128 + (ks % 4) * 32),
                                smem_desc_k_major(ka + (ks / 4) * BN * 128 + (ks % 4) * 32), idesc_s, ks > 0 ? 1u : 0u);
                        commit(smem_u32(&gb.s_full[sb]));
                        commit(smem_u32(&bars.k_empty[s]));
                        return true;
                    };
                    for (int i = 0; i < first && ok; ++i) ok = pass_tile(i);
                    if (ok && n_own > 0) ok = issue_scores(0);
                    if (ok && n_own > 1) ok = issue_scores(1);
                    for (int li = 0; li < n_own && ok; ++li) {
                        const int i = first + li, s = i % ST;
                        ok = mbar_wait(smem_u32(&gb.p_ready), li & 1, abort_flag, err_word, 2, wait_limit) &&
                             mbar_wait(smem_u32(&bars.v_full[s]), (i / ST) & 1, abort_flag, err_word, 2, wait_limit);
                        if (!ok) break;
                        fence_after();
                        const unsigned va = smem_u32(v_s + s * KT_BYTES);
#pragma unroll
                        for (int ks = 0; ks < BN / 16; ++ks)
                            mma_a_tmem(tmem_g + 2 * BN, tmem_g + (li & 1) * BN + ks * 8, smem_desc(va + ks * 16 * 128, BN * 128, 1024),
                                       idesc_pv, (li > 0 || ks > 0) ? 1u : 0u);
                        commit(smem_u32(&gb.pv_done));
                        commit(smem_u32(&bars.v_empty[s]));
                        if (li + 2 < n_own) ok = issue_scores(li + 2);
                    }
                    for (int i = last + 1; i < n_tiles && ok; ++i) ok = pass_tile(i);
                }
            } else {
                // ---- softmax: one thread per row; warp w may read tensor-memory lanes [32 (w % 4), + 32)
                const int quarter = warp & 3;
                const int r = quarter * 32 + lane;
                const bool row_ok = r < ntg * G;
                const int tok = tg0 + (row_ok ? r / G : 0), head = kvh * G + (row_ok ? r % G : 0);
                const int pos = row_ok ? b.positions[tok] : -1;   // a row without a token sees no key
                const int lo = window_lowest(p.window_kind, p.window_size, max(pos, 0));
                const float scale = p.softmax_scale * LOG2E;
                const unsigned lane_base = tmem_g + ((unsigned)(quarter * 32) << 16);
                float m_ref = -INFINITY, l = 0.f;
                bool ok = true;
                for (int li = 0; li < n_own; ++li) {
                    const int sb = li & 1;
                    ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&gb.s_full[sb]), (li >> 1) & 1, abort_flag, err_word, 3, wait_limit));
                    if (!ok) break;
                    fence_after();
                    float s[BN];
                    ld64(s, lane_base + sb * BN);
                    const int j0 = k_begin + (first + li) * BN;
                    const bool open = j0 >= lo_last && j0 + BN - 1 <= p_first;   // every key visible to every row with a token
                    // maximum of the raw scores (the scale is positive); four running values shorten the chain
                    float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                    if (!open) {                                   // a tile on a window's edge or on the diagonal
#pragma unroll
                        for (int e = 0; e < BN; ++e) {
                            const int j = j0 + e;
                            s[e] = (j >= lo && j <= pos) ? s[e] : -INFINITY;
                        }
                    }
#pragma unroll
                    for (int e = 0; e < BN; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], s[e]);
                    const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale;
                    const bool need = mx > m_ref + RESCALE_STEP;
                    float corr = 1.f;
                    if (need) { corr = exp2f(m_ref - mx); l *= corr; m_ref = mx; }
                    const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
                    // Over the key tiles that both own, the two row tiles take turns at the exponentials (key tile i
                    // of the first row tile, key tile i of the second, key tile i + 1 of the first, ...): the
                    // special-function units serve one at full rate while the tensor cores work for the other,
                    // instead of both halves of the block computing and then both waiting.  Both count their
                    // turns from the first shared key tile, so each is at most one phase behind the other's barrier.
                    const int turn = first + li - shared_lo;
                    const bool takes_turns = turn >= 0 && first + li <= shared_hi;
                    if (takes_turns && (g == 1 || turn > 0)) {
                        const int before = g == 0 ? turn - 1 : turn;      // the other row tile's turn before this one
                        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.g[g ^ 1].exp_done), before & 1, abort_flag, err_word, 3, wait_limit));
                        if (!ok) break;
                    }
                    unsigned packed[BN / 2];
                    float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int e = 0; e < BN; e += 2) {
                        const float a = ex2(fmaf(s[e], scale, neg_m)), bb = ex2(fmaf(s[e + 1], scale, neg_m));
                        sum4[(e >> 1) & 3] += a + bb;
                        packed[e / 2] = pack_bf16(a, bb);
                    }
                    __syncwarp();
                    if (takes_turns && lane == 0) mbar_arrive(smem_u32(&gb.exp_done));
                    const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
                    l += sum;
                    if (li > 0) {
                        // The product of the tile before must have left O before its rows are rescaled.  The wait is
                        // made for every tile, needed or not: a wait by parity is only right while the waiter is
                        // at most one phase behind the barrier.
                        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&gb.pv_done), (li - 1) & 1, abort_flag, err_word, 3, wait_limit));
                        if (!ok) break;
                        if (__any_sync(0xffffffffu, need)) {
                            fence_after();
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
                    st32(lane_base + sb * BN, packed);              // P over the first half of the score tile just read
                    fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&gb.p_ready));
                }
                if (ok && n_own > 0)
                    ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&gb.pv_done), (n_own - 1) & 1, abort_flag, err_word, 3, wait_limit));
                if (ok && n_own > 0) {
                    fence_after();
                    const float inv = 1.0f / fmaxf(l, 1e-30f);
                    __nv_bfloat16* dst = (__nv_bfloat16*)p.out + ((size_t)tok * nq + head) * HD;
#pragma unroll 1
                    for (int c0 = 0; c0 < HD; c0 += 32) {
                        float o[32];
                        ld32(o, lane_base + 2 * BN + c0);          // warp-collective: every lane takes part
                        if (!row_ok) continue;
#pragma unroll
                        for (int e = 0; e < 32; e += 8)
                            *(uint4*)(dst + c0 + e) = make_uint4(pack_bf16(o[e] * inv, o[e + 1] * inv), pack_bf16(o[e + 2] * inv, o[e + 3] * inv),
                                                                 pack_bf16(o[e + 4] * inv, o[e + 5] * inv), pack_bf16(o[e + 6] * inv, o[e + 7] * inv));
                    }
                }
            }
        }
        // end of the item: everything asynchronous has been waited for; renew the barriers
        fence_before();
        __syncthreads();
        fence_after();
        if (*abort_flag) break;
        if (threadIdx.x == 0) init_barriers(true);
        __syncthreads();
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
           int n_sm, cudaStream_t st) {
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
    const size_t smem = 2 * (size_t)NKB * BM * 128 + 2 * ST * (size_t)NKB * BN * 128;
    auto k = attn_tc_kernel<NKB>;
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return SPITE_LAUNCH_FAILED;
    const long long items = (long long)n_blocks * nkv;
    const int grid = (int)(items < n_sm ? items : n_sm);
    SPITE_LAUNCH(k, grid, THREADS, smem, st, mq, mk, mv, p, b, c, x, box_tokens, n_blocks, s_waits);
    return spite_launch_status();
}

}  // namespace

// `tokens_per_block`: tokens of one row tile, tokens_per_block * (query heads per kv head) <= 128; a block
// serves two row tiles.  `n_blocks` = sum over the served segments of ceil(tokens / (2 tokens_per_block)),
// computed by the caller; `n_sm`: number of multiprocessors (one persistent block each).
SPITE_API int spite_paged_attention_tc(const AttentionParams* p, const StepTokens* b, const PagedCache* c,
                                       const AttnMmaExtra* x, int n_blocks, int n_sm, void* stream) {
    if (n_sm < 1) return SPITE_BAD_ARG;
    if (!p || !b || !c || !x || !p->q || !p->out || !x->cu_seqlens || !c->kv) return SPITE_BAD_ARG;
    if (!b->positions || !b->block_table || b->n_tokens < 0 || b->table_width < 1) return SPITE_BAD_ARG;
    if (p->num_heads < 1 || c->num_kv_heads < 1 || p->num_heads % c->num_kv_heads) return SPITE_BAD_ARG;
    if (p->window_kind < 0 || p->window_kind > 2) return SPITE_BAD_ARG;
    if (p->window_kind != SPITE_WINDOW_FULL && p->window_size < 1) return SPITE_BAD_ARG;
    if (x->n_segments < 1 || x->tokens_per_block < 1 || n_blocks < 0 || c->n_pages < 1 || c->page_size < 1) return SPITE_BAD_ARG;
    const int G = p->num_heads / c->num_kv_heads;
    if ((c->head_dim != 64 && c->head_dim != 128) || G > BM || c->page_size % BN) return SPITE_UNSUPPORTED;
    if (x->tokens_per_block * G > BM) return SPITE_BAD_ARG;
    if ((long long)n_blocks * c->num_kv_heads > 0x7fffffffll || p->num_heads > 256 * c->num_kv_heads) return SPITE_UNSUPPORTED;
    if ((long long)c->n_pages * c->num_kv_heads * c->page_size > 0x7fffffffll) return SPITE_UNSUPPORTED;   // TMA coordinates are int32
    if ((((uintptr_t)p->q | (uintptr_t)p->out | (uintptr_t)c->kv) & 15) || (c->v_offset & 7)) return SPITE_UNSUPPORTED;
    if (b->n_tokens == 0 || n_blocks == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    return c->head_dim == 64 ? launch<1>(*p, *b, *c, *x, n_blocks, n_sm, st) : launch<2>(*p, *b, *c, *x, n_blocks, n_sm, st);
}
