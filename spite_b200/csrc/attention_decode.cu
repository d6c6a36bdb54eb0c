// Attention of decoded tokens over the paged cache (bfloat16, head sizes 64 and 128, pages of a
// multiple of 64 keys, up to 16 query heads per kv head): few query rows, a long context, so the
// kernel is a stream of keys and values through shared memory and nothing else matters.
//
// A block serves the (token, query head of one kv group) rows of up to `tokens_per_block` tokens of
// one request, for one kv head and one split of the keys.  One producer thread brings tiles of 64
// keys and 64 values, which are whole boxes of one page (a page holds one kv head's rows contiguously),
// into a ring of shared-memory stages with TMA (cp.async.bulk.tensor, 128-byte swizzle, no cluster
// multicast) and marks them to leave L2 first; four consumer warps take 16 keys of every tile each
// (ldmatrix + mma.sync m16n8k16, float32 running maximum and sum per warp) and merge their states in
// shared memory at the end.  With several splits a block leaves its unnormalised partial result in a
// scratch buffer and takes a ticket; the block that takes a (request block, kv head)'s last ticket
// merges the splits in split order, so no second kernel runs and the order of the additions does
// not depend on which block came last.
//
// Every wait on a barrier is bounded (tcgen05.cuh): a wait that runs out records a code, raises the
// block's abort flag, and the block leaves without writing its result.
//
// Score, mask and softmax: crates/spite-compute/src/flash_attn.rs:111-156; the local window rule
// is the architecture's (same chunk), see attention.cuh.
#include "attention.cuh"
#include "tcgen05.cuh"

namespace {
using namespace tc;

constexpr int CONSUMERS = 4;
constexpr int THREADS = (CONSUMERS + 1) * 32;
constexpr int BN = 64;                                    // keys of a tile
constexpr int MERGE_BATCH = 24;                           // partial results a thread asks for together when splits are merged
constexpr int BOX_BYTES = BN * 128;                       // 64 rows of 64 elements
constexpr int MAX_STAGES = 8;

__device__ int g_attn_decode_error = 0;
}  // namespace
// 1: the producer waited for a free stage, 2: a consumer waited for a tile.  (`extra_tx` is not used here.)
SPITE_WAIT_CONTROLS(attention_decode, g_attn_decode_error)
namespace {

struct Tail {
    unsigned long long full[MAX_STAGES], empty[MAX_STAGES];
    int abort_flag, last;
};

__device__ __forceinline__ void mma16816(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ unsigned pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *(unsigned*)&v;
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(CONSUMERS * 32) : "memory"); }

// Element (row r, 16-byte chunk ch of the head) of a tile of 64 rows: the head's elements come in boxes
// of 64 (128 bytes a row), inside a box TMA has xor-ed the chunk index with the row's low bits.
__device__ __forceinline__ unsigned tile_addr(unsigned base, int r, int ch) {
    return base + (ch >> 3) * BOX_BYTES + r * 128 + (((ch & 7) ^ (r & 7)) << 4);
}

// NKB = head_dim / 64.  grid (blocks over the served segments, kv heads, splits).
template <int NKB>
__global__ void __launch_bounds__(THREADS) attn_decode_kernel(const __grid_constant__ CUtensorMap map_k,
                                                              const __grid_constant__ CUtensorMap map_v,
                                                              const AttentionParams p, const StepTokens b,
                                                              const PagedCache c, const AttnDecodeExtra x,
                                                              const int n_stages, const int ring_bytes,
                                                              const WaitControl waits) {
    constexpr int HD = 64 * NKB, NK = 4 * NKB;            // NK: 16-element steps of the head
    constexpr int STAGE = 2 * NKB * BOX_BYTES;            // keys, then values
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    Tail* tail = (Tail*)(smem + ring_bytes);               // the ring of stages, later the merge buffers, lie before it
    volatile int* abort_flag = &tail->abort_flag;
    int* const err_word = waits.error_word ? waits.error_word : &g_attn_decode_error;
    const long long wait_limit = waits.limit_cycles;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < n_stages; ++s) { mbar_init(smem_u32(&tail->full[s]), 1); mbar_init(smem_u32(&tail->empty[s]), CONSUMERS); }
        tail->abort_flag = 0;
        tail->last = 0;
        mbar_init_fence();
    }
    if (warp == CONSUMERS && lane == 0) {                    // the tensor maps are needed first thing after the wait
        asm volatile("prefetch.tensormap [%0];\n" ::"l"((unsigned long long)&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"((unsigned long long)&map_v) : "memory");
    }
    __syncthreads();

    // What follows up to the wait reads only what no kernel of this step writes: the step's positions and
    // block tables (copied to the device before the step's first kernel) and, if the caller says that the
    // cache rows of earlier steps are settled, the tiles that lie wholly before the request's first token
    // of this step.  Their loads are under way while the kernel before (which writes q and this step's
    // keys) still runs.
    const int nq = p.num_heads, nkv = c.num_kv_heads, G = nq / nkv;
    // which request and which of its tokens
    int idx = blockIdx.x, seg = -1, t0 = 0, nt = 0, seg_lo = 0;
    for (int s = 0; s < x.n_segments; ++s) {
        const int lo = x.cu_seqlens[s], n = x.cu_seqlens[s + 1] - lo;
        if (n < x.seg_min_tokens || n > x.seg_max_tokens) continue;   // another kernel serves this segment
        const int blocks = (n + x.tokens_per_block - 1) / x.tokens_per_block;
        if (idx < blocks) { seg = s; seg_lo = lo; t0 = lo + idx * x.tokens_per_block; nt = min(x.tokens_per_block, lo + n - t0); break; }
        idx -= blocks;
    }
    if (seg < 0) { pdl_wait(); pdl_launch_dependents(); return; }   // (every thread of the block: no barrier is left waiting)
    const int kvh = blockIdx.y, split = blockIdx.z;
    const int n_rows = nt * G;
    const int* table = b.block_table + (size_t)seg * b.table_width;

    // tiles of 64 keys this block walks: its share of [lowest visible key of the first token, last token]
    const int p_first = b.positions[t0], p_last = b.positions[t0 + nt - 1];
    const int lo_first = window_lowest(p.window_kind, p.window_size, p_first);
    const int tile_lo = lo_first / BN;
    const int n_tiles = p_last / BN + 1 - tile_lo;
    const int sb = tile_lo + (int)((long long)n_tiles * split / x.n_splits);
    const int se = tile_lo + (int)((long long)n_tiles * (split + 1) / x.n_splits);

    auto issue_tile = [&](int ti, int s, unsigned long long policy) {
        const int j0 = ti * BN;
        const int page = max(table[j0 / c.page_size], 0);     // a tile with a visible key lies in a held page
        const int row = (page * nkv + kvh) * c.page_size + j0 % c.page_size;
        const unsigned bar = smem_u32(&tail->full[s]), dst = smem_u32(smem + (size_t)s * STAGE);
        mbar_expect_tx(bar, STAGE);
#pragma unroll
        for (int kb = 0; kb < NKB; ++kb) {
            tma_load_2d_hint(dst + kb * BOX_BYTES, &map_k, kb * 64, row, bar, policy);
            tma_load_2d_hint(dst + (NKB + kb) * BOX_BYTES, &map_v, kb * 64, row, bar, policy);
        }
    };
    int early = 0;                                            // tiles requested before the wait (producer thread only)
    if (x.cache_settled && warp == CONSUMERS && lane == 0) {
        const int settled_end = b.positions[seg_lo] / BN;     // tiles [.., settled_end) hold rows of earlier steps only
        const unsigned long long policy = l2_evict_first();
        while (early < n_stages && sb + early < se && sb + early < settled_end) { issue_tile(sb + early, early, policy); ++early; }
    }
    pdl_wait();
    pdl_launch_dependents();

    float o[2 * NK][4];
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    bool ok = true;

    if (warp == CONSUMERS) {
        // ---- producer
        if (lane == 0) {
            const unsigned long long policy = l2_evict_first();       // the cache is read once a step
            int s = 0, issued = 0;
            unsigned ph = 0;
            for (int ti = sb; ti < se; ++ti, ++issued, s = (s + 1 == n_stages ? 0 : s + 1), ph ^= (s == 0)) {
                if (issued < early) continue;                         // requested before the wait
                if (!mbar_wait(smem_u32(&tail->empty[s]), ph ^ 1, abort_flag, err_word, 1, wait_limit)) break;
                issue_tile(ti, s, policy);
            }
            if (*abort_flag) {
                // copies in flight must land before the block gives its shared memory back
                for (int j = max(0, issued - n_stages); j < issued; ++j)
                    mbar_drain(smem_u32(&tail->full[j % n_stages]), (j / n_stages) & 1, wait_limit);
            }
        }
    } else {
        // ---- consumers: warp w takes keys 16 w .. 16 w + 15 of every tile
        const int g = lane >> 2, cc = lane & 3;
        int row_pos[2], row_lo[2];
        bool row_ok[2];
        unsigned qa[NK][4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = g + 8 * h;
            row_ok[h] = r < n_rows;
            const int tok = t0 + (row_ok[h] ? r / G : 0);
            const int head = kvh * G + (row_ok[h] ? r % G : 0);
            row_pos[h] = b.positions[tok];
            row_lo[h] = window_lowest(p.window_kind, p.window_size, row_pos[h]);
            const __nv_bfloat16* qrow = (const __nv_bfloat16*)p.q + ((size_t)tok * nq + head) * HD;
#pragma unroll
            for (int kk = 0; kk < NK; ++kk) {
                const unsigned* src = (const unsigned*)(qrow + 16 * kk + 2 * cc);
                qa[kk][h] = row_ok[h] ? src[0] : 0u;            // k = 2c, 2c+1
                qa[kk][2 + h] = row_ok[h] ? src[4] : 0u;        // k = 2c+8, 2c+9
            }
        }
#pragma unroll
        for (int n = 0; n < 2 * NK; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[n][e] = 0.f;

        int s = 0;
        unsigned ph = 0;
        for (int ti = sb; ti < se; ++ti, s = (s + 1 == n_stages ? 0 : s + 1), ph ^= (s == 0)) {
            ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&tail->full[s]), ph, abort_flag, err_word, 2, wait_limit));
            if (!ok) break;
            const unsigned kbase = smem_u32(smem + (size_t)s * STAGE), vbase = kbase + NKB * BOX_BYTES;
            const int j0 = ti * BN + 16 * warp;                  // this warp's first key
            // a warp whose 16 keys no row may see skips them (the first and the last tile of a window)
            if (j0 + 15 >= lo_first && j0 <= p_last) {
                // scores of 16 rows x 16 keys
                float sc[2][4];
#pragma unroll
                for (int n = 0; n < 2; ++n) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) sc[n][e] = 0.f;
                    const int r = 16 * warp + n * 8 + (lane & 7);
#pragma unroll
                    for (int kk = 0; kk < NK; kk += 2) {
                        unsigned kb[4];
                        ldmatrix_x4(kb, tile_addr(kbase, r, 2 * kk + (lane >> 3)));
                        mma16816(sc[n], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], kb[0], kb[1]);
                        mma16816(sc[n], qa[kk + 1][0], qa[kk + 1][1], qa[kk + 1][2], qa[kk + 1][3], kb[2], kb[3]);
                    }
                }
                // mask, running maximum and sum (float32)
                float corr[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float mx = -INFINITY;
#pragma unroll
                    for (int n = 0; n < 2; ++n)
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int j = j0 + 8 * n + 2 * cc + e;
                            const bool vis = row_ok[h] && j >= row_lo[h] && j <= row_pos[h];
                            const float v = vis ? sc[n][2 * h + e] * p.softmax_scale : -INFINITY;
                            sc[n][2 * h + e] = v;
                            mx = fmaxf(mx, v);
                        }
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                    const float m_new = fmaxf(m_run[h], mx);
                    corr[h] = (m_new == -INFINITY) ? 1.f : expf(m_run[h] - m_new);
                    float sum = 0.f;
#pragma unroll
                    for (int n = 0; n < 2; ++n)
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const float pv = (m_new == -INFINITY) ? 0.f : expf(sc[n][2 * h + e] - m_new);
                            sc[n][2 * h + e] = pv;
                            sum += pv;
                        }
                    l_run[h] = l_run[h] * corr[h] + sum;
                    m_run[h] = m_new;
                }
#pragma unroll
                for (int n = 0; n < 2 * NK; ++n) {
                    o[n][0] *= corr[0]; o[n][1] *= corr[0];
                    o[n][2] *= corr[1]; o[n][3] *= corr[1];
                }
                // values: O += P V
                const unsigned pa0 = pack_bf16(sc[0][0], sc[0][1]), pa1 = pack_bf16(sc[0][2], sc[0][3]);
                const unsigned pa2 = pack_bf16(sc[1][0], sc[1][1]), pa3 = pack_bf16(sc[1][2], sc[1][3]);
#pragma unroll
                for (int jj = 0; jj < NK; ++jj) {
                    unsigned vb[4];
                    const int r = 16 * warp + (lane & 7) + 8 * ((lane >> 3) & 1);
                    ldmatrix_x4_trans(vb, tile_addr(vbase, r, 2 * jj + (lane >> 4)));
                    mma16816(o[2 * jj], pa0, pa1, pa2, pa3, vb[0], vb[1]);
                    mma16816(o[2 * jj + 1], pa0, pa1, pa2, pa3, vb[2], vb[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tail->empty[s]));
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
        }
    }
    __syncthreads();                                         // every tile has been read (or the block has given up)
    if (*abort_flag) return;
    if (warp == CONSUMERS) return;

    // ---- the four warps' states meet in shared memory (the tiles are dead: reuse their memory)
    const int g = lane >> 2, cc = lane & 3;
    float* o_s = (float*)smem;                               // [CONSUMERS][16][HD]
    float* m_s = o_s + CONSUMERS * 16 * HD;                  // [CONSUMERS][16]
    float* l_s = m_s + CONSUMERS * 16;
#pragma unroll
    for (int n = 0; n < 2 * NK; ++n) {
        float* dst = o_s + ((size_t)warp * 16 + g) * HD + 8 * n + 2 * cc;
        dst[0] = o[n][0]; dst[1] = o[n][1];
        dst[8 * HD] = o[n][2]; dst[8 * HD + 1] = o[n][3];
    }
    if (cc == 0) {
        m_s[warp * 16 + g] = m_run[0]; m_s[warp * 16 + g + 8] = m_run[1];
        l_s[warp * 16 + g] = l_run[0]; l_s[warp * 16 + g + 8] = l_run[1];
    }
    consumer_sync();
    // partial results: [block][kv head][split][16 rows][HD + 4]; elements HD and HD + 1 hold maximum and sum
    constexpr int ROW = HD + 4;                              // a multiple of four floats: rows are read 16 bytes at a time
    float* part_all = x.partial + ((size_t)blockIdx.x * nkv + kvh) * x.n_splits * 16 * ROW;
    float* part = part_all + (size_t)split * 16 * ROW;
    for (int e = threadIdx.x; e < n_rows * HD; e += CONSUMERS * 32) {
        const int r = e / HD, d = e % HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < CONSUMERS; ++w) m = fmaxf(m, m_s[w * 16 + r]);
        float l = 0.f, acc = 0.f;
        if (m > -INFINITY) {
#pragma unroll
            for (int w = 0; w < CONSUMERS; ++w) {
                const float f = expf(m_s[w * 16 + r] - m);
                l += l_s[w * 16 + r] * f;
                acc += o_s[((size_t)w * 16 + r) * HD + d] * f;
            }
        }
        if (x.n_splits == 1) {
            const int tok = t0 + r / G, head = kvh * G + r % G;
            ((__nv_bfloat16*)p.out)[((size_t)tok * nq + head) * HD + d] = __float2bfloat16_rn(acc / fmaxf(l, 1e-30f));
        } else {
            __stcg(part + r * ROW + d, acc);
            if (d == 0) { __stcg(part + r * ROW + HD, m); __stcg(part + r * ROW + HD + 1, l); }
        }
    }
    if (x.n_splits == 1) return;

    // ---- The block that brings the last partial result merges them all, in split order.  (Measured and not
    //      kept: merging in two rounds, groups of splits first; a second fence and ticket cost more than the
    //      shorter sums saved: 23.7 against 22.0 us at 37 splits, 22.0 against 17.6 us at 18.)
    consumer_sync();
    if (threadIdx.x == 0) {
        __threadfence();                                     // after the barrier: it covers what the other threads stored
        int* ticket = x.tickets + (size_t)blockIdx.x * nkv + kvh;
        const int arrived = atomicAdd(ticket, 1);
        tail->last = (arrived == x.n_splits - 1);
        if (tail->last) *ticket = 0;                         // as the next launch expects it
    }
    consumer_sync();
    if (!tail->last) return;
    __threadfence();
    // What the merge costs is the latency of its loads from L2 (partial results that other multiprocessors have
    // just written), so they are made few rounds of many.  A thread sums four output elements over the splits, in
    // split order; the partial outputs of its first elements are asked for at once, MERGE_BATCH splits together,
    // then every split's maximum and sum in one round, from which the splits' weights follow while the first
    // loads are still on their way.  (A loop over the splits whose length the compiler does not know would wait
    // for every load before it asks for the next: 6 us for 24 splits.)
    const int count = x.n_splits;
    float* w_s = (float*)smem;                               // [16][count] weights of the splits
    float* l_sp = w_s + 16 * count;                          // [16][count] their sums
    float* inv_s = l_sp + 16 * count;                        // [16] inverse of the merged sums
    const int n_items = n_rows * (HD / 4);
    float4 v[MERGE_BATCH];
    auto ask = [&](int e, int sp0) {
        const int r = e / (HD / 4), d4 = e % (HD / 4);
        const float4* from = (const float4*)(part_all + (size_t)r * ROW) + d4;
#pragma unroll
        for (int j = 0; j < MERGE_BATCH; ++j)
            v[j] = e < n_items && sp0 + j < count ? __ldcg(from + (size_t)(sp0 + j) * (16 * ROW / 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    ask(threadIdx.x, 0);
    for (int i = threadIdx.x; i < n_rows * count; i += CONSUMERS * 32) {
        const int r = i / count, sp = i % count;
        const float2 ml = __ldcg((const float2*)(part_all + ((size_t)sp * 16 + r) * ROW + HD));
        w_s[r * count + sp] = ml.x;
        l_sp[r * count + sp] = ml.y;
    }
    consumer_sync();
    for (int r = warp; r < n_rows; r += CONSUMERS) {
        float m = -INFINITY;
        for (int sp = lane; sp < count; sp += 32) m = fmaxf(m, w_s[r * count + sp]);
        m = warp_max(m);
        float l = 0.f;
        for (int sp0 = 0; sp0 < count; sp0 += 32) {           // sums in split order: lane order within 32, then the next 32
            const int sp = sp0 + lane;
            float ls = 0.f;
            if (sp < count) {
                const float ms = w_s[r * count + sp];
                const float w = ms > -INFINITY ? expf(ms - m) : 0.f;
                ls = l_sp[r * count + sp] * w;
                w_s[r * count + sp] = w;
            }
            l += warp_sum(ls);
        }
        if (lane == 0) inv_s[r] = 1.0f / fmaxf(l, 1e-30f);
    }
    consumer_sync();
    for (int e = threadIdx.x; e < n_items; e += CONSUMERS * 32) {
        const int r = e / (HD / 4), d4 = e % (HD / 4);
        const float* w = w_s + r * count;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sp0 = 0; sp0 < count; sp0 += MERGE_BATCH) {
            if (e != (int)threadIdx.x || sp0 > 0) ask(e, sp0);   // (the first batch of the first item is here already)
#pragma unroll
            for (int j = 0; j < MERGE_BATCH; ++j) {
                const float ws = sp0 + j < count ? w[sp0 + j] : 0.f;
                acc.x = fmaf(v[j].x, ws, acc.x); acc.y = fmaf(v[j].y, ws, acc.y);
                acc.z = fmaf(v[j].z, ws, acc.z); acc.w = fmaf(v[j].w, ws, acc.w);
            }
        }
        const float inv = inv_s[r];
        const int tok = t0 + r / G, head = kvh * G + r % G;
        const unsigned lo = pack_bf16(acc.x * inv, acc.y * inv), hi = pack_bf16(acc.z * inv, acc.w * inv);
        *(uint2*)((__nv_bfloat16*)p.out + ((size_t)tok * nq + head) * HD + 4 * d4) = make_uint2(lo, hi);
    }
}

template <int NKB>
int launch(const AttentionParams& p, const StepTokens& b, const PagedCache& c, const AttnDecodeExtra& x,
           int n_blocks, int n_stages, cudaStream_t st) {
    const int hd = 64 * NKB;
    CUtensorMap mk, mv;
    cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)c.n_pages * c.num_kv_heads * c.page_size};
    cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)BN};
    if (!make_map(&mk, c.kv, 2, dims, strides, box)) return SPITE_LAUNCH_FAILED;
    if (!make_map(&mv, (const __nv_bfloat16*)c.kv + c.v_offset, 2, dims, strides, box)) return SPITE_LAUNCH_FAILED;
    const size_t stage = 2 * (size_t)NKB * BOX_BYTES;
    const size_t merge = (size_t)CONSUMERS * 16 * hd * 4 + CONSUMERS * 16 * 2 * 4;
    const size_t weights = (size_t)(2 * 16 * x.n_splits + 16) * 4;
    size_t ring = (size_t)n_stages * stage;
    if (ring < merge) ring = merge;
    if (ring < weights) ring = weights;
    ring = (ring + 15) & ~(size_t)15;
    const size_t smem = ring + sizeof(Tail) + 1024;
    if (smem > 227 * 1024) return SPITE_UNSUPPORTED;
    auto k = attn_decode_kernel<NKB>;
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
        cudaFuncSetAttribute(k, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess)
        return SPITE_LAUNCH_FAILED;
    dim3 grid(n_blocks, c.num_kv_heads, x.n_splits);
    SPITE_LAUNCH(k, grid, THREADS, smem, st, mk, mv, p, b, c, x, n_stages, (int)ring, s_waits);
    return spite_launch_status();
}

}  // namespace

// `n_blocks` = sum over the segments this kernel serves of ceil(tokens / tokens_per_block), computed by the
// caller; `n_stages` (2..8) tiles of 64 keys and values are in flight per block.  With splits, `partial` holds
// n_blocks * kv heads * splits * 16 * (head_dim + 4) floats and `tickets` n_blocks * kv heads ints that are zero
// before the first call (the kernel leaves them zero); calls that share them must not overlap.
SPITE_API int spite_paged_attention_decode(const AttentionParams* p, const StepTokens* b, const PagedCache* c,
                                           const AttnDecodeExtra* x, int n_blocks, int n_stages, void* stream) {
    if (!p || !b || !c || !x || !p->q || !p->out || !x->cu_seqlens || !c->kv) return SPITE_BAD_ARG;
    if (!b->positions || !b->block_table || !b->seg_of_token || b->n_tokens < 0 || b->table_width < 1)
        return SPITE_BAD_ARG;
    if (p->num_heads < 1 || c->num_kv_heads < 1 || p->num_heads % c->num_kv_heads) return SPITE_BAD_ARG;
    if (p->window_kind < 0 || p->window_kind > 2) return SPITE_BAD_ARG;
    if (p->window_kind != SPITE_WINDOW_FULL && p->window_size < 1) return SPITE_BAD_ARG;
    if (x->n_splits < 1 || x->n_segments < 1 || x->tokens_per_block < 1 || n_blocks < 0) return SPITE_BAD_ARG;
    if (c->n_pages < 1 || c->page_size < 1 || n_stages < 2 || n_stages > MAX_STAGES) return SPITE_BAD_ARG;
    const int G = p->num_heads / c->num_kv_heads;
    if ((c->head_dim != 64 && c->head_dim != 128) || G > 16 || c->page_size % BN) return SPITE_UNSUPPORTED;
    if (x->tokens_per_block * G > 16) return SPITE_BAD_ARG;
    if (x->n_splits > 1 && (!x->partial || !x->tickets)) return SPITE_BAD_ARG;
    if (x->n_splits > 1024 || c->num_kv_heads > 65535 || x->n_splits > 65535) return SPITE_UNSUPPORTED;
    if ((((uintptr_t)p->q | (uintptr_t)p->out | (uintptr_t)c->kv | (uintptr_t)x->partial) & 15) || (c->v_offset & 7))
        return SPITE_UNSUPPORTED;                              // TMA, 16-byte loads of partial results, 8-byte stores
    if (b->n_tokens == 0 || n_blocks == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    return c->head_dim == 64 ? launch<1>(*p, *b, *c, *x, n_blocks, n_stages, st)
                             : launch<2>(*p, *b, *c, *x, n_blocks, n_stages, st);
}
