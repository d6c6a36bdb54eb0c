// Attention over the paged cache on the tensor cores (bfloat16, head sizes 16..128
// in steps of 16, up to 16 query heads per kv head, pages of a multiple of 16 keys).
//
// The rows of the score matrix are (token, query head of one kv group) pairs, up to
// 16 per block, all of one request; their keys and values are therefore loaded once
// for the whole group.  A block's four warps take turns on tiles of 16 keys
// (cp.async into shared memory, double buffered per warp), each with its own running
// maximum and sum in float32; the warps' states are merged in shared memory at the
// end.  With several splits along the keys (decode: few rows, long context) a block
// writes an unnormalised partial result and a second kernel merges the splits; the
// order of the merge is fixed by the split count.
//
// Score, mask and softmax: crates/spite-compute/src/flash_attn.rs:111-156; the local
// window rule is the architecture's (same chunk), see attention.cuh.
#include "attention.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int TILE = 16;

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
__device__ __forceinline__ void ldmatrix_x2(unsigned (&r)[2], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// 16 bytes of the cache: read once a step, so marked to leave L2 first
__device__ __forceinline__ void cp_async16(unsigned dst, const void* src, unsigned long long policy) {
    asm volatile("cp.async.cg.shared.global.L2::cache_hint.L2::256B [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "l"(policy));
}
__device__ __forceinline__ unsigned long long l2_evict_first() {
    unsigned long long policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ unsigned pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *(unsigned*)&v;
}

// NK = head_dim / 16
template <int NK>
__global__ void __launch_bounds__(WARPS * 32) attn_mma_kernel(const AttentionParams p, const StepTokens b,
                                                              const PagedCache c, const AttnMmaExtra x) {
    constexpr int HD = 16 * NK;
    constexpr int CH = 2 * NK;                          // 16-byte chunks per key row
    constexpr int SWZ = (CH % 8 == 0) ? 7 : 0;          // xor of the chunk index with the row, where rows alias
    constexpr int TILE_BYTES = TILE * HD * 2;
    extern __shared__ __align__(128) unsigned char smem[];
    pdl_wait();
    pdl_launch_dependents();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, cc = lane & 3;
    const int nq = p.num_heads, nkv = c.num_kv_heads, G = nq / nkv;

    // which request and which of its tokens
    int idx = blockIdx.x, seg = -1, t0 = 0, nt = 0;
    for (int s = 0; s < x.n_segments; ++s) {
        const int lo = x.cu_seqlens[s], n = x.cu_seqlens[s + 1] - lo;
        if (n < x.seg_min_tokens || n > x.seg_max_tokens) continue;   // another kernel serves this segment
        const int blocks = (n + x.tokens_per_block - 1) / x.tokens_per_block;
        if (idx < blocks) { seg = s; t0 = lo + idx * x.tokens_per_block; nt = min(x.tokens_per_block, lo + n - t0); break; }
        idx -= blocks;
    }
    if (seg < 0) return;
    const int kvh = blockIdx.y, split = blockIdx.z;
    const int n_rows = nt * G;
    const int* table = b.block_table + (size_t)seg * b.table_width;

    // the two rows of this lane: g and g + 8
    int row_pos[2], row_lo[2];
    bool row_ok[2];
    const __nv_bfloat16* qrow[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = g + 8 * h;
        row_ok[h] = r < n_rows;
        const int tok = t0 + (row_ok[h] ? r / G : 0);
        const int head = kvh * G + (row_ok[h] ? r % G : 0);
        row_pos[h] = b.positions[tok];
        row_lo[h] = window_lowest(p.window_kind, p.window_size, row_pos[h]);
        qrow[h] = (const __nv_bfloat16*)p.q + ((size_t)tok * nq + head) * HD;
    }
    unsigned qa[NK][4];
#pragma unroll
    for (int kk = 0; kk < NK; ++kk) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const unsigned* src = (const unsigned*)(qrow[h] + 16 * kk + 2 * cc);
            qa[kk][h] = row_ok[h] ? src[0] : 0u;            // k = 2c, 2c+1
            qa[kk][2 + h] = row_ok[h] ? src[4] : 0u;        // k = 2c+8, 2c+9
        }
    }

    // tiles of 16 keys this block and this warp walk
    const int p_first = b.positions[t0], p_last = b.positions[t0 + nt - 1];
    const int tile_lo = window_lowest(p.window_kind, p.window_size, p_first) / TILE;
    const int tile_hi = p_last / TILE + 1;
    const int n_tiles = tile_hi - tile_lo;
    const int sb = tile_lo + (int)((long long)n_tiles * split / x.n_splits);
    const int se = tile_lo + (int)((long long)n_tiles * (split + 1) / x.n_splits);

    unsigned char* my = smem + (size_t)warp * 4 * TILE_BYTES;       // [stage][K, V][16][HD]
    const unsigned my_addr = (unsigned)__cvta_generic_to_shared(my);
    const __nv_bfloat16* kbase = (const __nv_bfloat16*)c.kv;
    const __nv_bfloat16* vbase = kbase + c.v_offset;

    const unsigned long long kv_policy = l2_evict_first();
    auto issue = [&](int stage, int ti) {
        const int j0 = ti * TILE;
        const int page = table[j0 / c.page_size];
        const size_t off = (((size_t)max(page, 0) * nkv + kvh) * c.page_size + j0 % c.page_size) * HD;
        const unsigned kdst = my_addr + stage * 2 * TILE_BYTES, vdst = kdst + TILE_BYTES;
#pragma unroll
        for (int i = 0; i < NK; ++i) {
            const int e = lane + 32 * i;
            const int r = e / CH, ch = e % CH;
            const unsigned d = r * (HD * 2) + ((ch ^ (r & SWZ)) << 4);
            cp_async16(kdst + d, kbase + off + (size_t)r * HD + ch * 8, kv_policy);
            cp_async16(vdst + d, vbase + off + (size_t)r * HD + ch * 8, kv_policy);
        }
    };

    float o[2 * NK][4];
#pragma unroll
    for (int n = 0; n < 2 * NK; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    int ti = sb + warp;
    if (ti < se) issue(0, ti);
    cp_async_commit();
    int stage = 0;
    for (; ti < se; ti += WARPS, stage ^= 1) {
        if (ti + WARPS < se) issue(stage ^ 1, ti + WARPS);
        cp_async_commit();
        cp_async_wait<1>();
        __syncwarp();
        const unsigned kaddr = my_addr + stage * 2 * TILE_BYTES, vaddr = kaddr + TILE_BYTES;

        // scores of 16 rows x 16 keys
        float s[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
            const int r = n * 8 + (lane & 7);
#pragma unroll
            for (int kk = 0; kk + 1 < NK; kk += 2) {
                unsigned kb[4];
                const int ch = 2 * kk + (lane >> 3);
                ldmatrix_x4(kb, kaddr + r * (HD * 2) + ((ch ^ (r & SWZ)) << 4));
                mma16816(s[n], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], kb[0], kb[1]);
                mma16816(s[n], qa[kk + 1][0], qa[kk + 1][1], qa[kk + 1][2], qa[kk + 1][3], kb[2], kb[3]);
            }
            if (NK & 1) {
                unsigned kb[2];
                const int ch = 2 * (NK - 1) + ((lane >> 3) & 1);
                ldmatrix_x2(kb, kaddr + r * (HD * 2) + ((ch ^ (r & SWZ)) << 4));
                mma16816(s[n], qa[NK - 1][0], qa[NK - 1][1], qa[NK - 1][2], qa[NK - 1][3], kb[0], kb[1]);
            }
        }
        // mask, running maximum and sum (float32)
        const int j0 = ti * TILE;
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float mx = -INFINITY;
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = j0 + 8 * n + 2 * cc + e;
                    const bool ok = row_ok[h] && j >= row_lo[h] && j <= row_pos[h];
                    const float v = ok ? s[n][2 * h + e] * p.softmax_scale : -INFINITY;
                    s[n][2 * h + e] = v;
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
                    const float pv = (m_new == -INFINITY) ? 0.f : expf(s[n][2 * h + e] - m_new);
                    s[n][2 * h + e] = pv;
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
        const unsigned pa0 = pack_bf16(s[0][0], s[0][1]), pa1 = pack_bf16(s[0][2], s[0][3]);
        const unsigned pa2 = pack_bf16(s[1][0], s[1][1]), pa3 = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int jj = 0; jj < NK; ++jj) {
            unsigned vb[4];
            const int r = (lane & 7) + 8 * ((lane >> 3) & 1);
            const int ch = 2 * jj + (lane >> 4);
            ldmatrix_x4_trans(vb, vaddr + r * (HD * 2) + ((ch ^ (r & SWZ)) << 4));
            mma16816(o[2 * jj], pa0, pa1, pa2, pa3, vb[0], vb[1]);
            mma16816(o[2 * jj + 1], pa0, pa1, pa2, pa3, vb[2], vb[3]);
        }
        __syncwarp();
    }
    cp_async_wait<0>();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    __syncthreads();                                         // the tiles are dead: reuse their memory

    float* o_s = (float*)smem;                               // [WARPS][16][HD]
    float* m_s = o_s + WARPS * 16 * HD;                      // [WARPS][16]
    float* l_s = m_s + WARPS * 16;
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
    __syncthreads();
    for (int e = threadIdx.x; e < n_rows * HD; e += WARPS * 32) {
        const int r = e / HD, d = e % HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) m = fmaxf(m, m_s[w * 16 + r]);
        float l = 0.f, acc = 0.f;
        if (m > -INFINITY) {
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float f = expf(m_s[w * 16 + r] - m);
                l += l_s[w * 16 + r] * f;
                acc += o_s[((size_t)w * 16 + r) * HD + d] * f;
            }
        }
        const int tok = t0 + r / G, head = kvh * G + r % G;
        if (x.n_splits == 1) {
            ((__nv_bfloat16*)p.out)[((size_t)tok * nq + head) * HD + d] = __float2bfloat16_rn(acc / fmaxf(l, 1e-30f));
        } else {
            // partial results are indexed by the block's place among this kernel's blocks, not by the
            // token's place in the step: a long prompt portion beside one decoded token costs no scratch
            const size_t slot = (((size_t)blockIdx.x * x.tokens_per_block + r / G) * nq + head) * x.n_splits + split;
            x.o_part[slot * HD + d] = acc;
            if (d == 0) { x.ml_part[slot * 2] = m; x.ml_part[slot * 2 + 1] = l; }
        }
    }
}

// grid (blocks of the kernel above) * tokens_per_block * heads, block 128: merge the splits of one
// (token, head).  Thread s takes split s's maximum and sum (at most MERGE_THREADS splits); the weights
// 2^.. of the splits go through shared memory, then every thread sums its output elements over the
// splits in ascending order.
constexpr int MERGE_THREADS = 128;
__global__ void __launch_bounds__(MERGE_THREADS) attn_merge_kernel(const float* __restrict__ o_part,
                                                                   const float* __restrict__ ml_part,
                                                                   __nv_bfloat16* __restrict__ out, int n_splits, int hd,
                                                                   int num_heads, const AttnMmaExtra x) {
    __shared__ float w_s[MERGE_THREADS];
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch_dependents();
    const size_t row = blockIdx.x;
    const int head = (int)(row % num_heads);
    const int local = (int)((row / num_heads) % x.tokens_per_block);
    int idx = (int)(row / num_heads / x.tokens_per_block), tok = -1;
    for (int s = 0; s < x.n_segments; ++s) {                // the same walk as the kernel above
        const int lo = x.cu_seqlens[s], n = x.cu_seqlens[s + 1] - lo;
        if (n < x.seg_min_tokens || n > x.seg_max_tokens) continue;
        const int blocks = (n + x.tokens_per_block - 1) / x.tokens_per_block;
        if (idx < blocks) {
            const int t = lo + idx * x.tokens_per_block + local;
            if (t < lo + n) tok = t;
            break;
        }
        idx -= blocks;
    }
    if (tok < 0) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float ms = -INFINITY, ls = 0.f;
    if (tid < n_splits) {
        const float2 ml = *(const float2*)(ml_part + (row * n_splits + tid) * 2);
        ms = ml.x; ls = ml.y;
    }
    float m = warp_max(ms);
    if (lane == 0) scratch[warp] = m;
    __syncthreads();
    m = fmaxf(fmaxf(scratch[0], scratch[1]), fmaxf(scratch[2], scratch[3]));
    const float w = ms > -INFINITY ? expf(ms - m) : 0.f;
    w_s[tid] = w;
    const float l = block_sum(ls * w, scratch);             // syncs: w_s is visible afterwards
    const float inv = 1.0f / fmaxf(l, 1e-30f);
    const float* o = o_part + row * n_splits * hd;
    __nv_bfloat16* dst = out + ((size_t)tok * num_heads + head) * hd;
    for (int d = tid; d < hd; d += MERGE_THREADS) {
        float acc = 0.f;
#pragma unroll 4
        for (int s = 0; s < n_splits; ++s) acc = fmaf(o[(size_t)s * hd + d], w_s[s], acc);
        dst[d] = __float2bfloat16_rn(acc * inv);
    }
}

template <int NK>
int launch(const AttentionParams& p, const StepTokens& b, const PagedCache& c, const AttnMmaExtra& x,
           int n_blocks, cudaStream_t st) {
    const size_t tiles = (size_t)WARPS * 4 * TILE * 16 * NK * 2;
    const size_t merge = (size_t)WARPS * 16 * 16 * NK * 4 + WARPS * 16 * 2 * 4;
    const size_t smem = tiles > merge ? tiles : merge;
    auto k = attn_mma_kernel<NK>;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return SPITE_LAUNCH_FAILED;
    dim3 grid(n_blocks, c.num_kv_heads, x.n_splits);
    SPITE_LAUNCH(k, grid, WARPS * 32, smem, st, p, b, c, x);
    return spite_launch_status();
}

}  // namespace

// `n_blocks` = sum over the segments this kernel serves of ceil(tokens / tokens_per_block), computed by the
// caller.  With splits, `o_part` holds n_blocks * tokens_per_block * heads * splits * head_dim floats and
// `ml_part` two floats per (row, head, split).
SPITE_API int spite_paged_attention_mma(const AttentionParams* p, const StepTokens* b, const PagedCache* c,
                                        const AttnMmaExtra* x, int n_blocks, void* stream) {
    if (!p || !b || !c || !x || !p->q || !p->out || !x->cu_seqlens || !c->kv) return SPITE_BAD_ARG;
    if (!b->positions || !b->block_table || !b->seg_of_token || b->n_tokens < 0 || b->table_width < 1)
        return SPITE_BAD_ARG;
    if (p->num_heads < 1 || c->num_kv_heads < 1 || p->num_heads % c->num_kv_heads) return SPITE_BAD_ARG;
    if (p->window_kind < 0 || p->window_kind > 2) return SPITE_BAD_ARG;
    if (p->window_kind != SPITE_WINDOW_FULL && p->window_size < 1) return SPITE_BAD_ARG;
    if (x->n_splits < 1 || x->n_segments < 1 || x->tokens_per_block < 1 || n_blocks < 0) return SPITE_BAD_ARG;
    const int G = p->num_heads / c->num_kv_heads;
    if (c->head_dim % 16 || c->head_dim > 128 || G > 16 || c->page_size % 16) return SPITE_UNSUPPORTED;
    if (x->tokens_per_block * G > 16) return SPITE_BAD_ARG;
    if (x->n_splits > 1 && (!x->o_part || !x->ml_part)) return SPITE_BAD_ARG;
    if (x->n_splits > MERGE_THREADS || c->num_kv_heads > 65535) return SPITE_UNSUPPORTED;
    if (b->n_tokens == 0 || n_blocks == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    int rc;
    switch (c->head_dim / 16) {
        case 1: rc = launch<1>(*p, *b, *c, *x, n_blocks, st); break;
        case 2: rc = launch<2>(*p, *b, *c, *x, n_blocks, st); break;
        case 3: rc = launch<3>(*p, *b, *c, *x, n_blocks, st); break;
        case 4: rc = launch<4>(*p, *b, *c, *x, n_blocks, st); break;
        case 5: rc = launch<5>(*p, *b, *c, *x, n_blocks, st); break;
        case 6: rc = launch<6>(*p, *b, *c, *x, n_blocks, st); break;
        case 7: rc = launch<7>(*p, *b, *c, *x, n_blocks, st); break;
        default: rc = launch<8>(*p, *b, *c, *x, n_blocks, st); break;
    }
    if (rc != SPITE_OK || x->n_splits == 1) return rc;
    SPITE_LAUNCH(attn_merge_kernel, n_blocks * x->tokens_per_block * p->num_heads, MERGE_THREADS, 0, st,
                 (const float*)x->o_part, (const float*)x->ml_part, (__nv_bfloat16*)p->out, x->n_splits,
                 c->head_dim, p->num_heads, *x);
    return spite_launch_status();
}
