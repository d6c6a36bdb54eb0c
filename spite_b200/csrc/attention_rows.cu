// Attention over the paged cache for prompt portions (bfloat16, head sizes 16..128 in
// steps of 16, up to 16 query heads per kv head, pages of a multiple of 32 keys).
//
// A block owns 64 rows of the score matrix, (token, query head of one kv group) pairs of
// consecutive tokens of one request; each of its four warps owns 16 of them from the
// first key to the last and needs no merge.  The block walks tiles of 32 keys that all its
// threads load together (cp.async into a ring of three shared-memory stages), so a key and
// a value row are fetched once for 64 rows of scores, and for every head of the kv group.
// Running maximum and sum are float32.  A warp skips the tiles that lie wholly behind the
// positions of its own rows.
//
// Score, mask and softmax: crates/spite-compute/src/flash_attn.rs:111-156; the local window
// rule is the architecture's (same chunk), see attention.cuh.
#include "attention.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int ROWS = WARPS * 16;
constexpr int TILE = 32;
constexpr int STAGES = 3;

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
__device__ __forceinline__ void cp_async16(unsigned dst, const void* src) {
    asm volatile("cp.async.cg.shared.global.L2::256B [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ unsigned pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *(unsigned*)&v;
}

// NK = head_dim / 16
template <int NK>
__global__ void __launch_bounds__(WARPS * 32) attn_rows_kernel(const AttentionParams p, const StepTokens b,
                                                               const PagedCache c, const AttnMmaExtra x) {
    constexpr int HD = 16 * NK;
    constexpr int CH = 2 * NK;                          // 16-byte chunks per key row
    constexpr int SWZ = (CH % 8 == 0) ? 7 : 0;          // xor of the chunk index with the row, where rows alias
    constexpr int TILE_BYTES = TILE * HD * 2;
    extern __shared__ __align__(128) unsigned char smem[];   // [stage][K, V][32][HD]
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
    const int kvh = blockIdx.y;
    const int n_rows = nt * G;
    const int* table = b.block_table + (size_t)seg * b.table_width;

    // the two rows of this lane: 16 * warp + g and + 8
    int row_pos[2], row_lo[2];
    bool row_ok[2];
    const __nv_bfloat16* qrow[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = 16 * warp + g + 8 * h;
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
            qa[kk][h] = row_ok[h] ? src[0] : 0u;
            qa[kk][2 + h] = row_ok[h] ? src[4] : 0u;
        }
    }
    // the last position any row of this warp can see (rows ascend with the token)
    const int warp_last_row = min(16 * warp + 15, n_rows - 1);
    const int warp_max_pos = warp_last_row >= 0 && 16 * warp < n_rows ? b.positions[t0 + warp_last_row / G] : -1;

    const int p_first = b.positions[t0], p_last = b.positions[t0 + nt - 1];
    const int tile_lo = window_lowest(p.window_kind, p.window_size, p_first) / TILE;
    const int tile_hi = p_last / TILE + 1;

    const unsigned smem_addr = (unsigned)__cvta_generic_to_shared(smem);
    const __nv_bfloat16* kbase = (const __nv_bfloat16*)c.kv;
    const __nv_bfloat16* vbase = kbase + c.v_offset;

    auto issue = [&](int stage, int ti) {
        const int j0 = ti * TILE;
        const int page = table[j0 / c.page_size];
        const size_t off = (((size_t)max(page, 0) * nkv + kvh) * c.page_size + j0 % c.page_size) * HD;
        const unsigned kdst = smem_addr + stage * 2 * TILE_BYTES, vdst = kdst + TILE_BYTES;
        constexpr int CHUNKS = TILE * CH;                     // 16-byte chunks of one tile
        for (int e = threadIdx.x; e < CHUNKS; e += WARPS * 32) {
            const int r = e / CH, ch = e % CH;
            const unsigned d = r * (HD * 2) + ((ch ^ (r & SWZ)) << 4);
            cp_async16(kdst + d, kbase + off + (size_t)r * HD + ch * 8);
            cp_async16(vdst + d, vbase + off + (size_t)r * HD + ch * 8);
        }
    };

    float o[2 * NK][4];
#pragma unroll
    for (int n = 0; n < 2 * NK; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    // ring of STAGES tiles, STAGES - 1 in flight
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (tile_lo + s < tile_hi) issue(s, tile_lo + s);
        cp_async_commit();
    }
    int stage = 0;
    for (int ti = tile_lo; ti < tile_hi; ++ti) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();                                     // tile ti has landed; the stage refilled below is free
        {
            const int nxt = ti + STAGES - 1;
            int ns = stage + STAGES - 1;
            if (ns >= STAGES) ns -= STAGES;
            if (nxt < tile_hi) issue(ns, nxt);
            cp_async_commit();
        }
        const int j0 = ti * TILE;
        if (j0 <= warp_max_pos) {                            // else every key of the tile is behind this warp's rows
            const unsigned kaddr = smem_addr + stage * 2 * TILE_BYTES, vaddr = kaddr + TILE_BYTES;
            float s[4][4];
#pragma unroll
            for (int n = 0; n < 4; ++n) {
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
            float corr[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float mx = -INFINITY;
#pragma unroll
                for (int n = 0; n < 4; ++n)
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
                for (int n = 0; n < 4; ++n)
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
#pragma unroll
            for (int half = 0; half < 2; ++half) {           // 16 keys per k step of P V
                const unsigned pa0 = pack_bf16(s[2 * half][0], s[2 * half][1]), pa1 = pack_bf16(s[2 * half][2], s[2 * half][3]);
                const unsigned pa2 = pack_bf16(s[2 * half + 1][0], s[2 * half + 1][1]);
                const unsigned pa3 = pack_bf16(s[2 * half + 1][2], s[2 * half + 1][3]);
#pragma unroll
                for (int jj = 0; jj < NK; ++jj) {
                    unsigned vb[4];
                    const int r = 16 * half + (lane & 7) + 8 * ((lane >> 3) & 1);
                    const int ch = 2 * jj + (lane >> 4);
                    ldmatrix_x4_trans(vb, vaddr + r * (HD * 2) + ((ch ^ (r & SWZ)) << 4));
                    mma16816(o[2 * jj], pa0, pa1, pa2, pa3, vb[0], vb[1]);
                    mma16816(o[2 * jj + 1], pa0, pa1, pa2, pa3, vb[2], vb[3]);
                }
            }
        }
        if (++stage == STAGES) stage = 0;
    }
    cp_async_wait<0>();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
        if (!row_ok[h]) continue;
        const int r = 16 * warp + g + 8 * h;
        const int tok = t0 + r / G, head = kvh * G + r % G;
        const float inv = 1.0f / fmaxf(l_run[h], 1e-30f);
        __nv_bfloat16* dst = (__nv_bfloat16*)p.out + ((size_t)tok * nq + head) * HD + 2 * cc;
#pragma unroll
        for (int n = 0; n < 2 * NK; ++n)
            *(unsigned*)(dst + 8 * n) = pack_bf16(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
    }
}

template <int NK>
int launch(const AttentionParams& p, const StepTokens& b, const PagedCache& c, const AttnMmaExtra& x,
           int n_blocks, cudaStream_t st) {
    const size_t smem = (size_t)STAGES * 2 * TILE * 16 * NK * 2;
    auto k = attn_rows_kernel<NK>;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return SPITE_LAUNCH_FAILED;
    dim3 grid(n_blocks, c.num_kv_heads);
    SPITE_LAUNCH(k, grid, WARPS * 32, smem, st, p, b, c, x);
    return spite_launch_status();
}

}  // namespace

// `n_blocks` = sum over the served segments of ceil(tokens / tokens_per_block), computed by the caller.
SPITE_API int spite_paged_attention_rows(const AttentionParams* p, const StepTokens* b, const PagedCache* c,
                                         const AttnMmaExtra* x, int n_blocks, void* stream) {
    if (!p || !b || !c || !x || !p->q || !p->out || !x->cu_seqlens || !c->kv) return SPITE_BAD_ARG;
    if (!b->positions || !b->block_table || b->n_tokens < 0 || b->table_width < 1) return SPITE_BAD_ARG;
    if (p->num_heads < 1 || c->num_kv_heads < 1 || p->num_heads % c->num_kv_heads) return SPITE_BAD_ARG;
    if (p->window_kind < 0 || p->window_kind > 2) return SPITE_BAD_ARG;
    if (p->window_kind != SPITE_WINDOW_FULL && p->window_size < 1) return SPITE_BAD_ARG;
    if (x->n_segments < 1 || x->tokens_per_block < 1 || n_blocks < 0) return SPITE_BAD_ARG;
    const int G = p->num_heads / c->num_kv_heads;
    if (c->head_dim % 16 || c->head_dim > 128 || G > 16 || c->page_size % TILE) return SPITE_UNSUPPORTED;
    if (x->tokens_per_block * G > ROWS) return SPITE_BAD_ARG;
    if (c->num_kv_heads > 65535) return SPITE_UNSUPPORTED;
    if (b->n_tokens == 0 || n_blocks == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    switch (c->head_dim / 16) {
        case 1: return launch<1>(*p, *b, *c, *x, n_blocks, st);
        case 2: return launch<2>(*p, *b, *c, *x, n_blocks, st);
        case 3: return launch<3>(*p, *b, *c, *x, n_blocks, st);
        case 4: return launch<4>(*p, *b, *c, *x, n_blocks, st);
        case 5: return launch<5>(*p, *b, *c, *x, n_blocks, st);
        case 6: return launch<6>(*p, *b, *c, *x, n_blocks, st);
        case 7: return launch<7>(*p, *b, *c, *x, n_blocks, st);
        default: return launch<8>(*p, *b, *c, *x, n_blocks, st);
    }
}
