// Attention over the paged cache, general kernels (any head size that is a
// multiple of 2 up to 256, any number of heads and groups, both element types).
//
//  * qk_prepare: position encoding of q and k (neighbouring elements or the two halves of
//    the rotating part pair up), per-head RMS norm after or before it with or without gains,
//    the temperature factor of layers without rotation, and the append of k and v to
//    their pages, in one pass over the projection's output (one warp per head).
//  * paged_attention: one warp per (token, query head) walks the visible keys in
//    tiles of 32, keeps a running maximum and sum (all in float32) and gathers the
//    values.  It serves prompt portions and decoded tokens alike, since every key of
//    the step is in the cache before it runs.
#include "attention.cuh"

namespace {

// Two neighbouring elements with one load or store.
__device__ __forceinline__ void load_pair(const float* p, float& a, float& b) { const float2 v = *(const float2*)p; a = v.x; b = v.y; }
__device__ __forceinline__ void load_pair(const __nv_bfloat16* p, float& a, float& b) {
    const __nv_bfloat162 v = *(const __nv_bfloat162*)p;
    a = __low2float(v); b = __high2float(v);
}
__device__ __forceinline__ void store_pair(float* p, float a, float b) { *(float2*)p = make_float2(a, b); }
__device__ __forceinline__ void store_pair(__nv_bfloat16* p, float a, float b) { *(__nv_bfloat162*)p = __floats2bfloat162_rn(a, b); }

// grid (tokens, ceil(heads_total / heads_per_block)), block 32 * warps: a warp takes the heads
// blockIdx.y * heads_per_block + warp, + warps, ... of q, k and v, one at a time.
// HALVES: the two halves of the rotating part pair up (else neighbours; then every index below is known when
// the kernel is compiled, and a pair moves as one word).
template <typename T, bool HALVES>
__global__ void __launch_bounds__(256) qk_prepare_kernel(const QkPrepareParams p, const StepTokens b,
                                                         const PagedCache c, const int heads_per_block) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int nq = p.num_heads, nkv = c.num_kv_heads, hd = c.head_dim;
    const int heads_total = nq + 2 * nkv;
    const int head_end = min(heads_total, (int)(blockIdx.y + 1) * heads_per_block);
    const int pos = b.positions[t];
    int page = -1;
    if (p.write_cache) {
        page = b.block_table[(size_t)b.seg_of_token[t] * b.table_width + pos / c.page_size];
        if (page >= c.n_pages) page = -1;                     // the host never lets this happen
    }
    // the temperature factor of this position (llama4.rs:177-183)
    float temp = 1.f;
    if (p.temperature_floor > 0) temp = logf((float)((pos + 1) / p.temperature_floor) + 1.0f) * p.temperature_scale + 1.0f;

    // Pair i of a head is the elements (e0, e1): the neighbours (2i, 2i+1), or, among the first
    // `rot` elements when halves pair up, (i, i + rot/2); pairs beyond the rotating part are the
    // neighbours that remain.  Lane l holds the pairs l, l + 32, ...; the rotation of a pair is the
    // same for every head: cos and sin of pos * inv_freq[i], once per warp.
    constexpr int MAXP = 4;                                  // pairs per lane: head_dim <= 256
    const int rot = p.inv_freq ? p.rotary_dim : 0;
    constexpr bool halves = HALVES;
    // cos and sin of a position's angles are the same for every head: the block computes each once (the exact
    // sincosf of an angle of thousands of radians is the most expensive thing here) and its warps read them
    __shared__ float cs_s[128], sn_s[128];
    for (int i = threadIdx.x; 2 * i < rot; i += blockDim.x) sincosf((float)pos * p.inv_freq[i], &sn_s[i], &cs_s[i]);
    __syncthreads();
    float cs[MAXP], sn[MAXP];
    int e0[MAXP], e1[MAXP];                                  // (neighbours: known at compile time, no registers)
#pragma unroll
    for (int r = 0; r < MAXP; ++r) {
        const int i = lane + 32 * r;
        cs[r] = 1.f; sn[r] = 0.f;
        e0[r] = 2 * i; e1[r] = 2 * i + 1;
        if (2 * i < rot) {
            cs[r] = cs_s[i]; sn[r] = sn_s[i];
            if (halves) { e0[r] = i; e1[r] = i + rot / 2; }
        }
    }

    // (Measured and not kept: a warp loading four heads before working on the first, 61 against 33 us for 2,048
    // tokens of 56 heads; one head a warp with more blocks, 51 us.)
    const bool norm = p.qk_norm_eps > 0.f;
    const bool norm_first = norm && p.norm_before_rotation;
    for (int head = blockIdx.y * heads_per_block + warp; head < head_end; head += n_warps) {
        const T* in = (const T*)p.qkv + (size_t)t * heads_total * hd + (size_t)head * hd;
        const bool is_q = head < nq, is_v = head >= nq + nkv;
        T* dst;
        if (is_q) {
            dst = (T*)p.q_out + ((size_t)t * nq + head) * hd;
        } else {
            if (page < 0) continue;                          // nothing to append (or no page: the host never lets this happen)
            const int kvh = is_v ? head - nq - nkv : head - nq;
            dst = (T*)c.kv + (is_v ? c.v_offset : 0) +
                  (((size_t)page * nkv + kvh) * c.page_size + pos % c.page_size) * hd;
        }
        if (is_v) {
            for (int i = lane; 2 * i < hd; i += 32) {
                float a, bb;
                load_pair(in + 2 * i, a, bb);
                store_pair(dst + 2 * i, a, bb);
            }
            continue;
        }
        // q or k (rotation: crates/spite-rope/src/lib.rs:83-91; norm after it: llama4.rs:161-176)
        const float* gain = is_q ? p.q_gain : p.k_gain;
        float x0[MAXP], x1[MAXP];
#pragma unroll
        for (int r = 0; r < MAXP; ++r) {
            x0[r] = x1[r] = 0.f;
            if (2 * (lane + 32 * r) < hd) {
                if (halves) { x0[r] = to_f32(in[e0[r]]); x1[r] = to_f32(in[e1[r]]); }
                else load_pair(in + e0[r], x0[r], x1[r]);
            }
        }
        if (norm_first) {
            float ss = 0.f;
#pragma unroll
            for (int r = 0; r < MAXP; ++r) ss += x0[r] * x0[r] + x1[r] * x1[r];
            ss = warp_sum(ss);
            const float mul = 1.0f / sqrtf(ss / (float)hd + p.qk_norm_eps);
#pragma unroll
            for (int r = 0; r < MAXP; ++r) {
                if (2 * (lane + 32 * r) >= hd) continue;
                x0[r] *= mul; x1[r] *= mul;
                if (gain) { x0[r] *= gain[e0[r]]; x1[r] *= gain[e1[r]]; }
            }
        }
        float ss = 0.f;
#pragma unroll
        for (int r = 0; r < MAXP; ++r) {
            if (2 * (lane + 32 * r) < rot) {
                const float ra = x0[r] * cs[r] - x1[r] * sn[r], rb = x0[r] * sn[r] + x1[r] * cs[r];
                x0[r] = ra; x1[r] = rb;
            }
            ss += x0[r] * x0[r] + x1[r] * x1[r];
        }
        float mul = 1.f;
        if (norm && !norm_first) {
            ss = warp_sum(ss);
            mul = 1.0f / sqrtf(ss / (float)hd + p.qk_norm_eps);
        }
        if (is_q) mul *= temp;
#pragma unroll
        for (int r = 0; r < MAXP; ++r) {
            if (2 * (lane + 32 * r) >= hd) continue;
            float a = x0[r] * mul, bb = x1[r] * mul;
            if (gain && norm && !norm_first) { a *= gain[e0[r]]; bb *= gain[e1[r]]; }
            if (halves) { dst[e0[r]] = from_f32<T>(a); dst[e1[r]] = from_f32<T>(bb); }
            else store_pair(dst + e0[r], a, bb);
        }
    }
}

// grid (tokens, ceil(nq / 4)), block 128: one warp per (token, query head).
// crates/spite-compute/src/flash_attn.rs:111-156 with the maximum and the sum kept
// as running values over tiles of 32 keys.
template <typename T>
__global__ void __launch_bounds__(128) paged_attention_kernel(const AttentionParams p, const StepTokens b,
                                                              const PagedCache c) {
    __shared__ float q_s[4][256];
    pdl_wait();
    pdl_launch_dependents();

    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * 4 + warp;
    const int nq = p.num_heads, nkv = c.num_kv_heads, hd = c.head_dim;
    if (h >= nq) return;
    const int kvh = h / (nq / nkv);
    const int pos = b.positions[t];
    const int seg = b.seg_of_token[t];
    const int* table = b.block_table + (size_t)seg * b.table_width;
    const int lo = window_lowest(p.window_kind, p.window_size, pos);

    const T* q = (const T*)p.q + ((size_t)t * nq + h) * hd;
    for (int i = lane; i < hd; i += 32) q_s[warp][i] = to_f32(q[i]);
    __syncwarp();

    const T* kbase = (const T*)c.kv;
    const T* vbase = (const T*)c.kv + c.v_offset;
    constexpr int MAXD = 8;                                  // head_dim <= 256
    float acc[MAXD];
#pragma unroll
    for (int r = 0; r < MAXD; ++r) acc[r] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int j0 = lo; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        float s = -INFINITY;
        long long row = -1;
        if (j <= pos) {
            const int page = table[j / c.page_size];
            row = (((long long)page * nkv + kvh) * c.page_size + j % c.page_size) * hd;
            const T* k = kbase + row;
            float dot = 0.f;
            for (int d = 0; d < hd; ++d) dot = fmaf(q_s[warp][d], to_f32(k[d]), dot);
            s = dot * p.softmax_scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = expf(m - m_new);                  // 0 on the first tile (m = -inf)
        const float pj = (j <= pos) ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(pj);
#pragma unroll
        for (int r = 0; r < MAXD; ++r) acc[r] *= corr;
        const int n_valid = min(32, pos - j0 + 1);
        for (int jj = 0; jj < n_valid; ++jj) {
            const float pw = __shfl_sync(0xffffffffu, pj, jj);
            const long long vrow = __shfl_sync(0xffffffffu, row, jj);
            const T* v = vbase + vrow;
#pragma unroll
            for (int r = 0; r < MAXD; ++r) {
                const int d = lane + 32 * r;
                if (d < hd) acc[r] = fmaf(pw, to_f32(v[d]), acc[r]);
            }
        }
        m = m_new;
    }
    const float inv = 1.0f / fmaxf(l, 1e-30f);
    T* out = (T*)p.out + ((size_t)t * nq + h) * hd;
#pragma unroll
    for (int r = 0; r < MAXD; ++r) {
        const int d = lane + 32 * r;
        if (d < hd) out[d] = from_f32<T>(acc[r] * inv);
    }
}

int check_common(const StepTokens* b, const PagedCache* c, int num_heads) {
    if (!b || !c || !b->positions || !b->seg_of_token || !b->block_table || !c->kv) return SPITE_BAD_ARG;
    if (b->n_tokens < 0 || b->table_width < 1 || c->n_pages < 1 || c->page_size < 1) return SPITE_BAD_ARG;
    if (num_heads < 1 || c->num_kv_heads < 1 || num_heads % c->num_kv_heads) return SPITE_BAD_ARG;
    if (c->head_dim < 2 || c->head_dim % 2) return SPITE_BAD_ARG;
    if (c->head_dim > 256) return SPITE_UNSUPPORTED;
    return SPITE_OK;
}

}  // namespace

SPITE_API int spite_qk_prepare(int dtype, const QkPrepareParams* p, const StepTokens* b,
                               const PagedCache* c, void* stream) {
    if (!p || !p->qkv || !p->q_out) return SPITE_BAD_ARG;
    const int chk = check_common(b, c, p->num_heads);
    if (chk != SPITE_OK) return chk;
    if (b->n_tokens == 0) return SPITE_OK;
    if (p->pairing != SPITE_PAIR_NEIGHBOURS && p->pairing != SPITE_PAIR_HALVES) return SPITE_BAD_ARG;
    if (p->inv_freq && (p->rotary_dim < 2 || p->rotary_dim % 2 || p->rotary_dim > c->head_dim)) return SPITE_BAD_ARG;
    if (p->pairing == SPITE_PAIR_HALVES && p->inv_freq && p->rotary_dim % 4) return SPITE_UNSUPPORTED;  // pairs beyond the rotating part start at an even pair index
    const int heads = p->num_heads + 2 * c->num_kv_heads;
    // few tokens: four heads a block, so that the step still fills the device; many: a block per token
    const bool many = b->n_tokens >= 1024;
    const int heads_per_block = many ? 16 : 4;
    const int threads = many ? 256 : 128;
    dim3 grid(b->n_tokens, (heads + heads_per_block - 1) / heads_per_block);
    if (grid.y > 65535) return SPITE_UNSUPPORTED;
    if (((uintptr_t)p->qkv | (uintptr_t)p->q_out | (uintptr_t)c->kv) & 7) return SPITE_UNSUPPORTED;   // pairs move as one word
    cudaStream_t st = (cudaStream_t)stream;
    const bool halves = p->pairing == SPITE_PAIR_HALVES && p->inv_freq;
    if (dtype != SPITE_DT_F32 && dtype != SPITE_DT_BF16) return SPITE_BAD_ARG;
    if (dtype == SPITE_DT_F32) {
        if (halves) SPITE_LAUNCH((qk_prepare_kernel<float, true>), grid, threads, 0, st, *p, *b, *c, heads_per_block);
        else SPITE_LAUNCH((qk_prepare_kernel<float, false>), grid, threads, 0, st, *p, *b, *c, heads_per_block);
    } else {
        if (halves) SPITE_LAUNCH((qk_prepare_kernel<__nv_bfloat16, true>), grid, threads, 0, st, *p, *b, *c, heads_per_block);
        else SPITE_LAUNCH((qk_prepare_kernel<__nv_bfloat16, false>), grid, threads, 0, st, *p, *b, *c, heads_per_block);
    }
    return spite_launch_status();
}

SPITE_API int spite_paged_attention(int dtype, const AttentionParams* p, const StepTokens* b,
                                    const PagedCache* c, void* stream) {
    if (!p || !p->q || !p->out) return SPITE_BAD_ARG;
    const int chk = check_common(b, c, p->num_heads);
    if (chk != SPITE_OK) return chk;
    if (p->window_kind < 0 || p->window_kind > 2) return SPITE_BAD_ARG;
    if (p->window_kind != SPITE_WINDOW_FULL && p->window_size < 1) return SPITE_BAD_ARG;
    if (b->n_tokens == 0) return SPITE_OK;
    dim3 grid(b->n_tokens, (p->num_heads + 3) / 4);
    if (grid.y > 65535) return SPITE_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == SPITE_DT_F32) SPITE_LAUNCH(paged_attention_kernel<float>, grid, 128, 0, st, *p, *b, *c);
    else if (dtype == SPITE_DT_BF16) SPITE_LAUNCH(paged_attention_kernel<__nv_bfloat16>, grid, 128, 0, st, *p, *b, *c);
    else return SPITE_BAD_ARG;
    return spite_launch_status();
}
