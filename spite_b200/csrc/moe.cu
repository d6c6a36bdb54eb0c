// Router of a mixture-of-experts feed-forward and the ordering of tokens by expert.
//
// logits: l = Wr x in float32 (crates/spite-models/src/moe.rs:65-66).
// select: the k largest raw logits are chosen, equal logits preferring the lower expert
//   id (moe.rs:110-116, a stable descending sort); the weight is sigmoid(logit)
//   (moe.rs:120).  No softmax, no renormalisation.
//   Choices are stored slot-major: expert_ids[slot][token], weights[slot][token].
// sort: for every choice slot a stable counting sort of the tokens by expert:
//   offsets[slot][e] .. offsets[slot][e+1] are the places of expert e's tokens in
//   sorted_rows[slot][:], in ascending token order.  No host round trip: the grouped
//   products read these arrays on the device.
//
// Two kernels.  The first computes the logits (8 tokens x 2 experts at a time, the block's 8
// warps splitting the width), one pair of experts a block, so that a few tokens still spread over
// several multiprocessors.  The second, one block per choice slot, selects and sorts.
// A logit is summed in an order fixed by the width alone.
#include "common.cuh"

namespace {

constexpr int MAX_EXPERTS = 1024;
constexpr int TB = 8;                  // tokens per block of the logits kernel
constexpr int EB = 2;                  // experts per block
constexpr int WARPS = 8;

__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
    const float4 t = *(const float4*)p;
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 t = *(const uint2*)p;
    const __nv_bfloat162 a = *(const __nv_bfloat162*)&t.x, b = *(const __nv_bfloat162*)&t.y;
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}

// grid (ceil(tokens / TB), ceil(experts / experts_per_block)), block 256.  A block computes the logits
// of TB tokens for experts_per_block experts, EB at a time; from the second pair on its tokens come
// out of the first-level cache.
template <typename T>
__global__ void __launch_bounds__(WARPS * 32) route_logits_kernel(const T* __restrict__ x, const float* __restrict__ wr,
                                                                 int n_tokens, int d, int n_experts, int experts_per_block,
                                                                 float* __restrict__ logits) {
    __shared__ float part[WARPS][EB * TB];
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * TB;
    const int e_end = min(n_experts, (int)(blockIdx.y + 1) * experts_per_block);
    const bool vec = (d % 4 == 0) && (((uintptr_t)wr & 15) == 0) && (((uintptr_t)x & 15) == 0);
    for (int e0 = blockIdx.y * experts_per_block; e0 < e_end; e0 += EB) {
        float acc[EB][TB];
#pragma unroll
        for (int e = 0; e < EB; ++e)
#pragma unroll
            for (int t = 0; t < TB; ++t) acc[e][t] = 0.f;

        if (vec) {
            const int n4 = d >> 2;                            // groups of four elements
            const int lo = (int)((long long)n4 * warp / WARPS), hi = (int)((long long)n4 * (warp + 1) / WARPS);
            for (int k4 = lo + lane; k4 < hi; k4 += 32) {
                float w[EB][4];
#pragma unroll
                for (int e = 0; e < EB; ++e) {
                    if (e0 + e < e_end) load4(wr + (size_t)(e0 + e) * d + 4 * k4, w[e]);
                    else w[e][0] = w[e][1] = w[e][2] = w[e][3] = 0.f;
                }
#pragma unroll
                for (int t = 0; t < TB; ++t) {
                    if (t0 + t < n_tokens) {
                        float xv[4];
                        load4(x + (size_t)(t0 + t) * d + 4 * k4, xv);
#pragma unroll
                        for (int e = 0; e < EB; ++e)
#pragma unroll
                            for (int i = 0; i < 4; ++i) acc[e][t] = fmaf(xv[i], w[e][i], acc[e][t]);
                    }
                }
            }
        } else {
            const int lo = (int)((long long)d * warp / WARPS), hi = (int)((long long)d * (warp + 1) / WARPS);
            for (int k = lo + lane; k < hi; k += 32) {
#pragma unroll
                for (int t = 0; t < TB; ++t) {
                    if (t0 + t < n_tokens) {
                        const float xv = to_f32(x[(size_t)(t0 + t) * d + k]);
#pragma unroll
                        for (int e = 0; e < EB; ++e)
                            if (e0 + e < e_end) acc[e][t] = fmaf(xv, wr[(size_t)(e0 + e) * d + k], acc[e][t]);
                    }
                }
            }
        }
        __syncthreads();                                      // the sums of the pair before have been read
#pragma unroll
        for (int e = 0; e < EB; ++e)
#pragma unroll
            for (int t = 0; t < TB; ++t) {
                const float s = warp_sum(acc[e][t]);
                if (lane == 0) part[warp][e * TB + t] = s;
            }
        __syncthreads();
        if (threadIdx.x < EB * TB) {
            const int e = threadIdx.x / TB, t = threadIdx.x % TB;
            if (e0 + e < e_end && t0 + t < n_tokens) {
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < WARPS; ++w) s += part[w][threadIdx.x];
                logits[(size_t)(t0 + t) * n_experts + e0 + e] = s;
            }
        }
    }
}

// grid top_k, block 1024: block `slot` picks every token's slot-th expert and sorts the tokens by it.
__global__ void __launch_bounds__(1024) select_and_sort_kernel(const float* __restrict__ logits, int n_tokens,
                                                               int n_experts, int top_k,
                                                               int* __restrict__ expert_ids, float* __restrict__ weights,
                                                               int* __restrict__ offsets,
                                                               int* __restrict__ sorted_rows) {
    __shared__ int counts[MAX_EXPERTS + 1];
    pdl_wait();
    pdl_launch_dependents();
    const int slot = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    int* ids = expert_ids + (size_t)slot * n_tokens;
    for (int t = threadIdx.x; t < n_tokens; t += blockDim.x) {
        // the slot-th element in the order (logit descending, expert id ascending)
        const float* l = logits + (size_t)t * n_experts;
        float prev_v = INFINITY;
        int prev_e = -1;
        float best_v = 0.f;
        int best_e = 0;
        for (int s = 0; s <= slot; ++s) {
            best_v = -INFINITY;
            best_e = -1;
            for (int e = 0; e < n_experts; ++e) {
                const float v = l[e];
                const bool after_prev = v < prev_v || (v == prev_v && e > prev_e);
                if (after_prev && (best_e < 0 || v > best_v)) { best_v = v; best_e = e; }
            }
            if (best_e < 0) { best_e = 0; best_v = l[0]; }    // logits that do not compare (NaN): still a valid id
            prev_v = best_v;
            prev_e = best_e;
        }
        ids[t] = best_e;
        weights[(size_t)slot * n_tokens + t] = 1.0f / (1.0f + expf(-best_v));
        atomicAdd(&counts[best_e + 1], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0)
        for (int e = 0; e < n_experts; ++e) counts[e + 1] += counts[e];
    __syncthreads();
    int* off = offsets + (size_t)slot * (n_experts + 1);
    for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) off[e] = counts[e];
    int* rows = sorted_rows + (size_t)slot * n_tokens;
    for (int e = warp; e < n_experts; e += nwarps) {
        int base = counts[e];
        if (counts[e + 1] == base) continue;
        for (int t0 = 0; t0 < n_tokens; t0 += 32) {
            const int t = t0 + lane;
            const bool mine = t < n_tokens && ids[t] == e;
            const unsigned mask = __ballot_sync(0xffffffffu, mine);
            if (mine) rows[base + __popc(mask & ((1u << lane) - 1u))] = t;
            base += __popc(mask);
        }
    }
}

}  // namespace

// `logits` [tokens, experts] float32 is always written (the caller owns it).
SPITE_API int spite_moe_route(int dtype, const void* x, const float* w_router, int n_tokens, int d,
                              int n_experts, int top_k, int* expert_ids, float* weights,
                              float* logits, int* offsets, int* sorted_rows, void* stream) {
    if (!x || !w_router || !expert_ids || !weights || !logits || !offsets || !sorted_rows) return SPITE_BAD_ARG;
    if (n_tokens < 0 || d <= 0 || n_experts < 1 || top_k < 1 || top_k > n_experts) return SPITE_BAD_ARG;
    if (n_experts > MAX_EXPERTS) return SPITE_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    if (n_tokens > 0) {
        // one pair of experts a block: measured faster than blocks that take several pairs and reuse
        // their tokens from the first-level cache (31 us against 40 and 53 us for 2048 tokens, 16 experts)
        const int per_block = EB;
        dim3 grid((n_tokens + TB - 1) / TB, (n_experts + per_block - 1) / per_block);
        if (grid.y > 65535) return SPITE_UNSUPPORTED;
        if (dtype == SPITE_DT_F32)
            SPITE_LAUNCH(route_logits_kernel<float>, grid, WARPS * 32, 0, st, (const float*)x, w_router, n_tokens, d,
                         n_experts, per_block, logits);
        else if (dtype == SPITE_DT_BF16)
            SPITE_LAUNCH(route_logits_kernel<__nv_bfloat16>, grid, WARPS * 32, 0, st, (const __nv_bfloat16*)x, w_router,
                         n_tokens, d, n_experts, per_block, logits);
        else
            return SPITE_BAD_ARG;
        if (cudaGetLastError() != cudaSuccess) return SPITE_LAUNCH_FAILED;
    }
    SPITE_LAUNCH(select_and_sort_kernel, top_k, 1024, 0, st, (const float*)logits, n_tokens, n_experts, top_k,
                 expert_ids, weights, offsets, sorted_rows);
    return spite_launch_status();
}
