// Router of a mixture-of-experts feed-forward and the ordering of tokens by expert.
//
// route: logits = Wr x in float32 (crates/spite-models/src/moe.rs:65-66); the k
//   largest raw logits are chosen, equal logits preferring the lower expert id
//   (moe.rs:110-116, a stable descending sort); the weight is sigmoid(logit)
//   (moe.rs:120).  No softmax, no renormalisation.
// Choices are stored slot-major: expert_ids[slot][token], weights[slot][token].
// sort: for every choice slot a stable counting sort of the tokens by expert:
//   offsets[slot][e] .. offsets[slot][e+1] are the places of expert e's tokens in
//   sorted_rows[slot][:], in ascending token order.  No host round trip: the grouped
//   products read these arrays on the device.
#include "common.cuh"

namespace {

constexpr int MAX_EXPERTS = 1024;

// grid tokens, block 256: the token's row is staged in shared memory as float32, every
// warp takes experts e = warp, warp + 8, ...; warp 0 then picks the k largest logits.
// A logit is summed in an order fixed by the width d alone.
template <typename T>
__global__ void __launch_bounds__(256) route_kernel(const T* __restrict__ x, const float* __restrict__ wr,
                                                    int n_tokens, int d, int n_experts, int top_k,
                                                    int* __restrict__ expert_ids, float* __restrict__ weights,
                                                    float* __restrict__ logits_out) {
    extern __shared__ __align__(16) float route_s[];         // [d] token, [n_experts] logits
    pdl_wait();
    pdl_launch_dependents();
    float* xs = route_s;
    float* lg = route_s + ((d + 3) & ~3);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const T* xr = x + (size_t)t * d;
    for (int k = threadIdx.x; k < d; k += blockDim.x) xs[k] = to_f32(xr[k]);
    __syncthreads();
    const bool vec = (d % 4 == 0) && (((uintptr_t)wr & 15) == 0);
    for (int e = warp; e < n_experts; e += 8) {
        const float* w = wr + (size_t)e * d;
        float s0 = 0.f, s1 = 0.f;
        if (vec) {
            const float4* w4 = (const float4*)w;
            const float4* x4 = (const float4*)xs;
            const int n4 = d >> 2;
            int k = lane;
            for (; k + 32 < n4; k += 64) {
                const float4 a = w4[k], b = w4[k + 32];
                const float4 xa = x4[k], xb = x4[k + 32];
                s0 = fmaf(xa.x, a.x, s0); s0 = fmaf(xa.y, a.y, s0); s0 = fmaf(xa.z, a.z, s0); s0 = fmaf(xa.w, a.w, s0);
                s1 = fmaf(xb.x, b.x, s1); s1 = fmaf(xb.y, b.y, s1); s1 = fmaf(xb.z, b.z, s1); s1 = fmaf(xb.w, b.w, s1);
            }
            for (; k < n4; k += 32) {
                const float4 a = w4[k];
                const float4 xa = x4[k];
                s0 = fmaf(xa.x, a.x, s0); s0 = fmaf(xa.y, a.y, s0); s0 = fmaf(xa.z, a.z, s0); s0 = fmaf(xa.w, a.w, s0);
            }
        } else {
            for (int k = lane; k < d; k += 32) s0 = fmaf(xs[k], w[k], s0);
        }
        const float sum = warp_sum(s0 + s1);
        if (lane == 0) {
            lg[e] = sum;
            if (logits_out) logits_out[(size_t)t * n_experts + e] = sum;
        }
    }
    __syncthreads();
    if (warp != 0) return;
    for (int slot = 0; slot < top_k; ++slot) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32) {
            const float v = lg[e];
            if (v > best || (v == best && e < best_e)) { best = v; best_e = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
        }
        if (best_e == 0x7fffffff) best_e = 0;                // all logits NaN: still a valid id
        if (lane == 0) {
            expert_ids[(size_t)slot * n_tokens + t] = best_e;
            weights[(size_t)slot * n_tokens + t] = 1.0f / (1.0f + expf(-best));
            lg[best_e] = -INFINITY;
        }
        __syncwarp();
    }
}

// grid top_k, block 1024: block `slot` sorts the tokens by their slot-th expert.
__global__ void __launch_bounds__(1024) sort_by_expert_kernel(const int* __restrict__ expert_ids, int n_tokens,
                                                              int n_experts, int top_k,
                                                              int* __restrict__ offsets,
                                                              int* __restrict__ sorted_rows) {
    __shared__ int counts[MAX_EXPERTS + 1];
    pdl_wait();
    pdl_launch_dependents();
    const int slot = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int t = threadIdx.x; t < n_tokens; t += blockDim.x)
        atomicAdd(&counts[expert_ids[(size_t)slot * n_tokens + t] + 1], 1);
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
            const bool mine = t < n_tokens && expert_ids[(size_t)slot * n_tokens + t] == e;
            const unsigned mask = __ballot_sync(0xffffffffu, mine);
            if (mine) rows[base + __popc(mask & ((1u << lane) - 1u))] = t;
            base += __popc(mask);
        }
    }
}

}  // namespace

SPITE_API int spite_moe_route(int dtype, const void* x, const float* w_router, int n_tokens, int d,
                              int n_experts, int top_k, int* expert_ids, float* weights,
                              float* logits_out, int* offsets, int* sorted_rows, void* stream) {
    if (!x || !w_router || !expert_ids || !weights || !offsets || !sorted_rows) return SPITE_BAD_ARG;
    if (n_tokens < 0 || d <= 0 || n_experts < 1 || top_k < 1 || top_k > n_experts) return SPITE_BAD_ARG;
    if (n_experts > MAX_EXPERTS) return SPITE_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    if (n_tokens > 0) {
        const size_t smem = ((size_t)((d + 3) & ~3) + n_experts) * sizeof(float);
        if (smem > 200 * 1024) return SPITE_UNSUPPORTED;
        cudaError_t attr = cudaSuccess;
        if (dtype == SPITE_DT_F32) {
            if (smem > 48 * 1024)
                attr = cudaFuncSetAttribute(route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (attr != cudaSuccess) return SPITE_LAUNCH_FAILED;
            SPITE_LAUNCH(route_kernel<float>, n_tokens, 256, smem, st, (const float*)x, w_router, n_tokens, d, n_experts,
                         top_k, expert_ids, weights, logits_out);
        } else if (dtype == SPITE_DT_BF16) {
            if (smem > 48 * 1024)
                attr = cudaFuncSetAttribute(route_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (attr != cudaSuccess) return SPITE_LAUNCH_FAILED;
            SPITE_LAUNCH(route_kernel<__nv_bfloat16>, n_tokens, 256, smem, st, (const __nv_bfloat16*)x, w_router, n_tokens, d,
                         n_experts, top_k, expert_ids, weights, logits_out);
        } else {
            return SPITE_BAD_ARG;
        }
        if (cudaGetLastError() != cudaSuccess) return SPITE_LAUNCH_FAILED;
    }
    SPITE_LAUNCH(sort_by_expert_kernel, top_k, 1024, 0, st, (const int*)expert_ids, n_tokens, n_experts, top_k, offsets,
                 sorted_rows);
    return spite_launch_status();
}
