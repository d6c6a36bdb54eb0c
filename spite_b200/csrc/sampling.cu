// Token sampling on the device.  A row of logits is worked on by a cluster of eight blocks that keep
// it in their shared memory (an eighth each; distributed shared memory carries the sums between them),
// so the twenty to forty passes of the pipeline below read shared memory, not L2; a row too long for
// that (more than 8 x 49,152 logits) is worked on by one block through a scratch row in global memory.
//
// The pipeline and its order are those of giveen/spite's sampler
// (crates/spite-sampling/src/lib.rs:273-296): repetition penalty over the distinct
// tokens of the trailing context (lib.rs:208-231), temperature (117-125), min-p
// (178-189), top-k (128-143), top-p (146-174), then the argmax when temperature <= 0
// (236-243; of equal maxima the highest index wins, as Rust's `max_by` returns the
// last) or a multinomial draw against unnormalised masses exp(l - max) with the
// 64-bit LCG of lib.rs:343-348 (first index whose running sum reaches u * total,
// 247-265).  Sums are float32 and are added in a fixed order (a thread's elements, the threads of
// a warp, the warps of a block, the blocks of a cluster by rank), so a row's result does not depend on
// the other rows or on timing.
#include "common.cuh"

namespace {

constexpr int THREADS = 1024;

__device__ __forceinline__ unsigned order_key(float v) {
    const unsigned u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < (THREADS >> 5) ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Largest index holding the maximum (argmax with ties to the highest index).
__device__ int block_argmax_last(const float* l, int n, float* fscratch, int* iscratch) {
    float best = -INFINITY;
    int idx = -1;
    for (int i = threadIdx.x; i < n; i += THREADS) {
        const float v = l[i];
        if (v > best || (v == best && i > idx) || idx < 0) { best = v; idx = i; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (oi >= 0 && (idx < 0 || ov > best || (ov == best && oi > idx))) { best = ov; idx = oi; }
    }
    __syncthreads();
    if (lane == 0) { fscratch[warp] = best; iscratch[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        best = lane < (THREADS >> 5) ? fscratch[lane] : -INFINITY;
        idx = lane < (THREADS >> 5) ? iscratch[lane] : -1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (oi >= 0 && (idx < 0 || ov > best || (ov == best && oi > idx))) { best = ov; idx = oi; }
        }
        if (lane == 0) iscratch[32] = idx;
    }
    __syncthreads();
    return iscratch[32];
}

// First index i (ascending) at which the running sum of f(0..i) reaches `target`;
// -1 if it never does.  Every thread owns a contiguous range of indices.
template <typename F>
__device__ int block_first_reaching(int n, float target, F f, float* fscratch, int* iscratch) {
    const int chunk = (n + THREADS - 1) / THREADS;
    const int lo = min(n, (int)threadIdx.x * chunk), hi = min(n, lo + chunk);
    float mine = 0.f;
    for (int i = lo; i < hi; ++i) mine += f(i);
    // exclusive scan of the per-thread sums: within a warp by shuffles, across warps serially
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    __syncthreads();
    if (lane == 31) fscratch[warp] = incl;
    if (threadIdx.x == 0) iscratch[32] = 0x7fffffff;
    __syncthreads();
    float before = 0.f;
    for (int w = 0; w < warp; ++w) before += fscratch[w];
    float run = before + (incl - mine);
    if (threadIdx.x == 0 || run < target) {
        // the crossing may lie in this range: walk it
        for (int i = lo; i < hi; ++i) {
            run += f(i);
            if (run >= target) { atomicMin(&iscratch[32], i); break; }
        }
    } else if (lo < hi) {
        // the sum before this range has reached the target already; if rounding kept the
        // owner of the crossing from seeing it, this range's first index stands in
        atomicMin(&iscratch[32], lo);
    }
    __syncthreads();
    const int r = iscratch[32];
    __syncthreads();
    return r == 0x7fffffff ? -1 : r;
}

struct SampleParams {
    const float* logits;          // [rows, vocab], not modified
    float* work;                  // [rows, vocab] scratch
    const float* temperature;     // per row; <= 0: argmax
    const int* top_k;             // per row; 0: off
    const float* top_p;           // per row; >= 1: off
    const float* min_p;           // per row; <= 0: off
    const float* repetition_penalty;  // per row; 1: off
    const int* context;           // tokens of all rows, row r at [context_offsets[r], context_offsets[r+1])
    const int* context_offsets;   // the window (`repeat_last_n`) is applied by the caller
    unsigned long long* rng_state;    // per row, advanced once per multinomial draw
    int* out_tokens;              // [rows]
    int vocab;
};

__global__ void __launch_bounds__(THREADS) sample_kernel(const SampleParams p) {
    __shared__ float fs[33];
    __shared__ int is[33];
    __shared__ int hist[256];
    const int r = blockIdx.x;
    const int V = p.vocab;
    const float* in = p.logits + (size_t)r * V;
    float* l = p.work + (size_t)r * V;
    const float T = p.temperature[r];

    for (int i = threadIdx.x; i < V; i += THREADS) l[i] = in[i];
    __syncthreads();
    const float pen = p.repetition_penalty ? p.repetition_penalty[r] : 1.f;
    if (fabsf(pen - 1.f) >= 1.1920929e-07f && p.context) {
        // every occurrence writes the same function of the unmodified logit
        for (int i = p.context_offsets[r] + threadIdx.x; i < p.context_offsets[r + 1]; i += THREADS) {
            const int tok = p.context[i];
            if (tok >= 0 && tok < V) { const float v = in[tok]; l[tok] = v > 0.f ? v / pen : v * pen; }
        }
        __syncthreads();
    }
    if (T > 0.f)
        for (int i = threadIdx.x; i < V; i += THREADS) l[i] = l[i] / T;
    __syncthreads();

    const float minp = p.min_p ? p.min_p[r] : 0.f;
    if (minp > 0.f) {
        float mx = -INFINITY;
        for (int i = threadIdx.x; i < V; i += THREADS) mx = fmaxf(mx, l[i]);
        mx = block_max(mx, fs);
        const float thresh = mx + logf(minp);
        for (int i = threadIdx.x; i < V; i += THREADS) if (l[i] < thresh) l[i] = -INFINITY;
        __syncthreads();
    }

    const int k = p.top_k ? p.top_k[r] : 0;
    if (k > 0 && k < V) {
        // k-th largest key by radix selection, 8 bits a pass
        unsigned prefix = 0, mask = 0;
        int remaining = k;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = threadIdx.x; b < 256; b += THREADS) hist[b] = 0;
            __syncthreads();
            for (int i = threadIdx.x; i < V; i += THREADS) {
                const unsigned key = order_key(l[i]);
                if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255], 1);
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                int b = 255, rem = remaining;
                for (; b > 0; --b) { if (hist[b] >= rem) break; rem -= hist[b]; }
                is[0] = b; is[1] = rem;
            }
            __syncthreads();
            prefix |= (unsigned)is[0] << shift;
            mask |= 255u << shift;
            remaining = is[1];
            __syncthreads();
        }
        for (int i = threadIdx.x; i < V; i += THREADS) if (order_key(l[i]) < prefix) l[i] = -INFINITY;
        __syncthreads();
    }

    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += THREADS) mx = fmaxf(mx, l[i]);
    mx = block_max(mx, fs);

    const float topp = p.top_p ? p.top_p[r] : 1.f;
    if (topp < 1.f && mx > -INFINITY) {
        float tot = 0.f;
        for (int i = threadIdx.x; i < V; i += THREADS) tot += expf(l[i] - mx);
        tot = block_sum(tot, fs);
        const float want = topp * tot;
        // largest key K with mass(key >= K) >= want, by bisection on the key bits
        unsigned K = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = K | (1u << bit);
            float m = 0.f;
            for (int i = threadIdx.x; i < V; i += THREADS) if (order_key(l[i]) >= cand) m += expf(l[i] - mx);
            m = block_sum(m, fs);
            if (m >= want) K = cand;
        }
        float above = 0.f, tie_mass = 0.f, ties = 0.f;
        for (int i = threadIdx.x; i < V; i += THREADS) {
            const unsigned key = order_key(l[i]);
            if (key > K) above += expf(l[i] - mx);
            else if (key == K) { ties += 1.f; tie_mass = expf(l[i] - mx); }
        }
        above = block_sum(above, fs);
        ties = block_sum(ties, fs);
        tie_mass = block_max(tie_mass, fs);
        // of equal logits at the cut, the sorted order keeps the lower indices first
        float keep = tie_mass > 0.f ? ceilf((want - above) / tie_mass) : ties;
        keep = fminf(fmaxf(keep, 1.f), ties);
        int last_tie = V;
        if (keep < ties) {
            auto is_tie = [&](int i) { return order_key(l[i]) == K ? 1.f : 0.f; };
            last_tie = block_first_reaching(V, keep, is_tie, fs, is);
        }
        for (int i = threadIdx.x; i < V; i += THREADS) {
            const unsigned key = order_key(l[i]);
            if (key < K || (key == K && i > last_tie)) l[i] = -INFINITY;
        }
        __syncthreads();
    }

    int token;
    if (T <= 0.f) {
        token = block_argmax_last(l, V, fs, is);
    } else {
        unsigned long long s = p.rng_state[r];
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        const float u = (float)(s >> 33) / 2147483648.0f;
        float tot = 0.f;
        for (int i = threadIdx.x; i < V; i += THREADS) tot += expf(l[i] - mx);
        tot = block_sum(tot, fs);
        const float target = u * tot;
        auto mass = [&](int i) { return expf(l[i] - mx); };
        token = block_first_reaching(V, target, mass, fs, is);
        if (token < 0) token = block_argmax_last(l, V, fs, is);
        if (threadIdx.x == 0) p.rng_state[r] = s;
    }
    if (threadIdx.x == 0) p.out_tokens[r] = token;
}

// ---------------------------------------------------------------------------------
// The same pipeline with a row spread over a cluster of CL blocks.  Block `rank` holds the elements
// [rank * per, rank * per + per) of the row in shared memory.  Whatever the blocks must agree on goes
// through `Shared::pub`: every block publishes one value (or its histogram), the cluster meets at a
// barrier, every block reads all CL values through distributed shared memory and combines them in
// rank order.  Two sets of slots are used in turn, so one barrier per exchange is enough: a block
// that writes a set again has passed the barrier of the exchange between, which every block reaches
// only after it has read the set.
// ---------------------------------------------------------------------------------
constexpr int CL = 8;
constexpr int CLUSTER_MAX_PER_BLOCK = 49152;                 // floats of a row a block can hold (192 KiB)

__device__ __forceinline__ unsigned cl_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cl_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ unsigned cl_load_u32(const void* own_smem, unsigned rank) {
    unsigned addr = (unsigned)__cvta_generic_to_shared(own_smem), remote, v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(addr), "r"(rank));
    asm volatile("ld.shared::cluster.u32 %0, [%1];\n" : "=r"(v) : "r"(remote) : "memory");
    return v;
}

struct ClusterShared {
    float fs[33];
    int is[33];
    unsigned pub[2][2];           // two sets of two published words (a value, an index)
    int hist[256];
    int hist_pub[2][256];
    int turn;                     // which set the next exchange uses (the same in every block)
};

// Every thread of every block gets the CL published words `which` (0 or 1) of all blocks, rank order, in out[].
__device__ __forceinline__ void cl_exchange(ClusterShared& sh, unsigned mine0, unsigned mine1, unsigned (&out0)[CL],
                                            unsigned (&out1)[CL]) {
    const int t = sh.turn;
    __syncthreads();                                         // everyone has read `turn` (and the last results)
    if (threadIdx.x == 0) { sh.pub[t][0] = mine0; sh.pub[t][1] = mine1; sh.turn = t ^ 1; }
    cl_sync();
#pragma unroll
    for (int r = 0; r < CL; ++r) { out0[r] = cl_load_u32(&sh.pub[t][0], r); out1[r] = cl_load_u32(&sh.pub[t][1], r); }
}
__device__ __forceinline__ float cl_sum(ClusterShared& sh, float block_value) {
    unsigned a[CL], b[CL];
    cl_exchange(sh, __float_as_uint(block_value), 0u, a, b);
    float v = 0.f;
#pragma unroll
    for (int r = 0; r < CL; ++r) v += __uint_as_float(a[r]);
    return v;
}
__device__ __forceinline__ float cl_max(ClusterShared& sh, float block_value) {
    unsigned a[CL], b[CL];
    cl_exchange(sh, __float_as_uint(block_value), 0u, a, b);
    float v = -INFINITY;
#pragma unroll
    for (int r = 0; r < CL; ++r) v = fmaxf(v, __uint_as_float(a[r]));
    return v;
}
__device__ __forceinline__ int cl_min_int(ClusterShared& sh, int block_value) {
    unsigned a[CL], b[CL];
    cl_exchange(sh, (unsigned)block_value, 0u, a, b);
    int v = 0x7fffffff;
#pragma unroll
    for (int r = 0; r < CL; ++r) v = min(v, (int)a[r]);
    return v;
}

// Sum over the block (every thread receives it), in the order of block_sum.
__device__ __forceinline__ float csum(ClusterShared& sh, float v) { return block_sum(v, sh.fs); }

// First global index (ascending) at which the running sum of f over the whole row reaches `target`; -1 if never.
// `n` elements of this block start at global index `lo`; every thread owns a contiguous range.
template <typename F>
__device__ int cl_first_reaching(ClusterShared& sh, int n, int lo_global, float target, F f) {
    const int chunk = (n + THREADS - 1) / THREADS;
    const int lo = min(n, (int)threadIdx.x * chunk), hi = min(n, lo + chunk);
    float mine = 0.f;
    for (int i = lo; i < hi; ++i) mine += f(i);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    __syncthreads();
    if (lane == 31) sh.fs[warp] = incl;
    __syncthreads();
    float before = 0.f, block_total = 0.f;
    for (int w = 0; w < (THREADS >> 5); ++w) { if (w < warp) before += sh.fs[w]; block_total += sh.fs[w]; }
    // the sums of the blocks before this one, in rank order
    unsigned a[CL], b[CL];
    cl_exchange(sh, __float_as_uint(block_total), 0u, a, b);
    float base = 0.f;
    const unsigned rank = cl_rank();
#pragma unroll
    for (int r = 0; r < CL; ++r) if ((unsigned)r < rank) base += __uint_as_float(a[r]);
    __syncthreads();
    if (threadIdx.x == 0) sh.is[32] = 0x7fffffff;
    __syncthreads();
    float run = base + before + (incl - mine);
    if ((rank == 0 && threadIdx.x == 0) || run < target) {
        for (int i = lo; i < hi; ++i) {                      // the crossing may lie in this range: walk it
            run += f(i);
            if (run >= target) { atomicMin(&sh.is[32], lo_global + i); break; }
        }
    } else if (lo < hi) {
        // the sum before this range has reached the target already; if rounding kept the owner of the
        // crossing from seeing it, this range's first index stands in
        atomicMin(&sh.is[32], lo_global + lo);
    }
    __syncthreads();
    const int r = cl_min_int(sh, sh.is[32]);
    return r == 0x7fffffff ? -1 : r;
}

__global__ void __launch_bounds__(THREADS) sample_cluster_kernel(const SampleParams p, const int per) {
    extern __shared__ float l[];                             // this block's part of the row
    __shared__ ClusterShared sh;
    const unsigned rank = cl_rank();
    const int r = blockIdx.x / CL;
    const int V = p.vocab;
    const int lo = (int)rank * per, n = max(0, min(per, V - lo));
    const float* in = p.logits + (size_t)r * V;
    const float T = p.temperature[r];
    if (threadIdx.x == 0) sh.turn = 0;

    for (int i = threadIdx.x; i < n; i += THREADS) l[i] = in[lo + i];
    __syncthreads();
    const float pen = p.repetition_penalty ? p.repetition_penalty[r] : 1.f;
    if (fabsf(pen - 1.f) >= 1.1920929e-07f && p.context) {
        // every occurrence writes the same function of the unmodified logit
        for (int i = p.context_offsets[r] + threadIdx.x; i < p.context_offsets[r + 1]; i += THREADS) {
            const int tok = p.context[i];
            if (tok >= lo && tok < lo + n) { const float v = in[tok]; l[tok - lo] = v > 0.f ? v / pen : v * pen; }
        }
        __syncthreads();
    }
    if (T > 0.f)
        for (int i = threadIdx.x; i < n; i += THREADS) l[i] = l[i] / T;
    __syncthreads();

    auto row_max = [&]() {
        float mx = -INFINITY;
        for (int i = threadIdx.x; i < n; i += THREADS) mx = fmaxf(mx, l[i]);
        return cl_max(sh, block_max(mx, sh.fs));
    };

    const float minp = p.min_p ? p.min_p[r] : 0.f;
    if (minp > 0.f) {
        const float thresh = row_max() + logf(minp);
        for (int i = threadIdx.x; i < n; i += THREADS) if (l[i] < thresh) l[i] = -INFINITY;
        __syncthreads();
    }

    const int k = p.top_k ? p.top_k[r] : 0;
    if (k > 0 && k < V) {
        // k-th largest key by radix selection, 8 bits a pass; the histograms of the blocks are added
        unsigned prefix = 0, mask = 0;
        int remaining = k;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = threadIdx.x; b < 256; b += THREADS) sh.hist[b] = 0;
            __syncthreads();
            for (int i = threadIdx.x; i < n; i += THREADS) {
                const unsigned key = order_key(l[i]);
                if ((key & mask) == prefix) atomicAdd(&sh.hist[(key >> shift) & 255], 1);
            }
            __syncthreads();
            const int t = sh.turn;
            for (int b = threadIdx.x; b < 256; b += THREADS) sh.hist_pub[t][b] = sh.hist[b];
            __syncthreads();
            if (threadIdx.x == 0) sh.turn = t ^ 1;
            cl_sync();
            for (int b = threadIdx.x; b < 256; b += THREADS) {
                int total = 0;
#pragma unroll
                for (int q = 0; q < CL; ++q) total += (int)cl_load_u32(&sh.hist_pub[t][b], q);
                sh.hist[b] = total;
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                int b = 255, rem = remaining;
                for (; b > 0; --b) { if (sh.hist[b] >= rem) break; rem -= sh.hist[b]; }
                sh.is[0] = b; sh.is[1] = rem;
            }
            __syncthreads();
            prefix |= (unsigned)sh.is[0] << shift;
            mask |= 255u << shift;
            remaining = sh.is[1];
            __syncthreads();
        }
        for (int i = threadIdx.x; i < n; i += THREADS) if (order_key(l[i]) < prefix) l[i] = -INFINITY;
        __syncthreads();
    }

    const float mx = row_max();

    const float topp = p.top_p ? p.top_p[r] : 1.f;
    if (topp < 1.f && mx > -INFINITY) {
        float tot = 0.f;
        for (int i = threadIdx.x; i < n; i += THREADS) tot += expf(l[i] - mx);
        tot = cl_sum(sh, csum(sh, tot));
        const float want = topp * tot;
        // largest key K with mass(key >= K) >= want, by bisection on the key bits
        unsigned K = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = K | (1u << bit);
            float m = 0.f;
            for (int i = threadIdx.x; i < n; i += THREADS) if (order_key(l[i]) >= cand) m += expf(l[i] - mx);
            m = cl_sum(sh, csum(sh, m));
            if (m >= want) K = cand;
        }
        float above = 0.f, tie_mass = 0.f, ties = 0.f;
        for (int i = threadIdx.x; i < n; i += THREADS) {
            const unsigned key = order_key(l[i]);
            if (key > K) above += expf(l[i] - mx);
            else if (key == K) { ties += 1.f; tie_mass = expf(l[i] - mx); }
        }
        above = cl_sum(sh, csum(sh, above));
        ties = cl_sum(sh, csum(sh, ties));
        tie_mass = cl_max(sh, block_max(tie_mass, sh.fs));
        // of equal logits at the cut, the sorted order keeps the lower indices first
        float keep = tie_mass > 0.f ? ceilf((want - above) / tie_mass) : ties;
        keep = fminf(fmaxf(keep, 1.f), ties);
        int last_tie = V;
        if (keep < ties) {
            auto is_tie = [&](int i) { return order_key(l[i]) == K ? 1.f : 0.f; };
            last_tie = cl_first_reaching(sh, n, lo, keep, is_tie);
        }
        for (int i = threadIdx.x; i < n; i += THREADS) {
            const unsigned key = order_key(l[i]);
            if (key < K || (key == K && lo + i > last_tie)) l[i] = -INFINITY;
        }
        __syncthreads();
    }

    auto row_argmax_last = [&]() {
        int idx = block_argmax_last(l, n, sh.fs, sh.is);         // -1 if this block holds nothing
        const float best = idx >= 0 ? l[idx] : -INFINITY;
        unsigned a[CL], b[CL];
        cl_exchange(sh, __float_as_uint(best), (unsigned)(idx >= 0 ? lo + idx : -1), a, b);
        float bv = -INFINITY;
        int bi = -1;
#pragma unroll
        for (int q = 0; q < CL; ++q) {                           // ties go to the highest index: later ranks win
            const float v = __uint_as_float(a[q]);
            const int i = (int)b[q];
            if (i >= 0 && (bi < 0 || v >= bv)) { bv = v; bi = i; }
        }
        return bi;
    };

    int token;
    if (T <= 0.f) {
        token = row_argmax_last();
    } else {
        unsigned long long s = p.rng_state[r];
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        const float u = (float)(s >> 33) / 2147483648.0f;
        float tot = 0.f;
        for (int i = threadIdx.x; i < n; i += THREADS) tot += expf(l[i] - mx);
        tot = cl_sum(sh, csum(sh, tot));
        const float target = u * tot;
        auto mass = [&](int i) { return expf(l[i] - mx); };
        token = cl_first_reaching(sh, n, lo, target, mass);
        if (token < 0) token = row_argmax_last();
        cl_sync();                                               // every block has read the state before it changes
        if (rank == 0 && threadIdx.x == 0) p.rng_state[r] = s;
    }
    if (rank == 0 && threadIdx.x == 0) p.out_tokens[r] = token;
    cl_sync();                                                   // no block leaves while another may still read its shared memory
}

__global__ void __launch_bounds__(THREADS) argmax_kernel(const float* logits, int vocab, int* out) {
    __shared__ float fs[33];
    __shared__ int is[33];
    const int idx = block_argmax_last(logits + (size_t)blockIdx.x * vocab, vocab, fs, is);
    if (threadIdx.x == 0) out[blockIdx.x] = idx;
}

// The same with a row spread over a cluster of CL blocks, an eighth each: one block alone reads a row of
// 202,048 logits in 25 us, which a decode step of one request would wait for.  The blocks' results meet in
// block 0 through distributed shared memory, in rank order, with the same rule for equal values.
__global__ void __launch_bounds__(THREADS) argmax_cluster_kernel(const float* logits, int vocab, int per, int* out) {
    __shared__ float fs[33];
    __shared__ int is[33];
    __shared__ unsigned pub[2];
    const unsigned rank = cl_rank();
    const int row = blockIdx.x / CL;
    const float* l = logits + (size_t)row * vocab;
    const int lo = min(vocab, (int)rank * per), n = min(vocab, lo + per) - lo;
    const int mine = n > 0 ? block_argmax_last(l + lo, n, fs, is) : -1;
    if (threadIdx.x == 0) {
        pub[0] = __float_as_uint(mine >= 0 ? l[lo + mine] : -INFINITY);
        pub[1] = (unsigned)(mine >= 0 ? lo + mine : -1);
    }
    cl_sync();
    if (rank == 0 && threadIdx.x == 0) {
        float best = -INFINITY;
        int idx = -1;
        for (unsigned r = 0; r < CL; ++r) {
            const float ov = __uint_as_float(cl_load_u32(&pub[0], r));
            const int oi = (int)cl_load_u32(&pub[1], r);
            if (oi >= 0 && (idx < 0 || ov > best || (ov == best && oi > idx))) { best = ov; idx = oi; }
        }
        out[row] = idx;
    }
    cl_sync();                                                   // no block leaves while block 0 may still read its shared memory
}

}  // namespace

SPITE_API int spite_argmax(const float* logits, int rows, int vocab, int* out, void* stream) {
    if (!logits || !out || rows < 0 || vocab < 1) return SPITE_BAD_ARG;
    if (rows == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (vocab >= 16384 && rows <= 0x7fffffff / CL) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)rows * CL);
        cfg.blockDim = dim3(THREADS);
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = CL;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        (void)cudaLaunchKernelEx(&cfg, argmax_cluster_kernel, logits, vocab, (vocab + CL - 1) / CL, out);
        return spite_launch_status();
    }
    argmax_kernel<<<rows, THREADS, 0, st>>>(logits, vocab, out);
    return spite_launch_status();
}

// Both entry points launch through here, so they give the same tokens: a cluster of eight blocks per row where
// a row fits their shared memory (`p.work` is not touched then), else one block per row on `p.work`.
static int launch_sample(const SampleParams& p, int rows, cudaStream_t st) {
    int per = ((p.vocab + CL - 1) / CL + 31) / 32 * 32;
    if (per <= CLUSTER_MAX_PER_BLOCK && rows <= 0x7fffffff / CL) {
        const size_t smem = (size_t)per * sizeof(float);
        if (cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return SPITE_LAUNCH_FAILED;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)rows * CL);
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = CL;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        (void)cudaLaunchKernelEx(&cfg, sample_cluster_kernel, p, per);
        return spite_launch_status();
    }
    sample_kernel<<<rows, THREADS, 0, st>>>(p);
    return spite_launch_status();
}

SPITE_API int spite_sample(const SampleParams* p, int rows, void* stream) {
    if (!p || !p->logits || !p->work || !p->temperature || !p->rng_state || !p->out_tokens) return SPITE_BAD_ARG;
    if (rows < 0 || p->vocab < 1) return SPITE_BAD_ARG;
    if (p->context && !p->context_offsets) return SPITE_BAD_ARG;
    if (rows == 0) return SPITE_OK;
    return launch_sample(*p, rows, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------
// spite_sample_noalloc: the same kernel with its scratch rows in a fixed array of
// this library instead of memory the caller allocates.  See sampling_noalloc.h for
// who needs this, the size limit, and the rules on sharing and on the first call.
// ---------------------------------------------------------------------------------
#include "sampling_noalloc.h"
#include <atomic>

// Scratch of the no-allocation entry point.  In host code this name is only a handle
// for cudaGetSymbolAddress; it is never passed to a kernel as if it were a pointer.
static __device__ __align__(256) float g_sample_noalloc_scratch[SPITE_SAMPLE_NOALLOC_MAX_FLOATS];

namespace {

constexpr int NOALLOC_MAX_DEVICES = 64;
// device address of the array, per device; atomic, since the first calls of two host threads may both look it
// up (they store the same value)
std::atomic<float*> g_noalloc_scratch_addr[NOALLOC_MAX_DEVICES] = {};

// The device address of the scratch array on the current device; looked up once per
// device with that device current.  Returns null if the runtime refuses.
float* noalloc_scratch_for_current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) return nullptr;
    float* ptr = g_noalloc_scratch_addr[dev].load(std::memory_order_acquire);
    if (!ptr) {
        if (cudaGetSymbolAddress((void**)&ptr, g_sample_noalloc_scratch) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        g_noalloc_scratch_addr[dev].store(ptr, std::memory_order_release);
    }
    return ptr;
}

}  // namespace

SPITE_API int spite_sample_noalloc(const SpiteSampleNoAllocArgs* a, void* stream) {
    if (!a || !a->logits || !a->temperature || !a->rng_state || !a->out_tokens) return SPITE_BAD_ARG;
    if (a->rows < 0 || a->vocab < 1) return SPITE_BAD_ARG;
    if (a->context && !a->context_offsets) return SPITE_BAD_ARG;
    if ((long long)a->rows * (long long)a->vocab > (long long)SPITE_SAMPLE_NOALLOC_MAX_FLOATS)
        return SPITE_UNSUPPORTED;                            // beyond the fixed scratch: nothing runs
    if (a->rows == 0) return SPITE_OK;
    float* scratch = noalloc_scratch_for_current_device();
    if (!scratch) return SPITE_LAUNCH_FAILED;
    SampleParams p;
    p.logits = a->logits;
    p.work = scratch;                                        // every element is written before it is read
    p.temperature = a->temperature;
    p.top_k = a->top_k;
    p.top_p = a->top_p;
    p.min_p = a->min_p;
    p.repetition_penalty = a->repetition_penalty;
    p.context = a->context;
    p.context_offsets = a->context_offsets;
    p.rng_state = a->rng_state;
    p.out_tokens = a->out_tokens;
    p.vocab = a->vocab;
    return launch_sample(p, a->rows, (cudaStream_t)stream);
}
