// Matrix product for the few tokens of a decode step, weights streamed through shared memory by TMA:
//   y[M, N] = epilogue( x[M, K] W[N, K]^T ),  at most 16 rows per group (32 for a one-group product),
//   bfloat16 inputs, float32 sums.
//
// With few tokens the product is bound by reading W once from HBM, and what decides the speed is how
// many bytes a multiprocessor keeps in flight and how quickly the stream starts again after the
// kernel before.  Here a producer warp keeps a ring of shared-memory stages full: per stage one TMA
// box of 128 weight rows x 64 k (128-byte swizzle; for SwiGLU 64 gate and 64 up rows) and the
// matching 64 k of the group's tokens (cp.async, same swizzle).  Eight consumer warps own 16 of the
// 128 rows each and multiply with mma.sync.m16n8k16 (weights as the 16-row operand from ldmatrix,
// tokens as the 8, 16 or 32 columns), so no sums cross warps.  Registers stay few, and two blocks (of this
// kernel, or the last of this and the first of the next) share a multiprocessor.
//
// Work items are (group with tokens, tile of weight rows, k split); blocks are persistent and
// take items with a stride of the grid, the ring running on across items.
//
// A product with few output rows (an output projection: 5120) has too few tiles of 128 rows for
// the resident blocks.  Two ways to more items, both chosen by the caller.  k slices inside the block
// (S = 2, 4, 8): a stage holds S boxes of 128/S rows x 64 k, S k blocks side by side, and the warps
// are 8/S row groups x S slices; a tile has 128/S rows and the slices' sums meet in shared memory
// when the item ends, in the order of the slices: no traffic, no waiting for another block.  And k
// splits across blocks: the partial tiles go through a float32 scratch in global memory, and the block
// that arrives last at the tile's ticket adds them in the order of the splits (a fence, an atomic and
// a second pass: about 2.7 us an item); or, with up to eight splits and one block per (tile, split),
// the splits of a tile are one thread-block cluster and their sums land in its first block's shared
// memory between two cluster barriers.  Every way a sum's order does not depend on timing.
// A one-group product knows its items without the step's earlier kernels: its producer requests the
// first weights before griddepcontrol.wait.
// (Dealing every block one equal run of k blocks across tile borders was measured too: faster alone,
// 219 against 248 us for 8 tokens over 7 experts, and no faster in the decode step, where blocks that
// finish early make room for the next kernel's blocks to start and fetch.)
#include "gemm.cuh"
#include "tcgen05.cuh"
#include <map>
#include <mutex>
#include <tuple>

namespace {
using namespace tc;

constexpr int ROWS = 128, BK = 64;                      // weight rows and k of a stage's boxes together: 128 x 64 elements
constexpr int W_BYTES = ROWS * BK * 2;                  // 16 KiB a stage, however it is cut
constexpr int CONSUMERS = 8;                            // warps; warp CONSUMERS is the producer
constexpr int THREADS = (CONSUMERS + 1) * 32;
constexpr int MAX_STAGES = 12;
constexpr int MAX_GROUPS = 1024;

__device__ int g_stream_error = 0;
}  // namespace
// 1: the producer waited for a free stage, 2: a consumer waited for a stage.  (`extra_tx` is not used here.)
SPITE_WAIT_CONTROLS(gemm_stream, g_stream_error)
namespace {

struct Tail {
    unsigned long long full[MAX_STAGES], empty[MAX_STAGES];
    int abort_flag, n_active, last;
    int active[MAX_GROUPS];
};
// After the tail, with k slices: the sums of the warps of slices 1 .. S - 1 on their way to the warps of slice 0,
// [warp - R][lane][NT / 2] floats.
constexpr int slices_bytes(int nt, int s) { return s > 1 ? (CONSUMERS - CONSUMERS / s) * 32 * (nt / 2) * 4 : 0; }

__device__ __forceinline__ void mma16816(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(unsigned& r0, unsigned& r1, unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void cp_async16(unsigned dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
// The mbarrier gets one arrival when this thread's cp.async copies so far have landed.
__device__ __forceinline__ void cp_async_arrive(unsigned bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(CONSUMERS * 32) : "memory"); }
// The same barrier, and whether any consumer thread brought `v`: one answer for all of them.  (The producer
// may raise the abort flag at any moment; consumers that each read it for themselves could disagree, and those
// that stay would wait at the next barrier for those that left.)
__device__ __forceinline__ bool consumer_sync_any(bool v) {
    unsigned any;
    asm volatile("{\n.reg .pred p, q;\nsetp.ne.u32 q, %1, 0;\nbar.red.or.pred p, 1, %2, q;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(any) : "r"((unsigned)v), "n"(CONSUMERS * 32) : "memory");
    return any != 0;
}

__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// Four floats into the shared memory of the cluster's block `rank`, at the place `own` has in this block's.
__device__ __forceinline__ void cluster_store4(const void* own, unsigned rank, const float (&v)[4]) {
    unsigned addr = (unsigned)__cvta_generic_to_shared(own), remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(addr), "r"(rank));
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"r"(remote), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]) : "memory");
}

struct Item {
    int group, lo, m;             // group, its first row in the sorted order, its tokens
    int tile, n0;                 // tile id (group slot x row tiles + row tile) and first output column
    int split, kb0, kb1;          // k split and its range of stages (64 S wide each)
};

// NT: token columns (8, 16 or 32).  S: k slices inside the block.  `n_splits` k splits per tile; `scratch` holds
// tiles x n_splits x NT x (128 / S) floats, `tickets` one zeroed int per tile (left zeroed).
// CL (with S = 1): the k splits of a tile are the blocks of one thread-block cluster, the grid has one block per
// (tile, split), and the splits' sums meet in the shared memory of the cluster's first block instead of in
// global memory: no scratch, no fence, no ticket, no second pass through L2.
template <int NT, int EPI, int S, bool CL>
__global__ void __launch_bounds__(THREADS, NT <= 16 ? 3 : 2)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const GemmParams p, const int n_stages,
                   const int n_splits, float* __restrict__ scratch, int* __restrict__ tickets, const WaitControl waits) {
    constexpr bool DUAL = (EPI == EPI_SWIGLU);
    constexpr int TR = ROWS / S;                                 // weight rows of a tile
    constexpr int R = CONSUMERS / S;                             // row groups of 16 (SwiGLU: 8 gate + 8 up) rows
    constexpr int COLS = DUAL ? TR / 2 : TR;                     // output columns of a tile
    constexpr int BOX_BYTES = TR * BK * 2;                       // one slice's weights
    constexpr int X_BYTES = NT * BK * 2;                         // one slice's tokens: 1 or 2 KiB
    constexpr int STAGE = W_BYTES + (S * X_BYTES < 1024 ? 1024 : S * X_BYTES);
    constexpr int NB = NT / 8;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    Tail* tail = (Tail*)(smem + (size_t)n_stages * STAGE);
    float* const slice_sums = (float*)(tail + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool grouped = p.group_offsets != nullptr;
    const int row_tiles = (p.N + COLS - 1) / COLS;
    const int num_kb = p.K / (BK * S);                        // stages along k
    const int w_rows = DUAL ? 2 * p.N : p.N;
    volatile int* abort_flag = &tail->abort_flag;
    int* const err_word = waits.error_word ? waits.error_word : &g_stream_error;
    const long long wait_limit = waits.limit_cycles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < n_stages; ++s) { mbar_init(smem_u32(&tail->full[s]), 33); mbar_init(smem_u32(&tail->empty[s]), CONSUMERS); }
        tail->abort_flag = 0;
        mbar_init_fence();
    }
    const unsigned long long w_policy = l2_evict_first();   // weights are read once a step: they should not push the tokens and the cache out of L2
    // A one-group product's first item is known now: request its first weights before waiting for
    // the kernels before (weights are written by no kernel of the step).
    int pre = 0;
    if (!grouped) {
        __syncthreads();
        if (warp == CONSUMERS && lane == 0 && (int)blockIdx.x < row_tiles * n_splits) {
            const int i = blockIdx.x;
            const int split = i % n_splits, rt = i / n_splits;
            const int kb0 = (int)((long long)num_kb * split / n_splits), kb1 = (int)((long long)num_kb * (split + 1) / n_splits);
            pre = min(n_stages, kb1 - kb0);
            for (int j = 0; j < pre; ++j) {
                const unsigned bar = smem_u32(&tail->full[j]), dst = smem_u32(smem + j * STAGE);
                mbar_expect_tx(bar, W_BYTES);
#pragma unroll
                for (int sl = 0; sl < S; ++sl) {
                    const int kx = ((kb0 + j) * S + sl) * BK;
                    if (DUAL) {
                        tma_load_2d_hint(dst + sl * BOX_BYTES, &map_w, kx, rt * COLS, bar, w_policy);
                        tma_load_2d_hint(dst + sl * BOX_BYTES + BOX_BYTES / 2, &map_w, kx, p.N + rt * COLS, bar, w_policy);
                    } else {
                        tma_load_2d_hint(dst + sl * BOX_BYTES, &map_w, kx, rt * COLS, bar, w_policy);
                    }
                }
            }
        }
    }
    pdl_wait();
    pdl_launch_dependents();

    // groups that have tokens, in group order
    if (warp == 0) {
        int n = 0;
        const int groups = grouped ? p.n_groups : 1;
        for (int e0 = 0; e0 < groups; e0 += 32) {
            const int e = e0 + lane;
            const int m = e < groups ? (grouped ? p.group_offsets[e + 1] - p.group_offsets[e] : p.M) : 0;
            const unsigned has = __ballot_sync(0xffffffffu, m > 0);
            if (m > 0) tail->active[n + __popc(has & ((1u << lane) - 1u))] = e;
            n += __popc(has);
        }
        if (lane == 0) tail->n_active = n;
    }
    __syncthreads();
    const int total = tail->n_active * row_tiles * n_splits;

    auto item_at = [&](int i) {
        Item it;
        it.split = i % n_splits;
        const int rt = (i / n_splits) % row_tiles, slot = i / (n_splits * row_tiles);
        it.group = tail->active[slot];
        it.lo = grouped ? p.group_offsets[it.group] : 0;
        it.m = min(NT, (grouped ? p.group_offsets[it.group + 1] : p.M) - it.lo);
        it.tile = slot * row_tiles + rt;
        it.n0 = rt * COLS;
        it.kb0 = (int)((long long)num_kb * it.split / n_splits);
        it.kb1 = (int)((long long)num_kb * (it.split + 1) / n_splits);
        return it;
    };

    if (warp == CONSUMERS) {
        // ---- producer
        int s = 0;
        unsigned ph = 0;
        int skip_tma = __shfl_sync(0xffffffffu, pre, 0);         // stages whose weights are on the way already
        bool ok = true;
        const __nv_bfloat16* X = (const __nv_bfloat16*)p.A;
        for (int i = blockIdx.x; i < total && ok; i += gridDim.x) {
            const Item it = item_at(i);
            // this lane's 16-byte chunks of a slice's token tile: chunk q = lane + 32 j, token q / 8, k chunk q % 8.
            // Up to 16 tokens their places are worked out once an item; with more (one-group products only, rows
            // in place) they are cheap enough to work out again for every stage, and sixteen pointers would
            // cost every thread of the block their registers.
            constexpr int KEPT = NT <= 16 ? NT / 4 : 1;
            const __nv_bfloat16* src[KEPT];
            unsigned off[KEPT];
            if (NT <= 16) {
#pragma unroll
                for (int j = 0; j < KEPT; ++j) {
                    const int q = lane + 32 * j, t = q >> 3, c = q & 7;
                    const int li = it.lo + min(t, it.m - 1);     // rows past the group's tokens repeat its last one; never stored
                    src[j] = X + (size_t)(p.a_rows ? p.a_rows[li] : li) * p.lda + c * 8;
                    off[j] = W_BYTES + t * 128 + ((c ^ (t & 7)) << 4);
                }
            }
            const int wy = it.group * w_rows + it.n0;
            for (int kb = it.kb0; kb < it.kb1; ++kb, s = (s + 1 == n_stages ? 0 : s + 1), ph ^= (s == 0)) {
                if (lane == 0) ok = mbar_wait(smem_u32(&tail->empty[s]), ph ^ 1, abort_flag, err_word, 1, wait_limit);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                const unsigned bar = smem_u32(&tail->full[s]), dst = smem_u32(smem + s * STAGE);
                if (skip_tma > 0) {
                    --skip_tma;
                } else if (lane == 0) {
                    mbar_expect_tx(bar, W_BYTES);
#pragma unroll
                    for (int sl = 0; sl < S; ++sl) {
                        const int kx = (kb * S + sl) * BK;
                        if (DUAL) {
                            tma_load_2d_hint(dst + sl * BOX_BYTES, &map_w, kx, wy, bar, w_policy);
                            tma_load_2d_hint(dst + sl * BOX_BYTES + BOX_BYTES / 2, &map_w, kx, wy + p.N, bar, w_policy);
                        } else {
                            tma_load_2d_hint(dst + sl * BOX_BYTES, &map_w, kx, wy, bar, w_policy);
                        }
                    }
                }
                if (NT <= 16) {
#pragma unroll
                    for (int sl = 0; sl < S; ++sl)
#pragma unroll
                        for (int j = 0; j < KEPT; ++j)
                            cp_async16(dst + sl * X_BYTES + off[j], src[j] + ((size_t)kb * S + sl) * BK);
                } else {
                    const int c = lane & 7;
#pragma unroll
                    for (int sl = 0; sl < S; ++sl)
#pragma unroll 4
                        for (int j = 0; j < NT / 4; ++j) {
                            const int t = (lane >> 3) + 4 * j;
                            const int li = it.lo + min(t, it.m - 1);
                            cp_async16(dst + sl * X_BYTES + W_BYTES + t * 128 + ((c ^ (t & 7)) << 4),
                                       X + (size_t)li * p.lda + c * 8 + ((size_t)kb * S + sl) * BK);
                        }
                }
                cp_async_arrive(bar);
            }
        }
        asm volatile("cp.async.wait_all;\n" ::: "memory");
        if (CL && (int)blockIdx.x < total) { cluster_sync(); cluster_sync(); }     // with the consumers, see below
    } else {
        // ---- consumers: warp w works on slice w / R; it owns rows 16 r .. 16 r + 15 (r = w % R) of the tile
        //      (SwiGLU: gate rows 8 r .. + 7 and the up rows of the same output columns as fragment rows 8 .. 15)
        const int g = lane >> 2, c = lane & 3;
        const int rg = warp % R, slice = warp / R;
        const int mrow = (lane & 7) + ((lane >> 3) & 1) * 8;     // fragment row this lane addresses for ldmatrix
        const int arow = DUAL ? (mrow < 8 ? 8 * rg + mrow : TR / 2 + 8 * rg + mrow - 8) : 16 * rg + mrow;
        const unsigned a_off = slice * BOX_BYTES + arow * 128, a_swz = arow & 7, a_k = lane >> 4;
        const int brow = lane & 7;
        const unsigned b_k = (lane >> 3) & 1;
        int s = 0;
        unsigned ph = 0;
        bool ok = true;
        for (int i = blockIdx.x; i < total; i += gridDim.x) {
            const Item it = item_at(i);
            float acc[NB][4];
#pragma unroll
            for (int j = 0; j < NB; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
            for (int kb = it.kb0; kb < it.kb1; ++kb, s = (s + 1 == n_stages ? 0 : s + 1), ph ^= (s == 0)) {
                ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&tail->full[s]), ph, abort_flag, err_word, 2, wait_limit));
                if (!ok) break;
                const unsigned wbase = smem_u32(smem + s * STAGE), xbase = wbase + W_BYTES + slice * X_BYTES;
#pragma unroll
                for (int ks = 0; ks < BK / 16; ++ks) {
                    unsigned a[4];
                    ldmatrix_x4(a, wbase + a_off + (((2 * ks + a_k) ^ a_swz) << 4));
#pragma unroll
                    for (int j = 0; j < NB; ++j) {
                        const int t = 8 * j + brow;
                        unsigned b0, b1;
                        ldmatrix_x2(b0, b1, xbase + t * 128 + (((2 * ks + b_k) ^ (t & 7)) << 4));
                        mma16816(acc[j], a, b0, b1);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&tail->empty[s]));
            }
            // A warp whose wait ran out leaves at once only if the epilogue has no block-wide steps; else it
            // goes through this item's barriers with the others (storing nothing) and all leave together.
            if (!ok && n_splits == 1 && S == 1) break;

            // ---- the k slices' sums meet in the warps of slice 0, in the order of the slices
            if (S > 1) {
                consumer_sync();                              // the sums of the item before have been read
                if (slice > 0) {
#pragma unroll
                    for (int j = 0; j < NB; ++j)
#pragma unroll
                        for (int e = 0; e < 4; ++e) slice_sums[((warp - R) * 32 + lane) * (4 * NB) + 4 * j + e] = acc[j][e];
                }
                const bool stop = consumer_sync_any(*abort_flag != 0);
                if (slice == 0) {
#pragma unroll
                    for (int sl = 1; sl < S; ++sl)
#pragma unroll
                        for (int j = 0; j < NB; ++j)
#pragma unroll
                            for (int e = 0; e < 4; ++e) acc[j][e] += slice_sums[(((sl - 1) * R + rg) * 32 + lane) * (4 * NB) + 4 * j + e];
                }
                if (n_splits == 1 && stop) break;             // the same answer in every warp
            }
            const bool writer = slice == 0;

            // ---- epilogue.  This lane holds, for token 8 j + 2 c + (e & 1), fragment rows g (e < 2) and g + 8.
            auto finish = [&](int t, int col, float v, float v2) {      // output column n0 + col of token t
                const int n = it.n0 + col;
                if (t >= it.m || n >= p.N) return;
                const int li = it.lo + t;
                const int ar = p.a_rows ? p.a_rows[li] : li;
                const int crow = p.c_rows ? p.c_rows[li] : li;
                const float sc = p.row_scale ? p.row_scale[p.scale_by_a_row ? ar : li] : 1.f;
                const size_t o = (size_t)crow * p.ldc + n;
                if (EPI == EPI_STORE) ((__nv_bfloat16*)p.C)[o] = __float2bfloat16_rn(v * sc);
                else if (EPI == EPI_STORE_F32) ((float*)p.C)[o] = v * sc;
                else if (EPI == EPI_ADD_F32) ((float*)p.C)[o] += v * sc;
                else ((__nv_bfloat16*)p.C)[o] = __float2bfloat16_rn(silu_f32(v * sc) * (v2 * sc));
            };
            if (CL) {
                // the k loops of all the cluster's blocks have ended (the first block's ring is free: the others'
                // sums land there); then the first block adds them in the order of the splits
                float* const landing = (float*)smem;              // [split - 1][warp][lane][4 NB]
                cluster_sync();
                const unsigned rank = cluster_rank();
                if (rank > 0 && ok) {
#pragma unroll
                    for (int j = 0; j < NB; ++j)
                        cluster_store4(landing + ((((size_t)rank - 1) * CONSUMERS + warp) * 32 + lane) * (4 * NB) + 4 * j, 0, acc[j]);
                }
                cluster_sync();
                if (rank == 0) {
                    for (int sp = 1; sp < n_splits; ++sp)
#pragma unroll
                        for (int j = 0; j < NB; ++j)
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                acc[j][e] += landing[((((size_t)sp - 1) * CONSUMERS + warp) * 32 + lane) * (4 * NB) + 4 * j + e];
                }
            }
            if (n_splits == 1 || CL) {
                if (writer && (!CL || cluster_rank() == 0)) {
#pragma unroll
                    for (int j = 0; j < NB; ++j)
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int t = 8 * j + 2 * c + e;
                            if (DUAL) {
                                finish(t, 8 * rg + g, acc[j][e], acc[j][e + 2]);
                            } else {
                                finish(t, 16 * rg + g, acc[j][e], 0.f);
                                finish(t, 16 * rg + g + 8, acc[j][e + 2], 0.f);
                            }
                        }
                }
                continue;
            }
            // partial tile: scratch[tile][split][token][tile row]; tile rows of the SwiGLU form: gate rows, then up rows
            float* part = scratch + ((size_t)it.tile * n_splits + it.split) * NT * TR;
            const int r_lo = DUAL ? 8 * rg + g : 16 * rg + g;
            const int r_hi = DUAL ? TR / 2 + 8 * rg + g : 16 * rg + g + 8;
            if (writer) {
#pragma unroll
                for (int j = 0; j < NB; ++j)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int t = 8 * j + 2 * c + e;
                        if (t < it.m && ok) {
                            __stcg(part + t * TR + r_lo, acc[j][e]);
                            __stcg(part + t * TR + r_hi, acc[j][e + 2]);
                        }
                    }
            }
            consumer_sync();
            if (threadIdx.x == 0) {
                __threadfence();                              // after the barrier: it covers what the other threads stored
                const int arrived = atomicAdd(&tickets[it.tile], 1);
                tail->last = (arrived == n_splits - 1);
                if (tail->last) tickets[it.tile] = 0;
            }
            consumer_sync();
            if (tail->last) {
                __threadfence();
                const float* all = scratch + (size_t)it.tile * n_splits * NT * TR;
                for (int idx = threadIdx.x; idx < COLS * it.m; idx += CONSUMERS * 32) {
                    const int col = idx % COLS, t = idx / COLS;
                    float v = 0.f, v2 = 0.f;
                    // eight splits' loads are on their way together: a loop whose length the compiler does not know
                    // would wait for every load (a trip to L2, often the other die's) before it asks for the next
                    for (int sp0 = 0; sp0 < n_splits; sp0 += 8) {
                        float a[8], b[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const bool in = sp0 + j < n_splits;
                            const float* from = all + ((size_t)(sp0 + j) * NT + t) * TR + col;
                            a[j] = in ? __ldcg(from) : 0.f;
                            b[j] = DUAL && in ? __ldcg(from + TR / 2) : 0.f;
                        }
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            v += a[j];
                            if (DUAL) v2 += b[j];
                        }
                    }
                    finish(t, col, v, v2);
                }
            }
            if (consumer_sync_any(*abort_flag != 0)) break;   // (`last` is read before the next item writes it)
            ok = true;
        }
    }
}

template <int NT, int EPI, int S, bool CL>
int launch(const GemmParams& p, int n_blocks, int smem_budget, int n_splits, float* scratch, int* tickets, cudaStream_t st) {
    constexpr bool DUAL = (EPI == EPI_SWIGLU);
    constexpr int TR = ROWS / S;
    constexpr int X_BYTES = NT * BK * 2;
    constexpr int STAGE = W_BYTES + (S * X_BYTES < 1024 ? 1024 : S * X_BYTES);
    const long long w_rows = (long long)(DUAL ? 2 : 1) * p.N * p.n_groups;
    CUtensorMap mw;
    cuuint64_t dims[2] = {(cuuint64_t)p.K, (cuuint64_t)w_rows};
    cuuint64_t strides[1] = {(cuuint64_t)p.K * 2};
    cuuint32_t box[2] = {BK, (cuuint32_t)(DUAL ? TR / 2 : TR)};
    if (!make_map(&mw, p.W, 2, dims, strides, box)) return SPITE_LAUNCH_FAILED;
    constexpr int FIXED = (int)sizeof(Tail) + slices_bytes(NT, S) + 1024;
    int n_stages = (smem_budget - FIXED) / STAGE;
    if (n_stages > MAX_STAGES) n_stages = MAX_STAGES;
    if (n_stages < 2) return SPITE_UNSUPPORTED;                    // (16 tokens x 8 slices are 32 KiB a stage)
    const size_t smem = (size_t)n_stages * STAGE + FIXED;
    auto k = gemm_stream_kernel<NT, EPI, S, CL>;
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
        cudaFuncSetAttribute(k, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess)
        return SPITE_LAUNCH_FAILED;
    const int cols = DUAL ? TR / 2 : TR;
    const long long tiles = (long long)((p.N + cols - 1) / cols) * (p.group_offsets ? (p.n_groups < p.M ? p.n_groups : p.M) : 1) * n_splits;
    if (!CL) {
        const int grid = (int)(tiles < n_blocks ? tiles : n_blocks);
        SPITE_LAUNCH(k, grid, THREADS, smem, st, mw, p, n_stages, n_splits, scratch, tickets, s_waits);
        return spite_launch_status();
    }
    // one block per (tile, split), the splits of a tile one cluster; all of them resident at once, or the caller
    // takes the other way (-2): a second round of clusters would cost more than the cluster saves
    if (n_splits < 2 || n_splits > 8 || tiles > n_blocks) return SPITE_UNSUPPORTED;
    if ((size_t)(n_splits - 1) * CONSUMERS * 32 * (NT / 2) * 4 > (size_t)n_stages * STAGE) return SPITE_UNSUPPORTED;   // the landing place is the ring
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)tiles);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)n_splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // how many clusters of this size are resident at once: asked once per (size, shared memory) and device
    static std::mutex lock;
    static std::map<std::tuple<int, int, size_t>, int> known;
    int fit = 0, dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return SPITE_LAUNCH_FAILED;
    {
        std::lock_guard<std::mutex> hold(lock);
        const auto key = std::make_tuple(dev, n_splits, smem);
        const auto it = known.find(key);
        if (it != known.end()) {
            fit = it->second;
        } else {
            if (cudaOccupancyMaxActiveClusters(&fit, k, &cfg) != cudaSuccess) { (void)cudaGetLastError(); fit = 0; }
            known[key] = fit;
        }
    }
    if ((long long)fit * n_splits < tiles) return SPITE_UNSUPPORTED;
    cfg.numAttrs = spite_pdl_enabled() ? 2 : 1;
    (void)cudaLaunchKernelEx(&cfg, k, mw, p, n_stages, n_splits, scratch, tickets, s_waits);
    return spite_launch_status();
}

template <int NT, int EPI>
int launch_slices(int k_slices, bool cluster, const GemmParams& p, int n_blocks, int smem_budget, int n_splits, float* scratch,
                  int* tickets, cudaStream_t st) {
    if (cluster) {
        if (k_slices != 1) return SPITE_BAD_ARG;
        if (NT > 16) return SPITE_UNSUPPORTED;
        return launch<NT <= 16 ? NT : 8, EPI, 1, true>(p, n_blocks, smem_budget, n_splits, scratch, tickets, st);
    }
    if (NT > 16) {                                             // many tokens: tiles of 128 or 64 rows (more slices, more of a
        switch (k_slices) {                                    // stage would be tokens than weights)
            case 1: return launch<NT, EPI, 1, false>(p, n_blocks, smem_budget, n_splits, scratch, tickets, st);
            case 2: return launch<NT, EPI, 2, false>(p, n_blocks, smem_budget, n_splits, scratch, tickets, st);
            default: return SPITE_UNSUPPORTED;
        }
    }
    switch (k_slices) {
        case 1: return launch<NT, EPI, 1, false>(p, n_blocks, smem_budget, n_splits, scratch, tickets, st);
        case 2: return launch<NT, EPI, 2, false>(p, n_blocks, smem_budget, n_splits, scratch, tickets, st);
        case 4: return launch<NT <= 16 ? NT : 8, EPI, 4, false>(p, n_blocks, smem_budget, n_splits, scratch, tickets, st);
        case 8: return EPI == EPI_SWIGLU ? SPITE_UNSUPPORTED       // (tiles of 8 gate and 8 up rows: nobody needs them)
                                         : launch<NT <= 16 ? NT : 8, EPI == EPI_SWIGLU ? EPI_STORE : EPI, 8, false>(p, n_blocks, smem_budget, n_splits, scratch, tickets, st);
        default: return SPITE_BAD_ARG;
    }
}

}  // namespace

// `max_rows_per_group` <= 16, or <= 32 for a one-group product with its rows in place (with 64 token columns the
// mma.sync path cannot keep up with the stream: 34 to 63 us for Scout's projections against 28 to 41 on tcgen05).
// `k_slices` (1, 2, 4 or 8; 8 not with SwiGLU): a tile has 128 / k_slices weight rows
// (SwiGLU: half of them gate, half up) and K must be a multiple of 64 k_slices.  `n_blocks`: resident blocks
// (two per multiprocessor fit when `smem_budget`, the bytes of shared memory a block may take, is at most about
// 110 KiB, three at 74 KiB).  `n_splits`: k splits per tile across blocks (1: no scratch needed).  `cluster`
// (with k_slices 1 and 2 to 8 splits): the splits of a tile are one thread-block cluster and meet in shared
// memory; needs no scratch and no tickets, and is refused (-2) when the (tile, split) blocks are not all
// resident at once.  `scratch`: groups-with-tokens x row tiles x n_splits x 16 x (128 / k_slices) floats;
// `tickets`: that many tiles' ints, zero before the first call; calls that share them must not overlap.
SPITE_API int spite_gemm_stream(const GemmParams* p, int max_rows_per_group, int k_slices, int cluster, int n_blocks,
                                int smem_budget, int n_splits, float* scratch, long long scratch_floats, int* tickets,
                                int n_tickets, void* stream) {
    if (!p || !p->A || !p->W || !p->C) return SPITE_BAD_ARG;
    if (p->M < 0 || p->N <= 0 || p->K <= 0 || p->lda < p->K || p->ldc < p->N || n_blocks < 1 || n_splits < 1) return SPITE_BAD_ARG;
    if (p->group_offsets ? p->n_groups < 1 : p->n_groups != 1) return SPITE_BAD_ARG;
    if (p->epilogue < 0 || p->epilogue > EPI_SWIGLU) return SPITE_BAD_ARG;
    if (k_slices != 1 && k_slices != 2 && k_slices != 4 && k_slices != 8) return SPITE_BAD_ARG;
    if (p->K % (BK * k_slices) || p->lda % 8 || (((uintptr_t)p->A | (uintptr_t)p->W) & 15)) return SPITE_UNSUPPORTED;
    if (k_slices == 8 && p->epilogue == EPI_SWIGLU) return SPITE_UNSUPPORTED;
    if (max_rows_per_group < 1 || max_rows_per_group > 32 || p->n_groups > MAX_GROUPS) return SPITE_UNSUPPORTED;
    if (max_rows_per_group > 16 && (p->group_offsets || p->a_rows)) return SPITE_UNSUPPORTED;
    if (p->n_groups > 1 && p->w_group_stride != (long long)(p->epilogue == EPI_SWIGLU ? 2 : 1) * p->N * p->K)
        return SPITE_UNSUPPORTED;                              // groups must be stacked without gaps
    if (p->M == 0) return SPITE_OK;
    const int stages_k = p->K / (BK * k_slices);
    if (n_splits > stages_k) n_splits = stages_k;
    const int nt = max_rows_per_group <= 8 ? 8 : max_rows_per_group <= 16 ? 16 : 32;
    const int tr = ROWS / k_slices;
    const int cols = p->epilogue == EPI_SWIGLU ? tr / 2 : tr;
    const long long tiles = (long long)((p->N + cols - 1) / cols) * (p->group_offsets ? (p->n_groups < p->M ? p->n_groups : p->M) : 1);
    if (cluster && (k_slices != 1 || n_splits < 2)) return SPITE_BAD_ARG;
    if (n_splits > 1 && !cluster) {
        if (!scratch || !tickets || tiles > n_tickets || tiles * n_splits * nt * tr > scratch_floats) return SPITE_BAD_ARG;
    }
    cudaStream_t st = (cudaStream_t)stream;
#define SPITE_STREAM_NT(N_, E) launch_slices<N_, E>(k_slices, cluster != 0, *p, n_blocks, smem_budget, n_splits, scratch, tickets, st)
#define SPITE_STREAM_CASE(E)                                                                                              \
    case E:                                                                                                               \
        return nt == 8 ? SPITE_STREAM_NT(8, E) : nt == 16 ? SPITE_STREAM_NT(16, E) : SPITE_STREAM_NT(32, E);
    switch (p->epilogue) {
        SPITE_STREAM_CASE(EPI_STORE)
        SPITE_STREAM_CASE(EPI_STORE_F32)
        SPITE_STREAM_CASE(EPI_ADD_F32)
        default: return nt == 8 ? SPITE_STREAM_NT(8, EPI_SWIGLU) : nt == 16 ? SPITE_STREAM_NT(16, EPI_SWIGLU)
                                                                 : SPITE_STREAM_NT(32, EPI_SWIGLU);
    }
#undef SPITE_STREAM_CASE
#undef SPITE_STREAM_NT
}
