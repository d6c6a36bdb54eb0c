// Grouped matrix product for prompt portions whose groups (experts) have few rows each, on the
// fifth-generation tensor cores with the operands swapped:
//   D[n, t] = sum_k W[g][n, k] X[t, k]        n: 128 weight rows of group g, t: the group's tokens
// The weights are the 128-row operand of tcgen05.mma and the tokens its columns, so a group's token
// count is rounded up to 16 (the granularity of the instruction's N), not to the 128 rows of a
// row tile: with 2,048 tokens over 16 experts (128 +- 11 tokens each) or 4,096 over 128 experts
// (32 each) a tile of 128 token rows is mostly, or half the time, empty, and every empty row costs
// tensor-core time and shared-memory traffic that this product, bound by reading the weights once,
// cannot spare.  In the accumulator a lane is a weight row (an output column) and a column a token,
// so a warp of the epilogue writes 32 consecutive output columns of one token: the scattered
// read-modify-write of the float32 residual rows is whole 128-byte lines.
//
// Persistent blocks (one per multiprocessor) walk items (group with tokens, tile of 128 weight rows),
// weight-row tiles fastest, so the blocks of a round read different weights and share a group's
// tokens through L2.  A group of more tokens than a tile holds (256; 128 for SwiGLU) is cut into
// tiles of equal size that the same block runs one after the other, so that the weight tile's
// second reading comes from L2.  Roles as in gemm_tc.cu:
//   warp 0    one lane issues TMA loads (128-byte swizzle) of the weight tile (for SwiGLU: the gate
//             tile and the matching up tile), 64 k at a time, into a ring of 128 KiB: the weights
//             come from HBM, and what a multiprocessor keeps in flight of them decides the speed;
//   warp 6    one lane does the same for the token tile, into a shorter ring of its own (the
//             tokens come from L2, and a deep ring for them would take the weights' room);
//   warp 1    allocates TMEM; one lane issues tcgen05.mma 128 x (tokens rounded up to 16) x 16;
//   warps 2-5 read an accumulator with tcgen05.ld (one weight row per thread, 32 tokens at a
//             time) and apply the epilogue while the tensor cores fill the other accumulator.
// Epilogues: add to the float32 residual stream scattered through c_rows (down product, up to 256
// tokens a tile), SwiGLU with a per-token scale (gate/up product, up to 128 tokens a tile).
// Every wait is bounded as in gemm_tc.cu; spite_gemm_tc_experts_error() reads the code.
//
// Rows of A are contiguous in group order (the caller gathers them); `a_rows`, if set, only
// indexes `row_scale`.  Edges in K are covered by TMA's zero fill, edges in N and in the tokens by
// bounds checks on stores (rows a tile reads beyond its group's are computed and dropped).
#include "gemm.cuh"
#include "tcgen05.cuh"

namespace {
using namespace tc;

constexpr int BM = 128, BK = 64, UMMA_K = 16;
constexpr int W_BYTES = BM * BK * 2;                     // 16 KiB: one tile of weight rows
constexpr int XBOX = 64, XBOX_BYTES = XBOX * BK * 2;     // tokens come in boxes of 64 rows, 8 KiB
constexpr int W_RING_BYTES = 128 * 1024, MAX_W_STAGES = 8;
constexpr int X_RING_BYTES = 80 * 1024, MAX_X_STAGES = 4;
constexpr int ACC_COLS = 256, TMEM_COLS = 512;
constexpr int THREADS = 224;
constexpr int MAX_LISTED = 512;                          // groups with tokens, kept as a list in shared memory

__device__ int g_experts_error = 0;
}  // namespace
// 1: loader waited for a free stage, 2: tensor-core issue waited for a stage, 3: epilogue waited
// for an accumulator, 4: tensor-core issue waited for a free accumulator.  (`extra_tx` is not used here.)
SPITE_WAIT_CONTROLS(gemm_tc_experts, g_experts_error)
namespace {

struct SharedTail {
    unsigned long long w_full[MAX_W_STAGES], w_empty[MAX_W_STAGES];
    unsigned long long x_full[MAX_X_STAGES], x_empty[MAX_X_STAGES];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];
    unsigned tmem_base;
    int abort_flag;
    int n_active;                                        // groups that have tokens
    int max_tokens;                                      // most tokens of a token tile (rounded up to 16)
    int g_id[MAX_LISTED], g_lo[MAX_LISTED], g_hi[MAX_LISTED];
};

struct Item {
    int group, lo, hi, n0;          // the group, its rows in group order, the first weight row of the tile
    int n_tt, per;                  // its token tiles and the tokens of each (a multiple of 16; the last may have fewer)
};

// TOK_MAX: most tokens of a tile (256; 128 for SwiGLU, which keeps two accumulators per tile).
template <int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_experts_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                       const GemmParams p, const WaitControl waits) {
    constexpr bool DUAL = (EPI == EPI_SWIGLU);
    constexpr int TOK_MAX = DUAL ? 128 : 256;
    constexpr int WT_BYTES = (DUAL ? 2 : 1) * W_BYTES;          // weight bytes of a stage
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* x_ring = smem + W_RING_BYTES;
    SharedTail* tail = (SharedTail*)(smem + W_RING_BYTES + X_RING_BYTES);
    pdl_wait();
    pdl_launch_dependents();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (p.K + BK - 1) / BK;
    const int w_rows = DUAL ? 2 * p.N : p.N;                  // weight rows of one group
    const int r_tiles = (p.N + BM - 1) / BM;                  // tiles of 128 weight rows (output columns)
    volatile int* abort_flag = &tail->abort_flag;
    int* const err_word = waits.error_word ? waits.error_word : &g_experts_error;
    const long long wait_limit = waits.limit_cycles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < MAX_W_STAGES; ++s) { mbar_init(smem_u32(&tail->w_full[s]), 1); mbar_init(smem_u32(&tail->w_empty[s]), 1); }
        for (int s = 0; s < MAX_X_STAGES; ++s) { mbar_init(smem_u32(&tail->x_full[s]), 1); mbar_init(smem_u32(&tail->x_empty[s]), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(smem_u32(&tail->acc_full[b]), 1); mbar_init(smem_u32(&tail->acc_empty[b]), 4); }
        tail->abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc(&tail->tmem_base, TMEM_COLS);
    if (warp == 2) {
        // the groups that have tokens, in group order: 32 groups at a time, places by a ballot
        int n = 0, most = 0;
        for (int g0 = 0; g0 < p.n_groups; g0 += 32) {
            const int g = g0 + lane;
            int lo = 0, hi = 0;
            if (g < p.n_groups) { lo = p.group_offsets[g]; hi = p.group_offsets[g + 1]; }
            const unsigned has = __ballot_sync(0xffffffffu, hi > lo);
            if (hi > lo) {
                const int at = n + __popc(has & ((1u << lane) - 1u));
                tail->g_id[at] = g; tail->g_lo[at] = lo; tail->g_hi[at] = hi;
                const int n_tt = (hi - lo + TOK_MAX - 1) / TOK_MAX;
                most = max(most, ((hi - lo + n_tt - 1) / n_tt + 15) / 16 * 16);
            }
            n += __popc(has);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) most = max(most, __shfl_xor_sync(0xffffffffu, most, o));
        if (lane == 0) { tail->n_active = n; tail->max_tokens = max(16, most); }
    }
    fence_before();
    __syncthreads();
    fence_after();
    const unsigned tmem = tail->tmem_base;
    const int total = tail->n_active * r_tiles;
    // a stage of the token ring holds as many boxes of 64 tokens as the largest token tile needs
    const int x_stage = (tail->max_tokens + XBOX - 1) / XBOX * XBOX_BYTES;
    const int nx = min(MAX_X_STAGES, X_RING_BYTES / x_stage);
    constexpr int nw = W_RING_BYTES / WT_BYTES;

    auto item_at = [&](int idx) {
        Item it;
        const int slot = idx / r_tiles;
        it.n0 = (idx % r_tiles) * BM;
        it.group = tail->g_id[slot]; it.lo = tail->g_lo[slot]; it.hi = tail->g_hi[slot];
        it.n_tt = (it.hi - it.lo + TOK_MAX - 1) / TOK_MAX;
        it.per = ((it.hi - it.lo + it.n_tt - 1) / it.n_tt + 15) / 16 * 16;
        return it;
    };
    // token tile j of an item: its first row, its tokens, and the instruction's N (tokens rounded up to 16)
    auto tokens_of = [&](const Item& it, int j, int& row0, int& rows, int& nt) {
        row0 = it.lo + j * it.per;
        rows = max(0, min(it.per, it.hi - row0));
        nt = max(16, (rows + 15) / 16 * 16);
    };

    if (warp == 0) {
        if (lane == 0) {
            // ---- weight loader.  The weights are read once (they should leave L2 first), unless the same block
            //      reads the tile again for the group's next token tile.
            const unsigned long long w_policy = l2_evict_first();
            int issued = 0, s = 0;
            unsigned ph = 0;
            bool ok = true;
            for (int idx = blockIdx.x; idx < total && ok; idx += gridDim.x) {
                const Item it = item_at(idx);
                const int wy = it.group * w_rows + it.n0;
                for (int j = 0; j < it.n_tt && ok; ++j) {
                    int row0, rows, nt;
                    tokens_of(it, j, row0, rows, nt);
                    if (rows == 0) continue;
                    const bool again = j + 1 < it.n_tt;
                    for (int kb = 0; kb < num_kb; ++kb, ++issued, s = (s + 1 == nw ? 0 : s + 1), ph ^= (s == 0)) {
                        ok = mbar_wait(smem_u32(&tail->w_empty[s]), ph ^ 1, abort_flag, err_word, 1, wait_limit);
                        if (!ok) break;
                        const unsigned bar = smem_u32(&tail->w_full[s]);
                        const unsigned dst = smem_u32(smem + (size_t)s * WT_BYTES);
                        mbar_expect_tx(bar, WT_BYTES);
                        if (again) {
                            tma_load_2d(dst, &map_w, kb * BK, wy, bar);
                            if (DUAL) tma_load_2d(dst + W_BYTES, &map_w, kb * BK, wy + p.N, bar);
                        } else {
                            tma_load_2d_hint(dst, &map_w, kb * BK, wy, bar, w_policy);
                            if (DUAL) tma_load_2d_hint(dst + W_BYTES, &map_w, kb * BK, wy + p.N, bar, w_policy);
                        }
                    }
                }
            }
            if (*abort_flag) {
                // copies in flight must land before the block gives its shared memory back
                for (int j = max(0, issued - nw); j < issued; ++j)
                    mbar_drain(smem_u32(&tail->w_full[j % nw]), (j / nw) & 1, wait_limit);
            }
        }
    } else if (warp == 6) {
        if (lane == 0) {
            // ---- token loader: the token tile of every k block, read by every weight-row tile of the group (from L2)
            int issued = 0, s = 0;
            unsigned ph = 0;
            bool ok = true;
            for (int idx = blockIdx.x; idx < total && ok; idx += gridDim.x) {
                const Item it = item_at(idx);
                for (int j = 0; j < it.n_tt && ok; ++j) {
                    int row0, rows, nt;
                    tokens_of(it, j, row0, rows, nt);
                    if (rows == 0) continue;
                    const int x_boxes = (nt + XBOX - 1) / XBOX;
                    for (int kb = 0; kb < num_kb; ++kb, ++issued, s = (s + 1 == nx ? 0 : s + 1), ph ^= (s == 0)) {
                        ok = mbar_wait(smem_u32(&tail->x_empty[s]), ph ^ 1, abort_flag, err_word, 1, wait_limit);
                        if (!ok) break;
                        const unsigned bar = smem_u32(&tail->x_full[s]);
                        const unsigned dst = smem_u32(x_ring + (size_t)s * x_stage);
                        mbar_expect_tx(bar, x_boxes * XBOX_BYTES);
                        for (int xb = 0; xb < x_boxes; ++xb)
                            tma_load_2d(dst + xb * XBOX_BYTES, &map_x, kb * BK, row0 + xb * XBOX, bar);
                    }
                }
            }
            if (*abort_flag) {
                for (int j = max(0, issued - nx); j < issued; ++j)
                    mbar_drain(smem_u32(&tail->x_full[j % nx]), (j / nx) & 1, wait_limit);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- tensor-core issue
            int lt = 0, sw = 0, sx = 0;
            unsigned phw = 0, phx = 0;
            bool ok = true;
            for (int idx = blockIdx.x; idx < total && ok; idx += gridDim.x) {
                const Item it = item_at(idx);
                for (int j = 0; j < it.n_tt && ok; ++j) {
                    int row0, rows, nt;
                    tokens_of(it, j, row0, rows, nt);
                    if (rows == 0) continue;
                    const unsigned idesc = make_idesc(BM, nt);
                    const int buf = lt & 1;
                    ok = mbar_wait(smem_u32(&tail->acc_empty[buf]), ((lt >> 1) & 1) ^ 1, abort_flag, err_word, 4, wait_limit);
                    if (!ok) break;
                    fence_after();
                    const unsigned d_tmem = tmem + buf * ACC_COLS;
                    for (int kb = 0; kb < num_kb; ++kb, sw = (sw + 1 == nw ? 0 : sw + 1), phw ^= (sw == 0),
                                                        sx = (sx + 1 == nx ? 0 : sx + 1), phx ^= (sx == 0)) {
                        ok = mbar_wait(smem_u32(&tail->x_full[sx]), phx, abort_flag, err_word, 2, wait_limit) &&
                             mbar_wait(smem_u32(&tail->w_full[sw]), phw, abort_flag, err_word, 2, wait_limit);
                        if (!ok) break;
                        fence_after();
                        const unsigned w_addr = smem_u32(smem + (size_t)sw * WT_BYTES);
                        const unsigned x_addr = smem_u32(x_ring + (size_t)sx * x_stage);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            const unsigned acc = (kb > 0 || k > 0) ? 1u : 0u;
                            const unsigned long long xd = smem_desc_k_major(x_addr + k * UMMA_K * 2);
                            mma(d_tmem, smem_desc_k_major(w_addr + k * UMMA_K * 2), xd, idesc, acc);
                            if (DUAL) mma(d_tmem + TOK_MAX, smem_desc_k_major(w_addr + W_BYTES + k * UMMA_K * 2), xd, idesc, acc);
                        }
                        commit(smem_u32(&tail->w_empty[sw]));   // both stages are free once these MMAs have read them
                        commit(smem_u32(&tail->x_empty[sx]));
                    }
                    if (ok) commit(smem_u32(&tail->acc_full[buf]));   // this accumulator is complete
                    ++lt;
                }
            }
        }
    } else {
        // ---- epilogue: warp w may read TMEM lanes [32 (w % 4), 32 (w % 4) + 32): weight rows n0 + 32 (w % 4) + lane
        const int quarter = warp & 3;
        int lt = 0;
        bool ok = true;
        for (int idx = blockIdx.x; idx < total && ok; idx += gridDim.x) {
          const Item item = item_at(idx);
          for (int j = 0; j < item.n_tt && ok; ++j) {
            struct { int row0, rows, nt, n0; } it;
            tokens_of(item, j, it.row0, it.rows, it.nt);
            it.n0 = item.n0;
            if (it.rows == 0) continue;
            const int buf = lt & 1;
            ok = mbar_wait(smem_u32(&tail->acc_full[buf]), (lt >> 1) & 1, abort_flag, err_word, 3, wait_limit);
            if (!ok) break;
            fence_after();
            const unsigned lane_addr = tmem + buf * ACC_COLS + ((unsigned)(quarter * 32) << 16);
            const int n = it.n0 + quarter * 32 + lane;          // this thread's output column
            const bool n_ok = n < p.N;
#pragma unroll 1
            for (int c0 = 0; c0 < it.nt; c0 += 32) {
                float v[32];
                ld32(v, lane_addr + c0);                        // warp-collective: every lane takes part
                // lane i looks up what token c0 + i needs; the values go round by shuffle
                const int li = it.row0 + c0 + lane;
                const bool t_ok = c0 + lane < it.rows;
                if (DUAL) {
                    float u[32];
                    ld32(u, lane_addr + TOK_MAX + c0);
                    float sc = 1.f;
                    if (t_ok && p.row_scale) sc = p.row_scale[(p.scale_by_a_row && p.a_rows) ? p.a_rows[li] : li];
                    __nv_bfloat16* out = (__nv_bfloat16*)p.C + (size_t)(it.row0 + c0) * p.ldc + n;
#pragma unroll
                    for (int t = 0; t < 32; ++t) {
                        const float s = __shfl_sync(0xffffffffu, sc, t);
                        if (c0 + t < it.rows && n_ok) out[(size_t)t * p.ldc] = __float2bfloat16_rn(silu_f32(v[t] * s) * (u[t] * s));
                    }
                } else {
                    int crow = 0;
                    float sc = 1.f;
                    if (t_ok) {
                        crow = p.c_rows ? p.c_rows[li] : li;
                        if (p.row_scale) sc = p.row_scale[(p.scale_by_a_row && p.a_rows) ? p.a_rows[li] : li];
                    }
                    // the old values of all the tokens first, so that their latencies overlap
                    float old[32];
#pragma unroll
                    for (int t = 0; t < 32; ++t) {
                        const int r = __shfl_sync(0xffffffffu, crow, t);
                        old[t] = (EPI == EPI_ADD_F32 && c0 + t < it.rows && n_ok) ? ((const float*)p.C)[(size_t)r * p.ldc + n] : 0.f;
                    }
#pragma unroll
                    for (int t = 0; t < 32; ++t) {
                        const int r = __shfl_sync(0xffffffffu, crow, t);
                        const float s = __shfl_sync(0xffffffffu, sc, t);
                        if (c0 + t < it.rows && n_ok) {
                            const float y = old[t] + v[t] * s;
                            if (EPI == EPI_STORE) ((__nv_bfloat16*)p.C)[(size_t)r * p.ldc + n] = __float2bfloat16_rn(y);
                            else ((float*)p.C)[(size_t)r * p.ldc + n] = y;
                        }
                    }
                }
            }
            // this warp has read its lanes of the accumulator: hand it back to the tensor cores
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tail->acc_empty[buf]));
            ++lt;
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

template <int EPI>
int launch(const GemmParams& p, int n_blocks, cudaStream_t st) {
    constexpr bool DUAL = (EPI == EPI_SWIGLU);
    const long long w_rows = (long long)(DUAL ? 2 : 1) * p.N * p.n_groups;
    CUtensorMap mx, mw;
    {
        cuuint64_t dims[2] = {(cuuint64_t)p.K, (cuuint64_t)p.M};
        cuuint64_t strides[1] = {(cuuint64_t)p.lda * 2};
        cuuint32_t box[2] = {BK, XBOX};
        if (!make_map(&mx, p.A, 2, dims, strides, box)) return SPITE_LAUNCH_FAILED;
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)p.K, (cuuint64_t)w_rows};
        cuuint64_t strides[1] = {(cuuint64_t)p.K * 2};
        cuuint32_t box[2] = {BK, BM};
        if (!make_map(&mw, p.W, 2, dims, strides, box)) return SPITE_LAUNCH_FAILED;
    }
    const size_t smem = (size_t)W_RING_BYTES + X_RING_BYTES + sizeof(SharedTail) + 1024;
    auto k = gemm_tc_experts_kernel<EPI>;
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return SPITE_LAUNCH_FAILED;
    SPITE_LAUNCH(k, n_blocks, THREADS, smem, st, mx, mw, p, s_waits);
    return spite_launch_status();
}

}  // namespace

// A grouped product (`group_offsets` set) with the SwiGLU epilogue or the add into the float32 residual
// stream (optionally scattered through `c_rows`).  `n_blocks`: number of multiprocessors (one persistent
// block each).  Groups of any size are taken (a large group is cut into token tiles and its weights
// are then read once per tile: the caller sends such products to the kernels with 128-row tiles).
SPITE_API int spite_gemm_tc_experts(const GemmParams* p, int n_blocks, void* stream) {
    if (!p || !p->A || !p->W || !p->C) return SPITE_BAD_ARG;
    if (p->M < 0 || p->N <= 0 || p->K <= 0 || p->lda < p->K || p->ldc < p->N || n_blocks < 1) return SPITE_BAD_ARG;
    if (!p->group_offsets || p->n_groups < 1) return SPITE_BAD_ARG;
    if (p->epilogue < 0 || p->epilogue > EPI_SWIGLU) return SPITE_BAD_ARG;
    if (p->epilogue != EPI_SWIGLU && p->epilogue != EPI_ADD_F32) return SPITE_UNSUPPORTED;
    // TMA: 16-byte aligned bases and row pitches
    if (p->K % 8 || p->lda % 8 || (((uintptr_t)p->A | (uintptr_t)p->W) & 15)) return SPITE_UNSUPPORTED;
    if (p->w_group_stride != (long long)(p->epilogue == EPI_SWIGLU ? 2 : 1) * p->N * p->K)
        return SPITE_UNSUPPORTED;                              // groups must be stacked without gaps
    if (p->n_groups > MAX_LISTED) return SPITE_UNSUPPORTED;    // the groups with tokens are listed in shared memory
    if (p->M == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    return p->epilogue == EPI_SWIGLU ? launch<EPI_SWIGLU>(*p, n_blocks, st) : launch<EPI_ADD_F32>(*p, n_blocks, st);
}
