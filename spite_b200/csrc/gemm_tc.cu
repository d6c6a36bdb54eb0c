// Matrix product for many tokens (prefill) on the fifth-generation tensor cores:
//   C[M, N] (=|+=) epilogue( A[M, K] W[N, K]^T ),  bfloat16 inputs, float32 sums in TMEM.
//
// Persistent blocks (one per multiprocessor) walk the output tiles of 128 rows x BN
// columns, BN = 64..256 chosen on the host so that the last wave of tiles is full.  Roles:
//   warp 0    one lane issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of the A
//             tile and the two halves of the W tile of a 64-wide k block into a ring of four to
//             eight shared-memory stages (192 KiB; narrower tiles get more stages);
//   warp 1    allocates TMEM (512 columns: two accumulators of up to 256); one lane issues
//             tcgen05.mma 128 x BN x 16, operands straight from shared memory through matrix
//             descriptors, commits each stage back to the loader and each finished
//             accumulator to the epilogue;
//   warps 2-5 read an accumulator with tcgen05.ld (one row per thread) and apply the
//             epilogue while the tensor cores fill the other accumulator.
// The two halves of the W tile are the next BN/2 output columns, or, for the SwiGLU
// epilogue, BN/2 gate rows and the matching BN/2 up rows; the main loop is the same.
// Epilogues: store, store float32, add to the float32 residual stream (optionally
// scattered through c_rows), SwiGLU with a per-row scale.
//
// Stages, accumulators and roles hand over through mbarriers.  Every wait is bounded:
// after its limit (about two seconds unless spite_gemm_tc_configure_waits says otherwise) a waiter
// raises an abort flag that all roles poll, records an error code (read by spite_gemm_tc_error(),
// or from the word the caller named), waits for its own copies in
// flight, and the block leaves through the common exit, where TMEM is freed.
//
// Rows of A are contiguous (a grouped product gets its rows gathered into expert order
// beforehand); `a_rows`, if set, only indexes `row_scale`.  Edges in M, N and K are
// covered by TMA's zero fill on loads and by bounds checks on stores.
#include "gemm_tc_epilogue.cuh"

namespace {
using namespace tc;

constexpr int BM = 128, BK = 64, UMMA_K = 16, MAX_STAGES = 8;
constexpr int A_BYTES = BM * BK * 2;                     // 16 KiB
constexpr int B_BYTES = 256 * BK * 2;                    // room for 256 weight rows, 32 KiB
constexpr int RING_BYTES = 4 * (A_BYTES + B_BYTES);      // 192 KiB of stages: 4 of the widest tile, up to 8 of narrower ones
constexpr int ACC_COLS = 256, TMEM_COLS = 512;
constexpr int THREADS = 192;
constexpr int MAX_LISTED = 1024;                         // row tiles of a grouped product kept as a list in shared memory

__device__ int g_tc_error = 0;
}  // namespace
// 1: loader waited for a free stage, 2: tensor-core issue waited for a tile, 3: epilogue waited
// for an accumulator, 4: tensor-core issue waited for a free accumulator.
SPITE_WAIT_CONTROLS(gemm_tc, g_tc_error)
namespace {

struct SharedTail {
    unsigned long long full[MAX_STAGES];
    unsigned long long empty[MAX_STAGES];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];
    unsigned tmem_base;
    int abort_flag;
    int n_row_tiles;                                     // row tiles that hold rows (grouped products: counted in the kernel)
    int rt_group[MAX_LISTED], rt_row0[MAX_LISTED], rt_rows[MAX_LISTED];
};

// The tile with running index `idx`: column tile idx / row_tiles, row tile idx % row_tiles.
// A grouped product cuts every group into row tiles of its own.  Their list is built once per
// block in shared memory, so that only tiles that hold rows are dealt out to the blocks; a
// product with more row tiles than the list takes (`listed` false) scans the group offsets instead
// and skips the empty tiles at the end of each column.
struct Tile {
    int group, row0, rows, n0;
    bool ok;
};
__device__ __forceinline__ Tile tile_at(const GemmParams& p, const SharedTail* tail, bool listed, int idx,
                                        int row_tiles, int cols_per_tile) {
    Tile t;
    const int rt = idx % row_tiles;
    t.n0 = (idx / row_tiles) * cols_per_tile;
    if (listed) {
        t.group = tail->rt_group[rt]; t.row0 = tail->rt_row0[rt]; t.rows = tail->rt_rows[rt];
        t.ok = true;
    } else {
        t.ok = locate_row_tile(p, rt, BM, t.group, t.row0, t.rows);
    }
    return t;
}

// `bnh`: weight rows per half of the W tile (32 .. 128 in steps of 16; 32 for SwiGLU); the MMA is 128 x 2 bnh x 16.
template <int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const GemmParams p, const int bnh, const int max_row_tiles, const int col_tiles, const int n_stages,
               const WaitControl waits) {
    constexpr bool DUAL = (EPI == EPI_SWIGLU);
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    SharedTail* tail = (SharedTail*)(smem + RING_BYTES);
    pdl_wait();
    pdl_launch_dependents();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (p.K + BK - 1) / BK;
    const int w_rows = DUAL ? 2 * p.N : p.N;
    const int cols_per_tile = DUAL ? bnh : 2 * bnh;          // output columns of one tile
    const unsigned stage_tx = A_BYTES + 2 * bnh * BK * 2;   // bytes of one stage, also its stride in the ring
    volatile int* abort_flag = &tail->abort_flag;
    int* const err_word = waits.error_word ? waits.error_word : &g_tc_error;
    const long long wait_limit = waits.limit_cycles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < n_stages; ++s) { mbar_init(smem_u32(&tail->full[s]), 1); mbar_init(smem_u32(&tail->empty[s]), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(smem_u32(&tail->acc_full[b]), 1); mbar_init(smem_u32(&tail->acc_empty[b]), 4); }
        tail->abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) {
        tmem_alloc(&tail->tmem_base, TMEM_COLS);
    }
    const bool listed = p.group_offsets != nullptr && max_row_tiles <= MAX_LISTED;
    if (warp == 2 && listed) {
        // the row tiles of all groups in group order: 32 groups at a time, places by a warp scan
        int base = 0;
        for (int g0 = 0; g0 < p.n_groups; g0 += 32) {
            const int g = g0 + lane;
            int lo = 0, hi = 0;
            if (g < p.n_groups) { lo = p.group_offsets[g]; hi = p.group_offsets[g + 1]; }
            const int cnt = hi > lo ? (hi - lo + BM - 1) / BM : 0;
            int incl = cnt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            const int at = base + incl - cnt;
            for (int i = 0; i < cnt && at + i < MAX_LISTED; ++i) {
                tail->rt_group[at + i] = g;
                tail->rt_row0[at + i] = lo + i * BM;
                tail->rt_rows[at + i] = min(BM, hi - lo - i * BM);
            }
            base += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) tail->n_row_tiles = min(base, MAX_LISTED);
    }
    fence_before();
    __syncthreads();
    fence_after();
    const unsigned tmem = tail->tmem_base;
    const int row_tiles = listed ? tail->n_row_tiles : max_row_tiles;
    const int total_tiles = row_tiles * col_tiles;

    if (warp == 0) {
        if (lane == 0) {
            // ---- loader
            // weights that one row tile alone uses are read once: they should leave L2 first
            const bool dense_once = !p.group_offsets && p.M <= BM;
            const unsigned long long w_policy = l2_evict_first();
            int it = 0;                                       // k blocks issued so far, over all tiles
            int s = 0;                                        // it % n_stages and the ring's phase, kept by counting
            unsigned ph = 0;
            bool ok = true;
            for (int idx = blockIdx.x; idx < total_tiles && ok; idx += gridDim.x) {
                const Tile t = tile_at(p, tail, listed, idx, row_tiles, cols_per_tile);
                if (!t.ok) continue;
                const bool w_once = p.group_offsets ? p.group_offsets[t.group + 1] - p.group_offsets[t.group] <= BM : dense_once;
                const int wy0 = t.group * w_rows + t.n0;
                const int wy1 = DUAL ? t.group * w_rows + p.N + t.n0 : wy0 + bnh;
                for (int kb = 0; kb < num_kb; ++kb, ++it, s = (s + 1 == n_stages ? 0 : s + 1), ph ^= (s == 0)) {
                    ok = mbar_wait(smem_u32(&tail->empty[s]), ph ^ 1, abort_flag, err_word, 1, wait_limit);
                    if (!ok) break;
                    const unsigned bar = smem_u32(&tail->full[s]);
                    const unsigned dst = smem_u32(smem + s * stage_tx);
                    mbar_expect_tx(bar, stage_tx + (it == 0 ? waits.extra_tx : 0));
                    tma_load_2d(dst, &map_a, kb * BK, t.row0, bar);
                    if (w_once) {
                        tma_load_2d_hint(dst + A_BYTES, &map_w, kb * BK, wy0, bar, w_policy);
                        tma_load_2d_hint(dst + A_BYTES + bnh * BK * 2, &map_w, kb * BK, wy1, bar, w_policy);
                    } else {
                        tma_load_2d(dst + A_BYTES, &map_w, kb * BK, wy0, bar);
                        tma_load_2d(dst + A_BYTES + bnh * BK * 2, &map_w, kb * BK, wy1, bar);
                    }
                }
            }
            if (*abort_flag) {
                // copies in flight must land before the block gives its shared memory back
                for (int j = max(0, it - n_stages); j < it; ++j)
                    mbar_drain(smem_u32(&tail->full[j % n_stages]), (j / n_stages) & 1, wait_limit);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- tensor-core issue
            const unsigned idesc = make_idesc(BM, 2 * bnh);
            int lt = 0, s = 0;
            unsigned ph = 0;
            bool ok = true;
            for (int idx = blockIdx.x; idx < total_tiles && ok; idx += gridDim.x) {
                const Tile t = tile_at(p, tail, listed, idx, row_tiles, cols_per_tile);
                if (!t.ok) continue;
                const int buf = lt & 1;
                ok = mbar_wait(smem_u32(&tail->acc_empty[buf]), ((lt >> 1) & 1) ^ 1, abort_flag, err_word, 4, wait_limit);
                if (!ok) break;
                fence_after();
                const unsigned d_tmem = tmem + buf * ACC_COLS;
                for (int kb = 0; kb < num_kb; ++kb, s = (s + 1 == n_stages ? 0 : s + 1), ph ^= (s == 0)) {
                    ok = mbar_wait(smem_u32(&tail->full[s]), ph, abort_flag, err_word, 2, wait_limit);
                    if (!ok) break;
                    fence_after();
                    const unsigned a_addr = smem_u32(smem + s * stage_tx);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        mma(d_tmem, smem_desc_k_major(a_addr + k * UMMA_K * 2), smem_desc_k_major(a_addr + A_BYTES + k * UMMA_K * 2),
                               idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    commit(smem_u32(&tail->empty[s]));      // the stage is free once these MMAs have read it
                }
                if (ok) commit(smem_u32(&tail->acc_full[buf]));   // this accumulator is complete
                ++lt;
            }
        }
    } else {
        // ---- epilogue: warp w may read TMEM lanes [32 (w % 4), 32 (w % 4) + 32)
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        int lt = 0;
        bool ok = true;
        for (int idx = blockIdx.x; idx < total_tiles && ok; idx += gridDim.x) {
            const Tile t = tile_at(p, tail, listed, idx, row_tiles, cols_per_tile);
            if (!t.ok) continue;
            const int buf = lt & 1;
            ok = mbar_wait(smem_u32(&tail->acc_full[buf]), (lt >> 1) & 1, abort_flag, err_word, 3, wait_limit);
            if (!ok) break;
            fence_after();
            drain_accumulator_row<EPI>(p, t.row0 + r, r < t.rows, t.n0, cols_per_tile, bnh,
                                       tmem + buf * ACC_COLS + ((unsigned)(quarter * 32) << 16));
            // this warp has read its lanes of the accumulator: hand it back to the tensor cores
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tail->acc_empty[buf]));
            ++lt;
        }
    }
    fence_before();
    __syncthreads();
    if (warp == 1) {
        fence_after();
        tmem_free(tmem, TMEM_COLS);
    }
}

// ---------------------------------------------------------------- host side
// Half-tile height that makes the tile waves fullest: fewest rounds of n_blocks tiles, weighted by
// the tile's width plus a fixed cost for filling and draining the pipeline.
int choose_bnh(const GemmParams& p, int row_tiles, int n_blocks) {
    const bool dual = p.epilogue == EPI_SWIGLU;
    int best = 128;
    long long best_cost = -1;
    for (int bnh = 128; bnh >= 32; bnh -= 16) {
        // the epilogue reads 32 columns at a time: SwiGLU tiles (bnh columns) come in steps of 32.  The
        // in-between widths pay only where a product has few rounds (measured: 2048 x 7168 x 5120 gains
        // 5 % from 160-column tiles, the same product with 8192 rows loses 3 %)
        if (bnh % 32 && dual) continue;
        const int cols = dual ? bnh : 2 * bnh;
        const long long tiles = (long long)((p.N + cols - 1) / cols) * row_tiles;
        const long long rounds = (tiles + n_blocks - 1) / n_blocks;
        if (bnh % 32 && rounds > 6) continue;
        const long long cost = rounds * (2 * bnh + 40);
        if (best_cost < 0 || cost < best_cost) { best = bnh; best_cost = cost; }
    }
    return best;
}

template <int EPI>
int launch(const GemmParams& p, int n_blocks, cudaStream_t st) {
    const int row_tiles = (p.M + BM - 1) / BM + (p.group_offsets ? p.n_groups : 0);
    const int bnh = choose_bnh(p, row_tiles, n_blocks);
    const int cols = (EPI == EPI_SWIGLU) ? bnh : 2 * bnh;
    const long long total = (long long)((p.N + cols - 1) / cols) * row_tiles;
    if (total > 0x7fffffff) return SPITE_UNSUPPORTED;
    const long long w_rows = (long long)(EPI == EPI_SWIGLU ? 2 : 1) * p.N * p.n_groups;
    CUtensorMap ma, mw;
    if (!make_matrix_map(&ma, p.A, p.M, p.K, p.lda, BM) || !make_matrix_map(&mw, p.W, w_rows, p.K, p.K, bnh))
        return SPITE_LAUNCH_FAILED;
    const size_t smem = (size_t)RING_BYTES + sizeof(SharedTail) + 1024;
    int n_stages = RING_BYTES / (A_BYTES + 2 * bnh * BK * 2);
    if (n_stages > MAX_STAGES) n_stages = MAX_STAGES;
    auto k = gemm_tc_kernel<EPI>;
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return SPITE_LAUNCH_FAILED;
    const int grid = (int)(total < n_blocks ? total : n_blocks);
    SPITE_LAUNCH(k, grid, THREADS, smem, st, ma, mw, p, bnh, row_tiles, (int)(total / row_tiles), n_stages, s_waits);
    return spite_launch_status();
}

}  // namespace

// `n_blocks`: number of multiprocessors (one persistent block each).
SPITE_API int spite_gemm_tc(const GemmParams* p, int n_blocks, void* stream) {
    if (!p || !p->A || !p->W || !p->C) return SPITE_BAD_ARG;
    if (p->M < 0 || p->N <= 0 || p->K <= 0 || p->lda < p->K || p->ldc < p->N || n_blocks < 1) return SPITE_BAD_ARG;
    if (p->group_offsets ? p->n_groups < 1 : p->n_groups != 1) return SPITE_BAD_ARG;
    if (p->epilogue < 0 || p->epilogue > EPI_SWIGLU) return SPITE_BAD_ARG;
    // TMA: 16-byte aligned bases and row pitches
    if (p->K % 8 || p->lda % 8 || (((uintptr_t)p->A | (uintptr_t)p->W) & 15)) return SPITE_UNSUPPORTED;
    if (p->n_groups > 1 && p->w_group_stride != (long long)(p->epilogue == EPI_SWIGLU ? 2 : 1) * p->N * p->K)
        return SPITE_UNSUPPORTED;                              // groups must be stacked without gaps
    if (p->M == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    switch (p->epilogue) {
        case EPI_STORE: return launch<EPI_STORE>(*p, n_blocks, st);
        case EPI_STORE_F32: return launch<EPI_STORE_F32>(*p, n_blocks, st);
        case EPI_ADD_F32: return launch<EPI_ADD_F32>(*p, n_blocks, st);
        default: return launch<EPI_SWIGLU>(*p, n_blocks, st);
    }
}
