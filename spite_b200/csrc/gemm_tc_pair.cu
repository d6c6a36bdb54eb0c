// Matrix product for many tokens on pairs of multiprocessors (tcgen05 cta_group::2):
//   C[M, N] (=|+=) epilogue( A[M, K] W[N, K]^T ),  bfloat16 inputs, float32 sums in TMEM.
//
// Two blocks of a cluster share one output tile of 256 rows x BN columns (BN = 64..256).  Each
// loads its own 128 rows of A and its own half of the W tile, so a multiprocessor moves 32 KiB
// into shared memory per 64-wide k block where the one-block kernel (gemm_tc.cu) moves 48 KiB,
// and the ring holds 6 to 10 stages.  The first block of the pair issues tcgen05.mma
// .cta_group::2 (256 x BN x 16): the tensor cores of both multiprocessors read A from their
// own shared memory and the two halves of W from both, and each leaves its 128 rows of the
// accumulator in its own tensor memory, where its own four epilogue warps fetch them.
// The one-block kernel is bound by shared-memory traffic (operand reads plus TMA writes exceed
// what a multiprocessor's shared memory takes per cycle at full tensor rate); the pair halves
// the W part of it.
//
// Roles per block: warp 0 loader (one lane; TMA with the pair's leader's mbarrier as the
// completion target), warp 1 TMEM allocation (both blocks, cta_group::2) and, in the leader
// only, MMA issue; warps 2-5 epilogue.  Barriers: `full` lives in the leader (it counts the bytes of
// both blocks' loads), `empty` and `acc_full` live in both (the leader's tcgen05.commit
// multicasts its arrival to the pair), `acc_empty` lives in the leader and takes the arrivals
// of both blocks' epilogue warps.  The SwiGLU form gives the leader the gate rows and the
// other block the up rows of W.
// A grouped product cuts every group into row tiles of up to 256 rows of its own (listed in shared
// memory by both blocks alike); rows of A are contiguous in group order (gathered beforehand), and
// `a_rows`, if set, only indexes `row_scale`.  A group's last tile is part-filled (128 rows wasted on
// average), so it pays only where the groups hold many hundreds of rows.
// Every wait is bounded (tcgen05.cuh); the blocks of a pair leave together through a cluster
// barrier, after which each frees its tensor memory.  No TMA multicast is used.
#include "gemm_tc_epilogue.cuh"

namespace {
using namespace tc;

constexpr int BM = 128, BK = 64, UMMA_K = 16, MAX_STAGES = 10;
constexpr int A_BYTES = BM * BK * 2;                     // 16 KiB: this block's rows of A
constexpr int RING_BYTES = 192 * 1024;
constexpr int ACC_COLS = 256, TMEM_COLS = 512;
constexpr int THREADS = 192;
constexpr int MAX_LISTED = 1024;                         // row tiles of a grouped product kept as a list in shared memory

__device__ int g_pair_error = 0;
}  // namespace
// 1: loader waited for a free stage, 2: tensor-core issue waited for a stage, 3: epilogue waited
// for an accumulator, 4: tensor-core issue waited for a free accumulator.  (`extra_tx` is not used here.)
SPITE_WAIT_CONTROLS(gemm_tc_pair, g_pair_error)
namespace {

struct SharedTail {
    unsigned long long full[MAX_STAGES];                 // used in the leader
    unsigned long long empty[MAX_STAGES];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];                     // used in the leader
    unsigned tmem_base;
    int abort_flag;
    int n_row_tiles;                                     // grouped products: row tiles (of up to 256 rows) that hold rows
    int rt_group[MAX_LISTED], rt_row0[MAX_LISTED], rt_rows[MAX_LISTED];
};

struct Tile {
    int group, row0, rows, n0;                           // rows: of the whole 256-row tile
};

__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// The address of the same shared-memory location in block `rank` of the cluster.
__device__ __forceinline__ unsigned in_block(unsigned smem_addr, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
// TMA tile load whose completion is counted by an mbarrier of the pair's leader.
__device__ __forceinline__ void tma_load_2d_pair(unsigned dst, const CUtensorMap* map, int x, int y, unsigned leader_bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 ::"r"(dst), "l"((unsigned long long)map), "r"(x), "r"(y), "r"(leader_bar) : "memory");
}
__device__ __forceinline__ void mma_pair(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                         unsigned idesc, unsigned accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the barrier at this offset in both blocks of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void commit_pair(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
                 ::"r"(bar), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(unsigned* slot, unsigned cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_free_pair(unsigned base, unsigned cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(base), "r"(cols) : "memory");
}

// `bnh`: weight rows each block loads per tile (32 .. 128); the MMA is 256 x 2 bnh x 16.
// Tile idx: column tile idx / row_tiles, row tile (256 rows) idx % row_tiles; the pairs walk them
// with a stride of the number of pairs.
template <int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const GemmParams p, const int bnh, const int dense_row_tiles, const int col_tiles, const int n_stages,
                    const WaitControl waits) {
    constexpr bool DUAL = (EPI == EPI_SWIGLU);
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    SharedTail* tail = (SharedTail*)(smem + RING_BYTES);
    pdl_wait();
    pdl_launch_dependents();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_rank();                    // 0: the leader
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int num_kb = (p.K + BK - 1) / BK;
    const int cols_per_tile = DUAL ? bnh : 2 * bnh;          // output columns of one tile
    const unsigned stage_bytes = A_BYTES + bnh * BK * 2;    // what this block loads per stage, also the ring's stride
    volatile int* abort_flag = &tail->abort_flag;
    int* const err_word = waits.error_word ? waits.error_word : &g_pair_error;
    const long long wait_limit = waits.limit_cycles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < n_stages; ++s) { mbar_init(smem_u32(&tail->full[s]), 1); mbar_init(smem_u32(&tail->empty[s]), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(smem_u32(&tail->acc_full[b]), 1); mbar_init(smem_u32(&tail->acc_empty[b]), 8); }
        tail->abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 2 && p.group_offsets) {
        // the row tiles of all groups in group order, up to 256 rows each: 32 groups at a time, places by a warp scan
        int base = 0;
        for (int g0 = 0; g0 < p.n_groups; g0 += 32) {
            const int g = g0 + lane;
            int lo = 0, hi = 0;
            if (g < p.n_groups) { lo = p.group_offsets[g]; hi = p.group_offsets[g + 1]; }
            const int cnt = hi > lo ? (hi - lo + 2 * BM - 1) / (2 * BM) : 0;
            int incl = cnt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            const int at = base + incl - cnt;
            for (int i = 0; i < cnt && at + i < MAX_LISTED; ++i) {
                tail->rt_group[at + i] = g;
                tail->rt_row0[at + i] = lo + i * 2 * BM;
                tail->rt_rows[at + i] = min(2 * BM, hi - lo - i * 2 * BM);
            }
            base += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) tail->n_row_tiles = min(base, MAX_LISTED);
    }
    __syncthreads();
    if (warp == 1) tmem_alloc_pair(&tail->tmem_base, TMEM_COLS);
    fence_before();
    cluster_sync();                                          // both blocks' barriers exist before either is signalled
    fence_after();
    const unsigned tmem = tail->tmem_base;
    const int row_tiles = p.group_offsets ? tail->n_row_tiles : dense_row_tiles;
    const int total_tiles = row_tiles * col_tiles;
    const int w_rows = DUAL ? 2 * p.N : p.N;
    auto tile_at = [&](int idx) {
        Tile t;
        const int rt = idx % row_tiles;
        t.n0 = (idx / row_tiles) * cols_per_tile;
        if (p.group_offsets) {
            t.group = tail->rt_group[rt]; t.row0 = tail->rt_row0[rt]; t.rows = tail->rt_rows[rt];
        } else {
            t.group = 0; t.row0 = rt * 2 * BM; t.rows = min(2 * BM, p.M - t.row0);
        }
        return t;
    };

    if (warp == 0) {
        if (lane == 0) {
            // ---- loader: this block's rows of A and its half of the W tile
            int it = 0, s = 0;
            unsigned ph = 0;
            bool ok = true;
            for (int idx = pair; idx < total_tiles && ok; idx += n_pairs) {
                const Tile t = tile_at(idx);
                const int row0 = t.row0 + (int)rank * BM;
                const int wy = t.group * w_rows + (DUAL ? (rank ? p.N + t.n0 : t.n0) : t.n0 + (int)rank * bnh);
                for (int kb = 0; kb < num_kb; ++kb, ++it, s = (s + 1 == n_stages ? 0 : s + 1), ph ^= (s == 0)) {
                    ok = mbar_wait(smem_u32(&tail->empty[s]), ph ^ 1, abort_flag, err_word, 1, wait_limit);
                    if (!ok) break;
                    const unsigned bar = in_block(smem_u32(&tail->full[s]), 0);
                    const unsigned dst = smem_u32(smem + s * stage_bytes);
                    if (rank == 0) mbar_expect_tx(smem_u32(&tail->full[s]), 2 * stage_bytes);
                    tma_load_2d_pair(dst, &map_a, kb * BK, row0, bar);
                    tma_load_2d_pair(dst + A_BYTES, &map_w, kb * BK, wy, bar);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---- tensor-core issue, for both blocks
            const unsigned idesc = make_idesc(2 * BM, 2 * bnh);
            int lt = 0, s = 0;
            unsigned ph = 0;
            bool ok = true;
            for (int idx = pair; idx < total_tiles && ok; idx += n_pairs) {
                const int buf = lt & 1;
                ok = mbar_wait(smem_u32(&tail->acc_empty[buf]), ((lt >> 1) & 1) ^ 1, abort_flag, err_word, 4, wait_limit);
                if (!ok) break;
                fence_after();
                const unsigned d_tmem = tmem + buf * ACC_COLS;
                for (int kb = 0; kb < num_kb; ++kb, s = (s + 1 == n_stages ? 0 : s + 1), ph ^= (s == 0)) {
                    ok = mbar_wait(smem_u32(&tail->full[s]), ph, abort_flag, err_word, 2, wait_limit);
                    if (!ok) break;
                    fence_after();
                    const unsigned a_addr = smem_u32(smem + s * stage_bytes);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        mma_pair(d_tmem, smem_desc_k_major(a_addr + k * UMMA_K * 2),
                                 smem_desc_k_major(a_addr + A_BYTES + k * UMMA_K * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    commit_pair(smem_u32(&tail->empty[s]));     // the stage is free in both blocks once these MMAs have read it
                }
                if (ok) commit_pair(smem_u32(&tail->acc_full[buf]));
                ++lt;
            }
        }
    } else {
        // ---- epilogue: this block's 128 rows; warp w may read TMEM lanes [32 (w % 4), 32 (w % 4) + 32)
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        int lt = 0;
        bool ok = true;
        for (int idx = pair; idx < total_tiles && ok; idx += n_pairs) {
            const Tile t = tile_at(idx);
            const int buf = lt & 1;
            ok = mbar_wait(smem_u32(&tail->acc_full[buf]), (lt >> 1) & 1, abort_flag, err_word, 3, wait_limit);
            if (!ok) break;
            fence_after();
            drain_accumulator_row<EPI>(p, t.row0 + (int)rank * BM + r, (int)rank * BM + r < t.rows, t.n0, cols_per_tile, bnh,
                                       tmem + buf * ACC_COLS + ((unsigned)(quarter * 32) << 16));
            // this warp has read its lanes of the accumulator: tell the leader
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(in_block(smem_u32(&tail->acc_empty[buf]), 0));
            ++lt;
        }
    }
    // Leave together: neither block may free its shared or tensor memory while the other's tensor
    // cores or copies can still touch it.  A block that gave up waiting has told its own roles; the
    // other block's waits run out by themselves.
    fence_before();
    __syncthreads();
    if (warp == 0 && lane == 0 && *abort_flag) {
        // this block's copies in flight land in its own shared memory: give them time
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) {}
    }
    cluster_sync();
    if (warp == 1) {
        fence_after();
        tmem_free_pair(tmem, TMEM_COLS);
    }
}

// Half-tile height that makes the tile waves fullest over `n_pairs` pairs (see gemm_tc.cu).
int choose_bnh(const GemmParams& p, int row_tiles, int n_pairs) {
    const bool dual = p.epilogue == EPI_SWIGLU;
    int best = 128;
    long long best_cost = -1;
    for (int bnh = 128; bnh >= 32; bnh -= 16) {
        if (bnh % 32 && dual) continue;                      // the epilogue reads 32 columns at a time
        const int cols = dual ? bnh : 2 * bnh;
        const long long tiles = (long long)((p.N + cols - 1) / cols) * row_tiles;
        const long long rounds = (tiles + n_pairs - 1) / n_pairs;
        if (bnh % 32 && rounds > 6) continue;
        const long long cost = rounds * (2 * bnh + 40);
        if (best_cost < 0 || cost < best_cost) { best = bnh; best_cost = cost; }
    }
    return best;
}

template <int EPI>
int launch(const GemmParams& p, int n_pairs, cudaStream_t st) {
    // grouped: an upper bound (every group may end in a part-filled tile); the kernel counts the tiles that hold rows
    const int row_tiles = (p.M + 2 * BM - 1) / (2 * BM) + (p.group_offsets ? p.n_groups : 0);
    if (p.group_offsets && row_tiles > MAX_LISTED) return SPITE_UNSUPPORTED;
    const int bnh = choose_bnh(p, p.group_offsets ? (p.M + 2 * BM - 1) / (2 * BM) + p.n_groups / 2 : row_tiles, n_pairs);
    const int cols = (EPI == EPI_SWIGLU) ? bnh : 2 * bnh;
    const int col_tiles = (p.N + cols - 1) / cols;
    const long long total = (long long)col_tiles * row_tiles;
    if (total > 0x7fffffff) return SPITE_UNSUPPORTED;
    const long long w_rows = (long long)(EPI == EPI_SWIGLU ? 2 : 1) * p.N * p.n_groups;
    CUtensorMap ma, mw;
    if (!make_matrix_map(&ma, p.A, p.M, p.K, p.lda, BM) || !make_matrix_map(&mw, p.W, w_rows, p.K, p.K, bnh))
        return SPITE_LAUNCH_FAILED;
    const size_t smem = (size_t)RING_BYTES + sizeof(SharedTail) + 1024;
    int n_stages = RING_BYTES / (A_BYTES + bnh * BK * 2);
    if (n_stages > MAX_STAGES) n_stages = MAX_STAGES;
    auto k = gemm_tc_pair_kernel<EPI>;
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return SPITE_LAUNCH_FAILED;
    const int pairs = (int)(total < n_pairs ? total : n_pairs);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = spite_pdl_enabled() ? 2 : 1;
    (void)cudaLaunchKernelEx(&cfg, k, ma, mw, p, bnh, row_tiles, col_tiles, n_stages, s_waits);
    return spite_launch_status();
}

}  // namespace

// `n_pairs`: half the number of multiprocessors (one persistent pair of blocks each).
SPITE_API int spite_gemm_tc_pair(const GemmParams* p, int n_pairs, void* stream) {
    if (!p || !p->A || !p->W || !p->C) return SPITE_BAD_ARG;
    if (p->M < 0 || p->N <= 0 || p->K <= 0 || p->lda < p->K || p->ldc < p->N || n_pairs < 1) return SPITE_BAD_ARG;
    if (p->group_offsets ? p->n_groups < 1 : p->n_groups != 1) return SPITE_BAD_ARG;
    if (p->n_groups > 1 && p->w_group_stride != (long long)(p->epilogue == EPI_SWIGLU ? 2 : 1) * p->N * p->K)
        return SPITE_UNSUPPORTED;                              // groups must be stacked without gaps
    if (p->epilogue < 0 || p->epilogue > EPI_SWIGLU) return SPITE_BAD_ARG;
    // TMA: 16-byte aligned bases and row pitches
    if (p->K % 8 || p->lda % 8 || (((uintptr_t)p->A | (uintptr_t)p->W) & 15)) return SPITE_UNSUPPORTED;
    if (p->M == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    switch (p->epilogue) {
        case EPI_STORE: return launch<EPI_STORE>(*p, n_pairs, st);
        case EPI_STORE_F32: return launch<EPI_STORE_F32>(*p, n_pairs, st);
        case EPI_ADD_F32: return launch<EPI_ADD_F32>(*p, n_pairs, st);
        default: return launch<EPI_SWIGLU>(*p, n_pairs, st);
    }
}
