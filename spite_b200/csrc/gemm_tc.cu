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
// after about two seconds a waiter raises an abort flag that all roles poll, records an
// error code that the host reads with spite_gemm_tc_error(), waits for its own copies in
// flight, and the block leaves through the common exit, where TMEM is freed.
//
// Rows of A are contiguous (a grouped product gets its rows gathered into expert order
// beforehand); `a_rows`, if set, only indexes `row_scale`.  Edges in M, N and K are
// covered by TMA's zero fill on loads and by bounds checks on stores.
#include "gemm.cuh"
#include <cuda.h>

namespace {

constexpr int BM = 128, BK = 64, UMMA_K = 16, MAX_STAGES = 8;
constexpr int A_BYTES = BM * BK * 2;                     // 16 KiB
constexpr int B_BYTES = 256 * BK * 2;                    // room for 256 weight rows, 32 KiB
constexpr int RING_BYTES = 4 * (A_BYTES + B_BYTES);      // 192 KiB of stages: 4 of the widest tile, up to 8 of narrower ones
constexpr int ACC_COLS = 256, TMEM_COLS = 512;
constexpr int THREADS = 192;
constexpr long long WAIT_CYCLES = 4000000000ll;          // about two seconds

__device__ int g_tc_error = 0;

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Waits for the phase of `parity`; gives up when the abort flag is up or time has run out.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, volatile int* abort_flag, int code) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_CYCLES) {
            *abort_flag = 1;
            atomicCAS(&g_tc_error, 0, code);
            return false;
        }
    }
}
__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 ::"r"(dst), "l"((unsigned long long)map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                       unsigned idesc, unsigned accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(float (&v)[32], unsigned taddr) {
    unsigned r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128
// bytes, 8-row groups 1024 bytes apart (stride byte offset), descriptor version 1.
__device__ __forceinline__ unsigned long long smem_desc(unsigned addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFF) >> 4);            // start address
    d |= (unsigned long long)1 << 16;                            // leading byte offset (unused with swizzle)
    d |= (unsigned long long)(1024 >> 4) << 32;                  // stride byte offset
    d |= (unsigned long long)1 << 46;                            // version
    d |= (unsigned long long)2 << 61;                            // SWIZZLE_128B
    return d;
}

// kind::f16 instruction descriptor: float32 accumulator, bfloat16 A and B, both K-major.
__host__ __device__ constexpr unsigned make_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}

struct SharedTail {
    unsigned long long full[MAX_STAGES];
    unsigned long long empty[MAX_STAGES];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];
    unsigned tmem_base;
    int abort_flag;
};

// The tile with running index `idx`: column tile idx / row_tiles, row tile idx % row_tiles.
struct Tile {
    int group, row0, rows, n0;
    bool ok;
};
__device__ __forceinline__ Tile tile_at(const GemmParams& p, int idx, int row_tiles, int cols_per_tile) {
    Tile t;
    t.n0 = (idx / row_tiles) * cols_per_tile;
    t.ok = locate_row_tile(p, idx % row_tiles, BM, t.group, t.row0, t.rows);
    return t;
}

// `bnh`: weight rows per half of the W tile (32, 64, 96 or 128); the MMA is 128 x 2 bnh x 16.
template <int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const GemmParams p, const int bnh, const int row_tiles, const int total_tiles, const int n_stages) {
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

    if (threadIdx.x == 0) {
        for (int s = 0; s < n_stages; ++s) { mbar_init(smem_u32(&tail->full[s]), 1); mbar_init(smem_u32(&tail->empty[s]), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(smem_u32(&tail->acc_full[b]), 1); mbar_init(smem_u32(&tail->acc_empty[b]), 4); }
        tail->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&tail->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = tail->tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            // ---- loader
            int it = 0;                                       // k blocks issued so far, over all tiles
            int s = 0;                                        // it % n_stages and the ring's phase, kept by counting
            unsigned ph = 0;
            bool ok = true;
            for (int idx = blockIdx.x; idx < total_tiles && ok; idx += gridDim.x) {
                const Tile t = tile_at(p, idx, row_tiles, cols_per_tile);
                if (!t.ok) continue;
                const int wy0 = t.group * w_rows + t.n0;
                const int wy1 = DUAL ? t.group * w_rows + p.N + t.n0 : wy0 + bnh;
                for (int kb = 0; kb < num_kb; ++kb, ++it, s = (s + 1 == n_stages ? 0 : s + 1), ph ^= (s == 0)) {
                    ok = mbar_wait(smem_u32(&tail->empty[s]), ph ^ 1, abort_flag, 1);
                    if (!ok) break;
                    const unsigned bar = smem_u32(&tail->full[s]);
                    const unsigned dst = smem_u32(smem + s * stage_tx);
                    mbar_expect_tx(bar, stage_tx);
                    tma_load_2d(dst, &map_a, kb * BK, t.row0, bar);
                    tma_load_2d(dst + A_BYTES, &map_w, kb * BK, wy0, bar);
                    tma_load_2d(dst + A_BYTES + bnh * BK * 2, &map_w, kb * BK, wy1, bar);
                }
            }
            if (*abort_flag) {
                // copies in flight must land before the block gives its shared memory back
                for (int j = max(0, it - n_stages); j < it; ++j) {
                    const long long t0 = clock64();
                    while (!mbar_try(smem_u32(&tail->full[j % n_stages]), (j / n_stages) & 1) &&
                           clock64() - t0 < WAIT_CYCLES) {}
                }
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
                const Tile t = tile_at(p, idx, row_tiles, cols_per_tile);
                if (!t.ok) continue;
                const int buf = lt & 1;
                ok = mbar_wait(smem_u32(&tail->acc_empty[buf]), ((lt >> 1) & 1) ^ 1, abort_flag, 4);
                if (!ok) break;
                tc_fence_after();
                const unsigned d_tmem = tmem + buf * ACC_COLS;
                for (int kb = 0; kb < num_kb; ++kb, s = (s + 1 == n_stages ? 0 : s + 1), ph ^= (s == 0)) {
                    ok = mbar_wait(smem_u32(&tail->full[s]), ph, abort_flag, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const unsigned a_addr = smem_u32(smem + s * stage_tx);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        tc_mma(d_tmem, smem_desc(a_addr + k * UMMA_K * 2), smem_desc(a_addr + A_BYTES + k * UMMA_K * 2),
                               idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    tc_commit(smem_u32(&tail->empty[s]));      // the stage is free once these MMAs have read it
                }
                if (ok) tc_commit(smem_u32(&tail->acc_full[buf]));   // this accumulator is complete
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
            const Tile t = tile_at(p, idx, row_tiles, cols_per_tile);
            if (!t.ok) continue;
            const int buf = lt & 1;
            ok = mbar_wait(smem_u32(&tail->acc_full[buf]), (lt >> 1) & 1, abort_flag, 3);
            if (!ok) break;
            tc_fence_after();
            const int li = t.row0 + r;
            const bool row_ok = r < t.rows;
            int crow = li, srow = li;
            float sc = 1.f;
            if (row_ok) {
                if (p.c_rows) crow = p.c_rows[li];
                if (p.row_scale) {
                    if (p.scale_by_a_row && p.a_rows) srow = p.a_rows[li];
                    sc = p.row_scale[srow];
                }
            }
            const unsigned lane_addr = tmem + buf * ACC_COLS + ((unsigned)(quarter * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < cols_per_tile; c0 += 32) {
                float v[32];
                tc_ld32(v, lane_addr + c0);                    // warp-collective: every lane takes part
                float u[32];
                if (DUAL) tc_ld32(u, lane_addr + bnh + c0);
                const int n = t.n0 + c0;
                if (!row_ok || n >= p.N) continue;
                const size_t o = (size_t)crow * p.ldc + n;
                const bool full = (n + 32 <= p.N);
                if (EPI == EPI_STORE || EPI == EPI_SWIGLU) {
                    __nv_bfloat16* dst = (__nv_bfloat16*)p.C + o;
                    float y[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) y[i] = DUAL ? silu_f32(v[i] * sc) * (u[i] * sc) : v[i] * sc;
                    if (full && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 q;
                            __nv_bfloat162 h0 = __floats2bfloat162_rn(y[i], y[i + 1]), h1 = __floats2bfloat162_rn(y[i + 2], y[i + 3]);
                            __nv_bfloat162 h2 = __floats2bfloat162_rn(y[i + 4], y[i + 5]), h3 = __floats2bfloat162_rn(y[i + 6], y[i + 7]);
                            q.x = *(unsigned*)&h0; q.y = *(unsigned*)&h1; q.z = *(unsigned*)&h2; q.w = *(unsigned*)&h3;
                            *(uint4*)(dst + i) = q;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (n + i < p.N) dst[i] = __float2bfloat16_rn(y[i]);
                    }
                } else {
                    float* dst = (float*)p.C + o;
                    if (full && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            float4 q = make_float4(v[i] * sc, v[i + 1] * sc, v[i + 2] * sc, v[i + 3] * sc);
                            if (EPI == EPI_ADD_F32) {
                                const float4 old = *(const float4*)(dst + i);
                                q.x += old.x; q.y += old.y; q.z += old.z; q.w += old.w;
                            }
                            *(float4*)(dst + i) = q;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (n + i < p.N) dst[i] = (EPI == EPI_ADD_F32 ? dst[i] : 0.f) + v[i] * sc;
                    }
                }
            }
            // this warp has read its lanes of the accumulator: hand it back to the tensor cores
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tail->acc_empty[buf]));
            ++lt;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

// A row-major [rows, cols] bfloat16 matrix with leading dimension ld; boxes of 64 columns x box_rows rows.
bool make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Half-tile height that makes the tile waves fullest: fewest rounds of n_blocks tiles, weighted by
// the tile's width plus a fixed cost for filling and draining the pipeline.
int choose_bnh(const GemmParams& p, int row_tiles, int n_blocks) {
    const bool dual = p.epilogue == EPI_SWIGLU;
    int best = 128;
    long long best_cost = -1;
    for (int bnh = 128; bnh >= 32; bnh -= 32) {
        const int cols = dual ? bnh : 2 * bnh;
        const long long tiles = (long long)((p.N + cols - 1) / cols) * row_tiles;
        const long long rounds = (tiles + n_blocks - 1) / n_blocks;
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
    if (!make_map(&ma, p.A, p.M, p.K, p.lda, BM) || !make_map(&mw, p.W, w_rows, p.K, p.K, bnh))
        return SPITE_LAUNCH_FAILED;
    const size_t smem = (size_t)RING_BYTES + sizeof(SharedTail) + 1024;
    int n_stages = RING_BYTES / (A_BYTES + 2 * bnh * BK * 2);
    if (n_stages > MAX_STAGES) n_stages = MAX_STAGES;
    auto k = gemm_tc_kernel<EPI>;
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return SPITE_LAUNCH_FAILED;
    const int grid = (int)(total < n_blocks ? total : n_blocks);
    SPITE_LAUNCH(k, grid, THREADS, smem, st, ma, mw, p, bnh, row_tiles, (int)total, n_stages);
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

// Error code recorded by a block that gave up waiting (0: none); reading it clears it.
// 1: loader waited for a free stage, 2: tensor-core issue waited for a tile, 3: epilogue waited
// for an accumulator, 4: tensor-core issue waited for a free accumulator.
SPITE_API int spite_gemm_tc_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int)) != cudaSuccess) return -3;
    if (v) cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
    return v;
}
