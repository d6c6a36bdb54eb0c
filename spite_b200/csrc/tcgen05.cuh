// PTX wrappers for the fifth-generation tensor cores and their plumbing: mbarriers, TMA tile
// loads, tcgen05 issue/commit/fences, tensor-memory loads and stores, and the shared-memory and
// instruction descriptors of kind::f16 products with bfloat16 inputs.
//
// Every wait on an mbarrier is bounded: a waiter that runs out of time raises the block's abort
// flag (which all waiters poll) and records a code in an error word, so that a kernel always
// reaches its common exit, where it frees its tensor memory.  The limit and the error word are
// launch arguments (`WaitControl`), kept per library and set with its `..._configure_waits`.
#pragma once
#include "common.cuh"
#include <cuda.h>

namespace tc {

constexpr long long WAIT_CYCLES = 4000000000ll;          // the default limit of a wait: about two seconds

// How the waits of one launch behave.
struct WaitControl {
    long long limit_cycles;     // a wait gives up after this many clock cycles
    int* error_word;            // where the first give-up of a launch records its code (device memory, or host
                                // memory that the device can write); null: the library's own word
    int extra_tx;               // bytes added to what a loader announces for its first stage.  Always 0 in
                                // use; a test sets it so that one barrier never completes and the waits on
                                // it run out, which is the one way to reach the give-up path on purpose.
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_inval(unsigned bar) { asm volatile("mbarrier.inval.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
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
// Waits for the phase of `parity`; gives up when the abort flag is up or time has run out.  The
// flag and the clock are looked at once in 32 polls, so that a waiting warp takes few issue slots
// from the warps that compute (mbarrier.try_wait itself suspends the thread for a while).
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, volatile int* abort_flag, int* error_word,
                                          int code, long long limit_cycles) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > limit_cycles) {
            *abort_flag = 1;
            // the first code stays; a plain store, because the word may lie in host memory
            volatile int* w = error_word;
            if (*w == 0) *w = code;
            __threadfence_system();
            return false;
        }
    }
}
// Waits, without an abort flag, until a copy that is already in flight has landed (or time runs out).
__device__ __forceinline__ void mbar_drain(unsigned bar, unsigned parity, long long limit_cycles) {
    const long long t0 = clock64();
    while (!mbar_try(bar, parity) && clock64() - t0 < limit_cycles) {}
}

__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 ::"r"(dst), "l"((unsigned long long)map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// The same with an L2 eviction policy (see l2_evict_first) for data that is read once.
__device__ __forceinline__ void tma_load_2d_hint(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar,
                                                 unsigned long long policy) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;\n"
                 ::"r"(dst), "l"((unsigned long long)map), "r"(x), "r"(y), "r"(bar), "l"(policy) : "memory");
}
__device__ __forceinline__ unsigned long long l2_evict_first() {
    unsigned long long policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void tma_load_3d(unsigned dst, const CUtensorMap* map, int x, int y, int z, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
                 ::"r"(dst), "l"((unsigned long long)map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
// Orders this thread's ordinary shared-memory writes before reads by the tensor cores or TMA.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mma(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                    unsigned idesc, unsigned accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same product with the A operand in tensor memory: row i of A in lane i, two consecutive k
// elements of 16 bits in one 32-bit column (the even k in the low half), so 16 k take 8 columns.
__device__ __forceinline__ void mma_a_tmem(unsigned d_tmem, unsigned a_tmem, unsigned long long b_desc,
                                           unsigned idesc, unsigned accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Tensor-memory allocation of `cols` columns (a power of two, 32..512) by one whole warp; the
// base address lands in *slot (shared memory).
__device__ __forceinline__ void tmem_alloc(unsigned* slot, unsigned cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_free(unsigned base, unsigned cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(base), "r"(cols) : "memory");
}

// 32 consecutive float32 columns of this thread's lane (warp w reads lanes 32 (w % 4) .. + 31).
__device__ __forceinline__ void ld32(float (&v)[32], unsigned taddr) {
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
// The same for 64 columns: both loads are issued before the one wait, so their latencies overlap.
__device__ __forceinline__ void ld64(float (&v)[64], unsigned taddr) {
    unsigned r[64];
#pragma unroll
    for (int h = 0; h < 2; ++h)
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                     "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                     "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
                     : "=r"(r[32 * h + 0]), "=r"(r[32 * h + 1]), "=r"(r[32 * h + 2]), "=r"(r[32 * h + 3]),
                       "=r"(r[32 * h + 4]), "=r"(r[32 * h + 5]), "=r"(r[32 * h + 6]), "=r"(r[32 * h + 7]),
                       "=r"(r[32 * h + 8]), "=r"(r[32 * h + 9]), "=r"(r[32 * h + 10]), "=r"(r[32 * h + 11]),
                       "=r"(r[32 * h + 12]), "=r"(r[32 * h + 13]), "=r"(r[32 * h + 14]), "=r"(r[32 * h + 15]),
                       "=r"(r[32 * h + 16]), "=r"(r[32 * h + 17]), "=r"(r[32 * h + 18]), "=r"(r[32 * h + 19]),
                       "=r"(r[32 * h + 20]), "=r"(r[32 * h + 21]), "=r"(r[32 * h + 22]), "=r"(r[32 * h + 23]),
                       "=r"(r[32 * h + 24]), "=r"(r[32 * h + 25]), "=r"(r[32 * h + 26]), "=r"(r[32 * h + 27]),
                       "=r"(r[32 * h + 28]), "=r"(r[32 * h + 29]), "=r"(r[32 * h + 30]), "=r"(r[32 * h + 31])
                     : "r"(taddr + 32 * h) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
// 32 consecutive 32-bit columns of this thread's lane, written and waited for.
__device__ __forceinline__ void st32(unsigned taddr, const unsigned (&v)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                 "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
                 ::"r"(taddr),
                   "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
                   "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
                   "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
                   "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
                 : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void st32(unsigned taddr, const float (&v)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                 "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
                 ::"r"(taddr),
                   "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
                   "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
                   "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
                   "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
                   "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
                   "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
                   "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
                   "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
                 : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1.
//  K-major operand (rows of 64 k elements = 128 bytes): 8-row groups `sbo` bytes apart; the
//    leading offset is not used.
//  MN-major operand (rows of 64 m/n elements, one row per k): 8-row groups `sbo` bytes apart,
//    the next 64 m/n elements `lbo` bytes on.
__device__ __forceinline__ unsigned long long smem_desc(unsigned addr, unsigned lbo, unsigned sbo) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFF) >> 4);            // start address
    d |= (unsigned long long)((lbo >> 4) & 0x3FFF) << 16;        // leading byte offset
    d |= (unsigned long long)((sbo >> 4) & 0x3FFF) << 32;        // stride byte offset
    d |= (unsigned long long)1 << 46;                            // version
    d |= (unsigned long long)2 << 61;                            // SWIZZLE_128B
    return d;
}
__device__ __forceinline__ unsigned long long smem_desc_k_major(unsigned addr) { return smem_desc(addr, 16, 1024); }

// kind::f16 instruction descriptor: float32 accumulator, bfloat16 A (K-major) and B (K-major, or
// MN-major when `b_mn_major`), tile m x n.
__host__ __device__ constexpr unsigned make_idesc(int m, int n, bool b_mn_major = false) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((unsigned)(n >> 3) << 17) |
           ((unsigned)(m >> 4) << 24);
}

// ---------------------------------------------------------------- host side: tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_fn() {
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

// L2 promotion of the TMA loads: 256 bytes (a load of a 128-byte row segment brings its neighbour along;
// every kernel here walks its rows onward, so the neighbour is the next k block).  Measured on B200 in the
// decode step against 128 bytes: 1,096 against 1,053 tokens/s.
static inline CUtensorMapL2promotion l2_promotion() { return CU_TENSOR_MAP_L2_PROMOTION_L2_256B; }

// bfloat16 tensor of `rank` dimensions (innermost first), 128-byte swizzle, zero fill outside.
// `strides_bytes` has rank - 1 entries (the innermost dimension is contiguous).
static inline bool make_map(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims,
                            const cuuint64_t* strides_bytes, const cuuint32_t* box) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), dims, strides_bytes, box,
              estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, l2_promotion(),
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tc

// The exported controls of a library whose kernels wait on mbarriers: `name` is the library's stem,
// `own_word` its `__device__ int` error word.
//   spite_<name>_configure_waits(limit_cycles, error_word, extra_tx)   later launches take these (<= 0 / null: defaults)
//   spite_<name>_error()   waits for the device, returns the code a give-up left (0: none) and clears it
#define SPITE_WAIT_CONTROLS(name, own_word)                                                              \
    namespace { tc::WaitControl s_waits = {tc::WAIT_CYCLES, nullptr, 0}; }                                \
    SPITE_API int spite_##name##_configure_waits(long long limit_cycles, int* error_word, int extra_tx) { \
        if (extra_tx < 0 || extra_tx % 16) return SPITE_BAD_ARG;                                          \
        s_waits.limit_cycles = limit_cycles > 0 ? limit_cycles : tc::WAIT_CYCLES;                         \
        s_waits.error_word = error_word;                                                                  \
        s_waits.extra_tx = extra_tx;                                                                      \
        return SPITE_OK;                                                                                  \
    }                                                                                                     \
    SPITE_API int spite_##name##_error() {                                                                \
        int v = 0, zero = 0;                                                                              \
        if (cudaDeviceSynchronize() != cudaSuccess) return SPITE_LAUNCH_FAILED;                           \
        if (s_waits.error_word) {                                                                         \
            if (cudaMemcpy(&v, s_waits.error_word, sizeof(int), cudaMemcpyDefault) != cudaSuccess)        \
                return SPITE_LAUNCH_FAILED;                                                               \
            if (v) cudaMemcpy(s_waits.error_word, &zero, sizeof(int), cudaMemcpyDefault);                 \
            return v;                                                                                     \
        }                                                                                                 \
        if (cudaMemcpyFromSymbol(&v, own_word, sizeof(int)) != cudaSuccess) return SPITE_LAUNCH_FAILED;   \
        if (v) cudaMemcpyToSymbol(own_word, &zero, sizeof(int));                                          \
        return v;                                                                                         \
    }
