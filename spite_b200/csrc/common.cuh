// Shared declarations of the sm_100a kernel libraries.
//
// Every library exports plain C functions.  A function takes device pointers,
// sizes and the CUDA stream to launch on, and returns a status:
//   0  launched
//  -1  an argument is malformed (null pointer, non-positive size)
//  -2  the size is outside what the kernel supports
//  -3  the launch itself failed (cudaGetLastError)
// Nothing is written when the status is negative.  The status convention follows
// the op contract of giveen/spite's kernel ABI (core/abi.h:218,365: 0 ok, -1, -2).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define SPITE_OK 0
#define SPITE_BAD_ARG (-1)
#define SPITE_UNSUPPORTED (-2)
#define SPITE_LAUNCH_FAILED (-3)

#define SPITE_DT_F32 0
#define SPITE_DT_BF16 1

#define SPITE_API extern "C" __attribute__((visibility("default")))

static inline int spite_launch_status() {
    return cudaGetLastError() == cudaSuccess ? SPITE_OK : SPITE_LAUNCH_FAILED;
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread receives the result.
// `scratch` holds 33 floats of shared memory.  The order of the additions is a
// function of the block size only.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// ---------------------------------------------------------------------------------
// Programmatic dependent launch.  Kernels of a step run back to back on one stream; with
// this launch attribute the next kernel's blocks may be set up while the last blocks of
// the current one still run.  Every kernel launched this way starts with pdl_wait(): it
// returns when the preceding kernel has finished and its writes are visible, so nothing
// a kernel reads or writes can race with its predecessor.  What a kernel does before
// pdl_wait() must not touch anything an earlier kernel of the step writes (weights only).
// SPITE_NO_PDL=1 in the environment switches the attribute off.
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

#include <cstdlib>
static inline bool spite_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("SPITE_NO_PDL");
        on = (e && e[0] && e[0] != '0') ? 0 : 1;
    }
    return on == 1;
}

template <typename... P, typename... A>
static inline void spite_launch_kernel(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                       A&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = spite_pdl_enabled() ? 1 : 0;
    (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<A&&>(args)...);
}
#define SPITE_LAUNCH(kernel, grid, block, smem, stream, ...) \
    spite_launch_kernel(kernel, dim3(grid), dim3(block), smem, stream, __VA_ARGS__)
