// Embedding gather and RMS norm.  Both are bound by memory traffic: one read of
// the row, one write.  The residual stream is float32; the norm writes the
// model's activation type.
#include "common.cuh"

// h[m, :] = table[token[m], :] * scale    (crates/spite-models/src/llama/llama4.rs:118-119; scale 1 there)
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ h, int d, int vocab, float scale) {
    pdl_wait();
    pdl_launch_dependents();
    const int m = blockIdx.x;
    const int tok = tokens[m];
    float* out = h + (size_t)m * d;
    if (tok < 0 || tok >= vocab) {          // the host rejects such ids before the launch
        for (int i = threadIdx.x; i < d; i += blockDim.x) out[i] = 0.f;
        return;
    }
    const T* row = table + (size_t)tok * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) out[i] = to_f32(row[i]) * scale;
}

// y[i, :] = x[r, :] * rsqrt(mean(x[r]^2) + eps) * gain      r = rows ? rows[i] : i
// (crates/spite-models/src/dense.rs:175-181; the sum runs in float32)
// One block per row.  The row stays in registers between the sum and the scaling: every thread
// holds up to VPT groups of four elements, loaded with one 16-byte read each.
__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) { *(float4*)p = make_float4(a, b, c, d); }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *(uint2*)p = make_uint2(*(unsigned*)&lo, *(unsigned*)&hi);
}

template <typename T, int VPT>
__global__ void rms_norm_vec_kernel(const float* __restrict__ x, const float* __restrict__ gain,
                                    const int* __restrict__ rows, T* __restrict__ y, int d, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    const float4* in = (const float4*)(x + (size_t)r * d);
    const int d4 = d >> 2;
    float4 v[VPT];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        v[k] = c < d4 ? in[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int k = 0; k < VPT; ++k) s += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
    s = block_sum(s, scratch);
    const float scale = 1.0f / sqrtf(s / (float)d + eps);
    T* out = y + (size_t)i * d;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < d4) {
            const float4 g = ((const float4*)gain)[c];
            store4(out + 4 * c, v[k].x * scale * g.x, v[k].y * scale * g.y, v[k].z * scale * g.z, v[k].w * scale * g.w);
        }
    }
}

// The same for widths that are no multiple of four, or too wide for the registers: two passes over the row.
template <typename T>
__global__ void rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ gain,
                                const int* __restrict__ rows, T* __restrict__ y, int d, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    const float* in = x + (size_t)r * d;
    float s = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) { float v = in[c]; s += v * v; }
    s = block_sum(s, scratch);
    const float scale = 1.0f / sqrtf(s / (float)d + eps);
    T* out = y + (size_t)i * d;
    for (int c = threadIdx.x; c < d; c += blockDim.x) out[c] = from_f32<T>(in[c] * scale * gain[c]);
}

// logits = cap * tanh(logits * scale / cap), or logits * scale without a cap (cap <= 0)
__global__ void transform_logits_kernel(float* __restrict__ logits, long long n, float scale, float cap) {
    pdl_wait();
    pdl_launch_dependents();
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float v = logits[i] * scale;
        logits[i] = cap > 0.f ? cap * tanhf(v * inv_cap) : v;
    }
}

// dst[i, :] = src[idx[i], :]   (rows of activations brought into expert order), 16 bytes per thread and step
__global__ void gather_rows_kernel(const uint4* __restrict__ src, const int* __restrict__ idx,
                                   uint4* __restrict__ dst, int row_vecs) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = blockIdx.x;
    const uint4* in = src + (size_t)idx[i] * row_vecs;
    uint4* out = dst + i * row_vecs;
    for (int c = threadIdx.x; c < row_vecs; c += blockDim.x) out[c] = in[c];
}

SPITE_API int spite_gather_rows(const void* src, const int* idx, void* dst, int n_rows, long long row_bytes,
                                void* stream) {
    if (!src || !idx || !dst || n_rows < 0 || row_bytes <= 0) return SPITE_BAD_ARG;
    if (row_bytes % 16 || (((uintptr_t)src | (uintptr_t)dst) & 15)) return SPITE_UNSUPPORTED;
    if (n_rows == 0) return SPITE_OK;
    SPITE_LAUNCH(gather_rows_kernel, n_rows, 128, 0, (cudaStream_t)stream, (const uint4*)src, idx, (uint4*)dst,
                 (int)(row_bytes / 16));
    return spite_launch_status();
}

// Zero pages of a paged cache: `base` holds `n_outer` blocks of `outer_stride` bytes (one per cache of a
// group and per keys / values), each with pages of `page_bytes`.  grid (pages to clear, n_outer).
struct PageList { int n; int ids[60]; };
template <typename Word>
__global__ void clear_pages_kernel(unsigned char* __restrict__ base, long long outer_stride, long long page_bytes,
                                   const PageList pages) {
    pdl_wait();
    pdl_launch_dependents();
    Word* dst = (Word*)(base + (size_t)blockIdx.y * outer_stride + (size_t)pages.ids[blockIdx.x] * page_bytes);
    const long long n = page_bytes / (long long)sizeof(Word);
    Word zero;
    memset(&zero, 0, sizeof(Word));
    for (long long i = threadIdx.x; i < n; i += blockDim.x) dst[i] = zero;
}

// `page_ids` is host memory (the ids are passed to the kernel by value, 60 a launch).
SPITE_API int spite_clear_pages(void* base, long long n_outer, long long outer_stride, long long page_bytes,
                                int n_pages_total, const int* page_ids, int n_ids, void* stream) {
    if (!base || n_outer < 1 || outer_stride < 1 || page_bytes < 1 || n_pages_total < 1 || n_ids < 0) return SPITE_BAD_ARG;
    if (n_ids > 0 && !page_ids) return SPITE_BAD_ARG;
    if (page_bytes % 4 || outer_stride % 4 || ((uintptr_t)base & 3) || n_outer > 65535) return SPITE_UNSUPPORTED;
    const bool wide = page_bytes % 16 == 0 && outer_stride % 16 == 0 && ((uintptr_t)base & 15) == 0;
    for (int i = 0; i < n_ids; ++i)
        if (page_ids[i] < 0 || page_ids[i] >= n_pages_total) return SPITE_BAD_ARG;
    for (int at = 0; at < n_ids; at += 60) {
        PageList list;
        list.n = n_ids - at < 60 ? n_ids - at : 60;
        for (int i = 0; i < list.n; ++i) list.ids[i] = page_ids[at + i];
        if (wide)
            SPITE_LAUNCH(clear_pages_kernel<uint4>, dim3(list.n, (unsigned)n_outer), 256, 0, (cudaStream_t)stream,
                         (unsigned char*)base, outer_stride, page_bytes, list);
        else
            SPITE_LAUNCH(clear_pages_kernel<unsigned>, dim3(list.n, (unsigned)n_outer), 256, 0, (cudaStream_t)stream,
                         (unsigned char*)base, outer_stride, page_bytes, list);
        if (spite_launch_status() != SPITE_OK) return SPITE_LAUNCH_FAILED;
    }
    return SPITE_OK;
}

SPITE_API int spite_transform_logits(float* logits, long long n, float scale, float softcap, void* stream) {
    if (!logits || n < 0 || !(scale == scale) || !(softcap == softcap)) return SPITE_BAD_ARG;
    if (n == 0) return SPITE_OK;
    const long long blocks = (n + 255) / 256;
    SPITE_LAUNCH(transform_logits_kernel, (int)(blocks < 4096 ? blocks : 4096), 256, 0, (cudaStream_t)stream, logits, n,
                 scale, softcap);
    return spite_launch_status();
}

SPITE_API int spite_embed(int dtype, const void* table, const int* tokens, float* h,
                          int n_tokens, int d, int vocab, float scale, void* stream) {
    if (!table || !tokens || !h || n_tokens < 0 || d <= 0 || vocab <= 0 || !(scale == scale)) return SPITE_BAD_ARG;
    if (n_tokens == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const int threads = d >= 1024 ? 256 : 128;
    if (dtype == SPITE_DT_F32)
        SPITE_LAUNCH(embed_kernel<float>, n_tokens, threads, 0, st, (const float*)table, tokens, h, d, vocab, scale);
    else if (dtype == SPITE_DT_BF16)
        SPITE_LAUNCH(embed_kernel<__nv_bfloat16>, n_tokens, threads, 0, st, (const __nv_bfloat16*)table, tokens, h, d, vocab, scale);
    else
        return SPITE_BAD_ARG;
    return spite_launch_status();
}

SPITE_API int spite_rms_norm(int out_dtype, const float* x, const float* gain, const int* rows,
                             void* y, int n_rows, int d, float eps, void* stream) {
    if (!x || !gain || !y || n_rows < 0 || d <= 0 || !(eps > 0.f)) return SPITE_BAD_ARG;
    if (n_rows == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (out_dtype != SPITE_DT_F32 && out_dtype != SPITE_DT_BF16) return SPITE_BAD_ARG;
    const bool f32 = out_dtype == SPITE_DT_F32;
    const bool aligned = d % 4 == 0 && ((((uintptr_t)x | (uintptr_t)gain | (uintptr_t)y) & 15) == 0);
    if (aligned && d <= 256 * 4 * 8) {
        // threads and groups per thread so that every thread has work: 128 x 1 up to 256 x 8
        const int d4 = d / 4;
        const int threads = d4 <= 128 ? 128 : 256;
        const int vpt = (d4 + threads - 1) / threads;
#define SPITE_RMS(V)                                                                                              \
        if (f32) SPITE_LAUNCH((rms_norm_vec_kernel<float, V>), n_rows, threads, 0, st, x, gain, rows, (float*)y, d, eps); \
        else SPITE_LAUNCH((rms_norm_vec_kernel<__nv_bfloat16, V>), n_rows, threads, 0, st, x, gain, rows, (__nv_bfloat16*)y, d, eps)
        if (vpt <= 1) { SPITE_RMS(1); }
        else if (vpt <= 2) { SPITE_RMS(2); }
        else if (vpt <= 4) { SPITE_RMS(4); }
        else if (vpt <= 5) { SPITE_RMS(5); }
        else { SPITE_RMS(8); }
#undef SPITE_RMS
        return spite_launch_status();
    }
    const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
    if (f32)
        SPITE_LAUNCH(rms_norm_kernel<float>, n_rows, threads, 0, st, x, gain, rows, (float*)y, d, eps);
    else
        SPITE_LAUNCH(rms_norm_kernel<__nv_bfloat16>, n_rows, threads, 0, st, x, gain, rows, (__nv_bfloat16*)y, d, eps);
    return spite_launch_status();
}
