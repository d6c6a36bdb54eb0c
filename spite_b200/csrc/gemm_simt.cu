// Matrix product on the CUDA cores with float32 multiply-adds.
//
// This is the kernel of the true 32-bit path (inputs, products, sums and outputs
// are IEEE float32; no tensor-core mode is involved) and the fallback of the
// bfloat16 path for shapes the tensor-core kernels refuse.  Every output element
// is summed over k in ascending order by one thread, so its value does not depend
// on how many rows the call has or which tile it falls into.
//
// Formula: crates/spite-models/src/dense.rs:224-270 (`out[r] = sum_c w[r,c] x[c]`).
#include "gemm.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename T, int EPI>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const GemmParams p) {
    constexpr bool DUAL = (EPI == EPI_SWIGLU);
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[DUAL ? 2 : 1][BK][BN + 4];
    __shared__ int a_row_s[BM];
    pdl_wait();
    pdl_launch_dependents();

    int group, row0, rows;
    if (!locate_row_tile(p, blockIdx.y, BM, group, row0, rows)) return;
    const int n0 = blockIdx.x * BN;
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;

    const T* A = (const T*)p.A;
    const T* W = (const T*)p.W + (size_t)group * p.w_group_stride;
    if (tid < BM) {
        const int i = row0 + tid;
        a_row_s[tid] = (tid < rows) ? (p.a_rows ? p.a_rows[i] : i) : -1;
    }
    __syncthreads();

    float acc[DUAL ? 2 : 1][TM][TN];
#pragma unroll
    for (int h = 0; h < (DUAL ? 2 : 1); ++h)
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) acc[h][i][j] = 0.f;

    const int lr = tid >> 2;          // tile row (A) or tile column (W) this thread loads
    const int lk = (tid & 3) * 4;     // first k of its 4 consecutive elements
    for (int k0 = 0; k0 < p.K; k0 += BK) {
        {
            const int ar = a_row_s[lr];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int k = k0 + lk + e;
                As[lk + e][lr] = (ar >= 0 && k < p.K) ? to_f32(A[(size_t)ar * p.lda + k]) : 0.f;
            }
            const int n = n0 + lr;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int k = k0 + lk + e;
                const bool ok = n < p.N && k < p.K;
                Ws[0][lk + e][lr] = ok ? to_f32(W[(size_t)n * p.K + k]) : 0.f;
                if (DUAL) Ws[DUAL ? 1 : 0][lk + e][lr] = ok ? to_f32(W[(size_t)(n + p.N) * p.K + k]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[0][k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[0][i][j] = fmaf(a[i], w[j], acc[0][i][j]);
            if (DUAL) {
#pragma unroll
                for (int j = 0; j < TN; ++j) w[j] = Ws[DUAL ? 1 : 0][k][tx * TN + j];
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j)
                        acc[DUAL ? 1 : 0][i][j] = fmaf(a[i], w[j], acc[DUAL ? 1 : 0][i][j]);
            }
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = ty * TM + i;
        if (r >= rows) continue;
        const int li = row0 + r;
        const int crow = p.c_rows ? p.c_rows[li] : li;
        float s = 1.f;
        if (p.row_scale) s = p.row_scale[p.scale_by_a_row ? a_row_s[r] : li];
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= p.N) continue;
            const size_t o = (size_t)crow * p.ldc + n;
            if (EPI == EPI_STORE) ((T*)p.C)[o] = from_f32<T>(acc[0][i][j] * s);
            else if (EPI == EPI_STORE_F32) ((float*)p.C)[o] = acc[0][i][j] * s;
            else if (EPI == EPI_ADD_F32) ((float*)p.C)[o] += acc[0][i][j] * s;
            else ((T*)p.C)[o] = from_f32<T>(silu_f32(acc[0][i][j] * s) * (acc[DUAL ? 1 : 0][i][j] * s));
        }
    }
}

template <typename T>
int launch(const GemmParams& p, cudaStream_t st) {
    const int row_tiles = (p.M + BM - 1) / BM + (p.group_offsets ? p.n_groups : 0);
    dim3 grid((p.N + BN - 1) / BN, row_tiles);
    if (grid.y > 65535) return SPITE_UNSUPPORTED;
    switch (p.epilogue) {
        case EPI_STORE: SPITE_LAUNCH((gemm_simt_kernel<T, EPI_STORE>), grid, 256, 0, st, p); break;
        case EPI_STORE_F32: SPITE_LAUNCH((gemm_simt_kernel<T, EPI_STORE_F32>), grid, 256, 0, st, p); break;
        case EPI_ADD_F32: SPITE_LAUNCH((gemm_simt_kernel<T, EPI_ADD_F32>), grid, 256, 0, st, p); break;
        case EPI_SWIGLU: SPITE_LAUNCH((gemm_simt_kernel<T, EPI_SWIGLU>), grid, 256, 0, st, p); break;
        default: return SPITE_BAD_ARG;
    }
    return spite_launch_status();
}

}  // namespace

int gemm_check(const GemmParams* p) {
    if (!p || !p->A || !p->W || !p->C) return SPITE_BAD_ARG;
    if (p->M < 0 || p->N <= 0 || p->K <= 0 || p->lda < p->K) return SPITE_BAD_ARG;
    if (p->group_offsets ? p->n_groups < 1 : p->n_groups != 1) return SPITE_BAD_ARG;
    if (p->epilogue < 0 || p->epilogue > EPI_SWIGLU || p->ldc < p->N) return SPITE_BAD_ARG;
    return SPITE_OK;
}

SPITE_API int spite_gemm_simt(int dtype, const GemmParams* p, void* stream) {
    const int c = gemm_check(p);
    if (c != SPITE_OK) return c;
    if (p->M == 0) return SPITE_OK;
    if (dtype == SPITE_DT_F32) return launch<float>(*p, (cudaStream_t)stream);
    if (dtype == SPITE_DT_BF16) return launch<__nv_bfloat16>(*p, (cudaStream_t)stream);
    return SPITE_BAD_ARG;
}
