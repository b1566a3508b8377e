// float32 matrix products on the CUDA cores: y = x . W^T with x [M, K] and W [N, K], both
// row-major (the layout of F.linear in engine/model.py:194, 208, 210-211, 218).  This is the
// true 32-bit path: plain FMA, no tensor cores, no TF32.  Each output element is the sum
// over k = 0 .. K-1 in that order, so a row's result does not depend on how many other
// rows are in the call.
//
// Variant "swiglu": W has 2*N rows (gate rows first, then up rows); the kernel keeps two
// accumulators and writes silu(gate) * up, so the [M, 2N] intermediate never exists.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;  // 256 threads, 4x4 outputs each

// Four consecutive k of one row; `vec` = the row starts are 16-byte aligned and K % 4 == 0.
__device__ __forceinline__ float4 load_k4(const float* row, int k, int K, bool vec) {
    if (vec) return *reinterpret_cast<const float4*>(row + k);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (k < K) v.x = row[k];
    if (k + 1 < K) v.y = row[k + 1];
    if (k + 2 < K) v.z = row[k + 2];
    if (k + 3 < K) v.w = row[k + 3];
    return v;
}

template <bool SWIGLU>
__global__ void __launch_bounds__(256)
sgemm_tn_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C,
                int M, int N, int K, int lda, int ldw, int ldc, bool vec) {
    pdl_trigger();
    pdl_wait();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[SWIGLU ? 2 : 1][BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tr = tid / 16, tc = tid % 16;        // thread's place in the 16x16 grid of 4x4 tiles
    const int lrow = tid / 4, lk = (tid % 4) * 4;  // loader: row 0..63, k offset 0,4,8,12

    float acc[SWIGLU ? 2 : 1][TM][TN];
#pragma unroll
    for (int s = 0; s < (SWIGLU ? 2 : 1); ++s)
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) acc[s][i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            const int r = m0 + lrow, k = k0 + lk;
            if (r < M && k < K) v = load_k4(A + (size_t)r * lda, k, K, vec);
            As[lk][lrow] = v.x; As[lk + 1][lrow] = v.y; As[lk + 2][lrow] = v.z; As[lk + 3][lrow] = v.w;
        }
#pragma unroll
        for (int s = 0; s < (SWIGLU ? 2 : 1); ++s) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            const int r = n0 + lrow, k = k0 + lk;
            if (r < N && k < K) v = load_k4(W + ((size_t)s * N + r) * ldw, k, K, vec);
            Ws[s][lk][lrow] = v.x; Ws[s][lk + 1][lrow] = v.y; Ws[s][lk + 2][lrow] = v.z; Ws[s][lk + 3][lrow] = v.w;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[SWIGLU ? 2 : 1][TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][tr * TM + i];
#pragma unroll
            for (int s = 0; s < (SWIGLU ? 2 : 1); ++s)
#pragma unroll
                for (int j = 0; j < TN; ++j) b[s][j] = Ws[s][k][tc * TN + j];
#pragma unroll
            for (int s = 0; s < (SWIGLU ? 2 : 1); ++s)
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j) acc[s][i][j] = fmaf(a[i], b[s][j], acc[s][i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = m0 + tr * TM + i;
        if (r >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int c = n0 + tc * TN + j;
            if (c >= N) continue;
            float v = acc[0][i][j];
            if (SWIGLU) v = v / (1.0f + expf(-v)) * acc[SWIGLU ? 1 : 0][i][j];
            C[(size_t)r * ldc + c] = v;
        }
    }
}

}  // namespace

// C[M, N] = A[M, K] . W[N, K]^T            (swiglu == 0)
// C[M, N] = silu(A . W[0:N]^T) * (A . W[N:2N]^T)   (swiglu != 0, W has 2N rows)
LLM_API int llm_gemm_f32(const float* A, const float* W, float* C, int M, int N, int K, int lda, int ldw,
                         int ldc, int swiglu, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    const bool vec = !(K % 4 || lda % 4 || ldw % 4) && !((uintptr_t)A & 15) && !((uintptr_t)W & 15);
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) LLM_FAIL(-1, "gemm_f32: M %d is too large", M);
    if (swiglu)
        llm_launch(sgemm_tn_kernel<true>, grid, 256, 0, stream, A, W, C, M, N, K, lda, ldw, ldc, vec);
    else
        llm_launch(sgemm_tn_kernel<false>, grid, 256, 0, stream, A, W, C, M, N, K, lda, ldw, ldc, vec);
    LLM_CHECK_LAUNCH("gemm_f32");
    return 0;
}

LLM_TRACE_EXPORT(gemm_f32)
