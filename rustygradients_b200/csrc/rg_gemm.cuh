// FP32-accurate tiled GEMM on the CUDA cores, used where the path is a dense
// contraction that must keep f32 parity: the prompt pass (Linear::forward on
// [B*T, in] rows, src/nn/linear.rs:50-56 -> src/ops/matmul.rs:51-72) and the
// Backend::matmul op (src/backend/cpu.rs:82-208).
//
//   C[z][m][n] = epi( sum_k A[z][m][k] * W[z][k][n] )
//   epi(v)     = act(v + bias[n]) + res[m][n]        (each part optional)
//
// W is row-major [K,N] like the reference's Linear weight ([in,out]); it may be
// f32 or bf16 (converted while staging into shared memory).  Accumulation is
// f32 FMA in k order inside a 64x64x16 tile.
#pragma once
#include "rg_internal.cuh"

#define RG_GEMM_BM 64
#define RG_GEMM_BN 64
#define RG_GEMM_BK 16

struct rg_gemm_args {
    const float* A;
    long long lda, strideA;
    const void* W;
    long long ldw, strideW;
    float* C;
    long long ldc, strideC;
    int M, N, K;
    const float* bias;  // [N] or null
    const float* res;   // [M][ldres] or null (may alias C)
    long long ldres;
    int act;            // -1 none, RG_ACT_RELU, RG_ACT_GELU_TANH
};

template <typename WT>
__global__ void __launch_bounds__(256) rg_gemm_kernel(rg_gemm_args p) {
    __shared__ float As[RG_GEMM_BK][RG_GEMM_BM + 4];
    __shared__ float Ws[RG_GEMM_BK][RG_GEMM_BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * RG_GEMM_BM, n0 = blockIdx.x * RG_GEMM_BN;
    const float* A = p.A + (long long)blockIdx.z * p.strideA;
    const WT* W = static_cast<const WT*>(p.W) + (long long)blockIdx.z * p.strideW;
    float* C = p.C + (long long)blockIdx.z * p.strideC;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    const int a_row = tid >> 2, a_k = (tid & 3) * 4;  // 64 rows x 16 k
    const int w_k = tid >> 4, w_n = (tid & 15) * 4;   // 16 k x 64 n

    for (int k0 = 0; k0 < p.K; k0 += RG_GEMM_BK) {
        {
            const int m = m0 + a_row;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int k = k0 + a_k + j;
                As[a_k + j][a_row] = (m < p.M && k < p.K) ? A[(long long)m * p.lda + k] : 0.f;
            }
            const int k = k0 + w_k;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int n = n0 + w_n + j;
                Ws[w_k][w_n + j] = (k < p.K && n < p.N) ? rg_to_float(W[(long long)k * p.ldw + n]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < RG_GEMM_BK; kk++) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + ty * 4 + i;
        if (m >= p.M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n >= p.N) continue;
            float v = acc[i][j];
            if (p.bias) v += p.bias[n];
            if (p.act >= 0) v = rg_apply_act(v, p.act);
            if (p.res) v += p.res[(long long)m * p.ldres + n];
            C[(long long)m * p.ldc + n] = v;
        }
    }
}

template <typename WT>
static inline cudaError_t rg_gemm_launch(cudaStream_t s, const rg_gemm_args& p, int batch) {
    if (p.M <= 0 || p.N <= 0 || batch <= 0) return cudaSuccess;
    dim3 grid(rg_cdiv(p.N, RG_GEMM_BN), rg_cdiv(p.M, RG_GEMM_BM), batch);
    rg_gemm_kernel<WT><<<grid, 256, 0, s>>>(p);
    return cudaGetLastError();
}
