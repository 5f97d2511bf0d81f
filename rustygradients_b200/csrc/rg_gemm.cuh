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

#include <algorithm>

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
    int splitk;         // > 1 (single-matrix calls only): blockIdx.z is a k-range; raw partial tiles go to
    long long split_stride;  // C + z * split_stride and rg_gemm_splitk_reduce_kernel finishes the job
};

template <typename WT>
__global__ void __launch_bounds__(256) rg_gemm_kernel(rg_gemm_args p) {
    __shared__ float As[RG_GEMM_BK][RG_GEMM_BM + 4];
    __shared__ float Ws[RG_GEMM_BK][RG_GEMM_BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * RG_GEMM_BM, n0 = blockIdx.x * RG_GEMM_BN;
    const bool split = p.splitk > 1;
    const float* A = p.A + (split ? 0 : (long long)blockIdx.z * p.strideA);
    const WT* W = static_cast<const WT*>(p.W) + (split ? 0 : (long long)blockIdx.z * p.strideW);
    float* C = p.C + (split ? (long long)blockIdx.z * p.split_stride : (long long)blockIdx.z * p.strideC);
    int kbeg = 0, kend = p.K;
    if (split) {
        const int per = ((p.K + p.splitk - 1) / p.splitk + RG_GEMM_BK - 1) / RG_GEMM_BK * RG_GEMM_BK;
        kbeg = blockIdx.z * per;
        kend = min(p.K, kbeg + per);
    }

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    const int a_row = tid >> 2, a_k = (tid & 3) * 4;  // 64 rows x 16 k
    const int w_k = tid >> 4, w_n = (tid & 15) * 4;   // 16 k x 64 n

    for (int k0 = kbeg; k0 < kend; k0 += RG_GEMM_BK) {
        {
            const int m = m0 + a_row;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int k = k0 + a_k + j;
                As[a_k + j][a_row] = (m < p.M && k < kend) ? A[(long long)m * p.lda + k] : 0.f;
            }
            const int k = k0 + w_k;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int n = n0 + w_n + j;
                Ws[w_k][w_n + j] = (k < kend && n < p.N) ? rg_to_float(W[(long long)k * p.ldw + n]) : 0.f;
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
            if (split) {
                C[(long long)m * p.N + n] = v;
                continue;
            }
            if (p.bias) v += p.bias[n];
            if (p.act >= 0) v = rg_apply_act(v, p.act);
            if (p.res) v += p.res[(long long)m * p.ldres + n];
            C[(long long)m * p.ldc + n] = v;
        }
    }
}

// C[m][n] = epi(sum over the k-splits of ws[z][m][n]), fixed order
static __global__ void rg_gemm_splitk_reduce_kernel(const float* __restrict__ ws, int splits, int M, int N, float* __restrict__ C,
                                                    long long ldc, const float* __restrict__ bias,
                                                    const float* __restrict__ res, long long ldres, int act) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)M * N) return;
    const int m = (int)(i / N), n = (int)(i - (size_t)m * N);
    float v = 0.f;
    for (int z = 0; z < splits; z++) v += ws[(size_t)z * M * N + i];
    if (bias) v += bias[n];
    if (act >= 0) v = rg_apply_act(v, act);
    if (res) v += res[(long long)m * ldres + n];
    C[(long long)m * ldc + n] = v;
}

// ws: optional split-k workspace (ws_floats floats).  When the tile grid would leave most SMs idle the k range is
// split over blockIdx.z and a second kernel sums the partial tiles in a fixed order and applies the epilogue.
template <typename WT>
static inline cudaError_t rg_gemm_launch(cudaStream_t s, const rg_gemm_args& p0, int batch, float* ws = nullptr,
                                         size_t ws_floats = 0, int sm_count = 148, int* launches = nullptr) {
    if (p0.M <= 0 || p0.N <= 0 || batch <= 0) return cudaSuccess;
    rg_gemm_args p = p0;
    p.splitk = 1, p.split_stride = 0;
    const int tiles = rg_cdiv(p.N, RG_GEMM_BN) * rg_cdiv(p.M, RG_GEMM_BM);
    int splits = 1;
    if (batch == 1 && ws && tiles * 2 <= sm_count) {
        splits = std::min(std::min(sm_count / tiles, p.K / (4 * RG_GEMM_BK)), 16);
        while (splits > 1 && (size_t)splits * p.M * p.N > ws_floats) splits--;
        if (splits < 2) splits = 1;
    }
    if (splits > 1) {
        const int per = ((p.K + splits - 1) / splits + RG_GEMM_BK - 1) / RG_GEMM_BK * RG_GEMM_BK;
        splits = (p.K + per - 1) / per;
    }
    if (splits <= 1) {
        dim3 grid(rg_cdiv(p.N, RG_GEMM_BN), rg_cdiv(p.M, RG_GEMM_BM), batch);
        rg_gemm_kernel<WT><<<grid, 256, 0, s>>>(p);
        if (launches) *launches = 1;
        return cudaGetLastError();
    }
    p.splitk = splits, p.split_stride = (long long)p.M * p.N, p.C = ws;
    dim3 grid(rg_cdiv(p.N, RG_GEMM_BN), rg_cdiv(p.M, RG_GEMM_BM), splits);
    rg_gemm_kernel<WT><<<grid, 256, 0, s>>>(p);
    rg_gemm_splitk_reduce_kernel<<<rg_cdiv((long long)p.M * p.N, 256), 256, 0, s>>>(ws, splits, p.M, p.N, p0.C, p0.ldc, p0.bias, p0.res,
                                                                                  p0.ldres, p0.act);
    if (launches) *launches = 2;
    return cudaGetLastError();
}
