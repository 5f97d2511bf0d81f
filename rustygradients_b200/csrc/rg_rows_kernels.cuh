// Kernels between the tensor-core projections of the GEMM-form token step (batches of 8 or more
// sequences, bf16 weights).  A projection with few rows is split over k; its raw partial tiles are summed
// here, in a fixed order, fused with whatever follows the projection in the block
// (src/nn/transformer.rs:51-65): bias + residual + the next LayerNorm (src/ops/norm.rs:41-52), or bias +
// activation (src/nn/feedforward.rs:43-45), and the result is written as the bf16 input rows of the next
// projection.  One CTA of 256 threads per row where a row statistic is needed.
#pragma once
#include "rg_internal.cuh"

__device__ __forceinline__ float rg_block_sum_256(float v, float* sm8) {
    v = rg_warp_sum(v);
    __syncthreads();  // sm8 may still be read from a previous call
    if ((threadIdx.x & 31) == 0) sm8[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) s += sm8[w];
    return s;
}

#define RG_ROWS_MAX_D 2048  // 8 values per thread

// v = x + bias + sum of the k-split partials (all optional but x); x <- v when store_x; out16 <- LN(v; gamma, beta).
// Two-pass statistics on the values held in registers: mean, then the biased variance of (v - mean).
static __global__ void __launch_bounds__(256) rg_rows_res_ln_bf16_kernel(const float* __restrict__ parts, int nparts, size_t pstride,
                                                                         const float* __restrict__ bias, float* __restrict__ x,
                                                                         int store_x, const float* __restrict__ gamma,
                                                                         const float* __restrict__ beta,
                                                                         __nv_bfloat16* __restrict__ out16, int D) {
    rg_pdl_sync();
    __shared__ float sm8[8];
    const size_t row = blockIdx.x;
    float v[RG_ROWS_MAX_D / 256];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < RG_ROWS_MAX_D / 256; i++) {
        const int k = threadIdx.x + i * 256;
        v[i] = 0.f;
        if (k < D) {
            float t = x[row * D + k];
            if (bias) t += bias[k];
            t += rg_sum_parts(parts + row * D + k, nparts, pstride);
            if (store_x) x[row * D + k] = t;
            v[i] = t;
            s += t;
        }
    }
    const float mean = rg_block_sum_256(s, sm8) / (float)D;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < RG_ROWS_MAX_D / 256; i++) {
        const int k = threadIdx.x + i * 256;
        if (k < D) q = fmaf(v[i] - mean, v[i] - mean, q);
    }
    const float rstd = 1.f / sqrtf(rg_block_sum_256(q, sm8) / (float)D + 1e-5f);
#pragma unroll
    for (int i = 0; i < RG_ROWS_MAX_D / 256; i++) {
        const int k = threadIdx.x + i * 256;
        if (k < D) out16[row * D + k] = __float2bfloat16_rn((v[i] - mean) * rstd * gamma[k] + beta[k]);
    }
}

// out16[m][n] = act(bias[n] + sum of the partials)
static __global__ void rg_rows_act_bf16_kernel(const float* __restrict__ parts, int nparts, size_t pstride,
                                               const float* __restrict__ bias, int N, size_t total, int act,
                                               __nv_bfloat16* __restrict__ out16) {
    rg_pdl_sync();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    float v = bias ? bias[i % N] : 0.f;
    v += rg_sum_parts(parts + i, nparts, pstride);
    if (act >= 0) v = rg_apply_act(v, act);
    out16[i] = __float2bfloat16_rn(v);
}
