// Kernels of the prompt pass / full forward (many rows per sequence).
#pragma once
#include "rg_internal.cuh"

// x[b,t,:] = wte[id[b,t]] + wpe[t]   (src/models/gpt.rs:62-75)
template <typename WT>
__global__ void rg_embed_rows_kernel(const uint32_t* __restrict__ tokens, int C, int T, const WT* __restrict__ wte,
                                     const WT* __restrict__ wpe, int D, long long ldt, float* __restrict__ x) {
    const int row = blockIdx.x;  // b*T + t
    const int b = row / T, t = row - b * T;
    const uint32_t tok = tokens[(size_t)b * C + t];
    for (int d = threadIdx.x; d < D; d += blockDim.x)
        x[(size_t)row * D + d] = rg_to_float(wte[(size_t)tok * ldt + d]) + rg_to_float(wpe[(size_t)t * ldt + d]);
}

// LayerNorm of `rows` rows (one warp each, Welford statistics); row r is read at
// x + r*ldx so the last-row-only path can stride over [B,T,D].
static __global__ void __launch_bounds__(256) rg_ln_rows_kernel(const float* __restrict__ x, long long ldx,
                                                                const float* __restrict__ gamma,
                                                                const float* __restrict__ beta, float* __restrict__ y,
                                                                size_t rows, int n, float eps) {
    const size_t row = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float* xr = x + row * ldx;
    float* yr = y + row * n;
    // per-lane Welford over a strided subset costs a division per element; a lane's (count, mean, M2) is
    // obtained instead from shifted sums with c = x[0] (exactly the quantities Welford maintains), then the
    // 32 lanes are merged pairwise with Chan's formula as before
    const float c = xr[0];
    float s1 = 0.f, s2 = 0.f, cnt = 0.f;
    for (int i = lane; i < n; i += 32) {
        const float d = xr[i] - c;
        s1 += d;
        s2 = fmaf(d, d, s2);
        cnt += 1.f;
    }
    rg_welford w;
    w.n = cnt;
    const float m1 = cnt > 0.f ? s1 / cnt : 0.f;
    w.mean = c + m1;
    w.m2 = fmaxf(s2 - s1 * m1, 0.f);
    w = rg_welford_warp(w);
    const float inv = 1.f / sqrtf(w.m2 / (float)n + eps);
    for (int i = lane; i < n; i += 32) yr[i] = (xr[i] - w.mean) * inv * gamma[i] + beta[i];
}

// k, v columns of qkv[B*T, 3D] -> cache [B][H][C][hd] (positions 0..T-1).
template <typename KT>
__global__ void rg_kv_scatter_kernel(const float* __restrict__ qkv, KT* __restrict__ kc, KT* __restrict__ vc, int T,
                                     int H, int hd, int C, int D) {
    const int row = blockIdx.x;  // b*T + t
    const int b = row / T, t = row - b * T;
    const float* src = qkv + (size_t)row * 3 * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const int h = i / hd, d = i - h * hd;
        const size_t dst = (((size_t)b * H + h) * C + t) * hd + d;
        if (sizeof(KT) == 4) {
            reinterpret_cast<float*>(kc)[dst] = src[D + i];
            reinterpret_cast<float*>(vc)[dst] = src[2 * D + i];
        } else {
            reinterpret_cast<__nv_bfloat16*>(kc)[dst] = __float2bfloat16_rn(src[D + i]);
            reinterpret_cast<__nv_bfloat16*>(vc)[dst] = __float2bfloat16_rn(src[2 * D + i]);
        }
    }
}

// Attention over T rows per head (src/nn/attention.rs:78-94): S = q.k^T, scale,
// optional causal mask, row softmax (max-subtracted), P.v; heads merged back to
// [B*T, D].  grid = (ceil(T/8), H, B); one warp per query row, keys staged in
// shared memory 32 at a time and shared by the 8 rows of the CTA.
template <typename KT, int HD>
__global__ void __launch_bounds__(256) rg_attn_rows_kernel(const float* __restrict__ qkv, const KT* __restrict__ kc,
                                                           const KT* __restrict__ vc, float* __restrict__ out, int T,
                                                           int H, int C, int D, float scale, int causal) {
    constexpr int DPL = HD / 32;  // output dims per lane
    __shared__ float Ks[32][HD + 1];
    __shared__ float Vs[32][HD];
    __shared__ float Qs[8][HD];
    const int h = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tq = blockIdx.x * 8 + warp;
    const bool row_ok = tq < T;
    if (row_ok)
        for (int d = lane; d < HD; d += 32) Qs[warp][d] = qkv[((size_t)b * T + tq) * 3 * D + h * HD + d];
    const KT* kb = kc + ((size_t)b * H + h) * C * HD;
    const KT* vb = vc + ((size_t)b * H + h) * C * HD;
    const int tmax = causal ? min(T, blockIdx.x * 8 + 8) : T;  // keys any row of this CTA may see
    float m = -INFINITY, l = 0.f, acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; i++) acc[i] = 0.f;

    for (int j0 = 0; j0 < tmax; j0 += 32) {
        __syncthreads();
        for (int i = threadIdx.x; i < 32 * HD; i += 256) {
            const int r = i / HD, d = i - r * HD;
            const int t = j0 + r;
            Ks[r][d] = t < tmax ? rg_to_float(kb[(size_t)t * HD + d]) : 0.f;
            Vs[r][d] = t < tmax ? rg_to_float(vb[(size_t)t * HD + d]) : 0.f;
        }
        __syncthreads();
        if (!row_ok) continue;
        const int t = j0 + lane;
        float sc = 0.f;
#pragma unroll 8
        for (int d = 0; d < HD; d++) sc = fmaf(Qs[warp][d], Ks[lane][d], sc);
        sc *= scale;
        const bool visible = t < T && (!causal || t <= tq);
        if (!visible) sc = -INFINITY;
        const float tile_max = rg_warp_max(sc);
        if (tile_max == -INFINITY) continue;  // nothing visible in this tile (warp-uniform)
        const float mn = fmaxf(m, tile_max);
        const float corr = __expf(m - mn);
        const float pr = visible ? __expf(sc - mn) : 0.f;
        l = l * corr + rg_warp_sum(pr);
#pragma unroll
        for (int i = 0; i < DPL; i++) acc[i] *= corr;
        for (int j = 0; j < 32; j++) {
            const float pj = __shfl_sync(RG_FULL_MASK, pr, j);
#pragma unroll
            for (int i = 0; i < DPL; i++) acc[i] = fmaf(pj, Vs[j][lane + 32 * i], acc[i]);
        }
        m = mn;
    }
    if (row_ok) {
        const float inv = 1.f / l;
#pragma unroll
        for (int i = 0; i < DPL; i++) out[((size_t)b * T + tq) * D + h * HD + lane + 32 * i] = acc[i] * inv;
    }
}

// Copy row T-1 of every sequence: x[B*T, D] -> y[B, D].
static __global__ void rg_last_rows_kernel(const float* __restrict__ x, float* __restrict__ y, int T, int D) {
    const int b = blockIdx.x;
    for (int d = threadIdx.x; d < D; d += blockDim.x) y[(size_t)b * D + d] = x[((size_t)b * T + T - 1) * D + d];
}

// Greedy pick over finished logits rows [B][V]; lowest index on ties.  Writes the
// pick to tokens[b][slot] when slot < C.
static __global__ void __launch_bounds__(1024) rg_argmax_rows_kernel(const float* __restrict__ logits, int V,
                                                                     uint32_t* __restrict__ picks,
                                                                     uint32_t* __restrict__ tokens, int C, int slot) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    const int b = blockIdx.x, tid = threadIdx.x;
    float best = -INFINITY;
    int besti = 0x7fffffff;
    for (int v = tid; v < V; v += blockDim.x) {
        const float x = logits[(size_t)b * V + v];
        if (x > best) best = x, besti = v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(RG_FULL_MASK, best, o);
        const int oi = __shfl_xor_sync(RG_FULL_MASK, besti, o);
        if (ov > best || (ov == best && oi < besti)) best = ov, besti = oi;
    }
    if ((tid & 31) == 0) bv[tid >> 5] = best, bi[tid >> 5] = besti;
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); w++)
            if (bv[w] > best || (bv[w] == best && bi[w] < besti)) best = bv[w], besti = bi[w];
        if (besti == 0x7fffffff) besti = 0;
        picks[b] = (uint32_t)besti;
        if (slot < C) tokens[(size_t)b * C + slot] = (uint32_t)besti;
    }
}
