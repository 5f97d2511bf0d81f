// Kernels of the KV-cache token step (one new token per sequence).
//
// Conventions shared by all of them:
//  * Linear weights are row-major [in,out] (= [K,N]) like the reference
//    (src/nn/linear.rs:14-19), leading dimension padded to a multiple of 8
//    elements so every 16-byte vector load is aligned and in bounds.
//  * A projection is split over column tiles AND over k-ranges.  Each CTA writes
//    its partial dot products to parts[ksplit][B][N]; nothing is accumulated with
//    atomics.  The consumer of a vector sums the partials in a fixed order while
//    it loads them, so results are bit-reproducible run to run.
//  * The position of the step lives in device memory (pos[0]) so the same
//    launch sequence can be replayed from a CUDA graph.
#pragma once
#include "rg_internal.cuh"

// ---------------------------------------------------------------------------
// how a projection receives its input vector
// ---------------------------------------------------------------------------
enum { RG_IN_REDUCE = 0, RG_IN_ATTN = 1 };
enum { RG_POST_NONE = 0, RG_POST_LN = 1, RG_POST_RELU = 2, RG_POST_GELU = 3 };

struct rg_vec_in {
    int kind;            // RG_IN_REDUCE: v = base + bias + sum(parts); RG_IN_ATTN: merge of split-T attention partials
    const float* base;   // [B][K] or null
    const float* bias;   // [K] or null
    const float* parts;  // [nparts][B][K]
    int nparts;
    int post;            // RG_POST_*
    const float* gamma;  // LayerNorm scale / shift when post == RG_POST_LN
    const float* beta;
    float* store;        // [B][K] or null: where v (before post) is kept as the new residual stream
    const float* ap;     // [B][H][NS][hd+2] attention partials (m, l, o[hd])
    int H, hd, NS;
};

struct rg_gemv_args {
    rg_vec_in in;
    const void* W;
    long long ldw;
    int K, N, B;
    int ksplit, krows;   // k-range of CTA y: [y*krows, min(K,(y+1)*krows))
    float* out;          // [ksplit][B][N]
};

// v[b][k] of the input vector, reduced in fixed order.
__device__ __forceinline__ float rg_vec_in_value(const rg_vec_in& in, int B, int K, int b, int k) {
    if (in.kind == RG_IN_REDUCE) {
        float v = in.base ? in.base[(size_t)b * K + k] : 0.f;
        if (in.bias) v += in.bias[k];
        return v + rg_sum_parts(in.parts + (size_t)b * K + k, in.nparts, (size_t)B * K);
    } else {
        const int h = k / in.hd, d = k - h * in.hd;
        const int rec = in.hd + 2;
        const float* p = in.ap + ((size_t)(b * in.H + h) * in.NS) * rec;
        float M = -INFINITY;
        for (int s = 0; s < in.NS; s++) M = fmaxf(M, p[s * rec]);
        if (M == -INFINITY) return 0.f;
        float num = 0.f, den = 0.f;
        for (int s = 0; s < in.NS; s++) {
            const float w = __expf(p[s * rec] - M);
            num += w * p[s * rec + 2 + d];
            den += w * p[s * rec + 1];
        }
        return num / den;
    }
}

template <typename WT>
struct rg_wvec;
template <>
struct rg_wvec<float> {
    static constexpr int N = 4;
    __device__ __forceinline__ static void load(const float* p, float (&w)[4]) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(p));
        w[0] = v.x, w[1] = v.y, w[2] = v.z, w[3] = v.w;
    }
};
template <>
struct rg_wvec<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ __forceinline__ static void load(const __nv_bfloat16* p, float (&w)[8]) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
        const unsigned int u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            w[2 * i] = __uint_as_float(u[i] << 16);
            w[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
        }
    }
};

// ---------------------------------------------------------------------------
// Fused [reduce partials (+bias +residual) -> LayerNorm | activation | attention
// merge] -> x.W for up to BT sequences.  Replaces, per call site, LayerNorm::forward
// + Linear::forward (src/nn/norm.rs:53-57, src/nn/linear.rs:50-56) or relu/GELU +
// Linear::forward (src/nn/feedforward.rs:40-48) of the reference for a single row.
//
// grid = (column tiles, k splits, batch tiles); 256 threads: the 8 warps take
// interleaved k rows of the tile, a lane owns 16 bytes of consecutive columns, so a
// warp reads 512 contiguous bytes of one weight row per load.
// ---------------------------------------------------------------------------
template <typename WT, int BT>
__global__ void __launch_bounds__(256) rg_gemv_kernel(rg_gemv_args p) {
    rg_pdl_sync();
    constexpr int VEC = rg_wvec<WT>::N;
    constexpr int NT = 32 * VEC;
    extern __shared__ float smem[];
    __shared__ float red[8][NT];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b0 = blockIdx.z * BT;
    const int nb = min(BT, p.B - b0);
    const int k0 = blockIdx.y * p.krows;
    const int k1 = min(p.K, k0 + p.krows);
    const bool ln = p.in.post == RG_POST_LN;
    const int xk0 = ln ? 0 : k0;               // first k held in xs
    const int xlen = ln ? p.K : (k1 - k0);
    float* xs = smem;                          // [BT][xlen]

    // ---- input vector ----
    for (int b = 0; b < nb; b++) {
        for (int i = tid; i < xlen; i += 256) {
            const int k = xk0 + i;
            float v = rg_vec_in_value(p.in, p.B, p.K, b0 + b, k);
            if (ln && p.in.store && blockIdx.x == 0 && blockIdx.y == 0) p.in.store[(size_t)(b0 + b) * p.K + k] = v;
            if (p.in.post == RG_POST_RELU) v = fmaxf(v, 0.f);
            else if (p.in.post == RG_POST_GELU) v = rg_gelu_tanh(v);
            xs[b * xlen + i] = v;
        }
    }
    __syncthreads();
    if (ln) {
        // one warp per sequence: Welford over the row, then normalise in place
        for (int b = warp; b < nb; b += 8) {
            float* xr = xs + b * xlen;
            rg_welford w = {0.f, 0.f, 0.f};
            for (int i = lane; i < p.K; i += 32) rg_welford_add(w, xr[i]);
            w = rg_welford_warp(w);
            const float inv = 1.f / sqrtf(w.m2 / (float)p.K + 1e-5f);
            for (int i = lane; i < p.K; i += 32) xr[i] = (xr[i] - w.mean) * inv * p.in.gamma[i] + p.in.beta[i];
        }
        __syncthreads();
    }

    // ---- partial dot products ----
    const int n = blockIdx.x * NT + lane * VEC;
    const bool col_ok = n < p.N;  // ldw is padded, so a vector that starts below N is readable
    const WT* W = static_cast<const WT*>(p.W) + n;
    float acc[BT][VEC];
#pragma unroll
    for (int b = 0; b < BT; b++)
#pragma unroll
        for (int j = 0; j < VEC; j++) acc[b][j] = 0.f;

    if (col_ok) {
        constexpr int U = 4;
        int k = k0 + warp;
        for (; k + 8 * (U - 1) < k1; k += 8 * U) {
            float w[U][VEC];
#pragma unroll
            for (int u = 0; u < U; u++) rg_wvec<WT>::load(W + (size_t)(k + 8 * u) * p.ldw, w[u]);
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int b = 0; b < BT; b++) {
                    const float xv = xs[b * xlen + (k + 8 * u - xk0)];
#pragma unroll
                    for (int j = 0; j < VEC; j++) acc[b][j] = fmaf(xv, w[u][j], acc[b][j]);
                }
        }
        for (; k < k1; k += 8) {
            float w[VEC];
            rg_wvec<WT>::load(W + (size_t)k * p.ldw, w);
#pragma unroll
            for (int b = 0; b < BT; b++) {
                const float xv = xs[b * xlen + (k - xk0)];
#pragma unroll
                for (int j = 0; j < VEC; j++) acc[b][j] = fmaf(xv, w[j], acc[b][j]);
            }
        }
    }

    // ---- combine the 8 warps in fixed order, one sequence at a time ----
#pragma unroll
    for (int b = 0; b < BT; b++) {
        if (b >= nb) break;
#pragma unroll
        for (int j = 0; j < VEC; j++) red[warp][lane * VEC + j] = acc[b][j];
        __syncthreads();
        for (int c = tid; c < NT; c += 256) {
            const int col = blockIdx.x * NT + c;
            if (col < p.N) {
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < 8; w++) s += red[w][c];
                p.out[((size_t)blockIdx.y * p.B + (b0 + b)) * p.N + col] = s;
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------
// Token + position embedding of the new token (src/models/gpt.rs:62-75 for one
// row).  Also publishes the step's position: it reads pos_next (written by the
// previous step's pick kernel) and stores it to pos, which every later kernel of
// the step reads.
// ---------------------------------------------------------------------------
template <typename WT>
__global__ void rg_embed_step_kernel(const uint32_t* __restrict__ tokens, int C, const WT* __restrict__ wte,
                                     const WT* __restrict__ wpe, int D, long long ldt, float* __restrict__ x,
                                     const int* __restrict__ pos_next, int* __restrict__ pos) {
    rg_pdl_sync();
    const int t = *pos_next;
    const int b = blockIdx.x;
    if (b == 0 && threadIdx.x == 0) *pos = t;
    const uint32_t tok = tokens[(size_t)b * C + t];
    for (int d = threadIdx.x; d < D; d += blockDim.x)
        x[(size_t)b * D + d] = rg_to_float(wte[(size_t)tok * ldt + d]) + rg_to_float(wpe[(size_t)t * ldt + d]);
}

// ---------------------------------------------------------------------------
// Attention of one new query row over the cached keys/values of its head
// (src/nn/attention.rs:78-94 restricted to the last row; rows above it are
// invisible, which is what makes the cache valid).  Split over the context:
// grid = (NS, H, B); CTA s covers positions [s*chunk, (s+1)*chunk) and emits a
// softmax partial (running max m, sum l, un-normalised output o[hd]).
// q, k, v of the new token arrive as split-k partials of the QKV projection and
// are reduced here (+bias); the CTA whose range holds the new position appends
// k, v to the cache.
// Cache layout: [B][H][C][hd] per layer, so one head's context is one
// contiguous stream.
// ---------------------------------------------------------------------------
struct rg_attn_step_args {
    const float* qkv_parts;  // [nparts][B][3D]
    int nparts;
    const float* qkv_bias;   // [3D]
    void* kcache;            // this layer: [B][H][C][hd]
    void* vcache;
    float* ap;               // [B][H][NS][hd+2]
    const int* pos;
    int B, H, C, D, NS;
    float scale;
    // With one slice per (sequence, head) the merge of slices is a division: when this is set (and NS == 1) the kernel
    // writes the finished head outputs o / l as bf16 rows [B][H * hd], the input of the out-projection, itself
    // (the same bits rg_attn_merge_kernel would produce from the record).
    __nv_bfloat16* out16 = nullptr;
};

#ifndef RG_ATTN_STEP_UNROLL
#define RG_ATTN_STEP_UNROLL 2
#endif
template <typename KT, int HD>
__global__ void __launch_bounds__(128) rg_attn_step_kernel(rg_attn_step_args p) {
    // Inside a launch chain this kernel may start while the QKV projection before it still runs.  The cached rows it
    // will stream do not depend on that projection, so the CTA asks for its slice of K and V to be brought into L2
    // before it waits.  The position read here may be one step old (the counter is advanced by an earlier kernel of the
    // chain): it only sizes the hint; everything that matters is read again after the wait.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 0) {
        const int hint = min(max(*reinterpret_cast<const volatile int*>(p.pos), 0), p.C - 1) + 1;
        const int hchunk = (hint + p.NS - 1) / p.NS;
        const int h0 = (int)blockIdx.x * hchunk, h1 = min(hint, h0 + hchunk);
        if (h0 < h1) {
            const size_t head = ((size_t)(blockIdx.z * p.H + blockIdx.y) * p.C + h0) * HD * sizeof(KT);
            const uint32_t bytes = (uint32_t)(h1 - h0) * HD * (uint32_t)sizeof(KT);
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(static_cast<const char*>(p.kcache) + head), "r"(bytes)
                         : "memory");
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(static_cast<const char*>(p.vcache) + head), "r"(bytes)
                         : "memory");
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    constexpr int VEC = 16 / sizeof(KT);  // elements per 16-byte load
    constexpr int LPR = HD / VEC;         // lanes per cached row
    constexpr int RPW = 32 / LPR;         // rows per warp per load
    constexpr int NG = 4 * RPW;           // lane groups per CTA
    __shared__ float sq[HD], sk[HD], sv[HD];
    __shared__ float gm[NG], gl[NG];
    __shared__ float go[NG][HD];

    const int s = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pos = *p.pos;
    const int T = pos + 1;
    const int chunk = (T + p.NS - 1) / p.NS;
    const int t0 = s * chunk;
    const int t1 = min(T, t0 + chunk);
    const int rec = HD + 2;
    float* out = p.ap + ((size_t)(b * p.H + h) * p.NS + s) * rec;
    if (t0 >= t1) {  // empty split
        if (tid == 0) out[0] = -INFINITY, out[1] = 0.f;
        for (int d = tid; d < HD; d += 128) out[2 + d] = 0.f;
        return;
    }
    // q (all CTAs) and the new k, v (all CTAs need k/v only if they own pos; cheap enough to reduce everywhere)
    const bool owns_new = (pos >= t0 && pos < t1);
    for (int i = tid; i < 3 * HD; i += 128) {
        const int which = i / HD, d = i - which * HD;
        if (which > 0 && !owns_new) continue;
        const int col = which * p.D + h * HD + d;
        float v = p.qkv_bias ? p.qkv_bias[col] : 0.f;
        v += rg_sum_parts(p.qkv_parts + (size_t)b * 3 * p.D + col, p.nparts, (size_t)p.B * 3 * p.D);
        if (which == 0) sq[d] = v;
        else if (which == 1) sk[d] = v;
        else sv[d] = v;
    }
    __syncthreads();
    KT* kc = static_cast<KT*>(p.kcache) + ((size_t)(b * p.H + h) * p.C) * HD;
    KT* vc = static_cast<KT*>(p.vcache) + ((size_t)(b * p.H + h) * p.C) * HD;
    if (owns_new) {
        for (int d = tid; d < HD; d += 128) {
            if (sizeof(KT) == 4) {
                reinterpret_cast<float*>(kc)[(size_t)pos * HD + d] = sk[d];
                reinterpret_cast<float*>(vc)[(size_t)pos * HD + d] = sv[d];
            } else {
                // the step attends to what later steps will read back: the rounded values
                const __nv_bfloat16 kb = __float2bfloat16_rn(sk[d]), vb = __float2bfloat16_rn(sv[d]);
                reinterpret_cast<__nv_bfloat16*>(kc)[(size_t)pos * HD + d] = kb;
                reinterpret_cast<__nv_bfloat16*>(vc)[(size_t)pos * HD + d] = vb;
                sk[d] = __bfloat162float(kb);
                sv[d] = __bfloat162float(vb);
            }
        }
        __syncthreads();
    }

    const int sub = lane % LPR, grp = lane / LPR;
    float qf[VEC];
#pragma unroll
    for (int j = 0; j < VEC; j++) qf[j] = sq[sub * VEC + j];
    float m = -INFINITY, l = 0.f, acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; j++) acc[j] = 0.f;

    // Several row groups per trip: all 16-byte loads of a trip are issued before anything is computed on them, which
    // multiplies the bytes a thread keeps in flight (the loop is bound by the latency of these loads, not by arithmetic).
    constexpr int UNR = RG_ATTN_STEP_UNROLL;
    for (int tb = t0 + warp * RPW; tb < t1; tb += UNR * 4 * RPW) {
        float kf[UNR][VEC], vf[UNR][VEC];
        bool okk[UNR];
#pragma unroll
        for (int u = 0; u < UNR; u++) {
            const int t = tb + u * 4 * RPW + grp;
            okk[u] = t < t1;
            if (okk[u] && t != pos) {
                rg_wvec<KT>::load(kc + (size_t)t * HD + sub * VEC, kf[u]);
                rg_wvec<KT>::load(vc + (size_t)t * HD + sub * VEC, vf[u]);
            } else {
#pragma unroll
                for (int j = 0; j < VEC; j++) {
                    kf[u][j] = okk[u] ? sk[sub * VEC + j] : 0.f;
                    vf[u][j] = okk[u] ? sv[sub * VEC + j] : 0.f;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < UNR; u++) {
            float dot = 0.f;
#pragma unroll
            for (int j = 0; j < VEC; j++) dot = fmaf(qf[j], kf[u][j], dot);
#pragma unroll
            for (int o = LPR / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(RG_FULL_MASK, dot, o);
            if (okk[u]) {
                const float sc = dot * p.scale;
                const float mn = fmaxf(m, sc);
                const float corr = __expf(m - mn), pr = __expf(sc - mn);
                l = l * corr + pr;
#pragma unroll
                for (int j = 0; j < VEC; j++) acc[j] = acc[j] * corr + pr * vf[u][j];
                m = mn;
            }
        }
    }
    // merge the lane groups of the CTA in fixed order
    const int g = warp * RPW + grp;
    if (sub == 0) gm[g] = m, gl[g] = l;
#pragma unroll
    for (int j = 0; j < VEC; j++) go[g][sub * VEC + j] = acc[j];
    __syncthreads();
    float M = -INFINITY;
    for (int i = 0; i < NG; i++) M = fmaxf(M, gm[i]);
    const bool finish = p.out16 != nullptr && p.NS == 1;
    float Lall = 0.f;
    if (finish)
        for (int i = 0; i < NG; i++)
            if (gm[i] != -INFINITY) Lall += __expf(gm[i] - M) * gl[i];
    for (int d = tid; d < HD; d += 128) {
        float o = 0.f;
        for (int i = 0; i < NG; i++)
            if (gm[i] != -INFINITY) o += __expf(gm[i] - M) * go[i][d];
        out[2 + d] = o;
        if (finish) p.out16[(size_t)(b * p.H + h) * HD + d] = __float2bfloat16_rn(o / Lall);
    }
    if (tid == 0) {
        float L = 0.f;
        for (int i = 0; i < NG; i++)
            if (gm[i] != -INFINITY) L += __expf(gm[i] - M) * gl[i];
        out[0] = M;
        out[1] = L;
    }
}

// ---------------------------------------------------------------------------
// Last stage of the step: logits = bias + sum of LM-head partials, greedy pick
// (= top_k 1 of src/wasm_api.rs:120-156; lowest index on ties), appended to the
// id buffer at pos+1.  One CTA per sequence.  Publishes pos_next.
// ---------------------------------------------------------------------------
struct rg_pick_args {
    const float* parts;  // [nparts][B][V]
    int nparts;
    const float* bias;   // [V]
    float* logits;       // [B][V]
    uint32_t* tokens;    // [B][C]
    uint32_t* picks;     // [B]
    const int* pos;
    int* pos_next;
    int B, V, C;
};

static __global__ void __launch_bounds__(1024) rg_pick_kernel(rg_pick_args p) {
    rg_pdl_sync();
    __shared__ float bv[32];
    __shared__ int bi[32];
    const int b = blockIdx.x, tid = threadIdx.x;
    const int pos = *p.pos;
    float best = -INFINITY;
    int besti = 0x7fffffff;
    const size_t stride = (size_t)p.B * p.V;
    // finished logits in place (one part, no bias): nothing to add and nothing to store, only the scan
    const bool in_place = p.nparts == 1 && !p.bias && p.parts == p.logits;
    // PU elements per thread and trip, their loads issued together (a load -> compare chain per element would cost one
    // memory latency each: V / 1024 = 49 of them for the full vocabulary; 16 at a time leaves 4 trips)
    constexpr int PU = 16;
    for (int v0 = tid; v0 < p.V; v0 += PU * blockDim.x) {
        float x[PU];
#pragma unroll
        for (int u = 0; u < PU; u++) {
            const int v = v0 + u * blockDim.x;
            x[u] = -INFINITY;
            if (v < p.V) {
                const float* pp = p.parts + (size_t)b * p.V + v;
                x[u] = in_place ? pp[0] : (p.bias ? p.bias[v] : 0.f) + rg_sum_parts(pp, p.nparts, stride);
            }
        }
#pragma unroll
        for (int u = 0; u < PU; u++) {
            const int v = v0 + u * blockDim.x;
            if (v < p.V) {
                if (!in_place) p.logits[(size_t)b * p.V + v] = x[u];
                if (x[u] > best) best = x[u], besti = v;  // ascending per thread: the first hit is its lowest index
            }
        }
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
        if (besti == 0x7fffffff) besti = 0;  // all-NaN row
        p.picks[b] = (uint32_t)besti;
        if (pos + 1 < p.C) p.tokens[(size_t)b * p.C + pos + 1] = (uint32_t)besti;
        if (b == 0) *p.pos_next = pos + 1;
    }
}

// Merge of the split-context attention partials into finished head outputs:
// out[b][h*hd + d] = sum_s w_s o_s[d] / sum_s w_s l_s with w_s = exp(m_s - max m).
static __global__ void rg_attn_merge_kernel(const float* __restrict__ ap, float* __restrict__ out, int B, int H, int hd, int NS,
                                            __nv_bfloat16* __restrict__ out16 = nullptr) {
    rg_pdl_sync();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= B * H * hd) return;
    rg_vec_in in;
    in.kind = RG_IN_ATTN, in.ap = ap, in.H = H, in.hd = hd, in.NS = NS;
    const int b = i / (H * hd), k = i - b * (H * hd);
    const float v = rg_vec_in_value(in, B, H * hd, b, k);
    if (out) out[i] = v;
    if (out16) out16[i] = __float2bfloat16_rn(v);  // the input rows of a tensor-core projection
}
