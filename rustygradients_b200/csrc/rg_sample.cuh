// Stochastic half of the token loop: top-k filter, temperature, inverse-CDF draw
// (src/wasm_api.rs:120-156), one CTA per sequence over a finished row of logits.
//
// Differences from the reference, all outside what its tests pin:
//  * the uniform draw comes from a counter-based generator keyed by (seed, sequence,
//    step) instead of thread_rng, so a run is reproducible;
//  * exp((l - max)/T) is used instead of exp(l/T): the same distribution after the
//    normalisation the reference applies, without its overflow to inf;
//  * among logits equal to the k-th largest the lowest indices are kept (the
//    reference's unstable sort leaves that order unspecified).
#pragma once
#include "rg_internal.cuh"

__host__ __device__ __forceinline__ unsigned long long rg_splitmix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
// uniform in [0,1) with 24 random bits
__host__ __device__ __forceinline__ float rg_uniform(unsigned long long seed, unsigned int seq, unsigned int step) {
    const unsigned long long h = rg_splitmix64(rg_splitmix64(seed ^ (0xD1B54A32D192ED03ull * (seq + 1))) + step);
    return (float)(h >> 40) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ unsigned int rg_float_key(float f) {  // order-preserving map to unsigned
    const unsigned int b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct rg_sample_args {
    const float* logits;  // [B][V]
    uint32_t* tokens;     // [B][C]
    uint32_t* picks;      // [B]
    int V, C, slot;       // the drawn id goes to tokens[b][slot] when slot < C
    int top_k;            // 0 or >= V: no filter
    float inv_temperature;
    unsigned long long seed;
    unsigned int step;
};

static __global__ void __launch_bounds__(1024) rg_sample_kernel(rg_sample_args p) {
    __shared__ unsigned int hist[256];
    __shared__ float fred[32];
    __shared__ float tsum[1024];
    __shared__ unsigned int s_prefix, s_need, s_eq_before[1024];
    __shared__ int s_result;
    const int b = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const float* lg = p.logits + (size_t)b * p.V;
    const int V = p.V;

    // ---- threshold = k-th largest logit (radix select on the order-preserving keys) ----
    unsigned int thr_key = 0, need_eq = 0;  // keep keys > thr_key, plus the first need_eq keys == thr_key
    const bool filter = p.top_k > 0 && p.top_k < V;
    if (filter) {
        unsigned int prefix = 0, mask = 0, need = (unsigned int)p.top_k;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int i = tid; i < 256; i += nt) hist[i] = 0;
            __syncthreads();
            for (int i = tid; i < V; i += nt) {
                const unsigned int k = rg_float_key(lg[i]);
                if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned int acc = 0;
                int d = 255;
                for (; d > 0; d--) {
                    if (acc + hist[d] >= need) break;
                    acc += hist[d];
                }
                s_prefix = prefix | ((unsigned int)d << shift);
                s_need = need - acc;  // how many are still wanted inside bin d
            }
            __syncthreads();
            prefix = s_prefix, need = s_need, mask |= 255u << shift;
            __syncthreads();
        }
        thr_key = prefix, need_eq = need;
    }
    // ---- row maximum (for a safe exponent) ----
    float mx = -INFINITY;
    for (int i = tid; i < V; i += nt) mx = fmaxf(mx, lg[i]);
    mx = rg_warp_max(mx);
    if ((tid & 31) == 0) fred[tid >> 5] = mx;
    __syncthreads();
    mx = fred[0];
    for (int w = 1; w < (nt >> 5); w++) mx = fmaxf(mx, fred[w]);
    // ---- each thread owns a contiguous run of ids: weights summed in id order ----
    const int per = (V + nt - 1) / nt;
    const int i0 = min(V, tid * per), i1 = min(V, i0 + per);
    unsigned int eq_mine = 0;
    if (filter)
        for (int i = i0; i < i1; i++) eq_mine += rg_float_key(lg[i]) == thr_key;
    s_eq_before[tid] = eq_mine;
    __syncthreads();
    if (tid == 0) {  // exclusive prefix of the tie counts, in id order
        unsigned int run = 0;
        for (int t = 0; t < nt; t++) {
            const unsigned int c = s_eq_before[t];
            s_eq_before[t] = run;
            run += c;
        }
    }
    __syncthreads();
    unsigned int eq_seen = s_eq_before[tid];
    float mine = 0.f;
    for (int i = i0; i < i1; i++) {
        const unsigned int k = rg_float_key(lg[i]);
        bool keep = true;
        if (filter) keep = k > thr_key || (k == thr_key && eq_seen++ < need_eq);
        if (keep) mine += expf((lg[i] - mx) * p.inv_temperature);
    }
    tsum[tid] = mine;
    __syncthreads();
    if (tid == 0) {
        float total = 0.f;
        for (int t = 0; t < nt; t++) total += tsum[t];
        const float target = rg_uniform(p.seed, (unsigned int)b, p.step) * total;
        float run = 0.f;
        int owner = -1;
        for (int t = 0; t < nt; t++) {
            if (target < run + tsum[t]) {
                owner = t;
                break;
            }
            run += tsum[t];
        }
        s_result = owner;
        fred[0] = target - run;  // what is left to cross inside the owner's run
    }
    __syncthreads();
    const int owner = s_result;
    if (owner < 0) {  // the walk never crossed (rounding): the reference falls through to id 0
        if (tid == 0) {
            p.picks[b] = 0;
            if (p.slot < p.C) p.tokens[(size_t)b * p.C + p.slot] = 0;
        }
        return;
    }
    if (tid == owner) {
        const float rest = fred[0];
        unsigned int eq2 = s_eq_before[tid];
        float run = 0.f;
        int pick = -1, last_kept = -1;
        for (int i = i0; i < i1; i++) {
            const unsigned int k = rg_float_key(lg[i]);
            bool keep = true;
            if (filter) keep = k > thr_key || (k == thr_key && eq2++ < need_eq);
            if (!keep) continue;
            last_kept = i;
            run += expf((lg[i] - mx) * p.inv_temperature);
            if (rest < run) {
                pick = i;
                break;
            }
        }
        if (pick < 0) pick = last_kept < 0 ? 0 : last_kept;
        p.picks[b] = (uint32_t)pick;
        if (p.slot < p.C) p.tokens[(size_t)b * p.C + p.slot] = (uint32_t)pick;
    }
}
