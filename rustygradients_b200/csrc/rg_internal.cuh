// Shared internals of the B200 GPT token-loop library: handle structs, error
// plumbing and small device helpers.  Not part of the public ABI.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdarg.h>
#include <stdio.h>

#include <cstring>
#include <memory>
#include <utility>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/rg_b200.h"

// ---------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------
rg_status rg_fail(rg_status st, const char* fmt, ...);
void rg_clear_error();

#define RG_CUDA(expr)                                                                       \
    do {                                                                                    \
        cudaError_t _e = (expr);                                                            \
        if (_e != cudaSuccess)                                                              \
            return rg_fail(RG_ERR_BACKEND, "CUDA error %d (%s) at %s:%d: %s", (int)_e,      \
                           cudaGetErrorName(_e), __FILE__, __LINE__, cudaGetErrorString(_e)); \
    } while (0)

#define RG_TRY(expr)                  \
    do {                              \
        rg_status _s = (expr);        \
        if (_s != RG_OK) return _s;   \
    } while (0)

// ---------------------------------------------------------------------------
// handles
// ---------------------------------------------------------------------------
struct rg_ctx {
    int device = 0;
    int sm_count = 148;
    cudaStream_t stream = nullptr;
    std::mutex mu;
    uint64_t launches = 0;
    int* d_flag = nullptr;  // device word kernels raise on invalid input
    int* h_flag = nullptr;  // pinned mirror
    bool pdl = false;        // launch with programmatic stream serialization (inside a chain of rg_pdl_sync kernels)
    float* tc_ws = nullptr;  // split-k workspace of the tensor-core GEMM (this context's stream only)
    size_t tc_ws_bytes = 0;
    // storages outlive nothing they need: a buffer frees itself on `stream` only while this is still true
    std::shared_ptr<bool> alive = std::make_shared<bool>(true);
};

// Op outputs come from the device's stream-ordered pool (cudaMallocAsync on the context's stream: a few microseconds
// against the ~0.5 ms of a cudaMalloc / cudaFree pair, which dominated every small op) and go back to it on the same
// stream, after the work that was enqueued on them.
struct rg_devbuf {
    void* ptr = nullptr;
    size_t bytes = 0;
    int device = 0;
    cudaStream_t stream = nullptr;
    std::shared_ptr<bool> ctx_alive;
    ~rg_devbuf();
};

struct rg_storage {
    rg_ctx* ctx = nullptr;
    std::shared_ptr<rg_devbuf> buf;  // reshape views alias the same buffer
    std::vector<size_t> shape;
    size_t len = 0;
    const float* data() const { return static_cast<const float*>(buf->ptr); }
    float* data() { return static_cast<float*>(buf->ptr); }
};

rg_status rg_alloc_storage(rg_ctx* ctx, const size_t* shape, int ndim, rg_storage** out);
rg_status rg_tc_wait_check(rg_ctx* ctx);  // after a synchronise: did a wait of a tensor-core kernel give up?

struct rg_ctx_guard {
    rg_ctx* c;
    explicit rg_ctx_guard(rg_ctx* ctx) : c(ctx) {
        c->mu.lock();
        cudaSetDevice(c->device);
    }
    ~rg_ctx_guard() { c->mu.unlock(); }
};

#define RG_LAUNCHED(ctx) ((ctx)->launches++)

#ifdef __CUDACC__
// Kernel launch that, when pdl is set, may begin before the previous kernel of the stream has finished (the kernel
// must call rg_pdl_sync() first thing).
template <typename... P, typename... A>
static inline cudaError_t rg_launch(bool pdl, void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, A&&... args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at, cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, P(std::forward<A>(args))...);
}
#endif

static inline int rg_cdiv(long long a, long long b) { return (int)((a + b - 1) / b); }

// ---------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------
#ifdef __CUDACC__

#define RG_FULL_MASK 0xffffffffu

__device__ __forceinline__ float rg_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(RG_FULL_MASK, v, o);
    return v;
}
__device__ __forceinline__ float rg_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(RG_FULL_MASK, v, o));
    return v;
}

// Welford triple (count, mean, M2) and Chan's pairwise merge: the one-pass
// statistics of fused::layer_norm_fused (src/backend/fused.rs:22-144).
struct rg_welford {
    float n, mean, m2;
};
__device__ __forceinline__ void rg_welford_add(rg_welford& w, float x) {
    w.n += 1.f;
    float d = x - w.mean;
    w.mean += d / w.n;
    w.m2 += d * (x - w.mean);
}
__device__ __forceinline__ rg_welford rg_welford_merge(rg_welford a, rg_welford b) {
    rg_welford r;
    r.n = a.n + b.n;
    if (r.n == 0.f) {
        r.mean = 0.f;
        r.m2 = 0.f;
        return r;
    }
    float d = b.mean - a.mean;
    float f = b.n / r.n;
    r.mean = a.mean + d * f;
    r.m2 = a.m2 + b.m2 + d * d * a.n * f;
    return r;
}
__device__ __forceinline__ rg_welford rg_welford_warp(rg_welford w) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        rg_welford t;
        t.n = __shfl_xor_sync(RG_FULL_MASK, w.n, o);
        t.mean = __shfl_xor_sync(RG_FULL_MASK, w.mean, o);
        t.m2 = __shfl_xor_sync(RG_FULL_MASK, w.m2, o);
        w = rg_welford_merge(w, t);
    }
    return w;
}

// tanh-GELU with the reference's constants (src/backend/fused.rs:152-163,
// src/backend/cuda_kernels.cu:120-131).
__device__ __forceinline__ float rg_gelu_tanh(float x) {
    const float c0 = 0.7978845608f, c1 = 0.044715f;
    float inner = c0 * (x + c1 * x * x * x);
    return 0.5f * x * (1.f + tanhf(inner));
}
__device__ __forceinline__ float rg_apply_act(float x, int act) {
    return act == RG_ACT_RELU ? fmaxf(x, 0.f) : rg_gelu_tanh(x);
}

// Sum of the k-split partials of one element, in index order, with 8 loads in flight at a time (a chain of dependent
// load-add steps would cost one memory latency per partial).
__device__ __forceinline__ float rg_sum_parts(const float* __restrict__ p, int nparts, size_t pstride) {
    float t = 0.f;
    int z = 0;
    for (; z + 8 <= nparts; z += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; u++) v[u] = p[(size_t)(z + u) * pstride];
#pragma unroll
        for (int u = 0; u < 8; u++) t += v[u];
    }
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; u++) v[u] = (z + u < nparts) ? p[(size_t)(z + u) * pstride] : 0.f;
#pragma unroll
    for (int u = 0; u < 8; u++) t += v[u];
    return t;
}

// Programmatic dependent launch: a kernel launched with the "programmatic stream serialization" attribute may start
// while its predecessor is still running; this call (first statement of every kernel of such a chain) lets this
// kernel's own successor be scheduled early and then waits until the predecessor has completed and its memory is
// visible.  Without the attribute both instructions return at once.
__device__ __forceinline__ void rg_pdl_sync() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ float rg_to_float(float v) { return v; }
__device__ __forceinline__ float rg_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

#endif  // __CUDACC__
