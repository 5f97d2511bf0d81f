// Context, storage handles and the op-level half of the C ABI: one kernel per
// method of the reference's Backend trait (src/backend/mod.rs:130-227), with the
// semantics of its CPU implementation (src/backend/cpu.rs).
#include "rg_internal.cuh"
#include "rg_gemm.cuh"

#include <string.h>

// ---------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------
static thread_local std::string g_last_error;

rg_status rg_fail(rg_status st, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return st;
}
void rg_clear_error() { g_last_error.clear(); }

extern "C" const char* rg_last_error(void) { return g_last_error.c_str(); }
extern "C" const char* rg_version(void) { return "rg_b200 0.1 (sm_100a)"; }

rg_devbuf::~rg_devbuf() {
    if (ptr) {
        int cur = 0;
        cudaGetDevice(&cur);
        if (cur != device) cudaSetDevice(device);
        // the context's stream still exists: stream-ordered free; else (context destroyed first, which synchronised
        // the stream) a plain free
        if (!(ctx_alive && *ctx_alive && cudaFreeAsync(ptr, stream) == cudaSuccess)) {
            cudaGetLastError();
            cudaFree(ptr);
        }
        if (cur != device) cudaSetDevice(cur);
    }
}

// ---------------------------------------------------------------------------
// context
// ---------------------------------------------------------------------------
extern "C" int rg_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

extern "C" rg_status rg_ctx_create(int device, rg_ctx** out) {
    if (!out) return rg_fail(RG_ERR_INVALID_INPUT, "rg_ctx_create: out is NULL");
    *out = nullptr;
    int n = rg_device_count();
    if (device < 0 || device >= n)
        return rg_fail(RG_ERR_BACKEND, "Failed to initialize CUDA device %d: %d device(s) visible", device, n);
    RG_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    RG_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return rg_fail(RG_ERR_BACKEND, "device %d is sm_%d%d; this library is built for sm_100a only", device,
                       prop.major, prop.minor);
    rg_ctx* c = new rg_ctx();
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    cudaError_t e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) {
        // keep freed op outputs in the device's pool instead of returning them to the driver at every synchronise
        cudaMemPool_t pool = nullptr;
        unsigned long long keep = ~0ull;
        if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess)
            cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
        cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMalloc(&c->d_flag, sizeof(int) * 4);
    if (e == cudaSuccess) e = cudaMemset(c->d_flag, 0, sizeof(int) * 4);
    if (e == cudaSuccess) e = cudaMallocHost(&c->h_flag, sizeof(int) * 4);
    if (e != cudaSuccess) {
        delete c;
        return rg_fail(RG_ERR_BACKEND, "rg_ctx_create: %s", cudaGetErrorString(e));
    }
    *out = c;
    return RG_OK;
}

extern "C" rg_status rg_ctx_destroy(rg_ctx* ctx) {
    if (!ctx) return RG_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    *ctx->alive = false;
    cudaStreamDestroy(ctx->stream);
    cudaFree(ctx->d_flag);
    cudaFree(ctx->tc_ws);
    cudaFreeHost(ctx->h_flag);
    delete ctx;
    return RG_OK;
}

// The bounded waits of the tensor-core GEMM and attention kernels raise the second flag word when they give up (tiles or
// split-k partials are then missing).  Called after a stream synchronise: reports it once and clears the word.
rg_status rg_tc_wait_check(rg_ctx* ctx) {
    int v = 0;
    RG_CUDA(cudaMemcpy(&v, ctx->d_flag + 1, sizeof(int), cudaMemcpyDeviceToHost));
    if (v) {
        RG_CUDA(cudaMemset(ctx->d_flag + 1, 0, sizeof(int)));
        return rg_fail(RG_ERR_TIMEOUT, "a bounded wait inside a tensor-core kernel gave up; its output is incomplete");
    }
    return RG_OK;
}

extern "C" rg_status rg_synchronize(rg_ctx* ctx) {
    if (!ctx) return rg_fail(RG_ERR_INVALID_INPUT, "rg_synchronize: ctx is NULL");
    rg_ctx_guard g(ctx);
    RG_CUDA(cudaStreamSynchronize(ctx->stream));
    return rg_tc_wait_check(ctx);
}

extern "C" void* rg_ctx_stream(rg_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }
extern "C" uint64_t rg_ctx_launch_count(rg_ctx* ctx) { return ctx ? ctx->launches : 0; }

// ---------------------------------------------------------------------------
// storage
// ---------------------------------------------------------------------------
static size_t shape_len(const size_t* shape, int ndim) {
    size_t n = 1;
    for (int i = 0; i < ndim; i++) n *= shape[i];
    return n;
}

rg_status rg_alloc_storage(rg_ctx* ctx, const size_t* shape, int ndim, rg_storage** out) {
    if (ndim < 0 || ndim > 8) return rg_fail(RG_ERR_DIMENSION, "storage rank %d not in 0..8", ndim);
    rg_storage* s = new rg_storage();
    s->ctx = ctx;
    s->shape.assign(shape, shape + ndim);
    s->len = shape_len(shape, ndim);
    s->buf = std::make_shared<rg_devbuf>();
    s->buf->device = ctx->device;
    s->buf->bytes = (s->len ? s->len : 1) * sizeof(float);
    s->buf->stream = ctx->stream;
    s->buf->ctx_alive = ctx->alive;
    cudaError_t e = cudaMallocAsync(&s->buf->ptr, s->buf->bytes, ctx->stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        const size_t want = s->buf->bytes;
        s->buf->ptr = nullptr;
        delete s;
        return rg_fail(RG_ERR_BACKEND, "Failed to allocate %zu bytes of CUDA memory: %s", want, cudaGetErrorString(e));
    }
    *out = s;
    return RG_OK;
}

__global__ void rg_fill_kernel(float* p, size_t n, float v) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) p[i] = v;
}

static rg_status make_filled(rg_ctx* ctx, const size_t* shape, int ndim, float v, rg_storage** out) {
    if (!ctx || !out || (ndim > 0 && !shape)) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    rg_ctx_guard g(ctx);
    RG_TRY(rg_alloc_storage(ctx, shape, ndim, out));
    size_t n = (*out)->len;
    if (n) {
        int blocks = (int)std::min<size_t>((n + 255) / 256, 148 * 8);
        rg_fill_kernel<<<blocks, 256, 0, ctx->stream>>>((*out)->data(), n, v);
        RG_LAUNCHED(ctx);
        RG_CUDA(cudaGetLastError());
    }
    return RG_OK;
}

extern "C" rg_status rg_zeros(rg_ctx* ctx, const size_t* shape, int ndim, rg_storage** out) {
    return make_filled(ctx, shape, ndim, 0.f, out);
}
extern "C" rg_status rg_ones(rg_ctx* ctx, const size_t* shape, int ndim, rg_storage** out) {
    return make_filled(ctx, shape, ndim, 1.f, out);
}

extern "C" rg_status rg_from_slice(rg_ctx* ctx, const float* data, size_t len, const size_t* shape, int ndim,
                                   rg_storage** out) {
    if (!ctx || !out || (len && !data) || (ndim > 0 && !shape)) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    if (ndim < 0 || ndim > 8) return rg_fail(RG_ERR_DIMENSION, "storage rank %d not in 0..8", ndim);
    if (shape_len(shape, ndim) != len)
        return rg_fail(RG_ERR_SHAPE, "Failed to create array from slice: shape holds %zu elements, slice has %zu",
                       shape_len(shape, ndim), len);
    rg_ctx_guard g(ctx);
    RG_TRY(rg_alloc_storage(ctx, shape, ndim, out));
    if (len) {
        cudaError_t e = cudaMemcpyAsync((*out)->data(), data, len * sizeof(float), cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);  // the host slice is only borrowed
        if (e != cudaSuccess) {
            delete *out;
            *out = nullptr;
            return rg_fail(RG_ERR_BACKEND, "Failed to copy to CUDA: %s", cudaGetErrorString(e));
        }
    }
    return RG_OK;
}

extern "C" rg_status rg_to_vec(rg_ctx* ctx, const rg_storage* st, float* outp, size_t cap) {
    if (!ctx || !st || (!outp && st->len)) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    if (cap < st->len) return rg_fail(RG_ERR_SHAPE, "rg_to_vec: capacity %zu < %zu elements", cap, st->len);
    rg_ctx_guard g(ctx);
    if (st->len) RG_CUDA(cudaMemcpyAsync(outp, st->data(), st->len * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    RG_CUDA(cudaStreamSynchronize(ctx->stream));
    return rg_tc_wait_check(ctx);
}

extern "C" rg_status rg_shape(const rg_storage* st, size_t* shape_out, int cap, int* ndim_out) {
    if (!st || !ndim_out) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    *ndim_out = (int)st->shape.size();
    if (shape_out)
        for (int i = 0; i < (int)st->shape.size() && i < cap; i++) shape_out[i] = st->shape[i];
    return RG_OK;
}

extern "C" size_t rg_storage_len(const rg_storage* st) { return st ? st->len : 0; }

extern "C" rg_status rg_storage_free(rg_storage* st) {
    if (!st) return RG_OK;
    if (st->ctx) {
        // the buffer may still be read by kernels queued on the context's stream
        rg_ctx_guard g(st->ctx);
        if (st->buf.use_count() == 1) cudaStreamSynchronize(st->ctx->stream);
        delete st;
    } else {
        delete st;
    }
    return RG_OK;
}

// ---------------------------------------------------------------------------
// elementwise ops with broadcasting
// ---------------------------------------------------------------------------
enum { OP_ADD = 0, OP_SUB = 1, OP_MUL = 2 };
enum { U_RELU = 0, U_SIGMOID = 1, U_EXP = 2, U_LOG = 3, U_POWF = 4, U_GELU = 5 };

struct bcast_dims {
    int ndim;
    unsigned int out[8];
    long long sa[8], sb[8];  // element strides, 0 on broadcast axes
};

template <int OP>
__device__ __forceinline__ float bin_op(float a, float b) {
    return OP == OP_ADD ? a + b : (OP == OP_SUB ? a - b : a * b);
}

template <int OP>
__global__ void rg_binary_same_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
                                      size_t n) {
    size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    size_t stride = (size_t)gridDim.x * blockDim.x * 4;
    for (; i + 3 < n; i += stride) {
        float4 x = *reinterpret_cast<const float4*>(a + i), y = *reinterpret_cast<const float4*>(b + i), z;
        z.x = bin_op<OP>(x.x, y.x);
        z.y = bin_op<OP>(x.y, y.y);
        z.z = bin_op<OP>(x.z, y.z);
        z.w = bin_op<OP>(x.w, y.w);
        *reinterpret_cast<float4*>(c + i) = z;
    }
    for (; i < n; i += stride)
        for (size_t j = i; j < n && j < i + 4; j++) c[j] = bin_op<OP>(a[j], b[j]);
}

template <int OP>
__global__ void rg_binary_bcast_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
                                       size_t n, bcast_dims d) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        size_t r = i;
        long long ia = 0, ib = 0;
        for (int k = d.ndim - 1; k >= 0; k--) {
            unsigned int q = (unsigned int)(r % d.out[k]);
            r /= d.out[k];
            ia += q * d.sa[k];
            ib += q * d.sb[k];
        }
        c[i] = bin_op<OP>(a[ia], b[ib]);
    }
}

static int grid_for(size_t n, int per_thread = 1) {
    size_t b = (n + 256ull * per_thread - 1) / (256ull * per_thread);
    return (int)std::max<size_t>(1, std::min<size_t>(b, 148 * 16));
}

static rg_status binary_op(rg_ctx* ctx, const rg_storage* a, const rg_storage* b, rg_storage** out, int op) {
    if (!ctx || !a || !b || !out) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    rg_ctx_guard g(ctx);
    const int na = (int)a->shape.size(), nb = (int)b->shape.size(), nd = std::max(na, nb);
    bcast_dims d;
    d.ndim = nd;
    std::vector<size_t> oshape(nd);
    long long stra = 1, strb = 1;
    for (int k = nd - 1; k >= 0; k--) {
        const int ka = k - (nd - na), kb = k - (nd - nb);
        const size_t da = ka >= 0 ? a->shape[ka] : 1, db = kb >= 0 ? b->shape[kb] : 1;
        if (da != db && da != 1 && db != 1)
            return rg_fail(RG_ERR_SHAPE, "Incompatible shapes for operation: cannot broadcast axis %d (%zu vs %zu)", k, da,
                           db);
        oshape[k] = std::max(da, db);
        if (da == 0 || db == 0) oshape[k] = 0;
        d.out[k] = (unsigned int)oshape[k];
        d.sa[k] = da == 1 ? 0 : stra;
        d.sb[k] = db == 1 ? 0 : strb;
        stra *= (long long)da;
        strb *= (long long)db;
    }
    RG_TRY(rg_alloc_storage(ctx, oshape.data(), nd, out));
    const size_t n = (*out)->len;
    if (!n) return RG_OK;
    const bool same = a->shape == b->shape;
    cudaStream_t s = ctx->stream;
#define RG_BIN(OPID)                                                                                             \
    if (same)                                                                                                    \
        rg_binary_same_kernel<OPID><<<grid_for(n, 4), 256, 0, s>>>(a->data(), b->data(), (*out)->data(), n);     \
    else                                                                                                         \
        rg_binary_bcast_kernel<OPID><<<grid_for(n), 256, 0, s>>>(a->data(), b->data(), (*out)->data(), n, d);
    if (op == OP_ADD) {
        RG_BIN(OP_ADD)
    } else if (op == OP_SUB) {
        RG_BIN(OP_SUB)
    } else {
        RG_BIN(OP_MUL)
    }
#undef RG_BIN
    RG_LAUNCHED(ctx);
    RG_CUDA(cudaGetLastError());
    return RG_OK;
}

extern "C" rg_status rg_add(rg_ctx* c, const rg_storage* a, const rg_storage* b, rg_storage** o) {
    return binary_op(c, a, b, o, OP_ADD);
}
extern "C" rg_status rg_sub(rg_ctx* c, const rg_storage* a, const rg_storage* b, rg_storage** o) {
    return binary_op(c, a, b, o, OP_SUB);
}
extern "C" rg_status rg_mul(rg_ctx* c, const rg_storage* a, const rg_storage* b, rg_storage** o) {
    return binary_op(c, a, b, o, OP_MUL);
}

template <int OP>
__global__ void rg_unary_kernel(const float* __restrict__ a, float* __restrict__ c, size_t n, float param) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        float x = a[i], y;
        if (OP == U_RELU) y = fmaxf(x, 0.f);
        else if (OP == U_SIGMOID) y = 1.f / (1.f + expf(-x));
        else if (OP == U_EXP) y = expf(x);
        else if (OP == U_LOG) y = logf(x);
        else if (OP == U_POWF) y = powf(x, param);
        else y = rg_gelu_tanh(x);
        c[i] = y;
    }
}

static rg_status unary_op(rg_ctx* ctx, const rg_storage* a, rg_storage** out, int op, float param) {
    if (!ctx || !a || !out) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    rg_ctx_guard g(ctx);
    RG_TRY(rg_alloc_storage(ctx, a->shape.data(), (int)a->shape.size(), out));
    const size_t n = a->len;
    if (!n) return RG_OK;
    const int gr = grid_for(n);
    cudaStream_t s = ctx->stream;
    switch (op) {
        case U_RELU: rg_unary_kernel<U_RELU><<<gr, 256, 0, s>>>(a->data(), (*out)->data(), n, param); break;
        case U_SIGMOID: rg_unary_kernel<U_SIGMOID><<<gr, 256, 0, s>>>(a->data(), (*out)->data(), n, param); break;
        case U_EXP: rg_unary_kernel<U_EXP><<<gr, 256, 0, s>>>(a->data(), (*out)->data(), n, param); break;
        case U_LOG: rg_unary_kernel<U_LOG><<<gr, 256, 0, s>>>(a->data(), (*out)->data(), n, param); break;
        case U_POWF: rg_unary_kernel<U_POWF><<<gr, 256, 0, s>>>(a->data(), (*out)->data(), n, param); break;
        default: rg_unary_kernel<U_GELU><<<gr, 256, 0, s>>>(a->data(), (*out)->data(), n, param); break;
    }
    RG_LAUNCHED(ctx);
    RG_CUDA(cudaGetLastError());
    return RG_OK;
}

extern "C" rg_status rg_relu(rg_ctx* c, const rg_storage* a, rg_storage** o) { return unary_op(c, a, o, U_RELU, 0.f); }
extern "C" rg_status rg_sigmoid(rg_ctx* c, const rg_storage* a, rg_storage** o) { return unary_op(c, a, o, U_SIGMOID, 0.f); }
extern "C" rg_status rg_exp(rg_ctx* c, const rg_storage* a, rg_storage** o) { return unary_op(c, a, o, U_EXP, 0.f); }
extern "C" rg_status rg_log(rg_ctx* c, const rg_storage* a, rg_storage** o) { return unary_op(c, a, o, U_LOG, 0.f); }
extern "C" rg_status rg_powf(rg_ctx* c, const rg_storage* a, float p, rg_storage** o) { return unary_op(c, a, o, U_POWF, p); }
extern "C" rg_status rg_gelu(rg_ctx* c, const rg_storage* a, rg_storage** o) { return unary_op(c, a, o, U_GELU, 0.f); }

// ---------------------------------------------------------------------------
// row ops: softmax, layer_norm, sparse cross entropy, sums
// ---------------------------------------------------------------------------
__device__ __forceinline__ float block_reduce_sum(float v, float* red) {
    v = rg_warp_sum(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (l == 0) red[w] = v;
    __syncthreads();
    float r = 0.f;
    for (int i = 0; i < nw; i++) r += red[i];  // fixed order: deterministic
    return r;
}
__device__ __forceinline__ float block_reduce_max(float v, float* red) {
    v = rg_warp_max(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (l == 0) red[w] = v;
    __syncthreads();
    float r = red[0];
    for (int i = 1; i < nw; i++) r = fmaxf(r, red[i]);
    return r;
}

// One CTA per row: max, exp and sum, divide (src/backend/cpu.rs:246-270).
__global__ void __launch_bounds__(256) rg_softmax_rows_kernel(const float* __restrict__ x, float* __restrict__ y, int n) {
    __shared__ float red[8];
    const float* xr = x + (size_t)blockIdx.x * n;
    float* yr = y + (size_t)blockIdx.x * n;
    float m = -INFINITY;
    for (int i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, xr[i]);
    m = block_reduce_max(m, red);
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float e = expf(xr[i] - m);
        yr[i] = e;
        s += e;
    }
    s = block_reduce_sum(s, red);
    for (int i = threadIdx.x; i < n; i += blockDim.x) yr[i] = yr[i] / s;
}

extern "C" rg_status rg_softmax(rg_ctx* ctx, const rg_storage* a, rg_storage** out) {
    if (!ctx || !a || !out) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    if (a->shape.empty()) return rg_fail(RG_ERR_DIMENSION, "softmax requires at least 1 dimension, got 0");
    rg_ctx_guard g(ctx);
    RG_TRY(rg_alloc_storage(ctx, a->shape.data(), (int)a->shape.size(), out));
    const size_t n = a->shape.back();
    if (!a->len) return RG_OK;
    const size_t rows = a->len / n;
    rg_softmax_rows_kernel<<<(unsigned)rows, 256, 0, ctx->stream>>>(a->data(), (*out)->data(), (int)n);
    RG_LAUNCHED(ctx);
    RG_CUDA(cudaGetLastError());
    return RG_OK;
}

// One warp per row, Welford statistics merged across lanes
// (src/backend/fused.rs:22-144); y = (x - mean) / sqrt(var + eps) * gamma + beta.
__global__ void __launch_bounds__(256) rg_layernorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                                const float* __restrict__ beta, float* __restrict__ y,
                                                                size_t rows, int n, float eps) {
    const size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float* xr = x + row * n;
    float* yr = y + row * n;
    rg_welford w = {0.f, 0.f, 0.f};
    for (int i = lane; i < n; i += 32) rg_welford_add(w, xr[i]);
    w = rg_welford_warp(w);
    const float inv = 1.f / sqrtf(w.m2 / (float)n + eps);
    for (int i = lane; i < n; i += 32) yr[i] = (xr[i] - w.mean) * inv * gamma[i] + beta[i];
}

extern "C" rg_status rg_layer_norm(rg_ctx* ctx, const rg_storage* x, const rg_storage* gamma, const rg_storage* beta,
                                   float epsilon, rg_storage** out) {
    if (!ctx || !x || !gamma || !beta || !out) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    if (x->shape.empty()) return rg_fail(RG_ERR_DIMENSION, "layer_norm requires at least 1 dimension, got 0");
    const size_t n = x->shape.back();
    if (gamma->len != n)
        return rg_fail(RG_ERR_SHAPE, "Invalid shape for gamma in LayerNorm: expected [1, %zu], got %zu elements", n,
                       gamma->len);
    if (beta->len != n)
        return rg_fail(RG_ERR_SHAPE, "Invalid shape for beta in LayerNorm: expected [1, %zu], got %zu elements", n,
                       beta->len);
    rg_ctx_guard g(ctx);
    RG_TRY(rg_alloc_storage(ctx, x->shape.data(), (int)x->shape.size(), out));
    if (!x->len) return RG_OK;
    const size_t rows = x->len / n;
    rg_layernorm_rows_kernel<<<rg_cdiv(rows, 8), 256, 0, ctx->stream>>>(x->data(), gamma->data(), beta->data(),
                                                                         (*out)->data(), rows, (int)n, epsilon);
    RG_LAUNCHED(ctx);
    RG_CUDA(cudaGetLastError());
    return RG_OK;
}

// Sum over `mid` of x[outer][mid][inner]; one thread per output element, fixed
// order (deterministic).  sum() is the case outer = inner = 1 handled by a
// single CTA tree.
__global__ void rg_sum_axis_kernel(const float* __restrict__ x, float* __restrict__ y, size_t outer, size_t mid, size_t inner) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= outer * inner) return;
    size_t o = i / inner, in = i % inner;
    const float* p = x + o * mid * inner + in;
    float s = 0.f;
    for (size_t k = 0; k < mid; k++) s += p[k * inner];
    y[i] = s;
}
__global__ void __launch_bounds__(1024) rg_sum_all_kernel(const float* __restrict__ x, float* __restrict__ y, size_t n) {
    __shared__ float red[32];
    float s = 0.f;
    for (size_t i = threadIdx.x; i < n; i += blockDim.x) s += x[i];
    s = block_reduce_sum(s, red);
    if (threadIdx.x == 0) y[0] = s;
}

extern "C" rg_status rg_sum(rg_ctx* ctx, const rg_storage* a, rg_storage** out) {
    if (!ctx || !a || !out) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    rg_ctx_guard g(ctx);
    size_t one = 1;
    RG_TRY(rg_alloc_storage(ctx, &one, 1, out));
    rg_sum_all_kernel<<<1, 1024, 0, ctx->stream>>>(a->data(), (*out)->data(), a->len);
    RG_LAUNCHED(ctx);
    RG_CUDA(cudaGetLastError());
    return RG_OK;
}

extern "C" rg_status rg_sum_axis(rg_ctx* ctx, const rg_storage* a, size_t axis, rg_storage** out) {
    if (!ctx || !a || !out) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    if (axis >= a->shape.size())
        return rg_fail(RG_ERR_SHAPE, "Axis %zu out of bounds for array of dimension %zu", axis, a->shape.size());
    rg_ctx_guard g(ctx);
    std::vector<size_t> os;
    size_t outer = 1, inner = 1;
    for (size_t k = 0; k < a->shape.size(); k++) {
        if (k < axis) outer *= a->shape[k];
        if (k > axis) inner *= a->shape[k];
        if (k != axis) os.push_back(a->shape[k]);
    }
    RG_TRY(rg_alloc_storage(ctx, os.data(), (int)os.size(), out));
    const size_t n = outer * inner;
    if (!n) return RG_OK;
    rg_sum_axis_kernel<<<rg_cdiv(n, 256), 256, 0, ctx->stream>>>(a->data(), (*out)->data(), outer, a->shape[axis], inner);
    RG_LAUNCHED(ctx);
    RG_CUDA(cudaGetLastError());
    return RG_OK;
}

// Row losses -log(softmax(logits)[target]) then their mean (cpu.rs:377-427).
__global__ void __launch_bounds__(256) rg_sce_rows_kernel(const float* __restrict__ logits, const float* __restrict__ targets,
                                                          float* __restrict__ loss, int n, int* flag) {
    __shared__ float red[8];
    const float* xr = logits + (size_t)blockIdx.x * n;
    float m = -INFINITY;
    for (int i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, xr[i]);
    m = block_reduce_max(m, red);
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += expf(xr[i] - m);
    s = block_reduce_sum(s, red);
    if (threadIdx.x == 0) {
        const float tf = targets[blockIdx.x];
        const long long t = (long long)tf;
        if (tf < 0.f || t >= n) {
            atomicExch(flag, 1);
            loss[blockIdx.x] = 0.f;
        } else {
            loss[blockIdx.x] = -logf(expf(xr[t] - m) / s);
        }
    }
}
__global__ void rg_scale_kernel(float* y, float f) { y[0] *= f; }

static rg_status read_flag(rg_ctx* ctx, int* value) {
    RG_CUDA(cudaMemcpyAsync(ctx->h_flag, ctx->d_flag, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    RG_CUDA(cudaStreamSynchronize(ctx->stream));
    *value = ctx->h_flag[0];
    if (*value) RG_CUDA(cudaMemsetAsync(ctx->d_flag, 0, sizeof(int), ctx->stream));
    return RG_OK;
}

extern "C" rg_status rg_sparse_cross_entropy(rg_ctx* ctx, const rg_storage* logits, const rg_storage* targets,
                                             rg_storage** out) {
    if (!ctx || !logits || !targets || !out) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    if (logits->shape.size() != 2) return rg_fail(RG_ERR_SHAPE, "Logits must be 2D, got %zuD", logits->shape.size());
    const size_t rows = logits->shape[0], n = logits->shape[1];
    if (targets->len != rows)
        return rg_fail(RG_ERR_SHAPE, "targets hold %zu elements for %zu rows of logits", targets->len, rows);
    rg_ctx_guard g(ctx);
    rg_storage* tmp = nullptr;
    RG_TRY(rg_alloc_storage(ctx, &rows, 1, &tmp));
    size_t one = 1;
    rg_status st = rg_alloc_storage(ctx, &one, 1, out);
    if (st != RG_OK) {
        delete tmp;
        return st;
    }
    if (rows) {
        rg_sce_rows_kernel<<<(unsigned)rows, 256, 0, ctx->stream>>>(logits->data(), targets->data(), tmp->data(), (int)n,
                                                                    ctx->d_flag);
        RG_LAUNCHED(ctx);
    }
    rg_sum_all_kernel<<<1, 1024, 0, ctx->stream>>>(tmp->data(), (*out)->data(), rows);
    rg_scale_kernel<<<1, 1, 0, ctx->stream>>>((*out)->data(), 1.f / (float)rows);
    ctx->launches += 2;
    int flag = 0;
    st = read_flag(ctx, &flag);
    delete tmp;
    if (st != RG_OK || flag) {
        delete *out;
        *out = nullptr;
        return st != RG_OK ? st : rg_fail(RG_ERR_SHAPE, "Target index out of bounds for %zu classes", n);
    }
    return RG_OK;
}

// ---------------------------------------------------------------------------
// reshape / transpose / embedding / matmul
// ---------------------------------------------------------------------------
extern "C" rg_status rg_reshape(rg_ctx* ctx, const rg_storage* a, const size_t* new_shape, int ndim, rg_storage** out) {
    if (!ctx || !a || !out || (ndim > 0 && !new_shape)) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    if (ndim < 0 || ndim > 8) return rg_fail(RG_ERR_DIMENSION, "storage rank %d not in 0..8", ndim);
    if (shape_len(new_shape, ndim) != a->len)
        return rg_fail(RG_ERR_SHAPE, "Reshape failed: cannot reshape %zu elements into %zu", a->len,
                       shape_len(new_shape, ndim));
    // Storages are immutable values, so the new handle can share the buffer.
    rg_storage* s = new rg_storage();
    s->ctx = ctx;
    s->buf = a->buf;
    s->shape.assign(new_shape, new_shape + ndim);
    s->len = a->len;
    *out = s;
    return RG_OK;
}

struct perm_dims {
    int ndim;
    unsigned int out[8];
    long long sin[8];  // input stride of output axis k
};
__global__ void rg_permute_kernel(const float* __restrict__ x, float* __restrict__ y, size_t n, perm_dims d) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        size_t r = i;
        long long src = 0;
        for (int k = d.ndim - 1; k >= 0; k--) {
            src += (long long)(r % d.out[k]) * d.sin[k];
            r /= d.out[k];
        }
        y[i] = x[src];
    }
}

extern "C" rg_status rg_transpose(rg_ctx* ctx, const rg_storage* a, size_t axis1, size_t axis2, rg_storage** out) {
    if (!ctx || !a || !out) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    const int nd = (int)a->shape.size();
    if (axis1 >= (size_t)nd || axis2 >= (size_t)nd)
        return rg_fail(RG_ERR_SHAPE, "Transpose axes (%zu, %zu) out of bounds for array of dimension %d", axis1, axis2, nd);
    rg_ctx_guard g(ctx);
    std::vector<long long> stride(nd);
    long long st = 1;
    for (int k = nd - 1; k >= 0; k--) {
        stride[k] = st;
        st *= (long long)a->shape[k];
    }
    std::vector<size_t> os = a->shape;
    std::swap(os[axis1], os[axis2]);
    perm_dims d;
    d.ndim = nd;
    for (int k = 0; k < nd; k++) {
        int src_axis = k == (int)axis1 ? (int)axis2 : (k == (int)axis2 ? (int)axis1 : k);
        d.out[k] = (unsigned int)os[k];
        d.sin[k] = stride[src_axis];
    }
    RG_TRY(rg_alloc_storage(ctx, os.data(), nd, out));
    if (!a->len) return RG_OK;
    rg_permute_kernel<<<grid_for(a->len), 256, 0, ctx->stream>>>(a->data(), (*out)->data(), a->len, d);
    RG_LAUNCHED(ctx);
    RG_CUDA(cudaGetLastError());
    return RG_OK;
}

// Row gather with f32-valued indices (cast like `as usize`, src/ops/embedding.rs:50).
__global__ void rg_embedding_rows_kernel(const float* __restrict__ idx, const float* __restrict__ table,
                                         float* __restrict__ y, size_t rows, int V, int D, int* flag) {
    const size_t row = blockIdx.x;
    if (row >= rows) return;
    const float f = idx[row];
    long long id = (long long)f;
    if (f < 0.f || id >= V) {
        if (threadIdx.x == 0) atomicExch(flag, 1);
        id = 0;
    }
    const float* src = table + (size_t)id * D;
    float* dst = y + row * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) dst[i] = src[i];
}

extern "C" rg_status rg_embedding(rg_ctx* ctx, const rg_storage* indices, const rg_storage* weights, rg_storage** out) {
    if (!ctx || !indices || !weights || !out) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    if (weights->shape.size() != 2)
        return rg_fail(RG_ERR_SHAPE, "Embedding weights must be 2D, got %zuD", weights->shape.size());
    if (indices->shape.size() != 1 && indices->shape.size() != 2)
        return rg_fail(RG_ERR_DIMENSION, "Operation requires a tensor with 2 dimensions, but got %zu", indices->shape.size());
    rg_ctx_guard g(ctx);
    const size_t V = weights->shape[0], D = weights->shape[1];
    std::vector<size_t> os = indices->shape;
    os.push_back(D);
    RG_TRY(rg_alloc_storage(ctx, os.data(), (int)os.size(), out));
    const size_t rows = indices->len;
    if (!rows || !D) return RG_OK;
    rg_embedding_rows_kernel<<<(unsigned)rows, 128, 0, ctx->stream>>>(indices->data(), weights->data(), (*out)->data(), rows,
                                                                      (int)V, (int)D, ctx->d_flag);
    RG_LAUNCHED(ctx);
    RG_CUDA(cudaGetLastError());
    int flag = 0;
    rg_status st = read_flag(ctx, &flag);
    if (st != RG_OK || flag) {
        delete *out;
        *out = nullptr;
        return st != RG_OK ? st : rg_fail(RG_ERR_INVALID_INPUT, "Invalid input: index out of bounds for vocabulary size %zu", V);
    }
    return RG_OK;
}

extern "C" rg_status rg_matmul(rg_ctx* ctx, const rg_storage* a, const rg_storage* b, rg_storage** out) {
    if (!ctx || !a || !b || !out) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    const int na = (int)a->shape.size(), nb = (int)b->shape.size();
    rg_ctx_guard g(ctx);
    rg_gemm_args p;
    memset(&p, 0, sizeof(p));
    p.act = -1;
    std::vector<size_t> os;
    int batch = 1;
    if (na == 2 && nb == 2) {
        if (a->shape[1] != b->shape[0])
            return rg_fail(RG_ERR_SHAPE, "Incompatible shapes for 2D dot product: [%zu, %zu] and [%zu, %zu]", a->shape[0],
                           a->shape[1], b->shape[0], b->shape[1]);
        p.M = (int)a->shape[0], p.K = (int)a->shape[1], p.N = (int)b->shape[1];
        os = {a->shape[0], b->shape[1]};
    } else if (na == 3 && nb == 2) {
        if (a->shape[2] != b->shape[0])
            return rg_fail(RG_ERR_SHAPE, "Incompatible shapes for 3D-2D dot product");
        p.M = (int)(a->shape[0] * a->shape[1]), p.K = (int)a->shape[2], p.N = (int)b->shape[1];
        os = {a->shape[0], a->shape[1], b->shape[1]};
    } else if (na == 3 && nb == 3) {
        if (b->shape[0] != a->shape[0] || b->shape[1] != a->shape[2])
            return rg_fail(RG_ERR_SHAPE, "Incompatible shapes for 3D matmul");
        batch = (int)a->shape[0];
        p.M = (int)a->shape[1], p.K = (int)a->shape[2], p.N = (int)b->shape[2];
        os = {a->shape[0], a->shape[1], b->shape[2]};
    } else if (na == 4 && nb == 4) {
        if (b->shape[0] != a->shape[0] || b->shape[1] != a->shape[1] || b->shape[2] != a->shape[3])
            return rg_fail(RG_ERR_SHAPE, "Incompatible shapes for 4D matmul");
        batch = (int)(a->shape[0] * a->shape[1]);
        p.M = (int)a->shape[2], p.K = (int)a->shape[3], p.N = (int)b->shape[3];
        os = {a->shape[0], a->shape[1], a->shape[2], b->shape[3]};
    } else {
        return rg_fail(RG_ERR_SHAPE, "Unsupported matmul dimensions: %dD and %dD", na, nb);
    }
    RG_TRY(rg_alloc_storage(ctx, os.data(), (int)os.size(), out));
    if (!(*out)->len) return RG_OK;
    p.A = a->data(), p.lda = p.K, p.strideA = (long long)p.M * p.K;
    p.W = b->data(), p.ldw = p.N, p.strideW = (long long)p.K * p.N;
    p.C = (*out)->data(), p.ldc = p.N, p.strideC = (long long)p.M * p.N;
    if (p.K == 0) {
        RG_CUDA(cudaMemsetAsync((*out)->data(), 0, (*out)->len * sizeof(float), ctx->stream));
        return RG_OK;
    }
    if (batch > 65535) return rg_fail(RG_ERR_UNSUPPORTED, "matmul batch %d exceeds 65535", batch);
    RG_CUDA(rg_gemm_launch<float>(ctx->stream, p, batch));
    RG_LAUNCHED(ctx);
    return RG_OK;
}
