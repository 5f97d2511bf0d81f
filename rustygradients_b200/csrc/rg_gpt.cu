// GPT model half of the C ABI: weight ingest, full forward, prompt pass, the
// KV-cache token step and the generate loop.  Mirrors GptConfig / GPTModel
// (src/models/gpt.rs) and WasmGptTrainer::generate (src/wasm_api.rs:97-163).
#include "rg_internal.cuh"
#include "rg_gpt.h"
#include "rg_gemm.cuh"
#include "rg_decode_kernels.cuh"
#include "rg_prefill_kernels.cuh"
#include "rg_rows_kernels.cuh"
#include "rg_sample.cuh"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>

#include <dlfcn.h>
#include <nccl.h>  // types and prototypes only: the library is resolved at run time

// ---------------------------------------------------------------------------
// tensor parallelism: NCCL resolved with dlopen (the process normally has it loaded already)
// ---------------------------------------------------------------------------
struct rg_nccl_api {
    decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
    decltype(&ncclCommInitRank) CommInitRank = nullptr;
    decltype(&ncclCommDestroy) CommDestroy = nullptr;
    decltype(&ncclAllReduce) AllReduce = nullptr;
    decltype(&ncclAllGather) AllGather = nullptr;
    decltype(&ncclGetErrorString) GetErrorString = nullptr;
    bool ok = false;
};
static rg_nccl_api g_nccl;
static rg_status load_nccl() {
    if (g_nccl.ok) return RG_OK;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return rg_fail(RG_ERR_BACKEND, "tensor parallelism needs NCCL: cannot load libnccl.so.2 (%s)", dlerror());
#define RG_SYM(name)                                                          \
    g_nccl.name = reinterpret_cast<decltype(g_nccl.name)>(dlsym(h, "nccl" #name)); \
    if (!g_nccl.name) return rg_fail(RG_ERR_BACKEND, "libnccl has no symbol nccl" #name);
    RG_SYM(GetUniqueId) RG_SYM(CommInitRank) RG_SYM(CommDestroy) RG_SYM(AllReduce) RG_SYM(AllGather) RG_SYM(GetErrorString)
#undef RG_SYM
    g_nccl.ok = true;
    return RG_OK;
}
#define RG_NCCL(expr)                                                                                      \
    do {                                                                                                   \
        ncclResult_t _r = (expr);                                                                          \
        if (_r != ncclSuccess)                                                                             \
            return rg_fail(RG_ERR_BACKEND, "NCCL error %d (%s) at %s:%d", (int)_r, g_nccl.GetErrorString(_r), \
                           __FILE__, __LINE__);                                                            \
    } while (0)

// out[i] = sum over the k-splits of parts[s][i] (+ bias[i % n_bias]), fixed order
// (rows of n_bias values each; out row stride ld_out, 0 = contiguous)
static __global__ void rg_reduce_parts_kernel(const float* __restrict__ parts, int nparts, size_t n,
                                              const float* __restrict__ bias, int n_bias, float* __restrict__ out,
                                              long long ld_out = 0) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = bias ? bias[i % n_bias] : 0.f;
    for (int s = 0; s < nparts; s++) v += parts[(size_t)s * n + i];
    if (ld_out) out[(i / n_bias) * ld_out + i % n_bias] = v;
    else out[i] = v;
}
static void tp_peer_close(rg_gpt* m);
static rg_status tp_check(rg_gpt* m);
// ---- token-step all-reduce over peer memory (tensor parallel) ---------------------------------------------
// One kernel = local reduction of the projection's k-split partial sums + all-reduce over the ranks.  Every
// rank stores its value of element i, together with a tag, as ONE 64-bit word into slot [parity][rank][i] of
// every rank's receive buffer (plain stores through NVLink to peer-mapped memory), then polls the tp_size
// words of element i in its own buffer until their tags match and adds them in rank order, so every rank
// obtains bit-identical sums.  Data and flag travel in the same word: no separate signal, no barrier.
// Two parities alternate between consecutive all-reduces: a rank can be at most one all-reduce ahead of a
// peer that is still reading, because the next one needs that peer's contribution.
// Every wait is bounded: after RG_TP_SPIN_LIMIT polls the thread sets *err and gives up.
#define RG_TP_MAX 16
#define RG_TP_SPIN_LIMIT (1u << 22)
struct rg_tp_ar_args {
    const float* parts;  // [nparts][cnt]
    int nparts;
    size_t cnt;
    float* out;  // [cnt]
    unsigned long long* peer[RG_TP_MAX];
    int T, rank;
    size_t slot;  // words per (parity, rank)
    const unsigned* epoch;
    int site, nsites;
    int* err;
    unsigned limit;  // polls after which a wait gives up
};
static __global__ void __launch_bounds__(256) rg_tp_allreduce_kernel(rg_tp_ar_args a) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.cnt) return;
    const unsigned seq = *a.epoch * (unsigned)a.nsites + (unsigned)a.site;
    const unsigned tag = seq + 1u;
    const size_t par = seq & 1u;
    float v = 0.f;
    for (int z = 0; z < a.nparts; z++) v += a.parts[(size_t)z * a.cnt + i];
    const unsigned long long word = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
    const size_t mine = (par * a.T + a.rank) * a.slot + i;
    for (int r = 0; r < a.T; r++)
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(a.peer[r] + mine), "l"(word) : "memory");
    const unsigned long long* own = a.peer[a.rank] + par * a.T * a.slot + i;
    float vals[RG_TP_MAX];
    unsigned pending = (1u << a.T) - 1u, spins = 0;
    while (pending) {
        unsigned long long w[RG_TP_MAX];
#pragma unroll
        for (int r = 0; r < RG_TP_MAX; r++)
            if (r < a.T && (pending & (1u << r)))
                asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w[r]) : "l"(own + (size_t)r * a.slot) : "memory");
#pragma unroll
        for (int r = 0; r < RG_TP_MAX; r++)
            if (r < a.T && (pending & (1u << r)) && (unsigned)(w[r] >> 32) == tag) {
                vals[r] = __uint_as_float((unsigned)w[r]);
                pending &= ~(1u << r);
            }
        if (pending && (++spins > a.limit || ((spins & 1023u) == 0 && *(volatile int*)a.err))) {
            *a.err = 1;
            break;
        }
    }
    float sum = 0.f;
#pragma unroll
    for (int r = 0; r < RG_TP_MAX; r++)
        if (r < a.T) sum += (pending & (1u << r)) ? 0.f : vals[r];
    a.out[i] = sum;
}
static __global__ void rg_bump_kernel(unsigned* p) { *p += 1u; }

// Row-split projection of the batched token step, tensor parallel: "sum the k-split partial tiles -> all-reduce over the
// ranks -> + bias + residual -> LayerNorm -> bf16 rows" in ONE kernel (one CTA per row, 256 threads, 8 values per thread
// at most).  The all-reduce is the one-shot exchange of rg_tp_allreduce_kernel done by the thread that owns the
// element: its local sum goes, tagged, into slot [parity][rank][row * D + k] of every rank's receive buffer, then the
// tp_size words of that element are collected from the own buffer (all requested together, bounded) and added in rank
// order.  Same slots, tags and parities as rg_tp_allreduce_kernel, so both forms of the step can alternate.
static __global__ void __launch_bounds__(256) rg_rows_res_ln_tp_bf16_kernel(rg_tp_ar_args a, const float* __restrict__ bias,
                                                                            float* __restrict__ x, const float* __restrict__ gamma,
                                                                            const float* __restrict__ beta,
                                                                            __nv_bfloat16* __restrict__ out16, int D) {
    rg_pdl_sync();
    __shared__ float sm8[8];
    const size_t row = blockIdx.x;
    const unsigned seq = *a.epoch * (unsigned)a.nsites + (unsigned)a.site;
    const unsigned tag = seq + 1u;
    const size_t par = seq & 1u;
    constexpr int PT = RG_ROWS_MAX_D / 256;
    float v[PT];
    // local sums out first, for every element of the thread, so that the peers' words travel while the rest is prepared
#pragma unroll
    for (int i = 0; i < PT; i++) {
        const int k = threadIdx.x + i * 256;
        v[i] = 0.f;
        if (k < D) {
            const size_t e = row * D + k;
            const float part = rg_sum_parts(a.parts + e, a.nparts, a.cnt);
            const unsigned long long word = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(part);
            const size_t mine = (par * a.T + a.rank) * a.slot + e;
            for (int r = 0; r < a.T; r++)
                asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(a.peer[r] + mine), "l"(word) : "memory");
        }
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < PT; i++) {
        const int k = threadIdx.x + i * 256;
        if (k < D) {
            const size_t e = row * D + k;
            const unsigned long long* own = a.peer[a.rank] + par * a.T * a.slot + e;
            float vals[RG_TP_MAX];
            unsigned pending = (1u << a.T) - 1u, spins = 0;
            while (pending) {
                unsigned long long w[RG_TP_MAX];
#pragma unroll
                for (int r = 0; r < RG_TP_MAX; r++)
                    if (r < a.T && (pending & (1u << r)))
                        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w[r]) : "l"(own + (size_t)r * a.slot) : "memory");
#pragma unroll
                for (int r = 0; r < RG_TP_MAX; r++)
                    if (r < a.T && (pending & (1u << r)) && (unsigned)(w[r] >> 32) == tag) {
                        vals[r] = __uint_as_float((unsigned)w[r]);
                        pending &= ~(1u << r);
                    }
                if (pending && (++spins > a.limit || ((spins & 1023u) == 0 && *(volatile int*)a.err))) {
                    *a.err = 1;
                    break;
                }
            }
            float sum = 0.f;
#pragma unroll
            for (int r = 0; r < RG_TP_MAX; r++)
                if (r < a.T) sum += (pending & (1u << r)) ? 0.f : vals[r];
            const float t = x[e] + (sum + (bias ? bias[k] : 0.f));
            x[e] = t;
            v[i] = t;
            s += t;
        }
    }
    const float mean = rg_block_sum_256(s, sm8) / (float)D;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < PT; i++) {
        const int k = threadIdx.x + i * 256;
        if (k < D) q = fmaf(v[i] - mean, v[i] - mean, q);
    }
    const float rstd = 1.f / sqrtf(rg_block_sum_256(q, sm8) / (float)D + 1e-5f);
#pragma unroll
    for (int i = 0; i < PT; i++) {
        const int k = threadIdx.x + i * 256;
        if (k < D) out16[row * D + k] = __float2bfloat16_rn((v[i] - mean) * rstd * gamma[k] + beta[k]);
    }
}

// x[m][n] += t[m][n] + bias[n]
static __global__ void rg_add_bias_res_kernel(float* __restrict__ x, const float* __restrict__ t,
                                              const float* __restrict__ bias, size_t rows, int N) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * N) return;
    x[i] += t[i] + bias[i % N];
}
// gathered [ranks][rows][Vpad] -> logits [rows][V]
static __global__ void rg_ungather_logits_kernel(const float* __restrict__ g, float* __restrict__ logits, size_t rows, int V,
                                                 int Vpad) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * V) return;
    const size_t r = i / V;
    const int v = (int)(i - r * V);
    const int rank = v / Vpad;
    logits[i] = g[((size_t)rank * rows + r) * Vpad + (v - rank * Vpad)];
}

// Wt[n][k] = W[k][n] (bf16), 32x32 tiles through shared memory
static __global__ void rg_transpose_bf16_kernel(const __nv_bfloat16* __restrict__ W, long long ldw, int K, int N,
                                                __nv_bfloat16* __restrict__ Wt) {
    __shared__ __nv_bfloat16 t[32][33];
    const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int k = k0 + i, n = n0 + threadIdx.x;
        t[i][threadIdx.x] = (k < K && n < N) ? W[(size_t)k * ldw + n] : __float2bfloat16_rn(0.f);
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int n = n0 + i, k = k0 + threadIdx.x;
        if (n < N && k < K) Wt[(size_t)n * K + k] = t[threadIdx.x][i];
    }
}
// f32 mode: Wt3[n][0:K] = hi(W[k][n]), [K:2K] = lo, [2K:3K] = hi
static __global__ void rg_split3_wt_kernel(const float* __restrict__ W, long long ldw, int K, int N, __nv_bfloat16* __restrict__ Wt3) {
    __shared__ float t[32][33];
    const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int k = k0 + i, n = n0 + threadIdx.x;
        t[i][threadIdx.x] = (k < K && n < N) ? W[(size_t)k * ldw + n] : 0.f;
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int n = n0 + i, k = k0 + threadIdx.x;
        if (n < N && k < K) {
            const float w = t[threadIdx.x][i];
            const __nv_bfloat16 hi = __float2bfloat16_rn(w);
            const __nv_bfloat16 lo = __float2bfloat16_rn(w - __bfloat162float(hi));
            __nv_bfloat16* row = Wt3 + (size_t)n * 3 * K;
            row[k] = hi, row[K + k] = lo, row[2 * K + k] = hi;
        }
    }
}
// f32 mode: A3[m][0:K] = hi(A[m][k]), [K:2K] = hi, [2K:3K] = lo
static __global__ void rg_split3_rows_kernel(const float* __restrict__ A, int K, size_t total, __nv_bfloat16* __restrict__ A3) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t mrow = i / K;
    const int k = (int)(i - mrow * K);
    const float a = A[i];
    const __nv_bfloat16 hi = __float2bfloat16_rn(a);
    const __nv_bfloat16 lo = __float2bfloat16_rn(a - __bfloat162float(hi));
    __nv_bfloat16* row = A3 + mrow * 3 * K;
    row[k] = hi, row[K + k] = hi, row[2 * K + k] = lo;
}
static __global__ void rg_to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, size_t n) {
    size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < n) {
        const float4 v = *reinterpret_cast<const float4*>(x + i);
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<__nv_bfloat162*>(y + i) = a;
        *reinterpret_cast<__nv_bfloat162*>(y + i + 2) = b;
    } else {
        for (; i < n; i++) y[i] = __float2bfloat16_rn(x[i]);
    }
}

static __global__ void rg_set_int2_kernel(int* a, int* b, int v) {
    *a = v;
    if (b) *b = v;
}

// ---------------------------------------------------------------------------
// allocation helpers
// ---------------------------------------------------------------------------
static rg_status dalloc(rg_gpt* m, void** p, size_t bytes) {
    *p = nullptr;
    cudaError_t e = cudaMalloc(p, bytes ? bytes : 16);
    if (e != cudaSuccess)
        return rg_fail(RG_ERR_BACKEND, "Failed to allocate %zu bytes of CUDA memory: %s", bytes, cudaGetErrorString(e));
    m->allocs.push_back(*p);
    return RG_OK;
}
static void dfree(rg_gpt* m, void* p) {
    if (!p) return;
    auto it = std::find(m->allocs.begin(), m->allocs.end(), p);
    if (it != m->allocs.end()) m->allocs.erase(it);
    cudaFree(p);
}
static long long round_up(long long a, long long b) { return (a + b - 1) / b * b; }

static int batch_tile(int B) { return B <= 1 ? 1 : (B <= 2 ? 2 : (B <= 4 ? 4 : 8)); }

static void plan_split(rg_gpt* m, rg_linear& lin) {
    const int NT = m->bf16 ? 256 : 128;
    const int ntiles = rg_cdiv(lin.N, NT);
    int ks = std::max(1, m->ctx->sm_count / ntiles);
    ks = std::min(ks, std::max(1, lin.K / 16));
    ks = std::min(ks, 32);
    lin.krows = (int)round_up(rg_cdiv(lin.K, ks), 8);
    lin.ksplit = rg_cdiv(lin.K, lin.krows);
}

static rg_status alloc_linear(rg_gpt* m, rg_linear& lin, int K, int N) {
    lin.K = K, lin.N = N;
    lin.ldw = round_up(N, 8);
    RG_TRY(dalloc(m, &lin.W, (size_t)K * lin.ldw * m->wsize));
    RG_CUDA(cudaMemset(lin.W, 0, (size_t)K * lin.ldw * m->wsize));
    RG_TRY(dalloc(m, (void**)&lin.b, (size_t)N * 4));
    // K-contiguous copy for the tensor-core GEMM.  bf16 mode: Wt[n][k].  f32 mode: Wt[n][3K] = [hi | lo | hi] with
    // w = hi + lo + O(2^-17 w) in bf16 pieces, multiplied against rows [a_hi | a_hi | a_lo]: three bf16 products
    // accumulated in fp32 reproduce the f32 product to ~2^-16 relative, well inside the f32-mode tolerance.
    if (m->use_tc && K % 64 == 0) RG_TRY(dalloc(m, &lin.Wt, (size_t)N * K * (m->bf16 ? 2 : 6)));
    plan_split(m, lin);
    RG_TRY(dalloc(m, (void**)&lin.parts, (size_t)lin.ksplit * m->Bmax * N * 4));
    return RG_OK;
}

// ---------------------------------------------------------------------------
// create / destroy
// ---------------------------------------------------------------------------
template <typename F>
static void set_smem_attr(F f, int bytes) {
    cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

extern "C" rg_status rg_gpt_create(rg_ctx* ctx, const rg_gpt_config* cfg, rg_gpt** out) {
    if (!ctx || !cfg || !out) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    *out = nullptr;
    if (!cfg->block_size || !cfg->vocab_size || !cfg->num_layers || !cfg->num_heads || !cfg->embedding_dim)
        return rg_fail(RG_ERR_INVALID_INPUT, "GptConfig fields must be non-zero");
    if (cfg->embedding_dim % cfg->num_heads != 0)
        return rg_fail(RG_ERR_INVALID_INPUT, "embed_dim must be divisible by num_heads (%zu %% %zu != 0)",
                       cfg->embedding_dim, cfg->num_heads);
    const size_t hd = cfg->embedding_dim / cfg->num_heads;
    if (hd != 32 && hd != 64 && hd != 128)
        return rg_fail(RG_ERR_UNSUPPORTED, "head_dim %zu not supported (32, 64 or 128)", hd);
    if (cfg->activation != RG_ACT_RELU && cfg->activation != RG_ACT_GELU_TANH)
        return rg_fail(RG_ERR_INVALID_INPUT, "unknown activation %d", cfg->activation);
    if (cfg->weight_dtype != RG_DTYPE_F32 && cfg->weight_dtype != RG_DTYPE_BF16)
        return rg_fail(RG_ERR_INVALID_INPUT, "unknown weight_dtype %d", cfg->weight_dtype);
    if (cfg->vocab_size >= (1u << 24))
        return rg_fail(RG_ERR_UNSUPPORTED, "vocab_size %zu: ids are carried as f32 and must stay below 2^24", cfg->vocab_size);
    rg_ctx_guard g(ctx);
    rg_gpt* m = new rg_gpt();
    m->ctx = ctx;
    m->cfg = *cfg;
    m->V = (int)cfg->vocab_size, m->D = (int)cfg->embedding_dim, m->L = (int)cfg->num_layers;
    m->H = (int)cfg->num_heads, m->hd = (int)hd, m->C = (int)cfg->block_size, m->F = 4 * m->D;
    m->Bmax = (int)std::max<size_t>(1, cfg->max_batch);
    m->bf16 = cfg->weight_dtype == RG_DTYPE_BF16;
    m->wsize = m->bf16 ? 2 : 4;
    m->ldt = round_up(m->D, 8);
    m->tp_size = std::max(1, cfg->tp_size), m->tp_rank = cfg->tp_size > 1 ? cfg->tp_rank : 0;
    if (m->tp_rank < 0 || m->tp_rank >= m->tp_size || m->tp_size > m->H) {
        const int r = m->tp_rank, t = m->tp_size;
        delete m;
        return rg_fail(RG_ERR_INVALID_INPUT, "tp_rank %d / tp_size %d not usable with %zu heads", r, t, cfg->num_heads);
    }
    {   // shard of this rank: whole heads, hidden columns in multiples of 8, one block of the vocabulary
        const int T = m->tp_size, r = m->tp_rank;
        m->Hl = m->H / T + (r < m->H % T ? 1 : 0);
        m->h0 = r * (m->H / T) + std::min(r, m->H % T);
        m->Dl = m->Hl * m->hd;
        const int F8 = m->F / 8;
        m->Fl = 8 * (F8 / T + (r < F8 % T ? 1 : 0));
        m->f0 = 8 * (r * (F8 / T) + std::min(r, F8 % T));
        m->Vpad = (int)round_up(rg_cdiv(m->V, T), 8);
        m->v0 = std::min(m->V, r * m->Vpad);
        m->Vl = std::max(0, std::min(m->Vpad, m->V - m->v0));
        if (T == 1) m->Vpad = m->V;
        if (m->Vl == 0) {
            delete m;
            return rg_fail(RG_ERR_INVALID_INPUT, "tp_size %d leaves rank %d without vocabulary", T, r);
        }
    }
    {
        const char* pf = getenv("RG_B200_PREFILL");
        m->use_tc = !(pf && strcmp(pf, "simt") == 0);
    }
    const char* ng = getenv("RG_B200_NO_GRAPH");
    m->use_graph = !(ng && ng[0] == '1');

    rg_status st = RG_OK;
    auto TRY = [&](rg_status s) {
        if (st == RG_OK) st = s;
    };
    TRY(dalloc(m, &m->wte, (size_t)m->V * m->ldt * m->wsize));
    TRY(dalloc(m, &m->wpe, (size_t)m->C * m->ldt * m->wsize));
    TRY(dalloc(m, (void**)&m->lnfg, m->D * 4));
    TRY(dalloc(m, (void**)&m->lnfb, m->D * 4));
    m->layers.resize(m->L);
    for (int l = 0; l < m->L && st == RG_OK; l++) {
        rg_layer& y = m->layers[l];
        TRY(alloc_linear(m, y.qkv, m->D, 3 * m->Dl));
        TRY(alloc_linear(m, y.o, m->Dl, m->D));
        TRY(alloc_linear(m, y.fc1, m->D, m->Fl));
        TRY(alloc_linear(m, y.fc2, m->Fl, m->D));
        TRY(dalloc(m, (void**)&y.ln1g, m->D * 4));
        TRY(dalloc(m, (void**)&y.ln1b, m->D * 4));
        TRY(dalloc(m, (void**)&y.ln2g, m->D * 4));
        TRY(dalloc(m, (void**)&y.ln2b, m->D * 4));
    }
    if (st == RG_OK) TRY(alloc_linear(m, m->head, m->D, m->Vl));
    const size_t kvsize = m->bf16 ? 2 : 4;
    m->kv_layer_bytes = (size_t)m->Bmax * m->Hl * m->C * m->hd * kvsize;
    TRY(dalloc(m, (void**)&m->kc, m->kv_layer_bytes * m->L));
    TRY(dalloc(m, (void**)&m->vc, m->kv_layer_bytes * m->L));
    // split of the context across CTAs in the token-step attention
    m->NS = std::max(1, std::min(16, rg_cdiv(ctx->sm_count, m->Hl)));
    TRY(dalloc(m, (void**)&m->xa, (size_t)m->Bmax * m->D * 4));
    TRY(dalloc(m, (void**)&m->xb, (size_t)m->Bmax * m->D * 4));
    TRY(dalloc(m, (void**)&m->ap, (size_t)m->Bmax * m->Hl * m->NS * (m->hd + 2) * 4));
    if (m->tp_size > 1) {
        TRY(dalloc(m, (void**)&m->tp_vec, (size_t)m->Bmax * m->D * 4));
        TRY(dalloc(m, (void**)&m->tp_local, (size_t)m->Bmax * m->Vpad * 4));
        TRY(dalloc(m, (void**)&m->tp_gather, (size_t)m->tp_size * m->Bmax * m->Vpad * 4));
    }
    TRY(dalloc(m, (void**)&m->logits, (size_t)m->Bmax * m->V * 4));
    TRY(dalloc(m, (void**)&m->tokens, (size_t)m->Bmax * m->C * 4));
    TRY(dalloc(m, (void**)&m->picks, (size_t)m->Bmax * 4));
    TRY(dalloc(m, (void**)&m->d_pos, 16));
    if (st != RG_OK) {
        rg_gpt_destroy(m);
        return st;
    }
    m->d_pos_next = m->d_pos + 1;
    cudaMemset(m->d_pos, 0, 16);
    cudaMemset(m->tokens, 0, (size_t)m->Bmax * m->C * 4);

    const int big = 100 * 1024;
    set_smem_attr(rg_gemv_kernel<float, 1>, big);
    set_smem_attr(rg_gemv_kernel<float, 2>, big);
    set_smem_attr(rg_gemv_kernel<float, 4>, big);
    set_smem_attr(rg_gemv_kernel<float, 8>, big);
    set_smem_attr(rg_gemv_kernel<__nv_bfloat16, 1>, big);
    set_smem_attr(rg_gemv_kernel<__nv_bfloat16, 2>, big);
    set_smem_attr(rg_gemv_kernel<__nv_bfloat16, 4>, big);
    set_smem_attr(rg_gemv_kernel<__nv_bfloat16, 8>, big);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        rg_gpt_destroy(m);
        return rg_fail(RG_ERR_BACKEND, "kernel attribute setup failed: %s (is the library built for this GPU?)",
                       cudaGetErrorString(e));
    }
    *out = m;
    return RG_OK;
}

extern "C" rg_status rg_gpt_destroy(rg_gpt* m) {
    if (!m) return RG_OK;
    cudaSetDevice(m->ctx->device);
    cudaStreamSynchronize(m->ctx->stream);
    if (m->graph) cudaGraphExecDestroy(m->graph);
    tp_peer_close(m);
    if (m->nccl_comm && g_nccl.ok) g_nccl.CommDestroy((ncclComm_t)m->nccl_comm);
    rg_mega_destroy(m);
    rg_cloop_destroy(m);
    for (void* p : m->allocs) cudaFree(p);
    delete m;
    return RG_OK;
}

extern "C" int rg_gpt_num_params(const rg_gpt* m) { return m ? 2 + 16 * m->L + 4 : 0; }

extern "C" rg_status rg_gpt_param_shape(const rg_gpt* m, int i, size_t s[2]) {
    if (!m || !s) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    const int n = rg_gpt_num_params(m);
    if (i < 0 || i >= n) return rg_fail(RG_ERR_INVALID_INPUT, "parameter index %d out of range 0..%d", i, n - 1);
    const size_t V = m->V, D = m->D, C = m->C, F = m->F;
    if (i == 0) { s[0] = V, s[1] = D; return RG_OK; }
    if (i == 1) { s[0] = C, s[1] = D; return RG_OK; }
    if (i >= n - 4) {
        const int j = i - (n - 4);
        if (j < 2) s[0] = 1, s[1] = D;
        else if (j == 2) s[0] = D, s[1] = V;
        else s[0] = 1, s[1] = V;
        return RG_OK;
    }
    const int j = (i - 2) % 16;
    switch (j) {
        case 0: case 2: case 4: case 6: s[0] = D, s[1] = D; break;
        case 10: s[0] = D, s[1] = F; break;
        case 11: s[0] = 1, s[1] = F; break;
        case 12: s[0] = F, s[1] = D; break;
        default: s[0] = 1, s[1] = D; break;
    }
    return RG_OK;
}

// ---------------------------------------------------------------------------
// weight ingest
// ---------------------------------------------------------------------------
static inline uint16_t f32_to_bf16_rne(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);  // NaN
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

// Copy a row-major [rows][cols] f32 host matrix into columns [col0, col0+cols) of a
// device matrix with leading dimension ld, converting to the weight dtype.
// The host block is rows x cols at src (row stride src_ld floats).
static rg_status upload_matrix(rg_gpt* m, void* dst, long long ld, int col0, const float* src, int rows, int cols,
                               long long src_ld = -1) {
    if (src_ld < 0) src_ld = cols;
    if (!m->bf16) {
        RG_CUDA(cudaMemcpy2D((float*)dst + col0, ld * 4, src, (size_t)src_ld * 4, (size_t)cols * 4, rows,
                             cudaMemcpyHostToDevice));
    } else {
        std::vector<uint16_t> tmp((size_t)rows * cols);
        for (int r = 0; r < rows; r++)
            for (int c = 0; c < cols; c++) tmp[(size_t)r * cols + c] = f32_to_bf16_rne(src[(size_t)r * src_ld + c]);
        RG_CUDA(cudaMemcpy2D((uint16_t*)dst + col0, ld * 2, tmp.data(), (size_t)cols * 2, (size_t)cols * 2, rows,
                             cudaMemcpyHostToDevice));
    }
    return RG_OK;
}
static rg_status upload_vec(float* dst, const float* src, int n) {
    RG_CUDA(cudaMemcpy(dst, src, (size_t)n * 4, cudaMemcpyHostToDevice));
    return RG_OK;
}

extern "C" rg_status rg_gpt_load_params(rg_gpt* m, const float* const* data, const size_t* const* shapes,
                                        const int* ndims, int n) {
    if (!m || !data || !shapes || !ndims) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    const int want = rg_gpt_num_params(m);
    if (n != want)
        return rg_fail(RG_ERR_SHAPE, "Mismatch in number of parameter tensors during loading: got %d, model has %d", n, want);
    for (int i = 0; i < n; i++) {
        size_t s[2];
        rg_gpt_param_shape(m, i, s);
        if (!data[i] || !shapes[i]) return rg_fail(RG_ERR_INVALID_INPUT, "parameter %d is NULL", i);
        if (ndims[i] != 2 || shapes[i][0] != s[0] || shapes[i][1] != s[1])
            return rg_fail(RG_ERR_SHAPE, "Mismatch in tensor shape during loading: parameter %d expected [%zu, %zu]", i, s[0],
                           s[1]);
    }
    rg_ctx_guard g(m->ctx);
    RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
    const int D = m->D, F = m->F, V = m->V, C = m->C;
    RG_TRY(upload_matrix(m, m->wte, m->ldt, 0, data[0], V, D));
    RG_TRY(upload_matrix(m, m->wpe, m->ldt, 0, data[1], C, D));
    for (int l = 0; l < m->L; l++) {
        const float* const* p = data + 2 + 16 * l;
        rg_layer& y = m->layers[l];
        const int Dl = m->Dl, c0 = m->h0 * m->hd;  // this rank's heads = columns [c0, c0 + Dl) of Wq, Wk, Wv
        for (int j = 0; j < 3; j++) {  // Wq | Wk | Wv side by side: one [D, 3 Dl] projection
            RG_TRY(upload_matrix(m, y.qkv.W, y.qkv.ldw, j * Dl, p[2 * j] + c0, D, Dl, D));
            RG_TRY(upload_vec(y.qkv.b + j * Dl, p[2 * j + 1] + c0, Dl));
        }
        RG_TRY(upload_matrix(m, y.o.W, y.o.ldw, 0, p[6] + (size_t)c0 * D, Dl, D, D));  // rows of Wo for the same heads
        RG_TRY(upload_vec(y.o.b, p[7], D));
        RG_TRY(upload_vec(y.ln1g, p[8], D));
        RG_TRY(upload_vec(y.ln1b, p[9], D));
        RG_TRY(upload_matrix(m, y.fc1.W, y.fc1.ldw, 0, p[10] + m->f0, D, m->Fl, F));  // hidden columns [f0, f0 + Fl)
        RG_TRY(upload_vec(y.fc1.b, p[11] + m->f0, m->Fl));
        RG_TRY(upload_matrix(m, y.fc2.W, y.fc2.ldw, 0, p[12] + (size_t)m->f0 * D, m->Fl, D, D));  // and the matching rows
        RG_TRY(upload_vec(y.fc2.b, p[13], D));
        RG_TRY(upload_vec(y.ln2g, p[14], D));
        RG_TRY(upload_vec(y.ln2b, p[15], D));
    }
    RG_TRY(upload_vec(m->lnfg, data[n - 4], D));
    RG_TRY(upload_vec(m->lnfb, data[n - 3], D));
    RG_TRY(upload_matrix(m, m->head.W, m->head.ldw, 0, data[n - 2] + m->v0, D, m->Vl, V));  // vocabulary slice
    RG_TRY(upload_vec(m->head.b, data[n - 1] + m->v0, m->Vl));
    if (m->bf16) {  // K-contiguous copies for the tensor-core prompt pass
        auto tr = [&](rg_linear& lin) {
            if (!lin.Wt) return;
            dim3 grid(rg_cdiv(lin.N, 32), rg_cdiv(lin.K, 32)), block(32, 8);
            rg_transpose_bf16_kernel<<<grid, block, 0, m->ctx->stream>>>((const __nv_bfloat16*)lin.W, lin.ldw, lin.K, lin.N,
                                                                        (__nv_bfloat16*)lin.Wt);
            RG_LAUNCHED(m->ctx);
        };
        for (auto& y : m->layers) tr(y.qkv), tr(y.o), tr(y.fc1), tr(y.fc2);
        tr(m->head);
        RG_CUDA(cudaGetLastError());
        RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
    }
    if (!m->bf16) {  // hi | lo | hi pieces for the f32-accurate tensor-core prompt pass
        auto sp = [&](rg_linear& lin) {
            if (!lin.Wt) return;
            dim3 grid(rg_cdiv(lin.N, 32), rg_cdiv(lin.K, 32)), block(32, 8);
            rg_split3_wt_kernel<<<grid, block, 0, m->ctx->stream>>>((const float*)lin.W, lin.ldw, lin.K, lin.N, (__nv_bfloat16*)lin.Wt);
            RG_LAUNCHED(m->ctx);
        };
        for (auto& y : m->layers) sp(y.qkv), sp(y.o), sp(y.fc1), sp(y.fc2);
        sp(m->head);
        RG_CUDA(cudaGetLastError());
        RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
    }
    m->loaded = true;
    m->pos = 0;
    m->curB = 0;
    RG_TRY(rg_mega_create(m));
    return rg_cloop_create(m);
}

// ---------------------------------------------------------------------------
// prompt pass / full forward
// ---------------------------------------------------------------------------
static rg_status ensure_rows(rg_gpt* m, size_t rows) {
    if (rows <= m->rowsCap) return RG_OK;
    RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
    dfree(m, m->px), dfree(m, m->pln), dfree(m, m->pqkv), dfree(m, m->pattn), dfree(m, m->ph), dfree(m, m->plast);
    dfree(m, m->ptp), dfree(m, m->pa16), dfree(m, m->pq16), dfree(m, m->pvt16);
    if (m->graph) cudaGraphExecDestroy(m->graph), m->graph = nullptr;  // a captured step may point into the old buffers
    m->px = m->pln = m->pqkv = m->pattn = m->ph = m->plast = m->ptp = nullptr;
    m->pa16 = m->pq16 = m->pvt16 = nullptr;
    m->rowsCap = 0;
    RG_TRY(dalloc(m, (void**)&m->px, rows * m->D * 4));
    RG_TRY(dalloc(m, (void**)&m->pln, rows * m->D * 4));
    RG_TRY(dalloc(m, (void**)&m->pqkv, rows * 3 * m->Dl * 4));
    RG_TRY(dalloc(m, (void**)&m->pattn, rows * m->Dl * 4));
    RG_TRY(dalloc(m, (void**)&m->ph, rows * m->Fl * 4));
    if (m->tp_size > 1) RG_TRY(dalloc(m, (void**)&m->ptp, rows * m->D * 4));
    if (!m->pws) {  // 32 MiB: enough to split the k range of every few-row projection of the supported shapes
        m->pwsFloats = (size_t)8 << 20;
        RG_TRY(dalloc(m, (void**)&m->pws, m->pwsFloats * 4));
    }
    if (m->use_tc)
        RG_TRY(dalloc(m, &m->pa16, std::max<size_t>(rows, 128) * (size_t)std::max(m->D, m->Fl) * (m->bf16 ? 2 : 6)));
    if (m->bf16 && m->use_tc && m->hd == 64) {
        RG_TRY(dalloc(m, &m->pq16, rows * m->Dl * 2));
        RG_TRY(dalloc(m, &m->pvt16, (rows + 64 * (size_t)std::max(m->Bmax, 1)) * m->Dl * 2));
    }
    RG_TRY(dalloc(m, (void**)&m->plast, (size_t)m->Bmax * m->D * 4));
    m->rowsCap = rows;
    return RG_OK;
}

static rg_status tp_ready(rg_gpt* m) {
    if (m->tp_size > 1 && !m->nccl_comm)
        return rg_fail(RG_ERR_INVALID_INPUT, "tensor-parallel model: call rg_gpt_tp_init on every rank first");
    return RG_OK;
}
static rg_status tp_allreduce(rg_gpt* m, float* buf, size_t n) {
    RG_NCCL(g_nccl.AllReduce(buf, buf, n, ncclFloat32, ncclSum, (ncclComm_t)m->nccl_comm, m->ctx->stream));
    RG_LAUNCHED(m->ctx);
    return RG_OK;
}
static rg_status tp_allgather(rg_gpt* m, const float* send, float* recv, size_t n_per_rank) {
    RG_NCCL(g_nccl.AllGather(send, recv, n_per_rank, ncclFloat32, (ncclComm_t)m->nccl_comm, m->ctx->stream));
    RG_LAUNCHED(m->ctx);
    return RG_OK;
}

static rg_status gemm(rg_gpt* m, const float* A, int M, const rg_linear& lin, float* Cout, const float* res, int act,
                      bool with_bias = true, long long ldc = -1) {
    rg_gemm_args p;
    memset(&p, 0, sizeof(p));
    p.A = A, p.lda = lin.K;
    p.W = lin.W, p.ldw = lin.ldw;
    p.C = Cout, p.ldc = ldc < 0 ? lin.N : ldc;
    p.M = M, p.N = lin.N, p.K = lin.K;
    p.bias = with_bias ? lin.b : nullptr, p.res = res, p.ldres = lin.N, p.act = act;
    if (m->bf16 && m->use_tc && lin.Wt && m->pa16 && M >= 8 && lin.K % 64 == 0) {
        // dense contraction on the tensor cores: bf16 operands (activations rounded on the way in), fp32 accumulate
        const size_t cnt = (size_t)M * lin.K;
        rg_to_bf16_kernel<<<rg_cdiv((long long)cnt, 1024), 256, 0, m->ctx->stream>>>(A, (__nv_bfloat16*)m->pa16, cnt);
        RG_LAUNCHED(m->ctx);
        rg_status st = rg_gemm_bf16_tc(m->ctx, m->pa16, M, lin.K, lin.Wt, lin.N, Cout, p.ldc, p.bias, res, lin.N, act);
        if (st == RG_OK) return RG_OK;
        if (st != RG_ERR_UNSUPPORTED) return st;
    }
    if (!m->bf16 && m->use_tc && lin.Wt && m->pa16 && M >= 32 && (3 * lin.K) % 64 == 0) {
        // f32 mode with enough rows for a tensor tile: split both operands into bf16 pieces (see lin.Wt) and run the
        // same tcgen05 GEMM over the concatenated K range
        const size_t cnt = (size_t)M * lin.K;
        rg_split3_rows_kernel<<<rg_cdiv((long long)cnt, 256), 256, 0, m->ctx->stream>>>(A, lin.K, cnt, (__nv_bfloat16*)m->pa16);
        RG_LAUNCHED(m->ctx);
        rg_status st = rg_gemm_bf16_tc(m->ctx, m->pa16, M, 3 * lin.K, lin.Wt, lin.N, Cout, p.ldc, p.bias, res, lin.N, act);
        if (st == RG_OK) return RG_OK;
        if (st != RG_ERR_UNSUPPORTED) return st;
    }
    int nl = 1;
    if (m->bf16) RG_CUDA(rg_gemm_launch<__nv_bfloat16>(m->ctx->stream, p, 1, m->pws, m->pwsFloats, m->ctx->sm_count, &nl));
    else RG_CUDA(rg_gemm_launch<float>(m->ctx->stream, p, 1, m->pws, m->pwsFloats, m->ctx->sm_count, &nl));
    m->ctx->launches += nl;
    return RG_OK;
}

template <typename KT>
static rg_status attn_rows(rg_gpt* m, int l, int B, int T) {
    const KT* kc = (const KT*)(m->kc + (size_t)l * m->kv_layer_bytes);
    const KT* vc = (const KT*)(m->vc + (size_t)l * m->kv_layer_bytes);
    cudaStream_t s = m->ctx->stream;
    rg_kv_scatter_kernel<KT><<<B * T, 256, 0, s>>>(m->pqkv, (KT*)kc, (KT*)vc, T, m->Hl, m->hd, m->C, m->Dl);
    const int causal = m->cfg.causal ? 1 : 0;
    if (sizeof(KT) == 2 && m->pq16 && m->pvt16 && B <= std::max(m->Bmax, 1)) {
        // bf16 mode, head_dim 64: attention of all rows on the tensor cores
        RG_LAUNCHED(m->ctx);
        rg_status st = rg_attn_bf16_tc(m->ctx, m->pqkv, kc, B, m->Hl, T, m->C, m->Dl, m->hd, causal, m->pq16, m->pvt16, m->pattn);
        if (st == RG_OK) return RG_OK;
        if (st != RG_ERR_UNSUPPORTED) return st;
        m->ctx->launches -= 1;
    }
    dim3 grid(rg_cdiv(T, 8), m->Hl, B);
    const float scale = 1.f / sqrtf((float)m->hd);
    if (m->hd == 32)
        rg_attn_rows_kernel<KT, 32><<<grid, 256, 0, s>>>(m->pqkv, kc, vc, m->pattn, T, m->Hl, m->C, m->Dl, scale, causal);
    else if (m->hd == 64)
        rg_attn_rows_kernel<KT, 64><<<grid, 256, 0, s>>>(m->pqkv, kc, vc, m->pattn, T, m->Hl, m->C, m->Dl, scale, causal);
    else
        rg_attn_rows_kernel<KT, 128><<<grid, 256, 0, s>>>(m->pqkv, kc, vc, m->pattn, T, m->Hl, m->C, m->Dl, scale, causal);
    m->ctx->launches += 2;
    RG_CUDA(cudaGetLastError());
    return RG_OK;
}

// x += A . W + b for a row-split projection: every rank holds a K-slice, the partial products are summed
// over the ranks (NCCL all-reduce over NVLink), bias and residual are added once.
static rg_status gemm_rowsplit_residual(rg_gpt* m, const float* A, int M, const rg_linear& lin, float* x) {
    if (m->tp_size == 1) return gemm(m, A, M, lin, x, x, -1);
    RG_TRY(gemm(m, A, M, lin, m->ptp, nullptr, -1, false));
    RG_TRY(tp_allreduce(m, m->ptp, (size_t)M * lin.N));
    rg_add_bias_res_kernel<<<rg_cdiv((long long)M * lin.N, 256), 256, 0, m->ctx->stream>>>(x, m->ptp, lin.b, (size_t)M, lin.N);
    RG_LAUNCHED(m->ctx);
    return RG_OK;
}

// room for the all-gather of `rows` rows of logits (allocates: never call inside a stream capture)
static rg_status ensure_gather(rg_gpt* m, int rows) {
    const size_t per = (size_t)rows * m->Vpad;
    if (m->tp_size == 1 || per * (m->tp_size + 1) <= m->pgatherCap) return RG_OK;
    RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
    dfree(m, m->pgather);
    m->pgather = nullptr, m->pgatherCap = 0;
    RG_TRY(dalloc(m, (void**)&m->pgather, per * (m->tp_size + 1) * 4));
    RG_CUDA(cudaMemset(m->pgather, 0, per * (m->tp_size + 1) * 4));
    m->pgatherCap = per * (m->tp_size + 1);
    if (m->graph) cudaGraphExecDestroy(m->graph), m->graph = nullptr;
    return RG_OK;
}

// logits of `rows` rows: local vocabulary slice, then (tensor parallel) all-gather and re-interleave
static rg_status head_logits(rg_gpt* m, const float* A, int rows, float* logits) {
    if (m->tp_size == 1) return gemm(m, A, rows, m->head, logits, nullptr, -1);
    const size_t per = (size_t)rows * m->Vpad;
    RG_TRY(ensure_gather(m, rows));
    float* local = m->pgather + per * m->tp_size;
    RG_CUDA(cudaMemsetAsync(local, 0, per * 4, m->ctx->stream));
    RG_TRY(gemm(m, A, rows, m->head, local, nullptr, -1, true, m->Vpad));
    RG_TRY(tp_allgather(m, local, m->pgather, per));
    rg_ungather_logits_kernel<<<rg_cdiv((long long)rows * m->V, 256), 256, 0, m->ctx->stream>>>(m->pgather, logits, (size_t)rows,
                                                                                                m->V, m->Vpad);
    RG_LAUNCHED(m->ctx);
    return RG_OK;
}

// Runs ids tokens[b][0..T) (already on the device) through the model.  With
// full != null writes logits of every row there ([B*T][V], device); otherwise
// computes the last row only into m->logits and its greedy pick into
// m->picks / tokens[b][T].
static rg_status run_rows(rg_gpt* m, int B, int T, float* full) {
    const int M = B * T, D = m->D;
    RG_TRY(tp_ready(m));
    RG_TRY(ensure_rows(m, (size_t)M));
    cudaStream_t s = m->ctx->stream;
    if (m->bf16)
        rg_embed_rows_kernel<__nv_bfloat16><<<M, 128, 0, s>>>(m->tokens, m->C, T, (const __nv_bfloat16*)m->wte,
                                                              (const __nv_bfloat16*)m->wpe, D, m->ldt, m->px);
    else
        rg_embed_rows_kernel<float><<<M, 128, 0, s>>>(m->tokens, m->C, T, (const float*)m->wte, (const float*)m->wpe, D,
                                                      m->ldt, m->px);
    RG_LAUNCHED(m->ctx);
    const int act = m->cfg.activation;
    for (int l = 0; l < m->L; l++) {
        rg_layer& y = m->layers[l];
        rg_ln_rows_kernel<<<rg_cdiv(M, 8), 256, 0, s>>>(m->px, D, y.ln1g, y.ln1b, m->pln, (size_t)M, D, 1e-5f);
        RG_LAUNCHED(m->ctx);
        RG_TRY(gemm(m, m->pln, M, y.qkv, m->pqkv, nullptr, -1));
        if (m->bf16) RG_TRY(attn_rows<__nv_bfloat16>(m, l, B, T));
        else RG_TRY(attn_rows<float>(m, l, B, T));
        RG_TRY(gemm_rowsplit_residual(m, m->pattn, M, y.o, m->px));
        rg_ln_rows_kernel<<<rg_cdiv(M, 8), 256, 0, s>>>(m->px, D, y.ln2g, y.ln2b, m->pln, (size_t)M, D, 1e-5f);
        RG_LAUNCHED(m->ctx);
        RG_TRY(gemm(m, m->pln, M, y.fc1, m->ph, nullptr, act));
        RG_TRY(gemm_rowsplit_residual(m, m->ph, M, y.fc2, m->px));
    }
    if (full) {
        rg_ln_rows_kernel<<<rg_cdiv(M, 8), 256, 0, s>>>(m->px, D, m->lnfg, m->lnfb, m->pln, (size_t)M, D, 1e-5f);
        RG_LAUNCHED(m->ctx);
        RG_TRY(head_logits(m, m->pln, M, full));
    } else {
        rg_ln_rows_kernel<<<rg_cdiv(B, 8), 256, 0, s>>>(m->px + (size_t)(T - 1) * D, (long long)T * D, m->lnfg, m->lnfb,
                                                        m->plast, (size_t)B, D, 1e-5f);
        RG_LAUNCHED(m->ctx);
        RG_TRY(head_logits(m, m->plast, B, m->logits));
        rg_argmax_rows_kernel<<<B, 1024, 0, s>>>(m->logits, m->V, m->picks, m->tokens, m->C, T);
        RG_LAUNCHED(m->ctx);
    }
    RG_CUDA(cudaGetLastError());
    return RG_OK;
}

static rg_status check_ready(rg_gpt* m, size_t B) {
    if (!m->loaded) return rg_fail(RG_ERR_INVALID_INPUT, "model parameters have not been loaded");
    if (B == 0 || B > (size_t)m->Bmax)
        return rg_fail(RG_ERR_INVALID_INPUT, "batch %zu outside 1..max_batch (%d)", B, m->Bmax);
    return RG_OK;
}

// ids [B][T] host -> tokens[b][0..T)
static rg_status upload_ids(rg_gpt* m, const uint32_t* ids, size_t B, size_t T) {
    for (size_t i = 0; i < B * T; i++)
        if (ids[i] >= (uint32_t)m->V)
            return rg_fail(RG_ERR_INVALID_INPUT, "Invalid input: index %u out of bounds for vocabulary size %d", ids[i], m->V);
    RG_CUDA(cudaMemcpy2DAsync(m->tokens, (size_t)m->C * 4, ids, T * 4, T * 4, B, cudaMemcpyHostToDevice, m->ctx->stream));
    return RG_OK;
}

extern "C" rg_status rg_gpt_forward(rg_gpt* m, const float* idx_f32, size_t B, size_t T, float* logits) {
    if (!m || !idx_f32 || !logits) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    RG_TRY(check_ready(m, B));
    if (T == 0) return rg_fail(RG_ERR_INVALID_INPUT, "empty sequence");
    if (T > (size_t)m->C)
        return rg_fail(RG_ERR_INVALID_INPUT, "Invalid input: index %zu out of bounds for vocabulary size %d (positions)", T - 1,
                       m->C);
    std::vector<uint32_t> ids(B * T);
    for (size_t i = 0; i < B * T; i++) {
        const float f = idx_f32[i];
        if (!(f >= 0.f) || (size_t)f >= (size_t)m->V)
            return rg_fail(RG_ERR_INVALID_INPUT, "Invalid input: index %g out of bounds for vocabulary size %d", (double)f, m->V);
        ids[i] = (uint32_t)f;  // `as usize` truncation, src/ops/embedding.rs:50
    }
    rg_ctx_guard g(m->ctx);
    RG_TRY(upload_ids(m, ids.data(), B, T));
    const size_t need = B * T * (size_t)m->V;
    if (need > m->plogitsCap) {
        RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
        dfree(m, m->plogits);
        m->plogits = nullptr, m->plogitsCap = 0;
        RG_TRY(dalloc(m, (void**)&m->plogits, need * 4));
        m->plogitsCap = need;
    }
    RG_TRY(run_rows(m, (int)B, (int)T, m->plogits));
    RG_CUDA(cudaMemcpyAsync(logits, m->plogits, need * 4, cudaMemcpyDeviceToHost, m->ctx->stream));
    RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
    m->pos = 0, m->curB = 0;  // the cache now holds this call's keys, not a generation context
    return rg_tc_wait_check(m->ctx);
}

static rg_status set_pos(rg_gpt* m, size_t T) {
    rg_set_int2_kernel<<<1, 1, 0, m->ctx->stream>>>(m->d_pos_next, m->d_pos, (int)T);
    RG_LAUNCHED(m->ctx);
    RG_CUDA(cudaGetLastError());
    m->pos = T;
    return RG_OK;
}

static rg_status prefill_locked(rg_gpt* m, const uint32_t* ids, size_t B, size_t T, float* logits_last, uint32_t* argmax) {
    if (T == 0) return rg_fail(RG_ERR_INVALID_INPUT, "empty prompt");
    if (T > (size_t)m->C) return rg_fail(RG_ERR_INVALID_INPUT, "prompt of %zu ids exceeds block_size %d", T, m->C);
    RG_TRY(upload_ids(m, ids, B, T));
    RG_TRY(run_rows(m, (int)B, (int)T, nullptr));
    RG_TRY(set_pos(m, T));
    m->curB = B;
    if (logits_last)
        RG_CUDA(cudaMemcpyAsync(logits_last, m->logits, B * (size_t)m->V * 4, cudaMemcpyDeviceToHost, m->ctx->stream));
    if (argmax) RG_CUDA(cudaMemcpyAsync(argmax, m->picks, B * 4, cudaMemcpyDeviceToHost, m->ctx->stream));
    if (logits_last || argmax) {
        RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
        return rg_tc_wait_check(m->ctx);
    }
    return RG_OK;
}

extern "C" rg_status rg_gpt_prefill(rg_gpt* m, const uint32_t* ids, size_t B, size_t T, float* logits_last,
                                    uint32_t* argmax) {
    if (!m || !ids) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    RG_TRY(check_ready(m, B));
    rg_ctx_guard g(m->ctx);
    return prefill_locked(m, ids, B, T, logits_last, argmax);
}

// ---------------------------------------------------------------------------
// token step
// ---------------------------------------------------------------------------
template <typename WT, int BT>
static void launch_gemv_bt(rg_gpt* m, const rg_gemv_args& a) {
    constexpr int NT = 32 * rg_wvec<WT>::N;
    dim3 grid(rg_cdiv(a.N, NT), a.ksplit, rg_cdiv(a.B, BT));
    const int xlen = a.in.post == RG_POST_LN ? a.K : a.krows;
    const size_t smem = (size_t)BT * xlen * 4;
    rg_launch(m->ctx->pdl, rg_gemv_kernel<WT, BT>, grid, dim3(256), smem, m->ctx->stream, a);
}
template <typename WT>
static void launch_gemv_wt(rg_gpt* m, const rg_gemv_args& a) {
    switch (batch_tile(a.B)) {
        case 1: launch_gemv_bt<WT, 1>(m, a); break;
        case 2: launch_gemv_bt<WT, 2>(m, a); break;
        case 4: launch_gemv_bt<WT, 4>(m, a); break;
        default: launch_gemv_bt<WT, 8>(m, a); break;
    }
}
static void launch_gemv(rg_gpt* m, const rg_linear& lin, const rg_vec_in& in, int B) {
    rg_gemv_args a;
    a.in = in;
    a.W = lin.W, a.ldw = lin.ldw, a.K = lin.K, a.N = lin.N, a.B = B;
    a.ksplit = lin.ksplit, a.krows = lin.krows, a.out = lin.parts;
    if (m->bf16) launch_gemv_wt<__nv_bfloat16>(m, a);
    else launch_gemv_wt<float>(m, a);
}

static rg_vec_in vec_reduce(const float* base, const float* bias, const rg_linear* producer, int post) {
    rg_vec_in in;
    memset(&in, 0, sizeof(in));
    in.kind = RG_IN_REDUCE;
    in.base = base, in.bias = bias;
    in.parts = producer ? producer->parts : nullptr;
    in.nparts = producer ? producer->ksplit : 0;
    in.post = post;
    return in;
}

template <typename KT>
static void launch_attn_step(rg_gpt* m, int l, int B) {
    rg_layer& y = m->layers[l];
    rg_attn_step_args a;
    a.qkv_parts = y.qkv.parts, a.nparts = y.qkv.ksplit, a.qkv_bias = y.qkv.b;
    a.kcache = m->kc + (size_t)l * m->kv_layer_bytes, a.vcache = m->vc + (size_t)l * m->kv_layer_bytes;
    a.ap = m->ap, a.pos = m->d_pos;
    a.B = B, a.H = m->Hl, a.C = m->C, a.D = m->Dl, a.NS = m->NS;
    a.scale = 1.f / sqrtf((float)m->hd);
    dim3 grid(m->NS, m->Hl, B);
    cudaStream_t s = m->ctx->stream;
    const bool pdl = m->ctx->pdl;
    if (m->hd == 32) rg_launch(pdl, rg_attn_step_kernel<KT, 32>, grid, dim3(128), 0, s, a);
    else if (m->hd == 64) rg_launch(pdl, rg_attn_step_kernel<KT, 64>, grid, dim3(128), 0, s, a);
    else rg_launch(pdl, rg_attn_step_kernel<KT, 128>, grid, dim3(128), 0, s, a);
}

// Enqueue the kernels of one token step for B sequences; returns how many.
// Tensor parallel: the k-split partials of a row-split projection are summed locally, then over the ranks;
// returns the "producer" the next stage reads (one part: the reduced vector).
static rg_linear tp_reduce(rg_gpt* m, const rg_linear& lin, int B, int* n, int site) {
    rg_linear r = lin;
    if (m->tp_size == 1) return r;
    const size_t cnt = (size_t)B * lin.N;
    if (m->tp_fused) {
        rg_tp_ar_args a;
        memset(&a, 0, sizeof(a));
        a.parts = lin.parts, a.nparts = lin.ksplit, a.cnt = cnt, a.out = m->tp_vec;
        for (int p = 0; p < m->tp_size; p++) a.peer[p] = m->tp_peer[p];
        a.T = m->tp_size, a.rank = m->tp_rank, a.slot = (size_t)m->Bmax * m->D;
        a.epoch = m->d_tp_epoch, a.site = site, a.nsites = 2 * m->L, a.err = m->d_tp_err, a.limit = RG_TP_SPIN_LIMIT;
        rg_tp_allreduce_kernel<<<rg_cdiv((long long)cnt, 256), 256, 0, m->ctx->stream>>>(a);
        *n += 1;
    } else {
        rg_reduce_parts_kernel<<<rg_cdiv((long long)cnt, 256), 256, 0, m->ctx->stream>>>(lin.parts, lin.ksplit, cnt, nullptr, 1,
                                                                                       m->tp_vec);
        g_nccl.AllReduce(m->tp_vec, m->tp_vec, cnt, ncclFloat32, ncclSum, (ncclComm_t)m->nccl_comm, m->ctx->stream);
        *n += 2;
    }
    r.parts = m->tp_vec, r.ksplit = 1;
    return r;
}

// Enqueue the kernels of one token step for B sequences; returns how many.
// While alive, projection / attention kernels of this context are launched with programmatic stream serialization
// (they all begin with rg_pdl_sync()); RG_B200_PDL=0 turns it off.
struct rg_pdl_scope {
    rg_ctx* c;
    explicit rg_pdl_scope(rg_ctx* ctx) : c(ctx) {
        const char* e = getenv("RG_B200_PDL");
        c->pdl = !(e && strcmp(e, "0") == 0);
    }
    ~rg_pdl_scope() { c->pdl = false; }
};

static int enqueue_step(rg_gpt* m, int B) {
    cudaStream_t s = m->ctx->stream;
    int n = 0;
    rg_pdl_scope pdl_scope(m->ctx);
    if (m->tp_fused) {
        rg_bump_kernel<<<1, 1, 0, s>>>(m->d_tp_epoch);  // every rank runs the same steps: the tags agree
        n++;
    }
    if (m->bf16)
        rg_embed_step_kernel<__nv_bfloat16><<<B, 128, 0, s>>>(m->tokens, m->C, (const __nv_bfloat16*)m->wte,
                                                              (const __nv_bfloat16*)m->wpe, m->D, m->ldt, m->xa,
                                                              m->d_pos_next, m->d_pos);
    else
        rg_embed_step_kernel<float><<<B, 128, 0, s>>>(m->tokens, m->C, (const float*)m->wte, (const float*)m->wpe, m->D,
                                                      m->ldt, m->xa, m->d_pos_next, m->d_pos);
    n++;
    const int act_post = m->cfg.activation == RG_ACT_RELU ? RG_POST_RELU : RG_POST_GELU;
    rg_linear prev_fc2;  // producer of the block input (reduced over the ranks when tensor parallel)
    const float* prev_b2 = nullptr;
    bool have_prev = false;
    for (int l = 0; l < m->L; l++) {
        rg_layer& y = m->layers[l];
        // x = x + b2 + fc2 partials of the previous block; LN1; QKV (this rank's heads)
        rg_vec_in in = vec_reduce(m->xa, prev_b2, have_prev ? &prev_fc2 : nullptr, RG_POST_LN);
        in.gamma = y.ln1g, in.beta = y.ln1b, in.store = m->xb;
        launch_gemv(m, y.qkv, in, B);
        if (m->bf16) launch_attn_step<__nv_bfloat16>(m, l, B);
        else launch_attn_step<float>(m, l, B);
        // merged heads -> output projection (row-split over the ranks' heads)
        rg_vec_in ia;
        memset(&ia, 0, sizeof(ia));
        ia.kind = RG_IN_ATTN, ia.ap = m->ap, ia.H = m->Hl, ia.hd = m->hd, ia.NS = m->NS, ia.post = RG_POST_NONE;
        launch_gemv(m, y.o, ia, B);
        const rg_linear o_red = tp_reduce(m, y.o, B, &n, 2 * l);
        // x = x + bo + partials; LN2; FC1 (this rank's hidden columns)
        rg_vec_in i1 = vec_reduce(m->xb, y.o.b, &o_red, RG_POST_LN);
        i1.gamma = y.ln2g, i1.beta = y.ln2b, i1.store = m->xa;
        launch_gemv(m, y.fc1, i1, B);
        // act(b1 + partials); FC2 (row-split)
        rg_vec_in i2 = vec_reduce(nullptr, y.fc1.b, &y.fc1, act_post);
        launch_gemv(m, y.fc2, i2, B);
        prev_fc2 = tp_reduce(m, y.fc2, B, &n, 2 * l + 1);
        prev_b2 = y.fc2.b;
        have_prev = true;
        n += 5;
    }
    rg_vec_in ih = vec_reduce(m->xa, prev_b2, &prev_fc2, RG_POST_LN);
    ih.gamma = m->lnfg, ih.beta = m->lnfb, ih.store = nullptr;
    launch_gemv(m, m->head, ih, B);
    rg_pick_args pa;
    pa.parts = m->head.parts, pa.nparts = m->head.ksplit, pa.bias = m->head.b, pa.logits = m->logits;
    pa.tokens = m->tokens, pa.picks = m->picks, pa.pos = m->d_pos, pa.pos_next = m->d_pos_next;
    pa.B = B, pa.V = m->V, pa.C = m->C;
    if (m->tp_size > 1) {
        // vocabulary slices: local logits (+bias) -> all-gather -> full rows in m->logits -> pick
        const size_t per = (size_t)B * m->Vpad;
        cudaMemsetAsync(m->tp_local, 0, per * 4, s);
        rg_reduce_parts_kernel<<<rg_cdiv((long long)B * m->Vl, 256), 256, 0, s>>>(m->head.parts, m->head.ksplit,
                                                                                 (size_t)B * m->Vl, m->head.b, m->Vl, m->tp_local,
                                                                                 m->Vpad);
        g_nccl.AllGather(m->tp_local, m->tp_gather, per, ncclFloat32, (ncclComm_t)m->nccl_comm, s);
        rg_ungather_logits_kernel<<<rg_cdiv((long long)B * m->V, 256), 256, 0, s>>>(m->tp_gather, m->logits, (size_t)B, m->V,
                                                                                   m->Vpad);
        pa.parts = m->logits, pa.nparts = 1, pa.bias = nullptr;
        n += 4;
    }
    rg_pick_kernel<<<B, 1024, 0, s>>>(pa);
    n += 2;
    return n;
}

// Token step for larger batches: with 8 or more sequences a projection is a (small-M) dense contraction, so the step
// runs on the prompt-pass kernels (LayerNorm rows, GEMM - tensor cores in bf16 mode -, row-split all-reduce when tensor
// parallel) around the KV-cache attention.  Returns the number of launches, or -1 on error.
static int enqueue_step_rows(rg_gpt* m, int B) {
    cudaStream_t s = m->ctx->stream;
    const uint64_t l0 = m->ctx->launches;
    const int D = m->D, act = m->cfg.activation;
    if (m->bf16)
        rg_embed_step_kernel<__nv_bfloat16><<<B, 128, 0, s>>>(m->tokens, m->C, (const __nv_bfloat16*)m->wte,
                                                              (const __nv_bfloat16*)m->wpe, D, m->ldt, m->px, m->d_pos_next,
                                                              m->d_pos);
    else
        rg_embed_step_kernel<float><<<B, 128, 0, s>>>(m->tokens, m->C, (const float*)m->wte, (const float*)m->wpe, D, m->ldt,
                                                      m->px, m->d_pos_next, m->d_pos);
    RG_LAUNCHED(m->ctx);
    for (int l = 0; l < m->L; l++) {
        rg_layer& y = m->layers[l];
        rg_ln_rows_kernel<<<rg_cdiv(B, 8), 256, 0, s>>>(m->px, D, y.ln1g, y.ln1b, m->pln, (size_t)B, D, 1e-5f);
        RG_LAUNCHED(m->ctx);
        if (gemm(m, m->pln, B, y.qkv, m->pqkv, nullptr, -1) != RG_OK) return -1;
        {   // attention over the cache: q, k, v rows are finished values here (one "partial", no bias left to add)
            rg_attn_step_args a;
            a.qkv_parts = m->pqkv, a.nparts = 1, a.qkv_bias = nullptr;
            a.kcache = m->kc + (size_t)l * m->kv_layer_bytes, a.vcache = m->vc + (size_t)l * m->kv_layer_bytes;
            a.ap = m->ap, a.pos = m->d_pos;
            a.B = B, a.H = m->Hl, a.C = m->C, a.D = m->Dl, a.NS = m->NS;
            a.scale = 1.f / sqrtf((float)m->hd);
            dim3 grid(m->NS, m->Hl, B);
            if (m->bf16) {
                if (m->hd == 32) rg_attn_step_kernel<__nv_bfloat16, 32><<<grid, 128, 0, s>>>(a);
                else if (m->hd == 64) rg_attn_step_kernel<__nv_bfloat16, 64><<<grid, 128, 0, s>>>(a);
                else rg_attn_step_kernel<__nv_bfloat16, 128><<<grid, 128, 0, s>>>(a);
            } else {
                if (m->hd == 32) rg_attn_step_kernel<float, 32><<<grid, 128, 0, s>>>(a);
                else if (m->hd == 64) rg_attn_step_kernel<float, 64><<<grid, 128, 0, s>>>(a);
                else rg_attn_step_kernel<float, 128><<<grid, 128, 0, s>>>(a);
            }
            rg_attn_merge_kernel<<<rg_cdiv(B * m->Dl, 256), 256, 0, s>>>(m->ap, m->pattn, B, m->Hl, m->hd, m->NS);
            m->ctx->launches += 2;
        }
        if (gemm_rowsplit_residual(m, m->pattn, B, y.o, m->px) != RG_OK) return -1;
        rg_ln_rows_kernel<<<rg_cdiv(B, 8), 256, 0, s>>>(m->px, D, y.ln2g, y.ln2b, m->pln, (size_t)B, D, 1e-5f);
        RG_LAUNCHED(m->ctx);
        if (gemm(m, m->pln, B, y.fc1, m->ph, nullptr, act) != RG_OK) return -1;
        if (gemm_rowsplit_residual(m, m->ph, B, y.fc2, m->px) != RG_OK) return -1;
    }
    rg_ln_rows_kernel<<<rg_cdiv(B, 8), 256, 0, s>>>(m->px, D, m->lnfg, m->lnfb, m->plast, (size_t)B, D, 1e-5f);
    RG_LAUNCHED(m->ctx);
    if (head_logits(m, m->plast, B, m->logits) != RG_OK) return -1;
    rg_pick_args pa;
    pa.parts = m->logits, pa.nparts = 1, pa.bias = nullptr, pa.logits = m->logits;
    pa.tokens = m->tokens, pa.picks = m->picks, pa.pos = m->d_pos, pa.pos_next = m->d_pos_next;
    pa.B = B, pa.V = m->V, pa.C = m->C;
    rg_pick_kernel<<<B, 1024, 0, s>>>(pa);
    RG_LAUNCHED(m->ctx);
    const int n = (int)(m->ctx->launches - l0);
    m->ctx->launches = l0;  // the caller accounts for the launches (once per replay when captured)
    return n;
}

static rg_status step_ready(rg_gpt* m, size_t steps) {
    if (!m->cfg.causal)
        return rg_fail(RG_ERR_UNSUPPORTED,
                       "the KV-cache token step needs causal attention; this model uses the reference's unmasked attention");
    if (m->curB == 0) return rg_fail(RG_ERR_INVALID_INPUT, "no context: call rg_gpt_prefill first");
    RG_TRY(tp_ready(m));
    if (m->pos + steps > (size_t)m->C)
        return rg_fail(RG_ERR_CONTEXT_FULL, "context full: position %zu + %zu steps exceeds block_size %d", m->pos, steps, m->C);
    return RG_OK;
}

// The same step with every small kernel between two projections folded into one: the tensor-core GEMM leaves raw
// k-split partial tiles, the attention kernel sums the q/k/v partials itself, and one kernel per projection does
// "sum partials + bias (+ residual + next LayerNorm | + activation) -> bf16 rows".  9 launches per block instead of 16.
static bool rows_tc_usable(const rg_gpt* m) {
    // Shards whose width is not a multiple of the GEMM's 64-wide k-blocks (hidden shard of 800 columns: GPT-2-XL shape on
    // 8 GPUs) keep the plain form: the kernel handles such a K (self-check: rg_debug_hook 8), but that configuration has not
    // been validated end to end on 8 GPUs.
    if (!(m->bf16 && m->use_tc && m->pa16) || m->D > RG_ROWS_MAX_D || m->D % 64 || m->Dl % 64 || m->Fl % 64) return false;
    if (m->tp_size > 1 && !(m->tp_fused && m->Bmax * (size_t)m->D >= 1)) return false;  // tensor parallel: the peer-memory exchange only
    for (const rg_layer& y : m->layers)
        if (!y.qkv.Wt || !y.o.Wt || !y.fc1.Wt || !y.fc2.Wt) return false;
    return m->head.Wt != nullptr;
}
static int enqueue_step_rows_tc(rg_gpt* m, int B) {
    cudaStream_t s = m->ctx->stream;
    const uint64_t l0 = m->ctx->launches;
    const int D = m->D, Dl = m->Dl, F = m->Fl, act = m->cfg.activation;  // Dl, Fl: this rank's shard (= D, F on one GPU)
    const bool tp = m->tp_size > 1;
    __nv_bfloat16* a16 = (__nv_bfloat16*)m->pa16;
    // every kernel of the step starts with rg_pdl_sync(): launched with programmatic stream serialization, the launch
    // latency of a kernel overlaps the execution of the one before it (RG_B200_PDL=0 turns the attribute off)
    rg_pdl_scope scope(m->ctx);
    const bool pdl = m->ctx->pdl;
    if (tp) {
        rg_bump_kernel<<<1, 1, 0, s>>>(m->d_tp_epoch);  // every rank runs the same steps: the tags of the exchanges agree
        m->ctx->launches += 1;
    }
    // a row-split projection (out-projection: site 0, FC2: site 1 of block l) ends with partial sums on every rank:
    // on one GPU the rows kernel adds bias + residual and normalises; tensor parallel, it also does the all-reduce
    auto rows_res_ln = [&](const float* parts_, int np_, const float* bias, const float* gamma, const float* beta, int site) {
        if (!tp) {
            rg_launch(pdl, rg_rows_res_ln_bf16_kernel, dim3(B), dim3(256), 0, s, parts_, np_, (size_t)B * D, bias, m->px, 1, gamma, beta,
                      a16, D);
        } else {
            rg_tp_ar_args a;
            memset(&a, 0, sizeof(a));
            a.parts = parts_, a.nparts = np_, a.cnt = (size_t)B * D, a.out = nullptr;
            for (int p = 0; p < m->tp_size; p++) a.peer[p] = m->tp_peer[p];
            a.T = m->tp_size, a.rank = m->tp_rank, a.slot = (size_t)m->Bmax * m->D;
            a.epoch = m->d_tp_epoch, a.site = site, a.nsites = 2 * m->L, a.err = m->d_tp_err, a.limit = RG_TP_SPIN_LIMIT;
            rg_launch(pdl, rg_rows_res_ln_tp_bf16_kernel, dim3(B), dim3(256), 0, s, a, bias, m->px, gamma, beta, a16, D);
        }
        RG_LAUNCHED(m->ctx);
    };
    rg_launch(pdl, rg_embed_step_kernel<__nv_bfloat16>, dim3(B), dim3(128), 0, s, m->tokens, m->C, (const __nv_bfloat16*)m->wte,
              (const __nv_bfloat16*)m->wpe, D, m->ldt, m->px, m->d_pos_next, m->d_pos);
    rg_launch(pdl, rg_rows_res_ln_bf16_kernel, dim3(B), dim3(256), 0, s, nullptr, 0, (size_t)0, nullptr, m->px, 0, m->layers[0].ln1g,
              m->layers[0].ln1b, a16, D);
    m->ctx->launches += 2;
    // context slices per (sequence, head): enough CTAs to fill the GPU a few times over, no more
    const int NS = std::max(1, std::min(m->NS, rg_cdiv(4 * m->ctx->sm_count, B * m->Hl)));
    const float* parts = nullptr;
    int np = 0;
    for (int l = 0; l < m->L; l++) {
        rg_layer& y = m->layers[l];
        if (rg_gemm_bf16_tc_parts(m->ctx, a16, B, D, y.qkv.Wt, 3 * Dl, &parts, &np) != RG_OK) return -1;
        {
            rg_attn_step_args a;
            a.qkv_parts = parts, a.nparts = np, a.qkv_bias = y.qkv.b;
            a.kcache = m->kc + (size_t)l * m->kv_layer_bytes, a.vcache = m->vc + (size_t)l * m->kv_layer_bytes;
            a.ap = m->ap, a.pos = m->d_pos;
            a.B = B, a.H = m->Hl, a.C = m->C, a.D = m->Dl, a.NS = NS;
            a.scale = 1.f / sqrtf((float)m->hd);
            if (NS == 1) a.out16 = a16;  // one slice per (sequence, head): the attention kernel finishes the rows itself
            dim3 grid(NS, m->Hl, B);
            if (m->hd == 32) rg_launch(pdl, rg_attn_step_kernel<__nv_bfloat16, 32>, grid, dim3(128), 0, s, a);
            else if (m->hd == 64) rg_launch(pdl, rg_attn_step_kernel<__nv_bfloat16, 64>, grid, dim3(128), 0, s, a);
            else rg_launch(pdl, rg_attn_step_kernel<__nv_bfloat16, 128>, grid, dim3(128), 0, s, a);
            m->ctx->launches += 1;
            if (NS > 1) {
                rg_launch(pdl, rg_attn_merge_kernel, dim3(rg_cdiv(B * Dl, 256)), dim3(256), 0, s, (const float*)m->ap, (float*)nullptr, B,
                          m->Hl, m->hd, NS, a16);
                m->ctx->launches += 1;
            }
        }
        if (rg_gemm_bf16_tc_parts(m->ctx, a16, B, Dl, y.o.Wt, D, &parts, &np) != RG_OK) return -1;
        rows_res_ln(parts, np, y.o.b, y.ln2g, y.ln2b, 2 * l);
        if (rg_gemm_bf16_tc_parts(m->ctx, a16, B, D, y.fc1.Wt, F, &parts, &np) != RG_OK) return -1;
        rg_launch(pdl, rg_rows_act_bf16_kernel, dim3(rg_cdiv((long long)B * F, 256)), dim3(256), 0, s, parts, np, (size_t)B * F,
                  (const float*)y.fc1.b, F, (size_t)B * F, act, a16);
        RG_LAUNCHED(m->ctx);
        if (rg_gemm_bf16_tc_parts(m->ctx, a16, B, F, y.fc2.Wt, D, &parts, &np) != RG_OK) return -1;
        const bool last = l + 1 == m->L;
        rows_res_ln(parts, np, y.fc2.b, last ? m->lnfg : m->layers[l + 1].ln1g, last ? m->lnfb : m->layers[l + 1].ln1b, 2 * l + 1);
    }
    if (!tp) {
        if (rg_gemm_bf16_tc(m->ctx, a16, B, D, m->head.Wt, m->V, m->logits, m->V, m->head.b, nullptr, 0, -1) != RG_OK) return -1;
    } else {
        // this rank's vocabulary slice -> all-gather of the padded slices -> [B][V] (the gather buffer exists: run_steps
        // made room for it before the capture)
        const size_t per = (size_t)B * m->Vpad;
        float* local = m->pgather + per * m->tp_size;
        // (the padding columns of `local` are zero since ensure_gather and are never written)
        if (rg_gemm_bf16_tc(m->ctx, a16, B, D, m->head.Wt, m->Vl, local, m->Vpad, m->head.b, nullptr, 0, -1) != RG_OK) return -1;
        if (tp_allgather(m, local, m->pgather, per) != RG_OK) return -1;
        rg_ungather_logits_kernel<<<rg_cdiv((long long)B * m->V, 256), 256, 0, s>>>(m->pgather, m->logits, (size_t)B, m->V, m->Vpad);
        RG_LAUNCHED(m->ctx);
    }
    rg_pick_args pa;
    pa.parts = m->logits, pa.nparts = 1, pa.bias = nullptr, pa.logits = m->logits;
    pa.tokens = m->tokens, pa.picks = m->picks, pa.pos = m->d_pos, pa.pos_next = m->d_pos_next;
    pa.B = B, pa.V = m->V, pa.C = m->C;
    rg_launch(pdl, rg_pick_kernel, dim3(B), dim3(1024), 0, s, pa);
    RG_LAUNCHED(m->ctx);
    const int n = (int)(m->ctx->launches - l0);
    m->ctx->launches = l0;
    return n;
}

static rg_status tp_check(rg_gpt* m);
// After a synchronise: has any bounded device wait given up (tensor-parallel all-reduce, the persistent token-loop
// kernels, the tensor-core kernels of the prompt pass and of the batched step)?
static rg_status waits_check(rg_gpt* m) {
    RG_TRY(tp_check(m));
    RG_TRY(rg_mega_check(m));
    RG_TRY(rg_cloop_check(m));
    return rg_tc_wait_check(m->ctx);
}

// need_logits: the caller reads the full logit rows afterwards.  A tensor-parallel persistent launch leaves every rank
// with its own vocabulary slice only (the ids are complete), so such a call takes the launch form, which gathers them.
static rg_status run_steps(rg_gpt* m, size_t steps, bool need_logits = false) {
    const int B = (int)m->curB;
    cudaStream_t s = m->ctx->stream;
    if (rg_cloop_supports(m, B)) {
        // one persistent kernel of thread-block clusters runs all the steps
        rg_status st = rg_cloop_run(m, B, m->pos, steps);
        if (st == RG_OK) {
            m->pos += steps;
            return RG_OK;
        }
        if (st != RG_ERR_UNSUPPORTED) return st;
        // no cluster shape of this GPU fits the model, or the clusters cannot all be resident: the forms below
        // compute the same thing
    }
    if (rg_mega_supports(m, B) && !(m->tp_size > 1 && need_logits)) {
        // one persistent cooperative kernel runs all the steps
        rg_status st = rg_mega_run(m, B, m->pos, steps);
        if (st == RG_OK) {
            m->pos += steps;
            return RG_OK;
        }
        if (st != RG_ERR_UNSUPPORTED) return st;
        // the model does not fit the persistent kernel, or its CTAs cannot all be resident at once (a GPU shared
        // with other work): the CUDA-graph step below computes the same thing
    }
    const bool rows_path = (m->bf16 && m->use_tc) ? B >= 8 : B >= 32;  // where a projection is worth a GEMM launch
    if (rows_path) {  // before capture: may allocate
        RG_TRY(ensure_rows(m, (size_t)std::max(B, 128)));
        RG_TRY(ensure_gather(m, B));
    }
    const char* rows_env = getenv("RG_B200_ROWS_STEP");  // "plain": one kernel per operation (for comparisons)
    const bool fuse_env = !(rows_env && strcmp(rows_env, "plain") == 0);
    const bool rows_fused = rows_path && fuse_env && rows_tc_usable(m);
    if (!m->use_graph) {
        for (size_t i = 0; i < steps; i++) {
            const int n = rows_path ? (rows_fused ? enqueue_step_rows_tc(m, B) : enqueue_step_rows(m, B)) : enqueue_step(m, B);
            if (n < 0) return RG_ERR_BACKEND;
            m->ctx->launches += n;
            RG_CUDA(cudaGetLastError());
        }
    } else {
        if (!m->graph || m->graphB != (size_t)B) {
            if (m->graph) cudaGraphExecDestroy(m->graph), m->graph = nullptr;
            cudaGraph_t gr = nullptr;
            RG_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
            m->kernels_per_step =
                rows_path ? (rows_fused ? enqueue_step_rows_tc(m, B) : enqueue_step_rows(m, B)) : enqueue_step(m, B);
            cudaError_t e = cudaStreamEndCapture(s, &gr);
            const cudaError_t le = cudaGetLastError();  // a launch that was rejected while capturing leaves its error here
            if (e == cudaSuccess && le != cudaSuccess) e = le;
            if (m->kernels_per_step < 0) {
                if (gr) cudaGraphDestroy(gr);
                return RG_ERR_BACKEND;
            }
            if (e != cudaSuccess) return rg_fail(RG_ERR_BACKEND, "graph capture failed: %s", cudaGetErrorString(e));
            e = cudaGraphInstantiate(&m->graph, gr, 0);
            cudaGraphDestroy(gr);
            if (e != cudaSuccess) return rg_fail(RG_ERR_BACKEND, "graph instantiate failed: %s", cudaGetErrorString(e));
            m->graphB = B;
        }
        for (size_t i = 0; i < steps; i++) RG_CUDA(cudaGraphLaunch(m->graph, s));
        m->ctx->launches += (uint64_t)m->kernels_per_step * steps;
    }
    m->pos += steps;
    return RG_OK;
}

extern "C" rg_status rg_gpt_decode_step(rg_gpt* m, const uint32_t* tok, float* logits, uint32_t* argmax) {
    if (!m || !tok) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    rg_ctx_guard g(m->ctx);
    RG_TRY(step_ready(m, 1));
    const size_t B = m->curB;
    for (size_t b = 0; b < B; b++)
        if (tok[b] >= (uint32_t)m->V)
            return rg_fail(RG_ERR_INVALID_INPUT, "Invalid input: index %u out of bounds for vocabulary size %d", tok[b], m->V);
    RG_CUDA(cudaMemcpy2DAsync(m->tokens + m->pos, (size_t)m->C * 4, tok, 4, 4, B, cudaMemcpyHostToDevice, m->ctx->stream));
    RG_TRY(run_steps(m, 1, logits != nullptr));
    if (logits) RG_CUDA(cudaMemcpyAsync(logits, m->logits, B * (size_t)m->V * 4, cudaMemcpyDeviceToHost, m->ctx->stream));
    if (argmax) RG_CUDA(cudaMemcpyAsync(argmax, m->picks, B * 4, cudaMemcpyDeviceToHost, m->ctx->stream));
    RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
    return waits_check(m);
}

extern "C" rg_status rg_gpt_decode_run(rg_gpt* m, size_t n_steps) {
    if (!m) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    rg_ctx_guard g(m->ctx);
    RG_TRY(step_ready(m, n_steps));
    return run_steps(m, n_steps);
}

extern "C" rg_status rg_gpt_rewind(rg_gpt* m, size_t T, const uint32_t* tok) {
    if (!m) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    rg_ctx_guard g(m->ctx);
    if (m->curB == 0) return rg_fail(RG_ERR_INVALID_INPUT, "no context: call rg_gpt_prefill first");
    if (T > m->pos) return rg_fail(RG_ERR_INVALID_INPUT, "cannot rewind forward: position %zu, asked for %zu", m->pos, T);
    if (T >= (size_t)m->C) return rg_fail(RG_ERR_CONTEXT_FULL, "position %zu is outside block_size %d", T, m->C);
    if (tok) {
        for (size_t b = 0; b < m->curB; b++)
            if (tok[b] >= (uint32_t)m->V) return rg_fail(RG_ERR_INVALID_INPUT, "Invalid input: index %u out of bounds", tok[b]);
        RG_CUDA(cudaMemcpy2DAsync(m->tokens + T, (size_t)m->C * 4, tok, 4, 4, m->curB, cudaMemcpyHostToDevice,
                                  m->ctx->stream));
    }
    return set_pos(m, T);
}

extern "C" rg_status rg_gpt_read_tokens(rg_gpt* m, size_t from, size_t n, uint32_t* out) {
    if (!m || !out) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    rg_ctx_guard g(m->ctx);
    if (m->curB == 0) return rg_fail(RG_ERR_INVALID_INPUT, "no context");
    if (from + n > (size_t)m->C) return rg_fail(RG_ERR_INVALID_INPUT, "ids [%zu, %zu) outside block_size %d", from, from + n, m->C);
    if (n)
        RG_CUDA(cudaMemcpy2DAsync(out, n * 4, m->tokens + from, (size_t)m->C * 4, n * 4, m->curB, cudaMemcpyDeviceToHost,
                                  m->ctx->stream));
    RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
    return waits_check(m);
}

extern "C" size_t rg_gpt_position(const rg_gpt* m) { return m ? m->pos : 0; }

extern "C" rg_status rg_gpt_reset(rg_gpt* m) {
    if (!m) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    rg_ctx_guard g(m->ctx);
    m->curB = 0;
    return set_pos(m, 0);
}

// ---------------------------------------------------------------------------
// generate
// ---------------------------------------------------------------------------
// Draw the id at `slot` of every sequence from the finished logits rows (m->logits).
static rg_status sample_rows(rg_gpt* m, int B, size_t slot, float temperature, size_t top_k, uint64_t seed, unsigned step) {
    rg_sample_args a;
    a.logits = m->logits, a.tokens = m->tokens, a.picks = m->picks;
    a.V = m->V, a.C = m->C, a.slot = (int)slot;
    a.top_k = top_k >= (size_t)m->V ? 0 : (int)top_k;
    a.inv_temperature = 1.f / temperature;
    a.seed = seed, a.step = step;
    rg_sample_kernel<<<B, 1024, 0, m->ctx->stream>>>(a);
    RG_LAUNCHED(m->ctx);
    RG_CUDA(cudaGetLastError());
    return RG_OK;
}

extern "C" rg_status rg_gpt_generate(rg_gpt* m, const uint32_t* prompt, size_t B, size_t P, size_t max_new,
                                     float temperature, size_t top_k, uint64_t seed, uint32_t* out) {
    if (!m || !prompt || (!out && max_new)) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    RG_TRY(check_ready(m, B));
    const bool greedy = top_k == 1;
    if (!greedy && !(temperature > 0.f)) return rg_fail(RG_ERR_INVALID_INPUT, "temperature must be positive, got %g", (double)temperature);
    if (P == 0) return rg_fail(RG_ERR_INVALID_INPUT, "empty prompt");
    if (max_new == 0) return RG_OK;
    rg_ctx_guard g(m->ctx);
    if (m->cfg.causal) {
        if (P + max_new - 1 > (size_t)m->C)
            return rg_fail(RG_ERR_CONTEXT_FULL,
                           "prompt %zu + %zu new ids needs %zu cache rows, block_size is %d (the KV cache cannot slide)", P,
                           max_new, P + max_new - 1, m->C);
        RG_TRY(prefill_locked(m, prompt, B, P, nullptr, nullptr));
        if (greedy) {
            if (max_new > 1) RG_TRY(run_steps(m, max_new - 1));
        } else {
            // one step at a time: the draw replaces the greedy pick the step left at the next position
            RG_TRY(sample_rows(m, (int)B, P, temperature, top_k, seed, 0));
            for (size_t i = 1; i < max_new; i++) {
                RG_TRY(run_steps(m, 1, true));
                RG_TRY(sample_rows(m, (int)B, P + i, temperature, top_k, seed, (unsigned)i));
            }
        }
        if (P + max_new <= (size_t)m->C) {
            RG_CUDA(cudaMemcpy2DAsync(out, max_new * 4, m->tokens + P, (size_t)m->C * 4, max_new * 4, B,
                                      cudaMemcpyDeviceToHost, m->ctx->stream));
        } else {  // the last pick has no slot in the id buffer: it is in picks
            if (max_new > 1)
                RG_CUDA(cudaMemcpy2DAsync(out, max_new * 4, m->tokens + P, (size_t)m->C * 4, (max_new - 1) * 4, B,
                                          cudaMemcpyDeviceToHost, m->ctx->stream));
            RG_CUDA(cudaMemcpy2DAsync(out + (max_new - 1), max_new * 4, m->picks, 4, 4, B, cudaMemcpyDeviceToHost,
                                      m->ctx->stream));
        }
        RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
        return waits_check(m);
    }
    // The reference's loop proper (no mask, so no cache): every new id re-runs the
    // whole window of the last block_size ids (wasm_api.rs:102-118).
    std::vector<std::vector<uint32_t>> ids(B);
    for (size_t b = 0; b < B; b++) ids[b].assign(prompt + b * P, prompt + (b + 1) * P);
    std::vector<uint32_t> window, picks(B);
    for (size_t i = 0; i < max_new; i++) {
        const size_t len = ids[0].size();
        const size_t T = std::min(len, (size_t)m->C), start = len - T;
        window.resize(B * T);
        for (size_t b = 0; b < B; b++) memcpy(&window[b * T], &ids[b][start], T * 4);
        RG_TRY(upload_ids(m, window.data(), B, T));
        RG_TRY(run_rows(m, (int)B, (int)T, nullptr));
        if (!greedy) RG_TRY(sample_rows(m, (int)B, (size_t)m->C, temperature, top_k, seed, (unsigned)i));
        RG_CUDA(cudaMemcpyAsync(picks.data(), m->picks, B * 4, cudaMemcpyDeviceToHost, m->ctx->stream));
        RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
        for (size_t b = 0; b < B; b++) {
            ids[b].push_back(picks[b]);
            out[b * max_new + i] = picks[b];
        }
    }
    m->pos = 0, m->curB = 0;
    return RG_OK;
}

extern "C" double rg_gpt_decode_step_bytes(const rg_gpt* m, size_t B, double mean_ctx) {
    if (!m) return 0.0;
    // per GPU: with tensor parallelism the projections, their split biases and the cache are this rank's shard; LayerNorm
    // parameters, the biases added after an all-reduce and the two embedding rows are read by every rank
    const double D = m->D, L = m->L, Dl = m->Dl, Fl = m->Fl, Vl = m->Vl;
    const double layer = (D * 3.0 * Dl + 3.0 * Dl) + (Dl * D + D) + (D * Fl + Fl) + (Fl * D + D) + 4.0 * D;
    const double w = L * layer + D * Vl + Vl + 4.0 * D;
    const double kv = m->bf16 ? 2.0 : 4.0;
    return (double)m->wsize * w + (double)B * kv * 2.0 * L * Dl * mean_ctx;
}

extern "C" rg_status rg_gpt_tp_unique_id(uint8_t id_out[128]) {
    if (!id_out) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    RG_TRY(load_nccl());
    ncclUniqueId id;
    RG_NCCL(g_nccl.GetUniqueId(&id));
    memcpy(id_out, id.internal, 128);
    return RG_OK;
}

static void tp_peer_close(rg_gpt* m) {
    for (int r = 0; r < RG_TP_MAX; r++) {
        if (m->tp_peer[r] && r != m->tp_rank) cudaIpcCloseMemHandle(m->tp_peer[r]);
        m->tp_peer[r] = nullptr;
    }
    m->tp_fused = false;
}

// A wait of the peer-memory all-reduce that ran out (a rank that never arrived) -> RG_ERR_TIMEOUT; call after a sync.
static rg_status tp_check(rg_gpt* m) {
    if (!m->tp_fused) return RG_OK;
    int err = 0;
    RG_CUDA(cudaMemcpy(&err, m->d_tp_err, 4, cudaMemcpyDeviceToHost));
    if (err) return rg_fail(RG_ERR_TIMEOUT, "tensor-parallel all-reduce: a peer's contribution did not arrive in time");
    return RG_OK;
}

// Maps every rank's receive buffer into every other rank (CUDA IPC; one process per GPU on one node) for the
// token step's one-shot all-reduce.  All ranks end up in the same mode: if any of them cannot map a peer
// (no peer access between the two GPUs, IPC unavailable) or RG_B200_TP_ALLREDUCE=nccl is set, all keep NCCL.
static rg_status tp_peer_setup(rg_gpt* m) {
    const int T = m->tp_size;
    cudaStream_t s = m->ctx->stream;
    const char* mode = getenv("RG_B200_TP_ALLREDUCE");
    int ok = (T <= RG_TP_MAX && !(mode && strcmp(mode, "nccl") == 0)) ? 1 : 0;
    const size_t ar_words = 2 * (size_t)T * m->Bmax * m->D;
    const size_t mega_words = 2 * (size_t)T * 4 * m->D + (size_t)T * m->ctx->sm_count * 4 * 2;  // 4 = sequences a persistent launch takes at most
    const size_t words = ar_words + mega_words;
    RG_TRY(dalloc(m, (void**)&m->tp_recv, words * 8));
    m->tp_mega_off = ar_words;
    RG_TRY(dalloc(m, (void**)&m->d_tp_epoch, 16));
    RG_CUDA(cudaMemsetAsync(m->tp_recv, 0, words * 8, s));  // tag 0 never matches: tags start at 1
    RG_CUDA(cudaMemsetAsync(m->d_tp_epoch, 0, 16, s));
    m->d_tp_err = reinterpret_cast<int*>(m->d_tp_epoch + 2);
    // exchange the IPC handles over the communicator that exists already
    cudaIpcMemHandle_t mine;
    memset(&mine, 0, sizeof(mine));
    if (cudaIpcGetMemHandle(&mine, m->tp_recv) != cudaSuccess) ok = 0, (void)cudaGetLastError();
    char* dh = nullptr;
    RG_TRY(dalloc(m, (void**)&dh, (size_t)(T + 1) * sizeof(mine)));
    RG_CUDA(cudaMemcpyAsync(dh + (size_t)T * sizeof(mine), &mine, sizeof(mine), cudaMemcpyHostToDevice, s));
    RG_NCCL(g_nccl.AllGather(dh + (size_t)T * sizeof(mine), dh, sizeof(mine), ncclInt8, (ncclComm_t)m->nccl_comm, s));
    std::vector<cudaIpcMemHandle_t> all((size_t)T);
    RG_CUDA(cudaMemcpyAsync(all.data(), dh, (size_t)T * sizeof(mine), cudaMemcpyDeviceToHost, s));
    RG_CUDA(cudaStreamSynchronize(s));
    for (int r = 0; r < T && ok; r++) {
        if (r == m->tp_rank) {
            m->tp_peer[r] = m->tp_recv;
            continue;
        }
        void* p = nullptr;
        if (cudaIpcOpenMemHandle(&p, all[(size_t)r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            (void)cudaGetLastError();
            ok = 0;
            break;
        }
        m->tp_peer[r] = static_cast<unsigned long long*>(p);
    }
    // unanimous decision: minimum of the ranks' flags
    float* df = reinterpret_cast<float*>(dh);
    const float okf = (float)ok;
    RG_CUDA(cudaMemcpyAsync(df, &okf, 4, cudaMemcpyHostToDevice, s));
    RG_NCCL(g_nccl.AllReduce(df, df, 1, ncclFloat32, ncclMin, (ncclComm_t)m->nccl_comm, s));
    float all_ok = 0.f;
    RG_CUDA(cudaMemcpyAsync(&all_ok, df, 4, cudaMemcpyDeviceToHost, s));
    RG_CUDA(cudaStreamSynchronize(s));
    dfree(m, dh);
    m->tp_fused = all_ok > 0.5f;
    if (!m->tp_fused) tp_peer_close(m);
    return RG_OK;
}

rg_status rg_tp_stream_barrier(rg_gpt* m) {
    if (m->tp_size <= 1 || !m->nccl_comm) return RG_OK;
    float* word = reinterpret_cast<float*>(m->d_tp_epoch + 3);  // stays 0
    RG_NCCL(g_nccl.AllReduce(word, word, 1, ncclFloat32, ncclSum, (ncclComm_t)m->nccl_comm, m->ctx->stream));
    return RG_OK;
}

extern "C" rg_status rg_gpt_tp_init(rg_gpt* m, const uint8_t id_in[128]) {
    if (!m || !id_in) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    if (m->tp_size <= 1) return rg_fail(RG_ERR_INVALID_INPUT, "the model was created with tp_size <= 1");
    if (m->nccl_comm) return rg_fail(RG_ERR_INVALID_INPUT, "the communicator exists already");
    RG_TRY(load_nccl());
    rg_ctx_guard g(m->ctx);
    ncclUniqueId id;
    memcpy(id.internal, id_in, 128);
    ncclComm_t comm = nullptr;
    RG_NCCL(g_nccl.CommInitRank(&comm, m->tp_size, id, m->tp_rank));
    m->nccl_comm = comm;
    return tp_peer_setup(m);
}

extern "C" int rg_gpt_tp_fused(const rg_gpt* m) { return m && m->tp_fused ? 1 : 0; }

extern "C" rg_status rg_gpt_trace_enable(rg_gpt* m, int on) {
    if (!m) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    m->trace_on = on != 0;
    return RG_OK;
}

extern "C" rg_status rg_gpt_trace_read(rg_gpt* m, uint64_t* out, size_t cap_rows, size_t* n_rows) {
    if (!m || !out || !n_rows) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    rg_ctx_guard g(m->ctx);
    if (rg_cloop_active(m)) return rg_cloop_trace(m, (unsigned long long*)out, cap_rows, n_rows);
    return rg_mega_trace(m, (unsigned long long*)out, cap_rows, n_rows);
}

// Test hook (see rg_b200.h): makes the failure paths of the bounded device waits reachable without a device fault.
extern "C" rg_status rg_debug_hook(rg_ctx* ctx, rg_gpt* m, int what, long long value) {
    switch (what) {
        case 1: {  // raise the flag word of the tensor-core kernels' waits, as a wait that gave up would
            if (!ctx) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
            rg_ctx_guard g(ctx);
            const int one = 1;
            RG_CUDA(cudaMemcpy(ctx->d_flag + 1, &one, sizeof(int), cudaMemcpyHostToDevice));
            return RG_OK;
        }
        case 2:  // cluster token loop: head cluster 0 withholds its out-projection partial of layer `value` (-1: off)
            if (!m) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
            rg_cloop_debug(m, (int)value, 0);
            return RG_OK;
        case 3:  // cluster token loop: iteration limit of every wait
            if (!m || value < 1000) return rg_fail(RG_ERR_INVALID_INPUT, "the limit must be at least 1000");
            rg_cloop_debug(m, m->cloop ? -2 : -1, (unsigned)value);
            return RG_OK;
        case 4:  // form of the token loop: 0 the default, 1 the cluster kernel, 2 the persistent kernel, 3 separate launches
            if (!m || value < 0 || value > 3) return rg_fail(RG_ERR_INVALID_INPUT, "form 0..3");
            m->use_cloop = value == 1 && m->cloop != nullptr;
            m->use_mega = (value == 0 || value == 2) && m->mega != nullptr;
            return RG_OK;
        case 5:  // persistent kernel: iteration limit of every wait (0: the built-in limit)
            if (!m || value < 0) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
            rg_mega_debug(m, (unsigned)value, -3);
            return RG_OK;
        case 6:  // persistent kernel: CTA 0 withholds its q|k|v outputs of block `value` (-1: off)
            if (!m) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
            rg_mega_debug(m, 0xffffffffu, (int)value);
            return RG_OK;
        case 7: {  // the tensor-parallel all-reduce kernel as rank 0 of 2 on one GPU; rank 1 never contributes: the wait must run out
            if (!ctx || value < 1000) return rg_fail(RG_ERR_INVALID_INPUT, "needs a context and a limit of at least 1000 polls");
            rg_ctx_guard g(ctx);
            const size_t cnt = 768;
            float *parts = nullptr, *out = nullptr;
            unsigned long long* recv = nullptr;
            unsigned* ep = nullptr;
            RG_CUDA(cudaMalloc(&parts, cnt * 4));
            RG_CUDA(cudaMalloc(&out, cnt * 4));
            RG_CUDA(cudaMalloc(&recv, 2 * 2 * 2 * cnt * 8));  // two receive buffers of [2 parities][2 ranks][cnt]
            RG_CUDA(cudaMalloc(&ep, 16));
            RG_CUDA(cudaMemset(parts, 0, cnt * 4));
            RG_CUDA(cudaMemset(recv, 0, 2 * 2 * 2 * cnt * 8));
            RG_CUDA(cudaMemset(ep, 0, 16));
            rg_tp_ar_args a;
            memset(&a, 0, sizeof(a));
            a.parts = parts, a.nparts = 1, a.cnt = cnt, a.out = out, a.T = 2, a.rank = 0, a.slot = cnt;
            a.peer[0] = recv, a.peer[1] = recv + 2 * 2 * cnt;
            a.epoch = ep, a.site = 0, a.nsites = 1, a.err = reinterpret_cast<int*>(ep + 2), a.limit = (unsigned)value;
            rg_tp_allreduce_kernel<<<rg_cdiv((long long)cnt, 256), 256, 0, ctx->stream>>>(a);
            RG_LAUNCHED(ctx);
            int err = 0;
            cudaError_t e = cudaStreamSynchronize(ctx->stream);
            if (e == cudaSuccess) e = cudaMemcpy(&err, a.err, 4, cudaMemcpyDeviceToHost);
            cudaFree(parts), cudaFree(out), cudaFree(recv), cudaFree(ep);
            RG_CUDA(e);
            if (err) return rg_fail(RG_ERR_TIMEOUT, "tensor-parallel all-reduce: a peer's contribution did not arrive in time");
            return RG_OK;
        }
        case 8: {  // the tensor-core GEMM against a plain dot product: 40 rows, 200 columns, K = value (any multiple of 8 >= 64)
            if (!ctx || value < 64 || value > 8192 || value % 8) return rg_fail(RG_ERR_INVALID_INPUT, "K must be a multiple of 8 in 64..8192");
            rg_ctx_guard g(ctx);
            const int M = 40, N = 200, K = (int)value;
            std::vector<__nv_bfloat16> ha((size_t)M * K), hw((size_t)N * K);
            std::vector<float> fa(ha.size()), fw(hw.size());
            uint32_t st = 12345u;
            auto next = [&]() { st = st * 1664525u + 1013904223u; return ((float)(st >> 8) * (1.f / 16777216.f) - 0.5f); };
            for (size_t i = 0; i < ha.size(); i++) ha[i] = __float2bfloat16_rn(next()), fa[i] = __bfloat162float(ha[i]);
            for (size_t i = 0; i < hw.size(); i++) hw[i] = __float2bfloat16_rn(next()), fw[i] = __bfloat162float(hw[i]);
            void *da = nullptr, *dw = nullptr;
            float* dc = nullptr;
            RG_CUDA(cudaMalloc(&da, std::max<size_t>(ha.size(), (size_t)128 * K) * 2));
            RG_CUDA(cudaMalloc(&dw, hw.size() * 2));
            RG_CUDA(cudaMalloc(&dc, (size_t)M * N * 4));
            RG_CUDA(cudaMemcpy(da, ha.data(), ha.size() * 2, cudaMemcpyHostToDevice));
            RG_CUDA(cudaMemcpy(dw, hw.data(), hw.size() * 2, cudaMemcpyHostToDevice));
            std::vector<float> got((size_t)M * N), parts_sum((size_t)M * N, 0.f);
            rg_status rs = rg_gemm_bf16_tc(ctx, da, M, K, dw, N, dc, N, nullptr, nullptr, 0, -1);
            if (rs == RG_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) rs = RG_ERR_BACKEND;
            if (rs == RG_OK) cudaMemcpy(got.data(), dc, got.size() * 4, cudaMemcpyDeviceToHost);
            const float* parts = nullptr;
            int np = 0;
            if (rs == RG_OK) rs = rg_gemm_bf16_tc_parts(ctx, da, M, K, dw, N, &parts, &np);
            if (rs == RG_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) rs = RG_ERR_BACKEND;
            if (rs == RG_OK) {
                std::vector<float> one((size_t)M * N);
                for (int z = 0; z < np; z++) {
                    cudaMemcpy(one.data(), parts + (size_t)z * M * N, one.size() * 4, cudaMemcpyDeviceToHost);
                    for (size_t i = 0; i < one.size(); i++) parts_sum[i] += one[i];
                }
            }
            cudaFree(da), cudaFree(dw), cudaFree(dc);
            if (rs != RG_OK) return rg_fail(rs, "tensor-core GEMM self-check: the kernel refused K = %d", K);
            double worst = 0.0;
            for (int mi = 0; mi < M; mi++)
                for (int n = 0; n < N; n++) {
                    double ref = 0.0;
                    for (int k = 0; k < K; k++) ref += (double)fa[(size_t)mi * K + k] * (double)fw[(size_t)n * K + k];
                    worst = std::max(worst, fabs(ref - (double)got[(size_t)mi * N + n]));
                    worst = std::max(worst, fabs(ref - (double)parts_sum[(size_t)mi * N + n]));
                }
            if (!(worst <= 1e-3 * sqrt((double)K)))
                return rg_fail(RG_ERR_BACKEND, "tensor-core GEMM self-check: K = %d, worst |diff| = %g (%d partial tiles)", K, worst, np);
            return RG_OK;
        }
        default:
            return rg_fail(RG_ERR_INVALID_INPUT, "unknown hook %d", what);
    }
}
