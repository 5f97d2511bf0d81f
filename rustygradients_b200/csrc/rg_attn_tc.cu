// Attention over all rows of a prompt on the tensor cores (bf16 mode, head_dim 64; sm_100a only):
// MultiHeadAttention::forward (src/nn/attention.rs:78-94) for T query rows per head at once,
//
//   S = Q K^T, scale after the product, optional causal mask, softmax over the keys
//   (max-subtracted, src/ops/elementwise.rs:144-157), O = P V
//
// as a streaming-softmax kernel: a CTA owns 128 query rows of one (sequence, head) and walks
// the keys 128 at a time.
//  * TMA (cp.async.bulk.tensor, 128-byte swizzle) stages the Q tile once and, per key tile, the
//    K rows straight out of the KV cache and the matching columns of V^T;
//  * one elected thread issues tcgen05.mma: S = Q K^T (M 128, N 128, K 64) into 128 TMEM columns,
//    later O_j = P V (M 128, N 64, K 128) into 64 more;
//  * four warps own one query row per thread: they read S with tcgen05.ld (two passes: row
//    maximum, then exponentials), keep the running maximum and sum, write P as bf16 into
//    shared memory in the swizzled K-major layout the MMA expects, and add O_j, rescaled, to
//    the fp32 output row they hold in registers.
// P and V enter the second product in bf16 with fp32 accumulation, which stays inside the
// bf16-mode tolerance.  No cluster multicast.  Every wait is bounded: on expiry the CTA raises
// an error word, still frees its TMEM and returns.
#include "rg_internal.cuh"

#include <cuda.h>

#define AT_BM 128   // query rows per CTA
#define AT_BN 128   // keys per tile
#define AT_HD 64
#define AT_THREADS 192
#define AT_SPIN_LIMIT (1u << 22)
#define AT_Q_BYTES (AT_BM * AT_HD * 2)        // 16 KB
#define AT_K_BYTES (AT_BN * AT_HD * 2)        // 16 KB
#define AT_V_BYTES (AT_HD * AT_BN * 2)        // 16 KB: two atoms [64 d][64 keys]
#define AT_P_BYTES (AT_BM * AT_BN * 2)        // 32 KB: two atoms [128 q][64 keys]
#define AT_SMEM_BYTES (AT_Q_BYTES + AT_K_BYTES + AT_V_BYTES + AT_P_BYTES + 1024 + 256)

struct at_args {
    float* out;      // [B*T][D]
    int T, H, D, C;  // rows per sequence, heads, model width (row stride of out), cache rows per head
    int causal;
    float scale_log2e;  // 1/sqrt(hd) * log2(e)
    int* err;
};

__device__ __forceinline__ uint32_t at_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool at_wait(uint64_t* bar, uint32_t parity, int* err) {
    uint32_t ok = 0, spins = 0;
    while (true) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(at_smem(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
        if (++spins > AT_SPIN_LIMIT) {
            atomicExch(err, 1);
            return false;
        }
    }
}

// K-major tile with 128-byte rows, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t at_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

#define AT_TMEM_LD32(r, taddr)                                                                                              \
    asm volatile(                                                                                                           \
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                                           \
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                                           \
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"                           \
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),       \
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),            \
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),           \
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])                         \
        : "r"(taddr)                                                                                                        \
        : "memory");                                                                                                        \
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory")

// qkv f32 [B*T][3D] -> Q as bf16 [B*H*T][64] and V^T as bf16 [B*H*64][Tp] (columns T..Tp-1 zero).
// grid (Tp/64, H, B), 256 threads: a 64 x 64 tile through shared memory.
static __global__ void __launch_bounds__(256) rg_attn_prep_kernel(const float* __restrict__ qkv, __nv_bfloat16* __restrict__ Qb,
                                                                  __nv_bfloat16* __restrict__ Vt, int T, int Tp, int H, int D) {
    __shared__ float tv[64][65];
    const int t0 = blockIdx.x * 64, h = blockIdx.y, b = blockIdx.z;
    const size_t bh = (size_t)b * H + h;
    for (int i = threadIdx.x; i < 64 * 64; i += 256) {
        const int tt = i >> 6, d = i & 63, t = t0 + tt;
        float q = 0.f, v = 0.f;
        if (t < T) {
            const float* row = qkv + ((size_t)b * T + t) * 3 * D;
            q = row[h * 64 + d];
            v = row[2 * D + h * 64 + d];
            Qb[(bh * T + t) * 64 + d] = __float2bfloat16_rn(q);
        }
        tv[tt][d] = v;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 64 * 64; i += 256) {
        const int d = i >> 6, tt = i & 63;
        Vt[(bh * 64 + d) * Tp + t0 + tt] = __float2bfloat16_rn(tv[tt][d]);
    }
}

__global__ void __launch_bounds__(AT_THREADS, 2)
rg_attn_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const at_args a) {
    extern __shared__ unsigned char at_smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(at_smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = base;
    unsigned char* sK = sQ + AT_Q_BYTES;
    unsigned char* sV = sK + AT_K_BYTES;
    unsigned char* sP = sV + AT_V_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sP + AT_P_BYTES);
    uint64_t *q_full = bars, *kv_full = bars + 1, *kv_empty = bars + 2, *s_full = bars + 3, *p_full = bars + 4, *o_full = bars + 5;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int bh = b * a.H + h;
    const int q0 = qt * AT_BM;
    const int ktiles_all = (a.T + AT_BN - 1) / AT_BN;
    const int nk = a.causal ? min(qt + 1, ktiles_all) : ktiles_all;  // key tiles this CTA visits

    if (threadIdx.x == 0) {
        for (int i = 0; i < 6; i++) {
            const uint32_t count = (i == 4) ? 4u : 1u;  // p_full: one arrival per softmax warp
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(at_smem(&bars[i])), "r"(count) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // 128 columns for S, 64 for the partial output: 256 is the next power of two
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;" ::"r"(at_smem(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + AT_BN;

    if (warp == 0) {
        // ===== TMA producer =====
        if (lane == 0) {
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(at_smem(q_full)), "r"((uint32_t)AT_Q_BYTES)
                         : "memory");
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                             at_smem(sQ)),
                         "l"(&tmQ), "r"(0), "r"(bh * a.T + q0), "r"(at_smem(q_full))
                         : "memory");
            for (int j = 0; j < nk; j++) {
                if (!at_wait(kv_empty, (uint32_t)(j & 1) ^ 1u, a.err)) break;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(at_smem(kv_full)),
                             "r"((uint32_t)(AT_K_BYTES + AT_V_BYTES))
                             : "memory");
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                        at_smem(sK)),
                    "l"(&tmK), "r"(0), "r"(bh * a.C + j * AT_BN), "r"(at_smem(kv_full))
                    : "memory");
#pragma unroll
                for (int at = 0; at < 2; at++)
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                            at_smem(sV + at * (AT_V_BYTES / 2))),
                        "l"(&tmV), "r"(j * AT_BN + at * 64), "r"(bh * AT_HD), "r"(at_smem(kv_full))
                        : "memory");
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer =====
        if (lane == 0) {
            const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(AT_BN >> 3) << 17) | ((uint32_t)(AT_BM >> 4) << 24);
            const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(AT_HD >> 3) << 17) | ((uint32_t)(AT_BM >> 4) << 24);
            bool ok = at_wait(q_full, 0, a.err);
            for (int j = 0; j < nk && ok; j++) {
                const uint32_t par = (uint32_t)(j & 1);
                ok = at_wait(kv_full, par, a.err);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int k = 0; k < AT_HD / 16; k++) {  // S = Q K^T
                    const uint64_t da = at_desc(at_smem(sQ) + k * 32), db = at_desc(at_smem(sK) + k * 32);
                    const uint32_t acc = k > 0 ? 1u : 0u;
                    asm volatile(
                        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_s),
                        "l"(da), "l"(db), "r"(idesc_s), "r"(acc)
                        : "memory");
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(at_smem(s_full))
                             : "memory");
                ok = at_wait(p_full, par, a.err);  // P of this tile is in shared memory (and S has been read)
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int at = 0; at < 2; at++)
#pragma unroll
                    for (int k = 0; k < 4; k++) {  // O_j = P V: keys at*64 + k*16 ...
                        const uint64_t da = at_desc(at_smem(sP + at * (AT_P_BYTES / 2)) + k * 32);
                        const uint64_t db = at_desc(at_smem(sV + at * (AT_V_BYTES / 2)) + k * 32);
                        const uint32_t acc = (at > 0 || k > 0) ? 1u : 0u;
                        asm volatile(
                            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_o),
                            "l"(da), "l"(db), "r"(idesc_o), "r"(acc)
                            : "memory");
                    }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(at_smem(o_full))
                             : "memory");
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(at_smem(kv_empty))
                             : "memory");
            }
        }
    } else {
        // ===== softmax / output warps 2..5: thread = query row (TMEM lane quarter = warp % 4) =====
        const int q = warp & 3;
        const int r = q * 32 + lane;   // row inside the tile
        const int qi = q0 + r;         // row inside the sequence
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        float m_run = -INFINITY, l_run = 0.f;
        float o[AT_HD];
#pragma unroll
        for (int d = 0; d < AT_HD; d++) o[d] = 0.f;
        bool ok = true;
        for (int j = 0; j < nk && ok; j++) {
            const uint32_t par = (uint32_t)(j & 1);
            ok = at_wait(s_full, par, a.err);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int kbase = j * AT_BN;
            // pass 1: row maximum over the visible keys of this tile
            float mx = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < AT_BN / 32; c++) {
                uint32_t s[32];
                AT_TMEM_LD32(s, tmem_s + lane_addr + (uint32_t)(c * 32));
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    const int kj = kbase + c * 32 + i;
                    const bool vis = kj < a.T && (!a.causal || kj <= qi);
                    if (vis) mx = fmaxf(mx, __uint_as_float(s[i]));
                }
            }
            const float m_new = fmaxf(m_run, mx * a.scale_log2e);  // in log2 units
            const float corr = (m_new == -INFINITY) ? 1.f : exp2f(m_run - m_new);
            // pass 2: p = 2^(s * scale * log2e - m_new), written as bf16 into the swizzled K-major P tile
            float lsum = 0.f;
#pragma unroll 1
            for (int c = 0; c < AT_BN / 32; c++) {
                uint32_t s[32];
                AT_TMEM_LD32(s, tmem_s + lane_addr + (uint32_t)(c * 32));
                unsigned char* atom = sP + (c >> 1) * (AT_P_BYTES / 2) + r * 128;
#pragma unroll
                for (int g = 0; g < 4; g++) {  // 8 keys = one 16-byte chunk
                    uint32_t packed[4];
#pragma unroll
                    for (int e2 = 0; e2 < 4; e2++) {
                        float p2[2];
#pragma unroll
                        for (int u = 0; u < 2; u++) {
                            const int i = g * 8 + e2 * 2 + u;
                            const int kj = kbase + c * 32 + i;
                            const bool vis = kj < a.T && (!a.causal || kj <= qi);
                            p2[u] = vis ? exp2f(fmaf(__uint_as_float(s[i]), a.scale_log2e, -m_new)) : 0.f;
                        }
                        const __nv_bfloat162 pk = __floats2bfloat162_rn(p2[0], p2[1]);
                        // the second product sees the rounded values: sum what it will use
                        lsum += __bfloat162float(pk.x) + __bfloat162float(pk.y);
                        packed[e2] = *reinterpret_cast<const uint32_t*>(&pk);
                    }
                    const int chunk = (c & 1) * 4 + g;  // 16-byte chunk of the 128-byte row
                    *reinterpret_cast<uint4*>(atom + ((chunk ^ (r & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                }
            }
            l_run = l_run * corr + lsum;
            m_run = m_new;
            // P is complete: make the generic-proxy writes visible to the tensor core, then signal
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(at_smem(p_full)) : "memory");
            ok = at_wait(o_full, par, a.err);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int c = 0; c < AT_HD / 32; c++) {
                uint32_t t[32];
                AT_TMEM_LD32(t, tmem_o + lane_addr + (uint32_t)(c * 32));
#pragma unroll
                for (int i = 0; i < 32; i++) o[c * 32 + i] = fmaf(o[c * 32 + i], corr, __uint_as_float(t[i]));
            }
        }
        if (ok && qi < a.T) {
            const float inv = 1.f / l_run;
            float* dst = a.out + ((size_t)b * a.T + qi) * a.D + h * AT_HD;
#pragma unroll
            for (int d = 0; d < AT_HD; d += 4)
                *reinterpret_cast<float4*>(dst + d) = make_float4(o[d] * inv, o[d + 1] * inv, o[d + 2] * inv, o[d + 3] * inv);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" ::"r"(tmem_base) : "memory");
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*at_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static at_encode_fn g_at_encode = nullptr;

static rg_status at_make_map(CUtensorMap* map, const void* base, uint64_t inner, uint64_t rows, uint32_t box_rows) {
    const cuuint64_t dims[2] = {inner, rows};
    const cuuint64_t strides[1] = {inner * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = g_at_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return rg_fail(RG_ERR_BACKEND, "cuTensorMapEncodeTiled failed with %d", (int)r);
    return RG_OK;
}

// qkv: f32 rows [B*T][3D] of this block; kcache: this block's K cache [B][H][C][64] (bf16, rows 0..T-1 already written);
// q16 / vt16: scratch of B*H*T*64 and B*H*64*Tp bf16 (Tp = T rounded up to 64); out: f32 [B*T][D].
// RG_ERR_UNSUPPORTED when the shape is outside the kernel's limits (the caller then uses the CUDA-core kernel).
rg_status rg_attn_bf16_tc(rg_ctx* ctx, const float* qkv, const void* kcache, int B, int H, int T, int C, int D, int hd, int causal,
                          void* q16, void* vt16, float* out) {
    if (hd != AT_HD || D != H * AT_HD || T <= 0 || (D & 3)) return RG_ERR_UNSUPPORTED;
    if (!g_at_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t er = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (er != cudaSuccess || !fn || qres != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return RG_ERR_UNSUPPORTED;
        }
        g_at_encode = reinterpret_cast<at_encode_fn>(fn);
        cudaError_t ea = cudaFuncSetAttribute(rg_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM_BYTES);
        if (ea != cudaSuccess) return rg_fail(RG_ERR_BACKEND, "rg_attn_tc_kernel: %s", cudaGetErrorString(ea));
    }
    const int Tp = (T + 63) / 64 * 64;
    rg_attn_prep_kernel<<<dim3(Tp / 64, H, B), 256, 0, ctx->stream>>>(qkv, (__nv_bfloat16*)q16, (__nv_bfloat16*)vt16, T, Tp, H, D);
    RG_LAUNCHED(ctx);
    CUtensorMap tmQ, tmK, tmV;
    RG_TRY(at_make_map(&tmQ, q16, AT_HD, (uint64_t)B * H * T, AT_BM));
    RG_TRY(at_make_map(&tmK, kcache, AT_HD, (uint64_t)B * H * C, AT_BN));
    RG_TRY(at_make_map(&tmV, vt16, (uint64_t)Tp, (uint64_t)B * H * AT_HD, AT_HD));
    at_args a;
    a.out = out, a.T = T, a.H = H, a.D = D, a.C = C, a.causal = causal;
    a.scale_log2e = (1.f / sqrtf((float)hd)) * 1.4426950408889634f;
    a.err = ctx->d_flag + 1;
    rg_attn_tc_kernel<<<dim3((T + AT_BM - 1) / AT_BM, H, B), AT_THREADS, AT_SMEM_BYTES, ctx->stream>>>(tmQ, tmK, tmV, a);
    RG_CUDA(cudaGetLastError());
    RG_LAUNCHED(ctx);
    return RG_OK;
}
