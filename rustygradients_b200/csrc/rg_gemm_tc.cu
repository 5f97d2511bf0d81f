// Tensor-core GEMM of the prompt pass in bf16-weight mode (sm_100a only):
//
//   C[M,N] (f32) = epi( A[M,K] (bf16, row-major) . Wt[N,K]^T (bf16, K contiguous) )
//   epi(v) = act(v + bias[n]) + res[m][n]
//
// This is Linear::forward (src/nn/linear.rs:50-56) on all rows of a prompt at once,
// the one place on the path that is a dense contraction.  5th-generation tensor cores:
//  * one CTA per SM walks the output tiles (persistent); operands are staged by TMA
//    (cp.async.bulk.tensor, 128-byte swizzle) into a 6-stage shared-memory ring, 128x64 bf16
//    tiles of A and of Wt per stage, and the producer runs ahead across tile boundaries;
//  * one elected thread issues tcgen05.mma (M=128, N=128, K=16, kind::f16, fp32
//    accumulate) with shared-memory matrix descriptors; two accumulators live in TMEM
//    (128 lanes x 128 columns each), so the epilogue of a tile overlaps the MMAs of the next;
//  * tcgen05.commit signals "stage consumed" and "accumulator complete" on mbarriers;
//  * eight epilogue warps read the accumulator back with tcgen05.ld (32 lanes x 32
//    columns at a time) and apply bias / activation / residual on the way to HBM.
// No cluster multicast anywhere.  Every wait is bounded: on expiry the CTA raises an
// error word, still frees its TMEM and returns.
#include "rg_internal.cuh"

#include <cuda.h>

#include <algorithm>

#define TC_BM 128
#define TC_BN 128
#define TC_BK 64
#define TC_STAGES 6
#define TC_THREADS 320  // TMA warp, MMA warp, 8 epilogue warps
#define TC_SPIN_LIMIT (1u << 22)
#define TC_STAGE_BYTES ((TC_BM + TC_BN) * TC_BK * 2)
#define TC_SMEM_BYTES (TC_STAGES * TC_STAGE_BYTES + 1024 + 256)

struct tc_epi {
    float* C;
    long long ldc;
    const float* bias;
    const float* res;
    long long ldres;
    int act;
    int M, N, K;
    int kb_per_split;  // k-blocks per CTA along z (split-k: partial tiles go to C + z * M * ldc, no epilogue terms)
    int* err;
};

__device__ __forceinline__ uint32_t tc_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool tc_wait(uint64_t* bar, uint32_t parity, int* err) {
    uint32_t ok = 0, spins = 0;
    while (true) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(tc_smem(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
        if (++spins > TC_SPIN_LIMIT) {
            atomicExch(err, 1);
            return false;
        }
    }
}

// Shared-memory matrix descriptor: K-major tile whose rows are 128 bytes (64 bf16), 128-byte swizzle,
// 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t tc_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);  // start address
    d |= (uint64_t)0 << 16;                       // leading byte offset: unused for swizzled K-major
    d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                       // descriptor version
    d |= (uint64_t)2 << 61;                       // 128-byte swizzle
    return d;
}

__global__ void __launch_bounds__(TC_THREADS, 1)
rg_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const tc_epi e) {
    // Inside a chain of dependent launches this kernel may start while its predecessor still runs.  Everything that does
    // not depend on the predecessor happens before the wait: barrier set-up, the TMEM allocation and the copies of the
    // WEIGHT tiles of the first TC_STAGES k-blocks (weights are never written by a kernel of the chain).  The activation
    // tiles, the residual reads and every store come after it.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ unsigned char tc_smem_raw[];
    // 1024-byte aligned tiles (the swizzle pattern is a function of the address)
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + TC_STAGES * TC_STAGE_BYTES);
    uint64_t* empty = full + TC_STAGES;
    uint64_t* acc_full = empty + TC_STAGES;  // [2]: accumulator b holds a finished tile
    uint64_t* acc_empty = acc_full + 2;      // [2]: the epilogue warps have read accumulator b
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = (e.N + TC_BN - 1) / TC_BN, tiles_m = (e.M + TC_BM - 1) / TC_BM;
    const int ntiles = tiles_n * tiles_m;
    const int kb_begin = blockIdx.z * e.kb_per_split;
    const int nkb = min(e.kb_per_split, (e.K + TC_BK - 1) / TC_BK - kb_begin);  // a ragged last k-block is zero-filled by TMA

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&full[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&empty[s])) : "memory");
        }
        for (int b = 0; b < 2; b++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&acc_full[b])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 8;" ::"r"(tc_smem(&acc_empty[b])) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // the MMA warp owns the tensor memory: two accumulators of 128 fp32 columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;" ::"r"(tc_smem(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    // weight tiles of the first k-blocks (the `empty` barriers of a fresh ring pass without a wait)
    uint32_t pre = 0;
    if (warp == 0 && lane == 0) {
        for (int tile = blockIdx.x; tile < ntiles && pre < TC_STAGES; tile += gridDim.x) {
            const int n0 = (tile % tiles_n) * TC_BN;
            for (int kb = 0; kb < nkb && pre < TC_STAGES; kb++, pre++) {
                unsigned char* b_dst = tiles + pre * TC_STAGE_BYTES + TC_BM * TC_BK * 2;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tc_smem(&full[pre])),
                             "r"((uint32_t)TC_STAGE_BYTES)
                             : "memory");
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                        tc_smem(b_dst)),
                    "l"(&tmB), "r"((kb_begin + kb) * TC_BK), "r"(n0), "r"(tc_smem(&full[pre]))
                    : "memory");
            }
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // Persistent tile loop: CTA x takes tiles x, x + gridDim.x, ...; n varies fastest, so the CTAs running at the same
    // time share rows of A in L2.  The three roles walk the same sequence, each with its own counters.
    if (warp == 0) {
        // ===== TMA producer: runs ahead across tile boundaries, up to TC_STAGES k-blocks =====
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                const int m0 = (tile / tiles_n) * TC_BM, n0 = (tile % tiles_n) * TC_BN;
                for (int kb = 0; kb < nkb; kb++, it++) {
                    const int s = it % TC_STAGES;
                    const uint32_t par = (it / TC_STAGES) & 1;
                    unsigned char* a_dst = tiles + s * TC_STAGE_BYTES;
                    unsigned char* b_dst = a_dst + TC_BM * TC_BK * 2;
                    if (it >= pre) {
                        ok = tc_wait(&empty[s], par ^ 1u, e.err);
                        if (!ok) break;
                        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tc_smem(&full[s])),
                                     "r"((uint32_t)TC_STAGE_BYTES)
                                     : "memory");
                    }
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                            tc_smem(a_dst)),
                        "l"(&tmA), "r"((kb_begin + kb) * TC_BK), "r"(m0), "r"(tc_smem(&full[s]))
                        : "memory");
                    if (it >= pre) asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                            tc_smem(b_dst)),
                        "l"(&tmB), "r"((kb_begin + kb) * TC_BK), "r"(n0), "r"(tc_smem(&full[s]))
                        : "memory");
                }
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer: accumulator (tile count & 1), so the epilogue of one tile overlaps the MMAs of the next =====
        if (lane == 0) {
            // instruction descriptor: D = f32, A = B = bf16, both K-major, N = 128, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
            uint32_t it = 0, tl = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, tl++) {
                const uint32_t buf = tl & 1u, use = tl >> 1;
                ok = tc_wait(&acc_empty[buf], (use & 1u) ^ 1u, e.err);  // passes at once for the first use of a buffer
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + buf * TC_BN;
                for (int kb = 0; kb < nkb; kb++, it++) {
                    const int s = it % TC_STAGES;
                    const uint32_t par = (it / TC_STAGES) & 1;
                    ok = tc_wait(&full[s], par, e.err);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = tc_smem(tiles + s * TC_STAGE_BYTES);
                    const uint32_t b_addr = a_addr + TC_BM * TC_BK * 2;
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; k++) {
                        const uint64_t da = tc_desc(a_addr + k * 32);  // 16 bf16 = 32 bytes further along K inside the swizzle span
                        const uint64_t db = tc_desc(b_addr + k * 32);
                        const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                        asm volatile(
                            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                            "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
                            : "memory");
                    }
                    // the stage is free again once these MMAs have read it
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_smem(&empty[s]))
                                 : "memory");
                }
                if (ok)
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                     tc_smem(&acc_full[buf]))
                                 : "memory");
            }
        }
    } else {
        // ===== epilogue warps 2..9: TMEM lane quarter = warp % 4; warps 2..5 take the left half of the columns,
        // warps 6..9 the right half (the epilogue, not the MMA, bounds a tile when K is short: with 4 warps a 128x128
        // tile of the out-projection took ~20 us to drain) =====
        const int q = warp & 3;
        const int c_begin = warp < 6 ? 0 : TC_BN / 64, c_end = c_begin + TC_BN / 64;
        uint32_t tl = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, tl++) {
            const int m0 = (tile / tiles_n) * TC_BM, n0 = (tile % tiles_n) * TC_BN;
            const uint32_t buf = tl & 1u, use = tl >> 1;
            ok = tc_wait(&acc_full[buf], use & 1u, e.err);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int m = m0 + q * 32 + lane;
#pragma unroll 1
            for (int c = c_begin; c < c_end; c++) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + buf * TC_BN + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                      "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
                      "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
                      "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (c == c_end - 1) {
                    // every column of this accumulator has been read: hand it back before the last stores
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc_smem(&acc_empty[buf])) : "memory");
                }
                float* Cz = e.C + (size_t)blockIdx.z * e.M * e.ldc;
                if (m < e.M) {
                    const int nc = n0 + c * 32;
                    float* crow = Cz + (long long)m * e.ldc + nc;
                    const float* rrow = e.res ? e.res + (long long)m * e.ldres + nc : nullptr;
                    // a thread holds 32 consecutive columns of its row: 128 contiguous bytes, moved as 8 x 16 bytes when
                    // the row segment, the bias and the residual are 16-byte aligned and entirely inside the matrix
                    const bool vec = nc + 32 <= e.N && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0) &&
                                     (!e.bias || (reinterpret_cast<uintptr_t>(e.bias + nc) & 15) == 0) &&
                                     (!rrow || (reinterpret_cast<uintptr_t>(rrow) & 15) == 0);
                    if (vec) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                                   __uint_as_float(r[j + 3]));
                            if (e.bias) {
                                const float4 b = __ldg(reinterpret_cast<const float4*>(e.bias + nc + j));
                                v.x += b.x, v.y += b.y, v.z += b.z, v.w += b.w;
                            }
                            if (e.act >= 0) {
                                v.x = rg_apply_act(v.x, e.act), v.y = rg_apply_act(v.y, e.act);
                                v.z = rg_apply_act(v.z, e.act), v.w = rg_apply_act(v.w, e.act);
                            }
                            if (rrow) {
                                const float4 q4 = *reinterpret_cast<const float4*>(rrow + j);
                                v.x += q4.x, v.y += q4.y, v.z += q4.z, v.w += q4.w;
                            }
                            *reinterpret_cast<float4*>(crow + j) = v;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const int n = nc + j;
                            if (n < e.N) {
                                float v = __uint_as_float(r[j]);
                                if (e.bias) v += e.bias[n];
                                if (e.act >= 0) v = rg_apply_act(v, e.act);
                                if (rrow) v += rrow[j];
                                crow[j] = v;
                            }
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" ::"r"(tmem_base) : "memory");
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*tc_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static tc_encode_fn g_encode = nullptr;

static rg_status tc_make_map(CUtensorMap* map, const void* base, int rows, int K) {
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {TC_BK, TC_BM};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return rg_fail(RG_ERR_BACKEND, "cuTensorMapEncodeTiled failed with %d", (int)r);
    return RG_OK;
}

// C[m][n] = epi(sum over the k-splits of ws[z][m][n]), fixed order
static __global__ void tc_splitk_reduce_kernel(const float* __restrict__ ws, int splits, int M, int N, float* __restrict__ C,
                                               long long ldc, const float* __restrict__ bias, const float* __restrict__ res,
                                               long long ldres, int act) {
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


// Returns RG_ERR_UNSUPPORTED (without touching C) when the shape is outside the kernel's limits.
// With few rows (one M tile) the k range is split over several CTAs so that the weights stream through
// many SMs at once; the partial tiles are summed, in a fixed order, by a second kernel that also applies
// the epilogue.  The split-k workspace is allocated on first use per context (not inside a stream capture:
// the prompt pass, which always runs first, goes through here too).
static rg_status tc_gemm(rg_ctx* ctx, const void* A16, int M, int K, const void* Wt16, int N, float* C, long long ldc,
                         const float* bias, const float* res, long long ldres, int act, const float** raw_parts, int* raw_nparts) {
    const bool raw = raw_parts != nullptr;
    // rows of both operands must start on 16-byte boundaries (K % 8); a last k-block that reaches past K is filled with
    // zeros by the tensor maps (out-of-bounds fill), on both operands
    if (K % 8 != 0 || K < TC_BK || M <= 0 || N <= 0) return RG_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(A16) & 15) || (reinterpret_cast<uintptr_t>(Wt16) & 15)) return RG_ERR_UNSUPPORTED;
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t er = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (er != cudaSuccess || !fn || qres != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return RG_ERR_UNSUPPORTED;
        }
        g_encode = reinterpret_cast<tc_encode_fn>(fn);
        cudaError_t ea = cudaFuncSetAttribute(rg_gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES);
        if (ea != cudaSuccess) return rg_fail(RG_ERR_BACKEND, "rg_gemm_tc_kernel: %s", cudaGetErrorString(ea));
    }
    {   // split-k workspace of this context: 64 MiB on the first call (the prompt pass, never inside a capture)
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        cudaStreamIsCapturing(ctx->stream, &cs);
        if (!ctx->tc_ws && cs == cudaStreamCaptureStatusNone) {
            if (cudaMalloc(&ctx->tc_ws, (size_t)64 << 20) == cudaSuccess) ctx->tc_ws_bytes = (size_t)64 << 20;
            else cudaGetLastError();
        }
    }
    CUtensorMap tmA, tmB;
    RG_TRY(tc_make_map(&tmA, A16, M, K));
    RG_TRY(tc_make_map(&tmB, Wt16, N, K));
    const int nkb = rg_cdiv(K, TC_BK), ntiles = rg_cdiv(N, TC_BN) * rg_cdiv(M, TC_BM);
    int splits = 1;
    if (M <= TC_BM && ntiles < ctx->sm_count / 2) splits = std::max(1, std::min(nkb / 3, ctx->sm_count / ntiles));  // at least 3 k-blocks per CTA (A/B: 2 and 4 are slower)
    const int kb_per = rg_cdiv(nkb, splits);
    splits = rg_cdiv(nkb, kb_per);
    tc_epi e;
    e.C = C, e.ldc = ldc, e.bias = bias, e.res = res, e.ldres = ldres, e.act = act, e.M = M, e.N = N, e.K = K;
    e.kb_per_split = kb_per;
    e.err = ctx->d_flag + 1;
    if (splits > 1) {
        const size_t need = (size_t)splits * M * N * 4;
        if (ctx->tc_ws_bytes < need) {
            cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
            cudaStreamIsCapturing(ctx->stream, &cs);
            if (cs != cudaStreamCaptureStatusNone) {
                splits = 1, e.kb_per_split = nkb;  // cannot allocate now: run unsplit
            } else {
                const size_t want = std::max(need, (size_t)64 << 20);
                if (ctx->tc_ws) cudaFree(ctx->tc_ws);
                ctx->tc_ws = nullptr, ctx->tc_ws_bytes = 0;
                if (cudaMalloc(&ctx->tc_ws, want) == cudaSuccess) ctx->tc_ws_bytes = want;
                else cudaGetLastError(), splits = 1, e.kb_per_split = nkb;
            }
        }
    }
    if (raw) {
        // the caller sums the partial tiles itself (fused with what follows the projection)
        if (ctx->tc_ws_bytes < (size_t)splits * M * N * 4) return RG_ERR_UNSUPPORTED;
        e.C = ctx->tc_ws, e.ldc = N, e.bias = nullptr, e.res = nullptr, e.act = -1;
        *raw_parts = e.C, *raw_nparts = splits;
    } else if (splits > 1) {
        e.C = ctx->tc_ws, e.ldc = N, e.bias = nullptr, e.res = nullptr, e.act = -1;
    }
    dim3 grid(std::min(ntiles, ctx->sm_count), 1, splits);  // persistent: one CTA per SM walks the tiles
    RG_CUDA(rg_launch(ctx->pdl, rg_gemm_tc_kernel, grid, dim3(TC_THREADS), TC_SMEM_BYTES, ctx->stream, tmA, tmB, e));
    RG_CUDA(cudaGetLastError());
    RG_LAUNCHED(ctx);
    if (splits > 1 && !raw) {
        tc_splitk_reduce_kernel<<<rg_cdiv((long long)M * N, 256), 256, 0, ctx->stream>>>(ctx->tc_ws, splits, M, N, C, ldc,
                                                                                         bias, res, ldres, act);
        RG_CUDA(cudaGetLastError());
        RG_LAUNCHED(ctx);
    }
    return RG_OK;
}

rg_status rg_gemm_bf16_tc(rg_ctx* ctx, const void* A16, int M, int K, const void* Wt16, int N, float* C, long long ldc,
                          const float* bias, const float* res, long long ldres, int act) {
    return tc_gemm(ctx, A16, M, K, Wt16, N, C, ldc, bias, res, ldres, act, nullptr, nullptr);
}

// Raw form for few rows: the accumulators of every k-split go to the per-device workspace as [nparts][M][N] (no bias,
// no activation); the caller's next kernel adds them up in order.  The workspace is reused by the next call.
rg_status rg_gemm_bf16_tc_parts(rg_ctx* ctx, const void* A16, int M, int K, const void* Wt16, int N, const float** parts,
                                int* nparts) {
    return tc_gemm(ctx, A16, M, K, Wt16, N, nullptr, N, nullptr, nullptr, 0, -1, parts, nparts);
}
