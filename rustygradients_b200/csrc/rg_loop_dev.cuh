// Device helpers shared by the persistent token-loop kernels: mbarrier and bulk-copy wrappers, tagged 64-bit
// exchange words, the shared-memory ring as the consumer warps see it, polling fetches of tagged vectors and the
// halving warp reduction.
#pragma once
#include "rg_gpt.h"

#define MG_THREADS 256
#define MG_SLOT_BYTES 32768
#define MG_ATTN_PASSES (MG_SLOT_BYTES / 4096)  // rows of a full K/V chunk that one lane group of one warp handles
#define MG_SPIN_LIMIT (1u << 21)
#define MG_BMAX 4

typedef unsigned long long mg_word;  // (tag << 32) | payload bits

// ---------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t mg_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mg_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mg_smem(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mg_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mg_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mg_mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(mg_smem(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void mg_bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(mg_smem(dst)),
                 "l"(src), "r"(bytes), "r"(mg_smem(bar))
                 : "memory");
}
__device__ __forceinline__ void mg_fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ mg_word mg_ld_word(const mg_word* p) {
    mg_word v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void mg_st_word(mg_word* p, uint32_t tag, uint32_t payload) {
    const mg_word v = ((mg_word)tag << 32) | payload;
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long mg_globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ int mg_ld_flag(const int* p) {
    int v;
    asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

template <typename T>
__device__ __forceinline__ T mg_from_float(float v);
template <>
__device__ __forceinline__ float mg_from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 mg_from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T>
struct mg_vec;
template <>
struct mg_vec<float> {
    static constexpr int N = 4;
    __device__ __forceinline__ static void unpack(const uint4& v, float (&w)[4]) {
        w[0] = __uint_as_float(v.x), w[1] = __uint_as_float(v.y), w[2] = __uint_as_float(v.z), w[3] = __uint_as_float(v.w);
    }
};
template <>
struct mg_vec<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ __forceinline__ static void unpack(const uint4& v, float (&w)[8]) {
        const unsigned int u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            w[2 * i] = __uint_as_float(u[i] << 16);
            w[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
        }
    }
};

// ---------------------------------------------------------------------------
// CTA layout: warps 0-7 (256 threads) are consumers; warp 8 is the producer (one
// elected lane issues the bulk copies).  Consumers synchronise among themselves
// on named barrier 1, so the producer never has to take part.
// ---------------------------------------------------------------------------
#define MG_TOTAL_THREADS (MG_THREADS + 32)

__device__ __forceinline__ void mg_csync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ bool mg_csync_or(bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.or.pred q, 1, 256, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(r)
        : "r"((uint32_t)(pred ? 1 : 0))
        : "memory");
    return r != 0;
}
__device__ __forceinline__ void mg_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mg_smem(bar)) : "memory");
}

// Per-thread control state.  `dead` becomes CTA-wide at the next op boundary.
struct mg_ctl {
    int* abort_flag;
    unsigned poll_sleep;  // ns to pause between two polls of words that were not valid yet (0 = none)
    unsigned limit;       // iterations after which a wait gives up (MG_SPIN_LIMIT unless a test lowers it)
    bool dead;
};
__device__ __forceinline__ void mg_give_up(mg_ctl& c) {
    atomicExch(c.abort_flag, 1);
    c.dead = true;
}

__device__ __forceinline__ int mg_attn_rows_per_chunk(int hd, int kvsize) { return MG_SLOT_BYTES / (hd * kvsize); }

// Consumer view of the ring.
struct mg_cons {
    unsigned char* slots;
    uint64_t *full, *empty;
    int nslot, slot;
    uint32_t parity;
};
__device__ __forceinline__ const unsigned char* mg_ring_wait(mg_cons& r, mg_ctl& ctl) {
    uint32_t spins = 0;
    while (!ctl.dead && !mg_mbar_try_wait(&r.full[r.slot], r.parity)) {
        if (++spins > ctl.limit || ((spins & 255u) == 0 && mg_ld_flag(ctl.abort_flag))) mg_give_up(ctl);
        if (ctl.poll_sleep) __nanosleep(ctl.poll_sleep);
    }
    // Telling the compiler that the pointer is a shared-memory pointer makes it emit ld.shared for what is read through
    // it.  A load through a generic pointer takes the global-memory path of the SM and queues behind the polling loads
    // (measured on the same loop: 2757 cycles generic, 3782 with other warps polling, 1437 with ld.shared).
    const unsigned char* s = r.slots + (size_t)r.slot * MG_SLOT_BYTES;
    __builtin_assume(__isShared(s));
    return s;
}
// Each consumer warp reports that it is done with the slot; the 8th report frees it.
__device__ __forceinline__ void mg_ring_release(mg_cons& r) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mg_mbar_arrive(&r.empty[r.slot]);
    if (++r.slot == r.nslot) r.slot = 0, r.parity ^= 1u;
}

template <bool SYS = false>
__device__ __forceinline__ void mg_ld_word2(const mg_word* p, mg_word& a, mg_word& b) {
    if constexpr (SYS)  // words that another GPU stores over NVLink
        asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
    else
        asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}

// Fetch one stage input vector of n values (n even) into dst (shared memory) from
// tagged words (16-byte aligned), polling until every word carries `tag`.  A thread owns
// the word pairs tid, tid + 256, ...; one 16-byte load brings a pair (each 8-byte half
// carries its own tag, so the halves validate independently), up to U loads are issued
// back to back before any is checked, and only the pairs that were not valid yet are
// read again, after a short pause that keeps the polling traffic of 148 CTAs off the L2.
// RT = false compiles the wait limit in and leaves the optional pause out (the noinline routines would otherwise read
// both from the caller's stack inside the polling loop: 3 % of the token time on the GPT-2-small shape).
template <int U = 8, bool RT = true, bool SYS = false>
__device__ __noinline__ void mg_fetch(const mg_word* src, int n, uint32_t tag, float* dst, mg_ctl& ctl) {
    __builtin_assume(__isShared(dst));
    const int npair = n >> 1;
    for (int base = threadIdx.x; base < npair; base += MG_THREADS * U) {
        uint32_t pending = 0;
#pragma unroll
        for (int u = 0; u < U; u++)
            if (base + u * MG_THREADS < npair) pending |= 1u << u;
        uint32_t spins = 0;
        while (pending != 0) {
            mg_word w[U][2];
#pragma unroll
            for (int u = 0; u < U; u++)
                if (pending & (1u << u)) mg_ld_word2<SYS>(src + 2 * (base + u * MG_THREADS), w[u][0], w[u][1]);
            uint32_t done = 0;
#pragma unroll
            for (int u = 0; u < U; u++) {
                if ((pending & (1u << u)) && (uint32_t)(w[u][0] >> 32) == tag && (uint32_t)(w[u][1] >> 32) == tag) {
                    const int i = 2 * (base + u * MG_THREADS);
                    *reinterpret_cast<float2*>(dst + i) =
                        make_float2(__uint_as_float((uint32_t)w[u][0]), __uint_as_float((uint32_t)w[u][1]));
                    done |= 1u << u;
                }
            }
            pending &= ~done;
            if (pending != 0) {
                if (++spins > (RT ? ctl.limit : MG_SPIN_LIMIT) || ((spins & 255u) == 0 && mg_ld_flag(ctl.abort_flag))) {
                    mg_give_up(ctl);
                    break;
                }
                if (RT && ctl.poll_sleep) __nanosleep(ctl.poll_sleep);
            }
        }
        if (ctl.dead) break;
    }
}

// Fetch of a stage input where every thread takes exactly the elements it will use itself: element k
// belongs to thread k mod 256, the same thread that owns weight row k in the dot products.  Nothing else
// reads dst[k], so no barrier is needed between this fetch and the dot products, and a thread starts its
// multiply-adds as soon as ITS words have arrived.  8-byte loads, up to U in flight per thread.
template <int U = 8, bool RT = true>
__device__ __noinline__ void mg_fetch_own(const mg_word* src, int n, uint32_t tag, float* dst, mg_ctl& ctl) {
    __builtin_assume(__isShared(dst));
    for (int base = threadIdx.x; base < n; base += MG_THREADS * U) {
        uint32_t pending = 0;
#pragma unroll
        for (int u = 0; u < U; u++)
            if (base + u * MG_THREADS < n) pending |= 1u << u;
        uint32_t spins = 0;
        while (pending != 0) {
            mg_word w[U];
#pragma unroll
            for (int u = 0; u < U; u++)
                if (pending & (1u << u)) w[u] = mg_ld_word(src + base + u * MG_THREADS);
            uint32_t done = 0;
#pragma unroll
            for (int u = 0; u < U; u++) {
                if ((pending & (1u << u)) && (uint32_t)(w[u] >> 32) == tag) {
                    dst[base + u * MG_THREADS] = __uint_as_float((uint32_t)w[u]);
                    done |= 1u << u;
                }
            }
            pending &= ~done;
            if (pending != 0) {
                if (++spins > (RT ? ctl.limit : MG_SPIN_LIMIT) || ((spins & 255u) == 0 && mg_ld_flag(ctl.abort_flag))) {
                    mg_give_up(ctl);
                    break;
                }
                if (RT && ctl.poll_sleep) __nanosleep(ctl.poll_sleep);
            }
        }
        if (ctl.dead) break;
    }
}

__device__ __forceinline__ float mg_block_max(float v, float* scratch) {
    v = rg_warp_max(v);
    mg_csync();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    mg_csync();
    float r = scratch[0];
#pragma unroll
    for (int i = 1; i < MG_THREADS / 32; i++) r = fmaxf(r, scratch[i]);
    return r;
}

// Sum N per-lane values across the warp with a halving exchange: while N is even each
// step sends half of the values to the partner lane and keeps the other half, so N
// halves per step; the remaining steps are plain butterflies.  On return v[0..count)
// of lane l holds the warp sums of indices base + [0, count).
template <int N, int O>
struct mg_halver {
    __device__ __forceinline__ static void run(float (&v)[N], int lane, int& base, int& count) {
        if constexpr (O == 0) {
            count = N;
        } else if constexpr (N % 2 == 0) {
            constexpr int H = N / 2;
            const bool upper = (lane & O) != 0;
            float keep[H];
#pragma unroll
            for (int i = 0; i < H; i++) {
                const float send = upper ? v[i] : v[i + H];
                const float recv = __shfl_xor_sync(RG_FULL_MASK, send, O);
                keep[i] = (upper ? v[i + H] : v[i]) + recv;
            }
            if (upper) base += H;
            mg_halver<H, O / 2>::run(reinterpret_cast<float(&)[H]>(keep), lane, base, count);
#pragma unroll
            for (int i = 0; i < H; i++) v[i] = keep[i];
        } else {
#pragma unroll
            for (int i = 0; i < N; i++) v[i] += __shfl_xor_sync(RG_FULL_MASK, v[i], O);
            mg_halver<N, O / 2>::run(v, lane, base, count);
        }
    }
    // lanes that differ only in bits consumed by plain butterflies hold identical sums: the lowest one writes
    __device__ __forceinline__ static bool writer(int lane) {
        int n = N, o = 16;
        while (o > 0 && n % 2 == 0) n /= 2, o >>= 1;
        return o == 0 || (lane & (2 * o - 1)) == 0;
    }
};
