// Token loop as ONE persistent kernel of thread-block clusters with specialised warps: n token steps of the
// KV-cache loop (src/wasm_api.rs:102-160 on a causal model), two grid-wide exchanges per transformer block
// (src/nn/transformer.rs:51-65).
//
// Decomposition over CTAs (sm_100a, one CTA per SM, clusters of `cs` CTAs):
//  * Cluster h < H is the HEAD CLUSTER of head h.  Its CTAs split the head's q|k|v columns (LayerNorm folded into the
//    projection), pass the 3*head_dim results to each other through distributed shared memory, attend over one slice
//    of the context each (src/nn/attention.rs:57-105, online softmax, K/V slices stream through the ring), pass the
//    (max, sum, output) records around the same way, merge them, and multiply the head's output with the head's ROWS
//    of Wo: a partial sum of the out-projection, the D columns split over the CTAs of the cluster.  H partial vectors
//    per block go to global memory as tagged words {value, tag}.
//  * EVERY CTA owns a slice of the hidden units: its columns of FC1 (LayerNorm folded), the activation, and ITS ROWS
//    of FC2 without leaving the CTA (src/nn/feedforward.rs:40-48).  The D-long partial sums of the CTAs of a cluster
//    are reduce-scattered through distributed shared memory; one partial vector per cluster goes to global memory.
//  * A consumer of such a set of partial vectors works per cluster as well: CTA r fetches slice r of every partial
//    vector (polling the tags), adds them in index order and stores the sums into all CTAs of its cluster.  Residual
//    and bias travel inside partial 0 (the cluster that produces it adds them), so the sum of the partials IS the
//    new residual stream and no CTA keeps residual state.
//
// Decomposition inside a CTA: 8 consumer warps in 4 roles of 2 warps, one role per SM sub-partition (warp w runs on
// scheduler w mod 4), plus the producer warp:
//      role 0 "exchange": embedding, fetch + sum + distribute of the partial vectors, the pick;
//      role 1 "rows":     the projections whose K rows are spread over threads (q|k|v, FC1, LM head);
//      role 2 "head":     attention over the context slice, merge, out-projection partial;
//      role 3 "columns":  FC2 rows of the hidden slice, reduce-scatter, partial vector of the cluster.
//    A role executes only its own few hundred instructions per block, which stay in its scheduler's instruction cache;
//    the same loop with every warp running every stage fetched most of its instructions from L2 (measured: 7 cycles
//    per instruction) and was three times slower.  Roles hand results to each other through shared memory and
//    mbarriers; nothing in the loop is a CTA-wide barrier.
//  * Weights are packed per CTA in consumption order and stream through a ring of 32 KB shared-memory slots (bulk
//    asynchronous copies issued by the producer warp, which runs ahead across stages and tokens); each chunk is
//    consumed by exactly one role.
//  * Inside a cluster, data moves by plain stores into the other CTA's shared memory; each sending warp then signals
//    the receivers' mbarrier once (arrive with release at cluster scope), the receivers wait with acquire.
//  * Every wait is bounded: on expiry the thread raises a global flag, every role of every CTA leaves, the host
//    reports RG_ERR_TIMEOUT.  No multicast load is used.
#include "rg_gpt.h"

#include <stdlib.h>
#include <string.h>

#include <algorithm>

#include "rg_loop_dev.cuh"

enum { CL_QKV = 0, CL_ATTN = 1, CL_OPROJ = 2, CL_FC1 = 3, CL_FC2 = 4, CL_HEAD = 5 };
enum { CL_FIRST = 1, CL_LAST = 2 };
enum { CL_ROLE_XCH = 0, CL_ROLE_ROWS = 1, CL_ROLE_HEAD = 2, CL_ROLE_COLS = 3 };
#define CL_MAX_CS 16
#define CL_RT 64     // threads of a role
#define CL_NVMAX 32  // accumulators (values x sequences) a thread carries through a row-split projection op
#define CL_NUT 8     // most 4-column units a thread owns in a column-split op

// Row-split projection (QKV, FC1, head): nq 4-column units [q0, q0 + nq), all K rows, chunks of kc rows laid out
// [unit][row][4 columns]; trailer [additive term per column][LayerNorm mean coefficient per column].
// Column-split product (out-projection partial, FC2): rows [k0, k0 + nq) of the matrix, columns [q0, q0 + nvalid),
// chunks of kc whole rows laid out [row][columns]; trailer = bias of the CTA's slice of a D-long vector.
struct cl_op {
    int type, layer;
    int nq;
    int nvalid;
    int q0;
    int K, kc, nchunks;
    int k0;
    int flags;
    int uv;   // 4
    int aux;  // QKV: head; FC1: offset of the op's first value in the CTA's hidden slice; head: pick slot
    long long src;
};

struct cl_cdesc {
    long long src;  // kind 0: byte offset into the packed weights; 2: the CTA's attention slices (expanded on the device)
    int bytes;
    int kind;
};

struct cl_params {
    const cl_op* ops;
    const int* cta_off;
    const cl_cdesc* cds;
    const int* cd_off;
    const unsigned char* wpack;
    unsigned long long* trace;

    const void *wte, *wpe;
    long long ldt;
    unsigned char *kc, *vc;
    size_t kv_layer_bytes;
    mg_word *buf_a, *buf_b, *buf_pick;
    float* logits;
    uint32_t *tokens, *picks;
    int *d_pos, *d_pos_next;
    int* abort_flag;
    int V, D, L, H, hd, C, F;
    int act;
    int pos0, n_steps;
    uint32_t epoch0;
    int nslot, max_ops, max_cd, n_pick_ctas;
    int cs, ncl;
    int su[CL_MAX_CS + 1];  // slice r of a D-long vector = elements [su[r], su[r+1]) (multiples of 4)
    int nh_cap;             // hidden units a CTA owns at most
    int n4_cap;             // 4-element groups in the largest slice
    int scr_bytes;          // scratch of the head role (attention partials)
    int qkv_signals;        // q|k|v ops of a head cluster (each signals the cluster once)
    uint32_t spin_limit;
    int poll_sleep;         // ns between two polls of words that were not valid yet (0: none)
    int withhold_layer;     // test hook: head cluster 0 does not publish its out-projection partial of this layer (-1: off)
    float scale;
};

// ---------------------------------------------------------------------------
// cluster helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cl_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cl_id() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cl_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cl_mapa(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
// plain stores into the shared memory of a CTA of the cluster (this one included)
__device__ __forceinline__ void cl_st1(uint32_t raddr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(raddr), "f"(v) : "memory");
}
__device__ __forceinline__ void cl_st2(uint32_t raddr, float a, float b) {
    asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(raddr), "f"(a), "f"(b) : "memory");
}
__device__ __forceinline__ void cl_st4(uint32_t raddr, float a, float b, float c, float d) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(raddr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
// 16 bytes into the shared memory of CTA `rank` of the cluster (this one included); the store completes 16 bytes on that
// CTA's mbarrier at the same offset as `bar`: data and signal travel together, no fence and no separate arrive.
// (Measured for 96 floats from each of 8 CTAs to each: 563 cycles per round this way, 1085 with plain remote stores
// followed by an arrive with release semantics, 1030 with a bulk copy out of a local staging buffer.)
__device__ __forceinline__ void cl_send4(uint32_t a_dst, uint32_t a_bar, uint32_t rank, float x, float y, float z, float w) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(cl_mapa(a_dst, rank)),
                 "f"(x), "f"(y), "f"(z), "f"(w), "r"(cl_mapa(a_bar, rank))
                 : "memory");
}
// the receiving side: one thread announces the bytes of the phase, every thread then waits for them (bounded)
__device__ __forceinline__ void cl_expect(uint64_t* bar, uint32_t bytes) { mg_mbar_expect_tx(bar, bytes); }

// One signal of the calling warp to every CTA of the cluster: everything the warp stored before it is visible to a
// thread that has seen the receiving barrier's phase complete (arrive.release / try_wait.acquire at cluster scope).
__device__ __forceinline__ void cl_signal_warp(uint64_t* bar, int cs) {
    __syncwarp();
    const int lane = threadIdx.x & 31;
    if (lane < cs) {
        const uint32_t rb = cl_mapa(mg_smem(bar), (uint32_t)lane);
        asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(rb) : "memory");
    }
}
// one arrival of the calling warp on a barrier of this CTA (hand-off between roles)
__device__ __forceinline__ void cl_arrive_warp(uint64_t* bar) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mg_mbar_arrive(bar);
}
__device__ __forceinline__ bool cl_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(mg_smem(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void cl_st_word2(mg_word* p, uint32_t tag, float a, float b) {
    const mg_word wa = ((mg_word)tag << 32) | __float_as_uint(a), wb = ((mg_word)tag << 32) | __float_as_uint(b);
    asm volatile("st.relaxed.gpu.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(wa), "l"(wb) : "memory");
}
// bounded wait on an mbarrier of this CTA
__device__ __forceinline__ void cl_wait(uint64_t* bar, uint32_t parity, mg_ctl& ctl, uint32_t limit) {
    uint32_t spins = 0;
    while (!ctl.dead && !cl_try_wait(bar, parity)) {
        if (++spins > limit || ((spins & 255u) == 0 && mg_ld_flag(ctl.abort_flag))) mg_give_up(ctl);
        if (ctl.poll_sleep) __nanosleep(ctl.poll_sleep);
    }
}
// barrier of the 64 threads of a role (named barriers 2..5) that also spreads `dead`
__device__ __forceinline__ bool cl_rsync_or(int role, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.or.pred q, %2, 64, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(r)
        : "r"((uint32_t)(pred ? 1 : 0)), "r"(2 + role)
        : "memory");
    return r != 0;
}

// a pair of alternating receive buffers with their barriers: index and the parity to wait for next (bit i)
struct cl_flip {
    int i;
    uint32_t ph;
    __device__ __forceinline__ uint32_t parity() const { return (ph >> i) & 1u; }
    __device__ __forceinline__ void done() { ph ^= 1u << i, i ^= 1; }  // after the use of buffer i
};

__device__ __forceinline__ void cl_ring_skip(mg_cons& r, int n) {
    const int s = r.slot + n;
    r.parity ^= (uint32_t)(s / r.nslot) & 1u;
    r.slot = s % r.nslot;
}

// Shared memory is read and written through 32-bit shared-state-space addresses in everything that is on the critical
// path.  A load through a generic pointer takes the global-memory path of the SM, where it queues behind the polling
// loads of the exchange role (measured: 2 to 8 times slower than ld.shared for the same loop).
__device__ __forceinline__ float cl_lds(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ float2 cl_lds2(uint32_t a) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ float4 cl_lds4(uint32_t a) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 cl_ldsu4(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ void cl_sts(uint32_t a, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory"); }
__device__ __forceinline__ void cl_sts4(uint32_t a, float4 v) {
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(a), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
// 4 weights of a unit (16 bytes of f32, 8 bytes of bf16) at shared address a
template <typename WT>
__device__ __forceinline__ void cl_ldw4(uint32_t a, float (&w)[4]) {
    if constexpr (sizeof(WT) == 4) {
        const float4 v = cl_lds4(a);
        w[0] = v.x, w[1] = v.y, w[2] = v.z, w[3] = v.w;
    } else {
        uint32_t x, y;
        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(x), "=r"(y) : "r"(a));
        w[0] = __uint_as_float(x << 16), w[1] = __uint_as_float(x & 0xffff0000u);
        w[2] = __uint_as_float(y << 16), w[3] = __uint_as_float(y & 0xffff0000u);
    }
}
// the ring as the consumer sees it, by shared address
__device__ __forceinline__ uint32_t cl_ring_wait(mg_cons& r, mg_ctl& ctl) { return mg_smem(mg_ring_wait(r, ctl)); }

// shared-memory map of a CTA (must match cl_smem_bytes on the host)
struct cl_mem {
    unsigned char* slots;
    uint64_t *full, *empty;
    uint64_t *barX, *barQ, *barR, *barF, *barH, *barA;
    cl_op* ops;
    cl_cdesc* cds;
    float *rxX, *rxQ, *rxR, *rxF;
    float *hs, *ovec, *colred, *scr;
    float *red, *stat, *pickbuf;
    float* bestv;
    int* besti;
    uint32_t* s_pick;
    int* s_flags;
};

template <int B>
__device__ __forceinline__ void cl_carve(const cl_params& p, unsigned char* sp, cl_mem& m) {
    m.slots = sp;
    sp += (size_t)p.nslot * MG_SLOT_BYTES;
    m.full = reinterpret_cast<uint64_t*>(sp);
    m.empty = m.full + 8;
    m.barX = m.full + 16, m.barQ = m.full + 18, m.barR = m.full + 20, m.barF = m.full + 22, m.barH = m.full + 24, m.barA = m.full + 26;
    sp += 32 * 8;
    m.ops = reinterpret_cast<cl_op*>(sp);
    sp += (size_t)p.max_ops * sizeof(cl_op);
    m.cds = reinterpret_cast<cl_cdesc*>(sp);
    sp += (size_t)p.max_cd * sizeof(cl_cdesc);
    sp = reinterpret_cast<unsigned char*>(((uintptr_t)sp + 15) & ~(uintptr_t)15);
    m.rxX = reinterpret_cast<float*>(sp);  // [2][B][D]
    sp += (size_t)2 * B * p.D * 4;
    m.rxF = reinterpret_cast<float*>(sp);  // [2][cs][B][n4_cap][4]
    sp += (size_t)2 * p.cs * B * p.n4_cap * 16;
    m.colred = reinterpret_cast<float*>(sp);  // [2][B][n4_cap][4] partial sums of the two row groups of a column-split op
    sp += (size_t)2 * B * p.n4_cap * 16;
    m.rxQ = reinterpret_cast<float*>(sp);  // [2][B][3 * head_dim]
    sp += (size_t)2 * B * 3 * p.hd * 4;
    m.rxR = reinterpret_cast<float*>(sp);  // [2][cs][B][hd + 4]
    sp += (size_t)2 * p.cs * B * (p.hd + 4) * 4;
    m.hs = reinterpret_cast<float*>(sp);  // [2][B][nh_cap]
    sp += (size_t)2 * B * p.nh_cap * 4;
    m.ovec = reinterpret_cast<float*>(sp);  // [B][hd]
    sp += (size_t)B * p.hd * 4;
    m.scr = reinterpret_cast<float*>(sp);  // attention partials of the head role
    sp += (size_t)p.scr_bytes;
    m.red = reinterpret_cast<float*>(sp);  // [2][2][CL_NVMAX]
    sp += 2 * 2 * CL_NVMAX * 4;
    m.stat = reinterpret_cast<float*>(sp);  // [2][2][B][4]
    sp += 2 * 2 * 4 * MG_BMAX * 4;
    m.pickbuf = reinterpret_cast<float*>(sp);  // [n_pick_ctas * B * 2]
    sp += (size_t)p.n_pick_ctas * B * 2 * 4;
    m.bestv = reinterpret_cast<float*>(sp);
    sp += CL_RT * 4;
    m.besti = reinterpret_cast<int*>(sp);
    sp += CL_RT * 4;
    m.s_pick = reinterpret_cast<uint32_t*>(sp);
    sp += MG_BMAX * 4;
    m.s_flags = reinterpret_cast<int*>(sp);  // [0] tokens whose pick this CTA has seen, [1] dead
}

#define CL_CLK(i)                                               \
    do {                                                        \
        if (TRACE && tw) tw[i] = (unsigned long long)clock64(); \
    } while (0)

template <bool TRACE>
__device__ __forceinline__ unsigned long long* cl_tw(const cl_params& p, int t, int oi) {
    if constexpr (TRACE) {
        if (p.trace != nullptr && t == p.n_steps - 1 && (threadIdx.x & 31) == 0) {
            const int w = (int)(threadIdx.x >> 5);
            unsigned long long* base = p.trace + ((size_t)blockIdx.x * p.max_ops + oi) * 72;
            if (w < 4) base[w] = mg_globaltimer();  // wall-clock start of the op, per role
            return base + 8 + w * 8;
        }
    }
    return nullptr;
}

// ---------------------------------------------------------------------------
// The producer: walks the CTA's copy schedule for every token of the run, waits for a free slot, issues the copy.
// K/V rows below the current position are final only once this CTA has seen the previous token's pick (the last CTA
// of the cluster appends row pos-1 during that token): s_progress counts the picks seen.
// ---------------------------------------------------------------------------
__device__ void cl_producer(const cl_params& p, const cl_cdesc* cd, int ncd, unsigned char* slots, uint64_t* full, uint64_t* empty,
                            int nslot, volatile int* s_progress, volatile int* s_dead, int kvsize, int B, int head, int rank) {
    int slot = 0;
    uint32_t parity = 0, issued = 0;
    bool stop = false;
    const int rc = mg_attn_rows_per_chunk(p.hd, kvsize);
    const size_t rb = (size_t)p.hd * kvsize;
    const uint32_t limit = p.spin_limit;
    for (int tok = 0; tok < p.n_steps && !stop; tok++) {
        const int pos = p.pos0 + tok;
        for (int i = 0; i < ncd && !stop; i++) {
            const cl_cdesc d = cd[i];
            int nseq = 1;
            if (d.kind == 2) {
                nseq = B;
                if (tok > 0) {
                    uint32_t spins = 0;
                    while (*s_progress < tok) {
                        if (++spins > limit || *s_dead) {
                            stop = true;
                            break;
                        }
                    }
                    if (stop) break;
                    mg_fence_proxy_async();
                }
            }
            for (int b = 0; b < nseq && !stop; b++) {
                int nch = 1, arows = 0;
                const unsigned char *kbase = nullptr, *vbase = nullptr;
                if (d.kind == 2) {
                    const int c = (pos + p.cs - 1) / p.cs;  // rows per slice
                    const int r_lo = rank * c;
                    const int r_hi = min(pos, r_lo + c);
                    arows = max(0, r_hi - r_lo);
                    nch = 2 * ((arows + rc - 1) / rc);
                    const size_t head_off = (((size_t)b * p.H + head) * p.C + r_lo) * rb + (size_t)d.src * p.kv_layer_bytes;
                    kbase = p.kc + head_off;
                    vbase = p.vc + head_off;
                }
                for (int j = 0; j < nch; j++) {
                    uint32_t spins = 0;
                    while (!mg_mbar_try_wait(&empty[slot], parity ^ 1u)) {
                        if (++spins > limit || *s_dead) {
                            stop = true;
                            break;
                        }
                        if (p.poll_sleep) __nanosleep(p.poll_sleep);
                    }
                    if (stop) break;
                    const unsigned char* src;
                    uint32_t bytes;
                    if (d.kind == 0) src = p.wpack + d.src, bytes = (uint32_t)d.bytes;
                    else {
                        const int jj = j >> 1;  // K rows of a range, then V rows of the same range
                        const int rows = min(rc, arows - jj * rc);
                        src = ((j & 1) ? vbase : kbase) + (size_t)jj * rc * rb;
                        bytes = (uint32_t)(rows * rb);
                    }
                    mg_mbar_expect_tx(&full[slot], bytes);
                    mg_bulk_g2s(slots + (size_t)slot * MG_SLOT_BYTES, src, bytes, &full[slot]);
                    issued++;
                    if (++slot == nslot) slot = 0, parity ^= 1u;
                }
            }
        }
    }
    if (stop) {
        const uint32_t n = issued < (uint32_t)nslot ? issued : (uint32_t)nslot;
        for (uint32_t i = 0; i < n; i++) {
            if (--slot < 0) slot = nslot - 1, parity ^= 1u;
            uint32_t spins = 0;
            while (!mg_mbar_try_wait(&full[slot], parity) && ++spins < limit) {
            }
        }
    }
}

// chunks of the ring that the attention op of this CTA takes at position pos
__device__ __forceinline__ int cl_attn_chunks(const cl_params& p, int pos, int me, int kvsize, int B) {
    const int csz = (pos + p.cs - 1) / p.cs;
    const int r_lo = me * csz;
    const int arows = max(0, min(pos, r_lo + csz) - r_lo);
    const int rc = mg_attn_rows_per_chunk(p.hd, kvsize);
    return 2 * ((arows + rc - 1) / rc) * B;
}

// ---------------------------------------------------------------------------
// role 0: the exchanges.  Fetch of a set of partial vectors: this CTA takes elements [e0, e0 + ne) of every partial
// (thread q owns one pair of elements and polls all P partials of it, up to 16 loads in flight), adds them in index
// order and stores the sums into xdst (same shared-memory offset) of every CTA of the cluster; both warps signal bar.
// ---------------------------------------------------------------------------
template <int B>
__device__ __forceinline__ void cl_consume(const mg_word* buf, int P, uint32_t tag, int D, int e0, int ne, float* xdst, uint64_t* bar,
                                           int cs, mg_ctl& ctl, uint32_t limit, int rt) {
    const int npair = ne >> 1, ntot = B * npair;  // npair is even: slices are multiples of 4 elements
    const uint32_t a_x = mg_smem(xdst), a_bar = mg_smem(bar);
    for (int q0 = 0; q0 < ntot; q0 += CL_RT) {
        const int qq = q0 + rt;
        const bool on = qq < ntot;
        const int b = on ? qq / npair : 0, pr = on ? qq - b * npair : 0;
        const mg_word* src = buf + (size_t)b * D + e0 + 2 * pr;
        float sx = 0.f, sy = 0.f;
        for (int p0 = 0; p0 < P && on && !ctl.dead; p0 += 16) {
            uint32_t pending = 0;
#pragma unroll
            for (int u = 0; u < 16; u++)
                if (p0 + u < P) pending |= 1u << u;
            const uint32_t want = pending;
            mg_word w[16][2];
            uint32_t spins = 0;
            while (pending != 0) {
#pragma unroll
                for (int u = 0; u < 16; u++)
                    if (pending & (1u << u)) mg_ld_word2(src + (size_t)(p0 + u) * B * D, w[u][0], w[u][1]);
                uint32_t done = 0;
#pragma unroll
                for (int u = 0; u < 16; u++)
                    if ((pending & (1u << u)) && (uint32_t)(w[u][0] >> 32) == tag && (uint32_t)(w[u][1] >> 32) == tag) done |= 1u << u;
                pending &= ~done;
                if (pending != 0) {
                    if (++spins > limit || ((spins & 255u) == 0 && mg_ld_flag(ctl.abort_flag))) {
                        mg_give_up(ctl);
                        break;
                    }
                    if (ctl.poll_sleep) __nanosleep(ctl.poll_sleep);
                }
            }
            if (ctl.dead) break;
#pragma unroll
            for (int u = 0; u < 16; u++)
                if (want & (1u << u)) {
                    sx += __uint_as_float((uint32_t)w[u][0]);
                    sy += __uint_as_float((uint32_t)w[u][1]);
                }
        }
        // two neighbouring pairs make one 16-byte store per destination
        const float nx = __shfl_down_sync(RG_FULL_MASK, sx, 1), ny = __shfl_down_sync(RG_FULL_MASK, sy, 1);
        if (on && (qq & 1) == 0) {
            const uint32_t a = a_x + (uint32_t)((b * D + e0 + 2 * pr) * 4);
            for (int d = 0; d < cs; d++) cl_send4(a, a_bar, (uint32_t)d, sx, sy, nx, ny);
        }
    }
}

template <typename WT, int B, bool TRACE>
__device__ __forceinline__ void cl_role_exchange(const cl_params& p, const cl_mem& m, int nops, int me, int cid, mg_ctl& ctl) {
    const int rt = threadIdx.x >> 7 << 5 | (threadIdx.x & 31);  // warps 0 and 4
    const int lane = threadIdx.x & 31, wr = threadIdx.x >> 7;
    const int D = p.D, cs = p.cs;
    const uint32_t limit = p.spin_limit;
    const int e0 = p.su[me], ne = p.su[me + 1] - p.su[me];
    const WT* wte = static_cast<const WT*>(p.wte);
    const WT* wpe = static_cast<const WT*>(p.wpe);
    int xi = 0;
    for (int t = 0; t < p.n_steps; t++) {
        const int pos = p.pos0 + t;
        const uint32_t tagbase = (p.epoch0 + (uint32_t)t) * (uint32_t)(p.L + 1);
        for (int oi = 0; oi < nops; oi++) {
            const cl_op& op = m.ops[oi];
            if (!(op.flags & CL_FIRST) || (op.type != CL_QKV && op.type != CL_FC1 && op.type != CL_HEAD)) continue;
            unsigned long long* tw = cl_tw<TRACE>(p, t, oi);
            CL_CLK(0);
            xi ^= 1;
            float* xn = m.rxX + (size_t)xi * B * D;
            const uint32_t tag = tagbase + (uint32_t)op.layer + 1u;
            if (op.type == CL_QKV && op.layer == 0) {
                // token + position embedding (src/models/gpt.rs:62-75): this CTA's slice for every CTA of the cluster
                const uint32_t a_x = mg_smem(xn), a_bar = mg_smem(&m.barX[xi]);
                const int n4s = ne >> 2;
                for (int i = rt; i < B * n4s; i += CL_RT) {
                    const int b = i / n4s, k = e0 + 4 * (i - b * n4s);
                    const uint32_t tok = t == 0 ? p.tokens[(size_t)b * p.C + pos] : m.s_pick[b];
                    float v[4];
#pragma unroll
                    for (int c = 0; c < 4; c++) v[c] = rg_to_float(wte[(size_t)tok * p.ldt + k + c]) + rg_to_float(wpe[(size_t)pos * p.ldt + k + c]);
                    for (int d = 0; d < cs; d++) cl_send4(a_x + (uint32_t)((b * D + k) * 4), a_bar, (uint32_t)d, v[0], v[1], v[2], v[3]);
                }
            } else {
                const bool from_a = op.type == CL_FC1;
                cl_consume<B>(from_a ? p.buf_a : p.buf_b, from_a ? p.H : p.ncl, from_a ? tag : tag - 1u, D, e0, ne, xn, &m.barX[xi], cs, ctl,
                              limit, rt);
            }
            CL_CLK(1);
            // A wait that gave up marks only the threads that waited.  Every lane of the warp must take the same way out:
            // the fetch above shuffles with a full mask, and lanes that stayed in this loop would wait there for lanes that
            // already sit at the role barrier below.
            if (__any_sync(RG_FULL_MASK, ctl.dead)) {
                ctl.dead = true;
                break;
            }
        }
        if (cl_rsync_or(CL_ROLE_XCH, ctl.dead)) {
            ctl.dead = true;
            break;
        }
        // ---- greedy pick (top_k = 1 of src/wasm_api.rs:120-156): best over all CTAs, lowest index on ties ----
        {
            const int n = p.n_pick_ctas * B * 2;
            const uint32_t ptag = tagbase + (uint32_t)p.L + 1u;
            for (int i = rt; i < n; i += CL_RT) {
                uint32_t spins = 0;
                mg_word w = mg_ld_word(p.buf_pick + i);
                while ((uint32_t)(w >> 32) != ptag) {
                    if (++spins > limit || ((spins & 255u) == 0 && mg_ld_flag(ctl.abort_flag))) {
                        mg_give_up(ctl);
                        break;
                    }
                    w = mg_ld_word(p.buf_pick + i);
                }
                m.pickbuf[i] = __uint_as_float((uint32_t)w);
            }
            // everything any CTA stored before its pick (cache rows included) is ordered before what follows here
            __threadfence();
            mg_fence_proxy_async();
            if (cl_rsync_or(CL_ROLE_XCH, ctl.dead)) {
                ctl.dead = true;
                break;
            }
            if (wr == 0) {
                for (int b = 0; b < B; b++) {
                    float bv = -INFINITY;
                    int bi = 0x7fffffff;
                    for (int r = lane; r < p.n_pick_ctas; r += 32) {
                        const float v = m.pickbuf[(r * B + b) * 2];
                        const int ix = (int)__float_as_uint(m.pickbuf[(r * B + b) * 2 + 1]);
                        if (v > bv || (v == bv && ix < bi)) bv = v, bi = ix;
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        const float ov = __shfl_xor_sync(RG_FULL_MASK, bv, o);
                        const int oi2 = __shfl_xor_sync(RG_FULL_MASK, bi, o);
                        if (ov > bv || (ov == bv && oi2 < bi)) bv = ov, bi = oi2;
                    }
                    if (lane == 0) {
                        if (bi == 0x7fffffff) bi = 0;
                        m.s_pick[b] = (uint32_t)bi;
                        if (blockIdx.x == 0) {
                            p.picks[b] = (uint32_t)bi;
                            if (pos + 1 < p.C) p.tokens[(size_t)b * p.C + pos + 1] = (uint32_t)bi;
                        }
                    }
                }
                if (lane == 0) *reinterpret_cast<volatile int*>(m.s_flags) = t + 1;  // the producer reads this
            }
            if (cl_rsync_or(CL_ROLE_XCH, ctl.dead)) {
                ctl.dead = true;
                break;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// role 1: row-split projections.  Thread rt takes rows rt, rt + 64, ... of every chunk and all NQA units.
// ---------------------------------------------------------------------------
template <typename WT, int B, int NQA>
__device__ __forceinline__ void cl_rows_dots(const cl_op& op, mg_cons& ring, mg_ctl& ctl, const float* xs, int XLEN, float* red, int rt,
                                             float& t0, float& t1, unsigned long long* tw) {
    constexpr int UB = 4 * (int)sizeof(WT);
    constexpr int NV = B * NQA * 4;
    const int lane = rt & 31, wr = rt >> 5;
    float acc[NV];
#pragma unroll
    for (int i = 0; i < NV; i++) acc[i] = 0.f;
    long long wcyc = 0;
    const uint32_t a_xs = mg_smem(xs);
    const int nchunks = op.nchunks, kc = op.kc, K = op.K;
    for (int j = 0; j < nchunks; j++) {
        const long long c0 = tw ? clock64() : 0;
        const uint32_t slot = cl_ring_wait(ring, ctl);
        if (tw) wcyc += clock64() - c0;
        const int kb = j * kc;
        const int rows = min(kc, K - kb);
        if (j == nchunks - 1 && rt < NV) {
            const uint32_t tr = slot + (uint32_t)(NQA * rows) * UB;
            t0 = cl_lds(tr + 4u * (rt / B));
            t1 = cl_lds(tr + 4u * (NQA * 4 + rt / B));
        }
        const uint32_t xr = a_xs + 4u * kb;
        // two rows per step: every load of the step is issued before the first multiply-add needs one (the loads are
        // volatile asm statements, which the compiler keeps in order and does not hoist above the arithmetic by itself)
        for (int r = rt; r < rows; r += 2 * CL_RT) {
            const bool two = r + CL_RT < rows;
            const int r1 = two ? r + CL_RT : r;
            float xv[2][B], w[2][NQA][4];
#pragma unroll
            for (int b = 0; b < B; b++) xv[0][b] = cl_lds(xr + 4u * (b * XLEN + r)), xv[1][b] = cl_lds(xr + 4u * (b * XLEN + r1));
#pragma unroll
            for (int q = 0; q < NQA; q++) {
                cl_ldw4<WT>(slot + ((uint32_t)(q * rows + r)) * UB, w[0][q]);
                cl_ldw4<WT>(slot + ((uint32_t)(q * rows + r1)) * UB, w[1][q]);
            }
            if (!two) {
#pragma unroll
                for (int b = 0; b < B; b++) xv[1][b] = 0.f;
            }
#pragma unroll
            for (int h = 0; h < 2; h++)
#pragma unroll
                for (int q = 0; q < NQA; q++)
#pragma unroll
                    for (int jj = 0; jj < 4; jj++)
#pragma unroll
                        for (int b = 0; b < B; b++) acc[(q * 4 + jj) * B + b] = fmaf(xv[h][b], w[h][q][jj], acc[(q * 4 + jj) * B + b]);
        }
        mg_ring_release(ring);
    }
    if (tw) tw[5] = (unsigned long long)wcyc, tw[6] = (unsigned long long)clock64();
    int base = 0, count = 0;
    mg_halver<NV, 16>::run(acc, lane, base, count);
    if (mg_halver<NV, 16>::writer(lane)) {
        const uint32_t a_red = mg_smem(red);
#pragma unroll
        for (int i = 0; i < NV; i++)
            if (i < count) cl_sts(a_red + 4u * (wr * CL_NVMAX + base + i), acc[i]);
    }
}

template <typename WT, int B, bool TRACE>
__device__ __forceinline__ void cl_role_rows(const cl_params& p, const cl_mem& m, int nops, int me, int cid, mg_ctl& ctl, mg_cons& ring) {
    constexpr int KVS = sizeof(WT);
    const int rt = ((threadIdx.x >> 5) >> 2) * 32 + (threadIdx.x & 31);  // warps 1 and 5
    const int lane = rt & 31, wr = rt >> 5;
    const int D = p.D, HD = p.hd, cs = p.cs, Q3 = 3 * p.hd;
    const uint32_t limit = p.spin_limit;
    cl_flip fx = {0, 0}, fq = {0, 0}, fh = {0, 0}, fa = {0, 0};
    const float* xcur = m.rxX;
    float mu[B], rstd[B];
#pragma unroll
    for (int b = 0; b < B; b++) mu[b] = 0.f, rstd[b] = 1.f;
    bool stats_pending = false;
    for (int t = 0; t < p.n_steps; t++) {
        const int pos = p.pos0 + t;
        const uint32_t tagbase = (p.epoch0 + (uint32_t)t) * (uint32_t)(p.L + 1);
        float my_best = -INFINITY;
        int my_besti = 0x7fffffff;
        for (int oi = 0; oi < nops; oi++) {
            const cl_op& op = m.ops[oi];
            const int type = op.type;
            if (type == CL_ATTN) {
                cl_ring_skip(ring, cl_attn_chunks(p, pos, me, KVS, B));
                continue;
            }
            if (type == CL_OPROJ || type == CL_FC2) {
                cl_ring_skip(ring, op.nchunks);
                continue;
            }
            unsigned long long* tw = cl_tw<TRACE>(p, t, oi);
            CL_CLK(0);
            float* red = m.red + (oi & 1) * (2 * CL_NVMAX);
            float* stat = m.stat + (oi & 1) * (2 * 4 * MG_BMAX);
            if (op.flags & CL_FIRST) {
                // the stage's input vector, complete, from the exchange role(s) of the cluster.  LayerNorm is folded into the
                // projection (gamma in the packed weights):
                //   LN(x).W + b = rstd * (sum_k x_k g_k W_kn - mean * sum_k g_k W_kn) + (sum_k beta_k W_kn + b_n)
                // (src/ops/norm.rs:41-52); the two column sums ride at the end of the op's weights.
                fx.i ^= 1;
                if (rt == 0) cl_expect(&m.barX[fx.i], (uint32_t)(B * D * 4));
                cl_wait(&m.barX[fx.i], fx.parity(), ctl, limit);
                fx.ph ^= 1u << fx.i;
                xcur = m.rxX + (size_t)fx.i * B * D;
                // statistics: per warp, shifted sums over the elements its threads own, shift = the warp's first element;
                // the two tuples are combined exactly after the dot products
#pragma unroll
                for (int b = 0; b < B; b++) {
                    const uint32_t xr = mg_smem(xcur + b * D);
                    const float c = __shfl_sync(RG_FULL_MASK, cl_lds(xr + 4u * (rt < D ? rt : 0)), 0);
                    float s0 = 0.f, s1 = 0.f, s2 = 0.f;
#pragma unroll 4
                    for (int i = rt; i < D; i += CL_RT) {
                        const float d = cl_lds(xr + 4u * i) - c;
                        s0 += 1.f;
                        s1 += d;
                        s2 = fmaf(d, d, s2);
                    }
                    s0 = rg_warp_sum(s0);
                    s1 = rg_warp_sum(s1);
                    s2 = rg_warp_sum(s2);
                    if (lane == 0) {
                        float* sc4 = stat + (wr * B + b) * 4;
                        sc4[0] = s0, sc4[1] = s1, sc4[2] = s2, sc4[3] = c;
                    }
                }
                stats_pending = true;
            }
            CL_CLK(1);
            float t0 = 0.f, t1 = 0.f;
            switch (op.nq) {
                case 1: cl_rows_dots<WT, B, 1>(op, ring, ctl, xcur, D, red, rt, t0, t1, tw); break;
                case 2: cl_rows_dots<WT, B, 2>(op, ring, ctl, xcur, D, red, rt, t0, t1, tw); break;
                case 3: cl_rows_dots<WT, B, 3>(op, ring, ctl, xcur, D, red, rt, t0, t1, tw); break;
                case 4: cl_rows_dots<WT, B, 4>(op, ring, ctl, xcur, D, red, rt, t0, t1, tw); break;
                case 5: if constexpr (B <= 1) cl_rows_dots<WT, B, 5>(op, ring, ctl, xcur, D, red, rt, t0, t1, tw); break;
                case 6: if constexpr (B <= 1) cl_rows_dots<WT, B, 6>(op, ring, ctl, xcur, D, red, rt, t0, t1, tw); break;
                case 7: if constexpr (B <= 1) cl_rows_dots<WT, B, 7>(op, ring, ctl, xcur, D, red, rt, t0, t1, tw); break;
                default: if constexpr (B <= 1) cl_rows_dots<WT, B, 8>(op, ring, ctl, xcur, D, red, rt, t0, t1, tw); break;
            }
            CL_CLK(2);
            if (cl_rsync_or(CL_ROLE_ROWS, ctl.dead)) {
                ctl.dead = true;
                return;
            }
            CL_CLK(3);
            if (stats_pending) {
                // combine the two shifted sums exactly (common shift C = the first warp's):
                //   sum(x - C) = s1 + n (c - C),  sum((x - C)^2) = s2 + 2 (c - C) s1 + n (c - C)^2
                // then mean = C + S1/N and the biased variance S2/N - (S1/N)^2, eps inside the sqrt (src/ops/norm.rs:41-52)
#pragma unroll
                for (int b = 0; b < B; b++) {
                    const float C = stat[b * 4 + 3];
                    float S0 = 0.f, S1 = 0.f, S2 = 0.f;
#pragma unroll
                    for (int w2 = 0; w2 < 2; w2++) {
                        const float* sc4 = stat + (w2 * B + b) * 4;
                        const float dc = sc4[3] - C;
                        S0 += sc4[0];
                        S1 += fmaf(sc4[0], dc, sc4[1]);
                        S2 += fmaf(sc4[0] * dc, dc, fmaf(2.f * dc, sc4[1], sc4[2]));
                    }
                    const float rn = 1.f / S0;
                    const float m1 = S1 * rn;
                    mu[b] = C + m1;
                    rstd[b] = rsqrtf(fmaxf(fmaf(-m1, m1, S2 * rn), 0.f) + 1e-5f);
                }
                stats_pending = false;
            }
            const int nv = B * op.nq * 4;  // finished values of this op: all in the role's first warp
            float sfin = 0.f;
            if (rt < nv) {
                const int b = rt % B;
                sfin = cl_lds(mg_smem(red) + 4u * rt) + cl_lds(mg_smem(red) + 4u * (CL_NVMAX + rt));
                sfin = fmaf(rstd[b], fmaf(-mu[b], t1, sfin), t0);
            }
            if (type == CL_QKV && wr == 0) {
                // q | k | v values of this op -> every CTA of the cluster, 4 columns (one unit) per store
                static_assert(B == 1, "the gather below assumes one sequence");
                const int col = op.q0 * 4 + rt;  // index in the head's q | k | v
                if (KVS == 2 && col >= HD) sfin = __bfloat162float(__float2bfloat16_rn(sfin));  // k, v as the cache will hold them
                const int l4 = lane & ~3;
                const float v0 = __shfl_sync(RG_FULL_MASK, sfin, l4), v1 = __shfl_sync(RG_FULL_MASK, sfin, l4 + 1);
                const float v2 = __shfl_sync(RG_FULL_MASK, sfin, l4 + 2), v3 = __shfl_sync(RG_FULL_MASK, sfin, l4 + 3);
                if (rt < nv && (lane & 3) == 0) {
                    const uint32_t a_rx = mg_smem(m.rxQ + (size_t)fq.i * B * Q3 + col), a_bar = mg_smem(&m.barQ[fq.i]);
                    for (int d = 0; d < cs; d++) cl_send4(a_rx, a_bar, (uint32_t)d, v0, v1, v2, v3);
                }
            }
            if (rt < nv) {
                const int b = rt % B, jq = rt / B;
                const float s = sfin;
                const int col = op.q0 * 4 + jq;
                if (type == CL_QKV) {
                } else if (type == CL_FC1) {
                    cl_sts(mg_smem(m.hs + (size_t)fh.i * B * p.nh_cap + b * p.nh_cap + op.aux + jq), rg_apply_act(s, p.act));
                } else if (col < p.V) {  // CL_HEAD
                    p.logits[(size_t)b * p.V + col] = s;
                    if (s > my_best || (s == my_best && col < my_besti)) my_best = s, my_besti = col;
                }
            }
            if (wr == 0 && type == CL_FC1) cl_arrive_warp(&m.barH[fh.i]);
            if (op.flags & CL_LAST) {
                if (type == CL_QKV) fq.i ^= 1;
                else if (type == CL_FC1) fh.i ^= 1;
            }
            CL_CLK(4);
            if (type == CL_HEAD && (op.flags & CL_LAST)) {
                // this CTA's candidate of the pick: the best of the first warp's threads, published once the head role has
                // fenced the cache rows it appended during this token
                if (wr == 0) {
                    if (cid < p.H) cl_wait(&m.barA[fa.i], fa.parity(), ctl, limit);
                    fa.done();
                    for (int b = 0; b < B; b++) {
                        float bv = (lane % B) == b ? my_best : -INFINITY;
                        int bi = (lane % B) == b ? my_besti : 0x7fffffff;
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) {
                            const float ov = __shfl_xor_sync(RG_FULL_MASK, bv, o);
                            const int oi2 = __shfl_xor_sync(RG_FULL_MASK, bi, o);
                            if (ov > bv || (ov == bv && oi2 < bi)) bv = ov, bi = oi2;
                        }
                        if (lane == 0) {
                            mg_word* dst = p.buf_pick + ((size_t)op.aux * B + b) * 2;
                            mg_st_word(dst, tagbase + (uint32_t)p.L + 1u, __float_as_uint(bv));
                            mg_st_word(dst + 1, tagbase + (uint32_t)p.L + 1u, (uint32_t)bi);
                        }
                    }
                } else {
                    fa.done();
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Column-split product of roles 2 and 3: out[c] = sum_r vin[r] * W[r][c] over the op's rows, columns in 4-column
// units.  The 64 threads form nrg row groups of 64 / nrg threads; a thread owns units ucol, ucol + 64 / nrg, ...
// (at most NUT) and the rows of its group.  Returns the thread's partial sums and the bias of element groups rt and
// rt + 64 of the CTA's slice (it rides behind the last chunk).
// ---------------------------------------------------------------------------
template <typename WT, int B, int NUT>
__device__ __forceinline__ void cl_cols_dots(const cl_op& op, int U, int nrg, mg_cons& ring, mg_ctl& ctl, const float* vin, int vstride,
                                             int rt, int n4, float (&acc)[NUT][B][4], float4 (&bias4)[2], unsigned long long* tw = nullptr) {
    constexpr int UB = 4 * (int)sizeof(WT);
    const int tpg = CL_RT / nrg;
    const int ucol = rt % tpg, rg = rt / tpg;
#pragma unroll
    for (int a = 0; a < NUT; a++)
#pragma unroll
        for (int b = 0; b < B; b++)
#pragma unroll
            for (int c = 0; c < 4; c++) acc[a][b][c] = 0.f;
    // units of this thread: ucol + a * tpg; a unit past the end reads unit ucol again and its sums are dropped by the caller
    uint32_t uoff[NUT];
#pragma unroll
    for (int a = 0; a < NUT; a++) uoff[a] = (uint32_t)((ucol + a * tpg < U ? ucol + a * tpg : (ucol < U ? ucol : 0)) * UB);
    long long wcyc = 0;
    const uint32_t a_vin = mg_smem(vin);
    const int nchunks = op.nchunks, kc = op.kc, nrows = op.nq;
    for (int j = 0; j < nchunks; j++) {
        const long long c0 = tw ? clock64() : 0;
        const uint32_t slot = cl_ring_wait(ring, ctl);
        if (tw) wcyc += clock64() - c0;
        const int kb = j * kc;
        const int rows = min(kc, nrows - kb);
        // two rows per step, all loads of the step first (see cl_rows_dots)
        for (int r = rg; r < rows; r += 2 * nrg) {
            const bool two = r + nrg < rows;
            const int r1 = two ? r + nrg : r;
            float hv[2][B], w[2][NUT][4];
#pragma unroll
            for (int b = 0; b < B; b++)
                hv[0][b] = cl_lds(a_vin + 4u * (b * vstride + kb + r)), hv[1][b] = cl_lds(a_vin + 4u * (b * vstride + kb + r1));
            const uint32_t rowp0 = slot + (uint32_t)(r * U) * UB, rowp1 = slot + (uint32_t)(r1 * U) * UB;
#pragma unroll
            for (int a = 0; a < NUT; a++) {
                cl_ldw4<WT>(rowp0 + uoff[a], w[0][a]);
                cl_ldw4<WT>(rowp1 + uoff[a], w[1][a]);
            }
            if (!two) {
#pragma unroll
                for (int b = 0; b < B; b++) hv[1][b] = 0.f;
            }
#pragma unroll
            for (int h = 0; h < 2; h++)
#pragma unroll
                for (int a = 0; a < NUT; a++)
#pragma unroll
                    for (int b = 0; b < B; b++)
#pragma unroll
                        for (int c = 0; c < 4; c++) acc[a][b][c] = fmaf(hv[h][b], w[h][a][c], acc[a][b][c]);
        }
        if (j == nchunks - 1) {
#pragma unroll
            for (int k = 0; k < 2; k++)
                if (rt + k * CL_RT < B * n4) bias4[k] = cl_lds4(slot + (uint32_t)(rows * U) * UB + 16u * ((rt + k * CL_RT) % n4));
        }
        if (tw && j < 2) tw[6 + j] = (unsigned long long)clock64();
        mg_ring_release(ring);
    }
    if (tw) tw[5] = (unsigned long long)wcyc;
}

// the same with the number of units per thread chosen at run time (the sums of the units beyond it are zero)
template <typename WT, int B>
__device__ __forceinline__ void cl_cols_dots_n(int nut, const cl_op& op, int U, int nrg, mg_cons& ring, mg_ctl& ctl, const float* vin,
                                               int vstride, int rt, int n4, float (&acc)[CL_NUT][B][4], float4 (&bias4)[2],
                                               unsigned long long* tw) {
#pragma unroll
    for (int a = 0; a < CL_NUT; a++)
#pragma unroll
        for (int b = 0; b < B; b++)
#pragma unroll
            for (int c = 0; c < 4; c++) acc[a][b][c] = 0.f;
#define CL_COLS_CASE(N)                                                                       \
    case N: {                                                                                 \
        float part[N][B][4];                                                                  \
        cl_cols_dots<WT, B, N>(op, U, nrg, ring, ctl, vin, vstride, rt, n4, part, bias4, tw); \
        _Pragma("unroll") for (int a = 0; a < N; a++) _Pragma("unroll") for (int b = 0; b < B; b++) \
            _Pragma("unroll") for (int c = 0; c < 4; c++) acc[a][b][c] = part[a][b][c];       \
    } break;
    switch (nut) {
        CL_COLS_CASE(1)
        CL_COLS_CASE(2)
        CL_COLS_CASE(3)
        CL_COLS_CASE(4)
        CL_COLS_CASE(5)
        CL_COLS_CASE(6)
        CL_COLS_CASE(7)
        default:
            CL_COLS_CASE(8)
    }
#undef CL_COLS_CASE
}

// ---------------------------------------------------------------------------
// role 2: attention over this CTA's slice of the context, merge over the cluster, out-projection partial
// ---------------------------------------------------------------------------
template <typename WT, int B, bool TRACE>
__device__ __forceinline__ void cl_role_head(const cl_params& p, const cl_mem& m, int nops, int me, int cid, mg_ctl& ctl, mg_cons& ring) {
    constexpr int VEC = mg_vec<WT>::N;  // K/V cache elements per 16 bytes
    constexpr int KVS = sizeof(WT);
    constexpr int NP = 8;  // rows of a lane group that are in flight together
    const int rt = ((threadIdx.x >> 5) >> 2) * 32 + (threadIdx.x & 31);  // warps 2 and 6
    const int lane = rt & 31, wr = rt >> 5;
    const int D = p.D, HD = p.hd, cs = p.cs, Q3 = 3 * p.hd;
    const uint32_t limit = p.spin_limit;
    const int e0 = p.su[me], ne = p.su[me + 1] - p.su[me], n4 = ne >> 2;
    cl_flip fx = {0, 0}, fq = {0, 0}, fr = {0, 0}, fa = {0, 0};
    // A CTA outside the head clusters has nothing for this role.  (It must not walk the tokens either: nothing would hold
    // it back, and a barrier that is signalled twice more before its waiter has looked reads as not signalled.)
    if (cid >= p.H) return;
    const int LPR = HD / VEC;   // lanes per cached row
    const int RPW = 32 / LPR;   // rows per warp per pass
    const int sub = lane % LPR, g2 = lane / LPR;
    const int rc = mg_attn_rows_per_chunk(HD, KVS);
    float* go = m.scr;                 // [2 * RPW][HD] attention output partials
    float* gml = m.scr + 2 * RPW * HD;  // [2][2 * RPW] partial max / sum
    for (int t = 0; t < p.n_steps; t++) {
        const int pos = p.pos0 + t;
        const uint32_t tagbase = (p.epoch0 + (uint32_t)t) * (uint32_t)(p.L + 1);
        bool appended = false;
        int xblock_i = 0;
        uint32_t xblock_par = 0;
        for (int oi = 0; oi < nops; oi++) {
            const cl_op& op = m.ops[oi];
            const int type = op.type;
            if (type == CL_QKV || type == CL_FC1 || type == CL_HEAD) {
                if (op.flags & CL_FIRST) {  // keep track of the input vector's buffer (the residual of partial 0 is read from it)
                    fx.i ^= 1;
                    if (type == CL_QKV) xblock_i = fx.i, xblock_par = fx.parity();
                    fx.ph ^= 1u << fx.i;
                }
                cl_ring_skip(ring, op.nchunks);
                continue;
            }
            if (type == CL_FC2) {
                cl_ring_skip(ring, op.nchunks);
                continue;
            }
            unsigned long long* tw = cl_tw<TRACE>(p, t, oi);
            CL_CLK(0);
            const uint32_t tag = tagbase + (uint32_t)op.layer + 1u;
            if (type == CL_ATTN) {
                // =================== attention of head cid, context slice `me` of cs ===================
                if (rt == 0) cl_expect(&m.barQ[fq.i], (uint32_t)(B * Q3 * 4));
                cl_wait(&m.barQ[fq.i], fq.parity(), ctl, limit);
                const float* sq = m.rxQ + (size_t)fq.i * B * Q3;
                fq.done();
                CL_CLK(1);
                const bool is_last = me == cs - 1;  // this CTA also takes the new row and appends it to the cache
                const int csz = (pos + cs - 1) / cs;
                const int r_lo = me * csz;
                const int arows = max(0, min(pos, r_lo + csz) - r_lo);
                const int nk = (arows + rc - 1) / rc;
                float* recs = m.rxR + (size_t)fr.i * cs * B * (HD + 4);
                const uint32_t a_go = mg_smem(go), a_gml = mg_smem(gml);
                for (int b = 0; b < B; b++) {
                    const uint32_t sqb = mg_smem(sq + b * Q3);
                    float qf[VEC];
#pragma unroll
                    for (int j = 0; j < VEC; j++) qf[j] = cl_lds(sqb + 4u * (sub * VEC + j));
                    float mx = -INFINITY, l = 0.f, acc[VEC];
#pragma unroll
                    for (int j = 0; j < VEC; j++) acc[j] = 0.f;
                    for (int j = 0; j < nk; j++) {
                        const int rows = min(rc, arows - j * rc);
                        // K rows and V rows of the same positions are consecutive chunks: both are held while the rows are
                        // walked in groups of NP passes of the two warps
                        const uint32_t kslot = cl_ring_wait(ring, ctl);
                        mg_cons vring = ring;
                        if (++vring.slot == vring.nslot) vring.slot = 0, vring.parity ^= 1u;
                        const uint32_t vslot = cl_ring_wait(vring, ctl);
                        for (int g0 = 0; g0 < rows; g0 += NP * 2 * RPW) {
                            float sreg[NP];
                            uint4 raw[NP];
#pragma unroll
                            for (int u = 0; u < NP; u++) {
                                const int rr = min(g0 + (u * 2 + wr) * RPW + g2, rows - 1);
                                raw[u] = cl_ldsu4(kslot + ((uint32_t)(rr * LPR + sub)) * 16);
                            }
#pragma unroll
                            for (int u = 0; u < NP; u++) {
                                float kf[VEC];
                                mg_vec<WT>::unpack(raw[u], kf);
                                float dot = 0.f;
#pragma unroll
                                for (int jj = 0; jj < VEC; jj++) dot = fmaf(qf[jj], kf[jj], dot);
                                sreg[u] = dot;
                            }
                            for (int o = LPR >> 1; o > 0; o >>= 1) {
#pragma unroll
                                for (int u = 0; u < NP; u++) sreg[u] += __shfl_xor_sync(RG_FULL_MASK, sreg[u], o);
                            }
                            float cm = -INFINITY;
#pragma unroll
                            for (int u = 0; u < NP; u++) {
                                const int rr = g0 + (u * 2 + wr) * RPW + g2;
                                sreg[u] = rr < rows ? sreg[u] * p.scale : -INFINITY;
                                cm = fmaxf(cm, sreg[u]);
                            }
                            const float mn = fmaxf(mx, cm);
                            const float msafe = mn == -INFINITY ? 0.f : mn;  // a group that has seen no row yet
                            const float corr = __expf(mx - msafe);           // exp(-inf) = 0 while mx is still -inf
                            mx = mn;
                            float psum = 0.f;
#pragma unroll
                            for (int u = 0; u < NP; u++) {
                                sreg[u] = __expf(sreg[u] - msafe);  // masked rows: exp(-inf) = 0
                                psum += sreg[u];
                            }
                            l = l * corr + psum;
#pragma unroll
                            for (int jj = 0; jj < VEC; jj++) acc[jj] *= corr;
#pragma unroll
                            for (int u = 0; u < NP; u++) {
                                const int rr = min(g0 + (u * 2 + wr) * RPW + g2, rows - 1);
                                raw[u] = cl_ldsu4(vslot + ((uint32_t)(rr * LPR + sub)) * 16);
                            }
#pragma unroll
                            for (int u = 0; u < NP; u++) {
                                float vf[VEC];
                                mg_vec<WT>::unpack(raw[u], vf);
#pragma unroll
                                for (int jj = 0; jj < VEC; jj++) acc[jj] = fmaf(sreg[u], vf[jj], acc[jj]);
                            }
                        }
                        mg_ring_release(ring);
                        mg_ring_release(ring);
                    }
                    // the new row's score (both warps compute it: cheaper than sharing it)
                    float s_new = -INFINITY;
                    if (is_last) {
                        float dot = 0.f;
                        for (int d = lane; d < HD; d += 32) dot = fmaf(cl_lds(sqb + 4u * d), cl_lds(sqb + 4u * (HD + d)), dot);
                        s_new = rg_warp_sum(dot) * p.scale;
                    }
                    CL_CLK(2);
                    const int ng = 2 * RPW;
                    const int grp = wr * RPW + g2;  // partial index
                    if (sub == 0) cl_sts(a_gml + 4u * grp, mx), cl_sts(a_gml + 4u * (ng + grp), l);
#pragma unroll
                    for (int j = 0; j < VEC; j++) cl_sts(a_go + 4u * (grp * HD + sub * VEC + j), acc[j]);
                    if (cl_rsync_or(CL_ROLE_HEAD, ctl.dead)) {
                        ctl.dead = true;
                        return;
                    }
                    // this CTA's record: running max, sum and un-normalised output over its slice (+ the new row), stored into
                    // the record array of every CTA of the cluster
                    // (loads first, arithmetic after: at most 8 partials)
                    float gm[8], gl[8];
#pragma unroll
                    for (int g = 0; g < 8; g++) {
                        gm[g] = g < ng ? cl_lds(a_gml + 4u * g) : -INFINITY;
                        gl[g] = g < ng ? cl_lds(a_gml + 4u * (ng + g)) : 0.f;
                    }
                    float M = s_new;
#pragma unroll
                    for (int g = 0; g < 8; g++) M = fmaxf(M, gm[g]);
                    float den = 0.f, wn = 0.f;
                    const bool any = M != -INFINITY;
                    if (any && is_last) wn = __expf(s_new - M), den = wn;
#pragma unroll
                    for (int g = 0; g < 8; g++) {
                        gm[g] = any ? __expf(gm[g] - M) : 0.f;  // weight of partial g (0 for a group that saw no row)
                        den = fmaf(gm[g], gl[g], den);
                    }
                    // record layout: [HD un-normalised outputs][max, sum, 0, 0]; 4 values per store
                    const uint32_t a_rec = mg_smem(recs + ((size_t)me * B + b) * (HD + 4)), a_bar = mg_smem(&m.barR[fr.i]);
                    for (int e0r = 0; e0r < HD; e0r += CL_RT) {
                        const int e = e0r + rt;
                        float num = 0.f;
                        if (e < HD) {
                            float gv[8];
#pragma unroll
                            for (int g = 0; g < 8; g++) gv[g] = g < ng ? cl_lds(a_go + 4u * (g * HD + e)) : 0.f;
                            if (is_last) num = wn * cl_lds(sqb + 4u * (2 * HD + e));
#pragma unroll
                            for (int g = 0; g < 8; g++) num = fmaf(gm[g], gv[g], num);
                        }
                        const int l4 = lane & ~3;
                        const float v0 = __shfl_sync(RG_FULL_MASK, num, l4), v1 = __shfl_sync(RG_FULL_MASK, num, l4 + 1);
                        const float v2 = __shfl_sync(RG_FULL_MASK, num, l4 + 2), v3 = __shfl_sync(RG_FULL_MASK, num, l4 + 3);
                        if (e < HD && (lane & 3) == 0)
                            for (int d = 0; d < cs; d++) cl_send4(a_rec + 4u * e, a_bar, (uint32_t)d, v0, v1, v2, v3);
                    }
                    if (rt == 0)
                        for (int d = 0; d < cs; d++) cl_send4(a_rec + 4u * HD, a_bar, (uint32_t)d, M, den, 0.f, 0.f);
                    if (B > 1 && cl_rsync_or(CL_ROLE_HEAD, ctl.dead)) {  // go / gml are reused by the next sequence
                        ctl.dead = true;
                        return;
                    }
                }
                CL_CLK(3);
                if (is_last) {
                    // append k, v of the new row to the cache (generic-proxy stores; fenced once per token, see below)
                    for (int i = rt; i < B * 2 * HD; i += CL_RT) {
                        const int b = i / (2 * HD), r2 = i - b * 2 * HD;
                        const int which = r2 / HD, d = r2 - which * HD;
                        const size_t row = (((size_t)b * p.H + cid) * p.C + pos) * HD;
                        unsigned char* base = (which == 0 ? p.kc : p.vc) + (size_t)op.layer * p.kv_layer_bytes;
                        const float v = sq[b * Q3 + (which + 1) * HD + d];
                        if (KVS == 4) reinterpret_cast<float*>(base)[row + d] = v;
                        else reinterpret_cast<__nv_bfloat16*>(base)[row + d] = __float2bfloat16_rn(v);
                    }
                    appended = true;
                }
                CL_CLK(4);
                continue;
            }
            // =================== out-projection partial: the head's rows of Wo, this CTA's slice of the columns ===================
            {
                if (rt == 0) cl_expect(&m.barR[fr.i], (uint32_t)(cs * B * (HD + 4) * 4));
                cl_wait(&m.barR[fr.i], fr.parity(), ctl, limit);
                const float* recs = m.rxR + (size_t)fr.i * cs * B * (HD + 4);
                fr.done();
                // records of all context slices of the head -> merged, normalised head output
                const uint32_t a_recs = mg_smem(recs), a_ovec = mg_smem(m.ovec);
                for (int e = rt; e < B * HD; e += CL_RT) {
                    const int b = e / HD, row = e - b * HD;
                    // (loads first, arithmetic after)
                    float rm[CL_MAX_CS], rl[CL_MAX_CS], rv[CL_MAX_CS];
#pragma unroll
                    for (int s = 0; s < CL_MAX_CS; s++) {
                        const uint32_t r0 = a_recs + 4u * (((s < cs ? s : 0) * B + b) * (HD + 4));
                        const float2 ml = cl_lds2(r0 + 4u * HD);
                        rm[s] = s < cs ? ml.x : -INFINITY, rl[s] = ml.y, rv[s] = cl_lds(r0 + 4u * row);
                    }
                    float M = -INFINITY;
#pragma unroll
                    for (int s = 0; s < CL_MAX_CS; s++) M = fmaxf(M, rm[s]);
                    float o = 0.f, den = 0.f;
#pragma unroll
                    for (int s = 0; s < CL_MAX_CS; s++) {
                        const float w = __expf(rm[s] - M);  // 0 for an empty slice and beyond the cluster
                        o = fmaf(w, rv[s], o);
                        den = fmaf(w, rl[s], den);
                    }
                    cl_sts(a_ovec + 4u * e, __fdividef(o, den));
                }
                if (cl_rsync_or(CL_ROLE_HEAD, ctl.dead)) {
                    ctl.dead = true;
                    return;
                }
                CL_CLK(1);
                const int U = op.nvalid >> 2;             // = n4
                const int nrg = U <= CL_RT / 2 ? 2 : 1;   // two row groups when half of the threads cover the columns
                const int nut = (U + CL_RT / nrg - 1) / (CL_RT / nrg);
                float acc[CL_NUT][B][4];
                float4 bias4[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};  // zero outside cluster 0
                cl_cols_dots_n<WT, B>(nut, op, U, nrg, ring, ctl, m.ovec, HD, rt, n4, acc, bias4, tw);
                CL_CLK(2);
                // the row groups' partial sums -> colred[group][b][unit]
                const int tpg = CL_RT / nrg, ucol = rt % tpg, rg = rt / tpg;
#pragma unroll
                for (int a = 0; a < CL_NUT; a++) {
                    const int u = ucol + a * tpg;
                    if (a < nut && u < U) {
#pragma unroll
                        for (int b = 0; b < B; b++)
                            cl_sts4(mg_smem(m.colred) + 16u * ((rg * B + b) * p.n4_cap + u), make_float4(acc[a][b][0], acc[a][b][1], acc[a][b][2], acc[a][b][3]));
                    }
                }
                if (cl_rsync_or(CL_ROLE_HEAD, ctl.dead)) {
                    ctl.dead = true;
                    return;
                }
                CL_CLK(3);
                if (cid == 0) cl_wait(&m.barX[xblock_i], xblock_par, ctl, limit);  // the block's input (complete long ago)
                for (int i = rt; i < B * n4; i += CL_RT) {
                    const int b = i / n4, ul = i - b * n4;
                    float4 s = cl_lds4(mg_smem(m.colred) + 16u * (b * p.n4_cap + ul));
                    if (nrg == 2) {
                        const float4 s1 = cl_lds4(mg_smem(m.colred) + 16u * ((B + b) * p.n4_cap + ul));
                        s.x += s1.x, s.y += s1.y, s.z += s1.z, s.w += s1.w;
                    }
                    const int col = e0 + 4 * ul;
                    const float4 bb = i < CL_RT ? bias4[0] : bias4[1];
                    s.x += bb.x, s.y += bb.y, s.z += bb.z, s.w += bb.w;
                    if (cid == 0) {  // the residual travels in partial 0
                        const float4 xb = cl_lds4(mg_smem(m.rxX + (size_t)xblock_i * B * D + b * D + col));
                        s.x += xb.x, s.y += xb.y, s.z += xb.z, s.w += xb.w;
                    }
                    if (!(cid == 0 && op.layer == p.withhold_layer)) {
                        mg_word* dst = p.buf_a + ((size_t)cid * B + b) * D + col;
                        cl_st_word2(dst, tag, s.x, s.y);
                        cl_st_word2(dst + 2, tag, s.z, s.w);
                    }
                }
                CL_CLK(4);
            }
        }
        // The appended rows are generic-proxy stores that later tokens read with bulk copies, possibly from another CTA of
        // the cluster: one proxy fence + gpu-scope fence per token, before this CTA publishes its pick, orders them all;
        // every CTA fences again after it has read the token's picks.
        if (appended) {
            mg_fence_proxy_async();
            __threadfence();
        }
        cl_arrive_warp(&m.barA[fa.i]);
        fa.i ^= 1;
    }
}

// ---------------------------------------------------------------------------
// role 3: FC2 rows of this CTA's hidden units -> partial sums over all D columns, reduce-scatter over the cluster
// ---------------------------------------------------------------------------
template <typename WT, int B, bool TRACE>
__device__ __forceinline__ void cl_role_cols(const cl_params& p, const cl_mem& m, int nops, int me, int cid, mg_ctl& ctl, mg_cons& ring) {
    constexpr int KVS = sizeof(WT);
    const int rt = ((threadIdx.x >> 5) >> 2) * 32 + (threadIdx.x & 31);  // warps 3 and 7
    const int D = p.D, cs = p.cs;
    const uint32_t limit = p.spin_limit;
    const int e0 = p.su[me], ne = p.su[me + 1] - p.su[me], n4 = ne >> 2;
    const int D4 = D >> 2;
    cl_flip fx = {0, 0}, fh = {0, 0}, ff = {0, 0};
    int xmid_i = 0;
    uint32_t xmid_par = 0;
    for (int t = 0; t < p.n_steps; t++) {
        const int pos = p.pos0 + t;
        const uint32_t tagbase = (p.epoch0 + (uint32_t)t) * (uint32_t)(p.L + 1);
        for (int oi = 0; oi < nops; oi++) {
            const cl_op& op = m.ops[oi];
            const int type = op.type;
            if (type == CL_ATTN) {
                cl_ring_skip(ring, cl_attn_chunks(p, pos, me, KVS, B));
                continue;
            }
            if (type != CL_FC2) {
                if ((op.flags & CL_FIRST) && type != CL_OPROJ) {
                    fx.i ^= 1;
                    if (type == CL_FC1) xmid_i = fx.i, xmid_par = fx.parity();
                    fx.ph ^= 1u << fx.i;
                }
                cl_ring_skip(ring, op.nchunks);
                continue;
            }
            unsigned long long* tw = cl_tw<TRACE>(p, t, oi);
            CL_CLK(0);
            const uint32_t tag = tagbase + (uint32_t)op.layer + 1u;
            cl_wait(&m.barH[fh.i], fh.parity(), ctl, limit);  // the activated hidden units of this CTA
            const float* hs = m.hs + (size_t)fh.i * B * p.nh_cap;
            fh.done();
            CL_CLK(1);
            float acc[CL_NUT][B][4];
            float4 bias4[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};  // zero outside cluster 0
            cl_cols_dots_n<WT, B>((D4 + CL_RT - 1) / CL_RT, op, D4, 1, ring, ctl, hs, p.nh_cap, rt, n4, acc, bias4, tw);
            CL_CLK(2);
            // reduce-scatter: unit u goes to the rank whose slice holds it
            {
                const uint32_t a_rx = mg_smem(m.rxF + (size_t)(ff.i * cs + me) * B * p.n4_cap * 4), a_barf = mg_smem(&m.barF[ff.i]);
                if (rt == 0) cl_expect(&m.barF[ff.i], (uint32_t)(cs * B * n4 * 16));
#pragma unroll
                for (int a = 0; a < CL_NUT; a++) {
                    const int u = rt + a * CL_RT;
                    if (u < D4) {
                        int d = 0;
                        while (d + 1 < cs && 4 * u >= p.su[d + 1]) d++;
                        const int ul = u - (p.su[d] >> 2);
#pragma unroll
                        for (int b = 0; b < B; b++)
                            cl_send4(a_rx + (uint32_t)((b * p.n4_cap + ul) * 16), a_barf, (uint32_t)d, acc[a][b][0], acc[a][b][1], acc[a][b][2],
                                     acc[a][b][3]);
                    }
                }
            }
            cl_wait(&m.barF[ff.i], ff.parity(), ctl, limit);
            CL_CLK(3);
            if (cid == 0) cl_wait(&m.barX[xmid_i], xmid_par, ctl, limit);  // the stage's input (complete long ago)
            for (int i = rt; i < B * n4; i += CL_RT) {
                const int b = i / n4, ul = i - b * n4;
                float s[4] = {0.f, 0.f, 0.f, 0.f};
                const uint32_t a_rxf = mg_smem(m.rxF);
                for (int r = 0; r < cs; r++) {
                    const float4 v = cl_lds4(a_rxf + 16u * (((ff.i * cs + r) * B + b) * p.n4_cap + ul));
                    s[0] += v.x, s[1] += v.y, s[2] += v.z, s[3] += v.w;
                }
                const int col = e0 + 4 * ul;
                const float4 bb = i < CL_RT ? bias4[0] : bias4[1];
                s[0] += bb.x, s[1] += bb.y, s[2] += bb.z, s[3] += bb.w;
                if (cid == 0) {  // the residual travels in partial 0
                    const float4 xb = cl_lds4(mg_smem(m.rxX + (size_t)xmid_i * B * D + b * D + col));
                    s[0] += xb.x, s[1] += xb.y, s[2] += xb.z, s[3] += xb.w;
                }
                mg_word* dst = p.buf_b + ((size_t)cid * B + b) * D + col;
                cl_st_word2(dst, tag, s[0], s[1]);
                cl_st_word2(dst + 2, tag, s[2], s[3]);
            }
            ff.done();
            CL_CLK(4);
            if (cl_rsync_or(CL_ROLE_COLS, ctl.dead)) {
                ctl.dead = true;
                return;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
template <typename WT, int B, bool TRACE>
__global__ void __launch_bounds__(MG_TOTAL_THREADS, 1) rg_cluster_loop_kernel(const cl_params p) {
    constexpr int KVS = sizeof(WT);  // the KV cache has the weight dtype
    constexpr int NWARP = MG_THREADS / 32;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x;
    const int cs = p.cs, me = (int)cl_rank(), cid = (int)cl_id();
    cl_mem m;
    cl_carve<B>(p, smem_raw, m);

    const int op0 = p.cta_off[cta];
    const int nops = p.cta_off[cta + 1] - op0;
    const int cd0 = p.cd_off[cta];
    const int ncd = p.cd_off[cta + 1] - cd0;
    for (int i = tid; i < nops * (int)(sizeof(cl_op) / 4); i += MG_TOTAL_THREADS)
        reinterpret_cast<int*>(m.ops)[i] = reinterpret_cast<const int*>(p.ops + op0)[i];
    for (int i = tid; i < ncd * (int)(sizeof(cl_cdesc) / 4); i += MG_TOTAL_THREADS)
        reinterpret_cast<int*>(m.cds)[i] = reinterpret_cast<const int*>(p.cds + cd0)[i];
    __syncthreads();
    if (tid == 0) {
        int nfc1 = 0;  // FC1 ops of a block: each hands its hidden values to the columns role with one arrival
        for (int i = 0; i < nops; i++)
            if (m.ops[i].type == CL_FC1 && m.ops[i].layer == 0) nfc1++;
        for (int i = 0; i < p.nslot; i++) mg_mbar_init(&m.full[i], 1), mg_mbar_init(&m.empty[i], 2);
        for (int i = 0; i < 2; i++) {
            // exchange barriers: the waiting role announces the bytes of a phase (one arrival), the data completes them
            mg_mbar_init(&m.barX[i], 1);
            mg_mbar_init(&m.barQ[i], 1);
            mg_mbar_init(&m.barR[i], 1);
            mg_mbar_init(&m.barF[i], 1);
            mg_mbar_init(&m.barH[i], nfc1 > 0 ? nfc1 : 1);
            mg_mbar_init(&m.barA[i], 2);                                       // both head-role warps, once per token
        }
        m.s_flags[0] = 0, m.s_flags[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    cl_sync_all();  // every CTA of the cluster has its barriers ready before anyone signals them

    if (warp == NWARP) {
        // =================== producer warp ===================
        if (lane == 0) cl_producer(p, m.cds, ncd, m.slots, m.full, m.empty, p.nslot, m.s_flags, m.s_flags + 1, KVS, B, cid, me);
        __syncwarp();
    } else {
        mg_ctl ctl;
        ctl.abort_flag = p.abort_flag;
        ctl.poll_sleep = (unsigned)p.poll_sleep;
        ctl.limit = p.spin_limit;
        ctl.dead = false;
        mg_cons ring;
        ring.slots = m.slots, ring.full = m.full, ring.empty = m.empty, ring.nslot = p.nslot, ring.slot = 0, ring.parity = 0;
        const int role = warp & 3;
        if (role == CL_ROLE_XCH) cl_role_exchange<WT, B, TRACE>(p, m, nops, me, cid, ctl);
        else if (role == CL_ROLE_ROWS) cl_role_rows<WT, B, TRACE>(p, m, nops, me, cid, ctl, ring);
        else if (role == CL_ROLE_HEAD) cl_role_head<WT, B, TRACE>(p, m, nops, me, cid, ctl, ring);
        else cl_role_cols<WT, B, TRACE>(p, m, nops, me, cid, ctl, ring);
        // a role that leaves early (a wait gave up somewhere) tells the producer to stop and drain
        if (ctl.dead || mg_ld_flag(p.abort_flag)) {
            *reinterpret_cast<volatile int*>(m.s_flags + 1) = 1;
            for (int i = 0; i < 64; i++) __nanosleep(1000);  // stores of other CTAs may still be on their way into this CTA
        } else if (cta == 0 && tid == 0) {
            *p.d_pos_next = p.pos0 + p.n_steps;
            *p.d_pos = p.pos0 + p.n_steps - 1;
        }
    }
    __syncthreads();  // joins the producer warp: no copy of ours is in flight past this point
    cl_sync_all();    // no CTA of the cluster leaves while another may still write into its shared memory
}


// ---------------------------------------------------------------------------
// packing: row-major [K][ldw] weights -> per-CTA streams in consumption order.
//  projections: [chunk][unit][row][unit bytes], the last chunk followed by the trailer
//      [additive term per column][LayerNorm mean coefficient per column];
//  column-split products (out-projection partial, FC2): the CTA's rows and columns as they are, [row][column],
//      followed by the bias of the CTA's slice of the output vector.
// Units or rows outside the matrix (padding, CTAs without a real share) are stored as zeros.
// ---------------------------------------------------------------------------
template <typename WT>
static __global__ void cl_pack_kernel(const WT* __restrict__ W, long long ldw, int Wrows, int Wcols, const float* __restrict__ bias,
                                      const float* __restrict__ gamma, const float* __restrict__ beta, const cl_op* __restrict__ ops,
                                      const int* __restrict__ cta_off, int type, int layer, unsigned char* __restrict__ dst, int D, int hd,
                                      int cs) {
    const int cta = blockIdx.x;
    for (int oi = cta_off[cta]; oi < cta_off[cta + 1]; oi++) {
        const cl_op op = ops[oi];
        if (op.type != type || op.layer != layer) continue;
        if (type == CL_FC2 || type == CL_OPROJ) {
            // rows [k0, k0 + nq), columns [q0, q0 + nvalid) as they are; then the bias of elements [aux, aux + K) of the output
            // vector, which only partial 0 (cluster 0) carries
            WT* out = reinterpret_cast<WT*>(dst + op.src);
            const size_t total = (size_t)op.nq * op.nvalid;
            for (size_t e = threadIdx.x; e < total; e += blockDim.x) {
                const int r = (int)(e / op.nvalid), c = (int)(e - (size_t)r * op.nvalid);
                out[e] = (op.k0 + r < Wrows && op.q0 + c < Wcols) ? W[(size_t)(op.k0 + r) * ldw + op.q0 + c] : mg_from_float<WT>(0.f);
            }
            float* tail = reinterpret_cast<float*>(dst + op.src + total * sizeof(WT));
            for (int e = threadIdx.x; e < op.K; e += blockDim.x) tail[e] = (cta / cs == 0) ? bias[op.aux + e] : 0.f;
            continue;
        }
        const int UB = op.uv * (int)sizeof(WT);
        auto column = [&](int q, int i, bool& ok) {
            int col = (op.q0 + q) * op.uv + i;
            if (type == CL_QKV) {
                const int which = col / hd;
                col = which * D + op.aux * hd + (col - which * hd);
            }
            ok = q < op.nvalid && col < Wcols;
            return col;
        };
        const int total = op.nq * op.K;
        for (int e = threadIdx.x; e < total; e += blockDim.x) {
            const int k = e / op.nq, q = e - k * op.nq;
            const int j = k / op.kc, r = k - j * op.kc;
            const int rows = min(op.kc, op.K - j * op.kc);
            WT* dstp = reinterpret_cast<WT*>(dst + op.src + ((size_t)j * op.nq * op.kc + (size_t)q * rows + r) * UB);
            const float gk = gamma != nullptr ? gamma[op.k0 + k] : 1.f;  // LayerNorm stage: store gamma_k * W_kn (exact when gamma is 1)
            for (int i = 0; i < op.uv; i++) {
                bool ok;
                const int col = column(q, i, ok);
                ok = ok && op.k0 + k < Wrows;
                const WT w = ok ? W[(size_t)(op.k0 + k) * ldw + col] : mg_from_float<WT>(0.f);
                dstp[i] = gamma != nullptr ? mg_from_float<WT>(gk * rg_to_float(w)) : w;
            }
        }
        // trailer: plain stage: bias, 0.  LayerNorm stage: sum_k beta_k W_kn + bias_n, sum_k gamma_k W_kn (as stored).
        float* tail = reinterpret_cast<float*>(dst + op.src + (size_t)op.nq * op.K * UB);
        const bool with_bias = true;
        for (int e = threadIdx.x; e < op.nq * op.uv; e += blockDim.x) {
            bool ok;
            const int col = column(e / op.uv, e % op.uv, ok);
            float add = (ok && with_bias) ? bias[col] : 0.f, coef = 0.f;
            if (gamma != nullptr && ok) {
                for (int k = 0; k < op.K; k++) {
                    const float w = rg_to_float(W[(size_t)k * ldw + col]);
                    add = fmaf(beta[k], w, add);
                    coef += rg_to_float(mg_from_float<WT>(gamma[k] * w));
                }
            }
            tail[e] = add;
            tail[op.nq * op.uv + e] = coef;
        }
    }
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
struct rg_cloop {
    int G = 0, cs = 0, ncl = 0;
    std::vector<cl_op> ops;
    std::vector<int> cta_off;
    std::vector<cl_cdesc> cds;
    std::vector<int> cd_off;
    cl_op* d_ops = nullptr;
    int* d_cta_off = nullptr;
    cl_cdesc* d_cds = nullptr;
    int* d_cd_off = nullptr;
    unsigned char* d_wpack = nullptr;
    size_t wpack_bytes = 0;
    unsigned long long* d_trace = nullptr;
    mg_word *buf_a = nullptr, *buf_b = nullptr, *buf_pick = nullptr, *buf_base = nullptr;
    size_t buf_bytes = 0;
    int* d_abort = nullptr;
    int max_ops = 0, max_cd = 0, nslot = 0;
    int su[CL_MAX_CS + 1] = {};
    int nh_cap = 0, n4_cap = 0, scr_bytes = 0, qkv_signals = 1;
    size_t smem_bytes = 0;
    int built_for_B = 0;
    bool unusable = false;  // no cluster shape of this GPU fits the model
    uint32_t spin_limit = MG_SPIN_LIMIT;
    int withhold_layer = -1;
    std::vector<void*> allocs;
};

static rg_status cl_dalloc(rg_cloop* g, void** p, size_t bytes) {
    cudaError_t e = cudaMalloc(p, bytes ? bytes : 16);
    if (e != cudaSuccess) {
        *p = nullptr;
        return rg_fail(RG_ERR_BACKEND, "Failed to allocate %zu bytes of CUDA memory: %s", bytes, cudaGetErrorString(e));
    }
    g->allocs.push_back(*p);
    return RG_OK;
}

static size_t cl_smem_bytes(const rg_gpt* m, const rg_cloop* g, int B, int nslot) {
    // mirrors cl_carve
    size_t s = (size_t)nslot * MG_SLOT_BYTES + 32 * 8;
    s += (size_t)g->max_ops * sizeof(cl_op) + (size_t)g->max_cd * sizeof(cl_cdesc) + 16;
    s += (size_t)2 * B * m->D * 4 + (size_t)2 * g->cs * B * g->n4_cap * 16 + (size_t)2 * B * g->n4_cap * 16;
    s += (size_t)2 * B * 3 * m->hd * 4 + (size_t)2 * g->cs * B * (m->hd + 4) * 4 + (size_t)2 * B * g->nh_cap * 4 + (size_t)B * m->hd * 4;
    s += (size_t)g->scr_bytes + 2 * 2 * (size_t)CL_NVMAX * 4 + 2 * 2 * 4 * MG_BMAX * 4 + (size_t)g->G * B * 2 * 4;
    s += 2 * (size_t)CL_RT * 4 + MG_BMAX * 4 + 16;
    return s + 128;
}

template <typename WT, int B, bool TRACE>
static cudaError_t cl_launch_t(rg_gpt* m, rg_cloop* g, cl_params& prm) {
    auto kern = rg_cluster_loop_kernel<WT, B, TRACE>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g->smem_bytes);
    if (e != cudaSuccess) return e;
    if (g->cs > 8) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(g->G), cfg.blockDim = dim3(MG_TOTAL_THREADS), cfg.dynamicSmemBytes = g->smem_bytes, cfg.stream = m->ctx->stream;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = g->cs, at[0].val.clusterDim.y = 1, at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeCooperative;  // all CTAs resident at once, or the launch fails
    at[1].val.cooperative = 1;
    // RG_B200_NO_COOP=1 drops the co-residency guarantee (a profiler that replays the kernel cannot launch it otherwise);
    // the bounded waits still end a launch whose clusters are not all resident
    const char* nc = getenv("RG_B200_NO_COOP");
    cfg.attrs = at, cfg.numAttrs = (nc && nc[0] == '1') ? 1 : 2;
    return cudaLaunchKernelEx(&cfg, kern, prm);
}

// How many clusters of `cs` CTAs (one CTA per SM, the kernel's full shared memory) can be resident at once.
template <typename WT>
static int cl_max_clusters(int cs) {
    auto kern = rg_cluster_loop_kernel<WT, 1, false>;
    const int smem = 227 * 1024;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return cudaGetLastError(), 0;
    if (cs > 8 && cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess)
        return cudaGetLastError(), 0;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(cs * 64), cfg.blockDim = dim3(MG_TOTAL_THREADS), cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = cs, at[0].val.clusterDim.y = 1, at[0].val.clusterDim.z = 1;
    cfg.attrs = at, cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) return cudaGetLastError(), 0;
    return n;
}

// Cluster shape: the head clusters need at least H clusters, and every CTA of a head cluster at least one q|k|v unit.
static bool cl_choose_shape(rg_gpt* m, rg_cloop* g) {
    const int HU = 3 * m->hd / 4;  // 4-column units of a head's q | k | v
    int cand[8] = {8, 6, 4, 5, 3, 2, 0, 0}, ncand = 6;
    if (const char* e = getenv("RG_B200_CLUSTER")) {
        const int v = atoi(e);
        if (v >= 1 && v <= CL_MAX_CS) cand[0] = v, ncand = 1;
    }
    for (int i = 0; i < ncand; i++) {
        const int cs = cand[i];
        if (cs > HU || m->D / 4 < cs) continue;
        int n = m->bf16 ? cl_max_clusters<__nv_bfloat16>(cs) : cl_max_clusters<float>(cs);
        if (const char* e = getenv("RG_B200_CLUSTERS_MAX")) n = std::min(n, atoi(e));
        if (n >= m->H) {
            g->cs = cs, g->ncl = n, g->G = n * cs;
            return true;
        }
    }
    return false;
}

// Build the per-CTA op lists and copy schedules for batch B.
static void cl_build_program(rg_gpt* m, rg_cloop* g, int B) {
    const int G = g->G, cs = g->cs, ws = (int)m->wsize;
    const int KVEC = m->bf16 ? 8 : 4;  // K/V cache elements per 16 bytes
    const int D = m->D, HD = m->hd, F = m->F;
    // 4-column units per row-split op: at most 32 accumulators per thread, and 256 rows of them + the trailer must fit a slot
    const int NQMAX = std::max(1, (m->bf16 ? 8 : 7) / B);
    std::vector<std::vector<cl_op>> per(G);
    {   // slices of a D-long vector over the ranks of a cluster, in groups of 4 elements
        const int U = D / 4, base = U / cs, extra = U % cs;
        g->su[0] = 0;
        for (int r = 0; r < cs; r++) g->su[r + 1] = g->su[r] + (base + (r < extra ? 1 : 0)) * 4;
        g->n4_cap = base + (extra ? 1 : 0);
        const int RPW = 32 / (HD / KVEC);
        g->scr_bytes = (2 * RPW * HD + 8 * RPW) * 4 + 64;
    }
    // row-split projection op over all K rows
    auto make_dots = [&](int type, int layer, int K, int q0, int nq, int aux) {
        cl_op op;
        memset(&op, 0, sizeof(op));
        op.type = type, op.layer = layer, op.K = K, op.q0 = q0, op.nq = nq, op.nvalid = nq, op.uv = 4, op.aux = aux;
        const int ub = 4 * ws;
        // rows per chunk: a multiple of 256, a single chunk when K is small; only the last chunk carries the trailer
        int kc = K;
        const int trailer = 2 * nq * 4 * 4;
        if (K > 256) {
            kc = std::max(256, (int)(MG_SLOT_BYTES / ((size_t)nq * ub)) / 256 * 256);
            kc = std::min(kc, (K + 255) / 256 * 256);
            auto last_rows = [&](int c) { return K % c == 0 ? c : K % c; };
            while (kc > 256 && (size_t)nq * last_rows(kc) * ub + trailer > MG_SLOT_BYTES) kc -= 256;
        }
        op.kc = std::max(kc, 1);
        op.nchunks = rg_cdiv(K, op.kc);
        return op;
    };
    auto add_split = [&](std::vector<cl_op>& list, int type, int layer, int K, int q0, int n, int aux, bool aux_counts) {
        // n units from q0 in ops of at most NQMAX units, sizes as even as possible
        const int nops = std::max(1, rg_cdiv(n, NQMAX));
        int done = 0;
        for (int i = 0; i < nops; i++) {
            const int take = n / nops + (i < n % nops ? 1 : 0);
            cl_op op = make_dots(type, layer, K, q0 + done, take, aux_counts ? aux + done * 4 : aux);
            op.flags = (i == 0 ? CL_FIRST : 0) | (i == nops - 1 ? CL_LAST : 0);
            list.push_back(op);
            done += take;
        }
    };
    // column-split product: rows [k0, k0 + rows) of the matrix, columns [c0, c0 + nc), bias of elements [t0, t0 + tn)
    auto make_cols = [&](int type, int layer, int k0, int rows, int c0, int nc, int t0, int tn) {
        cl_op op;
        memset(&op, 0, sizeof(op));
        op.type = type, op.layer = layer, op.k0 = k0, op.nq = rows, op.q0 = c0, op.nvalid = nc, op.aux = t0, op.K = tn, op.uv = 4;
        op.kc = std::max(1, (int)((MG_SLOT_BYTES - (size_t)tn * 4) / ((size_t)nc * ws)));
        op.kc = std::min(op.kc, rows);
        op.nchunks = rg_cdiv(rows, op.kc);
        op.flags = CL_FIRST | CL_LAST;
        return op;
    };
    const int HU = 3 * HD / 4;
    const int F4 = F / 4;
    const int f_base = F4 / G, f_extra = F4 % G;
    g->nh_cap = 4 * std::max(1, f_base + (f_extra ? 1 : 0));
    for (int l = 0; l < m->L; l++) {
        for (int c = 0; c < G; c++) {
            const int cl = c / cs, r = c % cs;
            const int s0 = g->su[r], sn = g->su[r + 1] - g->su[r];
            if (cl < m->H) {
                const int a0 = r * (HU / cs) + std::min(r, HU % cs), an = HU / cs + (r < HU % cs ? 1 : 0);
                add_split(per[c], CL_QKV, l, D, a0, an, cl, false);
                cl_op at;
                memset(&at, 0, sizeof(at));
                at.type = CL_ATTN, at.layer = l, at.flags = CL_FIRST | CL_LAST, at.aux = cl;
                per[c].push_back(at);
                // out-projection partial: the head's rows of Wo, this rank's slice of the columns
                per[c].push_back(make_cols(CL_OPROJ, l, cl * HD, HD, s0, sn, s0, sn));
            }
            // FC1 columns / FC2 rows of this CTA's hidden units (a CTA without a share works on zeros)
            int fq0 = c * f_base + std::min(c, f_extra), fn = f_base + (c < f_extra ? 1 : 0);
            if (fn == 0) fq0 = F4, fn = 1;
            add_split(per[c], CL_FC1, l, D, fq0, fn, 0, true);
            per[c].push_back(make_cols(CL_FC2, l, 4 * fq0, 4 * fn, 0, D, s0, sn));
        }
    }
    {   // LM head: 4-column units over all CTAs
        const int VU = rg_cdiv(m->V, 4), base = VU / G, extra = VU % G;
        for (int c = 0; c < G; c++) {
            int q0 = c * base + std::min(c, extra), n = base + (c < extra ? 1 : 0);
            if (n == 0) q0 = VU, n = 1;
            add_split(per[c], CL_HEAD, m->L, D, q0, n, c, false);
        }
    }
    g->qkv_signals = 0;
    for (int c = 0; c < cs; c++)
        for (const cl_op& op : per[c])
            if (op.type == CL_QKV && op.layer == 0) g->qkv_signals++;
    g->qkv_signals = std::max(1, g->qkv_signals);
    g->ops.clear();
    g->cta_off.assign(G + 1, 0);
    g->max_ops = 1;
    size_t off = 0;
    for (int c = 0; c < G; c++) {
        g->cta_off[c] = (int)g->ops.size();
        for (cl_op& op : per[c]) {
            if (op.type == CL_FC2 || op.type == CL_OPROJ) {
                op.src = (long long)off;
                off += (size_t)op.nq * op.nvalid * ws + (size_t)op.K * 4;
            } else if (op.type != CL_ATTN) {
                op.src = (long long)off;
                off += (size_t)op.nq * op.K * op.uv * ws + 2 * (size_t)op.nq * op.uv * 4;
            }
            off = (off + 15) & ~(size_t)15;
            g->ops.push_back(op);
        }
        g->max_ops = std::max(g->max_ops, (int)per[c].size());
    }
    g->cta_off[G] = (int)g->ops.size();
    g->wpack_bytes = off + 16;
    g->cds.clear();
    g->cd_off.assign(G + 1, 0);
    g->max_cd = 1;
    for (int c = 0; c < G; c++) {
        g->cd_off[c] = (int)g->cds.size();
        for (int oi = g->cta_off[c]; oi < g->cta_off[c + 1]; oi++) {
            const cl_op& op = g->ops[oi];
            if (op.type == CL_ATTN) {
                g->cds.push_back({(long long)op.layer, 0, 2});
            } else if (op.type == CL_FC2 || op.type == CL_OPROJ) {
                for (int j = 0; j < op.nchunks; j++) {
                    const int rows = std::min(op.kc, op.nq - j * op.kc);
                    int bytes = rows * op.nvalid * ws;
                    if (j == op.nchunks - 1) bytes += op.K * 4;
                    bytes = (bytes + 15) & ~15;
                    g->cds.push_back({op.src + (long long)j * op.kc * op.nvalid * ws, bytes, 0});
                }
            } else {
                for (int j = 0; j < op.nchunks; j++) {
                    const int rows = std::min(op.kc, op.K - j * op.kc);
                    const int ub = op.uv * ws;
                    int bytes = op.nq * rows * ub;
                    if (j == op.nchunks - 1) bytes += 2 * op.nq * op.uv * 4;
                    bytes = (bytes + 15) & ~15;
                    g->cds.push_back({op.src + (long long)j * op.nq * op.kc * ub, bytes, 0});
                }
            }
        }
        g->max_cd = std::max(g->max_cd, (int)g->cds.size() - g->cd_off[c]);
    }
    g->cd_off[G] = (int)g->cds.size();
}

template <typename WT>
static void cl_pack_all(rg_gpt* m, rg_cloop* g) {
    cudaStream_t s = m->ctx->stream;
    for (int l = 0; l < m->L; l++) {
        rg_layer& y = m->layers[l];
        const rg_linear* lins[4] = {&y.qkv, &y.o, &y.fc1, &y.fc2};
        const int types[4] = {CL_QKV, CL_OPROJ, CL_FC1, CL_FC2};
        const float* gam[4] = {y.ln1g, nullptr, y.ln2g, nullptr};
        const float* bet[4] = {y.ln1b, nullptr, y.ln2b, nullptr};
        for (int i = 0; i < 4; i++)
            cl_pack_kernel<WT><<<g->G, 256, 0, s>>>((const WT*)lins[i]->W, lins[i]->ldw, lins[i]->K, lins[i]->N, lins[i]->b, gam[i], bet[i],
                                                    g->d_ops, g->d_cta_off, types[i], l, g->d_wpack, m->D, m->hd, g->cs);
    }
    cl_pack_kernel<WT><<<g->G, 256, 0, s>>>((const WT*)m->head.W, m->head.ldw, m->head.K, m->head.N, m->head.b, m->lnfg, m->lnfb,
                                            g->d_ops, g->d_cta_off, CL_HEAD, m->L, g->d_wpack, m->D, m->hd, g->cs);
    m->ctx->launches += 4 * m->L + 1;
}

static rg_status cl_prepare(rg_gpt* m, int B) {
    rg_cloop* g = m->cloop;
    if (g->built_for_B == B) return RG_OK;
    if (g->unusable) return RG_ERR_UNSUPPORTED;
    RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
    for (void* p : g->allocs) cudaFree(p);
    g->allocs.clear();
    g->built_for_B = 0;
    if (!cl_choose_shape(m, g)) {
        g->unusable = true;
        return RG_ERR_UNSUPPORTED;
    }
    cl_build_program(m, g, B);
    g->nslot = 0;
    for (int ns = 6; ns >= 3; ns--) {
        const size_t need = cl_smem_bytes(m, g, B, ns);
        if (need <= 227 * 1024) {
            g->nslot = ns;
            g->smem_bytes = need;
            break;
        }
    }
    if (g->nslot == 0 || B * g->n4_cap > 2 * CL_RT) {
        g->unusable = true;
        return RG_ERR_UNSUPPORTED;
    }
    RG_TRY(cl_dalloc(g, (void**)&g->d_ops, g->ops.size() * sizeof(cl_op)));
    RG_TRY(cl_dalloc(g, (void**)&g->d_cta_off, (g->G + 1) * sizeof(int)));
    RG_TRY(cl_dalloc(g, (void**)&g->d_cds, g->cds.size() * sizeof(cl_cdesc)));
    RG_TRY(cl_dalloc(g, (void**)&g->d_cd_off, (g->G + 1) * sizeof(int)));
    RG_TRY(cl_dalloc(g, (void**)&g->d_wpack, g->wpack_bytes));
    RG_TRY(cl_dalloc(g, (void**)&g->d_trace, (size_t)g->G * g->max_ops * 72 * 8));
    RG_CUDA(cudaMemset(g->d_trace, 0, (size_t)g->G * g->max_ops * 72 * 8));
    RG_TRY(cl_dalloc(g, (void**)&g->d_abort, 16));
    const size_t wa = (size_t)m->H * B * m->D, wb = (size_t)g->ncl * B * m->D, wp = (size_t)g->G * B * 2;
    const size_t words = ((wa + 63) & ~(size_t)63) + ((wb + 63) & ~(size_t)63) + wp + 64;
    RG_TRY(cl_dalloc(g, (void**)&g->buf_base, words * 8));
    g->buf_bytes = words * 8;
    g->buf_a = g->buf_base;
    g->buf_b = g->buf_a + ((wa + 63) & ~(size_t)63);
    g->buf_pick = g->buf_b + ((wb + 63) & ~(size_t)63);
    RG_CUDA(cudaMemset(g->buf_base, 0, g->buf_bytes));
    RG_CUDA(cudaMemset(g->d_abort, 0, 16));
    RG_CUDA(cudaMemset(g->d_wpack, 0, g->wpack_bytes));
    m->epoch = 0;
    RG_CUDA(cudaMemcpy(g->d_ops, g->ops.data(), g->ops.size() * sizeof(cl_op), cudaMemcpyHostToDevice));
    RG_CUDA(cudaMemcpy(g->d_cta_off, g->cta_off.data(), (g->G + 1) * sizeof(int), cudaMemcpyHostToDevice));
    RG_CUDA(cudaMemcpy(g->d_cds, g->cds.data(), g->cds.size() * sizeof(cl_cdesc), cudaMemcpyHostToDevice));
    RG_CUDA(cudaMemcpy(g->d_cd_off, g->cd_off.data(), (g->G + 1) * sizeof(int), cudaMemcpyHostToDevice));
    if (m->bf16) cl_pack_all<__nv_bfloat16>(m, g);
    else cl_pack_all<float>(m, g);
    RG_CUDA(cudaGetLastError());
    RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
    g->built_for_B = B;
    if (getenv("RG_B200_DEBUG"))
        fprintf(stderr, "[rg_b200] cluster token loop: %d clusters of %d CTAs, %d ring slots, %zu bytes of shared memory, %d ops and %d copies per CTA at most, %.1f MB packed\n",
                g->ncl, g->cs, g->nslot, g->smem_bytes, g->max_ops, g->max_cd, g->wpack_bytes / 1e6);
    return RG_OK;
}

bool rg_cloop_supports(const rg_gpt* m, int B) {
    if (!m->cloop || !m->use_cloop || m->cloop->unusable || !m->cfg.causal || m->tp_size != 1) return false;
    // (at most 8 attention partials per CTA: 4 cached rows per warp and pass, i.e. head_dim >= 32 in f32, >= 64 in bf16)
    const bool hd_ok = (m->hd == 32 && !m->bf16) || m->hd == 64 || m->hd == 128;
    return B == 1 && hd_ok && m->D % 8 == 0 && m->D / 4 <= CL_NUT * CL_RT && m->F == 4 * m->D && m->H <= 64;
}

rg_status rg_cloop_create(rg_gpt* m) {
    rg_cloop_destroy(m);
    // The kernel of rg_mega.cu is the default form of the token loop (it is the faster one on the benchmark workload);
    // RG_B200_DECODE=cluster, or rg_debug_hook(4, 1), selects this one.
    const char* mode = getenv("RG_B200_DECODE");
    m->use_cloop = mode && strcmp(mode, "cluster") == 0;
    if (!m->cfg.causal) return RG_OK;
    m->cloop = new rg_cloop();
    if (const char* e = getenv("RG_B200_SPIN_LIMIT")) m->cloop->spin_limit = (uint32_t)std::max(1000, atoi(e));
    return RG_OK;
}

void rg_cloop_destroy(rg_gpt* m) {
    if (!m->cloop) return;
    for (void* p : m->cloop->allocs) cudaFree(p);
    delete m->cloop;
    m->cloop = nullptr;
}

void rg_cloop_debug(rg_gpt* m, int withhold_layer, unsigned spin_limit) {
    if (!m->cloop) return;
    if (withhold_layer != -2) m->cloop->withhold_layer = withhold_layer;
    if (spin_limit) m->cloop->spin_limit = spin_limit;
}

rg_status rg_cloop_run(rg_gpt* m, int B, size_t pos0, size_t n_steps) {
    if (n_steps == 0) return RG_OK;
    rg_cloop* g = m->cloop;
    rg_status st = cl_prepare(m, B);
    if (st != RG_OK) return st;
    // tags are (epoch * (L+1) + layer + 1) in 32 bits: start over long before they wrap
    if (((uint64_t)m->epoch + n_steps + 1) * (uint64_t)(m->L + 1) >= 0xfffffff0ull) {
        RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
        RG_CUDA(cudaMemset(g->buf_base, 0, g->buf_bytes));
        m->epoch = 0;
    }
    cl_params prm;
    memset(&prm, 0, sizeof(prm));
    prm.ops = g->d_ops, prm.cta_off = g->d_cta_off, prm.cds = g->d_cds, prm.cd_off = g->d_cd_off, prm.wpack = g->d_wpack;
    prm.trace = m->trace_on ? g->d_trace : nullptr;
    prm.wte = m->wte, prm.wpe = m->wpe, prm.ldt = m->ldt;
    prm.kc = (unsigned char*)m->kc, prm.vc = (unsigned char*)m->vc, prm.kv_layer_bytes = m->kv_layer_bytes;
    prm.buf_a = g->buf_a, prm.buf_b = g->buf_b, prm.buf_pick = g->buf_pick;
    prm.logits = m->logits, prm.tokens = m->tokens, prm.picks = m->picks, prm.d_pos = m->d_pos, prm.d_pos_next = m->d_pos_next;
    prm.abort_flag = g->d_abort;
    prm.V = m->V, prm.D = m->D, prm.L = m->L, prm.H = m->H, prm.hd = m->hd, prm.C = m->C, prm.F = m->F;
    prm.act = m->cfg.activation;
    prm.pos0 = (int)pos0, prm.n_steps = (int)n_steps, prm.epoch0 = m->epoch;
    prm.nslot = g->nslot, prm.max_ops = g->max_ops, prm.max_cd = g->max_cd, prm.n_pick_ctas = g->G;
    prm.cs = g->cs, prm.ncl = g->ncl;
    for (int i = 0; i <= CL_MAX_CS; i++) prm.su[i] = g->su[std::min(i, g->cs)];
    prm.nh_cap = g->nh_cap, prm.n4_cap = g->n4_cap, prm.scr_bytes = g->scr_bytes, prm.qkv_signals = g->qkv_signals;
    prm.spin_limit = g->spin_limit, prm.withhold_layer = g->withhold_layer;
    {
        const char* ps = getenv("RG_B200_POLL_SLEEP_NS");
        prm.poll_sleep = ps ? atoi(ps) : 0;
    }
    prm.scale = 1.f / sqrtf((float)m->hd);
    cudaError_t e;
    if (!m->bf16) e = prm.trace ? cl_launch_t<float, 1, true>(m, g, prm) : cl_launch_t<float, 1, false>(m, g, prm);
    else e = prm.trace ? cl_launch_t<__nv_bfloat16, 1, true>(m, g, prm) : cl_launch_t<__nv_bfloat16, 1, false>(m, g, prm);
    if (e == cudaErrorCooperativeLaunchTooLarge || e == cudaErrorLaunchOutOfResources || e == cudaErrorInvalidClusterSize) {
        cudaGetLastError();
        m->use_cloop = false;  // its clusters cannot be co-resident here: the caller uses another form of the step
        return RG_ERR_UNSUPPORTED;
    }
    if (e != cudaSuccess) return rg_fail(RG_ERR_BACKEND, "cluster token-loop kernel launch failed: %s", cudaGetErrorString(e));
    m->epoch += (uint32_t)n_steps;
    m->ctx->launches += 1;
    return RG_OK;
}

rg_status rg_cloop_check(rg_gpt* m) {
    rg_cloop* g = m->cloop;
    if (!g || !g->d_abort || !g->built_for_B) return RG_OK;
    int flag = 0;
    RG_CUDA(cudaMemcpyAsync(&flag, g->d_abort, sizeof(int), cudaMemcpyDeviceToHost, m->ctx->stream));
    RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
    if (flag) {
        cudaMemsetAsync(g->d_abort, 0, sizeof(int), m->ctx->stream);
        cudaMemsetAsync(g->buf_base, 0, g->buf_bytes, m->ctx->stream);
        m->epoch = 0;
        return rg_fail(RG_ERR_TIMEOUT, "a bounded wait inside the cluster token-loop kernel gave up; the step was abandoned");
    }
    return RG_OK;
}

// Rows of 12 like rg_mega_trace: cta, op index, type, layer, t0..t3 (ns: start, input ready, dot products done,
// outputs stored), four unused.
rg_status rg_cloop_trace(rg_gpt* m, unsigned long long* out, size_t cap_rows, size_t* n_rows) {
    rg_cloop* g = m->cloop;
    *n_rows = 0;
    if (!g || !g->built_for_B || !g->d_trace) return RG_OK;
    std::vector<unsigned long long> raw((size_t)g->G * g->max_ops * 72);
    RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
    RG_CUDA(cudaMemcpy(raw.data(), g->d_trace, raw.size() * 8, cudaMemcpyDeviceToHost));
    size_t n = 0;
    for (int c = 0; c < g->G; c++)
        for (int oi = g->cta_off[c]; oi < g->cta_off[c + 1]; oi++) {
            if (n >= cap_rows) break;
            const cl_op& op = g->ops[oi];
            const unsigned long long* t = &raw[((size_t)c * g->max_ops + (oi - g->cta_off[c])) * 72];
            unsigned long long* o = out + n * 12;
            o[0] = c, o[1] = oi - g->cta_off[c], o[2] = op.type, o[3] = op.layer;
            o[4] = t[0], o[5] = t[1], o[6] = t[2], o[7] = t[3], o[8] = t[4], o[9] = t[5], o[10] = t[6], o[11] = t[7];
            n++;
            for (int w = 0; w < 8 && n < cap_rows; w++) {  // SM cycle stamps of warp w: type 100 + w
                o = out + n * 12;
                o[0] = c, o[1] = oi - g->cta_off[c], o[2] = 100 + w, o[3] = op.layer;
                for (int i = 0; i < 8; i++) o[4 + i] = t[8 + w * 8 + i];
                n++;
            }
        }
    *n_rows = n;
    return RG_OK;
}

bool rg_cloop_active(const rg_gpt* m) { return m->cloop && m->cloop->built_for_B > 0 && m->use_cloop; }
