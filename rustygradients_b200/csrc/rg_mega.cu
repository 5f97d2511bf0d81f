// Persistent token-loop kernel: one cooperative launch runs n token steps of the
// KV-cache loop (src/wasm_api.rs:102-160 on a causal model) for up to 4
// sequences, with no kernel boundary between layers or tokens.
//
// Design (sm_100a, one CTA per SM, 256 threads):
//  * Every projection is split by OUTPUT COLUMNS only: a CTA owns a few 16-byte
//    column groups of a matrix and all K rows of them, so it produces finished
//    values (bias, activation and residual applied), never partial sums.
//  * The weights are re-packed at load into one stream per CTA, in the order the
//    CTA consumes them.  One elected thread moves that stream through a ring of
//    32 KB shared-memory slots with bulk asynchronous copies (cp.async.bulk +
//    mbarrier complete_tx).  The copies do not depend on activations, so they run
//    ahead across stage and token boundaries: HBM keeps streaming while a stage
//    waits for its input vector.
//  * Stages exchange finished vectors through global memory as 64-bit words
//    {value, tag}: the consumer polls the words it needs until their tag equals
//    the tag of the current (token, layer).  Data and flag travel in one store,
//    so there is no grid-wide barrier and no separate flag round trip.
//  * Attention of one (sequence, head) runs in one CTA: cached K rows then V rows
//    stream through the same ring (rows below the current position never change),
//    exact two-pass softmax in shared memory, the new row's k/v come straight from
//    the QKV stage and are appended to the cache.
//  * The residual stream lives with the CTA that owns its columns.
//  * Every wait (tagged words, mbarriers) is bounded: on expiry the CTA raises a
//    global flag, drains its own copies and returns; the host reports RG_ERR_TIMEOUT.
#include "rg_gpt.h"

#include <stdlib.h>
#include <string.h>

#include <algorithm>

#include "rg_loop_dev.cuh"


enum { MG_QKV = 0, MG_ATTN = 1, MG_OPROJ = 2, MG_FC1 = 3, MG_FC2 = 4, MG_HEAD = 5 };
enum { MG_FIRST = 1, MG_LAST = 2 };


#define MG_TP_MAX 16

struct mg_op {
    int type, layer;
    int nq, q0;  // projection: number of 16-byte column groups and the first one; attention: sequence b and head h
    int K, kc, nchunks;
    int flags;
    long long src;  // byte offset of this group's packed weights
    int aux;        // N=D stages: offset into the CTA's residual slice; head: rank of the CTA among head CTAs
    int uv;         // columns per column unit: a unit is 16 bytes of a weight row, or 8 bytes in the N = D stages
};

// One entry of a CTA's copy schedule for a token step.
struct mg_cdesc {
    long long src;  // kind 0: byte offset into the packed weights; 2: index of an attention op (its K/V slices)
    int bytes;
    int kind;
};

struct mg_params {
    const mg_op* ops;
    const int* cta_off;
    const mg_cdesc* cds;  // per-CTA copy schedule of one token step
    const int* cd_off;
    const unsigned char* wpack;
    unsigned long long* trace;  // optional [G][max_ops][4] timestamps of the last token step

    const void *wte, *wpe;
    long long ldt;
    unsigned char *kc, *vc;
    size_t kv_layer_bytes;
    mg_word *buf_qkv, *buf_a, *buf_xc, *buf_h, *buf_xe, *buf_pick;
    float* logits;
    uint32_t *tokens, *picks;
    int *d_pos, *d_pos_next;
    int* abort_flag;
    int V, D, L, H, hd, C, F;
    int act;
    int pos0, n_steps;
    uint32_t epoch0;
    int nslot, max_ops, max_cd, res_cap, n_pick_ctas;
    int poll_sleep;
    uint32_t spin_limit;  // iterations after which a wait gives up
    int withhold_layer;   // test hook: CTA 0 does not publish its q|k|v outputs of this block (-1: off)
    int S;  // CTAs that share one (sequence, head) in the attention stage, each a slice of the context
    float scale;
    // Tensor parallel: H, F and V above are THIS RANK's heads, hidden columns and vocabulary slice; D is the model
    // width; Dq = H * hd is the width of each of the q, k, v segments (= D without tensor parallelism).
    int Dq, XLEN, ldl, v0;  // XLEN: stride of the stage-input vectors (max(D, F)); ldl: row stride of `logits`
    int tp_rank, tp_size;
    int n_pick_of[MG_TP_MAX];  // head CTAs of every rank; rank r's picks start at r * pick_stride
    int pick_stride;
    mg_word* tp_xc[MG_TP_MAX];    // every rank's receive region of the out-projection partial sums: [tp_size][B][D] words
    mg_word* tp_xe[MG_TP_MAX];    // ... of the FC2 partial sums
    mg_word* tp_pick[MG_TP_MAX];  // ... of the picks: [tp_size][pick_stride][B][2]
};

struct rg_mega {
    int G = 0;
    std::vector<mg_op> ops;
    std::vector<int> cta_off;
    std::vector<mg_cdesc> cds;
    std::vector<int> cd_off;
    mg_op* d_ops = nullptr;
    int* d_cta_off = nullptr;
    mg_cdesc* d_cds = nullptr;
    int* d_cd_off = nullptr;
    int max_cd = 0;
    unsigned char* d_wpack = nullptr;
    size_t wpack_bytes = 0;
    unsigned long long* d_trace = nullptr;
    mg_word *buf_qkv = nullptr, *buf_a = nullptr, *buf_xc = nullptr, *buf_h = nullptr, *buf_xe = nullptr,
            *buf_pick = nullptr;
    size_t buf_bytes = 0;
    mg_word* buf_base = nullptr;
    int* d_abort = nullptr;
    int max_ops = 0, res_cap = 0, n_pick_ctas = 0, S = 1;
    int nslot = 0;
    size_t smem_bytes = 0;
    int built_for_B = 0;
    int place[6] = {0, 0, 0, 0, 0, 0};  // chosen position of every exchange vector inside its region
    bool placed = false;                // ... once mg_place_exchange has run
    uint32_t spin_limit = MG_SPIN_LIMIT;
    int withhold_layer = -1;
    std::vector<void*> allocs;
};


// The producer: walks the CTA's copy schedule for every token of the run, waits for
// a free slot, issues the copy.  K/V rows below the current position are final only
// once the consumers have passed the same attention op of the previous token (they
// append row pos-1 there); s_progress = token * nops + op index tells how far they are.
__device__ void mg_producer(const mg_params& p, const mg_cdesc* cd, int ncd, const mg_op* ops, int nops,
                            unsigned char* slots, uint64_t* full, uint64_t* empty, int nslot, volatile int* s_progress,
                            volatile int* s_dead, int kvsize) {
    int slot = 0;
    uint32_t parity = 0, issued = 0;
    bool stop = false;
    const int rc = mg_attn_rows_per_chunk(p.hd, kvsize);
    const size_t rb = (size_t)p.hd * kvsize;
    for (int tok = 0; tok < p.n_steps && !stop; tok++) {
        const int pos = p.pos0 + tok;
        for (int i = 0; i < ncd && !stop; i++) {
            const mg_cdesc d = cd[i];
            int nch = 1, r_lo = 0, arows = 0;
            const unsigned char *kbase = nullptr, *vbase = nullptr;
            if (d.kind == 2) {
                const mg_op& op = ops[(int)d.src];
                if (tok > 0) {
                    // cached rows may have been appended by another CTA during the previous token: wait until
                    // this CTA's consumers have finished that token (they fence after reading its picks)
                    const int need = tok * nops;
                    uint32_t spins = 0;
                    while (*s_progress < need) {
                        if (++spins > p.spin_limit || *s_dead) {
                            stop = true;
                            break;
                        }
                    }
                    if (stop) break;
                    mg_fence_proxy_async();
                }
                const int c = (pos + p.S - 1) / p.S;  // rows per split
                r_lo = op.aux * c;
                const int r_hi = min(pos, r_lo + c);
                arows = max(0, r_hi - r_lo);
                nch = 2 * ((arows + rc - 1) / rc);
                const size_t head_off = (((size_t)op.nq * p.H + op.q0) * p.C + r_lo) * rb + (size_t)op.layer * p.kv_layer_bytes;
                kbase = p.kc + head_off;
                vbase = p.vc + head_off;
            }
            for (int j = 0; j < nch; j++) {
                uint32_t spins = 0;
                while (!mg_mbar_try_wait(&empty[slot], parity ^ 1u)) {
                    if (++spins > p.spin_limit || *s_dead) {
                        stop = true;
                        break;
                    }
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
    if (stop) {
        // leaving early: wait (bounded) for the copies of ours that may still be in flight
        const uint32_t n = issued < (uint32_t)nslot ? issued : (uint32_t)nslot;
        for (uint32_t i = 0; i < n; i++) {
            if (--slot < 0) slot = nslot - 1, parity ^= 1u;
            uint32_t spins = 0;
            while (!mg_mbar_try_wait(&full[slot], parity) && ++spins < p.spin_limit) {
            }
        }
    }
}


// Dot products of one group (NQA active 16-byte column groups, all K rows) for B input
// vectors: streams the group's chunks out of the ring, then sums the per-thread partials
// over the CTA (halving exchange inside a warp, per-warp results to red[warp][value]).
// Value order: ((q * VEC + j) * B + b).  Returns through t0/t1 the two trailer values of
// the calling thread's output column (tid < B*NQA*VEC): additive term and LayerNorm
// mean coefficient.
template <typename WT, int B, int NQA, int UB, bool TRACE>
__device__ __forceinline__ void mg_group_dots(const mg_op& op, mg_cons& ring, mg_ctl& ctl, const float* xs, int XLEN,
                                              float* red, float& t0, float& t1, long long& wait_cyc,
                                              unsigned long long* tr_loop) {
    constexpr int UV = UB / (int)sizeof(WT);  // columns per unit
    constexpr int NV = B * NQA * UV;
    __builtin_assume(__isShared(xs)), __builtin_assume(__isShared(red));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    float acc[NV];
#pragma unroll
    for (int i = 0; i < NV; i++) acc[i] = 0.f;
    for (int j = 0; j < op.nchunks; j++) {
        long long c0 = 0;
        if constexpr (TRACE) c0 = clock64();
        const unsigned char* slot = mg_ring_wait(ring, ctl);
        if constexpr (TRACE) wait_cyc += clock64() - c0;
        const int kb = j * op.kc;
        const int rows = min(op.kc, op.K - kb);
        if (j == op.nchunks - 1 && tid < NV) {
            const float* tr = reinterpret_cast<const float*>(slot + (size_t)NQA * rows * UB);
            t0 = tr[tid / B];
            t1 = tr[NQA * UV + tid / B];
        }
#pragma unroll 2
        for (int r = tid; r < rows; r += MG_THREADS) {
            float xv[B];
#pragma unroll
            for (int b = 0; b < B; b++) xv[b] = xs[b * XLEN + kb + r];
#pragma unroll
            for (int q = 0; q < NQA; q++) {
                float w[UV];
                if constexpr (UB == 16) {
                    mg_vec<WT>::unpack(*reinterpret_cast<const uint4*>(slot + ((size_t)q * rows + r) * 16), w);
                } else {
                    const uint2 v = *reinterpret_cast<const uint2*>(slot + ((size_t)q * rows + r) * 8);
                    if constexpr (sizeof(WT) == 4) {
                        w[0] = __uint_as_float(v.x), w[1] = __uint_as_float(v.y);
                    } else {
                        w[0] = __uint_as_float(v.x << 16), w[1] = __uint_as_float(v.x & 0xffff0000u);
                        w[2] = __uint_as_float(v.y << 16), w[3] = __uint_as_float(v.y & 0xffff0000u);
                    }
                }
#pragma unroll
                for (int jj = 0; jj < UV; jj++)
#pragma unroll
                    for (int b = 0; b < B; b++)
                        acc[(q * UV + jj) * B + b] = fmaf(xv[b], w[jj], acc[(q * UV + jj) * B + b]);
            }
        }
        mg_ring_release(ring);
    }
    if (TRACE && tr_loop) *tr_loop = mg_globaltimer();
    int base = 0, count = 0;
    mg_halver<NV, 16>::run(acc, lane, base, count);
    if (mg_halver<NV, 16>::writer(lane)) {
#pragma unroll
        for (int i = 0; i < NV; i++)
            if (i < count) red[warp * NV + base + i] = acc[i];
    }
}

// Tensor parallel, row-split stages (out-projection, FC2): a rank holds a partial sum of element `elem`.  It goes,
// tagged, into every rank's receive region; then the same thread collects the tp_size partials of ITS element from its
// own region (`stride` words apart) and adds them in rank order, so every rank computes the same bits.  All words are
// requested together; only those not valid yet are read again.
// Bounded like every wait of the kernel.  Kept out of line: its 16 words in flight would otherwise cost the token loop
// registers it does not have.
__device__ __noinline__ float mg_tp_reduce(mg_word* const* regs, int rank, int T, size_t stride, size_t elem, uint32_t tag, float part,
                                           mg_ctl& ctl) {
    // this rank's partial sum, tagged, into slot [rank][elem] of every rank's region (plain stores; NVLink for the peers)
    const mg_word mine = ((mg_word)tag << 32) | __float_as_uint(part);
    for (int r = 0; r < T; r++)
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(regs[r] + (size_t)rank * stride + elem), "l"(mine) : "memory");
    const mg_word* own = regs[rank] + elem;
    float vals[MG_TP_MAX];
    uint32_t pending = (1u << T) - 1u, spins = 0;
    while (pending != 0) {
        mg_word w[MG_TP_MAX];
#pragma unroll
        for (int r = 0; r < MG_TP_MAX; r++)
            if (pending & (1u << r))
                asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w[r]) : "l"(own + (size_t)r * stride) : "memory");
#pragma unroll
        for (int r = 0; r < MG_TP_MAX; r++)
            if ((pending & (1u << r)) && (uint32_t)(w[r] >> 32) == tag) {
                vals[r] = __uint_as_float((uint32_t)w[r]);
                pending &= ~(1u << r);
            }
        if (pending != 0 && (++spins > ctl.limit || ((spins & 255u) == 0 && mg_ld_flag(ctl.abort_flag)))) {
            mg_give_up(ctl);
            break;
        }
    }
    float sum = 0.f;
#pragma unroll
    for (int r = 0; r < MG_TP_MAX; r++)
        if (r < T) sum += (pending & (1u << r)) ? 0.f : vals[r];
    return sum;
}

__device__ __noinline__ void mg_tp_publish_pick(mg_word* const* regs, int T, size_t slot, uint32_t tag, float best, int id) {
    const mg_word w0 = ((mg_word)tag << 32) | __float_as_uint(best), w1 = ((mg_word)tag << 32) | (uint32_t)id;
    for (int r = 0; r < T; r++) {
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(regs[r] + slot), "l"(w0) : "memory");
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(regs[r] + slot + 1), "l"(w1) : "memory");
    }
}

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
template <typename WT, int B, int NQ, bool TRACE, bool TP = false>
__global__ void __launch_bounds__(MG_TOTAL_THREADS, 1) rg_token_loop_kernel(const mg_params p) {
    constexpr int VEC = mg_vec<WT>::N;
    constexpr int KVS = sizeof(WT);  // the KV cache has the weight dtype
    constexpr int NOUT = B * NQ * VEC;  // most finished values a group can have
    constexpr int NWARP = MG_THREADS / 32;
    static_assert(NOUT <= MG_THREADS, "one thread per finished value");
    extern __shared__ __align__(128) unsigned char smem_raw[];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x;
    const int XLEN = p.XLEN;

    // ---- shared memory carve-up (must match mg_smem_bytes on the host) ----
    unsigned char* sp = smem_raw;
    unsigned char* slots = sp;
    sp += (size_t)p.nslot * MG_SLOT_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(sp);
    uint64_t* empty = full + 8;
    sp += 16 * 8;
    mg_op* ops = reinterpret_cast<mg_op*>(sp);
    sp += (size_t)p.max_ops * sizeof(mg_op);
    mg_cdesc* cds = reinterpret_cast<mg_cdesc*>(sp);
    sp += (size_t)p.max_cd * sizeof(mg_cdesc);
    float* xs = reinterpret_cast<float*>(sp);  // [B][XLEN] input vector of the current stage
    sp += (size_t)B * XLEN * 4;
    float* xemb = reinterpret_cast<float*>(sp);  // [B][D] token + position embedding of the step
    sp += (size_t)B * p.D * 4;
    float* go = reinterpret_cast<float*>(sp);  // [MG_THREADS * VEC] attention output partials
    sp += (size_t)MG_THREADS * VEC * 4;
    // xs, xemb and go are contiguous: the out-projection stage, which needs neither xemb nor go, lays the
    // attention records of all heads and its own input vectors over the three of them
    float* xres = reinterpret_cast<float*>(sp);  // [B][res_cap] this CTA's slice of the residual stream
    sp += (size_t)B * p.res_cap * 4;
    float* gml = reinterpret_cast<float*>(sp);  // [2][64] attention partial max / sum
    sp += 128 * 4;
    float* sqkv = reinterpret_cast<float*>(sp);  // q, k, v of the new row: 3 * 128
    sp += 3 * 128 * 4;
    float* red2 = reinterpret_cast<float*>(sp);  // [2][8][NOUT]: alternates per projection op (see below)
    sp += 2 * NWARP * NOUT * 4;
    float* scratch2 = reinterpret_cast<float*>(sp);  // [2][8][B][4] per-warp LayerNorm sums (count, s1, s2, shift)
    sp += 2 * NWARP * 4 * MG_BMAX * 4;
    float* bestv = reinterpret_cast<float*>(sp);  // [NOUT]
    sp += NOUT * 4;
    int* besti = reinterpret_cast<int*>(sp);  // [NOUT]
    sp += NOUT * 4;
    uint32_t* s_pick = reinterpret_cast<uint32_t*>(sp);  // [B]
    sp += MG_BMAX * 4;
    int* s_flags = reinterpret_cast<int*>(sp);  // [0] consumer progress, [1] dead
    sp += 4 * 4;
    float* awts = reinterpret_cast<float*>(sp);  // [256] normalised weights of the attention records
    sp += 256 * 4;
    float* pickbuf = reinterpret_cast<float*>(sp);  // [n_pick_ctas * B * 2]; tensor parallel: [tp_size][pick_stride][B][2]
    sp += ((size_t)(TP ? p.tp_size * p.pick_stride : p.n_pick_ctas) * B * 2 * 4 + 15) & ~(size_t)15;
    // tensor parallel: the ranks' receive regions and head-CTA counts, copied out of the kernel parameters (a parameter
    // array indexed by a run-time rank would be copied to local memory by every thread)
    sp = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(sp) + 15) & ~(uintptr_t)15);
    mg_word** s_tp = reinterpret_cast<mg_word**>(sp);  // [3][MG_TP_MAX]: out-projection partials, FC2 partials, picks
    int* s_npick = reinterpret_cast<int*>(sp + 3 * MG_TP_MAX * 8);  // [MG_TP_MAX]
    if constexpr (TP) {
        if (tid == 0) {
#pragma unroll
            for (int r = 0; r < MG_TP_MAX; r++)
                s_tp[r] = p.tp_xc[r], s_tp[MG_TP_MAX + r] = p.tp_xe[r], s_tp[2 * MG_TP_MAX + r] = p.tp_pick[r], s_npick[r] = p.n_pick_of[r];
        }
    }
    // every one of these is a shared-memory pointer: say so, so that ld.shared / st.shared are emitted (see mg_ring_wait)
    __builtin_assume(__isShared(slots)), __builtin_assume(__isShared(ops)), __builtin_assume(__isShared(cds));
    __builtin_assume(__isShared(xs)), __builtin_assume(__isShared(xemb)), __builtin_assume(__isShared(go));
    __builtin_assume(__isShared(xres)), __builtin_assume(__isShared(gml)), __builtin_assume(__isShared(sqkv));
    __builtin_assume(__isShared(red2)), __builtin_assume(__isShared(scratch2)), __builtin_assume(__isShared(bestv));
    __builtin_assume(__isShared(besti)), __builtin_assume(__isShared(s_pick)), __builtin_assume(__isShared(s_flags));
    __builtin_assume(__isShared(awts)), __builtin_assume(__isShared(pickbuf));

    const int op0 = p.cta_off[cta];
    const int nops = p.cta_off[cta + 1] - op0;
    const int cd0 = p.cd_off[cta];
    const int ncd = p.cd_off[cta + 1] - cd0;
    if (nops == 0) return;  // nothing depends on a CTA without work, and it depends on nothing
    for (int i = tid; i < nops * (int)(sizeof(mg_op) / 4); i += MG_TOTAL_THREADS)
        reinterpret_cast<int*>(ops)[i] = reinterpret_cast<const int*>(p.ops + op0)[i];
    for (int i = tid; i < ncd * (int)(sizeof(mg_cdesc) / 4); i += MG_TOTAL_THREADS)
        reinterpret_cast<int*>(cds)[i] = reinterpret_cast<const int*>(p.cds + cd0)[i];
    if (tid == 0) {
        for (int i = 0; i < p.nslot; i++) mg_mbar_init(&full[i], 1), mg_mbar_init(&empty[i], NWARP);
        s_flags[0] = -1, s_flags[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == NWARP) {
        // =================== producer warp ===================
        if (lane == 0)
            mg_producer(p, cds, ncd, ops, nops, slots, full, empty, p.nslot, s_flags, s_flags + 1, KVS);
        __syncwarp();
        __syncthreads();
        return;
    }

    // =================== consumer warps ===================
    mg_ctl ctl;
    ctl.abort_flag = p.abort_flag;
    ctl.poll_sleep = TRACE ? (unsigned)p.poll_sleep : 0u;
    ctl.limit = TRACE ? p.spin_limit : MG_SPIN_LIMIT;  // a run-time limit costs 3 % of the token time: instrumented build only
    ctl.dead = false;
    mg_cons ring;
    ring.slots = slots, ring.full = full, ring.empty = empty, ring.nslot = p.nslot, ring.slot = 0, ring.parity = 0;

    const WT* wte = static_cast<const WT*>(p.wte);
    const WT* wpe = static_cast<const WT*>(p.wpe);
    // residual slice of this CTA: column groups of the N = D stages (same in every layer)
    int res_q0 = 0, res_n = 0;
    for (int i = 0; i < nops; i++)
        if (ops[i].type == MG_OPROJ && ops[i].layer == 0) {
            if (res_n == 0) res_q0 = ops[i].q0 * ops[i].uv;  // first column of the slice
            res_n += ops[i].nq * ops[i].uv;
        }
    bool stats_pending = false;
    float mu[B], rstd[B];  // LayerNorm statistics of the current stage's input
#pragma unroll
    for (int b = 0; b < B; b++) mu[b] = 0.f, rstd[b] = 1.f;

    for (int t = 0; t < p.n_steps && !ctl.dead; t++) {
        const int pos = p.pos0 + t;
        const uint32_t tagbase = (p.epoch0 + (uint32_t)t) * (uint32_t)(p.L + 1);

        // ---- token + position embedding (src/models/gpt.rs:62-75), every CTA for itself ----
        for (int b = 0; b < B; b++) {
            const uint32_t tok = t == 0 ? p.tokens[(size_t)b * p.C + pos] : s_pick[b];
            for (int k = tid; k < p.D; k += MG_THREADS)
                xemb[b * p.D + k] = rg_to_float(wte[(size_t)tok * p.ldt + k]) + rg_to_float(wpe[(size_t)pos * p.ldt + k]);
        }
        mg_csync();
        for (int i = tid; i < B * res_n; i += MG_THREADS) {
            const int b = i / res_n, j = i - b * res_n;
            xres[b * p.res_cap + j] = xemb[b * p.D + res_q0 + j];
        }
        // thread-local best logit of the head stage (thread tid serves sequence tid % B)
        float my_best = -INFINITY;
        int my_besti = 0x7fffffff;

        // Deferred append of the new k, v row (held in sqkv since the attention op).  Generic-proxy stores that later
        // tokens read with bulk copies, possibly from another CTA: proxy fence + gpu-scope fence here, and every CTA
        // fences again after it has read the token's picks (which depend on this CTA's later stores).
        int append_layer = -1, append_b = 0, append_h = 0;
        auto flush_append = [&]() {
            if (append_layer < 0) return;
            const int HD = p.hd;
            const size_t row = (((size_t)append_b * p.H + append_h) * p.C + pos) * HD;
            WT* kdst = reinterpret_cast<WT*>(p.kc + (size_t)append_layer * p.kv_layer_bytes) + row;
            WT* vdst = reinterpret_cast<WT*>(p.vc + (size_t)append_layer * p.kv_layer_bytes) + row;
            for (int i = tid; i < 2 * HD; i += MG_THREADS) {
                const int which = i / HD, d = i - which * HD;
                const float v = sqkv[(which + 1) * 128 + d];
                WT* dst = which == 0 ? kdst : vdst;
                if (KVS == 4) reinterpret_cast<float*>(dst)[d] = v;
                else reinterpret_cast<__nv_bfloat16*>(dst)[d] = __float2bfloat16_rn(v);
            }
            mg_fence_proxy_async();
            __threadfence();
            append_layer = -1;
        };
        int prev_type = MG_ATTN;  // forces a barrier before the first op of the token
        for (int oi = 0; oi < nops; oi++) {
            const mg_op op = ops[oi];
            // A barrier at the start of an op is only needed when shared memory of the previous op could still be in
            // use: attention scratch (either side).  Between two projection ops (of one stage or of two) the barrier
            // after the previous dot products already ordered everything, and the partial-sum arrays alternate.
            if (op.type == MG_ATTN || prev_type == MG_ATTN) {
                if (mg_csync_or(ctl.dead)) ctl.dead = true;
            }
            if (ctl.dead) break;
            prev_type = op.type;
            if (tid == 0) *reinterpret_cast<volatile int*>(s_flags) = t * nops + oi;  // the producer reads this
            // The per-warp partial results alternate between two buffers: without a barrier between an op's input
            // fetch and its dot products, a warp could otherwise overwrite partials the previous op's epilogue still reads.
            float* red = red2 + (oi & 1) * (NWARP * NOUT);
            float* scratch = scratch2 + (oi & 1) * (NWARP * 4 * MG_BMAX);
            __builtin_assume(__isShared(red)), __builtin_assume(__isShared(scratch));
            const uint32_t tag = tagbase + (uint32_t)op.layer + 1u;
            const bool tracing = TRACE && p.trace != nullptr && t == p.n_steps - 1 && tid == 0;
            unsigned long long* tr = tracing ? p.trace + ((size_t)cta * p.max_ops + oi) * 8 : nullptr;
            long long wait_cyc = 0, poll_cyc = 0;
            if (tracing) tr[0] = mg_globaltimer();

            if (op.type == MG_ATTN) {
                flush_append();  // sqkv is about to be reused
                // =================== attention of (sequence b, head h) ===================
                // One CTA per (sequence, head).  Each warp owns every 8th group of cached rows and keeps its
                // own running softmax (max m, sum l, output o); K rows and V rows of the same positions arrive
                // as consecutive chunks.  The partials of all warps and the new row are merged at the end:
                // exactly softmax(q.K^T * scale).V with the row maximum subtracted (src/nn/attention.rs:78-94).
                const int b = op.nq, h = op.q0, HD = p.hd, S = p.S, sidx = op.aux;
                const int LPR = HD / VEC;   // lanes per cached row
                const int RPW = 32 / LPR;   // rows per warp per pass
                const int sub = lane % LPR, g2 = lane / LPR;
                const bool is_last = sidx == S - 1;  // this CTA also takes the new row and appends it to the cache
                const int csz = (pos + S - 1) / S;
                const int r_lo = sidx * csz;
                const int arows = max(0, min(pos, r_lo + csz) - r_lo);  // cached rows of this CTA's slice
                for (int i = tid; i < (is_last ? 3 : 1) * HD; i += MG_THREADS) {
                    const int which = i / HD, d = i - which * HD;
                    const mg_word* src = p.buf_qkv + (size_t)b * 3 * p.Dq + which * p.Dq + h * HD + d;
                    uint32_t spins = 0;
                    mg_word w = mg_ld_word(src);
                    while ((uint32_t)(w >> 32) != tag) {
                        if (++spins > ctl.limit || ((spins & 255u) == 0 && mg_ld_flag(ctl.abort_flag))) {
                            mg_give_up(ctl);
                            break;
                        }
                        w = mg_ld_word(src);
                    }
                    float v = __uint_as_float((uint32_t)w);
                    if (which > 0 && KVS == 2) v = __bfloat162float(__float2bfloat16_rn(v));  // what the cache will hold
                    sqkv[which * 128 + d] = v;
                }
                mg_csync();
                const int rc = mg_attn_rows_per_chunk(HD, KVS);  // = MG_ATTN_PASSES passes of the 8 warps
                const int nk = (arows + rc - 1) / rc;
                if (tracing) tr[1] = mg_globaltimer();
                float qf[VEC];
#pragma unroll
                for (int j = 0; j < VEC; j++) qf[j] = sqkv[sub * VEC + j];
                float m = -INFINITY, l = 0.f, acc[VEC];
#pragma unroll
                for (int j = 0; j < VEC; j++) acc[j] = 0.f;
                for (int j = 0; j < nk; j++) {
                    const int rows = min(rc, arows - j * rc);
                    float sreg[MG_ATTN_PASSES];
                    {   // scores of this warp's rows of the chunk: 8 independent rows in flight per lane group.
                        // Rows past the end are read from the last valid row and masked: no branches.
                        long long c0 = 0;
                        if constexpr (TRACE) c0 = clock64();
                        const unsigned char* slot = mg_ring_wait(ring, ctl);
                        if constexpr (TRACE) wait_cyc += clock64() - c0;
#pragma unroll
                        for (int u = 0; u < MG_ATTN_PASSES; u++) {
                            const int rr = min((u * NWARP + warp) * RPW + g2, rows - 1);
                            float kf[VEC];
                            mg_vec<WT>::unpack(*reinterpret_cast<const uint4*>(slot + ((size_t)rr * LPR + sub) * 16), kf);
                            float dot = 0.f;
#pragma unroll
                            for (int jj = 0; jj < VEC; jj++) dot = fmaf(qf[jj], kf[jj], dot);
                            sreg[u] = dot;
                        }
                        for (int o = LPR >> 1; o > 0; o >>= 1) {
#pragma unroll
                            for (int u = 0; u < MG_ATTN_PASSES; u++) sreg[u] += __shfl_xor_sync(RG_FULL_MASK, sreg[u], o);
                        }
                        mg_ring_release(ring);
                    }
                    float cm = -INFINITY;
#pragma unroll
                    for (int u = 0; u < MG_ATTN_PASSES; u++) {
                        const int rr = (u * NWARP + warp) * RPW + g2;
                        sreg[u] = rr < rows ? sreg[u] * p.scale : -INFINITY;
                        cm = fmaxf(cm, sreg[u]);
                    }
                    const float mn = fmaxf(m, cm);
                    const float msafe = mn == -INFINITY ? 0.f : mn;  // a group that has seen no row yet
                    const float corr = __expf(m - msafe);            // exp(-inf) = 0 while m is still -inf
                    m = mn;
                    float psum = 0.f;
#pragma unroll
                    for (int u = 0; u < MG_ATTN_PASSES; u++) {
                        sreg[u] = __expf(sreg[u] - msafe);  // masked rows: exp(-inf) = 0
                        psum += sreg[u];
                    }
                    l = l * corr + psum;
#pragma unroll
                    for (int jj = 0; jj < VEC; jj++) acc[jj] *= corr;
                    {
                        long long c0 = 0;
                        if constexpr (TRACE) c0 = clock64();
                        const unsigned char* slot = mg_ring_wait(ring, ctl);
                        if constexpr (TRACE) wait_cyc += clock64() - c0;
#pragma unroll
                        for (int u = 0; u < MG_ATTN_PASSES; u++) {
                            const int rr = min((u * NWARP + warp) * RPW + g2, rows - 1);
                            float vf[VEC];
                            mg_vec<WT>::unpack(*reinterpret_cast<const uint4*>(slot + ((size_t)rr * LPR + sub) * 16), vf);
#pragma unroll
                            for (int jj = 0; jj < VEC; jj++) acc[jj] = fmaf(sreg[u], vf[jj], acc[jj]);
                        }
                        mg_ring_release(ring);
                    }
                }
                // the new row's score (every warp computes it: cheaper than sharing it)
                float s_new = -INFINITY;
                if (is_last) {
                    float dot = 0.f;
                    for (int d = lane; d < HD; d += 32) dot = fmaf(sqkv[d], sqkv[128 + d], dot);
                    s_new = rg_warp_sum(dot) * p.scale;
                }
                const int grp = warp * RPW + g2;  // partial index, NWARP * RPW of them
                if (sub == 0) gml[grp] = m, gml[64 + grp] = l;
#pragma unroll
                for (int j = 0; j < VEC; j++) go[grp * HD + sub * VEC + j] = acc[j];
                if (tracing) tr[2] = mg_globaltimer();
                mg_csync();
                if (tid < HD) {
                    // this CTA's record: running max, sum and un-normalised output over its slice (+ the new row)
                    const int ng = NWARP * RPW;
                    float M = s_new;
                    for (int g = 0; g < ng; g++) M = fmaxf(M, gml[g]);
                    float num = 0.f, den = 0.f;
                    if (M != -INFINITY) {
                        if (is_last) {
                            const float wn = __expf(s_new - M);
                            num = wn * sqkv[256 + tid], den = wn;
                        }
                        for (int g = 0; g < ng; g++) {
                            const float w = __expf(gml[g] - M);  // 0 for a group that saw no row
                            num = fmaf(w, go[g * HD + tid], num);
                            den = fmaf(w, gml[64 + g], den);
                        }
                    }
                    mg_word* rec = p.buf_a + (((size_t)b * p.H + h) * S + sidx) * (HD + 2);
                    mg_st_word(rec + 2 + tid, tag, __float_as_uint(num));
                    if (tid == 0) {
                        mg_st_word(rec, tag, __float_as_uint(M));
                        mg_st_word(rec + 1, tag, __float_as_uint(den));
                    }
                }
                if (is_last) {
                    // k, v of the new row still have to be appended to the cache: not now, the out-projection is waiting
                    // for this CTA; flush_append() runs after the next projection's outputs are on their way
                    append_layer = op.layer, append_b = b, append_h = h;
                }
                if (tracing) tr[3] = mg_globaltimer(), tr[4] = (unsigned long long)wait_cyc, tr[5] = 0;
                continue;
            }

            // =================== projection stages ===================
            const bool ln_stage = op.type == MG_QKV || op.type == MG_FC1 || op.type == MG_HEAD;
            if (op.flags & MG_FIRST) {
                // the stage's input vector, complete, into xs.  For a LayerNorm stage the packed weights already
                // hold g_k W_kn; mean and 1/sqrt(var + eps) are applied to the finished dot products:
                //   LN(x).W + b = rstd * (sum_k x_k g_k W_kn - mean * sum_k g_k W_kn) + (sum_k beta_k W_kn + b_n)
                // (the two column sums are precomputed at load time and ride at the end of the group's weights).
                const mg_word* src =
                    op.type == MG_OPROJ ? p.buf_a : (op.type == MG_FC1 ? p.buf_xc : (op.type == MG_FC2 ? p.buf_h : p.buf_xe));
                const int n_in = op.type == MG_FC2 ? p.F : p.D;
                const uint32_t in_tag = (op.type == MG_QKV || op.type == MG_HEAD) ? tag - 1u : tag;  // previous block's output
                const bool local = op.type == MG_QKV && op.layer == 0;  // block 0 starts from the embedding
                long long c0 = 0;
                if constexpr (TRACE) c0 = clock64();
                if (ln_stage) {
                    // raw vector in (gamma is already folded into the packed weights), every thread its own elements.
                    // Statistics: per warp, shifted sums with the warp's first element as shift; the 8 (count, s1, s2,
                    // shift) tuples are combined exactly in the epilogue, after the barrier that follows the dot products.
#pragma unroll
                    for (int b = 0; b < B; b++) {
                        float* xr = xs + b * XLEN;
                        if (local) {
                            for (int i = tid; i < n_in; i += MG_THREADS) xr[i] = xemb[b * p.D + i];
                        } else {
                            mg_fetch_own<4, TRACE>(src + (size_t)b * n_in, n_in, in_tag, xr, ctl);
                        }
                        const float c = __shfl_sync(RG_FULL_MASK, tid < n_in ? xr[tid] : 0.f, 0);  // lane 0 of a warp always owns an element when n >= 256
                        float s0 = 0.f, s1 = 0.f, s2 = 0.f;
                        for (int i = tid; i < n_in; i += MG_THREADS) {
                            const float d = xr[i] - c;
                            s0 += 1.f;
                            s1 += d;
                            s2 = fmaf(d, d, s2);
                        }
                        s0 = rg_warp_sum(s0);
                        s1 = rg_warp_sum(s1);
                        s2 = rg_warp_sum(s2);
                        if (lane == 0) {
                            float* sc4 = scratch + (warp * B + b) * 4;
                            sc4[0] = s0, sc4[1] = s1, sc4[2] = s2, sc4[3] = c;
                        }
                    }
                    stats_pending = true;
                } else if (op.type == MG_OPROJ) {
                    // attention records of every (sequence, head, slice) -> merged, normalised head outputs
                    const int rec = p.hd + 2, nrec = B * p.H * p.S * rec;
                    mg_fetch<8, TRACE>(p.buf_a, nrec, in_tag, xs, ctl);
                    mg_csync();
                    if (tracing) tr[6] = mg_globaltimer();
                    float* vec = xs + ((nrec + 3) & ~3);
                    // normalised weight of every record, once per (sequence, head, slice): w_s = exp(m_s - M) / sum_s exp(m_s - M) l_s
                    const int nw = B * p.H * p.S;
                    // (4 lanes per (sequence, head): slices in parallel, max and sum by two shuffles each; S <= 4)
                    for (int i0 = 0; i0 < B * p.H; i0 += MG_THREADS / 4) {
                        const int i = i0 + (tid >> 2), sp2 = tid & 3;
                        const bool on = i < B * p.H && sp2 < p.S;
                        const float* r0 = xs + ((size_t)(on ? i : 0) * p.S + (on ? sp2 : 0)) * rec;
                        const float ms = on ? r0[0] : -INFINITY, ls = on ? r0[1] : 0.f;
                        float M = fmaxf(ms, __shfl_xor_sync(RG_FULL_MASK, ms, 1));
                        M = fmaxf(M, __shfl_xor_sync(RG_FULL_MASK, M, 2));
                        const float w = on ? __expf(ms - M) : 0.f;
                        float den = w * ls;
                        den += __shfl_xor_sync(RG_FULL_MASK, den, 1);
                        den += __shfl_xor_sync(RG_FULL_MASK, den, 2);
                        if (on && i * p.S + sp2 < 256) awts[i * p.S + sp2] = __fdividef(w, den);  // 0 for an empty slice
                    }
                    mg_csync();
                    const int hshift = 31 - __clz(p.hd);  // head_dim is 32, 64 or 128
#pragma unroll
                    for (int b = 0; b < B; b++) {
                        for (int k = tid; k < p.Dq; k += MG_THREADS) {
                            const int hh = k >> hshift, d = k & (p.hd - 1);
                            const int wi = (b * p.H + hh) * p.S;
                            const float* r0 = xs + (size_t)wi * rec + 2 + d;
                            float o = 0.f;
                            if (nw <= 256) {
                                for (int sp2 = 0; sp2 < p.S; sp2++) o = fmaf(awts[wi + sp2], r0[sp2 * rec], o);
                            } else {  // more records than the weight array holds: recompute the weights in place
                                const float* rr = xs + (size_t)wi * rec;
                                float M = -INFINITY, den = 0.f;
                                for (int sp2 = 0; sp2 < p.S; sp2++) M = fmaxf(M, rr[sp2 * rec]);
                                for (int sp2 = 0; sp2 < p.S; sp2++) {
                                    const float w = __expf(rr[sp2 * rec] - M);
                                    o = fmaf(w, r0[sp2 * rec], o);
                                    den = fmaf(w, rr[sp2 * rec + 1], den);
                                }
                                o = __fdividef(o, den);
                            }
                            vec[b * p.Dq + k] = o;  // element k stays with thread k mod 256: no barrier before the dot products
                        }
                    }
                } else {
#pragma unroll
                    for (int b = 0; b < B; b++) mg_fetch_own<16, TRACE>(src + (size_t)b * n_in, n_in, in_tag, xs + b * XLEN, ctl);
                    if (tracing) tr[6] = mg_globaltimer();
                }
                if constexpr (TRACE) poll_cyc += clock64() - c0;
            }
            if (tracing) tr[1] = mg_globaltimer();
            // ---- dot products of this group's columns over all K rows, summed over the CTA ----
            float t0 = 0.f, t1 = 0.f;
            const float* xin = xs;
            int xstride = XLEN;
            if (op.type == MG_OPROJ) xin = xs + ((B * p.H * p.S * (p.hd + 2) + 3) & ~3), xstride = p.Dq;
            __builtin_assume(__isShared(xin));
            if (op.uv == VEC) {
                switch (op.nq) {
                    case 1: mg_group_dots<WT, B, 1, 16, TRACE>(op, ring, ctl, xin, xstride, red, t0, t1, wait_cyc, tracing ? tr + 7 : nullptr); break;
                    case 2: if constexpr (NQ >= 2) mg_group_dots<WT, B, 2, 16, TRACE>(op, ring, ctl, xin, xstride, red, t0, t1, wait_cyc, tracing ? tr + 7 : nullptr); break;
                    case 3: if constexpr (NQ >= 3) mg_group_dots<WT, B, 3, 16, TRACE>(op, ring, ctl, xin, xstride, red, t0, t1, wait_cyc, tracing ? tr + 7 : nullptr); break;
                    case 4: if constexpr (NQ >= 4) mg_group_dots<WT, B, 4, 16, TRACE>(op, ring, ctl, xin, xstride, red, t0, t1, wait_cyc, tracing ? tr + 7 : nullptr); break;
                    case 5: if constexpr (NQ >= 5) mg_group_dots<WT, B, 5, 16, TRACE>(op, ring, ctl, xin, xstride, red, t0, t1, wait_cyc, tracing ? tr + 7 : nullptr); break;
                    default: if constexpr (NQ >= 6) mg_group_dots<WT, B, 6, 16, TRACE>(op, ring, ctl, xin, xstride, red, t0, t1, wait_cyc, tracing ? tr + 7 : nullptr); break;
                }
            } else {  // 8-byte units (N = D stages): half as many columns per unit, twice as many units allowed
                switch (op.nq) {
                    case 1: mg_group_dots<WT, B, 1, 8, TRACE>(op, ring, ctl, xin, xstride, red, t0, t1, wait_cyc, tracing ? tr + 7 : nullptr); break;
                    case 2: mg_group_dots<WT, B, 2, 8, TRACE>(op, ring, ctl, xin, xstride, red, t0, t1, wait_cyc, tracing ? tr + 7 : nullptr); break;
                    case 3: if constexpr (NQ >= 2) mg_group_dots<WT, B, 3, 8, TRACE>(op, ring, ctl, xin, xstride, red, t0, t1, wait_cyc, tracing ? tr + 7 : nullptr); break;
                    case 4: if constexpr (NQ >= 2) mg_group_dots<WT, B, 4, 8, TRACE>(op, ring, ctl, xin, xstride, red, t0, t1, wait_cyc, tracing ? tr + 7 : nullptr); break;
                    case 5: if constexpr (NQ >= 3) mg_group_dots<WT, B, 5, 8, TRACE>(op, ring, ctl, xin, xstride, red, t0, t1, wait_cyc, tracing ? tr + 7 : nullptr); break;
                    default: if constexpr (NQ >= 3) mg_group_dots<WT, B, 6, 8, TRACE>(op, ring, ctl, xin, xstride, red, t0, t1, wait_cyc, tracing ? tr + 7 : nullptr); break;
                }
            }
            if (mg_csync_or(ctl.dead)) ctl.dead = true;  // uniform from here on
            if (stats_pending && tid < NOUT) {
                // combine the per-warp shifted sums exactly (common shift C = the first warp's):
                //   sum(x - C) = s1 + n (c - C),  sum((x - C)^2) = s2 + 2 (c - C) s1 + n (c - C)^2
                // then mean = C + S1/N and the biased variance S2/N - (S1/N)^2, eps inside the sqrt (src/ops/norm.rs:41-52)
#pragma unroll
                for (int b = 0; b < B; b++) {
                    const float C = scratch[(0 * B + b) * 4 + 3];
                    float S0 = 0.f, S1 = 0.f, S2 = 0.f;
#pragma unroll
                    for (int w2 = 0; w2 < NWARP; w2++) {
                        const float* sc4 = scratch + (w2 * B + b) * 4;
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
            }
            stats_pending = false;
            if (tracing) tr[2] = mg_globaltimer();
            const int nv = B * op.nq * op.uv;
            if (tid < nv) {
                const int b = tid % B, jq = tid / B;
                float s = 0.f;
#pragma unroll
                for (int w2 = 0; w2 < NWARP; w2++) s += red[w2 * nv + tid];
                const int col = op.q0 * op.uv + jq;
                if constexpr (TP) {
                    // Row-split stages (out-projection, FC2): this rank holds a partial sum.  It goes, tagged, into
                    // every rank's receive region (plain stores, NVLink for the peers); then the same thread collects
                    // the tp_size partials of ITS element from its own region and adds them in rank order, so every
                    // rank computes the same bits.  Bias and residual are added once, after the sum.
                    if (op.type == MG_OPROJ || op.type == MG_FC2) {
                        s = mg_tp_reduce(s_tp + (op.type == MG_OPROJ ? 0 : MG_TP_MAX), p.tp_rank, p.tp_size, (size_t)B * p.D,
                                         (size_t)b * p.D + col, tag, s, ctl);
                    }
                }
                s = ln_stage ? fmaf(rstd[b], fmaf(-mu[b], t1, s), t0) : s + t0;
                if (op.type == MG_QKV) {
                    if (!(TRACE && cta == 0 && op.layer == p.withhold_layer))
                        mg_st_word(p.buf_qkv + (size_t)b * 3 * p.Dq + col, tag, __float_as_uint(s));
                } else if (op.type == MG_OPROJ) {
                    const float v = xres[b * p.res_cap + op.aux + jq] + s;
                    xres[b * p.res_cap + op.aux + jq] = v;
                    mg_st_word(p.buf_xc + (size_t)b * p.D + col, tag, __float_as_uint(v));
                } else if (op.type == MG_FC1) {
                    const float v = rg_apply_act(s, p.act);
                    mg_st_word(p.buf_h + (size_t)b * p.F + col, tag, __float_as_uint(v));
                } else if (op.type == MG_FC2) {
                    const float v = xres[b * p.res_cap + op.aux + jq] + s;
                    xres[b * p.res_cap + op.aux + jq] = v;
                    mg_st_word(p.buf_xe + (size_t)b * p.D + col, tag, __float_as_uint(v));
                } else if (col < p.V) {  // MG_HEAD
                    p.logits[(size_t)b * p.ldl + col] = s;
                    const int id = p.v0 + col;
                    if (s > my_best || (s == my_best && id < my_besti)) my_best = s, my_besti = id;
                }
            }
            if (tracing) tr[3] = mg_globaltimer(), tr[4] = (unsigned long long)wait_cyc, tr[5] = (unsigned long long)poll_cyc;
            flush_append();  // off the critical path: this op's outputs are already stored
            if (op.type == MG_HEAD && (op.flags & MG_LAST)) {
                // this CTA's best logit per sequence -> its slot of the pick buffer
                if (tid < NOUT) bestv[tid] = my_best, besti[tid] = my_besti;
                mg_csync();
                if (tid < B) {
                    float bv = -INFINITY;
                    int bi = 0x7fffffff;
                    for (int i = tid; i < NOUT; i += B) {  // thread i served sequence i % B
                        const float v = bestv[i];
                        const int ix = besti[i];
                        if (v > bv || (v == bv && ix < bi)) bv = v, bi = ix;
                    }
                    const uint32_t ptag = tagbase + (uint32_t)p.L + 1u;
                    if constexpr (TP) {  // every rank needs every rank's candidates
                        mg_tp_publish_pick(s_tp + 2 * MG_TP_MAX, p.tp_size, (((size_t)p.tp_rank * p.pick_stride + op.aux) * B + tid) * 2, ptag,
                                           bv, bi);
                    } else {
                        mg_word* dst = p.buf_pick + ((size_t)op.aux * B + tid) * 2;
                        mg_st_word(dst, ptag, __float_as_uint(bv));
                        mg_st_word(dst + 1, ptag, (uint32_t)bi);
                    }
                }
            }
        }
        if (ctl.dead) break;
        flush_append();

        // ---- greedy pick (top_k = 1 of src/wasm_api.rs:120-156): best over all CTAs, lowest index on ties ----
        if constexpr (TP) {
            for (int r = 0; r < p.tp_size; r++)
                mg_fetch<8, TRACE, true>(s_tp[2 * MG_TP_MAX + p.tp_rank] + (size_t)r * p.pick_stride * B * 2, s_npick[r] * B * 2,
                                         tagbase + (uint32_t)p.L + 1u, pickbuf + (size_t)r * p.pick_stride * B * 2, ctl);
        } else {
            mg_fetch<8, TRACE>(p.buf_pick, p.n_pick_ctas * B * 2, tagbase + (uint32_t)p.L + 1u, pickbuf, ctl);
        }
        // everything any CTA stored before its pick (cache rows included) is ordered before what follows here
        __threadfence();
        mg_fence_proxy_async();
        mg_csync();
        if (warp < B) {  // warp b scans the candidates of sequence b
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            for (int rk = 0; rk < (TP ? p.tp_size : 1); rk++) {
                const float* pb = pickbuf + (size_t)rk * p.pick_stride * B * 2;
                const int n = TP ? s_npick[rk] : p.n_pick_ctas;
                for (int r = lane; r < n; r += 32) {
                    const float v = pb[(r * B + warp) * 2];
                    const int ix = (int)__float_as_uint(pb[(r * B + warp) * 2 + 1]);
                    if (v > bv || (v == bv && ix < bi)) bv = v, bi = ix;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(RG_FULL_MASK, bv, o);
                const int oi2 = __shfl_xor_sync(RG_FULL_MASK, bi, o);
                if (ov > bv || (ov == bv && oi2 < bi)) bv = ov, bi = oi2;
            }
            if (lane == 0) {
                if (bi == 0x7fffffff) bi = 0;
                s_pick[warp] = (uint32_t)bi;
                if (cta == 0) {
                    p.picks[warp] = (uint32_t)bi;
                    if (pos + 1 < p.C) p.tokens[(size_t)warp * p.C + pos + 1] = (uint32_t)bi;
                }
            }
        }
        mg_csync();
    }

    // ---- exit ----
    const bool died = mg_csync_or(ctl.dead);
    if (tid == 0) {
        if (died) *reinterpret_cast<volatile int*>(s_flags + 1) = 1;  // tells the producer to stop and drain
        else if (cta == 0) {
            *p.d_pos_next = p.pos0 + p.n_steps;
            *p.d_pos = p.pos0 + p.n_steps - 1;
        }
    }
    __syncthreads();  // joins the producer warp: no copy of ours is in flight past this point
}

// ---------------------------------------------------------------------------
// packing: row-major [K][ldw] -> per-CTA streams of [chunk][column group][row][16 bytes]
// ---------------------------------------------------------------------------
template <typename WT>
static __global__ void mg_pack_kernel(const WT* __restrict__ W, long long ldw, const float* __restrict__ bias, int N,
                                      const float* __restrict__ gamma, const float* __restrict__ beta,
                                      const mg_op* __restrict__ ops, const int* __restrict__ cta_off, int type, int layer,
                                      unsigned char* __restrict__ dst) {
    constexpr int VEC = 16 / sizeof(WT);
    const int cta = blockIdx.x;
    for (int oi = cta_off[cta]; oi < cta_off[cta + 1]; oi++) {
        const mg_op op = ops[oi];
        if (op.type != type || op.layer != layer) continue;
        const int total = op.nq * op.K;
        const int UB = op.uv * (int)sizeof(WT);  // 16 or 8 bytes per unit and row
        for (int e = threadIdx.x; e < total; e += blockDim.x) {
            const int k = e / op.nq, q = e - k * op.nq;
            const int j = k / op.kc, r = k - j * op.kc;
            const int rows = min(op.kc, op.K - j * op.kc);
            const WT* srcp = W + (size_t)k * ldw + (size_t)(op.q0 + q) * op.uv;
            WT* dstp = reinterpret_cast<WT*>(dst + op.src + ((size_t)j * op.nq * op.kc + (size_t)q * rows + r) * UB);
            const float gk = gamma != nullptr ? gamma[k] : 1.f;  // LayerNorm stage: store gamma_k * W_kn (exact when gamma is 1)
            for (int i = 0; i < op.uv; i++) dstp[i] = gamma != nullptr ? mg_from_float<WT>(gk * rg_to_float(srcp[i])) : srcp[i];
        }
        // trailer of the last chunk, per column of the group: [additive term][mean coefficient].
        // plain stage: bias, 0.  LayerNorm stage: sum_k beta_k W_kn + bias_n, sum_k gamma_k W_kn.
        float* tail = reinterpret_cast<float*>(dst + op.src + (size_t)op.nq * op.K * UB);
        for (int e = threadIdx.x; e < op.nq * op.uv; e += blockDim.x) {
            const int col = op.q0 * op.uv + e;
            float add = col < N ? bias[col] : 0.f, coef = 0.f;
            if (gamma != nullptr && col < N) {
                for (int k = 0; k < op.K; k++) {
                    const float w = rg_to_float(W[(size_t)k * ldw + col]);
                    add = fmaf(beta[k], w, add);
                    coef += rg_to_float(mg_from_float<WT>(gamma[k] * w));  // the folded weight as stored
                }
            }
            tail[e] = add;
            tail[op.nq * op.uv + e] = coef;
        }
    }
}

// ---------------------------------------------------------------------------
// host: program builder
// ---------------------------------------------------------------------------
static int mg_variant(int B) { return B == 1 ? 0 : (B == 2 ? 1 : (B == 4 ? 2 : -1)); }
static int mg_nq_for(bool bf16, int B) {
    if (!bf16) return B == 1 ? 6 : (B == 2 ? 4 : 2);
    return B == 1 ? 3 : (B == 2 ? 2 : 1);
}

static rg_status mg_dalloc(rg_mega* g, void** p, size_t bytes) {
    cudaError_t e = cudaMalloc(p, bytes ? bytes : 16);
    if (e != cudaSuccess) {
        *p = nullptr;
        return rg_fail(RG_ERR_BACKEND, "Failed to allocate %zu bytes of CUDA memory: %s", bytes, cudaGetErrorString(e));
    }
    g->allocs.push_back(*p);
    return RG_OK;
}

static size_t mg_smem_bytes(const rg_gpt* m, int B, int NQ, int nslot, int max_ops, int max_cd, int res_cap, int n_pick) {
    const int VEC = m->bf16 ? 8 : 4;
    const int NOUT = B * NQ * VEC;
    size_t s = (size_t)nslot * MG_SLOT_BYTES + 128 + (size_t)max_ops * sizeof(mg_op) + (size_t)max_cd * sizeof(mg_cdesc);
    s += (size_t)B * std::max(m->D, m->Fl) * 4 + (size_t)B * m->D * 4 + (size_t)B * res_cap * 4 + (size_t)MG_THREADS * VEC * 4 + 128 * 4 + 3 * 128 * 4;
    s += 2 * 8 * (size_t)NOUT * 4 + 2 * 8 * 4 * MG_BMAX * 4 + 2 * (size_t)NOUT * 4 + MG_BMAX * 4 + 16 + 256 * 4 + (((size_t)n_pick * B * 2 * 4 + 15) & ~(size_t)15);
    s += 16 + 3 * MG_TP_MAX * 8 + MG_TP_MAX * 4;  // tensor parallel: pointer table and head-CTA counts
    return s + 128;
}

// Build the per-CTA op lists for batch B (the column-group limit per op depends on B).
static void mg_build_program(rg_gpt* m, rg_mega* g, int B) {
    const int G = g->G, VEC = m->bf16 ? 8 : 4, NQ = mg_nq_for(m->bf16, B);
    std::vector<std::vector<mg_op>> per(G);
    // slices of the context per (sequence, head): as many as there are CTAs for, at most 4, and only as many as
    // let the out-projection stage hold all attention records plus its input vectors in the xs/xemb/go overlay
    // (a tensor-parallel rank builds the program of its own shard: Hl heads, Fl hidden columns, Vl vocabulary entries)
    const int H = m->Hl, Dq = m->Dl, F = m->Fl, XL = std::max(m->D, m->Fl);
    g->S = std::max(1, std::min(4, G / std::max(1, B * H)));
    if (const char* e = getenv("RG_B200_ATTN_SLICES")) g->S = std::max(1, std::min(g->S, atoi(e)));  // experiments: fewer slices
    while (g->S > 1 && (size_t)B * H * g->S * (m->hd + 2) + 4 + (size_t)B * Dq >
                           (size_t)B * XL + (size_t)B * m->D + (size_t)MG_THREADS * VEC)
        g->S--;
    int rot = 0;
    auto add_projection = [&](int type, int layer, int K, int N, int fixed_rot, int ub) {
        const int UV = ub / (int)m->wsize;         // columns per unit
        const int NQU = ub == 16 ? NQ : std::min(6, 2 * NQ);  // units per op
        const int Q = rg_cdiv(N, UV);
        const int base = Q / G, extra = Q % G;
        const int r0 = fixed_rot >= 0 ? fixed_rot : rot;
        const int active = std::min(G, Q);
        for (int r = 0; r < active; r++) {
            const int c = (r + r0) % G;
            int nq = base + (r < extra ? 1 : 0);
            int q = r * base + std::min(r, extra);
            int aux = 0;
            bool first = true;
            while (nq > 0) {
                mg_op op;
                memset(&op, 0, sizeof(op));
                op.type = type, op.layer = layer, op.K = K;
                op.nq = std::min(nq, NQU), op.q0 = q, op.uv = UV;
                // rows per chunk: a multiple of 256 so that row k of every chunk is handled by thread k mod 256
                // (the thread that fetched input element k); a single chunk when K is small.  Only the last
                // chunk carries the trailer (256 bytes set aside).
                int kc = K;
                if (K > 256) {
                    kc = std::max(256, (int)(MG_SLOT_BYTES / ((size_t)op.nq * ub)) / 256 * 256);
                    kc = std::min(kc, (K + 255) / 256 * 256);
                    auto last_rows = [&](int c) { return K % c == 0 ? c : K % c; };
                    while (kc > 256 && (size_t)op.nq * last_rows(kc) * ub + 256 > MG_SLOT_BYTES) kc -= 256;
                }
                op.kc = std::max(kc, 1);
                op.nchunks = rg_cdiv(K, op.kc);
                op.flags = first ? MG_FIRST : 0;
                op.aux = type == MG_HEAD ? r : aux;
                first = false;
                aux += op.nq * UV;
                q += op.nq, nq -= op.nq;
                if (nq == 0) op.flags |= MG_LAST;
                per[c].push_back(op);
            }
        }
        if (fixed_rot < 0) rot = (rot + extra) % G;
        return active;
    };
    const int extraD = rg_cdiv(m->D, VEC / 2) % G;
    rot = extraD;  // stages with N != D put their larger shares on other CTAs than the N = D stages do
    for (int l = 0; l < m->L; l++) {
        add_projection(MG_QKV, l, m->D, 3 * Dq, -1, 16);
        for (int pr = 0; pr < B * H * g->S; pr++) {  // one CTA per (sequence, head, slice), from the top of the grid down
            mg_op op;
            memset(&op, 0, sizeof(op));
            const int bh = pr / g->S;
            op.type = MG_ATTN, op.layer = l, op.nq = bh / H, op.q0 = bh % H, op.aux = pr % g->S, op.K = g->S;
            op.flags = MG_FIRST | MG_LAST;
            per[(G - 1) - (pr % G)].push_back(op);
        }
        add_projection(MG_OPROJ, l, Dq, m->D, 0, 8);
        add_projection(MG_FC1, l, m->D, F, -1, 16);
        add_projection(MG_FC2, l, F, m->D, 0, 8);
    }
    g->n_pick_ctas = add_projection(MG_HEAD, m->L, m->D, m->Vl, -1, 16);
    g->ops.clear();
    g->cta_off.assign(G + 1, 0);
    g->max_ops = 1;
    g->res_cap = VEC;
    size_t off = 0;
    for (int c = 0; c < G; c++) {
        g->cta_off[c] = (int)g->ops.size();
        int res = 0;
        for (mg_op& op : per[c]) {
            if (op.type != MG_ATTN) {
                op.src = (long long)off;
                off += (size_t)op.nq * op.K * op.uv * m->wsize + 2 * (size_t)op.nq * op.uv * 4;
                off = (off + 15) & ~(size_t)15;
            }
            if (op.type == MG_OPROJ && op.layer == 0) res += op.nq * op.uv;
            g->ops.push_back(op);
        }
        g->max_ops = std::max(g->max_ops, (int)per[c].size());
        g->res_cap = std::max(g->res_cap, res);
    }
    g->cta_off[G] = (int)g->ops.size();
    g->wpack_bytes = off;
    // the copy schedule: one entry per chunk of a projection, one per attention op (expanded on the device)
    g->cds.clear();
    g->cd_off.assign(G + 1, 0);
    g->max_cd = 1;
    for (int c = 0; c < G; c++) {
        g->cd_off[c] = (int)g->cds.size();
        for (int oi = g->cta_off[c]; oi < g->cta_off[c + 1]; oi++) {
            const mg_op& op = g->ops[oi];
            if (op.type == MG_ATTN) {
                g->cds.push_back({(long long)(oi - g->cta_off[c]), 0, 2});
                continue;
            }
            for (int j = 0; j < op.nchunks; j++) {
                const int rows = std::min(op.kc, op.K - j * op.kc);
                const int ub = op.uv * (int)m->wsize;
                int bytes = op.nq * rows * ub;
                if (j == op.nchunks - 1) bytes += 2 * op.nq * op.uv * 4;  // trailer
                bytes = (bytes + 15) & ~15;
                g->cds.push_back({op.src + (long long)j * op.nq * op.kc * ub, bytes, 0});
            }
        }
        g->max_cd = std::max(g->max_cd, (int)g->cds.size() - g->cd_off[c]);
    }
    g->cd_off[G] = (int)g->cds.size();
}

template <typename WT>
static void mg_pack_all(rg_gpt* m, rg_mega* g) {
    cudaStream_t s = m->ctx->stream;
    for (int l = 0; l < m->L; l++) {
        rg_layer& y = m->layers[l];
        const rg_linear* lins[4] = {&y.qkv, &y.o, &y.fc1, &y.fc2};
        const int types[4] = {MG_QKV, MG_OPROJ, MG_FC1, MG_FC2};
        const float* gam[4] = {y.ln1g, nullptr, y.ln2g, nullptr};
        const float* bet[4] = {y.ln1b, nullptr, y.ln2b, nullptr};
        for (int i = 0; i < 4; i++)
            mg_pack_kernel<WT><<<g->G, 256, 0, s>>>((const WT*)lins[i]->W, lins[i]->ldw, lins[i]->b, lins[i]->N, gam[i], bet[i],
                                                    g->d_ops, g->d_cta_off, types[i], l, g->d_wpack);
    }
    mg_pack_kernel<WT><<<g->G, 256, 0, s>>>((const WT*)m->head.W, m->head.ldw, m->head.b, m->head.N, m->lnfg, m->lnfb, g->d_ops,
                                            g->d_cta_off, MG_HEAD, m->L, g->d_wpack);

    m->ctx->launches += 4 * m->L + 1;
}

template <typename WT, int B, int NQ, bool TRACE, bool TP = false>
static cudaError_t mg_launch_t(rg_gpt* m, rg_mega* g, mg_params& prm) {
    auto kern = rg_token_loop_kernel<WT, B, NQ, TRACE, TP>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g->smem_bytes);
    if (e != cudaSuccess) return e;
    void* args[] = {&prm};
    return cudaLaunchCooperativeKernel((void*)kern, dim3(g->G), dim3(MG_TOTAL_THREADS), args, g->smem_bytes, m->ctx->stream);
}

template <typename WT, int B, int NQ>
static cudaError_t mg_launch(rg_gpt* m, rg_mega* g, mg_params& prm) {
    // the instrumented build is also the one that honours a lowered wait limit and the withheld signal of the tests
    const bool instrumented = prm.trace || prm.spin_limit != MG_SPIN_LIMIT || prm.withhold_layer != -1 || prm.poll_sleep;
    // tensor parallel: one instance, with the run-time wait limit (NVLink latency, not instruction count, bounds its stages)
    if (prm.tp_size > 1) return mg_launch_t<WT, B, NQ, true, true>(m, g, prm);
    return instrumented ? mg_launch_t<WT, B, NQ, true>(m, g, prm) : mg_launch_t<WT, B, NQ, false>(m, g, prm);
}

// Where the exchange buffers sit inside their allocation decides which L2 slices serve the words that all 148 CTAs
// poll, and the per-token time moves by up to 4 % with it (measured: 192.8 ... 200.4 us on the GPT-2-small shape,
// reproducible per position).  The allocation therefore has room for MG_PLACE_CANDIDATES positions 4 KB apart and
// the first long enough run times a few token steps at each of them and keeps the fastest.
#define MG_PLACE_CANDIDATES 8
#define MG_PLACE_STEP_WORDS 512
#define MG_PLACE_BUFS 6
// Every exchange vector (q|k|v, attention records, x after the out-projection, hidden, x after FC2, picks) has its
// own region with room for MG_PLACE_CANDIDATES positions; cand[i] selects the position of vector i.
static void mg_exchange_sizes(const rg_gpt* m, const rg_mega* g, int B, size_t (&sz)[MG_PLACE_BUFS]) {
    sz[0] = (size_t)B * 3 * m->Dl;
    sz[1] = (size_t)B * m->Hl * g->S * (m->hd + 2);
    sz[2] = (size_t)B * m->D;
    sz[3] = (size_t)B * m->Fl;
    sz[4] = (size_t)B * m->D;
    sz[5] = (size_t)g->n_pick_ctas * B * 2;
}
static void mg_set_exchange(const rg_gpt* m, rg_mega* g, int B, const int (&cand)[MG_PLACE_BUFS]) {
    size_t sz[MG_PLACE_BUFS];
    mg_exchange_sizes(m, g, B, sz);
    mg_word** dst[MG_PLACE_BUFS] = {&g->buf_qkv, &g->buf_a, &g->buf_xc, &g->buf_h, &g->buf_xe, &g->buf_pick};
    mg_word* w = g->buf_base;
    for (int i = 0; i < MG_PLACE_BUFS; i++) {
        *dst[i] = w + (size_t)cand[i] * MG_PLACE_STEP_WORDS;
        w += ((sz[i] + 511) & ~(size_t)511) + (size_t)MG_PLACE_CANDIDATES * MG_PLACE_STEP_WORDS;
    }
}

// (Re)build program, packed weights and exchange buffers for batch B.
static rg_status mg_prepare(rg_gpt* m, int B) {
    rg_mega* g = m->mega;
    if (g->built_for_B == B) return RG_OK;
    RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
    for (void* p : g->allocs) cudaFree(p);
    g->allocs.clear();
    g->built_for_B = 0;
    mg_build_program(m, g, B);
    const int NQ = mg_nq_for(m->bf16, B);
    // ring depth: as many 32 KB slots as fit beside the rest (at most 6)
    g->nslot = 0;
    for (int ns = 6; ns >= 2; ns--) {
        const size_t need = mg_smem_bytes(m, B, NQ, ns, g->max_ops, g->max_cd, g->res_cap, m->tp_size > 1 ? m->tp_size * g->G : g->n_pick_ctas);
        if (need <= 227 * 1024) {
            g->nslot = ns;
            g->smem_bytes = need;
            break;
        }
    }
    if (g->nslot == 0) return rg_fail(RG_ERR_UNSUPPORTED, "model too large for the persistent token-loop kernel's shared memory");
    RG_TRY(mg_dalloc(g, (void**)&g->d_ops, g->ops.size() * sizeof(mg_op)));
    RG_TRY(mg_dalloc(g, (void**)&g->d_cta_off, (g->G + 1) * sizeof(int)));
    RG_TRY(mg_dalloc(g, (void**)&g->d_cds, g->cds.size() * sizeof(mg_cdesc)));
    RG_TRY(mg_dalloc(g, (void**)&g->d_cd_off, (g->G + 1) * sizeof(int)));
    RG_TRY(mg_dalloc(g, (void**)&g->d_wpack, g->wpack_bytes));
    RG_TRY(mg_dalloc(g, (void**)&g->d_trace, (size_t)g->G * g->max_ops * 8 * 8));
    RG_CUDA(cudaMemset(g->d_trace, 0, (size_t)g->G * g->max_ops * 8 * 8));
    RG_TRY(mg_dalloc(g, (void**)&g->d_abort, 16));
    size_t words = 0;
    {
        size_t sz[MG_PLACE_BUFS];
        mg_exchange_sizes(m, g, B, sz);
        for (size_t v : sz) words += ((v + 511) & ~(size_t)511) + (size_t)MG_PLACE_CANDIDATES * MG_PLACE_STEP_WORDS;
    }
    RG_TRY(mg_dalloc(g, (void**)&g->buf_base, words * 8));
    g->buf_bytes = words * 8;
    for (int& c : g->place) c = 0;
    mg_set_exchange(m, g, B, g->place);
    g->placed = m->tp_size > 1;  // (tensor parallel: no placement runs, they would have to be agreed between the ranks)
    RG_CUDA(cudaMemset(g->buf_base, 0, g->buf_bytes));
    RG_CUDA(cudaMemset(g->d_abort, 0, 16));
    // Tags restart with the local buffers.  Not so across ranks: the peers' words in this rank's receive regions keep
    // their tags, so a tensor-parallel model never reuses a tag (all ranks count the same steps).
    if (m->tp_size == 1) m->epoch = 0;
    RG_CUDA(cudaMemcpy(g->d_ops, g->ops.data(), g->ops.size() * sizeof(mg_op), cudaMemcpyHostToDevice));
    RG_CUDA(cudaMemcpy(g->d_cta_off, g->cta_off.data(), (g->G + 1) * sizeof(int), cudaMemcpyHostToDevice));
    RG_CUDA(cudaMemcpy(g->d_cds, g->cds.data(), g->cds.size() * sizeof(mg_cdesc), cudaMemcpyHostToDevice));
    RG_CUDA(cudaMemcpy(g->d_cd_off, g->cd_off.data(), (g->G + 1) * sizeof(int), cudaMemcpyHostToDevice));
    if (m->bf16) mg_pack_all<__nv_bfloat16>(m, g);
    else mg_pack_all<float>(m, g);
    RG_CUDA(cudaGetLastError());
    RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
    g->built_for_B = B;
    return RG_OK;
}

bool rg_mega_supports(const rg_gpt* m, int B) {
    if (m->tp_size > 1 && !(m->tp_fused && m->tp_mega_off != 0 && B <= MG_BMAX)) return false;  // needs the peer-mapped regions
    return m->mega != nullptr && m->use_mega && m->cfg.causal && mg_variant(B) >= 0 && m->hd <= 128;
}

rg_status rg_mega_create(rg_gpt* m) {
    rg_mega_destroy(m);
    const char* mode = getenv("RG_B200_DECODE");
    m->use_mega = !(mode && strcmp(mode, "graph") == 0);
    if (!m->cfg.causal) return RG_OK;
    m->mega = new rg_mega();
    m->mega->G = m->ctx->sm_count;
    return RG_OK;
}

void rg_mega_debug(rg_gpt* m, unsigned spin_limit, int withhold_layer) {
    if (!m->mega) return;
    if (spin_limit != 0xffffffffu) m->mega->spin_limit = spin_limit ? spin_limit : MG_SPIN_LIMIT;
    if (withhold_layer != -3) m->mega->withhold_layer = withhold_layer;
}

void rg_mega_destroy(rg_gpt* m) {
    if (!m->mega) return;
    for (void* p : m->mega->allocs) cudaFree(p);
    delete m->mega;
    m->mega = nullptr;
}

// One cooperative launch of n_steps token steps from position pos0 (the model's state says which ids to start from).
static rg_status mg_run_once(rg_gpt* m, int B, size_t pos0, size_t n_steps) {
    rg_mega* g = m->mega;
    // tags are (epoch * (L+1) + layer + 1) in 32 bits: start over long before they wrap
    if (((uint64_t)m->epoch + n_steps + 1) * (uint64_t)(m->L + 1) >= 0xfffffff0ull) {
        if (m->tp_size > 1) {  // cannot clear the peers' words from here: the launch form takes over
            m->use_mega = false;
            return RG_ERR_UNSUPPORTED;
        }
        RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
        RG_CUDA(cudaMemset(g->buf_base, 0, g->buf_bytes));
        m->epoch = 0;
    }
    mg_params prm;
    memset(&prm, 0, sizeof(prm));
    prm.ops = g->d_ops, prm.cta_off = g->d_cta_off, prm.wpack = g->d_wpack;
    prm.cds = g->d_cds, prm.cd_off = g->d_cd_off, prm.max_cd = g->max_cd;
    prm.trace = m->trace_on ? g->d_trace : nullptr;
    prm.wte = m->wte, prm.wpe = m->wpe, prm.ldt = m->ldt;
    prm.kc = (unsigned char*)m->kc, prm.vc = (unsigned char*)m->vc, prm.kv_layer_bytes = m->kv_layer_bytes;
    prm.buf_qkv = g->buf_qkv, prm.buf_a = g->buf_a, prm.buf_xc = g->buf_xc, prm.buf_h = g->buf_h, prm.buf_xe = g->buf_xe;
    prm.buf_pick = g->buf_pick;
    prm.logits = m->logits + m->v0, prm.tokens = m->tokens, prm.picks = m->picks, prm.d_pos = m->d_pos, prm.d_pos_next = m->d_pos_next;
    prm.abort_flag = g->d_abort;
    prm.V = m->Vl, prm.D = m->D, prm.L = m->L, prm.H = m->Hl, prm.hd = m->hd, prm.C = m->C, prm.F = m->Fl;
    prm.Dq = m->Dl, prm.XLEN = std::max(m->D, m->Fl), prm.ldl = m->V, prm.v0 = m->v0;
    prm.tp_rank = m->tp_rank, prm.tp_size = m->tp_size, prm.pick_stride = g->G;
    if (m->tp_size > 1) {
        // the peers' regions inside every rank's receive buffer (rg_gpt.cu lays them out: see rg_tp_mega_words)
        const size_t xwords = (size_t)m->tp_size * MG_BMAX * m->D;
        for (int r = 0; r < m->tp_size; r++) {
            mg_word* base = reinterpret_cast<mg_word*>(m->tp_peer[r]) + m->tp_mega_off;
            prm.tp_xc[r] = base, prm.tp_xe[r] = base + xwords, prm.tp_pick[r] = base + 2 * xwords;
            // head CTAs of rank r: what add_projection(MG_HEAD) gives for its vocabulary slice
            const int v0r = std::min(m->V, r * m->Vpad), vlr = std::max(0, std::min(m->Vpad, m->V - v0r));
            prm.n_pick_of[r] = std::min(g->G, rg_cdiv(vlr, 16 / (int)m->wsize));
        }
    } else {
        prm.n_pick_of[0] = g->n_pick_ctas;
    }
    prm.act = m->cfg.activation;
    prm.pos0 = (int)pos0, prm.n_steps = (int)n_steps, prm.epoch0 = m->epoch;
    prm.S = g->S;
    prm.spin_limit = g->spin_limit, prm.withhold_layer = g->withhold_layer;
    {
        const char* ps = getenv("RG_B200_POLL_SLEEP_NS");
        prm.poll_sleep = ps ? atoi(ps) : 0;
    }
    prm.nslot = g->nslot, prm.max_ops = g->max_ops, prm.res_cap = g->res_cap, prm.n_pick_ctas = g->n_pick_ctas;
    prm.scale = 1.f / sqrtf((float)m->hd);
    cudaError_t e;
    if (!m->bf16) {
        if (B == 1) e = mg_launch<float, 1, 6>(m, g, prm);
        else if (B == 2) e = mg_launch<float, 2, 4>(m, g, prm);
        else e = mg_launch<float, 4, 2>(m, g, prm);
    } else {
        if (B == 1) e = mg_launch<__nv_bfloat16, 1, 3>(m, g, prm);
        else if (B == 2) e = mg_launch<__nv_bfloat16, 2, 2>(m, g, prm);
        else e = mg_launch<__nv_bfloat16, 4, 1>(m, g, prm);
    }
    if (e == cudaErrorCooperativeLaunchTooLarge || e == cudaErrorLaunchOutOfResources) {
        cudaGetLastError();
        m->use_mega = false;  // its CTAs cannot be co-resident here: use the CUDA-graph step from now on
        return RG_ERR_UNSUPPORTED;
    }
    if (e != cudaSuccess)
        return rg_fail(RG_ERR_BACKEND, "persistent token-loop kernel launch failed: %s", cudaGetErrorString(e));
    m->epoch += (uint32_t)n_steps;
    m->ctx->launches += 1;
    return RG_OK;
}

// Chooses the position of every exchange vector: one vector at a time, MG_PLACE_TOKENS token steps are timed at each
// of its candidate positions (the others fixed) and the fastest is kept; a stage's latency depends on where its own
// input vector lives, so the per-vector optima add up.  The trial runs start from the caller's position and recompute
// exactly what the real run computes next (same cache rows, same ids), so they leave nothing behind but their tags,
// which are older than any tag used later.
#define MG_PLACE_TOKENS 16
static rg_status mg_place_exchange(rg_gpt* m, int B, size_t pos0) {
    rg_mega* g = m->mega;
    g->placed = true;
    const char* env = getenv("RG_B200_EXCH_PLACE");  // "off": keep every vector at position 0
    if (env && strcmp(env, "off") == 0) return RG_OK;
    const bool tr = m->trace_on;
    m->trace_on = false;
    cudaEvent_t e0, e1;
    RG_CUDA(cudaEventCreate(&e0));
    RG_CUDA(cudaEventCreate(&e1));
    rg_status st = RG_OK;
    auto timed = [&](float* ms) {
        cudaEventRecord(e0, m->ctx->stream);
        st = mg_run_once(m, B, pos0, MG_PLACE_TOKENS);
        cudaEventRecord(e1, m->ctx->stream);
        if (st != RG_OK) return;
        if (cudaEventSynchronize(e1) != cudaSuccess) {
            st = rg_fail(RG_ERR_BACKEND, "persistent token-loop kernel failed during placement: %s",
                         cudaGetErrorString(cudaGetLastError()));
            return;
        }
        cudaEventElapsedTime(ms, e0, e1);
    };
    float ms = 0.f;
    timed(&ms);  // warm-up (instruction cache, packed weights of the first steps in L2)
    for (int i = 0; i < MG_PLACE_BUFS - 1 && st == RG_OK; i++) {  // the pick vector (last) is tiny: left where it is
        int best = 0;
        float best_ms = 1e30f;
        for (int c = 0; c < MG_PLACE_CANDIDATES && st == RG_OK; c++) {
            g->place[i] = c;
            mg_set_exchange(m, g, B, g->place);
            float t0 = 1e30f, t1 = 1e30f;
            timed(&t0);
            if (st == RG_OK) timed(&t1);
            const float t = std::min(t0, t1);
            if (t < best_ms) best_ms = t, best = c;
        }
        g->place[i] = best;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    m->trace_on = tr;
    if (st != RG_OK) return st;
    mg_set_exchange(m, g, B, g->place);
    return rg_mega_check(m);
}

rg_status rg_mega_run(rg_gpt* m, int B, size_t pos0, size_t n_steps) {
    if (n_steps == 0) return RG_OK;
    rg_status st = mg_prepare(m, B);
    if (st == RG_ERR_UNSUPPORTED) {  // fall back to the graph path for this model from now on
        m->use_mega = false;
        return st;
    }
    RG_TRY(st);
    if (!m->mega->placed && n_steps >= 2 * MG_PLACE_TOKENS && pos0 + MG_PLACE_TOKENS < (size_t)m->C) {
        st = mg_place_exchange(m, B, pos0);
        if (st != RG_OK) return st;  // RG_ERR_UNSUPPORTED included: the caller falls back to the graph step
    }
    // tensor parallel: the ranks' kernels wait for each other's words, so they should start together; a small collective
    // on the stream, after this rank's (possibly long) preparation, lines the launches up
    if (m->tp_size > 1) RG_TRY(rg_tp_stream_barrier(m));
    return mg_run_once(m, B, pos0, n_steps);
}

rg_status rg_mega_check(rg_gpt* m) {
    if (!m->mega || !m->mega->d_abort || !m->mega->built_for_B) return RG_OK;
    int flag = 0;
    RG_CUDA(cudaMemcpyAsync(&flag, m->mega->d_abort, sizeof(int), cudaMemcpyDeviceToHost, m->ctx->stream));
    RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
    if (flag) {
        cudaMemsetAsync(m->mega->d_abort, 0, sizeof(int), m->ctx->stream);
        cudaMemsetAsync(m->mega->buf_base, 0, m->mega->buf_bytes, m->ctx->stream);
        if (m->tp_size == 1) m->epoch = 0;
        else m->use_mega = false;  // the ranks may no longer agree on the step count: the launch form from now on
        return rg_fail(RG_ERR_TIMEOUT, "a bounded wait inside the persistent token-loop kernel gave up; the step was abandoned");
    }
    return RG_OK;
}

// Timestamps (ns, %globaltimer) of the last token step of the last run, per CTA and op:
// [start, input ready, dot products done, outputs stored] then SM cycles spent waiting for ring slots and
// for the input vector, then two more timestamps (input words all valid; chunk loop finished).
// Rows of 12: cta, op index, type, layer, t0..t3, wait cycles, poll cycles, t_fetched, t_loop.
rg_status rg_mega_trace(rg_gpt* m, unsigned long long* out, size_t cap_rows, size_t* n_rows) {
    rg_mega* g = m->mega;
    *n_rows = 0;
    if (!g || !g->built_for_B || !g->d_trace) return RG_OK;
    std::vector<unsigned long long> raw((size_t)g->G * g->max_ops * 8);
    RG_CUDA(cudaStreamSynchronize(m->ctx->stream));
    RG_CUDA(cudaMemcpy(raw.data(), g->d_trace, raw.size() * 8, cudaMemcpyDeviceToHost));
    size_t n = 0;
    for (int c = 0; c < g->G; c++)
        for (int oi = g->cta_off[c]; oi < g->cta_off[c + 1]; oi++) {
            if (n >= cap_rows) break;
            const mg_op& op = g->ops[oi];
            const unsigned long long* t = &raw[((size_t)c * g->max_ops + (oi - g->cta_off[c])) * 8];
            unsigned long long* o = out + n * 12;
            o[0] = c, o[1] = oi - g->cta_off[c], o[2] = op.type, o[3] = op.layer;
            o[4] = t[0], o[5] = t[1], o[6] = t[2], o[7] = t[3], o[8] = t[4], o[9] = t[5], o[10] = t[6], o[11] = t[7];
            n++;
        }
    *n_rows = n;
    return RG_OK;
}

// ---------------------------------------------------------------------------
// Host-only check of the token-loop program (no device is touched): builds the per-CTA op lists of one tensor-parallel
// rank of a model shape exactly as rg_mega_run would and verifies what the kernel relies on.
// out[0] context slices per head, [1] most ops of a CTA, [2] ring slots that fit, [3] shared memory bytes,
// [4] CTAs with LM-head work, [5] packed weight bytes, [6] ops in total, [7] number of violations found:
// a projection column or an attention (sequence, head, slice) that is covered zero times or twice, a chunk larger than a
// ring slot, a residual slice larger than res_cap.  out[2] = 0 means the program does not fit the SM's shared memory (the
// library then runs the step as separate launches).
// ---------------------------------------------------------------------------
extern "C" rg_status rg_token_loop_plan(int D, int H, int L, int V, int tp_size, int tp_rank, int bf16, int batch, int sm_count,
                                               long long* out) {
    if (!out || D <= 0 || H <= 0 || L <= 0 || V <= 0 || tp_size <= 0 || tp_rank < 0 || tp_rank >= tp_size || sm_count <= 0 ||
        D % H || mg_variant(batch) < 0 || tp_size > H)
        return rg_fail(RG_ERR_INVALID_INPUT, "rg_token_loop_plan: shape or rank out of range");
    rg_gpt m;
    m.D = D, m.H = H, m.hd = D / H, m.L = L, m.V = V, m.F = 4 * D, m.C = 1024, m.Bmax = batch;
    m.bf16 = bf16 != 0, m.wsize = bf16 ? 2 : 4;
    m.tp_size = tp_size, m.tp_rank = tp_rank;
    {   // the shard arithmetic of rg_gpt_create
        const int T = tp_size, r = tp_rank, F8 = m.F / 8;
        m.Hl = H / T + (r < H % T ? 1 : 0), m.h0 = r * (H / T) + std::min(r, H % T), m.Dl = m.Hl * m.hd;
        m.Fl = 8 * (F8 / T + (r < F8 % T ? 1 : 0)), m.f0 = 8 * (r * (F8 / T) + std::min(r, F8 % T));
        m.Vpad = (rg_cdiv(V, T) + 7) / 8 * 8;
        m.v0 = std::min(V, r * m.Vpad), m.Vl = std::max(0, std::min(m.Vpad, V - m.v0));
        if (T == 1) m.Vpad = V;
    }
    if (m.Vl <= 0 || m.hd > 128) return rg_fail(RG_ERR_UNSUPPORTED, "rg_token_loop_plan: shape outside the kernel's limits");
    rg_mega g;
    g.G = sm_count;
    mg_build_program(&m, &g, batch);
    const int B = batch, NQ = mg_nq_for(m.bf16, B);
    long long bad = 0;
    int nslot = 0;
    size_t smem = 0;
    for (int ns = 6; ns >= 2 && !nslot; ns--) {
        const size_t need = mg_smem_bytes(&m, B, NQ, ns, g.max_ops, g.max_cd, g.res_cap, tp_size > 1 ? tp_size * g.G : g.n_pick_ctas);
        if (need <= 227 * 1024) nslot = ns, smem = need;
    }
    // coverage: per (type, layer) the column units of all CTAs tile [0, N) exactly once
    const int Ns[6] = {3 * m.Dl, 0, D, m.Fl, D, m.Vl};
    for (int l = 0; l <= L; l++) {
        for (int type : {MG_QKV, MG_OPROJ, MG_FC1, MG_FC2, MG_HEAD}) {
            if ((type == MG_HEAD) != (l == L)) continue;
            const int N = Ns[type];
            std::vector<int> seen((size_t)N, 0);
            for (const mg_op& op : g.ops) {
                if (op.type != type || op.layer != l) continue;
                for (int c = op.q0 * op.uv; c < (op.q0 + op.nq) * op.uv; c++)
                    if (c < N) seen[(size_t)c]++;
            }
            for (int c = 0; c < N; c++)
                if (seen[(size_t)c] != 1) bad++;
        }
        if (l == L) break;
        std::vector<int> pairs((size_t)B * m.Hl * g.S, 0);
        for (const mg_op& op : g.ops)
            if (op.type == MG_ATTN && op.layer == l) {
                const size_t i = ((size_t)op.nq * m.Hl + op.q0) * g.S + op.aux;
                if (op.nq >= B || op.q0 >= m.Hl || op.aux >= g.S) bad++;
                else pairs[i]++;
            }
        for (int v : pairs)
            if (v != 1) bad++;
    }
    // every copy of the schedule fits a ring slot
    for (const mg_cdesc& cd : g.cds)
        if (cd.kind == 0 && (cd.bytes <= 0 || (size_t)cd.bytes > MG_SLOT_BYTES || (cd.bytes & 15))) bad++;
    // every CTA's residual slice fits
    for (int c = 0; c < g.G; c++) {
        int res = 0;
        for (int oi = g.cta_off[c]; oi < g.cta_off[c + 1]; oi++)
            if (g.ops[oi].type == MG_OPROJ && g.ops[oi].layer == 0) res += g.ops[oi].nq * g.ops[oi].uv;
        if (res > g.res_cap) bad++;
    }
    out[0] = g.S, out[1] = g.max_ops, out[2] = nslot, out[3] = (long long)smem, out[4] = g.n_pick_ctas;
    out[5] = (long long)g.wpack_bytes, out[6] = (long long)g.ops.size(), out[7] = bad;
    return RG_OK;
}

