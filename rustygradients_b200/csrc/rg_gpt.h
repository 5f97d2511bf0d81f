// Model state shared by the translation units of the GPT half of the library.
#pragma once
#include "rg_internal.cuh"

struct rg_mega;   // persistent token-loop kernel state (rg_mega.cu)
struct rg_cloop;  // persistent token-loop kernel of thread-block clusters (rg_cloop.cu)

struct rg_linear {
    void* W = nullptr;  // [K][ldw] f32 or bf16
    void* Wt = nullptr;  // bf16 mode: [N][K] copy (K contiguous) for the tensor-core prompt pass
    long long ldw = 0;
    float* b = nullptr;  // [N]
    int K = 0, N = 0;
    int ksplit = 1, krows = 0;  // split of the token-step projection
    float* parts = nullptr;     // [ksplit][Bmax][N]
};

struct rg_layer {
    rg_linear qkv, o, fc1, fc2;
    float *ln1g = nullptr, *ln1b = nullptr, *ln2g = nullptr, *ln2b = nullptr;
};

struct rg_gpt {
    rg_ctx* ctx = nullptr;
    rg_gpt_config cfg;
    int V = 0, D = 0, L = 0, H = 0, hd = 0, C = 0, F = 0, Bmax = 1;
    // tensor-parallel shard of this rank (the full sizes when tp_size == 1): heads [h0, h0+Hl), hidden columns
    // [f0, f0+Fl), vocabulary [v0, v0+Vl); Dl = Hl * hd; Vpad = vocabulary slice size of every rank but the last
    int tp_rank = 0, tp_size = 1;
    int Hl = 0, h0 = 0, Dl = 0, Fl = 0, f0 = 0, Vl = 0, v0 = 0, Vpad = 0;
    void* nccl_comm = nullptr;
    float *tp_vec = nullptr, *tp_gather = nullptr, *tp_local = nullptr;  // token-step collectives
    float *ptp = nullptr, *pgather = nullptr;                           // prompt-pass collectives
    // one-shot all-reduce of the token step over peer memory: every rank's receive buffer
    // [2 parities][tp_size ranks][Bmax * D] of {f32 value, 32-bit tag} words, mapped into every other rank
    unsigned long long* tp_recv = nullptr;
    unsigned long long* tp_peer[16] = {};
    bool tp_fused = false;
    // after the all-reduce slots, the same buffer holds the receive regions of the tensor-parallel persistent token loop
    // (rg_mega.cu): [tp_size][4][D] out-projection partials, the same for FC2, [tp_size][SMs][4][2] picks; in words
    size_t tp_mega_off = 0;
    unsigned* d_tp_epoch = nullptr;  // token steps enqueued so far (tags)
    int* d_tp_err = nullptr;         // set by a wait that gave up
    size_t pgatherCap = 0;
    bool bf16 = false, loaded = false;
    size_t wsize = 4;
    long long ldt = 0;  // leading dimension of the two embedding tables
    void *wte = nullptr, *wpe = nullptr;
    float *lnfg = nullptr, *lnfb = nullptr;
    rg_linear head;
    std::vector<rg_layer> layers;
    std::vector<void*> allocs;

    // KV cache: [L][Bmax][H][C][hd], f32 or bf16
    char *kc = nullptr, *vc = nullptr;
    size_t kv_layer_bytes = 0;

    // token-step state
    float *xa = nullptr, *xb = nullptr, *ap = nullptr, *logits = nullptr;
    uint32_t *tokens = nullptr, *picks = nullptr;
    int *d_pos = nullptr, *d_pos_next = nullptr;
    int NS = 1;
    size_t pos = 0, curB = 0;
    cudaGraphExec_t graph = nullptr;
    size_t graphB = 0;
    int kernels_per_step = 0;
    bool use_graph = true;

    // prompt-pass buffers, grown on demand
    size_t rowsCap = 0;
    float *px = nullptr, *pln = nullptr, *pqkv = nullptr, *pattn = nullptr, *ph = nullptr, *plast = nullptr;
    void *pq16 = nullptr, *pvt16 = nullptr;  // bf16 Q rows and V^T of the tensor-core attention of the prompt pass
    void* pa16 = nullptr;  // bf16 copy of the current GEMM input rows
    float* pws = nullptr;  // split-k workspace of the CUDA-core GEMM
    size_t pwsFloats = 0;
    bool use_tc = true;
    float* plogits = nullptr;
    size_t plogitsCap = 0;

    // persistent token-loop kernel (null when the model shape is outside its limits)
    rg_mega* mega = nullptr;
    bool use_mega = true;
    // the same loop as a kernel of thread-block clusters (tried first; null or unusable -> the kernel above)
    rg_cloop* cloop = nullptr;
    bool use_cloop = true;
    bool trace_on = false;
    uint32_t epoch = 0;  // token steps run so far by the persistent kernel (tags of its exchange buffers)
};

// rg_gemm_tc.cu: RG_ERR_UNSUPPORTED when the shape is outside the tensor-core kernel's limits
rg_status rg_gemm_bf16_tc(rg_ctx* ctx, const void* A16, int M, int K, const void* Wt16, int N, float* C, long long ldc,
                          const float* bias, const float* res, long long ldres, int act);

rg_status rg_gemm_bf16_tc_parts(rg_ctx* ctx, const void* A16, int M, int K, const void* Wt16, int N, const float** parts,
                                int* nparts);

// rg_attn_tc.cu: RG_ERR_UNSUPPORTED when the shape is outside the tensor-core attention kernel's limits
rg_status rg_attn_bf16_tc(rg_ctx* ctx, const float* qkv, const void* kcache, int B, int H, int T, int C, int D, int hd, int causal,
                          void* q16, void* vt16, float* out);

// rg_gpt.cu: a one-element all-reduce on the model's stream (tensor parallel only)
rg_status rg_tp_stream_barrier(rg_gpt* m);

// rg_mega.cu
rg_status rg_mega_create(rg_gpt* m);            // after the weights are on the device
void rg_mega_destroy(rg_gpt* m);
bool rg_mega_supports(const rg_gpt* m, int B);
rg_status rg_mega_run(rg_gpt* m, int B, size_t pos0, size_t n_steps);  // enqueue n_steps token steps
rg_status rg_mega_check(rg_gpt* m);
// test hooks: spin_limit 0xffffffff and withhold_layer -3 keep the current values
void rg_mega_debug(rg_gpt* m, unsigned spin_limit, int withhold_layer);
rg_status rg_mega_trace(rg_gpt* m, unsigned long long* out, size_t cap_rows, size_t* n_rows);             // after a synchronise: did a bounded wait give up?


// rg_cloop.cu: same contract as the rg_mega_* functions
rg_status rg_cloop_create(rg_gpt* m);
void rg_cloop_destroy(rg_gpt* m);
bool rg_cloop_supports(const rg_gpt* m, int B);
rg_status rg_cloop_run(rg_gpt* m, int B, size_t pos0, size_t n_steps);
rg_status rg_cloop_check(rg_gpt* m);
rg_status rg_cloop_trace(rg_gpt* m, unsigned long long* out, size_t cap_rows, size_t* n_rows);
bool rg_cloop_active(const rg_gpt* m);
// test hook: head cluster 0 withholds its partial of `withhold_layer` (-1: off); spin_limit 0 keeps the current limit
void rg_cloop_debug(rg_gpt* m, int withhold_layer, unsigned spin_limit);
