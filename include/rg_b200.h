/*
 * rg_b200.h - C ABI of the B200 (sm_100a) GPT token-loop library.
 *
 * Every entry point is what a foreign-function binding for RustyGradients
 * (crate rusty-gradients 0.2.0) would bind for this path: plain pointers and
 * sizes, opaque handles, a status code per call.  The comment above each
 * declaration names the reference interface it replaces (file:line inside the
 * crate).  Host pointers are borrowed for the duration of the call only.
 *
 * Threading: an rg_ctx may be used from any thread, one call at a time per
 * context; an rg_gpt has a single owner (the reference's model is !Send,
 * src/tensor.rs:23).  One context per GPU.
 */
#ifndef RG_B200_H
#define RG_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define RG_API __attribute__((visibility("default")))
#else
#define RG_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- errors: src/error.rs:13-50 (RustyGradientsError) plus the two variants
 * the reference's CUDA backend assumes, src/backend/cuda.rs:41-45,50 -------- */
typedef enum rg_status {
    RG_OK = 0,
    RG_ERR_SHAPE = 1,         /* ShapeError / ShapeMismatch            */
    RG_ERR_DIMENSION = 2,     /* DimensionError {expected, actual}     */
    RG_ERR_INVALID_INPUT = 3, /* InvalidInput (id >= vocab, T > block) */
    RG_ERR_BACKEND = 4,       /* BackendError (CUDA / NCCL failure)    */
    RG_ERR_UNSUPPORTED = 5,   /* where the reference has unimplemented!() (src/backend/cuda.rs:436-494) */
    RG_ERR_CONTEXT_FULL = 6,  /* decode past block_size (the reference slides its window, src/wasm_api.rs:103) */
    RG_ERR_TIMEOUT = 7,       /* a bounded device-side wait gave up    */
    RG_ERR_SERIALIZATION = 8, /* SerializationError (malformed file, dtype other than F32) */
    RG_ERR_IO = 9             /* IoError (missing file, missing required weight: src/models/hf_loader.rs:233-238) */
} rg_status;

/* Message of the last failing call on this thread (maps to the String payload
 * of the enum variants above). Never NULL. */
RG_API const char* rg_last_error(void);
RG_API const char* rg_version(void);

typedef struct rg_ctx rg_ctx;         /* CudaBackend, src/backend/cuda.rs:77-83       */
typedef struct rg_storage rg_storage; /* CudaStorage {data, shape, device}, src/backend/cuda.rs:29-33 */
typedef struct rg_gpt rg_gpt;         /* GPTModel, src/models/gpt.rs:17-24            */

/* ---- context ------------------------------------------------------------ */
/* CudaBackend::device_count / is_available, src/backend/cuda.rs:128-135 */
RG_API int rg_device_count(void);
/* CudaBackend::new(device_index), src/backend/cuda.rs:87-125; Device::cuda(index), src/backend/mod.rs:72-77 */
RG_API rg_status rg_ctx_create(int device, rg_ctx** out);
RG_API rg_status rg_ctx_destroy(rg_ctx* ctx);
/* Backend::synchronize, src/backend/mod.rs:137-138 */
RG_API rg_status rg_synchronize(rg_ctx* ctx);
/* The cudaStream_t every call of this context enqueues on (for event timing). */
RG_API void* rg_ctx_stream(rg_ctx* ctx);
/* Number of kernels this context has launched since creation. */
RG_API uint64_t rg_ctx_launch_count(rg_ctx* ctx);

/* ---- storage: Backend memory operations, src/backend/mod.rs:140-155 ---------- */
/* Backend::zeros / ones */
RG_API rg_status rg_zeros(rg_ctx* ctx, const size_t* shape, int ndim, rg_storage** out);
RG_API rg_status rg_ones(rg_ctx* ctx, const size_t* shape, int ndim, rg_storage** out);
/* Backend::from_slice(&[f32], &[usize]); len != prod(shape) is RG_ERR_SHAPE (src/backend/cpu.rs:54-57) */
RG_API rg_status rg_from_slice(rg_ctx* ctx, const float* data, size_t len, const size_t* shape, int ndim,
                        rg_storage** out);
/* Backend::to_vec: copies prod(shape) floats to out (cap = capacity in floats) and synchronises */
RG_API rg_status rg_to_vec(rg_ctx* ctx, const rg_storage* st, float* out, size_t cap);
/* Backend::shape */
RG_API rg_status rg_shape(const rg_storage* st, size_t* shape_out, int cap, int* ndim_out);
RG_API size_t rg_storage_len(const rg_storage* st); /* CudaStorage::len, src/backend/cuda.rs:65-67 */
RG_API rg_status rg_storage_free(rg_storage* st);   /* Drop of the Storage value         */

/* ---- ops: one per Backend trait method, src/backend/mod.rs:157-226.  Each
 * returns a new owned storage; inputs are never modified. ------------------ */
/* add / sub / mul with numpy-style broadcasting (src/backend/cpu.rs:68-80; bias add
 * [B,T,N]+[1,N], 0-D scale and residuals on the model path, src/ops/basic_ops.rs:45-148) */
RG_API rg_status rg_add(rg_ctx* ctx, const rg_storage* a, const rg_storage* b, rg_storage** out);
RG_API rg_status rg_sub(rg_ctx* ctx, const rg_storage* a, const rg_storage* b, rg_storage** out);
RG_API rg_status rg_mul(rg_ctx* ctx, const rg_storage* a, const rg_storage* b, rg_storage** out);
/* matmul 2Dx2D, 3Dx3D, 4Dx4D (src/backend/cpu.rs:82-208) and 3Dx2D (src/ops/matmul.rs:51-72) */
RG_API rg_status rg_matmul(rg_ctx* ctx, const rg_storage* a, const rg_storage* b, rg_storage** out);
/* relu / sigmoid / exp / log / powf (src/backend/cpu.rs:213-244; kernels src/backend/cuda_kernels.cu:81-171) */
RG_API rg_status rg_relu(rg_ctx* ctx, const rg_storage* a, rg_storage** out);
RG_API rg_status rg_sigmoid(rg_ctx* ctx, const rg_storage* a, rg_storage** out);
RG_API rg_status rg_exp(rg_ctx* ctx, const rg_storage* a, rg_storage** out);
RG_API rg_status rg_log(rg_ctx* ctx, const rg_storage* a, rg_storage** out);
RG_API rg_status rg_powf(rg_ctx* ctx, const rg_storage* a, float power, rg_storage** out);
/* tanh-GELU: fused::gelu_fused, src/backend/fused.rs:151-175; kernel gelu_forward,
 * src/backend/cuda_kernels.cu:120-131 (loaded by the reference but never given a trait method) */
RG_API rg_status rg_gelu(rg_ctx* ctx, const rg_storage* a, rg_storage** out);
/* softmax over the last axis, max-subtracted (src/backend/cpu.rs:246-270; src/backend/cuda.rs:404-432) */
RG_API rg_status rg_softmax(rg_ctx* ctx, const rg_storage* a, rg_storage** out);
/* sum -> shape [1] (src/backend/cpu.rs:274-277), sum_axis (src/backend/cpu.rs:279-291) */
RG_API rg_status rg_sum(rg_ctx* ctx, const rg_storage* a, rg_storage** out);
RG_API rg_status rg_sum_axis(rg_ctx* ctx, const rg_storage* a, size_t axis, rg_storage** out);
/* reshape (element count must match, src/backend/cpu.rs:292-296) and transpose of two axes,
 * materialised (src/backend/cpu.rs:298-311) */
RG_API rg_status rg_reshape(rg_ctx* ctx, const rg_storage* a, const size_t* new_shape, int ndim, rg_storage** out);
RG_API rg_status rg_transpose(rg_ctx* ctx, const rg_storage* a, size_t axis1, size_t axis2, rg_storage** out);
/* embedding: f32-valued indices [B,T] or [B], weights [V,D] (src/backend/cpu.rs:315-363) */
RG_API rg_status rg_embedding(rg_ctx* ctx, const rg_storage* indices, const rg_storage* weights, rg_storage** out);
/* layer_norm over the last axis, one-pass Welford statistics, biased variance,
 * eps inside the sqrt (src/backend/cpu.rs:365-375 -> src/backend/fused.rs:22-144); gamma/beta hold D values */
RG_API rg_status rg_layer_norm(rg_ctx* ctx, const rg_storage* x, const rg_storage* gamma, const rg_storage* beta,
                        float epsilon, rg_storage** out);
/* sparse_cross_entropy: mean over rows of -log softmax(logits)[target] (src/backend/cpu.rs:377-427) */
RG_API rg_status rg_sparse_cross_entropy(rg_ctx* ctx, const rg_storage* logits, const rg_storage* targets,
                                  rg_storage** out);

/* ---- GPT model: src/models/gpt.rs ---------------------------------------- */
enum { RG_ACT_RELU = 0, RG_ACT_GELU_TANH = 1 };
enum { RG_DTYPE_F32 = 0, RG_DTYPE_BF16 = 1 };

/* GptConfig (src/models/gpt.rs:8-14) plus the switches this engine adds. */
typedef struct rg_gpt_config {
    size_t block_size;
    size_t vocab_size;
    size_t num_layers;
    size_t num_heads;
    size_t embedding_dim;
    int causal;        /* 0: the reference's unmasked attention (src/nn/attention.rs:78-94); 1: causal, enables the KV cache */
    int activation;    /* RG_ACT_RELU (src/nn/feedforward.rs:43-45) or RG_ACT_GELU_TANH (src/backend/fused.rs:151-175) */
    int weight_dtype;  /* RG_DTYPE_F32, or RG_DTYPE_BF16: matrices, tables and KV cache kept in bf16 */
    size_t max_batch;  /* sequences the KV cache is sized for */
    int tp_rank;       /* tensor parallelism: this process's rank ... */
    int tp_size;       /* ... of tp_size (0 or 1 = none).  One process and one GPU per rank. */
} rg_gpt_config;

/* GPTModel::new(config), src/models/gpt.rs:27-54 (asserts embedding_dim % num_heads == 0, src/nn/attention.rs:38-41) */
RG_API rg_status rg_gpt_create(rg_ctx* ctx, const rg_gpt_config* cfg, rg_gpt** out);
RG_API rg_status rg_gpt_destroy(rg_gpt* m);
/* Module::parameters() order, src/models/gpt.rs:85-93: number of tensors (2 + 16 L + 4) and the shape of tensor i */
RG_API int rg_gpt_num_params(const rg_gpt* m);
RG_API rg_status rg_gpt_param_shape(const rg_gpt* m, int i, size_t shape_out[2]);
/* Weight ingest with the shape asserts of WasmGptTrainer::loadWeightsFromJson,
 * src/wasm_api.rs:182-199: n tensors in parameters() order, f32, W as [in,out]. */
RG_API rg_status rg_gpt_load_params(rg_gpt* m, const float* const* data, const size_t* const* shapes,
                             const int* ndims, int n);
/* Module::forward(&idx) -> logits, src/models/gpt.rs:58-83: idx_f32 [B,T] host (ids carried as
 * f32 like src/wasm_api.rs:106), logits [B,T,V] host.  Honours cfg.causal / activation. */
RG_API rg_status rg_gpt_forward(rg_gpt* m, const float* idx_f32, size_t B, size_t T, float* logits);
/* First half of the token loop (src/wasm_api.rs:103-118) for a causal model: runs the
 * prompt [B,T] once, fills the KV cache, leaves position = T.  Optional outputs:
 * last-row logits [B,V] and their argmax [B] (host). */
RG_API rg_status rg_gpt_prefill(rg_gpt* m, const uint32_t* ids, size_t B, size_t T, float* logits_last,
                         uint32_t* argmax);
/* One iteration of the loop body (src/wasm_api.rs:102-160) on the KV cache: feeds
 * tok[B] (host) at the current position, returns logits [B,V] (or NULL) and the
 * greedy pick [B] (or NULL). */
RG_API rg_status rg_gpt_decode_step(rg_gpt* m, const uint32_t* tok, float* logits, uint32_t* argmax);
/* WasmGptTrainer::generate(prompt_ids, max_new_tokens, temperature, top_k),
 * src/wasm_api.rs:97-163, batched over B prompts of equal length P; out [B,max_new].
 * top_k == 1 is greedy (argmax, lowest index on ties).  Other top_k draw from a
 * counter-based generator seeded with `seed` (the reference uses thread_rng). */
RG_API rg_status rg_gpt_generate(rg_gpt* m, const uint32_t* prompt, size_t B, size_t P, size_t max_new,
                          float temperature, size_t top_k, uint64_t seed, uint32_t* out);
/* Device-resident greedy loop: n_steps iterations of the loop body starting from the
 * pick left by prefill / the previous step, ids never leave the GPU.  Asynchronous. */
RG_API rg_status rg_gpt_decode_run(rg_gpt* m, size_t n_steps);
/* Rewind the position to T (the cache rows below T stay valid) and make `tok[B]`
 * (host) the next token to feed. */
RG_API rg_status rg_gpt_rewind(rg_gpt* m, size_t T, const uint32_t* tok);
/* Copy generated ids [B, n] starting at absolute position `from` to the host; synchronises. */
RG_API rg_status rg_gpt_read_tokens(rg_gpt* m, size_t from, size_t n, uint32_t* out);
RG_API size_t rg_gpt_position(const rg_gpt* m);
/* Forget the cached context (start of a new generate call). */
RG_API rg_status rg_gpt_reset(rg_gpt* m);
/* Algorithmic bytes one decode step reads ON THIS GPU at context length T for B sequences
 * (weights + biases + LN + one table row pair + K/V of every cached position; with tensor
 * parallelism the shard of this rank plus the replicated LayerNorm / bias terms). */
RG_API double rg_gpt_decode_step_bytes(const rg_gpt* m, size_t B, double mean_ctx);

/* Tensor parallelism (nothing to mirror: the reference has no multi-device path).  With
 * cfg.tp_size > 1 every rank creates the same model with its own tp_rank, loads the SAME full
 * parameter list (it keeps only its shard: heads of Wq/Wk/Wv and the matching rows of Wo, columns
 * of W1 with the matching rows of W2, a vocabulary slice of the LM head) and joins one NCCL
 * communicator: rank 0 calls rg_gpt_tp_unique_id, the 128 bytes travel to the other ranks by any
 * host channel, then every rank calls rg_gpt_tp_init (collective).  Each block then costs two
 * all-reduces of [B, embedding_dim] over NVLink, the head one all-gather of logits. */
RG_API rg_status rg_gpt_tp_unique_id(uint8_t id_out[128]);
RG_API rg_status rg_gpt_tp_init(rg_gpt* m, const uint8_t id[128]);
/* 1 when the token step's all-reduces run as the library's own one-shot kernel over peer-mapped memory
 * (NVLink stores + tagged words), 0 when they go through NCCL (RG_B200_TP_ALLREDUCE=nccl, or a GPU pair
 * without peer access).  No counterpart in the reference. */
RG_API int rg_gpt_tp_fused(const rg_gpt* m);

/* Profiling aid of the persistent token-loop kernel (engine-only, nothing to mirror in the
 * reference): when enabled, the last token step of every rg_gpt_decode_run records device
 * timestamps per CTA and stage.  rg_gpt_trace_read returns rows of 12 uint64:
 * cta, op index, stage (0 QKV, 1 attention, 2 out-proj, 3 FC1, 4 FC2, 5 LM head), layer,
 * ns timestamps (stage start, input vector ready, dot products done, outputs stored), then SM
 * cycles spent waiting for weight/KV chunks and for the input vector, then two more ns timestamps:
 * all input words valid, chunk loop finished (0 where a stage does not record them). */
RG_API rg_status rg_gpt_trace_enable(rg_gpt* m, int on);
RG_API rg_status rg_gpt_trace_read(rg_gpt* m, uint64_t* out, size_t cap_rows, size_t* n_rows);

/* Test hook, no counterpart in the reference: makes the failure paths of the bounded device waits reachable without
 * a device fault.  what = 1 (ctx): raise the flag word that a tensor-core kernel's wait raises when it gives up, so
 * that the next synchronising call reports RG_ERR_TIMEOUT.  what = 2 (m): the persistent cluster kernel's head
 * cluster 0 withholds its partial vector of block `value` (-1: off), so every wait that depends on it runs out.
 * what = 3 (m): iteration limit of that kernel's waits (>= 1000).  what = 4 (m): form of the token loop (0 default,
 * 1 cluster kernel, 2 persistent kernel, 3 separate launches).  what = 5 (m): iteration limit of the persistent
 * kernel's waits (0: built-in).  what = 6 (m): CTA 0 of the persistent kernel withholds its q|k|v outputs of block
 * `value` (-1: off).  what = 7 (ctx): runs the tensor-parallel all-reduce kernel as rank 0 of 2 on this GPU with a
 * limit of `value` polls while nothing plays rank 1, and reports the RG_ERR_TIMEOUT that a missing peer produces.
 * what = 8 (ctx): self-check of the tensor-core projection kernel on a 40 x 200 product with K = `value` (a multiple of
 * 8 in 64..8192; a K that is not a multiple of the kernel's 64-wide k-blocks exercises the zero-filled last block),
 * both with its own epilogue and as raw k-split partial tiles, against a float64 dot product; RG_ERR_BACKEND with the
 * worst difference in rg_last_error() when it is off.  The unused handle may be NULL. */
RG_API rg_status rg_debug_hook(rg_ctx* ctx, rg_gpt* m, int what, long long value);

/* Diagnostic, no counterpart in the reference, touches no device: builds the op program the persistent token-loop
 * kernel would run for one tensor-parallel rank (tp_rank of tp_size; 1 for a single GPU) of a model shape
 * (hidden = 4 * d_model, head size d_model / heads) with `batch` sequences (1, 2 or 4) on a GPU with `sm_count` SMs, and
 * checks the properties the kernel relies on.  out[8]: context slices per head, most ops of a CTA, ring slots that fit,
 * shared-memory bytes, CTAs with LM-head work, packed weight bytes, ops in total, number of violations (a projection
 * column or an attention (sequence, head, slice) covered zero times or twice, a chunk larger than a ring slot, a residual
 * slice beyond its capacity).  0 ring slots: the program does not fit shared memory and the library would run the step as
 * separate launches instead.  RG_ERR_INVALID_INPUT / RG_ERR_UNSUPPORTED for shapes outside
 * the kernel's limits. */
RG_API rg_status rg_token_loop_plan(int d_model, int heads, int layers, int vocab, int tp_size, int tp_rank, int bf16, int batch,
                                    int sm_count, long long* out);

/* ---- allocation-free projection ------------------------------------------- */
/* No counterpart in the reference.  y[N] = x[K] . W[K,N] + bias[N] (bias may be NULL)
 * for a caller that cannot allocate device memory (inside a capture/replay region,
 * a latency-critical loop, or a host that owns the whole device heap): all four
 * pointers are DEVICE pointers the caller already owns, f32, W row-major and
 * 16-byte aligned with N a multiple of 4.  The split-k partial sums live in a fixed
 * 2 MiB array inside the library image (held by every GPU that loads the library
 * until exit), which limits N to 16384 and K to 32768; larger sizes return
 * RG_ERR_INVALID_INPUT.  Runs on the current device, on `stream` (a cudaStream_t that
 * belongs to the current device: the scratch address used is that device's).
 * The first call on each device also looks up the array's address: make that
 * call before any stream capture begins.  All calls share the array, so calls that
 * overlap on the GPU race; nothing in it needs clearing between calls.  Never calls
 * cudaMalloc / cudaFree or any allocating library routine. */
RG_API rg_status rg_linear_row_noalloc(const float* x, const float* W, const float* bias, float* y, size_t K,
                                       size_t N, void* stream);

/* ---- weight ingest from disk (the step before the path) -------------------- */
/* Names under which a safetensors file holds the model's tensors. */
typedef enum rg_names {
    RG_NAMES_AUTO = 0,   /* Hugging Face names if `wte.weight` is present, else the crate's */
    RG_NAMES_RUSTY = 1,  /* token_embedding.weight, position_embedding.weight, layer_{l}.attn.{q,k,v,out_proj}.weight
                          * (or the fused layer_{l}.attn.qkv.weight [D,3D] + attn.proj.weight), layer_{l}.ffn.fc{1,2}.weight,
                          * layer_{l}.ln{1,2}.{gamma,beta}, output_projection.weight: examples/serialization_demo.rs:24-101,
                          * examples/train_gpt_e2e.rs:146-160.  Optional: `.bias` of every projection (0 when absent),
                          * ln_f.{gamma,beta} (1 / 0 when absent) */
    RG_NAMES_HF_GPT2 = 2 /* wte, wpe, h.{l}.attn.c_attn / c_proj, h.{l}.ln_1 / ln_2, h.{l}.mlp.c_fc / c_proj, ln_f, with or
                          * without the `transformer.` prefix: src/models/hf_loader.rs:256-276.  c_attn [D,3D] is split into
                          * q | k | v; the LM head is lm_head.weight or the token table, transposed, with a zero bias */
} rg_names;

/* ModelMetadata {model_type, vocab_size, embedding_dim, num_layers, num_heads, block_size, dropout}
 * (src/serialization/mod.rs:28-37) from the sidecar `<weights>.safetensors.json` that save_model writes
 * (src/serialization/safetensors_format.rs:76-81) or from the "metadata" object of a JsonCheckpoint
 * (src/serialization/mod.rs:68-74).  Sets the five GptConfig fields of *cfg and leaves the others alone. */
RG_API rg_status rg_model_metadata_read(const char* path, rg_gpt_config* cfg);
/* load_model (src/serialization/safetensors_format.rs:89-138) + the copy into the model the reference never
 * finished (src/models/hf_loader.rs:290-296).  F32 tensors only (RG_ERR_SERIALIZATION otherwise, as :111-116);
 * a missing required tensor is RG_ERR_IO, a wrong shape RG_ERR_SHAPE.  `names` is an rg_names value. */
RG_API rg_status rg_gpt_load_safetensors(rg_gpt* m, const char* path, int names);
/* WasmGptTrainer::loadWeightsFromJson (src/wasm_api.rs:179-199): a JSON array of {shape, data} in parameters()
 * order, or a JsonCheckpoint {metadata, weights, step, loss} (src/serialization/mod.rs:52-74, :104-113). */
RG_API rg_status rg_gpt_load_json(rg_gpt* m, const char* path);

/* ---- tokenizers (text in / text out around the path; host code) ------------ */
typedef struct rg_tokenizer rg_tokenizer;
/* CharTokenizer::new(text): ids = rank among the sorted distinct characters (src/tokenization/char_tokenizer.rs:34-60) */
RG_API rg_status rg_tokenizer_char_from_text(const char* text_utf8, size_t len, rg_tokenizer** out);
/* CharTokenizer::from_vocab(&[char]): Unicode scalar values in id order (src/tokenization/char_tokenizer.rs:63-84) */
RG_API rg_status rg_tokenizer_char_from_vocab(const uint32_t* codepoints, size_t n, rg_tokenizer** out);
/* BPETokenizer::load (src/tokenization/bpe_tokenizer.rs:224-247): {token_to_id, id_to_token, merges, vocab_size} */
RG_API rg_status rg_tokenizer_bpe_load(const char* path, rg_tokenizer** out);
/* Tokenizer::vocab_size (src/tokenization/mod.rs) */
RG_API rg_status rg_tokenizer_vocab_size(const rg_tokenizer* t, size_t* out);
/* Tokenizer::encode (char_tokenizer.rs:95-100, bpe_tokenizer.rs:250-267).  *n_out receives the number of ids;
 * ids_out may be NULL to ask for it only; a too small `cap` or text that is not UTF-8 is RG_ERR_INVALID_INPUT. */
RG_API rg_status rg_tokenizer_encode(const rg_tokenizer* t, const char* text_utf8, size_t len, uint32_t* ids_out, size_t cap,
                                     size_t* n_out);
/* Tokenizer::decode (char_tokenizer.rs:102-107, bpe_tokenizer.rs:269-275); unknown ids are skipped.  UTF-8, not
 * NUL-terminated; *len_out receives the byte length; out may be NULL to ask for it only. */
RG_API rg_status rg_tokenizer_decode(const rg_tokenizer* t, const uint32_t* ids, size_t n, char* out, size_t cap, size_t* len_out);
RG_API void rg_tokenizer_free(rg_tokenizer* t);

#ifdef __cplusplus
}
#endif
#endif /* RG_B200_H */
