// TEST INFRASTRUCTURE, not product code: host launchers around the reference's OWN CUDA kernels
// (src/backend/cuda_kernels.cu of the reference tree), compiled IN PLACE from where that file lies: the include below
// resolves through the -I path oracle/build_ref.py passes, nothing of the reference is copied into this repository.
// Launch shapes follow the reference's wrapper (src/backend/cuda_kernels_wrapper.rs:109-126: 256 threads per block,
// ceil(n / 256) blocks for the elementwise kernels; :228-252: one block of 256 threads per row and 2 KB of dynamic
// shared memory for softmax and layernorm).  Used by tests/ only: op-level outputs of the reference's kernels on this
// GPU pin the library's ops, and their device time is measured beside the library's.
#include "cuda_kernels.cu"

#include <cuda_runtime.h>

#define REF_API extern "C" __attribute__((visibility("default")))

static inline int ref_blocks(int n) { return (n + 255) / 256; }

// kind: 0 add, 1 mul, 2 sub (a, b -> out); 3 relu, 4 sigmoid, 5 gelu, 6 exp, 7 log (a -> out); 8 softmax rows,
// 9 layernorm rows (a = input, b = gamma, c = beta).  Returns a cudaError_t.
static int ref_launch(int kind, const float* a, const float* b, const float* c, float* out, int batch, int n, float eps,
                      cudaStream_t s) {
    const int total = batch * n;
    switch (kind) {
        case 0: elementwise_add<<<ref_blocks(total), 256, 0, s>>>(a, b, out, total); break;
        case 1: elementwise_mul<<<ref_blocks(total), 256, 0, s>>>(a, b, out, total); break;
        case 2: elementwise_sub<<<ref_blocks(total), 256, 0, s>>>(a, b, out, total); break;
        case 3: relu_forward<<<ref_blocks(total), 256, 0, s>>>(a, out, total); break;
        case 4: sigmoid_forward<<<ref_blocks(total), 256, 0, s>>>(a, out, total); break;
        case 5: gelu_forward<<<ref_blocks(total), 256, 0, s>>>(a, out, total); break;
        case 6: exp_forward<<<ref_blocks(total), 256, 0, s>>>(a, out, total); break;
        case 7: log_forward<<<ref_blocks(total), 256, 0, s>>>(a, out, total); break;
        case 8: softmax_forward<<<batch, 256, 512 * sizeof(float), s>>>(a, out, batch, n); break;
        case 9: layernorm_forward<<<batch, 256, 512 * sizeof(float), s>>>(a, b, c, out, batch, n, eps); break;
        default: return (int)cudaErrorInvalidValue;
    }
    return (int)cudaGetLastError();
}

// Host arrays in, host array out (sizes: a, out = batch * n; b = batch * n for kinds 0-2, n for kind 9; c = n).
REF_API int ref_run(int kind, const float* a, const float* b, const float* c, float* out, int batch, int n, float eps) {
    if (batch <= 0 || n <= 0 || (long long)batch * n > (1ll << 28)) return (int)cudaErrorInvalidValue;
    const size_t bytes = (size_t)batch * n * sizeof(float);
    const size_t bbytes = kind <= 2 ? bytes : (size_t)n * sizeof(float);
    float *da = nullptr, *db = nullptr, *dc = nullptr, *dout = nullptr;
    cudaError_t e = cudaMalloc(&da, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&dout, bytes);
    if (e == cudaSuccess && b) e = cudaMalloc(&db, bbytes);
    if (e == cudaSuccess && c) e = cudaMalloc(&dc, (size_t)n * sizeof(float));
    if (e == cudaSuccess) e = cudaMemcpy(da, a, bytes, cudaMemcpyHostToDevice);
    if (e == cudaSuccess && b) e = cudaMemcpy(db, b, bbytes, cudaMemcpyHostToDevice);
    if (e == cudaSuccess && c) e = cudaMemcpy(dc, c, (size_t)n * sizeof(float), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = (cudaError_t)ref_launch(kind, da, db, dc, dout, batch, n, eps, 0);
    if (e == cudaSuccess) e = cudaMemcpy(out, dout, bytes, cudaMemcpyDeviceToHost);
    cudaFree(da), cudaFree(db), cudaFree(dc), cudaFree(dout);
    return (int)e;
}

// Device time of `iters` launches on synthetic device data (ms per launch in *ms); inputs are filled once with a ramp.
REF_API int ref_time(int kind, int batch, int n, int iters, float* ms) {
    if (batch <= 0 || n <= 0 || iters <= 0 || (long long)batch * n > (1ll << 28)) return (int)cudaErrorInvalidValue;
    const size_t count = (size_t)batch * n, bytes = count * sizeof(float);
    float *da = nullptr, *db = nullptr, *dc = nullptr, *dout = nullptr;
    float* h = (float*)malloc(bytes);
    if (!h) return (int)cudaErrorMemoryAllocation;
    for (size_t i = 0; i < count; i++) h[i] = 0.25f + (float)(i % 1013) * (1.0f / 1013.0f);
    cudaError_t e = cudaMalloc(&da, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&db, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&dc, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&dout, bytes);
    if (e == cudaSuccess) e = cudaMemcpy(da, h, bytes, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(db, h, bytes, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(dc, h, bytes, cudaMemcpyHostToDevice);
    free(h);
    cudaEvent_t t0 = nullptr, t1 = nullptr;
    if (e == cudaSuccess) e = cudaEventCreate(&t0);
    if (e == cudaSuccess) e = cudaEventCreate(&t1);
    for (int w = 0; w < 3 && e == cudaSuccess; w++) e = (cudaError_t)ref_launch(kind, da, db, dc, dout, batch, n, 1e-5f, 0);
    if (e == cudaSuccess) e = cudaEventRecord(t0, 0);
    for (int i = 0; i < iters && e == cudaSuccess; i++) e = (cudaError_t)ref_launch(kind, da, db, dc, dout, batch, n, 1e-5f, 0);
    if (e == cudaSuccess) e = cudaEventRecord(t1, 0);
    if (e == cudaSuccess) e = cudaEventSynchronize(t1);
    float total = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&total, t0, t1);
    *ms = total / (float)iters;
    if (t0) cudaEventDestroy(t0);
    if (t1) cudaEventDestroy(t1);
    cudaFree(da), cudaFree(db), cudaFree(dc), cudaFree(dout);
    return (int)e;
}
