// rg_linear_row_noalloc: one row through a Linear layer, y = x.W + b, for callers
// that cannot allocate device memory.
//
// Who this is for: code that runs where cudaMalloc is off limits - inside a
// region that is being captured or replayed, inside a real-time loop that must
// not take the allocator's locks or trigger a device synchronisation, or under
// a host framework that owns the whole device heap and hands out fixed
// buffers.  Such a caller already owns x, W, b and y on the device; what it
// cannot supply is the temporary that the split-k projection kernel needs for
// its partial sums.  Here that temporary is a fixed array inside the library
// image instead of an allocation.
//
// Cost and limits: the array (RG_NOALLOC_SCRATCH_BYTES = 2 MiB) is part of the
// module, so every GPU that loads this library holds it until the process
// exits.  N (outputs) is limited to RG_NOALLOC_MAX_N and K (inputs) to
// RG_NOALLOC_MAX_K; larger sizes are refused, never truncated.
//
// Sharing: all calls on a device use the same array and it keeps whatever the
// previous call left in it.  Nothing here needs the array to start at zero -
// every slot that is read in a call was written earlier in that same call - so
// nothing is cleared.  Two calls that overlap on the GPU (different streams, or
// two host threads) race on the array and give wrong results: serialise them.
//
// Set-up: the first call on each device looks up the array's device address
// (cudaGetSymbolAddress) and caches it for that device.  Make that first call
// outside of any stream capture.
#include "rg_internal.cuh"
#include "rg_decode_kernels.cuh"

#define RG_NOALLOC_MAX_N 16384
#define RG_NOALLOC_MAX_K 32768
#define RG_NOALLOC_MAX_SPLIT 32
#define RG_NOALLOC_SCRATCH_BYTES (RG_NOALLOC_MAX_SPLIT * RG_NOALLOC_MAX_N * 4)
#define RG_NOALLOC_MAX_DEVICES 64

// In host code this name is only a handle for the symbol, not a device address:
// host code below obtains the address with cudaGetSymbolAddress.
static __device__ __align__(256) float rg_noalloc_scratch[RG_NOALLOC_MAX_SPLIT * RG_NOALLOC_MAX_N];

static float* g_scratch_addr[RG_NOALLOC_MAX_DEVICES];  // per device, filled on first use
static std::mutex g_scratch_mu;

// y[n] = bias[n] + sum over the k-splits of the partial dot products, fixed order.
static __global__ void rg_noalloc_finish_kernel(const float* __restrict__ parts, int nparts, int N,
                                                const float* __restrict__ bias, float* __restrict__ y) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    float v = bias ? bias[n] : 0.f;
    for (int s = 0; s < nparts; s++) v += parts[(size_t)s * N + n];
    y[n] = v;
}

extern "C" rg_status rg_linear_row_noalloc(const float* x, const float* W, const float* bias, float* y, size_t K,
                                           size_t N, void* stream) {
    if (!x || !W || !y) return rg_fail(RG_ERR_INVALID_INPUT, "rg_linear_row_noalloc: x, W and y must be device pointers");
    if (K == 0 || N == 0) return rg_fail(RG_ERR_INVALID_INPUT, "rg_linear_row_noalloc: K and N must be non-zero");
    if (N > RG_NOALLOC_MAX_N)
        return rg_fail(RG_ERR_INVALID_INPUT, "rg_linear_row_noalloc: N = %zu exceeds the built-in scratch limit of %d outputs", N,
                       RG_NOALLOC_MAX_N);
    if (K > RG_NOALLOC_MAX_K)
        return rg_fail(RG_ERR_INVALID_INPUT, "rg_linear_row_noalloc: K = %zu exceeds the limit of %d inputs", K,
                       RG_NOALLOC_MAX_K);
    if (N % 4 != 0 || (reinterpret_cast<uintptr_t>(W) & 15) != 0)
        return rg_fail(RG_ERR_INVALID_INPUT,
                       "rg_linear_row_noalloc: W must be 16-byte aligned with N a multiple of 4 (got N = %zu)", N);
    int dev = 0;
    RG_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= RG_NOALLOC_MAX_DEVICES) return rg_fail(RG_ERR_BACKEND, "device index %d not supported", dev);
    float* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_scratch_mu);
        if (!g_scratch_addr[dev]) {
            float* p = nullptr;
            cudaError_t e = cudaGetSymbolAddress((void**)&p, rg_noalloc_scratch);
            if (e != cudaSuccess || !p)
                return rg_fail(RG_ERR_BACKEND, "rg_linear_row_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev,
                               cudaGetErrorString(e));
            g_scratch_addr[dev] = p;
        }
        scratch = g_scratch_addr[dev];
    }
    // split of the k range: about one CTA per SM, at least 16 rows per split
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int ntiles = rg_cdiv((long long)N, 128);
    int ks = std::max(1, sms / ntiles);
    ks = std::min(ks, std::max(1, (int)(K / 16)));
    ks = std::max(ks, rg_cdiv((long long)K, 8192));  // a split's slice of x must fit the default 48 KB of shared memory
    ks = std::min(ks, RG_NOALLOC_MAX_SPLIT);
    int krows = (int)((rg_cdiv((long long)K, ks) + 7) / 8 * 8);
    ks = rg_cdiv((long long)K, krows);

    rg_gemv_args a;
    memset(&a, 0, sizeof(a));
    a.in.kind = RG_IN_REDUCE;
    a.in.base = x;  // the input row itself: no partials to sum, no bias, no post-op
    a.in.post = RG_POST_NONE;
    a.W = W, a.ldw = (long long)N, a.K = (int)K, a.N = (int)N, a.B = 1;
    a.ksplit = ks, a.krows = krows, a.out = scratch;
    cudaStream_t s = (cudaStream_t)stream;
    rg_gemv_kernel<float, 1><<<dim3(ntiles, ks, 1), 256, (size_t)krows * 4, s>>>(a);
    RG_CUDA(cudaGetLastError());
    rg_noalloc_finish_kernel<<<rg_cdiv((long long)N, 256), 256, 0, s>>>(scratch, ks, (int)N, bias, y);
    RG_CUDA(cudaGetLastError());
    return RG_OK;
}
