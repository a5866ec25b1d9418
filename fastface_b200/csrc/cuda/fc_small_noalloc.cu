// fc_small_noalloc.cu -- the small-batch FC for callers that must not allocate.
//
// Who this is for: code that runs where cudaMalloc / cudaFree are off the table -- inside a
// latency-critical serving loop that cannot take the implicit device-wide synchronisation an
// allocation brings, inside a host callback or a plug-in that is handed device buffers but
// no allocator, or in a process whose memory budget is fixed up front.  Such a caller owns
// its input and output buffers already; what it cannot supply is the split-K kernel's
// int32 accumulator.  Here that accumulator is a fixed array in the library's own device
// image, so the call allocates nothing at all.
//
// Limits and sharing rules:
//   * batch <= 16 and N <= 512 (the array is 64 ticket counters + 16 x 512 int32 sums = 32.25 KiB;
//     every GPU that loads the library carries it until the process exits);
//   * all calls on one device share the one array.  It is cleared at the start of each call
//     on the caller's stream, so calls issued back to back on one stream are fine, but two
//     calls that can overlap on the GPU (different streams, different host threads) race on it;
//   * the first call on a device looks up the array's device address (a one-time set-up with
//     that device current).  Make that first call outside any stream capture.
//   * the kernel reads act and w sixteen bytes at a time: both pointers must be 16-byte aligned,
//     K a positive multiple of 16 (so every row keeps that alignment) and N a multiple of 8;
//     w_scale, bias and out must be 4-byte aligned.  All of this is checked on the host before
//     anything is launched: a sliced or offset buffer is refused (-1), never faulted on.

#include "ffcu_internal.cuh"

#define FC_NOALLOC_MAX_BATCH 16
#define FC_NOALLOC_MAX_N 512
#define FC_NOALLOC_MAX_DEVICES 64

// The split-K accumulator.  In host code this name is only a handle for the symbol, not a
// device address: the address each device gives it comes from cudaGetSymbolAddress below.
static __device__ __align__(256) int g_fc_noalloc_scratch[FFCU_FC_SMALL_TICKETS + FC_NOALLOC_MAX_BATCH * FC_NOALLOC_MAX_N];

static int* g_scratch_addr[FC_NOALLOC_MAX_DEVICES];   // per device, filled on first use

// Device code may name the array directly; this kernel zeroes the part a call will use.
static __global__ void fc_noalloc_clear_kernel(int n)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) g_fc_noalloc_scratch[i] = 0;
}

// Small-batch FC without any allocation: out[b][n] = bias[n] + (float)dot(act[b], w[n]) * w_scale[n].
// All pointers are DEVICE pointers owned by the caller: act int8 [batch][K], w int8 [N][K],
// w_scale / bias f32 [N], out f32 [batch][N].  mode: 0 strict, 1 contract (as ffcu_set_mode).
// stream: a cudaStream_t passed as void* (NULL = the default stream).  Returns 0, or a negative
// code with the reason in ffcu_last_error().
extern "C" int ffcu_fc_small_noalloc(const int8_t* act, const int8_t* w, const float* w_scale, const float* bias,
                                     int batch, int N, int K, int mode, float* out, void* stream)
{
    if (!act || !w || !w_scale || !bias || !out) { ffcu_set_error("ffcu_fc_small_noalloc: NULL pointer"); return -1; }
    if (batch < 1 || batch > FC_NOALLOC_MAX_BATCH || N < 1 || N > FC_NOALLOC_MAX_N) {
        ffcu_set_error("ffcu_fc_small_noalloc: batch %d / N %d exceed the built-in accumulator (batch <= %d, N <= %d); "
                       "use the allocating path (fastface_embed_batch) for larger problems",
                       batch, N, FC_NOALLOC_MAX_BATCH, FC_NOALLOC_MAX_N);
        return -2;
    }
    if (mode != 0 && mode != 1) { ffcu_set_error("ffcu_fc_small_noalloc: mode must be 0 or 1"); return -1; }
    if (K < 16 || K % 16 != 0 || N % 8 != 0) {
        ffcu_set_error("ffcu_fc_small_noalloc: K = %d must be a positive multiple of 16 and N = %d a multiple of 8", K, N);
        return -1;
    }
    if ((((uintptr_t)act | (uintptr_t)w) & 15u) != 0) {
        ffcu_set_error("ffcu_fc_small_noalloc: act and w must be 16-byte aligned (the kernel reads them 16 bytes at a time)");
        return -1;
    }
    if ((((uintptr_t)w_scale | (uintptr_t)bias | (uintptr_t)out) & 3u) != 0) {
        ffcu_set_error("ffcu_fc_small_noalloc: w_scale, bias and out must be 4-byte aligned");
        return -1;
    }
    int dev = -1;
    FFCU_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= FC_NOALLOC_MAX_DEVICES) { ffcu_set_error("ffcu_fc_small_noalloc: device ordinal %d not supported", dev); return -3; }
    if (!g_scratch_addr[dev]) {
        // one-time set-up for this device (it is the current one): resolve the symbol to the
        // address it has on this GPU
        int* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&p, g_fc_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            ffcu_set_error("ffcu_fc_small_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return -100;
        }
        g_scratch_addr[dev] = p;
    }
    int* scratch = g_scratch_addr[dev];
    cudaStream_t s = (cudaStream_t)stream;
    // the array keeps whatever the last call (or an aborted one) left: start from zero
    const int used = FFCU_FC_SMALL_TICKETS + batch * N;    // ticket counters, then the sums this call adds into
    fc_noalloc_clear_kernel<<<(used + 255) / 256, 256, 0, s>>>(used);
    FFCU_CHECK(cudaGetLastError());
    return ffcu_launch_fc_small(act, w, w_scale, bias, batch, N, K, mode, scratch, out, s);
}
