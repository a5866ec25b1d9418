// peak_probe.cu -- measures what the tensor cores deliver for tcgen05.mma kind::i8 with
// operands already in shared memory (no global loads): the practical ceiling the
// convolution kernels are compared against.  One persistent CTA per SM issues `iters`
// rounds of four 128 x BN x 32 MMAs on the same two shared-memory tiles.
#include "conv_tc_common.cuh"

template <int BN>
__global__ void __launch_bounds__(128, 1) mma_peak_kernel(int iters, int* err)
{
    extern __shared__ uint8_t smem_raw[];
    // round up to 1024 bytes by pointer arithmetic on the __shared__ array (an integer round-trip
    // would hide the address space from the compiler and turn every table read into a generic load)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    __shared__ uint64_t done_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    constexpr int KC = 128;
    constexpr uint32_t IDESC = idesc_i8(BN);
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < (TC_TILE_M + BN) * KC / 4; i += blockDim.x) ((uint32_t*)smem)[i] = 0x01010101u * (i & 3);
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&done_bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"((uint32_t)BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    if (threadIdx.x == 0) {
        const uint64_t da = smem_desc<KC>(smem_u32(smem));
        const uint64_t db = smem_desc<KC>(smem_u32(smem) + TC_TILE_M * KC);
        for (int it = 0; it < iters; it++) {
#pragma unroll
            for (int k = 0; k < 4; k++) umma_i8(tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), IDESC, (it | k) ? 1u : 0u);
        }
        umma_commit(smem_u32(&done_bar));
        mbar_wait(smem_u32(&done_bar), 0, &abort_flag, err, FFCU_ERR_MMA_TIMEOUT);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)BN) : "memory");
    }
}

// Dense INT8 tensor throughput in TOP/s (2 ops per MAC) for M=128, N=bn, operands in shared
// memory, all SMs busy.  Returns 0 on success.
extern "C" int ffcu_i8_mma_peak(int device, int bn, int iters, float* tops, float* ms_out)
{
    if (!tops || iters < 1 || (bn != 64 && bn != 128 && bn != 256)) { ffcu_set_error("ffcu_i8_mma_peak: bad arguments"); return -1; }
    FFCU_CHECK(cudaSetDevice(device));
    int n_sm = 0;
    FFCU_CHECK(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, device));
    int* d_err = nullptr;
    FFCU_CHECK(cudaMalloc(&d_err, sizeof(int)));
    FFCU_CHECK(cudaMemset(d_err, 0, sizeof(int)));
    const int smem = (TC_TILE_M + bn) * 128 + 1024 + 4096;
    cudaEvent_t e0, e1;
    FFCU_CHECK(cudaEventCreate(&e0)); FFCU_CHECK(cudaEventCreate(&e1));
    float best = 1e30f;
    for (int rep = 0; rep < 4; rep++) {
        FFCU_CHECK(cudaEventRecord(e0));
        if (bn == 64) {
            FFCU_CHECK(cudaFuncSetAttribute(mma_peak_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            mma_peak_kernel<64><<<n_sm, 128, smem>>>(iters, d_err);
        } else if (bn == 128) {
            FFCU_CHECK(cudaFuncSetAttribute(mma_peak_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            mma_peak_kernel<128><<<n_sm, 128, smem>>>(iters, d_err);
        } else {
            FFCU_CHECK(cudaFuncSetAttribute(mma_peak_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            mma_peak_kernel<256><<<n_sm, 128, smem>>>(iters, d_err);
        }
        FFCU_CHECK(cudaEventRecord(e1));
        FFCU_CHECK(cudaEventSynchronize(e1));
        float ms = 0;
        FFCU_CHECK(cudaEventElapsedTime(&ms, e0, e1));
        if (rep > 0 && ms < best) best = ms;
    }
    int herr = 0;
    FFCU_CHECK(cudaMemcpy(&herr, d_err, sizeof(int), cudaMemcpyDeviceToHost));
    cudaFree(d_err); cudaEventDestroy(e0); cudaEventDestroy(e1);
    if (herr) { ffcu_set_error("peak probe: device error word %d", herr); return 1000 + herr; }
    const double ops = 2.0 * (double)n_sm * iters * 4.0 * TC_TILE_M * bn * 32.0;
    *tops = (float)(ops / (best * 1e-3) / 1e12);
    if (ms_out) *ms_out = best;
    return 0;
}
