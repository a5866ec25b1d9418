// peak_probe.cu -- measures what the tensor cores deliver for tcgen05.mma kind::i8 with
// operands already in shared memory (no global loads): the practical ceiling the
// convolution kernels are compared against.  One persistent CTA per SM issues `iters`
// rounds of four 128 x BN x 32 MMAs on the same two shared-memory tiles.
#include "conv_tc_common.cuh"

// wait flavours for the hand-shake experiment: 0 = the kernels' bounded try_wait loop,
// 1 = non-blocking test_wait spin, 2 = try_wait with a zero suspend-time hint
__device__ __forceinline__ void probe_wait(int flavour, uint32_t bar, uint32_t parity, int* abort_flag, int* err)
{
    if (flavour == 0) { mbar_wait(bar, parity, abort_flag, err, FFCU_ERR_MMA_TIMEOUT); return; }
    for (int i = 0; i < 100000000; i++) {
        uint32_t ok;
        if (flavour == 1)
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        else
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(ok) : "r"(bar), "r"(parity), "r"(0u) : "memory");
        if (ok) return;
    }
    *abort_flag = 1;
}

template <int BN>
__global__ void __launch_bounds__(608, 1) mma_peak_kernel(int iters, int* err, int mode)
{
    extern __shared__ uint8_t smem_raw[];
    // round up to 1024 bytes by pointer arithmetic on the __shared__ array (an integer round-trip
    // would hide the address space from the compiler and turn every table read into a generic load)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    __shared__ uint64_t done_bar;
    __shared__ uint64_t scratch_bar;
    __shared__ uint64_t ring_full[16], ring_empty[16];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    constexpr int KC = 128;
    constexpr uint32_t IDESC = idesc_i8(BN);
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < (TC_TILE_M + BN) * KC / 4; i += blockDim.x) ((uint32_t*)smem)[i] = 0x01010101u * (i & 3);
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&done_bar), 1);
        mbar_init(smem_u32(&scratch_bar), 1);
        for (int i = 0; i < 16; i++) { mbar_init(smem_u32(&ring_full[i]), 1); mbar_init(smem_u32(&ring_empty[i]), 1); }
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
        if (mode == 0) {
            for (int it = 0; it < iters; it++) {
#pragma unroll
                for (int k = 0; k < 4; k++) umma_i8(tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), IDESC, (it | k) ? 1u : 0u);
            }
        } else if (mode & 1024) {
            // bit 10: the single-thread ring, with each round's barrier test issued one round early so
            // its latency overlaps the MMA issue of the round before
            const int nst = (mode & 128) ? 8 : ((mode & 256) ? 16 : 4);
            int stage = 0; uint32_t phase = 0;
            uint32_t ready = 1;
            for (int it = 0; it < iters; it++) {
                if (!ready) probe_wait(0, smem_u32(&ring_empty[stage]), phase ^ 1, &abort_flag, err);
                // test the NEXT stage now, consume the answer next round
                int ns = stage + 1; uint32_t np = phase; if (ns == nst) { ns = 0; np ^= 1; }
                uint32_t nr = 1;
                if (it + 1 >= nst)
                    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                                 : "=r"(nr) : "r"(smem_u32(&ring_empty[ns])), "r"(np ^ 1) : "memory");
                const uint32_t off = (uint32_t)((stage & 3) * 64);
#pragma unroll
                for (int k = 0; k < 4; k++) umma_i8(tmem, da + (uint64_t)(off + 2 * k), db + (uint64_t)(off + 2 * k), IDESC, (it | k) ? 1u : 0u);
                umma_commit(smem_u32(&ring_empty[stage]));
                ready = nr;
                stage = ns; phase = np;
            }
        } else if (mode & 8) {
            // bit 3: the convolution kernels' stage hand-shake, four stages, no copies: a second
            // thread waits for a stage to be released by the commit and marks it full again
            int stage = 0; uint32_t phase = 0;
            const int nst = (mode & 128) ? 8 : ((mode & 256) ? 16 : 4);     // bits 7, 8: ring of 8 / 16 stages
            for (int it = 0; it < iters; it++) {
                // bit 9: no second thread; the issuer itself waits for the commit of the round that used this stage last
                if (mode & 512) { if (it >= nst) probe_wait((mode >> 4) & 3, smem_u32(&ring_empty[stage]), phase ^ 1, &abort_flag, err); }
                else probe_wait((mode >> 4) & 3, smem_u32(&ring_full[stage]), phase, &abort_flag, err);
                if (!(mode & 64)) tc_fence_after();       // bit 6: no tcgen05 fence after the wait
                const uint32_t off = (uint32_t)((stage & 3) * 64);
#pragma unroll
                for (int k = 0; k < 4; k++) umma_i8(tmem, da + (uint64_t)(off + 2 * k), db + (uint64_t)(off + 2 * k), IDESC, (it | k) ? 1u : 0u);
                umma_commit(smem_u32(&ring_empty[stage]));
                if (++stage == nst) { stage = 0; phase ^= 1; }
            }
        } else {
            // issue-pattern experiments ($FF_PROBE_MODE): bit 0 = the descriptors move from round to
            // round as a stage ring's would, bit 1 = one commit per round on a scratch barrier
            int stage = 0;
            for (int it = 0; it < iters; it++) {
                const uint32_t off = (mode & 1) ? (uint32_t)(stage * 64) : 0u;
#pragma unroll
                for (int k = 0; k < 4; k++) umma_i8(tmem, da + (uint64_t)(off + 2 * k), db + (uint64_t)(off + 2 * k), IDESC, (it | k) ? 1u : 0u);
                if (mode & 2) umma_commit(smem_u32(&scratch_bar));
                if (++stage == 4) stage = 0;
            }
        }
        umma_commit(smem_u32(&done_bar));
        mbar_wait(smem_u32(&done_bar), 0, &abort_flag, err, FFCU_ERR_MMA_TIMEOUT);
    } else if (threadIdx.x == 32 && (mode & 8) && !(mode & 512)) {
        int stage = 0; uint32_t phase = 0;
        const int nst = (mode & 128) ? 8 : ((mode & 256) ? 16 : 4);
        for (int it = 0; it < iters; it++) {
            probe_wait((mode >> 4) & 3, smem_u32(&ring_empty[stage]), phase ^ 1, &abort_flag, err);
            mbar_arrive(smem_u32(&ring_full[stage]));
            if (++stage == nst) { stage = 0; phase ^= 1; }
        }
    } else if (warp >= 4) {
        // bit 2 of the mode launches 15 more warps that poll the completion barrier the way the
        // convolution kernels' epilogue warps poll for an accumulator
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
    const char* me = getenv("FF_PROBE_MODE");
    const int mode = me ? atoi(me) : 0;
    cudaEvent_t e0, e1;
    FFCU_CHECK(cudaEventCreate(&e0)); FFCU_CHECK(cudaEventCreate(&e1));
    float best = 1e30f;
    for (int rep = 0; rep < 4; rep++) {
        FFCU_CHECK(cudaEventRecord(e0));
        if (bn == 64) {
            FFCU_CHECK(cudaFuncSetAttribute(mma_peak_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            mma_peak_kernel<64><<<n_sm, (mode & 4) ? 608 : 128, smem>>>(iters, d_err, mode);
        } else if (bn == 128) {
            FFCU_CHECK(cudaFuncSetAttribute(mma_peak_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            mma_peak_kernel<128><<<n_sm, (mode & 4) ? 608 : 128, smem>>>(iters, d_err, mode);
        } else {
            FFCU_CHECK(cudaFuncSetAttribute(mma_peak_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            mma_peak_kernel<256><<<n_sm, (mode & 4) ? 608 : 128, smem>>>(iters, d_err, mode);
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
