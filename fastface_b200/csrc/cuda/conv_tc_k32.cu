// conv_tc_k32.cu -- the stem convolution (3 -> 64 channels, 3x3) as a K = 32 tensor-core GEMM.
#include "conv_tc_common.cuh"

// ---------------------------------------------------------------------------
// The stem's K is 27 (3 channels x 9 taps): no TMA box can gather it from the image, so a
// CUDA-core pass (stem_pack_kernel) quantises the input and writes one 32-byte im2col row
// per output pixel ([kh][kw][c] bytes + 5 zeros).  This kernel multiplies those rows by the
// 64 x 32 weight matrix: per 128-pixel tile ONE TMA box {32 B, 128 rows} and ONE
// tcgen05.mma (128 x 64 x 32), then the shared epilogue (PReLU, requantise, fused BN).  The
// weights (2 KB) stay in shared memory; eight accumulators in TMEM; two issuer warps on alternate
// tiles; everything else (warp roles, barriers, bounded waits, teardown) as in the
// weight-stationary kernel.  The tile index space is the flat pixel index: the epilogue sees a
// 1 x n_pixels "image" (TW = 128, tiles_w = total tiles).
// ---------------------------------------------------------------------------
#define K32_A_BYTES (TC_TILE_M * 32)

template <bool CONTRACT, int EPI>
__global__ void __launch_bounds__(TC_THREADS, 1)
conv_k32_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const TcParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int BN = 64;
    constexpr int W_BYTES = BN * 32;
    constexpr uint32_t TMEM_COLS = TC_NACC(BN) * BN;
    constexpr uint32_t IDESC = idesc_i8(BN);

    uint8_t* s_w = smem;                                        // [64][32]
    uint8_t* s_a = smem + W_BYTES;                              // [stages][128][32]
    float* tab = (float*)(s_a + (size_t)p.stages * K32_A_BYTES);
    uint8_t* lut = (uint8_t*)(tab + p.ntab * TC_MAX_COUT);
    TcShared* sh = (TcShared*)(lut + p.lut_bytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    tc_load_tables(tab, p);
    tc_load_lut(lut, p, 0, BN);
    tc_setup(sh, p.stages, TMEM_COLS, warp, p.epi_wps);
    tc_pdl_sync();
    const uint32_t tmem_base = sh->tmem_base;
    volatile int* abort_flag = &sh->abort_flag;

    if (warp == 0) {
        const uint32_t wbar = smem_u32(&sh->w_full);
        if (lane == 0) {
            mbar_expect_tx(wbar, W_BYTES);
            tma_load_4d(smem_u32(s_w), &mapB, wbar, 0, 0, 0, 0);
        }
        __syncwarp();
        int stage = 0; uint32_t phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
            ok = mbar_wait(smem_u32(&sh->empty[stage]), phase ^ 1, abort_flag, p.err, FFCU_ERR_EMPTY_TIMEOUT);
            if (!ok) break;
            const uint32_t bar = smem_u32(&sh->full[stage]);
            if (lane == 0) {
                mbar_expect_tx(bar, K32_A_BYTES);
                tma_load_4d(smem_u32(s_a + (size_t)stage * K32_A_BYTES), &mapA, bar, 0, tile * TC_TILE_M, 0, 0);
            }
            __syncwarp();
            if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
    } else if (warp == 1 || warp == TC_ISSUER2_WARP) {
        const int me = (warp == 1) ? 0 : 1;
        bool ok = mbar_wait(smem_u32(&sh->w_full), 0, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT);
        tc_fence_after();
        const uint64_t dw = smem_desc_sw32(smem_u32(s_w));
        const uint32_t leader = (lane == 0) ? 1u : 0u;
        uint32_t ready_a = 0, ready_f = 0;
        for (int tile = blockIdx.x + me * gridDim.x, local = me; tile < p.total_tiles && ok; tile += 2 * gridDim.x, local += 2) {
            const int stage = local % p.stages;
            const uint32_t phase = (uint32_t)(local / p.stages) & 1;
            const int a = local % TC_NACC(BN);
            const uint32_t aphase = (uint32_t)(local / TC_NACC(BN)) & 1;
            if (!ready_a) {
                ok = mbar_wait(smem_u32(&sh->acc_empty[a]), aphase ^ 1, abort_flag, p.err, FFCU_ERR_TMEM_TIMEOUT);
                if (!ok) break;
            }
            if (!ready_f) {
                ok = mbar_wait(smem_u32(&sh->full[stage]), phase, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT, p.full_wait);
                if (!ok) break;
            }
            {
                const int nl = local + 2;
                ready_a = mbar_test(smem_u32(&sh->acc_empty[nl % TC_NACC(BN)]), ((uint32_t)(nl / TC_NACC(BN)) & 1) ^ 1);
                ready_f = mbar_test(smem_u32(&sh->full[nl % p.stages]), (uint32_t)(nl / p.stages) & 1);
            }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(a * BN);
            const uint64_t da = smem_desc_sw32(smem_u32(s_a + (size_t)stage * K32_A_BYTES));
            if (!TC_DBG(p, 2)) umma_i8_w(leader, d_tmem, da, dw, IDESC, 0u);
            umma_commit_w(leader, smem_u32(&sh->empty[stage]));
            umma_commit_w(leader, smem_u32(&sh->acc_full[a]));
        }
    } else {
        tc_epilogue_role<BN, CONTRACT, false, EPI>(p, tab, lut, sh, tmem_base, abort_flag, warp, lane,
                                                   blockIdx.x, gridDim.x, p.total_tiles, 1, 0, 0u);
    }
    tc_teardown(abort_flag, tmem_base, TMEM_COLS, warp);
}

template <bool CONTRACT, int EPI>
static int launch_k(int grid, int smem, cudaStream_t s, const CUtensorMap& mapA, const CUtensorMap& mapB, const TcParams& prm)
{
    auto kern = conv_k32_kernel<CONTRACT, EPI>;
    static int smem_set[64] = {};      // per device: the attribute belongs to the device's copy of the function
    int dev = 0;
    FFCU_CHECK(cudaGetDevice(&dev));
    if (smem_set[dev & 63] < smem) {
        FFCU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        smem_set[dev & 63] = smem;
    }
    return tc_launch_ex(kern, grid, smem, s, false, mapA, mapB, prm);
}

int tc_launch_k32(int mode, int epi, int grid, int smem, cudaStream_t s,
                  const CUtensorMap& mapA, const CUtensorMap& mapB, const TcParams& prm)
{
    if (!mode) return launch_k<false, EPI_RUNTIME>(grid, smem, s, mapA, mapB, prm);
    switch (epi) {
    case EPI_SLOPE_BN: return launch_k<true, EPI_SLOPE_BN>(grid, smem, s, mapA, mapB, prm);
    case EPI_SLOPE:    return launch_k<true, EPI_SLOPE>(grid, smem, s, mapA, mapB, prm);
    default:           return launch_k<true, EPI_RUNTIME>(grid, smem, s, mapA, mapB, prm);
    }
}
