// conv_tc_generic.cu -- one-CTA implicit-GEMM kernel, one TMA box per filter tap.
#include "conv_tc_common.cuh"

// ---------------------------------------------------------------------------
// generic kernel: one TMA box per filter tap and channel slice
// ---------------------------------------------------------------------------
template <int BN, int KC, bool CONTRACT, bool OUT_F32, int EPI>
__global__ void __launch_bounds__(TC_THREADS, 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const TcParams p)
{
    extern __shared__ uint8_t smem_raw[];
    // stage ring must start on a 1024-byte boundary (swizzle atoms)
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int A_BYTES = TC_TILE_M * KC;
    constexpr int B_BYTES = BN * KC;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;    // 128 / 256 / 512: powers of two
    constexpr uint32_t IDESC = idesc_i8(BN);

    float* tab = (float*)(smem + (size_t)p.stages * STAGE_BYTES);       // [TC_NTAB][TC_MAX_COUT]
    TcShared* sh = (TcShared*)(tab + TC_NTAB * TC_MAX_COUT);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int kblocks = p.taps * p.cin_blocks;

    tc_load_tables(tab, p);
    tc_setup(sh, p.stages, TMEM_COLS, warp);
    const uint32_t tmem_base = sh->tmem_base;
    volatile int* abort_flag = &sh->abort_flag;

    if (warp == 0) {
        if (lane == 0) {
            // TMA producer
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
                const int tn = tile % p.tiles_n;
                int m = tile / p.tiles_n;
                const int tw = m % p.tiles_w; m /= p.tiles_w;
                const int th = m % p.tiles_h;
                const int tb = m / p.tiles_h;
                const int x0 = tw * p.TW * p.stride - p.pad;
                const int y0 = th * p.TH * p.stride - p.pad;
                const int b0 = tb * p.TB;
                const int n0 = tn * BN;
                for (int kb = 0; kb < kblocks; kb++) {
                    ok = mbar_wait(smem_u32(&sh->empty[stage]), phase ^ 1, abort_flag, p.err, FFCU_ERR_EMPTY_TIMEOUT);
                    if (!ok) break;
                    const int tap = kb / p.cin_blocks;
                    const int c0 = (kb - tap * p.cin_blocks) * KC;
                    const int kh = tap / p.Kw, kw = tap - kh * p.Kw;
                    const uint32_t bar = smem_u32(&sh->full[stage]);
                    const uint32_t sa = smem_u32(smem + (size_t)stage * STAGE_BYTES);
                    mbar_expect_tx(bar, STAGE_BYTES);
                    tma_load_4d(sa, &mapA, bar, c0, x0 + kw, y0 + kh, b0);
                    tma_load_2d(sa + A_BYTES, &mapB, bar, tap * p.Cp + c0, n0);
                    if (++stage == p.stages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // MMA issuer
            int stage = 0; uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x, local++) {
                const int a = local & 1;
                const uint32_t aphase = (uint32_t)(local >> 1) & 1;
                ok = mbar_wait(smem_u32(&sh->acc_empty[a]), aphase ^ 1, abort_flag, p.err, FFCU_ERR_TMEM_TIMEOUT);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(a * BN);
                for (int kb = 0; kb < kblocks; kb++) {
                    ok = mbar_wait(smem_u32(&sh->full[stage]), phase, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + (size_t)stage * STAGE_BYTES);
                    const uint64_t da = smem_desc<KC>(sa);
                    const uint64_t db = smem_desc<KC>(sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < KC / 32; k++)
                        umma_i8(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), IDESC, (kb | k) ? 1u : 0u);
                    umma_commit(smem_u32(&sh->empty[stage]));   // frees the stage once these MMAs have read it
                    if (++stage == p.stages) { stage = 0; phase ^= 1; }
                }
                if (ok) umma_commit(smem_u32(&sh->acc_full[a]));
            }
        }
    } else {
        tc_epilogue_role<BN, CONTRACT, OUT_F32, EPI>(p, tab, sh, tmem_base, abort_flag, warp, lane,
                                                blockIdx.x, gridDim.x, p.total_tiles, 1, 0, 0u);
    }
    tc_teardown(abort_flag, tmem_base, TMEM_COLS, warp);
}


template <int BN, int KC, bool CONTRACT, bool F32, int EPI>
static int launch_g(int grid, int smem, cudaStream_t s, const CUtensorMap& mapA, const CUtensorMap& mapB, const TcParams& prm)
{
    auto kern = conv_tc_kernel<BN, KC, CONTRACT, F32, EPI>;
    static int smem_set[64] = {};      // per device: the attribute belongs to the device's copy of the function
    int dev = 0;
    FFCU_CHECK(cudaGetDevice(&dev));
    if (smem_set[dev & 63] < smem) {
        FFCU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        smem_set[dev & 63] = smem;
    }
    kern<<<grid, TC_THREADS, smem, s>>>(mapA, mapB, prm);
    FFCU_CHECK(cudaGetLastError());
    return 0;
}

template <int BN, int KC>
static int launch_g_bn(int mode, int epi, bool f32, int grid, int smem, cudaStream_t s,
                       const CUtensorMap& mapA, const CUtensorMap& mapB, const TcParams& prm)
{
    if (f32) return mode ? launch_g<BN, KC, true, true, EPI_PLAIN>(grid, smem, s, mapA, mapB, prm)
                         : launch_g<BN, KC, false, true, EPI_PLAIN>(grid, smem, s, mapA, mapB, prm);
    if (!mode) return launch_g<BN, KC, false, false, EPI_RUNTIME>(grid, smem, s, mapA, mapB, prm);
    switch (epi) {
    case EPI_PLAIN:  return launch_g<BN, KC, true, false, EPI_PLAIN>(grid, smem, s, mapA, mapB, prm);
    case EPI_SLOPE:  return launch_g<BN, KC, true, false, EPI_SLOPE>(grid, smem, s, mapA, mapB, prm);
    case EPI_RES_BN: return launch_g<BN, KC, true, false, EPI_RES_BN>(grid, smem, s, mapA, mapB, prm);
    case EPI_RES:    return launch_g<BN, KC, true, false, EPI_RES>(grid, smem, s, mapA, mapB, prm);
    default:         return launch_g<BN, KC, true, false, EPI_RUNTIME>(grid, smem, s, mapA, mapB, prm);
    }
}

int tc_launch_generic(int bn, int kc, int mode, int epi, bool f32, int grid, int smem, cudaStream_t s,
                      const CUtensorMap& mapA, const CUtensorMap& mapB, const TcParams& prm)
{
    if (kc == 128) {
        if (bn == 64) return launch_g_bn<64, 128>(mode, epi, f32, grid, smem, s, mapA, mapB, prm);
        if (bn == 128) return launch_g_bn<128, 128>(mode, epi, f32, grid, smem, s, mapA, mapB, prm);
        return launch_g_bn<256, 128>(mode, epi, f32, grid, smem, s, mapA, mapB, prm);
    }
    if (bn == 64) return launch_g_bn<64, 64>(mode, epi, f32, grid, smem, s, mapA, mapB, prm);
    if (bn == 128) return launch_g_bn<128, 64>(mode, epi, f32, grid, smem, s, mapA, mapB, prm);
    ffcu_set_error("no kernel for BN=%d with 64-byte K blocks", bn);
    return -1;
}
