// conv_tc_ws.cu -- weight-stationary implicit-GEMM kernel for the 64-input-channel layers.
#include "conv_tc_common.cuh"

// ---------------------------------------------------------------------------
// weight-stationary kernel for the 64-input-channel 3x3 stride-1 layers
// (112x112 and 56x56 maps: 20% of the network's MACs but, tap by tap, its largest
// shared-memory fill traffic).
//   * all 9 weight taps ([tap][BN rows][64 B], 36 KB or 72 KB) are loaded once per CTA
//     and stay in shared memory for every tile the CTA processes;
//   * output tile = 8 wide x 16 high pixels of one image.  Per tile ONE box
//     {64 B, 10, 18, 1} is loaded: columns x0-1 .. x0+8, rows y0-1 .. y0+16.  An 8-row
//     swizzle group of the A operand is one image row of the tile, groups are 10 lines
//     (640 B) apart, and tap (kh, kw) is the same buffer read from descriptor start
//     + (kh * 10 + kw) * 64 B.  Activation bytes fetched per tile drop from 9 x 128 to
//     180 rows of 64 B.
// ---------------------------------------------------------------------------

template <int BN, bool CONTRACT, int EPI>
__global__ void __launch_bounds__(TC_THREADS, 1)
conv_ws_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const TcParams p)
{
    tc_pdl_trigger();
    extern __shared__ uint8_t smem_raw[];
    // round up to 1024 bytes by pointer arithmetic on the __shared__ array (an integer round-trip
    // would hide the address space from the compiler and turn every table read into a generic load)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int KC = 64;
    constexpr int W_TAP_BYTES = BN * KC;
    constexpr int W_BYTES = 9 * W_TAP_BYTES;
    constexpr uint32_t TMEM_COLS = TC_NACC(BN) * BN;
    constexpr uint32_t IDESC = idesc_i8(BN);

    uint8_t* s_w = smem;                                        // [9][BN][64]
    uint8_t* s_a = smem + W_BYTES;                              // [stages][3][144][64]
    float* tab = (float*)(s_a + (size_t)p.stages * WS_A_BYTES);
    uint8_t* lut = (uint8_t*)(tab + p.ntab * TC_MAX_COUT);                  // [BN][256] fused-BN table (lut_bytes may be 0)
    TcShared* sh = (TcShared*)(lut + p.lut_bytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    tc_load_tables(tab, p);
    tc_load_lut(lut, p, 0 * BN, BN);
    tc_setup(sh, p.stages, TMEM_COLS, warp, p.epi_wps);
    tc_pdl_wait();
    const uint32_t tmem_base = sh->tmem_base;
    volatile int* abort_flag = &sh->abort_flag;

    if (warp == 0) {
        {
            // the warp loops and waits together (lanes stay converged); lanes 0..8 fetch one weight tap each, lane 0 the boxes
            const uint32_t wbar = smem_u32(&sh->w_full);
            if (lane == 0) mbar_expect_tx(wbar, W_BYTES);
            __syncwarp();
            if (lane < 9) tma_load_4d(smem_u32(s_w + lane * W_TAP_BYTES), &mapB, wbar, lane * p.Cp, 0, 0, 0);
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            TileWalk wk;
            walk_init(wk, p, blockIdx.x, gridDim.x);
            for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x, walk_next(wk, p)) {
                const int tw = wk.tw, th = wk.th, b = wk.tb;
                ok = mbar_wait(smem_u32(&sh->empty[stage]), phase ^ 1, abort_flag, p.err, FFCU_ERR_EMPTY_TIMEOUT);
                if (!ok) break;
                const uint32_t bar = smem_u32(&sh->full[stage]);
                const uint32_t sa = smem_u32(s_a + (size_t)stage * WS_A_BYTES);
                if (TC_DBG(p, 1)) { if (lane == 0) mbar_arrive(bar); if (++stage == p.stages) { stage = 0; phase ^= 1; } continue; }
                if (lane == 0) {
                    mbar_expect_tx(bar, WS_BOX_ROWS * 64);
                    tma_load_4d(sa, &mapA, bar, 0, tw * WS_TW - 1, th * WS_TH - 1, b);
                }
                __syncwarp();
                if (++stage == p.stages) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1 || warp == TC_ISSUER2_WARP) {
        {
            // Two MMA issuers take alternate tiles: a tile is 18 short MMAs (128 x BN x 32), and one
            // thread cannot issue them as fast as the tensor pipe retires them.  Each issuer derives
            // its ring positions from the tile's index, so the two never touch the same stage or
            // accumulator.  The warp loops and waits together, lane 0 issues.
            const int me = (warp == 1) ? 0 : 1;
            bool ok = mbar_wait(smem_u32(&sh->w_full), 0, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT);
            tc_fence_after();
            const uint64_t dw = smem_desc<KC>(smem_u32(s_w));
            const uint32_t leader = (lane == 0) ? 1u : 0u;
            uint32_t ready_a = 0, ready_f = 0;           // answers of the early tests for this issuer's next tile
            // ring positions carried forward by additions (both rings are even: +2 keeps this issuer on its own slots)
            const int stages = p.stages;
            int stage = me; uint32_t phase = 0;
            int a = me; uint32_t aphase = 0;
            for (int tile = blockIdx.x + me * gridDim.x; tile < p.total_tiles && ok; tile += 2 * gridDim.x) {
                if (!ready_a) {
                    ok = mbar_wait(smem_u32(&sh->acc_empty[a]), aphase ^ 1, abort_flag, p.err, FFCU_ERR_TMEM_TIMEOUT);
                    if (!ok) break;
                }
                if (!ready_f) {
                    ok = mbar_wait(smem_u32(&sh->full[stage]), phase, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT, p.full_wait);
                    if (!ok) break;
                }
                int ns = stage + 2; uint32_t np = phase;
                if (ns >= stages) { ns -= stages; np ^= 1; }
                int na = a + 2; uint32_t nap = aphase;
                if (na >= TC_NACC(BN)) { na -= TC_NACC(BN); nap ^= 1; }
                // test the barriers of this issuer's next tile now, use the answers next round
                ready_a = mbar_test(smem_u32(&sh->acc_empty[na]), nap ^ 1);
                ready_f = mbar_test(smem_u32(&sh->full[ns]), np);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(a * BN);
                const uint64_t da0 = smem_desc_sbo<KC>(smem_u32(s_a + (size_t)stage * WS_A_BYTES), WS_PITCH * 64);
                {
                if (!TC_DBG(p, 2))
#pragma unroll
                for (int kw = 0; kw < 3; kw++)
#pragma unroll
                    for (int kh = 0; kh < 3; kh++) {
                        // tap (kh, kw): start = (kh * pitch + kw) lines of 64 B (>> 4)
                        const uint64_t da = da0 + (uint64_t)(((kh * WS_PITCH + kw) * 64) >> 4);
                        const uint64_t db = dw + (uint64_t)(((kh * 3 + kw) * W_TAP_BYTES) >> 4);
#pragma unroll
                        for (int k = 0; k < 2; k++)
                            umma_i8_w(leader, d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), IDESC, (kw | kh | k) ? 1u : 0u);
                    }
                umma_commit_w(leader, smem_u32(&sh->empty[stage]));
                umma_commit_w(leader, smem_u32(&sh->acc_full[a]));
                }
                stage = ns; phase = np; a = na; aphase = nap;
            }
        }
    } else {
        tc_epilogue_role<BN, CONTRACT, false, EPI, (EPI != EPI_RUNTIME)>(p, tab, lut, sh, tmem_base, abort_flag, warp, lane,
                                             blockIdx.x, gridDim.x, p.total_tiles, 1, 0, 0u);
    }
    tc_teardown(abort_flag, tmem_base, TMEM_COLS, warp);
}



template <int BN, bool CONTRACT, int EPI>
static int launch_w(int grid, int smem, cudaStream_t s, const CUtensorMap& mapA, const CUtensorMap& mapB, const TcParams& prm)
{
    auto kern = conv_ws_kernel<BN, CONTRACT, EPI>;
    static int smem_set[64] = {};      // per device: the attribute belongs to the device's copy of the function
    int dev = 0;
    FFCU_CHECK(cudaGetDevice(&dev));
    if (smem_set[dev & 63] < smem) {
        FFCU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        smem_set[dev & 63] = smem;
    }
    return tc_launch_ex(kern, grid, smem, s, 1, mapA, mapB, prm);
}

template <int BN>
static int launch_w_bn(int mode, int epi, int grid, int smem, cudaStream_t s,
                       const CUtensorMap& mapA, const CUtensorMap& mapB, const TcParams& prm)
{
    if (!mode) return launch_w<BN, false, EPI_RUNTIME>(grid, smem, s, mapA, mapB, prm);
    switch (epi) {
    case EPI_PLAIN:  return launch_w<BN, true, EPI_PLAIN>(grid, smem, s, mapA, mapB, prm);
    case EPI_SLOPE:  return launch_w<BN, true, EPI_SLOPE>(grid, smem, s, mapA, mapB, prm);
    case EPI_RES_BN: return launch_w<BN, true, EPI_RES_BN>(grid, smem, s, mapA, mapB, prm);
    case EPI_RES:    return launch_w<BN, true, EPI_RES>(grid, smem, s, mapA, mapB, prm);
    default:         return launch_w<BN, true, EPI_RUNTIME>(grid, smem, s, mapA, mapB, prm);
    }
}

int tc_launch_ws(int bn, int mode, int epi, int grid, int smem, cudaStream_t s,
                 const CUtensorMap& mapA, const CUtensorMap& mapB, const TcParams& prm)
{
    if (bn == 64) return launch_w_bn<64>(mode, epi, grid, smem, s, mapA, mapB, prm);
    return launch_w_bn<128>(mode, epi, grid, smem, s, mapA, mapB, prm);
}
