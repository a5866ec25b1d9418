// conv_tc_generic.cu -- one-CTA implicit-GEMM kernel, one TMA box per filter tap.
#include "conv_tc_common.cuh"

// ---------------------------------------------------------------------------
// generic kernel: one TMA box per filter tap and channel slice
// ---------------------------------------------------------------------------
template <int BN, int KC, bool CONTRACT, bool OUT_F32, int EPI>
__global__ void __launch_bounds__(TC_THREADS, 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const TcParams p)
{
    tc_pdl_trigger();
    extern __shared__ uint8_t smem_raw[];
    // stage ring must start on a 1024-byte boundary (swizzle atoms)
    // round up to 1024 bytes by pointer arithmetic on the __shared__ array (an integer round-trip
    // would hide the address space from the compiler and turn every table read into a generic load)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int A_BYTES = TC_TILE_M * KC;
    constexpr int B_BYTES = BN * KC;
    constexpr int SUB_BYTES = A_BYTES + B_BYTES;          // one K block: [A 128 x KC | B BN x KC]
    constexpr uint32_t TMEM_COLS = TC_NACC(BN) * BN;        // the whole accumulator ring: 512 columns
    constexpr uint32_t IDESC = idesc_i8(BN);

    float* tab = (float*)(smem + (size_t)p.stages * p.group * SUB_BYTES);       // [p.ntab][TC_MAX_COUT]
    uint8_t* lut = (uint8_t*)(tab + p.ntab * TC_MAX_COUT);                  // [BN][256] fused-BN table (lut_bytes may be 0)
    TcShared* sh = (TcShared*)(lut + p.lut_bytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int kblocks = p.taps * p.cin_blocks;

    tc_load_tables(tab, p);
    tc_load_lut(lut, p, (int)(blockIdx.x % p.tiles_n) * BN, BN);
    tc_setup(sh, p.stages, TMEM_COLS, warp, p.epi_wps);
    const uint32_t tmem_base = sh->tmem_base;
    volatile int* abort_flag = &sh->abort_flag;

    if (warp == 0) {
        const int G = p.group;
        {
            // TMA producer.  The whole warp runs the loop (lanes stay converged; a lone lane
            // looping while its 31 siblings sit at the final barrier was measured slower);
            // lanes 0 .. 2G-1 issue.  A pipeline stage holds G consecutive K blocks; lane 2g fetches the
            // activation box of block g, lane 2g+1 its weight box, all in ONE instruction (both
            // tensor maps are 4-D).  One barrier hand-shake per stage: the hand-shake, not the copy,
            // is what a single-thread loop pays for, so it is amortised over G blocks.  Each lane
            // carries its own (kh, kw, c0) forward by G blocks per step: no divisions in the loop.
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            const bool issuer = lane < 2 * G;
            const int g = issuer ? (lane >> 1) : 0;
            const bool is_a = (lane & 1) == 0;
            const CUtensorMap* map = is_a ? &mapA : &mapB;
            const uint32_t smem0 = smem_u32(smem) + (uint32_t)(g * SUB_BYTES) + (is_a ? 0u : (uint32_t)A_BYTES);
            const uint32_t full0 = smem_u32(&sh->full[0]), empty0 = smem_u32(&sh->empty[0]);
            const int stage_bytes = G * SUB_BYTES;
            const int n_steps = kblocks / G;
            const int tn = blockIdx.x % p.tiles_n;
            // this lane's first block of a tile: kb = g
            int c0_first = g * KC, kw_first = 0, kh_first = 0;
            while (c0_first >= p.Cp) { c0_first -= p.Cp; if (++kw_first == p.Kw) { kw_first = 0; kh_first++; } }
            // The weights do not depend on the previous kernel: the weight boxes of the first tile's
            // first steps (as many as the ring holds) are requested before the programmatic-dependency
            // wait, the activation boxes after it.  Each slot's byte count is armed here for both.
            int pre = 0;
            if ((int)blockIdx.x < p.total_tiles && !TC_DBG(p, 1)) {
                pre = n_steps < p.stages ? n_steps : p.stages;
                int c0 = c0_first, kw = kw_first, kh = kh_first;
#pragma unroll 1
                for (int it = 0; it < pre; it++) {
                    if (lane == 0) mbar_expect_tx(full0 + it * 8, G * SUB_BYTES);
                    __syncwarp();
                    if (issuer && !is_a)
                        tma_load_4d(smem0 + it * stage_bytes, map, full0 + it * 8, (kh * p.Kw + kw) * p.Cp + c0, tn * BN, 0, 0);
                    c0 += G * KC;
                    while (c0 >= p.Cp) { c0 -= p.Cp; if (++kw == p.Kw) { kw = 0; kh++; } }
                }
            }
            tc_pdl_wait();
            TileWalk wk;
            walk_init(wk, p, blockIdx.x / p.tiles_n, gridDim.x / p.tiles_n);
            for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x, walk_next(wk, p)) {
                const int tw = wk.tw, th = wk.th, tb = wk.tb;   // tb may be past the batch: TMA zero-fills
                const int x0 = tw * p.TW * p.stride - p.pad;
                const int y0 = th * p.TH * p.stride - p.pad;
                const int c3 = is_a ? tb * p.TB : 0;
                int c0 = c0_first, kw = kw_first, kh = kh_first;
#pragma unroll 1
                for (int it = 0; it < n_steps; it++) {
                    const bool first_fill = it < pre;          // slot is fresh and its weight box is on its way
                    if (!first_fill) {
                        ok = mbar_wait(empty0 + stage * 8, phase ^ 1, abort_flag, p.err, FFCU_ERR_EMPTY_TIMEOUT);
                        if (!ok) break;
                    }
                    if (TC_DBG(p, 1)) { if (lane == 0) mbar_arrive(full0 + stage * 8); }
                    else if (tile == (int)blockIdx.x && it == p.drop_stage) {
                        // armed by ffcu_test_arm_timeout for one launch: this step's data never arrives
                    } else {
                        if (!first_fill) {
                            if (lane == 0) mbar_expect_tx(full0 + stage * 8, G * SUB_BYTES);
                            __syncwarp();                       // the byte count is armed before any copy can land
                        }
                        const int tapk = (kh * p.Kw + kw) * p.Cp + c0;
                        if (issuer && (is_a || !first_fill))
                            tma_load_4d(smem0 + stage * stage_bytes, map, full0 + stage * 8,
                                        is_a ? c0 : tapk, is_a ? x0 + kw : tn * BN, is_a ? y0 + kh : 0, c3);
                    }
                    c0 += G * KC;
                    while (c0 >= p.Cp) { c0 -= p.Cp; if (++kw == p.Kw) { kw = 0; kh++; } }
                    if (++stage == p.stages) { stage = 0; phase ^= 1; }
                }
                pre = 0;
            }
        }
    } else if (warp == 1) {
        const int G = p.group;
        const int n_steps = kblocks / G;
        {
            // MMA issuer: the warp loops and waits together, lane 0 issues
            int stage = 0; uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            const int stage_bytes = G * SUB_BYTES;
            const uint32_t full0 = smem_u32(&sh->full[0]), empty0 = smem_u32(&sh->empty[0]);
            const uint64_t da0 = smem_desc<KC>(smem_u32(smem));
            const uint64_t db0 = smem_desc<KC>(smem_u32(smem) + A_BYTES);
            const uint32_t leader = (lane == 0) ? 1u : 0u;
            uint32_t ready = 0;                          // answer of the early test for the upcoming stage
            for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x, local++) {
                const int a = local % TC_NACC(BN);
                const uint32_t aphase = (uint32_t)(local / TC_NACC(BN)) & 1;
                ok = mbar_wait(smem_u32(&sh->acc_empty[a]), aphase ^ 1, abort_flag, p.err, FFCU_ERR_TMEM_TIMEOUT);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(a * BN);
#pragma unroll 1
                for (int it = 0; it < n_steps; it++) {
                    if (!ready) {
                        ok = mbar_wait(full0 + stage * 8, phase, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT, p.full_wait);
                        if (!ok) break;
                    }
                    // test the next stage now, use the answer next round
                    int ns = stage + 1; uint32_t np = phase;
                    if (ns == p.stages) { ns = 0; np ^= 1; }
                    ready = mbar_test(full0 + ns * 8, np);
                    tc_fence_after();
                    {
                        uint32_t soff = (uint32_t)((stage * stage_bytes) >> 4);
                        if (!TC_DBG(p, 2))
#pragma unroll 1
                        for (int g = 0; g < G; g++, soff += (uint32_t)(SUB_BYTES >> 4)) {
#pragma unroll
                            for (int k = 0; k < KC / 32; k++)
                                umma_i8_w(leader, d_tmem, da0 + (uint64_t)(soff + 2 * k), db0 + (uint64_t)(soff + 2 * k), IDESC, (it | g | k) ? 1u : 0u);
                        }
                        umma_commit_w(leader, empty0 + stage * 8);   // frees the stage once these MMAs have read it
                    }
                    stage = ns; phase = np;
                }
                if (ok) umma_commit_w(leader, smem_u32(&sh->acc_full[a]));
            }
        }
    } else {
        tc_pdl_wait();
        tc_epilogue_role<BN, CONTRACT, OUT_F32, EPI, (KC == 64 && EPI != EPI_RUNTIME && !OUT_F32)>(p, tab, lut, sh, tmem_base, abort_flag, warp, lane,
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
    return tc_launch_ex(kern, grid, smem, s, 1, mapA, mapB, prm);
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
