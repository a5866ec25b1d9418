// conv_tc_ws2.cu -- weight-stationary kernel for the 64-input-channel 3x3 stride-1 layers, CTA pair.
#include "conv_tc_common.cuh"

// ---------------------------------------------------------------------------
// The one-CTA weight-stationary kernel issues 18 tcgen05.mma of 128 x BN x 32 per tile.  With
// BN = 64 such an instruction is 32 cycles of tensor work, but one thread issues an MMA with
// changing descriptors only about every 70 cycles, so the issue rate bounds the K loop.  Here two
// CTAs of a TPC work as a pair (cta_group::2): each holds its own 8 x 16-pixel activation tile and
// HALF of the weights (BN / 2 output channels x 9 taps), and one instruction issued by the
// leader covers both tiles (M = 256): half the instructions per output, and half the weight
// bytes resident per SM.
//   * every TMA load is issued by the CTA that owns the destination shared memory and counts its
//     bytes on the LEADER's barrier (no multicast);
//   * the leader's commit arrives on the stage-empty / accumulator-full barriers of both CTAs;
//   * both CTAs' epilogue warps arrive on the leader's accumulator-empty barrier;
//   * two issuer warps of the leader take alternate pair tiles;
//   * activation tile, tap addressing (descriptor start offsets into one box) and epilogue are
//     those of the one-CTA kernel; pairing, barriers and teardown those of the per-tap pair kernel.
// ---------------------------------------------------------------------------
template <int BN, bool CONTRACT, int EPI>
__global__ void __launch_bounds__(TC_THREADS, 1)
conv_ws2_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const TcParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int KC = 64;
    constexpr int W_TAP_BYTES = (BN / 2) * KC;            // this CTA's half of one tap
    constexpr int W_BYTES = 9 * W_TAP_BYTES;
    constexpr uint32_t TMEM_COLS = TC_NACC(BN) * BN;
    constexpr uint32_t IDESC = idesc_i8(BN, 256);

    uint8_t* s_w = smem;                                        // [9][BN/2][64]
    uint8_t* s_a = smem + W_BYTES;                              // [stages][WS_A_BYTES]
    float* tab = (float*)(s_a + (size_t)p.stages * WS_A_BYTES);
    uint8_t* lut = (uint8_t*)(tab + p.ntab * TC_MAX_COUT);
    TcShared* sh = (TcShared*)(lut + p.lut_bytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();            // 0 = leader
    const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int m_tiles = p.tiles_w * p.tiles_h * p.tiles_b;
    const int total = (m_tiles + 1) >> 1;                // pair tiles (tiles_n == 1)

    tc_load_tables(tab, p);
    tc_load_lut(lut, p, 0, BN);
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) { mbar_init(smem_u32(&sh->full[s]), 1); mbar_init(smem_u32(&sh->empty[s]), 1); }
        for (int a = 0; a < TC_MAX_ACC; a++) { mbar_init(smem_u32(&sh->acc_full[a]), 1); mbar_init(smem_u32(&sh->acc_empty[a]), 2 * TC_EPI_ACTIVE(BN)); }
        mbar_init(smem_u32(&sh->w_full), 1);
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&sh->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                  // peer's barriers are initialised
    tc_fence_after();
    tc_pdl_sync();
    const uint32_t tmem_base = sh->tmem_base;
    volatile int* abort_flag = &sh->abort_flag;

    if (warp == 0) {
        // TMA producer (both CTAs): lanes 0..8 fetch this CTA's half of one weight tap each, then
        // lane 0 one activation box per tile.  Bytes are counted on the leader's barriers.
        const uint32_t wbar = smem_u32(&sh->w_full);
        const uint32_t wbar_leader = map_to_cta(wbar, 0);
        const uint32_t full0 = smem_u32(&sh->full[0]);
        const uint32_t full0_leader = map_to_cta(full0, 0);
        if (rank == 0 && lane == 0) mbar_expect_tx(wbar, 2 * W_BYTES);
        __syncwarp();
        if (lane < 9) tma2_load_4d(smem_u32(s_w + lane * W_TAP_BYTES), &mapB, wbar_leader, lane * p.Cp, (int)rank * (BN / 2), 0, 0);
        int stage = 0; uint32_t phase = 0;
        bool ok = true;
        TileWalk wk;
        walk_init(wk, p, pair_id * 2 + (int)rank, n_pairs * 2);
        for (int tile = pair_id; tile < total && ok; tile += n_pairs, walk_next(wk, p)) {
            const int tw = wk.tw, th = wk.th, b = wk.tb;  // b may be past the batch: TMA zero-fills
            ok = mbar_wait(smem_u32(&sh->empty[stage]), phase ^ 1, abort_flag, p.err, FFCU_ERR_EMPTY_TIMEOUT);
            if (!ok) break;
            if (p.dbg & 1) {
                if (rank == 0 && lane == 0) mbar_arrive(full0 + stage * 8);
            } else if (lane == 0) {
                if (rank == 0) mbar_expect_tx(full0 + stage * 8, 2 * WS_BOX_ROWS * 64);
                tma2_load_4d(smem_u32(s_a + (size_t)stage * WS_A_BYTES), &mapA, full0_leader + stage * 8,
                             0, tw * WS_TW - 1, th * WS_TH - 1, b);
            }
            __syncwarp();
            if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
    } else if (warp == 1 || warp == TC_ISSUER2_WARP) {
        if (rank == 0) {
            // MMA issuers (leader CTA), alternate pair tiles; ring positions from the tile's index
            const int me = (warp == 1) ? 0 : 1;
            bool ok = mbar_wait_cluster(smem_u32(&sh->w_full), 0, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT);
            tc_fence_after();
            const uint64_t dw = smem_desc<KC>(smem_u32(s_w));
            const uint32_t leader = (lane == 0) ? 1u : 0u;
            uint32_t ready_a = 0, ready_f = 0;           // answers of the early tests for this issuer's next tile
            for (int tile = pair_id + me * n_pairs, local = me; tile < total && ok; tile += 2 * n_pairs, local += 2) {
                const int stage = local % p.stages;
                const uint32_t phase = (uint32_t)(local / p.stages) & 1;
                const int a = local % TC_NACC(BN);
                const uint32_t aphase = (uint32_t)(local / TC_NACC(BN)) & 1;
                if (!ready_a) {
                    ok = mbar_wait_cluster(smem_u32(&sh->acc_empty[a]), aphase ^ 1, abort_flag, p.err, FFCU_ERR_TMEM_TIMEOUT);
                    if (!ok) break;
                }
                if (!ready_f) {
                    ok = mbar_wait_cluster(smem_u32(&sh->full[stage]), phase, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT);
                    if (!ok) break;
                }
                {
                    const int nl = local + 2;
                    ready_a = mbar_test_cluster(smem_u32(&sh->acc_empty[nl % TC_NACC(BN)]), ((uint32_t)(nl / TC_NACC(BN)) & 1) ^ 1);
                    ready_f = mbar_test_cluster(smem_u32(&sh->full[nl % p.stages]), (uint32_t)(nl / p.stages) & 1);
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(a * BN);
                const uint64_t da0 = smem_desc_sbo<KC>(smem_u32(s_a + (size_t)stage * WS_A_BYTES), WS_PITCH * 64);
                if (!(p.dbg & 2))
#pragma unroll
                for (int kw = 0; kw < 3; kw++)
#pragma unroll
                    for (int kh = 0; kh < 3; kh++) {
                        // tap (kh, kw): the same box, (kh * pitch + kw) lines further on
                        const uint64_t da = da0 + (uint64_t)(((kh * WS_PITCH + kw) * 64) >> 4);
                        const uint64_t db = dw + (uint64_t)(((kh * 3 + kw) * W_TAP_BYTES) >> 4);
#pragma unroll
                        for (int k = 0; k < 2; k++)
                            umma2_i8_w(leader, d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), IDESC, (kw | kh | k) ? 1u : 0u);
                    }
                umma2_commit_both_w(leader, smem_u32(&sh->empty[stage]));
                umma2_commit_both_w(leader, smem_u32(&sh->acc_full[a]));
            }
        }
    } else {
        const uint32_t leader_acc_empty = map_to_cta(smem_u32(&sh->acc_empty[0]), 0);
        tc_epilogue_role<BN, CONTRACT, false, EPI>(p, tab, lut, sh, tmem_base, abort_flag, warp, lane,
                                                   pair_id, n_pairs, total, 2, (int)rank, leader_acc_empty);
    }

    // ---- teardown: neither CTA may leave while its partner can still read its smem / TMEM ----
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
    }
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

template <int BN, bool CONTRACT, int EPI>
static int launch_w2(int grid, int smem, cudaStream_t s, const CUtensorMap& mapA, const CUtensorMap& mapB, const TcParams& prm)
{
    auto kern = conv_ws2_kernel<BN, CONTRACT, EPI>;
    static int smem_set[64] = {};      // per device: the attribute belongs to the device's copy of the function
    int dev = 0;
    FFCU_CHECK(cudaGetDevice(&dev));
    if (smem_set[dev & 63] < smem) {
        FFCU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        smem_set[dev & 63] = smem;
    }
    return tc_launch_ex(kern, grid, smem, s, true, mapA, mapB, prm);
}

template <int BN>
static int launch_w2_bn(int mode, int epi, int grid, int smem, cudaStream_t s,
                        const CUtensorMap& mapA, const CUtensorMap& mapB, const TcParams& prm)
{
    if (!mode) return launch_w2<BN, false, EPI_RUNTIME>(grid, smem, s, mapA, mapB, prm);
    switch (epi) {
    case EPI_PLAIN:  return launch_w2<BN, true, EPI_PLAIN>(grid, smem, s, mapA, mapB, prm);
    case EPI_SLOPE:  return launch_w2<BN, true, EPI_SLOPE>(grid, smem, s, mapA, mapB, prm);
    case EPI_RES_BN: return launch_w2<BN, true, EPI_RES_BN>(grid, smem, s, mapA, mapB, prm);
    case EPI_RES:    return launch_w2<BN, true, EPI_RES>(grid, smem, s, mapA, mapB, prm);
    default:         return launch_w2<BN, true, EPI_RUNTIME>(grid, smem, s, mapA, mapB, prm);
    }
}

int tc_launch_ws2(int bn, int mode, int epi, int grid, int smem, cudaStream_t s,
                  const CUtensorMap& mapA, const CUtensorMap& mapB_half, const TcParams& prm)
{
    if (bn == 128) return launch_w2_bn<128>(mode, epi, grid, smem, s, mapA, mapB_half, prm);
    return launch_w2_bn<64>(mode, epi, grid, smem, s, mapA, mapB_half, prm);
}
