// conv_tc_pair.cu -- CTA-pair (cta_group::2) implicit-GEMM kernel for >= 128 input channels.
#include "conv_tc_common.cuh"

// ---------------------------------------------------------------------------
// CTA-pair kernel (cta_group::2) for the layers with >= 128 input channels.
// Two CTAs on one TPC compute a 256-pixel x BN tile: each loads its own 128 pixel rows
// of A and HALF of the weight tile (BN/2 rows), and one tcgen05.mma.cta_group::2 issued
// by the leader CTA reads both halves from both shared memories.  Per CTA the bytes
// fetched from L2 per MAC drop by a third (BN = 256: 16 KB + 16 KB instead of
// 16 KB + 32 KB per 128 x 256 x 128 MACs), which is what bounds these layers.
//   * every TMA load is issued by the CTA that owns the destination shared memory and
//     counts its bytes on the LEADER's full barrier (no multicast);
//   * the leader's commit arrives on the empty / accumulator-full barriers of both CTAs;
//   * both CTAs' epilogue warps arrive on the leader's accumulator-empty barrier;
//   * the pair synchronises (cluster barrier) after set-up and before teardown so neither
//     CTA's shared memory or TMEM goes away while the other may still touch it.
// ---------------------------------------------------------------------------
template <int BN, bool CONTRACT, bool OUT_F32, int EPI>
__global__ void __launch_bounds__(TC_THREADS, 1)
conv_tc2_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const TcParams p)
{
    tc_pdl_trigger();
    extern __shared__ uint8_t smem_raw[];
    // round up to 1024 bytes by pointer arithmetic on the __shared__ array (an integer round-trip
    // would hide the address space from the compiler and turn every table read into a generic load)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int KC = 128;
    constexpr int A_BYTES = TC_TILE_M * KC;
    constexpr int B_BYTES = (BN / 2) * KC;
    constexpr int SUB_BYTES = A_BYTES + B_BYTES;          // one K block: [A 128 x 128 | B-half BN/2 x 128]
    constexpr uint32_t TMEM_COLS = TC_NACC(BN) * BN;
    constexpr uint32_t IDESC = idesc_i8(BN, 256);

    float* tab = (float*)(smem + (size_t)p.stages * p.group * SUB_BYTES);
    uint8_t* lut = (uint8_t*)(tab + p.ntab * TC_MAX_COUT);                  // [BN][256] fused-BN table (lut_bytes may be 0)
    TcShared* sh = (TcShared*)(lut + p.lut_bytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();            // 0 = leader
    const int kblocks = p.taps * p.cin_blocks;
    const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int m_tiles = p.tiles_w * p.tiles_h * p.tiles_b;
    const int total = p.tiles_n * ((m_tiles + 1) >> 1);  // pair tiles

    tc_load_tables(tab, p);
    tc_load_lut(lut, p, (int)(pair_id % p.tiles_n) * BN, BN);
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) { mbar_init(smem_u32(&sh->full[s]), 1); mbar_init(smem_u32(&sh->empty[s]), 1); }
        for (int a = 0; a < TC_MAX_ACC; a++) { mbar_init(smem_u32(&sh->acc_full[a]), 1); mbar_init(smem_u32(&sh->acc_empty[a]), 2 * p.epi_wps); }
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
    tc_pdl_wait();
    const uint32_t tmem_base = sh->tmem_base;
    volatile int* abort_flag = &sh->abort_flag;

    if (warp == 0) {
        const int G = p.group;
        {
            // TMA producer.  The whole warp runs the loop (lanes stay converged); lanes
            // 0 .. 2G-1 issue.  A pipeline stage holds G consecutive K blocks; lane 2g fetches the
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
            const uint32_t full0_leader = map_to_cta(full0, 0);
            const int stage_bytes = G * SUB_BYTES;
            const int n_steps = kblocks / G;
            const int tn = pair_id % p.tiles_n;
            TileWalk wk;
            walk_init(wk, p, (pair_id / p.tiles_n) * 2 + (int)rank, (n_pairs / p.tiles_n) * 2);
            for (int tile = pair_id; tile < total && ok; tile += n_pairs, walk_next(wk, p)) {
                const int tw = wk.tw, th = wk.th, tb = wk.tb;   // tb may be past the batch: TMA zero-fills
                const int x0 = tw * p.TW * p.stride - p.pad;
                const int y0 = th * p.TH * p.stride - p.pad;
                const int c3 = is_a ? tb * p.TB : 0;
                // this lane's first block: kb = g
                int c0 = g * KC, kw = 0, kh = 0;
                while (c0 >= p.Cp) { c0 -= p.Cp; if (++kw == p.Kw) { kw = 0; kh++; } }
#pragma unroll 1
                for (int it = 0; it < n_steps; it++) {
                    ok = mbar_wait(empty0 + stage * 8, phase ^ 1, abort_flag, p.err, FFCU_ERR_EMPTY_TIMEOUT);
                    if (!ok) break;
                    if (TC_DBG(p, 1)) { if (rank == 0 && lane == 0) mbar_arrive(full0 + stage * 8); }
                    else {
                        if (rank == 0 && lane == 0) mbar_expect_tx(full0 + stage * 8, 2 * G * SUB_BYTES);
                        __syncwarp();                           // the byte count is armed before any copy can land
                        const int tapk = (kh * p.Kw + kw) * p.Cp + c0;
                        if (issuer) tma2_load_4d(smem0 + stage * stage_bytes, map, full0_leader + stage * 8,
                                    is_a ? c0 : tapk, is_a ? x0 + kw : tn * BN + (int)rank * (BN / 2), is_a ? y0 + kh : 0, c3);
                    }
                    c0 += G * KC;
                    while (c0 >= p.Cp) { c0 -= p.Cp; if (++kw == p.Kw) { kw = 0; kh++; } }
                    if (++stage == p.stages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        const int G = p.group;
        const int n_steps = kblocks / G;
        if (rank == 0) {
            // MMA issuer (leader CTA): the warp loops and waits together, lane 0 issues
            int stage = 0; uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            const int stage_bytes = G * SUB_BYTES;
            const uint32_t full0 = smem_u32(&sh->full[0]), empty0 = smem_u32(&sh->empty[0]);
            const uint64_t da0 = smem_desc<KC>(smem_u32(smem));
            const uint64_t db0 = smem_desc<KC>(smem_u32(smem) + A_BYTES);
            const uint32_t leader = (lane == 0) ? 1u : 0u;
            uint32_t ready = 0;                          // answer of the early test for the upcoming stage
            for (int tile = pair_id; tile < total && ok; tile += n_pairs, local++) {
                const int a = local % TC_NACC(BN);
                const uint32_t aphase = (uint32_t)(local / TC_NACC(BN)) & 1;
                ok = mbar_wait_cluster(smem_u32(&sh->acc_empty[a]), aphase ^ 1, abort_flag, p.err, FFCU_ERR_TMEM_TIMEOUT);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(a * BN);
#pragma unroll 1
                for (int it = 0; it < n_steps; it++) {
                    if (!ready) {
                        ok = mbar_wait_cluster(full0 + stage * 8, phase, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT, p.full_wait);
                        if (!ok) break;
                    }
                    // test the next stage now, use the answer next round
                    int ns = stage + 1; uint32_t np = phase;
                    if (ns == p.stages) { ns = 0; np ^= 1; }
                    ready = mbar_test_cluster(full0 + ns * 8, np);
                    tc_fence_after();
                    {
                        uint32_t soff = (uint32_t)((stage * stage_bytes) >> 4);
                        if (!TC_DBG(p, 2))
#pragma unroll 1
                        for (int g = 0; g < G; g++, soff += (uint32_t)(SUB_BYTES >> 4)) {
#pragma unroll
                            for (int k = 0; k < KC / 32; k++)
                                umma2_i8_w(leader, d_tmem, da0 + (uint64_t)(soff + 2 * k), db0 + (uint64_t)(soff + 2 * k), IDESC, (it | g | k) ? 1u : 0u);
                        }
                        umma2_commit_both_w(leader, empty0 + stage * 8);   // frees the stage once these MMAs have read it
                    }
                    stage = ns; phase = np;
                }
                if (ok) umma2_commit_both_w(leader, smem_u32(&sh->acc_full[a]));
            }
        }
    } else {
        const uint32_t leader_acc_empty = map_to_cta(smem_u32(&sh->acc_empty[0]), 0);
        tc_epilogue_role<BN, CONTRACT, OUT_F32, EPI>(p, tab, lut, sh, tmem_base, abort_flag, warp, lane,
                                                pair_id, n_pairs, total, 2, (int)rank, leader_acc_empty);
    }

    // ---- teardown: neither CTA may leave while its partner can still read its smem / TMEM ----
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
#pragma unroll 1
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
    }
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}


template <int BN, bool CONTRACT, bool F32, int EPI>
static int launch_p(int grid, int smem, cudaStream_t s, const CUtensorMap& mapA, const CUtensorMap& mapB, const TcParams& prm)
{
    auto kern = conv_tc2_kernel<BN, CONTRACT, F32, EPI>;
    static int smem_set[64] = {};      // per device: the attribute belongs to the device's copy of the function
    int dev = 0;
    FFCU_CHECK(cudaGetDevice(&dev));
    if (smem_set[dev & 63] < smem) {
        FFCU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        smem_set[dev & 63] = smem;
    }
    return tc_launch_ex(kern, grid, smem, s, 2, mapA, mapB, prm);
}

template <int BN>
static int launch_p_bn(int mode, int epi, bool f32, int grid, int smem, cudaStream_t s,
                       const CUtensorMap& mapA, const CUtensorMap& mapB, const TcParams& prm)
{
    if (f32) return mode ? launch_p<BN, true, true, EPI_PLAIN>(grid, smem, s, mapA, mapB, prm)
                         : launch_p<BN, false, true, EPI_PLAIN>(grid, smem, s, mapA, mapB, prm);
    if (!mode) return launch_p<BN, false, false, EPI_RUNTIME>(grid, smem, s, mapA, mapB, prm);
    switch (epi) {
    case EPI_PLAIN:  return launch_p<BN, true, false, EPI_PLAIN>(grid, smem, s, mapA, mapB, prm);
    case EPI_SLOPE:  return launch_p<BN, true, false, EPI_SLOPE>(grid, smem, s, mapA, mapB, prm);
    case EPI_RES_BN: return launch_p<BN, true, false, EPI_RES_BN>(grid, smem, s, mapA, mapB, prm);
    case EPI_RES:    return launch_p<BN, true, false, EPI_RES>(grid, smem, s, mapA, mapB, prm);
    default:         return launch_p<BN, true, false, EPI_RUNTIME>(grid, smem, s, mapA, mapB, prm);
    }
}

int tc_launch_pair(int bn, int mode, int epi, bool f32, int grid, int smem, cudaStream_t s,
                   const CUtensorMap& mapA, const CUtensorMap& mapB, const TcParams& prm)
{
    if (bn == 256) return launch_p_bn<256>(mode, epi, f32, grid, smem, s, mapA, mapB, prm);
    return launch_p_bn<128>(mode, epi, f32, grid, smem, s, mapA, mapB, prm);
}
