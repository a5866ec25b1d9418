// conv_tc_wsp.cu -- weight-stationary CTA-pair kernel for the 3x3 stride-1 128 -> 128 layers (28x28 maps).
#include "conv_tc_common.cuh"

// ---------------------------------------------------------------------------
// Why: with 128 x 128 tiles the per-tap kernels move, per K block, as many bytes into shared memory
// (16 KB of activations + 8 KB of weights per CTA) as the tensor core reads out of it, and the two
// together ask more of the 128 B/cycle shared-memory path than it has: these layers ran at a third
// of the tensor rate.  Here nothing but the activations moves:
//   * the layer's weights (9 taps x 128 x 128 int8 = 144 KB) stay in shared memory for the CTA
//     pair's lifetime, half of the output channels in each CTA (cta_group::2 reads both halves);
//   * a tile is 128 consecutive LINES of one image stored with a row pitch of P = W + 2 lines (a
//     zero column either side): line l = row * P + column + 1.  One TMA box {128 B, P, 8, 1} per
//     tile, starting at column -1 and one row above the tile's first row, brings every line the
//     tile's nine taps touch (rows and columns outside the image are zero-filled: the conv's
//     padding).  Tap (kh, kw) of output line l reads line l + (kh-1) * P + (kw-1): the same
//     buffer, with the A descriptor's start moved by that many lines (the tensor core applies the
//     128-byte swizzle to absolute shared-memory addresses, as the TMA write did).  The two pitch
//     columns and the lines past the last row are positions without an output (6.7 % + the last
//     tile's tail); the epilogue skips them.
//   * a pair works on the SAME tile index of two consecutive images, so both CTAs' buffers have
//     the tile's first line at the same offset and one descriptor serves the pair.
// Activation bytes fetched per tile: 240 lines instead of 9 x 128; weights: none.
// Warp roles, barriers, bounded waits and teardown as in the per-tap pair kernel; two issuer
// warps (leader CTA) take alternate tiles as in the 64-channel weight-stationary kernel.
// ---------------------------------------------------------------------------
template <bool CONTRACT, int EPI>
__global__ void __launch_bounds__(TC_THREADS, 1)
conv_wsp_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const TcParams p)
{
    tc_pdl_trigger();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int BN = 128, KC = 128;
    constexpr int W_TAP_BYTES = (BN / 2) * KC;            // this CTA's half of one tap: 64 output channels
    constexpr int W_BYTES = 9 * W_TAP_BYTES;
    constexpr uint32_t TMEM_COLS = TC_NACC(BN) * BN;
    constexpr uint32_t IDESC = idesc_i8(BN, 256);
    const int P = p.flat_P;
    const int box_bytes = P * WSP_BOX_ROWS * KC;
    const int a_stride = (WSP_GUARD_BYTES + box_bytes + 1023) & ~1023;

    uint8_t* s_w = smem;                                  // [9][64][128]
    uint8_t* s_a = smem + W_BYTES;                        // [stages][guard | box]
    float* tab = (float*)(s_a + (size_t)p.stages * a_stride);
    uint8_t* lut = (uint8_t*)(tab + p.ntab * TC_MAX_COUT);
    TcShared* sh = (TcShared*)(lut + p.lut_bytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();              // 0 = leader
    const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int total = p.total_tiles;                      // pair tiles: (images / 2) x tiles per image

    tc_load_tables(tab, p);
    tc_load_lut(lut, p, 0, BN);
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
    cluster_sync_all();                                   // peer's barriers are initialised
    tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;
    volatile int* abort_flag = &sh->abort_flag;

    if (warp == 0) {
        // TMA producer (both CTAs).  The weights do not depend on the previous kernel: they are
        // requested before the programmatic-dependency wait, the activations after it.
        const uint32_t wbar_leader = map_to_cta(smem_u32(&sh->w_full), 0);
        // (a copy that lands before the leader has armed the byte count only drives the count negative
        // for a moment; the phase cannot complete before the leader's own arrival)
        if (rank == 0 && lane == 0) mbar_expect_tx(smem_u32(&sh->w_full), 2 * W_BYTES);
        __syncwarp();
        if (lane < 9) tma2_load_4d(smem_u32(s_w + lane * W_TAP_BYTES), &mapB, wbar_leader, lane * p.Cp, (int)rank * (BN / 2), 0, 0);
        tc_pdl_wait();
        const uint32_t full0 = smem_u32(&sh->full[0]), empty0 = smem_u32(&sh->empty[0]);
        const uint32_t full0_leader = map_to_cta(full0, 0);
        int stage = 0; uint32_t phase = 0;
        bool ok = true;
        TileWalk wk;
        walk_init(wk, p, pair_id * 2 + (int)rank, n_pairs * 2);
        for (int tile = pair_id; tile < total && ok; tile += n_pairs, walk_next(wk, p)) {
            const int b = wk.tw, t = wk.th;               // image (may be one past the batch: zero-filled), tile in image
            const int base_row = (t * TC_TILE_M) / P - 1;
            ok = mbar_wait(empty0 + stage * 8, phase ^ 1, abort_flag, p.err, FFCU_ERR_EMPTY_TIMEOUT);
            if (!ok) break;
            if (TC_DBG(p, 1)) { if (rank == 0 && lane == 0) mbar_arrive(full0 + stage * 8); }
            else {
                if (rank == 0 && lane == 0) mbar_expect_tx(full0 + stage * 8, 2 * box_bytes);
                __syncwarp();
                if (lane == 0) tma2_load_4d(smem_u32(s_a + (size_t)stage * a_stride + WSP_GUARD_BYTES), &mapA,
                                            full0_leader + stage * 8, 0, -1, base_row, b);
            }
            __syncwarp();
            if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
    } else if (warp == 1 || warp == TC_ISSUER2_WARP) {
        tc_pdl_wait();
        if (rank == 0) {
            // Two MMA issuers (leader CTA) take alternate tiles; each derives its ring positions from
            // the tile's index.  The warp loops and waits together, lane 0 issues.
            const int me = (warp == 1) ? 0 : 1;
            bool ok = mbar_wait_cluster(smem_u32(&sh->w_full), 0, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT);
            tc_fence_after();
            const uint64_t dw = smem_desc<KC>(smem_u32(s_w));
            const uint32_t leader = (lane == 0) ? 1u : 0u;
            uint32_t ready_a = 0, ready_f = 0;
            TileWalk wk;
            walk_init(wk, p, (pair_id + me * n_pairs) * 2, n_pairs * 4);
            // ring positions carried forward by additions (both rings are even: +2 keeps this issuer on its own slots)
            const int stages = p.stages;
            int stage = me; uint32_t phase = 0;
            int a = me; uint32_t aphase = 0;
            int ns = 0, na = 0; uint32_t np = 0, nap = 0;
            for (int tile = pair_id + me * n_pairs; tile < total && ok;
                 tile += 2 * n_pairs, walk_next(wk, p), stage = ns, phase = np, a = na, aphase = nap) {
                if (!ready_a) {
                    ok = mbar_wait_cluster(smem_u32(&sh->acc_empty[a]), aphase ^ 1, abort_flag, p.err, FFCU_ERR_TMEM_TIMEOUT);
                    if (!ok) break;
                }
                if (!ready_f) {
                    ok = mbar_wait_cluster(smem_u32(&sh->full[stage]), phase, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT, p.full_wait);
                    if (!ok) break;
                }
                {   // test the barriers of this issuer's next tile now, use the answers next round
                    ns = stage + 2; np = phase;
                    if (ns >= stages) { ns -= stages; np ^= 1; }
                    na = a + 2; nap = aphase;
                    if (na >= TC_NACC(BN)) { na -= TC_NACC(BN); nap ^= 1; }
                    ready_a = mbar_test_cluster(smem_u32(&sh->acc_empty[na]), nap ^ 1);
                    ready_f = mbar_test_cluster(smem_u32(&sh->full[ns]), np);
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(a * BN);
                // first line of the tile inside the box: one row below the box's first row, plus the tile's column offset
                const int t = wk.th;
                const int off = t * TC_TILE_M - ((t * TC_TILE_M) / P - 1) * P;
                const uint64_t da0 = smem_desc<KC>(smem_u32(s_a + (size_t)stage * a_stride + WSP_GUARD_BYTES));
                if (!TC_DBG(p, 2)) {
#pragma unroll 1
                    for (int kh = 0; kh < 3; kh++)
#pragma unroll
                        for (int kw = 0; kw < 3; kw++) {
                            const int line = off + (kh - 1) * P + (kw - 1);        // >= -1: the guard in front of the box
                            const uint64_t da = da0 + (uint64_t)(int64_t)((line * KC) >> 4);
                            const uint64_t db = dw + (uint64_t)(((kh * 3 + kw) * W_TAP_BYTES) >> 4);
#pragma unroll
                            for (int k = 0; k < KC / 32; k++)
                                umma2_i8_w(leader, d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), IDESC, (kh | kw | k) ? 1u : 0u);
                        }
                }
                umma2_commit_both_w(leader, smem_u32(&sh->empty[stage]));
                umma2_commit_both_w(leader, smem_u32(&sh->acc_full[a]));
            }
        }
    } else {
        tc_pdl_wait();
        const uint32_t leader_acc_empty = map_to_cta(smem_u32(&sh->acc_empty[0]), 0);
        tc_epilogue_role<BN, CONTRACT, false, EPI>(p, tab, lut, sh, tmem_base, abort_flag, warp, lane,
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

template <bool CONTRACT, int EPI>
static int launch_wsp(int grid, int smem, cudaStream_t s, const CUtensorMap& mapA, const CUtensorMap& mapB, const TcParams& prm)
{
    auto kern = conv_wsp_kernel<CONTRACT, EPI>;
    static int smem_set[64] = {};      // per device: the attribute belongs to the device's copy of the function
    int dev = 0;
    FFCU_CHECK(cudaGetDevice(&dev));
    if (smem_set[dev & 63] < smem) {
        FFCU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        smem_set[dev & 63] = smem;
    }
    return tc_launch_ex(kern, grid, smem, s, 2, mapA, mapB, prm);
}

int tc_launch_wsp(int mode, int epi, int grid, int smem, cudaStream_t s,
                  const CUtensorMap& mapA, const CUtensorMap& mapB_half, const TcParams& prm)
{
    if (!mode) return launch_wsp<false, EPI_RUNTIME>(grid, smem, s, mapA, mapB_half, prm);
    switch (epi) {
    case EPI_PLAIN:  return launch_wsp<true, EPI_PLAIN>(grid, smem, s, mapA, mapB_half, prm);
    case EPI_SLOPE:  return launch_wsp<true, EPI_SLOPE>(grid, smem, s, mapA, mapB_half, prm);
    case EPI_RES_BN: return launch_wsp<true, EPI_RES_BN>(grid, smem, s, mapA, mapB_half, prm);
    case EPI_RES:    return launch_wsp<true, EPI_RES>(grid, smem, s, mapA, mapB_half, prm);
    default:         return launch_wsp<true, EPI_RUNTIME>(grid, smem, s, mapA, mapB_half, prm);
    }
}
