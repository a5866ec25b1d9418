// conv_tc_shift.cu -- CTA-pair kernel for the 3x3 stride-1 layers with >= 128 input channels:
// the activation patch stays in shared memory for all nine taps.
#include "conv_tc_common.cuh"

// ---------------------------------------------------------------------------
// The per-tap kernels fetch a tile's activations nine times (once per filter tap) and its
// weights once; at 128 x BN tiles that is more L2 -> shared-memory traffic than the tensor
// pipe's appetite allows (BN = 128: 96 bytes per cycle per SM).  Here a tile is TR image
// rows of ONE image, stored in shared memory with a row pitch of P pixels (P >= W + 1,
// P * TR = 128): one TMA box {128 B, P, TR + 2, 1} starting at (x, y) = (-1, y0 - 1) per
// 128-channel slice, out-of-range pixels zero-filled.  Output position m = r * P + x of the
// tile (r < TR, x < P; x >= W are padding positions whose results are dropped) reads, for
// tap (kh, kw), shared-memory line m + kh * P + kw.  So the A operand of every tap is the
// same buffer, addressed with the descriptor's start address moved by (kh * P + kw) lines:
// the tensor core applies the 128-byte swizzle to absolute shared-memory addresses, the same
// rule the TMA write used, so a start that is not a multiple of 8 lines still reads the
// right bytes.  The zero column at x = W doubles as the x = -1 column of the next row.
// Per tile each CTA now fetches (TR + 2) * P lines per slice once, plus its half of the weights.
//
// K loop order: slice c (128 channels), then tap.  Rings: NA activation-slice buffers
// (a_full / a_empty), `stages` weight stages of `group` taps each (full / empty).
// CTA pairing, barriers and teardown are those of the per-tap pair kernel.
// ---------------------------------------------------------------------------
template <int BN, bool CONTRACT, int EPI>
__global__ void __launch_bounds__(TC_THREADS, 1)
conv_shift_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const TcParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int KC = 128;
    constexpr int B_BYTES = (BN / 2) * KC;                // one tap of one slice: this CTA's half of the weights
    constexpr uint32_t TMEM_COLS = TC_NACC(BN) * BN;
    constexpr uint32_t IDESC = idesc_i8(BN, 256);

    uint8_t* s_a = smem;                                                    // [na][a_stride]
    uint8_t* s_b = smem + (size_t)p.na * p.a_stride;                        // [stages][group][B_BYTES]
    float* tab = (float*)(s_b + (size_t)p.stages * p.group * B_BYTES);
    uint8_t* lut = (uint8_t*)(tab + p.ntab * TC_MAX_COUT);
    TcShared* sh = (TcShared*)(lut + p.lut_bytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();            // 0 = leader
    const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int m_tiles = p.tiles_w * p.tiles_h * p.tiles_b;
    const int total = p.tiles_n * ((m_tiles + 1) >> 1);  // pair tiles
    const int G = p.group;
    const int steps_per_slice = 9 / G;
    const int a_box_bytes = p.TW * (p.TH + 2) * KC;

    tc_load_tables(tab, p);
    tc_load_lut(lut, p, (int)(pair_id % p.tiles_n) * BN, BN);
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) { mbar_init(smem_u32(&sh->full[s]), 1); mbar_init(smem_u32(&sh->empty[s]), 1); }
        for (int s = 0; s < TC_MAX_ABUF; s++) { mbar_init(smem_u32(&sh->a_full[s]), 1); mbar_init(smem_u32(&sh->a_empty[s]), 1); }
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
        // TMA producer (both CTAs): lane 0 fetches the activation slices, lanes 0 .. G-1 one
        // weight tap each.  Bytes are counted on the leader's barriers.
        const uint32_t full0 = smem_u32(&sh->full[0]), empty0 = smem_u32(&sh->empty[0]);
        const uint32_t afull0 = smem_u32(&sh->a_full[0]), aempty0 = smem_u32(&sh->a_empty[0]);
        const uint32_t full0_leader = map_to_cta(full0, 0), afull0_leader = map_to_cta(afull0, 0);
        int stage = 0; uint32_t phase = 0;
        int abuf = 0; uint32_t aphase = 0;
        bool ok = true;
        const int tn = pair_id % p.tiles_n;
        TileWalk wk;
        walk_init(wk, p, (pair_id / p.tiles_n) * 2 + (int)rank, (n_pairs / p.tiles_n) * 2);
        for (int tile = pair_id; tile < total && ok; tile += n_pairs, walk_next(wk, p)) {
            const int y0 = wk.th * p.TH - 1;              // tiles_w == 1: a tile spans the image width
            const int b = wk.tb;                          // may be past the batch: TMA zero-fills
            for (int c = 0; c < p.cin_blocks && ok; c++) {
                ok = mbar_wait(aempty0 + abuf * 8, aphase ^ 1, abort_flag, p.err, FFCU_ERR_EMPTY_TIMEOUT);
                if (!ok) break;
                if (!(p.dbg & 1)) {
                    if (lane == 0) {
                        if (rank == 0) mbar_expect_tx(afull0 + abuf * 8, 2 * a_box_bytes);
                        tma2_load_4d(smem_u32(s_a + (size_t)abuf * p.a_stride), &mapA, afull0_leader + abuf * 8, c * KC, -1, y0, b);
                    }
                } else if (rank == 0 && lane == 0) mbar_arrive(afull0 + abuf * 8);
                __syncwarp();
                if (++abuf == p.na) { abuf = 0; aphase ^= 1; }
                for (int st = 0; st < steps_per_slice; st++) {
                    ok = mbar_wait(empty0 + stage * 8, phase ^ 1, abort_flag, p.err, FFCU_ERR_EMPTY_TIMEOUT);
                    if (!ok) break;
                    if (!(p.dbg & 1)) {
                        if (rank == 0 && lane == 0) mbar_expect_tx(full0 + stage * 8, 2 * G * B_BYTES);
                        __syncwarp();                   // the byte count is armed before any copy can land
                        if (lane < G) {
                            const int tap = st * G + lane;
                            tma2_load_4d(smem_u32(s_b + ((size_t)stage * G + lane) * B_BYTES), &mapB, full0_leader + stage * 8,
                                         tap * p.Cp + c * KC, tn * BN + (int)rank * (BN / 2), 0, 0);
                        }
                    } else if (rank == 0 && lane == 0) mbar_arrive(full0 + stage * 8);
                    __syncwarp();
                    if (++stage == p.stages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (rank == 0) {
            // MMA issuer (leader CTA): the warp loops and waits together, lane 0 issues
            const uint32_t full0 = smem_u32(&sh->full[0]), empty0 = smem_u32(&sh->empty[0]);
            const uint32_t afull0 = smem_u32(&sh->a_full[0]), aempty0 = smem_u32(&sh->a_empty[0]);
            int stage = 0; uint32_t phase = 0;
            int abuf = 0; uint32_t aphase = 0;
            int local = 0;
            bool ok = true;
            const uint64_t db0 = smem_desc<KC>(smem_u32(s_b));
            const uint32_t leader = (lane == 0) ? 1u : 0u;
            for (int tile = pair_id; tile < total && ok; tile += n_pairs, local++) {
                const int a = local % TC_NACC(BN);
                const uint32_t accphase = (uint32_t)(local / TC_NACC(BN)) & 1;
                ok = mbar_wait_cluster(smem_u32(&sh->acc_empty[a]), accphase ^ 1, abort_flag, p.err, FFCU_ERR_TMEM_TIMEOUT);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(a * BN);
                for (int c = 0; c < p.cin_blocks && ok; c++) {
                    ok = mbar_wait_cluster(afull0 + abuf * 8, aphase, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT);
                    if (!ok) break;
                    const uint64_t da0 = smem_desc<KC>(smem_u32(s_a + (size_t)abuf * p.a_stride));
                    for (int st = 0; st < steps_per_slice; st++) {
                        ok = mbar_wait_cluster(full0 + stage * 8, phase, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT);
                        if (!ok) break;
                        tc_fence_after();
                        {
                            if (!(p.dbg & 2))
                            for (int g = 0; g < G; g++) {
                                const int tap = st * G + g;
                                const int kh = tap / 3, kw = tap - 3 * kh;
                                // tap (kh, kw): the same activation buffer, (kh * P + kw) lines further on
                                const uint32_t aoff = (uint32_t)(((kh * p.TW + kw) * KC) >> 4);
                                const uint32_t boff = (uint32_t)(((stage * G + g) * B_BYTES) >> 4);
#pragma unroll
                                for (int k = 0; k < KC / 32; k++)
                                    umma2_i8_w(leader, d_tmem, da0 + (uint64_t)(aoff + 2 * k), db0 + (uint64_t)(boff + 2 * k), IDESC, (c | st | g | k) ? 1u : 0u);
                            }
                            umma2_commit_both_w(leader, empty0 + stage * 8);      // frees the weight stage in both CTAs
                        }
                        if (++stage == p.stages) { stage = 0; phase ^= 1; }
                    }
                    if (ok) umma2_commit_both_w(leader, aempty0 + abuf * 8);   // this slice's nine taps have been read
                    if (++abuf == p.na) { abuf = 0; aphase ^= 1; }
                }
                if (ok) umma2_commit_both_w(leader, smem_u32(&sh->acc_full[a]));
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
static int launch_s(int grid, int smem, cudaStream_t s, const CUtensorMap& mapA, const CUtensorMap& mapB, const TcParams& prm)
{
    auto kern = conv_shift_kernel<BN, CONTRACT, EPI>;
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
static int launch_s_bn(int mode, int epi, int grid, int smem, cudaStream_t s,
                       const CUtensorMap& mapA, const CUtensorMap& mapB, const TcParams& prm)
{
    if (!mode) return launch_s<BN, false, EPI_RUNTIME>(grid, smem, s, mapA, mapB, prm);
    switch (epi) {
    case EPI_PLAIN:  return launch_s<BN, true, EPI_PLAIN>(grid, smem, s, mapA, mapB, prm);
    case EPI_SLOPE:  return launch_s<BN, true, EPI_SLOPE>(grid, smem, s, mapA, mapB, prm);
    case EPI_RES_BN: return launch_s<BN, true, EPI_RES_BN>(grid, smem, s, mapA, mapB, prm);
    case EPI_RES:    return launch_s<BN, true, EPI_RES>(grid, smem, s, mapA, mapB, prm);
    default:         return launch_s<BN, true, EPI_RUNTIME>(grid, smem, s, mapA, mapB, prm);
    }
}

int tc_launch_shift(int bn, int mode, int epi, int grid, int smem, cudaStream_t s,
                    const CUtensorMap& mapA, const CUtensorMap& mapB, const TcParams& prm)
{
    if (bn == 256) return launch_s_bn<256>(mode, epi, grid, smem, s, mapA, mapB, prm);
    return launch_s_bn<128>(mode, epi, grid, smem, s, mapA, mapB, prm);
}
