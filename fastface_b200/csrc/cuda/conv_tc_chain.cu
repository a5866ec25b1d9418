// conv_tc_chain.cu -- batch-1 latency path: a run of consecutive 3x3 stride-1 convolutions of one
// shape (the 26 layers of the 14x14 stage, the 4 of the 7x7 stage) in ONE launch of one cluster of
// eight CTAs, with the activations resident in shared memory.
//
// At batch 1 a 14x14 layer is 8 tiles (2 row tiles x 4 column tiles of 64 channels); as separate
// launches each layer pays kernel completion + dependency release + a TMA round trip for 50 KB of
// activations before its first MMA.  Here the eight CTAs of a cluster take one tile each and keep the
// rows of the current layer's input their row tile reads in their own shared memory (double-buffered),
// laid out the way a TMA load with 128-byte swizzle would have left them: line (row + 1) * P + (col + 1)
// of 128 channels per plane, P = pitch in lines, zero lines for the padding.  Filter tap (kh, kw) is then
// the same buffer read (kh * P + kw) lines further on (the tensor core applies the swizzle to absolute
// shared-memory addresses), so the activations need no loads at all.  A CTA's epilogue requantises its
// 128 x 64 result to int8 (the fused BN's output where the layer has one) and writes each 16-byte piece
// straight into the NEXT layer's buffer of every CTA whose row tile reads that row, with st.async stores
// that count their bytes on the receiving CTA's barrier: "input complete" is a byte count, no fence or
// barrier round.  The weights stream through a TMA ring that runs ahead across layer boundaries, since
// they depend on nothing.  Global memory still receives every output (the residual two layers on is
// read from there, and the kernel after the chain).  Replaces, per layer, what conv_tc_kernel does
// (reference kernels/conv2d_nhwc.c:179-220, kernels/int8_epilogue.c:25-112, :253-318); same
// arithmetic, same bytes.
//
// Every wait is bounded as in the other kernels (the limit is a launch parameter); nobody leaves before
// the whole cluster has arrived at the final barrier, so no CTA's shared memory is written after it has
// exited.
#include "conv_tc_common.cuh"

struct ChainShared {
    uint64_t full[CHAIN_MAX_STAGES];
    uint64_t empty[CHAIN_MAX_STAGES];
    uint64_t act_full[2];                 // buffer b holds every byte this CTA needs of the next layer to read it
    uint64_t a0_full;                     // the first layer's input has landed (TMA)
    uint64_t acc_full;
    uint64_t acc_empty;                   // the sixteen epilogue warps have read the accumulator
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void chain_bar_sync_epi()
{
    asm volatile("bar.sync 1, %0;" ::"n"(CHAIN_EPI_THREADS) : "memory");
}

// Two MMA issuers (warps 1 and 18; each warp loops and waits together, lane 0 issues).  One thread issues an
// N = 64 MMA about every 70 cycles and pays a few hundred more per pipeline stage, which is slower than the
// tensor core retires them (51 cycles): the issuers take alternate stages of the weight ring, each
// accumulating into its own 64 TMEM columns; the epilogue adds the two (integer adds commute).  The ring is
// even, so a slot is always the same issuer's (a parity wait cannot tell "this fill" from "two fills ago",
// and with an odd ring the fill in between would be the other issuer's to consume).  PLANES (C / 128) and
// TPS (filter taps per stage) are compile-time so that a stage's MMAs are one straight-line block, and the
// ring / layer bookkeeping is carried forward by additions only.
template <int PLANES, int TPS>
__device__ __forceinline__ void chain_issuer_role(const ChainParams& p, ChainShared* sh, int me, int lane, uint32_t rank,
                                                  uint32_t tmem_base, uint32_t s_a_addr, uint32_t s_b_addr,
                                                  int tile_line0, uint32_t in_bytes)
{
    (void)rank;
    constexpr uint32_t IDESC = idesc_i8(CHAIN_BN);
    constexpr int B_BLOCK = CHAIN_BN * 128;
    constexpr int S = 9 / TPS;                              // stages per layer (odd)
    constexpr int STAGE_BYTES = TPS * PLANES * B_BLOCK;
    volatile int* abort_flag = &sh->abort_flag;
    const uint32_t full0 = smem_u32(&sh->full[0]), empty0 = smem_u32(&sh->empty[0]);
    const int stages = p.stages, n_layers = p.n_layers;
    const uint32_t leader = (lane == 0) ? 1u : 0u;
    const uint32_t d_tmem = tmem_base + (uint32_t)(me * CHAIN_BN);
    const uint64_t db_base = smem_desc<128>(s_b_addr);
    const uint32_t a_buf_bytes = (uint32_t)(PLANES * p.plane_bytes);
    const uint64_t dplane = (uint64_t)(p.plane_bytes >> 4);
    const uint32_t P8 = (uint32_t)(p.P * 8);                // one padded row, in descriptor units (16 bytes)
    uint64_t da_layer = 0;                                  // descriptor of the tile's first line in the layer's buffer
    uint32_t ready = 0;                                     // answer of the early test for this issuer's next stage
    uint32_t first = 0;                                     // non-zero after this issuer's first MMA of the layer
    int stage = me; uint32_t phase = 0;                     // ring slot of this issuer's current stage
    int L = 0, st = me;                                     // layer, stage within the layer
    bool new_layer = true;
    bool ok = true;
#pragma unroll 1
    while (L < n_layers) {
        if (new_layer) {
            new_layer = false;
            const int buf = L & 1;
            // arm the barrier of the buffer the peers fill during this layer (bytes that land before this
            // only drive the count negative for a moment: the phase cannot complete before this arrival)
            if (me == 0 && L + 1 < n_layers && lane == 0) mbar_expect_tx(smem_u32(&sh->act_full[buf ^ 1]), in_bytes);
            if (L == 0) ok = mbar_wait(smem_u32(&sh->a0_full), 0, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT, p.wait_cycles);
            else {
                ok = mbar_wait_cluster(smem_u32(&sh->act_full[buf]), (uint32_t)((L - 1) >> 1) & 1, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT, p.wait_cycles);
                if (ok) ok = mbar_wait(smem_u32(&sh->acc_empty), (uint32_t)(L - 1) & 1, abort_flag, p.err, FFCU_ERR_TMEM_TIMEOUT, p.wait_cycles);
            }
            if (!ok) break;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_after();
#ifdef FF_TC_TIMING
            if (p.ts && rank == 0 && lane == 0 && me == 0) p.ts[4 * L + 0] = globaltimer_ns();      // input complete
#endif
            da_layer = smem_desc<128>(s_a_addr + (uint32_t)buf * a_buf_bytes + (uint32_t)(tile_line0 * 128));
            first = 0;
        }
        if (!ready) {
            ok = mbar_wait(full0 + stage * 8, phase, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT, p.wait_cycles);
            if (!ok) break;
        }
        // this issuer's next stage: test its barrier now, use the answer next round (a test takes a few hundred cycles)
        int ns = stage + 2; uint32_t np = phase;
        if (ns >= stages) { ns -= stages; np ^= 1; }
        ready = mbar_test(full0 + ns * 8, np);
        tc_fence_after();
        {
            // first tap of the stage: (kh, kw) = (st, 0) when a stage is a filter row, (st / 3, st % 3) otherwise
            const int kh = (TPS == 3) ? st : st / 3;
            const int kw0 = (TPS == 3) ? 0 : st - 3 * kh;
            const uint64_t da0 = da_layer + (uint64_t)((uint32_t)kh * P8 + (uint32_t)kw0 * 8u);
            const uint64_t db0 = db_base + (uint64_t)((uint32_t)(stage * STAGE_BYTES) >> 4);
#pragma unroll
            for (int g = 0; g < TPS; g++)
#pragma unroll
                for (int pl = 0; pl < PLANES; pl++)
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        umma_i8_w(leader, d_tmem, da0 + (uint64_t)(g * 8 + 2 * k) + (uint64_t)pl * dplane,
                                  db0 + (uint64_t)(((g * PLANES + pl) * B_BLOCK >> 4) + 2 * k), IDESC,
                                  (g | pl | k) ? 1u : first);
            first = 1;
        }
        umma_commit_w(leader, empty0 + stage * 8);
        stage = ns; phase = np;
        st += 2;
        if (st >= S) {                                      // that was this issuer's last stage of the layer
            umma_commit_w(leader, smem_u32(&sh->acc_full));
#ifdef FF_TC_TIMING
            if (p.ts && rank == 0 && lane == 0 && st - 2 == S - 1) p.ts[4 * L + 1] = globaltimer_ns();   // last MMA issued
#endif
            st -= S; L++; new_layer = true;
        }
    }
}

template <bool CONTRACT>
__global__ void __launch_bounds__(TC_THREADS, 1)
conv_chain_kernel(const __grid_constant__ CUtensorMap mapA, const ChainParams p)
{
    tc_pdl_trigger();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr uint32_t TMEM_COLS = 2 * CHAIN_BN;          // one accumulator per MMA issuer
    constexpr uint32_t IDESC = idesc_i8(CHAIN_BN);
    constexpr int B_BLOCK = CHAIN_BN * 128;               // one plane of one tap: 64 output channels x 128 input channels

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int tile_m = (int)rank / p.tiles_n;
    const int tile_n = (int)rank % p.tiles_n;
    const int a_buf_bytes = p.planes * p.plane_bytes;
    const int stage_bytes = p.tps * p.planes * B_BLOCK;
    // Row tile t produces output rows [t * 128 / P, (t * 128 + 127) / P] (clipped to the map) and reads the
    // input rows one above and one below: a CTA receives only those rows of every layer's result.
    // A CTA keeps only the lines its row tile reads: a window of p.win_rows padded rows starting at the
    // first output row of its tile (padded row index = output row + kh).  base_line(t) is a multiple of 8
    // lines, so a line's swizzle phase is the same in every window.
    auto base_line = [&](int t) { return ((t * TC_TILE_M) / p.P) * p.P; };
    auto rows_lo = [&](int t) { return (t * TC_TILE_M) / p.P - 1; };
    auto rows_hi = [&](int t) { const int h = (t * TC_TILE_M + TC_TILE_M - 1) / p.P; return (h < p.H - 1 ? h : p.H - 1) + 1; };
    uint8_t* s_a = smem;                                  // [2][planes][plane_bytes]
    uint8_t* s_b = s_a + 2 * a_buf_bytes;                 // [stages][planes][B_BLOCK]
    uint8_t* s_lut = s_b + p.stages * stage_bytes;        // [64][256]
    float* s_tab = (float*)(s_lut + CHAIN_BN * 256);      // [5][64]: w_scale, bias, slope, res_scale, inv_out of the current layer
    ChainShared* sh = (ChainShared*)(s_tab + 5 * CHAIN_BN);

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) { mbar_init(smem_u32(&sh->full[s]), 1); mbar_init(smem_u32(&sh->empty[s]), 1); }
        mbar_init(smem_u32(&sh->act_full[0]), 1);          // one arming arrival; the rest is byte counting
        mbar_init(smem_u32(&sh->act_full[1]), 1);
        mbar_init(smem_u32(&sh->a0_full), 1);
        mbar_init(smem_u32(&sh->acc_full), 2);              // both issuers' MMAs of the layer are complete
        mbar_init(smem_u32(&sh->acc_empty), CHAIN_EPI_WARPS);
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&sh->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                   // every peer's barriers are initialised
    tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;
    volatile int* abort_flag = &sh->abort_flag;
    const uint32_t full0 = smem_u32(&sh->full[0]), empty0 = smem_u32(&sh->empty[0]);

    if (warp == 0) {
        // Weight producer.  One stage = p.tps filter taps of this CTA's 64 output channels (planes boxes of
        // 8 KB each); the ring runs ahead across layers.  The first layer's activations are requested once the
        // ring is full of weights: they are the only thing that depends on the previous kernel.
        const int G = p.tps;                                  // filter taps per stage
        const int total_steps = p.n_layers * (9 / G);
        const int pre = p.stages < total_steps ? p.stages : total_steps;
        int stage = 0; uint32_t phase = 0;
        bool ok = true;
        int L = 0, tap = 0;
        const int my_g = lane / p.planes, my_pl = lane - my_g * p.planes;   // this lane's box within a stage
        const bool loader = lane < G * p.planes;
#pragma unroll 1
        for (int gs = 0; gs < total_steps && ok; gs++) {
            if (gs == pre) {
                tc_pdl_wait();
                if (lane == 0) mbar_expect_tx(smem_u32(&sh->a0_full), 2 * a_buf_bytes);
                __syncwarp();
                // both buffers: the copy into the second one only puts the zero lines of the padding in place
                if (lane < 2 * p.planes)
                    tma_load_4d(smem_u32(s_a) + lane * p.plane_bytes, &mapA, smem_u32(&sh->a0_full),
                                (lane % p.planes) * 128, -1, (tile_m * TC_TILE_M) / p.P - 1, 0);
            }
            ok = mbar_wait(empty0 + stage * 8, phase ^ 1, abort_flag, p.err, FFCU_ERR_EMPTY_TIMEOUT, p.wait_cycles);
            if (!ok) break;
#ifdef FF_TC_TIMING
            if (p.dbg & 1) {
                if (lane == 0) mbar_arrive(full0 + stage * 8);
                if (++stage == p.stages) { stage = 0; phase ^= 1; }
                tap += G;
                if (tap == 9) { tap = 0; L++; }
                continue;
            }
#endif
            if (lane == 0) mbar_expect_tx(full0 + stage * 8, stage_bytes);
            __syncwarp();
            if (gs == p.drop_step && rank == 0) {
                // armed by ffcu_test_arm_chain_timeout for one launch: CTA 0 never requests this stage's weights, so its
                // issuer's (shortened) wait runs out and, for want of CTA 0's results, every peer's does after it
                if (++stage == p.stages) { stage = 0; phase ^= 1; }
                tap += G;
                if (tap == 9) { tap = 0; L++; }
                continue;
            }
            if (tap == 0 && loader) {
                // the layer's tensor map sits in global memory, put there by a host copy: order this thread's
                // use of it (through the tensor-map proxy) after that write
                asm volatile("fence.proxy.tensormap::generic.acquire.sys [%0], 128;" ::"l"(&p.layers[L].mapB) : "memory");
            }
            if (loader)
                tma_load_4d(smem_u32(s_b) + stage * stage_bytes + lane * B_BLOCK, &p.layers[L].mapB, full0 + stage * 8,
                            (tap + my_g) * p.C + my_pl * 128, tile_n * CHAIN_BN, 0, 0);
            if (++stage == p.stages) { stage = 0; phase ^= 1; }
            tap += G;
            if (tap == 9) { tap = 0; L++; }
        }
    } else if (warp == 1 || warp == TC_ISSUER2_WARP) {
        const int me = (warp == 1) ? 0 : 1;
        const int tile_line0 = tile_m * TC_TILE_M - base_line(tile_m);
        const int my_lo = rows_lo(tile_m) < 0 ? 0 : rows_lo(tile_m);
        const int my_hi = rows_hi(tile_m) > p.H - 1 ? p.H - 1 : rows_hi(tile_m);
        const uint32_t in_bytes = (uint32_t)((my_hi - my_lo + 1) * p.W * p.C);
        if (p.planes == 2 && p.tps == 3)      chain_issuer_role<2, 3>(p, sh, me, lane, rank, tmem_base, smem_u32(s_a), smem_u32(s_b), tile_line0, in_bytes);
        else if (p.planes == 2)               chain_issuer_role<2, 1>(p, sh, me, lane, rank, tmem_base, smem_u32(s_a), smem_u32(s_b), tile_line0, in_bytes);
        else                                  chain_issuer_role<4, 1>(p, sh, me, lane, rank, tmem_base, smem_u32(s_a), smem_u32(s_b), tile_line0, in_bytes);
    } else {
        // Epilogue: sixteen warps on the CTA's one tile, warp = (TMEM lane quarter, 16-channel group).
        const int q = warp & 3;
        const int cg = (warp - 2) >> 2;
        const int qpos = tile_m * TC_TILE_M + q * 32 + lane;      // position r * P + c of this thread's output
        const int r = qpos / p.P, c = qpos - r * p.P;
        const bool valid = (c < p.W) && (r < p.H);
        const int cb = tile_n * CHAIN_BN + cg * 16;                // first of this thread's 16 channels
        const size_t o = (size_t)(r * p.W + c) * p.C + cb;
        // where this output sits in the next layer's input: line (r + 1) * P + (c + 1), 16-byte chunk swizzled
        const int out_line = qpos + p.P + 1;
        const uint32_t nx_off = (uint32_t)((cb >> 7) * p.plane_bytes + out_line * 128 + ((((cb & 127) >> 4) ^ (out_line & 7)) << 4));
        const uint32_t taddr = tmem_base + (uint32_t)(cg * 16) + ((uint32_t)(q * 32) << 16);
        const uint32_t lut_base = smem_u32(s_lut) + (uint32_t)(cg * 16) * 256u;
        uint32_t dest_mask = 0;                                    // peers whose row tile reads this thread's output row
        for (int rk = 0; rk < CHAIN_CLUSTER; rk++) {
            const int t = rk / p.tiles_n;
            if (valid && r >= rows_lo(t) && r <= rows_hi(t)) dest_mask |= 1u << rk;
        }
        const int et = threadIdx.x - 64;                           // 0 .. 511 among the epilogue threads
        int lut_layer = -1;                                        // layer whose table s_lut holds
        bool ok = true;
        tc_pdl_wait();
#pragma unroll 1
        for (int L = 0; L < p.n_layers; L++) {
            // All epilogue warps are past the previous layer (its table reads included).  The two barriers
            // are executed by every warp in every iteration, whatever its ok flag: none may be left waiting.
            chain_bar_sync_epi();
            const ChainLayer* cl = p.layers + L;
            const int8_t* lutp = cl->lut;
            int8_t* out2 = cl->out2;
            const bool has_bn2 = (out2 != nullptr) && (lutp != nullptr);
            if (ok) {
                const int8_t* src = nullptr;
                if (has_bn2) { if (lut_layer != L) { src = lutp; lut_layer = L; } }
                else if (L + 1 < p.n_layers) {
                    // this layer reads no table: fetch the next layer's while the MMAs run
                    const int8_t* nl = p.layers[L + 1].lut;
                    if (nl && p.layers[L + 1].out2) { src = nl; lut_layer = L + 1; }
                }
                if (src) {
                    const int4* s4 = (const int4*)(src + (size_t)tile_n * CHAIN_BN * 256) + et * 2;
                    int4* d4 = (int4*)s_lut + et * 2;
                    d4[0] = __ldg(s4); d4[1] = __ldg(s4 + 1);
                }
                if (et < 5 * CHAIN_BN) {
                    // this layer's per-channel constants for the CTA's 64 channels
                    const int t = et >> 6, ch = et & 63;
                    const float* tp = t == 0 ? cl->w_scale : t == 1 ? cl->bias : t == 2 ? cl->slope : t == 3 ? cl->res_scale : cl->inv_out;
                    s_tab[et] = tp ? __ldg(tp + tile_n * CHAIN_BN + ch) : 0.0f;
                }
            }
            chain_bar_sync_epi();
            if (!ok) continue;
            const int8_t* res = cl->res;
            int8_t* out = cl->out;
            const bool has_res = (res != nullptr) && (cl->res_scale != nullptr);
            const bool has_slope = cl->slope != nullptr;
            int rw[4] = {0, 0, 0, 0};
            if (has_res && valid) {
                // written by a peer's epilogue two layers ago (or by an earlier kernel): read past L1
                asm volatile("ld.global.cg.v4.b32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(rw[0]), "=r"(rw[1]), "=r"(rw[2]), "=r"(rw[3]) : "l"(res + o));
            }
            ok = mbar_wait(smem_u32(&sh->acc_full), (uint32_t)L & 1, abort_flag, p.err, FFCU_ERR_EPI_TIMEOUT, p.wait_cycles);
            if (!ok) continue;
            tc_fence_after();
#ifdef FF_TC_TIMING
            if (p.ts && rank == 0 && warp == 2 && lane == 0) p.ts[4 * L + 2] = globaltimer_ns();   // accumulator complete
#endif
            int v[16], v2[16];
            tmem_ld16_issue(taddr, v);
            tmem_ld16_issue(taddr + CHAIN_BN, v2);                 // the second issuer's partial sums
            tmem_ld_wait(v);
            tmem_ld_wait(v2);
#pragma unroll
            for (int i = 0; i < 16; i++) v[i] += v2[i];
            int ow[4], ow2[4];
#pragma unroll
            for (int g = 0; g < 4; g++) {
                const int rr = rw[g];
                const float* tg = s_tab + cg * 16 + 4 * g;
                const float4 ws = *(const float4*)(tg), bi = *(const float4*)(tg + CHAIN_BN), sl = *(const float4*)(tg + 2 * CHAIN_BN);
                const float4 rs = *(const float4*)(tg + 3 * CHAIN_BN), iv = *(const float4*)(tg + 4 * CHAIN_BN);
                const float f0 = ffcu_conv_fp<CONTRACT>(v[4 * g + 0], ws.x, bi.x, has_res, (int)(int8_t)(rr & 0xff), rs.x, has_slope, sl.x);
                const float f1 = ffcu_conv_fp<CONTRACT>(v[4 * g + 1], ws.y, bi.y, has_res, (int)(int8_t)((rr >> 8) & 0xff), rs.y, has_slope, sl.y);
                const float f2 = ffcu_conv_fp<CONTRACT>(v[4 * g + 2], ws.z, bi.z, has_res, (int)(int8_t)((rr >> 16) & 0xff), rs.z, has_slope, sl.z);
                const float f3 = ffcu_conv_fp<CONTRACT>(v[4 * g + 3], ws.w, bi.w, has_res, rr >> 24, rs.w, has_slope, sl.w);
                const int w = ffcu_pack4(ffcu_requant_nosat<false>(f0, iv.x), ffcu_requant_nosat<false>(f1, iv.y),
                                         ffcu_requant_nosat<false>(f2, iv.z), ffcu_requant_nosat<false>(f3, iv.w));
                ow[g] = w;
                ow2[g] = 0;
                if (has_bn2) {
                    const uint32_t row = lut_base + (uint32_t)(4 * g) * 256u;
                    uint32_t b0, b1, b2, b3;
                    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(b0) : "r"(row + ((uint32_t)w & 0xffu)));
                    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(b1) : "r"(row + 256u + (((uint32_t)w >> 8) & 0xffu)));
                    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(b2) : "r"(row + 512u + (((uint32_t)w >> 16) & 0xffu)));
                    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(b3) : "r"(row + 768u + ((uint32_t)w >> 24)));
                    ow2[g] = (int)(b0 | (b1 << 8) | (b2 << 16) | (b3 << 24));
                }
            }
            if (L + 1 < p.n_layers) {
                // the next layer's input: straight into the peers' shared memory; each 16-byte store counts
                // its bytes on the destination CTA's barrier when it has landed
                const uint32_t dst = smem_u32(s_a) + (uint32_t)(((L + 1) & 1) * a_buf_bytes) + nx_off;
                const uint32_t bar = smem_u32(&sh->act_full[(L + 1) & 1]);
                const int n0 = has_bn2 ? ow2[0] : ow[0], n1 = has_bn2 ? ow2[1] : ow[1];
                const int n2 = has_bn2 ? ow2[2] : ow[2], n3 = has_bn2 ? ow2[3] : ow[3];
#pragma unroll
                for (uint32_t rk = 0; rk < CHAIN_CLUSTER; rk++)
                    if (dest_mask & (1u << rk))
                        asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
                                     ::"r"(map_to_cta(dst - (uint32_t)(base_line((int)rk / p.tiles_n) * 128), rk)),
                                       "r"(n0), "r"(n1), "r"(n2), "r"(n3), "r"(map_to_cta(bar, rk)) : "memory");
            }
            tc_fence_before();                                     // this warp's TMEM reads are complete
            __syncwarp();
            if (lane == 0) mbar_arrive_relaxed(smem_u32(&sh->acc_empty));
#ifdef FF_TC_TIMING
            if (p.ts && rank == 0 && warp == 2 && lane == 0) p.ts[4 * L + 3] = globaltimer_ns();   // results sent
#endif
            if (valid) {
                *(int4*)(out + o) = make_int4(ow[0], ow[1], ow[2], ow[3]);
                if (has_bn2) *(int4*)(out2 + o) = make_int4(ow2[0], ow2[1], ow2[2], ow2[3]);
            }
        }
    }
    // teardown: nobody leaves (and frees shared memory a peer may still write) before the whole cluster is here
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

int tc_launch_chain(int mode, int smem, cudaStream_t s, const CUtensorMap& mapA, const ChainParams& prm)
{
    static int smem_set[2][64] = {};      // per device: the attribute belongs to the device's copy of the function
    int dev = 0;
    FFCU_CHECK(cudaGetDevice(&dev));
    if (smem_set[mode ? 1 : 0][dev & 63] < smem) {
        if (mode) FFCU_CHECK(cudaFuncSetAttribute(conv_chain_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        else      FFCU_CHECK(cudaFuncSetAttribute(conv_chain_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        smem_set[mode ? 1 : 0][dev & 63] = smem;
    }
    if (mode) return tc_launch_ex(conv_chain_kernel<true>, CHAIN_CLUSTER, smem, s, CHAIN_CLUSTER, mapA, prm);
    return tc_launch_ex(conv_chain_kernel<false>, CHAIN_CLUSTER, smem, s, CHAIN_CLUSTER, mapA, prm);
}

// Can this device co-schedule one cluster of the chain kernel (eight CTAs with `smem` bytes each in one GPC)?
// Asked once per plan; a device that cannot keeps the per-layer launches.
bool tc_chain_fits(int smem)
{
    if (cudaFuncSetAttribute(conv_chain_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess ||
        cudaFuncSetAttribute(conv_chain_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(CHAIN_CLUSTER);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CHAIN_CLUSTER; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, conv_chain_kernel<true>, &cfg) != cudaSuccess) { cudaGetLastError(); return false; }
    return n >= 1;
}
