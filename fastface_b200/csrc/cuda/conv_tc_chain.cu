// conv_tc_chain.cu -- batch-1 latency path: a run of consecutive 3x3 stride-1 convolutions of one
// shape (the 26 layers of the 14x14 stage, the 4 of the 7x7 stage) in ONE launch of one cluster of
// eight CTAs, with the activations resident in shared memory.
//
// At batch 1 a 14x14 layer is 8 tiles (2 row tiles x 4 column tiles of 64 channels); as separate
// launches each layer pays kernel completion + dependency release + a TMA round trip for 50 KB of
// activations before its first MMA.  Here the eight CTAs of a cluster take one tile each and keep
// the WHOLE input tensor of the current layer in their own shared memory, laid out the way a TMA
// load with 128-byte swizzle would have left it: line (row + 1) * P + (col + 1) of 128 channels per
// plane, P = pitch in lines, zero lines for the padding.  Filter tap (kh, kw) is then the same buffer
// read (kh * P + kw) lines further on (the tensor core applies the swizzle to absolute shared-memory
// addresses), so the activations need no loads at all.  A CTA's epilogue writes its 128 x 64 result,
// already requantised to int8 (the fused BN's output where the layer has one), into the NEXT layer's
// buffer of all eight CTAs (st.shared::cluster) and arrives on their barriers; the weights stream
// through a TMA ring that runs ahead across layer boundaries, since they depend on nothing.
// Global memory still receives every output (the residual two layers on reads it from there, and the
// kernel after the chain).  Replaces, per layer, what conv_tc_kernel does (reference
// kernels/conv2d_nhwc.c:179-220, kernels/int8_epilogue.c:25-112, :253-318); same arithmetic, same bytes.
//
// Every wait is bounded as in the other kernels; nobody leaves before the whole cluster has
// arrived at the final barrier, so no CTA's shared memory is written after it has exited.
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

template <bool CONTRACT>
__global__ void __launch_bounds__(TC_THREADS, 1)
conv_chain_kernel(const __grid_constant__ CUtensorMap mapA, const ChainParams p)
{
    tc_pdl_trigger();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr uint32_t TMEM_COLS = 64;
    constexpr uint32_t IDESC = idesc_i8(CHAIN_BN);
    constexpr int B_BLOCK = CHAIN_BN * 128;               // one plane of one tap: 64 output channels x 128 input channels

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int tile_m = (int)rank / p.tiles_n;
    const int tile_n = (int)rank % p.tiles_n;
    const int a_buf_bytes = p.planes * p.plane_bytes;
    const int stage_bytes = p.planes * B_BLOCK;
    // Row tile t produces output rows [t * 128 / P, (t * 128 + 127) / P] (clipped to the map) and reads the
    // input rows one above and one below: a CTA receives only those rows of every layer's result.
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
        mbar_init(smem_u32(&sh->acc_full), 1);
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
        // Weight producer.  One stage = one filter tap of this CTA's 64 output channels (planes boxes of
        // 8 KB); the ring runs ahead across layers.  The first layer's activations are requested once the
        // ring is full of weights: they are the only thing that depends on the previous kernel.
        const int total_steps = p.n_layers * 9;
        const int pre = p.stages < total_steps ? p.stages : total_steps;
        int stage = 0; uint32_t phase = 0;
        bool ok = true;
        int L = 0, tap = 0;
#pragma unroll 1
        for (int gs = 0; gs < total_steps && ok; gs++) {
            if (gs == pre) {
                tc_pdl_wait();
                if (lane == 0) mbar_expect_tx(smem_u32(&sh->a0_full), 2 * a_buf_bytes);
                __syncwarp();
                // both buffers: the copy into the second one only puts the zero lines of the padding in place
                if (lane < 2 * p.planes)
                    tma_load_4d(smem_u32(s_a) + lane * p.plane_bytes, &mapA, smem_u32(&sh->a0_full),
                                (lane % p.planes) * 128, -1, -1, 0);
            }
            ok = mbar_wait(empty0 + stage * 8, phase ^ 1, abort_flag, p.err, FFCU_ERR_EMPTY_TIMEOUT);
            if (!ok) break;
            if (lane == 0) mbar_expect_tx(full0 + stage * 8, stage_bytes);
            __syncwarp();
            if (tap == 0 && lane < p.planes) {
                // the layer's tensor map sits in global memory, put there by a host copy: order this thread's
                // use of it (through the tensor-map proxy) after that write
                asm volatile("fence.proxy.tensormap::generic.acquire.sys [%0], 128;" ::"l"(&p.layers[L].mapB) : "memory");
            }
            if (lane < p.planes)
                tma_load_4d(smem_u32(s_b) + stage * stage_bytes + lane * B_BLOCK, &p.layers[L].mapB, full0 + stage * 8,
                            tap * p.C + lane * 128, tile_n * CHAIN_BN, 0, 0);
            if (p.l2_ahead && L + 1 < p.n_layers && lane < p.planes) {
                // the same tap of the NEXT layer's weights: into L2 now, so that its TMA load a layer later is a hit
                asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];"
                             ::"l"(&p.layers[L + 1].mapB), "r"(tap * p.C + lane * 128), "r"(tile_n * CHAIN_BN), "r"(0), "r"(0) : "memory");
            }
            if (++stage == p.stages) { stage = 0; phase ^= 1; }
            if (++tap == 9) { tap = 0; L++; }
        }
    } else if (warp == 1) {
        // MMA issuer: the warp loops and waits together, lane 0 issues
        int stage = 0; uint32_t phase = 0;
        bool ok = true;
        const uint32_t leader = (lane == 0) ? 1u : 0u;
        const uint64_t da_base = smem_desc<128>(smem_u32(s_a));
        const uint64_t db_base = smem_desc<128>(smem_u32(s_b));
        uint32_t ready = 0;                                 // answer of the early test for the upcoming stage
        // bytes of one layer's result this CTA receives: its rows x W positions x C channels
        const int my_lo = rows_lo(tile_m) < 0 ? 0 : rows_lo(tile_m);
        const int my_hi = rows_hi(tile_m) > p.H - 1 ? p.H - 1 : rows_hi(tile_m);
        const uint32_t in_bytes = (uint32_t)((my_hi - my_lo + 1) * p.W * p.C);
#pragma unroll 1
        for (int L = 0; L < p.n_layers && ok; L++) {
            const int buf = L & 1;
            // arm the barrier of the buffer the peers fill during this layer (bytes that land before this
            // only drive the count negative for a moment: the phase cannot complete before this arrival)
            if (L + 1 < p.n_layers && lane == 0) mbar_expect_tx(smem_u32(&sh->act_full[buf ^ 1]), in_bytes);
            if (L == 0) ok = mbar_wait(smem_u32(&sh->a0_full), 0, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT);
            else {
                ok = mbar_wait_cluster(smem_u32(&sh->act_full[buf]), (uint32_t)((L - 1) >> 1) & 1, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT);
                if (ok) ok = mbar_wait(smem_u32(&sh->acc_empty), (uint32_t)(L - 1) & 1, abort_flag, p.err, FFCU_ERR_TMEM_TIMEOUT);
            }
            if (!ok) break;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_after();
#ifdef FF_TC_TIMING
            if (p.ts && rank == 0 && lane == 0) p.ts[4 * L + 0] = globaltimer_ns();      // input complete
#endif
            const uint32_t a_off0 = (uint32_t)(buf * a_buf_bytes + tile_m * TC_TILE_M * 128);
            uint64_t da_row = da_base + (uint64_t)(a_off0 >> 4);   // descriptor of tap (kh, 0), plane 0
            int kw = 0;
#pragma unroll 1
            for (int tap = 0; tap < 9; tap++) {
                if (!ready) {
                    ok = mbar_wait(full0 + stage * 8, phase, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT);
                    if (!ok) break;
                }
                // test the next stage now, use the answer next round (a barrier test takes a few hundred cycles)
                int ns = stage + 1; uint32_t np = phase;
                if (ns == p.stages) { ns = 0; np ^= 1; }
                ready = mbar_test(full0 + ns * 8, np);
                tc_fence_after();
                uint64_t da = da_row + (uint64_t)(kw * 8);          // one line = 128 bytes = 8 descriptor units
#ifdef FF_TC_TIMING
                if (p.l2_ahead & 2) da = da_row;                    // timing experiment: every tap from an atom-aligned start (wrong results)
#endif
                uint64_t db = db_base + (uint64_t)((uint32_t)(stage * stage_bytes) >> 4);
#pragma unroll 1
                for (int pl = 0; pl < p.planes; pl++, da += (uint64_t)(p.plane_bytes >> 4), db += (uint64_t)(B_BLOCK >> 4)) {
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        umma_i8_w(leader, tmem_base, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), IDESC, (tap | pl | k) ? 1u : 0u);
                }
                umma_commit_w(leader, empty0 + stage * 8);
                stage = ns; phase = np;
                if (++kw == 3) { kw = 0; da_row += (uint64_t)(p.P * 8); }
            }
            if (ok) umma_commit_w(leader, smem_u32(&sh->acc_full));
#ifdef FF_TC_TIMING
            if (p.ts && rank == 0 && lane == 0) p.ts[4 * L + 1] = globaltimer_ns();      // last MMA issued
#endif
        }
    } else if (warp < TC_ISSUER2_WARP) {
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
            ok = mbar_wait(smem_u32(&sh->acc_full), (uint32_t)L & 1, abort_flag, p.err, FFCU_ERR_EPI_TIMEOUT);
            if (!ok) continue;
            tc_fence_after();
#ifdef FF_TC_TIMING
            if (p.ts && rank == 0 && warp == 2 && lane == 0) p.ts[4 * L + 2] = globaltimer_ns();   // accumulator complete
#endif
            int v[16];
            tmem_ld16(taddr, v);
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
                                     ::"r"(map_to_cta(dst, rk)), "r"(n0), "r"(n1), "r"(n2), "r"(n3), "r"(map_to_cta(bar, rk)) : "memory");
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
