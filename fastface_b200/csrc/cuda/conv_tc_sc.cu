// conv_tc_sc.cu -- a residual block's stride-2 3x3 convolution and its 1x1 stride-2 shortcut in ONE launch.
//
// In the down-sampling blocks the op list ends with  conv 3x3 stride 2 (main path)  ->  conv 1x1 stride 2 on the
// block's input with the ADD fused (residual = the main path's int8 output) [-> BN of the next block].  Both produce
// the same output tile, so one CTA computes both: the main convolution's K loop into one TMEM accumulator, then the
// shortcut's one or two K blocks (its own input and weight tensor maps) into a second one, and a single epilogue
// requantises the main accumulator to int8 exactly as its own launch would (reference
// kernels/int8_epilogue.c:25-112), feeds those bytes as the residual into the shortcut's epilogue and applies the
// fused BN's byte table.  Same bytes as the two launches; the main path's tensor is not written at all unless another
// layer reads it.  Used where the call's column tile is 64 channels wide: every down-sampling block at small batch
// (a launch less per block: ~4 us of a 300 us forward each), the 112x112 one at any batch.
//
// Structure and bounded waits as conv_tc_kernel (conv_tc_generic.cu); 64-column tiles, four tile slots of two
// accumulators in the 512 TMEM columns.
#include "conv_tc_common.cuh"

#define SC_BN 64
#define SC_SLOTS (TC_NACC(SC_BN) / 2)          // tiles in flight: two accumulators each

__device__ __forceinline__ void sc_load_tables(float* tab, const EpiTables& t, int Cout)
{
#pragma unroll 1
    for (int i = threadIdx.x; i < Cout; i += TC_THREADS) {
        tab[0 * TC_MAX_COUT + i] = t.w_scale[i];
        tab[1 * TC_MAX_COUT + i] = t.bias[i];
        tab[2 * TC_MAX_COUT + i] = t.slope ? t.slope[i] : 0.0f;
        tab[3 * TC_MAX_COUT + i] = t.res_scale ? t.res_scale[i] : 0.0f;
        tab[4 * TC_MAX_COUT + i] = t.inv_out ? t.inv_out[i] : 0.0f;
    }
}

template <int KC, bool CONTRACT>
__global__ void __launch_bounds__(TC_THREADS, 1)
conv_sc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
               const __grid_constant__ CUtensorMap mapA2, const __grid_constant__ CUtensorMap mapB2,
               const TcParams p, const ScParams q)
{
    tc_pdl_trigger();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int BN = SC_BN;
    constexpr int A_BYTES = TC_TILE_M * KC;
    constexpr int B_BYTES = BN * KC;
    constexpr int SUB_BYTES = A_BYTES + B_BYTES;          // one K block: [A 128 x KC | B 64 x KC]
    constexpr uint32_t TMEM_COLS = TC_NACC(BN) * BN;
    constexpr uint32_t IDESC = idesc_i8(BN);

    float* tab1 = (float*)(smem + (size_t)p.stages * p.group * SUB_BYTES);     // main path: [5][TC_MAX_COUT]
    float* tab2 = tab1 + 5 * TC_MAX_COUT;                                       // shortcut:  [5][TC_MAX_COUT]
    uint8_t* lut = (uint8_t*)(tab2 + 5 * TC_MAX_COUT);                          // [64][256] fused-BN table of the block's output
    TcShared* sh = (TcShared*)(lut + q.lut_bytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int kblocks = p.taps * p.cin_blocks;
    const int G = p.group;
    const int n_steps = kblocks / G;
    const int tn = blockIdx.x % p.tiles_n;

    sc_load_tables(tab1, p.t, p.Cout);
    sc_load_tables(tab2, q.t2, p.Cout);
    if (q.lut_bytes) {
        const int4* src = (const int4*)(q.t2.bn_lut + (size_t)tn * BN * 256);
        int4* dst = (int4*)lut;
#pragma unroll 1
        for (int i = threadIdx.x; i < BN * 16; i += TC_THREADS) dst[i] = __ldg(src + i);
    }
    tc_setup(sh, p.stages, TMEM_COLS, warp, p.epi_wps);
    const uint32_t tmem_base = sh->tmem_base;
    volatile int* abort_flag = &sh->abort_flag;
    const uint32_t full0 = smem_u32(&sh->full[0]), empty0 = smem_u32(&sh->empty[0]);
    const int stage_bytes = G * SUB_BYTES;

    if (warp == 0) {
        // TMA producer: per tile the main path's K loop (lane 2g: activation box of block g, lane 2g+1: its weight
        // box, G blocks per stage), then ONE stage with the shortcut's kb_sc blocks from its own tensor maps.
        int stage = 0; uint32_t phase = 0;
        bool ok = true;
        const bool issuer = lane < 2 * G;
        const int g = issuer ? (lane >> 1) : 0;
        const bool is_a = (lane & 1) == 0;
        const CUtensorMap* map = is_a ? &mapA : &mapB;
        const CUtensorMap* map2 = is_a ? &mapA2 : &mapB2;
        const uint32_t smem0 = smem_u32(smem) + (uint32_t)(g * SUB_BYTES) + (is_a ? 0u : (uint32_t)A_BYTES);
        int c0_first = g * KC, kw_first = 0, kh_first = 0;
        while (c0_first >= p.Cp) { c0_first -= p.Cp; if (++kw_first == p.Kw) { kw_first = 0; kh_first++; } }
        tc_pdl_wait();
        TileWalk wk;
        walk_init(wk, p, blockIdx.x / p.tiles_n, gridDim.x / p.tiles_n);
        for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x, walk_next(wk, p)) {
            const int tw = wk.tw, th = wk.th, tb = wk.tb;
            const int x0 = tw * p.TW * p.stride - p.pad;
            const int y0 = th * p.TH * p.stride - p.pad;
            const int c3 = is_a ? tb * p.TB : 0;
            int c0 = c0_first, kw = kw_first, kh = kh_first;
#pragma unroll 1
            for (int it = 0; it <= n_steps; it++) {
                ok = mbar_wait(empty0 + stage * 8, phase ^ 1, abort_flag, p.err, FFCU_ERR_EMPTY_TIMEOUT);
                if (!ok) break;
                if (it < n_steps) {
                    if (lane == 0) mbar_expect_tx(full0 + stage * 8, G * SUB_BYTES);
                    __syncwarp();                           // the byte count is armed before any copy can land
                    const int tapk = (kh * p.Kw + kw) * p.Cp + c0;
                    if (issuer)
                        tma_load_4d(smem0 + stage * stage_bytes, map, full0 + stage * 8,
                                    is_a ? c0 : tapk, is_a ? x0 + kw : tn * BN, is_a ? y0 + kh : 0, c3);
                    c0 += G * KC;
                    while (c0 >= p.Cp) { c0 -= p.Cp; if (++kw == p.Kw) { kw = 0; kh++; } }
                } else {
                    // the shortcut: 1x1, stride 2, no padding: input pixel (2 * oh, 2 * ow) of the block's input
                    if (lane == 0) mbar_expect_tx(full0 + stage * 8, q.kb_sc * SUB_BYTES);
                    __syncwarp();
                    if (lane < 2 * q.kb_sc)
                        tma_load_4d(smem0 + stage * stage_bytes, map2, full0 + stage * 8,
                                    g * KC, is_a ? tw * p.TW * 2 : tn * BN, is_a ? th * p.TH * 2 : 0, c3);
                }
                if (++stage == p.stages) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        // MMA issuer: the warp loops and waits together, lane 0 issues
        int stage = 0; uint32_t phase = 0;
        int ts = 0; uint32_t tphase = 0;                    // tile slot (two accumulators) and its phase
        bool ok = true;
        const uint64_t da0 = smem_desc<KC>(smem_u32(smem));
        const uint64_t db0 = smem_desc<KC>(smem_u32(smem) + A_BYTES);
        const uint32_t leader = (lane == 0) ? 1u : 0u;
        uint32_t ready = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
            ok = mbar_wait(smem_u32(&sh->acc_empty[ts]), tphase ^ 1, abort_flag, p.err, FFCU_ERR_TMEM_TIMEOUT);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_main = tmem_base + (uint32_t)(2 * ts * BN);
            const uint32_t d_sc = d_main + BN;
#pragma unroll 1
            for (int it = 0; it <= n_steps; it++) {
                if (!ready) {
                    ok = mbar_wait(full0 + stage * 8, phase, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT, p.full_wait);
                    if (!ok) break;
                }
                int ns = stage + 1; uint32_t np = phase;
                if (ns == p.stages) { ns = 0; np ^= 1; }
                ready = mbar_test(full0 + ns * 8, np);
                tc_fence_after();
                uint32_t soff = (uint32_t)((stage * stage_bytes) >> 4);
                const int nb = it < n_steps ? G : q.kb_sc;
                const uint32_t d = it < n_steps ? d_main : d_sc;
#pragma unroll 1
                for (int g = 0; g < nb; g++, soff += (uint32_t)(SUB_BYTES >> 4)) {
#pragma unroll
                    for (int k = 0; k < KC / 32; k++)
                        umma_i8_w(leader, d, da0 + (uint64_t)(soff + 2 * k), db0 + (uint64_t)(soff + 2 * k), IDESC,
                                  ((it < n_steps ? it : 0) | g | k) ? 1u : 0u);
                }
                umma_commit_w(leader, empty0 + stage * 8);
                stage = ns; phase = np;
            }
            if (ok) umma_commit_w(leader, smem_u32(&sh->acc_full[ts]));
            if (++ts == SC_SLOTS) { ts = 0; tphase ^= 1; }
        }
    } else if (warp < TC_ISSUER2_WARP) {
        // Epilogue: 16 / wps sets of wps warps on alternate tiles; a warp = (TMEM lane quarter, column group).
        tc_pdl_wait();
        const int wps = p.epi_wps;
        const int sets = TC_EPI_TOTAL_WARPS / wps;
        const int cols = BN / (wps >> 2);
        const int n_chunks = cols >> 4;
        const int qd = warp & 3;
        const int set = (warp - 2) / wps;
        const int cg = ((warp - 2) % wps) >> 2;
        const int row = qd * 32 + lane;
        const int iw = row % p.TW;
        const int ih = (row / p.TW) % p.TH;
        const int ib = row / (p.TW * p.TH);
        const bool has_slope1 = p.t.slope != nullptr, has_slope2 = q.t2.slope != nullptr;
        const bool has_bn2 = q.out2_sc != nullptr && q.lut_bytes != 0;
        const int c0 = tn * BN + cg * cols;
        const uint32_t lut0 = smem_u32(lut) + (uint32_t)(cg * cols) * 256u;
        // this set's tiles: set, set + sets, ... of the CTA's; tile slot and phase follow the CTA's tile count
        int local = set;
        bool ok = true;
        TileWalk wk;
        walk_init(wk, p, (int)(blockIdx.x + set * gridDim.x) / p.tiles_n, (int)(gridDim.x * sets) / p.tiles_n);
        for (int tile = blockIdx.x + set * gridDim.x; tile < p.total_tiles && ok;
             tile += gridDim.x * sets, local += sets, walk_next(wk, p)) {
            const int ow = wk.tw * p.TW + iw, oh = wk.th * p.TH + ih, b = wk.tb * p.TB + ib;
            const bool valid = (ow < p.Wo) && (oh < p.Ho) && (b < p.batch);
            const size_t o0 = (((size_t)b * p.Ho + oh) * p.Wo + ow) * p.Cout + c0;
            const int ts = local % SC_SLOTS;
            const uint32_t tphase = (uint32_t)(local / SC_SLOTS) & 1;
            ok = mbar_wait(smem_u32(&sh->acc_full[ts]), tphase, abort_flag, p.err, FFCU_ERR_EPI_TIMEOUT);
            if (!ok) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + (uint32_t)(2 * ts * BN + cg * cols) + ((uint32_t)(qd * 32) << 16);
#pragma unroll 1
            for (int ch = 0; ch < n_chunks; ch++) {
                int va[16], vb[16];
                tmem_ld16_issue(taddr + (uint32_t)(16 * ch), va);
                tmem_ld16_issue(taddr + (uint32_t)(BN + 16 * ch), vb);
                tmem_ld_wait(va);
                tmem_ld_wait(vb);
                const int cb = c0 + 16 * ch;
                int wm[4], wo[4], wo2[4];
#pragma unroll
                for (int g = 0; g < 4; g++) {
                    const float* t1 = tab1 + cb + 4 * g;
                    const float* t2 = tab2 + cb + 4 * g;
                    const float4 ws1 = *(const float4*)(t1), bi1 = *(const float4*)(t1 + TC_MAX_COUT), sl1 = *(const float4*)(t1 + 2 * TC_MAX_COUT);
                    const float4 iv1 = *(const float4*)(t1 + 4 * TC_MAX_COUT);
                    const float4 ws2 = *(const float4*)(t2), bi2 = *(const float4*)(t2 + TC_MAX_COUT), sl2 = *(const float4*)(t2 + 2 * TC_MAX_COUT);
                    const float4 rs2 = *(const float4*)(t2 + 3 * TC_MAX_COUT), iv2 = *(const float4*)(t2 + 4 * TC_MAX_COUT);
                    // the main path's int8 output, exactly as its own launch would have stored it
                    const float m0 = ffcu_conv_fp_f<CONTRACT>(__int2float_rn(va[4 * g + 0]), ws1.x, bi1.x, false, 0.0f, 0.0f, has_slope1, sl1.x);
                    const float m1 = ffcu_conv_fp_f<CONTRACT>(__int2float_rn(va[4 * g + 1]), ws1.y, bi1.y, false, 0.0f, 0.0f, has_slope1, sl1.y);
                    const float m2 = ffcu_conv_fp_f<CONTRACT>(__int2float_rn(va[4 * g + 2]), ws1.z, bi1.z, false, 0.0f, 0.0f, has_slope1, sl1.z);
                    const float m3 = ffcu_conv_fp_f<CONTRACT>(__int2float_rn(va[4 * g + 3]), ws1.w, bi1.w, false, 0.0f, 0.0f, has_slope1, sl1.w);
                    const int w1 = ffcu_pack4(ffcu_requant_nosat<false>(m0, iv1.x), ffcu_requant_nosat<false>(m1, iv1.y),
                                              ffcu_requant_nosat<false>(m2, iv1.z), ffcu_requant_nosat<false>(m3, iv1.w));
                    wm[g] = w1;
                    // ... is the shortcut's residual
                    const uint32_t rx = (uint32_t)w1 ^ 0x80808080u;
                    const float f0 = ffcu_conv_fp_f<CONTRACT>(__int2float_rn(vb[4 * g + 0]), ws2.x, bi2.x, true, ffcu_byte2f<0>(rx), rs2.x, has_slope2, sl2.x);
                    const float f1 = ffcu_conv_fp_f<CONTRACT>(__int2float_rn(vb[4 * g + 1]), ws2.y, bi2.y, true, ffcu_byte2f<1>(rx), rs2.y, has_slope2, sl2.y);
                    const float f2 = ffcu_conv_fp_f<CONTRACT>(__int2float_rn(vb[4 * g + 2]), ws2.z, bi2.z, true, ffcu_byte2f<2>(rx), rs2.z, has_slope2, sl2.z);
                    const float f3 = ffcu_conv_fp_f<CONTRACT>(__int2float_rn(vb[4 * g + 3]), ws2.w, bi2.w, true, ffcu_byte2f<3>(rx), rs2.w, has_slope2, sl2.w);
                    const int w = ffcu_pack4(ffcu_requant_nosat<false>(f0, iv2.x), ffcu_requant_nosat<false>(f1, iv2.y),
                                             ffcu_requant_nosat<false>(f2, iv2.z), ffcu_requant_nosat<false>(f3, iv2.w));
                    wo[g] = w;
                    wo2[g] = 0;
                    if (has_bn2) {
                        const uint32_t rowa = lut0 + (uint32_t)(16 * ch + 4 * g) * 256u;
                        uint32_t b0, b1, b2, b3;
                        asm volatile("ld.shared.u8 %0, [%1];" : "=r"(b0) : "r"(rowa + ((uint32_t)w & 0xffu)));
                        asm volatile("ld.shared.u8 %0, [%1];" : "=r"(b1) : "r"(rowa + 256u + (((uint32_t)w >> 8) & 0xffu)));
                        asm volatile("ld.shared.u8 %0, [%1];" : "=r"(b2) : "r"(rowa + 512u + (((uint32_t)w >> 16) & 0xffu)));
                        asm volatile("ld.shared.u8 %0, [%1];" : "=r"(b3) : "r"(rowa + 768u + ((uint32_t)w >> 24)));
                        wo2[g] = (int)(b0 | (b1 << 8) | (b2 << 16) | (b3 << 24));
                    }
                }
                if (valid) {
                    const size_t o = o0 + 16 * ch;
                    if (q.write_main) *(int4*)((int8_t*)p.out + o) = make_int4(wm[0], wm[1], wm[2], wm[3]);
                    *(int4*)(q.out_sc + o) = make_int4(wo[0], wo[1], wo[2], wo[3]);
                    if (has_bn2) *(int4*)(q.out2_sc + o) = make_int4(wo2[0], wo2[1], wo2[2], wo2[3]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_relaxed(smem_u32(&sh->acc_empty[ts]));
        }
    }
    tc_teardown(abort_flag, tmem_base, TMEM_COLS, warp);
}

template <int KC, bool CONTRACT>
static int launch_sc(int grid, int smem, cudaStream_t s, const CUtensorMap& mapA, const CUtensorMap& mapB,
                     const CUtensorMap& mapA2, const CUtensorMap& mapB2, const TcParams& prm, const ScParams& q)
{
    auto kern = conv_sc_kernel<KC, CONTRACT>;
    static int smem_set[64] = {};      // per device: the attribute belongs to the device's copy of the function
    int dev = 0;
    FFCU_CHECK(cudaGetDevice(&dev));
    if (smem_set[dev & 63] < smem) {
        FFCU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        smem_set[dev & 63] = smem;
    }
    return tc_launch_ex(kern, grid, smem, s, 1, mapA, mapB, mapA2, mapB2, prm, q);
}

int tc_launch_sc(int kc, int mode, int grid, int smem, cudaStream_t s, const CUtensorMap& mapA, const CUtensorMap& mapB,
                 const CUtensorMap& mapA2, const CUtensorMap& mapB2, const TcParams& prm, const ScParams& q)
{
    if (kc == 128) return mode ? launch_sc<128, true>(grid, smem, s, mapA, mapB, mapA2, mapB2, prm, q)
                               : launch_sc<128, false>(grid, smem, s, mapA, mapB, mapA2, mapB2, prm, q);
    return mode ? launch_sc<64, true>(grid, smem, s, mapA, mapB, mapA2, mapB2, prm, q)
                : launch_sc<64, false>(grid, smem, s, mapA, mapB, mapA2, mapB2, prm, q);
}
