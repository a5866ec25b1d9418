// conv_tc_stem.cu -- the stem in ONE launch: input quantisation, im2col rows built in shared memory,
// K = 32 tensor-core GEMM, PReLU / requantisation / fused BN epilogue.
#include "conv_tc_common.cuh"

// ---------------------------------------------------------------------------
// The stem's K is 27 (3 channels x 9 taps): no TMA box can gather it from the image.  Instead of a
// separate pass that writes 32-byte im2col rows to global memory for a GEMM kernel to read back,
// two producer warps of this kernel build the rows directly in the shared-memory stage the MMA
// reads:
//   * a tile is 16 x 8 output pixels of one image.  A producer warp loads the tile's 18 x 10 input
//     patch (fp32, or 8-bit pixels, which stand for (p - 127.5) / 127.5 with the wrapper's two fp32
//     roundings, fastface.py:11), quantises each value once (quantize_fp32_nhwc_to_int8,
//     reference kernels/int8_epilogue.c:231-247: lrintf = round-half-even, clamp to [-128, 127]; for
//     8-bit input through a 3 x 256 table of exactly that arithmetic, built at kernel start) and
//     keeps it as one word per pixel in a small per-warp buffer; pixels outside the image are zero;
//   * each lane then forms four output pixels' rows: bytes [kh][kw][c] (27 values) + 5 zero bytes, and
//     stores them where a TMA load with 32-byte swizzle would have put them (row r at r * 32, its two
//     16-byte halves exchanged when bit 2 of r is set), so the K-major operand descriptor is the usual
//     one.  A proxy fence makes the stores visible to the tensor core before the stage's barrier is
//     arrived on;
//   * warp 1 issues ONE tcgen05.mma (128 x 64 x 32) per tile; sixteen epilogue warps as everywhere.
// The two producers take alternate tiles (the stage ring is even), and each has its next tile's
// patch loads in flight while it packs the current one.
// Traffic per face: 150 528 B (or 37 632 B) read, 2 x 802 816 B written; nothing in between.
// ---------------------------------------------------------------------------
#define STEM_TW 16
#define STEM_TH 8
#define STEM_PW (STEM_TW + 2)
#define STEM_PH (STEM_TH + 2)
#define STEM_PATCH (STEM_PW * STEM_PH)        // 180 input pixels
#define STEM_PER_LANE ((STEM_PATCH + 31) / 32)
#define STEM_A_BYTES (TC_TILE_M * 32)

// The tile's input patch into registers: fp32 values, or (8-bit input) the raw pixel values, which the
// quantiser then looks up; positions outside the image are marked so that they quantise to zero.
template <bool IN_U8>
__device__ __forceinline__ void stem_load_patch(const void* in_any, int b, int y0, int x0, int lane, float (&f)[STEM_PER_LANE][3])
{
#pragma unroll
    for (int i = 0; i < STEM_PER_LANE; i++) {
        const int px = lane + 32 * i;
        const int py = y0 - 1 + px / STEM_PW, pxx = x0 - 1 + px % STEM_PW;
        f[i][0] = f[i][1] = f[i][2] = IN_U8 ? -1.0f : 0.0f;
        if (px < STEM_PATCH && py >= 0 && py < 112 && pxx >= 0 && pxx < 112) {
            const size_t e = (((size_t)b * 112 + py) * 112 + pxx) * 3;
            if (IN_U8) {
                const uint8_t* x = (const uint8_t*)in_any + e;
                f[i][0] = (float)__ldg(x); f[i][1] = (float)__ldg(x + 1); f[i][2] = (float)__ldg(x + 2);
            } else {
                const float* x = (const float*)in_any + e;
                f[i][0] = __ldg(x); f[i][1] = __ldg(x + 1); f[i][2] = __ldg(x + 2);
            }
        }
    }
}

template <bool CONTRACT, int EPI, bool IN_U8>
__global__ void __launch_bounds__(TC_THREADS, 1)
conv_stem_kernel(const __grid_constant__ CUtensorMap mapB, const TcParams p, const void* __restrict__ in_any,
                 const float* __restrict__ inv3)
{
    tc_pdl_trigger();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int BN = 64;
    constexpr int W_BYTES = BN * 32;
    constexpr uint32_t TMEM_COLS = TC_NACC(BN) * BN;
    constexpr uint32_t IDESC = idesc_i8(BN);
    __shared__ uint32_t s_patch[2][STEM_PATCH];                 // quantised patch of each producer warp, one word per pixel
    __shared__ int8_t s_qlut[3][256];                           // 8-bit input: quantised value of every pixel value, per channel

    uint8_t* s_w = smem;                                        // [64][32]
    uint8_t* s_a = smem + W_BYTES;                              // [stages][128][32]
    float* tab = (float*)(s_a + (size_t)p.stages * STEM_A_BYTES);
    uint8_t* lut = (uint8_t*)(tab + p.ntab * TC_MAX_COUT);
    TcShared* sh = (TcShared*)(lut + p.lut_bytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    tc_load_tables(tab, p);
    tc_load_lut(lut, p, 0, BN);
    if (IN_U8) {
        // An 8-bit pixel has 256 values: normalise and quantise each once, with the arithmetic of the fp32
        // path ((p - 127.5) / 127.5 in fp32, then x * inv, lrintf, clamp), and let the producers look it up.
        for (int i = threadIdx.x; i < 3 * 256; i += TC_THREADS) {
            const int c = i >> 8, v = i & 255;
            const float x = __fdiv_rn(__fsub_rn((float)v, 127.5f), 127.5f);
            s_qlut[c][v] = (int8_t)max(-128, min(127, __float2int_rn(__fmul_rn(x, __ldg(inv3 + c)))));
        }
    }
    tc_setup(sh, p.stages, TMEM_COLS, warp, p.epi_wps);
    tc_pdl_wait();
    const uint32_t tmem_base = sh->tmem_base;
    volatile int* abort_flag = &sh->abort_flag;

    if (warp == 0 || warp == TC_ISSUER2_WARP) {
        // ---- producers: quantise + pack, alternate tiles ----
        const int me = (warp == 0) ? 0 : 1;
        if (me == 0 && lane == 0) {                              // the 2 KB weight matrix, once
            mbar_expect_tx(smem_u32(&sh->w_full), W_BYTES);
            tma_load_4d(smem_u32(s_w), &mapB, smem_u32(&sh->w_full), 0, 0, 0, 0);
        }
        const float i0 = __ldg(inv3), i1 = __ldg(inv3 + 1), i2 = __ldg(inv3 + 2);
        uint32_t* patch = s_patch[me];
        bool ok = true;
        TileWalk wk;
        walk_init(wk, p, blockIdx.x + me * gridDim.x, 2 * gridDim.x);
        float f[STEM_PER_LANE][3];
        int tile = blockIdx.x + me * gridDim.x;
        if (tile < p.total_tiles) stem_load_patch<IN_U8>(in_any, wk.tb, wk.th * STEM_TH, wk.tw * STEM_TW, lane, f);
        for (int local = me; tile < p.total_tiles && ok; tile += 2 * gridDim.x, local += 2) {
            // quantise this tile's patch (already in registers) into the warp's buffer
#pragma unroll
            for (int i = 0; i < STEM_PER_LANE; i++) {
                const int px = lane + 32 * i;
                int q0, q1, q2;
                if (IN_U8) {
                    const int v0 = (int)f[i][0], v1 = (int)f[i][1], v2 = (int)f[i][2];
                    q0 = v0 < 0 ? 0 : s_qlut[0][v0]; q1 = v1 < 0 ? 0 : s_qlut[1][v1]; q2 = v2 < 0 ? 0 : s_qlut[2][v2];
                } else {
                    q0 = max(-128, min(127, __float2int_rn(__fmul_rn(f[i][0], i0))));
                    q1 = max(-128, min(127, __float2int_rn(__fmul_rn(f[i][1], i1))));
                    q2 = max(-128, min(127, __float2int_rn(__fmul_rn(f[i][2], i2))));
                }
                if (px < STEM_PATCH) patch[px] = (uint32_t)((q0 & 0xff) | ((q1 & 0xff) << 8) | ((q2 & 0xff) << 16));
            }
            // next tile's loads go out now and land while this one is packed
            walk_next(wk, p);
            if (tile + 2 * (int)gridDim.x < p.total_tiles)
                stem_load_patch<IN_U8>(in_any, wk.tb, wk.th * STEM_TH, wk.tw * STEM_TW, lane, f);
            __syncwarp();
            const int stage = local % p.stages;
            const uint32_t phase = (uint32_t)(local / p.stages) & 1;
            ok = mbar_wait(smem_u32(&sh->empty[stage]), phase ^ 1, abort_flag, p.err, FFCU_ERR_EMPTY_TIMEOUT);
            if (!ok) break;
            uint8_t* dst = s_a + (size_t)stage * STEM_A_BYTES;
#pragma unroll
            for (int j = 0; j < TC_TILE_M / 32; j++) {
                const int r = lane + 32 * j;                     // output pixel of the tile: row r of the A operand
                const int ty = r / STEM_TW, tx = r % STEM_TW;
                uint32_t a[9];
#pragma unroll
                for (int kh = 0; kh < 3; kh++)
#pragma unroll
                    for (int kw = 0; kw < 3; kw++) a[kh * 3 + kw] = patch[(ty + kh) * STEM_PW + tx + kw];
                // nine (c0, c1, c2, 0) words -> 27 consecutive bytes + 5 zeros
                int4 lo, hi;
                lo.x = (int)__byte_perm(a[0], a[1], 0x4210);
                lo.y = (int)__byte_perm(a[1], a[2], 0x5421);
                lo.z = (int)__byte_perm(a[2], a[3], 0x6542);
                lo.w = (int)__byte_perm(a[4], a[5], 0x4210);
                hi.x = (int)__byte_perm(a[5], a[6], 0x5421);
                hi.y = (int)__byte_perm(a[6], a[7], 0x6542);
                hi.z = (int)(a[8] & 0x00ffffffu);
                hi.w = 0;
                // 32-byte swizzle: the row's two 16-byte halves swap when bit 7 of the row's byte offset is set
                const int sw = (r >> 2) & 1;
                int4* row = (int4*)(dst + r * 32);
                row[sw] = lo;
                row[sw ^ 1] = hi;
            }
            // generic-proxy stores -> visible to the tensor core (async proxy), then hand the stage over
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh->full[stage]));
        }
    } else if (warp == 1) {
        bool ok = mbar_wait(smem_u32(&sh->w_full), 0, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT);
        tc_fence_after();
        const uint64_t dw = smem_desc_sw32(smem_u32(s_w));
        const uint32_t leader = (lane == 0) ? 1u : 0u;
        for (int tile = blockIdx.x, local = 0; tile < p.total_tiles && ok; tile += gridDim.x, local++) {
            const int stage = local % p.stages;
            const uint32_t phase = (uint32_t)(local / p.stages) & 1;
            const int a = local % TC_NACC(BN);
            const uint32_t aphase = (uint32_t)(local / TC_NACC(BN)) & 1;
            ok = mbar_wait(smem_u32(&sh->acc_empty[a]), aphase ^ 1, abort_flag, p.err, FFCU_ERR_TMEM_TIMEOUT);
            if (!ok) break;
            ok = mbar_wait(smem_u32(&sh->full[stage]), phase, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT, p.full_wait);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(a * BN);
            const uint64_t da = smem_desc_sw32(smem_u32(s_a + (size_t)stage * STEM_A_BYTES));
            if (!TC_DBG(p, 2)) umma_i8_w(leader, d_tmem, da, dw, IDESC, 0u);
            umma_commit_w(leader, smem_u32(&sh->empty[stage]));
            umma_commit_w(leader, smem_u32(&sh->acc_full[a]));
        }
    } else {
        tc_epilogue_role<BN, CONTRACT, false, EPI, (EPI != EPI_RUNTIME)>(p, tab, lut, sh, tmem_base, abort_flag, warp, lane,
                                                   blockIdx.x, gridDim.x, p.total_tiles, 1, 0, 0u);
    }
    tc_teardown(abort_flag, tmem_base, TMEM_COLS, warp);
}

template <bool CONTRACT, int EPI, bool IN_U8>
static int launch_stem(int grid, int smem, cudaStream_t s, const CUtensorMap& mapB, const TcParams& prm, const void* in_any,
                       const float* inv3)
{
    auto kern = conv_stem_kernel<CONTRACT, EPI, IN_U8>;
    static int smem_set[64] = {};      // per device: the attribute belongs to the device's copy of the function
    int dev = 0;
    FFCU_CHECK(cudaGetDevice(&dev));
    if (smem_set[dev & 63] < smem) {
        FFCU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        smem_set[dev & 63] = smem;
    }
    return tc_launch_ex(kern, grid, smem, s, 1, mapB, prm, in_any, inv3);
}

int tc_launch_stem(int mode, int epi, int in_u8, int grid, int smem, cudaStream_t s, const CUtensorMap& mapB,
                   const TcParams& prm, const void* in_any, const float* inv3)
{
#define STEM_PICK(C_, E_) (in_u8 ? launch_stem<C_, E_, true>(grid, smem, s, mapB, prm, in_any, inv3) \
                                 : launch_stem<C_, E_, false>(grid, smem, s, mapB, prm, in_any, inv3))
    if (!mode) return STEM_PICK(false, EPI_RUNTIME);
    switch (epi) {
    case EPI_SLOPE_BN: return STEM_PICK(true, EPI_SLOPE_BN);
    case EPI_SLOPE:    return STEM_PICK(true, EPI_SLOPE);
    default:           return STEM_PICK(true, EPI_RUNTIME);
    }
#undef STEM_PICK
}
