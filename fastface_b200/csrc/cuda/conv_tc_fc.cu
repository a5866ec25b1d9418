// conv_tc_fc.cu -- the FC layer (512 outputs over K = 25088) as a split-K tensor-core GEMM.
//
// As one 128-row x 64-column tile per CTA the FC is eight CTAs per 128 faces, each streaming its
// whole K (4.8 MB of operand boxes through one SM's TMA: 47 us whatever the batch up to 256).  Here a
// (row tile, column tile) is cut into `splits` K ranges, one CTA each: with 14 ranges a 128-face FC
// runs on 112 SMs.  A CTA adds its int32 partial sums into a scratch array (red.global.add: integer
// addition, so any order gives the same bits), takes a ticket, and the CTA that takes the last ticket
// of its tile turns the sums into floats exactly as the one-CTA form does (reference
// kernels/gemm_int8_matvec.c: out = (float)dot * w_scale + bias), leaving sums and ticket zero for the
// next call.
#include "conv_tc_common.cuh"

#define FCT_BN 64
#define FCT_KC 128
#define FCT_A_BYTES (TC_TILE_M * FCT_KC)
#define FCT_B_BYTES (FCT_BN * FCT_KC)
#define FCT_SUB_BYTES (FCT_A_BYTES + FCT_B_BYTES)

template <bool CONTRACT>
__global__ void __launch_bounds__(TC_THREADS, 1)
fc_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const FcTcParams p)
{
    tc_pdl_trigger();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    TcShared* sh = (TcShared*)(smem + (size_t)p.stages * p.group * FCT_SUB_BYTES);
    __shared__ int s_last;
    constexpr uint32_t TMEM_COLS = FCT_BN;
    constexpr uint32_t IDESC = idesc_i8(FCT_BN);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // CTA -> (column tile, row tile, K range); the column tile varies fastest so that the CTAs of one
    // K range (which read the same activation boxes) are launched together
    const int tn = blockIdx.x % p.tiles_n;
    const int tm = (blockIdx.x / p.tiles_n) % p.tiles_m;
    const int split = blockIdx.x / (p.tiles_n * p.tiles_m);
    const int G = p.group;
    const int n_steps = p.blocks_per_split / G;
    const int kb0 = split * p.blocks_per_split;

    tc_setup(sh, p.stages, TMEM_COLS, warp, 4);
    const uint32_t tmem_base = sh->tmem_base;
    volatile int* abort_flag = &sh->abort_flag;
    const uint32_t full0 = smem_u32(&sh->full[0]), empty0 = smem_u32(&sh->empty[0]);
    const int stage_bytes = G * FCT_SUB_BYTES;

    if (warp == 0) {
        // TMA producer: lane 2g fetches the activation box of the stage's K block g, lane 2g + 1 its weight box.
        // The weights do not depend on the previous kernel: the weight boxes of the first ring-full of steps are
        // requested before the programmatic-dependency wait.
        const bool issuer = lane < 2 * G;
        const int g = issuer ? (lane >> 1) : 0;
        const bool is_a = (lane & 1) == 0;
        const CUtensorMap* map = is_a ? &mapA : &mapB;
        const uint32_t smem0 = smem_u32(smem) + (uint32_t)(g * FCT_SUB_BYTES) + (is_a ? 0u : (uint32_t)FCT_A_BYTES);
        const int pre = n_steps < p.stages ? n_steps : p.stages;
#pragma unroll 1
        for (int it = 0; it < pre; it++) {
            if (lane == 0) mbar_expect_tx(full0 + it * 8, G * FCT_SUB_BYTES);
            __syncwarp();
            if (issuer && !is_a) tma_load_4d(smem0 + it * stage_bytes, map, full0 + it * 8, (kb0 + it * G + g) * FCT_KC, tn * FCT_BN, 0, 0);
        }
        tc_pdl_wait();
        int stage = 0; uint32_t phase = 0;
        bool ok = true;
#pragma unroll 1
        for (int it = 0; it < n_steps && ok; it++) {
            const bool first_fill = it < pre;
            if (!first_fill) {
                ok = mbar_wait(empty0 + stage * 8, phase ^ 1, abort_flag, p.err, FFCU_ERR_EMPTY_TIMEOUT, p.wait_cycles);
                if (!ok) break;
                if (lane == 0) mbar_expect_tx(full0 + stage * 8, G * FCT_SUB_BYTES);
                __syncwarp();
            }
            if (it == p.drop_step) {
                // armed by the timeout test for one launch: this step's activations never arrive
            } else if (issuer && (is_a || !first_fill)) {
                const int c0 = (kb0 + it * G + g) * FCT_KC;
                tma_load_4d(smem0 + stage * stage_bytes, map, full0 + stage * 8, c0, is_a ? 0 : tn * FCT_BN, 0, is_a ? tm * TC_TILE_M : 0);
            }
            if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
    } else if (warp == 1) {
        // MMA issuer: the warp loops and waits together, lane 0 issues
        int stage = 0; uint32_t phase = 0;
        bool ok = true;
        const uint64_t da0 = smem_desc<FCT_KC>(smem_u32(smem));
        const uint64_t db0 = smem_desc<FCT_KC>(smem_u32(smem) + FCT_A_BYTES);
        const uint32_t leader = (lane == 0) ? 1u : 0u;
#pragma unroll 1
        for (int it = 0; it < n_steps; it++) {
            ok = mbar_wait(full0 + stage * 8, phase, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT, p.wait_cycles);
            if (!ok) break;
            tc_fence_after();
            uint32_t soff = (uint32_t)((stage * stage_bytes) >> 4);
#pragma unroll 1
            for (int g = 0; g < G; g++, soff += (uint32_t)(FCT_SUB_BYTES >> 4)) {
#pragma unroll
                for (int k = 0; k < FCT_KC / 32; k++)
                    umma_i8_w(leader, tmem_base, da0 + (uint64_t)(soff + 2 * k), db0 + (uint64_t)(soff + 2 * k), IDESC, (it | g | k) ? 1u : 0u);
            }
            umma_commit_w(leader, empty0 + stage * 8);
            if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit_w(leader, smem_u32(&sh->acc_full[0]));
    } else if (warp < 6) {
        // Epilogue: four warps, one TMEM lane quarter (32 faces) each, all 64 columns.  A TMEM load gives a lane one
        // face's columns; global memory wants a warp on consecutive columns of ONE face (a face's row of sums is 2 KB
        // from the next: 32 lanes on 32 faces would be 32 sectors per instruction).  So the warp turns its 32 x 64
        // block through shared memory: the pipeline ring is idle once the accumulator is complete (every MMA has read
        // its operands, no copy is in flight), and 65-word rows keep both directions free of bank conflicts.
        tc_pdl_wait();                                       // the scratch sums and tickets belong to the previous call until here
        const int q = warp & 3;
        const int b0 = tm * TC_TILE_M + q * 32;              // first face of this warp's quarter
        const int rows = p.batch - b0 < 32 ? p.batch - b0 : 32;      // faces of the quarter that exist (may be <= 0)
        const int n0 = tn * FCT_BN;
        int* stg = (int*)smem + (warp - 2) * (32 * 65);
        const float ws0 = __ldg(p.w_scale + n0 + lane), ws1 = __ldg(p.w_scale + n0 + 32 + lane);
        const float bi0 = __ldg(p.bias + n0 + lane), bi1 = __ldg(p.bias + n0 + 32 + lane);
        bool ok = mbar_wait(smem_u32(&sh->acc_full[0]), 0, abort_flag, p.err, FFCU_ERR_EPI_TIMEOUT, p.wait_cycles);
        if (ok) {
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
            for (int ch = 0; ch < FCT_BN / 16; ch++) {
                int v[16];
                tmem_ld16_issue(taddr + (uint32_t)(16 * ch), v);
                tmem_ld_wait(v);
#pragma unroll
                for (int i = 0; i < 16; i++) stg[lane * 65 + 16 * ch + i] = v[i];
            }
            tc_fence_before();
            __syncwarp();
#pragma unroll 1
            for (int r = 0; r < rows; r++) {
                const int x0 = stg[r * 65 + lane], x1 = stg[r * 65 + 32 + lane];
                const size_t o = (size_t)(b0 + r) * p.N + n0 + lane;
                if (p.splits == 1) {
                    p.out[o] = ffcu_fc_fp<CONTRACT>(x0, ws0, bi0);
                    p.out[o + 32] = ffcu_fc_fp<CONTRACT>(x1, ws1, bi1);
                } else {
                    atomicAdd(p.sums + o, x0);
                    atomicAdd(p.sums + o + 32, x1);
                }
            }
        }
        if (p.splits > 1) {
            // every epilogue thread's additions are out (or the CTA has given up) before the ticket is taken
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (warp == 2 && lane == 0)
                s_last = (!*abort_flag && atomicAdd(p.tickets + tm * p.tiles_n + tn, 1) == p.splits - 1) ? 1 : 0;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (s_last) {
                __threadfence();                             // the other CTAs' additions are visible from here on
                // eight faces' sums are requested before the first is used: one L2 round trip per eight rows, not per row
#pragma unroll 1
                for (int r0 = 0; r0 < rows; r0 += 8) {
                    int d0[8], d1[8];
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        const size_t o = (size_t)(b0 + r0 + k) * p.N + n0 + lane;
                        d0[k] = 0; d1[k] = 0;
                        if (r0 + k < rows) { d0[k] = __ldcg(p.sums + o); d1[k] = __ldcg(p.sums + o + 32); }
                    }
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        if (r0 + k >= rows) break;
                        const size_t o = (size_t)(b0 + r0 + k) * p.N + n0 + lane;
                        p.sums[o] = 0; p.sums[o + 32] = 0;   // clean for the next call
                        p.out[o] = ffcu_fc_fp<CONTRACT>(d0[k], ws0, bi0);
                        p.out[o + 32] = ffcu_fc_fp<CONTRACT>(d1[k], ws1, bi1);
                    }
                }
                if (warp == 2 && lane == 0) p.tickets[tm * p.tiles_n + tn] = 0;
            }
        }
    }
    tc_teardown(abort_flag, tmem_base, TMEM_COLS, warp);
}

int tc_launch_fc(int mode, int grid, int smem, cudaStream_t s, const CUtensorMap& mapA, const CUtensorMap& mapB, const FcTcParams& prm)
{
    static int smem_set[64][2] = {};   // per device and instantiation: the attribute belongs to the device's copy of the function
    int dev = 0;
    FFCU_CHECK(cudaGetDevice(&dev));
    if (mode) {
        auto kern = fc_tc_kernel<true>;
        if (smem_set[dev & 63][1] < smem) {
            FFCU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            smem_set[dev & 63][1] = smem;
        }
        return tc_launch_ex(kern, grid, smem, s, 1, mapA, mapB, prm);
    }
    auto kern = fc_tc_kernel<false>;
    if (smem_set[dev & 63][0] < smem) {
        FFCU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        smem_set[dev & 63][0] = smem;
    }
    return tc_launch_ex(kern, grid, smem, s, 1, mapA, mapB, prm);
}
