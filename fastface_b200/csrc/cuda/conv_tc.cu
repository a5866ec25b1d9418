// conv_tc.cu -- INT8 implicit-GEMM convolution / FC on the sm_100a tensor cores.
//
// Takes over the reference's im2col + VNNI GEMM + fused epilogue
// (kernels/conv2d_nhwc.c:179-220, kernels/gemm_int8_v2.c:86-110,
// kernels/int8_epilogue.c:25-112) and, as a 1x1 "conv" over a [B,1,1,K] tensor,
// the final Linear (kernels/gemm_int8_matvec.c:33-81).
//
//   D[128 pixels x BN channels] (int32, TMEM) += A[128 x 32B] (smem) * B[BN x 32B] (smem)
//
// * A is never materialised: for each filter tap (kh,kw) and each KC-byte slice of
//   the input channels one 4-D TMA box {KC, TW, TH, TB} of the NHWC activation
//   tensor, shifted by the tap, lands in shared memory as 128 K-major rows.
//   Out-of-bounds rows/columns are zero-filled by TMA (= the conv's zero padding);
//   stride-2 convs use the tensor map's element strides.
// * B is the weight matrix repacked [Cout][kh][kw][Cin], a 2-D TMA box {KC, BN}.
// * tcgen05.mma kind::i8, cta_group::1, M=128, N=BN, K=32 per instruction;
//   accumulators double-buffered in TMEM so the epilogue of tile i overlaps the
//   MMAs of tile i+1.
// * Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer (+TMEM alloc),
//   warps 2..9 = epilogue (tcgen05.ld -> exact fp32 chain -> int8 NHWC stores).
// * Every wait is bounded; on expiry the kernel records an error word, drains
//   and frees its TMEM, and returns.  No cluster launch, no multicast.

#include "ffcu_internal.cuh"

#include <stdio.h>
#include <string.h>

#define TC_TILE_M 128
#define TC_MAX_COUT 512
#define TC_WAIT_NS 2000000000ull   // 2 s per wait

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t globaltimer_ns()
{
    uint64_t t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false (and raises the CTA-wide abort flag + the global error
// word) when the barrier did not flip within TC_WAIT_NS or another role already aborted.
__device__ __noinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err, int code)
{
    if (mbar_try(bar, parity)) return true;
    uint64_t t0 = globaltimer_ns();
    for (uint32_t spin = 1;; spin++) {
        if (mbar_try(bar, parity)) return true;
        if ((spin & 63u) == 0) {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > TC_WAIT_NS) {
                *abort_flag = 1;
                atomicCAS(err, 0, code);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3)
{
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after()  { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the mbarrier once every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, int (&v)[32])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                   "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                   "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major shared-memory matrix descriptor: rows of ROWB bytes (= swizzle span), 8-row groups
// 8*ROWB bytes apart, descriptor version 1 (sm_100), layout 2 = 128B swizzle / 4 = 64B swizzle.
template <int ROWB>
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr)
{
    uint64_t d = (uint64_t)((saddr >> 4) & 0x3fff);
    d |= (uint64_t)1 << 16;                              // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)((8 * ROWB) >> 4) << 32;              // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                              // version
    d |= (uint64_t)(ROWB == 128 ? 2 : 4) << 61;          // swizzle mode
    return d;
}

// kind::i8 instruction descriptor: D=s32, A=B=s8, both K-major, M=128, N=BN.
__host__ __device__ constexpr uint32_t idesc_i8(int bn)
{
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(TC_TILE_M >> 4) << 24);
}

// ---------------------------------------------------------------------------
// kernel parameters, shared state, epilogue
// ---------------------------------------------------------------------------
struct TcParams {
    EpiTables t;
    const int8_t* res;
    int32_t* acc_out;
    void* out;
    int8_t* out2;            // fused BN second output (NULL: none)
    int* err;
    int batch, Ho, Wo, Cout;
    int taps, Kw, cin_blocks, Cp;
    int stride, pad;
    int TW, TH, TB;
    int tiles_w, tiles_h, tiles_b, tiles_n, total_tiles;
    int stages;
};

#define TC_MAX_STAGES 8
#define TC_NTAB 9          // w_scale, bias, slope, res_scale, inv_out, bn_in, bn_scale, bn_offset, bn_inv
#define TC_EPI_WARPS 8     // warps 2..9: two per TMEM lane quarter, each takes half the columns
#define TC_THREADS (32 * (2 + TC_EPI_WARPS))

struct TcShared {                 // lives after the stage ring and the tables
    uint64_t full[TC_MAX_STAGES];
    uint64_t empty[TC_MAX_STAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t w_full;              // weight-stationary kernel: weights have landed
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void tc_load_tables(float* tab, const TcParams& p)
{
    for (int i = threadIdx.x; i < p.Cout; i += TC_THREADS) {
        tab[0 * TC_MAX_COUT + i] = p.t.w_scale[i];
        tab[1 * TC_MAX_COUT + i] = p.t.bias[i];
        tab[2 * TC_MAX_COUT + i] = p.t.slope ? p.t.slope[i] : 0.0f;
        tab[3 * TC_MAX_COUT + i] = p.t.res_scale ? p.t.res_scale[i] : 0.0f;
        tab[4 * TC_MAX_COUT + i] = p.t.inv_out ? p.t.inv_out[i] : 0.0f;
        if (p.out2) {
            tab[5 * TC_MAX_COUT + i] = p.t.bn_in[i];
            tab[6 * TC_MAX_COUT + i] = p.t.bn_scale[i];
            tab[7 * TC_MAX_COUT + i] = p.t.bn_offset[i];
            tab[8 * TC_MAX_COUT + i] = p.t.bn_inv[i];
        }
    }
}

// One 32-column chunk of one accumulator row: v[32] int32 -> outputs at element offset o
// (= pixel * Cout + first channel cb).  Replaces fused_epilogue_int8 for those 32 values
// (reference kernels/int8_epilogue.c:25-112), optionally followed by the next BN pass
// (:253-318) as a second output.
template <bool CONTRACT, bool OUT_F32>
__device__ __forceinline__ void tc_epilogue_chunk(const TcParams& p, const float* tab, const int (&v)[32],
                                                  const int (&rw)[8], int cb, size_t o, bool has_res,
                                                  bool has_slope, bool has_bn2)
{
    if (p.acc_out) {
        int4* dst = (int4*)(p.acc_out + o);
#pragma unroll
        for (int g = 0; g < 8; g++) dst[g] = make_int4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
    }
    if (OUT_F32) {
        float4* dst = (float4*)((float*)p.out + o);
#pragma unroll
        for (int g = 0; g < 8; g++) {
            const float4 ws = *(const float4*)&tab[0 * TC_MAX_COUT + cb + 4 * g];
            const float4 bi = *(const float4*)&tab[1 * TC_MAX_COUT + cb + 4 * g];
            float4 r;
            r.x = ffcu_fc_fp<CONTRACT>(v[4 * g + 0], ws.x, bi.x);
            r.y = ffcu_fc_fp<CONTRACT>(v[4 * g + 1], ws.y, bi.y);
            r.z = ffcu_fc_fp<CONTRACT>(v[4 * g + 2], ws.z, bi.z);
            r.w = ffcu_fc_fp<CONTRACT>(v[4 * g + 3], ws.w, bi.w);
            dst[g] = r;
        }
        return;
    }
    int ow_[8], ow2_[8];
#pragma unroll
    for (int g = 0; g < 8; g++) {
        const float4 ws = *(const float4*)&tab[0 * TC_MAX_COUT + cb + 4 * g];
        const float4 bi = *(const float4*)&tab[1 * TC_MAX_COUT + cb + 4 * g];
        const float4 sl = *(const float4*)&tab[2 * TC_MAX_COUT + cb + 4 * g];
        const float4 rs = *(const float4*)&tab[3 * TC_MAX_COUT + cb + 4 * g];
        const float4 iv = *(const float4*)&tab[4 * TC_MAX_COUT + cb + 4 * g];
        const int r = rw[g];
        float f0 = ffcu_conv_fp<CONTRACT>(v[4 * g + 0], ws.x, bi.x, has_res, (int)(int8_t)(r & 0xff), rs.x, has_slope, sl.x);
        float f1 = ffcu_conv_fp<CONTRACT>(v[4 * g + 1], ws.y, bi.y, has_res, (int)(int8_t)((r >> 8) & 0xff), rs.y, has_slope, sl.y);
        float f2 = ffcu_conv_fp<CONTRACT>(v[4 * g + 2], ws.z, bi.z, has_res, (int)(int8_t)((r >> 16) & 0xff), rs.z, has_slope, sl.z);
        float f3 = ffcu_conv_fp<CONTRACT>(v[4 * g + 3], ws.w, bi.w, has_res, (int)(int8_t)((r >> 24) & 0xff), rs.w, has_slope, sl.w);
        int q0 = ffcu_requant_nosat(f0, iv.x), q1 = ffcu_requant_nosat(f1, iv.y);
        int q2 = ffcu_requant_nosat(f2, iv.z), q3 = ffcu_requant_nosat(f3, iv.w);
        ow_[g] = ffcu_pack4(q0, q1, q2, q3);
        if (has_bn2) {
            q0 = max(-128, min(127, q0)); q1 = max(-128, min(127, q1));
            q2 = max(-128, min(127, q2)); q3 = max(-128, min(127, q3));
            const float4 bi_ = *(const float4*)&tab[5 * TC_MAX_COUT + cb + 4 * g];
            const float4 bs_ = *(const float4*)&tab[6 * TC_MAX_COUT + cb + 4 * g];
            const float4 bo_ = *(const float4*)&tab[7 * TC_MAX_COUT + cb + 4 * g];
            const float4 bv_ = *(const float4*)&tab[8 * TC_MAX_COUT + cb + 4 * g];
            int b0 = ffcu_bn_q_nosat(q0, bi_.x, bs_.x, bo_.x, bv_.x), b1 = ffcu_bn_q_nosat(q1, bi_.y, bs_.y, bo_.y, bv_.y);
            int b2 = ffcu_bn_q_nosat(q2, bi_.z, bs_.z, bo_.z, bv_.z), b3 = ffcu_bn_q_nosat(q3, bi_.w, bs_.w, bo_.w, bv_.w);
            ow2_[g] = ffcu_pack4(b0, b1, b2, b3);
        }
    }
    int4* dst = (int4*)((int8_t*)p.out + o);
    dst[0] = make_int4(ow_[0], ow_[1], ow_[2], ow_[3]);
    dst[1] = make_int4(ow_[4], ow_[5], ow_[6], ow_[7]);
    if (has_bn2) {
        int4* dst2 = (int4*)(p.out2 + o);
        dst2[0] = make_int4(ow2_[0], ow2_[1], ow2_[2], ow2_[3]);
        dst2[1] = make_int4(ow2_[4], ow2_[5], ow2_[6], ow2_[7]);
    }
}

// Epilogue role shared by both kernels.  Warps 2..9: warp w reads TMEM lanes
// [32*(w%4), +32) (the hardware's per-warp lane window) and the column half (w-2)/4.
template <int BN, bool CONTRACT, bool OUT_F32>
__device__ __forceinline__ void tc_epilogue_role(const TcParams& p, const float* tab, TcShared* sh,
                                                 uint32_t tmem_base, volatile int* abort_flag, int warp, int lane)
{
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int CHUNKS = BN / 32;                       // 2, 4 or 8
    constexpr int PER = CHUNKS / 2;
    const int row = q * 32 + lane;
    const int iw = row % p.TW;
    const int ih = (row / p.TW) % p.TH;
    const int ib = row / (p.TW * p.TH);
    const bool has_res = (p.res != nullptr) && (p.t.res_scale != nullptr);
    const bool has_slope = p.t.slope != nullptr;
    const bool has_bn2 = p.out2 != nullptr;
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x, local++) {
        const int tn = tile % p.tiles_n;
        int m = tile / p.tiles_n;
        const int tw = m % p.tiles_w; m /= p.tiles_w;
        const int th = m % p.tiles_h;
        const int tb = m / p.tiles_h;
        const int ow = tw * p.TW + iw, oh = th * p.TH + ih, b = tb * p.TB + ib;
        const bool valid = (ow < p.Wo) && (oh < p.Ho) && (b < p.batch);
        const size_t pix = ((size_t)b * p.Ho + oh) * p.Wo + ow;
        const int n0 = tn * BN;
        const int a = local & 1;
        const uint32_t aphase = (uint32_t)(local >> 1) & 1;
        // the residual operand does not depend on the accumulator: fetch the first chunk's
        // 32 bytes before waiting for the MMAs, the next chunk's while computing this one
        int rw[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        const size_t o0 = pix * p.Cout + n0 + half * PER * 32;
        if (has_res && valid) {
            const int4* rp = (const int4*)(p.res + o0);
            int4 r0 = rp[0], r1 = rp[1];
            rw[0] = r0.x; rw[1] = r0.y; rw[2] = r0.z; rw[3] = r0.w;
            rw[4] = r1.x; rw[5] = r1.y; rw[6] = r1.z; rw[7] = r1.w;
        }
        ok = mbar_wait(smem_u32(&sh->acc_full[a]), aphase, abort_flag, p.err, FFCU_ERR_EPI_TIMEOUT);
        if (!ok) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + (uint32_t)(a * BN) + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
        for (int jj = 0; jj < PER; jj++) {
            const int j = half * PER + jj;
            int v[32];
            tmem_ld32(taddr + (uint32_t)(j * 32), v);
            if (!valid) continue;
            int rn[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (has_res && jj + 1 < PER) {
                const int4* rp = (const int4*)(p.res + o0 + (size_t)(jj + 1) * 32);
                int4 r0 = rp[0], r1 = rp[1];
                rn[0] = r0.x; rn[1] = r0.y; rn[2] = r0.z; rn[3] = r0.w;
                rn[4] = r1.x; rn[5] = r1.y; rn[6] = r1.z; rn[7] = r1.w;
            }
            const int cb = n0 + j * 32;
            tc_epilogue_chunk<CONTRACT, OUT_F32>(p, tab, v, rw, cb, pix * p.Cout + cb, has_res, has_slope, has_bn2);
#pragma unroll
            for (int g = 0; g < 8; g++) rw[g] = rn[g];
        }
        // this warp's TMEM reads are complete (tcgen05.wait::ld inside tmem_ld32)
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh->acc_empty[a]));
    }
}

__device__ __forceinline__ void tc_setup(TcShared* sh, int stages, uint32_t tmem_cols, int warp)
{
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) { mbar_init(smem_u32(&sh->full[s]), 1); mbar_init(smem_u32(&sh->empty[s]), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(smem_u32(&sh->acc_full[a]), 1); mbar_init(smem_u32(&sh->acc_empty[a]), TC_EPI_WARPS); }
        mbar_init(smem_u32(&sh->w_full), 1);
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&sh->tmem_base)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
}

__device__ __forceinline__ void tc_teardown(volatile int* abort_flag, uint32_t tmem_base, uint32_t tmem_cols, int warp)
{
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        // a wait ran out: give bulk copies still in flight time to land before the
        // shared memory is handed back (bounded: about 1 ms)
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

// ---------------------------------------------------------------------------
// generic kernel: one TMA box per filter tap and channel slice
// ---------------------------------------------------------------------------
template <int BN, int KC, bool CONTRACT, bool OUT_F32>
__global__ void __launch_bounds__(TC_THREADS, 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const TcParams p)
{
    extern __shared__ uint8_t smem_raw[];
    // stage ring must start on a 1024-byte boundary (swizzle atoms)
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int A_BYTES = TC_TILE_M * KC;
    constexpr int B_BYTES = BN * KC;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;    // 128 / 256 / 512: powers of two
    constexpr uint32_t IDESC = idesc_i8(BN);

    float* tab = (float*)(smem + (size_t)p.stages * STAGE_BYTES);       // [TC_NTAB][TC_MAX_COUT]
    TcShared* sh = (TcShared*)(tab + TC_NTAB * TC_MAX_COUT);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int kblocks = p.taps * p.cin_blocks;

    tc_load_tables(tab, p);
    tc_setup(sh, p.stages, TMEM_COLS, warp);
    const uint32_t tmem_base = sh->tmem_base;
    volatile int* abort_flag = &sh->abort_flag;

    if (warp == 0) {
        if (lane == 0) {
            // TMA producer
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
                const int tn = tile % p.tiles_n;
                int m = tile / p.tiles_n;
                const int tw = m % p.tiles_w; m /= p.tiles_w;
                const int th = m % p.tiles_h;
                const int tb = m / p.tiles_h;
                const int x0 = tw * p.TW * p.stride - p.pad;
                const int y0 = th * p.TH * p.stride - p.pad;
                const int b0 = tb * p.TB;
                const int n0 = tn * BN;
                for (int kb = 0; kb < kblocks; kb++) {
                    ok = mbar_wait(smem_u32(&sh->empty[stage]), phase ^ 1, abort_flag, p.err, FFCU_ERR_EMPTY_TIMEOUT);
                    if (!ok) break;
                    const int tap = kb / p.cin_blocks;
                    const int c0 = (kb - tap * p.cin_blocks) * KC;
                    const int kh = tap / p.Kw, kw = tap - kh * p.Kw;
                    const uint32_t bar = smem_u32(&sh->full[stage]);
                    const uint32_t sa = smem_u32(smem + (size_t)stage * STAGE_BYTES);
                    mbar_expect_tx(bar, STAGE_BYTES);
                    tma_load_4d(sa, &mapA, bar, c0, x0 + kw, y0 + kh, b0);
                    tma_load_2d(sa + A_BYTES, &mapB, bar, tap * p.Cp + c0, n0);
                    if (++stage == p.stages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // MMA issuer
            int stage = 0; uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x, local++) {
                const int a = local & 1;
                const uint32_t aphase = (uint32_t)(local >> 1) & 1;
                ok = mbar_wait(smem_u32(&sh->acc_empty[a]), aphase ^ 1, abort_flag, p.err, FFCU_ERR_TMEM_TIMEOUT);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(a * BN);
                for (int kb = 0; kb < kblocks; kb++) {
                    ok = mbar_wait(smem_u32(&sh->full[stage]), phase, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + (size_t)stage * STAGE_BYTES);
                    const uint64_t da = smem_desc<KC>(sa);
                    const uint64_t db = smem_desc<KC>(sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < KC / 32; k++)
                        umma_i8(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), IDESC, (kb | k) ? 1u : 0u);
                    umma_commit(smem_u32(&sh->empty[stage]));   // frees the stage once these MMAs have read it
                    if (++stage == p.stages) { stage = 0; phase ^= 1; }
                }
                if (ok) umma_commit(smem_u32(&sh->acc_full[a]));
            }
        }
    } else {
        tc_epilogue_role<BN, CONTRACT, OUT_F32>(p, tab, sh, tmem_base, abort_flag, warp, lane);
    }
    tc_teardown(abort_flag, tmem_base, TMEM_COLS, warp);
}

// ---------------------------------------------------------------------------
// weight-stationary kernel for the 64-input-channel 3x3 stride-1 layers
// (112x112 and 56x56 maps: 20% of the network's MACs but, tap by tap, its largest
// shared-memory fill traffic).
//   * all 9 weight taps ([tap][BN rows][64 B], 36 KB or 72 KB) are loaded once per CTA
//     and stay in shared memory for every tile the CTA processes;
//   * output tile = 8 wide x 16 high pixels of one image.  Per tile three boxes
//     {64 B, 8, 18, 1} are loaded, one per kw, each holding rows y0-1 .. y0+16: an 8-row
//     swizzle group is one image row of the box, so the three kh taps are the same box
//     read at group offsets 0, 1, 2 (descriptor start + kh * 512 B).  Activation bytes
//     fetched per tile drop from 9 x 128 to 3 x 144 rows.
// ---------------------------------------------------------------------------
#define WS_TW 8
#define WS_TH 16
#define WS_BOX_ROWS (WS_TW * (WS_TH + 2))          // 144 rows of 64 B per kw box
#define WS_A_BYTES (3 * WS_BOX_ROWS * 64)          // 27 648 B per tile

template <int BN, bool CONTRACT>
__global__ void __launch_bounds__(TC_THREADS, 1)
conv_ws_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const TcParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int KC = 64;
    constexpr int W_TAP_BYTES = BN * KC;
    constexpr int W_BYTES = 9 * W_TAP_BYTES;
    constexpr uint32_t TMEM_COLS = 2 * BN;
    constexpr uint32_t IDESC = idesc_i8(BN);

    uint8_t* s_w = smem;                                        // [9][BN][64]
    uint8_t* s_a = smem + W_BYTES;                              // [stages][3][144][64]
    float* tab = (float*)(s_a + (size_t)p.stages * WS_A_BYTES);
    TcShared* sh = (TcShared*)(tab + TC_NTAB * TC_MAX_COUT);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    tc_load_tables(tab, p);
    tc_setup(sh, p.stages, TMEM_COLS, warp);
    const uint32_t tmem_base = sh->tmem_base;
    volatile int* abort_flag = &sh->abort_flag;

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t wbar = smem_u32(&sh->w_full);
            mbar_expect_tx(wbar, W_BYTES);
            for (int tap = 0; tap < 9; tap++)
                tma_load_2d(smem_u32(s_w + tap * W_TAP_BYTES), &mapB, wbar, tap * p.Cp, 0);
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
                int m = tile;
                const int tw = m % p.tiles_w; m /= p.tiles_w;
                const int th = m % p.tiles_h;
                const int b = m / p.tiles_h;
                ok = mbar_wait(smem_u32(&sh->empty[stage]), phase ^ 1, abort_flag, p.err, FFCU_ERR_EMPTY_TIMEOUT);
                if (!ok) break;
                const uint32_t bar = smem_u32(&sh->full[stage]);
                const uint32_t sa = smem_u32(s_a + (size_t)stage * WS_A_BYTES);
                mbar_expect_tx(bar, WS_A_BYTES);
                for (int kw = 0; kw < 3; kw++)
                    tma_load_4d(sa + kw * (WS_BOX_ROWS * 64), &mapA, bar, 0, tw * WS_TW + kw - 1, th * WS_TH - 1, b);
                if (++stage == p.stages) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = mbar_wait(smem_u32(&sh->w_full), 0, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT);
            tc_fence_after();
            int stage = 0; uint32_t phase = 0;
            int local = 0;
            const uint64_t dw = smem_desc<KC>(smem_u32(s_w));
            for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x, local++) {
                const int a = local & 1;
                const uint32_t aphase = (uint32_t)(local >> 1) & 1;
                ok = mbar_wait(smem_u32(&sh->acc_empty[a]), aphase ^ 1, abort_flag, p.err, FFCU_ERR_TMEM_TIMEOUT);
                if (!ok) break;
                ok = mbar_wait(smem_u32(&sh->full[stage]), phase, abort_flag, p.err, FFCU_ERR_TMA_TIMEOUT);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(a * BN);
                const uint64_t da0 = smem_desc<KC>(smem_u32(s_a + (size_t)stage * WS_A_BYTES));
#pragma unroll
                for (int kw = 0; kw < 3; kw++)
#pragma unroll
                    for (int kh = 0; kh < 3; kh++) {
                        // box kw, image rows kh .. kh+15: start = kw * 9216 + kh * 512 bytes (>> 4)
                        const uint64_t da = da0 + (uint64_t)((kw * WS_BOX_ROWS * 64 + kh * WS_TW * 64) >> 4);
                        const uint64_t db = dw + (uint64_t)(((kh * 3 + kw) * W_TAP_BYTES) >> 4);
#pragma unroll
                        for (int k = 0; k < 2; k++)
                            umma_i8(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), IDESC, (kw | kh | k) ? 1u : 0u);
                    }
                umma_commit(smem_u32(&sh->empty[stage]));
                umma_commit(smem_u32(&sh->acc_full[a]));
                if (++stage == p.stages) { stage = 0; phase ^= 1; }
            }
        }
    } else {
        tc_epilogue_role<BN, CONTRACT, false>(p, tab, sh, tmem_base, abort_flag, warp, lane);
    }
    tc_teardown(abort_flag, tmem_base, TMEM_COLS, warp);
}

// ---------------------------------------------------------------------------
// host side: tile geometry, tensor maps, launch
// ---------------------------------------------------------------------------
typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static encode_tiled_fn get_encode()
{
    static encode_tiled_fn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (encode_tiled_fn)p;
    }
    return fn;
}

struct TcGeom { int TW, TH, TB; CUtensorMap mapA; bool valid; };

struct TcPlan {
    ffcu_layer d;
    int max_batch;
    int BN, KC, stages, smem_bytes;
    bool out_f32;
    const int8_t* d_in;
    CUtensorMap mapB;
    int n_sm;
    TcGeom geoms[8];
    int n_geoms;
    bool ws;                 // weight-stationary kernel (64-channel 3x3 stride-1 layers)
    CUtensorMap mapA_ws;     // box {64, 8, 18, 1}
    int ws_stages, ws_smem_bytes;
};

// Output-tile shape {TW, TH, TB} with TW*TH*TB = 128 that wastes the fewest rows for this
// feature-map size and batch; ties go to the widest tile.
static void pick_geometry(int Wo, int Ho, int batch, int* TW, int* TH, int* TB)
{
    double best = 1e300; int bw = 1, bh = 1, bb = 128;
    for (int tw = 128; tw >= 1; tw >>= 1)
        for (int th = 128 / tw; th >= 1; th >>= 1) {
            int tb = 128 / (tw * th);
            double padded = (double)((Wo + tw - 1) / tw * tw) * ((Ho + th - 1) / th * th) * ((batch + tb - 1) / tb * tb);
            if (padded < best) { best = padded; bw = tw; bh = th; bb = tb; }
        }
    *TW = bw; *TH = bh; *TB = bb;
}

static bool encode_A(const TcPlan* p, TcGeom* g)
{
    encode_tiled_fn enc = get_encode();
    if (!enc) { ffcu_set_error("cuTensorMapEncodeTiled is not available"); return false; }
    const ffcu_layer& d = p->d;
    const cuuint64_t Cp = (cuuint64_t)d.Cin_pad;
    cuuint64_t dims[4] = {Cp, (cuuint64_t)d.W, (cuuint64_t)d.H, (cuuint64_t)p->max_batch};
    cuuint64_t strides[3] = {Cp, Cp * d.W, Cp * d.W * d.H};
    cuuint32_t box[4] = {(cuuint32_t)p->KC, (cuuint32_t)(g->TW * d.stride), (cuuint32_t)(g->TH * d.stride), (cuuint32_t)g->TB};
    cuuint32_t estr[4] = {1, (cuuint32_t)d.stride, (cuuint32_t)d.stride, 1};
    if (d.stride > 1) {      // a unit-extent dimension needs no traversal stride
        if (g->TW == 1) { box[1] = 1; estr[1] = 1; }
        if (g->TH == 1) { box[2] = 1; estr[2] = 1; }
    }
    CUresult r = enc(&g->mapA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)p->d_in, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE,
                     p->KC == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { ffcu_set_error("cuTensorMapEncodeTiled(A) failed: %d", (int)r); return false; }
    return true;
}

TcPlan* ffcu_tc_plan(const ffcu_layer& L, int max_batch, const int8_t* d_in, const int8_t* d_w, int device)
{
    if (L.kind != FFCU_CONV && L.kind != FFCU_FC) return nullptr;
    const int Cp = L.Cin_pad;
    if (Cp % 64 != 0 || L.Cout % 64 != 0 || L.Cout > TC_MAX_COUT) return nullptr;
    if (L.stride < 1 || L.stride > 2 || L.Kh * L.Kw > 9) return nullptr;
    if (L.stride == 2 && getenv("FF_TC_STRIDE2") && atoi(getenv("FF_TC_STRIDE2")) == 0) return nullptr;
    encode_tiled_fn enc = get_encode();
    if (!enc) return nullptr;
    TcPlan* p = new TcPlan();
    p->d = L; p->max_batch = max_batch; p->d_in = d_in; p->n_geoms = 0;
    p->out_f32 = (L.kind == FFCU_FC);
    p->KC = (Cp % 128 == 0) ? 128 : 64;
    p->BN = L.Cout >= 256 ? 256 : L.Cout;
    const char* bn_env = getenv("FF_TC_BN");
    if (bn_env) { int v = atoi(bn_env); if ((v == 64 || v == 128 || v == 256) && L.Cout % v == 0) p->BN = v; }
    const int stage_bytes = (TC_TILE_M + p->BN) * p->KC;
    const int fixed = TC_NTAB * TC_MAX_COUT * 4 + (int)sizeof(TcShared) + 1024;
    int stages = (232448 - fixed) / stage_bytes;
    if (stages > TC_MAX_STAGES) stages = TC_MAX_STAGES;
    if (stages < 2) { delete p; return nullptr; }
    p->stages = stages;
    p->smem_bytes = stages * stage_bytes + fixed;
    cudaDeviceGetAttribute(&p->n_sm, cudaDevAttrMultiProcessorCount, device);
    // weights: [Cout][taps*Cp] K-major
    cuuint64_t Ktot = (cuuint64_t)L.Kh * L.Kw * Cp;
    cuuint64_t dims[2] = {Ktot, (cuuint64_t)L.Cout};
    cuuint64_t strides[1] = {Ktot};
    cuuint32_t box[2] = {(cuuint32_t)p->KC, (cuuint32_t)p->BN};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&p->mapB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)d_w, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE,
                     p->KC == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { ffcu_set_error("cuTensorMapEncodeTiled(B) failed: %d", (int)r); delete p; return nullptr; }
    // weight-stationary variant
    p->ws = false;
    const char* ws_env = getenv("FF_TC_WS");
    if (L.kind == FFCU_CONV && Cp == 64 && L.Kh == 3 && L.Kw == 3 && L.stride == 1 && L.pad == 1 &&
        (L.Cout == 64 || L.Cout == 128) && p->BN == L.Cout && L.W % WS_TW == 0 && L.H >= WS_TH &&
        !(ws_env && ws_env[0] == '0')) {
        cuuint64_t adims[4] = {64, (cuuint64_t)L.W, (cuuint64_t)L.H, (cuuint64_t)max_batch};
        cuuint64_t astr[3] = {64, (cuuint64_t)64 * L.W, (cuuint64_t)64 * L.W * L.H};
        cuuint32_t abox[4] = {64, WS_TW, WS_TH + 2, 1};
        cuuint32_t aes[4] = {1, 1, 1, 1};
        r = enc(&p->mapA_ws, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)d_in, adims, astr, abox, aes,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r == CUDA_SUCCESS) {
            const int wbytes = 9 * p->BN * 64;
            int st = (232448 - wbytes - fixed) / WS_A_BYTES;
            if (st > TC_MAX_STAGES) st = TC_MAX_STAGES;
            if (st >= 2) { p->ws = true; p->ws_stages = st; p->ws_smem_bytes = wbytes + st * WS_A_BYTES + fixed; }
        }
    }
    return p;
}

void ffcu_tc_free(TcPlan* p) { delete p; }

template <int BN, int KC>
static int launch_variant(const TcPlan* p, const TcGeom* g, const TcParams& prm, int mode, int grid, cudaStream_t s)
{
#define TC_LAUNCH(CONTRACT, F32)                                                                         \
    do {                                                                                                 \
        auto kern = conv_tc_kernel<BN, KC, CONTRACT, F32>;                                               \
        FFCU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, p->smem_bytes)); \
        kern<<<grid, TC_THREADS, p->smem_bytes, s>>>(g->mapA, p->mapB, prm);                             \
    } while (0)
    if (p->out_f32) { if (mode) TC_LAUNCH(true, true); else TC_LAUNCH(false, true); }
    else            { if (mode) TC_LAUNCH(true, false); else TC_LAUNCH(false, false); }
#undef TC_LAUNCH
    FFCU_CHECK(cudaGetLastError());
    return 0;
}

int ffcu_tc_launch(const TcPlan* cp, int batch, int mode, const EpiTables& t, const int8_t* res,
                   int32_t* acc_out, void* out, int8_t* out_bn2, int* d_err, cudaStream_t s)
{
    TcPlan* p = const_cast<TcPlan*>(cp);
    if (batch < 1 || batch > p->max_batch) { ffcu_set_error("tc launch: batch out of range"); return -1; }
    const ffcu_layer& d = p->d;
    if (p->ws) {
        TcParams prm;
        prm.t = t; prm.res = res; prm.acc_out = acc_out; prm.out = out; prm.err = d_err;
        prm.out2 = (out_bn2 && t.bn_in) ? out_bn2 : nullptr;
        prm.batch = batch; prm.Ho = d.Ho; prm.Wo = d.Wo; prm.Cout = d.Cout;
        prm.taps = 9; prm.Kw = 3; prm.Cp = 64; prm.cin_blocks = 1; prm.stride = 1; prm.pad = 1;
        prm.TW = WS_TW; prm.TH = WS_TH; prm.TB = 1;
        prm.tiles_w = d.Wo / WS_TW; prm.tiles_h = (d.Ho + WS_TH - 1) / WS_TH; prm.tiles_b = batch; prm.tiles_n = 1;
        prm.total_tiles = prm.tiles_w * prm.tiles_h * batch;
        prm.stages = p->ws_stages;
        int grid = prm.total_tiles < p->n_sm ? prm.total_tiles : p->n_sm;
#define WS_LAUNCH(BNV, CONTRACT)                                                                            \
        do {                                                                                                \
            auto kern = conv_ws_kernel<BNV, CONTRACT>;                                                      \
            FFCU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, p->ws_smem_bytes)); \
            kern<<<grid, TC_THREADS, p->ws_smem_bytes, s>>>(p->mapA_ws, p->mapB, prm);                      \
        } while (0)
        if (p->BN == 64) { if (mode) WS_LAUNCH(64, true); else WS_LAUNCH(64, false); }
        else             { if (mode) WS_LAUNCH(128, true); else WS_LAUNCH(128, false); }
#undef WS_LAUNCH
        FFCU_CHECK(cudaGetLastError());
        return 0;
    }
    int TW, TH, TB;
    pick_geometry(d.Wo, d.Ho, batch, &TW, &TH, &TB);
    TcGeom* g = nullptr;
    for (int i = 0; i < p->n_geoms; i++)
        if (p->geoms[i].TW == TW && p->geoms[i].TH == TH && p->geoms[i].TB == TB) g = &p->geoms[i];
    if (!g) {
        if (p->n_geoms == 8) p->n_geoms = 0;
        g = &p->geoms[p->n_geoms];
        g->TW = TW; g->TH = TH; g->TB = TB;
        if (!encode_A(p, g)) return -1;
        p->n_geoms++;
    }
    TcParams prm;
    prm.t = t; prm.res = res; prm.acc_out = acc_out; prm.out = out; prm.err = d_err;
    prm.out2 = (out_bn2 && t.bn_in) ? out_bn2 : nullptr;
    prm.batch = batch; prm.Ho = d.Ho; prm.Wo = d.Wo; prm.Cout = d.Cout;
    prm.taps = d.Kh * d.Kw; prm.Kw = d.Kw; prm.Cp = d.Cin_pad; prm.cin_blocks = d.Cin_pad / p->KC;
    prm.stride = d.stride; prm.pad = d.pad;
    prm.TW = TW; prm.TH = TH; prm.TB = TB;
    prm.tiles_w = (d.Wo + TW - 1) / TW; prm.tiles_h = (d.Ho + TH - 1) / TH; prm.tiles_b = (batch + TB - 1) / TB;
    prm.tiles_n = d.Cout / p->BN;
    prm.total_tiles = prm.tiles_w * prm.tiles_h * prm.tiles_b * prm.tiles_n;
    prm.stages = p->stages;
    int grid = prm.total_tiles < p->n_sm ? prm.total_tiles : p->n_sm;
    if (p->KC == 128) {
        if (p->BN == 64) return launch_variant<64, 128>(p, g, prm, mode, grid, s);
        if (p->BN == 128) return launch_variant<128, 128>(p, g, prm, mode, grid, s);
        return launch_variant<256, 128>(p, g, prm, mode, grid, s);
    }
    if (p->BN == 64) return launch_variant<64, 64>(p, g, prm, mode, grid, s);
    if (p->BN == 128) return launch_variant<128, 64>(p, g, prm, mode, grid, s);
    return launch_variant<256, 64>(p, g, prm, mode, grid, s);
}
