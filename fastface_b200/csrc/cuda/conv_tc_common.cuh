// conv_tc_common.cuh -- shared pieces of the INT8 implicit-GEMM convolution / FC on the sm_100a tensor cores.
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
// * tcgen05.mma kind::i8, M=128 per CTA (cta_group::1) or M=256 per CTA pair
//   (cta_group::2), N=BN, K=32 per instruction; a ring of 512/BN accumulators in
//   TMEM so the epilogue of one tile overlaps the MMAs of the next ones.
// * Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer (+TMEM alloc),
//   warps 2..17 = epilogue, two sets of eight (tcgen05.ld -> exact fp32 chain ->
//   int8 NHWC stores), warp 18 = second MMA issuer in the kernels whose tiles are
//   a handful of MMAs (weight-stationary and stem kernels).
// * Every wait is bounded; on expiry the kernel records an error word, drains
//   and frees its TMEM, and returns.  The CTA-pair kernel is a cluster of two;
//   no TMA load is multicast.

#pragma once
#include "ffcu_internal.cuh"

#include <stdio.h>
#include <string.h>
#include <type_traits>

#define TC_TILE_M 128
#define TC_MAX_COUT 512

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
// Arrive that publishes nothing but "my tcgen05.ld reads are done" (see mbar_arrive_cluster).
__device__ __forceinline__ void mbar_arrive_relaxed(uint32_t bar)
{
    asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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

__device__ __forceinline__ bool mbar_try_cluster(uint32_t bar, uint32_t parity);
// Bounded wait.  Returns false (and raises the CTA-wide abort flag + the global error
// word) when the barrier did not flip within `limit` SM cycles (TC_WAIT_CYCLES, about 2 s,
// unless the launch says otherwise) or another role already aborted.  The clock is only
// consulted after a burst of failed polls, so a wait that succeeds quickly costs nothing
// but the polls.
#define TC_WAIT_CYCLES 4000000000ll
template <bool CLUSTER>
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err, int code,
                                            long long limit)
{
#pragma unroll 1
    for (int i = 0; i < 256; i++)
        if (CLUSTER ? mbar_try_cluster(bar, parity) : mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
#pragma unroll 1
    for (uint32_t spin = 1;; spin++) {
        if (CLUSTER ? mbar_try_cluster(bar, parity) : mbar_try(bar, parity)) return true;
        if ((spin & 255u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > limit) {
                *abort_flag = 1;
                atomicCAS(err, 0, code);
                return false;
            }
        }
    }
}
// The first polls are inline (a wait that is already satisfied, or nearly, costs a few instructions);
// the long form with the clock and the abort flag is one shared function, not a copy per wait site.
template <bool CLUSTER>
__device__ __forceinline__ bool mbar_wait_impl(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err, int code,
                                               long long limit)
{
    if (CLUSTER ? mbar_try_cluster(bar, parity) : mbar_try(bar, parity)) return true;
    if (CLUSTER ? mbar_try_cluster(bar, parity) : mbar_try(bar, parity)) return true;
    return mbar_wait_slow<CLUSTER>(bar, parity, abort_flag, err, code, limit);
}
__device__ __forceinline__ bool mbar_try_cluster(uint32_t bar, uint32_t parity);
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err, int code,
                                          long long limit = TC_WAIT_CYCLES)
{
    return mbar_wait_impl<false>(bar, parity, abort_flag, err, code, limit);
}
// Same, for a barrier that CTAs of the pair arrive on remotely (cluster-scope acquire).
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err, int code,
                                                  long long limit = TC_WAIT_CYCLES)
{
    return mbar_wait_impl<true>(bar, parity, abort_flag, err, code, limit);
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
// Warp-uniform issue: every lane executes the surrounding code (so the descriptor arithmetic is
// uniform across the warp and needs no per-lane-to-uniform register moves), `leader` is
// non-zero in the one lane whose instruction takes effect.
__device__ __forceinline__ void umma_i8_w(uint32_t leader, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                 "@q tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader) : "memory");
}
__device__ __forceinline__ void umma_commit_w(uint32_t leader, uint32_t bar)
{
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
                 "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(bar), "r"(leader) : "memory");
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

// ---- CTA-pair (cta_group::2) helpers: cluster of two CTAs on one TPC -------------------
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank)
{
    uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank)); return r;
}
// Remote arrive on the leader CTA's barrier.  Relaxed: what the arrive publishes is "this
// warp's tcgen05.ld reads have completed" (tcgen05.wait::ld has returned and
// tcgen05.fence::before_thread_sync precedes the arrive); a release at cluster scope would also
// wait for the warp's global stores to drain, which nobody on the other side reads.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA loads of a CTA pair: the data lands in the issuing CTA's shared memory, the bytes are
// counted on the LEADER CTA's mbarrier (a shared::cluster address).  No multicast.
__device__ __forceinline__ void tma2_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t leader_bar,
                                             int c0, int c1, int c2, int c3)
{
    asm volatile("cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(dst), "l"(map), "r"(leader_bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma2_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t leader_bar, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(leader_bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void umma2_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma2_i8_w(uint32_t leader, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                 "@q tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader) : "memory");
}
__device__ __forceinline__ void umma2_commit_both_w(uint32_t leader, uint32_t bar)
{
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %2, 0;\n\t"
                 "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n\t}"
                 ::"r"(bar), "h"((uint16_t)3), "r"(leader) : "memory");
}
// arrives, once the pair's MMAs issued so far are complete, on the mbarrier at this offset in BOTH CTAs
__device__ __forceinline__ void umma2_commit_both(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ bool mbar_try_cluster(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Non-blocking barrier tests.  A barrier test takes a few hundred cycles to answer; an issuer
// loop that tests the barrier of the NEXT stage before issuing this stage's MMAs, and reads the
// answer a round later, keeps that latency off its critical path (measured with the probe:
// 163 -> 110 cycles per MMA at four MMAs per stage).
__device__ __forceinline__ uint32_t mbar_test(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ uint32_t mbar_test_cluster(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int (&v)[16])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld(uint32_t taddr, int (&v)[32]) { tmem_ld32(taddr, v); }
__device__ __forceinline__ void tmem_ld(uint32_t taddr, int (&v)[16]) { tmem_ld16(taddr, v); }

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

// 32-byte rows with 32-byte swizzle (K = 32 operands: the stem's im2col rows), 8-row groups 256 B apart.
__device__ __forceinline__ uint64_t smem_desc_sw32(uint32_t saddr)
{
    uint64_t d = (uint64_t)((saddr >> 4) & 0x3fff);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(256 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)6 << 61;                              // swizzle mode: 32 B
    return d;
}

// Same with an explicit stride between 8-row groups.
template <int ROWB>
__device__ __forceinline__ uint64_t smem_desc_sbo(uint32_t saddr, uint32_t sbo_bytes)
{
    uint64_t d = (uint64_t)((saddr >> 4) & 0x3fff);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(sbo_bytes >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)(ROWB == 128 ? 2 : 4) << 61;
    return d;
}

// kind::i8 instruction descriptor: D=s32, A=B=s8, both K-major, M=128, N=BN.
__host__ __device__ constexpr uint32_t idesc_i8(int bn, int m = TC_TILE_M)
{
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
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
    int lut_bytes;           // shared-memory bytes of the fused BN's table (BN * 256, or 0)
    int group;               // K blocks per pipeline stage (one barrier hand-shake per `group` blocks)
    int ntab;                // per-channel tables held in shared memory: 5, or 9 when the fused BN is computed arithmetically
    int flat_P;              // > 0: flat-pitch tiles (weight-stationary pair kernel): a tile is 128 consecutive lines of
                             // an image laid out with a row pitch of flat_P = W + 2 lines (one zero column either side);
                             // the tile walk's digits are then (image, tile-in-image) instead of (w, h, batch) tiles
    int epi_wps;             // epilogue warps per set, 4 or 8 (16 / epi_wps sets take alternate tiles)
    long long full_wait;     // cycle limit of the MMA issuer's wait for a pipeline stage's data (TC_WAIT_CYCLES)
    int drop_stage;          // >= 0: the producer neither arms nor loads this K step of its first tile, so the
                             // issuer's wait for it must run out (ffcu_test_arm_timeout; -1 in every other launch)
#ifdef FF_TC_TIMING
    int dbg;                 // timing experiments: bit 0 = skip the TMA loads, bit 1 = skip the MMAs, bit 2 = no global memory in the epilogue, bit 3 = no epilogue arithmetic
#endif
};
#ifdef FF_TC_TIMING
#define TC_DBG(p, bit) ((p).dbg & (bit))
#else
#define TC_DBG(p, bit) 0
#endif

// Epilogue variants.  All but EPI_RUNTIME fix the presence of PReLU / residual / fused BN at
// compile time, which turns the per-element code into one straight-line block the scheduler
// can interleave across elements (the run-time form branches per element and runs several
// times slower).
enum { EPI_RUNTIME = 0, EPI_PLAIN = 1, EPI_SLOPE = 2, EPI_RES_BN = 3, EPI_RES = 4, EPI_SLOPE_BN = 5 };

#define TC_MAX_STAGES 8
#define TC_NTAB 9          // most tables a kernel holds: w_scale, bias, slope, res_scale, inv_out | fused BN without a byte table: in_scale, scale, offset, inv_out (TcParams::ntab is the count in use)
// Accumulator ring in TMEM: 512 columns hold 512 / BN tiles.  With short K loops (the
// 64-channel layers) a tile's MMAs take less time than the hand-shake round trip to the
// epilogue warps and back, so the issuer must be able to run several tiles ahead.
#define TC_MAX_ACC 8
#define TC_NACC(BN) (512 / (BN) > TC_MAX_ACC ? TC_MAX_ACC : 512 / (BN))
// Warp 0: TMA producer, warp 1: MMA issuer, warps 2 .. 17: epilogue, warp 18: second MMA issuer
// (weight-stationary and stem kernels, idle elsewhere).
#define TC_ISSUER2_WARP 18
#define TC_THREADS (32 * 19)

struct TcShared {                 // lives after the stage ring and the tables
    uint64_t full[TC_MAX_STAGES];
    uint64_t empty[TC_MAX_STAGES];
    uint64_t acc_full[TC_MAX_ACC];
    uint64_t acc_empty[TC_MAX_ACC];
    uint64_t w_full;              // weight-stationary kernel: weights have landed
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void tc_load_tables(float* tab, const TcParams& p)
{
#pragma unroll 1
    for (int i = threadIdx.x; i < p.Cout; i += TC_THREADS) {
        tab[0 * TC_MAX_COUT + i] = p.t.w_scale[i];
        tab[1 * TC_MAX_COUT + i] = p.t.bias[i];
        tab[2 * TC_MAX_COUT + i] = p.t.slope ? p.t.slope[i] : 0.0f;
        tab[3 * TC_MAX_COUT + i] = p.t.res_scale ? p.t.res_scale[i] : 0.0f;
        tab[4 * TC_MAX_COUT + i] = p.t.inv_out ? p.t.inv_out[i] : 0.0f;
        if (p.out2 && !p.lut_bytes) {
            tab[5 * TC_MAX_COUT + i] = p.t.bn_in[i];
            tab[6 * TC_MAX_COUT + i] = p.t.bn_scale[i];
            tab[7 * TC_MAX_COUT + i] = p.t.bn_offset[i];
            tab[8 * TC_MAX_COUT + i] = p.t.bn_inv[i];
        }
    }
}

// The fused BN pass as a byte table in shared memory: lut[c * 256 + (uint8_t)q] for the BN
// channels [c0, c0 + bn) of this CTA's column tile (a CTA keeps one column tile for its lifetime).
__device__ __forceinline__ void tc_load_lut(uint8_t* lut, const TcParams& p, int c0, int bn)
{
    if (!p.out2 || !p.lut_bytes) return;
    const int4* src = (const int4*)(p.t.bn_lut + (size_t)c0 * 256);
    int4* dst = (int4*)lut;
#pragma unroll 1
    for (int i = threadIdx.x; i < bn * 16; i += TC_THREADS) dst[i] = __ldg(src + i);
}

// 32-byte global accesses (sm_100 has 256-bit vector loads / stores): one full sector per
// thread per instruction instead of two half-sector 16-byte accesses.
__device__ __forceinline__ void st_global_32B(void* ptr, const int (&w)[8])
{
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"l"(ptr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
}
__device__ __forceinline__ void ld_global_32B(const void* ptr, int (&w)[8])
{
    asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]) : "l"(ptr));
}

// ---------------------------------------------------------------------------
// Epilogue.  Replaces fused_epilogue_int8 (reference kernels/int8_epilogue.c:25-112), optionally
// followed by the next BN pass (:253-318) as a second output.
// ---------------------------------------------------------------------------

// Compile-time loop: f(std::integral_constant<int, 0>{}) ... f(integral_constant<N-1>), so the index
// can feed template arguments and immediate operands.
template <int N>
struct TcUnroll {
    template <typename F>
    __device__ __forceinline__ static void run(F&& f)
    {
        TcUnroll<N - 1>::run(f);
        f(std::integral_constant<int, N - 1>{});
    }
};
template <>
struct TcUnroll<0> {
    template <typename F>
    __device__ __forceinline__ static void run(F&&) {}
};

// TMEM -> registers, 16 columns of this warp's 32 lanes.  The load is asynchronous: the
// registers hold the data only after tmem_ld_wait, which names them as in/out operands so that
// no use of them can be scheduled above it.
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, int (&v)[16])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait(int (&v)[16])
{
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
                   "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])
                 :: "memory");
}

// One entry of the fused BN's byte table: entry (uint8_t)q of the row ROW rows past the one at
// shared-memory address lut_base.  The table is 256-byte aligned, so a row's address with the
// index byte dropped into its low byte IS the entry's address: one byte-permute instead of an
// extract and an add.  K = which byte of the packed word w holds q.
template <int K, int ROW>
__device__ __forceinline__ uint32_t tc_lut_byte(uint32_t w, uint32_t lut_base)
{
    uint32_t addr, r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(addr) : "r"(w), "r"(lut_base), "n"(0x7650 | K));
    asm("ld.shared.u8 %0, [%1 + %2];" : "=r"(r) : "r"(addr), "n"(ROW * 256));
    return r;
}

// Sixteen columns of one accumulator row: v[16] int32 at channels cb .. cb + 15 -> four packed
// int8 words (and four more for the fused BN's output).  CI = 0 / 1: first or second chunk of the
// pair whose 32 table rows start at shared-memory address lut_pr.
template <bool CONTRACT, int EPI, bool CHECK, int CI, bool ACC22 = false>
__device__ __forceinline__ void tc_epilogue16(const TcParams& p, const float* tab, uint32_t lut_pr,
                                              const int (&v)[16], const int* rw, int cb,
                                              bool rt_res, bool rt_slope, bool rt_bn2, int (&ow)[4], int (&ow2)[4])
{
    const bool has_res = (EPI == EPI_RUNTIME) ? rt_res : (EPI == EPI_RES_BN || EPI == EPI_RES);
    const bool has_slope = (EPI == EPI_RUNTIME) ? rt_slope : (EPI == EPI_SLOPE || EPI == EPI_SLOPE_BN);
    const bool has_bn2 = (EPI == EPI_RUNTIME) ? rt_bn2 : (EPI == EPI_RES_BN || EPI == EPI_SLOPE_BN);
    TcUnroll<4>::run([&](auto gc) {
        constexpr int g = decltype(gc)::value;
        const float4 ws = *(const float4*)&tab[0 * TC_MAX_COUT + cb + 4 * g];
        const float4 bi = *(const float4*)&tab[1 * TC_MAX_COUT + cb + 4 * g];
        const float4 sl = *(const float4*)&tab[2 * TC_MAX_COUT + cb + 4 * g];
        const float4 rs = *(const float4*)&tab[3 * TC_MAX_COUT + cb + 4 * g];
        const float4 iv = *(const float4*)&tab[4 * TC_MAX_COUT + cb + 4 * g];
        // int -> float: the residual's bytes never need the conversion unit (ffcu_byte2f is exact for every byte);
        // the accumulator does not either where the launcher has the layer's 22-bit bound (ACC22)
        const uint32_t rx = has_res ? ((uint32_t)rw[g] ^ 0x80808080u) : 0x80808080u;
        const float a0 = ACC22 ? ffcu_i2f_22(v[4 * g + 0]) : __int2float_rn(v[4 * g + 0]);
        const float a1 = ACC22 ? ffcu_i2f_22(v[4 * g + 1]) : __int2float_rn(v[4 * g + 1]);
        const float a2 = ACC22 ? ffcu_i2f_22(v[4 * g + 2]) : __int2float_rn(v[4 * g + 2]);
        const float a3 = ACC22 ? ffcu_i2f_22(v[4 * g + 3]) : __int2float_rn(v[4 * g + 3]);
        const float f0 = ffcu_conv_fp_f<CONTRACT>(a0, ws.x, bi.x, has_res, ffcu_byte2f<0>(rx), rs.x, has_slope, sl.x);
        const float f1 = ffcu_conv_fp_f<CONTRACT>(a1, ws.y, bi.y, has_res, ffcu_byte2f<1>(rx), rs.y, has_slope, sl.y);
        const float f2 = ffcu_conv_fp_f<CONTRACT>(a2, ws.z, bi.z, has_res, ffcu_byte2f<2>(rx), rs.z, has_slope, sl.z);
        const float f3 = ffcu_conv_fp_f<CONTRACT>(a3, ws.w, bi.w, has_res, ffcu_byte2f<3>(rx), rs.w, has_slope, sl.w);
        const int w = ffcu_pack4(ffcu_requant_nosat<CHECK>(f0, iv.x), ffcu_requant_nosat<CHECK>(f1, iv.y),
                                 ffcu_requant_nosat<CHECK>(f2, iv.z), ffcu_requant_nosat<CHECK>(f3, iv.w));
        ow[g] = w;
        if (EPI == EPI_RUNTIME && has_bn2 && !p.lut_bytes) {
            // BN of the four int8 results by arithmetic (no byte table in shared memory)
            const float4 b_in = *(const float4*)&tab[5 * TC_MAX_COUT + cb + 4 * g];
            const float4 b_sc = *(const float4*)&tab[6 * TC_MAX_COUT + cb + 4 * g];
            const float4 b_of = *(const float4*)&tab[7 * TC_MAX_COUT + cb + 4 * g];
            const float4 b_iv = *(const float4*)&tab[8 * TC_MAX_COUT + cb + 4 * g];
            const int a0 = (int)(int8_t)(w & 0xff), a1 = (int)(int8_t)((w >> 8) & 0xff);
            const int a2 = (int)(int8_t)((w >> 16) & 0xff), a3 = w >> 24;
            ow2[g] = ffcu_pack4(ffcu_bn_q_nosat<CHECK>(a0, b_in.x, b_sc.x, b_of.x, b_iv.x),
                                ffcu_bn_q_nosat<CHECK>(a1, b_in.y, b_sc.y, b_of.y, b_iv.y),
                                ffcu_bn_q_nosat<CHECK>(a2, b_in.z, b_sc.z, b_of.z, b_iv.z),
                                ffcu_bn_q_nosat<CHECK>(a3, b_in.w, b_sc.w, b_of.w, b_iv.w));
        } else if (has_bn2) {
#ifdef FF_TC_TIMING
            if (TC_DBG(p, 32)) { ow2[g] = w ^ 0x01010101; return; }     // timing experiment: no table look-ups (wrong results)
#endif
            // BN of the four int8 results just packed: one table row per channel, indexed by the byte
            constexpr int R = CI * 16 + 4 * g;
            const uint32_t b0 = tc_lut_byte<0, R + 0>((uint32_t)w, lut_pr), b1 = tc_lut_byte<1, R + 1>((uint32_t)w, lut_pr);
            const uint32_t b2 = tc_lut_byte<2, R + 2>((uint32_t)w, lut_pr), b3 = tc_lut_byte<3, R + 3>((uint32_t)w, lut_pr);
            ow2[g] = (int)__byte_perm(__byte_perm(b0, b1, 0x1140), __byte_perm(b2, b3, 0x1140), 0x5410);
        } else {
            ow2[g] = 0;
        }
    });
}

// FC variant: sixteen f32 outputs, out = fmaf((float)dot, w_scale, bias) (or the unfused order).
template <bool CONTRACT>
__device__ __forceinline__ void tc_fc16(const TcParams& p, const float* tab, const int (&v)[16], int cb, size_t o)
{
    float4* dst = (float4*)((float*)p.out + o);
#pragma unroll
    for (int g = 0; g < 4; g++) {
        const float4 ws = *(const float4*)&tab[0 * TC_MAX_COUT + cb + 4 * g];
        const float4 bi = *(const float4*)&tab[1 * TC_MAX_COUT + cb + 4 * g];
        float4 r;
        r.x = ffcu_fc_fp<CONTRACT>(v[4 * g + 0], ws.x, bi.x);
        r.y = ffcu_fc_fp<CONTRACT>(v[4 * g + 1], ws.y, bi.y);
        r.z = ffcu_fc_fp<CONTRACT>(v[4 * g + 2], ws.z, bi.z);
        r.w = ffcu_fc_fp<CONTRACT>(v[4 * g + 3], ws.w, bi.w);
        dst[g] = r;
    }
}

// Programmatic dependent launch.  Each tensor-core kernel is launched with
// cudaLaunchAttributeProgrammaticStreamSerialization.  tc_pdl_trigger, the kernel's first
// statement, lets the NEXT kernel of the stream become resident at once (on SMs this one leaves
// free: always the case at small batch, where a launch is 8-16 CTAs), so that its launch latency
// and set-up (barriers, TMEM, the per-channel tables, which no kernel writes) are hidden several
// kernels deep.  tc_pdl_wait blocks until the PREVIOUS kernel has completed and its stores are
// visible; every warp that touches activations executes it first.  Nothing a previous kernel
// produced, and nothing it may still read, is touched before that point.
__device__ __forceinline__ void tc_pdl_trigger()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void tc_pdl_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Launch with the programmatic-serialisation attribute, as clusters of `cluster` CTAs when that is
// 2 or more (the CTA-pair kernels, the eight-CTA layer chain).  $FF_PDL=0 launches the plain way.
template <typename... KArgs, typename... Args>
static int tc_launch_ex(void (*kern)(KArgs...), int grid, int smem, cudaStream_t s, int cluster, Args&&... args)
{
    static int pdl = -1;
    if (pdl < 0) { const char* e = getenv("FF_PDL"); pdl = (e && e[0] == '0') ? 0 : 1; }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (cluster >= 2) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)cluster; attr[n].val.clusterDim.y = 1; attr[n].val.clusterDim.z = 1;
        n++;
    }
    if (pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    cfg.attrs = attr; cfg.numAttrs = n;
    FFCU_CHECK(cudaLaunchKernelEx(&cfg, kern, args...));
    return 0;
}

// Tile walk.  A CTA visits tiles first, first + step, ...; the launchers keep step a multiple of
// tiles_n, so the column tile never changes and the row-tile index m advances by a constant.
// Its (w, h, batch) digits are carried forward with two compare-and-carry steps per tile: the
// three divisions a fresh decomposition costs are a third of a small tile's epilogue.
struct TileWalk { int tw, th, tb, dw, dh, db; };
__device__ __forceinline__ void walk_init(TileWalk& w, const TcParams& p, int first_m, int step_m)
{
    int m = first_m;
    w.tw = m % p.tiles_w; m /= p.tiles_w; w.th = m % p.tiles_h; w.tb = m / p.tiles_h;
    m = step_m;
    w.dw = m % p.tiles_w; m /= p.tiles_w; w.dh = m % p.tiles_h; w.db = m / p.tiles_h;
}
__device__ __forceinline__ void walk_next(TileWalk& w, const TcParams& p)
{
    w.tw += w.dw;
    int c = (w.tw >= p.tiles_w) ? 1 : 0;
    w.tw -= c ? p.tiles_w : 0;
    w.th += w.dh + c;
    c = (w.th >= p.tiles_h) ? 1 : 0;
    w.th -= c ? p.tiles_h : 0;
    w.tb += w.db + c;
}

// Epilogue warps: sixteen (warps 2..17), organised as 16 / wps sets of wps warps (TcParams::epi_wps,
// 4 or 8).  Set s takes the CTA's tiles s, s + sets, ...; within a set, warp e covers the TMEM lane
// quarter its index gives it (hardware: warp w reads lanes [32*(w%4), +32)) and column group e / 4 of
// wps / 4.  With four warps per set each warp walks all columns of its 32 rows, so the per-tile
// bookkeeping (tile walk, addresses, two barrier operations) is spread over twice the elements: the
// choice for narrow tiles at large batch.  Eight warps per set halve a tile's latency: the choice
// when a CTA sees only a few tiles.  The sets never exceed the accumulator ring.
#define TC_EPI_TOTAL_WARPS 16

// Epilogue role shared by all kernels.  A warp walks its column range in pairs of 16-column chunks:
// the tcgen05.ld of the next chunk is in flight while the current one is computed, each pair ends in
// 32-byte global stores, the residual's bytes are fetched one pair ahead.  The specialised variants
// (EPI != EPI_RUNTIME) assume what their launcher guarantees: the layer has the no-overflow proof, a
// fused BN comes with its byte table, no accumulator dump is asked for; everything else runs the
// EPI_RUNTIME variant.
template <int BN, bool CONTRACT, bool OUT_F32, int EPI, bool ACC22 = false>
__device__ __forceinline__ void tc_epilogue_role(const TcParams& p, const float* tab, const uint8_t* lut, TcShared* sh,
                                                 uint32_t tmem_base, volatile int* abort_flag, int warp, int lane,
                                                 int first, int step, int total, int m_mul, int m_off,
                                                 uint32_t remote_acc_empty /* 0: local barrier */)
{
    if (warp >= TC_ISSUER2_WARP) return;                  // not an epilogue warp
    const int wps = p.epi_wps;
    const int sets = TC_EPI_TOTAL_WARPS / wps;
    const int cols = BN / (wps >> 2);                     // columns this warp covers
    const int n_pairs = cols >> 5;                        // pairs of 16-column chunks
    const int q = warp & 3;
    const int set = (warp - 2) / wps;                     // which of the CTA's tiles this warp takes
    const int cg = ((warp - 2) % wps) >> 2;               // column group of this warp
    const int row = q * 32 + lane;
    const int iw = row % p.TW;
    const int ih = (row / p.TW) % p.TH;
    const int ib = row / (p.TW * p.TH);
    const bool has_res = (EPI == EPI_RUNTIME) ? ((p.res != nullptr) && (p.t.res_scale != nullptr))
                                              : (EPI == EPI_RES_BN || EPI == EPI_RES);
    const bool has_slope = p.t.slope != nullptr;
    const bool has_bn2 = (EPI == EPI_RUNTIME) ? (p.out2 != nullptr) : (EPI == EPI_RES_BN || EPI == EPI_SLOPE_BN);
    const bool check = (EPI == EPI_RUNTIME) && !p.t.no_overflow;
    const bool dump = (EPI == EPI_RUNTIME) && p.acc_out != nullptr;
    int local = set;
    bool ok = true;
    const int tn = first % p.tiles_n;
    const int c0 = tn * BN + cg * cols;                   // first channel of this warp's range
    const uint32_t lut0 = smem_u32(lut) + (uint32_t)(cg * cols) * 256u;
    first += set * step;
    step *= sets;
    TileWalk wk;
    walk_init(wk, p, (first / p.tiles_n) * m_mul + m_off, (step / p.tiles_n) * m_mul);
    for (int tile = first; tile < total && ok; tile += step, local += sets, walk_next(wk, p)) {
        int ow, oh, b;
        bool valid;
        if (p.flat_P) {
            // line l = tile * 128 + row of the image's padded-pitch layout: row l / P, column l % P - 1;
            // the pitch's two extra columns and the lines past the last row are positions without an output
            const int l = wk.th * TC_TILE_M + row;
            oh = l / p.flat_P;
            ow = l - oh * p.flat_P - 1;
            b = wk.tw;
            valid = (ow >= 0) && (ow < p.Wo) && (oh < p.Ho) && (b < p.batch);
        } else {
            ow = wk.tw * p.TW + iw; oh = wk.th * p.TH + ih; b = wk.tb * p.TB + ib;
            valid = (ow < p.Wo) && (oh < p.Ho) && (b < p.batch);
        }
        const size_t o0 = (((size_t)b * p.Ho + oh) * p.Wo + ow) * p.Cout + c0;
        const int a = local % TC_NACC(BN);
        const uint32_t aphase = (uint32_t)(local / TC_NACC(BN)) & 1;
        // the residual operand does not depend on the accumulator: the first 64 channels' bytes are
        // fetched before waiting for the MMAs, further ones two chunk pairs ahead of their use
        int rw[8], rn[8];
#pragma unroll
        for (int g = 0; g < 8; g++) { rw[g] = 0; rn[g] = 0; }
        if (has_res && valid && !TC_DBG(p, 4)) {
            ld_global_32B(p.res + o0, rw);
            if (n_pairs > 1) ld_global_32B(p.res + o0 + 32, rn);
        }
        ok = mbar_wait(smem_u32(&sh->acc_full[a]), aphase, abort_flag, p.err, FFCU_ERR_EPI_TIMEOUT);
        if (!ok) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + (uint32_t)(a * BN + cg * cols) + ((uint32_t)(q * 32) << 16);
        int v0[16], v1[16];
        tmem_ld16_issue(taddr, v0);
        tmem_ld_wait(v0);
#pragma unroll 1
        for (int pr = 0; pr < n_pairs; pr++) {
            const bool more = pr + 1 < n_pairs;
            const int cb = c0 + pr * 32;
            const size_t o = o0 + pr * 32;
            const uint32_t lut_pr = lut0 + (uint32_t)pr * (32u * 256u);
            tmem_ld16_issue(taddr + (uint32_t)(pr * 32 + 16), v1);            // lands while v0 is computed
            int w0[4], w0b[4], w1[4], w1b[4];
            if (valid && !TC_DBG(p, 8)) {
                if (dump) {
                    const int d0[8] = {v0[0], v0[1], v0[2], v0[3], v0[4], v0[5], v0[6], v0[7]};
                    const int d1[8] = {v0[8], v0[9], v0[10], v0[11], v0[12], v0[13], v0[14], v0[15]};
                    st_global_32B(p.acc_out + o, d0);
                    st_global_32B(p.acc_out + o + 8, d1);
                }
                if (OUT_F32) tc_fc16<CONTRACT>(p, tab, v0, cb, o);
                else if (check) tc_epilogue16<CONTRACT, EPI, true, 0>(p, tab, lut_pr, v0, rw, cb, has_res, has_slope, has_bn2, w0, w0b);
                else            tc_epilogue16<CONTRACT, EPI, false, 0, ACC22>(p, tab, lut_pr, v0, rw, cb, has_res, has_slope, has_bn2, w0, w0b);
            }
            tmem_ld_wait(v1);
            if (more) tmem_ld16_issue(taddr + (uint32_t)(pr * 32 + 32), v0);  // lands while v1 is computed
            if (valid && !TC_DBG(p, 8)) {
                if (dump) {
                    const int d0[8] = {v1[0], v1[1], v1[2], v1[3], v1[4], v1[5], v1[6], v1[7]};
                    const int d1[8] = {v1[8], v1[9], v1[10], v1[11], v1[12], v1[13], v1[14], v1[15]};
                    st_global_32B(p.acc_out + o + 16, d0);
                    st_global_32B(p.acc_out + o + 24, d1);
                }
                if (OUT_F32) tc_fc16<CONTRACT>(p, tab, v1, cb + 16, o + 16);
                else {
                    if (check) tc_epilogue16<CONTRACT, EPI, true, 1>(p, tab, lut_pr, v1, rw + 4, cb + 16, has_res, has_slope, has_bn2, w1, w1b);
                    else       tc_epilogue16<CONTRACT, EPI, false, 1, ACC22>(p, tab, lut_pr, v1, rw + 4, cb + 16, has_res, has_slope, has_bn2, w1, w1b);
                    if (!TC_DBG(p, 4)) {
                        const int w8[8] = {w0[0], w0[1], w0[2], w0[3], w1[0], w1[1], w1[2], w1[3]};
                        st_global_32B((int8_t*)p.out + o, w8);
                        if (has_bn2) {
                            const int w8b[8] = {w0b[0], w0b[1], w0b[2], w0b[3], w1b[0], w1b[1], w1b[2], w1b[3]};
                            st_global_32B(p.out2 + o, w8b);
                        }
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < 8; g++) rw[g] = rn[g];
            if (has_res && pr + 2 < n_pairs && valid && !TC_DBG(p, 4)) ld_global_32B(p.res + o + 64, rn);   // two pairs ahead
            if (more) tmem_ld_wait(v0);
        }
        // this warp's TMEM reads are complete (the last tcgen05.wait::ld has returned)
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
            if (remote_acc_empty) mbar_arrive_cluster(remote_acc_empty + (uint32_t)(a * 8));
            else mbar_arrive_relaxed(smem_u32(&sh->acc_empty[a]));
        }
    }
}

__device__ __forceinline__ void tc_setup(TcShared* sh, int stages, uint32_t tmem_cols, int warp, int epi_active)
{
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) { mbar_init(smem_u32(&sh->full[s]), 1); mbar_init(smem_u32(&sh->empty[s]), 1); }
        for (int a = 0; a < TC_MAX_ACC; a++) { mbar_init(smem_u32(&sh->acc_full[a]), 1); mbar_init(smem_u32(&sh->acc_empty[a]), epi_active); }
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
#pragma unroll 1
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}


// Kernel launchers, one translation unit per kernel family (they compile in parallel).
// epi is an EPI_* value; f32 selects the FC epilogue (f32 output, no requantisation).
int tc_launch_generic(int bn, int kc, int mode, int epi, bool f32, int grid, int smem, cudaStream_t s,
                      const CUtensorMap& mapA, const CUtensorMap& mapB, const TcParams& prm);
int tc_launch_ws(int bn, int mode, int epi, int grid, int smem, cudaStream_t s,
                 const CUtensorMap& mapA, const CUtensorMap& mapB, const TcParams& prm);
int tc_launch_pair(int bn, int mode, int epi, bool f32, int grid, int smem, cudaStream_t s,
                   const CUtensorMap& mapA, const CUtensorMap& mapB, const TcParams& prm);
int tc_launch_stem(int mode, int epi, int in_u8, int grid, int smem, cudaStream_t s, const CUtensorMap& mapB,
                   const TcParams& prm, const void* in_any, const float* inv3);
int tc_launch_wsp(int mode, int epi, int grid, int smem, cudaStream_t s,
                  const CUtensorMap& mapA, const CUtensorMap& mapB_half, const TcParams& prm);

// Stride-2 convolution + 1x1 shortcut in one launch (conv_tc_sc.cu)
struct ScParams {
    EpiTables t2;            // the shortcut layer's tables; res_scale scales the main path's int8 output
    int8_t* out_sc;          // the block's output (NHWC int8)
    int8_t* out2_sc;         // its fused BN output, or NULL
    int kb_sc;               // K blocks of the shortcut: its input channels / KC, rounded up (<= the main path's group)
    int write_main;          // 1: the main path's int8 output is stored too (TcParams::out): another layer reads it
    int lut_bytes;           // 64 * 256 when out2_sc comes through the byte table, else 0
};
int tc_launch_sc(int kc, int mode, int grid, int smem, cudaStream_t s, const CUtensorMap& mapA, const CUtensorMap& mapB,
                 const CUtensorMap& mapA2, const CUtensorMap& mapB2, const TcParams& prm, const ScParams& q);

// Split-K FC (conv_tc_fc.cu)
struct FcTcParams {
    const float* w_scale; const float* bias;
    float* out;              // [batch][N] f32
    int* sums;               // [rows][N] int32 partial sums, zero between calls
    int* tickets;            // [tiles_m * tiles_n] arrival counters, zero between calls
    int* err;
    int batch, N;
    int tiles_n, tiles_m, splits, blocks_per_split;   // grid = tiles_n * tiles_m * splits; K blocks of 128 per CTA
    int stages, group;
    int drop_step;           // >= 0: the producer leaves out this step's activation box (timeout test); -1 otherwise
    long long wait_cycles;   // limit of every barrier wait
};
int tc_launch_fc(int mode, int grid, int smem, cudaStream_t s, const CUtensorMap& mapA, const CUtensorMap& mapB, const FcTcParams& prm);

// Layer chain (conv_tc_chain.cu)
#define CHAIN_CLUSTER 8
#define CHAIN_BN 64
#define CHAIN_MAX_STAGES 8
#define CHAIN_EPI_WARPS 16
#define CHAIN_EPI_THREADS (32 * CHAIN_EPI_WARPS)

struct ChainLayer {                       // one layer of the chain, in global memory (256 bytes, 128-byte aligned)
    CUtensorMap mapB;                     // weights [Cout][9 * C] K-major, box {128, 64}
    const float* w_scale; const float* bias; const float* slope; const float* res_scale; const float* inv_out;
    const int8_t* lut;                    // fused BN byte table [Cout][256], or NULL
    const int8_t* res;                    // residual (NHWC int8), or NULL
    int8_t* out;                          // NHWC int8 output
    int8_t* out2;                         // fused BN second output, or NULL
    uint8_t pad_[256 - 128 - 9 * 8];
};
static_assert(sizeof(ChainLayer) == 256, "ChainLayer layout");

struct ChainParams {
    const ChainLayer* layers;
    int n_layers;
    int H, W, P, C;                       // feature map, pitch in lines, channels (in = out)
    int planes, plane_bytes;              // C / 128 planes of P * win_rows lines of 128 bytes
    int win_rows;                         // padded rows a CTA holds (the rows its row tile reads)
    int tiles_n;                          // C / 64 column tiles; CHAIN_CLUSTER / tiles_n row tiles
    int stages;                           // weight ring
    int tps;                              // filter taps per stage (1 or 3), planes x 8 KB each
    long long wait_cycles;                // limit of every barrier wait (TC_WAIT_CYCLES unless a test shortened it)
    int drop_step;                        // >= 0: CTA 0's producer leaves out this ring step (ffcu_test_arm_chain_timeout; -1 otherwise)
    int* err;
#ifdef FF_TC_TIMING
    unsigned long long* ts;               // timing build: per layer 4 time stamps of CTA 0 (ns)
    int dbg;                              // timing build: bit 0 = skip the weight loads (wrong results)
#endif
};

int tc_launch_chain(int mode, int smem, cudaStream_t s, const CUtensorMap& mapA, const ChainParams& prm);
bool tc_chain_fits(int smem);

// Flat-pitch weight-stationary pair kernel: activation buffer = guard + box of WSP_BOX_ROWS image rows
#define WSP_GUARD_BYTES 1024
#define WSP_BOX_ROWS 8

#define WS_TW 8
#define WS_TH 16
#ifndef WS_PITCH
#define WS_PITCH 10                                // pixels per image row of the activation box (>= WS_TW + 2)
#endif
#define WS_BOX_ROWS (WS_PITCH * (WS_TH + 2))       // rows of 64 B in the box
#define WS_A_BYTES ((WS_BOX_ROWS * 64 + 1023) / 1024 * 1024)
