// ffcu_internal.cuh -- shared declarations of the CUDA side (sm_100a only).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <limits.h>

#include "ff_cuda.h"

#define FFCU_MAX_BUFS 8

// Device error word values (first error wins).
enum {
    FFCU_ERR_NONE = 0,
    FFCU_ERR_TMA_TIMEOUT = 1,    // a bounded wait on a TMA "full" barrier ran out
    FFCU_ERR_MMA_TIMEOUT = 2,    // a bounded wait on an MMA-commit barrier ran out
    FFCU_ERR_EMPTY_TIMEOUT = 3,  // a bounded wait on a pipeline "empty" barrier ran out
    FFCU_ERR_EPI_TIMEOUT = 4,    // the epilogue's bounded wait on "accumulator ready" ran out
    FFCU_ERR_TMEM_TIMEOUT = 5    // a bounded wait on "accumulator drained" ran out
};

void ffcu_set_error(const char* fmt, ...);

#define FFCU_CHECK(expr)                                                                    \
    do {                                                                                    \
        cudaError_t _e = (expr);                                                            \
        if (_e != cudaSuccess) {                                                            \
            ffcu_set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
            return -100;                                                                    \
        }                                                                                   \
    } while (0)

// Per-output-channel tables of one conv / FC epilogue (device pointers).
struct EpiTables {
    const float* w_scale;
    const float* bias;
    const float* slope;      // NULL: no PReLU
    const float* res_scale;  // NULL: no residual
    const float* inv_out;
    // fused BN second output (all NULL when the layer has none)
    const float* bn_in;      // scale of the int8 value just produced
    const float* bn_scale;
    const float* bn_offset;
    const float* bn_inv;
    const int8_t* bn_lut;    // [Cout][256]: BN of every int8 value (ff_bn_lut_build), or NULL
    // 1 when the host has proved, from the weights and tables, that |t * inv + 0.5| stays far
    // below 2^31 for every int8 input: the kernels then skip the per-element emulation of
    // x86's out-of-range conversion result (it cannot trigger).
    int no_overflow;
    // 1 when the host has proved |accumulator| < 2^22 for every int8 input (128 * sum|w| per output channel):
    // the kernels may then convert the accumulator to float with one integer add and one float add instead
    // of the conversion unit (the 64-input-channel layers and the stem are bound by that unit).
    int acc22;
};

// ---------------------------------------------------------------------------
// The reference's fp32 arithmetic, one rounding per stated operation.
// ---------------------------------------------------------------------------

// Requantise: q = t * inv; r = q + copysign(0.5, q); truncate; clamp to [-128, 127]
// (reference kernels/int8_epilogue.c:80-87).  x86 cvttps2dq returns INT_MIN for NaN
// and for |r| >= 2^31, which the clamp turns into -128; reproduced here because
// __float2int_rz saturates instead.
__device__ __forceinline__ int ffcu_requant(float t, float inv)
{
    float q = __fmul_rn(t, inv);
    float half = __int_as_float(0x3f000000 | (__float_as_int(q) & 0x80000000));
    float r = __fadd_rn(q, half);
    int i = __float2int_rz(r);
    if (!(fabsf(r) < 2147483648.0f)) i = INT_MIN;
    return max(-128, min(127, i));
}

// Same rounding as ffcu_requant, but the clamp is left to the caller (ffcu_pack4 saturates).
// CHECK = false is for layers whose EpiTables::no_overflow is set.
template <bool CHECK = true>
__device__ __forceinline__ int ffcu_requant_nosat(float t, float inv)
{
    float q = __fmul_rn(t, inv);
    float half = __int_as_float(0x3f000000 | (__float_as_int(q) & 0x80000000));
    float r = __fadd_rn(q, half);
    int i = __float2int_rz(r);
    if (CHECK) { if (!(fabsf(r) < 2147483648.0f)) i = INT_MIN; }
    return i;
}

// Four int32 -> four int8 with saturation to [-128, 127], packed little-endian (a = byte 0).
__device__ __forceinline__ int ffcu_pack4(int a, int b, int c, int d)
{
    int hi, out;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(d), "r"(c));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(b), "r"(a), "r"(hi));
    return out;
}

// BN of an already-clamped int8 value, unclamped result (see ffcu_bn_q).
template <bool CHECK = true>
__device__ __forceinline__ int ffcu_bn_q_nosat(int a, float in_scale, float bn_scale, float bn_offset, float inv)
{
    float t = __fmul_rn(__int2float_rn(a), in_scale);
    t = __fmaf_rn(t, bn_scale, bn_offset);
    return ffcu_requant_nosat<CHECK>(t, inv);
}

// (float)acc without the conversion unit, exact for -2^22 <= acc < 2^22: the bit pattern of 1.5 * 2^23 plus acc
// is the float 12582912 + acc (one unit in the last place is 1 in that binade); subtracting the constant is exact.
__device__ __forceinline__ float ffcu_i2f_22(int acc)
{
    return __fadd_rn(__int_as_float(acc + 0x4B400000), -12582912.0f);
}
// (float)(int8_t) of byte K of a packed word, given wx = word ^ 0x80808080 (each byte + 128 as unsigned): the
// byte dropped into the low byte of 2^23's bit pattern is the float 8388608 + byte + 128.  Always exact.
template <int K>
__device__ __forceinline__ float ffcu_byte2f(uint32_t wx)
{
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(wx), "r"(0x4B000000u), "n"(0x7650 | K));
    return __fadd_rn(__uint_as_float(d), -8388736.0f);
}

// Conv epilogue value before requantisation, from operands already converted to float.
template <bool CONTRACT>
__device__ __forceinline__ float ffcu_conv_fp_f(float t, float ws, float bias, bool has_res, float resf,
                                                float rs, bool has_slope, float slope)
{
    if (CONTRACT) {
        t = __fmaf_rn(t, ws, bias);
        if (has_res) t = __fmaf_rn(resf, rs, t);
    } else {
        t = __fadd_rn(__fmul_rn(t, ws), bias);
        if (has_res) t = __fadd_rn(t, __fmul_rn(resf, rs));
    }
    if (has_slope && t < 0.0f) t = __fmul_rn(t, slope);
    return t;
}

// Conv epilogue value before requantisation (reference kernels/int8_epilogue.c:53-76).
// CONTRACT selects the evaluation gcc produces for that source under the reference
// Makefile's flags: the "* w_scale + bias" and "res * res_scale + t" pairs become fmas.
template <bool CONTRACT>
__device__ __forceinline__ float ffcu_conv_fp(int acc, float ws, float bias, bool has_res, int res,
                                              float rs, bool has_slope, float slope)
{
    float t = __int2float_rn(acc);            // (float)acc, then * in_scale (1.0f): exact
    if (CONTRACT) {
        t = __fmaf_rn(t, ws, bias);
        if (has_res) t = __fmaf_rn(__int2float_rn(res), rs, t);
    } else {
        t = __fadd_rn(__fmul_rn(t, ws), bias);
        if (has_res) t = __fadd_rn(t, __fmul_rn(__int2float_rn(res), rs));
    }
    if (has_slope && t < 0.0f) t = __fmul_rn(t, slope);
    return t;
}

// Standalone BN pass (reference kernels/int8_epilogue.c:272-303): explicit fma in the source.
__device__ __forceinline__ int ffcu_bn_q(int a, float in_scale, float bn_scale, float bn_offset, float inv)
{
    float t = __fmul_rn(__int2float_rn(a), in_scale);
    t = __fmaf_rn(t, bn_scale, bn_offset);
    return ffcu_requant(t, inv);
}

// FC output (reference kernels/gemm_int8_matvec.c:78-79): bias + (float)dot * 1.0f * w_scale.
template <bool CONTRACT>
__device__ __forceinline__ float ffcu_fc_fp(int dot, float ws, float bias)
{
    float t = __int2float_rn(dot);
    return CONTRACT ? __fmaf_rn(t, ws, bias) : __fadd_rn(bias, __fmul_rn(t, ws));
}

// ---------------------------------------------------------------------------
// Kernel launchers (kernels_simt.cu)
// ---------------------------------------------------------------------------
int ffcu_launch_quant(const float* in, int n_pix, const float* inv3, int8_t* out4, cudaStream_t s);
int ffcu_launch_conv_simt(const ffcu_layer& L, int batch, int mode, const int8_t* in, const int8_t* w,
                          const EpiTables& t, const int8_t* res, int32_t* acc_out, int8_t* out,
                          int8_t* out_bn2, cudaStream_t s);
// Fused stem: fp32 input -> per-channel int8 quantise -> conv3x3 3->64 -> epilogue (+BN second output).
// q_out (optional) receives the quantised input as 4-byte pixels.
int ffcu_launch_stem(const void* in_any, int in_u8, const float* inv3, const int8_t* w, const EpiTables& t, int batch,
                     int mode, int8_t* out, int8_t* out_bn2, int8_t* q_out, cudaStream_t s);
int ffcu_launch_bn(const int8_t* in, int8_t* out, size_t n_pos, int C, const float* in_scale,
                   const float* bn_scale, const float* bn_offset, const float* inv_out, cudaStream_t s);
int ffcu_launch_fc_simt(const int8_t* act, const int8_t* w, const float* w_scale, const float* bias,
                        int batch, int N, int K, int mode, float* out, cudaStream_t s);

// Small-batch (<= 16) split-K FC; scratch is an int32 [batch][N] accumulator, zero on entry and exit.
#define FFCU_FC_SMALL_MAX_BATCH 16
#define FFCU_FC_SMALL_TICKETS 64          // ticket counters at the head of the small-batch FC scratch (one per 8 outputs)
int ffcu_launch_fc_small(const int8_t* act, const int8_t* w, const float* w_scale, const float* bias,
                         int batch, int N, int K, int mode, int* scratch, float* out, cudaStream_t s);

// ---------------------------------------------------------------------------
// Tensor-core implicit GEMM (conv_tc.cu)
// ---------------------------------------------------------------------------
// A down-sampling block's stride-2 3x3 convolution and its 1x1 stride-2 shortcut (+ ADD + fused BN) in one launch.
struct ScPlan;
ScPlan* ffcu_sc_plan(const ffcu_layer& main, const ffcu_layer& sc, int max_batch, const int8_t* d_in_main, const int8_t* d_w_main,
                     const int8_t* d_in_sc, const int8_t* d_w_sc, int device);
void    ffcu_sc_free(ScPlan* sp);
int     ffcu_sc_launch(const ScPlan* sp, int batch, int mode, const EpiTables& t1, const EpiTables& t2, int8_t* out_main,
                       int write_main, int8_t* out_sc, int8_t* out2_sc, int* d_err, cudaStream_t s);
// Layer chain (batch 1): consecutive 3x3 stride-1 C -> C convolutions of one feature-map size in one launch.
struct ChainPlan;
struct ChainLayerDesc { const int8_t* w; EpiTables t; const int8_t* res; int8_t* out; int8_t* out2; };
ChainPlan* ffcu_chain_plan(int H, int W, int C, const int8_t* d_in, const ChainLayerDesc* layers, int n_layers, int device);
void       ffcu_chain_free(ChainPlan* p);
int        ffcu_chain_launch(const ChainPlan* p, int mode, int* d_err, cudaStream_t s);
struct TcPlan;   // opaque: tile shape, TMA descriptors, launch geometry for one layer
int ffcu_stem_weight_k32(const int8_t* d_w, int8_t* d_wk, int Cout, cudaStream_t s);
// Tensor-core stem (one launch): plan over the repacked weights d_wk [64][32]
struct StemTcPlan;
StemTcPlan* ffcu_stem_tc_plan(int max_batch, const int8_t* d_wk, bool has_bn2, int device);
void ffcu_stem_tc_free(StemTcPlan* p);
// Column-tile width (64 / 128 / 256) for a call of `batch` faces, and the plan for one width.
int     ffcu_tc_pick_bn(const ffcu_layer& L, int batch, int device, int fill_div = 0);
#define FFCU_FC_TC_TICKETS 256      // (128-face row tile, 64-column tile) pairs the split-K FC can count: 4096 faces x 512 outputs
int     ffcu_fc_tc_launch(const TcPlan* p, int batch, int mode, const EpiTables& t, float* out, int* scratch, int scratch_rows,
                          int* d_err, cudaStream_t s);
// NULL when the layer shape is not covered by the tensor-core kernels.
int ffcu_stem_fused_launch(const StemTcPlan* p, const void* in_any, int in_u8, const float* inv3, int batch, int mode,
                           const EpiTables& t, int8_t* out, int8_t* out_bn2, int* d_err, cudaStream_t s);
// NULL when the layer shape is not covered by the tensor-core kernels.
TcPlan* ffcu_tc_plan(const ffcu_layer& L, int max_batch, const int8_t* d_in, const int8_t* d_w, int device, int bn);
void    ffcu_tc_free(TcPlan* p);
int     ffcu_tc_launch(const TcPlan* p, int batch, int mode, const EpiTables& t, const int8_t* res,
                       int32_t* acc_out, void* out, int8_t* out_bn2, int* d_err, cudaStream_t s);
