/* ff_cuda.h -- C-ABI shim between the C99 host code and the CUDA (sm_100a) side.
 *
 * Plain pointers and sizes only.  The C99 host parses the model files, resolves
 * every scale the reference's driver loop (libfastface.c:349-466) would pick at
 * run time into per-channel arrays, assigns activation buffers, and hands the
 * resulting static layer list to the device context through these calls.  Each
 * entry names the reference function whose work it takes over.
 */
#ifndef FF_CUDA_H
#define FF_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ffcu_ctx ffcu_ctx;

enum { FFCU_QUANT = 0, FFCU_CONV = 1, FFCU_BN = 2, FFCU_FC = 3 };

/* One step of the static layer plan.  All arrays are host pointers that
 * ffcu_add_layer copies to the device; they need not outlive the call. */
typedef struct {
    int kind;            /* FFCU_*                                                   */
    int op_index;        /* FFW4 op index (dump-point id)                            */
    int src_buf;         /* activation buffer ids; FFCU_QUANT reads the fp32 input   */
    int dst_buf;         /* FFCU_FC writes the f32 embedding buffer                  */
    int res_buf;         /* residual operand of a fused ADD, or -1                   */
    int Cin, Cout, Kh, Kw, stride, pad;
    int H, W, Ho, Wo;    /* per-face input / output extent                           */
    /* FFCU_CONV: int8 weights repacked [Cout][Kh][Kw][Cin_pad] (Cin_pad = Cin rounded
     * up to 4); FFCU_FC: [N][K] with K in (h,w,c) order.                             */
    const int8_t* w;
    size_t w_bytes;
    int Cin_pad;
    /* per-output-channel fp32 tables, each [Cout] (or [C] for BN); NULL = unused   */
    const float* w_scale;    /* conv/FC dequant scale                                */
    const float* bias;       /* conv/FC bias                                         */
    const float* slope;      /* fused PReLU                                          */
    const float* res_scale;  /* scale of the residual operand                        */
    const float* inv_out;    /* requant multiplier 1/(s+1e-9f) (conv, BN, input)     */
    const float* in_scale;   /* BN: scale of the int8 input                          */
    const float* bn_scale;   /* BN                                                   */
    const float* bn_offset;  /* BN                                                   */
    /* FFCU_CONV only: a BN pass fused as a SECOND output of the epilogue.  The int8 result q
     * is stored to dst_buf as usual and BN(q) (same arithmetic as a FFCU_BN layer reading
     * dst_buf) is stored to bn2_dst_buf.  bn2_dst_buf < 0: none.                            */
    int bn2_dst_buf;
    int bn2_op_index;          /* FFW4 op index of the fused BN (dump-point id)             */
    const float* bn2_in_scale;
    const float* bn2_scale;
    const float* bn2_offset;
    const float* bn2_inv_out;
    /* Optional: the same BN as a table, [Cout][256] int8 indexed by the int8 value's byte
     * (two's complement, 0..255); ff_bn_lut_build fills it.  NULL: the kernels compute BN. */
    const int8_t* bn2_lut;
} ffcu_layer;

/* BN + requantisation of every int8 input value, per channel: lut[c*256 + (uint8_t)q] =
 * bn_prelu_requant_int8 (reference kernels/int8_epilogue.c:253-318) applied to q in channel c.
 * Plain host arithmetic with one IEEE rounding per operation, bit-identical to the kernels. */
void ff_bn_lut_build(const float* in_scale, const float* bn_scale, const float* bn_offset,
                     const float* inv_out, int C, int8_t* lut);

/* Devices visible to the process; <0 on a CUDA error. */
int ffcu_device_count(void);

/* Device context: n_bufs int8 activation buffers of max_batch*bytes_per_face each,
 * an fp32 input and an f32 output buffer for max_batch faces, streams, pinned
 * staging.  Takes over the buffer allocation of libfastface.c:301-308. */
ffcu_ctx* ffcu_create(int device, int max_batch, int n_bufs, size_t bytes_per_face);
void      ffcu_destroy(ffcu_ctx* c);

/* Append one layer (uploads its weights and tables).  Returns the layer id, <0 on error.
 * Takes over pack_conv_weight_nhwc's device-side half (kernels/conv2d_nhwc.c:79-100). */
int ffcu_add_layer(ffcu_ctx* c, const ffcu_layer* l);

/* Fix the plan: picks kernels/tiles per layer, encodes TMA descriptors. */
int ffcu_finalize(ffcu_ctx* c);

/* mode: 0 strict, 1 contract (fp32 evaluation order of the conv/FC epilogue). */
int ffcu_set_mode(ffcu_ctx* c, int mode);

/* Forward n <= max_batch faces: host fp32 in -> host f32 out, copies included.
 * Asynchronous on the context's stream; ffcu_wait blocks until it is done and
 * returns 0 or the device error word.  Takes over the op loop of
 * arcface_forward_int8_batched.c:339-516. */
int ffcu_submit(ffcu_ctx* c, const float* host_in, int n, float* host_out);
/* Same forward from 8-bit pixels [n][112][112][3]: the fused stem forms (p - 127.5f) / 127.5f in
 * fp32 (the value the reference's wrapper computes on the host, fastface.py:11) and quantises it as
 * quantize_fp32_nhwc_to_int8 does (kernels/int8_epilogue.c:231-247).  A quarter of the bytes
 * cross PCIe.  Needs the fused stem (the default). */
int ffcu_submit_u8(ffcu_ctx* c, const uint8_t* host_pixels, int n, float* host_out);
int ffcu_wait(ffcu_ctx* c);

/* Same forward with dump points; fn is called on the host after each layer. */
typedef void (*ffcu_trace_fn)(void* user, int op_index, int kind,
                              const void* data, unsigned long long n_elems);
int ffcu_trace(ffcu_ctx* c, const float* host_in, int n, float* host_out,
               ffcu_trace_fn fn, void* user);

/* iters forwards over n faces already on the device; CUDA-event milliseconds. */
int ffcu_bench_resident(ffcu_ctx* c, const float* host_in, int n, int iters, float* ms);

int ffcu_launches_per_forward(const ffcu_ctx* c);

/* Per-layer timing: after one full forward over n resident faces, each layer is
 * launched `iters` times back to back between two CUDA events on the compute stream;
 * ms[k] receives the total for layer k.  Returns the layer count (<0 on error). */
int ffcu_bench_layers(ffcu_ctx* c, const float* host_in, int n, int iters, float* ms, int cap);

/* Layer count and description of layer k (pointer members are NULL in *out);
 * *uses_tc = 1 when the tensor-core implicit-GEMM kernel runs it. */
int ffcu_layer_count(const ffcu_ctx* c);
int ffcu_layer_info(const ffcu_ctx* c, int k, ffcu_layer* out, int* uses_tc);

/* Standalone kernels on raw device-independent host buffers, for the single-layer
 * parity tests: runs one conv layer (int8 NHWC in, optional residual) and returns
 * int32 accumulators and/or the int8 epilogue output. impl: 0 = tensor-core
 * implicit GEMM, 1 = SIMT reference kernel. */
int ffcu_conv_once(int device, const ffcu_layer* l, int batch, int mode, int impl,
                   const int8_t* in, const int8_t* res, int32_t* acc_out, int8_t* out, int8_t* out_bn2);

/* The same layer, timed: after one run (whose int8 output is returned), `iters` more launches between
 * two CUDA events on the layer's stream; *ms = mean milliseconds per launch.  The single-layer
 * microbenchmark (the reference's bench_batched_conv.c measures its CPU kernels the same way). */
int ffcu_conv_bench(int device, const ffcu_layer* l, int batch, int mode, int impl,
                    const int8_t* in, const int8_t* res, int8_t* out, int8_t* out_bn2, int iters, float* ms);

/* 3x3 stride-1 pad-1 convolution by exact-integer Winograd F(2,3) on the CUDA cores (reference
 * kernels/winograd_int8_ref.c:117-179; int16 transformed operands, which the int8 tensor cores
 * cannot take): host tensors in int8 [B][H][W][Cin], w int8 OIHW -> out int32 [B][H][W][Cout],
 * equal to 4 x the direct convolution's accumulators (:237-259).  *ms = mean CUDA-event time of
 * `iters` runs of the convolution kernel (the weight transform is a load-time step and not timed).
 * Needs H, W multiples of 8, Cin a multiple of 16 (<= 128), Cout a multiple of 64.  Kept as the
 * measured alternative to the implicit GEMM; the forward pass does not use it. */
int ffcu_winograd_f23_once(int device, const int8_t* in, const int8_t* w_oihw, int B, int H, int W, int Cin,
                           int Cout, int iters, int32_t* out, float* ms);

/* Test hook for the bounded waits (no counterpart in the reference): arms the NEXT launch of the
 * one-CTA per-tap convolution kernel so that its TMA producer leaves out K step `drop_stage` of
 * its first tile, and the MMA issuer's wait for that step's data gives up after
 * `full_wait_cycles` SM cycles instead of the default two seconds.  The kernel then takes its
 * abort path: it records the error word, every role leaves its loop, tensor memory is freed and
 * the launch returns; ffcu_conv_once / ffcu_wait report 1000 + the error word.  Nothing faults,
 * traps or spins without a limit, and the hook disarms itself after that one launch. */
void ffcu_test_arm_timeout(int drop_stage, long long full_wait_cycles);
/* The same for the batch-1 layer-chain kernel (a cluster of eight CTAs): CTA 0's weight producer leaves out
 * ring step drop_step of the next chain launch and every barrier wait of that launch is limited to
 * wait_cycles.  CTA 0's MMA issuer gives up first; the other seven, waiting for results CTA 0 never
 * sends, give up one limit later; all eight meet at the final cluster barrier, free their tensor memory
 * and return; the call reports 1000 + the error word.  Disarms itself after that one launch. */
void ffcu_test_arm_chain_timeout(int drop_step, long long wait_cycles);
/* The same for the split-K FC kernel: the activation box of K step drop_step never arrives in any CTA of the next FC
 * launch and every barrier wait of that launch is limited to wait_cycles; every CTA gives up, takes no ticket, frees
 * its tensor memory and returns; the call reports 1000 + the error word and clears the kernel's scratch sums. */
void ffcu_test_arm_fc_timeout(int drop_step, long long wait_cycles);

/* Small-batch FC (batch <= 16, N <= 512) that allocates nothing: no counterpart in the
 * reference.  For callers that hold device buffers but cannot call cudaMalloc -- a serving loop
 * that cannot afford an allocation's device-wide synchronisation, a plug-in given buffers but no
 * allocator, a process with a fixed memory budget.  The split-K int32 accumulator the kernel
 * needs is a fixed 32 KiB array inside the library's device image.  act int8 [batch][K],
 * w int8 [N][K], w_scale / bias f32 [N], out f32 [batch][N]: all DEVICE pointers; stream is a
 * cudaStream_t (NULL = default stream).  Sizes beyond the limit return -2 with a message.
 * act and w must be 16-byte aligned, K a positive multiple of 16, N a multiple of 8, and
 * w_scale / bias / out 4-byte aligned; anything else returns -1 before a kernel is launched.
 * Every call on a device shares the one array (cleared at the start of each call): calls that
 * can overlap on the GPU race.  The first call on a device resolves the array's address; make
 * it outside any stream capture.  Computes out = bias + (float)dot * w_scale exactly as the FC
 * of fastface_embed (reference kernels/gemm_int8_matvec.c:78-79). */
int ffcu_fc_small_noalloc(const int8_t* act, const int8_t* w, const float* w_scale, const float* bias,
                          int batch, int N, int K, int mode, float* out, void* stream);

/* Cosine-similarity matrix out[n][m] of host embeddings a[n][512], b[m][512] with the float64
 * accumulation of the reference's Go wrapper (go/fastface/fastface.go:157-168), bit for bit. */
int ffcu_cos_sim_matrix(int device, const float* a, int n, const float* b, int m, float* out);

/* Dense INT8 tensor-core throughput (TOP/s, 2 ops per MAC) measured with operands already in
 * shared memory: M=128, N=bn (64/128/256), all SMs busy, `iters` rounds of four K=32 MMAs.
 * The practical ceiling the convolution kernels are compared against. */
int ffcu_i8_mma_peak(int device, int bn, int iters, float* tops, float* ms);

const char* ffcu_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* FF_CUDA_H */
