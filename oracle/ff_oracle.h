/* ff_oracle.h -- CPU restatement of the FastFace INT8 forward (TEST INFRASTRUCTURE).
 *
 * This is the checker the CUDA path is compared against.  It is plain,
 * portable C (no intrinsics) and is never linked into, loaded by or called
 * from the shipped library.  Each function names the reference file:line it
 * restates.  Parity of this restatement itself is pinned against the
 * reference's own code compiled from its sources (see oracle/Makefile and
 * tests/test_oracle_vs_reference.py) and against committed golden vectors
 * produced by that compiled reference (tests/golden/).
 */
#ifndef FF_ORACLE_H
#define FF_ORACLE_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    FFO_OP_CONV = 1, FFO_OP_BN = 2, FFO_OP_PRELU = 3, FFO_OP_ADD = 4,
    FFO_OP_GEMM = 5, FFO_OP_FLATTEN = 6, FFO_OP_SAVE_ID = 7, FFO_OP_BLOCK_START = 8
};

/* fp32 evaluation order of the conv epilogue.
 * FFO_STRICT   : every mul and add rounded separately, in source order
 *                (reference built with -ffp-contract=off).
 * FFO_CONTRACT : mul+add pairs fused the way gcc 13 contracts them under the
 *                reference Makefile's default flags (-O3, fp-contract=fast). */
enum { FFO_STRICT = 0, FFO_CONTRACT = 1 };

/* Trace record kinds handed to the callback. */
enum { FFO_TRACE_INPUT_I8 = 0, FFO_TRACE_CONV_ACC = 1, FFO_TRACE_CONV_OUT = 2,
       FFO_TRACE_BN_OUT = 3, FFO_TRACE_FC_OUT = 4 };

typedef void (*ffo_trace_cb)(void* user, int op_index, int kind,
                             const void* data, size_t n_elems);

typedef struct ffo_model ffo_model;

/* Load FFW4 + OPSC (+ optional OPSC2, may be NULL or a missing file).
 * Returns NULL on any failure the reference's fastface_create also fails on. */
ffo_model* ffo_load(const char* ffw4_path, const char* opsc_path, const char* opsc2_path);
void       ffo_free(ffo_model* m);
int        ffo_n_ops(const ffo_model* m);
int        ffo_has_per_channel(const ffo_model* m);

/* Forward B faces.  in: [B][112][112][3] f32, out: [B][512] f32.
 * mode is FFO_STRICT or FFO_CONTRACT.  cb may be NULL. */
int ffo_forward(const ffo_model* m, const float* in, int B, float* out,
                int mode, ffo_trace_cb cb, void* user);

/* Sequential per-channel calibration: runs the forward on the given faces and,
 * at every requantisation point, sets that op's per-channel output scale to
 * percentile(|fp|)/127 before quantising and moving on.  Writes OPSC and OPSC2
 * files.  Used only to produce the synthetic model's scale fixture. */
int ffo_calibrate(const char* ffw4_path, const float* in, int B, double percentile,
                  const char* opsc_out, const char* opsc2_out);

/* ---- single-kernel restatements (also used directly by the tests) ---- */

/* exact int8 x int8 -> int32 convolution, NHWC in, [B*Ho*Wo][Cout] out,
 * weights in the file's [Cout][Cin][Kh][Kw] order. */
void ffo_conv_i32(const int8_t* in, int B, int Cin, int H, int W,
                  const int8_t* w_oihw, int Cout, int Kh, int Kw, int stride, int pad,
                  int Ho, int Wo, int32_t* acc);

/* conv epilogue: any of bias / slope / add_src / add_scale_pc / inv_out_pc may be NULL
 * exactly as in the reference signature. */
void ffo_epilogue(const int32_t* acc, int n_pos, int Cout, float in_scale,
                  const float* w_scale, const float* bias, const float* slope,
                  const int8_t* add_src, float add_scale, const float* add_scale_pc,
                  const float* inv_out_pc, float out_scale, int mode, int8_t* out);

void ffo_bn_requant(const int8_t* in, float in_scale, const float* in_scale_pc,
                    const float* bn_scale, const float* bn_offset, const float* slope,
                    const float* inv_out_pc, float out_scale, int8_t* out, int n_pos, int C);

void ffo_quantize_input_pc(const float* in, int n_pos, int C, const float* inv_pc, int8_t* out);
void ffo_quantize_input(const float* in, int n, float scale, int8_t* out);

/* FC: acts are CHW-flattened int8 [K]; w is [N][K]. */
void ffo_fc(const int8_t* a, const int8_t* w, const float* w_scale, const float* bias,
            float a_scale, int N, int K, int mode, float* out);

float ffo_cos_sim(const float* a, const float* b, int n);

#ifdef __cplusplus
}
#endif
#endif
