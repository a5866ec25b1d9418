/* fastface.h -- C API of the B200 (sm_100a) FastFace INT8 ArcFace engine.
 *
 * Drop-in for the reference's fastface.h: the three original entry points keep
 * their names, argument meaning, return values and file conventions, so a
 * consumer of the CPU library relinks against libfastface_b200.so unchanged.
 *
 *     FastFace* ff = fastface_create("models/w600k_r50_ffw4.bin");
 *     float input[FASTFACE_INPUT_N];     // HWC float32, [-1, 1]
 *     float emb[FASTFACE_OUTPUT_N];      // raw (not L2-normalised)
 *     fastface_embed(ff, input, emb);
 *     fastface_destroy(ff);
 *
 * Files: the weights are FFW4 (reference kernels/ffw2_loader.c:94-157).  As in
 * the reference (libfastface.c:236-240) the activation scales are read from
 * "models/op_scales.bin" relative to the working directory (required) and from
 * $OPSC2_PATH, else "models/op_scales_v2.bin" (optional; without it the
 * per-tensor scales are used exactly as the reference does).
 *
 * Threading: one context per thread, as in the reference (fastface.h:11-12).
 * There is no CPU fallback: creation fails when no CUDA device is usable.
 */
#ifndef FASTFACE_H
#define FASTFACE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct FastFace FastFace;

#define FASTFACE_INPUT_N  37632   /* 3 * 112 * 112 */
#define FASTFACE_OUTPUT_N 512

/* Replaces fastface_create (reference fastface.h:29-31, libfastface.c:231-310).
 * Returns NULL on failure: unreadable file, bad magic (FFW2/FFW3 are rejected),
 * missing models/op_scales.bin, op-count mismatch, no usable GPU.
 * Devices: $FASTFACE_DEVICES (comma-separated ordinals, default "0");
 * largest batch per device per step: $FASTFACE_MAX_BATCH (default 256).
 * The file is copied to the device; it may be deleted afterwards. */
FastFace* fastface_create(const char* ffw4_path);

/* Replaces fastface_embed (reference fastface.h:33-35, libfastface.c:312-470).
 * One face: 37632 fp32 in, 512 fp32 out.  0 on success, -1 on NULL arguments,
 * other non-zero on a device error (see fastface_last_error). */
int fastface_embed(FastFace* ff, const float* input_hwc, float* out_emb);

/* Replaces fastface_destroy (reference fastface.h:37-38, libfastface.c:472-490).
 * NULL is a no-op. */
void fastface_destroy(FastFace* ff);

/* ---- additions (superset) ------------------------------------------- */

/* Explicit device list and per-device step batch. device_ids may be NULL
 * (then devices 0..n_devices-1). */
FastFace* fastface_create_ex(const char* ffw4_path, const int* device_ids, int n_devices,
                             int max_batch);

/* n faces, contiguous [n][112][112][3] in, [n][512] out.  Semantics of the
 * reference's batched driver (arcface_forward_int8_batched.c:339-516) and of
 * FastFace.embed_batch in its Python wrapper (fastface.py:109-117), for any
 * n >= 1: faces are split into contiguous chunks across the context's devices
 * and into steps of at most max_batch per device. */
int fastface_embed_batch(FastFace* ff, const float* input_hwc, int n, float* out_emb);

/* The same from 8-bit pixels, contiguous [n][112][112][3] uint8 (channel order as the fp32 entry).
 * No counterpart in the reference's C API: its callers normalise on the host,
 * x = (p - 127.5) / 127.5 in fp32 (fastface.py:11), and pass fp32.  This entry does that
 * normalisation on the device with the same two fp32 roundings, so the embeddings are bit for
 * bit those of fastface_embed_batch on the normalised floats, while a quarter of the input bytes
 * cross PCIe. */
int fastface_embed_batch_u8(FastFace* ff, const uint8_t* pixels_hwc, int n, float* out_emb);

/* How fastface_embed_batch splits n faces over n_devices: contiguous chunks of
 * ceil(n / n_devices) faces (the last may be shorter; devices beyond the data get none).
 * Fills starts[] / counts[] and returns the number of devices used.  Pure host arithmetic. */
int fastface_shard_plan(int n, int n_devices, int* starts, int* counts);

/* Cosine similarity of two 512-d embeddings, float64 accumulation, 0 when a
 * norm is 0 (reference go/fastface/fastface.go:157-168). */
float fastface_cos_sim(const float* a, const float* b);

/* All pairs at once: out[i * m + j] = fastface_cos_sim(a + 512 * i, b + 512 * j), computed on the
 * context's first device with the same float64 arithmetic (bit-identical values).  The reference's
 * consumers loop over pairs on the host (go/examples/findface/main.go, face_match.py). */
int fastface_cos_sim_matrix(const FastFace* ff, const float* a, int n, const float* b, int m, float* out);

/* fp32 evaluation order of the conv epilogue (see FF_EPILOGUE_* below);
 * default FF_EPILOGUE_CONTRACT, or $FF_EPILOGUE=strict|contract at create. */
#define FF_EPILOGUE_STRICT   0  /* reference built with -ffp-contract=off            */
#define FF_EPILOGUE_CONTRACT 1  /* reference built with its Makefile's default flags */
int fastface_set_epilogue_mode(FastFace* ff, int mode);

/* Per-layer dump points, the counterpart of tracing the reference's kernel calls:
 * kind 'Q' int8 quantised input [n][112][112][3], 'A' int32 conv accumulators,
 * 'O' int8 conv output, 'B' int8 BN output, 'F' f32 embeddings [n][512].
 * op_index is the FFW4 op index.  Runs on the context's first device, n <= max_batch. */
typedef void (*fastface_trace_fn)(void* user, int op_index, int kind,
                                  const void* data, unsigned long long n_elems);
int fastface_trace_batch(FastFace* ff, const float* input_hwc, int n, float* out_emb,
                         fastface_trace_fn fn, void* user);

/* Benchmark hook: `iters` forward passes of n faces already resident on the
 * context's first device (uploads input_hwc once), timed with CUDA events on
 * the compute stream.  Returns total milliseconds in *ms. */
int fastface_bench_resident(FastFace* ff, const float* input_hwc, int n, int iters, float* ms);

/* Benchmark hooks per layer of the static launch list: fastface_layer_count() layers;
 * fastface_layer_desc fills desc[12] = {kind (0 quantise, 1 conv, 2 BN, 3 FC), FFW4 op index,
 * Cin, Cout, Kh, Kw, stride, H, W, Ho, Wo, 1 if the tensor-core kernel runs it};
 * fastface_bench_layers times each layer `iters` times over n resident faces (ms[k] = total
 * CUDA-event milliseconds of layer k) and returns the layer count. */
int fastface_layer_count(const FastFace* ff);
int fastface_layer_desc(const FastFace* ff, int k, int* desc12);
int fastface_bench_layers(FastFace* ff, const float* input_hwc, int n, int iters, float* ms, int cap);

/* Number of kernel launches the last embed/bench call issued per forward pass. */
int fastface_launches_per_forward(const FastFace* ff);

/* Text of the last error on the calling thread ("" if none). */
const char* fastface_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* FASTFACE_H */
