/* ff_oracle.c -- CPU restatement of the FastFace INT8 forward (TEST INFRASTRUCTURE).
 *
 * Plain C99, no intrinsics, OpenMP only for speed.  Nothing in the shipped
 * library includes, links or calls this file; it exists to check the CUDA path.
 * Citations are paths inside the reference project (bauratynov/fastface).
 */
#include "ff_oracle.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    int type;
    int Cin, Cout, Kh, Kw, stride, pad;
    int8_t* w;          /* conv: [Cout][Cin][Kh][Kw] as stored in the file */
    float*  scale;      /* conv/gemm per-output scale */
    float*  bias;
    int     n;          /* BN / PReLU length */
    float*  bn_scale;
    float*  bn_offset;
    float*  slope;
    uint32_t N, K;      /* GEMM */
} ffo_op;

struct ffo_model {
    int n_ops;
    ffo_op* ops;
    /* OPSC  (libfastface.c:193-204) */
    float input_scale;
    float* scales;          /* [n_ops] */
    /* OPSC2 (libfastface.c:133-191) */
    int has_pc;
    int n_in;
    float* in_pc_scale;
    float* in_pc_inv;
    uint32_t* pc_len;       /* [n_ops] */
    float** pc_scale;       /* [n_ops] or NULL entries */
    float** pc_inv;
};

/* ------------------------------------------------------------------ */
/* fp32 helpers with the operation order made explicit                 */
/* ------------------------------------------------------------------ */

/* volatile stores stop the compiler from contracting a*b+c into an fma */
static inline float mul_rn(float a, float b) { volatile float r = a * b; return r; }
static inline float add_rn(float a, float b) { volatile float r = a + b; return r; }

/* kernels/int8_epilogue.c:81-87 -- add +/-0.5 (sign taken from the sign bit, so
 * -0 rounds with -0.5), truncate, clamp.  cvttps2dq yields INT_MIN for NaN and
 * for |r| >= 2^31, which the clamp then turns into -128. */
static inline int8_t requant_half_away(float q)
{
    uint32_t bits; memcpy(&bits, &q, 4);
    uint32_t hb = 0x3f000000u | (bits & 0x80000000u);
    float half; memcpy(&half, &hb, 4);
    float r = add_rn(q, half);
    int32_t i;
    if (r != r || r >= 2147483648.0f || r < -2147483648.0f) i = INT32_MIN;
    else i = (int32_t)r; /* C truncation toward zero */
    if (i < -128) i = -128;
    if (i > 127) i = 127;
    return (int8_t)i;
}

/* kernels/int8_epilogue.c:222,241 -- lrintf (ties to even) then clamp */
static inline int8_t quant_lrint(float v)
{
    long q = lrintf(v);
    int qi = (int)q;
    if (qi > 127) qi = 127;
    if (qi < -128) qi = -128;
    return (int8_t)qi;
}

/* ------------------------------------------------------------------ */
/* kernels                                                             */
/* ------------------------------------------------------------------ */

/* kernels/conv2d_nhwc.c:29-74 (im2col order kh,kw,ci; zero padding) +
 * kernels/gemm_int8_v2.c:42-110 (exact signed dot product after the +128 /
 * -128*colsum trick) restated as a direct convolution. */
void ffo_conv_i32(const int8_t* in, int B, int Cin, int H, int W,
                  const int8_t* w_oihw, int Cout, int Kh, int Kw, int stride, int pad,
                  int Ho, int Wo, int32_t* acc)
{
    /* repack to [Cout][Kh][Kw][Cin] so the inner loop is contiguous */
    size_t wn = (size_t)Cout * Cin * Kh * Kw;
    int8_t* wp = (int8_t*)malloc(wn);
    for (int co = 0; co < Cout; co++)
        for (int ci = 0; ci < Cin; ci++)
            for (int kh = 0; kh < Kh; kh++)
                for (int kw = 0; kw < Kw; kw++)
                    wp[(((size_t)co * Kh + kh) * Kw + kw) * Cin + ci] =
                        w_oihw[(((size_t)co * Cin + ci) * Kh + kh) * Kw + kw];
    long rows = (long)B * Ho;
    #pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; r++) {
        int b = (int)(r / Ho), oh = (int)(r % Ho);
        const int8_t* inb = in + (size_t)b * H * W * Cin;
        for (int ow = 0; ow < Wo; ow++) {
            int32_t* out = acc + (((size_t)b * Ho + oh) * Wo + ow) * Cout;
            for (int co = 0; co < Cout; co++) {
                int32_t s = 0;
                for (int kh = 0; kh < Kh; kh++) {
                    int ih = oh * stride - pad + kh;
                    if (ih < 0 || ih >= H) continue;
                    for (int kw = 0; kw < Kw; kw++) {
                        int iw = ow * stride - pad + kw;
                        if (iw < 0 || iw >= W) continue;
                        const int8_t* a = inb + ((size_t)ih * W + iw) * Cin;
                        const int8_t* ww = wp + (((size_t)co * Kh + kh) * Kw + kw) * Cin;
                        int32_t t = 0;
                        for (int ci = 0; ci < Cin; ci++) t += (int32_t)a[ci] * (int32_t)ww[ci];
                        s += t;
                    }
                }
                out[co] = s;
            }
        }
    }
    free(wp);
}

/* value before requantisation; kernels/int8_epilogue.c:53-76 */
static inline float epilogue_fp(int32_t acc, float in_scale, float ws, const float* bias, int co,
                                const int8_t* add_row, float add_scale_eff,
                                const float* slope, int mode)
{
    float t = mul_rn((float)acc, in_scale);
    if (mode == FFO_CONTRACT) {
        if (bias) t = fmaf(t, ws, bias[co]); else t = mul_rn(t, ws);
        if (add_row) t = fmaf((float)add_row[co], add_scale_eff, t);
    } else {
        t = mul_rn(t, ws);
        if (bias) t = add_rn(t, bias[co]);
        if (add_row) t = add_rn(t, mul_rn((float)add_row[co], add_scale_eff));
    }
    if (slope && t < 0.0f) t = mul_rn(t, slope[co]);
    return t;
}

/* kernels/int8_epilogue.c:25-112 (AVX2 branch; every Cout is a multiple of 8) */
void ffo_epilogue(const int32_t* acc, int n_pos, int Cout, float in_scale,
                  const float* w_scale, const float* bias, const float* slope,
                  const int8_t* add_src, float add_scale, const float* add_scale_pc,
                  const float* inv_out_pc, float out_scale, int mode, int8_t* out)
{
    float inv_scalar = 1.0f / (out_scale + 1e-9f);
    #pragma omp parallel for schedule(static)
    for (int p = 0; p < n_pos; p++) {
        const int32_t* ar = acc + (size_t)p * Cout;
        const int8_t* addr = add_src ? add_src + (size_t)p * Cout : NULL;
        int8_t* o = out + (size_t)p * Cout;
        for (int co = 0; co < Cout; co++) {
            float as = add_scale_pc ? add_scale_pc[co] : add_scale;
            float t = epilogue_fp(ar[co], in_scale, w_scale[co], bias, co, addr, as, slope, mode);
            float inv = inv_out_pc ? inv_out_pc[co] : inv_scalar;
            o[co] = requant_half_away(mul_rn(t, inv));
        }
    }
}

/* kernels/int8_epilogue.c:253-318 -- explicit fmadd in the source, so identical
 * in both build modes. */
static inline float bn_fp(int8_t a, float is, const float* bn_scale, const float* bn_offset,
                          const float* slope, int c)
{
    float t = mul_rn((float)a, is);
    if (bn_scale) t = fmaf(t, bn_scale[c], bn_offset[c]);
    if (slope && t < 0.0f) t = mul_rn(t, slope[c]);
    return t;
}

void ffo_bn_requant(const int8_t* in, float in_scale, const float* in_scale_pc,
                    const float* bn_scale, const float* bn_offset, const float* slope,
                    const float* inv_out_pc, float out_scale, int8_t* out, int n_pos, int C)
{
    float inv_scalar = 1.0f / (out_scale + 1e-9f);
    #pragma omp parallel for schedule(static)
    for (int p = 0; p < n_pos; p++) {
        const int8_t* ir = in + (size_t)p * C;
        int8_t* o = out + (size_t)p * C;
        for (int c = 0; c < C; c++) {
            float is = in_scale_pc ? in_scale_pc[c] : in_scale;
            float t = bn_fp(ir[c], is, bn_scale, bn_offset, slope, c);
            float inv = inv_out_pc ? inv_out_pc[c] : inv_scalar;
            o[c] = requant_half_away(mul_rn(t, inv));
        }
    }
}

/* kernels/int8_epilogue.c:231-247 */
void ffo_quantize_input_pc(const float* in, int n_pos, int C, const float* inv_pc, int8_t* out)
{
    for (long p = 0; p < n_pos; p++)
        for (int c = 0; c < C; c++)
            out[p * C + c] = quant_lrint(mul_rn(in[p * C + c], inv_pc[c]));
}

/* kernels/int8_epilogue.c:218-227 */
void ffo_quantize_input(const float* in, int n, float scale, int8_t* out)
{
    float inv = 1.0f / (scale + 1e-9f);
    for (long i = 0; i < n; i++) out[i] = quant_lrint(mul_rn(in[i], inv));
}

/* kernels/gemm_int8_matvec.c:33-81 -- exact signed dot, then
 * out = bias + (float)dot * A_scale * W_scale. */
void ffo_fc(const int8_t* a, const int8_t* w, const float* w_scale, const float* bias,
            float a_scale, int N, int K, int mode, float* out)
{
    #pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        const int8_t* wr = w + (size_t)n * K;
        int32_t s = 0;
        for (int k = 0; k < K; k++) s += (int32_t)a[k] * (int32_t)wr[k];
        float t = mul_rn((float)s, a_scale);
        if (mode == FFO_CONTRACT) out[n] = fmaf(t, w_scale[n], bias[n]);
        else out[n] = add_rn(bias[n], mul_rn(t, w_scale[n]));
    }
}

/* go/fastface/fastface.go:157-168 -- float64 accumulation, 0 when a norm is 0 */
float ffo_cos_sim(const float* a, const float* b, int n)
{
    double dot = 0, na = 0, nb = 0;
    for (int i = 0; i < n; i++) {
        dot += (double)a[i] * (double)b[i];
        na += (double)a[i] * (double)a[i];
        nb += (double)b[i] * (double)b[i];
    }
    if (na == 0 || nb == 0) return 0.0f;
    return (float)(dot / (sqrt(na) * sqrt(nb)));
}

/* ------------------------------------------------------------------ */
/* file formats                                                        */
/* ------------------------------------------------------------------ */

static uint8_t* read_file(const char* path, size_t* size)
{
    FILE* f = fopen(path, "rb");
    if (!f) return NULL;
    fseek(f, 0, SEEK_END);
    long n = ftell(f);
    fseek(f, 0, SEEK_SET);
    uint8_t* buf = (uint8_t*)malloc((size_t)n + 1);
    if (!buf || fread(buf, 1, (size_t)n, f) != (size_t)n) { fclose(f); free(buf); return NULL; }
    fclose(f);
    *size = (size_t)n;
    return buf;
}

static float* dup_f32(const uint8_t* p, size_t n)
{
    float* r = (float*)malloc((n ? n : 1) * sizeof(float));
    memcpy(r, p, n * sizeof(float));
    return r;
}

/* kernels/ffw2_loader.c:71-159 -- FFW4 only (FFW2/FFW3 need a runtime in_scale
 * the FFW4 path fixes to 1.0; they are rejected here). */
static int parse_ffw4(const uint8_t* d, size_t size, ffo_model* m)
{
    if (size < 8 || memcmp(d, "FFW4", 4) != 0) return -3;
    uint32_t n_ops; memcpy(&n_ops, d + 4, 4);
    if (n_ops == 0 || n_ops > 100000) return -3;
    m->n_ops = (int)n_ops;
    m->ops = (ffo_op*)calloc(n_ops, sizeof(ffo_op));
    const uint8_t* p = d + 8;
    const uint8_t* end = d + size;
#define NEED(nbytes) do { if ((size_t)(end - p) < (size_t)(nbytes)) return -5; } while (0)
    for (uint32_t i = 0; i < n_ops; i++) {
        ffo_op* op = &m->ops[i];
        NEED(1);
        op->type = *p++;
        switch (op->type) {
        case FFO_OP_CONV: {
            uint16_t v[6]; NEED(12); memcpy(v, p, 12); p += 12;
            op->Cin = v[0]; op->Cout = v[1]; op->Kh = v[2]; op->Kw = v[3];
            op->stride = v[4]; op->pad = v[5];
            size_t we = (size_t)op->Cout * op->Cin * op->Kh * op->Kw;
            NEED(we + 8u * op->Cout);
            op->w = (int8_t*)malloc(we); memcpy(op->w, p, we); p += we;
            op->scale = dup_f32(p, op->Cout); p += 4u * op->Cout;
            op->bias  = dup_f32(p, op->Cout); p += 4u * op->Cout;
            break;
        }
        case FFO_OP_BN: {
            uint16_t n; NEED(2); memcpy(&n, p, 2); p += 2; op->n = n;
            NEED(8u * n);
            op->bn_scale = dup_f32(p, n); p += 4u * n;
            op->bn_offset = dup_f32(p, n); p += 4u * n;
            break;
        }
        case FFO_OP_PRELU: {
            uint16_t n; NEED(2); memcpy(&n, p, 2); p += 2; op->n = n;
            NEED(4u * n);
            op->slope = dup_f32(p, n); p += 4u * n;
            break;
        }
        case FFO_OP_ADD: case FFO_OP_FLATTEN: case FFO_OP_SAVE_ID: case FFO_OP_BLOCK_START:
            break;
        case FFO_OP_GEMM: {
            NEED(8); memcpy(&op->N, p, 4); memcpy(&op->K, p + 4, 4); p += 8;
            size_t we = (size_t)op->N * op->K;
            NEED(we + 8u * op->N);
            op->w = (int8_t*)malloc(we); memcpy(op->w, p, we); p += we;
            op->scale = dup_f32(p, op->N); p += 4u * op->N;
            op->bias  = dup_f32(p, op->N); p += 4u * op->N;
            break;
        }
        default:
            return -4;
        }
    }
#undef NEED
    return 0;
}

/* libfastface.c:193-204 */
static int parse_opsc(const char* path, ffo_model* m)
{
    size_t size; uint8_t* d = read_file(path, &size);
    if (!d) return -1;
    if (size < 12 || memcmp(d, "OPSC", 4) != 0) { free(d); return -2; }
    uint32_t n; memcpy(&n, d + 4, 4);
    if ((int)n != m->n_ops || size < 12 + 4u * (size_t)n) { free(d); return -3; }
    memcpy(&m->input_scale, d + 8, 4);
    m->scales = dup_f32(d + 12, n);
    free(d);
    return 0;
}

/* libfastface.c:133-191 -- inv = 1.0f / (scale + 1e-9f) in fp32 */
static int parse_opsc2(const char* path, ffo_model* m)
{
    size_t size; uint8_t* d = read_file(path, &size);
    if (!d) return -1;
    if (size < 13 || memcmp(d, "OPSC2", 5) != 0) { free(d); return -2; }
    uint32_t n_ops, n_in; memcpy(&n_ops, d + 5, 4); memcpy(&n_in, d + 9, 4);
    if ((int)n_ops != m->n_ops) { free(d); return -3; }
    const uint8_t* p = d + 13; const uint8_t* end = d + size;
    if ((size_t)(end - p) < 4u * (size_t)n_in) { free(d); return -5; }
    m->n_in = (int)n_in;
    m->in_pc_scale = dup_f32(p, n_in); p += 4u * n_in;
    m->in_pc_inv = (float*)malloc((n_in ? n_in : 1) * sizeof(float));
    for (uint32_t c = 0; c < n_in; c++) m->in_pc_inv[c] = 1.0f / (m->in_pc_scale[c] + 1e-9f);
    m->pc_len = (uint32_t*)calloc(n_ops, sizeof(uint32_t));
    m->pc_scale = (float**)calloc(n_ops, sizeof(float*));
    m->pc_inv = (float**)calloc(n_ops, sizeof(float*));
    for (uint32_t i = 0; i < n_ops; i++) {
        if ((size_t)(end - p) < 4) { free(d); return -5; }
        uint32_t nch; memcpy(&nch, p, 4); p += 4;
        m->pc_len[i] = nch;
        if (nch == 0) continue;
        if (nch > 32768 || (size_t)(end - p) < 4u * (size_t)nch) { free(d); return -4; }
        m->pc_scale[i] = dup_f32(p, nch); p += 4u * nch;
        m->pc_inv[i] = (float*)malloc(nch * sizeof(float));
        for (uint32_t c = 0; c < nch; c++) m->pc_inv[i][c] = 1.0f / (m->pc_scale[i][c] + 1e-9f);
    }
    m->has_pc = 1;
    free(d);
    return 0;
}

void ffo_free(ffo_model* m)
{
    if (!m) return;
    for (int i = 0; i < m->n_ops; i++) {
        ffo_op* op = &m->ops[i];
        free(op->w); free(op->scale); free(op->bias);
        free(op->bn_scale); free(op->bn_offset); free(op->slope);
        if (m->pc_scale) free(m->pc_scale[i]);
        if (m->pc_inv) free(m->pc_inv[i]);
    }
    free(m->ops); free(m->scales); free(m->in_pc_scale); free(m->in_pc_inv);
    free(m->pc_len); free(m->pc_scale); free(m->pc_inv);
    free(m);
}

/* libfastface.c:231-240 */
ffo_model* ffo_load(const char* ffw4_path, const char* opsc_path, const char* opsc2_path)
{
    ffo_model* m = (ffo_model*)calloc(1, sizeof(ffo_model));
    size_t size; uint8_t* d = read_file(ffw4_path, &size);
    if (!d) { free(m); return NULL; }
    int rc = parse_ffw4(d, size, m);
    free(d);
    if (rc != 0) { ffo_free(m); return NULL; }
    if (parse_opsc(opsc_path, m) != 0) { ffo_free(m); return NULL; }
    if (opsc2_path) parse_opsc2(opsc2_path, m);   /* missing or bad file: per-tensor fallback */
    return m;
}

int ffo_n_ops(const ffo_model* m) { return m->n_ops; }
int ffo_has_per_channel(const ffo_model* m) { return m->has_pc; }

/* ------------------------------------------------------------------ */
/* driver: libfastface.c:243-269 (shape pre-pass) and :312-470 (op loop);
 * batched form arcface_forward_int8_batched.c:339-516                  */
/* ------------------------------------------------------------------ */

typedef struct { int C, H, W; } shape3;

static int cmp_f32(const void* a, const void* b)
{
    float x = *(const float*)a, y = *(const float*)b;
    return (x > y) - (x < y);
}

/* per-channel percentile(|t|)/127 over [n_pos][C]; installs scale + inverse for op idx */
static void calib_set(ffo_model* m, int idx, const float* t, long n_pos, int C, double pct)
{
    float* sc = (float*)malloc(C * sizeof(float));
    float* inv = (float*)malloc(C * sizeof(float));
    #pragma omp parallel for schedule(dynamic)
    for (int c = 0; c < C; c++) {
        float* col = (float*)malloc(n_pos * sizeof(float));
        for (long p = 0; p < n_pos; p++) col[p] = fabsf(t[p * C + c]);
        qsort(col, n_pos, sizeof(float), cmp_f32);
        long k = (long)ceil(pct * 0.01 * (double)n_pos) - 1;
        if (k < 0) k = 0;
        if (k >= n_pos) k = n_pos - 1;
        float v = col[k];
        if (!(v > 1e-6f)) v = col[n_pos - 1];
        if (!(v > 1e-6f)) v = 1e-6f;
        sc[c] = v / 127.0f;
        inv[c] = 1.0f / (sc[c] + 1e-9f);
        free(col);
    }
    free(m->pc_scale[idx]); free(m->pc_inv[idx]);
    m->pc_scale[idx] = sc; m->pc_inv[idx] = inv; m->pc_len[idx] = (uint32_t)C;
    float mx = 0; for (int c = 0; c < C; c++) if (sc[c] > mx) mx = sc[c];
    m->scales[idx] = mx;
}

static int forward_impl(ffo_model* m, const float* in, int B, float* out, int mode,
                        ffo_trace_cb cb, void* user, double calib_pct)
{
    const int n_ops = m->n_ops;
    uint8_t* is_shortcut = (uint8_t*)calloc(n_ops, 1);
    shape3* in_shape = (shape3*)calloc(n_ops, sizeof(shape3));
    shape3* shape_after = (shape3*)calloc(n_ops, sizeof(shape3));
    for (int i = 1; i < n_ops; i++)
        if (m->ops[i].type == FFO_OP_CONV && m->ops[i - 1].type == FFO_OP_SAVE_ID) is_shortcut[i] = 1;
    shape3 cur = {3, 112, 112}, block_in = cur;
    size_t max_act = (size_t)3 * 112 * 112;
    for (int i = 0; i < n_ops; i++) {
        ffo_op* op = &m->ops[i];
        shape3 s = is_shortcut[i] ? block_in : cur;
        in_shape[i] = s;
        if (op->type == FFO_OP_CONV) {
            if (op->Cin != s.C || op->stride < 1) { free(is_shortcut); free(in_shape); free(shape_after); return -2; }
            cur.H = (s.H + 2 * op->pad - op->Kh) / op->stride + 1;
            cur.W = (s.W + 2 * op->pad - op->Kw) / op->stride + 1;
            cur.C = op->Cout;
            size_t n = (size_t)cur.C * cur.H * cur.W;
            if (n > max_act) max_act = n;
        } else if (op->type == FFO_OP_GEMM) { cur.C = (int)op->N; cur.H = 1; cur.W = 1; }
        shape_after[i] = cur;
        if (op->type == FFO_OP_BLOCK_START) block_in = cur;
    }

    size_t act_bytes = (size_t)B * max_act + 64;
    int8_t* act_a = (int8_t*)malloc(act_bytes);
    int8_t* act_b = (int8_t*)malloc(act_bytes);
    int8_t* block_buf = (int8_t*)malloc(act_bytes);
    int32_t* conv_out = (int32_t*)malloc(act_bytes * sizeof(int32_t));
    float* fp_tmp = calib_pct > 0 ? (float*)malloc(act_bytes * sizeof(float)) : NULL;
    int8_t* id_slots[24]; float id_scales[24] = {0}; const float* id_scales_pc[24] = {0};
    for (int k = 0; k < 24; k++) id_slots[k] = (int8_t*)malloc(act_bytes);

    const int NIN = 3 * 112 * 112;
    if (m->has_pc && m->in_pc_inv && m->n_in >= 3)
        ffo_quantize_input_pc(in, B * 112 * 112, 3, m->in_pc_inv, act_a);
    else
        ffo_quantize_input(in, B * NIN, m->input_scale, act_a);
    if (cb) cb(user, -1, FFO_TRACE_INPUT_I8, act_a, (size_t)B * NIN);

    int8_t* A = act_a; int8_t* BB = act_b;
    float A_scale = m->input_scale;
    const float* A_scale_pc = m->has_pc ? m->in_pc_scale : NULL;
    int save_idx = 0, add_idx = 0;
    float block_scale = m->input_scale; (void)block_scale;
    memcpy(block_buf, act_a, (size_t)B * NIN);

    for (int i = 0; i < n_ops; i++) {
        ffo_op* op = &m->ops[i];
        shape3 si = in_shape[i], so = shape_after[i];
        int HWi = si.H * si.W, HWo = so.H * so.W;
        float next_scale = m->scales[i];
        if (next_scale <= 0) next_scale = A_scale;
        switch (op->type) {
        case FFO_OP_CONV: {
            const int8_t* conv_in = is_shortcut[i] ? block_buf : A;
            const float conv_in_scale = 1.0f;   /* FFW4: libfastface.c:362 */
            const float* fuse_prelu = NULL; const int8_t* add_src = NULL;
            float add_scale = 0.0f; const float* add_scale_pc = NULL;
            float eff_next = next_scale; int skip = 0, add_fused = 0, eff_idx = i;
            if (i + 1 < n_ops && m->ops[i + 1].type == FFO_OP_PRELU) {
                fuse_prelu = m->ops[i + 1].slope;
                eff_next = m->scales[i + 1]; if (eff_next <= 0) eff_next = next_scale;
                skip = 1; eff_idx = i + 1;
            } else if (i + 1 < n_ops && m->ops[i + 1].type == FFO_OP_ADD) {
                add_src = id_slots[add_idx % 24]; add_scale = id_scales[add_idx % 24];
                add_scale_pc = id_scales_pc[add_idx % 24];
                eff_next = m->scales[i + 1]; if (eff_next <= 0) eff_next = next_scale;
                skip = 1; add_fused = 1; eff_idx = i + 1;
            }
            ffo_conv_i32(conv_in, B, si.C, si.H, si.W, op->w, op->Cout, op->Kh, op->Kw,
                         op->stride, op->pad, so.H, so.W, conv_out);
            long n_pos = (long)B * HWo;
            if (cb) cb(user, i, FFO_TRACE_CONV_ACC, conv_out, (size_t)n_pos * op->Cout);
            if (calib_pct > 0) {
                #pragma omp parallel for schedule(static)
                for (long p = 0; p < n_pos; p++)
                    for (int co = 0; co < op->Cout; co++) {
                        float as = add_scale_pc ? add_scale_pc[co] : add_scale;
                        fp_tmp[p * op->Cout + co] = epilogue_fp(conv_out[p * op->Cout + co], conv_in_scale,
                            op->scale[co], op->bias, co, add_src ? add_src + p * op->Cout : NULL, as,
                            fuse_prelu, mode);
                    }
                calib_set(m, eff_idx, fp_tmp, n_pos, op->Cout, calib_pct);
                eff_next = m->scales[eff_idx];
            }
            const float* pc_inv = (m->has_pc && m->pc_inv) ? m->pc_inv[eff_idx] : NULL;
            ffo_epilogue(conv_out, (int)n_pos, op->Cout, conv_in_scale, op->scale, op->bias,
                         fuse_prelu, add_src, add_scale, add_scale_pc, pc_inv, eff_next, mode, BB);
            if (cb) cb(user, i, FFO_TRACE_CONV_OUT, BB, (size_t)n_pos * op->Cout);
            { int8_t* t = A; A = BB; BB = t; }
            A_scale = eff_next;
            if (m->has_pc && m->pc_scale && m->pc_scale[eff_idx]) A_scale_pc = m->pc_scale[eff_idx];
            if (skip) i++;
            if (add_fused) add_idx++;
            break;
        }
        case FFO_OP_BN: {
            long n_pos = (long)B * HWi;
            const float* in_pc = (m->has_pc && A_scale_pc) ? A_scale_pc : NULL;
            if (calib_pct > 0) {
                #pragma omp parallel for schedule(static)
                for (long p = 0; p < n_pos; p++)
                    for (int c = 0; c < si.C; c++)
                        fp_tmp[p * si.C + c] = bn_fp(A[p * si.C + c], in_pc ? in_pc[c] : A_scale,
                                                     op->bn_scale, op->bn_offset, NULL, c);
                calib_set(m, i, fp_tmp, n_pos, si.C, calib_pct);
                next_scale = m->scales[i];
            }
            const float* inv = (m->has_pc && m->pc_inv && m->pc_inv[i] && m->pc_len[i] == (uint32_t)si.C)
                               ? m->pc_inv[i] : NULL;
            ffo_bn_requant(A, A_scale, in_pc, op->bn_scale, op->bn_offset, NULL, inv, next_scale,
                           A, (int)n_pos, si.C);
            if (cb) cb(user, i, FFO_TRACE_BN_OUT, A, (size_t)n_pos * si.C);
            A_scale = next_scale;
            if (m->has_pc && m->pc_scale && m->pc_scale[i]) A_scale_pc = m->pc_scale[i];
            break;
        }
        case FFO_OP_PRELU: {   /* standalone PReLU: never reached with the IR-ResNet op order */
            long n_pos = (long)B * HWi;
            const float* in_pc = (m->has_pc && A_scale_pc) ? A_scale_pc : NULL;
            const float* inv = (m->has_pc && m->pc_inv) ? m->pc_inv[i] : NULL;
            ffo_bn_requant(A, A_scale, in_pc, NULL, NULL, op->slope, inv, next_scale, A, (int)n_pos, si.C);
            A_scale = next_scale;
            if (m->has_pc && m->pc_scale && m->pc_scale[i]) A_scale_pc = m->pc_scale[i];
            break;
        }
        case FFO_OP_BLOCK_START:
            memcpy(block_buf, A, (size_t)B * si.C * HWi);
            block_scale = A_scale;
            break;
        case FFO_OP_ADD:
            /* unfused ADD never occurs in the FFW4 op order (every ADD follows a CONV) */
            for (int k = 0; k < 24; k++) free(id_slots[k]);
            free(act_a); free(act_b); free(block_buf); free(conv_out); free(fp_tmp);
            free(is_shortcut); free(in_shape); free(shape_after);
            return -3;
        case FFO_OP_SAVE_ID:
            memcpy(id_slots[save_idx % 24], A, (size_t)B * si.C * HWi);
            id_scales[save_idx % 24] = A_scale;
            id_scales_pc[save_idx % 24] = A_scale_pc;
            save_idx++;
            break;
        case FFO_OP_FLATTEN: {   /* libfastface.c:456-464 NHWC -> CHW per face */
            size_t face = (size_t)si.C * HWi;
            for (int b = 0; b < B; b++)
                for (int c = 0; c < si.C; c++)
                    for (int hw = 0; hw < HWi; hw++)
                        BB[b * face + (size_t)c * HWi + hw] = A[b * face + (size_t)hw * si.C + c];
            { int8_t* t = A; A = BB; BB = t; }
            break;
        }
        case FFO_OP_GEMM:
            for (int b = 0; b < B; b++)
                ffo_fc(A + (size_t)b * op->K, op->w, op->scale, op->bias, 1.0f,
                       (int)op->N, (int)op->K, mode, out + (size_t)b * op->N);
            if (cb) cb(user, i, FFO_TRACE_FC_OUT, out, (size_t)B * op->N);
            break;
        }
    }
    for (int k = 0; k < 24; k++) free(id_slots[k]);
    free(act_a); free(act_b); free(block_buf); free(conv_out); free(fp_tmp);
    free(is_shortcut); free(in_shape); free(shape_after);
    return 0;
}

int ffo_forward(const ffo_model* m, const float* in, int B, float* out,
                int mode, ffo_trace_cb cb, void* user)
{
    if (!m || !in || !out || B < 1) return -1;
    return forward_impl((ffo_model*)m, in, B, out, mode, cb, user, 0.0);
}

int ffo_calibrate(const char* ffw4_path, const float* in, int B, double percentile,
                  const char* opsc_out, const char* opsc2_out)
{
    ffo_model* m = (ffo_model*)calloc(1, sizeof(ffo_model));
    size_t size; uint8_t* d = read_file(ffw4_path, &size);
    if (!d) { free(m); return -1; }
    int rc = parse_ffw4(d, size, m);
    free(d);
    if (rc != 0) { ffo_free(m); return rc; }
    int n = m->n_ops;
    m->input_scale = 1.0f / 127.0f;
    m->scales = (float*)calloc(n, sizeof(float));
    m->has_pc = 1; m->n_in = 3;
    m->in_pc_scale = (float*)malloc(3 * sizeof(float));
    m->in_pc_inv = (float*)malloc(3 * sizeof(float));
    for (int c = 0; c < 3; c++) { m->in_pc_scale[c] = 1.0f / 127.0f; m->in_pc_inv[c] = 1.0f / (m->in_pc_scale[c] + 1e-9f); }
    m->pc_len = (uint32_t*)calloc(n, sizeof(uint32_t));
    m->pc_scale = (float**)calloc(n, sizeof(float*));
    m->pc_inv = (float**)calloc(n, sizeof(float*));
    float* out = (float*)malloc((size_t)B * 512 * sizeof(float));
    rc = forward_impl(m, in, B, out, FFO_CONTRACT, NULL, NULL, percentile);
    free(out);
    if (rc == 0) {
        FILE* f = fopen(opsc_out, "wb");
        uint32_t un = (uint32_t)n;
        fwrite("OPSC", 1, 4, f); fwrite(&un, 4, 1, f); fwrite(&m->input_scale, 4, 1, f);
        fwrite(m->scales, 4, n, f); fclose(f);
        f = fopen(opsc2_out, "wb");
        uint32_t nin = 3;
        fwrite("OPSC2", 1, 5, f); fwrite(&un, 4, 1, f); fwrite(&nin, 4, 1, f);
        fwrite(m->in_pc_scale, 4, 3, f);
        for (int i = 0; i < n; i++) {
            fwrite(&m->pc_len[i], 4, 1, f);
            if (m->pc_len[i]) fwrite(m->pc_scale[i], 4, m->pc_len[i], f);
        }
        fclose(f);
    }
    ffo_free(m);
    return rc;
}
