/* ff_model.h -- in-memory form of the reference's model files (C99 host side). */
#ifndef FF_MODEL_H
#define FF_MODEL_H

#include <stddef.h>
#include <stdint.h>

enum {
    FF_OP_CONV = 1, FF_OP_BN = 2, FF_OP_PRELU = 3, FF_OP_ADD = 4,
    FF_OP_GEMM = 5, FF_OP_FLATTEN = 6, FF_OP_SAVE_ID = 7, FF_OP_BLOCK_START = 8
};

/* One FFW4 op.  Arrays are owned, aligned copies (the file stores them unaligned). */
typedef struct {
    int type;
    int Cin, Cout, Kh, Kw, stride, pad;   /* CONV */
    int8_t* w;                            /* CONV [Cout][Cin][Kh][Kw]; GEMM [N][K] */
    float* scale;                         /* CONV/GEMM per-output dequant scale */
    float* bias;                          /* CONV/GEMM */
    int n;                                /* BN / PRELU length */
    float* bn_scale;
    float* bn_offset;
    float* slope;
    uint32_t N, K;                        /* GEMM */
} ff_op;

typedef struct {
    int n_ops;
    ff_op* ops;
    /* OPSC: per-tensor scales, 0 means "inherit the current scale" */
    float input_scale;
    float* scales;
    /* OPSC2: per-channel scales and their fp32 inverses 1/(s + 1e-9f) */
    int has_pc;
    int n_in;
    float* in_pc_scale;
    float* in_pc_inv;
    uint32_t* pc_len;
    float** pc_scale;
    float** pc_inv;
} ff_model;

/* 0 on success; negative codes: -1 open/read, -3 bad magic or version, -4 bad op type,
 * -5 truncated file. */
int  ff_model_load_ffw4(ff_model* m, const char* path);
/* 0 on success; -1 open, -2 magic, -3 op-count mismatch or truncated. */
int  ff_model_load_opsc(ff_model* m, const char* path);
/* 0 on success; non-zero leaves the model on per-tensor scales (not an error). */
int  ff_model_load_opsc2(ff_model* m, const char* path);
void ff_model_free(ff_model* m);

void ff_set_error(const char* fmt, ...);

#endif
