/* ff_plan.c -- turn the FFW4 op list into a static list of kernel launches.
 *
 * The reference interprets the op list on every call (libfastface.c:349-466):
 * it looks one op ahead to fuse PRELU / ADD into the conv epilogue, swaps two
 * activation buffers, copies snapshots on BLOCK_START / SAVE_ID and carries the
 * "current scale" (scalar and per-channel) along.  None of that depends on the
 * input, so it is done once here:
 *   - every scale argument a kernel call would receive becomes a per-channel
 *     array (a scalar fallback is broadcast, which is arithmetically identical);
 *   - BLOCK_START / SAVE_ID copies become buffer aliases with reference counts;
 *   - FLATTEN (NHWC -> CHW, libfastface.c:456-464) is folded into a permutation
 *     of the FC weights' K axis, which leaves the int32 dot products unchanged.
 */
#define _POSIX_C_SOURCE 200809L
#include "ff_plan.h"

#include <limits.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#define FF_MAX_BUFS 8
#define FF_ID_SLOTS 24            /* ring size of the reference's id_slots (libfastface.c:226) */

static void* pool_alloc(ff_plan* p, size_t bytes)
{
    void* q = NULL;
    if (posix_memalign(&q, 64, bytes ? ((bytes + 63) & ~(size_t)63) : 64) != 0) return NULL;
    if (p->pool_n == p->pool_cap) {
        p->pool_cap = p->pool_cap ? p->pool_cap * 2 : 256;
        p->pool = (void**)realloc(p->pool, (size_t)p->pool_cap * sizeof(void*));
    }
    p->pool[p->pool_n++] = q;
    return q;
}

/* per-channel array from either a per-channel source or a broadcast scalar */
static const float* per_channel(ff_plan* p, const float* pc, float scalar, int C)
{
    float* a = (float*)pool_alloc(p, (size_t)C * sizeof(float));
    for (int c = 0; c < C; c++) a[c] = pc ? pc[c] : scalar;
    return a;
}

static const float* copy_f32(ff_plan* p, const float* src, int n)
{
    float* a = (float*)pool_alloc(p, (size_t)n * sizeof(float));
    memcpy(a, src, (size_t)n * sizeof(float));
    return a;
}

/* kernels/int8_epilogue.c:272-303 evaluated for all 256 int8 inputs of each channel.  Built
 * with -ffp-contract=off: every line below is one IEEE operation, as in the CUDA kernels. */
void ff_bn_lut_build(const float* in_scale, const float* bn_scale, const float* bn_offset,
                     const float* inv_out, int C, int8_t* lut)
{
    for (int c = 0; c < C; c++)
        for (int ub = 0; ub < 256; ub++) {
            const int q = (int)(int8_t)(uint8_t)ub;
            float t = (float)q * in_scale[c];
            t = fmaf(t, bn_scale[c], bn_offset[c]);
            const float qq = t * inv_out[c];
            uint32_t bits; memcpy(&bits, &qq, 4);
            const uint32_t hb = 0x3f000000u | (bits & 0x80000000u);
            float half; memcpy(&half, &hb, 4);
            const float r = qq + half;
            int i;
            if (!(fabsf(r) < 2147483648.0f)) i = INT_MIN;      /* cvttps2dq on overflow / NaN */
            else i = (int)r;
            if (i < -128) i = -128;
            if (i > 127) i = 127;
            lut[c * 256 + ub] = (int8_t)i;
        }
}

typedef struct { int C, H, W; } shape3;

typedef struct {
    int ref[FF_MAX_BUFS];
    int used;
} bufset;

static int buf_get(bufset* b)
{
    for (int i = 0; i < FF_MAX_BUFS; i++)
        if (b->ref[i] == 0) { b->ref[i] = 1; if (i + 1 > b->used) b->used = i + 1; return i; }
    return -1;
}
/* a free buffer other than x, y and z (the operands of the launch that will also write it) */
static int buf_get_not(bufset* b, int x, int y, int z)
{
    for (int i = 0; i < FF_MAX_BUFS; i++)
        if (b->ref[i] == 0 && i != x && i != y && i != z) { b->ref[i] = 1; if (i + 1 > b->used) b->used = i + 1; return i; }
    return -1;
}

/* [conv 3x3 stride 2][conv 1x1 stride 2 on the block's input, ADD of the former's output fused] may go out as ONE
 * launch (conv_tc_sc.cu) that reads the first conv's input while it writes the second conv's outputs: when `sc` is such
 * a second conv (the layer before it produced its residual), the buffer the first conv reads, else -1.  That buffer is
 * free by the time the second conv is planned, and must not be handed to either of its outputs. */
static int pair_input_buf(const ff_plan* p, const ffcu_layer* sc)
{
    if (sc < p->layers + 1 || sc->kind != FFCU_CONV || sc->res_buf < 0) return -1;
    const ffcu_layer* m = sc - 1;
    return (m->kind == FFCU_CONV && m->dst_buf == sc->res_buf) ? m->src_buf : -1;
}
static void buf_hold(bufset* b, int i) { if (i >= 0) b->ref[i]++; }
static void buf_drop(bufset* b, int i) { if (i >= 0 && b->ref[i] > 0) b->ref[i]--; }

static ffcu_layer* push_layer(ff_plan* p, int* cap)
{
    if (p->n_layers == *cap) {
        *cap = *cap ? *cap * 2 : 128;
        p->layers = (ffcu_layer*)realloc(p->layers, (size_t)*cap * sizeof(ffcu_layer));
    }
    ffcu_layer* l = &p->layers[p->n_layers++];
    memset(l, 0, sizeof *l);
    l->src_buf = l->dst_buf = l->res_buf = -1;
    l->bn2_dst_buf = -1; l->bn2_op_index = -1;
    return l;
}

int ff_plan_build(ff_plan* p, const ff_model* m)
{
    memset(p, 0, sizeof *p);
    int cap = 0;
    bufset bs; memset(&bs, 0, sizeof bs);
    const int n_ops = m->n_ops;
    const char* fb = getenv("FF_FUSE_BN");
    const int fuse_bn = !(fb && fb[0] == '0');

    /* scale state carried by the reference loop */
    float A_scale = m->input_scale;
    const float* A_pc = m->has_pc ? m->in_pc_scale : NULL;
    int A_pc_len = m->has_pc ? m->n_in : 0;
    float id_scale[FF_ID_SLOTS] = {0};
    const float* id_pc[FF_ID_SLOTS] = {0};
    int id_pc_len[FF_ID_SLOTS] = {0};
    int id_buf[FF_ID_SLOTS];
    for (int k = 0; k < FF_ID_SLOTS; k++) id_buf[k] = -1;
    int save_idx = 0, add_idx = 0;

    shape3 cur = {3, 112, 112}, block_in = cur;
    int flat_C = 0, flat_HW = 0;
    size_t max_face = (size_t)4 * 112 * 112;

    /* input quantisation (libfastface.c:335-338); stored with a zero 4th channel */
    int cur_buf = buf_get(&bs);
    {
        ffcu_layer* l = push_layer(p, &cap);
        l->kind = FFCU_QUANT; l->op_index = -1; l->dst_buf = cur_buf;
        l->Cin = 3; l->Cout = 4; l->H = l->Ho = 112; l->W = l->Wo = 112;
        if (m->has_pc && m->in_pc_inv) {
            if (m->n_in < 3) { ff_set_error("OPSC2 has %d input channels, need 3", m->n_in); return -2; }
            l->inv_out = per_channel(p, m->in_pc_inv, 0.0f, 3);
        } else {
            l->inv_out = per_channel(p, NULL, 1.0f / (m->input_scale + 1e-9f), 3);
        }
    }
    int block_buf = cur_buf; buf_hold(&bs, block_buf);

    for (int i = 0; i < n_ops; i++) {
        const ff_op* op = &m->ops[i];
        float next_scale = m->scales[i];
        if (next_scale <= 0) next_scale = A_scale;
        switch (op->type) {
        case FF_OP_CONV: {
            int shortcut = (i > 0 && m->ops[i - 1].type == FF_OP_SAVE_ID);
            shape3 si = shortcut ? block_in : cur;
            if (op->Cin != si.C || op->stride < 1 || op->Kh < 1 || op->Kw < 1) {
                ff_set_error("op %d: conv expects %d input channels, tensor has %d", i, op->Cin, si.C);
                return -2;
            }
            int Ho = (si.H + 2 * op->pad - op->Kh) / op->stride + 1;
            int Wo = (si.W + 2 * op->pad - op->Kw) / op->stride + 1;
            int Cout = op->Cout;
            const float* slope = NULL;
            int add_fused = 0, eff_idx = i, skip = 0;
            float eff_next = next_scale;
            if (i + 1 < n_ops && m->ops[i + 1].type == FF_OP_PRELU) {
                if (m->ops[i + 1].n != Cout) { ff_set_error("op %d: PReLU size mismatch", i + 1); return -2; }
                slope = m->ops[i + 1].slope;
                eff_next = m->scales[i + 1]; if (eff_next <= 0) eff_next = next_scale;
                skip = 1; eff_idx = i + 1;
            } else if (i + 1 < n_ops && m->ops[i + 1].type == FF_OP_ADD) {
                add_fused = 1;
                eff_next = m->scales[i + 1]; if (eff_next <= 0) eff_next = next_scale;
                skip = 1; eff_idx = i + 1;
            }
            ffcu_layer* l = push_layer(p, &cap);
            l->kind = FFCU_CONV; l->op_index = i;
            l->src_buf = shortcut ? block_buf : cur_buf;
            l->Cin = op->Cin; l->Cout = Cout; l->Kh = op->Kh; l->Kw = op->Kw;
            l->stride = op->stride; l->pad = op->pad;
            l->H = si.H; l->W = si.W; l->Ho = Ho; l->Wo = Wo;
            /* weights: [Cout][Cin][Kh][Kw] -> [Cout][Kh][Kw][Cin_pad]; K order (kh,kw,ci)
             * as in pack_conv_weight_nhwc (kernels/conv2d_nhwc.c:79-100) */
            int Cp = (op->Cin + 3) & ~3;
            l->Cin_pad = Cp;
            l->w_bytes = (size_t)Cout * op->Kh * op->Kw * Cp;
            int8_t* w = (int8_t*)pool_alloc(p, l->w_bytes);
            memset(w, 0, l->w_bytes);
            for (int co = 0; co < Cout; co++)
                for (int ci = 0; ci < op->Cin; ci++)
                    for (int kh = 0; kh < op->Kh; kh++)
                        for (int kw = 0; kw < op->Kw; kw++)
                            w[(((size_t)co * op->Kh + kh) * op->Kw + kw) * Cp + ci] =
                                op->w[(((size_t)co * op->Cin + ci) * op->Kh + kh) * op->Kw + kw];
            l->w = w;
            l->w_scale = copy_f32(p, op->scale, Cout);     /* in_scale is 1.0f for FFW4 (libfastface.c:362) */
            l->bias = copy_f32(p, op->bias, Cout);
            if (slope) l->slope = copy_f32(p, slope, Cout);
            if (add_fused) {
                int s = add_idx % FF_ID_SLOTS;
                if (id_buf[s] < 0) { ff_set_error("op %d: ADD without a saved identity", i + 1); return -2; }
                l->res_buf = id_buf[s];
                const float* rpc = m->has_pc ? id_pc[s] : NULL;
                if (rpc && id_pc_len[s] != Cout) { ff_set_error("op %d: identity scale length %d != %d", i, id_pc_len[s], Cout); return -2; }
                l->res_scale = per_channel(p, rpc, id_scale[s], Cout);
            }
            const float* inv_pc = m->has_pc ? m->pc_inv[eff_idx] : NULL;
            if (inv_pc && (int)m->pc_len[eff_idx] != Cout) {
                ff_set_error("op %d: OPSC2 has %u channels, conv has %d", eff_idx, m->pc_len[eff_idx], Cout);
                return -2;
            }
            l->inv_out = per_channel(p, inv_pc, 1.0f / (eff_next + 1e-9f), Cout);
            int dst = buf_get_not(&bs, pair_input_buf(p, l), -1, -1);
            if (dst < 0) { ff_set_error("activation buffer pool exhausted"); return -2; }
            l->dst_buf = dst;
            if (add_fused) { int s = add_idx % FF_ID_SLOTS; buf_drop(&bs, id_buf[s]); id_buf[s] = -1; add_idx++; }
            buf_drop(&bs, cur_buf); cur_buf = dst;
            cur.C = Cout; cur.H = Ho; cur.W = Wo;
            size_t n = (size_t)Cout * Ho * Wo; if (n > max_face) max_face = n;
            A_scale = eff_next;
            if (m->has_pc && m->pc_scale[eff_idx]) { A_pc = m->pc_scale[eff_idx]; A_pc_len = (int)m->pc_len[eff_idx]; }
            if (skip) i++;
            break;
        }
        case FF_OP_BN: {
            int C = cur.C;
            if (op->n != C) { ff_set_error("op %d: BN size %d != %d channels", i, op->n, C); return -2; }
            const float* in_pc = (m->has_pc && A_pc) ? A_pc : NULL;
            if (in_pc && A_pc_len < C) { ff_set_error("op %d: input scale length %d < %d", i, A_pc_len, C); return -2; }
            const float* inv_pc = (m->has_pc && m->pc_inv[i] && (int)m->pc_len[i] == C) ? m->pc_inv[i] : NULL;
            ffcu_layer* prev = p->n_layers ? &p->layers[p->n_layers - 1] : NULL;
            const int can_fuse = fuse_bn && prev && prev->kind == FFCU_CONV && prev->dst_buf == cur_buf
                                 && prev->bn2_dst_buf < 0 && prev->Cout == C;
            /* a fused second output must not land in a buffer the same launch still reads */
            int dst = can_fuse ? buf_get_not(&bs, prev->src_buf, prev->res_buf, pair_input_buf(p, prev)) : buf_get(&bs);
            if (dst < 0) { ff_set_error("activation buffer pool exhausted"); return -2; }
            /* The BN input is always the tensor the previous launch wrote; BN is a pure
             * per-element function of that int8 value, so it rides along as a second output of
             * the producing conv's epilogue (saves one read of the tensor and one launch). */
            if (can_fuse) {
                prev->bn2_dst_buf = dst; prev->bn2_op_index = i;
                prev->bn2_in_scale = per_channel(p, in_pc, A_scale, C);
                prev->bn2_scale = copy_f32(p, op->bn_scale, C);
                prev->bn2_offset = copy_f32(p, op->bn_offset, C);
                prev->bn2_inv_out = per_channel(p, inv_pc, 1.0f / (next_scale + 1e-9f), C);
                int8_t* lut = (int8_t*)pool_alloc(p, (size_t)C * 256);
                ff_bn_lut_build(prev->bn2_in_scale, prev->bn2_scale, prev->bn2_offset, prev->bn2_inv_out, C, lut);
                prev->bn2_lut = lut;
            } else {
                ffcu_layer* l = push_layer(p, &cap);
                l->kind = FFCU_BN; l->op_index = i;
                l->src_buf = cur_buf;
                l->Cin = l->Cout = C; l->H = l->Ho = cur.H; l->W = l->Wo = cur.W;
                l->in_scale = per_channel(p, in_pc, A_scale, C);
                l->bn_scale = copy_f32(p, op->bn_scale, C);
                l->bn_offset = copy_f32(p, op->bn_offset, C);
                l->inv_out = per_channel(p, inv_pc, 1.0f / (next_scale + 1e-9f), C);
                l->dst_buf = dst;
            }
            buf_drop(&bs, cur_buf); cur_buf = dst;
            A_scale = next_scale;
            if (m->has_pc && m->pc_scale[i]) { A_pc = m->pc_scale[i]; A_pc_len = (int)m->pc_len[i]; }
            break;
        }
        case FF_OP_BLOCK_START:
            buf_drop(&bs, block_buf); block_buf = cur_buf; buf_hold(&bs, block_buf);
            block_in = cur;
            break;
        case FF_OP_SAVE_ID: {
            int s = save_idx % FF_ID_SLOTS;
            buf_drop(&bs, id_buf[s]);
            id_buf[s] = cur_buf; buf_hold(&bs, cur_buf);
            id_scale[s] = A_scale; id_pc[s] = A_pc; id_pc_len[s] = A_pc_len;
            save_idx++;
            break;
        }
        case FF_OP_FLATTEN:
            flat_C = cur.C; flat_HW = cur.H * cur.W;
            break;
        case FF_OP_GEMM: {
            int C = flat_C ? flat_C : cur.C * cur.H * cur.W, HW = flat_C ? flat_HW : 1;
            if ((size_t)op->K != (size_t)C * HW) { ff_set_error("op %d: GEMM K=%u but tensor has %d values", i, op->K, C * HW); return -2; }
            ffcu_layer* l = push_layer(p, &cap);
            l->kind = FFCU_FC; l->op_index = i; l->src_buf = cur_buf;
            l->Cin = (int)op->K; l->Cin_pad = (int)op->K; l->Cout = (int)op->N;
            l->Kh = l->Kw = 1; l->stride = 1; l->H = l->W = l->Ho = l->Wo = 1;
            l->w_bytes = (size_t)op->N * op->K;
            int8_t* w = (int8_t*)pool_alloc(p, l->w_bytes);
            for (uint32_t n = 0; n < op->N; n++)
                for (int c = 0; c < C; c++)
                    for (int hw = 0; hw < HW; hw++)
                        w[(size_t)n * op->K + (size_t)hw * C + c] = op->w[(size_t)n * op->K + (size_t)c * HW + hw];
            l->w = w;
            l->w_scale = copy_f32(p, op->scale, (int)op->N);  /* A_scale is 1.0f for FFW4 (libfastface.c:449) */
            l->bias = copy_f32(p, op->bias, (int)op->N);
            cur.C = (int)op->N; cur.H = cur.W = 1;
            break;
        }
        case FF_OP_PRELU:
        case FF_OP_ADD:
            /* Every PRELU / ADD of the IR-ResNet export directly follows a CONV and is fused
             * above; the reference's standalone forms are dead code for FFW4. */
            ff_set_error("op %d: standalone %s is not supported", i, op->type == FF_OP_ADD ? "ADD" : "PRELU");
            return -2;
        default:
            ff_set_error("op %d: unknown type %d", i, op->type);
            return -2;
        }
    }
    if (p->n_layers == 0 || p->layers[p->n_layers - 1].kind != FFCU_FC || p->layers[p->n_layers - 1].Cout != 512) {
        ff_set_error("model does not end in a 512-wide GEMM");
        return -2;
    }
    p->n_bufs = bs.used;
    p->bytes_per_face = max_face;
    return 0;
}

void ff_plan_free(ff_plan* p)
{
    if (!p) return;
    for (int i = 0; i < p->pool_n; i++) free(p->pool[i]);
    free(p->pool); free(p->layers);
    memset(p, 0, sizeof *p);
}
