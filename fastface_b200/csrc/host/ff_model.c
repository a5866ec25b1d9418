/* ff_model.c -- readers for FFW4 weights and OPSC / OPSC2 activation scales.
 *
 * Formats (little-endian, packed):
 *   FFW4  : reference kernels/ffw2_loader.c:3-12,94-157
 *   OPSC  : reference libfastface.c:193-204
 *   OPSC2 : reference libfastface.c:133-191
 * The reference maps the file and points into it; here everything is copied
 * into aligned arrays because the next stop is a device upload.
 */
#define _POSIX_C_SOURCE 200809L
#include "ff_model.h"

#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static _Thread_local char g_err[512];

void ff_set_error(const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}

const char* ff_host_error(void) { return g_err; }

/* ---- byte cursor ---------------------------------------------------- */

typedef struct { const uint8_t* p; const uint8_t* end; int bad; } cursor;

static void cur_take(cursor* c, void* dst, size_t n)
{
    if (c->bad || (size_t)(c->end - c->p) < n) { c->bad = 1; memset(dst, 0, n); return; }
    memcpy(dst, c->p, n);
    c->p += n;
}

static uint16_t cur_u16(cursor* c) { uint16_t v; cur_take(c, &v, 2); return v; }
static uint32_t cur_u32(cursor* c) { uint32_t v; cur_take(c, &v, 4); return v; }

static void* cur_array(cursor* c, size_t n_elems, size_t elem)
{
    size_t bytes = n_elems * elem;
    if (c->bad || (size_t)(c->end - c->p) < bytes) { c->bad = 1; return NULL; }
    void* dst = NULL;
    if (posix_memalign(&dst, 64, bytes ? ((bytes + 63) & ~(size_t)63) : 64) != 0) { c->bad = 1; return NULL; }
    memcpy(dst, c->p, bytes);
    c->p += bytes;
    return dst;
}

static uint8_t* slurp(const char* path, size_t* size)
{
    FILE* f = fopen(path, "rb");
    if (!f) return NULL;
    if (fseek(f, 0, SEEK_END) != 0) { fclose(f); return NULL; }
    long n = ftell(f);
    if (n < 0) { fclose(f); return NULL; }
    rewind(f);
    uint8_t* buf = (uint8_t*)malloc((size_t)n + 1);
    if (!buf) { fclose(f); return NULL; }
    size_t got = fread(buf, 1, (size_t)n, f);
    fclose(f);
    if (got != (size_t)n) { free(buf); return NULL; }
    *size = (size_t)n;
    return buf;
}

/* ---- FFW4 ------------------------------------------------------------ */

int ff_model_load_ffw4(ff_model* m, const char* path)
{
    memset(m, 0, sizeof *m);
    size_t size = 0;
    uint8_t* data = slurp(path, &size);
    if (!data) { ff_set_error("cannot read %s", path); return -1; }
    if (size < 8 || memcmp(data, "FFW", 3) != 0) { free(data); ff_set_error("bad magic in %s", path); return -3; }
    if (data[3] != '4') {
        /* FFW2/FFW3 carry a run-time activation scale per conv (libfastface.c:361-362);
         * only the folded FFW4 form is supported. */
        free(data); ff_set_error("%s: only FFW4 is supported (found FFW%c)", path, data[3]); return -3;
    }
    cursor c = { data + 4, data + size, 0 };
    uint32_t n_ops = cur_u32(&c);
    if (n_ops == 0 || n_ops > (1u << 20)) { free(data); ff_set_error("implausible op count %u", n_ops); return -3; }
    m->n_ops = (int)n_ops;
    m->ops = (ff_op*)calloc(n_ops, sizeof(ff_op));
    int rc = 0;
    for (uint32_t i = 0; i < n_ops && !c.bad; i++) {
        ff_op* op = &m->ops[i];
        uint8_t t = 0; cur_take(&c, &t, 1);
        op->type = t;
        if (t == FF_OP_CONV) {
            op->Cin = cur_u16(&c); op->Cout = cur_u16(&c); op->Kh = cur_u16(&c);
            op->Kw = cur_u16(&c); op->stride = cur_u16(&c); op->pad = cur_u16(&c);
            op->w = (int8_t*)cur_array(&c, (size_t)op->Cout * op->Cin * op->Kh * op->Kw, 1);
            op->scale = (float*)cur_array(&c, op->Cout, 4);
            op->bias = (float*)cur_array(&c, op->Cout, 4);
        } else if (t == FF_OP_BN) {
            op->n = cur_u16(&c);
            op->bn_scale = (float*)cur_array(&c, op->n, 4);
            op->bn_offset = (float*)cur_array(&c, op->n, 4);
        } else if (t == FF_OP_PRELU) {
            op->n = cur_u16(&c);
            op->slope = (float*)cur_array(&c, op->n, 4);
        } else if (t == FF_OP_GEMM) {
            op->N = cur_u32(&c); op->K = cur_u32(&c);
            op->w = (int8_t*)cur_array(&c, (size_t)op->N * op->K, 1);
            op->scale = (float*)cur_array(&c, op->N, 4);
            op->bias = (float*)cur_array(&c, op->N, 4);
        } else if (t == FF_OP_ADD || t == FF_OP_FLATTEN || t == FF_OP_SAVE_ID || t == FF_OP_BLOCK_START) {
            /* markers: no payload */
        } else {
            ff_set_error("bad op type %d at op %u", (int)t, i);
            rc = -4;
            break;
        }
    }
    if (rc == 0 && c.bad) { ff_set_error("%s is truncated", path); rc = -5; }
    free(data);
    if (rc != 0) ff_model_free(m);
    return rc;
}

/* ---- OPSC ------------------------------------------------------------ */

int ff_model_load_opsc(ff_model* m, const char* path)
{
    size_t size = 0;
    uint8_t* data = slurp(path, &size);
    if (!data) { ff_set_error("open %s fail", path); return -1; }
    int rc = 0;
    if (size < 12 || memcmp(data, "OPSC", 4) != 0) rc = -2;
    if (rc == 0) {
        cursor c = { data + 4, data + size, 0 };
        uint32_t n = cur_u32(&c);
        cur_take(&c, &m->input_scale, 4);
        if ((int)n != m->n_ops) { ff_set_error("op_scales count mismatch: %u vs %d ops", n, m->n_ops); rc = -3; }
        else {
            m->scales = (float*)cur_array(&c, n, 4);
            if (c.bad) { ff_set_error("%s is truncated", path); rc = -3; }
        }
    } else ff_set_error("%s: not an OPSC file", path);
    free(data);
    return rc;
}

/* ---- OPSC2 ----------------------------------------------------------- */

static void free_pc(ff_model* m)
{
    if (m->pc_scale) for (int i = 0; i < m->n_ops; i++) free(m->pc_scale[i]);
    if (m->pc_inv) for (int i = 0; i < m->n_ops; i++) free(m->pc_inv[i]);
    free(m->pc_scale); free(m->pc_inv); free(m->pc_len);
    free(m->in_pc_scale); free(m->in_pc_inv);
    m->pc_scale = m->pc_inv = NULL; m->pc_len = NULL;
    m->in_pc_scale = m->in_pc_inv = NULL;
    m->has_pc = 0; m->n_in = 0;
}

int ff_model_load_opsc2(ff_model* m, const char* path)
{
    size_t size = 0;
    uint8_t* data = slurp(path, &size);
    if (!data) return -1;
    if (size < 13 || memcmp(data, "OPSC2", 5) != 0) { free(data); return -2; }
    cursor c = { data + 5, data + size, 0 };
    uint32_t n_ops = cur_u32(&c);
    uint32_t n_in = cur_u32(&c);
    if ((int)n_ops != m->n_ops) {
        fprintf(stderr, "OPSC2 n_ops mismatch: %u vs expected %d\n", n_ops, m->n_ops);
        free(data);
        return -3;
    }
    int rc = 0;
    m->n_in = (int)n_in;
    m->in_pc_scale = (float*)cur_array(&c, n_in, 4);
    m->in_pc_inv = (float*)calloc(n_in ? n_in : 1, sizeof(float));
    m->pc_len = (uint32_t*)calloc(n_ops, sizeof(uint32_t));
    m->pc_scale = (float**)calloc(n_ops, sizeof(float*));
    m->pc_inv = (float**)calloc(n_ops, sizeof(float*));
    if (!c.bad)
        for (uint32_t k = 0; k < n_in; k++)
            m->in_pc_inv[k] = 1.0f / (m->in_pc_scale[k] + 1e-9f);   /* libfastface.c:150-152 */
    for (uint32_t i = 0; i < n_ops && !c.bad; i++) {
        uint32_t nch = cur_u32(&c);
        if (nch == 0) continue;
        if (nch > 32768) { rc = -4; break; }                          /* libfastface.c:177 */
        m->pc_len[i] = nch;
        m->pc_scale[i] = (float*)cur_array(&c, nch, 4);
        if (c.bad) break;
        m->pc_inv[i] = (float*)malloc(nch * sizeof(float));
        for (uint32_t k = 0; k < nch; k++)
            m->pc_inv[i][k] = 1.0f / (m->pc_scale[i][k] + 1e-9f);   /* libfastface.c:181-183 */
    }
    if (c.bad) rc = -5;
    free(data);
    if (rc != 0) { free_pc(m); return rc; }
    m->has_pc = 1;
    return 0;
}

void ff_model_free(ff_model* m)
{
    if (!m) return;
    free_pc(m);
    for (int i = 0; i < m->n_ops && m->ops; i++) {
        ff_op* op = &m->ops[i];
        free(op->w); free(op->scale); free(op->bias);
        free(op->bn_scale); free(op->bn_offset); free(op->slope);
    }
    free(m->ops); free(m->scales);
    memset(m, 0, sizeof *m);
}
