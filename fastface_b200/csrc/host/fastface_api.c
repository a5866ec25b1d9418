/* fastface_api.c -- the public C API (include/fastface.h) on top of the CUDA shim.
 *
 * Mirrors the reference's libfastface.c: fastface_create loads FFW4 + OPSC
 * (+ OPSC2), builds everything that does not depend on the input, and
 * fastface_embed runs one forward pass.  The op loop itself lives on the GPU
 * side as a static launch list (ff_plan.c, csrc/cuda/).
 *
 * Multi-GPU: faces are independent, so a context that owns several devices
 * splits a batch into contiguous chunks, one host thread per device, with no
 * exchange between devices.
 */
#define _POSIX_C_SOURCE 200809L
#include "fastface.h"
#include "ff_cuda.h"
#include "ff_model.h"
#include "ff_plan.h"

#include <math.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define FF_MAX_DEVICES 16

const char* ff_host_error(void);

struct FastFace {
    int n_dev;
    int max_batch;
    ffcu_ctx* dev[FF_MAX_DEVICES];
    int dev_id[FF_MAX_DEVICES];
    int n_ops;
};

static _Thread_local char g_api_err[512];

static void api_error(const char* msg) { snprintf(g_api_err, sizeof g_api_err, "%s", msg ? msg : ""); }

const char* fastface_last_error(void)
{
    if (g_api_err[0]) return g_api_err;
    const char* h = ff_host_error();
    if (h && h[0]) return h;
    return ffcu_last_error();
}

static int parse_device_list(const char* s, int* ids, int max)
{
    int n = 0;
    while (s && *s && n < max) {
        char* end = NULL;
        long v = strtol(s, &end, 10);
        if (end == s) break;
        ids[n++] = (int)v;
        s = (*end == ',') ? end + 1 : end;
    }
    return n;
}

FastFace* fastface_create_ex(const char* ffw4_path, const int* device_ids, int n_devices, int max_batch)
{
    g_api_err[0] = 0;
    if (!ffw4_path) { api_error("NULL path"); return NULL; }
    if (n_devices < 1 || n_devices > FF_MAX_DEVICES) { api_error("bad device count"); return NULL; }
    if (max_batch < 1) max_batch = 1;

    ff_model model;
    if (ff_model_load_ffw4(&model, ffw4_path) != 0) { fprintf(stderr, "fastface: %s\n", ff_host_error()); return NULL; }
    /* same file convention as libfastface.c:236-240 */
    if (ff_model_load_opsc(&model, "models/op_scales.bin") != 0) {
        fprintf(stderr, "fastface: %s\n", ff_host_error());
        ff_model_free(&model);
        return NULL;
    }
    const char* v2 = getenv("OPSC2_PATH");
    if (!v2) v2 = "models/op_scales_v2.bin";
    if (ff_model_load_opsc2(&model, v2) == 0) {
        size_t total = 0;
        for (int i = 0; i < model.n_ops; i++) total += model.pc_len[i];
        fprintf(stderr, "OPSC2: loaded per-channel scales (total floats=%zu, input_pc_ch=%d)\n", total, model.n_in);
    }

    ff_plan plan;
    if (ff_plan_build(&plan, &model) != 0) {
        fprintf(stderr, "fastface: %s\n", ff_host_error());
        ff_plan_free(&plan); ff_model_free(&model);
        return NULL;
    }

    int avail = ffcu_device_count();
    if (avail <= 0) {
        api_error("no CUDA device available (this library has no CPU path)");
        fprintf(stderr, "fastface: %s\n", g_api_err);
        ff_plan_free(&plan); ff_model_free(&model);
        return NULL;
    }

    FastFace* ff = (FastFace*)calloc(1, sizeof(FastFace));
    if (!ff) {
        api_error("out of memory");
        fprintf(stderr, "fastface: %s\n", g_api_err);
        ff_plan_free(&plan); ff_model_free(&model);
        return NULL;
    }
    ff->n_dev = n_devices; ff->max_batch = max_batch; ff->n_ops = model.n_ops;
    int mode = FF_EPILOGUE_CONTRACT;
    const char* em = getenv("FF_EPILOGUE");
    if (em && strcmp(em, "strict") == 0) mode = FF_EPILOGUE_STRICT;
    int ok = 1;
    for (int d = 0; d < n_devices && ok; d++) {
        int id = device_ids ? device_ids[d] : d;
        ff->dev_id[d] = id;
        if (id < 0 || id >= avail) { api_error("device ordinal out of range"); ok = 0; break; }
        ff->dev[d] = ffcu_create(id, max_batch, plan.n_bufs, plan.bytes_per_face);
        if (!ff->dev[d]) { ok = 0; break; }
        for (int k = 0; k < plan.n_layers && ok; k++)
            if (ffcu_add_layer(ff->dev[d], &plan.layers[k]) < 0) ok = 0;
        if (ok && ffcu_finalize(ff->dev[d]) != 0) ok = 0;
        if (ok) ffcu_set_mode(ff->dev[d], mode);
    }
    ff_plan_free(&plan);
    ff_model_free(&model);
    if (!ok) {
        fprintf(stderr, "fastface: %s\n", fastface_last_error());
        fastface_destroy(ff);
        return NULL;
    }
    return ff;
}

FastFace* fastface_create(const char* ffw4_path)
{
    int ids[FF_MAX_DEVICES];
    int n = parse_device_list(getenv("FASTFACE_DEVICES"), ids, FF_MAX_DEVICES);
    if (n == 0) { ids[0] = 0; n = 1; }
    int mb = 256;
    const char* e = getenv("FASTFACE_MAX_BATCH");
    if (e && atoi(e) > 0) mb = atoi(e);
    return fastface_create_ex(ffw4_path, ids, n, mb);
}

void fastface_destroy(FastFace* ff)
{
    if (!ff) return;
    for (int d = 0; d < ff->n_dev; d++) ffcu_destroy(ff->dev[d]);
    free(ff);
}

/* one device's share of a batch, in steps of max_batch */
typedef struct {
    ffcu_ctx* ctx; const float* in; float* out; int n; int max_batch; int rc;
    const uint8_t* in_u8;      /* non-NULL: 8-bit pixel input instead of `in` */
    char err[256];             /* the CUDA side's message, copied on the thread that ran the job */
} dev_job;

static void* dev_job_run(void* arg)
{
    dev_job* j = (dev_job*)arg;
    j->rc = 0;
    for (int done = 0; done < j->n; ) {
        int step = j->n - done < j->max_batch ? j->n - done : j->max_batch;
        int rc = j->in_u8
            ? ffcu_submit_u8(j->ctx, j->in_u8 + (size_t)done * FASTFACE_INPUT_N, step, j->out + (size_t)done * FASTFACE_OUTPUT_N)
            : ffcu_submit(j->ctx, j->in + (size_t)done * FASTFACE_INPUT_N, step, j->out + (size_t)done * FASTFACE_OUTPUT_N);
        if (rc != 0) { j->rc = rc; break; }
        done += step;
    }
    int rc = ffcu_wait(j->ctx);
    if (j->rc == 0) j->rc = rc;
    /* the CUDA side keeps its last message per thread: take it here, where it was set */
    j->err[0] = 0;
    if (j->rc != 0) snprintf(j->err, sizeof j->err, "%s", ffcu_last_error());
    return NULL;
}

int fastface_shard_plan(int n, int n_devices, int* starts, int* counts)
{
    if (n < 1 || n_devices < 1 || !starts || !counts) return 0;
    int per = (n + n_devices - 1) / n_devices, used = 0, start = 0;
    for (int d = 0; d < n_devices && start < n; d++) {
        int cnt = n - start < per ? n - start : per;
        starts[used] = start; counts[used] = cnt;
        start += cnt; used++;
    }
    return used;
}

static int embed_batch_any(FastFace* ff, const float* input_hwc, const uint8_t* pixels_hwc, int n, float* out_emb);

int fastface_embed_batch(FastFace* ff, const float* input_hwc, int n, float* out_emb)
{
    if (!ff || !input_hwc || !out_emb || n < 1) return -1;
    return embed_batch_any(ff, input_hwc, NULL, n, out_emb);
}

int fastface_embed_batch_u8(FastFace* ff, const uint8_t* pixels_hwc, int n, float* out_emb)
{
    if (!ff || !pixels_hwc || !out_emb || n < 1) return -1;
    return embed_batch_any(ff, NULL, pixels_hwc, n, out_emb);
}

static int embed_batch_any(FastFace* ff, const float* input_hwc, const uint8_t* pixels_hwc, int n, float* out_emb)
{
    g_api_err[0] = 0;
    dev_job jobs[FF_MAX_DEVICES];
    pthread_t th[FF_MAX_DEVICES];
    int starts[FF_MAX_DEVICES], counts[FF_MAX_DEVICES];
    int used = fastface_shard_plan(n, ff->n_dev, starts, counts);
    for (int d = 0; d < used; d++)
        jobs[d] = (dev_job){ ff->dev[d], input_hwc ? input_hwc + (size_t)starts[d] * FASTFACE_INPUT_N : NULL,
                             out_emb + (size_t)starts[d] * FASTFACE_OUTPUT_N, counts[d], ff->max_batch, 0,
                             pixels_hwc ? pixels_hwc + (size_t)starts[d] * FASTFACE_INPUT_N : NULL, {0} };
    if (used == 1) {
        dev_job_run(&jobs[0]);
    } else {
        int started[FF_MAX_DEVICES];
        for (int d = 0; d < used; d++) started[d] = pthread_create(&th[d], NULL, dev_job_run, &jobs[d]) == 0;
        for (int d = 0; d < used; d++) {
            if (started[d]) pthread_join(th[d], NULL);
            else dev_job_run(&jobs[d]);          /* no thread to be had: run this device's share here */
        }
    }
    for (int d = 0; d < used; d++)
        if (jobs[d].rc != 0) { api_error(jobs[d].err); return jobs[d].rc; }
    return 0;
}

int fastface_embed(FastFace* ff, const float* input_hwc, float* out_emb)
{
    if (!ff || !input_hwc || !out_emb) return -1;
    return fastface_embed_batch(ff, input_hwc, 1, out_emb);
}

float fastface_cos_sim(const float* a, const float* b)
{
    if (!a || !b) return 0.0f;
    double dot = 0.0, na = 0.0, nb = 0.0;
    for (int i = 0; i < FASTFACE_OUTPUT_N; i++) {
        double x = (double)a[i], y = (double)b[i];
        dot += x * y; na += x * x; nb += y * y;
    }
    if (na == 0.0 || nb == 0.0) return 0.0f;
    return (float)(dot / (sqrt(na) * sqrt(nb)));
}

int fastface_cos_sim_matrix(const FastFace* ff, const float* a, int n, const float* b, int m, float* out)
{
    if (!ff || !a || !b || !out || n < 1 || m < 1) return -1;
    return ffcu_cos_sim_matrix(ff->dev_id[0], a, n, b, m, out);
}

int fastface_set_epilogue_mode(FastFace* ff, int mode)
{
    if (!ff || (mode != FF_EPILOGUE_STRICT && mode != FF_EPILOGUE_CONTRACT)) return -1;
    for (int d = 0; d < ff->n_dev; d++)
        if (ffcu_set_mode(ff->dev[d], mode) != 0) return -2;
    return 0;
}

int fastface_trace_batch(FastFace* ff, const float* input_hwc, int n, float* out_emb,
                         fastface_trace_fn fn, void* user)
{
    if (!ff || !input_hwc || !out_emb || n < 1 || n > ff->max_batch) return -1;
    return ffcu_trace(ff->dev[0], input_hwc, n, out_emb, (ffcu_trace_fn)fn, user);
}

int fastface_bench_resident(FastFace* ff, const float* input_hwc, int n, int iters, float* ms)
{
    if (!ff || !input_hwc || !ms || n < 1 || n > ff->max_batch || iters < 1) return -1;
    return ffcu_bench_resident(ff->dev[0], input_hwc, n, iters, ms);
}

int fastface_launches_per_forward(const FastFace* ff)
{
    return ff ? ffcu_launches_per_forward(ff->dev[0]) : 0;
}

int fastface_layer_count(const FastFace* ff) { return ff ? ffcu_layer_count(ff->dev[0]) : 0; }

int fastface_layer_desc(const FastFace* ff, int k, int* desc12)
{
    if (!ff || !desc12) return -1;
    ffcu_layer l; int tc = 0;
    if (ffcu_layer_info(ff->dev[0], k, &l, &tc) != 0) return -1;
    int v[12] = { l.kind, l.op_index, l.Cin, l.Cout, l.Kh, l.Kw, l.stride, l.H, l.W, l.Ho, l.Wo, tc };
    memcpy(desc12, v, sizeof v);
    return 0;
}

int fastface_bench_layers(FastFace* ff, const float* input_hwc, int n, int iters, float* ms, int cap)
{
    if (!ff || !input_hwc || !ms || n < 1 || n > ff->max_batch || iters < 1) return -1;
    return ffcu_bench_layers(ff->dev[0], input_hwc, n, iters, ms, cap);
}
