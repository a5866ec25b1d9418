/* fastface_cli.c -- command-line driver with the reference CLI's interface.
 *
 * Mirrors arcface_forward_int8_batched.c:206-573 (and arcface_forward_int8.c for
 * --batch 1) so scripts and the reference's Python / Go wrappers can drive the
 * GPU engine unchanged:
 *
 *   fastface_int8_b200 <weights.ffw4> [--batch B] [--in faces.f32 --out emb.f32]
 *                      [--server] [--devices 0,1,..]
 *
 *   --in/--out : read B faces (B*37632 f32), write B embeddings (B*512 f32), exit.
 *   --server   : loop: read B*37632 f32 from stdin, write B*512 f32 to stdout
 *                (the wrappers' protocol, fastface.py:96-117); a partial batch aborts
 *                with exit code 4 like the reference (:543-546).
 *   otherwise  : the reference's bench loop, 5 trials x 30 iterations on srand(42)
 *                synthetic faces, same report lines (:555-573).
 * models/op_scales.bin (+ op_scales_v2.bin / $OPSC2_PATH) are looked up relative to the
 * working directory exactly as the reference does.
 */
#define _POSIX_C_SOURCE 200809L
#include "fastface.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

static double now_s(void)
{
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + (double)ts.tv_nsec * 1e-9;
}

int main(int argc, char** argv)
{
    const char* path = (argc > 1) ? argv[1] : "models/w600k_r50_ffw4.bin";
    const char *in_path = NULL, *out_path = NULL, *devices = NULL;
    int B = 8, server = 0;
    for (int i = 2; i < argc; i++) {
        if (!strcmp(argv[i], "--in") && i + 1 < argc) in_path = argv[++i];
        else if (!strcmp(argv[i], "--out") && i + 1 < argc) out_path = argv[++i];
        else if (!strcmp(argv[i], "--batch") && i + 1 < argc) B = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--devices") && i + 1 < argc) devices = argv[++i];
        else if (!strcmp(argv[i], "--server")) server = 1;
        else if (!strcmp(argv[i], "--threads") && i + 1 < argc) i++;       /* accepted, meaningless here */
    }
    { const char* e = getenv("BATCH"); if (e) B = atoi(e); }
    if (B < 1) B = 1;
    FILE* info = server ? stderr : stdout;
    fprintf(info, "Batch size B=%d\n", B);

    int ids[16], n_dev = 0;
    for (const char* s = devices; s && *s && n_dev < 16;) {
        char* end; long v = strtol(s, &end, 10);
        if (end == s) break;
        ids[n_dev++] = (int)v;
        s = (*end == ',') ? end + 1 : end;
    }
    if (n_dev == 0) { ids[0] = 0; n_dev = 1; }
    FastFace* ff = fastface_create_ex(path, ids, n_dev, B);
    if (!ff) { fprintf(stderr, "load fail: %s\n", fastface_last_error()); return 1; }
    fprintf(info, "FastFace INT8 (B200)  devices=%d\n", n_dev);

    const size_t n_in = (size_t)B * FASTFACE_INPUT_N, n_out = (size_t)B * FASTFACE_OUTPUT_N;
    float* in = (float*)malloc(n_in * sizeof(float));
    float* out = (float*)malloc(n_out * sizeof(float));
    if (!in || !out) return 1;

    if (in_path && out_path) {
        FILE* f = fopen(in_path, "rb");
        if (!f) return 2;
        size_t got = fread(in, sizeof(float), n_in, f);
        fclose(f);
        if (got != n_in) { fprintf(stderr, "short input (%zu/%zu floats)\n", got, n_in); return 2; }
        if (fastface_embed_batch(ff, in, B, out) != 0) { fprintf(stderr, "embed failed: %s\n", fastface_last_error()); return 3; }
        fprintf(stderr, "final_emb[0..4] = %g %g %g %g %g\n", out[0], out[1], out[2], out[3], out[4]);
        f = fopen(out_path, "wb");
        if (!f) return 2;
        fwrite(out, sizeof(float), n_out, f);
        fclose(f);
        fastface_destroy(ff);
        return 0;
    }

    if (server) {
        fprintf(stderr, "Batched server mode ready. Awaiting %zu-float batches (B=%d x 3x112x112).\n", n_in, B);
        for (;;) {
            size_t got = fread(in, sizeof(float), n_in, stdin);
            if (got == 0) break;
            if (got != n_in) { fprintf(stderr, "partial batch read (%zu/%zu floats) -- abort\n", got, n_in); return 4; }
            if (fastface_embed_batch(ff, in, B, out) != 0) { fprintf(stderr, "embed failed: %s\n", fastface_last_error()); return 3; }
            if (fwrite(out, sizeof(float), n_out, stdout) != n_out) { fprintf(stderr, "partial write\n"); return 5; }
            fflush(stdout);
        }
        fastface_destroy(ff);
        return 0;
    }

    srand(42);
    for (size_t i = 0; i < n_in; i++) in[i] = ((rand() % 2001) - 1000) / 1000.0f;
    if (fastface_embed_batch(ff, in, B, out) != 0) { fprintf(stderr, "embed failed: %s\n", fastface_last_error()); return 3; }
    fprintf(stderr, "First pass OK\nfinal_emb[0..4] = %g %g %g %g %g\n", out[0], out[1], out[2], out[3], out[4]);
    const int ITER = 30;
    double best = 1e9;
    for (int trial = 0; trial < 5; trial++) {
        double t0 = now_s();
        for (int it = 0; it < ITER; it++) fastface_embed_batch(ff, in, B, out);
        double dt = (now_s() - t0) / ITER;
        if (dt < best) best = dt;
        printf("Trial %d: %.3f ms/batch = %.4f ms/face  (%.1f face/s)\n", trial, dt * 1000, dt * 1000 / B, B / dt);
    }
    printf("\n========== INT8 BATCHED END-TO-END RESULT (B=%d) ==========\n", B);
    printf("Best: %.3f ms/batch = %.4f ms/face  (%.1f face/s)\n", best * 1000, best * 1000 / B, B / best);
    printf("==========================================================\n");
    fastface_destroy(ff);
    free(in); free(out);
    return 0;
}
