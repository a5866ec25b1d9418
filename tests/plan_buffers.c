/* Test helper: builds the static launch list for a model with the library's own host sources and prints, per launch,
 * the layer shape and the activation buffers it reads and writes.  Compiled by tests/test_host_cpu.py (gcc, no GPU). */
#include <stdio.h>
#include <string.h>
#include "ff_model.h"
#include "ff_plan.h"

int main(int argc, char** argv)
{
    if (argc < 4) { fprintf(stderr, "usage: plan_buffers model.ffw4 op_scales.bin op_scales_v2.bin\n"); return 2; }
    ff_model m; ff_plan p;
    memset(&m, 0, sizeof m);
    if (ff_model_load_ffw4(&m, argv[1]) != 0 || ff_model_load_opsc(&m, argv[2]) != 0 || ff_model_load_opsc2(&m, argv[3]) != 0) {
        fprintf(stderr, "load failed\n");
        return 1;
    }
    if (ff_plan_build(&p, &m) != 0) { fprintf(stderr, "plan failed\n"); return 1; }
    for (int i = 0; i < p.n_layers; i++) {
        const ffcu_layer* l = &p.layers[i];
        printf("L %d kind %d cin %d cout %d k %d stride %d h %d src %d dst %d res %d bn2 %d\n", i, l->kind, l->Cin, l->Cout,
               l->Kh, l->stride, l->H, l->src_buf, l->dst_buf, l->res_buf, l->bn2_dst_buf);
    }
    printf("N_BUFS %d\n", p.n_bufs);
    return 0;
}
