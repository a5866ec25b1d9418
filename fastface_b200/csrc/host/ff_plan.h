/* ff_plan.h -- static layer plan derived from the FFW4 op list (C99 host side). */
#ifndef FF_PLAN_H
#define FF_PLAN_H

#include "ff_model.h"
#include "ff_cuda.h"

typedef struct {
    int n_layers;
    ffcu_layer* layers;      /* arrays inside are owned by the plan (see pool) */
    int n_bufs;              /* activation buffers the plan needs */
    size_t bytes_per_face;   /* largest int8 activation tensor of one face */
    void** pool;             /* every allocation the layers point into */
    int pool_n, pool_cap;
} ff_plan;

/* Walks the op list the way the reference's driver loop does
 * (libfastface.c:243-269 shape pre-pass, :349-466 op loop), resolving at build
 * time which scale each kernel call would receive, and emits one ffcu_layer per
 * kernel launch.  0 on success. */
int  ff_plan_build(ff_plan* p, const ff_model* m);
void ff_plan_free(ff_plan* p);

#endif
