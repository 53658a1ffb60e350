/* lf_gpu_sm100.c -- LFortran's GPU offload ABI over the sm_100a driver shim.
 *
 * Same contract as the reference's src/runtime/lf_gpu.c (over nv_rt) and
 * src/runtime/lf_gpu_hsa.c (over bc_runtime): buffers are copied in when they are
 * set and copied back after the launch, scalars travel by value, the launch hands
 * the driver one pointer per parameter, and every failure is fatal.
 *
 * What differs from the reference by design: kernels are heap objects rather than
 * a static pool of eight; the copies in and back are enqueued on the device's
 * stream together with the kernel, so one launch costs a single wait instead of
 * one per buffer; and a kernel that no file provides is looked up in the image
 * embedded in the library. */
#define _POSIX_C_SOURCE 200809L
#include "lf_gpu.h"
#include "booth_sm100.h"

#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define LF_MAX_ARGS 32      /* the parameter cap of the reference (src/runtime/lf_gpu.c:18) */
#define LF_SCAL_MAX 16      /* widest by-value scalar (src/runtime/lf_gpu.c:20) */
#define LF_PATH_MAX 512

struct lfortran_gpu_ctx {
    sm100_dev_t *dev;
    lfortran_gpu_kernel *kernels;      /* live kernels, newest first */
    int live;
};

typedef struct {
    void       *host;                  /* array to copy back into */
    sm100_ptr_t dptr;
    size_t      size;
    uint8_t     scal[LF_SCAL_MAX];
    int         is_buf, used;
} lf_arg_t;

struct lfortran_gpu_kernel {
    sm100_kern_t kern;
    lf_arg_t     args[LF_MAX_ARGS];
    int          nargs;
    lfortran_gpu_ctx    *ctx;
    lfortran_gpu_kernel *next;
};

static lfortran_gpu_ctx g_ctx;

static void lf_die(const lfortran_gpu_ctx *ctx, const char *what, long rc)
{
    const char *why = (ctx != NULL && ctx->dev != NULL) ? sm100_rt_errs(ctx->dev) : "";
    fprintf(stderr, "lf_gpu_sm100: %s failed (rc=%ld)%s%s\n", what, rc, why[0] ? ": " : "", why);
    exit(1);
}

static int lf_readable(const char *path)
{
    FILE *f = fopen(path, "rb");
    if (f == NULL) return 0;
    fclose(f);
    return 1;
}

lfortran_gpu_ctx *lfortran_gpu_init(void)
{
    int rc;
    if (g_ctx.live) return &g_ctx;
    rc = sm100_rt_init(&g_ctx.dev, -1);
    if (rc != SM100_OK) lf_die(NULL, "sm100_rt_init", rc);
    g_ctx.kernels = NULL;
    g_ctx.live = 1;
    return &g_ctx;
}

void lfortran_gpu_shutdown(lfortran_gpu_ctx *ctx)
{
    if (ctx == NULL || !ctx->live) return;
    while (ctx->kernels != NULL) lfortran_gpu_release_kernel(ctx->kernels);
    sm100_rt_shut(ctx->dev);
    ctx->dev = NULL;
    ctx->live = 0;
}

lfortran_gpu_kernel *lfortran_gpu_load_kernel(lfortran_gpu_ctx *ctx, const char *source,
                                              const char *entry_point)
{
    char path[LF_PATH_MAX];
    const char *env, *file = NULL;
    lfortran_gpu_kernel *k;
    int rc;

    if (ctx == NULL || !ctx->live || entry_point == NULL) lf_die(ctx, "load_kernel args", 0);
    if (source != NULL && source[0] != '\0') {
        file = source;
    } else if ((env = getenv("BOOTH_CUBIN")) != NULL && env[0] != '\0') {
        file = env;
    } else {
        (void)snprintf(path, sizeof path, "%s.cubin", entry_point);
        if (lf_readable(path)) file = path;
    }
    k = (lfortran_gpu_kernel *)calloc(1, sizeof *k);
    if (k == NULL) lf_die(ctx, "kernel object", (long)sizeof *k);
    rc = file != NULL ? sm100_rt_load(ctx->dev, file, entry_point, &k->kern)
                      : sm100_rt_load_builtin(ctx->dev, entry_point, &k->kern);
    if (rc != SM100_OK) {
        fprintf(stderr, "lf_gpu_sm100: could not load '%s' from %s\n", entry_point,
                file != NULL ? file : "the built-in image");
        lf_die(ctx, "sm100_rt_load", rc);
    }
    k->ctx = ctx;
    k->next = ctx->kernels;
    ctx->kernels = k;
    return k;
}

void lfortran_gpu_release_kernel(lfortran_gpu_kernel *k)
{
    lfortran_gpu_kernel **link;
    int j;

    if (k == NULL || k->ctx == NULL) return;
    for (link = &k->ctx->kernels; *link != NULL && *link != k; link = &(*link)->next) { }
    if (*link == NULL) return;                         /* not one of ours, or released before */
    *link = k->next;
    (void)sm100_rt_sync(k->ctx->dev);
    for (j = 0; j < k->nargs; j++)
        if (k->args[j].is_buf && k->args[j].dptr != 0) sm100_rt_free(k->ctx->dev, k->args[j].dptr);
    sm100_rt_unload(k->ctx->dev, &k->kern);
    k->ctx = NULL;
    free(k);
}

void lfortran_gpu_set_buffer_arg(lfortran_gpu_kernel *k, int idx, void *ptr, size_t size)
{
    lf_arg_t *a;
    int rc;

    if (k == NULL || k->ctx == NULL || idx < 0 || idx >= LF_MAX_ARGS) return;
    a = &k->args[idx];
    if (a->is_buf && a->dptr != 0 && a->size != size) {        /* keep an allocation of the same size */
        (void)sm100_rt_sync(k->ctx->dev);
        sm100_rt_free(k->ctx->dev, a->dptr);
        a->dptr = 0;
    }
    if (!a->is_buf) a->dptr = 0;
    if (a->dptr == 0) {
        a->dptr = sm100_rt_alloc(k->ctx->dev, size ? size : 1);
        if (a->dptr == 0) lf_die(k->ctx, "sm100_rt_alloc", (long)size);
    }
    if (size != 0) {
        rc = sm100_rt_h2d_async(k->ctx->dev, a->dptr, ptr, size);
        if (rc != SM100_OK) lf_die(k->ctx, "sm100_rt_h2d", rc);
    }
    a->host = ptr;
    a->size = size;
    a->is_buf = 1;
    a->used = 1;
    if (idx >= k->nargs) k->nargs = idx + 1;
}

void lfortran_gpu_set_scalar_arg(lfortran_gpu_kernel *k, int idx, const void *val, size_t size)
{
    lf_arg_t *a;

    if (k == NULL || k->ctx == NULL || idx < 0 || idx >= LF_MAX_ARGS) return;
    if (val == NULL || size == 0 || size > LF_SCAL_MAX) lf_die(k->ctx, "scalar arg too wide", (long)size);
    a = &k->args[idx];
    if (a->is_buf && a->dptr != 0) {
        (void)sm100_rt_sync(k->ctx->dev);
        sm100_rt_free(k->ctx->dev, a->dptr);
        a->dptr = 0;
    }
    memset(a->scal, 0, sizeof a->scal);
    memcpy(a->scal, val, size);
    a->size = size;
    a->is_buf = 0;
    a->used = 1;
    if (idx >= k->nargs) k->nargs = idx + 1;
}

void lfortran_gpu_launch(lfortran_gpu_ctx *ctx, lfortran_gpu_kernel *k, int grid[3], int block[3])
{
    void *argv[LF_MAX_ARGS];
    int j, rc;

    if (ctx == NULL || !ctx->live || k == NULL || k->ctx != ctx) return;
    if (grid == NULL || block == NULL) lf_die(ctx, "launch dims", 0);
    if (grid[0] < 1 || grid[1] < 1 || grid[2] < 1 || block[0] < 1 || block[1] < 1 || block[2] < 1)
        lf_die(ctx, "launch dims non-positive", grid[0]);
    for (j = 0; j < k->nargs; j++) {
        if (!k->args[j].used) lf_die(ctx, "argument gap", j);
        argv[j] = k->args[j].is_buf ? (void *)&k->args[j].dptr : (void *)k->args[j].scal;
    }
    rc = sm100_rt_launch(ctx->dev, &k->kern, (uint32_t)grid[0], (uint32_t)grid[1], (uint32_t)grid[2],
                         (uint32_t)block[0], (uint32_t)block[1], (uint32_t)block[2], 0u, argv);
    if (rc != SM100_OK) lf_die(ctx, "sm100_rt_launch", rc);
    /* The copies back queue up behind the kernel on the same stream. */
    for (j = 0; j < k->nargs; j++) {
        if (!k->args[j].is_buf || k->args[j].dptr == 0 || k->args[j].size == 0) continue;
        rc = sm100_rt_d2h_async(ctx->dev, k->args[j].host, k->args[j].dptr, k->args[j].size);
        if (rc != SM100_OK) lf_die(ctx, "sm100_rt_d2h", rc);
    }
    rc = sm100_rt_sync(ctx->dev);
    if (rc != SM100_OK) lf_die(ctx, "sm100_rt_sync", rc);
}

void lfortran_gpu_sync(lfortran_gpu_ctx *ctx)
{
    if (ctx == NULL || !ctx->live) return;
    (void)sm100_rt_sync(ctx->dev);
}
