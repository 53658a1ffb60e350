/* lf_offload.c -- the call sequence an LFortran-compiled `do concurrent` loop makes
 * through the eight-function offload ABI (include/lf_gpu.h), written out in C99.
 *
 * Three loops are offloaded the way the Fortran runtime would do it: host arrays are
 * handed over with set_buffer_arg, scalars with set_scalar_arg, the launch returns with
 * the results back in the same host arrays.
 *
 *   y = a*x + y            kernel "saxpy"       (float *y, float *x, float a, int n)
 *   out = x + y            kernel "vector_add"  (float *x, float *y, float *out, int n, int block)
 *   s = s + sum(x)         kernel "reduce_sum"  (float *s, float *x, int n)
 *
 * Built two ways. Against libbooth_sm100 alone, the library's own implementation of the
 * ABI runs all three; argv[1], when given, is the cubin to load, else the kernels come
 * from the image embedded in the library. With -DLF_SLOT_ABI the executable carries the
 * reference's src/runtime/lf_gpu_hsa.c, unchanged, which packs every parameter into an
 * 8-byte slot and dispatches through bc_*; that packing equals CUDA's natural parameter
 * layout only for kernels without two adjacent 4-byte parameters that are both read, so
 * this build runs vector_add (its last parameter is unused) and reduce_sum and needs the
 * cubin path in argv[1].
 *
 *   gcc -std=c99 -O2 -I include examples/lf_offload.c -L booth_b200/lib -lbooth_sm100 -lm -o lf_offload
 */
#include "lf_gpu.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>

static float unit(unsigned *s)          /* small LCG: inputs in [-1, 1) */
{
    *s = *s * 1664525u + 1013904223u;
    return (float)(*s >> 8) * (1.0f / 8388608.0f) - 1.0f;
}

int main(int argc, char **argv)
{
    const char *cubin = argc > 1 ? argv[1] : NULL;
    const int n = argc > 2 ? atoi(argv[2]) : 1000003;
    int grid[3] = { (n + 255) / 256, 1, 1 }, block[3] = { 256, 1, 1 };
    int bad = 0, i, bs = 256;
    unsigned seed = 0xB0070007u;
    float a = 2.5f;
    float *x = malloc((size_t)n * 4), *y = malloc((size_t)n * 4), *y0 = malloc((size_t)n * 4), *out = malloc((size_t)n * 4);
    lfortran_gpu_ctx *ctx;
    lfortran_gpu_kernel *k;

    if (!x || !y || !y0 || !out) { fprintf(stderr, "FAIL: host memory\n"); return 1; }
    for (i = 0; i < n; i++) { x[i] = unit(&seed); y[i] = y0[i] = unit(&seed); out[i] = -7.0f; }
    ctx = lfortran_gpu_init();
    if (ctx != lfortran_gpu_init()) { fprintf(stderr, "FAIL: second init returned another context\n"); return 1; }

#ifndef LF_SLOT_ABI
    k = lfortran_gpu_load_kernel(ctx, cubin, "saxpy");
    lfortran_gpu_set_buffer_arg(k, 0, y, (size_t)n * 4);
    lfortran_gpu_set_buffer_arg(k, 1, x, (size_t)n * 4);
    lfortran_gpu_set_scalar_arg(k, 2, &a, sizeof a);
    lfortran_gpu_set_scalar_arg(k, 3, &n, sizeof n);
    lfortran_gpu_launch(ctx, k, grid, block);
    lfortran_gpu_sync(ctx);
    for (i = 0; i < n; i++) {
        volatile float p = a * x[i];            /* product rounded before the sum, as the kernel does */
        if (y[i] != p + y0[i]) bad++;
    }
    printf("saxpy      n=%d: %d mismatches\n", n, bad);
    /* the same kernel object again: the Fortran loop runs twice */
    lfortran_gpu_set_buffer_arg(k, 0, y, (size_t)n * 4);
    lfortran_gpu_launch(ctx, k, grid, block);
    for (i = 0; i < n; i++) {
        volatile float p = a * x[i], q = p + y0[i];
        if (y[i] != p + q) bad++;
    }
    printf("saxpy x2   n=%d: %d mismatches\n", n, bad);
    lfortran_gpu_release_kernel(k);
    for (i = 0; i < n; i++) y[i] = y0[i];
#endif

    k = lfortran_gpu_load_kernel(ctx, cubin, "vector_add");
    lfortran_gpu_set_buffer_arg(k, 0, x, (size_t)n * 4);
    lfortran_gpu_set_buffer_arg(k, 1, y, (size_t)n * 4);
    lfortran_gpu_set_buffer_arg(k, 2, out, (size_t)n * 4);
    lfortran_gpu_set_scalar_arg(k, 3, &n, sizeof n);
    lfortran_gpu_set_scalar_arg(k, 4, &bs, sizeof bs);
    lfortran_gpu_launch(ctx, k, grid, block);
    {
        int before = bad;
        for (i = 0; i < n; i++) if (out[i] != x[i] + y[i]) bad++;
        printf("vector_add n=%d: %d mismatches\n", n, bad - before);
    }

    {
        lfortran_gpu_kernel *r = lfortran_gpu_load_kernel(ctx, cubin, "reduce_sum");
        float s = 1.0f;
        double want = 1.0;
        int rgrid[3] = { 296, 1, 1 };
        for (i = 0; i < n; i++) want += (double)x[i];
        lfortran_gpu_set_buffer_arg(r, 0, &s, sizeof s);
        lfortran_gpu_set_buffer_arg(r, 1, x, (size_t)n * 4);
        lfortran_gpu_set_scalar_arg(r, 2, &n, sizeof n);
        lfortran_gpu_launch(ctx, r, rgrid, block);
        lfortran_gpu_sync(ctx);
        printf("reduce_sum n=%d: %.6f (host %.6f)\n", n, s, want);
        if (fabs((double)s - want) > 1e-3 * (1.0 + fabs(want)) + 1e-4 * sqrt((double)n)) bad++;
        /* r is left loaded on purpose: shutdown releases what the program forgot */
    }
    lfortran_gpu_release_kernel(k);
    lfortran_gpu_release_kernel(NULL);
    lfortran_gpu_shutdown(ctx);
    lfortran_gpu_shutdown(ctx);
    free(x); free(y); free(y0); free(out);
    if (bad) { printf("FAIL\n"); return 1; }
    printf("lf_offload: ok\n");
    return 0;
}
