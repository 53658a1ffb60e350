/* nv_rt_time.c -- time a saxpy kernel loaded by name through the nv_rt_* API.
 *
 * Written against include/nv_rt.h only. The kernel file may be PTX text (for
 * instance what the reference compiler emits with --nvidia-ptx for
 * tests/canonical.cu:168-173), a cubin or a fatbin, as long as it exports
 * saxpy(float *y, float *x, float a, int n), or, when the kernel name given starts
 * with 'v', vector_add(float *x, float *y, float *out, int n, int block). Two launch
 * shapes are timed: one
 * thread per element in blocks of 256, which is how examples/launch_saxpy.c:83-87
 * launches, and, when blocks_per_sm is given, a fixed grid of that many 128-thread
 * blocks per SM for kernels that stride over the vector themselves.
 *
 *   gcc -std=c99 -O2 -I include examples/nv_rt_time.c -L booth_b200/lib -lbooth_sm100 -o nv_rt_time
 *   ./nv_rt_time <kernel file> [log2_n] [blocks_per_sm] [kernel name, default saxpy]
 */
#define _POSIX_C_SOURCE 200809L
#include "nv_rt.h"

#include <stdio.h>
#include <stdlib.h>
#include <time.h>

static double now(void)
{
    struct timespec t;
    clock_gettime(CLOCK_MONOTONIC, &t);
    return (double)t.tv_sec + 1e-9 * (double)t.tv_nsec;
}

static int timed(nv_dev_t *dev, nv_kern_t *k, unsigned grid, unsigned block, void **args, int reps, double *sec)
{
    int i;
    double t0;
    for (i = 0; i < 3; i++)
        if (nv_rt_launch(dev, k, grid, 1, 1, block, 1, 1, 0, args) != NV_RT_OK) return 1;
    if (nv_rt_sync(dev) != NV_RT_OK) return 1;
    t0 = now();
    for (i = 0; i < reps; i++)
        if (nv_rt_launch(dev, k, grid, 1, 1, block, 1, 1, 0, args) != NV_RT_OK) return 1;
    if (nv_rt_sync(dev) != NV_RT_OK) return 1;
    *sec = (now() - t0) / reps;
    return 0;
}

int main(int argc, char **argv)
{
    const int lg = argc > 2 ? atoi(argv[2]) : 28;
    const int bpsm = argc > 3 ? atoi(argv[3]) : 0;
    const char *name = argc > 4 ? argv[4] : "saxpy";
    const int n = 1 << (lg < 10 ? 10 : lg > 30 ? 30 : lg);
    const float a = 0.0f;                 /* y stays y: any number of repetitions leaves the data bounded */
    const size_t bytes = (size_t)n * 4;
    nv_dev_t dev;
    nv_kern_t k;
    CUdevptr x, y, o = 0;
    int vadd, bs = 256;
    float *h;
    double sec;
    void *args[5];
    int i, rc = 1;

    if (argc < 2) { fprintf(stderr, "usage: %s <kernel file> [log2_n] [blocks_per_sm] [kernel name]\n", argv[0]); return 2; }
    if (nv_rt_init(&dev) != NV_RT_OK) return 1;
    if (nv_rt_load(&dev, argv[1], name, &k) != NV_RT_OK) { nv_rt_shut(&dev); return 1; }
    vadd = name[0] == 'v';
    x = nv_rt_alloc(&dev, bytes);
    y = nv_rt_alloc(&dev, bytes);
    if (vadd) o = nv_rt_alloc(&dev, bytes);
    h = malloc(bytes);
    if (!x || !y || !h || (vadd && !o)) { fprintf(stderr, "FAIL: memory\n"); goto out; }
    for (i = 0; i < n; i++) h[i] = (float)(i & 1023) * 0.25f;
    if (nv_rt_h2d(&dev, x, h, bytes) != NV_RT_OK || nv_rt_h2d(&dev, y, h, bytes) != NV_RT_OK) goto out;
    if (vadd) { args[0] = &x; args[1] = &y; args[2] = &o; args[3] = (void *)&n; args[4] = &bs; }
    else { args[0] = &y; args[1] = &x; args[2] = (void *)&a; args[3] = (void *)&n; }

    if (timed(&dev, &k, (unsigned)((n + 255) / 256), 256, args, 20, &sec)) goto out;
    printf("one thread per element, 256-thread blocks: n=2^%d  %.3f ms  %.1f GB/s\n", lg, sec * 1e3, 12.0 * n / sec / 1e9);
    if (bpsm > 0) {
        if (timed(&dev, &k, 148u * (unsigned)bpsm, 128, args, 20, &sec)) goto out;
        printf("%d blocks of 128 threads per SM:            n=2^%d  %.3f ms  %.1f GB/s\n", bpsm, lg, sec * 1e3,
               12.0 * n / sec / 1e9);
    }
    if (nv_rt_d2h(&dev, h, vadd ? o : y, bytes) != NV_RT_OK) goto out;
    for (i = 0; i < n; i++)
        if (h[i] != (float)(i & 1023) * (vadd ? 0.5f : 0.25f)) { fprintf(stderr, "FAIL: result[%d] = %g\n", i, h[i]); goto out; }
    printf("nv_rt_time: ok\n");
    rc = 0;
out:
    nv_rt_free(&dev, x);
    nv_rt_free(&dev, y);
    nv_rt_free(&dev, o);
    nv_rt_unload(&dev, &k);
    nv_rt_shut(&dev);
    free(h);
    return rc;
}
