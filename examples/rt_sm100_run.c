/* rt_sm100_run.c -- drive the B200 through Booth's run-side contract.
 *
 * The program uses nothing but the descriptor operations of src/exec/exec.h
 * (open, load, alloc, h2d, run, sync, d2h, ...), the way src/exec/execs.c
 * dispatches them, to run the saxpy kernel of the sm_100a image and compare it
 * with the separately rounded host result (mulss then addss, as the reference's
 * x86-64 backend computes it).
 *
 *   gcc -std=c99 -O2 -I include [-I <booth>/src/exec -DUSE_BOOTH_EXEC_H] examples/rt_sm100_run.c \
 *       -L booth_b200/lib -lbooth_sm100 -o rt_sm100_run
 *   ./rt_sm100_run booth_b200/lib/booth_sm100.cubin
 */
#ifdef USE_BOOTH_EXEC_H
#include "exec.h"            /* the reference's own header: the descriptor must fit its types */
#endif
#include "rt_sm100.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define N 100003

int main(int argc, char **argv)
{
    const char *cubin = argc > 1 ? argv[1] : "booth_sm100.cubin";
    const rt_desc_t *t = &rt_sm100;
    unsigned char dev[RT_DEV_MAX], kern[RT_KERN_MAX];
    if (t->dev_size > RT_DEV_MAX || t->kern_size > RT_KERN_MAX) { printf("FAIL: handle sizes\n"); return 1; }
    memset(dev, 0, sizeof dev);
    memset(kern, 0, sizeof kern);
    int rc = t->open(dev);
    if (rc != RT_OK) { printf("FAIL: open: %s\n", t->errs(rc)); return 1; }

    /* host-detectable failures come back as contract codes */
    if (t->load(dev, "/nonexistent.cubin", "saxpy", kern) != RT_EIO) { printf("FAIL: EIO\n"); return 1; }
    if (t->load(dev, cubin, "no_such_kernel", kern) != RT_EKERN) { printf("FAIL: EKERN\n"); return 1; }
    rc = t->load(dev, cubin, "saxpy", kern);
    if (rc != RT_OK) { printf("FAIL: load: %s\n", t->errs(rc)); return 1; }

    float *x = (float *)malloc(N * sizeof(float)), *y = (float *)malloc(N * sizeof(float));
    float *want = (float *)malloc(N * sizeof(float));
    const float a = 2.5f;
    for (int i = 0; i < N; i++) {
        x[i] = (float)(i % 977) * 0.37f - 100.0f;
        y[i] = (float)(i % 613) * -0.011f + 3.0f;
        volatile float p = a * x[i];           /* product rounded on its own */
        want[i] = p + y[i];
    }
    rt_ptr dx = t->alloc(dev, N * sizeof(float)), dy = t->alloc(dev, N * sizeof(float));
    if (!dx || !dy) { printf("FAIL: alloc\n"); return 1; }
    t->trak(dev, dy, N * sizeof(float), "y", 0);
    if (t->h2d(dev, dx, x, N * sizeof(float)) || t->h2d(dev, dy, y, N * sizeof(float))) { printf("FAIL: h2d\n"); return 1; }

    int n = N;
    rt_arg_t args[4] = { { &dy, sizeof dy }, { &dx, sizeof dx }, { &a, sizeof a }, { &n, sizeof n } };
    rt_dim_t dim = { { (N + 255) / 256, 1, 1 }, { 256, 1, 1 }, 0 };
    rc = t->run(dev, kern, &dim, args, 4);
    if (rc == RT_OK) rc = t->sync(dev);
    if (rc != RT_OK) { printf("FAIL: run: %s\n", t->errs(rc)); return 1; }
    if (t->d2h(dev, y, dy, N * sizeof(float))) { printf("FAIL: d2h\n"); return 1; }

    int bad = 0;
    for (int i = 0; i < N; i++) if (memcmp(&y[i], &want[i], 4) != 0) bad++;

    /* memory both sides can reach */
    void *hp = NULL; rt_ptr dp = 0;
    if (t->hmap(dev, &hp, &dp, 4096) != RT_OK || !hp || !dp) { printf("FAIL: hmap\n"); return 1; }
    t->hfre(dev, hp);

    t->dfre(dev, dx); t->dfre(dev, dy);
    t->unload(dev, kern);
    t->shut(dev);
    if (bad) { printf("FAIL: %d of %d elements differ\n", bad, N); return 1; }
    printf("PASS: descriptor '%s' (%s) ran saxpy on %d elements, bit-exact\n", t->name, t->artefact, N);
    return 0;
}
