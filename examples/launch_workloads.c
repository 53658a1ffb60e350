/* launch_workloads.c -- the five workloads from one C99 host process on 1..8 B200s.
 *
 * A host program in the style of the reference's examples/launch_saxpy.c, written
 * against include/booth_sm100.h only (C99, no CUDA headers). One process drives
 * every visible GPU: inputs are the seeded Philox stream, each device takes a
 * contiguous range of the vectors / a disjoint range of Monte Carlo paths, the
 * per-device sums are combined with one NCCL all-reduce (sm100_comm_init_all).
 * With two or more devices the all-reduced totals are checked against a
 * single-device run of the whole problem on device 0.
 *
 *   gcc -std=c99 -O2 -I include examples/launch_workloads.c -L booth_b200/lib -lbooth_sm100 -lm -o launch_workloads
 *   ./launch_workloads [ngpu] [log2_elements_per_gpu] [log2_paths_per_gpu]
 */
#include "booth_sm100.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#define MAXDEV 8
#define CHECK(call) do { int rc_ = (call); if (rc_ != SM100_OK) { \
    fprintf(stderr, "FAIL: %s -> %d (line %d)\n", #call, rc_, __LINE__); return 1; } } while (0)

int main(int argc, char **argv)
{
    int have = sm100_rt_device_count();
    if (have < 1) { fprintf(stderr, "FAIL: no CUDA device (%d)\n", have); return 1; }
    int ng = argc > 1 ? atoi(argv[1]) : have;
    if (ng > have) ng = have;
    if (ng > MAXDEV) ng = MAXDEV;
    const long long n = 1ll << (argc > 2 ? atoi(argv[2]) : 26);
    const long long paths = 1ll << (argc > 3 ? atoi(argv[3]) : 22);
    const uint32_t seed = 0xB0070000u;

    sm100_dev_t *dev[MAXDEV];
    sm100_ptr_t x[MAXDEV], y[MAXDEV], out[MAXDEV];
    for (int g = 0; g < ng; g++) {
        CHECK(sm100_rt_init(&dev[g], g));
        x[g] = sm100_rt_alloc(dev[g], (size_t)n * 4);
        y[g] = sm100_rt_alloc(dev[g], (size_t)n * 4);
        out[g] = sm100_rt_alloc(dev[g], 64);
        if (!x[g] || !y[g] || !out[g]) { fprintf(stderr, "FAIL: alloc on device %d\n", g); return 1; }
    }
    sm100_comm_t *comm = NULL;
    if (ng > 1) CHECK(sm100_comm_init_all(&comm, dev, ng));

    /* saxpy on contiguous shards of one global pair of vectors; no collective */
    float ms[MAXDEV];
    for (int g = 0; g < ng; g++) {
        CHECK(booth_sm100_fill(dev[g], x[g], g * n, n, seed + 1, 0, BOOTH_FILL_F32_PM1));
        CHECK(booth_sm100_fill(dev[g], y[g], g * n, n, seed + 1, 1, BOOTH_FILL_F32_PM1));
    }
    for (int g = 0; g < ng; g++) CHECK(sm100_rt_sync(dev[g]));
    for (int g = 0; g < ng; g++) { CHECK(sm100_rt_tic(dev[g])); CHECK(booth_sm100_saxpy(dev[g], y[g], x[g], 2.5f, n)); }
    float worst = 0.f;
    for (int g = 0; g < ng; g++) { CHECK(sm100_rt_toc(dev[g], &ms[g])); if (ms[g] > worst) worst = ms[g]; }
    printf("saxpy      %d x 2^%d elements: %.3f ms, %.1f GB/s aggregate\n", ng, (int)log2((double)n), worst,
           12.0 * (double)n * ng / (worst * 1e-3) / 1e9);

    /* int32 and fp32 sums: per-device reduction, then one all-reduce of one element */
    int isum[MAXDEV]; double fsum[MAXDEV];
    for (int pass = 0; pass < 2; pass++) {
        for (int g = 0; g < ng; g++)
            CHECK(booth_sm100_fill(dev[g], x[g], g * n, n, seed + 2, (uint32_t)pass, pass ? BOOTH_FILL_F32_01 : BOOTH_FILL_I32_1000));
        for (int g = 0; g < ng; g++)
            CHECK(pass ? booth_sm100_reduce_f32(dev[g], x[g], n, out[g]) : booth_sm100_reduce_i32(dev[g], x[g], n, out[g]));
        if (comm) {
            CHECK(sm100_comm_group_begin());
            for (int g = 0; g < ng; g++) CHECK(sm100_comm_allreduce_sum_dev(comm, g, out[g], 1, pass ? SM100_F64 : SM100_I32));
            CHECK(sm100_comm_group_end());
        }
        for (int g = 0; g < ng; g++)
            CHECK(pass ? sm100_rt_d2h(dev[g], &fsum[g], out[g], 8) : sm100_rt_d2h(dev[g], &isum[g], out[g], 4));
    }
    for (int g = 1; g < ng; g++)
        if (isum[g] != isum[0] || fsum[g] != fsum[0]) { printf("FAIL: ranks disagree after the all-reduce\n"); return 1; }
    printf("sum int32  %d x 2^%d: %d      sum fp32: %.6f\n", ng, (int)log2((double)n), isum[0], fsum[0]);

    /* Asian option: disjoint Philox subsequences per device, all-reduce of four doubles */
    booth_asian_t prm;
    const float dt = 1.0f / 252.0f;
    prm.s0 = 100.f; prm.strike = 100.f; prm.nstep = 252; prm.k0 = seed + 5; prm.k1 = 0; prm.precise = 0;
    prm.drift = (0.05f - 0.5f * 0.2f * 0.2f) * dt;
    prm.vol = 0.2f * sqrtf(dt);
    double mc[MAXDEV][4];
    for (int g = 0; g < ng; g++) CHECK(booth_sm100_asian(dev[g], &prm, g * paths, paths, out[g]));
    if (comm) {
        CHECK(sm100_comm_group_begin());
        for (int g = 0; g < ng; g++) CHECK(sm100_comm_allreduce_sum_dev(comm, g, out[g], 4, SM100_F64));
        CHECK(sm100_comm_group_end());
    }
    for (int g = 0; g < ng; g++) CHECK(sm100_rt_d2h(dev[g], mc[g], out[g], 32));
    const double tot = (double)paths * ng, disc = exp(-0.05);
    printf("asian      %d x 2^%d paths: arithmetic %.6f  geometric %.6f (closed form 5.5655)\n", ng,
           (int)log2((double)paths), disc * mc[0][0] / tot, disc * mc[0][1] / tot);

    int bad = 0;
    if (ng > 1) {
        /* the same totals from device 0 alone over the whole ranges */
        double whole[4];
        CHECK(booth_sm100_asian(dev[0], &prm, 0, paths * ng, out[0]));
        CHECK(sm100_rt_d2h(dev[0], whole, out[0], 32));
        for (int k = 0; k < 4; k++) if (fabs(whole[k] - mc[0][k]) > 1e-12 * fabs(whole[k])) bad++;
        int iw = 0;
        for (int g = 0; g < ng; g++) {           /* int32 sum of every shard on device 0, added on the host */
            int part;
            CHECK(booth_sm100_fill(dev[0], x[0], g * n, n, seed + 2, 0, BOOTH_FILL_I32_1000));
            CHECK(booth_sm100_reduce_i32(dev[0], x[0], n, out[0]));
            CHECK(sm100_rt_d2h(dev[0], &part, out[0], 4));
            iw = (int)((unsigned)iw + (unsigned)part);
        }
        if (iw != isum[0]) bad++;
    }
    if (fabs(disc * mc[0][1] / tot - 5.5655) > 0.05) bad++;

    if (comm) sm100_comm_destroy(comm);
    for (int g = 0; g < ng; g++) {
        sm100_rt_free(dev[g], x[g]); sm100_rt_free(dev[g], y[g]); sm100_rt_free(dev[g], out[g]);
        sm100_rt_shut(dev[g]);
    }
    if (bad) { printf("FAIL: %d cross-check(s) failed\n", bad); return 1; }
    printf("PASS: %d device(s)\n", ng);
    return 0;
}
