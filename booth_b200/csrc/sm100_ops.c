/* sm100_ops.c -- the five workloads, launched with geometry tuned for a B200.
 *
 * Each function enqueues work on the device's stream and returns; results stay
 * in device memory (sm100_rt_sync / sm100_rt_d2h fetch them). The kernels come
 * from the image embedded in the library. There is no host-side arithmetic on
 * the data anywhere in this file, and no fallback: a failed launch is reported.
 *
 * The CPU-launcher symbols at the end (vector_add, matmul, matmul_k, saxpy) have
 * the signatures the reference's x86-64 objects export
 * (examples/cpu_launch_vadd.c:23-24, examples/cpu_launch_matmul.c:22-26); they
 * take host pointers, stage them through the GPU and copy the result back. */
#define _POSIX_C_SOURCE 200809L
#include <limits.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "sm100_internal.h"

static int env_int(const char *name, int dflt, int lo, int hi)
{
    const char *e = getenv(name);
    if (!e || !*e) return dflt;
    int v = atoi(e);
    if (v < lo) v = lo;
    if (v > hi) v = hi;
    return v;
}

static int bad_arg(sm100_dev_t *dev, const char *what)
{
    if (dev) snprintf(dev->err, sizeof dev->err, "%s", what);
    fprintf(stderr, "sm100_rt: %s\n", what);
    return SM100_ERR_ARG;
}

/* Scratch layout: the arrival counter and the GEMM status word in the first
 * 256 bytes, partials after. */
#define SCRATCH_TICKET   SM100_SCRATCH_TICKET
#define SCRATCH_PARTIALS SM100_SCRATCH_PARTIALS

/* Streaming kernels: 128-thread blocks; one block iteration (a tile) covers 128
 * threads x 2 x 32 bytes per input. Vectors of 2^28 elements and more get three
 * persistent blocks per SM: HBM throughput on a B200 peaks sharply at 384 threads
 * per SM for both kernels (saxpy at 2^30 elements: 6.94 TB/s at 3 blocks per SM,
 * 6.52 at 5, 6.73 at 32; vector add at 2^29: 6.94 at 3, 6.53 at 5, 6.79 at 32).
 * Shorter vectors stream for tens of microseconds and are dominated by the two
 * ends of the launch: up to 128 blocks per SM, in practice one tile each, let the
 * hardware scheduler even those out (saxpy at 2^24: 7.5 TB/s against 6.1 at 3
 * persistent blocks per SM; vector add: 6.45 against 5.96; at 2^27 the two
 * geometries meet). BOOTH_SM100_STREAM_BPSM / _BLOCK override. */
static unsigned stream_grid(sm100_dev_t *dev, long long n, unsigned block, unsigned unroll)
{
    const int bpsm = env_int("BOOTH_SM100_STREAM_BPSM", n < (1ll << 28) ? 128 : 3, 1, 128);
    long long tiles = ((n >> 3) + (long long)block * unroll - 1) / ((long long)block * unroll);
    long long g = (long long)dev->sm_count * bpsm;
    if (tiles < g) g = tiles;
    if (g < 1) g = 1;
    return (unsigned)g;
}

int booth_sm100_fill(sm100_dev_t *dev, sm100_ptr_t dst, long long first, long long n,
                     uint32_t seed, uint32_t stream, int kind)
{
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    if (n < 0 || first < 0 || kind < 0 || kind > BOOTH_FILL_U32_RAW || (n > 0 && (!dst || (dst & 3))))
        return bad_arg(dev, "booth_sm100_fill: bad argument");
    if (n == 0) return SM100_OK;
    long long nblk = ((first + n + 3) >> 2) - (first >> 2);
    long long g = (nblk + 255) / 256;
    if (g > (long long)dev->sm_count * 16) g = (long long)dev->sm_count * 16;
    void *args[] = { &dst, &first, &n, &seed, &stream, &kind };
    return sm100_launch_k(dev, SM100_K_FILL, (unsigned)g, 256, 0, args);
}

int booth_sm100_vadd(sm100_dev_t *dev, sm100_ptr_t x, sm100_ptr_t y, sm100_ptr_t out, long long n)
{
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    if (n < 0 || n > INT_MAX) return bad_arg(dev, "booth_sm100_vadd: n must be in [0, 2^31)");
    if (n == 0) return SM100_OK;
    if (!x || !y || !out || ((x | y | out) & 3))
        return bad_arg(dev, "booth_sm100_vadd: vectors must be non-NULL and 4-byte aligned");
    int ni = (int)n, bs = 256;
    const unsigned block = (unsigned)env_int("BOOTH_SM100_STREAM_BLOCK", 128, 32, 1024);
    void *args[] = { &x, &y, &out, &ni, &bs };
    return sm100_launch_k_overlapped(dev, SM100_K_VADD, stream_grid(dev, n, block, 2), block, 0, args);
}

int booth_sm100_saxpy(sm100_dev_t *dev, sm100_ptr_t y, sm100_ptr_t x, float a, long long n)
{
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    if (n < 0 || n > INT_MAX) return bad_arg(dev, "booth_sm100_saxpy: n must be in [0, 2^31)");
    if (n == 0) return SM100_OK;
    if (!x || !y || ((x | y) & 3))
        return bad_arg(dev, "booth_sm100_saxpy: vectors must be non-NULL and 4-byte aligned");
    int ni = (int)n;
    const unsigned block = (unsigned)env_int("BOOTH_SM100_STREAM_BLOCK", 128, 32, 1024);
    void *args[] = { &y, &x, &a, &ni };
    return sm100_launch_k_overlapped(dev, SM100_K_SAXPY, stream_grid(dev, n, block, 2), block, 0, args);
}

/* Reductions: 256-thread blocks, eight 16-byte loads per thread in flight. The
 * int32 kernel (32 registers) runs best at 8 blocks per SM (7.3 TB/s at 2^30
 * elements against 7.1 at 6 and 6.6 at 4); the fp32 kernel (62 registers, built
 * for at most 256 threads per block and 4 blocks per SM) at 3 (7.3 TB/s; 2 to 16
 * differ by about a percent). BOOTH_SM100_REDUCE_BPSM / _BLOCK override. */
static int reduce_common(sm100_dev_t *dev, int which, sm100_ptr_t in, long long n, sm100_ptr_t out, unsigned out_align,
                         int dflt_bpsm, unsigned max_block)
{
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    /* Checked here, before any GPU work: a misaligned result address would fault on the device. */
    if (n < 0 || !out || (out & (out_align - 1)) || (in & 3) || (n > 0 && !in))
        return bad_arg(dev, "booth_sm100_reduce: bad argument (in: 4-byte aligned, non-NULL when n > 0; "
                            "out: aligned to its own size, 4 bytes for the int32 sum, 8 for the fp32 sum)");
    unsigned block = (unsigned)env_int("BOOTH_SM100_REDUCE_BLOCK", 256, 32, 1024) & ~31u;
    if (block > max_block) block = max_block;
    const int bpsm = env_int("BOOTH_SM100_REDUCE_BPSM", dflt_bpsm, 1, 32);
    long long tiles = ((n >> 2) + (long long)block * 8 - 1) / ((long long)block * 8);
    long long g = (long long)dev->sm_count * bpsm;
    if (tiles < g) g = tiles;
    if (g < 1) g = 1;
    CUdeviceptr sc = sm100_scratch(dev, SCRATCH_PARTIALS + (size_t)g * 8);
    if (!sc) return SM100_ERR_ARG;
    CUdeviceptr partials = sc + SCRATCH_PARTIALS, ticket = sc + SCRATCH_TICKET;
    void *args[] = { &in, &n, &partials, &ticket, &out };
    return sm100_launch_k(dev, which, (unsigned)g, block, 0, args);
}

int booth_sm100_reduce_i32(sm100_dev_t *dev, sm100_ptr_t in, long long n, sm100_ptr_t out)
{
    return reduce_common(dev, SM100_K_REDUCE_I32, in, n, out, 4, 8, 1024);
}

int booth_sm100_reduce_f32(sm100_dev_t *dev, sm100_ptr_t in, long long n, sm100_ptr_t out)
{
    return reduce_common(dev, SM100_K_REDUCE_F32, in, n, out, 8, 3, 256);
}

int booth_sm100_asian(sm100_dev_t *dev, const booth_asian_t *p, long long path0,
                      long long npaths, sm100_ptr_t out)
{
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    if (!p || !out || (out & 7) || npaths < 0 || path0 < 0 || p->nstep <= 0 || (p->nstep & 3))
        return bad_arg(dev, "booth_sm100_asian: bad argument (nstep must be a positive multiple of 4, out 8-byte aligned)");
    /* 256-thread blocks, two resident per SM (116 registers). Thirty-two blocks per SM
     * in the grid, i.e. a hundred-odd paths per thread at 2^26 paths: the finer grain
     * evens out the end of the launch (1.5 % more paths per second than 8 blocks per
     * SM, 7 % more than 2; beyond 48 the per-block reduction starts to show). */
    const unsigned block = 256;
    const int bpsm = env_int("BOOTH_SM100_ASIAN_BPSM", 32, 1, 128);
    long long g = (npaths + block - 1) / block;
    if (g > (long long)dev->sm_count * bpsm) g = (long long)dev->sm_count * bpsm;
    if (g < 1) g = 1;
    CUdeviceptr sc = sm100_scratch(dev, SCRATCH_PARTIALS + (size_t)g * 32);
    if (!sc) return SM100_ERR_ARG;
    CUdeviceptr partials = sc + SCRATCH_PARTIALS, ticket = sc + SCRATCH_TICKET;
    unsigned long long p0 = (unsigned long long)path0, np = (unsigned long long)npaths;
    booth_asian_t q = *p;
    void *args[] = { &out, &p0, &np, &q.k0, &q.k1, &q.s0, &q.strike, &q.drift, &q.vol,
                     &q.nstep, &partials, &ticket };
    return sm100_launch_k(dev, p->precise ? SM100_K_ASIAN_MC_PRECISE : SM100_K_ASIAN_MC,
                          (unsigned)g, block, 0, args);
}

int booth_sm100_asian_paths(sm100_dev_t *dev, const booth_asian_t *p, long long path0,
                            long long npaths, sm100_ptr_t arith, sm100_ptr_t geom)
{
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    if (!p || !arith || !geom || ((arith | geom) & 3) || npaths < 0 || path0 < 0 || p->nstep <= 0 || (p->nstep & 3))
        return bad_arg(dev, "booth_sm100_asian_paths: bad argument");
    if (npaths == 0) return SM100_OK;
    long long g = (npaths + 255) / 256;
    if (g > (long long)dev->sm_count * 8) g = (long long)dev->sm_count * 8;
    booth_asian_t q = *p;
    void *args[] = { &arith, &geom, &path0, &npaths, &q.k0, &q.k1, &q.s0, &q.strike,
                     &q.drift, &q.vol, &q.nstep };
    return sm100_launch_k(dev, p->precise ? SM100_K_ASIAN_PATHS_PRECISE : SM100_K_ASIAN_PATHS,
                          (unsigned)g, 256, 0, args);
}

/* ---- host-side generator: the same stream as the fill_philox kernel ---- */

static void philox_block(uint32_t c[4], uint32_t k0, uint32_t k1)
{
    for (int r = 0; r < 10; r++) {
        uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
        uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0;
        uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
        c[0] = n0; c[1] = (uint32_t)p1; c[2] = n2; c[3] = (uint32_t)p0;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
}

void booth_sm100_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4])
{
    uint32_t c[4] = { ctr[0], ctr[1], ctr[2], ctr[3] };
    philox_block(c, key[0], key[1]);
    memcpy(out, c, sizeof c);
}

typedef struct { uint32_t *dst; long long first, lo, hi; uint32_t seed, stream; int kind; } fill_job_t;

static void *fill_worker(void *arg)
{
    fill_job_t *j = (fill_job_t *)arg;
    long long i = j->lo;
    while (i < j->hi) {
        long long e = j->first + i;
        unsigned long long ctr = (unsigned long long)(e >> 2);
        uint32_t c[4] = { (uint32_t)ctr, (uint32_t)(ctr >> 32), 0, 0 };
        philox_block(c, j->seed, j->stream);
        for (int l = (int)(e & 3); l < 4 && i < j->hi; l++, i++) {
            uint32_t x = c[l], v;
            if (j->kind == BOOTH_FILL_I32_1000) {
                v = (uint32_t)((int)(x % 2001u) - 1000);
            } else if (j->kind == BOOTH_FILL_U32_RAW) {
                v = x;
            } else {
                float u = (float)(x >> 8) * 5.9604644775390625e-8f;
                float f = j->kind == BOOTH_FILL_F32_PM1 ? 2.0f * u - 1.0f : u;
                memcpy(&v, &f, 4);
            }
            j->dst[i] = v;
        }
    }
    return NULL;
}

void booth_sm100_fill_host(void *dst, long long first, long long n, uint32_t seed,
                           uint32_t stream, int kind, int threads)
{
    if (!dst || n <= 0) return;
    if (threads < 1) threads = 1;
    if (threads > 64) threads = 64;
    if (n < (1 << 16)) threads = 1;
    pthread_t tid[64];
    fill_job_t job[64];
    for (int t = 0; t < threads; t++) {
        job[t].dst = (uint32_t *)dst; job[t].first = first;
        job[t].lo = n * t / threads; job[t].hi = n * (t + 1) / threads;
        job[t].seed = seed; job[t].stream = stream; job[t].kind = kind;
    }
    for (int t = 1; t < threads; t++) pthread_create(&tid[t], NULL, fill_worker, &job[t]);
    fill_worker(&job[0]);
    for (int t = 1; t < threads; t++) pthread_join(tid[t], NULL);
}

/* ---- host-pointer streaming: H2D, kernel and D2H pipelined over chunks ---- */

static int stage_setup(sm100_dev_t *dev)
{
    if (dev->stage_ready) return SM100_OK;
    const sm100_api_t *a = dev->api;
    CUstream s_out = NULL, s_in = NULL;
    CUevent ev[3][SM100_STAGE_SLOTS];
    CUdeviceptr stage = 0;
    memset(ev, 0, sizeof ev);
    CUresult cr = a->StreamCreate(&s_out, CU_STREAM_NON_BLOCKING);
    if (cr == CUDA_SUCCESS) cr = a->StreamCreate(&s_in, CU_STREAM_NON_BLOCKING);
    for (int k = 0; k < 3 && cr == CUDA_SUCCESS; k++)
        for (int i = 0; i < SM100_STAGE_SLOTS && cr == CUDA_SUCCESS; i++)
            cr = a->EventCreate(&ev[k][i], CU_EVENT_DISABLE_TIMING);
    if (cr == CUDA_SUCCESS) cr = a->MemAlloc(&stage, (size_t)SM100_STAGE_SLOTS * 2 * SM100_STAGE_BYTES);
    if (cr != CUDA_SUCCESS) {
        /* nothing half-built is kept: the next call starts over */
        for (int k = 0; k < 3; k++)
            for (int i = 0; i < SM100_STAGE_SLOTS; i++)
                if (ev[k][i]) a->EventDestroy(ev[k][i]);
        if (s_in) a->StreamDestroy(s_in);
        if (s_out) a->StreamDestroy(s_out);
        return sm100_fail(dev, "setting up the staging ring (two streams, nine events, 384 MiB)", cr);
    }
    dev->stream_out = s_out; dev->stream_in = s_in; dev->stage = stage;
    for (int i = 0; i < SM100_STAGE_SLOTS; i++) {
        dev->ev_uploaded[i] = ev[0][i]; dev->ev_computed[i] = ev[1][i]; dev->ev_drained[i] = ev[2][i];
    }
    dev->stage_ready = 1;
    return SM100_OK;
}

/* out[i] = op(x[i], y[i]) for host vectors. The vectors are cut into chunks of
 * 16 Mi elements and go through three streams: uploads (H2D of x and y) on one,
 * the kernel on the device's own stream, copies back (D2H) on a third, chained by
 * one event per staging slot and step. The upload of chunk i+1 therefore never
 * queues behind the kernel of chunk i, and both directions of the link stay busy.
 * Three staging slots of 2 x 64 MiB on the device; a slot is refilled once its
 * copy back has finished. */
static int stream_host(sm100_dev_t *dev, int saxpy, const float *x, const float *y, float *out, float a, long long n)
{
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    if (n < 0 || (n > 0 && (!x || !y || !out)) || (((uintptr_t)x | (uintptr_t)y | (uintptr_t)out) & 3))
        return bad_arg(dev, "booth_sm100_*_host: bad argument (vectors non-NULL and 4-byte aligned)");
    if (n == 0) return SM100_OK;
    if ((rc = stage_setup(dev)) != SM100_OK) return rc;
    const sm100_api_t *api = dev->api;
    const long long chunk = SM100_STAGE_BYTES / 4;
    CUresult cr = CUDA_SUCCESS;
    long long done = 0;
    /* work already queued on the device's stream (the caller's earlier calls) comes first */
    cr = api->EventRecord(dev->ev_computed[0], dev->stream);
    if (cr == CUDA_SUCCESS) cr = api->StreamWaitEvent(dev->stream_in, dev->ev_computed[0], 0);
    for (long long i = 0; done < n && cr == CUDA_SUCCESS; i++, done += chunk) {
        const int slot = (int)(i % SM100_STAGE_SLOTS);
        const long long m = n - done < chunk ? n - done : chunk;
        const CUdeviceptr dx = dev->stage + (size_t)slot * 2 * SM100_STAGE_BYTES, dy = dx + SM100_STAGE_BYTES;
        if (i >= SM100_STAGE_SLOTS) cr = api->StreamWaitEvent(dev->stream_in, dev->ev_drained[slot], 0);
        if (cr == CUDA_SUCCESS) cr = api->MemcpyHtoDAsync(dx, x + done, (size_t)m * 4, dev->stream_in);
        if (cr == CUDA_SUCCESS) cr = api->MemcpyHtoDAsync(dy, y + done, (size_t)m * 4, dev->stream_in);
        if (cr == CUDA_SUCCESS) cr = api->EventRecord(dev->ev_uploaded[slot], dev->stream_in);
        if (cr == CUDA_SUCCESS) cr = api->StreamWaitEvent(dev->stream, dev->ev_uploaded[slot], 0);
        if (cr != CUDA_SUCCESS) break;
        /* saxpy writes y in place; vector add writes its sum over the staged y */
        rc = saxpy ? booth_sm100_saxpy(dev, dy, dx, a, m) : booth_sm100_vadd(dev, dx, dy, dy, m);
        if (rc != SM100_OK) break;
        cr = api->EventRecord(dev->ev_computed[slot], dev->stream);
        if (cr == CUDA_SUCCESS) cr = api->StreamWaitEvent(dev->stream_out, dev->ev_computed[slot], 0);
        if (cr == CUDA_SUCCESS) cr = api->MemcpyDtoHAsync(out + done, dy, (size_t)m * 4, dev->stream_out);
        if (cr == CUDA_SUCCESS) cr = api->EventRecord(dev->ev_drained[slot], dev->stream_out);
    }
    /* All three streams are drained on every way out: copies from x and y and into
     * out may still be in flight, and the caller owns those buffers again on return. */
    const CUresult d0 = api->StreamSynchronize(dev->stream_in), d1 = api->StreamSynchronize(dev->stream_out),
                   d2 = api->StreamSynchronize(dev->stream);
    if (rc != SM100_OK) return rc;
    if (cr == CUDA_SUCCESS) cr = d0 != CUDA_SUCCESS ? d0 : d1 != CUDA_SUCCESS ? d1 : d2;
    return cr == CUDA_SUCCESS ? SM100_OK : sm100_fail(dev, "host-pointer streaming", cr);
}

/* How fast this GPU's host link moves page-locked memory: `bytes` up alone, down
 * alone, then both at once on two streams, each repeated `reps` times; GB/s. */
int booth_sm100_link_probe(sm100_dev_t *dev, size_t bytes, int reps, double gbs[4])
{
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    if (!gbs || bytes < 4096 || reps < 1) return bad_arg(dev, "booth_sm100_link_probe: bad argument");
    if ((rc = stage_setup(dev)) != SM100_OK) return rc;
    const sm100_api_t *api = dev->api;
    void *hup = NULL, *hdn = NULL;
    CUdeviceptr dup = 0, ddn = 0;
    CUevent e0 = NULL, e1 = NULL, f0 = NULL, f1 = NULL;
    CUresult cr = api->MemHostAlloc(&hup, bytes, CU_MEMHOSTALLOC_PORTABLE);
    if (cr == CUDA_SUCCESS) cr = api->MemHostAlloc(&hdn, bytes, CU_MEMHOSTALLOC_PORTABLE);
    if (cr == CUDA_SUCCESS) cr = api->MemAlloc(&dup, bytes);
    if (cr == CUDA_SUCCESS) cr = api->MemAlloc(&ddn, bytes);
    if (cr == CUDA_SUCCESS) cr = api->EventCreate(&e0, CU_EVENT_DEFAULT);
    if (cr == CUDA_SUCCESS) cr = api->EventCreate(&e1, CU_EVENT_DEFAULT);
    if (cr == CUDA_SUCCESS) cr = api->EventCreate(&f0, CU_EVENT_DEFAULT);
    if (cr == CUDA_SUCCESS) cr = api->EventCreate(&f1, CU_EVENT_DEFAULT);
    if (cr == CUDA_SUCCESS) { memset(hup, 1, bytes); memset(hdn, 0, bytes); }
    if (cr == CUDA_SUCCESS) cr = api->StreamSynchronize(dev->stream);
    for (int mode = 0; mode < 3 && cr == CUDA_SUCCESS; mode++) {          /* up, down, both */
        for (int r = -1; r < reps && cr == CUDA_SUCCESS; r++) {           /* r = -1: untimed warm-up */
            if (r == 0) {
                cr = api->EventRecord(e0, dev->stream_in);
                if (cr == CUDA_SUCCESS) cr = api->EventRecord(f0, dev->stream_out);
            }
            if (cr == CUDA_SUCCESS && mode != 1) cr = api->MemcpyHtoDAsync(dup, hup, bytes, dev->stream_in);
            if (cr == CUDA_SUCCESS && mode != 0) cr = api->MemcpyDtoHAsync(hdn, ddn, bytes, dev->stream_out);
            if (r == -1 && cr == CUDA_SUCCESS) {
                cr = api->StreamSynchronize(dev->stream_in);
                if (cr == CUDA_SUCCESS) cr = api->StreamSynchronize(dev->stream_out);
            }
        }
        if (cr == CUDA_SUCCESS) cr = api->EventRecord(e1, dev->stream_in);
        if (cr == CUDA_SUCCESS) cr = api->EventRecord(f1, dev->stream_out);
        if (cr == CUDA_SUCCESS) cr = api->StreamSynchronize(dev->stream_in);
        if (cr == CUDA_SUCCESS) cr = api->StreamSynchronize(dev->stream_out);
        float up_ms = 0.0f, dn_ms = 0.0f;
        if (cr == CUDA_SUCCESS) cr = api->EventElapsedTime(&up_ms, e0, e1);
        if (cr == CUDA_SUCCESS) cr = api->EventElapsedTime(&dn_ms, f0, f1);
        const double vol = (double)bytes * reps / 1e9;
        if (mode == 0) gbs[0] = up_ms > 0 ? vol / (up_ms * 1e-3) : 0.0;
        if (mode == 1) gbs[1] = dn_ms > 0 ? vol / (dn_ms * 1e-3) : 0.0;
        if (mode == 2) { gbs[2] = up_ms > 0 ? vol / (up_ms * 1e-3) : 0.0; gbs[3] = dn_ms > 0 ? vol / (dn_ms * 1e-3) : 0.0; }
    }
    if (e0) api->EventDestroy(e0);
    if (e1) api->EventDestroy(e1);
    if (f0) api->EventDestroy(f0);
    if (f1) api->EventDestroy(f1);
    if (dup) api->MemFree(dup);
    if (ddn) api->MemFree(ddn);
    if (hup) api->MemFreeHost(hup);
    if (hdn) api->MemFreeHost(hdn);
    return cr == CUDA_SUCCESS ? SM100_OK : sm100_fail(dev, "link probe", cr);
}

int booth_sm100_saxpy_host(sm100_dev_t *dev, float *y, const float *x, float a, long long n)
{
    return stream_host(dev, 1, x, y, y, a, n);
}

int booth_sm100_vadd_host(sm100_dev_t *dev, const float *x, const float *y, float *out, long long n)
{
    return stream_host(dev, 0, x, y, out, 0.0f, n);
}

/* ---- CPU-launcher symbols ---- */

static sm100_dev_t *g_host_dev;
static pthread_mutex_t g_host_mu = PTHREAD_MUTEX_INITIALIZER;

static void host_die(const char *what)
{
    fprintf(stderr, "sm100_rt: %s failed on the GPU path; there is no CPU fallback\n", what);
    abort();
}

static sm100_dev_t *host_dev(const char *what)
{
    pthread_mutex_lock(&g_host_mu);
    if (!g_host_dev && sm100_rt_init(&g_host_dev, -1) != SM100_OK) {
        pthread_mutex_unlock(&g_host_mu);
        host_die(what);
    }
    pthread_mutex_unlock(&g_host_mu);
    return g_host_dev;
}

/* The reference's objects are plain functions that several host threads may call at
 * once on disjoint ranges; here such calls share one device and one staging ring,
 * so they take turns. */
static void host_stream(const char *what, int is_saxpy, const float *x, const float *y, float *out, float a, long long m)
{
    sm100_dev_t *d = host_dev(what);
    pthread_mutex_lock(&g_host_mu);
    const int rc = stream_host(d, is_saxpy, x, y, out, a, m);
    pthread_mutex_unlock(&g_host_mu);
    if (rc != SM100_OK) host_die(what);
}

void vector_add(float *x, float *y, float *out, int n_elements, int block_size, int nthreads)
{
    /* One call of the CPU launcher covers element indices [0, nthreads): the
     * kernel's masks are dropped there (src/triton/lower.c:713-760), n_elements
     * is not consulted. */
    (void)n_elements; (void)block_size;
    if (nthreads <= 0) return;
    host_stream("vector_add", 0, x, y, out, 0.0f, nthreads);
}

void vadd(const float *a, const float *b, float *c, int n, int nthreads)
{
    /* tests/ocaml/vadd_k.bir: c[i] = a[i] + b[i] for the threads with i < n. */
    long long m = nthreads < n ? nthreads : n;
    if (m <= 0) return;
    host_stream("vadd", 0, a, b, c, 0.0f, m);
}

void saxpy(float *y, float *x, float a, int n, int nthreads)
{
    /* tests/canonical.cu:168-173: threads with idx >= n do nothing. */
    long long m = nthreads < n ? nthreads : n;
    if (m <= 0) return;
    host_stream("saxpy", 1, x, y, y, a, m);
}

/* Extent, in floats, of a strided 4 x K (or K x 4) operand starting at its base. */
static size_t span(int r, int sr, int c, int sc)
{
    long long m = (long long)(r - 1) * (sr > 0 ? sr : 0) + (long long)(c - 1) * (sc > 0 ? sc : 0) + 1;
    return (size_t)m;
}

static void tile_matmul(const char *what, float *a, float *b, float *c, int K, int block_k,
                        int sam, int sak, int sbk, int sbn, int scm, int scn, int accumulate,
                        int nthreads)
{
    if (nthreads <= 0) return;
    if (sam < 0 || sak < 0 || sbk < 0 || sbn < 0 || scm < 0 || scn < 0 || K <= 0) {
        fprintf(stderr, "sm100_rt: %s: negative strides are not supported\n", what);
        abort();
    }
    sm100_dev_t *d = host_dev(what);
    size_t na = span(4, sam, K, sak), nb = span(K, sbk, 4, sbn), nc = span(4, scm, 4, scn);
    /* Callers walk a matrix tile by tile with one call each (the reference's harnesses do),
     * so the device buffers and the kernel handle are kept between calls: one allocation
     * that only grows, cut into the three operands at 256-byte boundaries. */
    static sm100_ptr_t buf;
    static size_t buf_bytes;
    static sm100_kern_t k;
    const size_t oa = 0, ob = (na * 4 + 255) & ~(size_t)255, oc = ob + ((nb * 4 + 255) & ~(size_t)255);
    const size_t need = oc + nc * 4;
    pthread_mutex_lock(&g_host_mu);
    if (need > buf_bytes) {
        if (buf) sm100_rt_free(d, buf);
        buf_bytes = need < (1u << 20) ? (1u << 20) : need * 2;
        buf = sm100_rt_alloc(d, buf_bytes);
        if (!buf) { buf_bytes = 0; pthread_mutex_unlock(&g_host_mu); host_die(what); }
    }
    if (!k.func && sm100_rt_load_builtin(d, "matmul_tile", &k)) { pthread_mutex_unlock(&g_host_mu); host_die(what); }
    sm100_ptr_t da = buf + oa, db = buf + ob, dc = buf + oc;
    void *args[] = { &da, &db, &dc, &K, &block_k, &sam, &sak, &sbk, &sbn, &scm, &scn, &accumulate };
    /* The strided tile of c is written in place: bring the surrounding floats
     * over first so the copy back leaves them untouched. The three uploads and the launch
     * are queued on the device's stream; the copy back waits for them. */
    int bad = sm100_rt_h2d_async(d, da, a, na * 4) || sm100_rt_h2d_async(d, db, b, nb * 4) ||
              sm100_rt_h2d_async(d, dc, c, nc * 4) ||
              sm100_rt_launch(d, &k, 1, 1, 1, 32, 1, 1, 0, args) ||
              sm100_rt_d2h(d, c, dc, nc * 4);
    pthread_mutex_unlock(&g_host_mu);
    if (bad) host_die(what);
}

void matmul(float *a, float *b, float *c, int stride_am, int stride_ak, int stride_bk,
            int stride_bn, int stride_cm, int stride_cn, int nthreads)
{
    tile_matmul("matmul", a, b, c, 4, 4, stride_am, stride_ak, stride_bk, stride_bn,
                stride_cm, stride_cn, 0, nthreads);
}

void matmul_k(float *a, float *b, float *c, int K, int stride_am, int stride_ak, int stride_bk,
              int stride_bn, int stride_cm, int stride_cn, int nthreads)
{
    tile_matmul("matmul_k", a, b, c, K, 2, stride_am, stride_ak, stride_bk, stride_bn,
                stride_cm, stride_cn, 1, nthreads);
}

/* ---- fp32 GEMM, 3xTF32 on tcgen05 ---- */

static int tmap_2d(sm100_dev_t *dev, CUtensorMap *map, CUdeviceptr base, int rows, int K, int box_rows)
{
    /* Row-major [rows][K] fp32; a box is 32 floats (one 128-byte swizzle row) wide. */
    cuuint64_t dims[2] = { (cuuint64_t)K, (cuuint64_t)rows };
    cuuint64_t strides[1] = { (cuuint64_t)K * 4 };
    cuuint32_t box[2] = { 32, (cuuint32_t)box_rows };
    cuuint32_t estr[2] = { 1, 1 };
    CUresult cr = dev->api->TensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)(uintptr_t)base,
                                                 dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return cr == CUDA_SUCCESS ? SM100_OK : sm100_fail(dev, "cuTensorMapEncodeTiled", cr);
}

int booth_sm100_gemm(sm100_dev_t *dev, sm100_ptr_t c, sm100_ptr_t a, sm100_ptr_t b, int M, int N, int K)
{
    return booth_sm100_gemm_ex(dev, c, a, b, M, N, K, 0);
}

int booth_sm100_gemm_wait_limit(sm100_dev_t *dev, unsigned ms)
{
    if (!dev || ms < 1 || ms > 60000) return bad_arg(dev, "booth_sm100_gemm_wait_limit: 1 to 60000 ms");
    dev->gemm_wait_ms = ms;
    return SM100_OK;
}

/* The four tensor maps of a GEMM describe the planes in the workspace; they depend
 * only on where the workspace lies and on the padded extents, so they are encoded
 * once and reused while those repeat (a benchmark loop, a solver's iterations). */
static int gemm_maps(sm100_dev_t *dev, CUdeviceptr ws, int Mp, int Np, int Kp, int box_b, CUtensorMap **out)
{
    if (!dev->gemm_maps) {
        void *p = NULL;
        if (posix_memalign(&p, 64, 4 * sizeof(CUtensorMap)) != 0) return bad_arg(dev, "out of host memory");
        dev->gemm_maps = (CUtensorMap *)p;
        dev->gemm_maps_key.valid = 0;
    }
    *out = dev->gemm_maps;
    if (dev->gemm_maps_key.valid && dev->gemm_maps_key.ws == ws && dev->gemm_maps_key.Mp == Mp &&
        dev->gemm_maps_key.Np == Np && dev->gemm_maps_key.Kp == Kp && dev->gemm_maps_key.box_b == box_b)
        return SM100_OK;
    dev->gemm_maps_key.valid = 0;
    const size_t a_bytes = (size_t)Mp * Kp * 4, b_bytes = (size_t)Np * Kp * 4;
    int rc;
    if ((rc = tmap_2d(dev, &dev->gemm_maps[0], ws, Mp, Kp, 128)) != SM100_OK) return rc;
    if ((rc = tmap_2d(dev, &dev->gemm_maps[1], ws + a_bytes, Mp, Kp, 128)) != SM100_OK) return rc;
    if ((rc = tmap_2d(dev, &dev->gemm_maps[2], ws + 2 * a_bytes, Np, Kp, box_b)) != SM100_OK) return rc;
    if ((rc = tmap_2d(dev, &dev->gemm_maps[3], ws + 2 * a_bytes + b_bytes, Np, Kp, box_b)) != SM100_OK) return rc;
    dev->gemm_maps_key.ws = ws; dev->gemm_maps_key.Mp = Mp; dev->gemm_maps_key.Np = Np;
    dev->gemm_maps_key.Kp = Kp; dev->gemm_maps_key.box_b = box_b; dev->gemm_maps_key.valid = 1;
    return SM100_OK;
}

/* How many CTA pairs of the persistent kernel the GPU holds at once: asked of the
 * driver once per device (cuOccupancyMaxActiveClusters), else one pair per two SMs.
 * BOOTH_SM100_GEMM_CLUSTERS overrides. The grid never exceeds it, so every cluster
 * is resident and the one cross-cluster wait (for a partial sum) cannot starve. */
static int gemm_cluster_capacity(sm100_dev_t *dev)
{
    if (dev->gemm_clusters > 0) return dev->gemm_clusters;
    int n = dev->sm_count / 2;
    if (dev->api->OccupancyMaxActiveClusters) {
        CUlaunchAttribute attr;
        memset(&attr, 0, sizeof attr);
        attr.id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
        attr.value.clusterDim.x = 2; attr.value.clusterDim.y = 1; attr.value.clusterDim.z = 1;
        CUlaunchConfig cfg;
        memset(&cfg, 0, sizeof cfg);
        cfg.gridDimX = (unsigned)(dev->sm_count & ~1); cfg.gridDimY = 1; cfg.gridDimZ = 1;
        cfg.blockDimX = 384; cfg.blockDimY = 1; cfg.blockDimZ = 1;
        cfg.sharedMemBytes = 197632;
        cfg.hStream = dev->stream;
        cfg.attrs = &attr; cfg.numAttrs = 1;
        /* the kernel's dynamic shared memory limit must be raised before the question makes sense */
        if (dev->api->FuncSetAttribute(dev->k[SM100_K_GEMM_PERSIST], CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, 197632) == CUDA_SUCCESS) {
            int got = 0;
            if (dev->api->OccupancyMaxActiveClusters(&got, dev->k[SM100_K_GEMM_PERSIST], &cfg) == CUDA_SUCCESS && got > 0 && got < n)
                n = got;
        }
    }
    n = env_int("BOOTH_SM100_GEMM_CLUSTERS", n, 1, 256);
    if (n < 1) { bad_arg(dev, "booth_sm100_gemm: the GPU holds no CTA pair of the persistent kernel"); return 0; }
    dev->gemm_clusters = n;
    return n;
}

int booth_sm100_gemm_ex(sm100_dev_t *dev, sm100_ptr_t c, sm100_ptr_t a, sm100_ptr_t b, int M, int N, int K,
                        unsigned flags)
{
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    if (!c || !a || !b || M <= 0 || N <= 0 || K <= 0 || ((a | b | c) & 3) ||
        (long long)M + 255 > INT_MAX || (long long)N + 255 > INT_MAX || (long long)K + 31 > INT_MAX)
        return bad_arg(dev, "booth_sm100_gemm: need positive M, N, K and 4-byte aligned pointers");
    /* 256-wide tiles. The 128-wide forms (BOOTH_SM100_GEMM_BN=128) fill the last
     * wave of mid-sized problems better but measured slower everywhere (4096^3:
     * 184 against 226 TFLOP/s with CTA pairs): the narrower MMA re-reads A twice as
     * often from shared memory. */
    const int bn = env_int("BOOTH_SM100_GEMM_BN", 256, 128, 256) == 128 ? 128 : 256;
    /* Padded extents: whole tiles. CTA pairs (256-row tiles) when the rows come
     * out even, or when M is large enough that rounding up to 256 wastes little;
     * BOOTH_SM100_GEMM_2CTA=0 forces the one-CTA form. */
    int Mp = (M + 127) / 128 * 128;
    int pair = env_int("BOOTH_SM100_GEMM_2CTA", 1, 0, 1) && (Mp % 256 == 0 || M >= 2048);
    if (pair) Mp = (M + 255) / 256 * 256;
    int Np = (N + 255) / 256 * 256, Kp = (K + 31) / 32 * 32;
    const size_t a_bytes = (size_t)Mp * Kp * 4, b_bytes = (size_t)Np * Kp * 4, planes = 2 * a_bytes + 2 * b_bytes;
    /* The persistent form (one cluster per SM pair walks a list of tiles, the tail's K
     * chunks dealt out evenly) serves the 256 x 256 pair tiles; BOOTH_SM100_GEMM_PERSIST=0
     * falls back to one tile per cluster. Its workspace:
     *   [ 16 KiB header: 16 hand-over words per cluster, compared with a per-call tag,
     *     so nothing is cleared between calls (a fresh workspace is zeros, a tag never is) ]
     *   [ planes A_hi, A_lo, Bt_hi, Bt_lo ]
     *   [ one 256 KiB slot of partial sums per cluster ]
     * (the other forms leave the header alone and use the planes only). */
    const int persist = pair && bn == 256 && env_int("BOOTH_SM100_GEMM_PERSIST", 1, 0, 1);
    int clusters = 0;
    if (persist && (clusters = gemm_cluster_capacity(dev)) < 1) return SM100_ERR_CUDA;
    const size_t hdr = 256 * 16 * 4, slot_bytes = (size_t)2 * 8 * 128 * 32 * 4;
    CUdeviceptr ws = sm100_gemm_ws(dev, hdr + planes + (size_t)clusters * slot_bytes);
    if (!ws) return SM100_ERR_CUDA;
    const CUdeviceptr base = ws + hdr;
    CUdeviceptr a_hi = base, a_lo = base + a_bytes, b_hi = base + 2 * a_bytes, b_lo = b_hi + b_bytes;
    CUdeviceptr partial_ws = base + planes, flags_ptr = ws;
    CUtensorMap *maps = NULL;
    if ((rc = gemm_maps(dev, base, Mp, Np, Kp, pair ? bn / 2 : bn, &maps)) != SM100_OK) return rc;

    const unsigned shmem = 197632;     /* stages * stage bytes + 1024: 2 x 96 KB, 3 x 64 KB or 4 x 48 KB, the same for every form */
    if (!dev->gemm_smem_set) {
        CUresult cr = CUDA_SUCCESS;
        static const int forms[5] = { SM100_K_GEMM_TF32X3, SM100_K_GEMM_TF32X3_N128, SM100_K_GEMM_TF32X3_2CTA,
                                      SM100_K_GEMM_TF32X3_2CTA_N128, SM100_K_GEMM_PERSIST };
        for (int i = 0; i < 5 && cr == CUDA_SUCCESS; i++)
            cr = dev->api->FuncSetAttribute(dev->k[forms[i]], CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)shmem);
        if (cr != CUDA_SUCCESS) return sm100_fail(dev, "raising the GEMM kernel's shared memory limit", cr);
        dev->gemm_smem_set = 1;
    }
    CUdeviceptr status = dev->scratch + SM100_SCRATCH_GEMM_STATUS;
    if (!dev->gemm_pending) {
        CUresult cr = dev->api->MemsetD8Async(status, 0, 4, dev->stream);
        if (cr != CUDA_SUCCESS) return sm100_fail(dev, "clearing the GEMM status word", cr);
    }

    int tiles = pair && bn == 256 ? (Mp / 256) * (Np / 256) : 0, split_from = tiles, shared = 0, tail_split = 0, launch_clusters = 0;
    if (persist) {
        /* The tail (tiles % clusters) is dealt out by K chunks of 128 when that leaves every
         * cluster at least four chunks and a real share of the pairs would otherwise idle. */
        const int rem = tiles % clusters, nck = (Kp / 32 + 3) / 4;
        tail_split = rem > 0 && rem <= clusters - clusters / 8 && (long long)rem * nck / clusters >= 4 &&
                     env_int("BOOTH_SM100_GEMM_SPLIT_TAIL", 1, 0, 1);
        launch_clusters = tail_split || tiles >= clusters ? clusters : tiles;
    } else if (tiles && env_int("BOOTH_SM100_GEMM_SPLIT_TAIL", 1, 0, 1)) {
        /* One tile per cluster, a short last wave: when the tiles left over after the full
         * waves occupy at most half of the SM pairs, each of them is shared by two clusters
         * that take half of K each and add into a zeroed C (4096^3: 256 tiles on 74 pairs are
         * 3 waves + 34 tiles; sharing them turns the fourth wave into half a wave). */
        const int slots = dev->sm_count / 2, rem = slots > 0 ? tiles % slots : 0;
        if (rem > 0 && 2 * rem <= slots && (Kp / 32) % 2 == 0 && Kp >= 1024) { shared = rem; split_from = tiles - rem; }
    }

    /* 1. One launch ahead of the contraction: split A, split + transpose B (both write
     * zeros into the padding) and zero the tiles of C that clusters of the one-tile form
     * share. A is split one 16-byte chunk per thread
     * (measured 6.0 / 6.7 TB/s at 4096^2 / 8192^2 against 5.2 / 5.7 for eight persistent
     * blocks per SM), B in 64 x 64 tiles. The planes of B can stay from the previous call
     * when the caller says B has not changed and they are still where that call put them. */
    const int keep_b = (flags & BOOTH_GEMM_B_UNCHANGED) && dev->gemm_b.valid && dev->gemm_b.b == b &&
                       dev->gemm_b.planes == b_hi && dev->gemm_b.K == K && dev->gemm_b.N == N;
    if (!keep_b) dev->gemm_b.valid = 0;
    long long a_chunks = (long long)Mp * (Kp / 4), a_blocks = (a_chunks + 255) / 256;
    long long b_blocks = keep_b ? 0 : (long long)(Np / 64) * ((Kp + 63) / 64);
    if (a_blocks + b_blocks + shared > 0x7fffffffll) a_blocks = 0x7fffffffll - b_blocks - shared;
    if (a_blocks < 1) return bad_arg(dev, "booth_sm100_gemm: operands too large for one launch");
    unsigned ua = (unsigned)a_blocks, ub = (unsigned)b_blocks;
    int tiles_n = Np / 256;
    void *pa[] = { &a, &a_hi, &a_lo, &M, &K, &Mp, &Kp, &b, &b_hi, &b_lo, &N, &Np, &c, &tiles_n, &split_from, &ua, &ub };
    if ((rc = sm100_launch_k_overlapped(dev, SM100_K_GEMM_PREPASS, ua + ub + (unsigned)shared, 256, 0, pa)) != SM100_OK) return rc;

    /* 2. The tiled contraction. Barrier waits inside the kernel give up after
     * gemm_wait_ms (booth_sm100_gemm_wait_limit; 4 s unless set). With
     * BOOTH_GEMM_TEST_SILENT_PRODUCER the TMA producers issue nothing, the waits run
     * out, the kernel reports and returns: the tests' way to see that path. */
    unsigned long long wait_ns = (unsigned long long)dev->gemm_wait_ms * 1000000ull;
    int silent = (flags & BOOTH_GEMM_TEST_SILENT_PRODUCER) ? 1 : 0;
    if (persist) {
        if (++dev->gemm_epoch == 0) dev->gemm_epoch = 1;            /* this call's tag; zero is what a fresh workspace holds */
        unsigned epoch = dev->gemm_epoch;
        void *gp[] = { &maps[0], &maps[1], &maps[2], &maps[3], &c, &M, &N, &Np, &Kp, &tail_split, &status, &wait_ns, &silent,
                       &partial_ws, &flags_ptr, &epoch };
        rc = sm100_launch_k3_overlapped(dev, SM100_K_GEMM_PERSIST, 2u * (unsigned)launch_clusters, 1, 1, 384, 1, 1, shmem, gp);
    } else {
        void *ga[] = { &maps[0], &maps[1], &maps[2], &maps[3], &c, &M, &N, &Np, &Kp, &split_from, &status, &wait_ns, &silent };
        if (pair)
            rc = sm100_launch_k3_overlapped(dev, bn == 256 ? SM100_K_GEMM_TF32X3_2CTA : SM100_K_GEMM_TF32X3_2CTA_N128,
                                            2u * ((unsigned)(Mp / 256) * (unsigned)(Np / bn) + (unsigned)shared), 1, 1, 320, 1, 1, shmem, ga);
        else
            rc = sm100_launch_k3_overlapped(dev, bn == 256 ? SM100_K_GEMM_TF32X3 : SM100_K_GEMM_TF32X3_N128,
                                            (unsigned)(Np / bn), (unsigned)(Mp / 128), 1, 320, 1, 1, shmem, ga);
    }
    if (rc == SM100_OK) {
        dev->gemm_pending = 1;
        if (!keep_b) { dev->gemm_b.b = b; dev->gemm_b.planes = b_hi; dev->gemm_b.K = K; dev->gemm_b.N = N; dev->gemm_b.valid = 1; }
    }
    return rc;
}
