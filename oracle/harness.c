/* harness.c -- host driver that runs the CPU-launcher kernels on T pthreads.
 *
 * TEST INFRASTRUCTURE ONLY (checker and timed CPU baseline; never the product).
 *
 * It is linked twice: with the objects the reference compiler emits
 * (oracle/_ref/libbooth_ref.so) and with the C restatement in port.c
 * (oracle/libbooth_port.so). Both libraries export the same orc_* entry points,
 * so a test can run either and compare them.
 *
 * One call of a CPU-launcher kernel is one block of serially executed threads
 * (src/cpu/cpu_emit.c:426-431,783-790), so the harness cuts every workload into
 * disjoint ranges, hands each range to the kernel with offset pointers and the
 * range length as nthreads, and spreads the ranges over pthreads. The emitted
 * kernels keep all state in their own stack frame, so concurrent calls on
 * disjoint data are safe. nthreads is declared long long because the emitted
 * prologue stores and compares the whole 64-bit slot (src/cpu/cpu_emit.c:410-429). */
#define _POSIX_C_SOURCE 200809L
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include <unistd.h>

extern void vector_add(float *x, float *y, float *out, int n_elements,
                       int block_size, long long nthreads);
extern void saxpy(float *y, float *x, float a, int n, long long nthreads);
extern void reduce_chunk_i32(int *partial, int *in, int chunk, long long nthreads);
extern void reduce_chunk_f32(float *partial, float *in, int chunk, long long nthreads);
extern void matmul(float *a, float *b, float *c, int sam, int sak, int sbk,
                   int sbn, int scm, int scn, long long nthreads);
extern void matmul_k(float *a, float *b, float *c, int K, int sam, int sak,
                     int sbk, int sbn, int scm, int scn, long long nthreads);
extern void asian_paths(float *arith, float *geom, long long path0,
                        unsigned int k0, unsigned int k1, float s0, float strike,
                        float drift, float vol, int nstep, long long nthreads);

extern void philox_words(unsigned int *out, unsigned int c0, unsigned int c1,
                         unsigned int c2, unsigned int c3, unsigned int k0,
                         unsigned int k1, long long nthreads);

/* ---- a small static-schedule parallel-for ---- */

typedef void (*orc_body_fn)(void *ctx, long long lo, long long hi);

typedef struct {
    orc_body_fn fn; void *ctx; long long lo, hi;
} orc_job_t;

static void *orc_tramp(void *p)
{
    orc_job_t *j = (orc_job_t *)p;
    if (j->hi > j->lo) j->fn(j->ctx, j->lo, j->hi);
    return NULL;
}

/* Splits [0,count) into `threads` contiguous ranges whose bounds are multiples
 * of `grain` (except the last) and runs fn on each. */
static void orc_parallel(orc_body_fn fn, void *ctx, long long count,
                         long long grain, int threads)
{
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    if (grain < 1) grain = 1;
    long long units = (count + grain - 1) / grain;
    if (units < threads) threads = (int)(units > 0 ? units : 1);
    pthread_t tid[256];
    orc_job_t job[256];
    for (int t = 0; t < threads; t++) {
        long long u0 = units * t / threads, u1 = units * (t + 1) / threads;
        job[t].fn = fn; job[t].ctx = ctx;
        job[t].lo = u0 * grain;
        job[t].hi = u1 * grain < count ? u1 * grain : count;
    }
    for (int t = 1; t < threads; t++)
        pthread_create(&tid[t], NULL, orc_tramp, &job[t]);
    orc_tramp(&job[0]);
    for (int t = 1; t < threads; t++) pthread_join(tid[t], NULL);
}

int orc_cores(void)
{
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

double orc_now(void)
{
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

/* One kernel call never gets more than this many threads, so n_elements and
 * the int parameters of the kernels stay far from 2^31. */
#define ORC_CALL_MAX (1LL << 24)

/* ---- vadd ---- */
typedef struct { float *x, *y, *out; } vadd_ctx;
static void vadd_body(void *c, long long lo, long long hi)
{
    vadd_ctx *v = (vadd_ctx *)c;
    for (long long i = lo; i < hi; i += ORC_CALL_MAX) {
        long long m = hi - i < ORC_CALL_MAX ? hi - i : ORC_CALL_MAX;
        vector_add(v->x + i, v->y + i, v->out + i, (int)m, 256, m);
    }
}
void orc_vadd(float *x, float *y, float *out, long long n, int threads)
{
    vadd_ctx c = { x, y, out };
    orc_parallel(vadd_body, &c, n, 4096, threads);
}

/* ---- saxpy ---- */
typedef struct { float *y, *x; float a; } saxpy_ctx;
static void saxpy_body(void *c, long long lo, long long hi)
{
    saxpy_ctx *v = (saxpy_ctx *)c;
    for (long long i = lo; i < hi; i += ORC_CALL_MAX) {
        long long m = hi - i < ORC_CALL_MAX ? hi - i : ORC_CALL_MAX;
        saxpy(v->y + i, v->x + i, v->a, (int)m, m);
    }
}
void orc_saxpy(float *y, float *x, float a, long long n, int threads)
{
    saxpy_ctx c = { y, x, a };
    orc_parallel(saxpy_body, &c, n, 4096, threads);
}

/* ---- chunked sums ----
 * partial[] has ceil(n/chunk) entries; the last chunk may be short and is
 * produced by a one-thread call with chunk = its length. */
typedef struct { void *partial; void *in; long long n; int chunk; int is_f32; } red_ctx;
static void red_body(void *c, long long lo, long long hi)   /* lo,hi in chunks */
{
    red_ctx *r = (red_ctx *)c;
    long long full = r->n / r->chunk;
    for (long long t = lo; t < hi; ) {
        long long m = hi - t;
        if (t < full) {
            if (t + m > full) m = full - t;
            if (m > (1 << 18)) m = 1 << 18;
            if (r->is_f32)
                reduce_chunk_f32((float *)r->partial + t, (float *)r->in + t * r->chunk, r->chunk, m);
            else
                reduce_chunk_i32((int *)r->partial + t, (int *)r->in + t * r->chunk, r->chunk, m);
        } else {
            int tail = (int)(r->n - full * r->chunk);
            m = 1;
            if (r->is_f32)
                reduce_chunk_f32((float *)r->partial + t, (float *)r->in + t * r->chunk, tail, 1);
            else
                reduce_chunk_i32((int *)r->partial + t, (int *)r->in + t * r->chunk, tail, 1);
        }
        t += m;
    }
}

/* Wrapping int32 sum of in[0..n). */
int orc_reduce_i32(int *in, long long n, int chunk, int threads)
{
    if (n <= 0) return 0;
    long long np = (n + chunk - 1) / chunk;
    int *partial = (int *)malloc((size_t)np * sizeof(int));
    red_ctx c = { partial, in, n, chunk, 0 };
    orc_parallel(red_body, &c, np, 1, threads);
    uint32_t acc = 0;
    for (long long i = 0; i < np; i++) acc += (uint32_t)partial[i];
    free(partial);
    return (int)acc;
}

/* fp32 chunk sums combined in double, in chunk order. Returns the double; the
 * fp32 result of the workload is that value rounded to float. */
double orc_reduce_f32(float *in, long long n, int chunk, int threads)
{
    if (n <= 0) return 0.0;
    long long np = (n + chunk - 1) / chunk;
    float *partial = (float *)malloc((size_t)np * sizeof(float));
    red_ctx c = { partial, in, n, chunk, 1 };
    orc_parallel(red_body, &c, np, 1, threads);
    double acc = 0.0;
    for (long long i = 0; i < np; i++) acc += (double)partial[i];
    free(partial);
    return acc;
}

/* Plain double-precision sum, the ground truth quoted beside the fp32 result. */
typedef struct { float *in; double part[256]; long long lo[256]; int nslot; pthread_mutex_t mu; } f64_ctx;
static void f64_body(void *c, long long lo, long long hi)
{
    f64_ctx *f = (f64_ctx *)c;
    double acc = 0.0;
    for (long long i = lo; i < hi; i++) acc += (double)f->in[i];
    pthread_mutex_lock(&f->mu);
    f->part[f->nslot] = acc; f->lo[f->nslot] = lo; f->nslot++;
    pthread_mutex_unlock(&f->mu);
}
double orc_sum_f64(float *in, long long n, int threads)
{
    f64_ctx c; memset(&c, 0, sizeof c); c.in = in;
    pthread_mutex_init(&c.mu, NULL);
    orc_parallel(f64_body, &c, n, 4096, threads);
    double acc = 0.0;
    for (int i = 0; i < c.nslot; i++) acc += c.part[i];
    pthread_mutex_destroy(&c.mu);
    return acc;
}

/* ---- GEMM by 4x4 tiles: tests/tri_matmul_k.py called once per tile with
 * offset base pointers, as examples/cpu_launch_matmul.c:44 calls the single
 * tile. rows4[] lists the 4-row blocks of C to compute (NULL = all of them),
 * so a large GEMM can be checked on a sample of row blocks; the rows of C do
 * not depend on one another. */
typedef struct { float *a, *b, *c; int M, N, K; const int *rows4; } mm_ctx;
static void mm_body(void *cx, long long lo, long long hi)
{
    mm_ctx *g = (mm_ctx *)cx;
    for (long long r = lo; r < hi; r++) {
        int mb = g->rows4 ? g->rows4[r] : (int)r;
        for (int nb = 0; nb < g->N / 4; nb++)
            matmul_k(g->a + (size_t)mb * 4 * g->K, g->b + (size_t)nb * 4,
                     g->c + (size_t)mb * 4 * g->N + (size_t)nb * 4,
                     g->K, g->K, 1, g->N, 1, g->N, 1, 1);
    }
}
void orc_matmul(float *a, float *b, float *c, int M, int N, int K,
                const int *rows4, int nrows4, int threads)
{
    mm_ctx g = { a, b, c, M, N, K, rows4 };
    orc_parallel(mm_body, &g, rows4 ? nrows4 : M / 4, 1, threads);
}

/* Single 4x4x4 tile, the call of examples/cpu_launch_matmul.c:44. */
void orc_matmul_tile(float *a, float *b, float *c, int sam, int sak, int sbk,
                     int sbn, int scm, int scn)
{
    matmul(a, b, c, sam, sak, sbk, sbn, scm, scn, 1);
}

/* ---- Asian option: payoffs per path from the kernel, summed in double on the
 * host in path order within fixed blocks of ORC_MC_BLOCK paths, block sums
 * then added in block order, so the result does not depend on `threads`. */
#define ORC_MC_BLOCK 4096
typedef struct {
    long long path0, npaths; unsigned k0, k1; float s0, strike, drift, vol; int nstep;
    double *bsum;               /* 2 doubles per block */
    float *arith_out, *geom_out;/* optional per-path outputs */
} mc_ctx;
static void mc_body(void *cx, long long lo, long long hi)   /* in blocks */
{
    mc_ctx *m = (mc_ctx *)cx;
    float *pa = (float *)malloc(ORC_MC_BLOCK * sizeof(float));
    float *pg = (float *)malloc(ORC_MC_BLOCK * sizeof(float));
    for (long long b = lo; b < hi; b++) {
        long long first = b * ORC_MC_BLOCK;
        long long cnt = m->npaths - first < ORC_MC_BLOCK ? m->npaths - first : ORC_MC_BLOCK;
        asian_paths(pa, pg, m->path0 + first, m->k0, m->k1, m->s0, m->strike,
                    m->drift, m->vol, m->nstep, cnt);
        double sa = 0.0, sg = 0.0;
        for (long long i = 0; i < cnt; i++) { sa += (double)pa[i]; sg += (double)pg[i]; }
        m->bsum[2 * b] = sa; m->bsum[2 * b + 1] = sg;
        if (m->arith_out) memcpy(m->arith_out + first, pa, (size_t)cnt * sizeof(float));
        if (m->geom_out) memcpy(m->geom_out + first, pg, (size_t)cnt * sizeof(float));
    }
    free(pa); free(pg);
}
/* sums[0] = sum of arithmetic payoffs, sums[1] = sum of geometric payoffs
 * (undiscounted). arith_out / geom_out may be NULL. */
void orc_asian(long long path0, long long npaths, unsigned k0, unsigned k1,
               float s0, float strike, float drift, float vol, int nstep,
               int threads, double *sums, float *arith_out, float *geom_out)
{
    long long nb = (npaths + ORC_MC_BLOCK - 1) / ORC_MC_BLOCK;
    mc_ctx m = { path0, npaths, k0, k1, s0, strike, drift, vol, nstep,
                 (double *)calloc((size_t)(nb > 0 ? nb : 1) * 2, sizeof(double)),
                 arith_out, geom_out };
    orc_parallel(mc_body, &m, nb, 1, threads);
    double sa = 0.0, sg = 0.0;
    for (long long b = 0; b < nb; b++) { sa += m.bsum[2 * b]; sg += m.bsum[2 * b + 1]; }
    free(m.bsum);
    sums[0] = sa; sums[1] = sg;
}

/* ---- Philox4x32-10: the kernel object's words, and the seeded input stream ---- */

/* nblocks output blocks of the philox_words kernel (the reference compiler's
 * object in libbooth_ref, the restatement in libbooth_port): counter
 * (ctr[0] + t, ctr[1], ctr[2], ctr[3]), key (key[0], key[1]). */
void orc_philox_kernel(const unsigned *ctr, const unsigned *key, long long nblocks, unsigned *out)
{
    philox_words(out, ctr[0], ctr[1], ctr[2], ctr[3], key[0], key[1], nblocks);
}

/* The harness's own statement of the generator, used by orc_fill below to make
 * benchmark inputs without touching the product library. */
static void orc_philox_block(uint32_t c[4], uint32_t k0, uint32_t k1)
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

void orc_philox_host(const unsigned *ctr, const unsigned *key, unsigned *out)
{
    uint32_t c[4] = { ctr[0], ctr[1], ctr[2], ctr[3] };
    orc_philox_block(c, key[0], key[1]);
    for (int i = 0; i < 4; i++) out[i] = c[i];
}

/* The workloads' seeded input stream: element i is lane i%4 of the block with
 * counter (i/4 low word, i/4 high word, 0, 0) and key (seed, stream).
 *   kind 0: float in [-1,1)  2u-1, u = (x >> 8) * 2^-24      kind 1: float u in [0,1)
 *   kind 2: int32 in [-1000,1000]  (int)(x % 2001) - 1000    kind 3: the raw word x
 * dst[0] is element `first`. */
typedef struct { uint32_t *dst; long long first; uint32_t seed, stream; int kind; } fill_ctx;
static void fill_body(void *cx, long long lo, long long hi)
{
    fill_ctx *f = (fill_ctx *)cx;
    long long i = lo;
    while (i < hi) {
        long long e = f->first + i;
        unsigned long long ctr = (unsigned long long)e >> 2;
        uint32_t c[4] = { (uint32_t)ctr, (uint32_t)(ctr >> 32), 0, 0 };
        orc_philox_block(c, f->seed, f->stream);
        for (int l = (int)(e & 3); l < 4 && i < hi; l++, i++) {
            uint32_t x = c[l], v = x;
            if (f->kind == 2) {
                v = (uint32_t)((int)(x % 2001u) - 1000);
            } else if (f->kind != 3) {
                float u = (float)(x >> 8) * 5.9604644775390625e-8f;
                float g = f->kind == 0 ? 2.0f * u - 1.0f : u;
                memcpy(&v, &g, 4);
            }
            f->dst[i] = v;
        }
    }
}
void orc_fill(void *dst, long long first, long long n, unsigned seed, unsigned stream, int kind, int threads)
{
    fill_ctx c = { (uint32_t *)dst, first, seed, stream, kind };
    orc_parallel(fill_body, &c, n, 4096, threads);
}
