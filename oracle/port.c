/* port.c -- CPU restatement of the reference's x86-64 path for the five workloads.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker, never the product: only
 * the test-suite, the smoke check and the benchmark's cpu_baseline / reference
 * arm may build or call it. The product path is the sm_100a library and fails
 * loudly without it.
 *
 * Each function restates, in plain C, what the reference compiler's x86-64
 * backend (kath --cpu) emits for one kernel source, and exports it under the
 * same symbol and the same CPU-launcher ABI, kernel(params..., nthreads)
 * (src/cpu/cpu_emit.c:386-431,783-790: the body runs once per
 * tid in [0,nthreads) with blockIdx=0, gridDim=1, blockDim=nthreads).
 * Arithmetic rules carried over from the backend:
 *   - no FMA: every fmul and fadd is rounded on its own, mulss then addss
 *     (src/cpu/cpu_emit.c:538-542)  ->  build with -ffp-contract=off;
 *   - int32 add is a 64-bit add with a 32-bit store, i.e. wraps
 *     (src/cpu/cpu_emit.c:444-446)  ->  unsigned arithmetic here;
 *   - expf(x)=exp2f(x*1.4426950f), logf(x)=log2f(x)*0.6931472f,
 *     sinf/cosf(x)=libm(x*0.15915494f*6.2831855f), sqrtf=sqrtss
 *     (src/ir/bir_lower.c:1757-1811, src/cpu/cpu_emit.c:641-678).
 * Parity pin: tests/test_oracle.py checks these functions bit for bit against
 * the objects kath itself emits (oracle/_ref, built by oracle/Makefile from the
 * reference sources) and against the reference's own fixtures
 * (examples/cpu_launch_vadd.c:31-45, examples/cpu_launch_matmul.c:38-58,
 * tests/diff/vadd_io.h:12-22, tests/numeric/manifest.json:9-25,
 * examples/launch_saxpy.c:54-58); golden outputs of the kath objects are
 * committed under tests/golden/. */
#include <math.h>
#include <stdint.h>

/* tests/tri_vadd.py:6-16 through src/triton/lower.c:659-760: program_id is the
 * (always zero) block id, arange is the thread id, masks are dropped. */
void vector_add(float *x, float *y, float *out, int n_elements, int block_size,
                long long nthreads)
{
    (void)n_elements; (void)block_size;
    for (long long t = 0; t < nthreads; t++)
        out[t] = x[t] + y[t];
}

/* tests/canonical.cu:168-173: y[idx] = a*x[idx] + y[idx], guard idx < n. */
void saxpy(float *y, float *x, float a, int n, long long nthreads)
{
    for (long long t = 0; t < nthreads; t++) {
        if (t < (long long)n) {
            float p = a * x[t];
            y[t] = p + y[t];
        }
    }
}

/* oracle/kernels/reduce_chunk_i32.cu */
void reduce_chunk_i32(int *partial, int *in, int chunk, long long nthreads)
{
    for (long long t = 0; t < nthreads; t++) {
        const int *p = in + t * (long long)chunk;
        uint32_t acc = 0;
        for (int j = 0; j < chunk; j++) acc += (uint32_t)p[j];
        partial[t] = (int)acc;
    }
}

/* oracle/kernels/reduce_chunk_f32.cu */
void reduce_chunk_f32(float *partial, float *in, int chunk, long long nthreads)
{
    for (long long t = 0; t < nthreads; t++) {
        const float *p = in + t * (long long)chunk;
        float acc = 0.0f;
        for (int j = 0; j < chunk; j++) acc = acc + p[j];
        partial[t] = acc;
    }
}

/* tests/tri_matmul.py:8-25 through src/triton/lower.c:1001-1024: one 4x4 tile,
 * K = 4, tl.dot is a flat left-to-right sum of separately rounded products. */
void matmul(float *a, float *b, float *c, int sam, int sak, int sbk, int sbn,
            int scm, int scn, long long nthreads)
{
    for (long long t = 0; t < nthreads; t++)
        for (int m = 0; m < 4; m++)
            for (int n = 0; n < 4; n++) {
                float acc = a[m * sam] * b[n * sbn];
                for (int k = 1; k < 4; k++) {
                    float pr = a[m * sam + k * sak] * b[k * sbk + n * sbn];
                    acc = acc + pr;
                }
                c[m * scm + n * scn] = acc;
            }
}

/* tests/tri_matmul_k.py:8-23: 4x4 tile, runtime K loop in steps of BLOCK_K = 2;
 * per step acc[m,n] += (a[m,k]*b[k,n] + a[m,k+1]*b[k+1,n]), the inner pair
 * summed first (src/triton/lower.c:1012-1021), accumulators in a zeroed
 * scratch tile (src/triton/lower.c:964-982). */
void matmul_k(float *a, float *b, float *c, int K, int sam, int sak, int sbk,
              int sbn, int scm, int scn, long long nthreads)
{
    for (long long t = 0; t < nthreads; t++) {
        float acc[4][4];
        for (int m = 0; m < 4; m++) for (int n = 0; n < 4; n++) acc[m][n] = 0.0f;
        for (int k = 0; k < K; k += 2)
            for (int m = 0; m < 4; m++)
                for (int n = 0; n < 4; n++) {
                    float p0 = a[m * sam + k * sak] * b[k * sbk + n * sbn];
                    float p1 = a[m * sam + (k + 1) * sak] * b[(k + 1) * sbk + n * sbn];
                    float d = p0 + p1;
                    acc[m][n] = acc[m][n] + d;
                }
        for (int m = 0; m < 4; m++)
            for (int n = 0; n < 4; n++) c[m * scm + n * scn] = acc[m][n];
    }
}

/* ---- Asian-option paths: oracle/kernels/asian_paths.cu ---- */

static float bk_expf(float x) { return exp2f(x * 1.4426950f); }
static float bk_logf(float x) { return log2f(x) * 0.6931472f; }
static float bk_turn(float x) { float t = x * 0.15915494f; return t * 6.2831855f; }
static float bk_sinf(float x) { return sinf(bk_turn(x)); }
static float bk_cosf(float x) { return cosf(bk_turn(x)); }
static float u01(uint32_t x) { return ((float)(x >> 9) + 0.5f) * 1.1920928955078125e-7f; }

static void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1)
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

/* ---- raw Philox words: oracle/kernels/philox_words.cu ---- */
void philox_words(unsigned int *out, unsigned int c0, unsigned int c1, unsigned int c2,
                  unsigned int c3, unsigned int k0, unsigned int k1, long long nthreads)
{
    for (long long t = 0; t < nthreads; t++) {
        uint32_t c[4] = { c0 + (uint32_t)t, c1, c2, c3 };
        philox4x32_10(c, k0, k1);
        for (int i = 0; i < 4; i++) out[4 * t + i] = c[i];
    }
}

void asian_paths(float *arith, float *geom, long long path0, unsigned int k0,
                 unsigned int k1, float s0, float strike, float drift, float vol,
                 int nstep, long long nthreads)
{
    for (long long t = 0; t < nthreads; t++) {
        long long p = path0 + t;
        float s = s0, ls = 0.0f, sum_s = 0.0f, sum_l = 0.0f;
        int ncall = nstep / 4;
        for (int q = 0; q < ncall; q++) {
            uint32_t c[4] = { (uint32_t)p, (uint32_t)q, (uint32_t)((uint64_t)p >> 32), 0 };
            philox4x32_10(c, k0, k1);
            float u1 = u01(c[0]), u2 = u01(c[1]), u3 = u01(c[2]), u4 = u01(c[3]);
            float ra = sqrtf(-2.0f * bk_logf(u1));
            float rb = sqrtf(-2.0f * bk_logf(u3));
            float ta = 6.2831855f * u2, tb = 6.2831855f * u4;
            float z[4];
            z[0] = ra * bk_cosf(ta); z[1] = ra * bk_sinf(ta);
            z[2] = rb * bk_cosf(tb); z[3] = rb * bk_sinf(tb);
            for (int i = 0; i < 4; i++) {
                float vz = vol * z[i];
                float x = drift + vz;
                s = s * bk_expf(x);
                ls = ls + x;
                sum_s = sum_s + s;
                sum_l = sum_l + ls;
            }
        }
        float fn = (float)nstep;
        float am = sum_s / fn - strike;
        float gm = s0 * bk_expf(sum_l / fn) - strike;
        arith[t] = am > 0.0f ? am : 0.0f;
        geom[t] = gm > 0.0f ? gm : 0.0f;
    }
}
