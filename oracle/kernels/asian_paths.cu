/* Oracle kernel source (test infrastructure): Asian-option Monte Carlo paths.
 *
 * The reference's own pricer (src/ocaml/Asian.ml:8-72) draws its normals from a
 * counter hash; this source keeps its per-step update
 *     s = s * exp(drift + vol * z)
 * and its Box-Muller transform, and replaces the hash by Philox4x32-10.
 * It is written for the reference compiler's x86-64 backend (kath --cpu):
 *   - one thread per path, launched as kernel(params..., nthreads);
 *   - the high half of a 32x32 product comes from a 64-bit product, because the
 *     backend's 32-bit __umulhi is a widening multiply on sign-extended slots
 *     (src/cpu/cpu_emit.c:448);
 *   - no double arithmetic (the backend emits the ...ss form for every float
 *     op, src/cpu/cpu_emit.c:538-542,622-624): the kernel writes one fp32
 *     payoff pair per path and the host adds them up in double;
 *   - expf/logf/sinf/cosf go through the lowering in src/ir/bir_lower.c:1757-1811:
 *     expf(x) = exp2f(x*1.4426950f), logf(x) = log2f(x)*0.6931472f,
 *     sinf/cosf(x) = libm(x*0.15915494f*6.2831855f).
 * Counter = (path low word, call index q, path high word, 0); key = (k0, k1).
 * Call q yields four uniforms u = ((x >> 9) + 0.5) * 2^-23, exact in fp32 and
 * strictly inside (0,1), and from them the normals of monitoring steps
 * 4q .. 4q+3. nstep must be a multiple of 4. */

__device__ unsigned int mulhi32(unsigned int a, unsigned int b)
{
    unsigned long long p = (unsigned long long)a * (unsigned long long)b;
    return (unsigned int)(p >> 32);
}

__device__ float u01(unsigned int x)
{
    return ((float)(x >> 9) + 0.5f) * 1.1920928955078125e-7f;
}

__global__ void asian_paths(float *arith, float *geom, long long path0,
                            unsigned int k0, unsigned int k1,
                            float s0, float strike, float drift, float vol,
                            int nstep)
{
    int t = threadIdx.x;
    long long p = path0 + (long long)t;
    unsigned int plo = (unsigned int)p;
    unsigned int phi = (unsigned int)(p >> 32);

    float s = s0;
    float ls = 0.0f;
    float sum_s = 0.0f;
    float sum_l = 0.0f;
    int ncall = nstep / 4;

    for (int q = 0; q < ncall; q = q + 1) {
        unsigned int c0 = plo;
        unsigned int c1 = (unsigned int)q;
        unsigned int c2 = phi;
        unsigned int c3 = 0;
        unsigned int ka = k0;
        unsigned int kb = k1;
        for (int r = 0; r < 10; r = r + 1) {
            unsigned int hi0 = mulhi32(0xD2511F53u, c0);
            unsigned int lo0 = 0xD2511F53u * c0;
            unsigned int hi1 = mulhi32(0xCD9E8D57u, c2);
            unsigned int lo1 = 0xCD9E8D57u * c2;
            unsigned int n0 = hi1 ^ c1 ^ ka;
            unsigned int n2 = hi0 ^ c3 ^ kb;
            c0 = n0;
            c1 = lo1;
            c2 = n2;
            c3 = lo0;
            ka = ka + 0x9E3779B9u;
            kb = kb + 0xBB67AE85u;
        }
        float u1 = u01(c0);
        float u2 = u01(c1);
        float u3 = u01(c2);
        float u4 = u01(c3);
        float ra = sqrtf(-2.0f * logf(u1));
        float rb = sqrtf(-2.0f * logf(u3));
        float ta = 6.2831855f * u2;
        float tb = 6.2831855f * u4;
        float z0 = ra * cosf(ta);
        float z1 = ra * sinf(ta);
        float z2 = rb * cosf(tb);
        float z3 = rb * sinf(tb);

        float x0 = drift + vol * z0;
        s = s * expf(x0);
        ls = ls + x0;
        sum_s = sum_s + s;
        sum_l = sum_l + ls;

        float x1 = drift + vol * z1;
        s = s * expf(x1);
        ls = ls + x1;
        sum_s = sum_s + s;
        sum_l = sum_l + ls;

        float x2 = drift + vol * z2;
        s = s * expf(x2);
        ls = ls + x2;
        sum_s = sum_s + s;
        sum_l = sum_l + ls;

        float x3 = drift + vol * z3;
        s = s * expf(x3);
        ls = ls + x3;
        sum_s = sum_s + s;
        sum_l = sum_l + ls;
    }

    float fn = (float)nstep;
    float am = sum_s / fn - strike;
    float gm = s0 * expf(sum_l / fn) - strike;
    float pa = 0.0f;
    float pg = 0.0f;
    if (am > 0.0f) pa = am;
    if (gm > 0.0f) pg = gm;
    arith[t] = pa;
    geom[t] = pg;
}
