// asian.cu -- Asian-option Monte Carlo pricer for sm_100a, one path per thread.
//
// The model is the reference's pricer (src/ocaml/Asian.ml:32-72): per monitoring
// step s = s * exp(drift + vol*z), arithmetic-average call payoff, normals from
// Box-Muller; its counter-hash generator (src/ocaml/Asian.ml:8-27) is replaced by
// Philox4x32-10 and a geometric-average payoff is priced beside the arithmetic
// one. Everything a path needs lives in registers: the Philox state, the
// running price, its logarithm and the two running sums. Nothing is read from
// memory and only the reduced sums are written, so the kernel is bound by the
// special-function unit (ex2, lg2, sqrt, sin, cos: three MUFU operations per
// path-step) and by the generator's wide integer products on the heavy FMA pipe
// (pipe_probe.cu times the two groups alone), not by HBM.
//
// Random stream, identical to the CPU statement of the workload:
//   counter = (path low word, call index q, path high word, 0), key = (k0, k1);
//   call q gives four words x -> u = ((x >> 9) + 0.5) * 2^-23  (exact, in (0,1));
//   (u1,u2) and (u3,u4) give two Box-Muller pairs = the normals of steps 4q..4q+3.
// The uniform is formed without an integer-to-float conversion: the 23 bits are
// placed in the mantissa of 1.0f and (1 - 2^-24) is subtracted, which is exact.
//
// Two arithmetic flavours of the same path:
//   PRECISE  every operation rounded separately in the order of the CPU
//            statement (no FMA contraction), log2f/sinf/cosf/sqrtf from the CUDA
//            math library and 2^x from a polynomial on the FMA pipe (exp2_fma),
//            with the reference compiler's scalings
//            (src/ir/bir_lower.c:1757-1811): exp(x) = exp2(x*1.4426950f),
//            log(x) = log2(x)*0.6931472f, sin/cos(x) = f(x*0.15915494f*6.2831855f);
//   FAST     MUFU approximations (ex2/lg2/sqrt/sin/cos .approx), the step carried
//            in base-2 logarithms (drift and vol pre-scaled by log2(e), vol folded
//            into the Box-Muller radius so that one FMA forms the exponent), the
//            floating-point work of a Philox call on the packed fp32x2 forms, and
//            the price rebuilt from its running logarithm, s_j = s0 * 2^(l_j),
//            instead of a 252-long multiply chain.
// Payoffs are accumulated in double per thread, then warp shuffle -> shared ->
// per-block partials -> the block that takes the last ticket adds them in index
// order (no block waits for another).
#include "common.cuh"

// The 23 random bits as the mantissa of a float in [1, 2).
// One funnel shift, (0x7F : x) >> 9, is 0x3F800000 | (x >> 9). (Beside the scalar floating-point
// code of the earlier version a shift and an OR were 2 % faster; beside the packed forms the single
// instruction is, 4.89e9 against 4.80e9 paths/s, same bits.)
__device__ __forceinline__ float mantissa_word(uint32_t x) { return __uint_as_float(__funnelshift_r(x, 0x7Fu, 9)); }

__device__ __forceinline__ float u01(uint32_t x)
{
    // The mantissa word minus (1 - 2^-24): exact.
    return __fadd_rn(mantissa_word(x), -0.99999994f);
}

__device__ __forceinline__ float mufu_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float mufu_lg2(float x) { float y; asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float mufu_sqrt(float x) { float y; asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float mufu_sin(float x) { float y; asm("sin.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float mufu_cos(float x) { float y; asm("cos.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

// 2^x on the FMA pipe: x = n + f with |f| <= 1/2, e^(f ln 2) by its Taylor series to
// degree 8 (truncation 2e-10), scaled by 2^n through the exponent field. Unlike
// the MUFU ex2 its error has no measurable mean, which matters when 252 of them
// are multiplied together. Valid for |x| < 120.
__device__ __forceinline__ float exp2_fma(float x)
{
    const float n = rintf(x);
    const float t = __fmul_rn(__fsub_rn(x, n), 0.69314718f);
    float p = 2.4801587e-5f;                       // 1/8!
    p = fmaf(p, t, 1.9841270e-4f);                 // 1/7!
    p = fmaf(p, t, 1.3888889e-3f);                 // 1/6!
    p = fmaf(p, t, 8.3333333e-3f);                 // 1/5!
    p = fmaf(p, t, 4.1666667e-2f);                 // 1/4!
    p = fmaf(p, t, 1.6666667e-1f);                 // 1/3!
    p = fmaf(p, t, 0.5f);
    p = fmaf(p, t, 1.0f);
    p = fmaf(p, t, 1.0f);
    return __uint_as_float(__float_as_uint(p) + ((uint32_t)(int)n << 23));
}

struct Payoff { float arith, geom; };

template <bool PRECISE>
__device__ __forceinline__ Payoff asian_path(unsigned long long p, uint32_t k0, uint32_t k1,
                                             float s0, float strike, float drift, float vol, int nstep)
{
    const uint32_t plo = (uint32_t)p, phi = (uint32_t)(p >> 32);
    const int ncall = nstep >> 2;
    float sum_l = 0.0f;
    Payoff out;
    if (PRECISE) {
        float s = s0, ls = 0.0f, sum_s = 0.0f;
        for (int q = 0; q < ncall; q++) {
            const Philox4 r = philox4x32_10(plo, (uint32_t)q, phi, 0u, k0, k1);
            const float u1 = u01(r.x), u2 = u01(r.y), u3 = u01(r.z), u4 = u01(r.w);
            const float ra = __fsqrt_rn(__fmul_rn(-2.0f, __fmul_rn(log2f(u1), 0.6931472f)));
            const float rb = __fsqrt_rn(__fmul_rn(-2.0f, __fmul_rn(log2f(u3), 0.6931472f)));
            const float ta = __fmul_rn(__fmul_rn(__fmul_rn(6.2831855f, u2), 0.15915494f), 6.2831855f);
            const float tb = __fmul_rn(__fmul_rn(__fmul_rn(6.2831855f, u4), 0.15915494f), 6.2831855f);
            float z[4];
            z[0] = __fmul_rn(ra, cosf(ta)); z[1] = __fmul_rn(ra, sinf(ta));
            z[2] = __fmul_rn(rb, cosf(tb)); z[3] = __fmul_rn(rb, sinf(tb));
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float x = __fadd_rn(drift, __fmul_rn(vol, z[i]));
                s = __fmul_rn(s, exp2_fma(__fmul_rn(x, 1.4426950f)));
                ls = __fadd_rn(ls, x);
                sum_s = __fadd_rn(sum_s, s);
                sum_l = __fadd_rn(sum_l, ls);
            }
        }
        const float fn = (float)nstep;
        const float am = __fsub_rn(__fdiv_rn(sum_s, fn), strike);
        const float gm = __fsub_rn(__fmul_rn(s0, exp2_fma(__fmul_rn(__fdiv_rn(sum_l, fn), 1.4426950f))), strike);
        out.arith = am > 0.0f ? am : 0.0f;
        out.geom = gm > 0.0f ? gm : 0.0f;
    } else {
        // Step carried in log2 units: l_j = sum of the first j exponents, s_j = s0 * 2^l_j.
        // The price is rebuilt from its running logarithm at every step instead of
        // being multiplied up: the 252 exponentials of a path do not depend on one
        // another, and, more important, the tiny negative bias of the MUFU ex2
        // (-3e-9 relative per evaluation, measured) is applied once per price instead
        // of compounding over 252 products (which moved the price by -8.4e-6).
        //
        // vol is folded into the Box-Muller radius, vol*sqrt(-2 ln u) = sqrt((-2 ln2 vol^2) log2 u),
        // so a step's exponent is one FMA (radius * cos + drift), and the angle is one FMA of
        // the mantissa word. A Philox call yields two (cos, sin) pairs, i.e. four steps, and
        // its floating-point work runs on the packed fp32x2 forms of sm_100 (two lanes per
        // instruction): 11 instructions a call instead of 22 scalar ones. The running sums
        // are kept as (even step, odd step) pairs and joined at the end. Besides the three
        // MUFU operations of a step, the ten rounds of a call are 20 IMAD.WIDE on the heavy
        // FMA pipe at a quarter of the FP32 rate; fewer FP32 instructions leave that pipe to
        // them (4.79e9 against 4.60e9 paths per second; 4.89e9 with the funnel shift above). (vol below 1e-19, whose square
        // underflows, prices like vol = 0.)
        const float d2s = drift * 1.4426950f, v2 = vol * 1.4426950f;
        const float c_rv = (-2.0f * 0.6931472f) * (v2 * v2);            // -2 ln u * v2^2 = c_rv * log2 u
        const float2 c_rv2 = make_float2(c_rv, c_rv), d2 = make_float2(d2s, d2s);
        const float2 two_pi = make_float2(6.2831855f, 6.2831855f);
        const float2 ang0 = make_float2(-0.99999994f * 6.2831855f, -0.99999994f * 6.2831855f);
        const float2 minus1 = make_float2(-0.99999994f, -0.99999994f);
        float l = 0.0f;
        float2 sum_e2 = make_float2(0.0f, 0.0f), sum_l2 = make_float2(0.0f, 0.0f);
        // Seven Philox calls per trip (252 steps are 9 trips) give the scheduler
        // independent chains; measured 4 % faster than two per trip.
#pragma unroll 7
        for (int q = 0; q < ncall; q++) {
            const Philox4 r = philox4x32_10(plo, (uint32_t)q, phi, 0u, k0, k1);
            const float2 u13 = __fadd2_rn(make_float2(mantissa_word(r.x), mantissa_word(r.z)), minus1);
            const float2 t = __ffma2_rn(make_float2(mantissa_word(r.y), mantissa_word(r.w)), two_pi, ang0);
            const float2 rr = __fmul2_rn(c_rv2, make_float2(mufu_lg2(u13.x), mufu_lg2(u13.y)));
            const float ra = mufu_sqrt(rr.x), rb = mufu_sqrt(rr.y);
            const float2 xa = __ffma2_rn(make_float2(ra, ra), make_float2(mufu_cos(t.x), mufu_sin(t.x)), d2);
            const float2 xb = __ffma2_rn(make_float2(rb, rb), make_float2(mufu_cos(t.y), mufu_sin(t.y)), d2);
            const float2 la = __fadd2_rn(make_float2(l, l), make_float2(xa.x, xa.x + xa.y));
            const float2 lb = __fadd2_rn(make_float2(la.y, la.y), make_float2(xb.x, xb.x + xb.y));
            l = lb.y;
            sum_e2 = __fadd2_rn(sum_e2, make_float2(mufu_ex2(la.x), mufu_ex2(la.y)));
            sum_e2 = __fadd2_rn(sum_e2, make_float2(mufu_ex2(lb.x), mufu_ex2(lb.y)));
            sum_l2 = __fadd2_rn(sum_l2, la);
            sum_l2 = __fadd2_rn(sum_l2, lb);
        }
        const float sum_e = sum_e2.x + sum_e2.y;
        sum_l = sum_l2.x + sum_l2.y;
        const float inv_n = 1.0f / (float)nstep;
        const float am = s0 * (sum_e * inv_n) - strike;
        const float gm = s0 * exp2_fma(sum_l * inv_n) - strike;      // once per path: the accurate 2^x
        out.arith = am > 0.0f ? am : 0.0f;
        out.geom = gm > 0.0f ? gm : 0.0f;
    }
    return out;
}

__device__ __forceinline__ double warp_sum_d(double v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// out[0..3] = sum arith, sum geom, sum arith^2, sum geom^2 over paths
// [path0, path0+npaths). Launch with a 1-D grid of 1-D blocks whose size is a
// multiple of 32. partials needs 4 doubles per block, ticket starts at zero.
template <bool PRECISE>
__device__ __forceinline__ void asian_mc_body(double *out, unsigned long long path0,
                                              unsigned long long npaths, uint32_t k0, uint32_t k1,
                                              float s0, float strike, float drift, float vol,
                                              int nstep, double *partials, unsigned *ticket)
{
    __shared__ double sh[4][32];
    __shared__ unsigned s_last;
    double a1 = 0.0, g1 = 0.0, a2 = 0.0, g2 = 0.0;
    const unsigned long long T = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < npaths; i += T) {
        const Payoff pf = asian_path<PRECISE>(path0 + i, k0, k1, s0, strike, drift, vol, nstep);
        const double a = (double)pf.arith, g = (double)pf.geom;
        a1 += a; g1 += g; a2 += a * a; g2 += g * g;
    }
    const unsigned lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    a1 = warp_sum_d(a1); g1 = warp_sum_d(g1); a2 = warp_sum_d(a2); g2 = warp_sum_d(g2);
    if (lane == 0) { sh[0][wid] = a1; sh[1][wid] = g1; sh[2][wid] = a2; sh[3][wid] = g2; }
    __syncthreads();
    if (wid == 0) {
        double v[4];
#pragma unroll
        for (int k = 0; k < 4; k++) v[k] = warp_sum_d(lane < nwarp ? sh[k][lane] : 0.0);
        if (lane == 0) {
#pragma unroll
            for (int k = 0; k < 4; k++) partials[4 * blockIdx.x + k] = v[k];
            __threadfence();
            s_last = (atomicAdd(ticket, 1u) == gridDim.x - 1);
        }
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // Last block: 4 warps take one of the four sums each and add the block
    // partials in index order (lane-strided, then the butterfly).
    if (wid < 4) {
        double v = 0.0;
        for (unsigned b = lane; b < gridDim.x; b += 32) v += __ldcg(partials + 4 * b + wid);
        v = warp_sum_d(v);
        if (lane == 0) out[wid] = v;
    }
    if (threadIdx.x == 0) *ticket = 0u;
}

// The second launch bound frees the register budget (116 registers, two blocks per
// SM). The rate hardly depends on it: one to four blocks per SM and one to nine
// Philox calls per trip all land within 3 % of one another.
extern "C" __global__ void __launch_bounds__(256, 1)
asian_mc(double *out, unsigned long long path0, unsigned long long npaths, uint32_t k0, uint32_t k1,
         float s0, float strike, float drift, float vol, int nstep, double *partials, unsigned *ticket)
{
    asian_mc_body<false>(out, path0, npaths, k0, k1, s0, strike, drift, vol, nstep, partials, ticket);
}

extern "C" __global__ void __launch_bounds__(256, 1)
asian_mc_precise(double *out, unsigned long long path0, unsigned long long npaths, uint32_t k0, uint32_t k1,
                 float s0, float strike, float drift, float vol, int nstep, double *partials, unsigned *ticket)
{
    asian_mc_body<true>(out, path0, npaths, k0, k1, s0, strike, drift, vol, nstep, partials, ticket);
}

// Per-path payoffs with the parameter list of the CPU statement of the kernel:
// arith[t], geom[t] for path path0 + t, one thread per path (any 1-D launch;
// threads beyond npaths do nothing).
template <bool PRECISE>
__device__ __forceinline__ void asian_paths_body(float *arith, float *geom, long long path0, long long npaths,
                                                 uint32_t k0, uint32_t k1, float s0, float strike,
                                                 float drift, float vol, int nstep)
{
    const long long T = (long long)gridDim.x * blockDim.x;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < npaths; t += T) {
        const Payoff pf = asian_path<PRECISE>((unsigned long long)(path0 + t), k0, k1, s0, strike, drift, vol, nstep);
        arith[t] = pf.arith;
        geom[t] = pf.geom;
    }
}

extern "C" __global__ void asian_paths(float *arith, float *geom, long long path0, long long npaths,
                                       uint32_t k0, uint32_t k1, float s0, float strike,
                                       float drift, float vol, int nstep)
{
    asian_paths_body<false>(arith, geom, path0, npaths, k0, k1, s0, strike, drift, vol, nstep);
}

extern "C" __global__ void asian_paths_precise(float *arith, float *geom, long long path0, long long npaths,
                                               uint32_t k0, uint32_t k1, float s0, float strike,
                                               float drift, float vol, int nstep)
{
    asian_paths_body<true>(arith, geom, path0, npaths, k0, k1, s0, strike, drift, vol, nstep);
}
