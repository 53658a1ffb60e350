// stream.cu -- HBM-streaming kernels for sm_100a: vector_add, saxpy, fill_philox.
//
// vector_add and saxpy keep the names and parameter lists of the reference's
// kernel sources (tests/tri_vadd.py:6-9, tests/canonical.cu:168) because the
// launcher looks kernels up by bare name and the CALLER picks the launch
// geometry (examples/launch_saxpy.c:83-87 launches one thread per element).
// They are therefore correct for any grid and block shape: the threads of the
// launch are flattened and walk the vectors in tiles of 256-bit accesses. A
// launch far larger than any tuned one (one thread per element is eight times
// more threads than 32-byte chunks) keeps only its first blocks working; the
// others retire at once. saxpy_stream and vadd_stream are the same bodies for the
// library's own, tuned launches, with twice the loads in flight per thread and the
// registers that takes.
//
// Arithmetic matches the reference's x86-64 backend bit for bit: the product
// and the sum of saxpy are rounded separately (mulss then addss,
// src/cpu/cpu_emit.c:538-542), hence __fmul_rn/__fadd_rn, which the compiler
// never contracts into an FMA.
//
// Memory behaviour: every element is touched once. When the pointers allow it a
// thread moves 32 bytes per instruction (256-bit ld/st.global) and keeps two such
// loads per input in flight; a warp's accesses are contiguous 1 KiB rows. For
// vectors of 2^28 elements and more the host launches three persistent blocks of
// 128 threads per SM: HBM throughput on a B200 peaks sharply at 384 threads per
// SM (6.9 TB/s for both kernels, 6.5 at 640). Shorter vectors get up to 128
// blocks per SM, one tile each, so that the hardware scheduler evens out the two
// ends of a launch that lasts tens of microseconds.
// Algorithmic traffic is 12 bytes per element for both kernels.
#include "common.cuh"

// Threads per SM that an oversized launch of the by-name kernels keeps working.
#ifndef STREAM_KEEP_LONG
#define STREAM_KEEP_LONG 640      // vectors of 2^26 elements and more
#endif
#ifndef STREAM_BYNAME_REGS
#define STREAM_BYNAME_REGS 32
#endif
#define STREAM_KEEP_SHORT 1536

#define UNROLL 4      // 128-bit path: independent 16-byte loads per input per thread
#define UNROLL8 2     // 256-bit path: independent 32-byte loads per input per thread

// 256-bit global accesses (sm_100): one instruction moves 32 bytes per thread.
// Loads bypass L1 allocation; every element is used once.
struct __align__(32) f32x8 { float v[8]; };

__device__ __forceinline__ f32x8 ld256(const f32x8 *p)
{
    f32x8 r;
    asm volatile("ld.global.L1::no_allocate.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]),
                   "=f"(r.v[4]), "=f"(r.v[5]), "=f"(r.v[6]), "=f"(r.v[7]) : "l"(p));
    return r;
}
__device__ __forceinline__ void st256(f32x8 *p, const f32x8 &r)
{
    asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 :: "l"(p), "f"(r.v[0]), "f"(r.v[1]), "f"(r.v[2]), "f"(r.v[3]),
                    "f"(r.v[4]), "f"(r.v[5]), "f"(r.v[6]), "f"(r.v[7]) : "memory");
}

__device__ __forceinline__ float4 add4(float4 a, float4 b)
{
    return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
}
__device__ __forceinline__ float4 axpy4(float a, float4 x, float4 y)
{
    return make_float4(__fadd_rn(__fmul_rn(a, x.x), y.x), __fadd_rn(__fmul_rn(a, x.y), y.y),
                       __fadd_rn(__fmul_rn(a, x.z), y.z), __fadd_rn(__fmul_rn(a, x.w), y.w));
}

// One body for all four kernels: out[i] = op(x[i], y[i]) with op = x + y (SAXPY
// false) or fl(fl(a*x) + y) (SAXPY true). Three paths by pointer alignment: 32-byte
// vectors, 16-byte vectors, scalars; each ends with a scalar tail.
//
// ANY_LAUNCH: the geometry is the caller's. Blocks are handed to the SMs in index
// order, so when the launch has more than 128 blocks per SM the first `keep` (a
// few per SM) start together and stream the whole vector
// while the surplus blocks come and go beside them without touching memory; how
// fast the GPU hands out and retires empty blocks (1.77 per ns for 256-thread blocks,
// when nothing else occupies block slots) then sets the pace.
template <bool SAXPY>
__device__ __forceinline__ float op1(float a, float x, float y)
{
    return SAXPY ? __fadd_rn(__fmul_rn(a, x), y) : __fadd_rn(x, y);
}

template <bool SAXPY, bool ANY_LAUNCH, bool LEAN = false>
__device__ __forceinline__ void stream_body(const float *x, const float *y, float *out, float a, long long n)
{
    // Loads in flight per thread and input: two 32-byte (four 16-byte) in the library's own
    // launches; one (two) in the by-name kernels, which must live in 32 registers (see below).
    constexpr int U8 = LEAN ? 1 : UNROLL8, U4 = LEAN ? 2 : UNROLL;
    const unsigned tid = flat_tid(), B = flat_bdim();
    const unsigned long long bid = flat_bid();
    unsigned long long G = flat_gdim();
    if (ANY_LAUNCH) {
        unsigned nsm;
        asm("mov.u32 %0, %%nsmid;" : "=r"(nsm));
        if (G > 128ull * nsm) {                     // far beyond any tuned launch
            const unsigned per_sm = (n < (1ll << 26) ? STREAM_KEEP_SHORT : STREAM_KEEP_LONG) / B;
            const unsigned long long keep = (unsigned long long)nsm * (per_sm ? per_sm : 1u);
            if (bid >= keep) return;
            G = keep;
        }
    }
    // (The surplus blocks of an oversized launch have left above: they touch no memory,
    // and anything they execute first costs retirement rate, 3.0 against 4.3 TB/s.)
    // Launched with programmatic stream serialization (the library's own launches),
    // this grid is set up and its first blocks are placed while the previous kernel
    // on the stream is still finishing: wait here for that kernel's memory, then let
    // the next launch do the same behind this one. That hides the few microseconds
    // between back-to-back launches (2^24 elements: 8.1 against 7.5 TB/s). Waiting
    // first matters: releasing the next launch before the wait lets a whole chain of
    // grids pile up on the SMs and cost 14 % at 2^30 elements. Plain launches pass
    // straight through both instructions.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const uintptr_t bits = (uintptr_t)x | (uintptr_t)y | (uintptr_t)out;
    long long done;                     // elements covered by the vector part
    if ((bits & 31) == 0) {
        const long long nvec = n >> 3;
        const f32x8 *x8 = reinterpret_cast<const f32x8 *>(x);
        const f32x8 *y8 = reinterpret_cast<const f32x8 *>(y);
        f32x8 *o8 = reinterpret_cast<f32x8 *>(out);
        const long long tile = (long long)B * U8;
        const long long nfull = nvec / tile * tile;          // vectors covered by whole tiles
        // Branch-free main loop over whole tiles, so the loads of the next
        // iteration can be issued while this one's stores drain.
        for (long long base = (long long)bid * tile; base < nfull; base += (long long)G * tile) {
            f32x8 xv[U8], yv[U8];
#pragma unroll
            for (int j = 0; j < U8; j++) xv[j] = ld256(x8 + base + (long long)j * B + tid);
#pragma unroll
            for (int j = 0; j < U8; j++) yv[j] = ld256(y8 + base + (long long)j * B + tid);
#pragma unroll
            for (int j = 0; j < U8; j++) {
                f32x8 r;
#pragma unroll
                for (int e = 0; e < 8; e++) r.v[e] = op1<SAXPY>(a, xv[j].v[e], yv[j].v[e]);
                st256(o8 + base + (long long)j * B + tid, r);
            }
        }
        for (long long i = nfull + (long long)(bid * B + tid); i < nvec; i += (long long)(G * B)) {
            const f32x8 xv = ld256(x8 + i), yv = ld256(y8 + i);
            f32x8 r;
#pragma unroll
            for (int e = 0; e < 8; e++) r.v[e] = op1<SAXPY>(a, xv.v[e], yv.v[e]);
            st256(o8 + i, r);
        }
        done = nvec << 3;
    } else if ((bits & 15) == 0) {
        const long long nvec = n >> 2;
        const float4 *x4 = reinterpret_cast<const float4 *>(x);
        const float4 *y4 = reinterpret_cast<const float4 *>(y);
        float4 *o4 = reinterpret_cast<float4 *>(out);
        const long long tile = (long long)B * U4;
        for (long long base = (long long)bid * tile; base < nvec; base += (long long)G * tile) {
            if (base + tile <= nvec) {
                float4 xv[U4], yv[U4];
#pragma unroll
                for (int j = 0; j < U4; j++) xv[j] = __ldcs(x4 + base + (long long)j * B + tid);
#pragma unroll
                for (int j = 0; j < U4; j++) yv[j] = __ldcs(y4 + base + (long long)j * B + tid);
#pragma unroll
                for (int j = 0; j < U4; j++)
                    __stcs(o4 + base + (long long)j * B + tid, SAXPY ? axpy4(a, xv[j], yv[j]) : add4(xv[j], yv[j]));
            } else {
                for (int j = 0; j < U4; j++) {
                    const long long i = base + (long long)j * B + tid;
                    if (i < nvec) {
                        const float4 xv = __ldcs(x4 + i), yv = __ldcs(y4 + i);
                        __stcs(o4 + i, SAXPY ? axpy4(a, xv, yv) : add4(xv, yv));
                    }
                }
            }
        }
        done = nvec << 2;
    } else {
        done = 0;
    }
    // scalar remainder (the whole vector when the pointers are not 16-byte aligned)
    for (long long i = done + (long long)(bid * B + tid); i < n; i += (long long)(G * B))
        out[i] = op1<SAXPY>(a, x[i], y[i]);
}

// out[i] = x[i] + y[i] for i < n_elements. block_size is the Triton BLOCK_SIZE
// parameter of the reference kernel; the geometry comes from the launch itself.
// The by-name kernels are held to 32 registers (one 32-byte load per input in flight
// per thread instead of two): under a one-thread-per-element launch of 256-thread
// blocks that leaves room for eight blocks per SM, two or three that work and five
// slots through which the empty ones pass, and the launch then runs at the pace at
// which the GPU hands out blocks: 2^30 elements in 2.40 ms, 5.47 TB/s, where the same
// launch with n = 0 (every block empty) takes 2.37 ms. With 48 registers (five blocks
// per SM) it was 4.29 TB/s, with 40 (six) 4.83. Under a caller's moderate geometry
// the lean body reaches 6.3 to 6.6 TB/s (the library's own kernels 6.9).
extern "C" __global__ void __maxnreg__(STREAM_BYNAME_REGS) vector_add(const float *x, const float *y, float *out,
                                                      int n_elements, int block_size)
{
    (void)block_size;
    stream_body<false, true, true>(x, y, out, 0.0f, (long long)n_elements);
}
extern "C" __global__ void vadd_stream(const float *x, const float *y, float *out, int n_elements, int block_size)
{
    (void)block_size;
    stream_body<false, false>(x, y, out, 0.0f, (long long)n_elements);
}

// y[i] = a*x[i] + y[i] for i < n, product and sum rounded separately.
extern "C" __global__ void __maxnreg__(STREAM_BYNAME_REGS) saxpy(float *y, const float *x, float a, int n)
{
    stream_body<true, true, true>(x, y, y, a, (long long)n);
}
// The same for the library's own launches: tuned geometry, two 32-byte loads per input
// in flight. (Built with the geometry test and 48 registers like the by-name kernel
// used to be: that code reaches 6.92 TB/s at three 128-thread blocks per SM, the body
// without the test 5.8 at the same geometry; the optimum is that sharp.)
extern "C" __global__ void __maxnreg__(48) saxpy_stream(float *y, const float *x, float a, int n)
{
    stream_body<true, true, false>(x, y, y, a, (long long)n);
}

// ---- seeded inputs -------------------------------------------------------

__device__ __forceinline__ uint32_t fill_value(uint32_t x, int kind)
{
    if (kind == 2) return (uint32_t)((int)(x % 2001u) - 1000);
    if (kind == 3) return x;                                        // the raw word
    const float u = (float)(x >> 8) * 5.9604644775390625e-8f;       // exact, [0,1)
    const float v = kind == 0 ? __fadd_rn(__fmul_rn(2.0f, u), -1.0f) : u;
    return __float_as_uint(v);
}

// dst[j] = element (first + j), j in [0,n). Element i is lane i%4 of the Philox
// block with counter (i/4, 0, 0) and key (seed, stream).
extern "C" __global__ void fill_philox(uint32_t *dst, long long first, long long n,
                                       uint32_t seed, uint32_t stream, int kind)
{
    const long long blk0 = first >> 2;
    const long long nblk = ((first + n + 3) >> 2) - blk0;
    const long long T = (long long)flat_gdim() * flat_bdim();
    for (long long t = (long long)(flat_bid() * flat_bdim() + flat_tid()); t < nblk; t += T) {
        const unsigned long long ctr = (unsigned long long)(blk0 + t);
        const Philox4 r = philox4x32_10((uint32_t)ctr, (uint32_t)(ctr >> 32), 0u, 0u, seed, stream);
        const uint32_t v[4] = { r.x, r.y, r.z, r.w };
        const long long e0 = (long long)(ctr << 2);
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const long long j = e0 + l - first;
            if (j >= 0 && j < n) dst[j] = fill_value(v[l], kind);
        }
    }
}

// Raw Philox4x32-10 output for a caller-given counter and key: thread t of the
// launch writes the four words of the block with counter (c0 + t, c1, c2, c3) to
// out[4t .. 4t+3]. Looked up by name; it exists so that the generator can be
// checked on the device against the known-answer vectors published with Random123.
extern "C" __global__ void philox_words(uint32_t *out, uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                        uint32_t k0, uint32_t k1)
{
    const unsigned t = flat_bid() * flat_bdim() + flat_tid();
    const Philox4 r = philox4x32_10(c0 + t, c1, c2, c3, k0, k1);
    out[4 * t + 0] = r.x; out[4 * t + 1] = r.y; out[4 * t + 2] = r.z; out[4 * t + 3] = r.w;
}
