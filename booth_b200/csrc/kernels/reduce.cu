// reduce.cu -- global sum on sm_100a: warp shuffle tree, block pass, grid pass.
//
// The workload is the reference's reduction shape: per-thread serial partial
// sums, a shared-memory pass per block, one value per block
// (tests/tg_reduce.cu:4-26) and the grid-stride + shuffle + shared + atomic form
// (tests/canonical.cu:59-108). On a B200 it is a read-once stream (4 bytes per
// element), so each thread keeps eight independent 16-byte loads in flight with
// the streaming cache policy and the arithmetic hides under the loads.
//
// Stages:
//   1. thread:  grid-stride over 16-byte chunks, partial sums in registers
//               (int32: wrapping adds; fp32: four fp32 accumulator vectors);
//   2. warp:    __shfl_xor_sync butterfly (fp32 partials are widened to double
//               first, so everything above the thread level is double);
//   3. block:   one value per warp through shared memory, warp 0 finishes;
//   4. grid:    every block stores its value to partials[block], fences and takes
//               a ticket from an arrival counter; the block that draws the last
//               ticket adds the partials in index order and writes the result.
//               Nothing ever waits for another block, so there is no spin loop.
//               The last block puts the counter back to zero for the next launch.
// For a fixed launch geometry the result is bit-reproducible.
//
// Scratch: partials[] needs one slot per block, ticket one zero-initialised
// unsigned; both live in the device's scratch buffer owned by the host shim.
#include "common.cuh"

#define RED_UNROLL 8

// Sum over the warp; lane 0 always ends up with the total. A full warp uses the
// xor butterfly. A block whose size is not a multiple of 32 has one short warp;
// there the existing lanes are the low ones and a bounded shift-down tree is used.
template <typename T>
__device__ __forceinline__ T warp_sum(T v)
{
    const unsigned mask = __activemask();
    if (mask == 0xffffffffu) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    } else {
        const unsigned lane = flat_tid() & 31, cnt = __popc(mask);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const T t = __shfl_down_sync(mask, v, o);
            if (lane + o < cnt) v += t;
        }
    }
    return v;
}

// Sum over the block; the result is valid in thread 0. `sh` has 32 slots.
template <typename T>
__device__ __forceinline__ T block_sum(T v, T *sh)
{
    const unsigned tid = flat_tid(), lane = tid & 31, wid = tid >> 5;
    const unsigned nwarp = (flat_bdim() + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                    // sh may still be read from a previous call
    if (lane == 0) sh[wid] = v;
    __syncthreads();
    if (wid == 0) {
        v = lane < nwarp ? sh[lane] : T(0);
        v = warp_sum(v);
    }
    return v;
}

// Grid pass shared by both element types. Returns true in thread 0 of the block
// that drew the last ticket, with `total` holding the sum of all partials.
template <typename T>
__device__ __forceinline__ bool grid_sum(T block_value, T *partials, unsigned *ticket,
                                         T *sh, T &total)
{
    __shared__ unsigned s_last;
    const unsigned tid = flat_tid(), G = flat_gdim();
    if (tid == 0) {
        partials[flat_bid()] = block_value;
        __threadfence();
        s_last = (atomicAdd(ticket, 1u) == G - 1);
    }
    __syncthreads();
    if (!s_last) return false;
    __threadfence();
    T v = T(0);
    for (unsigned i = tid; i < G; i += flat_bdim()) v += __ldcg(partials + i);
    total = block_sum(v, sh);
    if (tid == 0) { *ticket = 0u; return true; }
    return false;
}

// Wrapping int32 sum of in[0..n) into *out.
extern "C" __global__ void reduce_sum_i32(const int *in, long long n, unsigned *partials,
                                          unsigned *ticket, int *out)
{
    __shared__ unsigned sh[32];
    const unsigned tid = flat_tid(), B = flat_bdim(), bid = flat_bid(), G = flat_gdim();
    // Peel up to three leading elements so the body is 16-byte aligned.
    long long head = (long long)(((16u - (unsigned)((uintptr_t)in & 15u)) & 15u) >> 2);
    if (head > n) head = n;
    const uint4 *v4 = reinterpret_cast<const uint4 *>(in + head);
    const long long nvec = (n - head) >> 2;
    unsigned acc = 0;
    const long long tile = (long long)B * RED_UNROLL;
    for (long long base = (long long)bid * tile; base < nvec; base += (long long)G * tile) {
        if (base + tile <= nvec) {
            uint4 v[RED_UNROLL];
#pragma unroll
            for (int j = 0; j < RED_UNROLL; j++) v[j] = __ldcs(v4 + base + (long long)j * B + tid);
#pragma unroll
            for (int j = 0; j < RED_UNROLL; j++) acc += (v[j].x + v[j].y) + (v[j].z + v[j].w);
        } else {
            for (int j = 0; j < RED_UNROLL; j++) {
                const long long i = base + (long long)j * B + tid;
                if (i < nvec) { const uint4 v = __ldcs(v4 + i); acc += (v.x + v.y) + (v.z + v.w); }
            }
        }
    }
    if (bid == 0) {
        const long long tail0 = head + (nvec << 2);
        for (long long i = tid; i < head; i += B) acc += (unsigned)in[i];
        for (long long i = tail0 + tid; i < n; i += B) acc += (unsigned)in[i];
    }
    const unsigned bsum = block_sum(acc, sh);
    unsigned total;
    if (grid_sum(bsum, partials, ticket, sh, total)) *out = (int)total;
}

// Sum of in[0..n) into *out (double). Per-thread partial sums are fp32. The launch
// bound is a scheduling hint that pays: told that four blocks share an SM, the
// compiler spends 62 registers instead of 54 and issues all eight loads of a trip
// ahead of the adds (7.3 TB/s at 2^30 elements against 7.0 without it).
extern "C" __global__ void __launch_bounds__(256, 4) reduce_sum_f32(const float *in, long long n, double *partials,
                                          unsigned *ticket, double *out)
{
    __shared__ double sh[32];
    const unsigned tid = flat_tid(), B = flat_bdim(), bid = flat_bid(), G = flat_gdim();
    long long head = (long long)(((16u - (unsigned)((uintptr_t)in & 15u)) & 15u) >> 2);
    if (head > n) head = n;
    const float4 *v4 = reinterpret_cast<const float4 *>(in + head);
    const long long nvec = (n - head) >> 2;
    float4 acc[4];
#pragma unroll
    for (int j = 0; j < 4; j++) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    const long long tile = (long long)B * RED_UNROLL;
    for (long long base = (long long)bid * tile; base < nvec; base += (long long)G * tile) {
        if (base + tile <= nvec) {
            float4 v[RED_UNROLL];
#pragma unroll
            for (int j = 0; j < RED_UNROLL; j++) v[j] = __ldcs(v4 + base + (long long)j * B + tid);
#pragma unroll
            for (int j = 0; j < RED_UNROLL; j++) {
                acc[j & 3].x += v[j].x; acc[j & 3].y += v[j].y;
                acc[j & 3].z += v[j].z; acc[j & 3].w += v[j].w;
            }
        } else {
            for (int j = 0; j < RED_UNROLL; j++) {
                const long long i = base + (long long)j * B + tid;
                if (i < nvec) {
                    const float4 v = __ldcs(v4 + i);
                    acc[0].x += v.x; acc[0].y += v.y; acc[0].z += v.z; acc[0].w += v.w;
                }
            }
        }
    }
    double d = 0.0;
#pragma unroll
    for (int j = 0; j < 4; j++)
        d += ((double)acc[j].x + (double)acc[j].y) + ((double)acc[j].z + (double)acc[j].w);
    if (bid == 0) {
        const long long tail0 = head + (nvec << 2);
        for (long long i = tid; i < head; i += B) d += (double)in[i];
        for (long long i = tail0 + tid; i < n; i += B) d += (double)in[i];
    }
    const double bsum = block_sum(d, sh);
    double total;
    if (grid_sum(bsum, partials, ticket, sh, total)) *out = total;
}
