// reduce_noalloc.cu -- fp32 sum for callers that are not allowed to allocate.
//
// Some hosts of this library cannot call cudaMalloc (or anything that does so
// on their behalf) at the moment they need a sum: code running inside a region
// where a framework has frozen its memory pool, real-time loops that forbid
// driver allocations, and plug-ins whose host owns every byte of device memory.
// booth_sm100_reduce_f32 keeps its per-block partial sums and its arrival
// counter in a scratch buffer that sm100_rt_init allocated; this entry point
// needs no device handle and no buffer from anybody: its scratch is a fixed
// array compiled into the library.
//
// What that costs and what the caller must know:
//   * the array (33,024 bytes) is part of the library's device image: every GPU
//     on which this entry point is used holds it from first use until exit;
//   * the input is cut into segments of 262,144 elements, one block and one
//     scratch slot per segment, 4,096 slots: n above 2^30 is refused;
//   * every call looks the array's device address up for the current device
//     (cudaGetSymbolAddress; the array's name in host code is only a stand-in,
//     not an address a kernel could use). The first such call on a device makes
//     the runtime load this library's device code there: make that first call
//     before any stream capture begins. Later calls are a table look-up, and
//     asking each time keeps the address right after the application has reset
//     the device;
//   * all calls share the one array and it keeps what the previous call left,
//     so each call first clears the arrival counter on the caller's stream.
//     Two calls that may run on the GPU at the same time (different streams,
//     different host threads) race on it: serialise them;
//   * nothing here calls cudaMalloc, cudaFree or a library routine that
//     allocates. The result is written to memory the caller passes.
//
// Because the segment size is fixed, the sum does not depend on the GPU or its SM
// count (the grid-sized booth_sm100_reduce_f32 does not promise that): the same
// input at the same 16-byte alignment gives the same bits everywhere. An input
// that is only 4-byte aligned is added up in a different order (scalar loads)
// and may differ from the aligned result in the last bits.
// in must be 4-byte aligned, out 8-byte aligned (it receives a double); both are
// checked here, before any GPU work, because the device would fault on them.
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

#include "booth_sm100.h"

namespace {

constexpr int NOALLOC_BLOCK = 256;
constexpr long long NOALLOC_SEGMENT = 1ll << 18;       // elements per block
constexpr int NOALLOC_SLOTS = 4096;                     // segment sums the scratch holds
constexpr long long NOALLOC_MAX_N = NOALLOC_SEGMENT * NOALLOC_SLOTS;
constexpr size_t NOALLOC_HEADER = 256;                  // arrival counter lives here

// [0,256): arrival counter (first 4 bytes). [256, ...): one double per segment.
static __device__ __align__(256) unsigned char g_scratch[NOALLOC_HEADER + NOALLOC_SLOTS * sizeof(double)];

__device__ __forceinline__ double warp_sum(double v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Valid in thread 0. sh has 32 slots. blockDim.x is NOALLOC_BLOCK.
__device__ __forceinline__ double block_sum(double v, double *sh)
{
    const unsigned lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) sh[wid] = v;
    __syncthreads();
    if (wid == 0) v = warp_sum(lane < NOALLOC_BLOCK / 32 ? sh[lane] : 0.0);
    return v;
}

// Block b sums its segment in[b*SEGMENT, min((b+1)*SEGMENT, n)): fp32 partial sums
// per thread, double above. The block that arrives last adds the segment sums in
// index order and writes *out. `scratch` is the device address of g_scratch.
__global__ void __launch_bounds__(NOALLOC_BLOCK)
reduce_f32_segments(const float *__restrict__ in, long long n, unsigned char *scratch, double *out)
{
    __shared__ double sh[32];
    __shared__ unsigned s_last;
    unsigned *ticket = reinterpret_cast<unsigned *>(scratch);
    double *partials = reinterpret_cast<double *>(scratch + NOALLOC_HEADER);
    const long long lo = (long long)blockIdx.x * NOALLOC_SEGMENT;
    const long long hi = lo + NOALLOC_SEGMENT < n ? lo + NOALLOC_SEGMENT : n;
    const float *p = in + lo;
    const long long len = hi > lo ? hi - lo : 0;
    double d = 0.0;
    if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
        const float4 *p4 = reinterpret_cast<const float4 *>(p);
        const long long nvec = len >> 2;
        float4 acc[4];
#pragma unroll
        for (int j = 0; j < 4; j++) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        long long i = threadIdx.x;
        for (; i + 3 * NOALLOC_BLOCK < nvec; i += 4 * NOALLOC_BLOCK) {
            float4 v[4];
#pragma unroll
            for (int j = 0; j < 4; j++) v[j] = __ldcs(p4 + i + j * NOALLOC_BLOCK);
#pragma unroll
            for (int j = 0; j < 4; j++) { acc[j].x += v[j].x; acc[j].y += v[j].y; acc[j].z += v[j].z; acc[j].w += v[j].w; }
        }
        for (; i < nvec; i += NOALLOC_BLOCK) {
            const float4 v = __ldcs(p4 + i);
            acc[0].x += v.x; acc[0].y += v.y; acc[0].z += v.z; acc[0].w += v.w;
        }
#pragma unroll
        for (int j = 0; j < 4; j++)
            d += ((double)acc[j].x + (double)acc[j].y) + ((double)acc[j].z + (double)acc[j].w);
        for (long long t = (nvec << 2) + threadIdx.x; t < len; t += NOALLOC_BLOCK) d += (double)p[t];
    } else {
        float acc = 0.f;
        for (long long t = threadIdx.x; t < len; t += NOALLOC_BLOCK) acc += p[t];
        d = (double)acc;
    }
    d = block_sum(d, sh);
    if (threadIdx.x == 0) {
        partials[blockIdx.x] = d;
        __threadfence();
        s_last = (atomicAdd(ticket, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    double v = 0.0;
    for (unsigned b = threadIdx.x; b < gridDim.x; b += NOALLOC_BLOCK) v += __ldcg(partials + b);
    v = block_sum(v, sh);
    if (threadIdx.x == 0) { *out = v; *ticket = 0u; }
}

int fail(const char *what, cudaError_t e)
{
    std::fprintf(stderr, "sm100_rt: booth_sm100_reduce_f32_noalloc: %s: %s\n", what, cudaGetErrorString(e));
    return SM100_ERR_CUDA;
}

}  // namespace

extern "C" int booth_sm100_reduce_f32_noalloc(sm100_ptr_t in, long long n, sm100_ptr_t out, void *stream)
{
    if (!out || (out & 7) || n < 0 || (n > 0 && !in) || (in & 3)) {
        std::fprintf(stderr, "sm100_rt: booth_sm100_reduce_f32_noalloc: bad argument (in: 4-byte aligned, "
                     "non-NULL when n > 0; out: 8-byte aligned)\n");
        return SM100_ERR_ARG;
    }
    if (n > NOALLOC_MAX_N) {
        std::fprintf(stderr, "sm100_rt: booth_sm100_reduce_f32_noalloc: n = %lld exceeds %lld, the capacity of the "
                     "built-in scratch (%d segment sums of %lld elements); use booth_sm100_reduce_f32\n",
                     n, NOALLOC_MAX_N, NOALLOC_SLOTS, NOALLOC_SEGMENT);
        return SM100_ERR_ARG;
    }
    // The device address of the array on the current device. In host code the name
    // g_scratch is not that address; only this call yields one a kernel can use.
    void *sym = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&sym, g_scratch);
    if (e != cudaSuccess) return fail("cudaGetSymbolAddress(scratch)", e);
    unsigned char *scratch = static_cast<unsigned char *>(sym);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The array keeps the previous call's contents; only the counter must be zero.
    e = cudaMemsetAsync(scratch, 0, NOALLOC_HEADER, s);
    if (e != cudaSuccess) return fail("clearing the arrival counter", e);
    long long blocks = (n + NOALLOC_SEGMENT - 1) / NOALLOC_SEGMENT;
    if (blocks < 1) blocks = 1;
    reduce_f32_segments<<<(unsigned)blocks, NOALLOC_BLOCK, 0, s>>>(
        reinterpret_cast<const float *>(static_cast<uintptr_t>(in)), n, scratch,
        reinterpret_cast<double *>(static_cast<uintptr_t>(out)));
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail("kernel launch", e);
    return SM100_OK;
}
