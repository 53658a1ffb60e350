// common.cuh -- helpers shared by the sm_100a kernels of the image.
#pragma once
#include <cstdint>

// The launcher lets the caller choose any grid and block shape, so kernels that
// are looked up by name flatten the launch to one dimension.
__device__ __forceinline__ unsigned flat_tid()
{
    return threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z);
}
__device__ __forceinline__ unsigned flat_bdim() { return blockDim.x * blockDim.y * blockDim.z; }
__device__ __forceinline__ unsigned flat_bid()
{
    return blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
}
__device__ __forceinline__ unsigned flat_gdim() { return gridDim.x * gridDim.y * gridDim.z; }

// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3").
// Each round is two 32x32->64 products (one IMAD.WIDE each) and two three-input
// xors; the key schedule is loop-invariant.
struct Philox4 { uint32_t x, y, z, w; };

__device__ __forceinline__ Philox4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                                 uint32_t k0, uint32_t k1)
{
#pragma unroll
    for (int r = 0; r < 10; r++) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        c0 = n0; c1 = (uint32_t)p1; c2 = n2; c3 = (uint32_t)p0;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    Philox4 o = { c0, c1, c2, c3 };
    return o;
}
