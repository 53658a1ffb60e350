// pipe_probe.cu -- how fast the SM runs the two instruction groups the pricer
// cannot do without, alone and together, when nothing waits for anything else.
//
// Per Philox call (four monitoring steps) asian_mc issues 12 MUFU operations
// and 20 IMAD.WIDE with 20 three-input xors (the two 32x32->64 products of each
// of the ten rounds), among 68 instructions in all. The special-function unit
// alone allows 16 lanes per clock per SM, which is the ceiling the pricer's
// roofline is quoted against; but IMAD.WIDE runs on the heavy FMA pipe at a
// quarter of the FP32 rate, and the two groups do not overlap fully. These
// kernels time them on independent chains held in registers:
//   probe_mufu            12 MUFU per trip
//   probe_imad_wide       20 IMAD.WIDE + 20 LOP3 per trip
//   probe_mufu_imad_wide  both
// The third is a subset of what the pricer issues per call, with no Box-Muller
// data flow and no floating-point work beside it, so its pace is a ceiling for
// the pricer on this SM. Each takes (out, trips, seed, key); out is written only
// if a sum hits an impossible value, which keeps the work alive. Launch with
// 256-thread blocks.
#include "common.cuh"

namespace probe {

__device__ __forceinline__ float ex2(float x)
{
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <bool MUFU, bool IMAD>
__device__ __forceinline__ void body(float *out, int trips, float seed, uint32_t key)
{
    float m[12];
#pragma unroll
    for (int j = 0; j < 12; j++) m[j] = seed + 0.001f * (float)(threadIdx.x + j);
    uint32_t c[2][4];
#pragma unroll
    for (int h = 0; h < 2; h++) { c[h][0] = threadIdx.x + h; c[h][1] = blockIdx.x; c[h][2] = h; c[h][3] = 7u; }
    for (int it = 0; it < trips; it++) {
        if (MUFU) {
#pragma unroll
            for (int j = 0; j < 12; j++) m[j] = ex2(m[j]);
        }
        if (IMAD) {
            // Two four-word Philox states, five rounds each: 20 wide products, 20 three-input xors.
#pragma unroll
            for (int r = 0; r < 5; r++) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const uint64_t p0 = (uint64_t)0xD2511F53u * c[h][0];
                    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c[h][2];
                    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[h][1] ^ key;
                    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[h][3] ^ (key + (uint32_t)r);
                    c[h][0] = n0; c[h][1] = (uint32_t)p1; c[h][2] = n2; c[h][3] = (uint32_t)p0;
                }
            }
        }
    }
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < 12; j++) acc += m[j];
#pragma unroll
    for (int h = 0; h < 2; h++) acc += (float)(c[h][0] ^ c[h][1] ^ c[h][2] ^ c[h][3]);
    if (acc == 12345.678f) out[0] = acc;
}

}  // namespace probe

extern "C" __global__ void __launch_bounds__(256, 2)
probe_mufu(float *out, int trips, float seed, uint32_t key) { probe::body<true, false>(out, trips, seed, key); }

extern "C" __global__ void __launch_bounds__(256, 2)
probe_imad_wide(float *out, int trips, float seed, uint32_t key) { probe::body<false, true>(out, trips, seed, key); }

extern "C" __global__ void __launch_bounds__(256, 2)
probe_mufu_imad_wide(float *out, int trips, float seed, uint32_t key) { probe::body<true, true>(out, trips, seed, key); }
