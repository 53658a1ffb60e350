// canonical.cu -- the reference's other launcher-dispatched kernels, by their own
// names and parameter lists, for host programs that load them by name.
//
//   matmul_general(C, A, B, M, N, K)   tests/canonical.cu:18-50  (16x16 shared tiles)
//   reduce_sum(output, input, n)       tests/canonical.cu:93-108 (grid-stride +
//                                      shuffle + shared + atomicAdd)
//
// The caller picks the launch geometry (the reference launches matmul_general
// with 16x16 blocks on a ceil(N/16) x ceil(M/16) grid), so both kernels walk
// their index space with strides of the whole launch and are correct for any
// grid and block. They are the call-compatible forms; the tuned paths are
// gemm_tf32x3 and reduce_sum_f32.
#include "common.cuh"

// C[row, col] = sum over k of A[row, k] * B[k, col], k ascending, product and sum
// rounded separately: the order and rounding of the reference kernel's inner
// loop, hence bit-identical to its x86-64 build and to a plain host triple loop.
extern "C" __global__ void matmul_general(float *C, const float *A, const float *B, int M, int N, int K)
{
    const unsigned cols_per_pass = gridDim.x * blockDim.x, rows_per_pass = gridDim.y * blockDim.y;
    for (unsigned row = blockIdx.y * blockDim.y + threadIdx.y; row < (unsigned)M; row += rows_per_pass)
        for (unsigned col = blockIdx.x * blockDim.x + threadIdx.x; col < (unsigned)N; col += cols_per_pass) {
            if (blockIdx.z != 0 || threadIdx.z != 0) continue;
            const float *a = A + (size_t)row * K;
            const float *b = B + col;
            float sum = 0.0f;
            for (int k = 0; k < K; k++) sum = __fadd_rn(sum, __fmul_rn(a[k], b[(size_t)k * N]));
            C[(size_t)row * N + col] = sum;
        }
}

// *output += sum of input[0..n): each block adds its grid-stride share with one
// atomicAdd, as the reference kernel does, so *output must hold the caller's
// starting value (normally 0) and the fp32 result depends on arrival order.
extern "C" __global__ void reduce_sum(float *output, const float *input, int n)
{
    __shared__ float warp_vals[32];
    const unsigned tid = flat_tid(), B = flat_bdim();
    float sum = 0.0f;
    for (long long i = (long long)flat_bid() * B + tid; i < n; i += (long long)flat_gdim() * B) sum += input[i];
    const unsigned mask = __activemask();
    const unsigned lane = tid & 31, wid = tid >> 5, cnt = __popc(mask);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float t = __shfl_down_sync(mask, sum, o);
        if (lane + o < cnt) sum += t;
    }
    if (lane == 0) warp_vals[wid] = sum;
    __syncthreads();
    if (tid == 0) {
        float total = 0.0f;
        for (unsigned w = 0; w < (B + 31) / 32; w++) total += warp_vals[w];
        atomicAdd(output, total);
    }
}
