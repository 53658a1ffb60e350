// canonical.cu -- the reference's other launcher-dispatched kernels, by their own
// names and parameter lists, for host programs that load them by name.
//
//   matmul_general(C, A, B, M, N, K)   tests/canonical.cu:18-50  (16x16 shared tiles)
//   reduce_sum(output, input, n)       tests/canonical.cu:93-108 (grid-stride +
//                                      shuffle + shared + atomicAdd)
//   dot_product(result, a, b, n)       tests/canonical.cu:149-161 (same reduction
//                                      over products)
//   r_2_1024_16_64(data0..data3, pos)  tests/tg_reduce.cu:4-26 (the tinygrad
//                                      attention reduction: masked 64-term sums
//                                      per thread, 16 threads combined)
//
// The caller picks the launch geometry (the reference launches matmul_general
// with 16x16 blocks on a ceil(N/16) x ceil(M/16) grid), so both kernels walk
// their index space with strides of the whole launch and are correct for any
// grid and block; so is dot_product. r_2_1024_16_64 has its geometry in its name
// (grid 1024 x 2, 16 threads) and takes its indices from the launch as the
// reference kernel does. They are the call-compatible forms; the tuned paths are
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

// Block sum of one value per thread, then one atomicAdd per block: shuffle tree
// inside each warp (partial warps included), per-warp sums through shared memory,
// thread 0 adds them in warp order.
__device__ __forceinline__ void block_sum_to(float *output, float sum)
{
    __shared__ float warp_vals[32];
    const unsigned tid = flat_tid(), B = flat_bdim();
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

// *output += sum of input[0..n): each block adds its grid-stride share with one
// atomicAdd, as the reference kernel does, so *output must hold the caller's
// starting value (normally 0) and the fp32 result depends on arrival order.
extern "C" __global__ void reduce_sum(float *output, const float *input, int n)
{
    const unsigned tid = flat_tid(), B = flat_bdim();
    float sum = 0.0f;
    for (long long i = (long long)flat_bid() * B + tid; i < n; i += (long long)flat_gdim() * B) sum += input[i];
    block_sum_to(output, sum);
}

// *result += sum of a[i]*b[i], i in [0,n): the same reduction over products, each
// product rounded before it is added (the reference's back ends never fuse).
extern "C" __global__ void dot_product(float *result, const float *a, const float *b, int n)
{
    const unsigned tid = flat_tid(), B = flat_bdim();
    float sum = 0.0f;
    for (long long i = (long long)flat_bid() * B + tid; i < n; i += (long long)flat_gdim() * B)
        sum = __fadd_rn(sum, __fmul_rn(a[i], b[i]));
    block_sum_to(result, sum);
}

// data0[x + 1024*y] = sum over l < 16, r < 64 of
//     [data1[64*l + r] == data2[start_pos + y]] * data3[1024*r + x + 65536*l]
// for block (x, y) of a 1024 x 2 grid of 16-thread blocks. Thread l forms its 64
// terms in order of r (the flag is multiplied in, never branched on, so a NaN or
// an infinity in data3 propagates as in the reference kernel); thread 0 then adds
// the sixteen partial sums in order of l, which it gets by shuffle instead of the
// shared array and barrier of the reference kernel. Same order of fp32 additions,
// hence the same bits.
extern "C" __global__ void __launch_bounds__(16)
r_2_1024_16_64(float *data0, const int *data1, const int *data2, const float *data3, const int start_pos)
{
    const int x = blockIdx.x, y = blockIdx.y, l = threadIdx.x;
    const int key = data2[start_pos + y];
    const int *flags = data1 + (l << 6);
    const float *col = data3 + x + ((size_t)l << 16);
    float acc = 0.0f;
#pragma unroll 16
    for (int r = 0; r < 64; r++)
        acc = __fadd_rn(acc, __fmul_rn(flags[r] == key ? 1.0f : 0.0f, col[(size_t)r << 10]));
    const unsigned mask = __activemask();
    float total = 0.0f;
#pragma unroll
    for (int k = 0; k < 16; k++) total = __fadd_rn(total, __shfl_sync(mask, acc, k));
    if (l == 0) data0[x + (y << 10)] = total;
}
