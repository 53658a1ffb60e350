// tile.cu -- the reference's single-tile Triton matmul kernels, as launched
// through the CPU-launcher symbols matmul / matmul_k.
//
// tests/tri_matmul.py:8-25 and tests/tri_matmul_k.py:8-23 compute one 4x4 output
// tile from strided operands. The reference lowers tl.dot to a flat,
// left-to-right sum of separately rounded products per BLOCK_K slice
// (src/triton/lower.c:1001-1024) and, in the K-loop kernel, adds each slice to a
// zero-initialised accumulator tile (src/triton/lower.c:964-982). One thread per
// output element repeats exactly that order, so the tile is bit-identical to the
// x86-64 backend's. This kernel exists for call compatibility with
// examples/cpu_launch_matmul.c; large GEMMs go through gemm_tf32x3.
extern "C" __global__ void matmul_tile(const float *a, const float *b, float *c, int K, int block_k,
                                       int sam, int sak, int sbk, int sbn, int scm, int scn,
                                       int accumulate)
{
    const int m = threadIdx.x >> 2, n = threadIdx.x & 3;
    if (threadIdx.x >= 16 || blockIdx.x != 0) return;
    float acc = 0.0f;
    for (int k0 = 0; k0 < K; k0 += block_k) {
        float d = __fmul_rn(a[(long long)m * sam + (long long)k0 * sak], b[(long long)k0 * sbk + (long long)n * sbn]);
        for (int k = k0 + 1; k < k0 + block_k; k++)
            d = __fadd_rn(d, __fmul_rn(a[(long long)m * sam + (long long)k * sak],
                                       b[(long long)k * sbk + (long long)n * sbn]));
        acc = accumulate ? __fadd_rn(acc, d) : d;
    }
    c[(long long)m * scm + (long long)n * scn] = acc;
}
