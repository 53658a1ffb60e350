/* Oracle kernel source (test infrastructure): stage 1 of the chunked fp32 sum.
 *
 * Same split-at-the-barrier shape as reduce_chunk_i32.cu. Each thread adds its
 * chunk serially with addss, one rounding per add (src/cpu/cpu_emit.c:538-542).
 * A single serial fp32 sum over 2^30 values in [0,1) saturates at 2^24, so the
 * chunk stays short (4096) and the partials are combined in double on the host. */
__global__ void reduce_chunk_f32(float *partial, float *in, int chunk)
{
    int t = threadIdx.x;
    int base = t * chunk;
    float acc = 0.0f;
    for (int j = 0; j < chunk; j = j + 1)
        acc = acc + in[base + j];
    partial[t] = acc;
}
