/* Oracle kernel source (test infrastructure): stage 1 of the chunked int32 sum.
 *
 * Compiled by the reference compiler's x86-64 backend (kath --cpu) and called
 * through the CPU-launcher convention kernel(params..., nthreads)
 * (src/cpu/cpu_emit.c:386-431): thread t sums its own chunk serially.
 * One launch is one block of serially executed threads and barriers are
 * no-ops there (src/cpu/cpu_emit.c:729), so the tg_reduce shape
 * (tests/tg_reduce.cu:4-26) is split at its barrier: this kernel is the part
 * before it, the combine of partial[] happens on the host.
 * Integer adds are 64-bit adds with a 32-bit store (src/cpu/cpu_emit.c:444-446),
 * i.e. wrapping int32 arithmetic. */
__global__ void reduce_chunk_i32(int *partial, int *in, int chunk)
{
    int t = threadIdx.x;
    int base = t * chunk;
    int acc = 0;
    for (int j = 0; j < chunk; j = j + 1)
        acc = acc + in[base + j];
    partial[t] = acc;
}
