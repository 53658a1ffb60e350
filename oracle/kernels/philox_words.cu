/* Oracle kernel source (test infrastructure): raw Philox4x32-10 output words.
 *
 * The same ten rounds, written the same way, as in asian_paths.cu beside this
 * file; here the four output words are stored as they are, so that the generator
 * every workload's inputs and every Monte Carlo path hang on can be compared with
 * the known-answer vectors published with the Random123 library (Salmon, Moraes,
 * Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11).
 * Written for the reference compiler's x86-64 backend (kath --cpu): the high half
 * of a 32x32 product comes from a 64-bit product because the backend's 32-bit
 * __umulhi multiplies sign-extended slots (src/cpu/cpu_emit.c:448).
 * Thread t computes the block with counter (c0 + t, c1, c2, c3), no carry out of
 * the first word, key (k0, k1), and stores out[4t .. 4t+3]. */

__device__ unsigned int mulhi32(unsigned int a, unsigned int b)
{
    unsigned long long p = (unsigned long long)a * (unsigned long long)b;
    return (unsigned int)(p >> 32);
}

__global__ void philox_words(unsigned int *out, unsigned int c0, unsigned int c1,
                             unsigned int c2, unsigned int c3,
                             unsigned int k0, unsigned int k1)
{
    int t = threadIdx.x;
    unsigned int x0 = c0 + (unsigned int)t;
    unsigned int x1 = c1;
    unsigned int x2 = c2;
    unsigned int x3 = c3;
    unsigned int ka = k0;
    unsigned int kb = k1;
    for (int r = 0; r < 10; r = r + 1) {
        unsigned int hi0 = mulhi32(0xD2511F53u, x0);
        unsigned int lo0 = 0xD2511F53u * x0;
        unsigned int hi1 = mulhi32(0xCD9E8D57u, x2);
        unsigned int lo1 = 0xCD9E8D57u * x2;
        unsigned int n0 = hi1 ^ x1 ^ ka;
        unsigned int n2 = hi0 ^ x3 ^ kb;
        x0 = n0;
        x1 = lo1;
        x2 = n2;
        x3 = lo0;
        ka = ka + 0x9E3779B9u;
        kb = kb + 0xBB67AE85u;
    }
    out[4 * t + 0] = x0;
    out[4 * t + 1] = x1;
    out[4 * t + 2] = x2;
    out[4 * t + 3] = x3;
}
