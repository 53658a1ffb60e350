// gemm_tf32x3.cu -- fp32 GEMM C = A.B on the sm_100a tensor cores with 3xTF32.
//
// The contraction is the reference's matmul (tests/tri_matmul_k.py:8-23,
// tests/canonical.cu:18-50): row-major fp32 A[M,K], B[K,N], C[M,N]. The tensor
// cores multiply TF32 (10-bit mantissa) operands, so every fp32 operand is split
// into hi = tf32(x) and lo = tf32(x - hi) and the product is rebuilt from three
// MMAs accumulated in fp32 in tensor memory:
//     a.b  ~=  a_lo.b_hi + a_hi.b_lo + a_hi.b_hi        (a_lo.b_lo ~ 2^-22 dropped)
// which keeps the result within ~1e-6 of an fp32 GEMM.
//
// Any positive M, N, K: the split kernels write the planes padded with zeros to
// whole tiles (Mp, Np, Kp), the contraction runs on the padded planes (K here is
// Kp), and the epilogue stores only the M x N that exist.
//
// Two launches per GEMM:
//   gemm_prepass    A[M,K]  -> A_hi, A_lo [Mp,Kp]          (elementwise, streaming)
//                   B[K,N]  -> Bt_hi, Bt_lo [Np,Kp]        (split + transpose through
//                   shared memory, so both MMA operands are K-major), and, for the
//                   one-tile-per-cluster pair form only, zeros in the tiles of C that
//                   two clusters add into
//   the contraction, in one of three forms: gemm_tf32x3 (below: one CTA per tile),
//                   gemm_tf32x3_2cta (a CTA pair per 256 x 256 tile) and
//                   gemm_tf32x3_persist (CTA pairs that stay and walk a list of
//                   tiles; the host's choice for 256-row tiles). The roles are the
//                   same in all three:
//   gemm_tf32x3     one 128 x BN tile of C per CTA:
//       warp 0, one lane : TMA producer. cp.async.bulk.tensor (128-byte swizzle, no
//                          multicast) brings the four operand tiles of a 32-wide
//                          K block into a ring of shared-memory stages and signals
//                          the stage's "full" mbarrier with the byte count.
//       warp 1, one lane : MMA issuer. Per K block 4 x 3 tcgen05.mma.kind::tf32
//                          (M=128, N=BN, K=8) into an fp32 accumulator of BN
//                          columns in TMEM; tcgen05.commit releases the stage
//                          ("empty" mbarrier) and, after each chunk of K, hands
//                          the accumulator to the epilogue warps.
//       warps 2-9        : running sum + epilogue. tcgen05.ld of each finished
//                          chunk, fp32 round-to-nearest adds into registers, and
//                          at the end 512-byte row segments stored to C.
// Every mbarrier wait is bounded by a wall-clock limit (%globaltimer, wait_ns); on
// expiry the kernel records a code in *status, lets copies in flight drain, frees
// its TMEM and returns, so a logic error cannot hang the device. silent_producer
// (host-side fault injection for the tests) keeps the TMA producer from issuing
// anything, so the MMA issuer's and the epilogue's waits run out and exactly that
// path is exercised.
#include "common.cuh"
#include <cuda.h>

namespace gemm {

constexpr int BM = 128;          // rows of C per CTA = TMEM lanes
constexpr int BK = 32;           // fp32 per K block = one 128-byte swizzle row
constexpr int UMMA_K = 8;        // K of one tcgen05.mma.kind::tf32

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long globaltimer()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// Where a wait reports to and how long it may last.
struct WaitCtl { int *status; unsigned long long limit_ns; };

// Bounded wait: false when the limit ran out (an error code has been recorded).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtl &w, int code)
{
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = globaltimer();
    while (!mbar_try_wait(bar, parity)) {
        if (globaltimer() - t0 > w.limit_ns) { atomicCAS(w.status, 0, code); return false; }
    }
    return true;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes,
// 128-byte swizzle: 8-row groups are 1024 bytes apart (SBO), descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr)
{
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor: D = fp32, A = B = TF32, both K-major, M = 128, N = bn.
__host__ __device__ constexpr uint32_t instr_desc(int bn)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}

__device__ __forceinline__ float to_tf32(float x)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

}  // namespace gemm

namespace gemm {

// A[M,K] row-major -> hi/lo planes [Mp,Kp] (Mp >= M, Kp >= K, Kp % 4 == 0), zero in
// the padding: hi = tf32(a), lo = tf32(a - hi). Without padding and with K % 4 == 0
// the planes are walked as one flat array of 16-byte chunks. Block `blk` of
// `nblk` blocks of 256 threads.
__device__ __forceinline__ void split_a_part(const float *__restrict__ a, float4 *__restrict__ hi, float4 *__restrict__ lo,
                                             int M, int K, int Mp, int Kp, unsigned blk, unsigned nblk)
{
    const long long T = (long long)nblk * 256;
    const long long kp4 = Kp >> 2, total = (long long)Mp * kp4;
    const bool flat = M == Mp && K == Kp && (((uintptr_t)a) & 15) == 0;
    for (long long i = (long long)blk * 256 + threadIdx.x; i < total; i += T) {
        float4 v;
        if (flat) {
            v = __ldcs(reinterpret_cast<const float4 *>(a) + i);
        } else {
            const long long row = i / kp4;
            const int k = (int)(i - row * kp4) << 2;
            const float *src = a + row * K + k;
            v.x = (row < M && k + 0 < K) ? src[0] : 0.0f;
            v.y = (row < M && k + 1 < K) ? src[1] : 0.0f;
            v.z = (row < M && k + 2 < K) ? src[2] : 0.0f;
            v.w = (row < M && k + 3 < K) ? src[3] : 0.0f;
        }
        float4 h, l;
        h.x = to_tf32(v.x); l.x = to_tf32(v.x - h.x);
        h.y = to_tf32(v.y); l.y = to_tf32(v.y - h.y);
        h.z = to_tf32(v.z); l.z = to_tf32(v.z - h.z);
        h.w = to_tf32(v.w); l.w = to_tf32(v.w - h.w);
        hi[i] = h;
        lo[i] = l;
    }
}

// B[K,N] row-major -> hi/lo planes of B^T, [Np,Kp] row-major, zero in the padding.
// One 64x64 tile (tile column bx of B^T rows, tile row by of K) through shared
// memory (padded against bank conflicts), 256 threads: rows of B are read in
// 256-byte runs (16-byte loads when N and the pointer allow), rows of B^T written
// in 256-byte runs of 16-byte stores.
__device__ __forceinline__ void split_bt_part(const float *__restrict__ b, float *__restrict__ hi, float *__restrict__ lo,
                                              int K, int N, int Kp, float (*tile)[65], int bx, int by)
{
    const int n0 = bx * 64, k0 = by * 64;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;          // 16 x 16
    const bool vec = (N & 3) == 0 && (((uintptr_t)b) & 15) == 0;
#pragma unroll
    for (int p = 0; p < 4; p++) {
        const int k = k0 + ty + 16 * p, n = n0 + 4 * tx;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k < K) {
            const float *src = b + (long long)k * N + n;
            if (vec && n + 3 < N) v = __ldcs(reinterpret_cast<const float4 *>(src));
            else {
                if (n + 0 < N) v.x = src[0];
                if (n + 1 < N) v.y = src[1];
                if (n + 2 < N) v.z = src[2];
                if (n + 3 < N) v.w = src[3];
            }
        }
        float *t = &tile[ty + 16 * p][4 * tx];
        t[0] = v.x; t[1] = v.y; t[2] = v.z; t[3] = v.w;
    }
    __syncthreads();
#pragma unroll
    for (int p = 0; p < 4; p++) {
        const int nl = ty + 16 * p, k = k0 + 4 * tx;                 // one row of B^T, four consecutive k
        if (k >= Kp) continue;
        float4 h, l;
        const float v0 = tile[4 * tx + 0][nl], v1 = tile[4 * tx + 1][nl], v2 = tile[4 * tx + 2][nl], v3 = tile[4 * tx + 3][nl];
        h.x = to_tf32(v0); l.x = to_tf32(v0 - h.x);
        h.y = to_tf32(v1); l.y = to_tf32(v1 - h.y);
        h.z = to_tf32(v2); l.z = to_tf32(v2 - h.z);
        h.w = to_tf32(v3); l.w = to_tf32(v3 - h.w);
        const long long o = (long long)(n0 + nl) * Kp + k;
        *reinterpret_cast<float4 *>(hi + o) = h;
        *reinterpret_cast<float4 *>(lo + o) = l;
    }
}

// Pair-tile index -> (tile row, tile column). Tiles are numbered in groups of
// eight tile rows, column by column inside a group, so the ~74 tiles that run at
// the same time form a block about 8 tall and 9 wide and share their A and B
// panels through L2 (a row-major numbering would touch every panel of B in
// every wave).
__device__ __forceinline__ void pair_tile_coords(int tile, int tiles_m, int tiles_n, int &tm, int &tn)
{
    constexpr int GROUP_M = 8;
    const int per_group = GROUP_M * tiles_n;
    const int g = tile / per_group, first_m = g * GROUP_M;
    const int rows = min(tiles_m - first_m, GROUP_M);
    const int in_group = tile - g * per_group;
    tm = first_m + in_group % rows;
    tn = in_group / rows;
}

// Zeroes one 256 x 256 tile of C (numbering of pair_tile_coords), clipped to
// M x N: a tile two clusters will add their halves of K into.
__device__ __forceinline__ void zero_tile_part(float *__restrict__ c, int M, int N, int tiles_n, int tile)
{
    int tm, tn;
    pair_tile_coords(tile, (M + 255) / 256, tiles_n, tm, tn);
    const int r0 = tm * 256, c0 = tn * 256;
    if ((N & 3) == 0 && (((uintptr_t)c) & 15) == 0) {
        for (int i = threadIdx.x; i < 256 * 64; i += 256) {
            const int r = r0 + (i >> 6), col = c0 + ((i & 63) << 2);
            if (r < M && col < N) *reinterpret_cast<float4 *>(c + (long long)r * N + col) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    } else {
        for (int i = threadIdx.x; i < 256 * 256; i += 256) {
            const int r = r0 + (i >> 8), col = c0 + (i & 255);
            if (r < M && col < N) c[(long long)r * N + col] = 0.0f;
        }
    }
}
}  // namespace gemm

// Everything the contraction needs beforehand, in ONE launch of 256-thread blocks
// (grid = a_blocks + b_blocks + n_zero):
//   blocks [0, a_blocks)                     split A into its hi/lo planes;
//   blocks [a_blocks, a_blocks + b_blocks)   split and transpose 64 x 64 tiles of B
//                                            (b_blocks = 0 when the planes of B are kept);
//   the last n_zero blocks                   zero the tiles of C that two clusters share
//                                            (one-tile-per-cluster contraction only).
// The parts are independent and all bound by HBM, so they stream side by side.
// Launched with programmatic stream serialization: the grid is set up while the
// previous kernel on the stream drains, waits for that kernel's memory (it may
// still be reading the planes, or writing a and b), then lets the contraction
// behind it do the same.
extern "C" __global__ void __launch_bounds__(256)
gemm_prepass(const float *__restrict__ a, float4 *__restrict__ a_hi, float4 *__restrict__ a_lo, int M, int K, int Mp, int Kp,
             const float *__restrict__ b, float *__restrict__ b_hi, float *__restrict__ b_lo, int N, int Np,
             float *__restrict__ c, int tiles_n, int tile_from, unsigned a_blocks, unsigned b_blocks)
{
    __shared__ float tile[64][65];            // [k][n], used by the B part
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const unsigned blk = blockIdx.x;
    if (blk < a_blocks) {
        gemm::split_a_part(a, a_hi, a_lo, M, K, Mp, Kp, blk, a_blocks);
    } else if (blk < a_blocks + b_blocks) {
        const unsigned t = blk - a_blocks, nbx = (unsigned)Np / 64u;
        gemm::split_bt_part(b, b_hi, b_lo, K, N, Kp, tile, (int)(t % nbx), (int)(t / nbx));
    } else {
        gemm::zero_tile_part(c, M, N, tiles_n, tile_from + (int)(blk - a_blocks - b_blocks));
    }
}

namespace gemm {
// One thread's HALF consecutive columns of one row of C, from its register sums.
// Whole 16-byte stores when the row segment lies inside C and is aligned, masked
// scalar stores at a ragged right edge; rows beyond M are padding and are dropped.
// add_row is the same for a tile whose K range is shared by two clusters: C was
// zeroed beforehand and both halves are added with fp32 atomics (two addends on
// zero: the sum does not depend on their order).
template <int HALF>
__device__ __forceinline__ void add_row(float *__restrict__ c, const float (&acc)[HALF], int row, int col0, int M, int N)
{
    if (row >= M) return;
    float *dst = c + (long long)row * N + col0;
#pragma unroll
    for (int j = 0; j < HALF; j++)
        if (col0 + j < N) atomicAdd(dst + j, acc[j]);
}

template <int HALF>
__device__ __forceinline__ void store_row(float *__restrict__ c, const float (&acc)[HALF], int row, int col0, int M, int N)
{
    if (row >= M) return;
    float *dst = c + (long long)row * N + col0;
    if (col0 + HALF <= N && (N & 3) == 0 && (((uintptr_t)c) & 15) == 0) {
#pragma unroll
        for (int j = 0; j < HALF / 4; j++)
            reinterpret_cast<float4 *>(dst)[j] = make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < HALF; j++)
            if (col0 + j < N) dst[j] = acc[j];
    }
}
}  // namespace gemm

// One 128 x BN tile of C per CTA; grid (N/BN, M/128), 320 threads,
// dynamic shared memory = STAGES * (2*128 + 2*BN) * 128 bytes + 1024 (alignment).
//
// Accumulation. The tensor core adds into its fp32 accumulator with truncation,
// so one long accumulation over K drifts (measured: relative error ~7e-9 * K).
// The K loop is therefore cut into chunks of CHUNK_KB K blocks (128 values of K):
// each chunk is accumulated in TMEM starting from zero, then the eight epilogue
// warps pull it into registers (tcgen05.ld) and add it to a running fp32 sum
// with round-to-nearest adds on the CUDA cores. Two TMEM accumulators alternate,
// so the MMA issuer starts the next chunk while the previous one is drained.
template <int BN, int STAGES>
__device__ __forceinline__ void gemm_tile(const CUtensorMap *map_a_hi, const CUtensorMap *map_a_lo,
                                          const CUtensorMap *map_b_hi, const CUtensorMap *map_b_lo,
                                          float *__restrict__ c, int M, int N, int K, int *status_word,
                                          unsigned long long wait_ns, int silent_producer)
{
    using namespace gemm;
    const WaitCtl status = { status_word, wait_ns };
    constexpr uint32_t A_BYTES = BM * BK * 4, B_BYTES = BN * BK * 4;
    constexpr uint32_t STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
    constexpr int CHUNK_KB = 4;                 // K blocks per TMEM accumulation
    constexpr int HALF = BN / 2;                // columns of C per epilogue warp
    constexpr uint32_t TMEM_COLS = 2 * BN;      // two accumulators

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
    __shared__ uint32_t s_tmem;

    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;    // swizzle atoms are 1024-byte aligned
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t acc_full0 = smem_u32(&bars[2 * STAGES]), acc_empty0 = smem_u32(&bars[2 * STAGES + 2]);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int nkb = K / BK;
    const int nchunk = (nkb + CHUNK_KB - 1) / CHUNK_KB;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; b++) { mbar_init(acc_full0 + 8 * b, 1); mbar_init(acc_empty0 + 8 * b, 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (warp == 0) {        // one warp allocates the tensor memory columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    // Everything above touched only this CTA's own shared and tensor memory, so
    // under programmatic stream serialization it overlaps the tail of the kernel
    // before (the operand split). The planes and C are touched only from here on.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");

    if (warp == 0) {
        // ---- TMA producer (one lane) ----
        if (lane == 0 && !silent_producer) {
            for (int kb = 0; kb < nkb; kb++) {
                const int s = kb % STAGES;
                const uint32_t ph = (uint32_t)(kb / STAGES) & 1u;
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, status, 1)) break;
                const uint32_t st = smem0 + (uint32_t)s * STAGE_BYTES, full = full0 + 8 * s;
                mbar_expect_tx(full, STAGE_BYTES);
                tma_load_2d(st, map_a_hi, full, kb * BK, m0);
                tma_load_2d(st + A_BYTES, map_a_lo, full, kb * BK, m0);
                tma_load_2d(st + 2 * A_BYTES, map_b_hi, full, kb * BK, n0);
                tma_load_2d(st + 2 * A_BYTES + B_BYTES, map_b_lo, full, kb * BK, n0);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---- MMA issuer (one lane) ----
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BN);
            bool ok = true;
            int kb = 0;
            for (int ch = 0; ch < nchunk && ok; ch++) {
                const uint32_t buf = (uint32_t)ch & 1u;
                ok = mbar_wait(acc_empty0 + 8 * buf, (((uint32_t)ch >> 1) & 1u) ^ 1u, status, 4);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tacc = tmem + buf * (uint32_t)BN;
                const int kb_end = min(kb + CHUNK_KB, nkb);
                for (bool first = true; kb < kb_end; kb++) {
                    const int s = kb % STAGES;
                    const uint32_t ph = (uint32_t)(kb / STAGES) & 1u;
                    ok = mbar_wait(full0 + 8 * s, ph, status, 2);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t st = smem0 + (uint32_t)s * STAGE_BYTES;
                    const uint64_t a_hi = smem_desc(st), a_lo = smem_desc(st + A_BYTES);
                    const uint64_t b_hi = smem_desc(st + 2 * A_BYTES), b_lo = smem_desc(st + 2 * A_BYTES + B_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) {
                        const uint64_t adv = (uint64_t)((k * UMMA_K * 4) >> 4);   // 32 bytes along K inside the swizzle row
                        umma_tf32(tacc, a_lo + adv, b_hi + adv, idesc, first ? 0u : 1u);
                        umma_tf32(tacc, a_hi + adv, b_lo + adv, idesc, 1u);
                        umma_tf32(tacc, a_hi + adv, b_hi + adv, idesc, 1u);
                        first = false;
                    }
                    umma_commit(empty0 + 8 * s);          // frees the stage once these MMAs have read it
                }
                umma_commit(acc_full0 + 8 * buf);         // arrives when the chunk's MMAs have finished
            }
        }
        __syncwarp();
    } else {
        // ---- accumulate + epilogue: warps 2..9. Warp w may touch TMEM lanes
        // 32*(w%4)..+31 (rows of the tile); warps 2-5 take the left half of the
        // columns, warps 6-9 the right half. ----
        const int q = warp & 3, h = (warp - 2) >> 2;
        float acc[HALF];
#pragma unroll
        for (int j = 0; j < HALF; j++) acc[j] = 0.0f;
        bool ok = true;
        for (int ch = 0; ch < nchunk; ch++) {
            const uint32_t buf = (uint32_t)ch & 1u;
            ok = __all_sync(0xffffffffu, ok && mbar_wait(acc_full0 + 8 * buf, ((uint32_t)ch >> 1) & 1u, status, 3));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tsrc = tmem + ((uint32_t)(q * 32) << 16) + buf * (uint32_t)BN + (uint32_t)(h * HALF);
#pragma unroll
            for (int cc = 0; cc < HALF / 32; cc++) {
                uint32_t r[32];
                tmem_ld32(tsrc + (uint32_t)(cc * 32), r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 32; j++) acc[cc * 32 + j] = __fadd_rn(acc[cc * 32 + j], __uint_as_float(r[j]));
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0)
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty0 + 8 * buf) : "memory");
        }
        if (__all_sync(0xffffffffu, ok && *(volatile int *)status_word == 0)) {
            store_row<HALF>(c, acc, m0 + q * 32 + lane, n0 + h * HALF, M, N);
        } else {
            // A wait ran out: give copies that may still be in flight time to
            // land before the shared memory is released.
            for (int i = 0; i < 64; i++) __nanosleep(4000);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

extern "C" __global__ void __launch_bounds__(320, 1)
gemm_tf32x3(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
            const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
            float *c, int M, int N, int Np, int K, int split_from, int *status, unsigned long long wait_ns, int silent_producer)
{
    (void)Np; (void)split_from;
    gemm_tile<256, 2>(&map_a_hi, &map_a_lo, &map_b_hi, &map_b_lo, c, M, N, K, status, wait_ns, silent_producer);
}

extern "C" __global__ void __launch_bounds__(320, 1)
gemm_tf32x3_n128(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                 const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
                 float *c, int M, int N, int Np, int K, int split_from, int *status, unsigned long long wait_ns, int silent_producer)
{
    (void)Np; (void)split_from;
    gemm_tile<128, 3>(&map_a_hi, &map_a_lo, &map_b_hi, &map_b_lo, c, M, N, K, status, wait_ns, silent_producer);
}


// ---------------------------------------------------------------------------
// Two-CTA form: a cluster of two CTAs on neighbouring SMs computes one 256 x 256
// tile of C with tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 8).
//
//   CTA r of the pair loads the 128 rows r*128.. of the A tile and the 128 rows
//   (values of n) r*128.. of the B^T tile, hi and lo planes: 64 KB per 32-wide K
//   block, so three stages fit where the one-CTA form has two, and every operand
//   byte that crosses L2 -> SM feeds 256 x 256 instead of 128 x 256 products.
//   Both producers signal the LEADER's "full" barrier (cp.async.bulk.tensor with
//   .cta_group::2 lets the completion land on the peer's mbarrier; no multicast).
//   The leader's single MMA thread issues for the pair; tcgen05.commit with
//   .multicast::cluster releases the stage in both CTAs and hands each CTA its
//   half of the accumulator (rows r*128.. live in CTA r's tensor memory).
//   Each CTA's warps 2-9 drain their own TMEM into register sums exactly as in
//   the one-CTA form; the peer's warps arrive on the leader's "accumulator empty"
//   barrier through its shared::cluster address.
// All waits stay bounded; both CTAs meet at a cluster barrier before any of them
// frees tensor memory or exits, so neither touches the other's shared memory
// after it is gone.
namespace gemm {

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank)
{
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_addr), "r"(rank));
    return a;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// The destination is this CTA's shared memory; the completion is counted on
// `bar`, a shared::cluster address that may belong to the peer CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_tf32_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the barrier at this shared-memory offset in both CTAs of the pair.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__host__ __device__ constexpr uint32_t instr_desc_pair(int bn)     // M = 256 across the pair
{
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

}  // namespace gemm

// grid.x = 2 * (M/256) * (N/BN), clusters of 2 along x, 320 threads, dynamic shared
// memory = STAGES * (32 KB + BN * 128 B) + 1024. BN = 256 with 3 stages is the
// form the host launches; BN = 128 with 4 stages is kept for experiments (it
// fills the last wave of mid-sized problems but the narrower MMA measured 20 %
// slower).
template <int BN, int STAGES>
__device__ __forceinline__ void gemm_pair_tile(const CUtensorMap &map_a_hi, const CUtensorMap &map_a_lo,
                                               const CUtensorMap &map_b_hi, const CUtensorMap &map_b_lo,
                                               float *__restrict__ c, int M, int N, int Np, int K, int split_from, int *status_word,
                                               unsigned long long wait_ns, int silent_producer)
{
    using namespace gemm;
    const WaitCtl status = { status_word, wait_ns };
    constexpr int HALF_N = BN / 2;
    constexpr uint32_t A_BYTES = BM * BK * 4, B_BYTES = HALF_N * BK * 4;
    constexpr uint32_t STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;          // per CTA
    constexpr int CHUNK_KB = 4;
    constexpr int HALF = BN / 2;                                         // columns per epilogue warp
    constexpr uint32_t TMEM_COLS = 2 * BN;

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
    __shared__ uint32_t s_tmem;

    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t acc_full0 = smem_u32(&bars[2 * STAGES]), acc_empty0 = smem_u32(&bars[2 * STAGES + 2]);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = Np / BN;
    // Clusters [0, split_from) compute one tile each over all of K. From
    // split_from on, two consecutive clusters share a tile and take half of K each
    // (the host uses this for the tiles of a short last wave).
    const int cl = blockIdx.x >> 1;
    const bool shared_tile = cl >= split_from;
    const int tile = shared_tile ? split_from + ((cl - split_from) >> 1) : cl;
    const int kpart = shared_tile ? ((cl - split_from) & 1) : 0;
    int tm, tn;
    pair_tile_coords(tile, (M + 255) / 256, tiles_n, tm, tn);
    const int m0 = tm * 256 + (int)rank * BM;                           // this CTA's rows of A and C
    const int n0 = tn * BN;
    const int nb0 = n0 + (int)rank * HALF_N;                            // this CTA's rows of B^T
    const int nkb = shared_tile ? (K / BK) / 2 : K / BK;             // K blocks this cluster covers
    const int kb0 = kpart * nkb;                                     // ... starting here
    const int nchunk = (nkb + CHUNK_KB - 1) / CHUNK_KB;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; b++) { mbar_init(acc_full0 + 8 * b, 1); mbar_init(acc_empty0 + 8 * b, 16); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (warp == 1) {        // the same warp in both CTAs allocates for the pair
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();     // both CTAs' barriers are initialised before anyone signals them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    asm volatile("griddepcontrol.wait;" ::: "memory");       // see the one-CTA form
    asm volatile("griddepcontrol.launch_dependents;");

    if (warp == 0) {
        // ---- TMA producer, one lane in each CTA; completions count on the leader's barrier ----
        if (lane == 0 && !silent_producer) {
            for (int kb = 0; kb < nkb; kb++) {
                const int s = kb % STAGES;
                const uint32_t ph = (uint32_t)(kb / STAGES) & 1u;
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, status, 1)) break;
                const uint32_t st = smem0 + (uint32_t)s * STAGE_BYTES;
                const uint32_t full_leader = map_to_cta(full0 + 8 * s, 0);
                if (leader) mbar_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);
                tma_load_2d_pair(st, &map_a_hi, full_leader, (kb0 + kb) * BK, m0);
                tma_load_2d_pair(st + A_BYTES, &map_a_lo, full_leader, (kb0 + kb) * BK, m0);
                tma_load_2d_pair(st + 2 * A_BYTES, &map_b_hi, full_leader, (kb0 + kb) * BK, nb0);
                tma_load_2d_pair(st + 2 * A_BYTES + B_BYTES, &map_b_lo, full_leader, (kb0 + kb) * BK, nb0);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---- MMA issuer: one lane of the leader CTA issues for the pair ----
        if (leader && lane == 0) {
            constexpr uint32_t idesc = instr_desc_pair(BN);
            bool ok = true;
            int kb = 0;
            for (int ch = 0; ch < nchunk && ok; ch++) {
                const uint32_t buf = (uint32_t)ch & 1u;
                ok = mbar_wait(acc_empty0 + 8 * buf, (((uint32_t)ch >> 1) & 1u) ^ 1u, status, 4);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tacc = tmem + buf * (uint32_t)BN;
                const int kb_end = min(kb + CHUNK_KB, nkb);
                for (bool first = true; kb < kb_end; kb++) {
                    const int s = kb % STAGES;
                    const uint32_t ph = (uint32_t)(kb / STAGES) & 1u;
                    ok = mbar_wait(full0 + 8 * s, ph, status, 2);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t st = smem0 + (uint32_t)s * STAGE_BYTES;
                    const uint64_t a_hi = smem_desc(st), a_lo = smem_desc(st + A_BYTES);
                    const uint64_t b_hi = smem_desc(st + 2 * A_BYTES), b_lo = smem_desc(st + 2 * A_BYTES + B_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) {
                        const uint64_t adv = (uint64_t)((k * UMMA_K * 4) >> 4);
                        umma_tf32_pair(tacc, a_lo + adv, b_hi + adv, idesc, first ? 0u : 1u);
                        umma_tf32_pair(tacc, a_hi + adv, b_lo + adv, idesc, 1u);
                        umma_tf32_pair(tacc, a_hi + adv, b_hi + adv, idesc, 1u);
                        first = false;
                    }
                    umma_commit_pair(empty0 + 8 * s);          // frees the stage in both CTAs
                }
                umma_commit_pair(acc_full0 + 8 * buf);         // each CTA's half of the chunk is complete
            }
        }
        __syncwarp();
    } else {
        // ---- running sum + epilogue, as in the one-CTA form, on this CTA's 128 rows ----
        const int q = warp & 3, h = (warp - 2) >> 2;
        float acc[HALF];
#pragma unroll
        for (int j = 0; j < HALF; j++) acc[j] = 0.0f;
        bool ok = true;
        for (int ch = 0; ch < nchunk; ch++) {
            const uint32_t buf = (uint32_t)ch & 1u;
            ok = __all_sync(0xffffffffu, ok && mbar_wait(acc_full0 + 8 * buf, ((uint32_t)ch >> 1) & 1u, status, 3));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tsrc = tmem + ((uint32_t)(q * 32) << 16) + buf * (uint32_t)BN + (uint32_t)(h * HALF);
#pragma unroll
            for (int cc = 0; cc < HALF / 32; cc++) {
                uint32_t r[32];
                tmem_ld32(tsrc + (uint32_t)(cc * 32), r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 32; j++) acc[cc * 32 + j] = __fadd_rn(acc[cc * 32 + j], __uint_as_float(r[j]));
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(acc_empty0 + 8 * buf, 0));   // the leader counts both CTAs
        }
        if (__all_sync(0xffffffffu, ok && *(volatile int *)status_word == 0)) {
            if (shared_tile) add_row<HALF>(c, acc, m0 + q * 32 + lane, n0 + h * HALF, M, N);
            else store_row<HALF>(c, acc, m0 + q * 32 + lane, n0 + h * HALF, M, N);
        } else {
            for (int i = 0; i < 64; i++) __nanosleep(4000);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();     // nobody frees or exits while the peer may still signal or read
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(320, 1)
gemm_tf32x3_2cta(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                 const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
                 float *__restrict__ c, int M, int N, int Np, int K, int split_from, int *status, unsigned long long wait_ns,
                 int silent_producer)
{
    gemm_pair_tile<256, 3>(map_a_hi, map_a_lo, map_b_hi, map_b_lo, c, M, N, Np, K, split_from, status, wait_ns, silent_producer);
}

extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(320, 1)
gemm_tf32x3_2cta_n128(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                      const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
                      float *__restrict__ c, int M, int N, int Np, int K, int split_from, int *status, unsigned long long wait_ns,
                 int silent_producer)
{
    gemm_pair_tile<128, 4>(map_a_hi, map_a_lo, map_b_hi, map_b_lo, c, M, N, Np, K, split_from, status, wait_ns, silent_producer);
}


// ---------------------------------------------------------------------------
// Persistent two-CTA form: one cluster per SM pair for the whole GEMM.
//
// The grid is 2 x C CTAs, C = the number of CTA pairs the GPU holds at once, and
// every cluster walks a list of work items instead of exiting after one tile:
//   * full waves: cluster cl computes tiles cl, cl + C, cl + 2C, ... over all of K
//     (the clusters of a wave run in step, so the ~C tiles in flight keep sharing
//     their A and B panels through L2 as in the one-tile-per-cluster form);
//   * the tail (tiles % C tiles that would leave most pairs idle): its K chunks are
//     dealt out evenly, cluster cl takes chunks [cl*U/C, (cl+1)*U/C) of the U chunks
//     of all tail tiles, so a tail tile may be shared by two or more clusters. The
//     cluster that holds a tile's first chunk owns the tile: the others write their
//     partial sums to a per-cluster slot of the workspace and publish them (one
//     word per epilogue warp, set to the call's tag, so nothing needs clearing), the
//     owner adds them to its own sum in cluster order and stores C. A partial is
//     always the FIRST thing its cluster does in the tail and the owner asks for
//     it LAST, so no cluster ever waits for work that waits for it; the wait is
//     bounded like every other wait here. No atomics on C, no zeroed C, and the
//     sum does not depend on timing.
// Staying resident saves the per-tile set-up (barriers, tensor memory) and lets
// the tensor pipe start the next item's first chunks while the eight epilogue
// warps still store the previous tile.
//
// 384 threads: warp 0 TMA producer, warp 1 MMA issuer (and tensor-memory
// allocation), warps 4-11 running sum + epilogue (warp w reads TMEM lanes
// 32*(w%4)..; warps 4-7 the left half of the columns, 8-11 the right half).
namespace gemm {

struct WorkItem { int tile, c0, c1; };          // chunks [c0, c1) of K for this tile

struct Schedule {
    int C, cl, nck, nfull, rem, split;
    long long u0, u1;                           // this cluster's chunks of the tail
    int w;                                      // iteration state
    long long u;
    __device__ __forceinline__ Schedule(int C_, int cl_, int tiles, int nck_, int split_)
        : C(C_), cl(cl_), nck(nck_), nfull(tiles / C_), rem(tiles % C_), split(split_)
    {
        const long long U = (long long)rem * nck;
        u0 = split ? (long long)cl * U / C : 0;
        u1 = split ? (long long)(cl + 1) * U / C : 0;
        w = 0; u = u0;
    }
    __device__ __forceinline__ long long tail_begin(int j) const { return (long long)j * ((long long)rem * nck) / C; }
    __device__ __forceinline__ bool next(WorkItem &it)
    {
        if (w < nfull) { it.tile = w * C + cl; it.c0 = 0; it.c1 = nck; w++; return true; }
        if (!split) {
            if (w == nfull && cl < rem) { it.tile = nfull * C + cl; it.c0 = 0; it.c1 = nck; w++; return true; }
            return false;
        }
        if (u < u1) {
            const long long t = u / nck;
            it.tile = nfull * C + (int)t;
            it.c0 = (int)(u - t * nck);
            const long long left = u1 - u;
            const int room = nck - it.c0;
            it.c1 = it.c0 + (int)(left < room ? left : room);
            u += it.c1 - it.c0;
            return true;
        }
        return false;
    }
};

// Bounded wait for a word in global memory to equal `tag`.
__device__ __forceinline__ bool flag_wait_eq(const unsigned *flag, unsigned tag, const WaitCtl &w, int code)
{
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v == tag) return true;
    const unsigned long long t0 = globaltimer();
    for (;;) {
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v == tag) return true;
        if (globaltimer() - t0 > w.limit_ns) { atomicCAS(w.status, 0, code); return false; }
        __nanosleep(128);
    }
}

// Makes this warp's partial sums visible and sets its hand-over word to the call's tag.
__device__ __forceinline__ void publish_partial(unsigned *flag, unsigned tag, int lane)
{
    __threadfence();
    __syncwarp();
    if (lane == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flag), "r"(tag) : "memory");
}

constexpr int PARTIAL_FLOATS = 2 * 8 * 128 * 32;     // one cluster's slot: [cta][epilogue warp][4 columns][lane][4]

}  // namespace gemm

extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(384, 1)
gemm_tf32x3_persist(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                    const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
                    float *__restrict__ c, int M, int N, int Np, int K, int tail_split,
                    int *status_word, unsigned long long wait_ns, int silent_producer,
                    float *__restrict__ partial_ws, unsigned *__restrict__ flags, unsigned epoch)
{
    using namespace gemm;
    constexpr int BN = 256, STAGES = 3, HALF_N = BN / 2, HALF = BN / 2, CHUNK_KB = 4;
    constexpr uint32_t A_BYTES = BM * BK * 4, B_BYTES = HALF_N * BK * 4;
    constexpr uint32_t STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;          // per CTA
    constexpr uint32_t TMEM_COLS = 2 * BN;
    const WaitCtl status = { status_word, wait_ns };

    extern __shared__ uint8_t smem_persist[];
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
    __shared__ uint32_t s_tmem;

    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const uint32_t smem0 = (smem_u32(smem_persist) + 1023u) & ~1023u;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t acc_full0 = smem_u32(&bars[2 * STAGES]), acc_empty0 = smem_u32(&bars[2 * STAGES + 2]);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (M + 255) / 256, tiles_n = Np / BN;
    const int nkb = K / BK, nck = (nkb + CHUNK_KB - 1) / CHUNK_KB;
    const int C = (int)(gridDim.x >> 1), cl = (int)(blockIdx.x >> 1);
    Schedule sched(C, cl, tiles_m * tiles_n, nck, tail_split);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; b++) { mbar_init(acc_full0 + 8 * b, 1); mbar_init(acc_empty0 + 8 * b, 16); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    asm volatile("griddepcontrol.wait;" ::: "memory");       // the planes, the flags and C are touched only from here on
    asm volatile("griddepcontrol.launch_dependents;");
    // Registers follow the roles (384 threads start with 168 each): the control warpgroup
    // gives up what it does not need, the two epilogue warpgroups (128 running sums per
    // thread) take it. Each warpgroup changes its share as the first thing in its branch.
    if (warp < 4) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
      if (warp == 0) {
        // ---- TMA producer, one lane in each CTA; completions count on the leader's barrier ----
        if (lane == 0 && !silent_producer) {
            uint32_t it = 0;                                           // K blocks issued so far, over all items
            WorkItem wi;
            bool ok = true;
            while (ok && sched.next(wi)) {
                int tm, tn;
                pair_tile_coords(wi.tile, tiles_m, tiles_n, tm, tn);
                const int m0 = tm * 256 + (int)rank * BM, nb0 = tn * BN + (int)rank * HALF_N;
                const int kb_end = min(wi.c1 * CHUNK_KB, nkb);
                for (int kb = wi.c0 * CHUNK_KB; kb < kb_end; kb++, it++) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, status, 1)) { ok = false; break; }
                    const uint32_t st = smem0 + s * STAGE_BYTES;
                    const uint32_t full_leader = map_to_cta(full0 + 8 * s, 0);
                    if (leader) mbar_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);
                    tma_load_2d_pair(st, &map_a_hi, full_leader, kb * BK, m0);
                    tma_load_2d_pair(st + A_BYTES, &map_a_lo, full_leader, kb * BK, m0);
                    tma_load_2d_pair(st + 2 * A_BYTES, &map_b_hi, full_leader, kb * BK, nb0);
                    tma_load_2d_pair(st + 2 * A_BYTES + B_BYTES, &map_b_lo, full_leader, kb * BK, nb0);
                }
            }
        }
        __syncwarp();
      } else if (warp == 1) {
        // ---- MMA issuer: one lane of the leader CTA issues for the pair ----
        if (leader && lane == 0) {
            constexpr uint32_t idesc = instr_desc_pair(BN);
            uint32_t it = 0, g = 0;                                    // K blocks and chunks consumed so far
            WorkItem wi;
            bool ok = true;
            while (ok && sched.next(wi)) {
                for (int ch = wi.c0; ch < wi.c1 && ok; ch++, g++) {
                    const uint32_t buf = g & 1u;
                    ok = mbar_wait(acc_empty0 + 8 * buf, ((g >> 1) & 1u) ^ 1u, status, 4);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t tacc = tmem + buf * (uint32_t)BN;
                    const int kb_end = min((ch + 1) * CHUNK_KB, nkb);
                    bool first = true;
                    for (int kb = ch * CHUNK_KB; kb < kb_end; kb++, it++) {
                        const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                        ok = mbar_wait(full0 + 8 * s, ph, status, 2);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t st = smem0 + s * STAGE_BYTES;
                        const uint64_t a_hi = smem_desc(st), a_lo = smem_desc(st + A_BYTES);
                        const uint64_t b_hi = smem_desc(st + 2 * A_BYTES), b_lo = smem_desc(st + 2 * A_BYTES + B_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; k++) {
                            const uint64_t adv = (uint64_t)((k * UMMA_K * 4) >> 4);
                            umma_tf32_pair(tacc, a_lo + adv, b_hi + adv, idesc, first ? 0u : 1u);
                            umma_tf32_pair(tacc, a_hi + adv, b_lo + adv, idesc, 1u);
                            umma_tf32_pair(tacc, a_hi + adv, b_hi + adv, idesc, 1u);
                            first = false;
                        }
                        umma_commit_pair(empty0 + 8 * s);          // frees the stage in both CTAs
                    }
                    if (ok) umma_commit_pair(acc_full0 + 8 * buf);     // each CTA's half of the chunk is complete
                }
            }
        }
        __syncwarp();
      }
    } else if (warp < 12) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
        // ---- running sum + epilogue on this CTA's 128 rows ----
        const int e = warp - 4, q = warp & 3, h = e >> 2;
        const uint32_t acc_empty_leader0 = map_to_cta(acc_empty0, 0);
        float acc[HALF];
        uint32_t g = 0;
        WorkItem wi;
        bool ok = true;
        // A partial handed over in the middle of the list is published one chunk later: its
        // stores are issued at once, but waiting for them to land there and then (the fence
        // before the release) held the drain up for 6 to 8 us beside the running loads, and
        // the tensor pipe, two chunks ahead at most, stalled for 3 of them.
        unsigned *unpublished = nullptr;
        while (ok && sched.next(wi)) {
#pragma unroll
            for (int j = 0; j < HALF; j++) acc[j] = 0.0f;
            for (int ch = wi.c0; ch < wi.c1; ch++, g++) {
                const uint32_t buf = g & 1u;
                ok = __all_sync(0xffffffffu, ok && mbar_wait(acc_full0 + 8 * buf, (g >> 1) & 1u, status, 3));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tsrc = tmem + ((uint32_t)(q * 32) << 16) + buf * (uint32_t)BN + (uint32_t)(h * HALF);
#pragma unroll
                for (int cc = 0; cc < HALF / 16; cc++) {
                    uint32_t r[16];
                    tmem_ld16(tsrc + (uint32_t)(cc * 16), r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 16; j++) acc[cc * 16 + j] = __fadd_rn(acc[cc * 16 + j], __uint_as_float(r[j]));
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(acc_empty_leader0 + 8 * buf);    // the leader counts both CTAs
                if (unpublished) { publish_partial(unpublished, epoch, lane); unpublished = nullptr; }
            }
            if (!ok) break;
            int tm, tn;
            pair_tile_coords(wi.tile, tiles_m, tiles_n, tm, tn);
            const int row = tm * 256 + (int)rank * BM + q * 32 + lane, col0 = tn * BN + h * HALF;
            // a warp's slot holds [group of 4 columns][lane][4]: every access is 16 bytes a lane, 512 a warp
            const size_t slot = (size_t)(rank * 8 + e) * 128 * 32;
            if (wi.c0 != 0) {
                // not this tile's owner: hand the partial sums over
                float4 *dst = reinterpret_cast<float4 *>(partial_ws + (size_t)cl * PARTIAL_FLOATS + slot) + lane;
#pragma unroll
                for (int j = 0; j < HALF / 4; j++)
                    dst[j * 32] = make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
                // one word per (cluster, CTA, epilogue warp), set to this call's tag: the owner's warp of
                // the same role is the only reader of this warp's sums
                unpublished = flags + cl * 16 + (int)rank * 8 + e;
            } else {
                if (wi.c1 != sched.nck) {
                    // owner of a shared tile: add the partials of the clusters that hold the rest of its K, always
                    // from the last cluster down. The last one holds the tile's end as the first item of its own
                    // list and has handed it over long ago; the ones between work on this tile to their very end,
                    // so their sums arrive last and are waited for last.
                    const long long tile_end = (long long)(wi.tile - sched.nfull * C + 1) * sched.nck;
                    // the last cluster whose share begins before the tile's end: floor(j U / C) < end <=> j U < end C
                    const int jlast = min(C - 1, (int)((tile_end * C - 1) / ((long long)sched.rem * sched.nck)));
                    for (int j = jlast; j > cl && ok; j--) {
                        if (sched.tail_begin(j + 1) == sched.tail_begin(j)) continue;   // that cluster has no work
                        // every lane does the acquire load itself (one broadcast access per warp), so each
                        // lane's reads of the partial sums below are ordered after the writer's release
                        const bool got = flag_wait_eq(flags + j * 16 + (int)rank * 8 + e, epoch, status, 5);
                        ok = __all_sync(0xffffffffu, got);
                        if (!ok) break;
                        const float4 *src = reinterpret_cast<const float4 *>(partial_ws + (size_t)j * PARTIAL_FLOATS + slot) + lane;
#pragma unroll
                        for (int jj = 0; jj < HALF / 4; jj++) {
                            const float4 v = __ldcg(src + jj * 32);
                            acc[4 * jj] = __fadd_rn(acc[4 * jj], v.x);
                            acc[4 * jj + 1] = __fadd_rn(acc[4 * jj + 1], v.y);
                            acc[4 * jj + 2] = __fadd_rn(acc[4 * jj + 2], v.z);
                            acc[4 * jj + 3] = __fadd_rn(acc[4 * jj + 3], v.w);
                        }
                    }
                    if (!ok) break;
                }
                if (*(volatile int *)status_word != 0) { ok = false; break; }
                store_row<HALF>(c, acc, row, col0, M, N);
            }
        }
        if (unpublished) publish_partial(unpublished, epoch, lane);      // the partial was this cluster's last work
        if (!__all_sync(0xffffffffu, ok)) {
            // A wait ran out: give copies that may still be in flight time to land
            // before the shared memory is released.
            for (int i = 0; i < 64; i++) __nanosleep(4000);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();     // nobody frees or exits while the peer may still signal or read
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}
