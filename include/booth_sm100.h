/* booth_sm100.h -- the B200 (sm_100a) execution path behind Booth's launcher.
 *
 * Three layers, all plain C ABI (pointers, sizes, integers; no C++ or Python
 * types), all served by libbooth_sm100.so:
 *
 *   1. sm100_rt_*      a thin shim over the CUDA driver API, the sm_100a twin of
 *                      the reference's nv_rt_* (src/nvidia/nv_rt.h:96-127,
 *                      src/nvidia/nv_rt.c:69-381). It dlopens libcuda.so.1, uses the
 *                      device's primary context (so NCCL and any other runtime-API
 *                      user in the process share it) and loads cubins built by nvcc
 *                      for sm_100a instead of JIT-compiling PTX.
 *   2. booth_sm100_*   the five workloads with launch geometry tuned for B200:
 *                      vector add, saxpy, sum reduction, fp32 GEMM (3xTF32 on
 *                      tcgen05) and the Asian-option Monte Carlo pricer, plus the
 *                      seeded input generator they are measured on.
 *   3. sm100_comm_*    the one collective the path has: an NCCL all-reduce of the
 *                      reduction / Monte Carlo partial sums.
 *
 * bc_runtime.h (same directory) is the reference's own launcher API on top of
 * layer 1. The CPU-launcher symbols at the end of this file let
 * examples/cpu_launch_vadd.c and examples/cpu_launch_matmul.c relink unchanged.
 *
 * There is no CPU fallback anywhere: without a driver, a B200 or the kernel
 * image every entry point returns an error code and prints one line that
 * starts with "sm100_rt:" on stderr. */
#ifndef BOOTH_SM100_H
#define BOOTH_SM100_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes: the numbering of src/nvidia/nv_rt.h:19-25, extended ---- */
#define SM100_OK            0
#define SM100_ERR_DL       -1   /* libcuda / libnccl could not be opened */
#define SM100_ERR_SYM      -2   /* an entry point is missing from the library */
#define SM100_ERR_CUDA     -3   /* a driver call returned an error */
#define SM100_ERR_NO_GPU   -4   /* no device, or the device is not sm_100 */
#define SM100_ERR_IO       -5   /* kernel image file unreadable */
#define SM100_ERR_KERN     -6   /* kernel name not found in the image */
#define SM100_ERR_ARG      -7   /* invalid argument (size, alignment, NULL) */
#define SM100_ERR_NCCL     -8   /* an NCCL call returned an error */

typedef struct sm100_dev sm100_dev_t;          /* one GPU: context, stream, kernels */
typedef unsigned long long sm100_ptr_t;        /* device address (CUdeviceptr) */

/* Kernel handle; replaces nv_kern_t (src/nvidia/nv_rt.h:42-46). */
typedef struct sm100_kern {
    void    *mod;            /* CUmodule, NULL when the kernel lives in the built-in image */
    void    *func;           /* CUfunction */
    uint32_t param_bytes;    /* size of the kernel's parameter block */
    uint32_t shared_bytes;   /* static shared memory */
    uint32_t local_bytes;    /* local memory per thread */
    uint32_t _pad;
    char     name[128];
} sm100_kern_t;

/* ---------------------------------------------------------------------------
 * Layer 1: driver shim
 * ------------------------------------------------------------------------- */

/* Replaces nv_rt_init (src/nvidia/nv_rt.c:69-156). ordinal < 0 reads the
 * environment variable BOOTH_DEVICE (default 0). Retains the primary context,
 * creates one stream, and loads the built-in sm_100a kernel image. */
int  sm100_rt_init(sm100_dev_t **out, int ordinal);
/* Replaces nv_rt_shut (src/nvidia/nv_rt.c:160-170). NULL is a no-op. */
void sm100_rt_shut(sm100_dev_t *dev);
/* Number of CUDA devices, or a negative status. */
int  sm100_rt_device_count(void);
const char *sm100_rt_name(const sm100_dev_t *dev);
int  sm100_rt_sm_count(const sm100_dev_t *dev);
int  sm100_rt_ordinal(const sm100_dev_t *dev);
/* Text of the last error recorded on this device ("" if none). */
const char *sm100_rt_errs(const sm100_dev_t *dev);

/* Replaces nv_rt_load (src/nvidia/nv_rt.c:172-248): path names a cubin or
 * fatbin built for sm_100a, or PTX text, which the driver compiles at load (its
 * error log is printed when that fails). */
int  sm100_rt_load(sm100_dev_t *dev, const char *path, const char *name,
                   sm100_kern_t *out);
/* Same, from the kernel image embedded in the library. */
int  sm100_rt_load_builtin(sm100_dev_t *dev, const char *name, sm100_kern_t *out);
/* Replaces nv_rt_unload (src/nvidia/nv_rt.c:252-257). */
void sm100_rt_unload(sm100_dev_t *dev, sm100_kern_t *kern);

/* Replace nv_rt_alloc / nv_rt_free (src/nvidia/nv_rt.c:261-278); 0 on failure. */
sm100_ptr_t sm100_rt_alloc(sm100_dev_t *dev, size_t size);
void        sm100_rt_free(sm100_dev_t *dev, sm100_ptr_t ptr);
/* Replace nv_rt_h2d / nv_rt_d2h (src/nvidia/nv_rt.c:280-300): synchronous. */
int  sm100_rt_h2d(sm100_dev_t *dev, sm100_ptr_t dst, const void *src, size_t size);
int  sm100_rt_d2h(sm100_dev_t *dev, void *dst, sm100_ptr_t src, size_t size);
/* Asynchronous copies on the device's stream (host memory should be pinned). */
int  sm100_rt_h2d_async(sm100_dev_t *dev, sm100_ptr_t dst, const void *src, size_t size);
int  sm100_rt_d2h_async(sm100_dev_t *dev, void *dst, sm100_ptr_t src, size_t size);
/* Fills size bytes with zero on the device's stream. */
int  sm100_rt_zero(sm100_dev_t *dev, sm100_ptr_t dst, size_t size);

/* Replaces nv_rt_launch (src/nvidia/nv_rt.c:304-327): args points at one
 * pointer per kernel parameter. Unlike the reference the launch is only
 * enqueued on the device's stream; sm100_rt_sync waits. */
int  sm100_rt_launch(sm100_dev_t *dev, const sm100_kern_t *kern,
                     uint32_t gx, uint32_t gy, uint32_t gz,
                     uint32_t bx, uint32_t by, uint32_t bz,
                     uint32_t shmem, void **args);
/* Launch with the packed parameter struct bc_dispatch receives
 * (src/runtime/bc_runtime.c:643-658); args_size beyond the kernel's own
 * parameter block is dropped, a shorter block is zero-padded. */
int  sm100_rt_launch_packed(sm100_dev_t *dev, const sm100_kern_t *kern,
                            uint32_t gx, uint32_t gy, uint32_t gz,
                            uint32_t bx, uint32_t by, uint32_t bz,
                            uint32_t shmem, const void *args, uint32_t args_size);
/* Replaces nv_rt_sync (src/nvidia/nv_rt.c:329-346); waits for the stream. */
int  sm100_rt_sync(sm100_dev_t *dev);

/* Pinned host memory; replace nv_rt_mmap / nv_rt_mfre (src/nvidia/nv_rt.c:348-381). */
int  sm100_rt_hostalloc(sm100_dev_t *dev, void **hp, size_t size);
/* Pinned host memory that kernels can address: *hp is the host pointer, *dp the
 * device address of the same bytes (nv_rt_mmap, src/nvidia/nv_rt.c:348-375).
 * Released with sm100_rt_hostfree. */
int  sm100_rt_hostmap(sm100_dev_t *dev, void **hp, sm100_ptr_t *dp, size_t size);
void sm100_rt_hostfree(sm100_dev_t *dev, void *hp);

/* Device-side timing on the device's stream: tic records an event, toc records
 * a second one, waits for it and returns the milliseconds between the two. */
int  sm100_rt_tic(sm100_dev_t *dev);
int  sm100_rt_toc(sm100_dev_t *dev, float *ms);
/* The stream all of this device's work is enqueued on (a CUstream / cudaStream_t),
 * for callers that want to order their own work or copies with it. */
void *sm100_rt_stream(const sm100_dev_t *dev);
/* Number of kernel launches this device has enqueued since sm100_rt_init. */
unsigned long long sm100_rt_launches(const sm100_dev_t *dev);

/* ---------------------------------------------------------------------------
 * Layer 2: workloads (all asynchronous on the device's stream; device pointers)
 * ------------------------------------------------------------------------- */

/* Seeded inputs. Element i is lane i%4 of Philox4x32-10 with counter
 * (i/4 low word, i/4 high word, 0, 0) and key (seed, stream):
 *   kind 0: float  uniform in [-1,1):   2*u - 1,  u = (x >> 8) * 2^-24
 *   kind 1: float  uniform in [0,1):    u
 *   kind 2: int32  uniform in [-1000,1000]:  (int)(x % 2001) - 1000
 *   kind 3: uint32 the generator's output word x itself
 * The device and host generators give identical bits. first is the index of
 * the first element written to dst (dst[0] is element `first`), so a shard can
 * be generated in place. */
#define BOOTH_FILL_F32_PM1   0
#define BOOTH_FILL_F32_01    1
#define BOOTH_FILL_I32_1000  2
#define BOOTH_FILL_U32_RAW   3
int  booth_sm100_fill(sm100_dev_t *dev, sm100_ptr_t dst, long long first,
                      long long n, uint32_t seed, uint32_t stream, int kind);
void booth_sm100_fill_host(void *dst, long long first, long long n,
                           uint32_t seed, uint32_t stream, int kind, int threads);
/* One Philox4x32-10 block on the host (Salmon et al., SC'11; the generator behind
 * the seeded inputs and the Monte Carlo pricer): counter ctr[0..3], key key[0..1].
 * The image also carries a kernel "philox_words(out, c0, c1, c2, c3, k0, k1)"
 * (sm100_rt_load_builtin) whose thread t writes the block of counter
 * (c0 + t, c1, c2, c3) to out[4t..4t+3]. Both exist so the generator can be held
 * against the known-answer vectors published with Random123; no counterpart in
 * the reference, whose pricer uses a counter hash (src/ocaml/Asian.ml:8-30). */
void booth_sm100_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]);

/* out[i] = x[i] + y[i]: tests/tri_vadd.py:6-16, tests/vector_add.cu:4-10.
 * Vectors of this and the next call: device addresses, 4-byte aligned (any
 * further alignment is found at run time), non-NULL when n > 0, n < 2^31; anything
 * else returns SM100_ERR_ARG before any GPU work. */
int  booth_sm100_vadd(sm100_dev_t *dev, sm100_ptr_t x, sm100_ptr_t y,
                      sm100_ptr_t out, long long n);
/* y[i] = a*x[i] + y[i], product and sum rounded separately:
 * tests/canonical.cu:168-173 as compiled by src/cpu/cpu_emit.c:538-542. */
int  booth_sm100_saxpy(sm100_dev_t *dev, sm100_ptr_t y, sm100_ptr_t x,
                       float a, long long n);
/* The same two operations on HOST vectors: chunks of 16 Mi elements are copied
 * in, computed and copied back in a three-slot pipeline on three streams (uploads,
 * kernels, copies back), so the host-to-device and device-to-host directions of
 * the link overlap and no upload queues behind a kernel. These calls
 * return when the result is in host memory. Page-locked host memory
 * (sm100_rt_hostalloc) runs at link speed; pageable memory works, staged by the
 * driver. They are what the CPU-launcher symbols vector_add and saxpy call
 * (examples/cpu_launch_vadd.c:35 hands host arrays to the kernel). */
int  booth_sm100_vadd_host(sm100_dev_t *dev, const float *x, const float *y, float *out, long long n);
int  booth_sm100_saxpy_host(sm100_dev_t *dev, float *y, const float *x, float a, long long n);
/* Measures the host link of this GPU with page-locked memory it allocates itself:
 * gbs[0] host-to-device alone, gbs[1] device-to-host alone, gbs[2] and gbs[3] the
 * two directions while both run at once (GB/s; `bytes` per copy, `reps` copies per
 * figure after one warm-up). The ceiling the *_host calls above can reach is
 * what this reports. No counterpart in the reference. */
int  booth_sm100_link_probe(sm100_dev_t *dev, size_t bytes, int reps, double gbs[4]);
/* Sum of n int32 with wrapping arithmetic into *out (one int32 on the device):
 * the tg_reduce / reduce_sum shape, tests/tg_reduce.cu:4-26,
 * tests/canonical.cu:59-108. For both sums in must be 4-byte aligned and out
 * aligned to the result's size (4 bytes here, 8 for the fp32 sum's double);
 * anything else returns SM100_ERR_ARG before any GPU work. */
int  booth_sm100_reduce_i32(sm100_dev_t *dev, sm100_ptr_t in, long long n,
                            sm100_ptr_t out);
/* Sum of n float into out[0] (double) on the device; fp32 per-thread partial
 * sums, combined in double. The workload's fp32 answer is (float)out[0]. */
int  booth_sm100_reduce_f32(sm100_dev_t *dev, sm100_ptr_t in, long long n,
                            sm100_ptr_t out);
/* The fp32 sum again, for callers that may not allocate device memory (no
 * cudaMalloc inside a frozen memory pool, in a real-time loop, or in a plug-in whose
 * host owns the GPU's memory). It takes no device handle: it runs on the CUDA
 * runtime's current device and on `stream` (a cudaStream_t, NULL for the default
 * stream) and keeps its segment sums in a 33,024-byte array built into the
 * library, so n is limited to 2^30 elements; larger n returns SM100_ERR_ARG.
 * out[0] (double, device memory, 8-byte aligned) receives the sum; in must be
 * 4-byte aligned; both are checked before any GPU work. The first call on a device
 * loads the library's device code there: make it before any stream capture. Calls
 * share the array: do not let two of them overlap on the GPU. This entry point has
 * no counterpart in the reference. */
int  booth_sm100_reduce_f32_noalloc(sm100_ptr_t in, long long n, sm100_ptr_t out, void *stream);
/* C[M,N] = A[M,K] * B[K,N], row-major fp32, 3xTF32 on the tensor cores:
 * the tests/tri_matmul_k.py:8-23 / tests/canonical.cu:18-50 contraction. Any
 * positive M, N, K (operands are padded to whole tiles in the workspace);
 * multiples of 256 / 256 / 32 waste nothing. Each operand is split into a TF32
 * value and a TF32 remainder and three products are accumulated in fp32 (K in
 * chunks of 128, the chunks added round-to-nearest): relative Frobenius error
 * about 1e-6 for finite inputs of ordinary range. An infinity or NaN in A or B
 * makes the elements of C it reaches NaN (the remainder of an infinity is a NaN),
 * where an fp32 product chain could give an infinity; remainders below 2^-126
 * count as zero. */
int  booth_sm100_gemm(sm100_dev_t *dev, sm100_ptr_t c, sm100_ptr_t a,
                      sm100_ptr_t b, int M, int N, int K);
/* The same with flags. BOOTH_GEMM_B_UNCHANGED: the caller states that b, K, N are
 * those of the previous GEMM on this device and that B's contents have not changed
 * since; the split, transposed copy of B kept in the workspace is then reused
 * instead of rebuilt (it is rebuilt anyway when the library finds a different
 * pointer, shape or workspace). For row blocks of A multiplied against one
 * replicated B, the reference's sharding of this workload. No counterpart in the
 * reference. */
#define BOOTH_GEMM_B_UNCHANGED 1u
/* Test hook, never set it in production: the kernel's TMA producers issue nothing,
 * so its bounded barrier waits run out and the failure report can be observed
 * without faulting the device (the call leaves C unwritten and the next wait on
 * the stream returns SM100_ERR_CUDA). */
#define BOOTH_GEMM_TEST_SILENT_PRODUCER 0x80000000u
int  booth_sm100_gemm_ex(sm100_dev_t *dev, sm100_ptr_t c, sm100_ptr_t a,
                         sm100_ptr_t b, int M, int N, int K, unsigned flags);
/* How long a barrier wait inside the GEMM kernel may last before the kernel gives
 * up, records which wait it was and returns (1..60000 ms; 4000 unless the
 * environment variable BOOTH_SM100_GEMM_WAIT_MS said otherwise at sm100_rt_init).
 * The outcome of a GEMM is reported by the next call that waits for the stream:
 * sm100_rt_sync, sm100_rt_d2h, sm100_rt_h2d, sm100_rt_toc (sm100_rt_free prints
 * it). */
int  booth_sm100_gemm_wait_limit(sm100_dev_t *dev, unsigned ms);

/* Asian-option Monte Carlo (src/ocaml/Asian.ml:32-72 with Philox4x32-10 in
 * place of its counter hash). drift = (r - sigma^2/2)*dt and vol = sigma*sqrt(dt)
 * are computed in fp32 by the caller; nstep must be a multiple of 4. */
typedef struct booth_asian {
    float    s0, strike, drift, vol;
    int32_t  nstep;
    uint32_t k0, k1;            /* Philox key */
    int32_t  precise;           /* 0: MUFU approximations, 1: libm-accurate functions */
} booth_asian_t;
/* Prices paths [path0, path0+npaths) and writes four doubles to out (8-byte
 * aligned) on the device: sum of arithmetic payoffs, sum of geometric payoffs, and the sums of
 * their squares (undiscounted). */
int  booth_sm100_asian(sm100_dev_t *dev, const booth_asian_t *p, long long path0,
                       long long npaths, sm100_ptr_t out);
/* Per-path payoffs, arith[i] and geom[i] for path path0+i (the oracle kernel's
 * own output, for per-path comparison). */
int  booth_sm100_asian_paths(sm100_dev_t *dev, const booth_asian_t *p,
                             long long path0, long long npaths,
                             sm100_ptr_t arith, sm100_ptr_t geom);

/* ---------------------------------------------------------------------------
 * Layer 3: the collective (NCCL over NVLink; libnccl.so.2 is dlopen'ed)
 * The reference has no counterpart: it drives one device only
 * (src/nvidia/nv_rt.c:132, src/runtime/bc_runtime.c:234-244).
 * ------------------------------------------------------------------------- */
typedef struct sm100_comm sm100_comm_t;
#define SM100_COMM_ID_BYTES 128
#define SM100_I32 0
#define SM100_F32 1
#define SM100_F64 2
/* One process per GPU: rank 0 makes an id, the host program hands it to every
 * rank (any transport), each rank calls init_rank with its own device. */
int  sm100_comm_unique_id(void *id128);
int  sm100_comm_init_rank(sm100_comm_t **out, sm100_dev_t *dev, int nranks,
                          int rank, const void *id128);
/* One process, ndev GPUs. */
int  sm100_comm_init_all(sm100_comm_t **out, sm100_dev_t **devs, int ndev);
/* In-place sum over all ranks of count elements at buf, on the device's stream
 * (communicator made by init_rank). */
int  sm100_comm_allreduce_sum(sm100_comm_t *comm, sm100_ptr_t buf, size_t count, int dtype);
/* The same for a communicator made by init_all: one call per device index,
 * all of them between group_begin and group_end. */
int  sm100_comm_allreduce_sum_dev(sm100_comm_t *comm, int index, sm100_ptr_t buf,
                                  size_t count, int dtype);
int  sm100_comm_group_begin(void);
int  sm100_comm_group_end(void);
void sm100_comm_destroy(sm100_comm_t *comm);

/* ---------------------------------------------------------------------------
 * CPU-launcher symbols (host pointers; stage to the GPU, launch, copy back)
 * The signatures are those of examples/cpu_launch_vadd.c:23-24 (also
 * tests/diff/diff_vadd.c:28-29) and examples/cpu_launch_matmul.c:22-26: the
 * kernel's own parameters followed by
 * nthreads (src/cpu/cpu_emit.c:386-431). They have no error channel; on failure
 * they print "sm100_rt: ..." and abort(), they never compute on the CPU.
 * Like the reference's objects they may be called from several host threads at
 * once (one range each); such calls share one device and take turns.
 * ------------------------------------------------------------------------- */
void vector_add(float *x, float *y, float *out, int n_elements, int block_size,
                int nthreads);
void matmul(float *a, float *b, float *c, int stride_am, int stride_ak,
            int stride_bk, int stride_bn, int stride_cm, int stride_cn,
            int nthreads);
void matmul_k(float *a, float *b, float *c, int K, int stride_am, int stride_ak,
              int stride_bk, int stride_bn, int stride_cm, int stride_cn,
              int nthreads);
void saxpy(float *y, float *x, float a, int n, int nthreads);
/* The guarded vector add of tests/ocaml/vadd_k.bir as tests/build/run_vadd.c:12
 * declares it: c[i] = a[i] + b[i] for i < min(n, nthreads). */
void vadd(const float *a, const float *b, float *c, int n, int nthreads);

#ifdef __cplusplus
}
#endif
#endif /* BOOTH_SM100_H */
