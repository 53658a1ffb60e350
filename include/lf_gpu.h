/* lf_gpu.h -- the eight-function offload ABI that LFortran-compiled programs call
 * to run a `do concurrent` kernel, served by the sm_100a runtime.
 *
 * Mirrors the declarations of the reference's src/runtime/lf_gpu.h:21-35 (same
 * names, argument order and meaning), so an object file that was compiled against
 * that header links against libbooth_sm100 unchanged. The reference implements the
 * ABI twice, over its CUDA launcher (src/runtime/lf_gpu.c) and over its HSA
 * launcher (src/runtime/lf_gpu_hsa.c); this is the third sibling, over sm100_rt_*.
 *
 * The ABI returns void everywhere and has no error channel: as in the reference
 * (src/runtime/lf_gpu.c:55-59) every failure prints one line on stderr and ends
 * the process with status 1, because handing garbage back to Fortran is worse.
 */
#ifndef BOOTH_SM100_LF_GPU_H
#define BOOTH_SM100_LF_GPU_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct lfortran_gpu_ctx    lfortran_gpu_ctx;
typedef struct lfortran_gpu_kernel lfortran_gpu_kernel;

/* Opens the device (ordinal from BOOTH_DEVICE, default 0). A second call returns
 * the live context (src/runtime/lf_gpu.c:82-94). */
lfortran_gpu_ctx    *lfortran_gpu_init(void);
/* Releases every kernel still loaded, then the device (src/runtime/lf_gpu.c:96-108).
 * NULL or an already closed context is a no-op. */
void                 lfortran_gpu_shutdown(lfortran_gpu_ctx *ctx);

/* Resolves entry_point in a cubin or fatbin built for sm_100a. The file is, in
 * order: `source` when non-empty, $BOOTH_CUBIN when set, "<entry_point>.cubin"
 * when that file exists (the search order of src/runtime/lf_gpu.c:61-78 with the
 * artefact kind changed), and last the kernel image embedded in the library. */
lfortran_gpu_kernel *lfortran_gpu_load_kernel(lfortran_gpu_ctx *ctx, const char *source,
                                              const char *entry_point);
/* Frees the kernel's device buffers and unloads it (src/runtime/lf_gpu.c:144-160). */
void                 lfortran_gpu_release_kernel(lfortran_gpu_kernel *k);

/* Parameter idx is a host array of `size` bytes: a device buffer is allocated and
 * the array copied in now; after the launch it is copied back into the same host
 * array (src/runtime/lf_gpu.c:164-188). idx outside [0,32) is ignored. */
void lfortran_gpu_set_buffer_arg(lfortran_gpu_kernel *k, int idx, void *ptr, size_t size);
/* Parameter idx is a scalar of `size` <= 16 bytes passed by value
 * (src/runtime/lf_gpu.c:190-207). */
void lfortran_gpu_set_scalar_arg(lfortran_gpu_kernel *k, int idx, const void *val, size_t size);

/* grid counts blocks, block counts threads; every entry must be >= 1. Returns
 * after the kernel has finished and every buffer argument is back in its host
 * array (src/runtime/lf_gpu.c:211-244). */
void lfortran_gpu_launch(lfortran_gpu_ctx *ctx, lfortran_gpu_kernel *k, int grid[3], int block[3]);
/* Waits for the device's stream. */
void lfortran_gpu_sync(lfortran_gpu_ctx *ctx);

#ifdef __cplusplus
}
#endif
#endif
