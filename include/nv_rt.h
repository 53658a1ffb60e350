/* nv_rt.h -- the reference's CUDA launcher API served by the sm_100a runtime.
 *
 * The reference's second launcher (src/nvidia/nv_rt.h:102-134, implemented in
 * src/nvidia/nv_rt.c:69-381) wraps the CUDA driver API for its host programs
 * (tests/build/gpu_vadd.c, gpu_reduce.c, gpu_scale.c, src/runtime/lf_gpu.c and the
 * harness tests/numeric/run_numeric.py:230-296 writes). libbooth_sm100 exports the
 * same twelve functions over its own driver shim, so those programs link against
 * the library in place of nv_rt.c, compiled against either this header or the
 * reference's: the two agree on every size, offset and status code.
 *
 * Differences a caller can see:
 *   - the device is BOOTH_DEVICE (default 0) and must be sm_100; its primary
 *     context is used rather than a new one;
 *   - nv_rt_load takes PTX text (compiled by the driver at load), a cubin or a fatbin;
 *   - work is ordered on one stream per device; copies are complete on return and
 *     nv_rt_sync waits for the kernels, as with the reference;
 *   - nv_dev_t carries no driver entry points: the slots the reference fills with
 *     function pointers stay NULL.
 */
#ifndef BOOTH_SM100_NV_RT_H
#define BOOTH_SM100_NV_RT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes (src/nvidia/nv_rt.h:19-25). */
#define NV_RT_OK           0
#define NV_RT_ERR_DL      -1   /* the CUDA driver library could not be opened */
#define NV_RT_ERR_SYM     -2   /* a driver entry point is missing */
#define NV_RT_ERR_CUDA    -3   /* a driver call failed */
#define NV_RT_ERR_NO_GPU  -4   /* no usable GPU */
#define NV_RT_ERR_IO      -5   /* kernel file unreadable */
#define NV_RT_ERR_KERN    -6   /* kernel name not in the module */

typedef unsigned long long CUdevptr;       /* device address (src/nvidia/nv_rt.h:38) */

/* Caller-owned kernel handle, 144 bytes (src/nvidia/nv_rt.h:42-46). */
typedef struct {
    void *mod;                 /* CUmodule */
    void *func;                /* CUfunction */
    char  name[128];
} nv_kern_t;

/* Caller-owned device record, 320 bytes with the reference's offsets
 * (src/nvidia/nv_rt.h:52-91): lib 0, ctx 8, dev 16, dev_name 20, sm_major 148,
 * sm_minor 152, twenty pointer slots from 160. */
typedef struct {
    void *lib;                 /* non-NULL while the device is open (here: the runtime's device object) */
    void *ctx;                 /* the CUDA context in use */
    int   dev;                 /* device ordinal */
    char  dev_name[128];
    int   sm_major;
    int   sm_minor;
    void *reserved[20];        /* the reference keeps driver entry points here; unused */
} nv_dev_t;

int  nv_rt_init(nv_dev_t *dev);
void nv_rt_shut(nv_dev_t *dev);

int  nv_rt_load(nv_dev_t *dev, const char *ptx_path, const char *kern_name, nv_kern_t *out);
void nv_rt_unload(nv_dev_t *dev, nv_kern_t *kern);

CUdevptr nv_rt_alloc(nv_dev_t *dev, size_t size);        /* 0 on failure */
void     nv_rt_free(nv_dev_t *dev, CUdevptr ptr);        /* 0 is a no-op */

int  nv_rt_h2d(nv_dev_t *dev, CUdevptr dst, const void *src, size_t size);
int  nv_rt_d2h(nv_dev_t *dev, void *dst, CUdevptr src, size_t size);

/* grid counts blocks, block counts threads; args holds one pointer per kernel
 * parameter. The launch is enqueued; nv_rt_sync waits (src/nvidia/nv_rt.c:304-346). */
int  nv_rt_launch(nv_dev_t *dev, nv_kern_t *kern, uint32_t gx, uint32_t gy, uint32_t gz,
                  uint32_t bx, uint32_t by, uint32_t bz, uint32_t shmem, void **args);
int  nv_rt_sync(nv_dev_t *dev);

/* Pinned host memory mapped into the device's address space: *hpp for the host,
 * *dpp for kernel arguments (src/nvidia/nv_rt.c:348-381). */
int  nv_rt_mmap(nv_dev_t *dev, void **hpp, CUdevptr *dpp, size_t sz);
void nv_rt_mfre(nv_dev_t *dev, void *hp);

#ifdef __cplusplus
}
#endif
#endif
