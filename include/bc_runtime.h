/* bc_runtime.h -- Booth's launcher C API, served by the B200 (sm_100a) runtime.
 *
 * This header declares exactly the interface of the reference's
 * src/runtime/bc_runtime.h:11-67, so a host program written against that file
 * (examples/launch_saxpy.c) compiles and links against libbooth_sm100 without
 * a change. Behind it sits the CUDA driver API instead of HSA:
 *
 *   bc_device_init      src/runtime/bc_runtime.c:326-443   open the driver, take a GPU
 *   bc_device_shutdown  src/runtime/bc_runtime.c:445-456
 *   bc_load_kernel      src/runtime/bc_runtime.c:463-557   path is a cubin/fatbin file
 *   bc_unload_kernel    src/runtime/bc_runtime.c:559-571
 *   bc_alloc / bc_free  src/runtime/bc_runtime.c:575-593   bc_free(NULL) is a no-op
 *   bc_trak             src/runtime/bc_runtime.c:595-602   label an allocation
 *   bc_copy_h2d / d2h   src/runtime/bc_runtime.c:604-624   synchronous copies
 *   bc_dispatch         src/runtime/bc_runtime.c:628-736   synchronous launch
 *
 * Differences a caller can observe: none in signatures, sizes or error codes.
 * The device is chosen by the environment variable BOOTH_DEVICE (default 0);
 * BC_RT_ERR_HSA means "a driver call failed". */
#ifndef BC_RUNTIME_H
#define BC_RUNTIME_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BC_RT_OK            0
#define BC_RT_ERR_DLOPEN   -1   /* the driver library could not be opened */
#define BC_RT_ERR_DLSYM    -2   /* a driver entry point is missing */
#define BC_RT_ERR_HSA      -3   /* a driver call returned an error */
#define BC_RT_ERR_NO_GPU   -4   /* no usable GPU */
#define BC_RT_ERR_NO_MEM   -5   /* a required memory pool is missing */
#define BC_RT_ERR_IO       -6   /* the kernel file could not be read */
#define BC_RT_ERR_SYMBOL   -7   /* no kernel of that name in the file */

/* Caller-owned kernel handle; field order and sizes as in the reference
 * (src/runtime/bc_runtime.h:24-32). Here kernel_object holds the CUfunction,
 * _exec the CUmodule, kernarg_size the kernel's parameter-block size,
 * group_size its static shared memory and private_size its local memory. */
typedef struct bc_kernel {
    uint64_t kernel_object;
    uint32_t kernarg_size;
    uint32_t group_size;
    uint32_t private_size;
    uint64_t _exec;
    uint64_t _reader;
} bc_kernel_t;

/* Caller-owned, stack-allocatable device context of 384 opaque bytes
 * (src/runtime/bc_runtime.h:36-39). */
#define BC_DEVICE_OPAQUE_SIZE 384
typedef struct bc_device {
    uint8_t _data[BC_DEVICE_OPAQUE_SIZE];
} bc_device_t;

int  bc_device_init(bc_device_t *dev);
void bc_device_shutdown(bc_device_t *dev);

/* kernel_name is the bare name ("saxpy"). */
int  bc_load_kernel(bc_device_t *dev, const char *hsaco_path,
                    const char *kernel_name, bc_kernel_t *out);
void bc_unload_kernel(bc_device_t *dev, bc_kernel_t *kern);

void *bc_alloc(bc_device_t *dev, size_t size);
void  bc_free(bc_device_t *dev, void *ptr);

/* Records a label for an allocation; a failed launch prints the labelled
 * buffers that were in flight. */
void bc_trak(bc_device_t *dev, void *ptr, size_t size,
             const char *label, int flags);

int bc_copy_h2d(bc_device_t *dev, void *dst, const void *src, size_t size);
int bc_copy_d2h(bc_device_t *dev, void *dst, const void *src, size_t size);

/* Launches and waits. grid counts blocks, block counts threads; a zero
 * dimension is taken as 1. args is the packed parameter struct in natural C
 * layout; bytes beyond the kernel's own parameter block are ignored. */
int bc_dispatch(bc_device_t *dev, const bc_kernel_t *kern,
                uint32_t grid_x, uint32_t grid_y, uint32_t grid_z,
                uint32_t block_x, uint32_t block_y, uint32_t block_z,
                const void *args, uint32_t args_size);

#ifdef __cplusplus
}
#endif
#endif /* BC_RUNTIME_H */
