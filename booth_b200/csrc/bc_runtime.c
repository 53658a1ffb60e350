/* bc_runtime.c -- Booth's launcher API (bc_*) on a B200.
 *
 * Same entry points, struct sizes, error codes and stderr prefix as the
 * reference's HSA launcher (src/runtime/bc_runtime.c:326-736), implemented on
 * the driver shim in sm100_shim.c. The 384 opaque bytes of bc_device_t hold a
 * tag and a pointer to the heap-allocated device; the reference keeps its HSA
 * function table in the same bytes (src/runtime/bc_runtime.c:213). Unlike the
 * reference, which reads kernel files into one static buffer
 * (src/runtime/bc_runtime.c:460-461), nothing here is shared between devices. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "bc_runtime.h"
#include "sm100_internal.h"

#define BC_TAG 0x30303153434f4f42ull   /* "BOOCS100" */

typedef struct {
    unsigned long long tag;
    sm100_dev_t *dev;
} bc_impl_t;

typedef char bc_impl_fits[(sizeof(bc_impl_t) <= BC_DEVICE_OPAQUE_SIZE) ? 1 : -1];
typedef char bc_kernel_is_40_bytes[(sizeof(bc_kernel_t) == 40) ? 1 : -1];

static sm100_dev_t *D_of(bc_device_t *dev)
{
    bc_impl_t im;
    if (!dev) return NULL;
    memcpy(&im, dev->_data, sizeof im);
    return im.tag == BC_TAG ? im.dev : NULL;
}

static int to_bc(int rc)
{
    switch (rc) {
    case SM100_OK:         return BC_RT_OK;
    case SM100_ERR_DL:     return BC_RT_ERR_DLOPEN;
    case SM100_ERR_SYM:    return BC_RT_ERR_DLSYM;
    case SM100_ERR_NO_GPU: return BC_RT_ERR_NO_GPU;
    case SM100_ERR_IO:     return BC_RT_ERR_IO;
    case SM100_ERR_KERN:   return BC_RT_ERR_SYMBOL;
    default:               return BC_RT_ERR_HSA;
    }
}

int bc_device_init(bc_device_t *dev)
{
    if (!dev) return BC_RT_ERR_NO_GPU;
    memset(dev, 0, sizeof *dev);
    sm100_dev_t *d = NULL;
    int rc = sm100_rt_init(&d, -1);
    if (rc != SM100_OK) {
        fprintf(stderr, "bc_runtime: device init failed (%d)\n", to_bc(rc));
        return to_bc(rc);
    }
    bc_impl_t im = { BC_TAG, d };
    memcpy(dev->_data, &im, sizeof im);
    fprintf(stderr, "bc_runtime: using %s\n", sm100_rt_name(d));
    return BC_RT_OK;
}

void bc_device_shutdown(bc_device_t *dev)
{
    sm100_dev_t *d = D_of(dev);
    if (d) sm100_rt_shut(d);
    if (dev) memset(dev, 0, sizeof *dev);
}

int bc_load_kernel(bc_device_t *dev, const char *hsaco_path,
                   const char *kernel_name, bc_kernel_t *out)
{
    sm100_dev_t *d = D_of(dev);
    if (!out) return BC_RT_ERR_SYMBOL;
    memset(out, 0, sizeof *out);
    if (!d) { fprintf(stderr, "bc_runtime: device not initialised\n"); return BC_RT_ERR_NO_GPU; }
    sm100_kern_t k;
    int rc = sm100_rt_load(d, hsaco_path, kernel_name, &k);
    if (rc == SM100_ERR_IO)
        fprintf(stderr, "bc_runtime: cannot open '%s'\n", hsaco_path);
    else if (rc == SM100_ERR_KERN)
        fprintf(stderr, "bc_runtime: kernel '%s' not found\n", kernel_name);
    if (rc != SM100_OK) return to_bc(rc);
    out->kernel_object = (uint64_t)(uintptr_t)k.func;
    out->kernarg_size = k.param_bytes;
    out->group_size = k.shared_bytes;
    out->private_size = k.local_bytes;
    out->_exec = (uint64_t)(uintptr_t)k.mod;
    out->_reader = 0;
    fprintf(stderr, "bc_runtime: loaded '%s' (kernarg=%u, lds=%u, scratch=%u)\n",
            kernel_name, out->kernarg_size, out->group_size, out->private_size);
    return BC_RT_OK;
}

void bc_unload_kernel(bc_device_t *dev, bc_kernel_t *kern)
{
    sm100_dev_t *d = D_of(dev);
    if (!kern) return;
    if (d && kern->_exec) {
        sm100_kern_t k;
        memset(&k, 0, sizeof k);
        k.mod = (void *)(uintptr_t)kern->_exec;
        sm100_rt_unload(d, &k);
    }
    memset(kern, 0, sizeof *kern);
}

void *bc_alloc(bc_device_t *dev, size_t size)
{
    sm100_dev_t *d = D_of(dev);
    if (!d) { fprintf(stderr, "bc_runtime: device not initialised\n"); return NULL; }
    sm100_ptr_t p = sm100_rt_alloc(d, size);
    if (!p) {
        fprintf(stderr, "bc_runtime: alloc %zu bytes failed\n", size);
        return NULL;
    }
    return (void *)(uintptr_t)p;
}

void bc_free(bc_device_t *dev, void *ptr)
{
    if (!ptr) return;
    sm100_dev_t *d = D_of(dev);
    if (!d) return;
    for (int i = 0; i < d->ntrak; i++)
        if (d->trak[i].ptr == (unsigned long long)(uintptr_t)ptr) {
            d->trak[i] = d->trak[d->ntrak - 1];
            d->ntrak--;
            break;
        }
    sm100_rt_free(d, (sm100_ptr_t)(uintptr_t)ptr);
}

void bc_trak(bc_device_t *dev, void *ptr, size_t size, const char *label, int flags)
{
    sm100_dev_t *d = D_of(dev);
    if (!d || !ptr || d->ntrak >= SM100_TRAK_MAX) return;
    int i = d->ntrak++;
    d->trak[i].ptr = (unsigned long long)(uintptr_t)ptr;
    d->trak[i].size = (unsigned long long)size;
    d->trak[i].flags = flags;
    snprintf(d->trak[i].label, sizeof d->trak[i].label, "%s", label ? label : "?");
}

int bc_copy_h2d(bc_device_t *dev, void *dst, const void *src, size_t size)
{
    sm100_dev_t *d = D_of(dev);
    if (!d) return BC_RT_ERR_NO_GPU;
    int rc = sm100_rt_h2d(d, (sm100_ptr_t)(uintptr_t)dst, src, size);
    if (rc != SM100_OK) fprintf(stderr, "bc_runtime: h2d copy failed\n");
    return to_bc(rc);
}

int bc_copy_d2h(bc_device_t *dev, void *dst, const void *src, size_t size)
{
    sm100_dev_t *d = D_of(dev);
    if (!d) return BC_RT_ERR_NO_GPU;
    int rc = sm100_rt_d2h(d, dst, (sm100_ptr_t)(uintptr_t)src, size);
    if (rc != SM100_OK) fprintf(stderr, "bc_runtime: d2h copy failed\n");
    return to_bc(rc);
}

int bc_dispatch(bc_device_t *dev, const bc_kernel_t *kern,
                uint32_t grid_x, uint32_t grid_y, uint32_t grid_z,
                uint32_t block_x, uint32_t block_y, uint32_t block_z,
                const void *args, uint32_t args_size)
{
    sm100_dev_t *d = D_of(dev);
    if (!d) return BC_RT_ERR_NO_GPU;
    if (!kern || !kern->kernel_object) {
        fprintf(stderr, "bc_runtime: dispatch without a loaded kernel\n");
        return BC_RT_ERR_SYMBOL;
    }
    /* Zero dimensions count as 1 (src/runtime/bc_runtime.c:636-641). */
    if (grid_x == 0)  grid_x = 1;
    if (grid_y == 0)  grid_y = 1;
    if (grid_z == 0)  grid_z = 1;
    if (block_x == 0) block_x = 1;
    if (block_y == 0) block_y = 1;
    if (block_z == 0) block_z = 1;

    sm100_kern_t k;
    memset(&k, 0, sizeof k);
    k.func = (void *)(uintptr_t)kern->kernel_object;
    k.param_bytes = kern->kernarg_size;
    sm100_func_name(d, k.func, k.name, sizeof k.name);      /* bc_kernel_t carries no name; ask the driver */
    int rc = sm100_rt_launch_packed(d, &k, grid_x, grid_y, grid_z, block_x, block_y, block_z,
                                    0, args, args_size);
    if (rc == SM100_OK) rc = sm100_rt_sync(d);
    if (rc != SM100_OK) fprintf(stderr, "bc_runtime: dispatch failed\n");
    return to_bc(rc);
}
