/* rt_sm100.c -- run-side descriptor "sm100" for Booth's src/exec contract.
 *
 * Implements every operation of rt_desc_t (src/exec/exec.h:69-93) on the driver
 * shim. The contract's handles are caller-held byte arrays (src/exec/exec.h:43-53):
 * the device handle stores a tag and the pointer to the shim's device, the
 * kernel handle stores the shim's kernel record. run receives {pointer, size}
 * pairs (src/exec/exec.h:29-32); the CUDA driver wants one pointer per
 * argument, so they pass straight through. */
#include <stdio.h>
#include <string.h>

#include "rt_sm100.h"
#include "sm100_internal.h"

typedef struct { unsigned long long tag; sm100_dev_t *d; } rt_sm100_dev;
#define RT_SM100_TAG 0x30303153545255ull

typedef char rt_dev_fits[(sizeof(rt_sm100_dev) <= RT_DEV_MAX) ? 1 : -1];
typedef char rt_kern_fits[(sizeof(sm100_kern_t) <= RT_KERN_MAX) ? 1 : -1];

static sm100_dev_t *D(void *dev)
{
    rt_sm100_dev h;
    if (!dev) return NULL;
    memcpy(&h, dev, sizeof h);
    return h.tag == RT_SM100_TAG ? h.d : NULL;
}

static int to_rt(int rc)
{
    switch (rc) {
    case SM100_OK:         return RT_OK;
    case SM100_ERR_DL:     return RT_ENODRV;
    case SM100_ERR_SYM:    return RT_ESYM;
    case SM100_ERR_NO_GPU: return RT_ENODEV;
    case SM100_ERR_IO:     return RT_EIO;
    case SM100_ERR_KERN:   return RT_EKERN;
    case SM100_ERR_ARG:    return RT_EINPUT;
    default:               return RT_EDRV;
    }
}

static int sm_open(void *dev)
{
    rt_sm100_dev h = { RT_SM100_TAG, NULL };
    int rc = sm100_rt_init(&h.d, -1);
    if (rc != SM100_OK) return to_rt(rc);
    memcpy(dev, &h, sizeof h);
    return RT_OK;
}

static void sm_shut(void *dev)
{
    sm100_dev_t *d = D(dev);
    if (d) sm100_rt_shut(d);
    if (dev) memset(dev, 0, sizeof(rt_sm100_dev));
}

static int sm_load(void *dev, const char *path, const char *kern, void *out)
{
    sm100_dev_t *d = D(dev);
    if (!d || !path || !kern || !out) return RT_EINPUT;
    sm100_kern_t k;
    int rc = sm100_rt_load(d, path, kern, &k);
    if (rc != SM100_OK) return to_rt(rc);
    memcpy(out, &k, sizeof k);
    return RT_OK;
}

static void sm_unload(void *dev, void *kern)
{
    sm100_dev_t *d = D(dev);
    if (!d || !kern) return;
    sm100_kern_t k;
    memcpy(&k, kern, sizeof k);
    sm100_rt_unload(d, &k);
    memset(kern, 0, sizeof k);
}

static rt_ptr sm_alloc(void *dev, size_t n)
{
    sm100_dev_t *d = D(dev);
    return d ? (rt_ptr)sm100_rt_alloc(d, n) : 0;
}

static void sm_dfre(void *dev, rt_ptr p)
{
    sm100_dev_t *d = D(dev);
    if (d && p) sm100_rt_free(d, (sm100_ptr_t)p);
}

static int sm_h2d(void *dev, rt_ptr dst, const void *src, size_t n)
{
    sm100_dev_t *d = D(dev);
    return d ? to_rt(sm100_rt_h2d(d, (sm100_ptr_t)dst, src, n)) : RT_EINPUT;
}

static int sm_d2h(void *dev, void *dst, rt_ptr src, size_t n)
{
    sm100_dev_t *d = D(dev);
    return d ? to_rt(sm100_rt_d2h(d, dst, (sm100_ptr_t)src, n)) : RT_EINPUT;
}

static int sm_run(void *dev, const void *kern, const rt_dim_t *dim, const rt_arg_t *args, uint32_t nargs)
{
    sm100_dev_t *d = D(dev);
    if (!d || !kern || !dim || (nargs && !args) || nargs > 64) return RT_EINPUT;
    sm100_kern_t k;
    memcpy(&k, kern, sizeof k);
    void *argv[64];
    uint32_t bytes = 0;
    for (uint32_t i = 0; i < nargs; i++) {
        if (!args[i].p || !args[i].size) return RT_EINPUT;
        argv[i] = (void *)(uintptr_t)args[i].p;
        /* the layout a packing target would build: each argument aligned to min(size, 8) */
        uint32_t al = args[i].size < 8u ? args[i].size : 8u;
        bytes = (bytes + al - 1) / al * al + args[i].size;
    }
    if (k.param_bytes && bytes > ((k.param_bytes + 7u) & ~7u)) {
        fprintf(stderr, "sm100_rt: kernel '%s' takes %u bytes of parameters, %u given\n", k.name, k.param_bytes, bytes);
        return RT_EINPUT;
    }
    uint32_t g[3], b[3];
    for (int i = 0; i < 3; i++) { g[i] = dim->grid[i] ? dim->grid[i] : 1; b[i] = dim->block[i] ? dim->block[i] : 1; }
    return to_rt(sm100_rt_launch(d, &k, g[0], g[1], g[2], b[0], b[1], b[2], dim->shmem, nargs ? argv : NULL));
}

static int sm_sync(void *dev)
{
    sm100_dev_t *d = D(dev);
    return d ? to_rt(sm100_rt_sync(d)) : RT_EINPUT;
}

/* Pinned host memory; with unified addressing the device sees it at the same address. */
static int sm_hmap(void *dev, void **hp, rt_ptr *dp, size_t n)
{
    sm100_dev_t *d = D(dev);
    if (!d || !hp || !dp) return RT_EINPUT;
    int rc = sm100_rt_hostalloc(d, hp, n);
    if (rc != SM100_OK) return to_rt(rc);
    *dp = (rt_ptr)(uintptr_t)*hp;
    return RT_OK;
}

static void sm_hfre(void *dev, void *hp)
{
    sm100_dev_t *d = D(dev);
    if (d && hp) sm100_rt_hostfree(d, hp);
}

static void sm_trak(void *dev, rt_ptr p, size_t n, const char *lbl, int fl)
{
    sm100_dev_t *d = D(dev);
    if (!d || !p || d->ntrak >= SM100_TRAK_MAX) return;
    int i = d->ntrak++;
    d->trak[i].ptr = (unsigned long long)p;
    d->trak[i].size = (unsigned long long)n;
    d->trak[i].flags = fl;
    snprintf(d->trak[i].label, sizeof d->trak[i].label, "%s", lbl ? lbl : "?");
}

static const char *sm_errs(int rc)
{
    switch (rc) {
    case RT_OK:      return "ok";
    case RT_ENODRV:  return "libcuda.so.1 could not be opened";
    case RT_ESYM:    return "the CUDA driver lacks an entry point this runtime needs";
    case RT_EDRV:    return "a CUDA driver call failed (see the sm100_rt: line on stderr)";
    case RT_ENODEV:  return "no sm_100 device";
    case RT_EIO:     return "the cubin could not be read";
    case RT_EKERN:   return "no kernel of that name in the cubin";
    case RT_EUNSUP:  return "not supported on sm100";
    case RT_EINPUT:  return "invalid argument";
    default:         return "unknown status";
    }
}

const rt_desc_t rt_sm100 = {
    "sm100", "cubin", (uint32_t)sizeof(rt_sm100_dev), (uint32_t)sizeof(sm100_kern_t),
    sm_open, sm_shut, sm_load, sm_unload, sm_alloc, sm_dfre, sm_h2d, sm_d2h, sm_run, sm_sync,
    sm_hmap, sm_hfre, sm_trak, sm_errs
};
