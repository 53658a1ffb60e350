/* nv_rt_sm100.c -- the reference's nv_rt_* launcher API (src/nvidia/nv_rt.h:102-134)
 * as a thin layer over sm100_rt_*: same signatures, same caller-owned records, same
 * status codes, one "nv_rt:" line on stderr per failure. The device object of the
 * runtime is kept in nv_dev_t.lib, which callers only test for NULL. */
#include "nv_rt.h"
#include "sm100_internal.h"

#include <stdio.h>
#include <string.h>

/* The layout the reference's callers were compiled against. */
typedef char nv_dev_size_check[sizeof(nv_dev_t) == 320 ? 1 : -1];
typedef char nv_kern_size_check[sizeof(nv_kern_t) == 144 ? 1 : -1];

static sm100_dev_t *nv_dev(const nv_dev_t *D)
{
    return D != NULL ? (sm100_dev_t *)D->lib : NULL;
}

/* sm100 status codes -1..-6 are the reference's; the two extra ones fold into
 * "a driver call failed". */
static int nv_rc(int rc)
{
    return (rc <= 0 && rc >= NV_RT_ERR_KERN) ? rc : NV_RT_ERR_CUDA;
}

static int nv_closed(const char *what)
{
    fprintf(stderr, "nv_rt: %s on a device that is not open\n", what);
    return NV_RT_ERR_CUDA;
}

static void nv_as_kern(const nv_kern_t *kern, sm100_kern_t *k)
{
    memset(k, 0, sizeof *k);
    k->mod = kern->mod;
    k->func = kern->func;
    memcpy(k->name, kern->name, sizeof k->name);
    k->name[sizeof k->name - 1] = 0;
}

int nv_rt_init(nv_dev_t *D)
{
    sm100_dev_t *dev = NULL;
    int rc;

    if (D == NULL) return NV_RT_ERR_CUDA;
    memset(D, 0, sizeof *D);
    rc = sm100_rt_init(&dev, -1);
    if (rc != SM100_OK) {
        fprintf(stderr, "nv_rt: device init failed (%d)\n", rc);
        return nv_rc(rc);
    }
    D->lib = dev;
    D->ctx = (void *)dev->ctx;
    D->dev = dev->ordinal;
    snprintf(D->dev_name, sizeof D->dev_name, "%s", dev->name);
    D->sm_major = dev->sm_major;
    D->sm_minor = dev->sm_minor;
    fprintf(stderr, "nv_rt: %s (sm_%d%d)\n", D->dev_name, D->sm_major, D->sm_minor);
    return NV_RT_OK;
}

void nv_rt_shut(nv_dev_t *D)
{
    if (D == NULL || D->lib == NULL) return;
    sm100_rt_shut(nv_dev(D));
    memset(D, 0, sizeof *D);
}

int nv_rt_load(nv_dev_t *D, const char *ptx_path, const char *kern_name, nv_kern_t *out)
{
    sm100_kern_t k;
    int rc;

    if (out == NULL) return NV_RT_ERR_CUDA;
    memset(out, 0, sizeof *out);
    if (nv_dev(D) == NULL) return nv_closed("nv_rt_load");
    rc = sm100_rt_load(nv_dev(D), ptx_path, kern_name, &k);
    if (rc != SM100_OK) {
        fprintf(stderr, "nv_rt: could not load kernel '%s' from %s (%d)\n",
                kern_name ? kern_name : "(null)", ptx_path ? ptx_path : "(null)", rc);
        return nv_rc(rc);
    }
    out->mod = k.mod;
    out->func = k.func;
    memcpy(out->name, k.name, sizeof out->name);
    fprintf(stderr, "nv_rt: loaded kernel '%s' from %s\n", kern_name, ptx_path);
    return NV_RT_OK;
}

void nv_rt_unload(nv_dev_t *D, nv_kern_t *kern)
{
    sm100_kern_t k;

    if (nv_dev(D) == NULL || kern == NULL || kern->mod == NULL) return;
    nv_as_kern(kern, &k);
    sm100_rt_unload(nv_dev(D), &k);
    memset(kern, 0, sizeof *kern);
}

CUdevptr nv_rt_alloc(nv_dev_t *D, size_t size)
{
    CUdevptr p;

    if (nv_dev(D) == NULL) { nv_closed("nv_rt_alloc"); return 0; }
    p = sm100_rt_alloc(nv_dev(D), size);
    if (p == 0) fprintf(stderr, "nv_rt: allocation of %llu bytes failed\n", (unsigned long long)size);
    return p;
}

void nv_rt_free(nv_dev_t *D, CUdevptr ptr)
{
    if (ptr != 0 && nv_dev(D) != NULL) sm100_rt_free(nv_dev(D), ptr);
}

int nv_rt_h2d(nv_dev_t *D, CUdevptr dst, const void *src, size_t size)
{
    int rc;

    if (nv_dev(D) == NULL) return nv_closed("nv_rt_h2d");
    rc = sm100_rt_h2d(nv_dev(D), dst, src, size);
    if (rc != SM100_OK) fprintf(stderr, "nv_rt: H2D copy failed (%d)\n", rc);
    return nv_rc(rc);
}

int nv_rt_d2h(nv_dev_t *D, void *dst, CUdevptr src, size_t size)
{
    int rc;

    if (nv_dev(D) == NULL) return nv_closed("nv_rt_d2h");
    rc = sm100_rt_d2h(nv_dev(D), dst, src, size);
    if (rc != SM100_OK) fprintf(stderr, "nv_rt: D2H copy failed (%d)\n", rc);
    return nv_rc(rc);
}

int nv_rt_launch(nv_dev_t *D, nv_kern_t *kern, uint32_t gx, uint32_t gy, uint32_t gz,
                 uint32_t bx, uint32_t by, uint32_t bz, uint32_t shmem, void **args)
{
    sm100_kern_t k;
    int rc;

    if (nv_dev(D) == NULL) return nv_closed("nv_rt_launch");
    if (kern == NULL || kern->func == NULL) {
        fprintf(stderr, "nv_rt: launch of a kernel that is not loaded\n");
        return NV_RT_ERR_CUDA;
    }
    nv_as_kern(kern, &k);
    rc = sm100_rt_launch(nv_dev(D), &k, gx, gy, gz, bx, by, bz, shmem, args);
    if (rc != SM100_OK) fprintf(stderr, "nv_rt: launch of '%s' failed (%d)\n", k.name, rc);
    return nv_rc(rc);
}

int nv_rt_sync(nv_dev_t *D)
{
    int rc;

    if (nv_dev(D) == NULL) return nv_closed("nv_rt_sync");
    rc = sm100_rt_sync(nv_dev(D));
    if (rc != SM100_OK) fprintf(stderr, "nv_rt: sync failed (%d)\n", rc);
    return nv_rc(rc);
}

int nv_rt_mmap(nv_dev_t *D, void **hpp, CUdevptr *dpp, size_t sz)
{
    int rc;

    if (hpp == NULL || dpp == NULL) return NV_RT_ERR_CUDA;
    *hpp = NULL;
    *dpp = 0;
    if (nv_dev(D) == NULL) return nv_closed("nv_rt_mmap");
    rc = sm100_rt_hostmap(nv_dev(D), hpp, dpp, sz);
    if (rc != SM100_OK) fprintf(stderr, "nv_rt: mapped host allocation of %llu bytes failed (%d)\n",
                                (unsigned long long)sz, rc);
    return nv_rc(rc);
}

void nv_rt_mfre(nv_dev_t *D, void *hp)
{
    if (hp != NULL && nv_dev(D) != NULL) sm100_rt_hostfree(nv_dev(D), hp);
}
