/* sm100_shim.c -- thin C99 shim over the CUDA driver API for B200 (sm_100a).
 *
 * The sm_100a counterpart of the reference's NVIDIA launcher
 * (src/nvidia/nv_rt.c:69-381): the driver library is opened at run time, so the
 * library itself links against nothing but libc/libdl and loads on a machine
 * without a GPU. Where the reference creates its own context
 * (src/nvidia/nv_rt.c:146) and JIT-compiles PTX (src/nvidia/nv_rt.c:172-248), this
 * shim retains the device's primary context, which is the one NCCL and the
 * CUDA runtime use, and loads machine code built by nvcc for sm_100a. Work goes
 * to one non-blocking stream per device rather than the NULL stream
 * (src/nvidia/nv_rt.c:304-327). */
#define _POSIX_C_SOURCE 200809L
#include <dlfcn.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "sm100_internal.h"

/* ---- driver table ---- */

static sm100_api_t g_api;
static int g_api_rc = 1;                 /* 1 = not tried yet */
static pthread_mutex_t g_api_mu = PTHREAD_MUTEX_INITIALIZER;

static int api_sym(void *lib, const char *name, void **out, int optional)
{
    *out = dlsym(lib, name);
    if (!*out && !optional) {
        fprintf(stderr, "sm100_rt: driver entry point '%s' not found\n", name);
        return SM100_ERR_SYM;
    }
    return SM100_OK;
}

static int api_load(void)
{
    const char *path = getenv("BOOTH_CUDA_LIB");
    if (!path || !*path) path = "libcuda.so.1";
    void *lib = dlopen(path, RTLD_NOW | RTLD_LOCAL);
    if (!lib) {
        fprintf(stderr, "sm100_rt: cannot open the CUDA driver '%s': %s\n", path, dlerror());
        return SM100_ERR_DL;
    }
    sm100_api_t *a = &g_api;
    a->lib = lib;
    int rc = SM100_OK;
#define SYM(field, name) if (rc == SM100_OK) rc = api_sym(lib, name, (void **)&a->field, 0)
#define OPT(field, name) api_sym(lib, name, (void **)&a->field, 1)
    SYM(Init, "cuInit");
    SYM(DeviceGetCount, "cuDeviceGetCount");
    SYM(DeviceGet, "cuDeviceGet");
    SYM(DeviceGetName, "cuDeviceGetName");
    SYM(DeviceGetAttribute, "cuDeviceGetAttribute");
    SYM(PrimaryCtxRetain, "cuDevicePrimaryCtxRetain");
    SYM(PrimaryCtxRelease, "cuDevicePrimaryCtxRelease_v2");
    SYM(CtxSetCurrent, "cuCtxSetCurrent");
    SYM(CtxGetCurrent, "cuCtxGetCurrent");
    SYM(ModuleLoadData, "cuModuleLoadData");
    SYM(ModuleLoadDataEx, "cuModuleLoadDataEx");
    SYM(ModuleUnload, "cuModuleUnload");
    SYM(ModuleGetFunction, "cuModuleGetFunction");
    SYM(FuncGetAttribute, "cuFuncGetAttribute");
    SYM(FuncSetAttribute, "cuFuncSetAttribute");
    OPT(FuncGetParamInfo, "cuFuncGetParamInfo");
    OPT(ModuleGetFunctionCount, "cuModuleGetFunctionCount");
    OPT(ModuleEnumerateFunctions, "cuModuleEnumerateFunctions");
    OPT(FuncGetName, "cuFuncGetName");
    SYM(MemAlloc, "cuMemAlloc_v2");
    SYM(MemFree, "cuMemFree_v2");
    SYM(MemcpyHtoD, "cuMemcpyHtoD_v2");
    SYM(MemcpyDtoH, "cuMemcpyDtoH_v2");
    SYM(MemcpyHtoDAsync, "cuMemcpyHtoDAsync_v2");
    SYM(MemcpyDtoHAsync, "cuMemcpyDtoHAsync_v2");
    SYM(MemsetD8Async, "cuMemsetD8Async");
    SYM(MemHostAlloc, "cuMemHostAlloc");
    SYM(MemFreeHost, "cuMemFreeHost");
    SYM(MemHostGetDevicePointer, "cuMemHostGetDevicePointer_v2");
    SYM(StreamCreate, "cuStreamCreate");
    SYM(StreamDestroy, "cuStreamDestroy_v2");
    SYM(StreamSynchronize, "cuStreamSynchronize");
    SYM(StreamWaitEvent, "cuStreamWaitEvent");
    SYM(EventCreate, "cuEventCreate");
    SYM(EventDestroy, "cuEventDestroy_v2");
    SYM(EventRecord, "cuEventRecord");
    SYM(EventSynchronize, "cuEventSynchronize");
    SYM(EventElapsedTime, "cuEventElapsedTime");
    SYM(LaunchKernel, "cuLaunchKernel");
    OPT(LaunchKernelEx, "cuLaunchKernelEx");
    OPT(OccupancyMaxActiveClusters, "cuOccupancyMaxActiveClusters");
    SYM(GetErrorString, "cuGetErrorString");
    SYM(TensorMapEncodeTiled, "cuTensorMapEncodeTiled");
#undef SYM
#undef OPT
    if (rc != SM100_OK) { dlclose(lib); a->lib = NULL; return rc; }
    CUresult cr = a->Init(0);
    if (cr != CUDA_SUCCESS) {
        const char *s = NULL;
        a->GetErrorString(cr, &s);
        fprintf(stderr, "sm100_rt: cuInit failed: %s\n", s ? s : "unknown error");
        return cr == CUDA_ERROR_NO_DEVICE ? SM100_ERR_NO_GPU : SM100_ERR_CUDA;
    }
    return SM100_OK;
}

static int api_get(const sm100_api_t **out)
{
    pthread_mutex_lock(&g_api_mu);
    if (g_api_rc == 1) g_api_rc = api_load();
    int rc = g_api_rc;
    pthread_mutex_unlock(&g_api_mu);
    *out = &g_api;
    return rc;
}

/* ---- errors ---- */

int sm100_fail(sm100_dev_t *dev, const char *what, CUresult rc)
{
    const char *s = NULL;
    if (g_api.GetErrorString) g_api.GetErrorString(rc, &s);
    if (!s) s = "unknown error";
    if (dev) snprintf(dev->err, sizeof dev->err, "%s: %s", what, s);
    fprintf(stderr, "sm100_rt: %s: %s\n", what, s);
    return SM100_ERR_CUDA;
}

static int fail_arg(sm100_dev_t *dev, const char *what)
{
    if (dev) snprintf(dev->err, sizeof dev->err, "%s", what);
    fprintf(stderr, "sm100_rt: %s\n", what);
    return SM100_ERR_ARG;
}

int sm100_enter(sm100_dev_t *dev)
{
    if (!dev) return fail_arg(NULL, "NULL device");
    CUresult rc = dev->api->CtxSetCurrent(dev->ctx);
    if (rc != CUDA_SUCCESS) return sm100_fail(dev, "cuCtxSetCurrent", rc);
    return SM100_OK;
}

/* ---- init / shut ---- */

static const char *const k_names[SM100_K_COUNT] = {
    "vadd_stream", "saxpy_stream", "fill_philox",
    "reduce_sum_i32", "reduce_sum_f32",
    "asian_mc", "asian_mc_precise",
    "asian_paths", "asian_paths_precise",
    "gemm_prepass", "gemm_tf32x3", "gemm_tf32x3_n128", "gemm_tf32x3_2cta", "gemm_tf32x3_2cta_n128", "gemm_tf32x3_persist",
};

int sm100_rt_device_count(void)
{
    const sm100_api_t *a;
    int rc = api_get(&a);
    if (rc != SM100_OK) return rc;
    int n = 0;
    CUresult cr = a->DeviceGetCount(&n);
    if (cr != CUDA_SUCCESS) return sm100_fail(NULL, "cuDeviceGetCount", cr);
    return n;
}

int sm100_rt_init(sm100_dev_t **out, int ordinal)
{
    if (!out) return fail_arg(NULL, "sm100_rt_init: NULL out");
    *out = NULL;
    const sm100_api_t *a;
    int rc = api_get(&a);
    if (rc != SM100_OK) return rc;

    if (ordinal < 0) {
        const char *e = getenv("BOOTH_DEVICE");
        ordinal = (e && *e) ? atoi(e) : 0;
    }
    int count = 0;
    CUresult cr = a->DeviceGetCount(&count);
    if (cr != CUDA_SUCCESS) return sm100_fail(NULL, "cuDeviceGetCount", cr);
    if (count <= 0 || ordinal >= count) {
        fprintf(stderr, "sm100_rt: no GPU with ordinal %d (%d present)\n", ordinal, count);
        return SM100_ERR_NO_GPU;
    }

    sm100_dev_t *d = (sm100_dev_t *)calloc(1, sizeof *d);
    if (!d) return fail_arg(NULL, "out of host memory");
    d->api = a;
    d->ordinal = ordinal;
    if ((cr = a->DeviceGet(&d->cudev, ordinal)) != CUDA_SUCCESS) {
        rc = sm100_fail(NULL, "cuDeviceGet", cr); free(d); return rc;
    }
    a->DeviceGetName(d->name, (int)sizeof d->name, d->cudev);
    a->DeviceGetAttribute(&d->sm_major, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR, d->cudev);
    a->DeviceGetAttribute(&d->sm_minor, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR, d->cudev);
    a->DeviceGetAttribute(&d->sm_count, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT, d->cudev);
    if (d->sm_major != 10) {
        fprintf(stderr, "sm100_rt: device %d (%s) is sm_%d%d; this library carries "
                "sm_100a code only\n", ordinal, d->name, d->sm_major, d->sm_minor);
        free(d);
        return SM100_ERR_NO_GPU;
    }
    if ((cr = a->PrimaryCtxRetain(&d->ctx, d->cudev)) != CUDA_SUCCESS) {
        rc = sm100_fail(NULL, "cuDevicePrimaryCtxRetain", cr); free(d); return rc;
    }
    if ((cr = a->CtxSetCurrent(d->ctx)) != CUDA_SUCCESS) {
        rc = sm100_fail(NULL, "cuCtxSetCurrent", cr); goto drop_ctx;
    }
    if ((cr = a->StreamCreate(&d->stream, CU_STREAM_NON_BLOCKING)) != CUDA_SUCCESS) {
        rc = sm100_fail(NULL, "cuStreamCreate", cr); goto drop_ctx;
    }
    if ((cr = a->EventCreate(&d->ev0, CU_EVENT_DEFAULT)) != CUDA_SUCCESS ||
        (cr = a->EventCreate(&d->ev1, CU_EVENT_DEFAULT)) != CUDA_SUCCESS) {
        rc = sm100_fail(NULL, "cuEventCreate", cr); goto drop_stream;
    }
    if ((cr = a->ModuleLoadData(&d->image, booth_sm100_image)) != CUDA_SUCCESS) {
        rc = sm100_fail(NULL, "cuModuleLoadData(built-in sm_100a image)", cr); goto drop_stream;
    }
    for (int i = 0; i < SM100_K_COUNT; i++) {
        cr = a->ModuleGetFunction(&d->k[i], d->image, k_names[i]);
        if (cr != CUDA_SUCCESS) {
            fprintf(stderr, "sm100_rt: built-in kernel '%s' missing from the image\n", k_names[i]);
            rc = SM100_ERR_KERN; goto drop_image;
        }
    }
    /* 1 MiB of device scratch: block partials and arrival counters. The
     * counters must start at zero; the kernels put them back to zero. */
    d->scratch_bytes = 1u << 20;
    if ((cr = a->MemAlloc(&d->scratch, d->scratch_bytes)) != CUDA_SUCCESS) {
        rc = sm100_fail(NULL, "cuMemAlloc(scratch)", cr); goto drop_image;
    }
    if ((cr = a->MemsetD8Async(d->scratch, 0, d->scratch_bytes, d->stream)) != CUDA_SUCCESS ||
        (cr = a->StreamSynchronize(d->stream)) != CUDA_SUCCESS) {
        rc = sm100_fail(NULL, "clearing scratch", cr); a->MemFree(d->scratch); goto drop_image;
    }
    {   /* limit of the GEMM kernel's barrier waits: BOOTH_SM100_GEMM_WAIT_MS at start-up, else 4 s */
        const char *e = getenv("BOOTH_SM100_GEMM_WAIT_MS");
        int ms = (e && *e) ? atoi(e) : 4000;
        d->gemm_wait_ms = (unsigned)(ms < 1 ? 1 : ms > 60000 ? 60000 : ms);
    }
    fprintf(stderr, "sm100_rt: device %d: %s (sm_%d%d, %d SMs)\n", ordinal, d->name,
            d->sm_major, d->sm_minor, d->sm_count);
    *out = d;
    return SM100_OK;

drop_image:
    a->ModuleUnload(d->image);
drop_stream:
    if (d->ev0) a->EventDestroy(d->ev0);
    if (d->ev1) a->EventDestroy(d->ev1);
    a->StreamDestroy(d->stream);
drop_ctx:
    a->PrimaryCtxRelease(d->cudev);
    free(d);
    return rc;
}

void sm100_rt_shut(sm100_dev_t *dev)
{
    if (!dev) return;
    const sm100_api_t *a = dev->api;
    if (a->CtxSetCurrent(dev->ctx) == CUDA_SUCCESS) {
        a->StreamSynchronize(dev->stream);
        if (dev->stage_ready) {
            a->StreamSynchronize(dev->stream_out);
            a->StreamSynchronize(dev->stream_in);
            for (int i = 0; i < SM100_STAGE_SLOTS; i++) {
                a->EventDestroy(dev->ev_uploaded[i]); a->EventDestroy(dev->ev_computed[i]); a->EventDestroy(dev->ev_drained[i]);
            }
            a->StreamDestroy(dev->stream_out);
            a->StreamDestroy(dev->stream_in);
            a->MemFree(dev->stage);
        }
        if (dev->gemm_ws) a->MemFree(dev->gemm_ws);
        if (dev->scratch) a->MemFree(dev->scratch);
        a->ModuleUnload(dev->image);
        a->EventDestroy(dev->ev0);
        a->EventDestroy(dev->ev1);
        a->StreamDestroy(dev->stream);
    }
    a->PrimaryCtxRelease(dev->cudev);
    free(dev->gemm_maps);
    free(dev);
}

const char *sm100_rt_name(const sm100_dev_t *dev) { return dev ? dev->name : ""; }
int sm100_rt_sm_count(const sm100_dev_t *dev) { return dev ? dev->sm_count : 0; }
int sm100_rt_ordinal(const sm100_dev_t *dev) { return dev ? dev->ordinal : -1; }
const char *sm100_rt_errs(const sm100_dev_t *dev) { return dev ? dev->err : ""; }
unsigned long long sm100_rt_launches(const sm100_dev_t *dev) { return dev ? dev->launches : 0; }
void *sm100_rt_stream(const sm100_dev_t *dev) { return dev ? (void *)dev->stream : NULL; }

/* ---- kernels ---- */

static void kern_describe(sm100_dev_t *dev, sm100_kern_t *k)
{
    const sm100_api_t *a = dev->api;
    int v = 0;
    if (a->FuncGetAttribute(&v, CU_FUNC_ATTRIBUTE_SHARED_SIZE_BYTES, (CUfunction)k->func) == CUDA_SUCCESS)
        k->shared_bytes = (uint32_t)v;
    if (a->FuncGetAttribute(&v, CU_FUNC_ATTRIBUTE_LOCAL_SIZE_BYTES, (CUfunction)k->func) == CUDA_SUCCESS)
        k->local_bytes = (uint32_t)v;
    /* Size of the parameter block = end of the last parameter. */
    k->param_bytes = 0;
    if (a->FuncGetParamInfo) {
        for (size_t i = 0; i < 64; i++) {
            size_t off = 0, sz = 0;
            if (a->FuncGetParamInfo((CUfunction)k->func, i, &off, &sz) != CUDA_SUCCESS) break;
            if (off + sz > k->param_bytes) k->param_bytes = (uint32_t)(off + sz);
        }
    }
}

/* The launcher looks kernels up by their bare source name (src/runtime/bc_runtime.h:44-46).
 * A cubin built by nvcc from a C++ source that does not say extern "C" carries
 * the Itanium-mangled name instead (_Z<length><name><parameters>): when the bare
 * name is absent, take the one kernel of the module whose mangled name starts
 * with that prefix. */
static int find_mangled(sm100_dev_t *dev, CUmodule mod, const char *name, CUfunction *out)
{
    const sm100_api_t *a = dev->api;
    if (!a->ModuleGetFunctionCount || !a->ModuleEnumerateFunctions || !a->FuncGetName) return 0;
    unsigned int count = 0;
    if (a->ModuleGetFunctionCount(&count, mod) != CUDA_SUCCESS || count == 0 || count > 4096) return 0;
    CUfunction *fs = (CUfunction *)malloc(count * sizeof *fs);
    if (!fs) return 0;
    char prefix[160];
    int plen = snprintf(prefix, sizeof prefix, "_Z%zu%s", strlen(name), name);
    int found = 0;
    if (plen > 0 && plen < (int)sizeof prefix &&
        a->ModuleEnumerateFunctions(fs, count, mod) == CUDA_SUCCESS) {
        for (unsigned int i = 0; i < count; i++) {
            const char *fn = NULL;
            if (a->FuncGetName(&fn, fs[i]) != CUDA_SUCCESS || !fn) continue;
            if (strncmp(fn, prefix, (size_t)plen) == 0) { *out = fs[i]; found++; }
        }
    }
    free(fs);
    return found == 1;
}

static int kern_from_module(sm100_dev_t *dev, CUmodule mod, int owns, const char *name,
                            sm100_kern_t *out)
{
    CUfunction f;
    CUresult cr = dev->api->ModuleGetFunction(&f, mod, name);
    if (cr != CUDA_SUCCESS && find_mangled(dev, mod, name, &f)) cr = CUDA_SUCCESS;
    if (cr != CUDA_SUCCESS) {
        snprintf(dev->err, sizeof dev->err, "kernel '%s' not found", name);
        fprintf(stderr, "sm100_rt: kernel '%s' not found in the image\n", name);
        if (owns) dev->api->ModuleUnload(mod);
        return SM100_ERR_KERN;
    }
    out->mod = owns ? (void *)mod : NULL;
    out->func = (void *)f;
    snprintf(out->name, sizeof out->name, "%s", name);
    kern_describe(dev, out);
    return SM100_OK;
}

int sm100_rt_load(sm100_dev_t *dev, const char *path, const char *name, sm100_kern_t *out)
{
    if (!dev || !path || !name || !out) return fail_arg(dev, "sm100_rt_load: NULL argument");
    memset(out, 0, sizeof *out);
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    FILE *fp = fopen(path, "rb");
    if (!fp) {
        snprintf(dev->err, sizeof dev->err, "cannot open '%s'", path);
        fprintf(stderr, "sm100_rt: cannot open '%s'\n", path);
        return SM100_ERR_IO;
    }
    fseek(fp, 0, SEEK_END);
    long sz = ftell(fp);
    fseek(fp, 0, SEEK_SET);
    if (sz <= 0) { fclose(fp); fprintf(stderr, "sm100_rt: '%s' is empty\n", path); return SM100_ERR_IO; }
    unsigned char *buf = (unsigned char *)malloc((size_t)sz + 1);
    if (!buf) { fclose(fp); return fail_arg(dev, "out of host memory"); }
    size_t got = fread(buf, 1, (size_t)sz, fp);
    fclose(fp);
    if (got != (size_t)sz) { free(buf); fprintf(stderr, "sm100_rt: short read on '%s'\n", path); return SM100_ERR_IO; }
    buf[sz] = 0;
    /* The file may be a cubin, a fatbin or PTX text (the reference's launcher loads
     * PTX, src/nvidia/nv_rt.c:172-248); for PTX the driver compiles it here, so ask
     * for its error log and print it when the load fails. */
    CUmodule mod;
    char jit_log[4096];
    jit_log[0] = 0;
    CUjit_option opts[2] = { CU_JIT_ERROR_LOG_BUFFER, CU_JIT_ERROR_LOG_BUFFER_SIZE_BYTES };
    void *vals[2] = { jit_log, (void *)(size_t)sizeof jit_log };
    CUresult cr = dev->api->ModuleLoadDataEx(&mod, buf, 2, opts, vals);
    free(buf);
    if (cr != CUDA_SUCCESS) {
        char what[600];
        snprintf(what, sizeof what, "loading '%s'", path);
        jit_log[sizeof jit_log - 1] = 0;
        if (jit_log[0]) fprintf(stderr, "sm100_rt: compiler log for '%s':\n%s\n", path, jit_log);
        return sm100_fail(dev, what, cr);
    }
    return kern_from_module(dev, mod, 1, name, out);
}

void sm100_func_name(sm100_dev_t *dev, void *func, char *out, size_t n)
{
    const char *name = NULL;
    if (dev && func && dev->api->FuncGetName && dev->api->FuncGetName(&name, (CUfunction)func) == CUDA_SUCCESS && name && *name)
        snprintf(out, n, "%s", name);
    else
        snprintf(out, n, "kernel");
}

int sm100_rt_load_builtin(sm100_dev_t *dev, const char *name, sm100_kern_t *out)
{
    if (!dev || !name || !out) return fail_arg(dev, "sm100_rt_load_builtin: NULL argument");
    memset(out, 0, sizeof *out);
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    return kern_from_module(dev, dev->image, 0, name, out);
}

void sm100_rt_unload(sm100_dev_t *dev, sm100_kern_t *kern)
{
    if (!dev || !kern) return;
    if (kern->mod && sm100_enter(dev) == SM100_OK)
        dev->api->ModuleUnload((CUmodule)kern->mod);
    memset(kern, 0, sizeof *kern);
}

/* ---- outcome of an enqueued GEMM ---- */

/* The GEMM kernel bounds its barrier waits and reports an expired one in a status
 * word instead of hanging. Every entry point that has just waited for the stream
 * (sync, the synchronous copies, toc, free) calls this, so a caller that goes from
 * booth_sm100_gemm straight to a copy back learns of it too. The stream must be
 * idle when this is called. */
int sm100_gemm_outcome(sm100_dev_t *dev)
{
    if (!dev->gemm_pending) return SM100_OK;
    int st = 0;
    dev->gemm_pending = 0;
    CUresult cr = dev->api->MemcpyDtoH(&st, dev->scratch + SM100_SCRATCH_GEMM_STATUS, sizeof st);
    if (cr != CUDA_SUCCESS) return sm100_fail(dev, "reading GEMM status", cr);
    if (st != 0) {
        snprintf(dev->err, sizeof dev->err, "gemm_tf32x3 gave up waiting on a barrier (code %d: "
                 "1 = producer, 2 = MMA issuer on operands, 3 = epilogue, 4 = MMA issuer on a free accumulator)", st);
        fprintf(stderr, "sm100_rt: %s\n", dev->err);
        return SM100_ERR_CUDA;
    }
    return SM100_OK;
}

/* ---- memory ---- */

sm100_ptr_t sm100_rt_alloc(sm100_dev_t *dev, size_t size)
{
    if (sm100_enter(dev) != SM100_OK) return 0;
    CUdeviceptr p = 0;
    CUresult cr = dev->api->MemAlloc(&p, size ? size : 1);
    if (cr != CUDA_SUCCESS) {
        char what[64];
        snprintf(what, sizeof what, "alloc %zu bytes", size);
        sm100_fail(dev, what, cr);
        return 0;
    }
    return (sm100_ptr_t)p;
}

void sm100_rt_free(sm100_dev_t *dev, sm100_ptr_t ptr)
{
    if (!ptr || sm100_enter(dev) != SM100_OK) return;
    /* cuMemFree itself waits for the work that may still use the block. Only a
     * GEMM whose outcome nobody has asked for yet needs a wait of our own: its
     * status is read (and a failure printed) before the memory goes away. */
    if (dev->gemm_pending && dev->api->StreamSynchronize(dev->stream) == CUDA_SUCCESS)
        (void)sm100_gemm_outcome(dev);
    dev->api->MemFree((CUdeviceptr)ptr);
}

int sm100_rt_h2d(sm100_dev_t *dev, sm100_ptr_t dst, const void *src, size_t size)
{
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    if (size == 0) return SM100_OK;
    /* Ordered on the device's own stream and complete on return. A plain
     * cuMemcpyHtoD from pageable memory may return while the DMA is still in
     * flight on the NULL stream, which this non-blocking stream does not wait
     * for: a kernel launched right after could read stale data. */
    CUresult cr = dev->api->MemcpyHtoDAsync((CUdeviceptr)dst, src, size, dev->stream);
    if (cr == CUDA_SUCCESS) cr = dev->api->StreamSynchronize(dev->stream);
    if (cr != CUDA_SUCCESS) return sm100_fail(dev, "h2d copy", cr);
    return sm100_gemm_outcome(dev);
}

int sm100_rt_d2h(sm100_dev_t *dev, void *dst, sm100_ptr_t src, size_t size)
{
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    if (size == 0) return SM100_OK;
    CUresult cr = dev->api->MemcpyDtoHAsync(dst, (CUdeviceptr)src, size, dev->stream);
    if (cr == CUDA_SUCCESS) cr = dev->api->StreamSynchronize(dev->stream);
    if (cr != CUDA_SUCCESS) return sm100_fail(dev, "d2h copy", cr);
    return sm100_gemm_outcome(dev);
}

int sm100_rt_h2d_async(sm100_dev_t *dev, sm100_ptr_t dst, const void *src, size_t size)
{
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    if (size == 0) return SM100_OK;
    CUresult cr = dev->api->MemcpyHtoDAsync((CUdeviceptr)dst, src, size, dev->stream);
    return cr == CUDA_SUCCESS ? SM100_OK : sm100_fail(dev, "h2d async copy", cr);
}

int sm100_rt_d2h_async(sm100_dev_t *dev, void *dst, sm100_ptr_t src, size_t size)
{
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    if (size == 0) return SM100_OK;
    CUresult cr = dev->api->MemcpyDtoHAsync(dst, (CUdeviceptr)src, size, dev->stream);
    return cr == CUDA_SUCCESS ? SM100_OK : sm100_fail(dev, "d2h async copy", cr);
}

int sm100_rt_zero(sm100_dev_t *dev, sm100_ptr_t dst, size_t size)
{
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    if (size == 0) return SM100_OK;
    CUresult cr = dev->api->MemsetD8Async((CUdeviceptr)dst, 0, size, dev->stream);
    return cr == CUDA_SUCCESS ? SM100_OK : sm100_fail(dev, "memset", cr);
}

int sm100_rt_hostalloc(sm100_dev_t *dev, void **hp, size_t size)
{
    if (!hp) return fail_arg(dev, "sm100_rt_hostalloc: NULL out");
    *hp = NULL;
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    CUresult cr = dev->api->MemHostAlloc(hp, size ? size : 1, CU_MEMHOSTALLOC_PORTABLE);
    return cr == CUDA_SUCCESS ? SM100_OK : sm100_fail(dev, "pinned host alloc", cr);
}

int sm100_rt_hostmap(sm100_dev_t *dev, void **hp, sm100_ptr_t *dp, size_t size)
{
    if (!hp || !dp) return fail_arg(dev, "sm100_rt_hostmap: NULL out");
    *hp = NULL;
    *dp = 0;
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    CUresult cr = dev->api->MemHostAlloc(hp, size ? size : 1, CU_MEMHOSTALLOC_PORTABLE | CU_MEMHOSTALLOC_DEVICEMAP);
    if (cr != CUDA_SUCCESS) return sm100_fail(dev, "mapped host alloc", cr);
    CUdeviceptr d = 0;
    cr = dev->api->MemHostGetDevicePointer(&d, *hp, 0);
    if (cr != CUDA_SUCCESS) {
        dev->api->MemFreeHost(*hp);
        *hp = NULL;
        return sm100_fail(dev, "device address of mapped host memory", cr);
    }
    *dp = (sm100_ptr_t)d;
    return SM100_OK;
}

void sm100_rt_hostfree(sm100_dev_t *dev, void *hp)
{
    if (!hp || sm100_enter(dev) != SM100_OK) return;
    dev->api->MemFreeHost(hp);
}

CUdeviceptr sm100_scratch(sm100_dev_t *dev, size_t bytes)
{
    if (bytes <= dev->scratch_bytes) return dev->scratch;
    snprintf(dev->err, sizeof dev->err, "scratch request %zu exceeds %zu", bytes, dev->scratch_bytes);
    fprintf(stderr, "sm100_rt: %s\n", dev->err);
    return 0;
}

CUdeviceptr sm100_gemm_ws(sm100_dev_t *dev, size_t bytes)
{
    if (bytes <= dev->gemm_ws_bytes) return dev->gemm_ws;
    const sm100_api_t *a = dev->api;
    a->StreamSynchronize(dev->stream);
    dev->gemm_b.valid = 0;
    if (dev->gemm_ws) { a->MemFree(dev->gemm_ws); dev->gemm_ws = 0; dev->gemm_ws_bytes = 0; }
    CUresult cr = a->MemAlloc(&dev->gemm_ws, bytes);
    if (cr != CUDA_SUCCESS) { sm100_fail(dev, "GEMM workspace alloc", cr); dev->gemm_ws = 0; return 0; }
    /* A fresh workspace starts as zeros: the persistent GEMM compares words in it with a
     * per-call tag that is never zero. */
    cr = a->MemsetD8Async(dev->gemm_ws, 0, bytes, dev->stream);
    if (cr != CUDA_SUCCESS) { sm100_fail(dev, "clearing the GEMM workspace", cr); a->MemFree(dev->gemm_ws); dev->gemm_ws = 0; return 0; }
    dev->gemm_ws_bytes = bytes;
    return dev->gemm_ws;
}

/* ---- launch ---- */

static void snap_dispatch(sm100_dev_t *dev, const char *kernel, unsigned gx, unsigned gy, unsigned gz,
                          unsigned bx, unsigned by, unsigned bz, unsigned shmem, const void *args, unsigned args_size)
{
    snprintf(dev->last.kernel, sizeof dev->last.kernel, "%.63s", kernel && *kernel ? kernel : "?");
    dev->last.grid[0] = gx; dev->last.grid[1] = gy; dev->last.grid[2] = gz;
    dev->last.block[0] = bx; dev->last.block[1] = by; dev->last.block[2] = bz;
    dev->last.shmem = shmem;
    dev->last.args_size = args_size;
    dev->last.snap_size = args_size < sizeof dev->last.args ? args_size : (unsigned)sizeof dev->last.args;
    if (args && dev->last.snap_size) memcpy(dev->last.args, args, dev->last.snap_size);
    else dev->last.snap_size = 0;
    dev->last.valid = 1;
}

static void dump_trak(sm100_dev_t *dev)
{
    if (dev->last.valid) {
        fprintf(stderr, "sm100_rt:   last dispatch: kernel '%s' grid %ux%ux%u block %ux%ux%u shmem %u, %u parameter bytes:",
                dev->last.kernel, dev->last.grid[0], dev->last.grid[1], dev->last.grid[2],
                dev->last.block[0], dev->last.block[1], dev->last.block[2], dev->last.shmem, dev->last.args_size);
        for (unsigned i = 0; i < dev->last.snap_size; i++)
            fprintf(stderr, "%s%02x", (i % 8) ? "" : " ", dev->last.args[i]);
        fprintf(stderr, "\n");
    }
    for (int i = 0; i < dev->ntrak; i++)
        fprintf(stderr, "sm100_rt:   buffer '%s' at 0x%llx, %llu bytes\n",
                dev->trak[i].label, dev->trak[i].ptr, dev->trak[i].size);
}

int sm100_rt_launch(sm100_dev_t *dev, const sm100_kern_t *kern,
                    uint32_t gx, uint32_t gy, uint32_t gz,
                    uint32_t bx, uint32_t by, uint32_t bz,
                    uint32_t shmem, void **args)
{
    if (!kern || !kern->func) return fail_arg(dev, "sm100_rt_launch: no kernel");
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    snap_dispatch(dev, kern->name, gx, gy, gz, bx, by, bz, shmem, NULL, 0);
    CUresult cr = dev->api->LaunchKernel((CUfunction)kern->func, gx, gy, gz, bx, by, bz,
                                         shmem, dev->stream, args, NULL);
    if (cr != CUDA_SUCCESS) {
        char what[192];
        snprintf(what, sizeof what, "cuLaunchKernel '%s' grid %ux%ux%u block %ux%ux%u",
                 kern->name, gx, gy, gz, bx, by, bz);
        rc = sm100_fail(dev, what, cr);
        dump_trak(dev);
        return rc;
    }
    dev->launches++;
    return SM100_OK;
}

int sm100_rt_launch_packed(sm100_dev_t *dev, const sm100_kern_t *kern,
                           uint32_t gx, uint32_t gy, uint32_t gz,
                           uint32_t bx, uint32_t by, uint32_t bz,
                           uint32_t shmem, const void *args, uint32_t args_size)
{
    if (!kern || !kern->func) return fail_arg(dev, "sm100_rt_launch_packed: no kernel");
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    unsigned char block[4096];
    size_t want = kern->param_bytes ? kern->param_bytes : args_size;
    if (want > sizeof block) return fail_arg(dev, "parameter block larger than 4096 bytes");
    memset(block, 0, want ? want : 1);
    if (args && args_size) memcpy(block, args, args_size < want ? args_size : want);
    snap_dispatch(dev, kern->name, gx, gy, gz, bx, by, bz, shmem, block, (unsigned)want);
    void *extra[] = {
        CU_LAUNCH_PARAM_BUFFER_POINTER, block,
        CU_LAUNCH_PARAM_BUFFER_SIZE, &want,
        CU_LAUNCH_PARAM_END
    };
    CUresult cr = dev->api->LaunchKernel((CUfunction)kern->func, gx, gy, gz, bx, by, bz,
                                         shmem, dev->stream, NULL, want ? extra : NULL);
    if (cr != CUDA_SUCCESS) {
        char what[192];
        snprintf(what, sizeof what, "cuLaunchKernel '%s' grid %ux%ux%u block %ux%ux%u args %u B",
                 kern->name, gx, gy, gz, bx, by, bz, args_size);
        rc = sm100_fail(dev, what, cr);
        dump_trak(dev);
        return rc;
    }
    dev->launches++;
    return SM100_OK;
}

int sm100_launch_k3(sm100_dev_t *dev, int which, unsigned gx, unsigned gy, unsigned gz,
                    unsigned bx, unsigned by, unsigned bz, unsigned shmem, void **args)
{
    CUresult cr = dev->api->LaunchKernel(dev->k[which], gx, gy, gz, bx, by, bz,
                                         shmem, dev->stream, args, NULL);
    if (cr != CUDA_SUCCESS) {
        char what[160];
        snprintf(what, sizeof what, "cuLaunchKernel '%s' grid %ux%ux%u block %ux%ux%u shmem %u",
                 k_names[which], gx, gy, gz, bx, by, bz, shmem);
        return sm100_fail(dev, what, cr);
    }
    dev->launches++;
    return SM100_OK;
}

int sm100_launch_k(sm100_dev_t *dev, int which, unsigned grid, unsigned block,
                   unsigned shmem, void **args)
{
    return sm100_launch_k3(dev, which, grid, 1, 1, block, 1, 1, shmem, args);
}

int sm100_launch_k3_overlapped(sm100_dev_t *dev, int which, unsigned gx, unsigned gy, unsigned gz,
                               unsigned bx, unsigned by, unsigned bz, unsigned shmem, void **args)
{
    static int enabled = -1;
    if (enabled < 0) {
        const char *e = getenv("BOOTH_SM100_PDL");
        enabled = !(e && e[0] == '0');
    }
    if (!enabled || !dev->api->LaunchKernelEx) return sm100_launch_k3(dev, which, gx, gy, gz, bx, by, bz, shmem, args);
    CUlaunchAttribute attr;
    memset(&attr, 0, sizeof attr);
    attr.id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
    attr.value.programmaticStreamSerializationAllowed = 1;
    CUlaunchConfig cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDimX = gx; cfg.gridDimY = gy; cfg.gridDimZ = gz;
    cfg.blockDimX = bx; cfg.blockDimY = by; cfg.blockDimZ = bz;
    cfg.sharedMemBytes = shmem;
    cfg.hStream = dev->stream;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    CUresult cr = dev->api->LaunchKernelEx(&cfg, dev->k[which], args, NULL);
    if (cr != CUDA_SUCCESS) {
        char what[160];
        snprintf(what, sizeof what, "cuLaunchKernelEx '%s' grid %ux%ux%u block %ux%ux%u shmem %u", k_names[which],
                 gx, gy, gz, bx, by, bz, shmem);
        return sm100_fail(dev, what, cr);
    }
    dev->launches++;
    return SM100_OK;
}

int sm100_launch_k_overlapped(sm100_dev_t *dev, int which, unsigned grid, unsigned block,
                              unsigned shmem, void **args)
{
    return sm100_launch_k3_overlapped(dev, which, grid, 1, 1, block, 1, 1, shmem, args);
}

int sm100_rt_sync(sm100_dev_t *dev)
{
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    CUresult cr = dev->api->StreamSynchronize(dev->stream);
    if (cr != CUDA_SUCCESS) { rc = sm100_fail(dev, "sync", cr); dump_trak(dev); return rc; }
    return sm100_gemm_outcome(dev);
}

int sm100_rt_tic(sm100_dev_t *dev)
{
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    CUresult cr = dev->api->EventRecord(dev->ev0, dev->stream);
    return cr == CUDA_SUCCESS ? SM100_OK : sm100_fail(dev, "cuEventRecord", cr);
}

int sm100_rt_toc(sm100_dev_t *dev, float *ms)
{
    int rc = sm100_enter(dev);
    if (rc != SM100_OK) return rc;
    CUresult cr = dev->api->EventRecord(dev->ev1, dev->stream);
    if (cr == CUDA_SUCCESS) cr = dev->api->EventSynchronize(dev->ev1);
    if (cr == CUDA_SUCCESS && ms) cr = dev->api->EventElapsedTime(ms, dev->ev0, dev->ev1);
    if (cr != CUDA_SUCCESS) return sm100_fail(dev, "event timing", cr);
    return sm100_gemm_outcome(dev);
}
