/* fake_cuda.c -- a stand-in for libcuda.so.1 for tests of the HOST side only.
 *
 * Test infrastructure, never part of the product: the tests build it into a
 * temporary directory and point the library at it with BOOTH_CUDA_LIB. It runs no
 * kernel and computes nothing: "device" memory is host memory, copies are memcpy,
 * and a launch only appends one line to the file named by FAKE_CUDA_LOG
 *
 *     launch <kernel> grid <x> <y> <z> block <x> <y> <z> shmem <bytes> overlap <0|1> packed <bytes>
 *
 * so that a test can check which kernels the host code launches, in which order
 * and with which geometry, without a GPU. FAKE_CUDA_FAIL=<entry point>:<k> makes
 * the k-th call of that entry point return an error (host-side fault injection).
 * FAKE_CUDA_GEMM_STATUS=<code> makes a launch of a gemm_tf32x3* kernel store that
 * code in the kernel's status word (its eleventh parameter), the way the real
 * kernel does when one of its bounded waits runs out.
 * The device it reports is an sm_100 part with 148 SMs.
 */
#define _POSIX_C_SOURCE 200809L
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef struct { char name[96]; int max_dyn_shmem; } fake_func_t;

static int fail_now(const char *entry)
{
    static char counted[32][48];
    static int counts[32], nct;
    const char *spec = getenv("FAKE_CUDA_FAIL");
    int i, k;
    size_t len;
    if (!spec) return 0;
    len = strlen(entry);
    if (strncmp(spec, entry, len) != 0 || spec[len] != ':') return 0;
    k = atoi(spec + len + 1);
    for (i = 0; i < nct; i++) if (strcmp(counted[i], entry) == 0) break;
    if (i == nct) { if (nct == 32) return 0; snprintf(counted[nct++], 48, "%s", entry); }
    return ++counts[i] == k;
}

static void logf_line(const char *line)
{
    const char *path = getenv("FAKE_CUDA_LOG");
    FILE *f;
    if (!path) return;
    f = fopen(path, "a");
    if (!f) return;
    fputs(line, f);
    fclose(f);
}

CUresult cuInit(unsigned flags) { (void)flags; return fail_now("cuInit") ? CUDA_ERROR_NO_DEVICE : CUDA_SUCCESS; }
CUresult cuDeviceGetCount(int *n) { *n = getenv("FAKE_CUDA_DEVICES") ? atoi(getenv("FAKE_CUDA_DEVICES")) : 1; return CUDA_SUCCESS; }
CUresult cuDeviceGet(CUdevice *d, int ordinal) { *d = ordinal; return CUDA_SUCCESS; }
CUresult cuDeviceGetName(char *name, int len, CUdevice d) { (void)d; snprintf(name, (size_t)len, "Fake B200 (host-logic tests)"); return CUDA_SUCCESS; }
CUresult cuDeviceGetAttribute(int *v, CUdevice_attribute a, CUdevice d)
{
    (void)d;
    if (a == CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR) *v = getenv("FAKE_CUDA_SM_MAJOR") ? atoi(getenv("FAKE_CUDA_SM_MAJOR")) : 10;
    else if (a == CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR) *v = 0;
    else if (a == CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT) *v = 148;
    else *v = 0;
    return CUDA_SUCCESS;
}
CUresult cuDevicePrimaryCtxRetain(CUcontext *c, CUdevice d) { *c = (CUcontext)(size_t)(0x1000 + d); return CUDA_SUCCESS; }
CUresult cuDevicePrimaryCtxRelease_v2(CUdevice d) { (void)d; return CUDA_SUCCESS; }
CUresult cuCtxSetCurrent(CUcontext c) { (void)c; return CUDA_SUCCESS; }
CUresult cuCtxGetCurrent(CUcontext *c) { *c = (CUcontext)(size_t)0x1000; return CUDA_SUCCESS; }

CUresult cuModuleLoadData(CUmodule *m, const void *image)
{
    (void)image;
    if (fail_now("cuModuleLoadData")) return CUDA_ERROR_INVALID_IMAGE;
    *m = (CUmodule)malloc(8);
    return CUDA_SUCCESS;
}
CUresult cuModuleLoadDataEx(CUmodule *m, const void *image, unsigned n, CUjit_option *o, void **v)
{
    (void)n; (void)o; (void)v;
    if (fail_now("cuModuleLoadDataEx")) return CUDA_ERROR_INVALID_PTX;
    return cuModuleLoadData(m, image);
}
CUresult cuModuleUnload(CUmodule m) { free(m); return CUDA_SUCCESS; }
CUresult cuModuleGetFunction(CUfunction *f, CUmodule m, const char *name)
{
    fake_func_t *fn;
    (void)m;
    if (strncmp(name, "no_such", 7) == 0) return CUDA_ERROR_NOT_FOUND;
    fn = (fake_func_t *)calloc(1, sizeof *fn);
    snprintf(fn->name, sizeof fn->name, "%s", name);
    *f = (CUfunction)fn;
    return CUDA_SUCCESS;
}
CUresult cuFuncGetAttribute(int *v, CUfunction_attribute a, CUfunction f) { (void)a; (void)f; *v = 0; return CUDA_SUCCESS; }
CUresult cuFuncSetAttribute(CUfunction f, CUfunction_attribute a, int v)
{
    if (a == CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES) ((fake_func_t *)f)->max_dyn_shmem = v;
    return CUDA_SUCCESS;
}
/* Parameter layouts of the two kernels the launcher tests dispatch with packed
 * arguments: saxpy(float *y, float *x, float a, int n) and everything else as one
 * pointer. */
CUresult cuFuncGetParamInfo(CUfunction f, size_t i, size_t *off, size_t *sz)
{
    static const size_t so[4] = { 0, 8, 16, 20 }, ss[4] = { 8, 8, 4, 4 };
    if (strcmp(((fake_func_t *)f)->name, "saxpy") == 0) {
        if (i >= 4) return CUDA_ERROR_INVALID_VALUE;
        *off = so[i]; *sz = ss[i];
        return CUDA_SUCCESS;
    }
    if (i >= 1) return CUDA_ERROR_INVALID_VALUE;
    *off = 0; *sz = 8;
    return CUDA_SUCCESS;
}

CUresult cuFuncGetName(const char **name, CUfunction f) { *name = ((fake_func_t *)f)->name; return CUDA_SUCCESS; }

CUresult cuMemAlloc_v2(CUdeviceptr *p, size_t n)
{
    if (fail_now("cuMemAlloc")) return CUDA_ERROR_OUT_OF_MEMORY;
    *p = (CUdeviceptr)(size_t)calloc(1, n ? n : 1);         /* large blocks are zero pages until touched */
    return *p ? CUDA_SUCCESS : CUDA_ERROR_OUT_OF_MEMORY;
}
CUresult cuMemFree_v2(CUdeviceptr p) { free((void *)(size_t)p); return CUDA_SUCCESS; }
CUresult cuMemcpyHtoD_v2(CUdeviceptr d, const void *s, size_t n) { memcpy((void *)(size_t)d, s, n); return CUDA_SUCCESS; }
CUresult cuMemcpyDtoH_v2(void *d, CUdeviceptr s, size_t n) { memcpy(d, (void *)(size_t)s, n); return CUDA_SUCCESS; }
CUresult cuMemcpyHtoDAsync_v2(CUdeviceptr d, const void *s, size_t n, CUstream st)
{
    char line[96];
    (void)st;
    if (fail_now("cuMemcpyHtoDAsync")) return CUDA_ERROR_INVALID_VALUE;
    memcpy((void *)(size_t)d, s, n);
    snprintf(line, sizeof line, "h2d %zu\n", n);
    logf_line(line);
    return CUDA_SUCCESS;
}
CUresult cuMemcpyDtoHAsync_v2(void *d, CUdeviceptr s, size_t n, CUstream st)
{
    char line[96];
    (void)st;
    if (fail_now("cuMemcpyDtoHAsync")) return CUDA_ERROR_INVALID_VALUE;
    memcpy(d, (void *)(size_t)s, n);
    snprintf(line, sizeof line, "d2h %zu\n", n);
    logf_line(line);
    return CUDA_SUCCESS;
}
CUresult cuMemsetD8Async(CUdeviceptr d, unsigned char v, size_t n, CUstream st) { (void)st; memset((void *)(size_t)d, v, n); return CUDA_SUCCESS; }
CUresult cuMemHostAlloc(void **p, size_t n, unsigned flags) { (void)flags; *p = calloc(1, n ? n : 1); return *p ? CUDA_SUCCESS : CUDA_ERROR_OUT_OF_MEMORY; }
CUresult cuMemFreeHost(void *p) { free(p); return CUDA_SUCCESS; }
CUresult cuMemHostGetDevicePointer_v2(CUdeviceptr *d, void *p, unsigned flags) { (void)flags; *d = (CUdeviceptr)(size_t)p; return CUDA_SUCCESS; }

CUresult cuStreamCreate(CUstream *s, unsigned flags) { (void)flags; *s = (CUstream)malloc(8); return CUDA_SUCCESS; }
CUresult cuStreamDestroy_v2(CUstream s) { free(s); return CUDA_SUCCESS; }
CUresult cuStreamSynchronize(CUstream s) { (void)s; return fail_now("cuStreamSynchronize") ? CUDA_ERROR_LAUNCH_FAILED : CUDA_SUCCESS; }
CUresult cuStreamWaitEvent(CUstream s, CUevent e, unsigned flags) { (void)s; (void)e; (void)flags; return CUDA_SUCCESS; }
CUresult cuEventCreate(CUevent *e, unsigned flags) { (void)flags; *e = (CUevent)malloc(8); return CUDA_SUCCESS; }
CUresult cuEventDestroy_v2(CUevent e) { free(e); return CUDA_SUCCESS; }
CUresult cuEventRecord(CUevent e, CUstream s) { (void)e; (void)s; return CUDA_SUCCESS; }
CUresult cuEventSynchronize(CUevent e) { (void)e; return CUDA_SUCCESS; }
CUresult cuEventElapsedTime(float *ms, CUevent a, CUevent b) { (void)a; (void)b; *ms = 1.0f; return CUDA_SUCCESS; }

static void gemm_status(CUfunction f, void **params)
{
    const char *code = getenv("FAKE_CUDA_GEMM_STATUS");
    if (code && params && strncmp(((fake_func_t *)f)->name, "gemm_tf32x3", 11) == 0)
        *(int *)(size_t)*(CUdeviceptr *)params[10] = atoi(code);
}

static CUresult record_launch(CUfunction f, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by, unsigned bz,
                              unsigned shmem, int overlap, void **extra)
{
    const fake_func_t *fn = (const fake_func_t *)f;
    char line[256];
    size_t packed = 0;
    if (fail_now("cuLaunchKernel")) return CUDA_ERROR_LAUNCH_OUT_OF_RESOURCES;
    if (gx == 0 || gy == 0 || gz == 0 || bx * by * bz == 0 || bx * by * bz > 1024) return CUDA_ERROR_INVALID_VALUE;
    if ((int)shmem > 48 * 1024 && (int)shmem > fn->max_dyn_shmem) return CUDA_ERROR_INVALID_VALUE;
    if (extra)
        for (int i = 0; extra[i] != CU_LAUNCH_PARAM_END; i += 2)
            if (extra[i] == CU_LAUNCH_PARAM_BUFFER_SIZE) packed = *(size_t *)extra[i + 1];
    snprintf(line, sizeof line, "launch %s grid %u %u %u block %u %u %u shmem %u overlap %d packed %zu\n",
             fn->name, gx, gy, gz, bx, by, bz, shmem, overlap, packed);
    logf_line(line);
    return CUDA_SUCCESS;
}
CUresult cuLaunchKernel(CUfunction f, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by, unsigned bz,
                        unsigned shmem, CUstream s, void **params, void **extra)
{
    (void)s;
    gemm_status(f, params);
    return record_launch(f, gx, gy, gz, bx, by, bz, shmem, 0, extra);
}
CUresult cuLaunchKernelEx(const CUlaunchConfig *c, CUfunction f, void **params, void **extra)
{
    int overlap = 0;
    gemm_status(f, params);
    for (unsigned i = 0; i < c->numAttrs; i++)
        if (c->attrs[i].id == CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION)
            overlap = c->attrs[i].value.programmaticStreamSerializationAllowed;
    return record_launch(f, c->gridDimX, c->gridDimY, c->gridDimZ, c->blockDimX, c->blockDimY, c->blockDimZ,
                         c->sharedMemBytes, overlap, extra);
}
CUresult cuGetErrorString(CUresult e, const char **s)
{
    *s = e == CUDA_ERROR_LAUNCH_OUT_OF_RESOURCES ? "fake: too many resources requested for launch"
       : e == CUDA_ERROR_OUT_OF_MEMORY ? "fake: out of memory"
       : e == CUDA_ERROR_INVALID_VALUE ? "fake: invalid argument" : "fake: error";
    return CUDA_SUCCESS;
}
CUresult cuTensorMapEncodeTiled(CUtensorMap *map, CUtensorMapDataType t, cuuint32_t rank, void *base, const cuuint64_t *dims,
                                const cuuint64_t *strides, const cuuint32_t *box, const cuuint32_t *estr,
                                CUtensorMapInterleave il, CUtensorMapSwizzle sw, CUtensorMapL2promotion l2,
                                CUtensorMapFloatOOBfill fill)
{
    char line[192];
    (void)t; (void)estr; (void)il; (void)sw; (void)l2; (void)fill;
    memset(map, 0, sizeof *map);
    if (rank != 2 || ((size_t)base & 15) || (strides[0] & 15)) return CUDA_ERROR_INVALID_VALUE;
    snprintf(line, sizeof line, "tensormap dims %llu %llu stride %llu box %u %u\n", (unsigned long long)dims[0],
             (unsigned long long)dims[1], (unsigned long long)strides[0], box[0], box[1]);
    logf_line(line);
    return CUDA_SUCCESS;
}
