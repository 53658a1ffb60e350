/* sm100_internal.h -- private state shared by the C files of libbooth_sm100. */
#ifndef SM100_INTERNAL_H
#define SM100_INTERNAL_H

#include <cuda.h>          /* types and enums only; every entry point is dlsym'ed */
#include "booth_sm100.h"

/* The driver entry points the library uses, by their exported (versioned)
 * names. Kept as one table so a missing symbol is reported by name. */
typedef struct sm100_api {
    void *lib;
    CUresult (*Init)(unsigned);
    CUresult (*DeviceGetCount)(int *);
    CUresult (*DeviceGet)(CUdevice *, int);
    CUresult (*DeviceGetName)(char *, int, CUdevice);
    CUresult (*DeviceGetAttribute)(int *, CUdevice_attribute, CUdevice);
    CUresult (*PrimaryCtxRetain)(CUcontext *, CUdevice);
    CUresult (*PrimaryCtxRelease)(CUdevice);
    CUresult (*CtxSetCurrent)(CUcontext);
    CUresult (*CtxGetCurrent)(CUcontext *);
    CUresult (*ModuleLoadData)(CUmodule *, const void *);
    CUresult (*ModuleLoadDataEx)(CUmodule *, const void *, unsigned, CUjit_option *, void **);
    CUresult (*ModuleUnload)(CUmodule);
    CUresult (*ModuleGetFunction)(CUfunction *, CUmodule, const char *);
    CUresult (*FuncGetAttribute)(int *, CUfunction_attribute, CUfunction);
    CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int);
    CUresult (*FuncGetParamInfo)(CUfunction, size_t, size_t *, size_t *);   /* optional */
    CUresult (*ModuleGetFunctionCount)(unsigned int *, CUmodule);           /* optional */
    CUresult (*ModuleEnumerateFunctions)(CUfunction *, unsigned int, CUmodule); /* optional */
    CUresult (*FuncGetName)(const char **, CUfunction);                     /* optional */
    CUresult (*MemAlloc)(CUdeviceptr *, size_t);
    CUresult (*MemFree)(CUdeviceptr);
    CUresult (*MemcpyHtoD)(CUdeviceptr, const void *, size_t);
    CUresult (*MemcpyDtoH)(void *, CUdeviceptr, size_t);
    CUresult (*MemcpyHtoDAsync)(CUdeviceptr, const void *, size_t, CUstream);
    CUresult (*MemcpyDtoHAsync)(void *, CUdeviceptr, size_t, CUstream);
    CUresult (*MemsetD8Async)(CUdeviceptr, unsigned char, size_t, CUstream);
    CUresult (*MemHostAlloc)(void **, size_t, unsigned);
    CUresult (*MemFreeHost)(void *);
    CUresult (*MemHostGetDevicePointer)(CUdeviceptr *, void *, unsigned);
    CUresult (*StreamCreate)(CUstream *, unsigned);
    CUresult (*StreamDestroy)(CUstream);
    CUresult (*StreamSynchronize)(CUstream);
    CUresult (*StreamWaitEvent)(CUstream, CUevent, unsigned);
    CUresult (*EventCreate)(CUevent *, unsigned);
    CUresult (*EventDestroy)(CUevent);
    CUresult (*EventRecord)(CUevent, CUstream);
    CUresult (*EventSynchronize)(CUevent);
    CUresult (*EventElapsedTime)(float *, CUevent, CUevent);
    CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned,
                             unsigned, unsigned, unsigned, unsigned, CUstream,
                             void **, void **);
    CUresult (*LaunchKernelEx)(const CUlaunchConfig *, CUfunction, void **, void **);   /* optional */
    CUresult (*OccupancyMaxActiveClusters)(int *, CUfunction, const CUlaunchConfig *);  /* optional */
    CUresult (*GetErrorString)(CUresult, const char **);
    CUresult (*TensorMapEncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t,
                                     void *, const cuuint64_t *, const cuuint64_t *,
                                     const cuuint32_t *, const cuuint32_t *,
                                     CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
} sm100_api_t;

#define SM100_TRAK_MAX 64
#define SM100_STAGE_SLOTS 3
#define SM100_STAGE_BYTES (64u << 20)      /* one operand chunk: 16 Mi floats */
/* Byte offsets inside the device scratch buffer. */
#define SM100_SCRATCH_TICKET       0
#define SM100_SCRATCH_GEMM_STATUS  128
#define SM100_SCRATCH_PARTIALS     256

/* Built-in kernels, resolved once per device from the embedded image. */
enum {
    SM100_K_VADD, SM100_K_SAXPY, SM100_K_FILL,
    SM100_K_REDUCE_I32, SM100_K_REDUCE_F32,
    SM100_K_ASIAN_MC, SM100_K_ASIAN_MC_PRECISE,
    SM100_K_ASIAN_PATHS, SM100_K_ASIAN_PATHS_PRECISE,
    SM100_K_GEMM_PREPASS, SM100_K_GEMM_TF32X3, SM100_K_GEMM_TF32X3_N128, SM100_K_GEMM_TF32X3_2CTA, SM100_K_GEMM_TF32X3_2CTA_N128, SM100_K_GEMM_PERSIST,
    SM100_K_COUNT
};

struct sm100_dev {
    const sm100_api_t *api;
    int         ordinal;
    CUdevice    cudev;
    CUcontext   ctx;
    CUstream    stream;
    CUevent     ev0, ev1;
    CUmodule    image;                 /* built-in kernel image */
    CUfunction  k[SM100_K_COUNT];
    char        name[128];
    int         sm_major, sm_minor, sm_count;
    unsigned long long launches;
    char        err[256];
    /* Scratch owned by the device: block partials and the arrival counter of
     * the reductions and the pricer. */
    CUdeviceptr scratch;
    size_t      scratch_bytes;
    /* GEMM workspace: the hi/lo planes of A and of B transposed. */
    CUdeviceptr gemm_ws;
    size_t      gemm_ws_bytes;
    /* Host-pointer streaming (booth_sm100_*_host): a ring of device staging slots, a
     * stream for the uploads, one for the copies back, and three events per slot. */
    CUstream    stream_out, stream_in;
    CUdeviceptr stage;                 /* SM100_STAGE_SLOTS x 2 x SM100_STAGE_BYTES */
    CUevent     ev_uploaded[SM100_STAGE_SLOTS], ev_computed[SM100_STAGE_SLOTS], ev_drained[SM100_STAGE_SLOTS];
    int         stage_ready;
    int         gemm_pending;          /* a GEMM was enqueued since the last status check */
    int         gemm_smem_set;         /* dynamic shared memory limit raised on the GEMM kernels */
    unsigned    gemm_wait_ms;          /* limit of the GEMM kernel's barrier waits */
    unsigned    gemm_epoch;            /* tag of the latest persistent GEMM call (never zero once used) */
    int         gemm_clusters;         /* CTA pairs of the persistent GEMM kernel this GPU holds at once (0 = not asked yet) */
    /* The GEMM's four tensor maps (64-byte aligned, allocated on first use) and what they were encoded for. */
    CUtensorMap *gemm_maps;
    struct { CUdeviceptr ws; int Mp, Np, Kp, box_b, valid; } gemm_maps_key;
    /* Which B the split planes in the workspace belong to (booth_sm100_gemm_ex reuses them on request). */
    struct { CUdeviceptr b, planes; int K, N, valid; } gemm_b;
    /* Snapshot of the most recent dispatch (kernel, geometry, first bytes of the
     * parameter block), printed with the labelled buffers when a launch or the
     * wait for it reports an error: the launcher's share of the reference's
     * ABEND dump (src/runtime/bc_runtime.c:661-675, src/runtime/bc_abend.h:57-71). */
    struct { char kernel[64]; unsigned grid[3], block[3], shmem, args_size, snap_size; unsigned char args[128]; int valid; } last;
    /* bc_trak labels. */
    struct { unsigned long long ptr, size; char label[24]; int flags; } trak[SM100_TRAK_MAX];
    int         ntrak;
};

/* Records and prints "sm100_rt: <what>: <driver text>"; returns SM100_ERR_CUDA. */
int  sm100_fail(sm100_dev_t *dev, const char *what, CUresult rc);
/* Makes the device's context current on the calling thread. */
int  sm100_enter(sm100_dev_t *dev);
/* Launch one of the built-in kernels on the device's stream. */
int  sm100_launch_k(sm100_dev_t *dev, int which, unsigned grid, unsigned block,
                    unsigned shmem, void **args);
int  sm100_launch_k3(sm100_dev_t *dev, int which, unsigned gx, unsigned gy, unsigned gz,
                     unsigned bx, unsigned by, unsigned bz, unsigned shmem, void **args);
/* The same for kernels that begin with griddepcontrol.wait: the launch may be set
 * up, and its first blocks placed, while the previous kernel on the stream is still
 * finishing (programmatic stream serialization). */
int  sm100_launch_k_overlapped(sm100_dev_t *dev, int which, unsigned grid, unsigned block,
                               unsigned shmem, void **args);
int  sm100_launch_k3_overlapped(sm100_dev_t *dev, int which, unsigned gx, unsigned gy, unsigned gz,
                                unsigned bx, unsigned by, unsigned bz, unsigned shmem, void **args);
/* The kernel's name as the driver knows it, for messages; "kernel" when the driver
 * cannot say (cuFuncGetName is a CUDA 12.3 entry point). */
void sm100_func_name(sm100_dev_t *dev, void *func, char *out, size_t n);
/* Grows the device-owned scratch / GEMM workspace; returns 0 on failure. */
CUdeviceptr sm100_scratch(sm100_dev_t *dev, size_t bytes);
CUdeviceptr sm100_gemm_ws(sm100_dev_t *dev, size_t bytes);

/* Reads the status word of a GEMM enqueued since the last check (the stream must
 * be idle): SM100_OK, or SM100_ERR_CUDA with the text recorded and printed. */
int  sm100_gemm_outcome(sm100_dev_t *dev);

/* The embedded sm_100a kernel image (image.S). */
extern const unsigned char booth_sm100_image[];
extern const unsigned char booth_sm100_image_end[];

#endif
