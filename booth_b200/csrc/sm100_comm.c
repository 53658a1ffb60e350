/* sm100_comm.c -- the one collective of the path: an NCCL all-reduce (sum) of
 * the per-GPU partial results of the reduction and of the Monte Carlo pricer.
 *
 * The reference drives a single device (src/nvidia/nv_rt.c:132,
 * src/runtime/bc_runtime.c:234-244) and has no collective; sharding is new here.
 * The payload is 1 to 4 numbers, so the all-reduce is latency-bound; it runs on
 * the device's own stream right behind the kernel that produced the partials.
 * libnccl.so.2 is opened at run time, like the driver, so a single-GPU user
 * needs no NCCL at all. */
#define _POSIX_C_SOURCE 200809L
#include <dlfcn.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "sm100_internal.h"

/* The slice of NCCL's ABI this file uses, declared here so the build needs no
 * NCCL headers (the reference does the same for the driver, src/nvidia/nv_rt.h:27-40).
 * Values are those of nccl.h, stable across NCCL 2.x. */
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
typedef int ncclDataType_t;
typedef int ncclRedOp_t;
typedef void *cudaStream_t;
#define ncclSuccess  0
#define ncclSum      0
#define ncclInt32    2
#define ncclFloat32  7
#define ncclFloat64  8

typedef struct {
    void *lib;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *);
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int);
    ncclResult_t (*CommInitAll)(ncclComm_t *, int, const int *);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t,
                              ncclComm_t, cudaStream_t);
    ncclResult_t (*GroupStart)(void);
    ncclResult_t (*GroupEnd)(void);
    const char *(*GetErrorString)(ncclResult_t);
} nccl_api_t;

static nccl_api_t g_nccl;
static int g_nccl_rc = 1;
static pthread_mutex_t g_nccl_mu = PTHREAD_MUTEX_INITIALIZER;

struct sm100_comm {
    int          ndev;             /* 1 in the one-process-per-GPU form */
    ncclComm_t   comm[16];
    sm100_dev_t *dev[16];
};

static int nccl_load(void)
{
    const char *path = getenv("BOOTH_NCCL_LIB");
    if (!path || !*path) path = "libnccl.so.2";
    void *lib = dlopen(path, RTLD_NOW | RTLD_LOCAL);
    if (!lib) {
        fprintf(stderr, "sm100_rt: cannot open NCCL '%s': %s\n", path, dlerror());
        return SM100_ERR_DL;
    }
    g_nccl.lib = lib;
    struct { void **p; const char *name; } syms[] = {
        { (void **)&g_nccl.GetUniqueId, "ncclGetUniqueId" },
        { (void **)&g_nccl.CommInitRank, "ncclCommInitRank" },
        { (void **)&g_nccl.CommInitAll, "ncclCommInitAll" },
        { (void **)&g_nccl.CommDestroy, "ncclCommDestroy" },
        { (void **)&g_nccl.AllReduce, "ncclAllReduce" },
        { (void **)&g_nccl.GroupStart, "ncclGroupStart" },
        { (void **)&g_nccl.GroupEnd, "ncclGroupEnd" },
        { (void **)&g_nccl.GetErrorString, "ncclGetErrorString" },
    };
    for (size_t i = 0; i < sizeof syms / sizeof syms[0]; i++) {
        *syms[i].p = dlsym(lib, syms[i].name);
        if (!*syms[i].p) {
            fprintf(stderr, "sm100_rt: NCCL entry point '%s' not found\n", syms[i].name);
            return SM100_ERR_SYM;
        }
    }
    return SM100_OK;
}

static int nccl_get(void)
{
    pthread_mutex_lock(&g_nccl_mu);
    if (g_nccl_rc == 1) g_nccl_rc = nccl_load();
    int rc = g_nccl_rc;
    pthread_mutex_unlock(&g_nccl_mu);
    return rc;
}

static int nccl_fail(const char *what, ncclResult_t r)
{
    fprintf(stderr, "sm100_rt: %s: %s\n", what, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "NCCL error");
    return SM100_ERR_NCCL;
}

int sm100_comm_unique_id(void *id128)
{
    int rc = nccl_get();
    if (rc != SM100_OK) return rc;
    if (!id128) return SM100_ERR_ARG;
    ncclUniqueId id;
    ncclResult_t r = g_nccl.GetUniqueId(&id);
    if (r != ncclSuccess) return nccl_fail("ncclGetUniqueId", r);
    memcpy(id128, &id, SM100_COMM_ID_BYTES);
    return SM100_OK;
}

int sm100_comm_init_rank(sm100_comm_t **out, sm100_dev_t *dev, int nranks, int rank, const void *id128)
{
    if (!out || !dev || !id128 || nranks < 1 || rank < 0 || rank >= nranks) {
        fprintf(stderr, "sm100_rt: sm100_comm_init_rank: bad argument (rank %d of %d)\n", rank, nranks);
        return SM100_ERR_ARG;
    }
    *out = NULL;
    int rc = nccl_get();
    if (rc != SM100_OK) return rc;
    if ((rc = sm100_enter(dev)) != SM100_OK) return rc;
    sm100_comm_t *c = (sm100_comm_t *)calloc(1, sizeof *c);
    if (!c) return SM100_ERR_ARG;
    ncclUniqueId id;
    memcpy(&id, id128, SM100_COMM_ID_BYTES);
    ncclResult_t r = g_nccl.CommInitRank(&c->comm[0], nranks, id, rank);
    if (r != ncclSuccess) { free(c); return nccl_fail("ncclCommInitRank", r); }
    c->ndev = 1;
    c->dev[0] = dev;
    *out = c;
    return SM100_OK;
}

int sm100_comm_init_all(sm100_comm_t **out, sm100_dev_t **devs, int ndev)
{
    if (!out || !devs || ndev < 1 || ndev > 16) {
        fprintf(stderr, "sm100_rt: sm100_comm_init_all: bad device count %d\n", ndev);
        return SM100_ERR_ARG;
    }
    *out = NULL;
    int rc = nccl_get();
    if (rc != SM100_OK) return rc;
    sm100_comm_t *c = (sm100_comm_t *)calloc(1, sizeof *c);
    if (!c) return SM100_ERR_ARG;
    int ords[16];
    for (int i = 0; i < ndev; i++) {
        if (!devs[i]) { free(c); return SM100_ERR_ARG; }
        ords[i] = devs[i]->ordinal; c->dev[i] = devs[i];
    }
    ncclResult_t r = g_nccl.CommInitAll(c->comm, ndev, ords);
    if (r != ncclSuccess) { free(c); return nccl_fail("ncclCommInitAll", r); }
    c->ndev = ndev;
    *out = c;
    return SM100_OK;
}

/* In the one-process form `buf` is the address on every device in turn: call
 * once per device, passing the communicator and that device's buffer; the
 * device is identified by the buffer's owner given through comm->dev order. */
static int allreduce_one(sm100_comm_t *comm, int i, sm100_ptr_t buf, size_t count, int dtype)
{
    ncclDataType_t dt = dtype == SM100_I32 ? ncclInt32 : dtype == SM100_F32 ? ncclFloat32 : ncclFloat64;
    int rc = sm100_enter(comm->dev[i]);
    if (rc != SM100_OK) return rc;
    ncclResult_t r = g_nccl.AllReduce((const void *)(uintptr_t)buf, (void *)(uintptr_t)buf, count, dt,
                                      ncclSum, comm->comm[i], (cudaStream_t)comm->dev[i]->stream);
    if (r != ncclSuccess) return nccl_fail("ncclAllReduce", r);
    return SM100_OK;
}

int sm100_comm_allreduce_sum(sm100_comm_t *comm, sm100_ptr_t buf, size_t count, int dtype)
{
    if (!comm || !buf || dtype < 0 || dtype > 2) return SM100_ERR_ARG;
    if (comm->ndev != 1) {
        fprintf(stderr, "sm100_rt: use sm100_comm_allreduce_sum_dev with a multi-device communicator\n");
        return SM100_ERR_ARG;
    }
    return allreduce_one(comm, 0, buf, count, dtype);
}

int sm100_comm_allreduce_sum_dev(sm100_comm_t *comm, int index, sm100_ptr_t buf, size_t count, int dtype)
{
    if (!comm || !buf || dtype < 0 || dtype > 2 || index < 0 || index >= comm->ndev) return SM100_ERR_ARG;
    return allreduce_one(comm, index, buf, count, dtype);
}

int sm100_comm_group_begin(void)
{
    int rc = nccl_get();
    if (rc != SM100_OK) return rc;
    ncclResult_t r = g_nccl.GroupStart();
    return r == ncclSuccess ? SM100_OK : nccl_fail("ncclGroupStart", r);
}

int sm100_comm_group_end(void)
{
    int rc = nccl_get();
    if (rc != SM100_OK) return rc;
    ncclResult_t r = g_nccl.GroupEnd();
    return r == ncclSuccess ? SM100_OK : nccl_fail("ncclGroupEnd", r);
}

void sm100_comm_destroy(sm100_comm_t *comm)
{
    if (!comm) return;
    for (int i = 0; i < comm->ndev; i++)
        if (comm->comm[i]) {
            if (sm100_enter(comm->dev[i]) == SM100_OK)
                comm->dev[i]->api->StreamSynchronize(comm->dev[i]->stream);
            g_nccl.CommDestroy(comm->comm[i]);
        }
    free(comm);
}
