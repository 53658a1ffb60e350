/* fake_nccl.c -- a stand-in for libnccl.so.2 for tests of the HOST side only.
 *
 * Test infrastructure, never part of the product (the tests point the library at
 * it with BOOTH_NCCL_LIB). It moves and adds nothing: every call appends a line to
 * the file named by FAKE_CUDA_LOG, and FAKE_NCCL_FAIL=<entry point>:<k> makes the
 * k-th call of that entry point return ncclSystemError, which is how the tests
 * stand in for a peer that died or a link that failed.
 */
#define _POSIX_C_SOURCE 200809L
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef struct fake_comm { int nranks, rank; } *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;

static int fail_now(const char *entry)
{
    static char counted[16][32];
    static int counts[16], nct;
    const char *spec = getenv("FAKE_NCCL_FAIL");
    size_t len = strlen(entry);
    int i;
    if (!spec || strncmp(spec, entry, len) != 0 || spec[len] != ':') return 0;
    for (i = 0; i < nct; i++) if (strcmp(counted[i], entry) == 0) break;
    if (i == nct) { if (nct == 16) return 0; snprintf(counted[nct++], 32, "%s", entry); }
    return ++counts[i] == atoi(spec + len + 1);
}

static void note(const char *fmt, long a, long b, long c)
{
    const char *path = getenv("FAKE_CUDA_LOG");
    FILE *f = path ? fopen(path, "a") : NULL;
    if (!f) return;
    fprintf(f, fmt, a, b, c);
    fclose(f);
}

int ncclGetUniqueId(ncclUniqueId *id) { memset(id, 0x5a, sizeof *id); return fail_now("ncclGetUniqueId") ? 2 : 0; }
int ncclCommInitRank(ncclComm_t *c, int nranks, ncclUniqueId id, int rank)
{
    if (fail_now("ncclCommInitRank") || id.internal[0] != 0x5a) return 2;
    *c = malloc(sizeof **c); (*c)->nranks = nranks; (*c)->rank = rank;
    note("nccl init_rank %ld of %ld%.0ld\n", rank, nranks, 0);
    return 0;
}
int ncclCommInitAll(ncclComm_t *c, int ndev, const int *devs)
{
    if (fail_now("ncclCommInitAll")) return 2;
    for (int i = 0; i < ndev; i++) { c[i] = malloc(sizeof **c); c[i]->nranks = ndev; c[i]->rank = i; }
    note("nccl init_all %ld devices, first ordinal %ld%.0ld\n", ndev, devs[0], 0);
    return 0;
}
int ncclCommDestroy(ncclComm_t c) { note("nccl destroy rank %ld%.0ld%.0ld\n", c->rank, 0, 0); free(c); return 0; }
int ncclAllReduce(const void *s, void *r, size_t count, int dtype, int op, ncclComm_t c, void *stream)
{
    (void)stream;
    if (fail_now("ncclAllReduce")) return 2;
    note("nccl allreduce rank %ld count %ld dtype %ld", c->rank, (long)count, dtype);
    note(" op %ld inplace %ld%.0ld\n", op, s == r, 0);
    return 0;
}
int ncclGroupStart(void) { note("nccl group_start%.0ld%.0ld%.0ld\n", 0, 0, 0); return 0; }
int ncclGroupEnd(void) { note("nccl group_end%.0ld%.0ld%.0ld\n", 0, 0, 0); return fail_now("ncclGroupEnd") ? 2 : 0; }
const char *ncclGetErrorString(int r) { return r == 2 ? "fake: unhandled system error" : "fake: error"; }
