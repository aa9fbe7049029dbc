/* Stand-in for libnccl used by the failure-path tests: the five entry points libvolta_b200 binds,
 * each failing on request.  FAKE_NCCL_FAIL names the call that fails ("uid", "init", "allreduce") and
 * FAKE_NCCL_CODE the NCCL result code it returns (default 2, ncclSystemError); FAKE_NCCL_WORLD, when
 * set, makes ncclCommInitRank refuse any other rank count with ncclInvalidArgument (4), the way a
 * launcher that started the wrong number of ranks is caught.  No GPU, no network. */
#include <stdlib.h>
#include <string.h>

typedef struct { char internal[128]; } ncclUniqueId;

static int fail_code(const char *what) {
    const char *f = getenv("FAKE_NCCL_FAIL");
    if (!f || strcmp(f, what) != 0) return 0;
    const char *c = getenv("FAKE_NCCL_CODE");
    return c ? atoi(c) : 2;
}

int ncclGetUniqueId(ncclUniqueId *id) {
    int rc = fail_code("uid");
    if (rc) return rc;
    memset(id, 0x5a, sizeof *id);
    return 0;
}

int ncclCommInitRank(void **comm, int nranks, ncclUniqueId id, int rank) {
    (void)id;
    int rc = fail_code("init");
    if (rc) return rc;
    const char *w = getenv("FAKE_NCCL_WORLD");
    if (w && atoi(w) != nranks) return 4;
    if (rank < 0 || rank >= nranks) return 4;
    *comm = malloc(16);
    return *comm ? 0 : 2;
}

int ncclCommDestroy(void *comm) {
    free(comm);
    return 0;
}

int ncclAllReduce(const void *send, void *recv, size_t count, int dtype, int op, void *comm, void *stream) {
    (void)send; (void)recv; (void)count; (void)dtype; (void)op; (void)comm; (void)stream;
    return fail_code("allreduce");
}

const char *ncclGetErrorString(int rc) {
    switch (rc) {
    case 0: return "no error";
    case 1: return "unhandled cuda error";
    case 2: return "unhandled system error";
    case 3: return "internal error";
    case 4: return "invalid argument";
    case 5: return "invalid usage";
    case 6: return "remote process exited or there was a network error";
    }
    return "unknown result code";
}
