#include "vb_dp.h"

#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

namespace vb {
namespace {

// Minimal slice of the NCCL API (nccl.h): opaque communicator, 128-byte id, enums as ints.
struct NcclId { char internal[128]; };
typedef int (*fn_get_unique_id)(NcclId *);
typedef int (*fn_comm_init_rank)(void **, int, NcclId, int);
typedef int (*fn_comm_destroy)(void *);
typedef int (*fn_all_reduce)(const void *, void *, size_t, int, int, void *, cudaStream_t);
typedef const char *(*fn_error_string)(int);
const int kNcclFloat32 = 7, kNcclSum = 0;

struct Api {
    void *lib = nullptr;
    fn_get_unique_id get_unique_id = nullptr;
    fn_comm_init_rank comm_init_rank = nullptr;
    fn_comm_destroy comm_destroy = nullptr;
    fn_all_reduce all_reduce = nullptr;
    fn_error_string error_string = nullptr;
    std::string why;
};

Api *api() {
    static Api a;
    static std::once_flag once;
    std::call_once(once, [] {
        // $VOLTA_B200_NCCL_LIB names the library to use (a site's own build; the failure-path tests point it
        // at a stand-in whose calls return NCCL error codes).  Otherwise prefer a copy the process has
        // already loaded (e.g. the one bundled with torch).
        const char *names[] = {"libnccl.so.2", "libnccl.so"};
        if (const char *own = getenv("VOLTA_B200_NCCL_LIB")) {
            a.lib = dlopen(own, RTLD_NOW | RTLD_LOCAL);
            if (!a.lib) {
                a.why = std::string("VOLTA_B200_NCCL_LIB: ") + dlerror();
                return;
            }
        }
        for (const char *nm : names) {
            if (a.lib) break;
            a.lib = dlopen(nm, RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
        }
        if (!a.lib)
            for (const char *nm : names) {
                a.lib = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
                if (a.lib) break;
            }
        if (!a.lib) {
            a.why = "NCCL not found (dlopen libnccl.so.2 failed)";
            return;
        }
        a.get_unique_id = (fn_get_unique_id)dlsym(a.lib, "ncclGetUniqueId");
        a.comm_init_rank = (fn_comm_init_rank)dlsym(a.lib, "ncclCommInitRank");
        a.comm_destroy = (fn_comm_destroy)dlsym(a.lib, "ncclCommDestroy");
        a.all_reduce = (fn_all_reduce)dlsym(a.lib, "ncclAllReduce");
        a.error_string = (fn_error_string)dlsym(a.lib, "ncclGetErrorString");
        if (!a.get_unique_id || !a.comm_init_rank || !a.comm_destroy || !a.all_reduce) {
            a.why = "NCCL library lacks a required symbol";
            a.lib = nullptr;
        }
    });
    return &a;
}

std::string describe(Api *a, const char *what, int rc) {
    std::string s = what;
    s += " failed: ";
    s += (a->error_string ? a->error_string(rc) : "unknown NCCL error");
    return s;
}

}  // namespace

int DpComm::unique_id(uint8_t out[128], std::string *why) {
    Api *a = api();
    if (!a->lib) {
        if (why) *why = a->why;
        return 1;
    }
    NcclId id;
    memset(&id, 0, sizeof id);
    int rc = a->get_unique_id(&id);
    if (rc) {
        if (why) *why = describe(a, "ncclGetUniqueId", rc);
        return rc;
    }
    memcpy(out, id.internal, 128);
    return 0;
}

int DpComm::init(const uint8_t idb[128], int world, int rank) {
    Api *a = api();
    if (!a->lib) {
        err_ = a->why;
        return 1;
    }
    // A fixed algorithm and protocol make the summation order a function of the rank count
    // and buffer size only, which is what run-to-run bit identity at a fixed GPU count
    // needs.  A caller's own setting wins.
    setenv("NCCL_ALGO", "Ring", 0);
    setenv("NCCL_PROTO", "Simple", 0);
    NcclId id;
    memcpy(id.internal, idb, 128);
    int rc = a->comm_init_rank(&comm_, world, id, rank);
    if (rc) {
        err_ = describe(a, "ncclCommInitRank", rc);
        comm_ = nullptr;
        return rc;
    }
    return 0;
}

int DpComm::all_reduce_sum(float *buf, int64_t count, cudaStream_t stream) {
    Api *a = api();
    if (!comm_) {
        err_ = "communicator not initialised";
        return 1;
    }
    int rc = a->all_reduce(buf, buf, (size_t)count, kNcclFloat32, kNcclSum, comm_, stream);
    if (rc) err_ = describe(a, "ncclAllReduce", rc);
    return rc;
}

DpComm::~DpComm() {
    Api *a = api();
    if (comm_ && a->lib) a->comm_destroy(comm_);
    comm_ = nullptr;
}

}  // namespace vb
