// Data-parallel communicator: NCCL resolved at run time with dlopen, so the library has no
// link-time dependency on it and single-GPU users never load it.  One sum-allreduce per layer
// over fp32 gradients is the only collective of the path; the reference has none.
#include <dlfcn.h>

#include <cstring>

#include "common.cuh"
#include "engine.h"

namespace flstm_b200 {

namespace {

// Minimal mirror of the NCCL C API types that cross the boundary (public, stable ABI).
struct NcclUniqueId { char internal[128]; };
typedef void *NcclComm;
enum { kNcclSuccess = 0, kNcclFloat32 = 7, kNcclSum = 0 };

struct NcclApi {
    void *handle = nullptr;
    int (*GetUniqueId)(NcclUniqueId *) = nullptr;
    int (*CommInitRank)(NcclComm *, int, NcclUniqueId, int) = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*CommAbort)(NcclComm) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    bool ok = false;
};

NcclApi &api() {
    static NcclApi a;
    static bool tried = false;
    if (tried) return a;
    tried = true;
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
        a.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (a.handle) break;
    }
    if (!a.handle) return a;
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(a.handle, "ncclGetUniqueId"));
    a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(a.handle, "ncclCommInitRank"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(a.handle, "ncclCommDestroy"));
    a.CommAbort = reinterpret_cast<decltype(a.CommAbort)>(dlsym(a.handle, "ncclCommAbort"));
    a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(dlsym(a.handle, "ncclAllReduce"));
    a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(dlsym(a.handle, "ncclGetErrorString"));
    a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.AllReduce && a.GetErrorString;
    return a;
}

int need_api() {
    if (!api().ok) return set_error(FLSTM_ERR_COMM, "libnccl.so.2 could not be loaded: %s", dlerror());
    return FLSTM_OK;
}

}  // namespace

struct Comm {
    NcclComm comm = nullptr;
    int rank = 0, world = 1;
};

int comm_unique_id(void *id128) {
    if (!id128) return set_error(FLSTM_ERR_INVALID, "null id");
    FLSTM_TRY(need_api());
    NcclUniqueId id;
    int r = api().GetUniqueId(&id);
    if (r != kNcclSuccess) return set_error(FLSTM_ERR_COMM, "ncclGetUniqueId: %s", api().GetErrorString(r));
    std::memcpy(id128, &id, sizeof(id));
    return FLSTM_OK;
}

int comm_create(const void *id128, int rank, int world, Comm **out) {
    if (world < 1 || rank < 0 || rank >= world) return set_error(FLSTM_ERR_INVALID, "bad rank %d of %d", rank, world);
    FLSTM_TRY(need_api());
    NcclUniqueId id;
    std::memcpy(&id, id128, sizeof(id));
    Comm *c = new Comm();
    c->rank = rank;
    c->world = world;
    int r = api().CommInitRank(&c->comm, world, id, rank);
    if (r != kNcclSuccess) {
        delete c;
        return set_error(FLSTM_ERR_COMM, "ncclCommInitRank: %s", api().GetErrorString(r));
    }
    *out = c;
    return FLSTM_OK;
}

void comm_destroy(Comm *c) {
    if (!c) return;
    if (c->comm && api().ok) api().CommDestroy(c->comm);
    delete c;
}

void comm_abort(Comm *c) {
    if (!c) return;
    if (c->comm && api().ok) {
        if (api().CommAbort) api().CommAbort(c->comm);
        else api().CommDestroy(c->comm);
    }
    delete c;
}

int comm_allreduce_sum_f32(Comm *c, float *buf, size_t count, cudaStream_t s) {
    if (!c || !c->comm) return set_error(FLSTM_ERR_COMM, "no communicator");
    int r = api().AllReduce(buf, buf, count, kNcclFloat32, kNcclSum, c->comm, s);
    if (r != kNcclSuccess) return set_error(FLSTM_ERR_COMM, "ncclAllReduce: %s", api().GetErrorString(r));
    return FLSTM_OK;
}

}  // namespace flstm_b200
