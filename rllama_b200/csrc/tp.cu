// NCCL bound at run time. The library does not link libnccl: a process that already holds a
// copy (for example the one bundled with PyTorch) must not get a second one, so the symbols
// are looked up in the loaded image first and only then in the system library.
#include "tp.h"

#include <dlfcn.h>

#include <cstring>

namespace {

struct UniqueId { char internal[128]; };
typedef int (*fn_get_unique_id)(UniqueId*);
typedef int (*fn_comm_init_rank)(void**, int, UniqueId, int);
typedef int (*fn_comm_destroy)(void*);
typedef int (*fn_all_reduce)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef int (*fn_all_gather)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef const char* (*fn_error_string)(int);

constexpr int kNcclFloat32 = 7;  // ncclDataType_t
constexpr int kNcclSum = 0;      // ncclRedOp_t

struct Api {
    void* handle = nullptr;
    fn_get_unique_id get_unique_id = nullptr;
    fn_comm_init_rank comm_init_rank = nullptr;
    fn_comm_destroy comm_destroy = nullptr;
    fn_all_reduce all_reduce = nullptr;
    fn_all_gather all_gather = nullptr;
    fn_error_string error_string = nullptr;
    bool tried = false;
} g_api;

int load_api() {
    if (g_api.handle) return RLB_OK;
    if (g_api.tried) return rlb_fail(RLB_ERR_COMM, "NCCL is not available in this process");
    g_api.tried = true;
    void* h = nullptr;
    if (const char* p = getenv("RLB_NCCL_LIB")) h = dlopen(p, RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // already mapped (e.g. by PyTorch)
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return rlb_fail(RLB_ERR_COMM, "cannot load libnccl.so.2: %s", dlerror());
    g_api.get_unique_id = (fn_get_unique_id)dlsym(h, "ncclGetUniqueId");
    g_api.comm_init_rank = (fn_comm_init_rank)dlsym(h, "ncclCommInitRank");
    g_api.comm_destroy = (fn_comm_destroy)dlsym(h, "ncclCommDestroy");
    g_api.all_reduce = (fn_all_reduce)dlsym(h, "ncclAllReduce");
    g_api.all_gather = (fn_all_gather)dlsym(h, "ncclAllGather");
    g_api.error_string = (fn_error_string)dlsym(h, "ncclGetErrorString");
    if (!g_api.get_unique_id || !g_api.comm_init_rank || !g_api.comm_destroy || !g_api.all_reduce || !g_api.all_gather)
        return rlb_fail(RLB_ERR_COMM, "libnccl lacks a required entry point");
    g_api.handle = h;
    return RLB_OK;
}

int check(int rc, const char* what) {
    if (rc == 0) return RLB_OK;
    return rlb_fail(RLB_ERR_COMM, "%s failed: %s", what, g_api.error_string ? g_api.error_string(rc) : "nccl error");
}

}  // namespace

int nccl_unique_id(void* id128) {
    RLB_TRY(load_api());
    UniqueId id;
    RLB_TRY(check(g_api.get_unique_id(&id), "ncclGetUniqueId"));
    memcpy(id128, &id, sizeof(id));
    return RLB_OK;
}

int nccl_init(TpNccl* t, const void* id128, int rank, int size) {
    RLB_TRY(load_api());
    UniqueId id;
    memcpy(&id, id128, sizeof(id));
    RLB_TRY(check(g_api.comm_init_rank(&t->comm, size, id, rank), "ncclCommInitRank"));
    t->rank = rank;
    t->size = size;
    return RLB_OK;
}

int nccl_destroy(TpNccl* t) {
    if (t->comm && g_api.comm_destroy) g_api.comm_destroy(t->comm);
    t->comm = nullptr;
    return RLB_OK;
}

int nccl_allreduce_f32(TpNccl* t, float* buf, size_t count, cudaStream_t stream) {
    if (!t->comm) return rlb_fail(RLB_ERR_STATE, "tensor-parallel model without an initialised NCCL communicator");
    return check(g_api.all_reduce(buf, buf, count, kNcclFloat32, kNcclSum, t->comm, stream), "ncclAllReduce");
}

int nccl_allgather_f32(TpNccl* t, const float* send, float* recv, size_t count_per_rank, cudaStream_t stream) {
    if (!t->comm) return rlb_fail(RLB_ERR_STATE, "tensor-parallel model without an initialised NCCL communicator");
    return check(g_api.all_gather(send, recv, count_per_rank, kNcclFloat32, t->comm, stream), "ncclAllGather");
}
