// thrml_comm: the library's handle on a NCCL communicator (one rank per process and GPU).
#include "comm.h"

#include <dlfcn.h>

#include <cstring>
#include <mutex>

using namespace thrml;

namespace thrml {

int32_t nccl_fail(const char* what, ncclResult_t r) {
    const NcclApi* api = nccl_api();
    const char* msg = api && api->GetErrorString ? api->GetErrorString(r) : "?";
    return fail(THRML_ERR_NCCL, std::string(what) + ": " + msg);
}

const NcclApi* nccl_api() {
    static NcclApi api;
    static bool tried = false, ok = false;
    static std::string why;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (!tried) {
        tried = true;
        // An already loaded libnccl.so.2 (for instance the one a host framework bundles) is found by its soname first.
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) {
            const char* e = dlerror();
            why = std::string("cannot load libnccl.so.2: ") + (e ? e : "unknown error");
        } else {
            bool all = true;
            auto get = [&](auto& fn, const char* name) {
                fn = reinterpret_cast<std::remove_reference_t<decltype(fn)>>(dlsym(h, name));
                if (!fn) { all = false; why = std::string("libnccl.so.2 lacks ") + name; }
            };
            get(api.GetVersion, "ncclGetVersion");
            get(api.GetUniqueId, "ncclGetUniqueId");
            get(api.CommInitRank, "ncclCommInitRank");
            get(api.CommDestroy, "ncclCommDestroy");
            get(api.CommAbort, "ncclCommAbort");
            get(api.CommCount, "ncclCommCount");
            get(api.CommUserRank, "ncclCommUserRank");
            get(api.AllReduce, "ncclAllReduce");
            get(api.Send, "ncclSend");
            get(api.Recv, "ncclRecv");
            get(api.GroupStart, "ncclGroupStart");
            get(api.GroupEnd, "ncclGroupEnd");
            get(api.GetErrorString, "ncclGetErrorString");
            ok = all;
        }
    }
    if (!ok) {
        fail(THRML_ERR_NCCL, why);
        return nullptr;
    }
    return &api;
}

}  // namespace thrml

extern "C" {

int32_t thrml_comm_unique_id(uint8_t* id_out) {
    if (!id_out) return fail(THRML_ERR_INVALID_ARG, "null id buffer");
    static_assert(NCCL_UNIQUE_ID_BYTES == THRML_COMM_ID_BYTES, "id size");
    const NcclApi* api = nccl_api();
    if (!api) return THRML_ERR_NCCL;
    ncclUniqueId id;
    NCCL_TRY(api, GetUniqueId(&id));
    std::memcpy(id_out, id.internal, THRML_COMM_ID_BYTES);
    return THRML_OK;
}

int32_t thrml_comm_create(thrml_ctx* ctx, const uint8_t* id, int32_t rank, int32_t world_size, thrml_comm** out) {
    if (!ctx || !id || !out) return fail(THRML_ERR_INVALID_ARG, "null argument");
    if (world_size < 1 || rank < 0 || rank >= world_size) return fail(THRML_ERR_INVALID_ARG, "rank out of range");
    const NcclApi* api = nccl_api();
    if (!api) return THRML_ERR_NCCL;
    CU_TRY(cudaSetDevice(ctx->device));
    ncclUniqueId uid;
    std::memcpy(uid.internal, id, THRML_COMM_ID_BYTES);
    ncclComm_t c = nullptr;
    NCCL_TRY(api, CommInitRank(&c, world_size, uid, rank));
    auto* h = new thrml_comm();
    h->ctx = ctx;
    h->device = ctx->device;
    h->nccl = c;
    h->rank = rank;
    h->world = world_size;
    h->owned = true;
    *out = h;
    return THRML_OK;
}

int32_t thrml_comm_adopt(thrml_ctx* ctx, void* nccl_comm, thrml_comm** out) {
    if (!ctx || !nccl_comm || !out) return fail(THRML_ERR_INVALID_ARG, "null argument");
    const NcclApi* api = nccl_api();
    if (!api) return THRML_ERR_NCCL;
    int rank = 0, world = 0;
    NCCL_TRY(api, CommUserRank(static_cast<ncclComm_t>(nccl_comm), &rank));
    NCCL_TRY(api, CommCount(static_cast<ncclComm_t>(nccl_comm), &world));
    auto* h = new thrml_comm();
    h->ctx = ctx;
    h->device = ctx->device;
    h->nccl = static_cast<ncclComm_t>(nccl_comm);
    h->rank = rank;
    h->world = world;
    h->owned = false;
    *out = h;
    return THRML_OK;
}

void thrml_comm_destroy(thrml_comm* c) {
    if (!c) return;
    if (c->owned && c->nccl) {  // handles may be destroyed in any order: the context is not touched here
        cudaSetDevice(c->device);
        cudaDeviceSynchronize();
        if (const NcclApi* api = nccl_api()) api->CommDestroy(c->nccl);
    }
    delete c;
}

int32_t thrml_comm_info(const thrml_comm* c, int32_t* rank_out, int32_t* world_out, int32_t* nccl_version_out) {
    if (!c) return fail(THRML_ERR_INVALID_ARG, "null communicator");
    if (rank_out) *rank_out = c->rank;
    if (world_out) *world_out = c->world;
    if (nccl_version_out) {
        const NcclApi* api = nccl_api();
        if (!api) return THRML_ERR_NCCL;
        int v = 0;
        NCCL_TRY(api, GetVersion(&v));
        *nccl_version_out = v;
    }
    return THRML_OK;
}

}  // extern "C"
