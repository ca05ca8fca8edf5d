// Multi-GPU communicator of the library: one process per GPU, NCCL underneath.
//
// NCCL is resolved at run time (dlopen of libnccl.so.2 on the first communicator call), so a single-GPU host needs no
// NCCL at all and a host that already loaded one (PyTorch bundles its own) shares that copy.  Only the types come from
// <nccl.h>.  Every failing NCCL call is reported as THRML_ERR_NCCL with NCCL's own message.
#pragma once
#include <nccl.h>

#include "ctx.h"

namespace thrml {

struct NcclApi {
    decltype(&ncclGetVersion) GetVersion = nullptr;
    decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
    decltype(&ncclCommInitRank) CommInitRank = nullptr;
    decltype(&ncclCommDestroy) CommDestroy = nullptr;
    decltype(&ncclCommAbort) CommAbort = nullptr;
    decltype(&ncclCommCount) CommCount = nullptr;
    decltype(&ncclCommUserRank) CommUserRank = nullptr;
    decltype(&ncclAllReduce) AllReduce = nullptr;
    decltype(&ncclSend) Send = nullptr;
    decltype(&ncclRecv) Recv = nullptr;
    decltype(&ncclGroupStart) GroupStart = nullptr;
    decltype(&ncclGroupEnd) GroupEnd = nullptr;
    decltype(&ncclGetErrorString) GetErrorString = nullptr;
};
// nullptr (with the error slot set) when no NCCL library can be loaded.
const NcclApi* nccl_api();
int32_t nccl_fail(const char* what, ncclResult_t r);

}  // namespace thrml

#define NCCL_TRY(api, call)                                            \
    do {                                                               \
        ncclResult_t r__ = (api)->call;                                \
        if (r__ != ncclSuccess) return thrml::nccl_fail(#call, r__);   \
    } while (0)

struct thrml_comm {
    thrml_ctx* ctx = nullptr;  // identity only (collectives check that their handles share it); never dereferenced after creation
    int device = 0;
    ncclComm_t nccl = nullptr;
    int32_t rank = 0, world = 1;
    bool owned = false;  // created by thrml_comm_create (destroyed with the handle) or adopted from the host
};
