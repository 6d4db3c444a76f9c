// NCCL bound at run time (dlopen), so the library loads and runs on one GPU
// without NCCL present and shares the copy a host process (e.g. torch) already
// loaded.  Only the calls the Lloyd loop needs.
#pragma once

#include <dlfcn.h>
#include <nccl.h>

#include <mutex>

#include "km_common.cuh"

namespace km {

struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                            cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t,
                            cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  void* handle = nullptr;

  static NcclApi* get() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
      const char* names[] = {"libnccl.so.2", "libnccl.so"};
      for (const char* nm : names) {
        api.handle = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
        if (api.handle) break;
      }
      if (!api.handle) return;
#define KM_SYM(field, sym) api.field = reinterpret_cast<decltype(api.field)>(dlsym(api.handle, sym))
      KM_SYM(GetUniqueId, "ncclGetUniqueId");
      KM_SYM(CommInitRank, "ncclCommInitRank");
      KM_SYM(CommInitAll, "ncclCommInitAll");
      KM_SYM(CommDestroy, "ncclCommDestroy");
      KM_SYM(AllReduce, "ncclAllReduce");
      KM_SYM(AllGather, "ncclAllGather");
      KM_SYM(GroupStart, "ncclGroupStart");
      KM_SYM(GroupEnd, "ncclGroupEnd");
      KM_SYM(GetErrorString, "ncclGetErrorString");
#undef KM_SYM
    });
    if (!api.handle || !api.AllReduce || !api.CommInitRank || !api.GetUniqueId) return nullptr;
    return &api;
  }
};

#define KM_NCCL(api, expr)                                                               \
  do {                                                                                   \
    ncclResult_t _r = (expr);                                                            \
    if (_r != ncclSuccess) {                                                             \
      ::km::set_error(std::string(#expr) + ": " +                                        \
                      ((api)->GetErrorString ? (api)->GetErrorString(_r) : "nccl error")); \
      return KM_ENCCL;                                                                   \
    }                                                                                    \
  } while (0)

}  // namespace km
