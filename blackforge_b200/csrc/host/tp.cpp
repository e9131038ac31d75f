#include "tp.hpp"

#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <string>

#include "../common.cuh"

namespace bfb200 {

namespace {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*getUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*commInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*allReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*commDestroy)(ncclComm_t) = nullptr;
    const char* (*getErrorString)(ncclResult_t) = nullptr;
};

NcclApi& api() {
    static NcclApi a;
    if (a.handle != nullptr) return a;
    a.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (a.handle == nullptr) a.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (a.handle == nullptr) bfb::fail(BFB_CUDA_ERROR, std::string("tensor parallelism: cannot load NCCL: ") + dlerror());
    auto sym = [&](const char* name) {
        void* p = dlsym(a.handle, name);
        if (p == nullptr) bfb::fail(BFB_CUDA_ERROR, std::string("tensor parallelism: NCCL symbol missing: ") + name);
        return p;
    };
    a.getUniqueId = reinterpret_cast<decltype(a.getUniqueId)>(sym("ncclGetUniqueId"));
    a.commInitRank = reinterpret_cast<decltype(a.commInitRank)>(sym("ncclCommInitRank"));
    a.allReduce = reinterpret_cast<decltype(a.allReduce)>(sym("ncclAllReduce"));
    a.commDestroy = reinterpret_cast<decltype(a.commDestroy)>(sym("ncclCommDestroy"));
    a.getErrorString = reinterpret_cast<decltype(a.getErrorString)>(sym("ncclGetErrorString"));
    return a;
}

ncclComm_t gComm = nullptr;
int gWorld = 1;

void check(ncclResult_t r, const char* what) {
    if (r != ncclSuccess) {
        bfb::fail(BFB_CUDA_ERROR, std::string("NCCL ") + what + " failed: " + api().getErrorString(r));
    }
}

}  // namespace

void tpUniqueId(void* hostId128) {
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is expected to be 128 bytes");
    bfb::require(hostId128 != nullptr, "tp_unique_id: null pointer");
    ncclUniqueId id;
    check(api().getUniqueId(&id), "getUniqueId");
    std::memcpy(hostId128, &id, sizeof(id));
}

void tpInit(const void* hostId128, int rank, int world) {
    bfb::require(hostId128 != nullptr, "tp_init: null id");
    bfb::require(world >= 1 && rank >= 0 && rank < world, "tp_init: bad rank / world");
    if (gComm != nullptr) tpDestroy();
    ncclUniqueId id;
    std::memcpy(&id, hostId128, sizeof(id));
    check(api().commInitRank(&gComm, world, id, rank), "commInitRank");
    gWorld = world;
}

void tpAllReduceSum(void* deviceBuffer, std::int64_t count, int dtype, void* stream) {
    if (gComm == nullptr) bfb::fail(BFB_INVALID_ARGUMENT, "tensor parallelism: communicator not initialised (bfb_tp_init)");
    bfb::require(dtype == BFB_F32 || dtype == BFB_BF16, "tp_allreduce: format must be f32 or bf16");
    if (count <= 0) return;
    check(api().allReduce(deviceBuffer, deviceBuffer, static_cast<size_t>(count), dtype == BFB_F32 ? ncclFloat32 : ncclBfloat16,
                          ncclSum, gComm, static_cast<cudaStream_t>(stream)),
          "allReduce");
}

void tpDestroy() {
    if (gComm != nullptr) {
        api().commDestroy(gComm);
        gComm = nullptr;
        gWorld = 1;
    }
}

bool tpReady() { return gComm != nullptr; }

}  // namespace bfb200
