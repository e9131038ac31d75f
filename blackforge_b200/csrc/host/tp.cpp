#include "tp.hpp"

#include <dlfcn.h>
#include <nccl.h>

#include <cstdlib>
#include <cstring>
#include <string>

#include "../common.cuh"
#include "watchdog.hpp"

namespace bfb200 {

namespace {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*getUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*commInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*allReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*groupStart)() = nullptr;
    ncclResult_t (*groupEnd)() = nullptr;
    ncclResult_t (*commDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*commAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*commGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
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
    a.groupStart = reinterpret_cast<decltype(a.groupStart)>(sym("ncclGroupStart"));
    a.groupEnd = reinterpret_cast<decltype(a.groupEnd)>(sym("ncclGroupEnd"));
    a.commDestroy = reinterpret_cast<decltype(a.commDestroy)>(sym("ncclCommDestroy"));
    a.commAbort = reinterpret_cast<decltype(a.commAbort)>(sym("ncclCommAbort"));
    a.commGetAsyncError = reinterpret_cast<decltype(a.commGetAsyncError)>(sym("ncclCommGetAsyncError"));
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

void tpAverageGradients(void* const* deviceBuffers, const std::int64_t* counts, int tensors, void* stream) {
    if (gComm == nullptr) bfb::fail(BFB_INVALID_ARGUMENT, "gradient average: communicator not initialised (bfb_tp_init)");
    bfb::require(tensors >= 0, "gradient average: negative tensor count");
    bfb::require(tensors == 0 || (deviceBuffers != nullptr && counts != nullptr), "gradient average: null table");
    for (int i = 0; i < tensors; ++i) {
        bfb::require(counts[i] >= 0, "gradient average: negative element count");
        bfb::require(counts[i] == 0 || deviceBuffers[i] != nullptr, "gradient average: null gradient buffer");
    }
    // one group: the library fuses the per-parameter reductions into as few launches as it can, so that the many small
    // tensors (biases, norms) cost no launch each
    check(api().groupStart(), "groupStart");
    ncclResult_t first = ncclSuccess;
    for (int i = 0; i < tensors && first == ncclSuccess; ++i) {
        if (counts[i] == 0) continue;
        first = api().allReduce(deviceBuffers[i], deviceBuffers[i], static_cast<size_t>(counts[i]), ncclFloat32, ncclAvg, gComm,
                                static_cast<cudaStream_t>(stream));
    }
    const ncclResult_t end = api().groupEnd();
    check(first, "allReduce (average)");
    check(end, "groupEnd");
}

void tpDestroy() {
    if (gComm != nullptr) {
        api().commDestroy(gComm);
        gComm = nullptr;
        gWorld = 1;
    }
}

bool tpReady() { return gComm != nullptr; }

std::int64_t tpTimeoutMs() {
    if (const char* e = std::getenv("BFB_TP_TIMEOUT_MS")) {
        const long long v = std::atoll(e);
        if (v > 0) return static_cast<std::int64_t>(v);
    }
    return 120000;
}

void tpSynchronize(void* stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (gComm == nullptr) {
        BFB_CUDA(cudaStreamSynchronize(s));
        return;
    }
    WatchdogHooks hooks;
    cudaError_t queryError = cudaSuccess;
    hooks.query = [&] {
        const cudaError_t e = cudaStreamQuery(s);
        if (e == cudaSuccess) return 0;
        if (e == cudaErrorNotReady) return 1;
        queryError = e;
        return 2;
    };
    hooks.asyncError = [&] {
        ncclResult_t state = ncclSuccess;
        if (api().commGetAsyncError(gComm, &state) != ncclSuccess) return 1;
        return (state == ncclSuccess || state == ncclInProgress) ? 0 : 1;
    };
    hooks.abort = [&] {
        // frees the communicator and makes its kernels on the device give up; the process group is gone afterwards
        api().commAbort(gComm);
        gComm = nullptr;
        gWorld = 1;
    };
    const std::int64_t limit = tpTimeoutMs();
    switch (waitWithDeadline(hooks, limit)) {
        case WatchdogOutcome::Completed: return;
        case WatchdogOutcome::TimedOut:
            bfb::fail(BFB_TIMEOUT, "tensor parallelism: the step did not finish within " + std::to_string(limit) +
                                       " ms (a rank is missing from a collective?); the communicator was aborted");
        case WatchdogOutcome::AsyncError:
            bfb::fail(BFB_CUDA_ERROR, "tensor parallelism: the communicator reported an asynchronous error and was aborted");
        case WatchdogOutcome::QueryError:
            bfb::fail(BFB_CUDA_ERROR, std::string("tensor parallelism: stream query failed: ") + cudaGetErrorString(queryError));
    }
}

}  // namespace bfb200
