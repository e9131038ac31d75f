// Device memory pool + process-wide helpers behind the C ABI.
//
// The pool keeps the reference's contract (exact-size free lists per device, memory is reused and
// never handed back to the driver on release, release must not throw) and adds a mutex, statistics
// and an explicit trim.
#include <atomic>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "pool.hpp"

namespace bfb {

std::string& lastErrorSlot() {
    thread_local std::string slot;
    return slot;
}

int64_t& launchCounter() {
    thread_local int64_t counter = 0;
    return counter;
}

int smCount() {
    static std::mutex mu;
    static std::unordered_map<int, int> cache;
    int dev = 0;
    BFB_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(dev);
    if (it != cache.end()) return it->second;
    int n = 0;
    BFB_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    cache[dev] = n;
    return n;
}

namespace {
std::atomic<int> gReservedSms{0};
}

namespace {
std::atomic<bool> gDynamicTiles{false};
constexpr int kTileCounters = 256;
}

void setDynamicTiles(bool on) { gDynamicTiles.store(on); }
bool dynamicTiles() { return gDynamicTiles.load(); }
int* nextTileCounter() {
    static std::mutex mu;
    static std::unordered_map<int, int*> perDevice;
    static std::unordered_map<int, unsigned> next;
    int dev = 0;
    BFB_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    int*& base = perDevice[dev];
    if (base == nullptr) BFB_CUDA(cudaMalloc(&base, kTileCounters * sizeof(int)));
    return base + (next[dev]++ % kTileCounters);
}

void setReservedSms(int count) { gReservedSms.store(count < 0 ? 0 : count); }
int reservedSms() { return gReservedSms.load(); }
int persistentSms() {
    const int all = smCount();
    const int left = (all - gReservedSms.load()) & ~1;
    return left < 2 ? (all < 2 ? all : 2) : left;
}

// ---- per-kernel timing -----------------------------------------------------------------------------
namespace {
struct ProfileRecord {
    int kind;
    cudaEvent_t start, stop;
    double work;
};
struct ProfileState {
    bool enabled = false;
    std::vector<ProfileRecord> records;
    std::vector<cudaEvent_t> spare;
    cudaEvent_t event() {
        if (!spare.empty()) {
            cudaEvent_t e = spare.back();
            spare.pop_back();
            return e;
        }
        cudaEvent_t e = nullptr;
        BFB_CUDA(cudaEventCreate(&e));
        return e;
    }
};
ProfileState& profileState() {
    thread_local ProfileState state;
    return state;
}
}  // namespace

void profileEnable(bool on) { profileState().enabled = on; }

void profileReset() {
    ProfileState& st = profileState();
    for (ProfileRecord& r : st.records) {
        st.spare.push_back(r.start);
        st.spare.push_back(r.stop);
    }
    st.records.clear();
}

void profileRead(int kind, double* milliseconds, int64_t* launches, double* work) {
    ProfileState& st = profileState();
    double ms = 0.0, w = 0.0;
    int64_t n = 0;
    for (ProfileRecord& r : st.records) {
        if (r.kind != kind) continue;
        BFB_CUDA(cudaEventSynchronize(r.stop));
        float t = 0.0f;
        BFB_CUDA(cudaEventElapsedTime(&t, r.start, r.stop));
        ms += t;
        w += r.work;
        ++n;
    }
    if (milliseconds != nullptr) *milliseconds = ms;
    if (launches != nullptr) *launches = n;
    if (work != nullptr) *work = w;
}

ProfileScope::ProfileScope(int kind, cudaStream_t stream, double work) : stream_(stream) {
    ProfileState& st = profileState();
    if (!st.enabled) return;
    ProfileRecord r{kind, st.event(), st.event(), work};
    BFB_CUDA(cudaEventRecord(r.start, stream));
    st.records.push_back(r);
    slot_ = static_cast<int>(st.records.size()) - 1;
}

ProfileScope::~ProfileScope() {
    if (slot_ < 0) return;
    ProfileState& st = profileState();
    if (slot_ < static_cast<int>(st.records.size())) cudaEventRecord(st.records[slot_].stop, stream_);
}

namespace {

struct DevicePool {
    std::unordered_map<size_t, std::vector<void*>> freeLists;
    size_t cachedBytes = 0;
    size_t liveBytes = 0;
};

std::mutex gPoolMutex;
std::unordered_map<int, DevicePool> gPools;

int currentDevice() {
    int dev = 0;
    BFB_CUDA(cudaGetDevice(&dev));
    return dev;
}

}  // namespace

namespace {
std::atomic<long long> gFailCountdown{0};
}

void poolFailAfter(long long nth) { gFailCountdown.store(nth > 0 ? nth : 0); }

void* poolAcquire(size_t bytes) {
    if (bytes == 0) return nullptr;
    if (gFailCountdown.load(std::memory_order_relaxed) > 0 && gFailCountdown.fetch_sub(1) == 1) {
        fail(BFB_CUDA_ERROR, "device pool: allocation of " + std::to_string(bytes) +
                                 " bytes failed (failure injected by bfb_pool_fail_after)");
    }
    int dev = currentDevice();
    {
        std::lock_guard<std::mutex> lock(gPoolMutex);
        DevicePool& pool = gPools[dev];
        auto it = pool.freeLists.find(bytes);
        if (it != pool.freeLists.end() && !it->second.empty()) {
            void* p = it->second.back();
            it->second.pop_back();
            pool.cachedBytes -= bytes;
            pool.liveBytes += bytes;
            return p;
        }
    }
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
        // one retry after giving cached buffers back, then report
        cudaGetLastError();
        poolTrim();
        e = cudaMalloc(&p, bytes);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        fail(BFB_CUDA_ERROR, "device pool: cudaMalloc of " + std::to_string(bytes) + " bytes failed: " +
                                 cudaGetErrorString(e));
    }
    std::lock_guard<std::mutex> lock(gPoolMutex);
    gPools[dev].liveBytes += bytes;
    return p;
}

void poolRelease(void* ptr, size_t bytes) noexcept {
    if (ptr == nullptr || bytes == 0) return;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return;
    try {
        std::lock_guard<std::mutex> lock(gPoolMutex);
        DevicePool& pool = gPools[dev];
        pool.freeLists[bytes].push_back(ptr);
        pool.cachedBytes += bytes;
        pool.liveBytes = pool.liveBytes >= bytes ? pool.liveBytes - bytes : 0;
    } catch (...) {
        cudaFree(ptr);
    }
}

void poolTrim() {
    int dev = currentDevice();
    std::vector<void*> victims;
    {
        std::lock_guard<std::mutex> lock(gPoolMutex);
        DevicePool& pool = gPools[dev];
        for (auto& kv : pool.freeLists) {
            for (void* p : kv.second) victims.push_back(p);
            kv.second.clear();
        }
        pool.cachedBytes = 0;
    }
    for (void* p : victims) cudaFree(p);
}

void poolStats(size_t* cached, size_t* live) {
    int dev = currentDevice();
    std::lock_guard<std::mutex> lock(gPoolMutex);
    DevicePool& pool = gPools[dev];
    if (cached != nullptr) *cached = pool.cachedBytes;
    if (live != nullptr) *live = pool.liveBytes;
}

}  // namespace bfb
