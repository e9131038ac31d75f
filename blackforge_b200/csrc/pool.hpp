// Device memory pool: exact-size free lists per device (the reference's devicePoolAcquire/Release
// contract, src/backend/cuda/device_pool.cu:29-65) with a lock, statistics and trim added.
#pragma once

#include <cstddef>

namespace bfb {

void* poolAcquire(size_t bytes);                  // throws bfb::Error(BFB_CUDA_ERROR) when out of memory
void poolRelease(void* ptr, size_t bytes) noexcept;  // same `bytes` as the acquire; never throws
void poolTrim();
void poolStats(size_t* cachedBytes, size_t* liveBytes);

// Fault injection for tests, on the host only: the `nth` acquisition from now on (1 = the next one), on any thread,
// fails as an exhausted device would (BFB_CUDA_ERROR) without touching the device; 0 disarms. One shot.
void poolFailAfter(long long nth);
}  // namespace bfb
