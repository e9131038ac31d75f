#include "widen.hpp"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <system_error>
#include <string>
#include <vector>

#if defined(__x86_64__) || defined(_M_X64)
#include <emmintrin.h>
#define BFB_WIDEN_SSE2 1
#endif

namespace bfb200 {

void widenBf16(const std::uint16_t* src, float* dst, std::size_t count) {
    std::size_t i = 0;
#ifdef BFB_WIDEN_SSE2
    // scalar head up to a 16-byte aligned destination, then 8 values per step with streaming stores: the
    // destination is written once and not read again here, so it should not displace the source from cache
    while (i < count && (reinterpret_cast<std::uintptr_t>(dst + i) & 15u) != 0u) {
        const std::uint32_t bits = static_cast<std::uint32_t>(src[i]) << 16;
        std::memcpy(dst + i, &bits, 4);
        ++i;
    }
    const __m128i zero = _mm_setzero_si128();
    for (; i + 8 <= count; i += 8) {
        const __m128i v = _mm_loadu_si128(reinterpret_cast<const __m128i*>(src + i));
        // interleaving zeros below each 16-bit value is the shift by 16
        _mm_stream_si128(reinterpret_cast<__m128i*>(dst + i), _mm_unpacklo_epi16(zero, v));
        _mm_stream_si128(reinterpret_cast<__m128i*>(dst + i + 4), _mm_unpackhi_epi16(zero, v));
    }
    _mm_sfence();
#endif
    for (; i < count; ++i) {
        const std::uint32_t bits = static_cast<std::uint32_t>(src[i]) << 16;
        std::memcpy(dst + i, &bits, 4);
    }
}

int defaultWidenThreads() {
    if (const char* e = std::getenv("BFB_HOST_THREADS")) {
        const int v = std::atoi(e);
        if (v >= 1) return std::min(v, 256);
    }
    unsigned hc = std::thread::hardware_concurrency();
    if (hc == 0) hc = 4;
    // one process per GPU on the same host (LOCAL_WORLD_SIZE as set by torchrun): the ranks share the cores
    if (const char* e = std::getenv("LOCAL_WORLD_SIZE")) {
        const int ranks = std::atoi(e);
        if (ranks > 1) hc = std::max(1u, hc / static_cast<unsigned>(ranks));
    }
    return static_cast<int>(std::min(hc, 16u));
}

WidenQueue::WidenQueue(int device, int threads) : device_(device), threads_(std::max(1, threads)) {
    coordinator_ = std::thread([this] { run(); });
}

WidenQueue::~WidenQueue() {
    {
        std::lock_guard<std::mutex> lock(mutex_);
        stop_ = true;
    }
    wake_.notify_all();
    if (coordinator_.joinable()) coordinator_.join();
}

std::size_t WidenQueue::submit(cudaEvent_t ready, const std::uint16_t* src, float* dst, std::size_t count) {
    std::size_t id;
    {
        std::lock_guard<std::mutex> lock(mutex_);
        jobs_.push_back(Job{ready, src, dst, count});
        id = submitted_++;
    }
    wake_.notify_all();
    return id;
}

void WidenQueue::wait(std::size_t job) {
    std::unique_lock<std::mutex> lock(mutex_);
    done_.wait(lock, [&] { return finished_ > job || error_ != nullptr; });
    if (error_ != nullptr) std::rethrow_exception(error_);
}

void WidenQueue::waitAll() {
    std::unique_lock<std::mutex> lock(mutex_);
    done_.wait(lock, [&] { return finished_ == submitted_ || error_ != nullptr; });
    if (error_ != nullptr) std::rethrow_exception(error_);
}

void WidenQueue::run() {
    try {
        if (cudaSetDevice(device_) != cudaSuccess) throw std::runtime_error("WidenQueue: cudaSetDevice failed");
        while (true) {
            Job job;
            {
                std::unique_lock<std::mutex> lock(mutex_);
                wake_.wait(lock, [&] { return stop_ || !jobs_.empty(); });
                if (jobs_.empty()) return;  // stop requested and nothing left
                job = jobs_.front();
                jobs_.pop_front();
            }
            const cudaError_t err = cudaEventSynchronize(job.ready);
            if (err != cudaSuccess) {
                throw std::runtime_error(std::string("WidenQueue: device-to-host copy failed: ") + cudaGetErrorString(err));
            }
            // contiguous chunks, multiples of 8 values so that each thread's stores stay aligned
            const std::size_t parts = static_cast<std::size_t>(threads_);
            const std::size_t chunk = ((job.count + parts - 1) / parts + 7) / 8 * 8;
            std::vector<std::thread> helpers;
            helpers.reserve(parts);
            std::size_t inlineFrom = parts;  // chunks from here on had no thread and are done by this one
            for (std::size_t t = 1; t < parts; ++t) {
                const std::size_t begin = t * chunk;
                if (begin >= job.count) break;
                const std::size_t n = std::min(chunk, job.count - begin);
                try {
                    helpers.emplace_back([=] { widenBf16(job.src + begin, job.dst + begin, n); });
                } catch (const std::system_error&) {
                    inlineFrom = t;
                    break;
                }
            }
            widenBf16(job.src, job.dst, std::min(chunk, job.count));
            for (std::size_t t = inlineFrom; t < parts && t * chunk < job.count; ++t) {
                widenBf16(job.src + t * chunk, job.dst + t * chunk, std::min(chunk, job.count - t * chunk));
            }
            for (std::thread& h : helpers) h.join();
            {
                std::lock_guard<std::mutex> lock(mutex_);
                ++finished_;
            }
            done_.notify_all();
        }
    } catch (...) {
        std::lock_guard<std::mutex> lock(mutex_);
        error_ = std::current_exception();
        done_.notify_all();
    }
}

}  // namespace bfb200
