// Host side of the bf16 result path: device results that are bf16 numbers cross PCIe as 2-byte values and are
// widened to the fp32 words the caller asked for by host threads, while the device works on the next slice.
#pragma once

#include <cuda_runtime.h>

#include <condition_variable>
#include <cstddef>
#include <cstdint>
#include <deque>
#include <exception>
#include <mutex>
#include <thread>

namespace bfb200 {

// dst[i] = the fp32 value of bf16 src[i] (exact), one thread.
void widenBf16(const std::uint16_t* src, float* dst, std::size_t count);

// Number of host threads a WidenQueue uses by default: the machine's hardware threads divided by the number of
// processes on this host (LOCAL_WORLD_SIZE, when a launcher set it), at most 16; the environment variable
// BFB_HOST_THREADS overrides it.
int defaultWidenThreads();

// Jobs run one at a time, in submission order, on a coordinator thread: wait for the job's CUDA event (the
// device-to-host copy that filled `src`), then widen with `threads` threads.
class WidenQueue {
public:
    WidenQueue(int device, int threads);
    ~WidenQueue();
    WidenQueue(const WidenQueue&) = delete;
    WidenQueue& operator=(const WidenQueue&) = delete;

    // Returns the job's number (0, 1, 2, ... in submission order).
    std::size_t submit(cudaEvent_t ready, const std::uint16_t* src, float* dst, std::size_t count);
    // Blocks until job `job` has been written to its destination; rethrows a failure of the coordinator.
    void wait(std::size_t job);
    void waitAll();

private:
    struct Job {
        cudaEvent_t ready;
        const std::uint16_t* src;
        float* dst;
        std::size_t count;
    };
    void run();

    int device_;
    int threads_;
    std::mutex mutex_;
    std::condition_variable wake_;
    std::condition_variable done_;
    std::deque<Job> jobs_;
    std::size_t submitted_ = 0;
    std::size_t finished_ = 0;
    bool stop_ = false;
    std::exception_ptr error_;
    std::thread coordinator_;
};

}  // namespace bfb200
