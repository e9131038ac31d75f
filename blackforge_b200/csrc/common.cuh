// Shared host-side plumbing for the C ABI: per-thread error text, status mapping, launch counting.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>

#include "../../include/bfb200.h"

namespace bfb {

// Errors follow the reference's convention so the C++ layer can let them propagate unchanged:
// argument problems are std::invalid_argument, everything else std::runtime_error (with the BFB_*
// status attached for the C boundary).
struct InvalidArgument : std::invalid_argument {
    using std::invalid_argument::invalid_argument;
};
struct RuntimeFailure : std::runtime_error {
    bfb_status status;
    RuntimeFailure(bfb_status s, const std::string& t) : std::runtime_error(t), status(s) {}
};

std::string& lastErrorSlot();
int64_t& launchCounter();

inline void noteLaunch(int n = 1) { launchCounter() += n; }

[[noreturn]] inline void fail(bfb_status s, const std::string& text) {
    if (s == BFB_INVALID_ARGUMENT) throw InvalidArgument(text);
    throw RuntimeFailure(s, text);
}

inline void require(bool ok, const char* text) {
    if (!ok) fail(BFB_INVALID_ARGUMENT, text);
}

inline void cudaCheck(cudaError_t e, const char* what, const char* file, int line) {
    if (e != cudaSuccess) {
        fail(BFB_CUDA_ERROR, std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ") at " +
                                 file + ":" + std::to_string(line));
    }
}
#define BFB_CUDA(expr) ::bfb::cudaCheck((expr), #expr, __FILE__, __LINE__)
#define BFB_LAUNCH_CHECK() ::bfb::cudaCheck(cudaGetLastError(), "kernel launch", __FILE__, __LINE__)

// Runs `fn`, converting exceptions into a status + last-error text.
template <typename Fn>
bfb_status guarded(Fn&& fn) noexcept {
    try {
        fn();
        return BFB_OK;
    } catch (const RuntimeFailure& e) {
        lastErrorSlot() = e.what();
        return e.status;
    } catch (const std::invalid_argument& e) {
        lastErrorSlot() = e.what();
        return BFB_INVALID_ARGUMENT;
    } catch (const std::exception& e) {
        lastErrorSlot() = e.what();
        return BFB_CUDA_ERROR;
    } catch (...) {
        lastErrorSlot() = "unknown failure";
        return BFB_CUDA_ERROR;
    }
}

// The status word a tensor-core kernel leaves behind (0 = ok): anything else means one of its bounded waits ran out.
inline void failOnDeviceStatus(int code) {
    if (code != 0) {
        fail(BFB_TIMEOUT, "a bounded wait inside a tensor-core kernel ran out (device code " + std::to_string(code) + ")");
    }
}

inline cudaStream_t asStream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

inline size_t dtypeBytes(int32_t dtype) {
    switch (dtype) {
        case BFB_F32: return 4;
        case BFB_BF16: return 2;
        case BFB_FP8_E4M3: return 1;
        default: fail(BFB_INVALID_ARGUMENT, "unknown element format");
    }
}

// Launch with programmatic stream serialisation: the kernel may begin (up to its griddepcontrol.wait) before the
// previous kernel on `stream` has finished. Only for kernels that call pdl_wait() before they touch global memory
// the previous kernel writes or reads. For chains of short kernels (a generation step), where launch latency and
// each kernel's prologue are a large part of the time.
template <typename... KArgs, typename... Args>
inline void launchDependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smemBytes, cudaStream_t stream,
                            Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    BFB_CUDA(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
}

// Number of SMs of the current device (cached per device).
int smCount();
// SMs the persistent kernels (tcgen05 GEMMs, flash attention) size their grids for: all of them, minus the ones a
// caller set aside for kernels of another stream that must run beside them (a collective that overlaps the GEMMs:
// a persistent grid over every SM would make it wait for a whole GEMM). Even, at least 2.
int persistentSms();
void setReservedSms(int count);
int reservedSms();
// Dynamic tile order for the CTA-pair GEMM (tiles drawn from a device counter instead of the static round-robin):
// for GEMMs that share the SMs with a kernel of another stream. nextTileCounter() lends one of a small rotating set
// of device counters of the current device; the caller zeroes it on its stream before the launch.
void setDynamicTiles(bool on);
bool dynamicTiles();
int* nextTileCounter();

// ---- per-kernel device timing (off by default) -----------------------------------------------------
// When enabled on the calling thread, a ProfileScope brackets one kernel launch with CUDA events on
// the launching stream and books the elapsed time and the launch's algorithmic work (FLOPs or bytes)
// under its kind. Reading a kind synchronises on its events.
enum ProfileKind {
    kProfGemmTc = 0,   // tcgen05 GEMM, work = 2*M*N*K FLOPs
    kProfAttnTc = 1,   // tcgen05 attention, work = FLOPs of the visible (query, key) pairs
    kProfRmsnorm = 2,  // work = bytes read + written
    kProfEmbed = 3,    // work = bytes read + written
    kProfCast = 4,     // work = bytes read + written
    kProfKindCount = 5
};
void profileEnable(bool on);
void profileReset();
void profileRead(int kind, double* milliseconds, int64_t* launches, double* work);
struct ProfileScope {
    ProfileScope(int kind, cudaStream_t stream, double work);
    ~ProfileScope();
    ProfileScope(const ProfileScope&) = delete;
    ProfileScope& operator=(const ProfileScope&) = delete;

private:
    int slot_ = -1;
    cudaStream_t stream_ = nullptr;
};

}  // namespace bfb
