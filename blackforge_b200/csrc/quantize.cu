// Per-tensor e4m3 quantisation of an activation: scale = 448 / max|x|, out = e4m3(x * scale).
// Three launches: (1) every block reduces its own 8192-element chunk to one partial maximum in a scratch
// array, (2) one block folds the partial maxima into {scale, 1/scale, 1/scale * weight inverse},
// (3) the conversion. No atomics, so the result does not depend on block scheduling.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <algorithm>
#include <mutex>
#include <string>
#include <unordered_map>

#include "common.cuh"
#include "kernels.hpp"
#include "pool.hpp"

namespace bfb {

namespace {

constexpr int kChunkThreads = 256;
constexpr int kChunkElems = 8192;  // elements reduced by one block

template <typename T>
__device__ __forceinline__ float absMax16(const T* p);
template <>
__device__ __forceinline__ float absMax16<float>(const float* p) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    return fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
}
template <>
__device__ __forceinline__ float absMax16<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
    return m;
}
template <typename T>
__device__ __forceinline__ float absOne(const T* p);
template <>
__device__ __forceinline__ float absOne<float>(const float* p) { return fabsf(*p); }
template <>
__device__ __forceinline__ float absOne<__nv_bfloat16>(const __nv_bfloat16* p) { return fabsf(__bfloat162float(*p)); }

template <typename T>
__global__ void __launch_bounds__(kChunkThreads)
partialAmaxKernel(const T* __restrict__ in, int64_t n, float* __restrict__ partial, int vectorised) {
    __shared__ float warpMax[kChunkThreads / 32];
    constexpr int kPerVec = 16 / static_cast<int>(sizeof(T));
    const int64_t begin = static_cast<int64_t>(blockIdx.x) * kChunkElems;
    const int64_t end = min(begin + static_cast<int64_t>(kChunkElems), n);
    float m = 0.0f;
    if (vectorised) {
        for (int64_t i = begin + static_cast<int64_t>(threadIdx.x) * kPerVec; i + kPerVec <= end;
             i += static_cast<int64_t>(kChunkThreads) * kPerVec) {
            m = fmaxf(m, absMax16<T>(in + i));
        }
        // tail of the last chunk that is not a whole vector
        const int64_t tail = begin + ((end - begin) / kPerVec) * kPerVec;
        for (int64_t i = tail + threadIdx.x; i < end; i += kChunkThreads) m = fmaxf(m, absOne<T>(in + i));
    } else {
        for (int64_t i = begin + threadIdx.x; i < end; i += kChunkThreads) m = fmaxf(m, absOne<T>(in + i));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if ((threadIdx.x & 31) == 0) warpMax[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = warpMax[0];
#pragma unroll
        for (int w = 1; w < kChunkThreads / 32; ++w) t = fmaxf(t, warpMax[w]);
        partial[blockIdx.x] = t;
    }
}

__global__ void __launch_bounds__(1024)
finalizeScaleKernel(const float* __restrict__ partial, int64_t count, float* __restrict__ scales,
                    const float* __restrict__ weightInverse) {
    __shared__ float warpMax[32];
    float m = 0.0f;
    for (int64_t i = threadIdx.x; i < count; i += blockDim.x) m = fmaxf(m, partial[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if ((threadIdx.x & 31) == 0) warpMax[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) t = fmaxf(t, warpMax[w]);
        const float s = t > 0.0f ? 448.0f / t : 1.0f;
        scales[0] = s;
        scales[1] = 1.0f / s;
        scales[2] = (1.0f / s) * (weightInverse != nullptr ? *weightInverse : 1.0f);
    }
}

// ---- rmsnorm + quantisation in two passes over x ---------------------------------------------------------
// Pass 1: one warp per row: r = 1 / sqrt(mean(x^2) + eps) to rowInv[row], and the block's maximum of
// |bf16(x * r)| (what a separate norm would have stored) to partial[block]. Pass 2: e4m3(bf16(x * r) * scale).
// x is read twice (2 + 2 bytes per element) and e4m3 written once, against 9 bytes per element for a norm that
// writes bf16, a maximum pass and a conversion pass.
constexpr int kNormThreads = 256;

__device__ __forceinline__ float bf16Rounded(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__global__ void __launch_bounds__(kNormThreads)
normAmaxKernel(const __nv_bfloat16* __restrict__ x, int64_t rows, int64_t dim, float eps, float* __restrict__ rowInv,
               float* __restrict__ partial, int vectorised) {
    __shared__ float warpMax[kNormThreads / 32];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int64_t warpsPerGrid = static_cast<int64_t>(gridDim.x) * (kNormThreads / 32);
    float blockMax = 0.0f;
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * (kNormThreads / 32) + warp; row < rows; row += warpsPerGrid) {
        const __nv_bfloat16* src = x + row * dim;
        float ss = 0.0f, mx = 0.0f;   // |x * r| is largest where |x| is: one pass gives both
        if (vectorised) {
            for (int64_t i = static_cast<int64_t>(lane) * 8; i < dim; i += 256) {
                const uint4 raw = *reinterpret_cast<const uint4*>(src + i);
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(h[j]);
                    ss = fmaf(f.x, f.x, fmaf(f.y, f.y, ss));
                    mx = fmaxf(mx, fmaxf(fabsf(f.x), fabsf(f.y)));
                }
            }
        } else {
            for (int64_t i = lane; i < dim; i += 32) {
                const float v = __bfloat162float(src[i]);
                ss = fmaf(v, v, ss);
                mx = fmaxf(mx, fabsf(v));
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
            mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        }
        const float inv = 1.0f / sqrtf(ss / static_cast<float>(dim) + eps);
        if (lane == 0) rowInv[row] = inv;
        // rounding to bf16 is monotonic, so the largest normalised magnitude is that of the largest |x|
        blockMax = fmaxf(blockMax, bf16Rounded(mx * inv));
    }
    if (lane == 0) warpMax[warp] = blockMax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = warpMax[0];
#pragma unroll
        for (int w = 1; w < kNormThreads / 32; ++w) t = fmaxf(t, warpMax[w]);
        partial[blockIdx.x] = t;
    }
}

// 8 elements per thread; dim is a multiple of 8, so a vector never straddles two rows.
__global__ void __launch_bounds__(kNormThreads)
normQuantizeKernel(const uint4* __restrict__ x, uint2* __restrict__ out, int64_t nVec, int64_t vecsPerRow,
                   const float* __restrict__ rowInv, const float* __restrict__ scales) {
    const float scale = scales[0];
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nVec; i += stride) {
        const float inv = __ldg(rowInv + i / vecsPerRow);
        const uint4 raw = x[i];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        uint2 packed;
        __nv_fp8x2_storage_t* o = reinterpret_cast<__nv_fp8x2_storage_t*>(&packed);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            o[j] = __nv_cvt_float2_to_fp8x2(make_float2(bf16Rounded(f.x * inv) * scale, bf16Rounded(f.y * inv) * scale),
                                            __NV_SATFINITE, __NV_E4M3);
        }
        out[i] = packed;
    }
}

__global__ void normQuantizeScalarKernel(const __nv_bfloat16* __restrict__ x, __nv_fp8_storage_t* __restrict__ out,
                                         int64_t n, int64_t dim, const float* __restrict__ rowInv,
                                         const float* __restrict__ scales) {
    const float scale = scales[0];
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float v = bf16Rounded(__bfloat162float(x[i]) * rowInv[i / dim]) * scale;
        out[i] = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
    }
}

// Pass 1 without reading x: the GEMM that wrote x left, per row and 128-column part, the sum of squares and the largest
// magnitude of the values it stored. One thread per row adds and maximises the parts (in index order, so the same
// bits on every run): r = 1 / sqrt(mean(x^2) + eps) to rowInv[row], the block's maximum of bf16(max|x| * r) to
// partial[block] — the figures normAmaxKernel would have found by reading x.
__global__ void __launch_bounds__(kNormThreads)
rowStatsAmaxKernel(const float* __restrict__ sumSqParts, const float* __restrict__ maxParts, int parts, int64_t rows,
                   int64_t dim, float eps, float* __restrict__ rowInv, float* __restrict__ partial) {
    __shared__ float warpMax[kNormThreads / 32];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kNormThreads;
    float best = 0.0f;
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * kNormThreads + threadIdx.x; row < rows; row += stride) {
        float ss = 0.0f, mx = 0.0f;
        for (int p = 0; p < parts; ++p) {
            ss += sumSqParts[static_cast<int64_t>(p) * rows + row];
            mx = fmaxf(mx, maxParts[static_cast<int64_t>(p) * rows + row]);
        }
        const float inv = 1.0f / sqrtf(ss / static_cast<float>(dim) + eps);
        rowInv[row] = inv;
        best = fmaxf(best, bf16Rounded(mx * inv));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = fmaxf(best, __shfl_xor_sync(0xFFFFFFFFu, best, o));
    if (lane == 0) warpMax[warp] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = warpMax[0];
#pragma unroll
        for (int w = 1; w < kNormThreads / 32; ++w) t = fmaxf(t, warpMax[w]);
        partial[blockIdx.x] = t;
    }
}

int normAmaxBlocks(int64_t rows) {
    return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>((rows + kNormThreads / 32 - 1) / (kNormThreads / 32),
                                                                 static_cast<int64_t>(smCount()) * 8)));
}

}  // namespace

int64_t rmsnormQuantizeScratchFloats(int64_t rows) { return rows + normAmaxBlocks(rows); }

void rmsnormQuantizeE4m3(const void* x, int64_t rows, int64_t dim, float eps, void* out, float* dScales,
                         const float* dWeightInverse, float* scratch, cudaStream_t stream, const float* sumSqParts,
                         const float* maxParts, int parts) {
    require(rows >= 0 && dim > 0, "rmsnorm_quantize_e4m3: bad sizes");
    require(dScales != nullptr && scratch != nullptr, "rmsnorm_quantize_e4m3: null scale or scratch pointer");
    if (rows > 0) require(x != nullptr && out != nullptr, "rmsnorm_quantize_e4m3: null pointer");
    const bool fromStats = sumSqParts != nullptr && maxParts != nullptr && parts > 0;
    float* rowInv = scratch;
    float* partial = scratch + rows;
    int blocks = normAmaxBlocks(rows);
    const bool vec = dim % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 8 == 0;
    const double elems = static_cast<double>(rows) * static_cast<double>(dim);
    if (rows > 0 && fromStats) {
        blocks = static_cast<int>(std::min<int64_t>((rows + kNormThreads - 1) / kNormThreads, blocks));
        ProfileScope prof(kProfRmsnorm, stream, static_cast<double>(rows) * parts * 8.0);
        rowStatsAmaxKernel<<<blocks, kNormThreads, 0, stream>>>(sumSqParts, maxParts, parts, rows, dim, eps, rowInv, partial);
        BFB_LAUNCH_CHECK();
        noteLaunch();
    } else if (rows > 0) {
        ProfileScope prof(kProfRmsnorm, stream, elems * 2.0);
        normAmaxKernel<<<blocks, kNormThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), rows, dim, eps, rowInv,
                                                            partial, vec ? 1 : 0);
        BFB_LAUNCH_CHECK();
        noteLaunch();
    }
    finalizeScaleKernel<<<1, 1024, 0, stream>>>(partial, rows > 0 ? blocks : 0, dScales, dWeightInverse);
    BFB_LAUNCH_CHECK();
    noteLaunch();
    if (rows == 0) return;
    ProfileScope prof(kProfCast, stream, elems * 3.0);
    const int64_t n = rows * dim;
    if (vec) {
        const int64_t nVec = n / 8;
        const int grid = static_cast<int>(std::min<int64_t>((nVec + kNormThreads - 1) / kNormThreads,
                                                            static_cast<int64_t>(smCount()) * 16));
        normQuantizeKernel<<<grid, kNormThreads, 0, stream>>>(static_cast<const uint4*>(x), static_cast<uint2*>(out), nVec,
                                                              dim / 8, rowInv, dScales);
    } else {
        const int grid = static_cast<int>(std::min<int64_t>((n + kNormThreads - 1) / kNormThreads,
                                                            static_cast<int64_t>(smCount()) * 16));
        normQuantizeScalarKernel<<<grid, kNormThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(x),
                                                                    static_cast<__nv_fp8_storage_t*>(out), n, dim, rowInv,
                                                                    dScales);
    }
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

int64_t quantizeScratchFloats(int64_t n) { return std::max<int64_t>(1, (n + kChunkElems - 1) / kChunkElems); }

void quantizeE4m3(const void* in, int inDtype, int64_t n, void* out, float* dScales, const float* dWeightInverse,
                  float* scratch, cudaStream_t stream) {
    require(n >= 0, "quantize_e4m3: negative size");
    require(inDtype == BFB_F32 || inDtype == BFB_BF16, "quantize_e4m3: input must be f32 or bf16");
    require(dScales != nullptr, "quantize_e4m3: null scale pointer");
    require(scratch != nullptr, "quantize_e4m3: null scratch pointer");
    if (n > 0) require(in != nullptr && out != nullptr, "quantize_e4m3: null pointer");
    const int64_t blocks = quantizeScratchFloats(n);
    require(blocks <= 0x7FFFFFFF, "quantize_e4m3: tensor too large for one launch");
    const int vectorised = reinterpret_cast<uintptr_t>(in) % 16 == 0 ? 1 : 0;
    if (n > 0) {
        if (inDtype == BFB_F32) {
            partialAmaxKernel<float><<<static_cast<unsigned>(blocks), kChunkThreads, 0, stream>>>(
                static_cast<const float*>(in), n, scratch, vectorised);
        } else {
            partialAmaxKernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), kChunkThreads, 0, stream>>>(
                static_cast<const __nv_bfloat16*>(in), n, scratch, vectorised);
        }
        BFB_LAUNCH_CHECK();
        noteLaunch();
    }
    finalizeScaleKernel<<<1, 1024, 0, stream>>>(scratch, n > 0 ? blocks : 0, dScales, dWeightInverse);
    BFB_LAUNCH_CHECK();
    noteLaunch();
    if (n > 0) castScaled(in, inDtype, out, BFB_FP8_E4M3, n, 1.0f, dScales, stream);
}

void quantizeE4m3FromMaxima(const void* in, int inDtype, int64_t n, void* out, float* dScales, const float* dWeightInverse,
                            const float* maxima, int64_t count, float* scratch, cudaStream_t stream) {
    require(n >= 0 && count >= 0, "quantize_e4m3: negative size");
    require(inDtype == BFB_F32 || inDtype == BFB_BF16, "quantize_e4m3: input must be f32 or bf16");
    require(dScales != nullptr && scratch != nullptr, "quantize_e4m3: null scale or scratch pointer");
    if (n > 0) require(in != nullptr && out != nullptr && maxima != nullptr && count > 0, "quantize_e4m3: null pointer");
    const int64_t blocks = quantizeScratchFloats(count);
    require(blocks <= 0x7FFFFFFF, "quantize_e4m3: too many maxima for one launch");
    if (n > 0) {
        // the maxima are magnitudes already; the kernel's fabs changes nothing
        partialAmaxKernel<float><<<static_cast<unsigned>(blocks), kChunkThreads, 0, stream>>>(
            maxima, count, scratch, reinterpret_cast<uintptr_t>(maxima) % 16 == 0 ? 1 : 0);
        BFB_LAUNCH_CHECK();
        noteLaunch();
    }
    finalizeScaleKernel<<<1, 1024, 0, stream>>>(scratch, n > 0 ? blocks : 0, dScales, dWeightInverse);
    BFB_LAUNCH_CHECK();
    noteLaunch();
    if (n > 0) castScaled(in, inDtype, out, BFB_FP8_E4M3, n, 1.0f, dScales, stream);
}

}  // namespace bfb

// ---- allocation-free variant ---------------------------------------------------------------------------
// Some hosts cannot let this library take device memory at call time: an engine that handed every byte of
// the GPU to its own arena at start-up, or a serving loop that must not reach cudaMalloc because it can
// stall the whole device. For them the partial maxima live in this fixed array instead of the pool. Every
// GPU on which the library is used keeps these 256 KiB until the process exits.
namespace bfb {
namespace {

constexpr int64_t kStaticScratchFloats = 65536;  // one partial maximum per 8192 elements -> 536 870 912 elements
__device__ __align__(256) float gQuantStaticScratch[kStaticScratchFloats];

// The array's name is only a host-side handle; kernels need its device address, which differs per device.
float* staticScratchForCurrentDevice() {
    static std::mutex mu;
    static std::unordered_map<int, float*> perDevice;
    int dev = 0;
    BFB_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    auto it = perDevice.find(dev);
    if (it != perDevice.end()) return it->second;
    float* ptr = nullptr;
    BFB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), gQuantStaticScratch));
    perDevice[dev] = ptr;
    return ptr;
}

}  // namespace
}  // namespace bfb

extern "C" bfb_status bfb_quantize_e4m3_static(const void* d_in, int32_t in_dtype, int64_t n, void* d_out,
                                               float* d_scales, const float* d_weight_inverse, void* stream) {
    return bfb::guarded([&] {
        bfb::require(n >= 0, "quantize_e4m3_static: negative size");
        if (bfb::quantizeScratchFloats(n) > bfb::kStaticScratchFloats) {
            bfb::fail(BFB_INVALID_ARGUMENT,
                      "quantize_e4m3_static: at most " + std::to_string(bfb::kStaticScratchFloats * 8192) +
                          " elements fit the built-in scratch array; use bfb_quantize_e4m3 for larger tensors");
        }
        float* scratch = bfb::staticScratchForCurrentDevice();
        // every block writes its own slot before the fold reads it, so nothing has to be cleared between calls
        bfb::quantizeE4m3(d_in, in_dtype, n, d_out, d_scales, d_weight_inverse, scratch, bfb::asStream(stream));
    });
}
