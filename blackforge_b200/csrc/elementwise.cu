// HBM-bound kernels of the forward path: token gather + positions, rmsnorm, softmax, elementwise
// ops, format conversion, amax and the one-off weight transpose. All are single-pass over their
// inputs, 128-bit vectorised where alignment allows, and sized to a multiple of the SM count.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <algorithm>
#include <cmath>

#include "common.cuh"
#include "kernels.hpp"
#include "ptx_sm100.cuh"

namespace bfb {

namespace {

constexpr int kThreads = 256;

inline int gridFor(int64_t work, int perBlock, int wavesCap = 32) {
    int64_t blocks = (work + perBlock - 1) / perBlock;
    int64_t cap = static_cast<int64_t>(smCount()) * wavesCap;
    return static_cast<int>(std::max<int64_t>(1, std::min(blocks, cap)));
}

__device__ __forceinline__ float bf16Round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ float warpSum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
__device__ __forceinline__ float warpMax(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

// Block-wide sum / max through one shared array of 32 floats.
__device__ __forceinline__ float blockSum(float v, float* scratch) {
    v = warpSum(v);
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    int nw = (blockDim.x + 31) >> 5;
    float t = (threadIdx.x < nw) ? scratch[threadIdx.x] : 0.0f;
    if (warp == 0) t = warpSum(t);
    if (threadIdx.x == 0) scratch[0] = t;
    __syncthreads();
    return scratch[0];
}
__device__ __forceinline__ float blockMax(float v, float* scratch) {
    v = warpMax(v);
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    int nw = (blockDim.x + 31) >> 5;
    float t = (threadIdx.x < nw) ? scratch[threadIdx.x] : -INFINITY;
    if (warp == 0) t = warpMax(t);
    if (threadIdx.x == 0) scratch[0] = t;
    __syncthreads();
    return scratch[0];
}

// ---- embedding gather + positional add --------------------------------------------------------
// One block walks token rows; a row of `dim` floats is copied with float4 loads when dim % 4 == 0.
template <bool kVec, bool kOutBf16>
__global__ void embedPosKernel(const float* __restrict__ ids, const float* __restrict__ table,
                               const float* __restrict__ pos, void* __restrict__ outRaw, int64_t tokens, int64_t seq,
                               int64_t vocab, int64_t dim, int64_t posOffset, int* oobCount) {
    for (int64_t t = blockIdx.x; t < tokens; t += gridDim.x) {
        float idf = ids[t];
        bool finite = fabsf(idf) < 2147483648.0f;  // false for NaN / inf too
        long long id = finite ? static_cast<long long>(lroundf(idf)) : -1;
        bool ok = id >= 0 && id < vocab;
        if (!ok && threadIdx.x == 0 && oobCount != nullptr) atomicAdd(oobCount, 1);
        const float* src = table + static_cast<int64_t>(ok ? id : 0) * dim;
        const float* prow = pos != nullptr ? pos + (posOffset + t % seq) * dim : nullptr;
        if constexpr (kVec) {
            int64_t nv = dim >> 2;
            for (int64_t i = threadIdx.x; i < nv; i += blockDim.x) {
                float4 v = ok ? __ldg(reinterpret_cast<const float4*>(src) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                if (prow != nullptr) {
                    float4 p = __ldg(reinterpret_cast<const float4*>(prow) + i);
                    v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
                }
                if constexpr (kOutBf16) {
                    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y);
                    __nv_bfloat162 hi = __floats2bfloat162_rn(v.z, v.w);
                    uint2 packed;
                    packed.x = *reinterpret_cast<uint32_t*>(&lo);
                    packed.y = *reinterpret_cast<uint32_t*>(&hi);
                    reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(outRaw) + t * dim)[i] = packed;
                } else {
                    reinterpret_cast<float4*>(static_cast<float*>(outRaw) + t * dim)[i] = v;
                }
            }
        } else {
            for (int64_t i = threadIdx.x; i < dim; i += blockDim.x) {
                float v = ok ? src[i] : 0.0f;
                if (prow != nullptr) v += prow[i];
                if constexpr (kOutBf16) {
                    static_cast<__nv_bfloat16*>(outRaw)[t * dim + i] = __float2bfloat16_rn(v);
                } else {
                    static_cast<float*>(outRaw)[t * dim + i] = v;
                }
            }
        }
    }
}

__global__ void addPositionalKernel(const float* __restrict__ in, const float* __restrict__ pos,
                                    float* __restrict__ out, int64_t total, int64_t seq, int64_t dim,
                                    int64_t posOffset) {
    int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        int64_t tok = i / dim;
        int64_t d = i - tok * dim;
        out[i] = in[i] + pos[(posOffset + tok % seq) * dim + d];
    }
}

// ---- rmsnorm ----------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
    float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
    uint2 t = *reinterpret_cast<const uint2*>(p);
    __nv_bfloat162 lo = *reinterpret_cast<__nv_bfloat162*>(&t.x);
    __nv_bfloat162 hi = *reinterpret_cast<__nv_bfloat162*>(&t.y);
    v[0] = __low2float(lo); v[1] = __high2float(lo); v[2] = __low2float(hi); v[3] = __high2float(hi);
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&v)[4]);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]);
    __nv_bfloat162 hi = __floats2bfloat162_rn(v[2], v[3]);
    uint2 t;
    t.x = *reinterpret_cast<uint32_t*>(&lo);
    t.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = t;
}

// Row held in registers (read once). kGroup threads cooperate on one row: 32 (a warp) or the whole
// block. Each thread keeps up to kMaxVec groups of 4 elements.
template <typename TIn, typename TOut, int kMaxVec, bool kBlockPerRow>
__global__ void rmsnormKernel(const TIn* __restrict__ x, TOut* __restrict__ out, int64_t rows, int64_t dim, float eps) {
    __shared__ float scratch[32];
    const int group = kBlockPerRow ? blockDim.x : 32;
    const int lane = kBlockPerRow ? threadIdx.x : (threadIdx.x & 31);
    const int64_t rowsPerBlock = kBlockPerRow ? 1 : (blockDim.x >> 5);
    const int64_t firstRow = static_cast<int64_t>(blockIdx.x) * rowsPerBlock + (kBlockPerRow ? 0 : (threadIdx.x >> 5));
    const int64_t rowStride = static_cast<int64_t>(gridDim.x) * rowsPerBlock;
    const int64_t nv = dim >> 2;
    // Block-per-row: every thread of the block walks the same rows, so barriers stay uniform.
    for (int64_t row = firstRow; row < rows; row += rowStride) {
        const TIn* src = x + row * dim;
        float vals[kMaxVec][4];
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < kMaxVec; ++j) {
            int64_t i = lane + static_cast<int64_t>(j) * group;
            if (i < nv) {
                load4<TIn>(src + i * 4, vals[j]);
                ss += vals[j][0] * vals[j][0] + vals[j][1] * vals[j][1] + vals[j][2] * vals[j][2] +
                      vals[j][3] * vals[j][3];
            }
        }
        float total = kBlockPerRow ? blockSum(ss, scratch) : warpSum(ss);
        float rms = sqrtf(total / static_cast<float>(dim) + eps);
        TOut* dst = out + row * dim;
#pragma unroll
        for (int j = 0; j < kMaxVec; ++j) {
            int64_t i = lane + static_cast<int64_t>(j) * group;
            if (i < nv) {
                float o[4] = {vals[j][0] / rms, vals[j][1] / rms, vals[j][2] / rms, vals[j][3] / rms};
                store4<TOut>(dst + i * 4, o);
            }
        }
    }
}

template <typename T>
__device__ __forceinline__ float toFloat(T v);
template <>
__device__ __forceinline__ float toFloat<float>(float v) { return v; }
template <>
__device__ __forceinline__ float toFloat<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T fromFloat(float v);
template <>
__device__ __forceinline__ float fromFloat<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 fromFloat<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// 16-byte vectors of TIn <-> floats
template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
    static constexpr int kN = 4;
    __device__ static void load(const float* p, float* v) {
        float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
};
template <>
struct Vec16<__nv_bfloat16> {
    static constexpr int kN = 8;
    __device__ static void load(const __nv_bfloat16* p, float* v) {
        uint4 t = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
};
template <typename TOut, int kN>
__device__ __forceinline__ void storeRun(TOut* p, const float* v) {
    if constexpr (sizeof(TOut) == 4) {
#pragma unroll
        for (int i = 0; i < kN; i += 4) *reinterpret_cast<float4*>(p + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    } else if constexpr (kN == 8) {
        uint4 t;
        uint32_t* w = reinterpret_cast<uint32_t*>(&t);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(p) = t;
    } else {
        uint2 t;
        __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]);
        __nv_bfloat162 hi = __floats2bfloat162_rn(v[2], v[3]);
        t.x = *reinterpret_cast<uint32_t*>(&lo);
        t.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = t;
    }
}

// One warp per row; every lane issues all of its 16-byte loads before the reduction, so a row of up to
// 32 * kVecs * 16 bytes is in flight at once and is read exactly once.
template <typename TIn, typename TOut, int kVecs>
__global__ void __launch_bounds__(kThreads)
rmsnormWarpKernel(const TIn* __restrict__ x, TOut* __restrict__ out, int64_t rows, int64_t dim, float eps) {
    constexpr int kN = Vec16<TIn>::kN;
    const int lane = threadIdx.x & 31;
    const int64_t warpsPerGrid = static_cast<int64_t>(gridDim.x) * (kThreads / 32);
    const int64_t nv = dim / kN;
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5); row < rows;
         row += warpsPerGrid) {
        const TIn* src = x + row * dim;
        float vals[kVecs][kN];
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int64_t i = lane + 32 * j;
            if (i < nv) Vec16<TIn>::load(src + i * kN, vals[j]);
        }
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            if (lane + 32 * j < nv) {
#pragma unroll
                for (int e = 0; e < kN; ++e) ss = fmaf(vals[j][e], vals[j][e], ss);
            }
        }
        const float total = warpSum(ss);
        const float rms = sqrtf(total / static_cast<float>(dim) + eps);
        // bf16 results are rounded to 8 bits anyway: one reciprocal per row instead of a division per element;
        // fp32 results keep the reference's x / rms
        const float inv = 1.0f / rms;
        TOut* dst = out + row * dim;
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int64_t i = lane + 32 * j;
            if (i < nv) {
                float o[kN];
#pragma unroll
                for (int e = 0; e < kN; ++e) o[e] = sizeof(TOut) == 2 ? vals[j][e] * inv : vals[j][e] / rms;
                storeRun<TOut, kN>(dst + i * kN, o);
            }
        }
    }
}

// The statistic of an rmsnorm alone: out[row] = sum of squares of the row. One warp per row, 16-byte loads.
template <typename TIn, bool kVector>
__global__ void __launch_bounds__(kThreads)
rowSumSquaresKernel(const TIn* __restrict__ x, float* __restrict__ out, int64_t rows, int64_t dim) {
    constexpr int kN = Vec16<TIn>::kN;
    const int lane = threadIdx.x & 31;
    const int64_t warpsPerGrid = static_cast<int64_t>(gridDim.x) * (kThreads / 32);
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5); row < rows;
         row += warpsPerGrid) {
        const TIn* src = x + row * dim;
        float s0 = 0.0f, s1 = 0.0f;
        if constexpr (kVector) {
            const int64_t nv = dim / kN;
            int64_t i = lane;
            for (; i + 32 < nv; i += 64) {   // two loads in flight per lane
                float a[kN], b[kN];
                Vec16<TIn>::load(src + i * kN, a);
                Vec16<TIn>::load(src + (i + 32) * kN, b);
#pragma unroll
                for (int e = 0; e < kN; ++e) {
                    s0 = fmaf(a[e], a[e], s0);
                    s1 = fmaf(b[e], b[e], s1);
                }
            }
            if (i < nv) {
                float a[kN];
                Vec16<TIn>::load(src + i * kN, a);
#pragma unroll
                for (int e = 0; e < kN; ++e) s0 = fmaf(a[e], a[e], s0);
            }
        } else {
            for (int64_t i = lane; i < dim; i += 32) {
                const float v = toFloat<TIn>(src[i]);
                s0 = fmaf(v, v, s0);
            }
        }
        const float total = warpSum(s0 + s1);
        if (lane == 0) out[row] = total;
    }
}

// Rows too long for one warp's registers: four warps share a row, each lane still holds its part in registers
// (read once, 16-byte accesses), and the four partial sums of squares meet in shared memory.
template <typename TIn, typename TOut, int kVecs>
__global__ void __launch_bounds__(kThreads)
rmsnormQuadKernel(const TIn* __restrict__ x, TOut* __restrict__ out, int64_t rows, int64_t dim, float eps) {
    constexpr int kN = Vec16<TIn>::kN;
    constexpr int kGroup = 4;                       // warps per row
    constexpr int kRowsPerBlock = kThreads / 32 / kGroup;
    __shared__ float partial[2][kThreads / 32];     // double-buffered by iteration: one barrier per row
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int group = warp / kGroup;
    const int64_t slot = (warp % kGroup) * 32 + lane;   // position among the 128 lanes of the row
    const int64_t nv = dim / kN;
    int parity = 0;
    // every warp of the block makes the same number of trips, so the barrier below is reached by all
    for (int64_t base = static_cast<int64_t>(blockIdx.x) * kRowsPerBlock; base < rows;
         base += static_cast<int64_t>(gridDim.x) * kRowsPerBlock, parity ^= 1) {
        const int64_t row = base + group;
        const bool active = row < rows;
        const TIn* src = x + row * dim;
        float vals[kVecs][kN];
        float ss = 0.0f;
        if (active) {
#pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                const int64_t i = slot + 128 * j;
                if (i < nv) Vec16<TIn>::load(src + i * kN, vals[j]);
            }
#pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                if (slot + 128 * j < nv) {
#pragma unroll
                    for (int e = 0; e < kN; ++e) ss = fmaf(vals[j][e], vals[j][e], ss);
                }
            }
        }
        const float mine = warpSum(ss);
        if (lane == 0) partial[parity][warp] = mine;
        __syncthreads();
        if (!active) continue;
        float total = 0.0f;
#pragma unroll
        for (int g = 0; g < kGroup; ++g) total += partial[parity][group * kGroup + g];
        const float rms = sqrtf(total / static_cast<float>(dim) + eps);
        const float inv = 1.0f / rms;
        TOut* dst = out + row * dim;
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int64_t i = slot + 128 * j;
            if (i < nv) {
                float o[kN];
#pragma unroll
                for (int e = 0; e < kN; ++e) o[e] = sizeof(TOut) == 2 ? vals[j][e] * inv : vals[j][e] / rms;
                storeRun<TOut, kN>(dst + i * kN, o);
            }
        }
    }
}

// Any dim, two passes over the row (second pass hits L1/L2).
template <typename TIn, typename TOut>
__global__ void rmsnormGenericKernel(const TIn* __restrict__ x, TOut* __restrict__ out, int64_t rows, int64_t dim,
                                     float eps) {
    __shared__ float scratch[32];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const TIn* src = x + row * dim;
        float ss = 0.0f;
        for (int64_t i = threadIdx.x; i < dim; i += blockDim.x) {
            float v = toFloat<TIn>(src[i]);
            ss += v * v;
        }
        float total = blockSum(ss, scratch);
        float rms = sqrtf(total / static_cast<float>(dim) + eps);
        for (int64_t i = threadIdx.x; i < dim; i += blockDim.x) {
            out[row * dim + i] = fromFloat<TOut>(toFloat<TIn>(src[i]) / rms);
        }
    }
}

template <typename TIn, typename TOut>
void rmsnormDispatch(const TIn* x, TOut* out, int64_t rows, int64_t dim, float eps, cudaStream_t stream) {
    bool aligned = (dim % 4 == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                   (reinterpret_cast<uintptr_t>(out) % 16 == 0);
    constexpr int kEpv = 16 / static_cast<int>(sizeof(TIn));  // elements per 16-byte load
    const bool wide = aligned && dim % kEpv == 0 && (dim * sizeof(TOut)) % 16 == 0;
    if (wide && dim <= 32 * 8 * kEpv) {
        // one warp per row, the whole row in flight as 16-byte loads before anything is reduced
        const int vecs = static_cast<int>((dim / kEpv + 31) / 32);
        const int rowsPerBlock = kThreads / 32;
        const int grid = gridFor(rows, rowsPerBlock, 8);
        if (vecs <= 2) rmsnormWarpKernel<TIn, TOut, 2><<<grid, kThreads, 0, stream>>>(x, out, rows, dim, eps);
        else if (vecs <= 4) rmsnormWarpKernel<TIn, TOut, 4><<<grid, kThreads, 0, stream>>>(x, out, rows, dim, eps);
        else rmsnormWarpKernel<TIn, TOut, 8><<<grid, kThreads, 0, stream>>>(x, out, rows, dim, eps);
    } else if (wide && dim <= 128 * 8 * kEpv) {
        const int vecs = static_cast<int>((dim / kEpv + 127) / 128);
        const int rowsPerBlock = kThreads / 32 / 4;
        const int grid = gridFor(rows, rowsPerBlock, 8);
        if (vecs <= 4) rmsnormQuadKernel<TIn, TOut, 4><<<grid, kThreads, 0, stream>>>(x, out, rows, dim, eps);
        else rmsnormQuadKernel<TIn, TOut, 8><<<grid, kThreads, 0, stream>>>(x, out, rows, dim, eps);
    } else if (aligned && dim <= 1024) {
        int rowsPerBlock = kThreads / 32;
        int grid = gridFor(rows, rowsPerBlock, 16);
        rmsnormKernel<TIn, TOut, 8, false><<<grid, kThreads, 0, stream>>>(x, out, rows, dim, eps);
    } else if (aligned && dim <= 8192) {
        int grid = gridFor(rows, 1, 16);
        rmsnormKernel<TIn, TOut, 8, true><<<grid, kThreads, 0, stream>>>(x, out, rows, dim, eps);
    } else {
        int grid = gridFor(rows, 1, 16);
        rmsnormGenericKernel<TIn, TOut><<<grid, kThreads, 0, stream>>>(x, out, rows, dim, eps);
    }
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

// ---- softmax ----------------------------------------------------------------------------------
__global__ void softmaxKernel(const float* __restrict__ x, float* __restrict__ out, int64_t rows, int64_t cols) {
    __shared__ float scratch[32];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float* src = x + row * cols;
        float mx = -INFINITY;
        for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) mx = fmaxf(mx, src[i]);
        mx = blockMax(mx, scratch);
        float sum = 0.0f;
        for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) sum += expf(src[i] - mx);
        sum = blockSum(sum, scratch);
        for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) out[row * cols + i] = expf(src[i] - mx) / sum;
    }
}

// ---- elementwise ------------------------------------------------------------------------------
__device__ __forceinline__ float siluF(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float geluF(float x) {
    float inner = 0.7978845608f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.0f + tanhf(inner));
}

template <int kOp>
__global__ void elementwiseKernel(const float* __restrict__ a, const float* __restrict__ b,
                                  const float* __restrict__ c, float* __restrict__ out, int64_t n, int64_t cols) {
    int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        float v = a[i];
        if constexpr (kOp == BFB_EW_ADD) v = v + b[i];
        if constexpr (kOp == BFB_EW_ADD_BIAS) v = v + b[i % cols];
        if constexpr (kOp == BFB_EW_ADD_BIAS_SILU) v = siluF(v + b[i % cols]);
        if constexpr (kOp == BFB_EW_ADD_BIAS_RESIDUAL) v = v + b[i % cols] + c[i];
        if constexpr (kOp == BFB_EW_SILU) v = siluF(v);
        if constexpr (kOp == BFB_EW_RELU) v = v > 0.0f ? v : 0.0f;
        if constexpr (kOp == BFB_EW_GELU) v = geluF(v);
        out[i] = v;
    }
}

__global__ void roundBf16Kernel(float* x, int64_t n) {
    int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        float v = x[i];
        x[i] = isfinite(v) ? bf16Round(v) : v;
    }
}

// ---- conversion -------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float loadAs(const void* p, int64_t i);
template <>
__device__ __forceinline__ float loadAs<float>(const void* p, int64_t i) { return static_cast<const float*>(p)[i]; }
template <>
__device__ __forceinline__ float loadAs<__nv_bfloat16>(const void* p, int64_t i) {
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}
template <>
__device__ __forceinline__ float loadAs<__nv_fp8_e4m3>(const void* p, int64_t i) {
    return static_cast<float>(static_cast<const __nv_fp8_e4m3*>(p)[i]);
}
template <typename T>
__device__ __forceinline__ void storeAs(void* p, int64_t i, float v);
template <>
__device__ __forceinline__ void storeAs<float>(void* p, int64_t i, float v) { static_cast<float*>(p)[i] = v; }
template <>
__device__ __forceinline__ void storeAs<__nv_bfloat16>(void* p, int64_t i, float v) {
    static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ void storeAs<__nv_fp8_e4m3>(void* p, int64_t i, float v) {
    // saturating round-to-nearest-even conversion (values beyond +-448 clamp)
    static_cast<__nv_fp8_storage_t*>(p)[i] = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

template <typename TIn, typename TOut>
__global__ void castKernel(const void* __restrict__ in, void* __restrict__ out, int64_t n, float scale,
                           const float* __restrict__ dScale) {
    float s = dScale != nullptr ? *dScale : scale;
    int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        storeAs<TOut>(out, i, loadAs<TIn>(in, i) * s);
    }
}

// bf16 -> e4m3, 8 elements per thread (128-bit loads, 64-bit stores): the hot conversion of the fp8 path.
__global__ void castBf16ToFp8Vec(const uint4* __restrict__ in, uint2* __restrict__ out, int64_t nVec, float scale,
                                 const float* __restrict__ dScale) {
    float s = dScale != nullptr ? *dScale : scale;
    int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nVec; i += stride) {
        uint4 raw = in[i];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        uint32_t packed[2] = {0u, 0u};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float2 f = __bfloat1622float2(h[j]);
            __nv_fp8x2_storage_t two = __nv_cvt_float2_to_fp8x2(make_float2(f.x * s, f.y * s), __NV_SATFINITE, __NV_E4M3);
            packed[j >> 1] |= static_cast<uint32_t>(two) << ((j & 1) * 16);
        }
        out[i] = make_uint2(packed[0], packed[1]);
    }
}

template <typename TIn>
__global__ void amaxKernel(const void* __restrict__ in, int64_t n, float* amaxOut) {
    __shared__ float scratch[32];
    float m = 0.0f;
    int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        m = fmaxf(m, fabsf(loadAs<TIn>(in, i)));
    }
    m = blockMax(m, scratch);
    // non-negative floats order like their bit patterns
    if (threadIdx.x == 0) atomicMax(reinterpret_cast<int*>(amaxOut), __float_as_int(m));
}

__global__ void fp8ScaleKernel(const float* amaxIn, float* scales) {
    float a = *amaxIn;
    float s = a > 0.0f ? 448.0f / a : 1.0f;
    scales[0] = s;
    scales[1] = 1.0f / s;
}

__global__ void fp8ActScaleKernel(const float* amaxIn, float* out, const float* weightInverse) {
    float a = *amaxIn;
    float s = a > 0.0f ? 448.0f / a : 1.0f;
    out[0] = s;
    out[1] = 1.0f / s;
    out[2] = (1.0f / s) * (*weightInverse);
}

// Seeded N(0, sigma) fill of a [rows, colsLocal] block of a [*, colsFull] tensor. Every value is a pure
// function of (seed, position in the FULL tensor), so tensor-parallel ranks that fill only their slice agree
// with a rank that fills everything.
__global__ void fillNormalKernel(float* __restrict__ out, int64_t rows, int64_t colsLocal, int64_t colsFull,
                                 int64_t rowOffset, int64_t colOffset, uint64_t seed, float sigma) {
    const int64_t total = rows * colsLocal;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t r = i / colsLocal, c = i - r * colsLocal;
        uint64_t z = seed * 0x9E3779B97F4A7C15ull + static_cast<uint64_t>((r + rowOffset) * colsFull + c + colOffset);
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;  // splitmix64 finaliser
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z ^= z >> 31;
        const float u1 = (static_cast<float>(static_cast<uint32_t>(z >> 32)) + 1.0f) * 2.3283064e-10f;  // (0, 1]
        const float u2 = static_cast<float>(static_cast<uint32_t>(z)) * 2.3283064e-10f;
        out[i] = sigma * sqrtf(-2.0f * __logf(u1)) * __cosf(6.2831853f * u2);
    }
}

// W[K,N] f32 -> W^T[N,K] in TOut, through a padded 32x32 shared tile.
template <typename TOut>
__global__ void transposeCastKernel(const float* __restrict__ w, void* __restrict__ out, int64_t k, int64_t n,
                                    float scale, const float* __restrict__ dScale) {
    __shared__ float tile[32][33];
    float s = dScale != nullptr ? *dScale : scale;
    int64_t tilesN = (n + 31) / 32;
    int64_t tilesK = (k + 31) / 32;
    for (int64_t t = blockIdx.x; t < tilesN * tilesK; t += gridDim.x) {
        int64_t tk = t / tilesN, tn = t % tilesN;
        __syncthreads();
        for (int r = threadIdx.y; r < 32; r += blockDim.y) {
            int64_t kk = tk * 32 + r, nn = tn * 32 + threadIdx.x;
            tile[r][threadIdx.x] = (kk < k && nn < n) ? w[kk * n + nn] : 0.0f;
        }
        __syncthreads();
        for (int r = threadIdx.y; r < 32; r += blockDim.y) {
            int64_t nn = tn * 32 + r, kk = tk * 32 + threadIdx.x;
            if (nn < n && kk < k) storeAs<TOut>(out, nn * k + kk, tile[threadIdx.x][r] * s);
        }
    }
}

// in [rows, cols] f32 -> bf16 copies in one pass over `in`: plain [rows, cols] (optional) and transposed [cols, rows].
// 64 x 64 tiles through shared memory; 16-byte reads, 8-byte plain and 16-byte transposed writes, so every access is
// whole sectors. rows % 8 == 0 and cols % 4 == 0 (the caller falls back to the scalar kernels otherwise).
constexpr int kPairTile = 64;
__global__ void __launch_bounds__(256)
castPairKernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ plain, __nv_bfloat16* __restrict__ transposed,
               int64_t rows, int64_t cols) {
    __shared__ __nv_bfloat16 tile[kPairTile][kPairTile + 2];
    const int64_t tilesC = (cols + kPairTile - 1) / kPairTile;
    const int64_t tilesR = (rows + kPairTile - 1) / kPairTile;
    for (int64_t t = blockIdx.x; t < tilesR * tilesC; t += gridDim.x) {
        const int64_t r0 = (t / tilesC) * kPairTile, c0 = (t % tilesC) * kPairTile;
        __syncthreads();
        // 64 rows x 16 float4: thread -> (row = i / 16, four columns at (i % 16) * 4)
#pragma unroll
        for (int i = threadIdx.x; i < kPairTile * 16; i += 256) {
            const int r = i >> 4, c = (i & 15) * 4;
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (r0 + r < rows && c0 + c < cols) v = *reinterpret_cast<const float4*>(in + (r0 + r) * cols + c0 + c);
            const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
            *reinterpret_cast<__nv_bfloat162*>(&tile[r][c]) = lo;
            *reinterpret_cast<__nv_bfloat162*>(&tile[r][c + 2]) = hi;
            if (plain != nullptr && r0 + r < rows && c0 + c < cols) {
                uint2 packed;
                packed.x = *reinterpret_cast<const uint32_t*>(&lo);
                packed.y = *reinterpret_cast<const uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(plain + (r0 + r) * cols + c0 + c) = packed;
            }
        }
        __syncthreads();
        // 32 pairs of output rows (input columns c, c + 1) x 8 pieces of 8 input rows: one 32-bit read serves both rows
        {
            const int i = threadIdx.x;
            const int c = (i >> 3) * 2, r = (i & 7) * 8;
            if (c0 + c < cols && r0 + r < rows) {
                uint32_t lo[4], hi[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t a = *reinterpret_cast<const uint32_t*>(&tile[r + 2 * j][c]);       // (c, c + 1) of row r + 2j
                    const uint32_t b = *reinterpret_cast<const uint32_t*>(&tile[r + 2 * j + 1][c]);
                    lo[j] = __byte_perm(a, b, 0x5410);   // column c of both rows
                    hi[j] = __byte_perm(a, b, 0x7632);   // column c + 1
                }
                *reinterpret_cast<uint4*>(transposed + (c0 + c) * rows + r0 + r) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                if (c0 + c + 1 < cols) {
                    *reinterpret_cast<uint4*>(transposed + (c0 + c + 1) * rows + r0 + r) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                }
            }
        }
    }
}

}  // namespace

// ---- host entry points ------------------------------------------------------------------------

void castPairBf16(const float* in, void* plain, void* transposed, int64_t rows, int64_t cols, cudaStream_t stream) {
    require(rows >= 0 && cols >= 0, "cast_pair: negative size");
    if (rows == 0 || cols == 0) return;
    require(in != nullptr && transposed != nullptr, "cast_pair: null pointer");
    auto aligned = [](const void* p, uintptr_t a) { return reinterpret_cast<uintptr_t>(p) % a == 0; };
    if (rows % 8 == 0 && cols % 4 == 0 && aligned(in, 16) && aligned(transposed, 16) && (plain == nullptr || aligned(plain, 8))) {
        const int64_t tiles = ((rows + kPairTile - 1) / kPairTile) * ((cols + kPairTile - 1) / kPairTile);
        const int grid = static_cast<int>(std::min<int64_t>(tiles, static_cast<int64_t>(smCount()) * 16));
        ProfileScope prof(kProfCast, stream, static_cast<double>(rows) * static_cast<double>(cols) * (plain != nullptr ? 8.0 : 6.0));
        castPairKernel<<<grid, 256, 0, stream>>>(in, static_cast<__nv_bfloat16*>(plain), static_cast<__nv_bfloat16*>(transposed),
                                                 rows, cols);
        BFB_LAUNCH_CHECK();
        noteLaunch();
        return;
    }
    if (plain != nullptr) castScaled(in, BFB_F32, plain, BFB_BF16, rows * cols, 1.0f, nullptr, stream);
    weightPrepare(in, transposed, BFB_BF16, rows, cols, 1.0f, nullptr, stream);
}


void embedPos(const float* ids, const float* table, const float* pos, void* out, int outDtype, int64_t batch,
              int64_t seq, int64_t vocab, int64_t dim, int64_t maxSeq, int64_t posOffset, int* oobCount,
              cudaStream_t stream) {
    require(batch >= 0 && seq >= 0 && vocab > 0 && dim > 0, "embed_pos: sizes must be positive");
    require(outDtype == BFB_F32 || outDtype == BFB_BF16, "embed_pos: output format must be f32 or bf16");
    if (pos != nullptr) require(posOffset >= 0 && posOffset + seq <= maxSeq, "embed_pos: sequence exceeds maxSeqLen");
    int64_t tokens = batch * seq;
    if (tokens == 0) return;
    require(ids != nullptr && table != nullptr && out != nullptr, "embed_pos: null pointer");
    bool vec = dim % 4 == 0 && reinterpret_cast<uintptr_t>(table) % 16 == 0 &&
               reinterpret_cast<uintptr_t>(out) % 16 == 0 && (pos == nullptr || reinterpret_cast<uintptr_t>(pos) % 16 == 0);
    int threads = static_cast<int>(std::min<int64_t>(256, std::max<int64_t>(32, ((vec ? dim / 4 : dim) + 31) / 32 * 32)));
    int grid = gridFor(tokens, 1, 16);
    bool bf = outDtype == BFB_BF16;
    ProfileScope prof(kProfEmbed, stream,
                      static_cast<double>(tokens) * static_cast<double>(dim) * ((pos != nullptr ? 8.0 : 4.0) + (bf ? 2.0 : 4.0)));
#define BFB_EMBED(V, B) \
    embedPosKernel<V, B><<<grid, threads, 0, stream>>>(ids, table, pos, out, tokens, seq, vocab, dim, posOffset, oobCount)
    if (vec && bf) BFB_EMBED(true, true);
    else if (vec) BFB_EMBED(true, false);
    else if (bf) BFB_EMBED(false, true);
    else BFB_EMBED(false, false);
#undef BFB_EMBED
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

void addPositional(const float* in, const float* pos, float* out, int64_t batch, int64_t seq, int64_t dim,
                   int64_t maxSeq, int64_t posOffset, cudaStream_t stream) {
    require(batch >= 0 && seq >= 0 && dim > 0, "add_positional: bad sizes");
    require(posOffset >= 0 && posOffset + seq <= maxSeq, "add_positional: sequence exceeds maxSeqLen");
    int64_t total = batch * seq * dim;
    if (total == 0) return;
    require(in != nullptr && pos != nullptr && out != nullptr, "add_positional: null pointer");
    addPositionalKernel<<<gridFor(total, kThreads), kThreads, 0, stream>>>(in, pos, out, total, seq, dim, posOffset);
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

void rmsnorm(const void* x, int xDtype, void* out, int outDtype, int64_t rows, int64_t dim, float eps,
             cudaStream_t stream) {
    require(rows >= 0 && dim > 0, "rmsnorm: bad sizes");
    require((xDtype == BFB_F32 || xDtype == BFB_BF16) && (outDtype == BFB_F32 || outDtype == BFB_BF16),
            "rmsnorm: formats must be f32 or bf16");
    if (rows == 0) return;
    require(x != nullptr && out != nullptr, "rmsnorm: null pointer");
    using bf = __nv_bfloat16;
    ProfileScope prof(kProfRmsnorm, stream,
                      static_cast<double>(rows) * static_cast<double>(dim) *
                          static_cast<double>(dtypeBytes(xDtype) + dtypeBytes(outDtype)));
    if (xDtype == BFB_F32 && outDtype == BFB_F32)
        rmsnormDispatch(static_cast<const float*>(x), static_cast<float*>(out), rows, dim, eps, stream);
    else if (xDtype == BFB_F32)
        rmsnormDispatch(static_cast<const float*>(x), static_cast<bf*>(out), rows, dim, eps, stream);
    else if (outDtype == BFB_F32)
        rmsnormDispatch(static_cast<const bf*>(x), static_cast<float*>(out), rows, dim, eps, stream);
    else
        rmsnormDispatch(static_cast<const bf*>(x), static_cast<bf*>(out), rows, dim, eps, stream);
}

void rowSumSquares(const void* x, int xDtype, float* out, int64_t rows, int64_t dim, cudaStream_t stream) {
    require(rows >= 0 && dim > 0, "row_sum_squares: bad sizes");
    require(xDtype == BFB_F32 || xDtype == BFB_BF16, "row_sum_squares: format must be f32 or bf16");
    if (rows == 0) return;
    require(x != nullptr && out != nullptr, "row_sum_squares: null pointer");
    ProfileScope prof(kProfRmsnorm, stream,
                      static_cast<double>(rows) * (static_cast<double>(dim) * dtypeBytes(xDtype) + 4.0));
    const int grid = gridFor(rows, kThreads / 32, 16);
    if (xDtype == BFB_F32) {
        const bool vec = dim % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0;
        if (vec) rowSumSquaresKernel<float, true><<<grid, kThreads, 0, stream>>>(static_cast<const float*>(x), out, rows, dim);
        else rowSumSquaresKernel<float, false><<<grid, kThreads, 0, stream>>>(static_cast<const float*>(x), out, rows, dim);
    } else {
        using bf = __nv_bfloat16;
        const bool vec = dim % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0;
        if (vec) rowSumSquaresKernel<bf, true><<<grid, kThreads, 0, stream>>>(static_cast<const bf*>(x), out, rows, dim);
        else rowSumSquaresKernel<bf, false><<<grid, kThreads, 0, stream>>>(static_cast<const bf*>(x), out, rows, dim);
    }
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

// ---- key/value cache append ---------------------------------------------------------------------
// Copies the K and V columns of freshly projected rows ([batch * newLen, ld], K at column kOff, V at vOff, `width`
// columns each) behind the `oldLen` rows every batch entry of the caches ([batch, capRows, width]) already holds.
template <typename V>
__global__ void appendKvKernel(const V* __restrict__ src, int64_t ldV, int64_t kOffV, int64_t vOffV, V* __restrict__ kCache,
                               V* __restrict__ vCache, int64_t batch, int64_t newLen, int64_t widthV, int64_t capRows,
                               int64_t oldLen) {
    if (threadIdx.x == 0) pdl_launch_dependents();
    pdl_wait();   // the new keys and values come from the kernel before; the caches may still be read by it
    const int64_t total = batch * newLen * widthV * 2;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t col = i % widthV;
        int64_t r = i / widthV;
        const int which = static_cast<int>(r & 1);   // 0: K, 1: V
        r >>= 1;
        const int64_t t = r % newLen, b = r / newLen;
        const V value = src[(b * newLen + t) * ldV + (which ? vOffV : kOffV) + col];
        V* dst = which ? vCache : kCache;
        dst[(b * capRows + oldLen + t) * widthV + col] = value;
    }
}

void appendKv(const void* src, int dtype, int64_t ld, int64_t kOffset, int64_t vOffset, void* kCache, void* vCache,
              int64_t batch, int64_t newLen, int64_t width, int64_t capRows, int64_t oldLen, cudaStream_t stream) {
    require(dtype == BFB_F32 || dtype == BFB_BF16, "append_kv: format must be f32 or bf16");
    require(batch >= 0 && newLen >= 0 && width > 0 && oldLen >= 0 && oldLen + newLen <= capRows, "append_kv: bad sizes");
    if (batch == 0 || newLen == 0) return;
    require(src != nullptr && kCache != nullptr && vCache != nullptr, "append_kv: null pointer");
    const int64_t eb = dtypeBytes(dtype);
    auto al16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    const bool vec = (width * eb) % 16 == 0 && (ld * eb) % 16 == 0 && (kOffset * eb) % 16 == 0 && (vOffset * eb) % 16 == 0 &&
                     al16(src) && al16(kCache) && al16(vCache);
    const int64_t per = vec ? 16 / eb : 1;
    const int64_t total = batch * newLen * (width / per) * 2;
    const int grid = static_cast<int>(std::min<int64_t>((total + kThreads - 1) / kThreads, static_cast<int64_t>(smCount()) * 8));
    if (vec) {
        launchDependent(appendKvKernel<uint4>, dim3(static_cast<unsigned>(grid)), dim3(kThreads), 0, stream,
                        static_cast<const uint4*>(src), ld / per, kOffset / per, vOffset / per, static_cast<uint4*>(kCache),
                        static_cast<uint4*>(vCache), batch, newLen, width / per, capRows, oldLen);
    } else if (dtype == BFB_F32) {
        appendKvKernel<float><<<grid, kThreads, 0, stream>>>(static_cast<const float*>(src), ld, kOffset, vOffset,
                                                             static_cast<float*>(kCache), static_cast<float*>(vCache),
                                                             batch, newLen, width, capRows, oldLen);
    } else {
        using bf = __nv_bfloat16;
        appendKvKernel<bf><<<grid, kThreads, 0, stream>>>(static_cast<const bf*>(src), ld, kOffset, vOffset,
                                                          static_cast<bf*>(kCache), static_cast<bf*>(vCache), batch,
                                                          newLen, width, capRows, oldLen);
    }
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

void softmaxRows(const float* x, float* out, int64_t rows, int64_t cols, cudaStream_t stream) {
    require(rows >= 0 && cols > 0, "softmax: bad sizes");
    if (rows == 0) return;
    require(x != nullptr && out != nullptr, "softmax: null pointer");
    softmaxKernel<<<gridFor(rows, 1, 16), kThreads, 0, stream>>>(x, out, rows, cols);
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

void elementwise(int op, const float* a, const float* b, const float* c, float* out, int64_t n, int64_t cols,
                 cudaStream_t stream) {
    require(n >= 0, "elementwise: negative size");
    require(op >= BFB_EW_ADD && op <= BFB_EW_GELU, "elementwise: unknown op");
    if (n == 0) return;
    require(a != nullptr && out != nullptr, "elementwise: null pointer");
    bool needsB = op <= BFB_EW_ADD_BIAS_RESIDUAL;
    if (needsB) require(b != nullptr, "elementwise: second operand missing");
    if (op == BFB_EW_ADD_BIAS || op == BFB_EW_ADD_BIAS_SILU || op == BFB_EW_ADD_BIAS_RESIDUAL)
        require(cols > 0 && n % cols == 0, "elementwise: bias length must divide the element count");
    if (op == BFB_EW_ADD_BIAS_RESIDUAL) require(c != nullptr, "elementwise: residual missing");
    int grid = gridFor(n, kThreads);
    switch (op) {
        case BFB_EW_ADD: elementwiseKernel<BFB_EW_ADD><<<grid, kThreads, 0, stream>>>(a, b, c, out, n, cols); break;
        case BFB_EW_ADD_BIAS: elementwiseKernel<BFB_EW_ADD_BIAS><<<grid, kThreads, 0, stream>>>(a, b, c, out, n, cols); break;
        case BFB_EW_ADD_BIAS_SILU: elementwiseKernel<BFB_EW_ADD_BIAS_SILU><<<grid, kThreads, 0, stream>>>(a, b, c, out, n, cols); break;
        case BFB_EW_ADD_BIAS_RESIDUAL: elementwiseKernel<BFB_EW_ADD_BIAS_RESIDUAL><<<grid, kThreads, 0, stream>>>(a, b, c, out, n, cols); break;
        case BFB_EW_SILU: elementwiseKernel<BFB_EW_SILU><<<grid, kThreads, 0, stream>>>(a, b, c, out, n, cols); break;
        case BFB_EW_RELU: elementwiseKernel<BFB_EW_RELU><<<grid, kThreads, 0, stream>>>(a, b, c, out, n, cols); break;
        default: elementwiseKernel<BFB_EW_GELU><<<grid, kThreads, 0, stream>>>(a, b, c, out, n, cols); break;
    }
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

void roundBf16InPlace(float* x, int64_t n, cudaStream_t stream) {
    if (n <= 0) return;
    roundBf16Kernel<<<gridFor(n, kThreads), kThreads, 0, stream>>>(x, n);
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

void castScaled(const void* in, int inDtype, void* out, int outDtype, int64_t n, float scale, const float* dScale,
                cudaStream_t stream) {
    require(n >= 0, "cast: negative size");
    dtypeBytes(inDtype);
    dtypeBytes(outDtype);
    if (n == 0) return;
    require(in != nullptr && out != nullptr, "cast: null pointer");
    using bf = __nv_bfloat16;
    ProfileScope prof(kProfCast, stream,
                      static_cast<double>(n) * static_cast<double>(dtypeBytes(inDtype) + dtypeBytes(outDtype)));
    using f8 = __nv_fp8_e4m3;
    if (inDtype == BFB_BF16 && outDtype == BFB_FP8_E4M3 && n % 8 == 0 && reinterpret_cast<uintptr_t>(in) % 16 == 0 &&
        reinterpret_cast<uintptr_t>(out) % 8 == 0) {
        int64_t nv = n / 8;
        castBf16ToFp8Vec<<<gridFor(nv, kThreads), kThreads, 0, stream>>>(static_cast<const uint4*>(in),
                                                                          static_cast<uint2*>(out), nv, scale, dScale);
        BFB_LAUNCH_CHECK();
        noteLaunch();
        return;
    }
    int grid = gridFor(n, kThreads);
#define BFB_CAST(TI, TO) castKernel<TI, TO><<<grid, kThreads, 0, stream>>>(in, out, n, scale, dScale)
    int key = inDtype * 3 + outDtype;
    switch (key) {
        case BFB_F32 * 3 + BFB_F32: BFB_CAST(float, float); break;
        case BFB_F32 * 3 + BFB_BF16: BFB_CAST(float, bf); break;
        case BFB_F32 * 3 + BFB_FP8_E4M3: BFB_CAST(float, f8); break;
        case BFB_BF16 * 3 + BFB_F32: BFB_CAST(bf, float); break;
        case BFB_BF16 * 3 + BFB_BF16: BFB_CAST(bf, bf); break;
        case BFB_BF16 * 3 + BFB_FP8_E4M3: BFB_CAST(bf, f8); break;
        case BFB_FP8_E4M3 * 3 + BFB_F32: BFB_CAST(f8, float); break;
        case BFB_FP8_E4M3 * 3 + BFB_BF16: BFB_CAST(f8, bf); break;
        default: BFB_CAST(f8, f8); break;
    }
#undef BFB_CAST
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

void amax(const void* in, int inDtype, int64_t n, float* dAmax, cudaStream_t stream) {
    require(n >= 0, "amax: negative size");
    require(inDtype == BFB_F32 || inDtype == BFB_BF16, "amax: input must be f32 or bf16");
    require(dAmax != nullptr, "amax: null result pointer");
    if (n == 0) return;
    require(in != nullptr, "amax: null pointer");
    int grid = gridFor(n, kThreads * 8, 4);
    if (inDtype == BFB_F32) amaxKernel<float><<<grid, kThreads, 0, stream>>>(in, n, dAmax);
    else amaxKernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(in, n, dAmax);
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

void fp8ScaleFromAmax(const float* dAmax, float* dScales, cudaStream_t stream) {
    require(dAmax != nullptr && dScales != nullptr, "fp8_scale_from_amax: null pointer");
    fp8ScaleKernel<<<1, 1, 0, stream>>>(dAmax, dScales);
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

void fp8ActScale(const float* dAmax, float* out, const float* dWeightInverse, cudaStream_t stream) {
    require(dAmax != nullptr && out != nullptr && dWeightInverse != nullptr, "fp8_act_scale: null pointer");
    fp8ActScaleKernel<<<1, 1, 0, stream>>>(dAmax, out, dWeightInverse);
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

void fillNormal(float* out, int64_t rows, int64_t colsLocal, int64_t colsFull, int64_t rowOffset, int64_t colOffset,
                uint64_t seed, float sigma, cudaStream_t stream) {
    require(rows >= 0 && colsLocal >= 0 && colsFull >= colsLocal, "fill_normal: bad sizes");
    if (rows * colsLocal == 0) return;
    require(out != nullptr, "fill_normal: null pointer");
    fillNormalKernel<<<gridFor(rows * colsLocal, kThreads), kThreads, 0, stream>>>(out, rows, colsLocal, colsFull,
                                                                                  rowOffset, colOffset, seed, sigma);
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

void weightPrepare(const float* w, void* out, int outDtype, int64_t k, int64_t n, float scale, const float* dScale,
                   cudaStream_t stream) {
    require(k > 0 && n > 0, "weight_prepare: bad sizes");
    require(w != nullptr && out != nullptr, "weight_prepare: null pointer");
    dtypeBytes(outDtype);
    int64_t tiles = ((n + 31) / 32) * ((k + 31) / 32);
    int grid = gridFor(tiles, 1, 32);
    dim3 block(32, 8);
    if (outDtype == BFB_F32) transposeCastKernel<float><<<grid, block, 0, stream>>>(w, out, k, n, scale, dScale);
    else if (outDtype == BFB_BF16) transposeCastKernel<__nv_bfloat16><<<grid, block, 0, stream>>>(w, out, k, n, scale, dScale);
    else transposeCastKernel<__nv_fp8_e4m3><<<grid, block, 0, stream>>>(w, out, k, n, scale, dScale);
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

}  // namespace bfb
