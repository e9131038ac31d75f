// CUDA-core online-softmax attention: any head_dim <= 256, f32 or bf16 data. It serves the fp32
// exactness path (tiny models, comparisons against the fp32 CPU backend) and head sizes the tcgen05
// kernel does not specialise. One warp owns one query row; keys stream through in ascending order
// with a running max / sum, so no score matrix is ever written.
#include <cuda_bf16.h>

#include <cmath>

#include "common.cuh"
#include "kernels.hpp"

namespace bfb {

namespace {

constexpr int kMaxPerLane = 8;  // head_dim <= 256
constexpr int kWarpsPerBlock = 8;

template <typename T>
__device__ __forceinline__ float ldf(const T* p);
template <>
__device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T>
__device__ __forceinline__ void stf(T* p, float v);
template <>
__device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
attentionSimtKernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ out,
                    float* __restrict__ mOut, float* __restrict__ lOut, int64_t batch, int64_t newLen,
                    int64_t totalLen, int64_t numHeads, int64_t headDim, int64_t ldQ, int64_t ldK, int64_t ldV,
                    int64_t ldO, float scale, int64_t oldLen, int causal, int64_t kvBatchRows) {
    const int lane = threadIdx.x & 31;
    const int64_t rowsTotal = batch * numHeads * newLen;
    const int64_t warpGlobal = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    const int64_t warpStride = static_cast<int64_t>(gridDim.x) * kWarpsPerBlock;
    const int per = static_cast<int>((headDim + 31) / 32);

    for (int64_t r = warpGlobal; r < rowsTotal; r += warpStride) {
        const int64_t i = r % newLen;
        const int64_t bh = r / newLen;
        const int64_t h = bh % numHeads;
        const int64_t b = bh / numHeads;
        const T* qRow = q + (b * newLen + i) * ldQ + h * headDim;
        float qReg[kMaxPerLane], acc[kMaxPerLane];
#pragma unroll
        for (int e = 0; e < kMaxPerLane; ++e) {
            int64_t d = lane + 32 * e;
            qReg[e] = (e < per && d < headDim) ? ldf<T>(qRow + d) : 0.0f;
            acc[e] = 0.0f;
        }
        float mRun = -INFINITY, lRun = 0.0f;
        int64_t lastKey = causal ? (oldLen + i) : (totalLen - 1);
        if (lastKey > totalLen - 1) lastKey = totalLen - 1;
        for (int64_t j = 0; j <= lastKey; ++j) {
            const T* kRow = k + (b * kvBatchRows + j) * ldK + h * headDim;
            float part = 0.0f;
#pragma unroll
            for (int e = 0; e < kMaxPerLane; ++e) {
                int64_t d = lane + 32 * e;
                if (e < per && d < headDim) part = fmaf(qReg[e], ldf<T>(kRow + d), part);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xFFFFFFFFu, part, o);
            const float score = part * scale;
            const float mNew = fmaxf(mRun, score);
            const float corr = expf(mRun - mNew);
            const float p = expf(score - mNew);
            const T* vRow = v + (b * kvBatchRows + j) * ldV + h * headDim;
#pragma unroll
            for (int e = 0; e < kMaxPerLane; ++e) {
                int64_t d = lane + 32 * e;
                if (e < per && d < headDim) acc[e] = acc[e] * corr + p * ldf<T>(vRow + d);
            }
            lRun = lRun * corr + p;
            mRun = mNew;
        }
        T* oRow = out + (b * newLen + i) * ldO + h * headDim;
#pragma unroll
        for (int e = 0; e < kMaxPerLane; ++e) {
            int64_t d = lane + 32 * e;
            if (e < per && d < headDim) stf<T>(oRow + d, acc[e] / lRun);
        }
        if (lane == 0) {
            if (mOut != nullptr) mOut[(b * numHeads + h) * newLen + i] = mRun;
            if (lOut != nullptr) lOut[(b * numHeads + h) * newLen + i] = lRun;
        }
    }
}

}  // namespace

void attentionForward(const AttentionArgs& a, cudaStream_t stream) {
    require(a.batch >= 0 && a.newLen >= 0 && a.totalLen >= 0, "attention: negative size");
    require(a.numHeads > 0 && a.headDim > 0, "attention: heads and head_dim must be positive");
    require(a.headDim <= 256, "attention: head_dim above 256 is not supported");
    require(a.dtype == BFB_F32 || a.dtype == BFB_BF16, "attention: data must be f32 or bf16");
    const int64_t dim = a.numHeads * a.headDim;
    require(a.ldQ >= dim && a.ldK >= dim && a.ldV >= dim && a.ldO >= dim, "attention: row stride below heads*head_dim");
    require(a.oldLen >= 0 && a.oldLen + a.newLen <= a.totalLen, "attention: old_len + new_len exceeds total_len");
    if (a.batch == 0 || a.newLen == 0) return;
    require(a.totalLen > 0, "attention: no keys");
    require(a.kvBatchRows == 0 || a.kvBatchRows >= a.totalLen, "attention: kv batch stride below total_len");
    const int64_t kvRows = a.kvBatchRows > 0 ? a.kvBatchRows : a.totalLen;
    require(a.q != nullptr && a.k != nullptr && a.v != nullptr && a.out != nullptr, "attention: null pointer");

    const bool tensorCores = !attentionDecodeEligible(a) && attentionUsesTensorCores(a);
    if (a.outMaxima != nullptr && !tensorCores) {
        fail(BFB_UNSUPPORTED, "attention: output maxima come from the tensor-core kernel only (bf16, head_dim 128, more than one query)");
    }
    if (attentionDecodeEligible(a)) {   // one query per sequence: stream K and V, nothing for a 128-row MMA to do
        attentionDecode(a, stream);
        return;
    }
    if (attentionUsesTensorCores(a)) {
        attentionTensorCore(a, stream);
        return;
    }
    const int64_t rows = a.batch * a.numHeads * a.newLen;
    int grid = static_cast<int>(std::min<int64_t>((rows + kWarpsPerBlock - 1) / kWarpsPerBlock,
                                                   static_cast<int64_t>(smCount()) * 32));
    if (a.dtype == BFB_F32) {
        attentionSimtKernel<float><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
            static_cast<const float*>(a.q), static_cast<const float*>(a.k), static_cast<const float*>(a.v),
            static_cast<float*>(a.out), a.m, a.l, a.batch, a.newLen, a.totalLen, a.numHeads, a.headDim, a.ldQ, a.ldK,
            a.ldV, a.ldO, a.scale, a.oldLen, a.causal, kvRows);
    } else {
        using bf = __nv_bfloat16;
        attentionSimtKernel<bf><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
            static_cast<const bf*>(a.q), static_cast<const bf*>(a.k), static_cast<const bf*>(a.v),
            static_cast<bf*>(a.out), a.m, a.l, a.batch, a.newLen, a.totalLen, a.numHeads, a.headDim, a.ldQ, a.ldK,
            a.ldV, a.ldO, a.scale, a.oldLen, a.causal, kvRows);
    }
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

}  // namespace bfb
