// Attention of a generation step: ONE new query per sequence and head (new_len = 1), head_dim 128, bf16, keys and
// values in the caches. Per query and key the arithmetic is 256 FMAs against 512 bytes of K and V, so the kernel is
// laid out for HBM bandwidth and runs on CUDA cores:
//   grid = (batch * heads) x splits; a CTA of 8 warps takes a contiguous range of keys of one (batch, head);
//   a warp takes one key at a time: its 32 lanes read the key's 128 dims as one coalesced 256-byte row (4 dims per
//   lane), the dot product with q is a 5-step shuffle reduction, the probability is the same in every lane, and
//   each lane accumulates its 4 output dims from the value row (again one coalesced row). Keys go in batches of 4
//   per warp; 48 warps per SM hide the latency. Online softmax per warp in log2 units; the 8 warps are merged through shared memory.
// With one split the CTA writes the bf16 output row (and the row statistics); with several, fp32 partial results
// {m, l, acc[128]} go to a workspace and attentionDecodeMergeKernel combines them in split order.
#include <cuda_bf16.h>

#include <algorithm>

#include "common.cuh"
#include "kernels.hpp"
#include "ptx_sm100.cuh"
#include "pool.hpp"

namespace bfb {

namespace {

constexpr int kDecodeDim = 128;
constexpr int kDecodeWarps = 8;
constexpr int kDecodeThreads = kDecodeWarps * 32;
constexpr int kKeysInFlight = 4;
constexpr int kPartialFloats = kDecodeDim + 2;   // m, l, acc[128]

__device__ __forceinline__ float ex2Decode(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {   // the query row
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

struct DecodeParams {
    const __nv_bfloat16* q;
    const __nv_bfloat16* k;
    const __nv_bfloat16* v;
    __nv_bfloat16* out;
    float* mOut;
    float* lOut;
    float* partial;     // [batch * heads][splits][kPartialFloats], or null when splits == 1
    int numHeads, totalLen, splits;
    int64_t ldQ, ldK, ldV, ldO, kvBatchRows;
    float scaleLog2;
};

__global__ void __launch_bounds__(kDecodeThreads, 6)
attentionDecodeKernel(DecodeParams p) {
    if (threadIdx.x == 0) pdl_launch_dependents();
    pdl_wait();   // the query and the newest keys and values come from the kernels before
    __shared__ float merge[kDecodeWarps][kPartialFloats];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int bh = static_cast<int>(blockIdx.x) / p.splits;
    const int split = static_cast<int>(blockIdx.x) - bh * p.splits;
    const int b = bh / p.numHeads, h = bh - b * p.numHeads;
    // this CTA's keys: a contiguous range, multiples of the warp count so the ranges differ by at most 8 keys
    const int perSplit = ((p.totalLen + p.splits - 1) / p.splits + kDecodeWarps - 1) / kDecodeWarps * kDecodeWarps;
    const int k0 = split * perSplit;
    const int k1 = min(p.totalLen, k0 + perSplit);

    float q[4];
    load4(p.q + static_cast<int64_t>(b) * p.ldQ + h * kDecodeDim + lane * 4, q);
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] *= p.scaleLog2;

    const __nv_bfloat16* kBase = p.k + (static_cast<int64_t>(b) * p.kvBatchRows) * p.ldK + h * kDecodeDim + lane * 4;
    const __nv_bfloat16* vBase = p.v + (static_cast<int64_t>(b) * p.kvBatchRows) * p.ldV + h * kDecodeDim + lane * 4;
    float m = -INFINITY, l = 0.0f;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};

    // Keys of this warp: k0 + warp, + 8, + 16, ... in batches of kKeysInFlight whose rows are requested together
    // and whose shuffle reductions run side by side. Latency is hidden by occupancy: the kernel needs 40 registers,
    // so 48 warps fit on an SM, and the host asks for enough key splits to have that many.
    for (int j0 = k0 + warp; j0 < k1; j0 += kDecodeWarps * kKeysInFlight) {
        uint2 kr[kKeysInFlight], vr[kKeysInFlight];
#pragma unroll
        for (int u = 0; u < kKeysInFlight; ++u) {
            const int j = min(j0 + u * kDecodeWarps, k1 - 1);   // a key past the end re-reads the last one, unused
            kr[u] = *reinterpret_cast<const uint2*>(kBase + static_cast<int64_t>(j) * p.ldK);
            vr[u] = *reinterpret_cast<const uint2*>(vBase + static_cast<int64_t>(j) * p.ldV);
        }
        float s[kKeysInFlight];
#pragma unroll
        for (int u = 0; u < kKeysInFlight; ++u) {
            const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&kr[u].x));
            const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&kr[u].y));
            s[u] = fmaf(q[3], c.y, fmaf(q[2], c.x, fmaf(q[1], a.y, q[0] * a.x)));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int u = 0; u < kKeysInFlight; ++u) s[u] += __shfl_xor_sync(0xFFFFFFFFu, s[u], o);
        }
        // the batch's maximum first: one rescale per batch instead of one per key
        float mNew = m;
#pragma unroll
        for (int u = 0; u < kKeysInFlight; ++u) {
            if (j0 + u * kDecodeWarps < k1) mNew = fmaxf(mNew, s[u]);
        }
        if (mNew > m) {   // the same decision in every lane: the sums are complete everywhere
            const float alpha = ex2Decode(m - mNew);
            l *= alpha;
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[i] *= alpha;
            m = mNew;
        }
#pragma unroll
        for (int u = 0; u < kKeysInFlight; ++u) {
            const float pr = (j0 + u * kDecodeWarps < k1) ? ex2Decode(s[u] - m) : 0.0f;
            l += pr;
            const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vr[u].x));
            const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vr[u].y));
            acc[0] = fmaf(pr, a.x, acc[0]);
            acc[1] = fmaf(pr, a.y, acc[1]);
            acc[2] = fmaf(pr, c.x, acc[2]);
            acc[3] = fmaf(pr, c.y, acc[3]);
        }
    }

    // merge the 8 warps: common maximum, rescaled sums
    if (lane == 0) {
        merge[warp][0] = m;
        merge[warp][1] = l;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) merge[warp][2 + lane * 4 + i] = acc[i];
    __syncthreads();
    if (warp != 0) return;
    float mAll = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) mAll = fmaxf(mAll, merge[w][0]);
    float lAll = 0.0f;
    float total[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) {
        const float mw = merge[w][0];
        const float f = mw == -INFINITY ? 0.0f : ex2Decode(mw - mAll);   // a warp without keys contributes nothing
        lAll = fmaf(merge[w][1], f, lAll);
#pragma unroll
        for (int i = 0; i < 4; ++i) total[i] = fmaf(merge[w][2 + lane * 4 + i], f, total[i]);
    }
    if (p.splits == 1) {
        const float inv = lAll > 0.0f ? 1.0f / lAll : 0.0f;
        __nv_bfloat16* dst = p.out + static_cast<int64_t>(b) * p.ldO + h * kDecodeDim + lane * 4;
        const __nv_bfloat162 lo = __floats2bfloat162_rn(total[0] * inv, total[1] * inv);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(total[2] * inv, total[3] * inv);
        uint2 packed;
        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(dst) = packed;
        if (lane == 0) {
            // statistics in natural-log units of the scaled scores, as the other kernels report them
            if (p.mOut != nullptr) p.mOut[bh] = mAll * 0.69314718056f;
            if (p.lOut != nullptr) p.lOut[bh] = lAll;
        }
    } else {
        float* dst = p.partial + (static_cast<int64_t>(bh) * p.splits + split) * kPartialFloats;
        if (lane == 0) {
            dst[0] = mAll;
            dst[1] = lAll;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[2 + lane * 4 + i] = total[i];
    }
}

// One warp per (batch, head): adds the splits in index order.
__global__ void attentionDecodeMergeKernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                                           float* __restrict__ mOut, float* __restrict__ lOut, int pairs, int splits,
                                           int numHeads, int64_t ldO) {
    if (threadIdx.x == 0) pdl_launch_dependents();
    pdl_wait();   // the partial results come from the kernel before
    const int lane = threadIdx.x & 31;
    const int bh = static_cast<int>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (bh >= pairs) return;
    const float* src = partial + static_cast<int64_t>(bh) * splits * kPartialFloats;
    float mAll = -INFINITY;
    for (int s = 0; s < splits; ++s) mAll = fmaxf(mAll, src[s * kPartialFloats]);
    float lAll = 0.0f;
    float total[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int s = 0; s < splits; ++s) {
        const float* ps = src + s * kPartialFloats;
        const float f = ps[0] == -INFINITY ? 0.0f : ex2Decode(ps[0] - mAll);
        lAll = fmaf(ps[1], f, lAll);
#pragma unroll
        for (int i = 0; i < 4; ++i) total[i] = fmaf(ps[2 + lane * 4 + i], f, total[i]);
    }
    const float inv = lAll > 0.0f ? 1.0f / lAll : 0.0f;
    const int b = bh / numHeads, h = bh - b * numHeads;
    __nv_bfloat16* dst = out + static_cast<int64_t>(b) * ldO + h * kDecodeDim + lane * 4;
    const __nv_bfloat162 lo = __floats2bfloat162_rn(total[0] * inv, total[1] * inv);
    const __nv_bfloat162 hi = __floats2bfloat162_rn(total[2] * inv, total[3] * inv);
    uint2 packed;
    packed.x = *reinterpret_cast<const uint32_t*>(&lo);
    packed.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = packed;
    if (lane == 0) {
        if (mOut != nullptr) mOut[bh] = mAll * 0.69314718056f;
        if (lOut != nullptr) lOut[bh] = lAll;
    }
}

}  // namespace

bool attentionDecodeEligible(const AttentionArgs& a) {
    if (a.dtype != BFB_BF16 || a.headDim != kDecodeDim || a.newLen != 1 || a.totalLen < 1) return false;
    if (a.ldQ % 4 || a.ldK % 4 || a.ldV % 4 || a.ldO % 4) return false;
    auto aligned8 = [](const void* ptr) { return reinterpret_cast<uintptr_t>(ptr) % 8 == 0; };
    if (!aligned8(a.q) || !aligned8(a.k) || !aligned8(a.v) || !aligned8(a.out)) return false;
    // the one query sees every key whether or not the mask is on: old_len + 1 == total_len
    if (a.causal && a.oldLen + 1 != a.totalLen) return false;
    return a.batch * a.numHeads <= 0x7FFFFF && a.totalLen <= 0x3FFFFFFF;
}

void attentionDecode(const AttentionArgs& a, cudaStream_t stream) {
    require(attentionDecodeEligible(a), "attention: the one-query kernel needs new_len 1, head_dim 128 and bf16 data");
    const int pairs = static_cast<int>(a.batch * a.numHeads);
    // Six CTAs (48 warps) fit on an SM. The keys are split until the grid is several times that, so that the last,
    // partly filled round of CTAs costs little; a split is worth at least 128 keys.
    const int wanted = (smCount() * 6 * 8 + pairs - 1) / pairs;
    const int splits = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(std::min(wanted, 32), a.totalLen / 128)));
    DecodeParams p;
    p.q = static_cast<const __nv_bfloat16*>(a.q);
    p.k = static_cast<const __nv_bfloat16*>(a.k);
    p.v = static_cast<const __nv_bfloat16*>(a.v);
    p.out = static_cast<__nv_bfloat16*>(a.out);
    p.mOut = a.m;
    p.lOut = a.l;
    p.numHeads = static_cast<int>(a.numHeads);
    p.totalLen = static_cast<int>(a.totalLen);
    p.splits = splits;
    p.ldQ = a.ldQ;
    p.ldK = a.ldK;
    p.ldV = a.ldV;
    p.ldO = a.ldO;
    p.kvBatchRows = a.kvBatchRows > 0 ? a.kvBatchRows : a.totalLen;
    p.scaleLog2 = a.scale * 1.4426950408889634f;
    const size_t wsBytes = splits > 1 ? static_cast<size_t>(pairs) * splits * kPartialFloats * sizeof(float) : 0;
    p.partial = splits > 1 ? static_cast<float*>(poolAcquire(wsBytes)) : nullptr;
    try {
        // the work figure of this kernel is the bytes of K and V it streams; the FLOP figure keeps the shared counter's unit
        ProfileScope prof(kProfAttnTc, stream, 4.0 * kDecodeDim * static_cast<double>(a.totalLen) * pairs);
        launchDependent(attentionDecodeKernel, dim3(static_cast<unsigned>(pairs * splits)), dim3(kDecodeThreads), 0, stream, p);
        BFB_LAUNCH_CHECK();
        noteLaunch();
        if (splits > 1) {
            launchDependent(attentionDecodeMergeKernel, dim3(static_cast<unsigned>((pairs + 7) / 8)), dim3(256), 0, stream,
                            p.partial, p.out, p.mOut, p.lOut, pairs, splits, p.numHeads, p.ldO);
            BFB_LAUNCH_CHECK();
            noteLaunch();
        }
    } catch (...) {
        if (p.partial != nullptr) poolRelease(p.partial, wsBytes);
        throw;
    }
    // work on `stream` is ordered before any later use of the buffer on the same stream
    if (p.partial != nullptr) poolRelease(p.partial, wsBytes);
}

}  // namespace bfb
