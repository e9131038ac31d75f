// Attention of a generation step: ONE new query per sequence and head (new_len = 1), head_dim 128, bf16, keys and
// values in the caches. Per query and key the arithmetic is 256 FMAs against 512 bytes of K and V, so the kernel is
// laid out for HBM bandwidth and runs on CUDA cores:
//   grid = (batch * heads) x splits; a CTA of 8 warps takes a contiguous range of keys of one (batch, head);
//   a half-warp takes one key at a time: its 16 lanes read the key's 128 dims as one coalesced 256-byte row (8 dims =
//   16 bytes per lane), the dot product with q is a 4-step shuffle reduction, the probability is the same in every
//   lane of the half, and each lane accumulates its 8 output dims from the value row (again one coalesced row). Keys
//   go in batches of 4 per half-warp; 32 warps per SM hide the latency. Online softmax per half-warp in log2 units;
//   the 16 half-warps are merged through shared memory.
// With one split the CTA writes the bf16 output row (and the row statistics); with several, fp32 partial results
// {m, l, acc[128]} go to a workspace and attentionDecodeMergeKernel combines them in split order. (Letting the CTA
// that finishes a (batch, head) last do that merge, behind a fence and a counter, saves the launch but no time: as
// a programmatic dependent the merge launch already overlaps the kernel's tail.)
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
constexpr int kDecodeGroups = kDecodeWarps * 2;   // half-warps: 16 lanes x 8 dims cover one key row
constexpr int kKeysInFlight = 4;
constexpr int kDecodeCtasPerSm = 4;
constexpr int kPartialFloats = kDecodeDim + 2;   // m, l, acc[128]

__device__ __forceinline__ float ex2Decode(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
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

__global__ void __launch_bounds__(kDecodeThreads, kDecodeCtasPerSm)
attentionDecodeKernel(DecodeParams p) {
    if (threadIdx.x == 0) pdl_launch_dependents();
    pdl_wait();   // the query and the newest keys and values come from the kernels before
    __shared__ float merge[kDecodeGroups][kPartialFloats];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int sub = lane & 15;                       // this lane's 8 dims: sub * 8 ...
    const int group = warp * 2 + (lane >> 4);        // the half-warp, which has its own keys and softmax state
    const int bh = static_cast<int>(blockIdx.x) / p.splits;
    const int split = static_cast<int>(blockIdx.x) - bh * p.splits;
    const int b = bh / p.numHeads, h = bh - b * p.numHeads;
    // this CTA's keys: a contiguous range, multiples of the group count so the ranges differ by at most 16 keys
    const int perSplit = ((p.totalLen + p.splits - 1) / p.splits + kDecodeGroups - 1) / kDecodeGroups * kDecodeGroups;
    const int k0 = split * perSplit;
    const int k1 = min(p.totalLen, k0 + perSplit);

    float q[8];
    unpack8(*reinterpret_cast<const uint4*>(p.q + static_cast<int64_t>(b) * p.ldQ + h * kDecodeDim + sub * 8), q);
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] *= p.scaleLog2;

    const __nv_bfloat16* kBase = p.k + (static_cast<int64_t>(b) * p.kvBatchRows) * p.ldK + h * kDecodeDim + sub * 8;
    const __nv_bfloat16* vBase = p.v + (static_cast<int64_t>(b) * p.kvBatchRows) * p.ldV + h * kDecodeDim + sub * 8;
    float m = -INFINITY, l = 0.0f;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;

    // Keys of this half-warp: k0 + group, + 16, + 32, ... in batches of kKeysInFlight whose rows are requested
    // together (16 bytes per lane and row) and whose shuffle reductions run side by side. A warp instruction thus
    // serves two keys, which matters: with one key per warp the kernel was bound by instruction issue (two thirds of
    // the issue slots busy at 56 % of the DRAM rate), not by memory. The loop trip count is the same for both halves
    // of a warp (keys past the end re-read the last one and count for nothing), so the shuffles stay convergent.
    for (int j0 = k0 + group; j0 - (lane >> 4) < k1; j0 += kDecodeGroups * kKeysInFlight) {
        uint4 kr[kKeysInFlight], vr[kKeysInFlight];
#pragma unroll
        for (int u = 0; u < kKeysInFlight; ++u) {
            const int j = max(k0, min(j0 + u * kDecodeGroups, k1 - 1));
            kr[u] = *reinterpret_cast<const uint4*>(kBase + static_cast<int64_t>(j) * p.ldK);
            vr[u] = *reinterpret_cast<const uint4*>(vBase + static_cast<int64_t>(j) * p.ldV);
        }
        float s[kKeysInFlight];
#pragma unroll
        for (int u = 0; u < kKeysInFlight; ++u) {
            float kf[8];
            unpack8(kr[u], kf);
            float d = q[0] * kf[0];
#pragma unroll
            for (int i = 1; i < 8; ++i) d = fmaf(q[i], kf[i], d);
            s[u] = d;
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
#pragma unroll
            for (int u = 0; u < kKeysInFlight; ++u) s[u] += __shfl_xor_sync(0xFFFFFFFFu, s[u], o);
        }
        // the batch's maximum first: one rescale per batch instead of one per key (branch-free: the two halves of
        // the warp decide differently)
        float mNew = m;
#pragma unroll
        for (int u = 0; u < kKeysInFlight; ++u) {
            if (j0 + u * kDecodeGroups < k1) mNew = fmaxf(mNew, s[u]);
        }
        const float alpha = mNew == -INFINITY ? 1.0f : ex2Decode(m - mNew);
        l *= alpha;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] *= alpha;
        m = mNew;
#pragma unroll
        for (int u = 0; u < kKeysInFlight; ++u) {
            const float pr = (j0 + u * kDecodeGroups < k1) ? ex2Decode(s[u] - m) : 0.0f;
            l += pr;
            float vf[8];
            unpack8(vr[u], vf);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(pr, vf[i], acc[i]);
        }
    }

    // merge the 16 half-warps: common maximum, rescaled sums
    if (sub == 0) {
        merge[group][0] = m;
        merge[group][1] = l;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) merge[group][2 + sub * 8 + i] = acc[i];
    __syncthreads();
    if (warp != 0) return;
    float mAll = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecodeGroups; ++w) mAll = fmaxf(mAll, merge[w][0]);
    float lAll = 0.0f;
    float total[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int w = 0; w < kDecodeGroups; ++w) {
        const float mw = merge[w][0];
        const float f = mw == -INFINITY ? 0.0f : ex2Decode(mw - mAll);   // a half-warp without keys contributes nothing
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
    if (a.ldQ % 8 || a.ldK % 8 || a.ldV % 8 || a.ldO % 4) return false;   // 16-byte loads of q, k, v; 8-byte stores
    auto aligned = [](const void* ptr, uintptr_t to) { return reinterpret_cast<uintptr_t>(ptr) % to == 0; };
    if (!aligned(a.q, 16) || !aligned(a.k, 16) || !aligned(a.v, 16) || !aligned(a.out, 8)) return false;
    // the one query sees every key whether or not the mask is on: old_len + 1 == total_len
    if (a.causal && a.oldLen + 1 != a.totalLen) return false;
    return a.batch * a.numHeads <= 0x7FFFFF && a.totalLen <= 0x3FFFFFFF;
}

void attentionDecode(const AttentionArgs& a, cudaStream_t stream) {
    require(attentionDecodeEligible(a), "attention: the one-query kernel needs new_len 1, head_dim 128 and bf16 data");
    const int pairs = static_cast<int>(a.batch * a.numHeads);
    // Four CTAs (32 warps, 64 registers a thread) fit on an SM. The keys are split until the grid is several times that, so that the last,
    // partly filled round of CTAs costs little; a split is worth at least 128 keys.
    const int wanted = (smCount() * kDecodeCtasPerSm * 8 + pairs - 1) / pairs;
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
