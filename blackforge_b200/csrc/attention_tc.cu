// tcgen05 flash attention for sm_100a: head_dim 128, bf16 operands, fp32 online softmax, causal
// (with a cache offset) or bidirectional. No score matrix is ever written to global memory.
//
// One CTA owns one 128-row query tile of one (batch, head). Roles:
//   warp 4      TMA producer: Q once, then K and V tiles (128 keys x 128 dims, two 64-wide swizzled
//               halves each) through a 4-slot shared-memory ring
//   warp 5      MMA issuer + TMEM owner: S = Q K^T (128x128x16 steps) into one of two S buffers, then
//               O_j = P V into one of two O buffers; S of the next tile is issued before P of the
//               current one is awaited, so the tensor core works under the softmax
//   warps 0-3   softmax: one thread per query row reads S from TMEM, keeps the running max and sum in
//               fp32 (base-2 exponentials with the scale folded in), writes P as bf16 into a
//               swizzled shared tile for the second MMA, and folds the previous tile's P V product
//               into a register accumulator with the usual rescaling
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512). Causal tiles above the diagonal
// are never visited; only tiles that straddle it are masked. All waits are bounded.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>

#include "common.cuh"
#include "kernels.hpp"
#include "ptx_sm100.cuh"

namespace bfb {

namespace {

constexpr int kD = 128;
constexpr int kBM = 128;
constexpr int kBN = 128;
constexpr int kHalfBytes = 128 * 128;       // one 64-wide half of a 128-row tile
constexpr int kTileBytes = 2 * kHalfBytes;  // 32 KiB
constexpr int kKvSlots = 4;
constexpr int kQOff = 0;
constexpr int kKvOff = kTileBytes;
constexpr int kPOff = kKvOff + kKvSlots * kTileBytes;
constexpr int kBarOff = kPOff + 2 * kTileBytes;
constexpr int kAttnSmemBytes = kBarOff + 256 + 1024;
constexpr int kAttnThreads = 192;
constexpr int kSoftmaxThreads = 128;
constexpr uint32_t kIdescQK = make_idesc(kBM, kBN, 1u, 0u);
constexpr uint32_t kIdescPV = make_idesc(kBM, kD, 1u, 1u);

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct AttnParams {
    __nv_bfloat16* out;
    float* mOut;
    float* lOut;
    int batch, newLen, totalLen, numHeads;
    int64_t ldO;
    float scaleLog2;
    int oldLen, causal, numQTiles;
};

__global__ void __launch_bounds__(kAttnThreads, 1)
attentionTcKernel(const __grid_constant__ CUtensorMap tmapQ, const __grid_constant__ CUtensorMap tmapK,
                  const __grid_constant__ CUtensorMap tmapV, AttnParams p, int* status) {
    extern __shared__ uint8_t smemRaw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kBarOff);
    uint64_t* qFull = bars;            // [1]
    uint64_t* kvFull = bars + 1;       // [4]
    uint64_t* kvEmpty = bars + 5;      // [4]
    uint64_t* sFull = bars + 9;        // [2]
    uint64_t* sFree = bars + 11;       // [2]
    uint64_t* pFull = bars + 13;       // [2]
    uint64_t* oFull = bars + 15;       // [2]
    uint64_t* oFree = bars + 17;       // [2]
    uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(bars + 19);
    volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // heaviest query tiles (most key tiles) are scheduled first
    const int bhCount = p.batch * p.numHeads;
    const int qt = p.numQTiles - 1 - static_cast<int>(blockIdx.x) / bhCount;
    const int bh = static_cast<int>(blockIdx.x) % bhCount;
    const int b = bh / p.numHeads;
    const int h = bh % p.numHeads;
    const int q0 = qt * kBM;
    int lastKey = p.totalLen - 1;
    if (p.causal) lastKey = min(lastKey, p.oldLen + q0 + kBM - 1);
    const int nKv = lastKey / kBN + 1;

    if (threadIdx.x == 0) {
        mbar_init(qFull, 1);
        for (int s = 0; s < kKvSlots; ++s) {
            mbar_init(&kvFull[s], 1);
            mbar_init(&kvEmpty[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sFull[i], 1);
            mbar_init(&sFree[i], kSoftmaxThreads);
            mbar_init(&pFull[i], kSoftmaxThreads);
            mbar_init(&oFull[i], 1);
            mbar_init(&oFree[i], kSoftmaxThreads);
        }
        *abortFlag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmapQ);
        tma_prefetch_desc(&tmapK);
        tma_prefetch_desc(&tmapV);
    }
    if (warp == 5) {
        tmem_alloc(tmemSlot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmemBase = *tmemSlot;

    if (warp == 4) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            mbar_arrive_expect_tx(qFull, kTileBytes);
            tma_load_3d(smem + kQOff, &tmapQ, qFull, h * kD, q0, b);
            tma_load_3d(smem + kQOff + kHalfBytes, &tmapQ, qFull, h * kD + 64, q0, b);
        }
        __syncwarp();
        bool alive = true;
        for (int idx = 0; idx < 2 * nKv && alive; ++idx) {
            const int slot = idx & (kKvSlots - 1);
            const uint32_t use = static_cast<uint32_t>(idx / kKvSlots);
            if (!warp_all(mbar_wait(&kvEmpty[slot], (use & 1u) ^ 1u, abortFlag, status, kDevTimeoutStageEmpty))) {
                alive = false;
                break;
            }
            if (lane == 0) {
                const int j = idx >> 1;
                const CUtensorMap* map = (idx & 1) ? &tmapV : &tmapK;
                uint8_t* dst = smem + kKvOff + slot * kTileBytes;
                mbar_arrive_expect_tx(&kvFull[slot], kTileBytes);
                tma_load_3d(dst, map, &kvFull[slot], h * kD, j * kBN, b);
                tma_load_3d(dst + kHalfBytes, map, &kvFull[slot], h * kD + 64, j * kBN, b);
            }
            __syncwarp();
        }
    } else if (warp == 5) {
        // ---------------- MMA issuer ----------------
        const uint32_t qAddr = smem_u32(smem + kQOff);
        const uint32_t kvAddr = smem_u32(smem + kKvOff);
        const uint32_t pAddr = smem_u32(smem + kPOff);
        auto issueQK = [&](int j) -> bool {  // S[j&1] = Q K(j)^T
            const int idx = 2 * j;
            const int slot = idx & (kKvSlots - 1);
            const uint32_t use = static_cast<uint32_t>(idx / kKvSlots);
            const uint32_t sUse = static_cast<uint32_t>(j >> 1);
            if (!warp_all(mbar_wait(&kvFull[slot], use & 1u, abortFlag, status, kDevTimeoutTmaFull))) return false;
            if (!warp_all(mbar_wait(&sFree[j & 1], (sUse & 1u) ^ 1u, abortFlag, status, kDevTimeoutAccEmpty))) return false;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t kAddr = kvAddr + slot * kTileBytes;
                const uint32_t dS = tmemBase + static_cast<uint32_t>((j & 1) * kBN);
#pragma unroll
                for (int kk = 0; kk < kD / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * kHalfBytes + (kk & 3) * 32;
                    umma_f16(dS, make_smem_desc_sw128(qAddr + off, 0, 1024), make_smem_desc_sw128(kAddr + off, 0, 1024),
                             kIdescQK, kk > 0 ? 1u : 0u);
                }
                umma_commit(&kvEmpty[slot]);
                umma_commit(&sFull[j & 1]);
            }
            __syncwarp();
            return true;
        };
        bool alive = warp_all(mbar_wait(qFull, 0, abortFlag, status, kDevTimeoutTmaFull));
        if (alive) alive = issueQK(0);
        for (int j = 0; j < nKv && alive; ++j) {
            if (j + 1 < nKv) {
                if (!issueQK(j + 1)) break;
            }
            const int idx = 2 * j + 1;
            const int slot = idx & (kKvSlots - 1);
            const uint32_t use = static_cast<uint32_t>(idx / kKvSlots);
            const uint32_t bufUse = static_cast<uint32_t>(j >> 1);
            if (!warp_all(mbar_wait(&pFull[j & 1], bufUse & 1u, abortFlag, status, kDevTimeoutSoftmax))) break;
            if (!warp_all(mbar_wait(&kvFull[slot], use & 1u, abortFlag, status, kDevTimeoutTmaFull))) break;
            if (!warp_all(mbar_wait(&oFree[j & 1], (bufUse & 1u) ^ 1u, abortFlag, status, kDevTimeoutAccEmpty))) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t vAddr = kvAddr + slot * kTileBytes;
                const uint32_t pBuf = pAddr + (j & 1) * kTileBytes;
                const uint32_t dO = tmemBase + 256u + static_cast<uint32_t>((j & 1) * kD);
#pragma unroll
                for (int kk = 0; kk < kBN / 16; ++kk) {
                    // P: K-major over keys (two 64-key halves). V: keys are rows (MN-major B): 8-key groups
                    // 1024 B apart, the two 64-wide halves of head_dim one half-tile apart.
                    const uint32_t pOff = (kk >> 2) * kHalfBytes + (kk & 3) * 32;
                    umma_f16(dO, make_smem_desc_sw128(pBuf + pOff, 0, 1024),
                             make_smem_desc_sw128(vAddr + kk * 2048, kHalfBytes, 1024), kIdescPV, kk > 0 ? 1u : 0u);
                }
                umma_commit(&kvEmpty[slot]);
                umma_commit(&oFull[j & 1]);
            }
            __syncwarp();
        }
    } else {
        // ---------------- softmax + accumulation (one thread per query row) ----------------
        const int r = threadIdx.x;  // 0..127
        const uint32_t laneBase = static_cast<uint32_t>(warp * 32) << 16;
        const int qPos = p.oldLen + q0 + r;
        float mRun = -INFINITY, lRun = 0.0f;
        float oAcc[kD];
#pragma unroll
        for (int i = 0; i < kD; ++i) oAcc[i] = 0.0f;
        bool alive = true;
        uint8_t* pRowBase = smem + kPOff + r * 128;
        const int sw = r & 7;

        for (int j = 0; j < nKv; ++j) {
            const int buf = j & 1;
            const uint32_t use = static_cast<uint32_t>(j >> 1);
            if (!warp_all(mbar_wait(&sFull[buf], use & 1u, abortFlag, status, kDevTimeoutAccFull))) {
                alive = false;
                break;
            }
            tc_fence_after();
            const uint32_t sAddr = tmemBase + laneBase + static_cast<uint32_t>(buf * kBN);
            const int key0 = j * kBN;
            const bool needMask = (p.causal && key0 + kBN - 1 > p.oldLen + q0) || (key0 + kBN > p.totalLen);
            const int keyLimit = p.causal ? min(qPos, p.totalLen - 1) : p.totalLen - 1;  // last visible key

            // pass 1: row maximum
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < kBN / 32; ++c) {
                uint32_t raw[32];
                tmem_ld_32x32(sAddr + static_cast<uint32_t>(c * 32), raw);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float s = __uint_as_float(raw[i]);
                    if (needMask && key0 + c * 32 + i > keyLimit) s = -INFINITY;
                    mx = fmaxf(mx, s);
                }
            }
            const float mNew = fmaxf(mRun, mx * p.scaleLog2);
            // a row with no visible key yet keeps everything at zero instead of producing NaN
            const float mUse = (mNew == -INFINITY) ? 0.0f : mNew;
            const float alpha = ex2(mRun - mUse);

            // pass 2: probabilities -> bf16 tile in shared memory, row sum in fp32
            float rowSum = 0.0f;
            uint8_t* pBuf = pRowBase + buf * kTileBytes;
#pragma unroll
            for (int c = 0; c < kBN / 32; ++c) {
                uint32_t raw[32];
                tmem_ld_32x32(sAddr + static_cast<uint32_t>(c * 32), raw);
                tmem_ld_wait();
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float s0 = __uint_as_float(raw[i]);
                    float s1 = __uint_as_float(raw[i + 1]);
                    float p0 = ex2(fmaf(s0, p.scaleLog2, -mUse));
                    float p1 = ex2(fmaf(s1, p.scaleLog2, -mUse));
                    if (needMask) {
                        if (key0 + c * 32 + i > keyLimit) p0 = 0.0f;
                        if (key0 + c * 32 + i + 1 > keyLimit) p1 = 0.0f;
                    }
                    rowSum += p0 + p1;
                    __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
                    packed[i >> 1] = *reinterpret_cast<uint32_t*>(&hh);
                }
                // 32 keys = four 16-byte chunks; chunk index inside the 128-byte row is XORed with row % 8
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int chunk = c * 4 + g;           // 0..15 over 128 keys
                    const int half = chunk >> 3;           // which 64-key half
                    const int cc = (chunk & 7) ^ sw;
                    *reinterpret_cast<uint4*>(pBuf + half * kHalfBytes + cc * 16) =
                        make_uint4(packed[g * 4], packed[g * 4 + 1], packed[g * 4 + 2], packed[g * 4 + 3]);
                }
            }
            tc_fence_before();
            mbar_arrive(&sFree[buf]);
            fence_proxy_async_smem();
            mbar_arrive(&pFull[buf]);
            lRun = lRun * alpha + rowSum;

            // fold the previous tile's P V into the register accumulator, then rescale to the new max
            if (j > 0) {
                const int pb = (j - 1) & 1;
                const uint32_t pUse = static_cast<uint32_t>((j - 1) >> 1);
                if (!warp_all(mbar_wait(&oFull[pb], pUse & 1u, abortFlag, status, kDevTimeoutAccFull))) {
                    alive = false;
                    break;
                }
                tc_fence_after();
                const uint32_t oAddr = tmemBase + laneBase + 256u + static_cast<uint32_t>(pb * kD);
#pragma unroll
                for (int c = 0; c < kD / 32; ++c) {
                    uint32_t raw[32];
                    tmem_ld_32x32(oAddr + static_cast<uint32_t>(c * 32), raw);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) oAcc[c * 32 + i] = (oAcc[c * 32 + i] + __uint_as_float(raw[i])) * alpha;
                }
                tc_fence_before();
                mbar_arrive(&oFree[pb]);
            }
            mRun = mNew;
        }

        if (alive) {
            const int pb = (nKv - 1) & 1;
            const uint32_t pUse = static_cast<uint32_t>((nKv - 1) >> 1);
            if (warp_all(mbar_wait(&oFull[pb], pUse & 1u, abortFlag, status, kDevTimeoutAccFull))) {
                tc_fence_after();
                const uint32_t oAddr = tmemBase + laneBase + 256u + static_cast<uint32_t>(pb * kD);
                const float inv = lRun > 0.0f ? 1.0f / lRun : 0.0f;
                const bool rowOk = q0 + r < p.newLen;
                __nv_bfloat16* dst =
                    p.out + (static_cast<int64_t>(b) * p.newLen + q0 + r) * p.ldO + static_cast<int64_t>(h) * kD;
#pragma unroll
                for (int c = 0; c < kD / 32; ++c) {
                    uint32_t raw[32];
                    tmem_ld_32x32(oAddr + static_cast<uint32_t>(c * 32), raw);
                    tmem_ld_wait();
                    if (rowOk) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            uint32_t w[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int e = g * 8 + 2 * i;
                                float a0 = (oAcc[c * 32 + e] + __uint_as_float(raw[e])) * inv;
                                float a1 = (oAcc[c * 32 + e + 1] + __uint_as_float(raw[e + 1])) * inv;
                                __nv_bfloat162 hh = __floats2bfloat162_rn(a0, a1);
                                w[i] = *reinterpret_cast<uint32_t*>(&hh);
                            }
                            *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
                if (rowOk) {
                    const int64_t statIdx = (static_cast<int64_t>(b) * p.numHeads + h) * p.newLen + q0 + r;
                    // statistics in natural-log units of the scaled scores, as the reference reports them
                    if (p.mOut != nullptr) p.mOut[statIdx] = mRun * 0.69314718056f;
                    if (p.lOut != nullptr) p.lOut[statIdx] = lRun;
                }
            }
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        if (*abortFlag != 0) {
            uint64_t t0 = global_timer_ns();
            while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
        tc_fence_after();
        tmem_dealloc(tmemBase, 512);
    }
}

void makeMap(TensorMapStorage* out, const void* base, int64_t dim, int64_t len, int64_t batch, int64_t ld) {
    uint64_t dims[3] = {static_cast<uint64_t>(dim), static_cast<uint64_t>(len), static_cast<uint64_t>(batch)};
    uint64_t strides[2] = {static_cast<uint64_t>(ld) * 2, static_cast<uint64_t>(ld) * 2 * static_cast<uint64_t>(len)};
    uint32_t box[3] = {64u, 128u, 1u};
    encodeTensorMap(out, base, 2, 3, dims, strides, box);
}

}  // namespace

bool attentionUsesTensorCores(const AttentionArgs& a) {
    if (a.dtype != BFB_BF16 || a.headDim != kD) return false;
    if (a.ldQ % 8 || a.ldK % 8 || a.ldV % 8 || a.ldO % 8) return false;
    auto aligned16 = [](const void* ptr) { return reinterpret_cast<uintptr_t>(ptr) % 16 == 0; };
    if (!aligned16(a.q) || !aligned16(a.k) || !aligned16(a.v) || !aligned16(a.out)) return false;
    if (a.batch * a.numHeads > 0x3FFFFF || a.totalLen > 0x3FFFFFFF || a.newLen > 0x3FFFFFFF) return false;
    return true;
}

void attentionTensorCore(const AttentionArgs& a, cudaStream_t stream) {
    const int64_t dim = a.numHeads * a.headDim;
    TensorMapStorage tq, tk, tv;
    makeMap(&tq, a.q, dim, a.newLen, a.batch, a.ldQ);
    makeMap(&tk, a.k, dim, a.totalLen, a.batch, a.ldK);
    makeMap(&tv, a.v, dim, a.totalLen, a.batch, a.ldV);
    AttnParams p;
    p.out = static_cast<__nv_bfloat16*>(a.out);
    p.mOut = a.m;
    p.lOut = a.l;
    p.batch = static_cast<int>(a.batch);
    p.newLen = static_cast<int>(a.newLen);
    p.totalLen = static_cast<int>(a.totalLen);
    p.numHeads = static_cast<int>(a.numHeads);
    p.ldO = a.ldO;
    p.scaleLog2 = a.scale * 1.4426950408889634f;
    p.oldLen = static_cast<int>(a.oldLen);
    p.causal = a.causal;
    p.numQTiles = static_cast<int>((a.newLen + kBM - 1) / kBM);
    const int64_t grid = static_cast<int64_t>(p.numQTiles) * a.batch * a.numHeads;
    require(grid <= 0x7FFFFFFF, "attention: too many query tiles for one launch");
    BFB_CUDA(cudaFuncSetAttribute(attentionTcKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmemBytes));
    // visible (query, key) pairs per (batch, head): causal rows see old_len + i + 1 keys
    const double nl = static_cast<double>(a.newLen), tl = static_cast<double>(a.totalLen);
    const double pairs = a.causal ? nl * static_cast<double>(a.oldLen) + nl * (nl + 1.0) / 2.0 : nl * tl;
    ProfileScope prof(kProfAttnTc, stream, 4.0 * kD * pairs * static_cast<double>(a.batch * a.numHeads));
    attentionTcKernel<<<static_cast<unsigned>(grid), kAttnThreads, kAttnSmemBytes, stream>>>(
        *reinterpret_cast<CUtensorMap*>(tq.bytes), *reinterpret_cast<CUtensorMap*>(tk.bytes),
        *reinterpret_cast<CUtensorMap*>(tv.bytes), p, a.dStatus);
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

}  // namespace bfb
