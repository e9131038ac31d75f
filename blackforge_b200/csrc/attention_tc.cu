// tcgen05 flash attention for sm_100a: head_dim 128, bf16 operands, fp32 online softmax, causal
// (with a cache offset) or bidirectional. No score matrix is ever written to global memory.
//
// One CTA owns one 128-row query tile of one (batch, head). With kParts softmax threads per query row
// (2 or 4) the roles are:
//   warps 0 .. 4*kParts-1   softmax. Warp w reads TMEM lanes 32*(w%4).. (its 32 query rows) and the
//               128/kParts key columns of part w/4. A thread reads its slice of S once, the parts of a row
//               exchange their maxima through shared memory, the probabilities are written back as bf16 INTO
//               TENSOR MEMORY over the scores they came from (two keys per 32-bit column), and the thread folds
//               its 128/kParts output columns of the previous tile's P V product into registers with one FMA
//               per element (acc = acc * alpha_prev + O_prev). Row sums stay per part and are combined at the end.
//   warp 4*kParts      TMA producer: Q once, then K and V tiles (128 keys x 128 dims, two 64-wide swizzled
//               halves each) through a 4-slot shared-memory ring
//   warp 4*kParts+1    MMA issuer + TMEM owner: S = Q K^T (128x128x16 steps, both operands from shared memory)
//               into one of two S buffers, then O_j = P V with P read from tensor memory and V from shared memory
//               into one of two O buffers; S of the next tile is issued before P of the current one is awaited,
//               so the tensor core works under the softmax
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P_j occupies the first 64 columns of S_j.
// Causal tiles above the diagonal are never visited; only tiles that straddle it are masked. All mbarrier
// waits are bounded.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdlib>

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
constexpr int kBarOff = kKvOff + kKvSlots * kTileBytes;
constexpr int kXchgOff = kBarOff + 256;     // float [2 buffers][kParts][128 rows]
constexpr uint32_t kIdescQK = make_idesc(kBM, kBN, 1u, 0u);
constexpr uint32_t kIdescPV = make_idesc(kBM, kD, 1u, 1u);

template <int kParts>
struct AttnCfg {
    static constexpr int kCols = 128 / kParts;  // key columns (and output columns) per softmax thread
    static constexpr int kSoftmaxWarps = 4 * kParts;
    static constexpr int kSoftmaxThreads = kSoftmaxWarps * 32;
    static constexpr int kThreads = kSoftmaxThreads + 64;
    static constexpr int kSmemBytes = kXchgOff + 2 * kParts * 128 * 4;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// barrier among the softmax warps only (the producer and MMA warps never join it)
template <int kThreads>
__device__ __forceinline__ void softmax_sync() {
    asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory");
}

struct AttnParams {
    __nv_bfloat16* out;
    float* mOut;
    float* lOut;
    int batch, newLen, totalLen, numHeads;
    int64_t ldO;
    float scaleLog2;
    int oldLen, causal, numQTiles;
    int headsPerGroup;  // (batch, head) pairs whose K + V are kept in L2 together
};

template <int kParts>
__global__ void __launch_bounds__(AttnCfg<kParts>::kThreads, 1)
attentionTcKernel(const __grid_constant__ CUtensorMap tmapQ, const __grid_constant__ CUtensorMap tmapK,
                  const __grid_constant__ CUtensorMap tmapV, AttnParams p, int* status) {
    using Cfg = AttnCfg<kParts>;
    constexpr int kCols = Cfg::kCols;
    constexpr int kChunks = kCols / 32;  // 32-column TMEM accesses per thread
    constexpr int kProducerWarp = Cfg::kSoftmaxWarps;
    constexpr int kMmaWarp = Cfg::kSoftmaxWarps + 1;

    extern __shared__ __align__(1024) uint8_t smem[];
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
    volatile int* softmaxStop = abortFlag + 1;  // agreed on at the softmax barrier so all softmax warps leave together
    float* xchg = reinterpret_cast<float*>(smem + kXchgOff);

    // The swizzled tiles need a 1024-byte aligned base; refuse to run otherwise (uniform across the CTA).
    if ((smem_u32(smem) & 1023u) != 0u) {
        if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0, kDevTimeoutOther);
        return;
    }

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // Launch order: (batch, head) pairs are taken in groups whose K and V fit in L2 together; inside a group the
    // heaviest query tiles (most key tiles) go first. All query tiles of a head therefore run close in time and
    // K/V come from DRAM once.
    const int bhCount = p.batch * p.numHeads;
    const int perGroup = p.headsPerGroup * p.numQTiles;
    const int fullGroups = bhCount / p.headsPerGroup;
    int group = static_cast<int>(blockIdx.x) / perGroup;
    int rem = static_cast<int>(blockIdx.x) - group * perGroup;
    int width = p.headsPerGroup;
    if (group >= fullGroups) {
        group = fullGroups;
        rem = static_cast<int>(blockIdx.x) - fullGroups * perGroup;
        width = bhCount - fullGroups * p.headsPerGroup;
    }
    const int qt = p.numQTiles - 1 - rem / width;
    const int bh = group * p.headsPerGroup + rem % width;
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
            mbar_init(&sFree[i], Cfg::kSoftmaxWarps);
            mbar_init(&pFull[i], Cfg::kSoftmaxWarps);
            mbar_init(&oFull[i], 1);
            mbar_init(&oFree[i], Cfg::kSoftmaxWarps);
        }
        *abortFlag = 0;
        *softmaxStop = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmapQ);
        tma_prefetch_desc(&tmapK);
        tma_prefetch_desc(&tmapV);
    }
    if (warp == kMmaWarp) {
        tmem_alloc(tmemSlot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmemBase = *tmemSlot;

    if (warp == kProducerWarp) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            mbar_arrive_expect_tx(qFull, kTileBytes);
            tma_load_3d(smem + kQOff, &tmapQ, qFull, h * kD, q0, b);
            tma_load_3d(smem + kQOff + kHalfBytes, &tmapQ, qFull, h * kD + 64, q0, b);
        }
        __syncwarp();
        for (int idx = 0; idx < 2 * nKv; ++idx) {
            const int slot = idx & (kKvSlots - 1);
            const uint32_t use = static_cast<uint32_t>(idx / kKvSlots);
            if (!warp_all(mbar_wait(&kvEmpty[slot], (use & 1u) ^ 1u, abortFlag, status, kDevTimeoutStageEmpty))) break;
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
    } else if (warp == kMmaWarp) {
        // ---------------- MMA issuer ----------------
        const uint32_t qAddr = smem_u32(smem + kQOff);
        const uint32_t kvAddr = smem_u32(smem + kKvOff);
        auto issueQK = [&](int j) -> bool {  // S[j&1] = Q K(j)^T
            const int idx = 2 * j;
            const int slot = idx & (kKvSlots - 1);
            const uint32_t use = static_cast<uint32_t>(idx / kKvSlots);
            const uint32_t sUse = static_cast<uint32_t>(j >> 1);
            if (!warp_all(mbar_wait(&kvFull[slot], use & 1u, abortFlag, status, kDevTimeoutTmaFull))) return false;
            // the buffer's previous scores were read and replaced by P, and the P V that reads them was issued
            // before this point (tensor-core operations of one thread complete in issue order)
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
                const uint32_t pTmem = tmemBase + static_cast<uint32_t>((j & 1) * kBN);  // P sits where S was
                const uint32_t dO = tmemBase + 256u + static_cast<uint32_t>((j & 1) * kD);
#pragma unroll
                for (int kk = 0; kk < kBN / 16; ++kk) {
                    // P from tensor memory: 16 keys = 8 packed columns per step. V: keys are rows (MN-major B):
                    // 8-key groups 1024 B apart, the two 64-wide halves of head_dim one half-tile apart.
                    umma_f16_ts(dO, pTmem + static_cast<uint32_t>(kk * 8),
                                make_smem_desc_sw128(vAddr + kk * 2048, kHalfBytes, 1024), kIdescPV, kk > 0 ? 1u : 0u);
                }
                umma_commit(&kvEmpty[slot]);
                umma_commit(&oFull[j & 1]);
            }
            __syncwarp();
        }
    } else {
        // ---------------- softmax + accumulation: kParts threads per query row ----------------
        const int quarter = warp & 3;
        const int part = warp >> 2;                 // which kCols key columns / output columns
        const int r = quarter * 32 + lane;          // query row inside the tile
        const uint32_t laneBase = static_cast<uint32_t>(quarter * 32) << 16;
        const int qPos = p.oldLen + q0 + r;
        const int keyLimit = p.causal ? min(qPos, p.totalLen - 1) : p.totalLen - 1;  // last visible key
        float mRun = -INFINITY, lRun = 0.0f, alphaPrev = 0.0f;
        float oAcc[kCols];
#pragma unroll
        for (int i = 0; i < kCols; ++i) oAcc[i] = 0.0f;
        bool alive = true;

        for (int j = 0; j < nKv; ++j) {
            const int buf = j & 1;
            const uint32_t use = static_cast<uint32_t>(j >> 1);
            // An abandoned wait is published and acted on after the next softmax barrier, where all softmax warps
            // see the same flag: they leave the loop in the same iteration and execute the same barrier count.
            if (alive && !warp_all(mbar_wait(&sFull[buf], use & 1u, abortFlag, status, kDevTimeoutAccFull))) {
                alive = false;
                *softmaxStop = 1;
            }
            const uint32_t sAddr = tmemBase + laneBase + static_cast<uint32_t>(buf * kBN + part * kCols);
            const int key0 = j * kBN + part * kCols;
            const bool needMask = (p.causal && j * kBN + kBN - 1 > p.oldLen + q0) || (j * kBN + kBN > p.totalLen);

            // this thread's scores, read once
            uint32_t s[kChunks][32];
            float mx = -INFINITY;
            if (alive) {
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < kChunks; ++c) tmem_ld_32x32(sAddr + static_cast<uint32_t>(c * 32), s[c]);
                tmem_ld_wait();
                if (needMask) {
#pragma unroll
                    for (int c = 0; c < kChunks; ++c)
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (key0 + c * 32 + i > keyLimit) s[c][i] = 0xFF800000u;  // -inf
                }
                // four independent chains instead of one long dependency
                float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                for (int c = 0; c < kChunks; ++c)
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        m0 = fmaxf(m0, __uint_as_float(s[c][i]));
                        m1 = fmaxf(m1, __uint_as_float(s[c][i + 1]));
                        m2 = fmaxf(m2, __uint_as_float(s[c][i + 2]));
                        m3 = fmaxf(m3, __uint_as_float(s[c][i + 3]));
                    }
                mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
            }
            float* slots = xchg + buf * kParts * 128 + r;   // [part][row]
            slots[part * 128] = mx;
            softmax_sync<Cfg::kSoftmaxThreads>();
            if (*softmaxStop != 0) {
                alive = false;
                break;
            }
#pragma unroll
            for (int q = 0; q < kParts; ++q) mx = fmaxf(mx, slots[q * 128]);
            const float mNew = fmaxf(mRun, mx * p.scaleLog2);
            // a row with no visible key yet keeps everything at zero instead of producing NaN
            const float mUse = (mNew == -INFINITY) ? 0.0f : mNew;
            const float alpha = ex2(mRun - mUse);

            // packed fp32 pairs: one FMA / ADD instruction serves two scores
            const uint64_t scale2 = pack_f32x2(p.scaleLog2, p.scaleLog2);
            const uint64_t negMax2 = pack_f32x2(-mUse, -mUse);
            uint64_t sumA = pack_f32x2(0.0f, 0.0f), sumB = sumA;
#pragma unroll
            for (int c = 0; c < kChunks; ++c) {
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    // masked entries hold -inf: ex2(-inf) = 0
                    const uint64_t arg = fma_f32x2(pack_f32x2(__uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1])),
                                                   scale2, negMax2);
                    float a0, a1;
                    unpack_f32x2(arg, a0, a1);
                    const float p0 = ex2(a0);
                    const float p1 = ex2(a1);
                    if ((i & 2) == 0) sumA = add_f32x2(sumA, pack_f32x2(p0, p1));
                    else sumB = add_f32x2(sumB, pack_f32x2(p0, p1));
                    __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
                    packed[i >> 1] = *reinterpret_cast<uint32_t*>(&hh);
                }
                // P replaces S in tensor memory: two bf16 keys per 32-bit column, so 128 keys take the first 64
                // columns of the S buffer and this thread's 32 keys of chunk c take 16 of them
                tmem_st_32x16(tmemBase + laneBase + static_cast<uint32_t>(buf * kBN + (part * kCols + c * 32) / 2), packed);
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();               // one arrival per warp: 256 per-thread arrivals on one word serialise
            if (lane == 0) {
                mbar_arrive(&pFull[buf]);   // P is in place ...
                mbar_arrive(&sFree[buf]);   // ... and S has been consumed: the buffer may be overwritten after P V
            }
            float sumLo, sumHi;
            unpack_f32x2(add_f32x2(sumA, sumB), sumLo, sumHi);
            lRun = lRun * alpha + (sumLo + sumHi);

            // fold the previous tile's P V (relative to the previous maximum) into the accumulator
            if (j > 0) {
                const int pb = (j - 1) & 1;
                const uint32_t pUse = static_cast<uint32_t>((j - 1) >> 1);
                if (warp_all(mbar_wait(&oFull[pb], pUse & 1u, abortFlag, status, kDevTimeoutAccFull))) {
                    tc_fence_after();
                    const uint32_t oAddr = tmemBase + laneBase + 256u + static_cast<uint32_t>(pb * kD + part * kCols);
                    uint32_t o[kChunks][32];
#pragma unroll
                    for (int c = 0; c < kChunks; ++c) tmem_ld_32x32(oAddr + static_cast<uint32_t>(c * 32), o[c]);
                    tmem_ld_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&oFree[pb]);
                    const uint64_t alpha2 = pack_f32x2(alphaPrev, alphaPrev);
#pragma unroll
                    for (int c = 0; c < kChunks; ++c)
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            unpack_f32x2(fma_f32x2(pack_f32x2(oAcc[c * 32 + i], oAcc[c * 32 + i + 1]), alpha2,
                                                   pack_f32x2(__uint_as_float(o[c][i]), __uint_as_float(o[c][i + 1]))),
                                         oAcc[c * 32 + i], oAcc[c * 32 + i + 1]);
                        }
                } else {
                    alive = false;
                    *softmaxStop = 1;
                }
            }
            alphaPrev = alpha;
            mRun = mNew;
        }

        // last tile's product, normalisation and store. Every softmax warp takes part in the two barriers
        // below even after an abandoned wait, so none is left behind.
        bool haveLast = false;
        uint32_t o[kChunks][32];
        if (alive && *softmaxStop == 0) {
            const int pb = (nKv - 1) & 1;
            const uint32_t pUse = static_cast<uint32_t>((nKv - 1) >> 1);
            if (warp_all(mbar_wait(&oFull[pb], pUse & 1u, abortFlag, status, kDevTimeoutAccFull))) {
                tc_fence_after();
                const uint32_t oAddr = tmemBase + laneBase + 256u + static_cast<uint32_t>(pb * kD + part * kCols);
#pragma unroll
                for (int c = 0; c < kChunks; ++c) tmem_ld_32x32(oAddr + static_cast<uint32_t>(c * 32), o[c]);
                tmem_ld_wait();
                haveLast = true;
            }
        }
        softmax_sync<Cfg::kSoftmaxThreads>();  // everyone is done with the maxima of the last tile
        xchg[part * 128 + r] = lRun;
        softmax_sync<Cfg::kSoftmaxThreads>();
        float lTotal = 0.0f;
#pragma unroll
        for (int q = 0; q < kParts; ++q) lTotal += xchg[q * 128 + r];
        if (haveLast) {
            const float inv = lTotal > 0.0f ? 1.0f / lTotal : 0.0f;
            const bool rowOk = q0 + r < p.newLen;
            if (rowOk) {
                __nv_bfloat16* dst = p.out + (static_cast<int64_t>(b) * p.newLen + q0 + r) * p.ldO +
                                     static_cast<int64_t>(h) * kD + part * kCols;
#pragma unroll
                for (int c = 0; c < kChunks; ++c) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint32_t w[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int e = g * 8 + 2 * i;
                            const float a0 = fmaf(oAcc[c * 32 + e], alphaPrev, __uint_as_float(o[c][e])) * inv;
                            const float a1 = fmaf(oAcc[c * 32 + e + 1], alphaPrev, __uint_as_float(o[c][e + 1])) * inv;
                            __nv_bfloat162 hh = __floats2bfloat162_rn(a0, a1);
                            w[i] = *reinterpret_cast<uint32_t*>(&hh);
                        }
                        *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
                if (part == 0) {
                    const int64_t statIdx = (static_cast<int64_t>(b) * p.numHeads + h) * p.newLen + q0 + r;
                    // statistics in natural-log units of the scaled scores, as the reference reports them
                    if (p.mOut != nullptr) p.mOut[statIdx] = mRun * 0.69314718056f;
                    if (p.lOut != nullptr) p.lOut[statIdx] = lTotal;
                }
            }
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
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

// BFB_ATTN_PARTS=2 in the environment selects two softmax threads per row instead of four (A/B measurements).
int softmaxParts() {
    static const int v = [] {
        const char* e = std::getenv("BFB_ATTN_PARTS");
        return (e != nullptr && std::atoi(e) == 2) ? 2 : 4;
    }();
    return v;
}

template <int kParts>
void launchAttention(const TensorMapStorage& tq, const TensorMapStorage& tk, const TensorMapStorage& tv,
                     const AttnParams& p, int64_t grid, int* status, cudaStream_t stream) {
    using Cfg = AttnCfg<kParts>;
    auto kernel = attentionTcKernel<kParts>;
    BFB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    kernel<<<static_cast<unsigned>(grid), Cfg::kThreads, Cfg::kSmemBytes, stream>>>(
        *reinterpret_cast<const CUtensorMap*>(tq.bytes), *reinterpret_cast<const CUtensorMap*>(tk.bytes),
        *reinterpret_cast<const CUtensorMap*>(tv.bytes), p, status);
}

}  // namespace

bool attentionUsesTensorCores(const AttentionArgs& a) {
    if (a.dtype != BFB_BF16 || a.headDim != kD) return false;
    if (a.ldQ % 8 || a.ldK % 8 || a.ldV % 8 || a.ldO % 8) return false;
    auto aligned16 = [](const void* ptr) { return reinterpret_cast<uintptr_t>(ptr) % 16 == 0; };
    if (!aligned16(a.q) || !aligned16(a.k) || !aligned16(a.v) || !aligned16(a.out)) return false;
    if (!(a.scale > 0.0f)) return false;  // masked scores are -inf before scaling
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
    // K + V of one (batch, head): 2 * total_len * 128 * 2 bytes; keep about 64 MB of them live in the 126 MB L2
    const int64_t kvBytes = 2 * a.totalLen * kD * 2;
    p.headsPerGroup = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(a.batch * a.numHeads, (64ll << 20) / kvBytes)));
    const int64_t grid = static_cast<int64_t>(p.numQTiles) * a.batch * a.numHeads;
    require(grid <= 0x7FFFFFFF, "attention: too many query tiles for one launch");
    // visible (query, key) pairs per (batch, head): causal rows see old_len + i + 1 keys
    const double nl = static_cast<double>(a.newLen), tl = static_cast<double>(a.totalLen);
    const double pairs = a.causal ? nl * static_cast<double>(a.oldLen) + nl * (nl + 1.0) / 2.0 : nl * tl;
    ProfileScope prof(kProfAttnTc, stream, 4.0 * kD * pairs * static_cast<double>(a.batch * a.numHeads));
    if (softmaxParts() == 2) launchAttention<2>(tq, tk, tv, p, grid, a.dStatus, stream);
    else launchAttention<4>(tq, tk, tv, p, grid, a.dStatus, stream);
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

}  // namespace bfb
