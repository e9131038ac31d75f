// tcgen05 flash attention for sm_100a: head_dim 128, bf16 operands, fp32 online softmax, causal
// (with a cache offset) or bidirectional. No score matrix is ever written to global memory.
//
// Persistent CTAs (one per SM) walk a list of work items; an item is a block of 256 query rows of one
// (batch, head), handled as two 128-row tiles, side A and side B, that share every K and V tile. Roles:
//   warps 0-3   softmax of side A, warps 4-7 softmax of side B: ONE thread per query row and no exchange between
//               threads. A thread reads its row of S (128 scores) from tensor memory, exponentiates against the
//               reference it carries over from the tile before (taking the tile's maximum on the way, on another
//               pipe), and writes the probabilities back as bf16 INTO TENSOR MEMORY over the scores (two keys per
//               32-bit column). The two sides are independent, so while one waits for its next scores the other
//               has the scheduler's exp unit to itself. At the end of an item a warp passes its 32 output rows
//               through a small swizzled staging tile in shared memory and a TMA store writes whole lines.
//   warp 8      TMA producer (one elected thread): Q of each item (both sides), K and V tiles (128 keys x 128 dims,
//               two 64-wide swizzled halves each) through a 4-slot ring. It runs ahead into the next item, so the
//               pipeline does not drain between items.
//   warp 9      MMA issuer (one elected thread) + TMEM owner. Per key tile and side: O += P V (P from tensor
//               memory, V from shared memory), then S = Q K^T of that side's NEXT key tile. Tensor-core operations
//               of one thread run in issue order, so the next scores overwrite P only after P V has read it.
//   warps 10-11 idle (they complete the warpgroup whose registers are handed to the softmax warps).
// O stays in tensor memory for the whole item and accumulates across key tiles. The exponent reference of a
// row follows the running maximum lazily: it moves (and O and the row sum are rescaled, and the tile is
// exponentiated again) only when the maximum has grown by more than 8 in log2 units, so probabilities stay below
// 2^8 and almost no tile pays for it.
// TMEM columns: S_A [0,128) S_B [128,256) O_A [256,384) O_B [384,512); P of a tile occupies the first 64
// columns of its S region. Key tiles above the causal diagonal are never visited; only tiles that straddle it
// are masked. All mbarrier waits are bounded.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdlib>
#include <map>
#include <mutex>
#include <queue>
#include <tuple>
#include <type_traits>
#include <vector>

#include "common.cuh"
#include "kernels.hpp"
#include "pool.hpp"
#include "ptx_sm100.cuh"

namespace bfb {

namespace {

constexpr int kD = 128;
constexpr int kBM = 128;                    // query rows per side
constexpr int kBN = 128;                    // keys per tile
constexpr int kItemRows = 2 * kBM;
constexpr int kHalfBytes = 128 * 128;       // one 64-wide half of a 128-row tile
constexpr int kTileBytes = 2 * kHalfBytes;  // 32 KiB
constexpr int kKvSlots = 4;
constexpr int kQOff = 0;                    // [2 sides] Q tiles of the current item
constexpr int kKvOff = 2 * kTileBytes;
constexpr int kStageBytes = 32 * 128;            // one softmax warp's 32 rows x 64 output values (bf16), swizzled
constexpr int kStageOff = kKvOff + kKvSlots * kTileBytes;   // [8 softmax warps]
constexpr int kBarOff = kStageOff + 8 * kStageBytes;
constexpr int kSmemBytes = kBarOff + 256;
constexpr int kFirstSoftmaxWarp = 0;
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kThreads = 384;
constexpr int kSoftmaxRegs = 232;           // 384 threads start with 168 registers each; the last warpgroup gives
constexpr int kOtherRegs = 40;              // 128 * (168 - 40), the two softmax warpgroups take 2 * 128 * (232 - 168)
constexpr float kRescaleSlack = 8.0f;       // log2 units the running maximum may lead the exponent reference
constexpr uint32_t kIdescQK = make_idesc(kBM, kBN, 1u, 0u);
constexpr uint32_t kIdescPV = make_idesc(kBM, kD, 1u, 1u);

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float max3f(float a, float b, float c) { return fmaxf(fmaxf(a, b), c); }

// A wait by every lane of a converged warp, with a warp-uniform outcome.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
    return warp_all(mbar_wait(bar, parity, abort_flag, status, code));
}

struct AttnParams {
    __nv_bfloat16* out;
    float* mOut;
    float* lOut;
    int batch, newLen, totalLen, numHeads;
    int64_t ldO;
    float scaleLog2;
    int oldLen, causal, numQBlocks;
    int totalItems;
    const int* schedule;   // [rounds][grid]: the item CTA c takes in round k, or -1
    int rounds;
    float* outMaxima;      // [batch][heads][ceil(newLen / 128)][4]: largest stored magnitude per 32 output rows, or null
};

struct Item {
    int b, h, q0;
    int nKv[2];   // key tiles side A / side B visits (0: the side has no query row)
    int n;        // max of the two
};

__device__ __forceinline__ int keyTiles(const AttnParams& p, int firstRow) {
    if (firstRow >= p.newLen) return 0;
    int lastKey = p.totalLen - 1;
    if (p.causal) lastKey = min(lastKey, p.oldLen + firstRow + kBM - 1);
    return lastKey / kBN + 1;
}

// An item is (batch * heads + head) * numQBlocks + query block.
__device__ __forceinline__ Item decodeItem(const AttnParams& p, int item) {
    const int bh = item / p.numQBlocks;
    const int qb = item - bh * p.numQBlocks;
    Item it;
    it.b = bh / p.numHeads;
    it.h = bh % p.numHeads;
    it.q0 = qb * kItemRows;
    it.nKv[0] = keyTiles(p, it.q0);
    it.nKv[1] = keyTiles(p, it.q0 + kBM);
    it.n = max(it.nKv[0], it.nKv[1]);
    return it;
}

// The k-th item of this CTA, or a value >= totalItems when it has none left: read from the schedule the host made
// for this shape (attentionSchedule below), which balances the CTAs' total work.
__device__ __forceinline__ int itemAtOf(const AttnParams& p, uint32_t k) {
    if (k >= static_cast<uint32_t>(p.rounds)) return p.totalItems;
    const int item = __ldg(p.schedule + static_cast<size_t>(k) * gridDim.x + blockIdx.x);
    return item < 0 ? p.totalItems : item;
}
#define itemAt(k) itemAtOf(p, (k))

__global__ void __launch_bounds__(kThreads, 1)
attentionTcKernel(const __grid_constant__ CUtensorMap tmapQ, const __grid_constant__ CUtensorMap tmapK,
                  const __grid_constant__ CUtensorMap tmapV, const __grid_constant__ CUtensorMap tmapO, AttnParams p,
                  int* status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kBarOff);
    uint64_t* qFull = bars;            // [1]
    uint64_t* qEmpty = bars + 1;       // [1]
    uint64_t* kvFull = bars + 2;       // [kKvSlots]
    uint64_t* kvEmpty = bars + 2 + kKvSlots;
    uint64_t* sFull = bars + 2 + 2 * kKvSlots;   // [2 sides]
    uint64_t* pFull = sFull + 2;       // [2]
    uint64_t* oFull = sFull + 4;       // [2]
    uint64_t* oFree = sFull + 6;       // [2]
    uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(sFull + 8);
    volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);

    // The swizzled tiles need a 1024-byte aligned base; refuse to run otherwise (uniform across the CTA).
    if ((smem_u32(smem) & 1023u) != 0u) {
        if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0, kDevTimeoutOther);
        return;
    }

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(&qFull[0], 1);
        mbar_init(&qEmpty[0], 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sFull[i], 1);
            mbar_init(&pFull[i], 4);   // one arrival per softmax warp of the side
            mbar_init(&oFull[i], 1);
            mbar_init(&oFree[i], 4);
        }
        for (int s = 0; s < kKvSlots; ++s) {
            mbar_init(&kvFull[s], 1);
            mbar_init(&kvEmpty[s], 1);
        }
        *abortFlag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmapQ);
        tma_prefetch_desc(&tmapK);
        tma_prefetch_desc(&tmapV);
        tma_prefetch_desc(&tmapO);
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
        // ---------------- TMA producer (one elected thread): runs ahead across items ----------------
        setmaxnreg_dec<kOtherRegs>();
        if (elect_one()) {
            uint32_t it = 0;     // items taken by this CTA so far
            uint32_t idx = 0;    // K/V tiles loaded so far (K of an item's key tile j, then its V)
            bool alive = true;
            for (int item = itemAt(0); item < p.totalItems && alive; item = itemAt(++it)) {
                const Item w = decodeItem(p, item);
                // Q of the item: its buffer is free once the previous item's last scores have been computed, which
                // is a whole key tile before this item's first scores are issued
                if (!mbar_wait(&qEmpty[0], (it & 1u) ^ 1u, abortFlag, status, kDevTimeoutStageEmpty)) break;
                {
                    uint8_t* dst = smem + kQOff;
                    const int sides = w.nKv[1] > 0 ? 2 : 1;
                    mbar_arrive_expect_tx(&qFull[0], sides * kTileBytes);
                    for (int s = 0; s < sides; ++s) {
                        tma_load_3d(dst + s * kTileBytes, &tmapQ, &qFull[0], w.h * kD, w.q0 + s * kBM, w.b);
                        tma_load_3d(dst + s * kTileBytes + kHalfBytes, &tmapQ, &qFull[0], w.h * kD + 64, w.q0 + s * kBM,
                                    w.b);
                    }
                }
                for (int t = 0; t < 2 * w.n; ++t, ++idx) {
                    const int slot = idx % kKvSlots;
                    const uint32_t use = idx / kKvSlots;
                    if (!mbar_wait(&kvEmpty[slot], (use & 1u) ^ 1u, abortFlag, status, kDevTimeoutStageEmpty)) {
                        alive = false;
                        break;
                    }
                    const int j = t >> 1;
                    const CUtensorMap* map = (t & 1) ? &tmapV : &tmapK;
                    uint8_t* dst = smem + kKvOff + slot * kTileBytes;
                    mbar_arrive_expect_tx(&kvFull[slot], kTileBytes);
                    tma_load_3d(dst, map, &kvFull[slot], w.h * kD, j * kBN, w.b);
                    tma_load_3d(dst + kHalfBytes, map, &kvFull[slot], w.h * kD + 64, j * kBN, w.b);
                }
            }
        }
        __syncwarp();
    } else if (warp == kMmaWarp) {
        // ---------------- MMA issuer (one elected thread) ----------------
        // The role runs on ONE thread chosen by elect.sync (the compiler then keeps the descriptors in uniform
        // registers; a test on the lane index made every instruction of the region several times slower). That
        // thread can run about six tcgen05.mma ahead of the tensor pipe, no further: whatever it does between two
        // batches beyond that is time the pipe stands still, and it shares its scheduler with two softmax warps, so
        // each of its instructions waits for an issue slot. Hence: descriptors are stepped with one integer add per
        // operand; everything that is normally long complete (the K/V tiles, the next item's Q) is checked BEFORE
        // the wait for the probabilities, the one wait that really takes time; a batch of P V is followed by the
        // next scores of the same side without a wait in between; completion is signalled once per side and key
        // tile (sFull, after the scores, which also covers the P V before them) and oFull only after an item's last
        // P V.
        setmaxnreg_dec<kOtherRegs>();
        if (elect_one()) {
            const uint32_t kvLoBase = smem_desc_lo(smem_u32(smem + kKvOff), 0);
            const uint32_t qLoBase = smem_desc_lo(smem_u32(smem + kQOff), 0);
            constexpr uint32_t kHi = smem_desc_hi_sw128(1024);
            uint32_t tilesDone[2] = {0u, 0u};   // P V products issued per side (phase of pFull)
            uint32_t itemsDone[2] = {0u, 0u};   // items whose output the side's softmax warps have taken (phase of oFree)

            auto waitKv = [&](uint32_t idx) -> bool {
                return mbar_wait(&kvFull[idx % kKvSlots], (idx / kKvSlots) & 1u, abortFlag, status, kDevTimeoutTmaFull);
            };
            // S_side = Q_side K^T for the key tile in ring entry kIdx
            auto issueQK = [&](int side, uint32_t kIdx) {
                const uint32_t qLo = qLoBase + side * (kTileBytes >> 4);
                const uint32_t kLo = kvLoBase + (kIdx % kKvSlots) * (kTileBytes >> 4);
                const uint32_t dS = tmemBase + static_cast<uint32_t>(side * kBN);
#pragma unroll
                for (int kk = 0; kk < kD / 16; ++kk) {
                    const uint32_t off = ((kk >> 2) * kHalfBytes + (kk & 3) * 32) >> 4;
                    umma_f16_words(dS, qLo + off, kHi, kLo + off, kHi, kIdescQK, kk > 0 ? 1u : 0u);
                }
                umma_commit(&sFull[side]);
            };
            // O_side (+)= P_side V for the key tile whose V is ring entry vIdx; `first` starts a new item's sum,
            // `last` ends it
            auto issuePV = [&](int side, uint32_t vIdx, bool first, bool last) -> bool {
                if (!mbar_wait(&pFull[side], tilesDone[side] & 1u, abortFlag, status, kDevTimeoutSoftmax)) return false;
                if (first) {
                    // the previous item's output must have left tensor memory
                    if (!mbar_wait(&oFree[side], (itemsDone[side] & 1u) ^ 1u, abortFlag, status, kDevTimeoutAccEmpty))
                        return false;
                    ++itemsDone[side];
                }
                tc_fence_after();
                // P from tensor memory (it sits where S was): 16 keys = 8 packed columns per step. V: keys are rows
                // (MN-major B): 8-key groups 1024 B apart, the two 64-wide halves of head_dim one half-tile apart.
                const uint32_t pTmem = tmemBase + static_cast<uint32_t>(side * kBN);
                const uint32_t dO = tmemBase + 256u + static_cast<uint32_t>(side * kD);
                const uint32_t vLo = kvLoBase + (vIdx % kKvSlots) * (kTileBytes >> 4) + ((kHalfBytes >> 4) << 16);
                const uint32_t accFirst = first ? 0u : 1u;
#pragma unroll
                for (int kk = 0; kk < kBN / 16; ++kk) {
                    umma_f16_ts_words(dO, pTmem + static_cast<uint32_t>(kk * 8), vLo + kk * (2048 >> 4), kHi, kIdescPV,
                                      kk > 0 ? 1u : accFirst);
                }
                if (last) umma_commit(&oFull[side]);
                ++tilesDone[side];
                return true;
            };
            auto waitQ = [&](uint32_t itemNo) -> bool {
                return mbar_wait(&qFull[0], itemNo & 1u, abortFlag, status, kDevTimeoutTmaFull);
            };

            int item = itemAt(0);
            if (item < p.totalItems) {
                uint32_t it = 0;
                uint32_t base = 0;   // ring entry of this item's K(0); K(j) is base + 2j, V(j) is base + 2j + 1
                Item w = decodeItem(p, item);
                bool alive = waitQ(0) && waitKv(0);
                if (alive) {
                    tc_fence_after();
                    issueQK(0, 0);
                    if (w.nKv[1] > 0) issueQK(1, 0);
                    umma_commit(&kvEmpty[0]);
                    if (w.n == 1) umma_commit(&qEmpty[0]);
                }
                while (alive) {
                    // the item that follows, if any: its first scores are issued under this item's last key tile
                    const int nextItem = itemAt(it + 1);
                    const bool haveNextItem = nextItem < p.totalItems;
                    Item nw = w;
                    if (haveNextItem) nw = decodeItem(p, nextItem);
                    const uint32_t nextBase = base + 2u * static_cast<uint32_t>(w.n);

                    for (int j = 0; j < w.n && alive; ++j) {
                        const uint32_t vIdx = base + 2u * j + 1u;
                        // the key tile whose scores are issued in this round
                        const bool inItem = j + 1 < w.n;
                        const bool haveNext = inItem || haveNextItem;
                        const uint32_t kIdx = inItem ? base + 2u * (j + 1) : nextBase;
                        const Item& kw = inItem ? w : nw;
                        const int kj = inItem ? j + 1 : 0;
                        // operands first: V of this key tile, K (and Q) of the next scores
                        if (!waitKv(vIdx)) { alive = false; break; }
                        if (haveNext && ((!inItem && !waitQ(it + 1)) || !waitKv(kIdx))) { alive = false; break; }
#pragma unroll
                        for (int side = 0; side < 2; ++side) {
                            if (j < w.nKv[side]) {
                                if (!issuePV(side, vIdx, j == 0, j == w.nKv[side] - 1)) { alive = false; break; }
                            }
                            if (haveNext && kj < kw.nKv[side]) issueQK(side, kIdx);
                        }
                        if (!alive) break;
                        umma_commit(&kvEmpty[vIdx % kKvSlots]);
                        if (haveNext) {
                            umma_commit(&kvEmpty[kIdx % kKvSlots]);
                            if (kj == kw.n - 1) umma_commit(&qEmpty[0]);   // those were the item's last scores
                        }
                    }
                    if (!alive || !haveNextItem) break;
                    item = nextItem;
                    w = nw;
                    base = nextBase;
                    ++it;
                }
            }
        }
        __syncwarp();
    } else if (warp >= kFirstSoftmaxWarp && warp < kFirstSoftmaxWarp + 8) {
        // ---------------- softmax: one thread per query row ----------------
        setmaxnreg_inc<kSoftmaxRegs>();
        const int side = (warp - kFirstSoftmaxWarp) >> 2;
        const int r = (warp & 3) * 32 + lane;       // query row inside the side's tile
        const uint32_t laneBase = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t sAddr = tmemBase + laneBase + static_cast<uint32_t>(side * kBN);
        const uint32_t oAddr = tmemBase + laneBase + 256u + static_cast<uint32_t>(side * kD);
        uint32_t tiles = 0;                         // key tiles this side has processed (phase of sFull)
        uint32_t sideItems = 0;                     // items this side has finished (phase of oFull)
        bool alive = true;

        for (uint32_t it = 0; alive; ++it) {
            const int item = itemAt(it);
            if (item >= p.totalItems) break;
            const Item w = decodeItem(p, item);
            const int nKv = w.nKv[side];
            if (nKv == 0) continue;
            const int row = w.q0 + side * kBM + r;
            const int qPos = p.oldLen + row;
            const int keyLimit = p.causal ? min(qPos, p.totalLen - 1) : p.totalLen - 1;  // last visible key
            const int firstRowPos = p.oldLen + w.q0 + side * kBM;
            float mRef = -INFINITY;    // exponent reference (log2 units); trails the true maximum by at most the slack
            float mTrue = -INFINITY;   // running maximum
            float lRun = 0.0f;         // row sum relative to mRef

            for (int j = 0; j < nKv; ++j, ++tiles) {
                if (!(warp_wait(&sFull[side], tiles & 1u, abortFlag, status, kDevTimeoutAccFull))) {
                    alive = false;
                    break;
                }
                tc_fence_after();
                uint32_t s[4][32];
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld_32x32(sAddr + static_cast<uint32_t>(c * 32), s[c]);
                tmem_ld_wait();
                const bool needMask = (p.causal && j * kBN + kBN - 1 > firstRowPos) || (j * kBN + kBN > p.totalLen);
                if (needMask) {
#pragma unroll
                    for (int c = 0; c < 4; ++c)
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (j * kBN + c * 32 + i > keyLimit) s[c][i] = 0xFF800000u;  // -inf
                }
                // Exponentials of the tile against the reference `ref` (log2 units), written over S as bf16 pairs (two
                // keys per 32-bit column: the 32 keys of chunk c take 16 columns, the tile the first 64 columns of the S
                // region); returns the row sum. With kTrackMax it also takes the maximum of the raw scores on the way,
                // which costs nothing next to the exponentials (other pipe). Packed fp32 pairs: one FMA / ADD instruction
                // serves two scores. Masked entries hold -inf: ex2(-inf) = 0.
                float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
                auto expPass = [&](float ref, auto trackMax) -> float {
                    constexpr bool kTrackMax = decltype(trackMax)::value;
                    const uint64_t scale2 = pack_f32x2(p.scaleLog2, p.scaleLog2);
                    const uint64_t negRef2 = pack_f32x2(-ref, -ref);
                    uint64_t sumA = pack_f32x2(0.0f, 0.0f), sumB = sumA;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t packed[16];
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            const float s0 = __uint_as_float(s[c][i]), s1 = __uint_as_float(s[c][i + 1]);
                            if (kTrackMax) {
                                if ((i & 6) == 0) m0 = max3f(m0, s0, s1);
                                else if ((i & 6) == 2) m1 = max3f(m1, s0, s1);
                                else if ((i & 6) == 4) m2 = max3f(m2, s0, s1);
                                else m3 = max3f(m3, s0, s1);
                            }
                            const uint64_t arg = fma_f32x2(pack_f32x2(s0, s1), scale2, negRef2);
                            float a0, a1;
                            unpack_f32x2(arg, a0, a1);
                            const float p0 = ex2(a0);
                            const float p1 = ex2(a1);
                            if ((i & 2) == 0) sumA = add_f32x2(sumA, pack_f32x2(p0, p1));
                            else sumB = add_f32x2(sumB, pack_f32x2(p0, p1));
                            __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
                            packed[i >> 1] = *reinterpret_cast<uint32_t*>(&hh);
                        }
                        tmem_st_32x16(sAddr + static_cast<uint32_t>(c * 16), packed);
                    }
                    float sumLo, sumHi;
                    unpack_f32x2(add_f32x2(sumA, sumB), sumLo, sumHi);
                    return sumLo + sumHi;
                };
                float tileSum;
                if (j == 0) {
                    // first key tile of the item: the reference is the tile's own maximum (four independent chains)
#pragma unroll
                    for (int c = 0; c < 4; ++c)
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            m0 = max3f(m0, __uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1]));
                            m1 = max3f(m1, __uint_as_float(s[c][i + 2]), __uint_as_float(s[c][i + 3]));
                            m2 = max3f(m2, __uint_as_float(s[c][i + 4]), __uint_as_float(s[c][i + 5]));
                            m3 = max3f(m3, __uint_as_float(s[c][i + 6]), __uint_as_float(s[c][i + 7]));
                        }
                    mRef = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * p.scaleLog2;
                    mTrue = mRef;
                    // a row with no visible key yet keeps everything at zero instead of producing NaN
                    tileSum = expPass((mRef == -INFINITY) ? 0.0f : mRef, std::false_type{});
                } else {
                    // Later tiles exponentiate against the reference they inherit and find their maximum on the way.
                    // The reference may trail the true maximum by kRescaleSlack, so the probabilities stay below
                    // 2^kRescaleSlack; only when a row's maximum has grown by more than that is the tile done again.
                    tileSum = expPass((mRef == -INFINITY) ? 0.0f : mRef, std::true_type{});
                    const float mTile = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * p.scaleLog2;
                    mTrue = fmaxf(mTrue, mTile);
                    const bool moved = mTile > mRef + kRescaleSlack;
                    if (__any_sync(0xFFFFFFFFu, moved)) {
                        // Rare: bring O and the row sum to the new reference. The previous tile's P V has finished:
                        // these scores were issued after it by the same thread, and sFull reports everything that
                        // thread had issued. The next P V is issued only after this warp reports P below.
                        const float alpha = moved ? ex2(mRef - mTile) : 1.0f;   // 0 when there was no visible key yet
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            uint32_t o[32];
                            tmem_ld_32x32(oAddr + static_cast<uint32_t>(c * 32), o);
                            tmem_ld_wait();
                            uint32_t lo[16], hi[16];
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                lo[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                                hi[i] = __float_as_uint(__uint_as_float(o[i + 16]) * alpha);
                            }
                            tmem_st_32x16(oAddr + static_cast<uint32_t>(c * 32), lo);
                            tmem_st_32x16(oAddr + static_cast<uint32_t>(c * 32 + 16), hi);
                        }
                        lRun *= alpha;
                        if (moved) mRef = mTile;
                        // every lane takes part (the stores to tensor memory are warp-wide); a row that has not
                        // moved gets the values it had
                        tileSum = expPass((mRef == -INFINITY) ? 0.0f : mRef, std::false_type{});
                    }
                }
                lRun += tileSum;
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();               // one arrival per warp: per-thread arrivals on one word serialise
                if (lane == 0) mbar_arrive(&pFull[side]);
            }
            if (!alive) break;

            // The item's output: wait for the last P V, normalise, hand the O region back. Each warp turns its 32
            // rows into bf16 in two halves of 64 values, lays a half out in its own staging tile (128-byte rows, the
            // 16-byte pieces of a row XOR-swizzled by the row so that the stores do not collide on banks: the layout
            // the tensor map expects) and lets the TMA engine write it: whole 128-byte lines, no store instruction
            // per row piece, and rows past the end of the sequence are clipped by the tensor map.
            if (!(warp_wait(&oFull[side], sideItems & 1u, abortFlag, status, kDevTimeoutAccFull))) break;
            ++sideItems;
            tc_fence_after();
            const float inv = lRun > 0.0f ? 1.0f / lRun : 0.0f;
            const bool store = row < p.newLen;
            float rowMax = 0.0f;   // largest |o| of this thread's row (an e4m3 quantisation of the output wants the maximum)
            uint8_t* stage = smem + kStageOff + (warp - kFirstSoftmaxWarp) * kStageBytes;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t o[2][32];
                tmem_ld_32x32(oAddr + static_cast<uint32_t>(h * 64), o[0]);
                tmem_ld_32x32(oAddr + static_cast<uint32_t>(h * 64 + 32), o[1]);
                tmem_ld_wait();
                if (h == 1) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&oFree[side]);
                }
                // the store issued from this tile before must have read it
                if (lane == 0) tma_store_wait_read();
                __syncwarp();
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    uint32_t wd[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int e = (g & 3) * 8 + 2 * i;
                        const float v0 = __uint_as_float(o[g >> 2][e]) * inv, v1 = __uint_as_float(o[g >> 2][e + 1]) * inv;
                        __nv_bfloat162 hh = __floats2bfloat162_rn(v0, v1);
                        wd[i] = *reinterpret_cast<uint32_t*>(&hh);
                        if (p.outMaxima != nullptr) rowMax = fmaxf(rowMax, fmaxf(fabsf(v0), fabsf(v1)));
                    }
                    *reinterpret_cast<uint4*>(stage + lane * 128 + ((g ^ (lane & 7)) << 4)) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    tma_store_3d(&tmapO, stage, w.h * kD + h * 64, w.q0 + side * kBM + (warp & 3) * 32, w.b);
                    tma_store_commit();
                }
            }
            if (p.outMaxima != nullptr) {
                // rounding to bf16 is monotonic: the largest stored magnitude is the rounded largest value
                float v = store ? __bfloat162float(__float2bfloat16_rn(rowMax)) : 0.0f;
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, off));
                const int rowBlocks = (p.newLen + kBM - 1) / kBM;
                const int64_t slot = ((static_cast<int64_t>(w.b) * p.numHeads + w.h) * rowBlocks + (w.q0 / kBM + side)) * 4 + (warp & 3);
                if (lane == 0 && w.q0 + side * kBM < p.newLen) p.outMaxima[slot] = v;
            }
            if (store) {
                const int64_t statIdx = (static_cast<int64_t>(w.b) * p.numHeads + w.h) * p.newLen + row;
                // statistics relative to the true running maximum, in natural-log units of the scaled scores
                if (p.mOut != nullptr) p.mOut[statIdx] = mTrue * 0.69314718056f;
                if (p.lOut != nullptr) p.lOut[statIdx] = (mTrue == -INFINITY) ? 0.0f : lRun * ex2(mRef - mTrue);
            }
        }
        if (lane == 0) tma_store_wait_all();
    } else {
        setmaxnreg_dec<kOtherRegs>();  // idle warps of the last warpgroup
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

// ---- which CTA takes which item, in what order ------------------------------------------------------------------
// Items differ in weight by up to the number of key tiles (a causal query block sees 2 to 2 * blocks key tiles), and
// a launch may hold only a few items per CTA, so a fixed round-robin can leave CTAs idle for a fifth of the kernel
// (measured: 790 to 1015 TFLOP/s on one shape depending on nothing but the order). The order is therefore planned on
// the host, once per shape and grid, and kept on the device:
//   * (batch, head) pairs are taken in groups whose K and V together fit an L2 budget (default 16 MB; the two halves
//     of the 126 MB L2 mirror lines that both dies read): a group's query blocks run close together in time, so K
//     and V come from DRAM about once;
//   * inside a group the heaviest query blocks come first, and every item goes to the CTA with the least work so far
//     (list scheduling: no CTA ends more than one item after the average), each CTA working through its list in order.
// Cost of an item: its key-tile rounds plus a fixed share for Q load, first scores and output (kItemOverhead).
struct ScheduleKey {
    int device, grid, batch, heads, newLen, totalLen, oldLen, causal;
    long long groupBytes;
    bool operator<(const ScheduleKey& o) const {
        return std::tie(device, grid, batch, heads, newLen, totalLen, oldLen, causal, groupBytes) <
               std::tie(o.device, o.grid, o.batch, o.heads, o.newLen, o.totalLen, o.oldLen, o.causal, o.groupBytes);
    }
};
struct ScheduleEntry {
    int* dev = nullptr;
    int rounds = 0;
    std::vector<int> host;   // kept: the asynchronous upload reads it
};
constexpr double kItemOverhead = 1.5;

int hostKeyTiles(const AttentionArgs& a, int64_t firstRow) {
    if (firstRow >= a.newLen) return 0;
    int64_t lastKey = a.totalLen - 1;
    if (a.causal) lastKey = std::min<int64_t>(lastKey, a.oldLen + firstRow + kBM - 1);
    return static_cast<int>(lastKey / kBN + 1);
}

const ScheduleEntry& attentionSchedule(const AttentionArgs& a, int grid, int numQBlocks, cudaStream_t stream) {
    static std::mutex mu;
    static std::map<ScheduleKey, ScheduleEntry> cache;
    static const long long groupBytes = [] {
        const char* e = std::getenv("BFB_ATTN_L2_MB");
        const long long mb = e != nullptr ? std::atoll(e) : 16;
        return std::max<long long>(1, mb) << 20;
    }();
    int device = 0;
    BFB_CUDA(cudaGetDevice(&device));
    const ScheduleKey key{device, grid, static_cast<int>(a.batch), static_cast<int>(a.numHeads), static_cast<int>(a.newLen),
                          static_cast<int>(a.totalLen), static_cast<int>(a.oldLen), a.causal, groupBytes};
    std::lock_guard<std::mutex> lock(mu);
    auto found = cache.find(key);
    if (found != cache.end()) return found->second;
    if (cache.size() >= 512) {
        // many different shapes (a server with free-form prompt lengths): start over; the buffers may still be in use
        BFB_CUDA(cudaDeviceSynchronize());
        for (auto& kv : cache) poolRelease(kv.second.dev, kv.second.host.size() * sizeof(int));
        cache.clear();
    }
    const int bhCount = static_cast<int>(a.batch * a.numHeads);
    std::vector<double> blockCost(static_cast<size_t>(numQBlocks));
    for (int qb = 0; qb < numQBlocks; ++qb) {
        const int64_t q0 = static_cast<int64_t>(qb) * kItemRows;
        blockCost[static_cast<size_t>(qb)] = std::max(hostKeyTiles(a, q0), hostKeyTiles(a, q0 + kBM)) + kItemOverhead;
    }
    std::vector<int> byWeight(static_cast<size_t>(numQBlocks));
    for (int qb = 0; qb < numQBlocks; ++qb) byWeight[static_cast<size_t>(qb)] = qb;
    std::stable_sort(byWeight.begin(), byWeight.end(), [&](int x, int y) { return blockCost[x] > blockCost[y]; });
    const long long kvBytes = 2ll * a.totalLen * kD * 2;
    const int perGroup = static_cast<int>(std::max<long long>(1, std::min<long long>(bhCount, groupBytes / std::max<long long>(kvBytes, 1))));
    // least-loaded CTA first; ties go to the lower index
    using Load = std::pair<double, int>;
    std::priority_queue<Load, std::vector<Load>, std::greater<Load>> loads;
    for (int c = 0; c < grid; ++c) loads.push({0.0, c});
    std::vector<std::vector<int>> lists(static_cast<size_t>(grid));
    for (int g0 = 0; g0 < bhCount; g0 += perGroup) {
        const int g1 = std::min(bhCount, g0 + perGroup);
        for (int qb : byWeight) {
            for (int bh = g0; bh < g1; ++bh) {
                Load l = loads.top();
                loads.pop();
                lists[static_cast<size_t>(l.second)].push_back(bh * numQBlocks + qb);
                l.first += blockCost[static_cast<size_t>(qb)];
                loads.push(l);
            }
        }
    }
    ScheduleEntry e;
    for (const auto& l : lists) e.rounds = std::max<int>(e.rounds, static_cast<int>(l.size()));
    e.host.assign(static_cast<size_t>(e.rounds) * grid, -1);
    for (int c = 0; c < grid; ++c)
        for (size_t k = 0; k < lists[static_cast<size_t>(c)].size(); ++k) e.host[k * grid + c] = lists[static_cast<size_t>(c)][k];
    e.dev = static_cast<int*>(poolAcquire(e.host.size() * sizeof(int)));
    ScheduleEntry& kept = cache[key] = std::move(e);
    BFB_CUDA(cudaMemcpyAsync(kept.dev, kept.host.data(), kept.host.size() * sizeof(int), cudaMemcpyHostToDevice, stream));
    return kept;
}

// `batchRows`: rows from one batch entry to the next (the length itself when densely packed, the capacity for a cache)
void makeMap(TensorMapStorage* out, const void* base, int64_t dim, int64_t len, int64_t batch, int64_t ld,
             int64_t batchRows, uint32_t boxRows = 128u) {
    uint64_t dims[3] = {static_cast<uint64_t>(dim), static_cast<uint64_t>(len), static_cast<uint64_t>(batch)};
    uint64_t strides[2] = {static_cast<uint64_t>(ld) * 2, static_cast<uint64_t>(ld) * 2 * static_cast<uint64_t>(batchRows)};
    uint32_t box[3] = {64u, boxRows, 1u};
    encodeTensorMap(out, base, 2, 3, dims, strides, box);
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

int64_t attentionMaximaCount(const AttentionArgs& a) {
    return a.batch * a.numHeads * ((a.newLen + kBM - 1) / kBM) * 4;
}

void attentionTensorCore(const AttentionArgs& a, cudaStream_t stream) {
    const int64_t dim = a.numHeads * a.headDim;
    TensorMapStorage tq, tk, tv, to;
    const int64_t kvRows = a.kvBatchRows > 0 ? a.kvBatchRows : a.totalLen;
    makeMap(&tq, a.q, dim, a.newLen, a.batch, a.ldQ, a.newLen);
    makeMap(&tk, a.k, dim, a.totalLen, a.batch, a.ldK, kvRows);
    makeMap(&tv, a.v, dim, a.totalLen, a.batch, a.ldV, kvRows);
    makeMap(&to, a.out, dim, a.newLen, a.batch, a.ldO, a.newLen, 32u);
    AttnParams p;
    p.out = static_cast<__nv_bfloat16*>(a.out);
    p.mOut = a.m;
    p.lOut = a.l;
    p.outMaxima = a.outMaxima;
    p.batch = static_cast<int>(a.batch);
    p.newLen = static_cast<int>(a.newLen);
    p.totalLen = static_cast<int>(a.totalLen);
    p.numHeads = static_cast<int>(a.numHeads);
    p.ldO = a.ldO;
    p.scaleLog2 = a.scale * 1.4426950408889634f;
    p.oldLen = static_cast<int>(a.oldLen);
    p.causal = a.causal;
    p.numQBlocks = static_cast<int>((a.newLen + kItemRows - 1) / kItemRows);
    const int64_t items = static_cast<int64_t>(p.numQBlocks) * a.batch * a.numHeads;
    require(items <= 0x7FFFFFFF, "attention: too many query blocks for one launch");
    p.totalItems = static_cast<int>(items);
    const int grid = static_cast<int>(std::min<int64_t>(items, persistentSms()));
    const ScheduleEntry& sched = attentionSchedule(a, grid, p.numQBlocks, stream);
    p.schedule = sched.dev;
    p.rounds = sched.rounds;
    // visible (query, key) pairs per (batch, head): causal rows see old_len + i + 1 keys
    const double nl = static_cast<double>(a.newLen), tl = static_cast<double>(a.totalLen);
    const double pairs = a.causal ? nl * static_cast<double>(a.oldLen) + nl * (nl + 1.0) / 2.0 : nl * tl;
    ProfileScope prof(kProfAttnTc, stream, 4.0 * kD * pairs * static_cast<double>(a.batch * a.numHeads));
    BFB_CUDA(cudaFuncSetAttribute(attentionTcKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    attentionTcKernel<<<static_cast<unsigned>(grid), kThreads, kSmemBytes, stream>>>(
        *reinterpret_cast<const CUtensorMap*>(tq.bytes), *reinterpret_cast<const CUtensorMap*>(tk.bytes),
        *reinterpret_cast<const CUtensorMap*>(tv.bytes), *reinterpret_cast<const CUtensorMap*>(to.bytes), p, a.dStatus);
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

}  // namespace bfb
