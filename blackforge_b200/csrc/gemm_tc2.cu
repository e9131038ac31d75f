// tcgen05 GEMM with CTA pairs (tcgen05.mma.cta_group::2): two CTAs of a cluster share one output tile
// of 256 rows x kAccN columns (kAccN = 256 or 512). Each CTA stages its own 128 rows of A and its half of
// the B^T rows per k-slice and holds the accumulator of its own 128 rows in tensor memory; the leader CTA
// issues every MMA (256 x 256 x 16 each) for both.
//
//   kAccN = 256  32 KiB per stage and CTA, 6-stage ring, two accumulator buffers: the epilogue of one tile
//                runs under the MMAs of the next.
//   kAccN = 512  48 KiB per stage, 4-stage ring, the whole tensor memory is one accumulator (two 256-column
//                halves fed by the same A slice). The epilogue is not hidden, but every byte of A is used for
//                twice as many FLOPs: 25 % fewer bytes come out of L2 per FLOP, which is what bounds the
//                256-wide tile (about 10 TB/s of L2 reads whatever the SM clock).
//
// Synchronisation across the pair:
//   full[s]      lives in the leader; both CTAs' TMA loads book their bytes on it
//   empty[s]     one per CTA; the leader's tcgen05.commit arrives on both
//   accFull[b]   one per CTA; same commit form, tells both epilogues the accumulator is complete
//   accEmpty[b]  lives in the leader; the epilogue threads of both CTAs arrive on it
//   tileFull[r]  one per CTA; the scheduler warp (leader) arrives after writing the tile index into both CTAs' rings
//   tileFree[r]  lives in the leader; every role warp of both CTAs arrives once it has read slot r
//
// Tile order: static round-robin (tile = pair + i * pairs), every role computing it for itself. With a device
// counter (setDynamicTiles) a scheduler warp in the leader CTA draws tiles with atomicAdd and hands them to the
// roles of both CTAs through a small ring of tile indices: pairs that start late, because SMs are held by a kernel
// of another stream (a collective that runs beside the GEMM), find the work done by the others instead of leaving
// a tail. The ring costs 2-4 % of an undisturbed GEMM, so it is only used when asked for.
// Operands: A [M,K] and B^T [N,K], K contiguous (bf16 or e4m3); C f32 or bf16 with the fused epilogues.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "kernels.hpp"
#include "ptx_sm100.cuh"

namespace bfb {

namespace {

constexpr int kPairM = 256;  // rows of the pair's tile (128 per CTA)
constexpr int kRowBytes2 = 128;
constexpr int kABytes2 = 128 * kRowBytes2;  // 16 KiB
constexpr int kThreads2 = 384;              // producer, MMA, TMEM, spare + 8 epilogue warps
constexpr int kEpilogueThreads2 = 256;
constexpr int kTileRing = 4;                // tile indices in flight between the scheduler warp and the roles
// arrivals that free a ring slot: two producers, the MMA warp, the epilogue warps of both CTAs
constexpr int kTileReaders = 2 + 1 + 2 * (kEpilogueThreads2 / 32);

template <int kAccN>
struct PairCfg {
    static constexpr int kBRows = kAccN / 2;                    // B^T rows staged by each CTA per k-slice
    static constexpr int kBBytes = kBRows * kRowBytes2;
    static constexpr int kStageBytes = kABytes2 + kBBytes;      // 32 or 48 KiB
    static constexpr int kStages = kAccN == 256 ? 6 : 4;
    static constexpr int kBufs = 512 / kAccN;                   // accumulator buffers in the 512 TMEM columns
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256 + 8 * 4096;   // + one 4 KiB staging tile per epilogue warp
};

struct PairTile {
    int m, n;
};

__device__ __forceinline__ PairTile pairTileCoord(int t, int tilesM, int tilesN, int groupN) {
    int fullGroups = tilesN / groupN;
    int perGroup = tilesM * groupN;
    int g = t / perGroup;
    int width = groupN;
    int r = t - g * perGroup;
    if (g >= fullGroups) {
        g = fullGroups;
        r = t - fullGroups * perGroup;
        width = tilesN - fullGroups * groupN;
    }
    PairTile c;
    c.m = r / width;
    c.n = g * groupN + r % width;
    return c;
}

struct PairEpilogue {
    void* c;
    const float* bias;
    const void* residual;
    float alpha;
    const float* dAlpha;
    int epilogue;
    int roundCBf16;
    const float* rowSumSq;   // [rowSumSqParts][m] partial sums of squares of A's rows, or null
    int rowSumSqParts;
    float rowInvDim;         // row scale = 1 / sqrt(sum * rowInvDim + rowEps)
    float rowEps;
    float* outSumSq;         // [ceil(n / 128)][m]: sums of squares of the stored values per 128-column part, or null
    float* outMaxAbs;        // same layout: largest magnitude of the stored values, or null
};

__device__ __forceinline__ float siluFast(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

template <int kElemBytes, typename TC, int kAccN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads2, 1)
gemmPairKernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB, PairEpilogue ep,
               int m, int n, int k, int tilesM, int tilesN, int groupN, int* status, int* tileCounter) {
    using Cfg = PairCfg<kAccN>;
    constexpr int kBlockK = kRowBytes2 / kElemBytes;
    constexpr int kMmaPerStage = 4;
    constexpr int kStages = Cfg::kStages;
    constexpr int kStageBytes = Cfg::kStageBytes;
    constexpr int kBufs = Cfg::kBufs;
    constexpr int kHalves = kAccN / 256;  // 256-column MMAs per k-step
    constexpr uint32_t kIdesc = make_idesc(kPairM, 256, kElemBytes == 2 ? 1u : 0u, 0u);

    extern __shared__ uint8_t smemRaw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
    uint64_t* fullBar = bars;
    uint64_t* emptyBar = bars + kStages;
    uint64_t* accFullBar = bars + 2 * kStages;
    uint64_t* accEmptyBar = accFullBar + 2;
    uint64_t* tileFullBar = accEmptyBar + 2;
    uint64_t* tileFreeBar = tileFullBar + kTileRing;
    uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(tileFreeBar + kTileRing);
    volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);
    volatile int* tileRing = reinterpret_cast<volatile int*>(tmemSlot + 2);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int numK = (k + kBlockK - 1) / kBlockK;
    const int totalTiles = tilesM * tilesN;
    const int clusterId = blockIdx.x >> 1;
    const int numClusters = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&fullBar[s], 1);
            mbar_init(&emptyBar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&accFullBar[b], 1);
            mbar_init(&accEmptyBar[b], 2 * (kEpilogueThreads2 / 32));  // one arrival per epilogue warp of both CTAs
        }
        for (int r = 0; r < kTileRing; ++r) {
            mbar_init(&tileFullBar[r], 1);
            mbar_init(&tileFreeBar[r], kTileReaders);
        }
        *abortFlag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmapA);
        tma_prefetch_desc(&tmapB);
    }
    if (warp == 2) {
        tmem_alloc(tmemSlot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers exist before any remote arrival or copy can reach them
    tc_fence_after();
    const uint32_t tmemBase = *tmemSlot;

    // next tile index for this warp (warp-uniform), -1 when there is none or the wait was abandoned
    int ringSlot = 0;
    uint32_t ringPhase = 0;
    int staticNext = clusterId;
    auto nextTile = [&]() -> int {
        if (tileCounter == nullptr) {   // static round-robin: no scheduler warp, no ring
            const int t = staticNext;
            staticNext += numClusters;
            return t < totalTiles ? t : -1;
        }
        if (!warp_all(mbar_wait_cluster(&tileFullBar[ringSlot], ringPhase, abortFlag, status, kDevTimeoutTile))) return -1;
        const int t = tileRing[ringSlot];
        __syncwarp();  // every lane has read the slot before it is handed back
        if (lane == 0) mbar_arrive_cluster(mapa_cluster(smem_u32(&tileFreeBar[ringSlot]), 0));
        if (++ringSlot == kTileRing) {
            ringSlot = 0;
            ringPhase ^= 1u;
        }
        return t;
    };

    if (warp == 3 && leader && tileCounter != nullptr) {
        // ---------------- tile scheduler (leader CTA, dynamic order only) ----------------
        const uint32_t peerRing = mapa_cluster(smem_u32(const_cast<int*>(tileRing)), 1);
        const uint32_t peerFull = mapa_cluster(smem_u32(tileFullBar), 1);
        int slot = 0;
        uint32_t phase = 0;
        while (true) {
            if (!warp_all(mbar_wait(&tileFreeBar[slot], phase ^ 1u, abortFlag, status, kDevTimeoutTile))) break;
            int t = 0;
            if (lane == 0) {
                t = atomicAdd(tileCounter, 1);
                if (t >= totalTiles) t = -1;
                tileRing[slot] = t;
                st_shared_cluster_u32(peerRing + static_cast<uint32_t>(slot) * 4u, static_cast<uint32_t>(t));
                mbar_arrive(&tileFullBar[slot]);
                mbar_arrive_cluster(peerFull + static_cast<uint32_t>(slot) * 8u);
            }
            t = __shfl_sync(0xFFFFFFFFu, t, 0);
            if (t < 0) break;   // the roles have been told; nothing more to hand out
            if (++slot == kTileRing) {
                slot = 0;
                phase ^= 1u;
            }
        }
    } else if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        int stage = 0;
        uint32_t phase = 0;
        bool alive = true;
        for (int t = nextTile(); t >= 0 && alive; t = nextTile()) {
            PairTile tc = pairTileCoord(t, tilesM, tilesN, groupN);
            const int rowA = tc.m * kPairM + static_cast<int>(rank) * 128;
            for (int kb = 0; kb < numK; ++kb) {
                if (!warp_all(mbar_wait(&emptyBar[stage], phase ^ 1u, abortFlag, status, kDevTimeoutStageEmpty))) {
                    alive = false;
                    break;
                }
                if (elect_one()) {
                    uint8_t* sa = smem + stage * kStageBytes;
                    uint8_t* sb = sa + kABytes2;
                    if (leader) mbar_arrive_expect_tx(&fullBar[stage], 2 * kStageBytes);
                    const uint32_t fullLeader = mapa_cluster(smem_u32(&fullBar[stage]), 0);
                    tma_load_2d_pair(sa, &tmapA, fullLeader, kb * kBlockK, rowA);
                    // each 256-column MMA takes 128 B^T rows from each CTA: this CTA's rows of column half h
#pragma unroll
                    for (int h = 0; h < kHalves; ++h) {
                        tma_load_2d_pair(sb + h * (128 * kRowBytes2), &tmapB, fullLeader, kb * kBlockK,
                                         tc.n * kAccN + h * 256 + static_cast<int>(rank) * 128);
                    }
                }
                __syncwarp();
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp == 1 && leader) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        // Static tile order: one elected thread runs the role (the compiler then keeps descriptors in uniform registers), and the
        // descriptors of a stage are its base words plus constants: one integer add per operand and MMA.
        if (tileCounter == nullptr && elect_one()) {
            constexpr uint32_t kHi = smem_desc_hi_sw128(1024);
            const uint32_t stage0Lo = smem_desc_lo(smem_u32(smem), 0);
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            bool alive = true;
            for (int t = staticNext; t < totalTiles && alive; t += numClusters, ++local) {
                const int buf = local % kBufs;
                const uint32_t accPhase = static_cast<uint32_t>(local / kBufs) & 1u;
                if (!mbar_wait(&accEmptyBar[buf], accPhase ^ 1u, abortFlag, status, kDevTimeoutAccEmpty)) break;
                tc_fence_after();
                const uint32_t dTmem = tmemBase + static_cast<uint32_t>(buf * kAccN);
                for (int kb = 0; kb < numK; ++kb) {
                    if (!mbar_wait(&fullBar[stage], phase, abortFlag, status, kDevTimeoutTmaFull)) {
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t aLo = stage0Lo + static_cast<uint32_t>(stage) * (kStageBytes >> 4);
                    const uint32_t bLo = aLo + (kABytes2 >> 4);
#pragma unroll
                    for (int kk = 0; kk < kMmaPerStage; ++kk) {
                        const uint32_t step = static_cast<uint32_t>((kk * 32) >> 4);
                        const uint32_t acc = (kb > 0 || kk > 0) ? 1u : 0u;
#pragma unroll
                        for (int h = 0; h < kHalves; ++h) {
                            const uint32_t bh = bLo + static_cast<uint32_t>(h * ((128 * kRowBytes2) >> 4)) + step;
                            const uint32_t d = dTmem + static_cast<uint32_t>(h * 256);
                            if constexpr (kElemBytes == 2) umma_f16_pair_words(d, aLo + step, kHi, bh, kHi, kIdesc, acc);
                            else umma_f8_pair_words(d, aLo + step, kHi, bh, kHi, kIdesc, acc);
                        }
                    }
                    umma_commit_pair(&emptyBar[stage]);
                    if (kb == numK - 1) umma_commit_pair(&accFullBar[buf]);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
        // dynamic tile order: the tile index arrives through the ring, read by the whole warp
        if (tileCounter != nullptr) {
        int stage = 0;
        uint32_t phase = 0;
        int local = 0;
        bool alive = true;
        for (int t = nextTile(); t >= 0 && alive; t = nextTile(), ++local) {
            const int buf = local % kBufs;
            const uint32_t accPhase = static_cast<uint32_t>(local / kBufs) & 1u;
            if (!warp_all(mbar_wait(&accEmptyBar[buf], accPhase ^ 1u, abortFlag, status, kDevTimeoutAccEmpty))) break;
            tc_fence_after();
            const uint32_t dTmem = tmemBase + static_cast<uint32_t>(buf * kAccN);
            for (int kb = 0; kb < numK; ++kb) {
                if (!warp_all(mbar_wait(&fullBar[stage], phase, abortFlag, status, kDevTimeoutTmaFull))) {
                    alive = false;
                    break;
                }
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t aAddr = smem_u32(smem + stage * kStageBytes);
                    const uint32_t bAddr = aAddr + kABytes2;
                    const uint64_t aDesc = make_smem_desc_sw128(aAddr, 0, 1024);
#pragma unroll
                    for (int kk = 0; kk < kMmaPerStage; ++kk) {
                        const uint64_t step = static_cast<uint64_t>((kk * 32) >> 4);
                        const uint32_t acc = (kb > 0 || kk > 0) ? 1u : 0u;
#pragma unroll
                        for (int h = 0; h < kHalves; ++h) {
                            const uint64_t bDesc = make_smem_desc_sw128(bAddr + h * (128 * kRowBytes2), 0, 1024);
                            const uint32_t d = dTmem + static_cast<uint32_t>(h * 256);
                            if constexpr (kElemBytes == 2) umma_f16_pair(d, aDesc + step, bDesc + step, kIdesc, acc);
                            else umma_f8_pair(d, aDesc + step, bDesc + step, kIdesc, acc);
                        }
                    }
                    umma_commit_pair(&emptyBar[stage]);
                    if (kb == numK - 1) umma_commit_pair(&accFullBar[buf]);
                }
                __syncwarp();
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
        }
    } else if (warp >= 4) {
        // ---------------- epilogue (both CTAs, 8 warps: lane quarter x column half) ----------------
        constexpr int kColsPerWarp = kAccN / 2;
        const int quarter = warp & 3;
        const int colHalf = (warp - 4) >> 2;
        const float scale = ep.dAlpha != nullptr ? *ep.dAlpha : ep.alpha;
        const bool hasBias =
            ep.epilogue == BFB_EPI_BIAS || ep.epilogue == BFB_EPI_BIAS_SILU || ep.epilogue == BFB_EPI_BIAS_RESIDUAL;
        const bool hasSilu = ep.epilogue == BFB_EPI_BIAS_SILU;
        const bool hasRes = ep.epilogue == BFB_EPI_BIAS_RESIDUAL || ep.epilogue == BFB_EPI_RESIDUAL;
        TC* cOut = static_cast<TC*>(ep.c);
        const TC* res = static_cast<const TC*>(ep.residual);
        uint8_t* stageTile = smem + kStages * kStageBytes + 256 + (warp - 4) * 4096;
        int local = 0;
        for (int t = nextTile(); t >= 0; t = nextTile(), ++local) {
            PairTile tc = pairTileCoord(t, tilesM, tilesN, groupN);
            const int buf = local % kBufs;
            const uint32_t accPhase = static_cast<uint32_t>(local / kBufs) & 1u;
            if (!warp_all(mbar_wait(&accFullBar[buf], accPhase, abortFlag, status, kDevTimeoutAccFull))) break;
            tc_fence_after();
            const int row = tc.m * kPairM + static_cast<int>(rank) * 128 + quarter * 32 + lane;
            const bool rowOk = row < m;
            // an rmsnorm of A's rows, applied to the product's rows instead
            float rowScale = scale;
            if (ep.rowSumSq != nullptr && rowOk) {
                float total = 0.0f;   // parts added in index order: the same sum whoever produced them
                for (int part = 0; part < ep.rowSumSqParts; ++part)
                    total += __ldg(ep.rowSumSq + static_cast<size_t>(part) * static_cast<size_t>(m) + row);
                rowScale = scale / sqrtf(total * ep.rowInvDim + ep.rowEps);
            }
            // Sums of squares of what this thread stores, one per 128-column part of the row, each written by
            // exactly one thread: no atomics, so the figures do not depend on timing or on the tile width.
            float sumSq = 0.0f, maxAbs = 0.0f;
            int part = -1;
            auto flushPart = [&]() {
                if (rowOk && part >= 0) {
                    const size_t at = static_cast<size_t>(part) * static_cast<size_t>(m) + row;
                    if (ep.outSumSq != nullptr) ep.outSumSq[at] = sumSq;
                    if (ep.outMaxAbs != nullptr) ep.outMaxAbs[at] = maxAbs;
                }
            };
            const uint32_t tBase = tmemBase + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(buf * kAccN + colHalf * kColsPerWarp);
            // The warp's 32 rows x 128 columns go out in rounds of 128 bytes per row (32 fp32 or 64 bf16 columns): a lane
            // finishes ITS row's values in registers (scale, bias, silu, residual, rounding, row statistics), lays them
            // into the warp's staging tile (16-byte pieces XOR-swizzled by the row: no bank conflicts either way), and the
            // warp writes the tile out four rows at a time, so that one store instruction covers four whole 128-byte
            // lines of C instead of 32 pieces of 32 different lines.
            constexpr int kRoundCols = 128 / static_cast<int>(sizeof(TC));      // columns per round
            constexpr int kPieceCols = 16 / static_cast<int>(sizeof(TC));       // columns per 16-byte piece
            const int row0 = tc.m * kPairM + static_cast<int>(rank) * 128 + quarter * 32;
#pragma unroll 1
            for (int round = 0; round < kColsPerWarp / kRoundCols; ++round) {
                const int col0 = tc.n * kAccN + colHalf * kColsPerWarp + round * kRoundCols;
                if (col0 >= n) break;
                if ((col0 >> 7) != part) {
                    flushPart();
                    part = col0 >> 7;
                    sumSq = 0.0f;
                    maxAbs = 0.0f;
                }
#pragma unroll
                for (int sub = 0; sub < kRoundCols / 32; ++sub) {
                    uint32_t raw[32];
                    tmem_ld_32x32(tBase + static_cast<uint32_t>(round * kRoundCols + sub * 32), raw);
                    tmem_ld_wait();
                    const size_t rowOff = static_cast<size_t>(row) * static_cast<size_t>(n);
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const int col = col0 + sub * 32 + g * 8;
                        const bool live = rowOk && col + 8 <= n;
                        float v[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(raw[g * 8 + j]) * rowScale;
                        if (hasBias && live) {
                            const float4 b0 = __ldg(reinterpret_cast<const float4*>(ep.bias + col));
                            const float4 b1 = __ldg(reinterpret_cast<const float4*>(ep.bias + col + 4));
                            v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
                            v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
                        }
                        if (hasSilu) {
#pragma unroll
                            for (int j = 0; j < 8; ++j) v[j] = siluFast(v[j]);
                        }
                        if constexpr (sizeof(TC) == 4) {
                            if (hasRes && live) {
                                const float4 r0 = *reinterpret_cast<const float4*>(res + rowOff + col);
                                const float4 r1 = *reinterpret_cast<const float4*>(res + rowOff + col + 4);
                                v[0] += r0.x; v[1] += r0.y; v[2] += r0.z; v[3] += r0.w;
                                v[4] += r1.x; v[5] += r1.y; v[6] += r1.z; v[7] += r1.w;
                            }
                            if (ep.roundCBf16) {
#pragma unroll
                                for (int j = 0; j < 8; ++j) v[j] = __bfloat162float(__float2bfloat16_rn(v[j]));
                            }
                            // pieces 2g and 2g + 1 of the row's 8 (one sub-block per round for fp32)
                            *reinterpret_cast<float4*>(stageTile + lane * 128 + (((2 * g) ^ (lane & 7)) << 4)) =
                                make_float4(v[0], v[1], v[2], v[3]);
                            *reinterpret_cast<float4*>(stageTile + lane * 128 + (((2 * g + 1) ^ (lane & 7)) << 4)) =
                                make_float4(v[4], v[5], v[6], v[7]);
                            if (live) {
                                if (ep.outSumSq != nullptr) {
#pragma unroll
                                    for (int j = 0; j < 8; ++j) sumSq = fmaf(v[j], v[j], sumSq);
                                }
                                if (ep.outMaxAbs != nullptr) {
#pragma unroll
                                    for (int j = 0; j < 8; ++j) maxAbs = fmaxf(maxAbs, fabsf(v[j]));
                                }
                            }
                        } else {
                            if (hasRes && live) {
                                const uint4 rr = *reinterpret_cast<const uint4*>(res + rowOff + col);
                                const __nv_bfloat162* rh = reinterpret_cast<const __nv_bfloat162*>(&rr);
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    float2 f = __bfloat1622float2(rh[j]);
                                    v[2 * j] += f.x;
                                    v[2 * j + 1] += f.y;
                                }
                            }
                            uint4 packed;
                            uint32_t* pw = reinterpret_cast<uint32_t*>(&packed);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                                pw[j] = *reinterpret_cast<uint32_t*>(&h);
                                if (live && (ep.outSumSq != nullptr || ep.outMaxAbs != nullptr)) {
                                    const float2 f = __bfloat1622float2(h);   // the values as stored
                                    sumSq = fmaf(f.x, f.x, fmaf(f.y, f.y, sumSq));
                                    maxAbs = fmaxf(maxAbs, fmaxf(fabsf(f.x), fabsf(f.y)));
                                }
                            }
                            // piece sub * 4 + g of the row's 8 (two sub-blocks per round for bf16)
                            *reinterpret_cast<uint4*>(stageTile + lane * 128 + (((sub * 4 + g) ^ (lane & 7)) << 4)) = packed;
                        }
                    }
                }
                __syncwarp();
                const int piece = lane & 7;
                const int colOut = col0 + piece * kPieceCols;
#pragma unroll
                for (int q4 = 0; q4 < 8; ++q4) {
                    const int rr = q4 * 4 + (lane >> 3);
                    const uint4 val = *reinterpret_cast<const uint4*>(stageTile + rr * 128 + ((piece ^ (rr & 7)) << 4));
                    if (row0 + rr < m && colOut + kPieceCols <= n) {
                        *reinterpret_cast<uint4*>(cOut + static_cast<size_t>(row0 + rr) * static_cast<size_t>(n) + colOut) = val;
                    }
                }
                __syncwarp();
            }
            tc_fence_before();
            __syncwarp();  // one (remote) arrival per warp instead of one per thread
            if (lane == 0) mbar_arrive_cluster(mapa_cluster(smem_u32(&accEmptyBar[buf]), 0));
            flushPart();
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's shared and tensor memory stay alive until the leader's MMAs are done with them
    if (warp == 2) {
        if (*abortFlag != 0) {
            uint64_t t0 = global_timer_ns();
            while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
        tc_fence_after();
        tmem_dealloc(tmemBase, 512);
    }
}

// BFB_GEMM_TILE_N=256 in the environment forces the 256-column tile (for A/B measurements).
int preferredTileN() {
    static const int v = [] {
        const char* e = std::getenv("BFB_GEMM_TILE_N");
        return (e != nullptr && std::atoi(e) == 256) ? 256 : 512;
    }();
    return v;
}

template <int kElemBytes, typename TC, int kAccN>
void launchPair(const GemmArgs& g, cudaStream_t stream) {
    using Cfg = PairCfg<kAccN>;
    constexpr int kBlockK = kRowBytes2 / kElemBytes;
    TensorMapStorage ta, tb;
    {
        uint64_t dims[2] = {static_cast<uint64_t>(g.k), static_cast<uint64_t>(g.m)};
        uint64_t strides[1] = {static_cast<uint64_t>(g.k) * kElemBytes};
        uint32_t box[2] = {static_cast<uint32_t>(kBlockK), 128u};
        encodeTensorMap(&ta, g.a, kElemBytes, 2, dims, strides, box);
    }
    {
        uint64_t dims[2] = {static_cast<uint64_t>(g.k), static_cast<uint64_t>(g.n)};
        uint64_t strides[1] = {static_cast<uint64_t>(g.k) * kElemBytes};
        uint32_t box[2] = {static_cast<uint32_t>(kBlockK), 128u};
        encodeTensorMap(&tb, g.b, kElemBytes, 2, dims, strides, box);
    }
    const int tilesM = static_cast<int>((g.m + kPairM - 1) / kPairM);
    const int tilesN = static_cast<int>((g.n + kAccN - 1) / kAccN);
    // about 4096 columns of B^T (16 MB at K = 2048) stay L2-resident per group
    const int maxGroup = 4096 / kAccN;
    const int groups = (tilesN + maxGroup - 1) / maxGroup;
    const int groupN = (tilesN + groups - 1) / groups;
    const int clusters = std::max(1, std::min(tilesM * tilesN, persistentSms() / 2));
    PairEpilogue ep{g.c, g.bias, g.residual, g.alpha, g.dAlpha, g.epilogue, g.roundCBf16,
                    g.rowSumSq, g.rowSumSqParts, g.rowInvDim, g.rowEps, g.outSumSq, g.outMaxAbs};
    auto kernel = gemmPairKernel<kElemBytes, TC, kAccN>;
    BFB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    int* tileCounter = nullptr;
    if (dynamicTiles() && tilesM * tilesN > clusters) {
        tileCounter = nextTileCounter();
        BFB_CUDA(cudaMemsetAsync(tileCounter, 0, sizeof(int), stream));
    }
    ProfileScope prof(kProfGemmTc, stream, 2.0 * static_cast<double>(g.m) * static_cast<double>(g.n) * static_cast<double>(g.k));
    kernel<<<2 * clusters, kThreads2, Cfg::kSmemBytes, stream>>>(*reinterpret_cast<CUtensorMap*>(ta.bytes),
                                                                 *reinterpret_cast<CUtensorMap*>(tb.bytes), ep,
                                                                 static_cast<int>(g.m), static_cast<int>(g.n),
                                                                 static_cast<int>(g.k), tilesM, tilesN, groupN, g.dStatus, tileCounter);
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

template <int kElemBytes, typename TC>
void launchPairAnyTile(const GemmArgs& g, cudaStream_t stream) {
    // The 512-column tile pays off once its exposed epilogue is small next to the k loop and there are enough
    // tiles. Measured at M = 65536: K = 2048 and 5632 lose 4-17 % to the 256-column tile, K = 16384 gains 17 %
    // (1587 vs 1358 TFLOP/s); BFB_GEMM_WIDE_K overrides the switch-over depth.
    static const int64_t wideK = [] {
        const char* e = std::getenv("BFB_GEMM_WIDE_K");
        return e != nullptr ? static_cast<int64_t>(std::atoll(e)) : static_cast<int64_t>(8192);
    }();
    const bool wide = preferredTileN() == 512 && g.n >= 512 && g.k >= wideK &&
                      ((g.m + 255) / 256) * ((g.n + 511) / 512) >= smCount() / 2;
    if (wide) launchPair<kElemBytes, TC, 512>(g, stream);
    else launchPair<kElemBytes, TC, 256>(g, stream);
}

}  // namespace

void gemmTensorCorePair(const GemmArgs& g, cudaStream_t stream) {
    const bool cf32 = g.cDtype == BFB_F32;
    using bf = __nv_bfloat16;
    if (g.abDtype == BFB_BF16) {
        if (cf32) launchPairAnyTile<2, float>(g, stream); else launchPairAnyTile<2, bf>(g, stream);
    } else {
        if (cf32) launchPairAnyTile<1, float>(g, stream); else launchPairAnyTile<1, bf>(g, stream);
    }
}

}  // namespace bfb
