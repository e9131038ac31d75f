// Backward of the causal attention core (fusedAttentionBackward, src/backend/cuda/fused_attention.cu:158-303,343-380
// in the reference): from dO, Q, K, V, O and the forward's row statistics (m, l) to dQ, dK, dV.
//
//   D_i  = sum_d O[i,d] dO[i,d]                      (attentionBackwardPrepKernel; also lse_i = m_i + ln l_i)
//   P    = exp(scale * Q K^T - lse)                   dP = dO V^T
//   dS   = scale * P o (dP - D)
//   dV   = P^T dO        dK = dS^T Q        dQ = dS K
//
// Two kernels:
//  * attentionBackwardTcKernel: tcgen05, head_dim 128, bf16 operands, fp32 accumulation. One CTA per (batch, head,
//    block of 128 keys); it walks the query blocks that see those keys. Everything is computed TRANSPOSED, with the
//    keys on the tensor-memory lanes: S^T = K Q^T and dP^T = V dO^T are ordinary shared-memory MMAs; a thread owns one
//    key row of both, so P^T and dS^T are written back as bf16 over them in tensor memory and are the TMEM operand of
//    dV += P^T dO and dK += dS^T Q, whose accumulators stay in tensor memory for the whole CTA. Only dS^T also goes
//    through shared memory, as the A operand of dQ = dS K (both tiles read MN-major: the dS^T tile with its query rows
//    and the K tile with head_dim contiguous). The dQ tile of a step is staged in the shared-memory slot that held the
//    step's Q and dO and ADDED to global memory by the TMA unit (cp.reduce.async.bulk.tensor), four instructions per
//    step; per-element atomics took a third of the step.
//    TMEM columns: S^T / P^T / dQ [0,128)  dP^T / dS^T [128,256)  dV [256,384)  dK [384,512).
//    dK and dV are written once (a CTA owns its keys), staged in the K and V tiles' shared memory and stored from there
//    a whole row per warp instruction; dQ is accumulated over the key blocks (zeroed by the host first), as the reference accumulates dK and dV
//    with atomics.
//  * attentionBackwardSimtKernel: any head_dim <= 256, fp32 or bf16 storage, one warp per query row; the shape-general
//    path, with the reference's own order of work.
// All mbarrier waits are bounded.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cmath>

#include "common.cuh"
#include "kernels.hpp"
#include "ptx_sm100.cuh"

namespace bfb {

namespace {

constexpr int kD = 128;
constexpr int kBlk = 128;                    // keys per CTA, query rows per step
constexpr int kHalfBytes = 128 * 128;        // one 64-wide half of a 128-row bf16 tile
constexpr int kTileBytes = 2 * kHalfBytes;   // 32 KiB
constexpr int kKOff = 0;
constexpr int kVOff = kTileBytes;
constexpr int kRingOff = 2 * kTileBytes;     // [2 stages][Q, dO]
constexpr int kDsOff = kRingOff + 4 * kTileBytes;
constexpr int kRowOff = kDsOff + kTileBytes; // [2 steps in flight][lse2, D][128] floats
constexpr int kBarOff = kRowOff + 2 * 2 * 128 * 4;
constexpr int kSmemBytes = kBarOff + 256;
constexpr int kSoftmaxWarps = 8;   // two per lane quadrant of tensor memory; each takes 64 of a step's 128 query columns
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kThreads = 320;
// A and B formats bf16, fp32 accumulate; bit 15 = A is MN-major, bit 16 = B is MN-major
constexpr uint32_t kIdescKK = make_idesc(128, 128, 1u, 0u);                  // both K-major
constexpr uint32_t kIdescKM = make_idesc(128, 128, 1u, 1u);                  // B MN-major (A from TMEM or K-major)
constexpr uint32_t kIdescMM = make_idesc(128, 128, 1u, 1u) | (1u << 15);     // A and B MN-major

__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct BwdParams {
    float* dQ;
    float* dK;
    float* dV;
    const float* lse2;   // [batch, heads, newLen]: (m + ln l) * log2(e)
    const float* dTerm;  // [batch, heads, newLen]: sum_d O dO
    int batch, newLen, totalLen, numHeads;
    int64_t ldDq, ldDk, ldDv;
    int prefetchAhead;     // a block asks for the K and V tiles of the block this many places after it
    float scale, scaleLog2;
    int oldLen, causal, numKvBlocks;
};

__global__ void __launch_bounds__(kThreads, 1)
attentionBackwardTcKernel(const __grid_constant__ CUtensorMap tmapQ, const __grid_constant__ CUtensorMap tmapK,
                          const __grid_constant__ CUtensorMap tmapV, const __grid_constant__ CUtensorMap tmapDo,
                          const __grid_constant__ CUtensorMap tmapDq, BwdParams p, int* status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kBarOff);
    uint64_t* kvFull = bars;          // [1]
    uint64_t* qFull = bars + 1;       // [2]
    uint64_t* dqStaged = bars + 3;    // [2] the step's dQ tile is in the slot its Q and dO came from (8 warps)
    uint64_t* sFull = bars + 5;       // S^T complete
    uint64_t* pFull = bars + 6;       // P^T written (4 warps)
    uint64_t* dsFull = bars + 7;      // dS^T written (4 warps)
    uint64_t* dqFull = bars + 8;      // dQ^T complete (and everything issued before it)
    uint64_t* dqFree = bars + 9;      // dQ^T read (4 warps): the S^T columns are free
    uint64_t* accFull = bars + 10;    // dV and dK complete
    uint64_t* rowFull = bars + 11;    // [2] row statistics of a step written (8 warps)
    uint64_t* slotFree = bars + 13;   // every product that reads the step's Q and dO tiles is complete
    uint64_t* dpFull = bars + 14;     // dP^T complete
    uint64_t* epiStaged = bars + 15;  // a gradient tile of the keys is in shared memory (8 warps)
    uint64_t* epiFree = bars + 16;    // ... and has been read out of it (8 warps)
    uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(bars + 17);
    volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);

    if ((smem_u32(smem) & 1023u) != 0u) {
        if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0, kDevTimeoutOther);
        return;
    }
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // work: key block 0 is seen by every query block, the last one by one: blocks differ in weight by the number of key blocks
    // (batch, head) pairs in groups of kGroup (their Q, K, V and dO together stay in L2: 2 MB a pair at 2048 rows); inside
    // a group the heaviest key blocks of all its pairs come first, so that the light ones fill the SMs at its end
    constexpr int kGroup = 8;
    const int numBh = p.batch * p.numHeads;
    const int perGroup = kGroup * p.numKvBlocks;
    auto decode = [&](int block, int* bOut, int* hOut) -> int {   // returns the block's first key
        const int group = block / perGroup;
        const int inGroup = block - group * perGroup;
        const int groupSize = min(kGroup, numBh - group * kGroup);
        const int bh = group * kGroup + inGroup % groupSize;
        *bOut = bh / p.numHeads;
        *hOut = bh % p.numHeads;
        return (inGroup / groupSize) * kBlk;
    };
    int b, h;
    const int k0 = decode(static_cast<int>(blockIdx.x), &b, &h);
    const int numQBlocks = (p.newLen + kBlk - 1) / kBlk;
    // first query block with a row that sees key k0: old_len + i >= k0
    const int firstQ = p.causal ? max(0, k0 - p.oldLen) / kBlk : 0;
    const int steps = max(0, numQBlocks - firstQ);

    // The first tiles are requested before anything else is set up: the producer thread initialises the three barriers
    // they complete on itself (the other roles look at them only after the CTA-wide barrier below).
    auto loadQdO = [&](int it) {
        uint8_t* slot = smem + kRingOff + (it & 1) * 2 * kTileBytes;
        const int q0 = (firstQ + it) * kBlk;
        mbar_arrive_expect_tx(&qFull[it & 1], 2 * kTileBytes);
        tma_load_3d(slot, &tmapQ, &qFull[it & 1], h * kD, q0, b);
        tma_load_3d(slot + kHalfBytes, &tmapQ, &qFull[it & 1], h * kD + 64, q0, b);
        tma_load_3d(slot + kTileBytes, &tmapDo, &qFull[it & 1], h * kD, q0, b);
        tma_load_3d(slot + kTileBytes + kHalfBytes, &tmapDo, &qFull[it & 1], h * kD + 64, q0, b);
    };
    if (warp == kProducerWarp && steps > 0 && elect_one()) {
        mbar_init(kvFull, 1);
        mbar_init(&qFull[0], 1);
        mbar_init(&qFull[1], 1);
        fence_mbar_init();
        mbar_arrive_expect_tx(kvFull, 2 * kTileBytes);
        tma_load_3d(smem + kKOff, &tmapK, kvFull, h * kD, k0, b);
        tma_load_3d(smem + kKOff + kHalfBytes, &tmapK, kvFull, h * kD + 64, k0, b);
        tma_load_3d(smem + kVOff, &tmapV, kvFull, h * kD, k0, b);
        tma_load_3d(smem + kVOff + kHalfBytes, &tmapV, kvFull, h * kD + 64, k0, b);
        loadQdO(0);
        if (steps > 1) loadQdO(1);
        // A block's K and V tiles are read by that block alone, so they would come from DRAM when it starts: the block
        // that takes an SM about one CTA from now has them brought into L2 here.
        const int ahead = static_cast<int>(blockIdx.x) + p.prefetchAhead;
        if (ahead < static_cast<int>(gridDim.x)) {
            int b2, h2;
            const int k2 = decode(ahead, &b2, &h2);
            tma_prefetch_l2_3d(&tmapK, h2 * kD, k2, b2);
            tma_prefetch_l2_3d(&tmapK, h2 * kD + 64, k2, b2);
            tma_prefetch_l2_3d(&tmapV, h2 * kD, k2, b2);
            tma_prefetch_l2_3d(&tmapV, h2 * kD + 64, k2, b2);
        }
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) mbar_init(&dqStaged[i], kSoftmaxWarps);
        mbar_init(sFull, 1);
        mbar_init(pFull, kSoftmaxWarps);
        mbar_init(dsFull, kSoftmaxWarps);
        mbar_init(dqFull, 1);
        mbar_init(dqFree, kSoftmaxWarps);
        mbar_init(accFull, 1);
        mbar_init(slotFree, 1);
        mbar_init(dpFull, 1);
        mbar_init(epiStaged, kSoftmaxWarps);
        mbar_init(epiFree, kSoftmaxWarps);
        mbar_init(&rowFull[0], kSoftmaxWarps);
        mbar_init(&rowFull[1], kSoftmaxWarps);
        *abortFlag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmapQ);
        tma_prefetch_desc(&tmapK);
        tma_prefetch_desc(&tmapV);
        tma_prefetch_desc(&tmapDo);
        tma_prefetch_desc(&tmapDq);
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
        // ---------------- TMA producer (one elected thread) ----------------
        if (elect_one() && steps > 0) {
            // Slot (it & 1) receives the Q and dO tiles of step it (those of steps 0 and 1 were requested above). Before
            // that, the dQ tile the gradient warps staged there for step it - 2 is added to global memory; the slot is
            // free again when that tile has been read. The CTA may end once the last tile has been read: the unit
            // completes the additions by itself.
            for (int it = 2; it < steps + 2; ++it) {
                const int stage = it & 1;
                uint8_t* slot = smem + kRingOff + stage * 2 * kTileBytes;
                if (!mbar_wait(&dqStaged[stage], ((it - 2) >> 1) & 1, abortFlag, status, kDevTimeoutStageEmpty)) break;
                const int qPrev = (firstQ + it - 2) * kBlk;
#pragma unroll
                for (int box = 0; box < 4; ++box) {
                    tma_reduce_add_3d(&tmapDq, slot + box * (kBlk * 128), h * kD + box * 32, qPrev, b);
                }
                tma_store_commit();
                tma_store_wait_read();
                if (it < steps) loadQdO(it);
            }
        }
        __syncwarp();
    } else if (warp == kMmaWarp) {
        // ---------------- MMA issuer (one elected thread) ----------------
        if (elect_one() && steps > 0) {
            constexpr uint32_t kHi = smem_desc_hi_sw128(1024);
            const uint32_t kLo = smem_desc_lo(smem_u32(smem + kKOff), 0);
            const uint32_t vLo = smem_desc_lo(smem_u32(smem + kVOff), 0);
            const uint32_t dsLoMn = smem_desc_lo(smem_u32(smem + kDsOff), kHalfBytes);
            const uint32_t kLoMn = smem_desc_lo(smem_u32(smem + kKOff), kHalfBytes);
            // The two 128-column regions swap roles every step: S^T of step it + 1 goes where dP^T / dS^T of step it was
            // (free as soon as dK of step it is issued: the pipe runs in order), dP^T of step it + 1 where S^T / P^T / dQ
            // of step it was (free when the gradient warps have read dQ). So the next S^T never waits for them.
            const uint32_t tDv = tmemBase + 256u, tDk = tmemBase + 384u;
            auto regionS = [&](int it) { return tmemBase + static_cast<uint32_t>((it & 1) * 128); };
            auto regionDp = [&](int it) { return tmemBase + static_cast<uint32_t>(((it & 1) ^ 1) * 128); };
            bool alive = mbar_wait(kvFull, 0, abortFlag, status, kDevTimeoutTmaFull);
            auto ringLo = [&](int it) { return smem_desc_lo(smem_u32(smem + kRingOff + (it & 1) * 2 * kTileBytes), 0); };
            auto issueDp = [&](int it) {                    // dP^T = V dO^T (reduction over head_dim)
                const uint32_t doLo = ringLo(it) + (kTileBytes >> 4);
#pragma unroll
                for (int kk = 0; kk < kD / 16; ++kk) {
                    const uint32_t off = ((kk >> 2) * kHalfBytes + (kk & 3) * 32) >> 4;
                    umma_f16_words(regionDp(it), vLo + off, kHi, doLo + off, kHi, kIdescKK, kk > 0 ? 1u : 0u);
                }
            };
            auto issueS = [&](int it) {                     // S^T = K Q^T
                const uint32_t qLo = ringLo(it);
#pragma unroll
                for (int kk = 0; kk < kD / 16; ++kk) {
                    const uint32_t off = ((kk >> 2) * kHalfBytes + (kk & 3) * 32) >> 4;
                    umma_f16_words(regionS(it), kLo + off, kHi, qLo + off, kHi, kIdescKK, kk > 0 ? 1u : 0u);
                }
            };
            // the bf16 operand a pair of warps leaves in tensor memory: query rows 0..63 over the first half of the
            // fp32 region, rows 64..127 over its second half (each warp writes only over columns it alone reads)
            auto aCol = [](int kk) { return static_cast<uint32_t>((kk >> 2) * 64 + (kk & 3) * 8); };
            if (alive && mbar_wait(&qFull[0], 0, abortFlag, status, kDevTimeoutTmaFull)) {
                tc_fence_after();
                issueS(0);
                umma_commit(sFull);
                issueDp(0);
                umma_commit(dpFull);
            } else {
                alive = false;
            }
            for (int it = 0; it < steps && alive; ++it) {
                const int stage = it & 1;
                const uint32_t par = static_cast<uint32_t>(it) & 1u;
                const uint32_t qLoMn = ringLo(it) + ((kHalfBytes >> 4) << 16);
                const uint32_t doLoMn = qLoMn + (kTileBytes >> 4);
                const uint32_t tS = regionS(it), tDp = regionDp(it);
                if (!mbar_wait(pFull, par, abortFlag, status, kDevTimeoutSoftmax)) { alive = false; break; }
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < kBlk / 16; ++kk) {    // dV += P^T dO (reduction over the query rows)
                    umma_f16_ts_words(tDv, tS + aCol(kk), doLoMn + kk * (2048 >> 4), kHi, kIdescKM, (it > 0 || kk > 0) ? 1u : 0u);
                }
                if (!mbar_wait(dsFull, par, abortFlag, status, kDevTimeoutSoftmax)) { alive = false; break; }
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < kBlk / 16; ++kk) {    // dQ = dS K (reduction over the keys), over S^T / P^T
                    umma_f16_words(tS, dsLoMn + kk * (2048 >> 4), kHi, kLoMn + kk * (2048 >> 4), kHi, kIdescMM, kk > 0 ? 1u : 0u);
                }
                umma_commit(dqFull);
#pragma unroll
                for (int kk = 0; kk < kBlk / 16; ++kk) {    // dK += dS^T Q
                    umma_f16_ts_words(tDk, tDp + aCol(kk), qLoMn + kk * (2048 >> 4), kHi, kIdescKM, (it > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(slotFree);   // dV and dK have read this step's dO and Q: their slot may take the dQ tile
                if (it + 1 < steps) {
                    if (!mbar_wait(&qFull[stage ^ 1], ((it + 1) >> 1) & 1, abortFlag, status, kDevTimeoutTmaFull)) { alive = false; break; }
                    tc_fence_after();
                    issueS(it + 1);
                    umma_commit(sFull);
                    if (!mbar_wait(dqFree, par, abortFlag, status, kDevTimeoutAccEmpty)) { alive = false; break; }
                    tc_fence_after();
                    issueDp(it + 1);
                    umma_commit(dpFull);
                }
            }
            if (alive) umma_commit(accFull);
        }
        __syncwarp();
    } else {
        // ---------------- gradient warps: a thread owns one key row and 64 of the step's 128 query columns ----------------
        const int quad = warp & 3, half = warp >> 2;
        const int keyRow = quad * 32 + lane;               // key inside the block; the query row when reading dQ
        const int keyPos = k0 + keyRow;
        const bool keyValid = keyPos < p.totalLen;
        const uint32_t laneBase = static_cast<uint32_t>(quad * 32) << 16;
        const uint32_t tHalf = tmemBase + laneBase + static_cast<uint32_t>(half * 64);   // + 128 for the other region
        uint8_t* dsRow = smem + kDsOff + half * kHalfBytes + keyRow * 128;
        const bool raggedKeys = k0 + kBlk > p.totalLen;
        bool alive = true;
        auto fetchStat = [&](int qBase) -> float {
            const int qi = qBase + keyRow;
            const bool ok = qi < p.newLen;
            const size_t at = (static_cast<size_t>(b) * p.numHeads + h) * p.newLen + (ok ? qi : 0);
            if (half == 0) return ok ? p.lse2[at] : INFINITY;
            return ok ? p.dTerm[at] : 0.0f;
        };
        if (steps > 0) {
            reinterpret_cast<float*>(smem + kRowOff)[half * 128 + keyRow] = fetchStat(firstQ * kBlk);
            __syncwarp();
            if (lane == 0) mbar_arrive(&rowFull[0]);
        }
        for (int it = 0; it < steps && alive; ++it) {
            const uint32_t par = static_cast<uint32_t>(it) & 1u;
            const int q0 = (firstQ + it) * kBlk;
            const uint32_t tS = tHalf + par * 128u, tDp = tHalf + (par ^ 1u) * 128u;   // the regions swap roles every step
            // statistics of the step's 128 query rows (lse2 from the first four warps, D from the others; a row past the
            // end gets +inf, which makes its probabilities zero): this step's are in shared memory already, the next
            // step's are fetched now and stored at the end of the step, so that no step waits for global memory
            const int stage = it & 1;
            float* lseS = reinterpret_cast<float*>(smem + kRowOff) + stage * 256;
            float* dS = lseS + 128;
            const float nextStat = it + 1 < steps ? fetchStat(q0 + kBlk) : 0.0f;
            if (!warp_all(mbar_wait(&rowFull[stage], (it >> 1) & 1, abortFlag, status, kDevTimeoutOther))) {
                alive = false;
                break;
            }
            if (!warp_all(mbar_wait(sFull, par, abortFlag, status, kDevTimeoutAccFull))) {
                alive = false;
                break;
            }
            tc_fence_after();
            // ---- P^T = exp2(S^T * scale_log2 - lse2[c]). Row c sees this key iff keyPos <= old_len + q0 + c: columns
            // below firstVisible are masked, which only the steps on the diagonal (or a ragged last key block) need.
            const int firstVisible = p.causal ? keyPos - p.oldLen - q0 : -1;
            const bool maskStep = raggedKeys || (p.causal && k0 + kBlk - 1 - p.oldLen - q0 > 0);
            const float* lseH = lseS + half * 64;
            const float* dH = dS + half * 64;
            uint32_t pk[2][16];   // P^T as bf16 pairs, kept for dS^T (chunk c reads columns [32c, 32c+32) of this warp's
                                  // half and writes [16c, 16c+16), which it has already read)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t sc[32];
                tmem_ld_32x32(tS + static_cast<uint32_t>(c * 32), sc);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    const float4 ls = *reinterpret_cast<const float4*>(lseH + c * 32 + i);
                    float pv[4];
                    pv[0] = ex2f(fmaf(__uint_as_float(sc[i]), p.scaleLog2, -ls.x));
                    pv[1] = ex2f(fmaf(__uint_as_float(sc[i + 1]), p.scaleLog2, -ls.y));
                    pv[2] = ex2f(fmaf(__uint_as_float(sc[i + 2]), p.scaleLog2, -ls.z));
                    pv[3] = ex2f(fmaf(__uint_as_float(sc[i + 3]), p.scaleLog2, -ls.w));
                    if (maskStep) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            if (!keyValid || half * 64 + c * 32 + i + e < firstVisible) pv[e] = 0.0f;
                        }
                    }
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(pv[0], pv[1]), h1 = __floats2bfloat162_rn(pv[2], pv[3]);
                    pk[c][i >> 1] = *reinterpret_cast<uint32_t*>(&h0);
                    pk[c][(i >> 1) + 1] = *reinterpret_cast<uint32_t*>(&h1);
                }
                tmem_st_32x16(tS + static_cast<uint32_t>(c * 16), pk[c]);
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(pFull);
            if (!warp_all(mbar_wait(dpFull, par, abortFlag, status, kDevTimeoutAccFull))) {
                alive = false;
                break;
            }
            tc_fence_after();
            // ---- dS^T = P^T o (scale dP^T - scale D[c]) (the statistics kernel stores D already scaled); written over
            // dP^T as the tensor-memory operand of dK, and to shared memory as the operand of dQ^T
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t dp[32];
                tmem_ld_32x32(tDp + static_cast<uint32_t>(c * 32), dp);
                tmem_ld_wait();
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    const float4 dt = *reinterpret_cast<const float4*>(dH + c * 32 + i);
                    const float2 pa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk[c][i >> 1]));
                    const float2 pb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk[c][(i >> 1) + 1]));
                    const float d0 = pa.x * fmaf(__uint_as_float(dp[i]), p.scale, -dt.x);
                    const float d1 = pa.y * fmaf(__uint_as_float(dp[i + 1]), p.scale, -dt.y);
                    const float d2 = pb.x * fmaf(__uint_as_float(dp[i + 2]), p.scale, -dt.z);
                    const float d3 = pb.y * fmaf(__uint_as_float(dp[i + 3]), p.scale, -dt.w);
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(d0, d1), h1 = __floats2bfloat162_rn(d2, d3);
                    packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h0);
                    packed[(i >> 1) + 1] = *reinterpret_cast<uint32_t*>(&h1);
                }
                tmem_st_32x16(tDp + static_cast<uint32_t>(c * 16), packed);
                // shared-memory copy: row = key, this warp's 64 query rows are one 128-byte row of its half tile, 16-byte
                // pieces swizzled by the row
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int piece = c * 4 + g;
                    *reinterpret_cast<uint4*>(dsRow + ((piece ^ (keyRow & 7)) << 4)) =
                        make_uint4(packed[g * 4], packed[g * 4 + 1], packed[g * 4 + 2], packed[g * 4 + 3]);
                }
            }
            tmem_st_wait();
            fence_proxy_async_smem();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(dsFull);
            // the statistics of the next step, fetched at the top of this one, go to the other buffer: every warp has
            // left the step that read it (this step's S^T needed all of them to finish the one before)
            if (it + 1 < steps) {
                float* nextRows = reinterpret_cast<float*>(smem + kRowOff) + (stage ^ 1) * 256 + half * 128;
                nextRows[keyRow] = nextStat;
                __syncwarp();
                if (lane == 0) mbar_arrive(&rowFull[stage ^ 1]);
            }
            // ---- dQ: lane = query row, columns = head_dim. The tile goes to the slot this step's Q and dO came from, as
            // four boxes of 32 floats x 128 rows in the 128-byte swizzle; the producer thread hands it to the TMA unit.
            if (!warp_all(mbar_wait(dqFull, par, abortFlag, status, kDevTimeoutAccFull))) {
                alive = false;
                break;
            }
            tc_fence_after();
            uint32_t dq[2][32];
            tmem_ld_32x32(tS, dq[0]);
            tmem_ld_32x32(tS + 32u, dq[1]);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(dqFree);       // the columns may take the next step's S^T
            // The first four warps write over the Q tile, which dK (issued after dQ) still reads; the others write over
            // the dO tile, whose last reader dV was issued before dQ and is complete with it. They go ahead, and so
            // reach the next step's exponentials while their scheduler's other warp is still here.
            if (half == 0 && !warp_all(mbar_wait(slotFree, par, abortFlag, status, kDevTimeoutAccFull))) {
                alive = false;
                break;
            }
            uint8_t* slot = smem + kRingOff + stage * 2 * kTileBytes;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint8_t* row = slot + (half * 2 + c) * (kBlk * 128) + keyRow * 128;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    *reinterpret_cast<uint4*>(row + ((j ^ (keyRow & 7)) << 4)) =
                        make_uint4(dq[c][j * 4], dq[c][j * 4 + 1], dq[c][j * 4 + 2], dq[c][j * 4 + 3]);
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&dqStaged[stage]);
        }
        // ---- dV (first four warps) and dK (the others) of this CTA's keys; keys that no query row sees get zeros
        if (steps == 0 && keyValid) {
            float* dst = (half == 0 ? p.dV : p.dK) +
                         (static_cast<size_t>(b) * p.totalLen + keyPos) * (half == 0 ? p.ldDv : p.ldDk) + static_cast<size_t>(h) * kD;
#pragma unroll 4
            for (int i = 0; i < kD; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
        if (alive && steps > 0 && warp_all(mbar_wait(accFull, 0, abortFlag, status, kDevTimeoutAccFull))) {
            // dV, then dK: a thread owns a key row of the accumulator, so the 64 KB tile is laid into the K and V tiles'
            // shared memory (no product reads them any more; four parts of 32 floats x 128 rows, 16-byte pieces swizzled by
            // the row) and leaves from there a row per warp instruction: 512 contiguous bytes. (Written by the TMA unit the
            // two tiles queued behind the last dQ tiles: 1 536 row segments of 128 bytes at about 5 cycles each, 7 500
            // cycles at the end of every CTA.)
            tc_fence_after();
            uint8_t* stageBase = smem + kKOff;
#pragma unroll 1
            for (int which = 0; which < 2; ++which) {
                if (which == 1 && !warp_all(mbar_wait(epiFree, 0, abortFlag, status, kDevTimeoutStageEmpty))) break;
                const uint32_t tAcc = tmemBase + laneBase + (which == 0 ? 256u : 384u) + static_cast<uint32_t>(half * 64);
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t acc[32];
                    tmem_ld_32x32(tAcc + static_cast<uint32_t>(c * 32), acc);
                    tmem_ld_wait();
                    uint8_t* row = stageBase + (half * 2 + c) * (kBlk * 128) + keyRow * 128;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        *reinterpret_cast<uint4*>(row + ((j ^ (keyRow & 7)) << 4)) =
                            make_uint4(acc[j * 4], acc[j * 4 + 1], acc[j * 4 + 2], acc[j * 4 + 3]);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(epiStaged);
                if (!warp_all(mbar_wait(epiStaged, static_cast<uint32_t>(which), abortFlag, status, kDevTimeoutOther))) break;
                // warp w writes key rows w, w + 8, ...; lane l the floats [4l, 4l + 4) of the row; rows past the last key
                // are left out
                const size_t ld = which == 0 ? p.ldDv : p.ldDk;
                float* dst = (which == 0 ? p.dV : p.dK) + (static_cast<size_t>(b) * p.totalLen + k0) * ld +
                             static_cast<size_t>(h) * kD + lane * 4;
                const uint8_t* part = stageBase + (lane >> 3) * (kBlk * 128);
                const int validRows = min(kBlk, p.totalLen - k0);
#pragma unroll 4
                for (int r = warp; r < validRows; r += kSoftmaxWarps) {
                    const uint4 v = *reinterpret_cast<const uint4*>(part + r * 128 + (((lane & 7) ^ (r & 7)) << 4));
                    *reinterpret_cast<uint4*>(dst + static_cast<size_t>(r) * ld) = v;
                }
                if (which == 0) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(epiFree);   // this warp has read its rows of dV out of the tiles
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

// D_i = dScale * sum_d O dO and lse2_i = (m_i + ln l_i) * log2(e), one warp per (batch, head, query row)
template <typename T>
__global__ void attentionBackwardPrepKernel(const T* out, const T* dOut, const float* m, const float* l, float* lse2,
                                            float* dTerm, int64_t rows, int numHeads, int64_t newLen, int headDim,
                                            int64_t ldO, int64_t ldDo, float dScale) {
    const int64_t warpId = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warpId >= rows) return;
    const int64_t i = warpId % newLen;
    const int64_t bh = warpId / newLen;
    const int64_t h = bh % numHeads, b = bh / numHeads;
    const T* o = out + (b * newLen + i) * ldO + h * headDim;
    const T* g = dOut + (b * newLen + i) * ldDo + h * headDim;
    float acc = 0.0f;
    for (int d = lane; d < headDim; d += 32) acc += static_cast<float>(o[d]) * static_cast<float>(g[d]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
    if (lane == 0) {
        dTerm[warpId] = acc * dScale;
        const float lv = l[warpId];
        // a row with no visible key (l == 0) never contributes: +inf makes every probability zero
        lse2[warpId] = lv > 0.0f ? (m[warpId] + logf(lv)) * 1.4426950408889634f : INFINITY;
    }
}

// Shape-general path: one warp per query row, the reference's order of work (fused_attention.cu:183-303): scores and
// dP by warp reductions, dQ in registers, dK / dV by atomics. T is the storage type of q, k, v, dO.
template <typename T>
__global__ void attentionBackwardSimtKernel(const T* q, const T* k, const T* v, const T* dOut, const float* lse2,
                                            const float* dTerm, float* dQ, float* dK, float* dV, int64_t rows, int numHeads,
                                            int64_t newLen, int64_t totalLen, int headDim, int64_t ldQ, int64_t ldK,
                                            int64_t ldV, int64_t ldDo, int64_t ldDq, int64_t ldDk, int64_t ldDv,
                                            float scale, int64_t oldLen, int causal) {
    constexpr int kMaxPerLane = 8;   // head_dim <= 256
    const int64_t warpId = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warpId >= rows) return;
    const int64_t i = warpId % newLen;
    const int64_t bh = warpId / newLen;
    const int64_t h = bh % numHeads, b = bh / numHeads;
    float qReg[kMaxPerLane], gReg[kMaxPerLane], dqAcc[kMaxPerLane];
#pragma unroll
    for (int e = 0; e < kMaxPerLane; ++e) {
        const int d = lane + e * 32;
        const bool ok = d < headDim;
        qReg[e] = ok ? static_cast<float>(q[(b * newLen + i) * ldQ + h * headDim + d]) : 0.0f;
        gReg[e] = ok ? static_cast<float>(dOut[(b * newLen + i) * ldDo + h * headDim + d]) : 0.0f;
        dqAcc[e] = 0.0f;
    }
    const float lseRow = lse2[warpId] * 0.6931471805599453f;   // back to natural-log units
    const float dRow = dTerm[warpId];
    const int64_t last = causal ? min(totalLen - 1, oldLen + i) : totalLen - 1;
    for (int64_t kp = 0; kp <= last; ++kp) {
        const T* kRow = k + (b * totalLen + kp) * ldK + h * headDim;
        const T* vRow = v + (b * totalLen + kp) * ldV + h * headDim;
        float sc = 0.0f, dp = 0.0f;
#pragma unroll
        for (int e = 0; e < kMaxPerLane; ++e) {
            const int d = lane + e * 32;
            if (d < headDim) {
                sc = fmaf(qReg[e], static_cast<float>(kRow[d]), sc);
                dp = fmaf(gReg[e], static_cast<float>(vRow[d]), dp);
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            sc += __shfl_xor_sync(0xFFFFFFFFu, sc, off);
            dp += __shfl_xor_sync(0xFFFFFFFFu, dp, off);
        }
        const float pr = expf(sc * scale - lseRow);
        const float ds = pr * (dp - dRow) * scale;
#pragma unroll
        for (int e = 0; e < kMaxPerLane; ++e) {
            const int d = lane + e * 32;
            if (d < headDim) {
                dqAcc[e] = fmaf(ds, static_cast<float>(kRow[d]), dqAcc[e]);
                atomicAdd(dK + (b * totalLen + kp) * ldDk + h * headDim + d, ds * qReg[e]);
                atomicAdd(dV + (b * totalLen + kp) * ldDv + h * headDim + d, pr * gReg[e]);
            }
        }
    }
#pragma unroll
    for (int e = 0; e < kMaxPerLane; ++e) {
        const int d = lane + e * 32;
        if (d < headDim) dQ[(b * newLen + i) * ldDq + h * headDim + d] = dqAcc[e];
    }
}

void makeMap3(TensorMapStorage* out, const void* base, int64_t dim, int64_t len, int64_t batch, int64_t ld) {
    uint64_t dims[3] = {static_cast<uint64_t>(dim), static_cast<uint64_t>(len), static_cast<uint64_t>(batch)};
    uint64_t strides[2] = {static_cast<uint64_t>(ld) * 2, static_cast<uint64_t>(ld) * 2 * static_cast<uint64_t>(len)};
    uint32_t box[3] = {64u, 128u, 1u};
    encodeTensorMap(out, base, 2, 3, dims, strides, box);
}

}  // namespace

bool attentionBackwardUsesTensorCores(const AttentionBackwardArgs& a) {
    if (a.dtype != BFB_BF16 || a.headDim != kD) return false;
    if (a.ldQ % 8 || a.ldK % 8 || a.ldV % 8 || a.ldDo % 8 || a.ldDq % 4 || a.ldDk % 4 || a.ldDv % 4) return false;
    auto aligned16 = [](const void* ptr) { return reinterpret_cast<uintptr_t>(ptr) % 16 == 0; };
    if (!aligned16(a.q) || !aligned16(a.k) || !aligned16(a.v) || !aligned16(a.dOut) || !aligned16(a.dQ) || !aligned16(a.dK) || !aligned16(a.dV))
        return false;
    if (a.batch * a.numHeads > 0x3FFFFF || a.totalLen > 0x3FFFFFFF || a.newLen > 0x3FFFFFFF) return false;
    return true;
}

void attentionBackward(const AttentionBackwardArgs& a, cudaStream_t stream) {
    require(a.batch >= 0 && a.newLen >= 0 && a.totalLen >= 0 && a.numHeads > 0 && a.headDim > 0, "attention_bwd: bad sizes");
    require(a.headDim <= 256, "attention_bwd: head_dim up to 256");
    require(a.totalLen >= a.oldLen + a.newLen || !a.causal, "attention_bwd: total_len must cover old_len + new_len");
    require(a.dtype == BFB_F32 || a.dtype == BFB_BF16, "attention_bwd: q, k, v, out and d_out are f32 or bf16");
    const int64_t rows = a.batch * a.numHeads * a.newLen;
    const size_t kvElems = static_cast<size_t>(a.batch) * a.totalLen;
    const int64_t dimAll = a.numHeads * a.headDim;
    require(a.ldQ >= dimAll && a.ldK >= dimAll && a.ldV >= dimAll && a.ldO >= dimAll && a.ldDo >= dimAll &&
                a.ldDq >= dimAll && a.ldDk >= dimAll && a.ldDv >= dimAll,
            "attention_bwd: row stride below heads*head_dim");
    if (kvElems > 0) require(a.dK != nullptr && a.dV != nullptr, "attention_bwd: null gradient pointer");
    if (rows > 0) {
        require(a.totalLen > 0, "attention_bwd: no keys");
        require(a.dOut != nullptr && a.q != nullptr && a.k != nullptr && a.v != nullptr && a.out != nullptr && a.m != nullptr &&
                    a.l != nullptr && a.dQ != nullptr,
                "attention_bwd: null pointer");
        require(a.lse2Scratch != nullptr && a.dTermScratch != nullptr, "attention_bwd: null scratch pointer");
    }
    const bool tensorCores = rows > 0 && attentionBackwardUsesTensorCores(a);
    // The CUDA-core kernel accumulates dK and dV with atomics: they start from zero. The tensor-core kernel writes every
    // element of both itself (a CTA owns its keys) and accumulates dQ, which then starts from zero.
    if (kvElems > 0 && !tensorCores) {
        BFB_CUDA(cudaMemset2DAsync(a.dK, static_cast<size_t>(a.ldDk) * 4, 0, static_cast<size_t>(a.numHeads * a.headDim) * 4, kvElems, stream));
        BFB_CUDA(cudaMemset2DAsync(a.dV, static_cast<size_t>(a.ldDv) * 4, 0, static_cast<size_t>(a.numHeads * a.headDim) * 4, kvElems, stream));
    }
    if (rows == 0) return;
    const int threads = 256;
    // the tensor-core kernel wants D already multiplied by the score scale
    const float dScale = tensorCores ? a.scale : 1.0f;
    const unsigned prepBlocks = static_cast<unsigned>((rows * 32 + threads - 1) / threads);
    if (a.dtype == BFB_F32) {
        attentionBackwardPrepKernel<float><<<prepBlocks, threads, 0, stream>>>(
            static_cast<const float*>(a.out), static_cast<const float*>(a.dOut), a.m, a.l, a.lse2Scratch, a.dTermScratch, rows,
            static_cast<int>(a.numHeads), a.newLen, static_cast<int>(a.headDim), a.ldO, a.ldDo, dScale);
    } else {
        attentionBackwardPrepKernel<__nv_bfloat16><<<prepBlocks, threads, 0, stream>>>(
            static_cast<const __nv_bfloat16*>(a.out), static_cast<const __nv_bfloat16*>(a.dOut), a.m, a.l, a.lse2Scratch,
            a.dTermScratch, rows, static_cast<int>(a.numHeads), a.newLen, static_cast<int>(a.headDim), a.ldO, a.ldDo, dScale);
    }
    BFB_LAUNCH_CHECK();
    noteLaunch();
    if (tensorCores) {
        BFB_CUDA(cudaMemset2DAsync(a.dQ, static_cast<size_t>(a.ldDq) * 4, 0, static_cast<size_t>(a.numHeads * a.headDim) * 4,
                                   static_cast<size_t>(a.batch) * a.newLen, stream));
        const int64_t dim = a.numHeads * a.headDim;
        TensorMapStorage tq, tk, tv, tg, tdq;
        {
            uint64_t dims[3] = {static_cast<uint64_t>(dim), static_cast<uint64_t>(a.newLen), static_cast<uint64_t>(a.batch)};
            uint64_t strides[2] = {static_cast<uint64_t>(a.ldDq) * 4, static_cast<uint64_t>(a.ldDq) * 4 * static_cast<uint64_t>(a.newLen)};
            uint32_t box[3] = {32u, 128u, 1u};
            encodeTensorMap(&tdq, a.dQ, 4, 3, dims, strides, box);
        }
        makeMap3(&tq, a.q, dim, a.newLen, a.batch, a.ldQ);
        makeMap3(&tk, a.k, dim, a.totalLen, a.batch, a.ldK);
        makeMap3(&tv, a.v, dim, a.totalLen, a.batch, a.ldV);
        makeMap3(&tg, a.dOut, dim, a.newLen, a.batch, a.ldDo);
        BwdParams p;
        p.dQ = a.dQ;
        p.dK = a.dK;
        p.dV = a.dV;
        p.lse2 = a.lse2Scratch;
        p.dTerm = a.dTermScratch;
        p.batch = static_cast<int>(a.batch);
        p.newLen = static_cast<int>(a.newLen);
        p.totalLen = static_cast<int>(a.totalLen);
        p.numHeads = static_cast<int>(a.numHeads);
        p.ldDq = a.ldDq;
        p.ldDk = a.ldDk;
        p.ldDv = a.ldDv;
        p.scale = a.scale;
        p.scaleLog2 = a.scale * 1.4426950408889634f;
        p.oldLen = static_cast<int>(a.oldLen);
        p.causal = a.causal;
        p.numKvBlocks = static_cast<int>((a.totalLen + kBlk - 1) / kBlk);
        p.prefetchAhead = smCount();   // one CTA per SM is resident
        const int64_t blocks = static_cast<int64_t>(p.numKvBlocks) * a.batch * a.numHeads;
        require(blocks <= 0x7FFFFFFF, "attention_bwd: too many key blocks for one launch");
        BFB_CUDA(cudaFuncSetAttribute(attentionBackwardTcKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        attentionBackwardTcKernel<<<static_cast<unsigned>(blocks), kThreads, kSmemBytes, stream>>>(
            *reinterpret_cast<const CUtensorMap*>(tq.bytes), *reinterpret_cast<const CUtensorMap*>(tk.bytes),
            *reinterpret_cast<const CUtensorMap*>(tv.bytes), *reinterpret_cast<const CUtensorMap*>(tg.bytes),
            *reinterpret_cast<const CUtensorMap*>(tdq.bytes), p, a.dStatus);
        BFB_LAUNCH_CHECK();
        noteLaunch();
        return;
    }
    const unsigned blocks = static_cast<unsigned>((rows * 32 + threads - 1) / threads);
    auto launch = [&](auto tag) {
        using T = decltype(tag);
        attentionBackwardSimtKernel<T><<<blocks, threads, 0, stream>>>(
            static_cast<const T*>(a.q), static_cast<const T*>(a.k), static_cast<const T*>(a.v), static_cast<const T*>(a.dOut),
            a.lse2Scratch, a.dTermScratch, a.dQ, a.dK, a.dV, rows, static_cast<int>(a.numHeads), a.newLen, a.totalLen,
            static_cast<int>(a.headDim), a.ldQ, a.ldK, a.ldV, a.ldDo, a.ldDq, a.ldDk, a.ldDv, a.scale, a.oldLen, a.causal);
    };
    if (a.dtype == BFB_F32) launch(float{}); else launch(__nv_bfloat16{});
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

}  // namespace bfb
