// tcgen05 GEMM for few rows (M <= 128: one generation step of a batch): C[M,N] = epilogue(A[M,K] * W^T), W [N,K].
//
// With a handful of rows the work is streaming W once, so the kernel is laid out for HBM bandwidth, not for the
// tensor pipe: the WEIGHT rows take the MMA's M side (128 per CTA) and the activation rows its N side (M padded
// to 16, 32, 64 or 128), and K is split across CTAs until about two CTAs per SM stream their own slices of W:
//   grid = ceil(N / 128) x splits, CTA (tile, split) computes W[tile*128 .. +128, k-slice] * A[:, k-slice]^T
//   warp 0      TMA producer: W slice (128 x 128 B, 128-byte swizzle) + A slice (mPad x 128 B) per stage, 3-6 stages
//               (about 100 KB, so that two CTAs share an SM)
//   warp 1      MMA issuer + TMEM owner: tcgen05.mma 128 x mPad x 16 (x32 for e4m3), fp32 accumulator in TMEM
//   warps 2-5   drain: tcgen05.ld the accumulator (lane = weight row = output column) and store the fp32 partial
//               products to a workspace [split][m][N]; for one activation row the 32 lanes write 32 consecutive floats
// A second, elementwise kernel adds the splits in index order (no atomics: the same bits on every run), applies
// row scale (folded rmsnorm), alpha, bias, silu, residual, stores C and, when asked, the per-128-column sums of
// squares of the stored values. Every mbarrier wait is bounded.
//
// Two single-launch forms were built, measured on the generation step of the 2B-class model and dropped: the last CTA
// of a column tile (a global counter) adding the splits from the workspace, 1.95 against 1.36 ms per step for the
// GEMMs; and the splits of a tile as one thread-block cluster (up to 16 CTAs) that leaves its partial tiles in shared
// memory and adds them through distributed shared memory after a cluster barrier, bit-identical but 3.09 against
// 2.62 ms for the whole step: clusters of CTAs with 100 KB of shared memory each place badly, and the dependent-launch
// overlap between consecutive kernels is worth more than the launch saved.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>

#include "common.cuh"
#include "kernels.hpp"
#include "pool.hpp"
#include "ptx_sm100.cuh"

namespace bfb {

namespace {

constexpr int kTileN = 128;                 // weight rows (output columns) per CTA
constexpr int kRowBytesS = 128;             // one swizzle atom of K per stage
constexpr int kMaxStagesS = 6;              // fewer for wider A slices: two CTAs share an SM's shared memory
constexpr int kSmemBudgetS = 110 * 1024;
constexpr int kWBytes = kTileN * kRowBytesS;   // 16 KiB
constexpr int kThreadsS = 192;
constexpr int kDrainWarps = 4;

__host__ __device__ constexpr int skinnyStageBytes(int mPad) { return kWBytes + mPad * kRowBytesS; }

template <int kElemBytes>
__global__ void __launch_bounds__(kThreadsS, 2)
gemmSkinnyKernel(const __grid_constant__ CUtensorMap tmapW, const __grid_constant__ CUtensorMap tmapA, float* ws, int m,
                 int n, int mPad, int tilesN, int numK, int blocksPerSplit, int stages, int* status) {
    constexpr int kBlockK = kRowBytesS / kElemBytes;
    constexpr int kUmmaK = 32 / kElemBytes;
    constexpr int kMmaPerStage = kBlockK / kUmmaK;  // 4

    extern __shared__ uint8_t smemRaw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
    const int stageBytes = skinnyStageBytes(mPad);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + stages * stageBytes);
    uint64_t* fullBar = bars;                 // [stages]
    uint64_t* emptyBar = bars + kMaxStagesS;  // [stages]
    uint64_t* accFullBar = bars + 2 * kMaxStagesS;
    uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(accFullBar + 1);
    volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tile = static_cast<int>(blockIdx.x) % tilesN;
    const int split = static_cast<int>(blockIdx.x) / tilesN;
    const int kbBegin = split * blocksPerSplit;
    const int kbEnd = min(numK, kbBegin + blocksPerSplit);
    const uint32_t tmemCols = mPad < 32 ? 32u : static_cast<uint32_t>(mPad);

    if (threadIdx.x == 0) {
        pdl_launch_dependents();   // the finish kernel may get ready; it waits for this grid before it reads
        for (int s = 0; s < stages; ++s) {
            mbar_init(&fullBar[s], 1);
            mbar_init(&emptyBar[s], 1);
        }
        mbar_init(accFullBar, 1);
        *abortFlag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmapW);
        tma_prefetch_desc(&tmapA);
    }
    if (warp == 1) {
        tmem_alloc(tmemSlot, tmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmemBase = *tmemSlot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        // The weights do not change during a pass, so their tiles of the first ring lap are requested while the
        // kernel before this one may still be running; the activation tiles (its output) follow once it is done.
        // Everything this kernel writes depends on those, so it also writes only after that.
        const int early = min(kbEnd - kbBegin, stages);
        if (lane == 0) {
            for (int it = 0; it < early; ++it) {
                mbar_arrive_expect_tx(&fullBar[it], static_cast<uint32_t>(stageBytes));
                tma_load_2d(smem + it * stageBytes, &tmapW, &fullBar[it], (kbBegin + it) * kBlockK, tile * kTileN);
            }
        }
        pdl_wait();
        if (lane == 0) {
            for (int it = 0; it < early; ++it) {
                tma_load_2d(smem + it * stageBytes + kWBytes, &tmapA, &fullBar[it], (kbBegin + it) * kBlockK, 0);
            }
        }
        __syncwarp();
        for (int kb = kbBegin + early, it = early; kb < kbEnd; ++kb, ++it) {
            const int s = it % stages;
            const uint32_t use = static_cast<uint32_t>(it / stages);
            if (!warp_all(mbar_wait(&emptyBar[s], (use & 1u) ^ 1u, abortFlag, status, kDevTimeoutStageEmpty))) break;
            if (lane == 0) {
                uint8_t* dst = smem + s * stageBytes;
                mbar_arrive_expect_tx(&fullBar[s], static_cast<uint32_t>(stageBytes));
                tma_load_2d(dst, &tmapW, &fullBar[s], kb * kBlockK, tile * kTileN);
                tma_load_2d(dst + kWBytes, &tmapA, &fullBar[s], kb * kBlockK, 0);
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        const uint32_t idesc = make_idesc(kTileN, static_cast<uint32_t>(mPad), kElemBytes == 2 ? 1u : 0u, 0u);
        bool alive = true;
        for (int kb = kbBegin, it = 0; kb < kbEnd; ++kb, ++it) {
            const int s = it % stages;
            const uint32_t use = static_cast<uint32_t>(it / stages);
            if (!warp_all(mbar_wait(&fullBar[s], use & 1u, abortFlag, status, kDevTimeoutTmaFull))) {
                alive = false;
                break;
            }
            tc_fence_after();
            if (lane == 0) {
                const uint32_t wAddr = smem_u32(smem + s * stageBytes);
                const uint32_t aAddr = wAddr + kWBytes;
#pragma unroll
                for (int j = 0; j < kMmaPerStage; ++j) {
                    const uint64_t wDesc = make_smem_desc_sw128(wAddr + j * 32, 0, 1024);
                    const uint64_t aDesc = make_smem_desc_sw128(aAddr + j * 32, 0, 1024);
                    const uint32_t acc = (it > 0 || j > 0) ? 1u : 0u;
                    if constexpr (kElemBytes == 2) umma_f16(tmemBase, wDesc, aDesc, idesc, acc);
                    else umma_f8(tmemBase, wDesc, aDesc, idesc, acc);
                }
                umma_commit(&emptyBar[s]);
            }
            __syncwarp();
        }
        if (alive) {
            if (lane == 0) umma_commit(accFullBar);
            __syncwarp();
        }
    } else {
        // ---------------- drain: accumulator -> fp32 partial products in the workspace ----------------
        const int quarter = warp & 3;   // TMEM lanes this warp may read
        if (warp_all(mbar_wait(accFullBar, 0u, abortFlag, status, kDevTimeoutAccFull))) {
            tc_fence_after();
            const int col = tile * kTileN + quarter * 32 + lane;   // output column = weight row
            const uint32_t tBase = tmemBase + (static_cast<uint32_t>(quarter * 32) << 16);
            float* dst = ws + static_cast<size_t>(split) * static_cast<size_t>(m) * static_cast<size_t>(n) + col;
            for (int c0 = 0; c0 < mPad; c0 += 16) {
                uint32_t raw[16];
                tmem_ld_32x16(tBase + static_cast<uint32_t>(c0), raw);
                tmem_ld_wait();
                if (col < n) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int row = c0 + j;
                        if (row < m) dst[static_cast<size_t>(row) * static_cast<size_t>(n)] = __uint_as_float(raw[j]);
                    }
                }
            }
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        if (*abortFlag != 0) {
            uint64_t t0 = global_timer_ns();
            while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
        tc_fence_after();
        tmem_dealloc(tmemBase, tmemCols);
    }
}

struct FinishParams {
    const float* ws;
    int splits;
    void* c;
    const float* bias;
    const void* residual;
    float alpha;
    const float* dAlpha;
    int epilogue;
    int roundCBf16;
    const float* rowSumSq;
    int rowSumSqParts;
    float rowInvDim;
    float rowEps;
    float* outSumSq;
};

__device__ __forceinline__ float siluSkinny(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// One warp per (row, 128-column part); a lane owns 4 consecutive columns.
template <typename TC>
__global__ void __launch_bounds__(256)
skinnyFinishKernel(FinishParams p, int m, int n, int parts) {
    if (threadIdx.x == 0) pdl_launch_dependents();
    pdl_wait();   // the partial products come from the kernel before
    const int lane = threadIdx.x & 31;
    const int unit = static_cast<int>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (unit >= m * parts) return;
    const int row = unit / parts;
    const int part = unit - row * parts;
    const int col = part * 128 + lane * 4;
    const bool hasBias = p.epilogue == BFB_EPI_BIAS || p.epilogue == BFB_EPI_BIAS_SILU || p.epilogue == BFB_EPI_BIAS_RESIDUAL;
    const bool hasSilu = p.epilogue == BFB_EPI_BIAS_SILU;
    const bool hasRes = p.epilogue == BFB_EPI_BIAS_RESIDUAL || p.epilogue == BFB_EPI_RESIDUAL;
    float scale = p.dAlpha != nullptr ? *p.dAlpha : p.alpha;
    if (p.rowSumSq != nullptr) {
        float total = 0.0f;
        for (int q = 0; q < p.rowSumSqParts; ++q) total += __ldg(p.rowSumSq + static_cast<size_t>(q) * m + row);
        scale = scale / sqrtf(total * p.rowInvDim + p.rowEps);
    }
    float sumSq = 0.0f;
    if (col < n) {   // n is a multiple of 8, so the 4 columns are in or out together
        const size_t off = static_cast<size_t>(row) * static_cast<size_t>(n) + col;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int s = 0; s < p.splits; ++s) {   // splits in index order
            const float4 v = *reinterpret_cast<const float4*>(p.ws + static_cast<size_t>(s) * m * n + off);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        float v[4] = {acc.x * scale, acc.y * scale, acc.z * scale, acc.w * scale};
        if (hasBias) {
            const float4 b = __ldg(reinterpret_cast<const float4*>(p.bias + col));
            v[0] += b.x; v[1] += b.y; v[2] += b.z; v[3] += b.w;
        }
        if (hasSilu) {
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = siluSkinny(v[j]);
        }
        if constexpr (sizeof(TC) == 4) {
            float* c = static_cast<float*>(p.c);
            if (hasRes) {
                const float4 r = *reinterpret_cast<const float4*>(static_cast<const float*>(p.residual) + off);
                v[0] += r.x; v[1] += r.y; v[2] += r.z; v[3] += r.w;
            }
            if (p.roundCBf16) {
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = __bfloat162float(__float2bfloat16_rn(v[j]));
            }
            *reinterpret_cast<float4*>(c + off) = make_float4(v[0], v[1], v[2], v[3]);
#pragma unroll
            for (int j = 0; j < 4; ++j) sumSq = fmaf(v[j], v[j], sumSq);
        } else {
            __nv_bfloat16* c = static_cast<__nv_bfloat16*>(p.c);
            if (hasRes) {
                const uint2 rr = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p.residual) + off);
                const __nv_bfloat162* rh = reinterpret_cast<const __nv_bfloat162*>(&rr);
                const float2 r0 = __bfloat1622float2(rh[0]), r1 = __bfloat1622float2(rh[1]);
                v[0] += r0.x; v[1] += r0.y; v[2] += r1.x; v[3] += r1.y;
            }
            uint2 packed;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(v[2], v[3]);
            packed.x = *reinterpret_cast<uint32_t*>(&h0);
            packed.y = *reinterpret_cast<uint32_t*>(&h1);
            *reinterpret_cast<uint2*>(c + off) = packed;
            const float2 f0 = __bfloat1622float2(h0), f1 = __bfloat1622float2(h1);   // the values as stored
            sumSq = fmaf(f0.x, f0.x, fmaf(f0.y, f0.y, fmaf(f1.x, f1.x, fmaf(f1.y, f1.y, sumSq))));
        }
    }
    if (p.outSumSq != nullptr) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sumSq += __shfl_xor_sync(0xFFFFFFFFu, sumSq, o);
        if (lane == 0) p.outSumSq[static_cast<size_t>(part) * m + row] = sumSq;
    }
}

int padRows(int64_t m) { return m <= 16 ? 16 : (m <= 32 ? 32 : (m <= 64 ? 64 : 128)); }

struct SkinnyPlan {
    int mPad, tilesN, numK, splits, blocksPerSplit, stages;
};

SkinnyPlan planSkinny(const GemmArgs& g) {
    const int elem = g.abDtype == BFB_BF16 ? 2 : 1;
    const int blockK = kRowBytesS / elem;
    SkinnyPlan p;
    p.mPad = padRows(g.m);
    p.tilesN = static_cast<int>((g.n + kTileN - 1) / kTileN);
    p.numK = static_cast<int>((g.k + blockK - 1) / blockK);
    // two CTAs fit on an SM: as many splits as keep all CTAs resident at once (one wave). The split depends on N and
    // K only, so a row gives the same bits whatever rows sit beside it
    p.stages = std::max(2, std::min(kMaxStagesS, kSmemBudgetS / skinnyStageBytes(p.mPad)));
    int splits = std::max(1, std::min({2 * smCount() / p.tilesN, p.numK, 16}));
    p.blocksPerSplit = (p.numK + splits - 1) / splits;
    p.splits = (p.numK + p.blocksPerSplit - 1) / p.blocksPerSplit;
    return p;
}

template <int kElemBytes>
void launchSkinny(const GemmArgs& g, const SkinnyPlan& p, float* ws, cudaStream_t stream) {
    constexpr int kBlockK = kRowBytesS / kElemBytes;
    TensorMapStorage tw, ta;
    {
        uint64_t dims[2] = {static_cast<uint64_t>(g.k), static_cast<uint64_t>(g.n)};
        uint64_t strides[1] = {static_cast<uint64_t>(g.k) * kElemBytes};
        uint32_t box[2] = {static_cast<uint32_t>(kBlockK), static_cast<uint32_t>(kTileN)};
        encodeTensorMap(&tw, g.b, kElemBytes, 2, dims, strides, box);
    }
    {
        uint64_t dims[2] = {static_cast<uint64_t>(g.k), static_cast<uint64_t>(g.m)};
        uint64_t strides[1] = {static_cast<uint64_t>(g.k) * kElemBytes};
        uint32_t box[2] = {static_cast<uint32_t>(kBlockK), static_cast<uint32_t>(p.mPad)};
        encodeTensorMap(&ta, g.a, kElemBytes, 2, dims, strides, box);
    }
    const int smemBytes = p.stages * skinnyStageBytes(p.mPad) + 1024 + 256;
    auto kernel = gemmSkinnyKernel<kElemBytes>;
    BFB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smemBytes));
    launchDependent(kernel, dim3(static_cast<unsigned>(p.tilesN * p.splits)), dim3(kThreadsS), static_cast<size_t>(smemBytes),
                    stream, *reinterpret_cast<CUtensorMap*>(tw.bytes), *reinterpret_cast<CUtensorMap*>(ta.bytes), ws,
                    static_cast<int>(g.m), static_cast<int>(g.n), p.mPad, p.tilesN, p.numK, p.blocksPerSplit, p.stages,
                    g.dStatus);
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

}  // namespace

bool gemmSkinnyEligible(const GemmArgs& g) {
    return g.m >= 1 && g.m <= 128 && g.bLayout == BFB_B_NK && g.k > 0 && gemmUsesTensorCores(g);
}

int64_t gemmSkinnyWorkspaceBytes(const GemmArgs& g) {
    const SkinnyPlan p = planSkinny(g);
    return static_cast<int64_t>(p.splits) * g.m * g.n * static_cast<int64_t>(sizeof(float));
}

void gemmSkinny(const GemmArgs& g, cudaStream_t stream) {
    require(gemmSkinnyEligible(g), "gemm: the few-rows kernel needs 1..128 rows, [N,K] weights and tensor-core formats");
    const SkinnyPlan p = planSkinny(g);
    const size_t need = static_cast<size_t>(gemmSkinnyWorkspaceBytes(g));
    float* ws = static_cast<float*>(g.workspace);
    bool own = false;
    if (ws == nullptr || g.workspaceBytes < need) {
        ws = static_cast<float*>(poolAcquire(need));
        own = true;
    }
    try {
        // work figure: the bytes of W, which is what this kernel is about
        ProfileScope prof(kProfGemmTc, stream, 2.0 * static_cast<double>(g.m) * static_cast<double>(g.n) * static_cast<double>(g.k));
        if (g.abDtype == BFB_BF16) launchSkinny<2>(g, p, ws, stream);
        else launchSkinny<1>(g, p, ws, stream);
        FinishParams f{ws, p.splits, g.c, g.bias, g.residual, g.alpha, g.dAlpha, g.epilogue, g.roundCBf16,
                       g.rowSumSq, g.rowSumSqParts, g.rowInvDim, g.rowEps, g.outSumSq};
        const int parts = static_cast<int>((g.n + 127) / 128);
        const int units = static_cast<int>(g.m) * parts;
        const int grid = (units + 7) / 8;
        if (g.cDtype == BFB_F32) {
            launchDependent(skinnyFinishKernel<float>, dim3(grid), dim3(256), 0, stream, f, static_cast<int>(g.m),
                            static_cast<int>(g.n), parts);
        } else {
            launchDependent(skinnyFinishKernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, f, static_cast<int>(g.m),
                            static_cast<int>(g.n), parts);
        }
        BFB_LAUNCH_CHECK();
        noteLaunch();
    } catch (...) {
        if (own) poolRelease(ws, need);
        throw;
    }
    // work on `stream` is ordered before any later use of the buffer on the same stream
    if (own) poolRelease(ws, need);
}

}  // namespace bfb
