// tcgen05 GEMM for sm_100a: C[M,N] = epilogue(alpha * A[M,K] * B), bf16 or e4m3 operands, fp32
// accumulation in tensor memory.
//
// One persistent CTA per SM walks 128x256 output tiles. Warp roles:
//   warp 0      TMA producer: 128-byte-swizzled A (128 x 128 B) and B (256 x 128 B) slices into a
//               4-stage shared-memory ring, completion counted on mbarriers
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (128x256x16 for bf16, x32 for e4m3)
//               into one of two 256-column TMEM accumulators, commits stage release + tile completion
//   warp 2      TMEM allocation / release
//   warps 4-7   epilogue: tcgen05.ld the finished accumulator (row per thread), apply alpha, bias,
//               silu, residual, convert and store, while the MMA warp already fills the other buffer
// Tiles are ordered in groups of N-tiles so that the B slices of a group stay in L2 while A streams
// through once per group. Every mbarrier wait is bounded; on expiry the CTA unwinds and reports
// through the status word.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "kernels.hpp"
#include "ptx_sm100.cuh"

namespace bfb {

namespace {

constexpr int kBlockM = 128;
constexpr int kBlockN = 256;
constexpr int kRowBytes = 128;  // one swizzle atom of K per stage (64 bf16 or 128 e4m3)
constexpr int kStages = 4;
constexpr int kABytes = kBlockM * kRowBytes;  // 16 KiB
constexpr int kBBytes = kBlockN * kRowBytes;  // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kTmemCols = 512;  // two 256-column accumulators
constexpr int kThreads = 256;
constexpr int kEpilogueThreads = 128;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;

struct TileCoord {
    int m, n;
};

// Group N-tiles so that a group's B slices stay L2-resident while all M-tiles sweep past them.
__device__ __forceinline__ TileCoord tileCoord(int t, int tilesM, int tilesN, int groupN) {
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
    TileCoord c;
    c.m = r / width;
    c.n = g * groupN + r % width;
    return c;
}

struct EpilogueParams {
    void* c;
    const float* bias;
    const void* residual;
    float alpha;
    const float* dAlpha;
    int epilogue;
    int roundCBf16;
};

__device__ __forceinline__ float siluDev(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// kElemBytes: 2 (bf16, kind::f16) or 1 (e4m3, kind::f8f6f4). kBMnMajor: B given as [K,N] row-major.
template <int kElemBytes, bool kBMnMajor, typename TC>
__global__ void __launch_bounds__(kThreads, 1)
gemmTcKernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB, EpilogueParams ep,
             int m, int n, int k, int tilesM, int tilesN, int groupN, int* status) {
    constexpr int kBlockK = kRowBytes / kElemBytes;  // elements of K per stage
    constexpr int kUmmaK = 32 / kElemBytes;          // K per tcgen05.mma
    constexpr int kMmaPerStage = kBlockK / kUmmaK;   // 4
    constexpr uint32_t kIdesc = make_idesc(kBlockM, kBlockN, kElemBytes == 2 ? 1u : 0u, kBMnMajor ? 1u : 0u);

    extern __shared__ uint8_t smemRaw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
    uint64_t* fullBar = bars;                   // [kStages] TMA bytes landed
    uint64_t* emptyBar = bars + kStages;        // [kStages] MMAs that read the stage are done
    uint64_t* accFullBar = bars + 2 * kStages;  // [2] accumulator complete
    uint64_t* accEmptyBar = accFullBar + 2;     // [2] epilogue drained the accumulator
    uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(accEmptyBar + 2);
    volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int numK = (k + kBlockK - 1) / kBlockK;
    const int totalTiles = tilesM * tilesN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&fullBar[s], 1);
            mbar_init(&emptyBar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&accFullBar[b], 1);
            mbar_init(&accEmptyBar[b], kEpilogueThreads);
        }
        *abortFlag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmapA);
        tma_prefetch_desc(&tmapB);
    }
    if (warp == 2) {
        tmem_alloc(tmemSlot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmemBase = *tmemSlot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        int stage = 0;
        uint32_t phase = 0;
        bool alive = true;
        for (int t = blockIdx.x; t < totalTiles && alive; t += gridDim.x) {
            TileCoord tc = tileCoord(t, tilesM, tilesN, groupN);
            for (int kb = 0; kb < numK; ++kb) {
                if (!warp_all(mbar_wait(&emptyBar[stage], phase ^ 1u, abortFlag, status, kDevTimeoutStageEmpty))) {
                    alive = false;
                    break;
                }
                if (lane == 0) {
                    uint8_t* sa = smem + stage * kStageBytes;
                    uint8_t* sb = sa + kABytes;
                    mbar_arrive_expect_tx(&fullBar[stage], kStageBytes);
                    tma_load_2d(sa, &tmapA, &fullBar[stage], kb * kBlockK, tc.m * kBlockM);
                    if constexpr (kBMnMajor) {
                        // four [kBlockK rows x 64 columns] boxes, one per 64-wide slice of N
#pragma unroll
                        for (int nb = 0; nb < kBlockN / 64; ++nb) {
                            tma_load_2d(sb + nb * (kBlockK * kRowBytes), &tmapB, &fullBar[stage],
                                        tc.n * kBlockN + nb * 64, kb * kBlockK);
                        }
                    } else {
                        tma_load_2d(sb, &tmapB, &fullBar[stage], kb * kBlockK, tc.n * kBlockN);
                    }
                }
                __syncwarp();
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        int stage = 0;
        uint32_t phase = 0;
        int local = 0;
        bool alive = true;
        for (int t = blockIdx.x; t < totalTiles && alive; t += gridDim.x, ++local) {
            const int buf = local & 1;
            const uint32_t accPhase = (local >> 1) & 1u;
            if (!warp_all(mbar_wait(&accEmptyBar[buf], accPhase ^ 1u, abortFlag, status, kDevTimeoutAccEmpty))) break;
            tc_fence_after();
            const uint32_t dTmem = tmemBase + static_cast<uint32_t>(buf * kBlockN);
            for (int kb = 0; kb < numK; ++kb) {
                if (!warp_all(mbar_wait(&fullBar[stage], phase, abortFlag, status, kDevTimeoutTmaFull))) {
                    alive = false;
                    break;
                }
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t aAddr = smem_u32(smem + stage * kStageBytes);
                    const uint32_t bAddr = aAddr + kABytes;
                    // K-major tiles: 8-row groups are 1024 B apart; MN-major B: 8 k-rows are 1024 B
                    // apart, consecutive 64-wide N slices are kBlockK * 128 B apart.
                    const uint64_t aDesc = make_smem_desc_sw128(aAddr, 0, 1024);
                    const uint64_t bDesc = kBMnMajor ? make_smem_desc_sw128(bAddr, kBlockK * kRowBytes, 1024)
                                                     : make_smem_desc_sw128(bAddr, 0, 1024);
#pragma unroll
                    for (int kk = 0; kk < kMmaPerStage; ++kk) {
                        const uint64_t aStep = static_cast<uint64_t>((kk * 32) >> 4);
                        const uint64_t bStep = kBMnMajor ? static_cast<uint64_t>((kk * kUmmaK * kRowBytes) >> 4)
                                                         : static_cast<uint64_t>((kk * 32) >> 4);
                        const uint32_t acc = (kb > 0 || kk > 0) ? 1u : 0u;
                        if constexpr (kElemBytes == 2) umma_f16(dTmem, aDesc + aStep, bDesc + bStep, kIdesc, acc);
                        else umma_f8(dTmem, aDesc + aStep, bDesc + bStep, kIdesc, acc);
                    }
                    umma_commit(&emptyBar[stage]);
                    if (kb == numK - 1) umma_commit(&accFullBar[buf]);
                }
                __syncwarp();
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp >= 4) {
        // ---------------- epilogue ----------------
        const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter + 32) belong to this warp
        const float scale = ep.dAlpha != nullptr ? *ep.dAlpha : ep.alpha;
        const bool hasBias =
            ep.epilogue == BFB_EPI_BIAS || ep.epilogue == BFB_EPI_BIAS_SILU || ep.epilogue == BFB_EPI_BIAS_RESIDUAL;
        const bool hasSilu = ep.epilogue == BFB_EPI_BIAS_SILU;
        const bool hasRes = ep.epilogue == BFB_EPI_BIAS_RESIDUAL || ep.epilogue == BFB_EPI_RESIDUAL;
        TC* cOut = static_cast<TC*>(ep.c);
        const TC* res = static_cast<const TC*>(ep.residual);
        int local = 0;
        for (int t = blockIdx.x; t < totalTiles; t += gridDim.x, ++local) {
            TileCoord tc = tileCoord(t, tilesM, tilesN, groupN);
            const int buf = local & 1;
            const uint32_t accPhase = (local >> 1) & 1u;
            if (!warp_all(mbar_wait(&accFullBar[buf], accPhase, abortFlag, status, kDevTimeoutAccFull))) break;
            tc_fence_after();
            const int row = tc.m * kBlockM + quarter * 32 + lane;
            const bool rowOk = row < m;
            const uint32_t tBase = tmemBase + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(buf * kBlockN);
#pragma unroll 1
            for (int chunk = 0; chunk < kBlockN / 32; ++chunk) {
                const int col0 = tc.n * kBlockN + chunk * 32;
                if (col0 >= n) break;  // uniform across the CTA
                uint32_t raw[32];
                tmem_ld_32x32(tBase + static_cast<uint32_t>(chunk * 32), raw);
                tmem_ld_wait();
                if (rowOk) {
                    const size_t rowOff = static_cast<size_t>(row) * static_cast<size_t>(n);
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const int col = col0 + g * 8;
                        if (col + 8 > n) break;
                        float v[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(raw[g * 8 + j]) * scale;
                        if (hasBias) {
                            const float4 b0 = __ldg(reinterpret_cast<const float4*>(ep.bias + col));
                            const float4 b1 = __ldg(reinterpret_cast<const float4*>(ep.bias + col + 4));
                            v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
                            v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
                        }
                        if (hasSilu) {
#pragma unroll
                            for (int j = 0; j < 8; ++j) v[j] = siluDev(v[j]);
                        }
                        if constexpr (sizeof(TC) == 4) {
                            if (hasRes) {
                                const float4 r0 = *reinterpret_cast<const float4*>(res + rowOff + col);
                                const float4 r1 = *reinterpret_cast<const float4*>(res + rowOff + col + 4);
                                v[0] += r0.x; v[1] += r0.y; v[2] += r0.z; v[3] += r0.w;
                                v[4] += r1.x; v[5] += r1.y; v[6] += r1.z; v[7] += r1.w;
                            }
                            if (ep.roundCBf16) {
#pragma unroll
                                for (int j = 0; j < 8; ++j) v[j] = __bfloat162float(__float2bfloat16_rn(v[j]));
                            }
                            float4* dst = reinterpret_cast<float4*>(cOut + rowOff + col);
                            dst[0] = make_float4(v[0], v[1], v[2], v[3]);
                            dst[1] = make_float4(v[4], v[5], v[6], v[7]);
                        } else {
                            if (hasRes) {
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
                            }
                            *reinterpret_cast<uint4*>(cOut + rowOff + col) = packed;
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&accEmptyBar[buf]);
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        if (*abortFlag != 0) {
            // give copies / MMAs still in flight time to land before the columns are handed back
            uint64_t t0 = global_timer_ns();
            while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
        tc_fence_after();
        tmem_dealloc(tmemBase, kTmemCols);
    }
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encodeFn() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
        if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeFn>(p);
    });
    if (fn == nullptr) fail(BFB_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
    return fn;
}

template <int kElemBytes, bool kBMnMajor, typename TC>
void launchTc(const GemmArgs& g, cudaStream_t stream) {
    constexpr int kBlockK = kRowBytes / kElemBytes;
    TensorMapStorage ta, tb;
    {
        uint64_t dims[2] = {static_cast<uint64_t>(g.k), static_cast<uint64_t>(g.m)};
        uint64_t strides[1] = {static_cast<uint64_t>(g.k) * kElemBytes};
        uint32_t box[2] = {static_cast<uint32_t>(kBlockK), static_cast<uint32_t>(kBlockM)};
        encodeTensorMap(&ta, g.a, kElemBytes, 2, dims, strides, box);
    }
    if (kBMnMajor) {
        uint64_t dims[2] = {static_cast<uint64_t>(g.n), static_cast<uint64_t>(g.k)};
        uint64_t strides[1] = {static_cast<uint64_t>(g.n) * kElemBytes};
        uint32_t box[2] = {64u, static_cast<uint32_t>(kBlockK)};
        encodeTensorMap(&tb, g.b, kElemBytes, 2, dims, strides, box);
    } else {
        uint64_t dims[2] = {static_cast<uint64_t>(g.k), static_cast<uint64_t>(g.n)};
        uint64_t strides[1] = {static_cast<uint64_t>(g.k) * kElemBytes};
        uint32_t box[2] = {static_cast<uint32_t>(kBlockK), static_cast<uint32_t>(kBlockN)};
        encodeTensorMap(&tb, g.b, kElemBytes, 2, dims, strides, box);
    }
    int tilesM = static_cast<int>((g.m + kBlockM - 1) / kBlockM);
    int tilesN = static_cast<int>((g.n + kBlockN - 1) / kBlockN);
    int groups = (tilesN + 15) / 16;
    int groupN = (tilesN + groups - 1) / groups;
    int grid = std::min(tilesM * tilesN, persistentSms());
    EpilogueParams ep{g.c, g.bias, g.residual, g.alpha, g.dAlpha, g.epilogue, g.roundCBf16};
    auto kernel = gemmTcKernel<kElemBytes, kBMnMajor, TC>;
    // per device, so set on every launch (the process may have switched devices)
    BFB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    ProfileScope prof(kProfGemmTc, stream, 2.0 * static_cast<double>(g.m) * static_cast<double>(g.n) * static_cast<double>(g.k));
    kernel<<<grid, kThreads, kSmemBytes, stream>>>(*reinterpret_cast<CUtensorMap*>(ta.bytes),
                                                   *reinterpret_cast<CUtensorMap*>(tb.bytes), ep,
                                                   static_cast<int>(g.m), static_cast<int>(g.n), static_cast<int>(g.k),
                                                   tilesM, tilesN, groupN, g.dStatus);
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

}  // namespace

void encodeTensorMap(TensorMapStorage* out, const void* base, int elemBytes, int rank, const uint64_t* dims,
                     const uint64_t* stridesBytes, const uint32_t* box) {
    cuuint64_t gdims[5];
    cuuint64_t gstrides[4];
    cuuint32_t gbox[5];
    cuuint32_t estr[5];
    for (int i = 0; i < rank; ++i) {
        gdims[i] = dims[i];
        gbox[i] = box[i];
        estr[i] = 1;
        if (i > 0) gstrides[i - 1] = stridesBytes[i - 1];
    }
    CUtensorMapDataType dt = elemBytes == 4   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                             : elemBytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                              : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    CUresult r = encodeFn()(reinterpret_cast<CUtensorMap*>(out->bytes), dt, static_cast<cuuint32_t>(rank),
                            const_cast<void*>(base), gdims, gstrides, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        fail(BFB_CUDA_ERROR, "cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(r)));
    }
}

bool gemmUsesTensorCores(const GemmArgs& g) {
    if (g.abDtype != BFB_BF16 && g.abDtype != BFB_FP8_E4M3) return false;
    const int64_t elem = g.abDtype == BFB_BF16 ? 2 : 1;
    const int64_t kAlign = 16 / elem;
    if (g.k < kAlign || g.k % kAlign != 0) return false;  // row pitch of A / B^T must be a multiple of 16 B
    if (g.n % 8 != 0) return false;                        // 16-byte result vectors; [K,N] pitch
    if (g.m < 1 || g.m > 0x7FFFFFFF || g.n > 0x7FFFFFFF || g.k > 0x7FFFFFFF) return false;
    if (g.abDtype == BFB_FP8_E4M3 && g.bLayout != BFB_B_NK) return false;
    auto aligned16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    if (!aligned16(g.a) || !aligned16(g.b) || !aligned16(g.c)) return false;
    if (g.residual != nullptr && !aligned16(g.residual)) return false;
    if (g.bias != nullptr && !aligned16(g.bias)) return false;
    return true;
}

// BFB_GEMM_PAIR=0 in the environment keeps every GEMM on the one-CTA kernel (for A/B measurements).
static bool pairKernelEnabled() {
    static const bool enabled = [] {
        const char* v = std::getenv("BFB_GEMM_PAIR");
        return v == nullptr || v[0] != '0';
    }();
    return enabled;
}

bool gemmSupportsRowStats(const GemmArgs& g) {
    return gemmUsesTensorCores(g) && g.bLayout == BFB_B_NK && pairKernelEnabled() && g.rowSumSqParts >= 1;
}

void gemmTensorCore(const GemmArgs& g, cudaStream_t stream) {
    // CTA pairs share 256-row tiles: worth it once there is more than one 128-row tile of work
    // ... or when row statistics are asked for, which only that kernel has (whatever the number of rows, so that
    // a sequence gives the same bits alone and inside a batch)
    const bool stats = g.rowSumSq != nullptr || g.outSumSq != nullptr || g.outMaxAbs != nullptr;
    if (g.bLayout == BFB_B_NK && (g.m > 128 || stats) && pairKernelEnabled()) {
        gemmTensorCorePair(g, stream);
        return;
    }
    const bool cf32 = g.cDtype == BFB_F32;
    using bf = __nv_bfloat16;
    if (g.abDtype == BFB_BF16) {
        if (g.bLayout == BFB_B_KN) {
            if (cf32) launchTc<2, true, float>(g, stream); else launchTc<2, true, bf>(g, stream);
        } else {
            if (cf32) launchTc<2, false, float>(g, stream); else launchTc<2, false, bf>(g, stream);
        }
    } else {
        if (cf32) launchTc<1, false, float>(g, stream); else launchTc<1, false, bf>(g, stream);
    }
}

}  // namespace bfb
