// CUDA-core GEMM: the exactness path (fp32 operands, fp32 accumulation in ascending-k order, as the
// reference's CPU loops and cublasSgemm contract) and the any-shape path for bf16 / e4m3 operands the
// tensor-core kernel's alignment rules exclude. 64x64 output tile, 16-deep k slices, 4x4 per thread.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "kernels.hpp"
#include "pool.hpp"

namespace bfb {

namespace {

constexpr int kTileM = 64, kTileN = 64, kTileK = 16;

template <typename T>
__device__ __forceinline__ float ldElem(const void* p, int64_t i);
template <>
__device__ __forceinline__ float ldElem<float>(const void* p, int64_t i) { return static_cast<const float*>(p)[i]; }
template <>
__device__ __forceinline__ float ldElem<__nv_bfloat16>(const void* p, int64_t i) {
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}
template <>
__device__ __forceinline__ float ldElem<__nv_fp8_e4m3>(const void* p, int64_t i) {
    return static_cast<float>(static_cast<const __nv_fp8_e4m3*>(p)[i]);
}

__device__ __forceinline__ float siluDev(float x) { return x / (1.0f + expf(-x)); }

template <typename TAb, typename TC>
__global__ void __launch_bounds__(256)
gemmSimtKernel(const void* __restrict__ a, const void* __restrict__ b, TC* c, int64_t m, int64_t n,
               int64_t k, int bLayout, int epilogue, const float* __restrict__ bias, const TC* residual,
               float alpha, const float* __restrict__ dAlpha, int roundCBf16) {
    __shared__ float sa[kTileK][kTileM + 1];
    __shared__ float sb[kTileK][kTileN + 1];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, each owns a 4x4 block
    const int64_t tilesN = (n + kTileN - 1) / kTileN;
    const int64_t tilesM = (m + kTileM - 1) / kTileM;
    const float scale = dAlpha != nullptr ? *dAlpha : alpha;

    for (int64_t tile = blockIdx.x; tile < tilesM * tilesN; tile += gridDim.x) {
        const int64_t m0 = (tile / tilesN) * kTileM, n0 = (tile % tilesN) * kTileN;
        float acc[4][4] = {};
        for (int64_t k0 = 0; k0 < k; k0 += kTileK) {
            __syncthreads();
            for (int i = tid; i < kTileM * kTileK; i += 256) {
                int r = i / kTileK, kk = i % kTileK;
                int64_t gm = m0 + r, gk = k0 + kk;
                sa[kk][r] = (gm < m && gk < k) ? ldElem<TAb>(a, gm * k + gk) : 0.0f;
            }
            if (bLayout == BFB_B_KN) {
                for (int i = tid; i < kTileN * kTileK; i += 256) {
                    int kk = i / kTileN, cidx = i % kTileN;
                    int64_t gk = k0 + kk, gn = n0 + cidx;
                    sb[kk][cidx] = (gk < k && gn < n) ? ldElem<TAb>(b, gk * n + gn) : 0.0f;
                }
            } else {
                for (int i = tid; i < kTileN * kTileK; i += 256) {
                    int cidx = i / kTileK, kk = i % kTileK;
                    int64_t gk = k0 + kk, gn = n0 + cidx;
                    sb[kk][cidx] = (gk < k && gn < n) ? ldElem<TAb>(b, gn * k + gk) : 0.0f;
                }
            }
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < kTileK; ++kk) {
                float av[4], bv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
                for (int j = 0; j < 4; ++j) bv[j] = sb[kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int64_t gm = m0 + ty * 4 + i;
            if (gm >= m) continue;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int64_t gn = n0 + tx * 4 + j;
                if (gn >= n) continue;
                float v = acc[i][j] * scale;
                if (epilogue == BFB_EPI_BIAS || epilogue == BFB_EPI_BIAS_SILU || epilogue == BFB_EPI_BIAS_RESIDUAL)
                    v += bias[gn];
                if (epilogue == BFB_EPI_BIAS_SILU) v = siluDev(v);
                if (epilogue == BFB_EPI_BIAS_RESIDUAL || epilogue == BFB_EPI_RESIDUAL) {
                    if constexpr (sizeof(TC) == 4) v += residual[gm * n + gn];
                    else v += __bfloat162float(residual[gm * n + gn]);
                }
                if constexpr (sizeof(TC) == 4) {
                    c[gm * n + gn] = roundCBf16 ? __bfloat162float(__float2bfloat16_rn(v)) : v;
                } else {
                    c[gm * n + gn] = __float2bfloat16_rn(v);
                }
            }
        }
    }
}

__global__ void matmulTransposeBKernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
                                       int64_t m, int64_t n, int64_t k) {
    int64_t total = m * n;
    int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        int64_t i = idx / n, j = idx % n;
        float s = 0.0f;
        for (int64_t p = 0; p < k; ++p) s = fmaf(a[i * k + p], b[j * k + p], s);
        c[idx] = s;
    }
}

template <typename TAb, typename TC>
void launchSimt(const GemmArgs& g, cudaStream_t stream) {
    int64_t tiles = ((g.m + kTileM - 1) / kTileM) * ((g.n + kTileN - 1) / kTileN);
    int grid = static_cast<int>(std::min<int64_t>(tiles, static_cast<int64_t>(smCount()) * 16));
    gemmSimtKernel<TAb, TC><<<grid, 256, 0, stream>>>(g.a, g.b, static_cast<TC*>(g.c), g.m, g.n, g.k, g.bLayout,
                                                       g.epilogue, g.bias, static_cast<const TC*>(g.residual), g.alpha,
                                                       g.dAlpha, g.roundCBf16);
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

}  // namespace

void gemm(const GemmArgs& g, cudaStream_t stream) {
    require(g.m >= 0 && g.n >= 0 && g.k >= 0, "gemm: negative size");
    require(g.abDtype == BFB_F32 || g.abDtype == BFB_BF16 || g.abDtype == BFB_FP8_E4M3, "gemm: unknown operand format");
    require(g.cDtype == BFB_F32 || g.cDtype == BFB_BF16, "gemm: result format must be f32 or bf16");
    require(g.bLayout == BFB_B_KN || g.bLayout == BFB_B_NK, "gemm: unknown B layout");
    require(g.epilogue >= BFB_EPI_NONE && g.epilogue <= BFB_EPI_RESIDUAL, "gemm: unknown epilogue");
    if (g.abDtype == BFB_FP8_E4M3) require(g.bLayout == BFB_B_NK, "gemm: e4m3 operands need the [N,K] weight layout");
    bool needsBias = g.epilogue == BFB_EPI_BIAS || g.epilogue == BFB_EPI_BIAS_SILU || g.epilogue == BFB_EPI_BIAS_RESIDUAL;
    bool needsRes = g.epilogue == BFB_EPI_BIAS_RESIDUAL || g.epilogue == BFB_EPI_RESIDUAL;
    if (g.m == 0 || g.n == 0) return;
    require(g.c != nullptr, "gemm: null result pointer");
    if (g.k > 0) require(g.a != nullptr && g.b != nullptr, "gemm: null operand pointer");
    if (needsBias) require(g.bias != nullptr, "gemm: bias missing");
    if (needsRes) require(g.residual != nullptr, "gemm: residual missing");

    if (g.preferSkinny != 0 && g.outMaxAbs == nullptr && gemmSkinnyEligible(g)) {
        gemmSkinny(g, stream);
        return;
    }
    if ((g.rowSumSq != nullptr || g.outSumSq != nullptr || g.outMaxAbs != nullptr) && !gemmSupportsRowStats(g)) {
        fail(BFB_UNSUPPORTED, "gemm: row statistics need the CTA-pair tensor-core kernel (bf16 or e4m3 operands, [N,K] weights, 16-byte aligned rows)");
    }
    if (gemmUsesTensorCores(g)) {
        gemmTensorCore(g, stream);
        return;
    }
    bool cf32 = g.cDtype == BFB_F32;
    using bf = __nv_bfloat16;
    using f8 = __nv_fp8_e4m3;
    if (g.abDtype == BFB_F32) {
        if (cf32) launchSimt<float, float>(g, stream); else launchSimt<float, bf>(g, stream);
    } else if (g.abDtype == BFB_BF16) {
        if (cf32) launchSimt<bf, float>(g, stream); else launchSimt<bf, bf>(g, stream);
    } else {
        if (cf32) launchSimt<f8, float>(g, stream); else launchSimt<f8, bf>(g, stream);
    }
}

namespace {
struct PoolScratch {
    void* ptr;
    size_t bytes;
    explicit PoolScratch(size_t b) : ptr(poolAcquire(b)), bytes(b) {}
    ~PoolScratch() { poolRelease(ptr, bytes); }
    PoolScratch(const PoolScratch&) = delete;
    PoolScratch& operator=(const PoolScratch&) = delete;
};
}  // namespace

// Both products run on the CTA-pair kernel, which wants its second operand as [N, K] with the reduction contiguous:
//   dA = G (m x n) times b16 read as [N' = k][K' = n]  — b's own layout, no transpose;
//   dB = A^T (k x m) times G^T read as [N' = n][K' = m] — a and grad go through a transposing cast (grad's plain and
//        transposed copies come from one pass over it), where the reference makes plain casts (toBf16,
//        ops_tensorcore.cu:401-403).
void matmulBf16Backward(const float* a, const float* b, const float* grad, float* dA, float* dB, int64_t m, int64_t k,
                        int64_t n, const void* bNatural16, cudaStream_t stream) {
    require(m >= 0 && k >= 0 && n >= 0, "matmul_bf16_backward: negative size");
    if (m == 0 || k == 0 || n == 0) {
        // the reference's zero fill of both results (ops_tensorcore.cu:412-415)
        if (m * k > 0) BFB_CUDA(cudaMemsetAsync(dA, 0, static_cast<size_t>(m * k) * 4, stream));
        if (k * n > 0) BFB_CUDA(cudaMemsetAsync(dB, 0, static_cast<size_t>(k * n) * 4, stream));
        return;
    }
    require(a != nullptr && b != nullptr && grad != nullptr && dA != nullptr && dB != nullptr,
            "matmul_bf16_backward: null pointer");
    PoolScratch g16(static_cast<size_t>(m * n) * 2), gT16(static_cast<size_t>(m * n) * 2), aT16(static_cast<size_t>(m * k) * 2);
    castPairBf16(grad, g16.ptr, gT16.ptr, m, n, stream);      // [m,n] and [n,m] in one pass over grad
    castPairBf16(a, nullptr, aT16.ptr, m, k, stream);         // [k,m]
    GemmArgs g;
    g.abDtype = BFB_BF16;
    g.cDtype = BFB_F32;
    g.bLayout = BFB_B_NK;
    g.a = g16.ptr;
    g.c = dA;
    g.m = m;
    g.n = k;
    g.k = n;
    if (bNatural16 != nullptr) {
        g.b = bNatural16;
        gemm(g, stream);
    } else {
        PoolScratch b16(static_cast<size_t>(k * n) * 2);
        castScaled(b, BFB_F32, b16.ptr, BFB_BF16, k * n, 1.0f, nullptr, stream);
        g.b = b16.ptr;
        gemm(g, stream);
    }
    g.a = aT16.ptr;
    g.b = gT16.ptr;
    g.c = dB;
    g.m = k;
    g.n = n;
    g.k = m;
    gemm(g, stream);
}

void matmulTransposeB(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k, cudaStream_t stream) {
    require(m >= 0 && n >= 0 && k >= 0, "matmul_transpose_b: negative size");
    if (m == 0 || n == 0) return;
    require(a != nullptr && b != nullptr && c != nullptr, "matmul_transpose_b: null pointer");
    int64_t total = m * n;
    int grid = static_cast<int>(std::min<int64_t>((total + 255) / 256, static_cast<int64_t>(smCount()) * 16));
    matmulTransposeBKernel<<<grid, 256, 0, stream>>>(a, b, c, m, n, k);
    BFB_LAUNCH_CHECK();
    noteLaunch();
}

}  // namespace bfb
