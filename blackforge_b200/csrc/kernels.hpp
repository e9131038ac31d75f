// Internal C++ entry points of the kernel layer. The C ABI (capi.cu) and the host-side operator
// layer (host/*.cpp) both call these; they throw bfb::Error and never fall back to the CPU.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace bfb {

void embedPos(const float* ids, const float* table, const float* pos, void* out, int outDtype, int64_t batch,
              int64_t seq, int64_t vocab, int64_t dim, int64_t maxSeq, int64_t posOffset, int* oobCount,
              cudaStream_t stream);
void addPositional(const float* in, const float* pos, float* out, int64_t batch, int64_t seq, int64_t dim,
                   int64_t maxSeq, int64_t posOffset, cudaStream_t stream);
// Key/value cache append: the K and V column blocks of `src` ([batch * newLen, ld]; K at column kOffset, V at
// vOffset, `width` columns each) go behind the oldLen rows each batch entry of the caches [batch, capRows, width] holds.
void appendKv(const void* src, int dtype, int64_t ld, int64_t kOffset, int64_t vOffset, void* kCache, void* vCache,
              int64_t batch, int64_t newLen, int64_t width, int64_t capRows, int64_t oldLen, cudaStream_t stream);
// out[row] = sum over the row of x^2 (the statistic of rmsnorm; see GemmArgs::rowSumSq).
void rowSumSquares(const void* x, int xDtype, float* out, int64_t rows, int64_t dim, cudaStream_t stream);
void rmsnorm(const void* x, int xDtype, void* out, int outDtype, int64_t rows, int64_t dim, float eps,
             cudaStream_t stream);
void softmaxRows(const float* x, float* out, int64_t rows, int64_t cols, cudaStream_t stream);
void elementwise(int op, const float* a, const float* b, const float* c, float* out, int64_t n, int64_t cols,
                 cudaStream_t stream);
void castScaled(const void* in, int inDtype, void* out, int outDtype, int64_t n, float scale, const float* dScale,
                cudaStream_t stream);
void amax(const void* in, int inDtype, int64_t n, float* dAmax, cudaStream_t stream);
void fp8ScaleFromAmax(const float* dAmax, float* dScales, cudaStream_t stream);
// out[0] = 448 / amax, out[1] = 1 / out[0], out[2] = out[1] * *dWeightInverse (the GEMM's alpha).
void fp8ActScale(const float* dAmax, float* out, const float* dWeightInverse, cudaStream_t stream);
void weightPrepare(const float* w, void* out, int outDtype, int64_t k, int64_t n, float scale, const float* dScale,
                   cudaStream_t stream);
// bf16 copies of in [rows, cols] (f32) in one pass over it: `plain` [rows, cols] (may be null) and `transposed`
// [cols, rows].
void castPairBf16(const float* in, void* plain, void* transposed, int64_t rows, int64_t cols, cudaStream_t stream);
// Per-tensor e4m3 quantisation: dScales[0] = 448 / max|in|, [1] = its inverse, [2] = inverse * *dWeightInverse
// (1 when null); out = e4m3(in * dScales[0]). `scratch` holds quantizeScratchFloats(n) floats of partial maxima.
int64_t quantizeScratchFloats(int64_t n);
void quantizeE4m3(const void* in, int inDtype, int64_t n, void* out, float* dScales, const float* dWeightInverse,
                  float* scratch, cudaStream_t stream);
// rmsnorm (no weights) of bf16 rows followed by per-tensor e4m3 quantisation, without storing the normalised rows:
// out = e4m3(bf16(x * r_row) * scale), scale = 448 / max|bf16(x * r_row)|; dScales as for quantizeE4m3. `scratch`
// holds rmsnormQuantizeScratchFloats(rows) floats.
// Per-tensor e4m3 quantisation of `in` whose maximum magnitude is the maximum of `maxima` (count floats, e.g. a
// GEMM's outMaxAbs): the maximum pass reads that small array instead of `in`. `scratch` holds
// quantizeScratchFloats(count) floats.
void quantizeE4m3FromMaxima(const void* in, int inDtype, int64_t n, void* out, float* dScales, const float* dWeightInverse,
                            const float* maxima, int64_t count, float* scratch, cudaStream_t stream);
int64_t rmsnormQuantizeScratchFloats(int64_t rows);
// `sumSqParts` / `maxParts` ([parts][rows], may be null): sums of squares and largest magnitudes of x per row and part,
// as the epilogue of the GEMM that wrote x leaves them (GemmArgs::outSumSq, outMaxAbs); with them the first pass reads
// those figures instead of x.
void rmsnormQuantizeE4m3(const void* x, int64_t rows, int64_t dim, float eps, void* out, float* dScales,
                         const float* dWeightInverse, float* scratch, cudaStream_t stream,
                         const float* sumSqParts = nullptr, const float* maxParts = nullptr, int parts = 0);
// Seeded N(0, sigma) values for the [rows, colsLocal] block at (rowOffset, colOffset) of a tensor with colsFull
// columns; a value depends only on the seed and its position in the full tensor.
void fillNormal(float* out, int64_t rows, int64_t colsLocal, int64_t colsFull, int64_t rowOffset, int64_t colOffset,
                uint64_t seed, float sigma, cudaStream_t stream);
// In-place rounding of an f32 buffer to bf16 precision (simulated `storage bf16` for the fp32 path).
void roundBf16InPlace(float* x, int64_t n, cudaStream_t stream);

struct GemmArgs {
    const void* a = nullptr;      // [M,K] row-major, abDtype
    const void* b = nullptr;      // [K,N] (BFB_B_KN) or [N,K] (BFB_B_NK), abDtype
    void* c = nullptr;            // [M,N], cDtype
    int64_t m = 0, n = 0, k = 0;
    int abDtype = 0, bLayout = 0, cDtype = 0, epilogue = 0;
    const float* bias = nullptr;
    const void* residual = nullptr;
    float alpha = 1.0f;
    const float* dAlpha = nullptr;
    int roundCBf16 = 0;
    int* dStatus = nullptr;
    // Row statistics (CTA-pair tensor-core kernel only, see gemmSupportsRowStats). With rowSumSq set, row i of
    // the product is multiplied by 1 / sqrt(s_i * rowInvDim + rowEps) before bias and activation, where s_i is
    // the sum over p < rowSumSqParts of rowSumSq[p * m + i]: an rmsnorm without weights commutes with the matrix
    // product, so A can be the un-normalised activation. With outSumSq set, the sums of squares of each stored
    // row (after rounding to the result format) are written per 128-column part to outSumSq[p * m + i],
    // p < ceil(n / 128): the next norm's statistic without another pass over C, and without atomics.
    const float* rowSumSq = nullptr;
    int rowSumSqParts = 1;
    float rowInvDim = 0.0f;
    float rowEps = 0.0f;
    float* outSumSq = nullptr;
    // Same layout and the same kernel as outSumSq: the largest magnitude of each stored row per 128-column part,
    // outMaxAbs[p * m + i]. The per-tensor maximum an e4m3 quantisation of C needs is then the maximum of a small
    // array instead of another pass over C.
    float* outMaxAbs = nullptr;
    // Few rows (a generation step): stream the weights through as many SMs as possible instead of tiling C (see
    // gemm_skinny.cu). Takes effect for 1..128 rows with [N,K] weights in a tensor-core format; has the row
    // statistics. `workspace` (gemmSkinnyWorkspaceBytes) is optional: without it the pool lends the memory.
    int preferSkinny = 0;
    void* workspace = nullptr;
    size_t workspaceBytes = 0;
};
void gemm(const GemmArgs& args, cudaStream_t stream);
bool gemmSupportsRowStats(const GemmArgs& args);
bool gemmSkinnyEligible(const GemmArgs& args);
int64_t gemmSkinnyWorkspaceBytes(const GemmArgs& args);
void gemmSkinny(const GemmArgs& args, cudaStream_t stream);
// True when the tcgen05 kernel takes this problem (otherwise the CUDA-core kernel runs).
bool gemmUsesTensorCores(const GemmArgs& args);
void matmulTransposeB(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k, cudaStream_t stream);
// Gradients of C = A B on the bf16 tensor-core route (matmulBf16Backward, src/backend/cuda/ops_tensorcore.cu:389-417):
// dA[m,k] = G[m,n] B^T and dB[k,n] = A^T G from fp32 a [m,k], b [k,n], grad [m,n]; operands rounded to bf16, fp32
// accumulation and results. `bNatural16` (may be null) is a ready bf16 copy of b in its own [k,n] layout.
void matmulBf16Backward(const float* a, const float* b, const float* grad, float* dA, float* dB, int64_t m, int64_t k,
                        int64_t n, const void* bNatural16, cudaStream_t stream);

struct AttentionArgs {
    const void* q = nullptr;
    const void* k = nullptr;
    const void* v = nullptr;
    void* out = nullptr;
    float* m = nullptr;
    float* l = nullptr;
    int dtype = 0;
    int64_t batch = 0, newLen = 0, totalLen = 0, numHeads = 0, headDim = 0;
    int64_t ldQ = 0, ldK = 0, ldV = 0, ldO = 0;
    // rows between one batch entry of K / V and the next; 0 means total_len (densely packed). A key/value cache
    // with room for more positions than it holds passes its capacity here.
    int64_t kvBatchRows = 0;
    float scale = 1.0f;
    int64_t oldLen = 0;
    int causal = 1;
    int* dStatus = nullptr;
    // Tensor-core kernel only (attentionUsesTensorCores): the largest magnitude of the stored output per 32 rows of a
    // (batch, head), attentionMaximaCount(args) floats, every one written: what a per-tensor e4m3 quantisation of the
    // output needs, without another pass over it. Null: not wanted.
    float* outMaxima = nullptr;
};
int64_t attentionMaximaCount(const AttentionArgs& args);
// One query per sequence and head against cached keys and values (a generation step): a bandwidth-oriented CUDA-core
// kernel, see attention_decode.cu.
bool attentionDecodeEligible(const AttentionArgs& args);
void attentionDecode(const AttentionArgs& args, cudaStream_t stream);
void attentionForward(const AttentionArgs& args, cudaStream_t stream);
bool attentionUsesTensorCores(const AttentionArgs& args);

// Backward of the attention core (attention_bwd.cu): dQ, dK, dV in fp32 from dOut, q, k, v, out (f32 or bf16, one
// type for all five) and the forward's row statistics m, l [batch, heads, new_len]. lse2Scratch and dTermScratch are
// caller-provided [batch * heads * new_len] floats. head_dim 128 in bf16 runs on the tensor cores.
struct AttentionBackwardArgs {
    const void* dOut = nullptr;
    const void* q = nullptr;
    const void* k = nullptr;
    const void* v = nullptr;
    const void* out = nullptr;
    const float* m = nullptr;
    const float* l = nullptr;
    float* dQ = nullptr;
    float* dK = nullptr;
    float* dV = nullptr;
    float* lse2Scratch = nullptr;
    float* dTermScratch = nullptr;
    int dtype = 0;
    int64_t batch = 0, newLen = 0, totalLen = 0, numHeads = 0, headDim = 0;
    int64_t ldQ = 0, ldK = 0, ldV = 0, ldO = 0, ldDo = 0, ldDq = 0, ldDk = 0, ldDv = 0;
    float scale = 1.0f;
    int64_t oldLen = 0;
    int causal = 1;
    int* dStatus = nullptr;
};
void attentionBackward(const AttentionBackwardArgs& args, cudaStream_t stream);
bool attentionBackwardUsesTensorCores(const AttentionBackwardArgs& args);

// Tensor-core kernels (gemm_tc.cu / attention_tc.cu); callers have checked eligibility.
void gemmTensorCore(const GemmArgs& args, cudaStream_t stream);
// CTA-pair variant (cta_group::2, 256 x 256 tiles); B must be [N,K].
void gemmTensorCorePair(const GemmArgs& args, cudaStream_t stream);
void attentionTensorCore(const AttentionArgs& args, cudaStream_t stream);

// Bounded-wait self-test (selftest.cu): device status code of a wait that was made to run out after `limitNs`.
int selfTestBoundedWait(unsigned long long limitNs, int* observedHost, cudaStream_t stream);

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time libcuda dependency).
// dims/strides innermost first; strides in bytes for dims 1..rank-1; elemBytes 1, 2 (bf16) or 4 (fp32).
struct TensorMapStorage {
    alignas(64) unsigned char bytes[128];
};
void encodeTensorMap(TensorMapStorage* out, const void* base, int elemBytes, int rank, const uint64_t* dims,
                     const uint64_t* stridesBytes, const uint32_t* box);

}  // namespace bfb
