// C++ host layer: the reference's backend operator interface re-created on top of the B200 kernels.
//
// Same names, argument meaning, ownership and error behaviour as blackforge::backend::cuda
// (include/blackforge/backend/cuda/{device_tensor,ops,fused_attention,model,executor,checkpoint,
// device_pool}.hpp in the reference project), in namespace bfb200 so both can be linked side by
// side. Shape / range violations throw std::invalid_argument, CUDA and file problems throw
// std::runtime_error. Tensors at this boundary are fp32 (DeviceTensor stores fp32 only, as in the
// reference); reduced-precision formats live inside Model::forward.
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <optional>
#include <string>
#include <vector>

#include "../../../include/bfb200.h"

namespace bfb200 {

// Host tensor: shape + row-major fp32 data (stand-in for blackforge::runtime::Tensor).
struct HostTensor {
    std::vector<std::size_t> shape;
    std::vector<float> data;
    [[nodiscard]] std::size_t elementCount() const;
};

// include/blackforge/backend/cuda/device_pool.hpp:47-54
void* devicePoolAcquire(std::size_t bytes);
void devicePoolRelease(void* ptr, std::size_t bytes);

// include/blackforge/backend/cuda/device_tensor.hpp:10-75 — move-only RAII fp32 buffer from the pool.
class DeviceTensor {
public:
    DeviceTensor() = default;
    explicit DeviceTensor(std::vector<std::size_t> shape);
    ~DeviceTensor();
    DeviceTensor(const DeviceTensor&) = delete;
    DeviceTensor& operator=(const DeviceTensor&) = delete;
    DeviceTensor(DeviceTensor&& other) noexcept;
    DeviceTensor& operator=(DeviceTensor&& other) noexcept;

    static DeviceTensor fromHost(const HostTensor& host);
    static DeviceTensor zeros(std::vector<std::size_t> shape);
    [[nodiscard]] HostTensor toHost() const;
    [[nodiscard]] DeviceTensor clone() const;
    [[nodiscard]] DeviceTensor reshaped(std::vector<std::size_t> newShape) &&;

    [[nodiscard]] float* data() { return data_; }
    [[nodiscard]] const float* data() const { return data_; }
    [[nodiscard]] const std::vector<std::size_t>& shape() const { return shape_; }
    [[nodiscard]] std::size_t rank() const { return shape_.size(); }
    [[nodiscard]] std::size_t dim(std::size_t axis) const { return shape_.at(axis); }
    [[nodiscard]] std::size_t elementCount() const;
    // Gives up ownership (for handing a result across the C ABI); release with devicePoolRelease.
    float* releaseOwnership();
    // Wraps memory owned by someone else; the caller must call releaseOwnership() before it dies.
    static DeviceTensor borrow(float* data, std::vector<std::size_t> shape);

private:
    float* data_ = nullptr;
    std::vector<std::size_t> shape_;
};

// ---- include/blackforge/backend/cuda/ops.hpp ------------------------------------------------------
DeviceTensor add(const DeviceTensor& a, const DeviceTensor& b);
DeviceTensor addBias(const DeviceTensor& input, const DeviceTensor& bias);
DeviceTensor addBiasSilu(const DeviceTensor& gemmOutput, const DeviceTensor& bias);
DeviceTensor addBiasResidual(const DeviceTensor& gemmOutput, const DeviceTensor& bias, const DeviceTensor& residual);
DeviceTensor matmul(const DeviceTensor& a, const DeviceTensor& b);
DeviceTensor matmulTransposeB(const DeviceTensor& a, const DeviceTensor& b);
DeviceTensor matmulBf16(const DeviceTensor& a, const DeviceTensor& b);
DeviceTensor matmulBf16CachedWeight(const DeviceTensor& a, const DeviceTensor& b);
void invalidateBf16WeightCache();
// include/blackforge/backend/cuda/autodiff.hpp:18-37: gradients of C = A B on the bf16 tensor-core route
// (dA = gradOutput B^T, dB = A^T gradOutput; fp32 tensors in and out). The CachedWeight form keeps a bf16 copy of B
// until invalidateBf16WeightCache().
struct MatmulGrad {
    DeviceTensor dA;
    DeviceTensor dB;
};
MatmulGrad matmulBf16Backward(const DeviceTensor& a, const DeviceTensor& b, const DeviceTensor& gradOutput);
MatmulGrad matmulBf16BackwardCachedWeight(const DeviceTensor& a, const DeviceTensor& b, const DeviceTensor& gradOutput);
// New: e4m3 operands with per-tensor amax scales, fp32 accumulate (the declared `compute fp8.e4m3`).
DeviceTensor matmulFp8(const DeviceTensor& a, const DeviceTensor& b);
DeviceTensor silu(const DeviceTensor& input);
DeviceTensor relu(const DeviceTensor& input);
DeviceTensor gelu(const DeviceTensor& input);
DeviceTensor rmsnorm(const DeviceTensor& input);
DeviceTensor softmax(const DeviceTensor& input);
DeviceTensor embeddingLookup(const DeviceTensor& tokenIds, const DeviceTensor& table);
DeviceTensor embeddingLookupPreValidated(const DeviceTensor& tokenIds, const DeviceTensor& table);
DeviceTensor addPositionalEmbedding(const DeviceTensor& input, const DeviceTensor& table);
DeviceTensor addPositionalEmbeddingAt(const DeviceTensor& input, const DeviceTensor& table, std::size_t offset);
DeviceTensor linear(const DeviceTensor& input, const DeviceTensor& weight, const DeviceTensor& bias);
DeviceTensor linearBf16(const DeviceTensor& input, const DeviceTensor& weight, const DeviceTensor& bias);
DeviceTensor feedForward(const DeviceTensor& input, const DeviceTensor& w1, const DeviceTensor& b1,
                         const DeviceTensor& w2, const DeviceTensor& b2);
DeviceTensor feedForwardBf16(const DeviceTensor& input, const DeviceTensor& w1, const DeviceTensor& b1,
                             const DeviceTensor& w2, const DeviceTensor& b2);
DeviceTensor selfAttention(const DeviceTensor& input, const DeviceTensor& wq, const DeviceTensor& wk,
                           const DeviceTensor& wv, const DeviceTensor& wout, std::size_t numHeads);
DeviceTensor selfAttentionBf16(const DeviceTensor& input, const DeviceTensor& wq, const DeviceTensor& wk,
                               const DeviceTensor& wv, const DeviceTensor& wout, std::size_t numHeads);

// include/blackforge/backend/cuda/ops.hpp:213-241 — autoregressive generation at the operator level. `k` / `v`
// are [batch, length, dim] and grow by the number of new positions on every call; one instance per layer.
// The result for the new positions equals what selfAttention() gives for them on the whole sequence so far.
struct KVCache {
    DeviceTensor k;
    DeviceTensor v;
    std::size_t length = 0;
};
DeviceTensor concatSeq(const DeviceTensor& a, const DeviceTensor& b);   // along dimension 1 of [batch, len, dim]
DeviceTensor selfAttentionIncremental(const DeviceTensor& newInput, const DeviceTensor& wq, const DeviceTensor& wk,
                                      const DeviceTensor& wv, const DeviceTensor& wout, std::size_t numHeads,
                                      KVCache& cache);
DeviceTensor selfAttentionIncrementalBf16(const DeviceTensor& newInput, const DeviceTensor& wq, const DeviceTensor& wk,
                                          const DeviceTensor& wv, const DeviceTensor& wout, std::size_t numHeads,
                                          KVCache& cache);

// include/blackforge/backend/cuda/fused_attention.hpp:42-57
struct FusedAttentionForwardResult {
    DeviceTensor output;
    DeviceTensor m;
    DeviceTensor l;
};
FusedAttentionForwardResult fusedAttentionForward(const DeviceTensor& q, const DeviceTensor& k, const DeviceTensor& v,
                                                  std::size_t numHeads, float scaleFactor, std::size_t oldLen);
// Same contract; operands are rounded to bf16 and run through the tensor-core kernel when head_dim is 128.
FusedAttentionForwardResult fusedAttentionForwardBf16(const DeviceTensor& q, const DeviceTensor& k,
                                                      const DeviceTensor& v, std::size_t numHeads, float scaleFactor,
                                                      std::size_t oldLen);

// include/blackforge/backend/cuda/fused_attention.hpp:59-76: gradients of the attention core from the forward's
// operands, output and row statistics. dQ [batch, new_len, dim]; dK, dV [batch, total_len, dim].
struct FusedAttentionGrad {
    DeviceTensor dQ;
    DeviceTensor dK;
    DeviceTensor dV;
};
FusedAttentionGrad fusedAttentionBackward(const DeviceTensor& dOutput, const DeviceTensor& q, const DeviceTensor& k,
                                          const DeviceTensor& v, const DeviceTensor& output, const DeviceTensor& m,
                                          const DeviceTensor& l, std::size_t numHeads, float scaleFactor,
                                          std::size_t oldLen);
// Same contract; operands are rounded to bf16 and run through the tensor-core kernel when head_dim is 128
// (gradients stay fp32).
FusedAttentionGrad fusedAttentionBackwardBf16(const DeviceTensor& dOutput, const DeviceTensor& q, const DeviceTensor& k,
                                              const DeviceTensor& v, const DeviceTensor& output, const DeviceTensor& m,
                                              const DeviceTensor& l, std::size_t numHeads, float scaleFactor,
                                              std::size_t oldLen);

// ---- model ------------------------------------------------------------------------------------------
using OpDesc = bfb_op_desc;

struct PrecisionPolicy {  // include/blackforge/ir/module.hpp:44-48, BFB_DT_* codes
    int storage = BFB_DT_FP32;
    int compute = BFB_DT_FP32;
    int accumulate = BFB_DT_FP32;
};

struct Parameter {  // include/blackforge/backend/cuda/model.hpp:15-19 (gradients belong to training)
    std::string name;
    DeviceTensor value;                  // this rank's part (the whole tensor when not tensor-parallel)
    std::vector<std::size_t> fullShape;  // shape in checkpoints
};

// include/blackforge/backend/cuda/model.hpp:57-113 (forward side).
// include/blackforge/backend/cpu/benchmark.hpp:14-45
struct OperationBenchmark {
    std::string operationName;   // "linear", "attention", ... (ir::opKindName)
    std::size_t operationIndex;  // position in the pipeline
    double meanMilliseconds;
};
struct BenchmarkResult {
    std::vector<std::size_t> inputShape;
    std::size_t warmupIterations = 0;
    std::size_t measuredIterations = 0;
    double meanMilliseconds = 0.0;
    double throughputSamplesPerSecond = 0.0;
    std::size_t estimatedMemoryBytes = 0;   // elements x 4 bytes of input, operation outputs and parameters
    std::vector<OperationBenchmark> perOperation;
};

class Model {
public:
    Model(const std::vector<OpDesc>& ops, std::int64_t inputLastDim, unsigned int seed = 42,
          std::optional<PrecisionPolicy> precision = std::nullopt, bool randomInit = true,
          std::string name = "model");
    ~Model();
    Model(const Model&) = delete;
    Model& operator=(const Model&) = delete;

    // Heads, feed-forward columns and logits columns sharded over `world` ranks; call before any
    // parameter is set. Outputs of a final linear are this rank's column slice.
    void setTensorParallel(int rank, int world);
    // How a tensor-parallel prompt pass hides its all-reduces: the batch is cut into `groups` groups of sequences
    // (1 = no overlap; fewer when the batch does not divide), and while one group's rows are summed over the ranks
    // on a second stream the next group computes; its GEMMs draw their tiles from a device counter (pairs the
    // collective's CTAs keep waiting then leave no tail) and its persistent kernels can leave `reservedSms` SMs free. Defaults: 2 and 0 (environment BFB_TP_CHUNKS, BFB_TP_RESERVE_SMS). Results do not depend on it.
    void setTensorParallelOverlap(int groups, int reservedSms);

    DeviceTensor forward(const DeviceTensor& input, bool inputRangeTrusted = false, void* stream = nullptr);
    // Under `storage bf16` every value of forward()'s result is a bf16 number held in an fp32 word. When the
    // pipeline runs from an embedding to a final linear, forwardBf16 writes those same numbers as 2-byte bf16
    // into `deviceOut16` (product(outputShape) elements) instead: half the bytes for a caller that moves them on.
    // include/blackforge/backend/cuda/model.hpp (forwardIncremental, resetGenerationState): autoregressive
    // generation. Each call takes the ids of the NEW positions only, [batch, newLen], and returns their outputs;
    // keys and values of earlier positions stay in per-layer caches, positions continue where the last call
    // stopped. The batch size is fixed by the first call after a reset. On the planned route (compute bf16 /
    // fp8.e4m3) the caches are preallocated bf16 buffers sized for the positional table (grown by doubling when
    // the pipeline has none), filled in place: no re-copy per token.
    DeviceTensor forwardIncremental(const DeviceTensor& newTokenIds, bool inputRangeTrusted = false, void* stream = nullptr);
    void resetGenerationState();
    [[nodiscard]] std::size_t generationPosition() const;
    [[nodiscard]] bool resultIsBf16Exact() const;
    void forwardBf16(const DeviceTensor& input, void* deviceOut16, bool inputRangeTrusted = false, void* stream = nullptr);

    [[nodiscard]] std::vector<Parameter*> parameters();
    [[nodiscard]] const std::string& name() const { return name_; }
    // Shape of forward()'s result for an input of this shape, without running anything.
    [[nodiscard]] std::vector<std::size_t> outputShape(const std::vector<std::size_t>& inputShape) const;
    // Structure only (no device memory touched): checkpoint order, names, full shapes.
    [[nodiscard]] std::size_t parameterCount() const;
    [[nodiscard]] const std::string& parameterName(std::size_t index) const;
    [[nodiscard]] const std::vector<std::size_t>& parameterShape(std::size_t index) const;
    void setParameter(std::size_t index, const float* hostFullValues);
    void getParameter(std::size_t index, float* hostFullValues);
    // Synthetic weights without a host round trip: seeded N(0, sigma), identical whatever the tensor-parallel split.
    void fillParameterNormal(std::size_t index, std::uint64_t seed, float sigma);
    // After conversion to bf16 / e4m3, drop the fp32 copies of the GEMM weights (inference on models whose fp32
    // weights would not fit next to the converted ones). Those parameters can no longer be read or set.
    void releaseMasterWeights();
    // Parameters changed: converted weights are rebuilt at the next forward.
    void invalidatePreparedWeights();
    [[nodiscard]] std::optional<std::size_t> firstLayerEmbeddingVocabSize() const;

    // include/blackforge/backend/cpu/benchmark.hpp:48-62 (runBenchmark), on the device and on the caller's input:
    // `warmupIterations` discarded passes, then `measuredIterations` timed ones. Times are device times between CUDA
    // events recorded on the forward's stream at the start of every pipeline operation: the per-operation figures
    // the reference's header says its CUDA side lacks (benchmark.hpp:34-43), taken inside the full pass instead of
    // operation by operation. An operation fused into its predecessor (positions into the embedding) reports 0.
    // Throws std::invalid_argument for an empty pipeline or measuredIterations == 0, as the reference does.
    BenchmarkResult benchmark(const DeviceTensor& input, std::size_t warmupIterations, std::size_t measuredIterations,
                              void* stream = nullptr);

    // Converted GEMM weights (bf16 or e4m3, transposed, with their scales) as the tensor-core route holds them: for a
    // cache file beside a checkpoint (loadCheckpointCached). The tag names compute format and tensor-parallel split
    // (empty for an fp32-compute model, which has no converted weights); the fingerprint covers the tag and every
    // parameter's name and shape. After adoptPreparedWeights() the fp32 copies of the GEMM weights do not exist.
    struct PreparedPiece {
        void* data;
        std::size_t bytes;
    };
    std::string preparedWeightsTag() const;
    std::uint64_t structureFingerprint() const;
    std::vector<PreparedPiece> preparedWeightPieces(bool allocate);
    void adoptPreparedWeights();
    bool parameterIsGemmWeight(std::size_t index) const;

    // A parameter seen as rows of the full (unsharded) tensor, and the rows this tensor-parallel rank holds a part
    // of: all of them, except for row-sharded matrices and sharded vectors (one element per row).
    struct RowView {
        std::size_t rows = 0, rowElems = 0;
        std::size_t firstNeededRow = 0, neededRows = 0;
    };
    RowView parameterRowView(std::size_t index) const;
    // Asynchronous upload of `rowCount` full-width rows (host memory, pinned for a truly asynchronous copy) starting
    // at row `firstRow` of the full tensor; this rank's columns are taken out of them where the parameter is
    // column-sharded. Returns the bytes sent to the device.
    std::size_t uploadParameterRows(std::size_t index, std::size_t firstRow, std::size_t rowCount, const float* hostRows,
                                    void* stream);

    struct Impl;

private:
    std::unique_ptr<Impl> impl_;
    std::string name_;
};

// include/blackforge/backend/cuda/checkpoint.hpp:24-27 — BFCKPT1 files. The loader streams: headers first, then
// whole rows through pinned buffers while earlier rows upload; a tensor-parallel rank reads only the rows it holds
// of row-sharded tensors. chunkBytes == 0 picks 4 MiB.
struct CheckpointEntry {
    std::string name;
    std::vector<std::size_t> shape;
    std::uint64_t dataOffset = 0, dataBytes = 0;
};
struct CheckpointLoadStats {
    std::size_t tensors = 0;
    std::uint64_t fileBytes = 0;      // fp32 payload of the file
    std::uint64_t readBytes = 0;      // read from the file by this rank
    std::uint64_t uploadedBytes = 0;  // sent to the device
    double seconds = 0.0;
    bool cacheHit = false;            // loadCheckpointCached: the converted weights came from the cache file
    std::uint64_t cacheBytes = 0;     // read from (hit) or written to (miss) the cache file
};
std::vector<CheckpointEntry> indexCheckpoint(const std::string& path);
void saveCheckpoint(Model& model, const std::string& path);
CheckpointLoadStats loadCheckpoint(Model& model, const std::string& path, std::size_t chunkBytes = 0);
// The same, with a cache of the CONVERTED GEMM weights beside the file (`<path>.bfb200cache.<format>.tp<r>of<w>`):
// written after the first load, and read instead of the fp32 GEMM weights on the next ones as long as the
// checkpoint's size and modification time and the model's structure are unchanged. A hit reads half (bf16) or a
// quarter (e4m3) of the bytes, skips the conversion pass and never creates the fp32 copies of the GEMM weights
// (they can then not be read back, set or saved). An fp32-compute model loads as loadCheckpoint does.
CheckpointLoadStats loadCheckpointCached(Model& model, const std::string& path, std::size_t chunkBytes = 0);

// include/blackforge/backend/cuda/executor.hpp:20-33 — weights regenerated from the seed on every run.
class Executor {
public:
    explicit Executor(unsigned int seed = 42) : seed_(seed) {}
    [[nodiscard]] HostTensor makeSyntheticInput(const std::vector<OpDesc>& ops, const std::vector<std::int64_t>& inputShape,
                                                std::size_t batchSize) const;
    [[nodiscard]] HostTensor run(const std::vector<OpDesc>& ops, std::int64_t inputLastDim, const HostTensor& input,
                                 const std::optional<PrecisionPolicy>& precision = std::nullopt) const;

private:
    unsigned int seed_;
};

// Seeded default initialisation shared by Model and Executor: uniform(-0.1, 0.1) from std::mt19937
// (src/backend/cpu/random_init.cpp:7-22) with seedFor(base, valueId, salt) = base ^ (valueId * salt).
HostTensor randomTensor(std::vector<std::size_t> shape, unsigned int seed);
HostTensor randomTokenIdTensor(std::vector<std::size_t> shape, std::size_t vocabSize, unsigned int seed);
unsigned int seedFor(unsigned int base, std::size_t valueId, unsigned int salt);

}  // namespace bfb200
