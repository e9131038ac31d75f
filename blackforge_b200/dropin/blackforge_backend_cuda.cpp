// Drop-in for the forward path of BlackForge's CUDA backend: this ONE translation unit defines the functions and
// classes that the reference declares in include/blackforge/backend/cuda/{device_pool,device_query,device_tensor,
// ops,fused_attention,model,executor,checkpoint}.hpp (namespace blackforge::backend::cuda), on top of the C ABI of
// libbfb200.so (include/bfb200.h). A BlackForge build compiles this file IN PLACE OF src/backend/cuda/{device_pool,
// device_query,device_tensor,ops_elementwise,ops_gemm,ops_tensorcore,ops_transformer,fused_attention,model,executor,
// checkpoint}.cu and links libbfb200.so; caller code written against the reference's headers (src/main.cpp:356-370,
// 803-829, the tests under tests/backend/cuda) compiles and runs unchanged for everything on the inference path.
//
// It needs the reference's headers to compile (-I<blackforge>/include) and nothing else from it. Same error
// behaviour as the reference: std::invalid_argument for shape / rank / range problems, std::runtime_error for
// everything else (cuda_check.hpp:14-53). Training (Model::backward, zeroGrad, the *ForwardCached and *Backward
// functions, train runners) is outside this backend: those members throw, the free functions are not defined here,
// except fusedAttentionBackward (the gradient of the attention core), which is.
//
// How the reference's private layout is served without touching its headers:
//  * DeviceTensor has no way to adopt memory; a result that arrives from the C ABI as a pool pointer is taken over
//    by the ordinary DeviceTensor(shape) constructor, which looks at a thread-local "next allocation is this
//    pointer" slot before it asks the pool (adoptNext below). No copy.
//  * Model has no member for a handle; handles live in a side table keyed by the Model's address.
//  * Model::parameters() hands out Parameter objects (name, value, grad) stored in the header's own LayerState
//    slots. They mirror the library's weights: forward() pushes a parameter into the library whenever its value
//    tensor was replaced (other device pointer) since the last push. Writing INTO an existing value buffer on the
//    device (an optimizer step) is not seen; that is training.
#include <cuda_runtime.h>

#include <cmath>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "blackforge/backend/cuda/checkpoint.hpp"
#include "blackforge/backend/cuda/device_pool.hpp"
#include "blackforge/backend/cuda/device_query.hpp"
#include "blackforge/backend/cuda/device_tensor.hpp"
#include "blackforge/backend/cuda/executor.hpp"
#include "blackforge/backend/cuda/fused_attention.hpp"
#include "blackforge/backend/cuda/model.hpp"
#include "blackforge/backend/cuda/ops.hpp"
#include "bfb200.h"

namespace blackforge::backend::cuda {

namespace {

// status of the C ABI -> the reference's exceptions
void check(bfb_status st) {
    if (st == BFB_OK) return;
    const std::string text = bfb_last_error();
    if (st == BFB_INVALID_ARGUMENT) throw std::invalid_argument(text);
    throw std::runtime_error(text);
}

thread_local float* tlsAdoptPtr = nullptr;
thread_local std::size_t tlsAdoptBytes = 0;

std::size_t countOf(const std::vector<std::size_t>& shape) {
    std::size_t n = 1;
    for (std::size_t d : shape) n *= d;
    return n;
}

// The next DeviceTensor(shape) of `bytes` bytes on this thread takes `ptr` (pool memory) instead of allocating.
DeviceTensor adopt(void* ptr, std::vector<std::size_t> shape) {
    tlsAdoptPtr = static_cast<float*>(ptr);
    tlsAdoptBytes = countOf(shape) * sizeof(float);
    return DeviceTensor(std::move(shape));
}

std::size_t rowsOf(const DeviceTensor& t) { return t.rank() == 0 ? 0 : t.elementCount() / t.dim(t.rank() - 1); }

struct Bf16Scratch {   // pool buffer of n bf16 values
    void* ptr = nullptr;
    std::size_t bytes = 0;
    explicit Bf16Scratch(std::size_t n) : bytes(n * 2) { ptr = devicePoolAcquire(bytes); }
    ~Bf16Scratch() { devicePoolRelease(ptr, bytes); }
    Bf16Scratch(const Bf16Scratch&) = delete;
    Bf16Scratch& operator=(const Bf16Scratch&) = delete;
};

void toBf16(const float* src, void* dst, std::size_t n) {
    check(bfb_cast(src, BFB_F32, dst, BFB_BF16, static_cast<int64_t>(n), 1.0f, nullptr, nullptr));
}

// C[m,n] = A[m,k] B[k,n] (+ epilogue), fp32 operands on CUDA cores or operands rounded to bf16 on tensor cores
DeviceTensor gemm(const float* a, const float* b, std::size_t m, std::size_t n, std::size_t k, bool bf16, int epilogue,
                  const float* bias, const float* residual, std::vector<std::size_t> outShape) {
    DeviceTensor c(std::move(outShape));
    if (m == 0 || n == 0) return c;
    if (k == 0) {
        check(bfb_memset_zero(c.data(), c.elementCount() * sizeof(float), nullptr));
        return c;
    }
    if (bf16) {
        Bf16Scratch a16(m * k), b16(k * n);
        toBf16(a, a16.ptr, m * k);
        toBf16(b, b16.ptr, k * n);
        check(bfb_gemm(a16.ptr, b16.ptr, c.data(), static_cast<int64_t>(m), static_cast<int64_t>(n), static_cast<int64_t>(k),
                       BFB_BF16, BFB_B_KN, BFB_F32, epilogue, bias, residual, 1.0f, nullptr, 0, nullptr, nullptr));
    } else {
        check(bfb_gemm(a, b, c.data(), static_cast<int64_t>(m), static_cast<int64_t>(n), static_cast<int64_t>(k), BFB_F32,
                       BFB_B_KN, BFB_F32, epilogue, bias, residual, 1.0f, nullptr, 0, nullptr, nullptr));
    }
    check(bfb_stream_synchronize(nullptr));
    return c;
}

void requireMatmulShapes(const DeviceTensor& a, const DeviceTensor& b, const char* who) {
    if (a.rank() != 2 || b.rank() != 2 || a.dim(1) != b.dim(0)) {
        throw std::invalid_argument(std::string(who) + ": incompatible shapes on the device");
    }
}

DeviceTensor unary(int op, const DeviceTensor& x) {
    DeviceTensor out(x.shape());
    check(bfb_elementwise(op, x.data(), nullptr, nullptr, out.data(), static_cast<int64_t>(x.elementCount()), 1, nullptr));
    return out;
}

DeviceTensor linearImpl(const DeviceTensor& input, const DeviceTensor& weight, const DeviceTensor& bias, bool bf16) {
    if (input.rank() < 2 || weight.rank() != 2 || input.dim(input.rank() - 1) != weight.dim(0)) {
        throw std::invalid_argument("linear: input [..., in] and weight [in, out] required");
    }
    if (bias.rank() != 1 || bias.dim(0) != weight.dim(1)) throw std::invalid_argument("linear: bias must be [out]");
    std::vector<std::size_t> outShape = input.shape();
    outShape.back() = weight.dim(1);
    return gemm(input.data(), weight.data(), rowsOf(input), weight.dim(1), weight.dim(0), bf16, BFB_EPI_BIAS, bias.data(),
                nullptr, std::move(outShape));
}

DeviceTensor feedForwardImpl(const DeviceTensor& input, const DeviceTensor& w1, const DeviceTensor& b1,
                             const DeviceTensor& w2, const DeviceTensor& b2, bool bf16) {
    if (input.rank() < 2 || w1.rank() != 2 || w2.rank() != 2 || input.dim(input.rank() - 1) != w1.dim(0) ||
        w1.dim(1) != w2.dim(0) || w2.dim(1) != w1.dim(0) || b1.rank() != 1 || b1.dim(0) != w1.dim(1) || b2.rank() != 1 ||
        b2.dim(0) != w2.dim(1)) {
        throw std::invalid_argument("feedForward: incompatible shapes");
    }
    const std::size_t rows = rowsOf(input), d = w1.dim(0), f = w1.dim(1);
    DeviceTensor normed = rmsnorm(input);
    DeviceTensor hidden = gemm(normed.data(), w1.data(), rows, f, d, bf16, BFB_EPI_BIAS_SILU, b1.data(), nullptr, {rows, f});
    return gemm(hidden.data(), w2.data(), rows, d, f, bf16, BFB_EPI_BIAS_RESIDUAL, b2.data(), input.data(), input.shape());
}

void requireAttentionShapes(const DeviceTensor& input, const DeviceTensor& wq, const DeviceTensor& wk,
                            const DeviceTensor& wv, const DeviceTensor& wout, std::size_t numHeads) {
    if (input.rank() != 3) throw std::invalid_argument("selfAttention: input [batch, seq, dim] required");
    const std::size_t d = input.dim(2);
    for (const DeviceTensor* w : {&wq, &wk, &wv, &wout}) {
        if (w->rank() != 2 || w->dim(0) != d || w->dim(1) != d) throw std::invalid_argument("selfAttention: weights must be [dim, dim]");
    }
    if (numHeads == 0 || d % numHeads != 0) throw std::invalid_argument("selfAttention: dim must divide by numHeads");
}

// causal multi-head attention core on fp32 q [batch, newLen, dim], k / v [batch, totalLen, dim]
DeviceTensor attentionCore(const DeviceTensor& q, const DeviceTensor& k, const DeviceTensor& v, std::size_t numHeads,
                           float scale, std::size_t oldLen, bool bf16, DeviceTensor* mOut, DeviceTensor* lOut) {
    const std::size_t batch = q.dim(0), newLen = q.dim(1), totalLen = k.dim(1), dim = q.dim(2), hd = dim / numHeads;
    DeviceTensor out(q.shape());
    float* m = mOut != nullptr ? mOut->data() : nullptr;
    float* l = lOut != nullptr ? lOut->data() : nullptr;
    const int64_t ld = static_cast<int64_t>(dim);
    if (bf16) {
        Bf16Scratch q16(q.elementCount()), k16(k.elementCount()), v16(v.elementCount()), o16(out.elementCount());
        toBf16(q.data(), q16.ptr, q.elementCount());
        toBf16(k.data(), k16.ptr, k.elementCount());
        toBf16(v.data(), v16.ptr, v.elementCount());
        check(bfb_attention_fwd(q16.ptr, k16.ptr, v16.ptr, o16.ptr, m, l, BFB_BF16, static_cast<int64_t>(batch),
                                static_cast<int64_t>(newLen), static_cast<int64_t>(totalLen), static_cast<int64_t>(numHeads),
                                static_cast<int64_t>(hd), ld, ld, ld, ld, scale, static_cast<int64_t>(oldLen), 1, nullptr, nullptr));
        check(bfb_cast(o16.ptr, BFB_BF16, out.data(), BFB_F32, static_cast<int64_t>(out.elementCount()), 1.0f, nullptr, nullptr));
        check(bfb_stream_synchronize(nullptr));
    } else {
        check(bfb_attention_fwd(q.data(), k.data(), v.data(), out.data(), m, l, BFB_F32, static_cast<int64_t>(batch),
                                static_cast<int64_t>(newLen), static_cast<int64_t>(totalLen), static_cast<int64_t>(numHeads),
                                static_cast<int64_t>(hd), ld, ld, ld, ld, scale, static_cast<int64_t>(oldLen), 1, nullptr, nullptr));
    }
    return out;
}

DeviceTensor selfAttentionImpl(const DeviceTensor& input, const DeviceTensor& wq, const DeviceTensor& wk,
                               const DeviceTensor& wv, const DeviceTensor& wout, std::size_t numHeads, bool bf16,
                               KVCache* cache) {
    requireAttentionShapes(input, wq, wk, wv, wout, numHeads);
    const std::size_t batch = input.dim(0), seq = input.dim(1), d = input.dim(2), rows = batch * seq;
    DeviceTensor normed = rmsnorm(input);
    DeviceTensor q = gemm(normed.data(), wq.data(), rows, d, d, bf16, BFB_EPI_NONE, nullptr, nullptr, input.shape());
    DeviceTensor k = gemm(normed.data(), wk.data(), rows, d, d, bf16, BFB_EPI_NONE, nullptr, nullptr, input.shape());
    DeviceTensor v = gemm(normed.data(), wv.data(), rows, d, d, bf16, BFB_EPI_NONE, nullptr, nullptr, input.shape());
    const float scale = 1.0f / std::sqrt(static_cast<float>(d / numHeads));
    DeviceTensor ctx;
    if (cache == nullptr) {
        ctx = attentionCore(q, k, v, numHeads, scale, 0, bf16, nullptr, nullptr);
    } else {
        // keys and values of all positions so far: [batch, old + new, dim], batch entries kept apart
        const std::size_t oldLen = cache->length;
        if (oldLen > 0 && cache->k.dim(0) != batch) throw std::invalid_argument("selfAttentionIncremental: batch size changed");
        DeviceTensor allK({batch, oldLen + seq, d}), allV({batch, oldLen + seq, d});
        for (std::size_t b = 0; b < batch; ++b) {
            if (oldLen > 0) {
                check(bfb_copy_d2d(allK.data() + b * (oldLen + seq) * d, cache->k.data() + b * oldLen * d, oldLen * d * sizeof(float), nullptr));
                check(bfb_copy_d2d(allV.data() + b * (oldLen + seq) * d, cache->v.data() + b * oldLen * d, oldLen * d * sizeof(float), nullptr));
            }
            check(bfb_copy_d2d(allK.data() + (b * (oldLen + seq) + oldLen) * d, k.data() + b * seq * d, seq * d * sizeof(float), nullptr));
            check(bfb_copy_d2d(allV.data() + (b * (oldLen + seq) + oldLen) * d, v.data() + b * seq * d, seq * d * sizeof(float), nullptr));
        }
        ctx = attentionCore(q, allK, allV, numHeads, scale, oldLen, bf16, nullptr, nullptr);
        check(bfb_stream_synchronize(nullptr));
        cache->k = std::move(allK);
        cache->v = std::move(allV);
        cache->length = oldLen + seq;
    }
    return gemm(ctx.data(), wout.data(), rows, d, d, bf16, BFB_EPI_RESIDUAL, nullptr, input.data(), input.shape());
}

// ---- Model side table --------------------------------------------------------------------------------------
struct ModelState {
    bfb_model* handle = nullptr;
    std::vector<const float*> pushed;   // device pointer of each parameter's value at the time it was last pushed
};
std::mutex gModelsMutex;
std::unordered_map<const Model*, ModelState> gModels;

ModelState& stateOf(const Model* m) {
    std::lock_guard<std::mutex> lock(gModelsMutex);
    auto it = gModels.find(m);
    if (it == gModels.end()) throw std::runtime_error("cuda::Model: unknown instance (moved or copied after construction?)");
    return it->second;
}

int dtypeCode(sema::DType t) {
    switch (t) {
        case sema::DType::FP8_E4M3: return BFB_DT_FP8_E4M3;
        case sema::DType::FP8_E5M2: return BFB_DT_FP8_E5M2;
        case sema::DType::FP16: return BFB_DT_FP16;
        case sema::DType::BF16: return BFB_DT_BF16;
        case sema::DType::TF32: return BFB_DT_TF32;
        default: return BFB_DT_FP32;
    }
}

int opCode(ir::OpKind k) {
    switch (k) {
        case ir::OpKind::Linear: return BFB_OP_LINEAR;
        case ir::OpKind::Silu: return BFB_OP_SILU;
        case ir::OpKind::Relu: return BFB_OP_RELU;
        case ir::OpKind::Gelu: return BFB_OP_GELU;
        case ir::OpKind::RmsNorm: return BFB_OP_RMSNORM;
        case ir::OpKind::Softmax: return BFB_OP_SOFTMAX;
        case ir::OpKind::Embedding: return BFB_OP_EMBEDDING;
        case ir::OpKind::PositionalEmbedding: return BFB_OP_POSITIONAL_EMBEDDING;
        case ir::OpKind::Attention: return BFB_OP_ATTENTION;
        case ir::OpKind::FeedForward: return BFB_OP_FEEDFORWARD;
        default: return BFB_OP_BIDIRECTIONAL_ATTENTION;
    }
}

// ir::ModelIR -> the C ABI's operation list and the width of the model's input (0 when symbolic)
std::vector<bfb_op_desc> describe(const ir::ModelIR& ir, int64_t* inputLastDim) {
    if (ir.pipelines.empty() || ir.pipelines.front().operations.empty()) {
        throw std::invalid_argument("cuda::Model: the model has no pipeline");
    }
    std::vector<bfb_op_desc> ops;
    for (const ir::Operation& op : ir.pipelines.front().operations) {
        bfb_op_desc d{};
        d.kind = opCode(op.kind);
        d.input = static_cast<int64_t>(op.input);
        d.output = static_cast<int64_t>(op.output);
        d.linear_out_features = op.linearOutFeatures;
        d.embedding_vocab_size = op.embeddingVocabSize;
        d.embedding_dim = op.embeddingDim;
        d.positional_max_seq_len = op.positionalMaxSeqLen;
        d.attention_num_heads = op.attentionNumHeads;
        d.feedforward_hidden_dim = op.feedForwardHiddenDim;
        ops.push_back(d);
    }
    const ir::Value& in = ir.valueById(ir.inputValue);
    *inputLastDim = (!in.shape.empty() && !in.shape.back().isSymbolic) ? in.shape.back().literalValue : 0;
    return ops;
}

bfb_precision precisionOf(const std::optional<ir::PrecisionPolicy>& p) {
    bfb_precision out{};
    if (p.has_value()) {
        out.present = 1;
        out.storage = dtypeCode(p->storage);
        out.compute = dtypeCode(p->compute);
        out.accumulate = dtypeCode(p->accumulate);
    }
    return out;
}

DeviceTensor paramFromLibrary(bfb_model* h, int index) {
    const int rank = bfb_model_param_rank(h, index);
    std::vector<int64_t> dims(static_cast<std::size_t>(std::max(rank, 1)));
    bfb_model_param_shape(h, index, dims.data());
    std::vector<std::size_t> shape(dims.begin(), dims.begin() + rank);
    std::vector<float> host(countOf(shape));
    check(bfb_model_param_get(h, index, host.data()));
    return DeviceTensor::fromHost(runtime::Tensor(std::move(shape), std::move(host)));
}

}  // namespace

// ---- device_pool.hpp:47-54 ------------------------------------------------------------------------------------
void* devicePoolAcquire(std::size_t bytes) {
    void* p = nullptr;
    check(bfb_pool_acquire(bytes, &p));
    return p;
}

void devicePoolRelease(void* ptr, std::size_t bytes) { bfb_pool_release(ptr, bytes); }

// ---- device_query.hpp:21-33 -----------------------------------------------------------------------------------
std::vector<CudaDeviceInfo> enumerateDevices() {
    int32_t count = 0;
    if (bfb_device_count(&count) != BFB_OK) return {};
    std::vector<CudaDeviceInfo> out;
    for (int i = 0; i < count; ++i) {
        cudaDeviceProp prop{};
        if (cudaGetDeviceProperties(&prop, i) != cudaSuccess) throw std::runtime_error("cudaGetDeviceProperties failed");
        out.push_back({i, prop.name, prop.major, prop.minor, prop.totalGlobalMem});
    }
    return out;
}

void setActiveDevice(int index) { check(bfb_set_device(index)); }

// ---- device_tensor.hpp ----------------------------------------------------------------------------------------
DeviceTensor::DeviceTensor(std::vector<std::size_t> shape) : shape_(std::move(shape)) {
    const std::size_t bytes = countOf(shape_) * sizeof(float);
    if (tlsAdoptPtr != nullptr && tlsAdoptBytes == bytes) {
        data_ = tlsAdoptPtr;   // a result of the library, taken over as it is
        tlsAdoptPtr = nullptr;
        return;
    }
    tlsAdoptPtr = nullptr;
    if (bytes > 0) data_ = static_cast<float*>(devicePoolAcquire(bytes));
}

DeviceTensor::~DeviceTensor() {
    if (data_ != nullptr) devicePoolRelease(data_, elementCount() * sizeof(float));
}

DeviceTensor::DeviceTensor(DeviceTensor&& other) noexcept : data_(other.data_), shape_(std::move(other.shape_)) {
    other.data_ = nullptr;
    other.shape_.clear();
}

DeviceTensor& DeviceTensor::operator=(DeviceTensor&& other) noexcept {
    if (this != &other) {
        if (data_ != nullptr) devicePoolRelease(data_, elementCount() * sizeof(float));
        data_ = other.data_;
        shape_ = std::move(other.shape_);
        other.data_ = nullptr;
        other.shape_.clear();
    }
    return *this;
}

std::size_t DeviceTensor::elementCount() const { return shape_.empty() ? 0 : countOf(shape_); }

DeviceTensor DeviceTensor::fromHost(const runtime::Tensor& host) {
    DeviceTensor t(host.shape());
    if (t.elementCount() > 0) {
        check(bfb_copy_h2d(t.data_, host.data().data(), t.elementCount() * sizeof(float), nullptr));
        check(bfb_stream_synchronize(nullptr));
    }
    return t;
}

DeviceTensor DeviceTensor::zeros(std::vector<std::size_t> shape) {
    DeviceTensor t(std::move(shape));
    if (t.elementCount() > 0) check(bfb_memset_zero(t.data_, t.elementCount() * sizeof(float), nullptr));
    return t;
}

runtime::Tensor DeviceTensor::toHost() const {
    std::vector<float> host(elementCount());
    if (!host.empty()) {
        check(bfb_copy_d2h(host.data(), data_, host.size() * sizeof(float), nullptr));
        check(bfb_stream_synchronize(nullptr));
    }
    return runtime::Tensor(shape_, std::move(host));
}

DeviceTensor DeviceTensor::clone() const {
    DeviceTensor t(shape_);
    if (t.elementCount() > 0) check(bfb_copy_d2d(t.data_, data_, t.elementCount() * sizeof(float), nullptr));
    return t;
}

DeviceTensor DeviceTensor::reshaped(std::vector<std::size_t> newShape) && {
    if (countOf(newShape) != elementCount()) throw std::invalid_argument("DeviceTensor::reshaped: element count differs");
    DeviceTensor t;
    t.data_ = data_;
    t.shape_ = std::move(newShape);
    data_ = nullptr;
    shape_.clear();
    return t;
}

// ---- ops.hpp:8-258 (forward side) ---------------------------------------------------------------------------------
DeviceTensor add(const DeviceTensor& a, const DeviceTensor& b) {
    if (a.shape() != b.shape()) throw std::invalid_argument("add: shapes differ");
    DeviceTensor out(a.shape());
    check(bfb_elementwise(BFB_EW_ADD, a.data(), b.data(), nullptr, out.data(), static_cast<int64_t>(a.elementCount()), 1, nullptr));
    return out;
}

DeviceTensor addBias(const DeviceTensor& input, const DeviceTensor& bias) {
    if (input.rank() < 1 || bias.rank() != 1 || bias.dim(0) != input.dim(input.rank() - 1)) {
        throw std::invalid_argument("addBias: bias must match the last dimension");
    }
    DeviceTensor out(input.shape());
    check(bfb_elementwise(BFB_EW_ADD_BIAS, input.data(), bias.data(), nullptr, out.data(),
                          static_cast<int64_t>(input.elementCount()), static_cast<int64_t>(bias.dim(0)), nullptr));
    return out;
}

DeviceTensor addBiasSilu(const DeviceTensor& gemmOutput, const DeviceTensor& bias) {
    if (gemmOutput.rank() < 1 || bias.rank() != 1 || bias.dim(0) != gemmOutput.dim(gemmOutput.rank() - 1)) {
        throw std::invalid_argument("addBiasSilu: bias must match the last dimension");
    }
    DeviceTensor out(gemmOutput.shape());
    check(bfb_elementwise(BFB_EW_ADD_BIAS_SILU, gemmOutput.data(), bias.data(), nullptr, out.data(),
                          static_cast<int64_t>(gemmOutput.elementCount()), static_cast<int64_t>(bias.dim(0)), nullptr));
    return out;
}

DeviceTensor addBiasResidual(const DeviceTensor& gemmOutput, const DeviceTensor& bias, const DeviceTensor& residual) {
    if (gemmOutput.rank() < 1 || bias.rank() != 1 || bias.dim(0) != gemmOutput.dim(gemmOutput.rank() - 1) ||
        residual.shape() != gemmOutput.shape()) {
        throw std::invalid_argument("addBiasResidual: incompatible shapes");
    }
    DeviceTensor out(gemmOutput.shape());
    check(bfb_elementwise(BFB_EW_ADD_BIAS_RESIDUAL, gemmOutput.data(), bias.data(), residual.data(), out.data(),
                          static_cast<int64_t>(gemmOutput.elementCount()), static_cast<int64_t>(bias.dim(0)), nullptr));
    return out;
}

DeviceTensor matmul(const DeviceTensor& a, const DeviceTensor& b) {
    requireMatmulShapes(a, b, "matmul");
    return gemm(a.data(), b.data(), a.dim(0), b.dim(1), a.dim(1), false, BFB_EPI_NONE, nullptr, nullptr, {a.dim(0), b.dim(1)});
}

DeviceTensor matmulTransposeB(const DeviceTensor& a, const DeviceTensor& b) {
    if (a.rank() != 2 || b.rank() != 2 || a.dim(1) != b.dim(1)) throw std::invalid_argument("matmulTransposeB: incompatible shapes");
    DeviceTensor c({a.dim(0), b.dim(0)});
    check(bfb_matmul_transpose_b(a.data(), b.data(), c.data(), static_cast<int64_t>(a.dim(0)), static_cast<int64_t>(b.dim(0)),
                                 static_cast<int64_t>(a.dim(1)), nullptr));
    return c;
}

DeviceTensor matmulBf16(const DeviceTensor& a, const DeviceTensor& b) {
    requireMatmulShapes(a, b, "matmulBf16");
    return gemm(a.data(), b.data(), a.dim(0), b.dim(1), a.dim(1), true, BFB_EPI_NONE, nullptr, nullptr, {a.dim(0), b.dim(1)});
}

// The operator-level call converts its weight on every call; Model keeps converted weights inside the library.
DeviceTensor matmulBf16CachedWeight(const DeviceTensor& a, const DeviceTensor& b) { return matmulBf16(a, b); }
void invalidateBf16WeightCache() {}

DeviceTensor silu(const DeviceTensor& input) { return unary(BFB_EW_SILU, input); }
DeviceTensor relu(const DeviceTensor& input) { return unary(BFB_EW_RELU, input); }
DeviceTensor gelu(const DeviceTensor& input) { return unary(BFB_EW_GELU, input); }

DeviceTensor rmsnorm(const DeviceTensor& input) {
    if (input.rank() < 1) throw std::invalid_argument("rmsnorm: rank >= 1 required");
    DeviceTensor out(input.shape());
    if (input.elementCount() > 0) {
        check(bfb_rmsnorm(input.data(), BFB_F32, out.data(), BFB_F32, static_cast<int64_t>(rowsOf(input)),
                          static_cast<int64_t>(input.dim(input.rank() - 1)), 1e-6f, nullptr));
    }
    return out;
}

DeviceTensor softmax(const DeviceTensor& input) {
    if (input.rank() < 1) throw std::invalid_argument("softmax: rank >= 1 required");
    DeviceTensor out(input.shape());
    if (input.elementCount() > 0) {
        check(bfb_softmax(input.data(), out.data(), static_cast<int64_t>(rowsOf(input)),
                          static_cast<int64_t>(input.dim(input.rank() - 1)), nullptr));
    }
    return out;
}

namespace {
DeviceTensor embeddingImpl(const DeviceTensor& tokenIds, const DeviceTensor& table, bool validate) {
    if (tokenIds.rank() != 2 || table.rank() != 2) throw std::invalid_argument("embeddingLookup: ids [batch, seq] and table [vocab, dim] required");
    DeviceTensor out({tokenIds.dim(0), tokenIds.dim(1), table.dim(1)});
    int32_t* oob = nullptr;
    if (validate) {
        oob = static_cast<int32_t*>(devicePoolAcquire(sizeof(int32_t)));
        check(bfb_memset_zero(oob, sizeof(int32_t), nullptr));
    }
    const bfb_status st = bfb_embed_pos(tokenIds.data(), table.data(), nullptr, out.data(), BFB_F32, static_cast<int64_t>(tokenIds.dim(0)),
                                        static_cast<int64_t>(tokenIds.dim(1)), static_cast<int64_t>(table.dim(0)),
                                        static_cast<int64_t>(table.dim(1)), 0, 0, oob, nullptr);
    int32_t bad = 0;
    if (validate) {
        if (st == BFB_OK) {
            bfb_copy_d2h(&bad, oob, sizeof(bad), nullptr);
            bfb_stream_synchronize(nullptr);
        }
        devicePoolRelease(oob, sizeof(int32_t));
    }
    check(st);
    if (bad != 0) throw std::invalid_argument("embeddingLookup: token id outside the vocabulary");
    return out;
}
}  // namespace

DeviceTensor embeddingLookup(const DeviceTensor& tokenIds, const DeviceTensor& table) { return embeddingImpl(tokenIds, table, true); }
DeviceTensor embeddingLookupPreValidated(const DeviceTensor& tokenIds, const DeviceTensor& table) {
    return embeddingImpl(tokenIds, table, false);
}

DeviceTensor addPositionalEmbeddingAt(const DeviceTensor& input, const DeviceTensor& table, std::size_t offset) {
    if (input.rank() != 3) throw std::invalid_argument("addPositionalEmbedding: input [batch, seq, dim] required");
    if (table.rank() != 2 || table.dim(1) != input.dim(2)) throw std::invalid_argument("addPositionalEmbedding: table must be [maxSeqLen, dim]");
    if (offset + input.dim(1) > table.dim(0)) throw std::invalid_argument("addPositionalEmbedding: sequence exceeds maxSeqLen of the table");
    DeviceTensor out(input.shape());
    check(bfb_add_positional(input.data(), table.data(), out.data(), static_cast<int64_t>(input.dim(0)),
                             static_cast<int64_t>(input.dim(1)), static_cast<int64_t>(input.dim(2)),
                             static_cast<int64_t>(table.dim(0)), static_cast<int64_t>(offset), nullptr));
    return out;
}

DeviceTensor addPositionalEmbedding(const DeviceTensor& input, const DeviceTensor& table) {
    return addPositionalEmbeddingAt(input, table, 0);
}

DeviceTensor linear(const DeviceTensor& input, const DeviceTensor& weight, const DeviceTensor& bias) {
    return linearImpl(input, weight, bias, false);
}
DeviceTensor linearBf16(const DeviceTensor& input, const DeviceTensor& weight, const DeviceTensor& bias) {
    return linearImpl(input, weight, bias, true);
}
DeviceTensor linearBf16CachedWeight(const DeviceTensor& input, const DeviceTensor& weight, const DeviceTensor& bias) {
    return linearImpl(input, weight, bias, true);
}

DeviceTensor feedForward(const DeviceTensor& input, const DeviceTensor& w1, const DeviceTensor& b1, const DeviceTensor& w2,
                         const DeviceTensor& b2) {
    return feedForwardImpl(input, w1, b1, w2, b2, false);
}
DeviceTensor feedForwardBf16(const DeviceTensor& input, const DeviceTensor& w1, const DeviceTensor& b1,
                             const DeviceTensor& w2, const DeviceTensor& b2) {
    return feedForwardImpl(input, w1, b1, w2, b2, true);
}

DeviceTensor selfAttention(const DeviceTensor& input, const DeviceTensor& wq, const DeviceTensor& wk, const DeviceTensor& wv,
                           const DeviceTensor& wout, std::size_t numHeads) {
    return selfAttentionImpl(input, wq, wk, wv, wout, numHeads, false, nullptr);
}
DeviceTensor selfAttentionBf16(const DeviceTensor& input, const DeviceTensor& wq, const DeviceTensor& wk,
                               const DeviceTensor& wv, const DeviceTensor& wout, std::size_t numHeads) {
    return selfAttentionImpl(input, wq, wk, wv, wout, numHeads, true, nullptr);
}
DeviceTensor selfAttentionIncremental(const DeviceTensor& newInput, const DeviceTensor& wq, const DeviceTensor& wk,
                                      const DeviceTensor& wv, const DeviceTensor& wout, std::size_t numHeads, KVCache& cache) {
    return selfAttentionImpl(newInput, wq, wk, wv, wout, numHeads, false, &cache);
}
DeviceTensor selfAttentionIncrementalBf16(const DeviceTensor& newInput, const DeviceTensor& wq, const DeviceTensor& wk,
                                          const DeviceTensor& wv, const DeviceTensor& wout, std::size_t numHeads,
                                          KVCache& cache) {
    return selfAttentionImpl(newInput, wq, wk, wv, wout, numHeads, true, &cache);
}

// ---- fused_attention.hpp:42-57 ---------------------------------------------------------------------------------
FusedAttentionForwardResult fusedAttentionForward(const DeviceTensor& q, const DeviceTensor& k, const DeviceTensor& v,
                                                  std::size_t numHeads, float scaleFactor, std::size_t oldLen) {
    if (q.rank() != 3 || k.rank() != 3 || v.rank() != 3 || k.shape() != v.shape() || q.dim(0) != k.dim(0) ||
        q.dim(2) != k.dim(2) || numHeads == 0 || q.dim(2) % numHeads != 0 || k.dim(1) != oldLen + q.dim(1)) {
        throw std::invalid_argument("fusedAttentionForward: incompatible shapes");
    }
    FusedAttentionForwardResult r;
    r.m = DeviceTensor({q.dim(0), numHeads, q.dim(1)});
    r.l = DeviceTensor({q.dim(0), numHeads, q.dim(1)});
    r.output = attentionCore(q, k, v, numHeads, scaleFactor, oldLen, false, &r.m, &r.l);
    return r;
}

// ---- fused_attention.hpp:59-76 ---------------------------------------------------------------------------------
// The one piece of the training side that is served: the gradient of the attention core, in the reference's fp32
// arithmetic (the tensor-core route of the library is reached through bfb_attention_bwd with bf16 operands).
FusedAttentionGrad fusedAttentionBackward(const DeviceTensor& dOutput, const DeviceTensor& q, const DeviceTensor& k,
                                          const DeviceTensor& v, const DeviceTensor& output, const DeviceTensor& m,
                                          const DeviceTensor& l, std::size_t numHeads, float scaleFactor,
                                          std::size_t oldLen) {
    if (q.rank() != 3 || k.rank() != 3 || v.rank() != 3 || k.shape() != v.shape() || q.dim(0) != k.dim(0) ||
        q.dim(2) != k.dim(2) || numHeads == 0 || q.dim(2) % numHeads != 0 || k.dim(1) != oldLen + q.dim(1) ||
        dOutput.shape() != q.shape() || output.shape() != q.shape() ||
        m.elementCount() != q.dim(0) * numHeads * q.dim(1) || l.elementCount() != m.elementCount()) {
        throw std::invalid_argument("fusedAttentionBackward: incompatible shapes");
    }
    const std::size_t batch = q.dim(0), newLen = q.dim(1), totalLen = k.dim(1), dim = q.dim(2), hd = dim / numHeads;
    FusedAttentionGrad g;
    g.dQ = DeviceTensor(q.shape());
    g.dK = DeviceTensor(k.shape());
    g.dV = DeviceTensor(k.shape());
    DeviceTensor scratch({2, batch, numHeads, newLen});
    const int64_t ld = static_cast<int64_t>(dim);
    check(bfb_attention_bwd(dOutput.data(), q.data(), k.data(), v.data(), output.data(), m.data(), l.data(), g.dQ.data(),
                            g.dK.data(), g.dV.data(), scratch.data(), BFB_F32, static_cast<int64_t>(batch),
                            static_cast<int64_t>(newLen), static_cast<int64_t>(totalLen), static_cast<int64_t>(numHeads),
                            static_cast<int64_t>(hd), ld, ld, ld, ld, scaleFactor, static_cast<int64_t>(oldLen), 1, nullptr,
                            nullptr));
    check(bfb_stream_synchronize(nullptr));   // the scratch tensor goes back to the pool on return
    return g;
}

// ---- model.hpp:57-113 -------------------------------------------------------------------------------------------
std::vector<Parameter*> Model::allParameterSlots(LayerState& layer) {
    std::vector<Parameter*> out;
    for (std::optional<Parameter>* slot : {&layer.weight, &layer.bias, &layer.embeddingTable, &layer.positionalTable,
                                           &layer.attnWq, &layer.attnWk, &layer.attnWv, &layer.attnWout, &layer.ffW1,
                                           &layer.ffB1, &layer.ffW2, &layer.ffB2}) {
        if (slot->has_value()) out.push_back(&slot->value());
    }
    return out;
}

Model::Model(const ir::ModelIR& modelIR, unsigned int seed, std::optional<ir::PrecisionPolicy> precision)
    : name_(modelIR.name) {
    int64_t inputLastDim = 0;
    const std::vector<bfb_op_desc> ops = describe(modelIR, &inputLastDim);
    const bfb_precision prec = precisionOf(precision);
    useTensorCoreLinear_ = precision.has_value() && precision->compute == sema::DType::BF16;
    bfb_model* handle = nullptr;
    check(bfb_model_create(ops.data(), static_cast<int32_t>(ops.size()), inputLastDim, seed, &prec, &handle));
    // the header's own parameter slots, in the library's (= the checkpoint's) order, holding copies of its weights
    int next = 0;
    try {
        for (const ir::Operation& op : modelIR.pipelines.front().operations) {
            LayerState layer;
            layer.kind = op.kind;
            auto take = [&](std::optional<Parameter>& slot) {
                Parameter p;
                p.name = bfb_model_param_name(handle, next);
                p.value = paramFromLibrary(handle, next);
                slot = std::move(p);
                ++next;
            };
            switch (op.kind) {
                case ir::OpKind::Linear: take(layer.weight); take(layer.bias); break;
                case ir::OpKind::Embedding:
                    take(layer.embeddingTable);
                    layer.embeddingVocabSize = static_cast<std::size_t>(op.embeddingVocabSize);
                    break;
                case ir::OpKind::PositionalEmbedding:
                    take(layer.positionalTable);
                    layer.positionalMaxSeqLen = static_cast<std::size_t>(op.positionalMaxSeqLen);
                    break;
                case ir::OpKind::Attention:
                case ir::OpKind::BidirectionalAttention:
                    take(layer.attnWq); take(layer.attnWk); take(layer.attnWv); take(layer.attnWout);
                    layer.attentionNumHeads = static_cast<std::size_t>(op.attentionNumHeads);
                    break;
                case ir::OpKind::FeedForward: take(layer.ffW1); take(layer.ffB1); take(layer.ffW2); take(layer.ffB2); break;
                default: break;
            }
            layers_.push_back(std::move(layer));
        }
        if (next != bfb_model_param_count(handle)) throw std::runtime_error("cuda::Model: parameter layout differs from the library's");
    } catch (...) {
        bfb_model_destroy(handle);
        throw;
    }
    ModelState st;
    st.handle = handle;
    for (Parameter* p : parameters()) st.pushed.push_back(p->value.data());
    std::lock_guard<std::mutex> lock(gModelsMutex);
    gModels[this] = std::move(st);
}

std::vector<Parameter*> Model::parameters() {
    std::vector<Parameter*> out;
    for (LayerState& layer : layers_) {
        for (Parameter* p : allParameterSlots(layer)) out.push_back(p);
    }
    return out;
}

namespace {
// parameters whose value tensor was replaced since the last push go to the library (checkpoint loads, tests that
// assign p->value); the library then rebuilds its converted weights at the next forward
void pushChangedParameters(Model& model, ModelState& st) {
    std::vector<Parameter*> params = model.parameters();
    for (std::size_t i = 0; i < params.size(); ++i) {
        if (params[i]->value.data() == st.pushed[i]) continue;
        const runtime::Tensor host = params[i]->value.toHost();
        check(bfb_model_param_set(st.handle, static_cast<int32_t>(i), host.data().data()));
        st.pushed[i] = params[i]->value.data();
    }
}

DeviceTensor runModel(Model& model, const DeviceTensor& input, bool trusted, bool incremental) {
    ModelState& st = stateOf(&model);
    pushChangedParameters(model, st);
    std::vector<int64_t> shape(input.shape().begin(), input.shape().end());
    float* out = nullptr;
    int64_t outShape[8] = {0};
    int32_t outRank = 0;
    check((incremental ? bfb_model_forward_incremental : bfb_model_forward)(
        st.handle, input.data(), shape.data(), static_cast<int32_t>(shape.size()), trusted ? 1 : 0, &out, outShape, &outRank,
        nullptr));
    return adopt(out, std::vector<std::size_t>(outShape, outShape + outRank));
}
}  // namespace

DeviceTensor Model::forward(const DeviceTensor& input, bool inputRangeTrusted) {
    return runModel(*this, input, inputRangeTrusted, false);
}

DeviceTensor Model::forwardIncremental(const DeviceTensor& newTokenIds) { return runModel(*this, newTokenIds, false, true); }

void Model::resetGenerationState() {
    check(bfb_model_reset_generation(stateOf(this).handle));
    generationPosition_ = 0;
}

void Model::backward(const DeviceTensor&, bool) {
    throw std::runtime_error("cuda::Model::backward: training is outside this backend (forward path only)");
}

void Model::zeroGrad() {
    throw std::runtime_error("cuda::Model::zeroGrad: training is outside this backend (forward path only)");
}

std::optional<std::size_t> Model::firstLayerEmbeddingVocabSize() const {
    if (!layers_.empty() && layers_.front().kind == ir::OpKind::Embedding) return layers_.front().embeddingVocabSize;
    return std::nullopt;
}

// ---- checkpoint.hpp:24-27 -----------------------------------------------------------------------------------------
void loadCheckpoint(Model& model, const std::string& path) {
    ModelState& st = stateOf(&model);
    pushChangedParameters(model, st);
    check(bfb_model_load_checkpoint(st.handle, path.c_str()));
    // the header's parameter objects follow the library
    std::vector<Parameter*> params = model.parameters();
    for (std::size_t i = 0; i < params.size(); ++i) {
        params[i]->value = paramFromLibrary(st.handle, static_cast<int>(i));
        st.pushed[i] = params[i]->value.data();
    }
}

void saveCheckpoint(Model& model, const std::string& path) {
    ModelState& st = stateOf(&model);
    pushChangedParameters(model, st);
    check(bfb_model_save_checkpoint(st.handle, path.c_str()));
}

// ---- executor.hpp:20-33 ---------------------------------------------------------------------------------------------
runtime::Tensor Executor::makeSyntheticInput(const ir::ModelIR& model, std::size_t batchSize) const {
    int64_t inputLastDim = 0;
    const std::vector<bfb_op_desc> ops = describe(model, &inputLastDim);
    const ir::Value& in = model.valueById(model.inputValue);
    std::vector<int64_t> declared;
    std::vector<std::size_t> shape;
    for (const ir::Dim& d : in.shape) {
        declared.push_back(d.isSymbolic ? -1 : d.literalValue);
        shape.push_back(d.isSymbolic ? batchSize : static_cast<std::size_t>(d.literalValue));
    }
    std::vector<float> data(countOf(shape));
    check(bfb_synthetic_input(ops.data(), static_cast<int32_t>(ops.size()), declared.data(), static_cast<int32_t>(declared.size()),
                              static_cast<int64_t>(batchSize), seed_, data.data()));
    return runtime::Tensor(std::move(shape), std::move(data));
}

runtime::Tensor Executor::run(const ir::ModelIR& model, const runtime::Tensor& input) const {
    int64_t inputLastDim = 0;
    const std::vector<bfb_op_desc> ops = describe(model, &inputLastDim);
    const bfb_precision none{};
    bfb_model* handle = nullptr;
    check(bfb_model_create(ops.data(), static_cast<int32_t>(ops.size()), inputLastDim, seed_, &none, &handle));
    std::vector<int64_t> shape(input.shape().begin(), input.shape().end());
    int64_t outShape[8] = {0};
    int32_t outRank = 0;
    bfb_status st = bfb_model_forward_host(handle, input.data().data(), shape.data(), static_cast<int32_t>(shape.size()), nullptr,
                                           outShape, &outRank);
    std::vector<float> out;
    std::vector<std::size_t> dims;
    if (st == BFB_OK) {
        dims.assign(outShape, outShape + outRank);
        out.resize(countOf(dims));
        st = bfb_model_forward_host(handle, input.data().data(), shape.data(), static_cast<int32_t>(shape.size()), out.data(),
                                    outShape, &outRank);
    }
    bfb_model_destroy(handle);
    check(st);
    return runtime::Tensor(std::move(dims), std::move(out));
}

}  // namespace blackforge::backend::cuda
