// DeviceTensor and the free-function operator API on fp32 device tensors.
// Each function checks shapes the way the reference's does (std::invalid_argument), then calls the
// kernel layer. Everything runs on the legacy default stream, like the reference.
#include <cmath>
#include <cstring>
#include <stdexcept>
#include <unordered_map>
#include <utility>

#include "../common.cuh"
#include "../kernels.hpp"
#include "../pool.hpp"
#include "bfb200.hpp"

namespace bfb200 {

using bfb::require;

std::size_t HostTensor::elementCount() const {
    std::size_t n = 1;
    for (std::size_t d : shape) n *= d;
    return n;
}

void* devicePoolAcquire(std::size_t bytes) { return bfb::poolAcquire(bytes); }
void devicePoolRelease(void* ptr, std::size_t bytes) { bfb::poolRelease(ptr, bytes); }

// ---- DeviceTensor -----------------------------------------------------------------------------------

namespace {
std::size_t countOf(const std::vector<std::size_t>& shape) {
    std::size_t n = 1;
    for (std::size_t d : shape) n *= d;
    return n;
}
}  // namespace

DeviceTensor::DeviceTensor(std::vector<std::size_t> shape) : shape_(std::move(shape)) {
    data_ = static_cast<float*>(bfb::poolAcquire(countOf(shape_) * sizeof(float)));
}

DeviceTensor::~DeviceTensor() {
    if (data_ != nullptr) bfb::poolRelease(data_, countOf(shape_) * sizeof(float));
}

DeviceTensor::DeviceTensor(DeviceTensor&& other) noexcept : data_(other.data_), shape_(std::move(other.shape_)) {
    other.data_ = nullptr;
    other.shape_.clear();
}

DeviceTensor& DeviceTensor::operator=(DeviceTensor&& other) noexcept {
    if (this != &other) {
        if (data_ != nullptr) bfb::poolRelease(data_, countOf(shape_) * sizeof(float));
        data_ = other.data_;
        shape_ = std::move(other.shape_);
        other.data_ = nullptr;
        other.shape_.clear();
    }
    return *this;
}

std::size_t DeviceTensor::elementCount() const { return countOf(shape_); }

DeviceTensor DeviceTensor::fromHost(const HostTensor& host) {
    require(host.data.size() == host.elementCount(), "DeviceTensor::fromHost: data size does not match shape");
    DeviceTensor t(host.shape);
    if (!host.data.empty()) {
        BFB_CUDA(cudaMemcpy(t.data_, host.data.data(), host.data.size() * sizeof(float), cudaMemcpyHostToDevice));
    }
    return t;
}

DeviceTensor DeviceTensor::zeros(std::vector<std::size_t> shape) {
    DeviceTensor t(std::move(shape));
    if (t.elementCount() > 0) BFB_CUDA(cudaMemset(t.data_, 0, t.elementCount() * sizeof(float)));
    return t;
}

HostTensor DeviceTensor::toHost() const {
    HostTensor h;
    h.shape = shape_;
    h.data.resize(elementCount());
    if (!h.data.empty()) {
        BFB_CUDA(cudaMemcpy(h.data.data(), data_, h.data.size() * sizeof(float), cudaMemcpyDeviceToHost));
    }
    return h;
}

DeviceTensor DeviceTensor::clone() const {
    DeviceTensor t(shape_);
    if (elementCount() > 0) {
        BFB_CUDA(cudaMemcpy(t.data_, data_, elementCount() * sizeof(float), cudaMemcpyDeviceToDevice));
    }
    return t;
}

DeviceTensor DeviceTensor::reshaped(std::vector<std::size_t> newShape) && {
    require(countOf(newShape) == elementCount(), "DeviceTensor::reshaped: element count differs");
    DeviceTensor t;
    t.data_ = data_;
    t.shape_ = std::move(newShape);
    data_ = nullptr;
    shape_.clear();
    return t;
}

DeviceTensor DeviceTensor::borrow(float* data, std::vector<std::size_t> shape) {
    DeviceTensor t;
    t.data_ = data;
    t.shape_ = std::move(shape);
    return t;
}

float* DeviceTensor::releaseOwnership() {
    float* p = data_;
    data_ = nullptr;
    shape_.clear();
    return p;
}

// ---- helpers ----------------------------------------------------------------------------------------

namespace {

// Scratch device buffer from the pool (any element format), released on scope exit.
struct Scratch {
    void* ptr = nullptr;
    std::size_t bytes = 0;
    explicit Scratch(std::size_t b) : ptr(bfb::poolAcquire(b)), bytes(b) {}
    ~Scratch() { bfb::poolRelease(ptr, bytes); }
    Scratch(const Scratch&) = delete;
    Scratch& operator=(const Scratch&) = delete;
    template <typename T>
    T* as() { return static_cast<T*>(ptr); }
};

std::size_t rowsOf(const DeviceTensor& t) { return t.elementCount() / t.shape().back(); }

std::vector<std::size_t> withLast(const DeviceTensor& t, std::size_t last) {
    std::vector<std::size_t> s = t.shape();
    s.back() = last;
    return s;
}

DeviceTensor unary(int op, const DeviceTensor& x) {
    DeviceTensor out(x.shape());
    bfb::elementwise(op, x.data(), nullptr, nullptr, out.data(), static_cast<int64_t>(x.elementCount()), 0, nullptr);
    return out;
}

// C = epilogue(A * W) with A, W fp32 device tensors; abDtype selects the arithmetic.
DeviceTensor gemmOp(const DeviceTensor& a2d, std::size_t m, std::size_t k, const DeviceTensor& w, int abDtype,
                    int epilogue, const float* bias, const float* residual, std::vector<std::size_t> outShape) {
    std::size_t n = w.dim(1);
    DeviceTensor out(std::move(outShape));
    bfb::GemmArgs g;
    g.m = static_cast<int64_t>(m);
    g.n = static_cast<int64_t>(n);
    g.k = static_cast<int64_t>(k);
    g.c = out.data();
    g.cDtype = BFB_F32;
    g.epilogue = epilogue;
    g.bias = bias;
    g.residual = residual;
    g.bLayout = BFB_B_KN;
    if (abDtype == BFB_F32) {
        g.a = a2d.data();
        g.b = w.data();
        g.abDtype = BFB_F32;
        bfb::gemm(g, nullptr);
        return out;
    }
    if (abDtype == BFB_BF16) {
        // the reference converts both operands on every call (ops_tensorcore.cu:316-317)
        Scratch a16(m * k * 2), w16(k * n * 2);
        bfb::castScaled(a2d.data(), BFB_F32, a16.ptr, BFB_BF16, static_cast<int64_t>(m * k), 1.0f, nullptr, nullptr);
        bfb::castScaled(w.data(), BFB_F32, w16.ptr, BFB_BF16, static_cast<int64_t>(k * n), 1.0f, nullptr, nullptr);
        g.a = a16.ptr;
        g.b = w16.ptr;
        g.abDtype = BFB_BF16;
        bfb::gemm(g, nullptr);
        return out;
    }
    // e4m3 with per-tensor amax scales
    Scratch a8(m * k), w8(k * n), stats(6 * sizeof(float));
    float* st = stats.as<float>();  // [0] amax a, [1] amax w, [2..3] scales a, [4..5] scales w
    BFB_CUDA(cudaMemsetAsync(st, 0, 6 * sizeof(float), nullptr));
    bfb::amax(a2d.data(), BFB_F32, static_cast<int64_t>(m * k), st + 0, nullptr);
    bfb::amax(w.data(), BFB_F32, static_cast<int64_t>(k * n), st + 1, nullptr);
    bfb::fp8ScaleFromAmax(st + 0, st + 2, nullptr);
    bfb::fp8ScaleFromAmax(st + 1, st + 4, nullptr);
    bfb::castScaled(a2d.data(), BFB_F32, a8.ptr, BFB_FP8_E4M3, static_cast<int64_t>(m * k), 1.0f, st + 2, nullptr);
    bfb::weightPrepare(w.data(), w8.ptr, BFB_FP8_E4M3, static_cast<int64_t>(k), static_cast<int64_t>(n), 1.0f, st + 4,
                       nullptr);
    // alpha = 1 / (scale_a * scale_w), computed on the host after a small copy (op-level API only)
    float hs[6];
    BFB_CUDA(cudaMemcpy(hs, st, sizeof(hs), cudaMemcpyDeviceToHost));
    g.a = a8.ptr;
    g.b = w8.ptr;
    g.abDtype = BFB_FP8_E4M3;
    g.bLayout = BFB_B_NK;
    g.alpha = hs[3] * hs[5];
    bfb::gemm(g, nullptr);
    return out;
}

void requireMatmulShapes(const DeviceTensor& a, const DeviceTensor& b, const char* name) {
    if (a.rank() != 2 || b.rank() != 2 || a.dim(1) != b.dim(0)) {
        throw std::invalid_argument(std::string(name) + ": incompatible shapes");
    }
}

DeviceTensor linearImpl(const DeviceTensor& input, const DeviceTensor& weight, const DeviceTensor& bias, int abDtype,
                        int epilogue, const float* residual, const char* name) {
    if (input.rank() < 2) throw std::invalid_argument(std::string(name) + ": input of rank >= 2 required");
    if (weight.rank() != 2 || input.shape().back() != weight.dim(0)) {
        throw std::invalid_argument(std::string(name) + ": weight must be [in_features, out_features]");
    }
    if (bias.rank() != 1 || bias.dim(0) != weight.dim(1)) {
        throw std::invalid_argument(std::string(name) + ": bias must be [out_features]");
    }
    return gemmOp(input, rowsOf(input), input.shape().back(), weight, abDtype, epilogue, bias.data(), residual,
                  withLast(input, weight.dim(1)));
}

FusedAttentionForwardResult attentionImpl(const DeviceTensor& q, const DeviceTensor& k, const DeviceTensor& v,
                                          std::size_t numHeads, float scaleFactor, std::size_t oldLen, bool bf16) {
    if (q.rank() != 3 || k.rank() != 3 || v.rank() != 3) {
        throw std::invalid_argument("fusedAttentionForward: q, k, v must be [batch, len, dim]");
    }
    std::size_t batch = q.dim(0), newLen = q.dim(1), dim = q.dim(2), totalLen = k.dim(1);
    if (k.dim(0) != batch || v.dim(0) != batch || k.dim(2) != dim || v.dim(2) != dim || v.dim(1) != totalLen) {
        throw std::invalid_argument("fusedAttentionForward: q, k, v shapes disagree");
    }
    if (numHeads == 0 || dim % numHeads != 0) {
        throw std::invalid_argument("fusedAttentionForward: numHeads must divide dim");
    }
    std::size_t headDim = dim / numHeads;
    if (headDim > 256) throw std::invalid_argument("fusedAttentionForward: head_dim above 256 is not supported");
    if (oldLen + newLen != totalLen) {
        throw std::invalid_argument("fusedAttentionForward: old_len + new_len must equal total_len");
    }
    FusedAttentionForwardResult r{DeviceTensor({batch, newLen, dim}), DeviceTensor({batch, numHeads, newLen}),
                                  DeviceTensor({batch, numHeads, newLen})};
    bfb::AttentionArgs a;
    a.batch = static_cast<int64_t>(batch);
    a.newLen = static_cast<int64_t>(newLen);
    a.totalLen = static_cast<int64_t>(totalLen);
    a.numHeads = static_cast<int64_t>(numHeads);
    a.headDim = static_cast<int64_t>(headDim);
    a.ldQ = a.ldK = a.ldV = a.ldO = static_cast<int64_t>(dim);
    a.scale = scaleFactor;
    a.oldLen = static_cast<int64_t>(oldLen);
    a.causal = 1;
    a.m = r.m.data();
    a.l = r.l.data();
    if (!bf16) {
        a.dtype = BFB_F32;
        a.q = q.data();
        a.k = k.data();
        a.v = v.data();
        a.out = r.output.data();
        bfb::attentionForward(a, nullptr);
        return r;
    }
    std::size_t nq = q.elementCount(), nk = k.elementCount();
    Scratch q16(nq * 2), k16(nk * 2), v16(nk * 2), o16(nq * 2);
    bfb::castScaled(q.data(), BFB_F32, q16.ptr, BFB_BF16, static_cast<int64_t>(nq), 1.0f, nullptr, nullptr);
    bfb::castScaled(k.data(), BFB_F32, k16.ptr, BFB_BF16, static_cast<int64_t>(nk), 1.0f, nullptr, nullptr);
    bfb::castScaled(v.data(), BFB_F32, v16.ptr, BFB_BF16, static_cast<int64_t>(nk), 1.0f, nullptr, nullptr);
    a.dtype = BFB_BF16;
    a.q = q16.ptr;
    a.k = k16.ptr;
    a.v = v16.ptr;
    a.out = o16.ptr;
    bfb::attentionForward(a, nullptr);
    bfb::castScaled(o16.ptr, BFB_BF16, r.output.data(), BFB_F32, static_cast<int64_t>(nq), 1.0f, nullptr, nullptr);
    return r;
}

FusedAttentionGrad attentionBackwardImpl(const DeviceTensor& dOutput, const DeviceTensor& q, const DeviceTensor& k,
                                         const DeviceTensor& v, const DeviceTensor& output, const DeviceTensor& m,
                                         const DeviceTensor& l, std::size_t numHeads, float scaleFactor,
                                         std::size_t oldLen, bool bf16) {
    if (q.rank() != 3 || k.rank() != 3 || v.rank() != 3) {
        throw std::invalid_argument("fusedAttentionBackward: q, k, v must be [batch, len, dim]");
    }
    std::size_t batch = q.dim(0), newLen = q.dim(1), dim = q.dim(2), totalLen = k.dim(1);
    if (k.dim(0) != batch || v.dim(0) != batch || k.dim(2) != dim || v.dim(2) != dim || v.dim(1) != totalLen ||
        dOutput.shape() != q.shape() || output.shape() != q.shape()) {
        throw std::invalid_argument("fusedAttentionBackward: operand shapes disagree");
    }
    if (numHeads == 0 || dim % numHeads != 0) {
        throw std::invalid_argument("fusedAttentionBackward: numHeads must divide dim");
    }
    std::size_t headDim = dim / numHeads;
    if (headDim > 256) throw std::invalid_argument("fusedAttentionBackward: head_dim above 256 is not supported");
    if (oldLen + newLen != totalLen) {
        throw std::invalid_argument("fusedAttentionBackward: old_len + new_len must equal total_len");
    }
    std::size_t statCount = batch * numHeads * newLen;
    if (m.elementCount() != statCount || l.elementCount() != statCount) {
        throw std::invalid_argument("fusedAttentionBackward: m and l must be [batch, heads, new_len]");
    }
    FusedAttentionGrad g{DeviceTensor({batch, newLen, dim}), DeviceTensor({batch, totalLen, dim}),
                         DeviceTensor({batch, totalLen, dim})};
    Scratch stats(std::max<std::size_t>(statCount, 1) * 2 * sizeof(float));
    bfb::AttentionBackwardArgs a;
    a.batch = static_cast<int64_t>(batch);
    a.newLen = static_cast<int64_t>(newLen);
    a.totalLen = static_cast<int64_t>(totalLen);
    a.numHeads = static_cast<int64_t>(numHeads);
    a.headDim = static_cast<int64_t>(headDim);
    a.ldQ = a.ldK = a.ldV = a.ldO = a.ldDo = a.ldDq = a.ldDk = a.ldDv = static_cast<int64_t>(dim);
    a.scale = scaleFactor;
    a.oldLen = static_cast<int64_t>(oldLen);
    a.causal = 1;
    a.m = m.data();
    a.l = l.data();
    a.dQ = g.dQ.data();
    a.dK = g.dK.data();
    a.dV = g.dV.data();
    a.lse2Scratch = stats.as<float>();
    a.dTermScratch = stats.as<float>() + statCount;
    if (!bf16) {
        a.dtype = BFB_F32;
        a.dOut = dOutput.data();
        a.q = q.data();
        a.k = k.data();
        a.v = v.data();
        a.out = output.data();
        bfb::attentionBackward(a, nullptr);
        return g;
    }
    std::size_t nq = q.elementCount(), nk = k.elementCount();
    Scratch q16(nq * 2), k16(nk * 2), v16(nk * 2), o16(nq * 2), g16(nq * 2);
    bfb::castScaled(q.data(), BFB_F32, q16.ptr, BFB_BF16, static_cast<int64_t>(nq), 1.0f, nullptr, nullptr);
    bfb::castScaled(k.data(), BFB_F32, k16.ptr, BFB_BF16, static_cast<int64_t>(nk), 1.0f, nullptr, nullptr);
    bfb::castScaled(v.data(), BFB_F32, v16.ptr, BFB_BF16, static_cast<int64_t>(nk), 1.0f, nullptr, nullptr);
    bfb::castScaled(output.data(), BFB_F32, o16.ptr, BFB_BF16, static_cast<int64_t>(nq), 1.0f, nullptr, nullptr);
    bfb::castScaled(dOutput.data(), BFB_F32, g16.ptr, BFB_BF16, static_cast<int64_t>(nq), 1.0f, nullptr, nullptr);
    a.dtype = BFB_BF16;
    a.dOut = g16.ptr;
    a.q = q16.ptr;
    a.k = k16.ptr;
    a.v = v16.ptr;
    a.out = o16.ptr;
    bfb::attentionBackward(a, nullptr);
    return g;
}

DeviceTensor selfAttentionImpl(const DeviceTensor& input, const DeviceTensor& wq, const DeviceTensor& wk,
                               const DeviceTensor& wv, const DeviceTensor& wout, std::size_t numHeads, bool bf16,
                               const char* name) {
    if (input.rank() != 3) throw std::invalid_argument(std::string(name) + ": input [batch, seq, dim] required");
    std::size_t batch = input.dim(0), seq = input.dim(1), dim = input.dim(2);
    if (numHeads == 0 || dim % numHeads != 0) {
        throw std::invalid_argument(std::string(name) + ": numHeads must divide dim");
    }
    for (const DeviceTensor* w : {&wq, &wk, &wv, &wout}) {
        if (w->rank() != 2 || w->dim(0) != dim || w->dim(1) != dim) {
            throw std::invalid_argument(std::string(name) + ": projection weights must be [dim, dim]");
        }
    }
    std::size_t headDim = dim / numHeads;
    float scaleFactor = 1.0f / std::sqrt(static_cast<float>(headDim));
    int ab = bf16 ? BFB_BF16 : BFB_F32;
    DeviceTensor normed = rmsnorm(input);
    std::size_t rows = batch * seq;
    DeviceTensor q = gemmOp(normed, rows, dim, wq, ab, BFB_EPI_NONE, nullptr, nullptr, {batch, seq, dim});
    DeviceTensor k = gemmOp(normed, rows, dim, wk, ab, BFB_EPI_NONE, nullptr, nullptr, {batch, seq, dim});
    DeviceTensor v = gemmOp(normed, rows, dim, wv, ab, BFB_EPI_NONE, nullptr, nullptr, {batch, seq, dim});
    FusedAttentionForwardResult attn = attentionImpl(q, k, v, numHeads, scaleFactor, 0, bf16);
    // residual add fused into the output projection
    return gemmOp(attn.output, rows, dim, wout, ab, BFB_EPI_RESIDUAL, nullptr, input.data(), {batch, seq, dim});
}

DeviceTensor selfAttentionIncrementalImpl(const DeviceTensor& newInput, const DeviceTensor& wq, const DeviceTensor& wk,
                                          const DeviceTensor& wv, const DeviceTensor& wout, std::size_t numHeads,
                                          KVCache& cache, bool bf16, const char* name) {
    if (newInput.rank() != 3) throw std::invalid_argument(std::string(name) + ": input [batch, seq, dim] required");
    std::size_t batch = newInput.dim(0), newLen = newInput.dim(1), dim = newInput.dim(2);
    if (numHeads == 0 || dim % numHeads != 0) {
        throw std::invalid_argument(std::string(name) + ": numHeads must divide dim");
    }
    for (const DeviceTensor* w : {&wq, &wk, &wv, &wout}) {
        if (w->rank() != 2 || w->dim(0) != dim || w->dim(1) != dim) {
            throw std::invalid_argument(std::string(name) + ": projection weights must be [dim, dim]");
        }
    }
    if (cache.length > 0 && (cache.k.rank() != 3 || cache.k.dim(0) != batch || cache.k.dim(2) != dim ||
                             cache.k.dim(1) != cache.length)) {
        throw std::invalid_argument(std::string(name) + ": the cache does not belong to this batch / width");
    }
    float scaleFactor = 1.0f / std::sqrt(static_cast<float>(dim / numHeads));
    int ab = bf16 ? BFB_BF16 : BFB_F32;
    // the norm is per position, so normalising the new positions alone is exact
    DeviceTensor normed = rmsnorm(newInput);
    std::size_t rows = batch * newLen;
    DeviceTensor q = gemmOp(normed, rows, dim, wq, ab, BFB_EPI_NONE, nullptr, nullptr, {batch, newLen, dim});
    DeviceTensor kNew = gemmOp(normed, rows, dim, wk, ab, BFB_EPI_NONE, nullptr, nullptr, {batch, newLen, dim});
    DeviceTensor vNew = gemmOp(normed, rows, dim, wv, ab, BFB_EPI_NONE, nullptr, nullptr, {batch, newLen, dim});
    const std::size_t oldLen = cache.length;
    if (oldLen == 0) {
        cache.k = std::move(kNew);
        cache.v = std::move(vNew);
    } else {
        cache.k = concatSeq(cache.k, kNew);
        cache.v = concatSeq(cache.v, vNew);
    }
    cache.length = oldLen + newLen;
    FusedAttentionForwardResult attn = attentionImpl(q, cache.k, cache.v, numHeads, scaleFactor, oldLen, bf16);
    return gemmOp(attn.output, rows, dim, wout, ab, BFB_EPI_RESIDUAL, nullptr, newInput.data(), {batch, newLen, dim});
}

DeviceTensor feedForwardImpl(const DeviceTensor& input, const DeviceTensor& w1, const DeviceTensor& b1,
                             const DeviceTensor& w2, const DeviceTensor& b2, bool bf16, const char* name) {
    if (input.rank() < 2) throw std::invalid_argument(std::string(name) + ": input of rank >= 2 required");
    int ab = bf16 ? BFB_BF16 : BFB_F32;
    DeviceTensor normed = rmsnorm(input);
    DeviceTensor hidden = linearImpl(normed, w1, b1, ab, BFB_EPI_BIAS_SILU, nullptr, name);
    if (w2.rank() != 2 || w2.dim(1) != input.shape().back()) {
        throw std::invalid_argument(std::string(name) + ": w2 must map back to the input width");
    }
    return linearImpl(hidden, w2, b2, ab, BFB_EPI_BIAS_RESIDUAL, input.data(), name);
}

}  // namespace

// ---- elementwise ------------------------------------------------------------------------------------

DeviceTensor add(const DeviceTensor& a, const DeviceTensor& b) {
    if (a.shape() != b.shape()) throw std::invalid_argument("add: shapes differ");
    DeviceTensor out(a.shape());
    bfb::elementwise(BFB_EW_ADD, a.data(), b.data(), nullptr, out.data(), static_cast<int64_t>(a.elementCount()), 0,
                     nullptr);
    return out;
}

namespace {
void requireBias(const DeviceTensor& input, const DeviceTensor& bias, const char* name) {
    if (input.rank() < 2 || bias.rank() != 1 || input.shape().back() != bias.dim(0)) {
        throw std::invalid_argument(std::string(name) + ": expected input [..., features] and bias [features]");
    }
}
}  // namespace

DeviceTensor addBias(const DeviceTensor& input, const DeviceTensor& bias) {
    requireBias(input, bias, "addBias");
    DeviceTensor out(input.shape());
    bfb::elementwise(BFB_EW_ADD_BIAS, input.data(), bias.data(), nullptr, out.data(),
                     static_cast<int64_t>(input.elementCount()), static_cast<int64_t>(bias.dim(0)), nullptr);
    return out;
}

DeviceTensor addBiasSilu(const DeviceTensor& gemmOutput, const DeviceTensor& bias) {
    requireBias(gemmOutput, bias, "addBiasSilu");
    DeviceTensor out(gemmOutput.shape());
    bfb::elementwise(BFB_EW_ADD_BIAS_SILU, gemmOutput.data(), bias.data(), nullptr, out.data(),
                     static_cast<int64_t>(gemmOutput.elementCount()), static_cast<int64_t>(bias.dim(0)), nullptr);
    return out;
}

DeviceTensor addBiasResidual(const DeviceTensor& gemmOutput, const DeviceTensor& bias, const DeviceTensor& residual) {
    requireBias(gemmOutput, bias, "addBiasResidual");
    if (gemmOutput.shape() != residual.shape()) throw std::invalid_argument("addBiasResidual: residual shape differs");
    DeviceTensor out(gemmOutput.shape());
    bfb::elementwise(BFB_EW_ADD_BIAS_RESIDUAL, gemmOutput.data(), bias.data(), residual.data(), out.data(),
                     static_cast<int64_t>(gemmOutput.elementCount()), static_cast<int64_t>(bias.dim(0)), nullptr);
    return out;
}

DeviceTensor silu(const DeviceTensor& input) { return unary(BFB_EW_SILU, input); }
DeviceTensor relu(const DeviceTensor& input) { return unary(BFB_EW_RELU, input); }
DeviceTensor gelu(const DeviceTensor& input) { return unary(BFB_EW_GELU, input); }

DeviceTensor rmsnorm(const DeviceTensor& input) {
    if (input.rank() < 2) throw std::invalid_argument("rmsnorm: input of rank >= 2 required");
    DeviceTensor out(input.shape());
    bfb::rmsnorm(input.data(), BFB_F32, out.data(), BFB_F32, static_cast<int64_t>(rowsOf(input)),
                 static_cast<int64_t>(input.shape().back()), 1e-6f, nullptr);
    return out;
}

DeviceTensor softmax(const DeviceTensor& input) {
    if (input.rank() < 2) throw std::invalid_argument("softmax: input of rank >= 2 required");
    DeviceTensor out(input.shape());
    bfb::softmaxRows(input.data(), out.data(), static_cast<int64_t>(rowsOf(input)),
                     static_cast<int64_t>(input.shape().back()), nullptr);
    return out;
}

// ---- matmul family ----------------------------------------------------------------------------------

DeviceTensor matmul(const DeviceTensor& a, const DeviceTensor& b) {
    requireMatmulShapes(a, b, "matmul");
    return gemmOp(a, a.dim(0), a.dim(1), b, BFB_F32, BFB_EPI_NONE, nullptr, nullptr, {a.dim(0), b.dim(1)});
}

DeviceTensor matmulTransposeB(const DeviceTensor& a, const DeviceTensor& b) {
    if (a.rank() != 2 || b.rank() != 2 || a.dim(1) != b.dim(1)) {
        throw std::invalid_argument("matmulTransposeB: incompatible shapes");
    }
    DeviceTensor out({a.dim(0), b.dim(0)});
    bfb::matmulTransposeB(a.data(), b.data(), out.data(), static_cast<int64_t>(a.dim(0)), static_cast<int64_t>(b.dim(0)),
                          static_cast<int64_t>(a.dim(1)), nullptr);
    return out;
}

DeviceTensor matmulBf16(const DeviceTensor& a, const DeviceTensor& b) {
    requireMatmulShapes(a, b, "matmulBf16");
    return gemmOp(a, a.dim(0), a.dim(1), b, BFB_BF16, BFB_EPI_NONE, nullptr, nullptr, {a.dim(0), b.dim(1)});
}

DeviceTensor matmulFp8(const DeviceTensor& a, const DeviceTensor& b) {
    requireMatmulShapes(a, b, "matmulFp8");
    return gemmOp(a, a.dim(0), a.dim(1), b, BFB_FP8_E4M3, BFB_EPI_NONE, nullptr, nullptr, {a.dim(0), b.dim(1)});
}

// bf16 [N,K] copies of weights, keyed by device pointer, valid until invalidateBf16WeightCache()
// (the reference keys on pointer + generation counter, ops_tensorcore.cu:98-131).
namespace {
struct CachedWeight {
    void* ptr;
    std::size_t bytes;
    std::size_t k, n;
};
// bf16 copies in the weight's own [K,N] layout, which the backward's dA = G B^T reads as its [N,K] operand
std::unordered_map<const float*, CachedWeight>& naturalWeightCache() {
    static std::unordered_map<const float*, CachedWeight> cache;
    return cache;
}
std::unordered_map<const float*, CachedWeight>& weightCache() {
    static std::unordered_map<const float*, CachedWeight> cache;
    return cache;
}
}  // namespace

void invalidateBf16WeightCache() {
    for (auto& kv : weightCache()) bfb::poolRelease(kv.second.ptr, kv.second.bytes);
    weightCache().clear();
    for (auto& kv : naturalWeightCache()) bfb::poolRelease(kv.second.ptr, kv.second.bytes);
    naturalWeightCache().clear();
}

namespace {
MatmulGrad matmulBackwardImpl(const DeviceTensor& a, const DeviceTensor& b, const DeviceTensor& gradOutput, bool cached,
                              const char* name) {
    if (a.rank() != 2 || b.rank() != 2 || gradOutput.rank() != 2 || a.dim(1) != b.dim(0) ||
        gradOutput.dim(0) != a.dim(0) || gradOutput.dim(1) != b.dim(1)) {
        throw std::invalid_argument(std::string(name) + ": incompatible shapes");
    }
    std::size_t m = a.dim(0), k = a.dim(1), n = b.dim(1);
    const void* natural = nullptr;
    if (cached && k * n > 0) {
        auto& cache = naturalWeightCache();
        auto it = cache.find(b.data());
        if (it == cache.end() || it->second.k != k || it->second.n != n) {
            if (it != cache.end()) {
                bfb::poolRelease(it->second.ptr, it->second.bytes);
                cache.erase(it);
            }
            CachedWeight cw{bfb::poolAcquire(k * n * 2), k * n * 2, k, n};
            bfb::castScaled(b.data(), BFB_F32, cw.ptr, BFB_BF16, static_cast<int64_t>(k * n), 1.0f, nullptr, nullptr);
            it = cache.emplace(b.data(), cw).first;
        }
        natural = it->second.ptr;
    }
    MatmulGrad g{DeviceTensor({m, k}), DeviceTensor({k, n})};
    bfb::matmulBf16Backward(a.data(), b.data(), gradOutput.data(), g.dA.data(), g.dB.data(), static_cast<int64_t>(m),
                            static_cast<int64_t>(k), static_cast<int64_t>(n), natural, nullptr);
    return g;
}
}  // namespace

MatmulGrad matmulBf16Backward(const DeviceTensor& a, const DeviceTensor& b, const DeviceTensor& gradOutput) {
    return matmulBackwardImpl(a, b, gradOutput, false, "matmulBf16Backward");
}

MatmulGrad matmulBf16BackwardCachedWeight(const DeviceTensor& a, const DeviceTensor& b, const DeviceTensor& gradOutput) {
    return matmulBackwardImpl(a, b, gradOutput, true, "matmulBf16BackwardCachedWeight");
}

DeviceTensor matmulBf16CachedWeight(const DeviceTensor& a, const DeviceTensor& b) {
    requireMatmulShapes(a, b, "matmulBf16CachedWeight");
    std::size_t m = a.dim(0), k = a.dim(1), n = b.dim(1);
    auto& cache = weightCache();
    auto it = cache.find(b.data());
    if (it == cache.end() || it->second.k != k || it->second.n != n) {
        if (it != cache.end()) {
            bfb::poolRelease(it->second.ptr, it->second.bytes);
            cache.erase(it);
        }
        CachedWeight cw{bfb::poolAcquire(k * n * 2), k * n * 2, k, n};
        bfb::weightPrepare(b.data(), cw.ptr, BFB_BF16, static_cast<int64_t>(k), static_cast<int64_t>(n), 1.0f, nullptr,
                           nullptr);
        it = cache.emplace(b.data(), cw).first;
    }
    Scratch a16(m * k * 2);
    bfb::castScaled(a.data(), BFB_F32, a16.ptr, BFB_BF16, static_cast<int64_t>(m * k), 1.0f, nullptr, nullptr);
    DeviceTensor out({m, n});
    bfb::GemmArgs g;
    g.a = a16.ptr;
    g.b = it->second.ptr;
    g.c = out.data();
    g.m = static_cast<int64_t>(m);
    g.n = static_cast<int64_t>(n);
    g.k = static_cast<int64_t>(k);
    g.abDtype = BFB_BF16;
    g.bLayout = BFB_B_NK;
    g.cDtype = BFB_F32;
    bfb::gemm(g, nullptr);
    return out;
}

DeviceTensor linear(const DeviceTensor& input, const DeviceTensor& weight, const DeviceTensor& bias) {
    return linearImpl(input, weight, bias, BFB_F32, BFB_EPI_BIAS, nullptr, "linear");
}

DeviceTensor linearBf16(const DeviceTensor& input, const DeviceTensor& weight, const DeviceTensor& bias) {
    return linearImpl(input, weight, bias, BFB_BF16, BFB_EPI_BIAS, nullptr, "linearBf16");
}

// ---- embedding / positions --------------------------------------------------------------------------

namespace {
DeviceTensor embeddingImpl(const DeviceTensor& tokenIds, const DeviceTensor& table, bool validate) {
    if (tokenIds.rank() != 2) throw std::invalid_argument("embeddingLookup: token ids must be [batch, seq]");
    if (table.rank() != 2) throw std::invalid_argument("embeddingLookup: table must be [vocabSize, dim]");
    std::size_t batch = tokenIds.dim(0), seq = tokenIds.dim(1), vocab = table.dim(0), dim = table.dim(1);
    DeviceTensor out({batch, seq, dim});
    if (!validate) {
        bfb::embedPos(tokenIds.data(), table.data(), nullptr, out.data(), BFB_F32, static_cast<int64_t>(batch),
                      static_cast<int64_t>(seq), static_cast<int64_t>(vocab), static_cast<int64_t>(dim), 0, 0, nullptr,
                      nullptr);
        return out;
    }
    // range check on the device: one counter comes back instead of the whole id tensor
    Scratch counter(sizeof(int));
    BFB_CUDA(cudaMemsetAsync(counter.ptr, 0, sizeof(int), nullptr));
    bfb::embedPos(tokenIds.data(), table.data(), nullptr, out.data(), BFB_F32, static_cast<int64_t>(batch),
                  static_cast<int64_t>(seq), static_cast<int64_t>(vocab), static_cast<int64_t>(dim), 0, 0,
                  counter.as<int>(), nullptr);
    int bad = 0;
    BFB_CUDA(cudaMemcpy(&bad, counter.ptr, sizeof(int), cudaMemcpyDeviceToHost));
    if (bad != 0) {
        throw std::invalid_argument("embeddingLookup: " + std::to_string(bad) + " token id(s) outside the vocabulary [0, " +
                                    std::to_string(vocab) + ")");
    }
    return out;
}
}  // namespace

DeviceTensor embeddingLookup(const DeviceTensor& tokenIds, const DeviceTensor& table) {
    return embeddingImpl(tokenIds, table, true);
}

DeviceTensor embeddingLookupPreValidated(const DeviceTensor& tokenIds, const DeviceTensor& table) {
    return embeddingImpl(tokenIds, table, false);
}

DeviceTensor addPositionalEmbeddingAt(const DeviceTensor& input, const DeviceTensor& table, std::size_t offset) {
    if (input.rank() != 3) throw std::invalid_argument("addPositionalEmbedding: input [batch, seq, dim] required");
    if (table.rank() != 2 || table.dim(1) != input.dim(2)) {
        throw std::invalid_argument("addPositionalEmbedding: table must be [maxSeqLen, dim]");
    }
    if (offset + input.dim(1) > table.dim(0)) {
        throw std::invalid_argument("addPositionalEmbedding: sequence exceeds maxSeqLen of the table");
    }
    DeviceTensor out(input.shape());
    bfb::addPositional(input.data(), table.data(), out.data(), static_cast<int64_t>(input.dim(0)),
                       static_cast<int64_t>(input.dim(1)), static_cast<int64_t>(input.dim(2)),
                       static_cast<int64_t>(table.dim(0)), static_cast<int64_t>(offset), nullptr);
    return out;
}

DeviceTensor addPositionalEmbedding(const DeviceTensor& input, const DeviceTensor& table) {
    return addPositionalEmbeddingAt(input, table, 0);
}

// ---- blocks -----------------------------------------------------------------------------------------

DeviceTensor feedForward(const DeviceTensor& input, const DeviceTensor& w1, const DeviceTensor& b1,
                         const DeviceTensor& w2, const DeviceTensor& b2) {
    return feedForwardImpl(input, w1, b1, w2, b2, false, "feedForward");
}

DeviceTensor feedForwardBf16(const DeviceTensor& input, const DeviceTensor& w1, const DeviceTensor& b1,
                             const DeviceTensor& w2, const DeviceTensor& b2) {
    return feedForwardImpl(input, w1, b1, w2, b2, true, "feedForwardBf16");
}

// ops_transformer.cu:159-167 (concatSeq): [batch, la, dim] ++ [batch, lb, dim] -> [batch, la + lb, dim].
DeviceTensor concatSeq(const DeviceTensor& a, const DeviceTensor& b) {
    if (a.rank() != 3 || b.rank() != 3 || a.dim(0) != b.dim(0) || a.dim(2) != b.dim(2)) {
        throw std::invalid_argument("concatSeq: tensors must be [batch, len, dim] with equal batch and dim");
    }
    const std::size_t batch = a.dim(0), la = a.dim(1), lb = b.dim(1), dim = a.dim(2);
    DeviceTensor out({batch, la + lb, dim});
    if (batch == 0 || dim == 0) return out;
    const std::size_t pitch = (la + lb) * dim * sizeof(float);
    // one strided copy per source: each batch entry is a "row" of la * dim (lb * dim) floats
    if (la > 0) {
        BFB_CUDA(cudaMemcpy2DAsync(out.data(), pitch, a.data(), la * dim * sizeof(float), la * dim * sizeof(float), batch,
                                   cudaMemcpyDeviceToDevice, nullptr));
    }
    if (lb > 0) {
        BFB_CUDA(cudaMemcpy2DAsync(out.data() + la * dim, pitch, b.data(), lb * dim * sizeof(float),
                                   lb * dim * sizeof(float), batch, cudaMemcpyDeviceToDevice, nullptr));
    }
    return out;
}

DeviceTensor selfAttentionIncremental(const DeviceTensor& newInput, const DeviceTensor& wq, const DeviceTensor& wk,
                                      const DeviceTensor& wv, const DeviceTensor& wout, std::size_t numHeads,
                                      KVCache& cache) {
    return selfAttentionIncrementalImpl(newInput, wq, wk, wv, wout, numHeads, cache, false, "selfAttentionIncremental");
}

DeviceTensor selfAttentionIncrementalBf16(const DeviceTensor& newInput, const DeviceTensor& wq, const DeviceTensor& wk,
                                          const DeviceTensor& wv, const DeviceTensor& wout, std::size_t numHeads,
                                          KVCache& cache) {
    return selfAttentionIncrementalImpl(newInput, wq, wk, wv, wout, numHeads, cache, true, "selfAttentionIncrementalBf16");
}

DeviceTensor selfAttention(const DeviceTensor& input, const DeviceTensor& wq, const DeviceTensor& wk,
                           const DeviceTensor& wv, const DeviceTensor& wout, std::size_t numHeads) {
    return selfAttentionImpl(input, wq, wk, wv, wout, numHeads, false, "selfAttention");
}

DeviceTensor selfAttentionBf16(const DeviceTensor& input, const DeviceTensor& wq, const DeviceTensor& wk,
                               const DeviceTensor& wv, const DeviceTensor& wout, std::size_t numHeads) {
    return selfAttentionImpl(input, wq, wk, wv, wout, numHeads, true, "selfAttentionBf16");
}

FusedAttentionForwardResult fusedAttentionForward(const DeviceTensor& q, const DeviceTensor& k, const DeviceTensor& v,
                                                  std::size_t numHeads, float scaleFactor, std::size_t oldLen) {
    return attentionImpl(q, k, v, numHeads, scaleFactor, oldLen, false);
}

FusedAttentionForwardResult fusedAttentionForwardBf16(const DeviceTensor& q, const DeviceTensor& k,
                                                      const DeviceTensor& v, std::size_t numHeads, float scaleFactor,
                                                      std::size_t oldLen) {
    return attentionImpl(q, k, v, numHeads, scaleFactor, oldLen, true);
}

FusedAttentionGrad fusedAttentionBackward(const DeviceTensor& dOutput, const DeviceTensor& q, const DeviceTensor& k,
                                          const DeviceTensor& v, const DeviceTensor& output, const DeviceTensor& m,
                                          const DeviceTensor& l, std::size_t numHeads, float scaleFactor,
                                          std::size_t oldLen) {
    return attentionBackwardImpl(dOutput, q, k, v, output, m, l, numHeads, scaleFactor, oldLen, false);
}

FusedAttentionGrad fusedAttentionBackwardBf16(const DeviceTensor& dOutput, const DeviceTensor& q, const DeviceTensor& k,
                                              const DeviceTensor& v, const DeviceTensor& output, const DeviceTensor& m,
                                              const DeviceTensor& l, std::size_t numHeads, float scaleFactor,
                                              std::size_t oldLen) {
    return attentionBackwardImpl(dOutput, q, k, v, output, m, l, numHeads, scaleFactor, oldLen, true);
}

}  // namespace bfb200
