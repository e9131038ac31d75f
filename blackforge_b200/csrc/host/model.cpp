// Model / Executor / checkpoints: the device side of the IR executor.
//
// Model::forward has two routes. Without a precision block (or with `compute fp32`) it interprets
// the pipeline op by op on fp32 tensors — the exactness route compared against the CPU backend.
// With `compute bf16` or `compute fp8.e4m3` it runs the planned route: weights converted once to
// K-major bf16 / e4m3 (Q, K, V fused into one matrix), activations kept in a reusable arena, and
// per block
//   rmsnorm -> [QKV GEMM] -> flash attention -> [out-proj GEMM + residual]
//   rmsnorm -> [GEMM + bias + silu] -> [GEMM + bias + residual]
// with every bias / activation / residual pass folded into a GEMM epilogue. On a bf16 residual stream with
// bf16 operands the rmsnorm is folded too: the GEMM after it reads x and scales its rows in the epilogue, and
// the GEMM that writes x delivers the row sums of squares the next norm needs. `storage bf16` keeps
// the residual stream in bf16 (each op output rounded once, the CPU backend's meaning of storage);
// otherwise it stays fp32. Results leave as fp32 tensors either way.
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <random>
#include <stdexcept>

#include "../common.cuh"
#include "../kernels.hpp"
#include "../pool.hpp"
#include "bfb200.hpp"
#include "tp.hpp"

namespace bfb200 {

using bfb::fail;
using bfb::require;

// ---- seeded default initialisation --------------------------------------------------------------------
// Salts per parameter slot (src/backend/cpu/model.cpp:14-26, src/backend/cuda/model.cu:17-28): part of
// the reproducibility contract of `run` without a checkpoint.
namespace {
constexpr unsigned int kWeightSalt = 0x2545F491U;
constexpr unsigned int kBiasSalt = 0x27D4EB2FU;
constexpr unsigned int kEmbeddingSalt = 0x85EBCA6BU;
constexpr unsigned int kPositionalSalt = 0xC2B2AE35U;
constexpr unsigned int kAttnWqSalt = 0x27D4EB2DU;
constexpr unsigned int kAttnWkSalt = 0x165667B1U;
constexpr unsigned int kAttnWvSalt = 0xD3A2646CU;
constexpr unsigned int kAttnWoutSalt = 0xFD7046C5U;
constexpr unsigned int kFFW1Salt = 0xB55A4F09U;
constexpr unsigned int kFFB1Salt = 0x5BD1E995U;
constexpr unsigned int kFFW2Salt = 0x9E3779B9U;
constexpr unsigned int kFFB2Salt = 0x1B873593U;
constexpr unsigned int kInputSalt = 0x9E3779B1U;
}  // namespace

HostTensor randomTensor(std::vector<std::size_t> shape, unsigned int seed) {
    std::mt19937 rng(seed);
    std::uniform_real_distribution<float> dist(-0.1F, 0.1F);
    HostTensor t;
    t.shape = std::move(shape);
    t.data.resize(t.elementCount());
    for (float& v : t.data) v = dist(rng);
    return t;
}

HostTensor randomTokenIdTensor(std::vector<std::size_t> shape, std::size_t vocabSize, unsigned int seed) {
    std::mt19937 rng(seed);
    std::uniform_int_distribution<std::size_t> dist(0, vocabSize > 0 ? vocabSize - 1 : 0);
    HostTensor t;
    t.shape = std::move(shape);
    t.data.resize(t.elementCount());
    for (float& v : t.data) v = static_cast<float>(dist(rng));
    return t;
}

unsigned int seedFor(unsigned int base, std::size_t valueId, unsigned int salt) {
    return base ^ (static_cast<unsigned int>(valueId) * salt);
}

// ---- Model::Impl ----------------------------------------------------------------------------------------

namespace {

enum class Shard { None, Cols, Rows, Vec };  // how a parameter is split across tensor-parallel ranks

enum class Mode { Fp32, Bf16, Fp8 };

struct DevBuf {
    void* ptr = nullptr;
    std::size_t bytes = 0;
    void reset() {
        if (ptr != nullptr) bfb::poolRelease(ptr, bytes);
        ptr = nullptr;
        bytes = 0;
    }
    void ensure(std::size_t need) {
        if (bytes == need && ptr != nullptr) return;
        reset();
        ptr = bfb::poolAcquire(need);
        bytes = need;
    }
};

struct ParamMeta {
    Shard shard = Shard::None;
    unsigned int salt = 0;
    std::size_t valueId = 0;
};

struct Layer {
    int kind = 0;
    std::size_t outputId = 0;
    std::size_t inFeat = 0, outFeat = 0;
    std::size_t heads = 0, hidden = 0, vocab = 0, maxSeq = 0;
    int p[4] = {-1, -1, -1, -1};  // parameter indices in slot order
    bool shardedLinear = false;
    // converted weights of the planned route (this rank's part)
    DevBuf w0, w1;   // attention: fused QKV^T, Wout^T; feed-forward: W1^T, W2^T; linear: W^T
    DevBuf scales;   // fp8: [0..1] scale/inverse of w0, [2..3] of w1
    // generation state of an attention layer: the planned route keeps bf16 caches [batch, cacheRows, dim / ranks]
    // that are filled in place; the fp32 route keeps the operator-level cache
    DevBuf kCache, vCache;
    std::size_t cacheRows = 0;
    KVCache opCache;
};

}  // namespace

struct Model::Impl {
    std::vector<OpDesc> ops;
    std::int64_t inputLastDim = 0;
    unsigned int seed = 42;
    std::optional<PrecisionPolicy> precision;
    int tpRank = 0, tpWorld = 1;
    Mode mode = Mode::Fp32;
    int streamDtype = BFB_F32;
    bool storageBf16 = false;
    bool randomInit = true;
    bool built = false;
    bool prepared = false;
    bool mastersReleased = false;  // fp32 copies of the GEMM weights dropped after conversion
    std::vector<Parameter> params;
    std::vector<ParamMeta> meta;
    std::vector<Layer> layers;
    std::map<std::string, DevBuf> arena;
    std::size_t genPosition = 0;   // positions already in the caches
    std::size_t genBatch = 0;      // batch size the caches were opened with
    DevBuf fp8Stats;  // per GEMM input: [amax, scale, inverse, alpha]
    DevBuf status;    // device status word for bounded waits + id range counter
    // Tensor-parallel prompt passes run the layers over `tpChunks` groups of sequences, the all-reduce of one group on
    // `commStream` beside the next group's GEMMs, which leave `tpReserveSms` SMs to it.
    // benchmark(): when set, the forward records a timing event on its stream before each pipeline operation it
    // starts (an operation fused into its predecessor records none) and one after the last
    struct OpMarks {
        std::vector<cudaEvent_t> events;
        std::vector<std::size_t> opIndex;   // pipeline position of the operation that starts at events[i]
        std::size_t used = 0;
        void mark(std::size_t op, cudaStream_t stream) {
            if (used == events.size()) {
                cudaEvent_t e = nullptr;
                BFB_CUDA(cudaEventCreate(&e));
                events.push_back(e);
                opIndex.push_back(0);
            }
            opIndex[used] = op;
            BFB_CUDA(cudaEventRecord(events[used++], stream));
        }
        ~OpMarks() {
            for (cudaEvent_t e : events) cudaEventDestroy(e);
        }
    };
    OpMarks* marks = nullptr;
    int tpChunks = 2;
    int tpReserveSms = 0;
    cudaStream_t commStream = nullptr;
    std::vector<cudaEvent_t> computed, reduced;

    Impl() {
        if (const char* e = std::getenv("BFB_TP_CHUNKS")) tpChunks = std::max(1, std::atoi(e));
        if (const char* e = std::getenv("BFB_TP_RESERVE_SMS")) tpReserveSms = std::max(0, std::atoi(e));
    }

    void ensureOverlapStreams(std::size_t chunks) {
        if (commStream == nullptr) {
            int least = 0, greatest = 0;
            BFB_CUDA(cudaDeviceGetStreamPriorityRange(&least, &greatest));
            BFB_CUDA(cudaStreamCreateWithPriority(&commStream, cudaStreamNonBlocking, greatest));
        }
        while (computed.size() < chunks) {
            cudaEvent_t a = nullptr, b = nullptr;
            BFB_CUDA(cudaEventCreateWithFlags(&a, cudaEventDisableTiming));
            BFB_CUDA(cudaEventCreateWithFlags(&b, cudaEventDisableTiming));
            computed.push_back(a);
            reduced.push_back(b);
        }
    }

    ~Impl() {
        for (cudaEvent_t e : computed) cudaEventDestroy(e);
        for (cudaEvent_t e : reduced) cudaEventDestroy(e);
        if (commStream != nullptr) cudaStreamDestroy(commStream);
        for (auto& l : layers) {
            l.w0.reset();
            l.w1.reset();
            l.scales.reset();
            l.kCache.reset();
            l.vCache.reset();
        }
        for (auto& kv : arena) kv.second.reset();
        fp8Stats.reset();
        status.reset();
    }

    void* buf(const std::string& name, std::size_t bytes) {
        DevBuf& b = arena[name];
        b.ensure(bytes);
        return b.ptr;
    }

    std::vector<std::size_t> localShape(const std::vector<std::size_t>& full, Shard s) const {
        std::vector<std::size_t> shape = full;
        if (tpWorld == 1) return shape;
        if (s == Shard::Cols) shape[1] /= static_cast<std::size_t>(tpWorld);
        if (s == Shard::Rows) shape[0] /= static_cast<std::size_t>(tpWorld);
        if (s == Shard::Vec) shape[0] /= static_cast<std::size_t>(tpWorld);
        return shape;
    }

    int addParam(const std::string& name, std::vector<std::size_t> fullShape, Shard shard, unsigned int salt,
                 std::size_t valueId) {
        Parameter prm;
        prm.name = name;
        prm.fullShape = std::move(fullShape);
        params.push_back(std::move(prm));
        meta.push_back(ParamMeta{shard, salt, valueId});
        return static_cast<int>(params.size()) - 1;
    }

    void buildStructure();
    void allocateParams();
    std::vector<char> gemmWeightMask() const;
    void setParam(std::size_t index, const float* hostFull);
    void getParam(std::size_t index, float* hostFull);
    void prepare(cudaStream_t stream);
    // incremental: `input` holds the ids of the new positions only; keys and values of earlier ones are cached
    DeviceTensor forwardFp32(const DeviceTensor& input, bool trusted, bool incremental);
    // out16 != nullptr: the final linear writes bf16 there and the returned tensor is empty
    DeviceTensor forwardPlanned(const DeviceTensor& input, bool trusted, cudaStream_t stream, void* out16,
                                bool incremental);
    void ensureCache(Layer& l, std::size_t batch, std::size_t width, std::size_t rowsNeeded, std::size_t rowsHint,
                     cudaStream_t stream);
    void resetGeneration();
    void checkStatus(cudaStream_t stream, bool checkIds, std::size_t vocab);
};

void Model::Impl::buildStructure() {
    std::size_t feat = inputLastDim > 0 ? static_cast<std::size_t>(inputLastDim) : 0;
    const std::size_t w = static_cast<std::size_t>(tpWorld);
    for (std::size_t i = 0; i < ops.size(); ++i) {
        const OpDesc& op = ops[i];
        Layer layer;
        layer.kind = op.kind;
        layer.outputId = static_cast<std::size_t>(op.output);
        layer.inFeat = feat;
        const std::string id = std::to_string(op.output);
        switch (op.kind) {
            case BFB_OP_LINEAR: {
                if (feat == 0) throw std::invalid_argument("Model: linear#" + id + " needs a concrete input width");
                if (op.linear_out_features <= 0) throw std::invalid_argument("Model: linear#" + id + " needs a positive width");
                std::size_t out = static_cast<std::size_t>(op.linear_out_features);
                layer.outFeat = out;
                layer.shardedLinear = tpWorld > 1 && i + 1 == ops.size();
                if (layer.shardedLinear && out % w != 0) {
                    throw std::invalid_argument("Model: output width of the last linear must divide by the tensor-parallel size");
                }
                Shard sw = layer.shardedLinear ? Shard::Cols : Shard::None;
                Shard sb = layer.shardedLinear ? Shard::Vec : Shard::None;
                layer.p[0] = addParam("linear" + id + ".weight", {feat, out}, sw, kWeightSalt, layer.outputId);
                layer.p[1] = addParam("linear" + id + ".bias", {out}, sb, kBiasSalt, layer.outputId);
                feat = out;
                break;
            }
            case BFB_OP_EMBEDDING: {
                if (op.embedding_vocab_size <= 0 || op.embedding_dim <= 0) {
                    throw std::invalid_argument("Model: embedding#" + id + " needs positive sizes");
                }
                layer.vocab = static_cast<std::size_t>(op.embedding_vocab_size);
                layer.outFeat = static_cast<std::size_t>(op.embedding_dim);
                layer.p[0] = addParam("embedding" + id + ".table", {layer.vocab, layer.outFeat}, Shard::None,
                                      kEmbeddingSalt, layer.outputId);
                feat = layer.outFeat;
                break;
            }
            case BFB_OP_POSITIONAL_EMBEDDING: {
                if (feat == 0) throw std::invalid_argument("Model: positional_embedding#" + id + " needs a concrete input width");
                if (op.positional_max_seq_len <= 0) throw std::invalid_argument("Model: positional_embedding#" + id + " needs a positive length");
                layer.maxSeq = static_cast<std::size_t>(op.positional_max_seq_len);
                layer.outFeat = feat;
                layer.p[0] = addParam("positional_embedding" + id + ".table", {layer.maxSeq, feat}, Shard::None,
                                      kPositionalSalt, layer.outputId);
                break;
            }
            case BFB_OP_ATTENTION: {
                if (feat == 0) throw std::invalid_argument("Model: attention#" + id + " needs a concrete input width");
                std::size_t heads = static_cast<std::size_t>(std::max<std::int64_t>(op.attention_num_heads, 0));
                if (heads == 0 || feat % heads != 0) {
                    throw std::invalid_argument("Model: 'attention#" + id + "' requires " + std::to_string(heads) +
                                                " heads to divide dim=" + std::to_string(feat));
                }
                if (tpWorld > 1 && heads % w != 0) {
                    throw std::invalid_argument("Model: attention heads must divide by the tensor-parallel size");
                }
                layer.heads = heads;
                layer.outFeat = feat;
                layer.p[0] = addParam("attention" + id + ".wq", {feat, feat}, Shard::Cols, kAttnWqSalt, layer.outputId);
                layer.p[1] = addParam("attention" + id + ".wk", {feat, feat}, Shard::Cols, kAttnWkSalt, layer.outputId);
                layer.p[2] = addParam("attention" + id + ".wv", {feat, feat}, Shard::Cols, kAttnWvSalt, layer.outputId);
                layer.p[3] = addParam("attention" + id + ".wout", {feat, feat}, Shard::Rows, kAttnWoutSalt, layer.outputId);
                break;
            }
            case BFB_OP_FEEDFORWARD: {
                if (feat == 0) throw std::invalid_argument("Model: feedforward#" + id + " needs a concrete input width");
                if (op.feedforward_hidden_dim <= 0) throw std::invalid_argument("Model: feedforward#" + id + " needs a positive hidden width");
                std::size_t hidden = static_cast<std::size_t>(op.feedforward_hidden_dim);
                if (tpWorld > 1 && hidden % w != 0) {
                    throw std::invalid_argument("Model: feed-forward width must divide by the tensor-parallel size");
                }
                layer.hidden = hidden;
                layer.outFeat = feat;
                layer.p[0] = addParam("feedforward" + id + ".w1", {feat, hidden}, Shard::Cols, kFFW1Salt, layer.outputId);
                layer.p[1] = addParam("feedforward" + id + ".b1", {hidden}, Shard::Vec, kFFB1Salt, layer.outputId);
                layer.p[2] = addParam("feedforward" + id + ".w2", {hidden, feat}, Shard::Rows, kFFW2Salt, layer.outputId);
                layer.p[3] = addParam("feedforward" + id + ".b2", {feat}, Shard::None, kFFB2Salt, layer.outputId);
                break;
            }
            case BFB_OP_BIDIRECTIONAL_ATTENTION:
                throw std::invalid_argument(
                    "Model: 'bidirectional_attention' is not available on the device backend (CPU only)");
            case BFB_OP_SILU:
            case BFB_OP_RELU:
            case BFB_OP_GELU:
            case BFB_OP_RMSNORM:
            case BFB_OP_SOFTMAX:
                layer.outFeat = feat;
                break;
            default:
                throw std::invalid_argument("Model: unknown operation kind " + std::to_string(op.kind));
        }
        layers.push_back(std::move(layer));
    }
}

// GEMM weights (attention wq/wk/wv/wout, feed-forward w1/w2, linear weight) by parameter index
std::vector<char> Model::Impl::gemmWeightMask() const {
    std::vector<char> mask(params.size(), 0);
    for (const Layer& l : layers) {
        if (l.kind != BFB_OP_ATTENTION && l.kind != BFB_OP_FEEDFORWARD && l.kind != BFB_OP_LINEAR) continue;
        const int weightSlots[3][4] = {{0, 1, 2, 3}, {0, 2, -1, -1}, {0, -1, -1, -1}};
        const int* slots = l.kind == BFB_OP_ATTENTION ? weightSlots[0] : l.kind == BFB_OP_FEEDFORWARD ? weightSlots[1] : weightSlots[2];
        for (int i = 0; i < 4; ++i) {
            if (slots[i] >= 0) mask[l.p[slots[i]]] = 1;
        }
    }
    return mask;
}

void Model::Impl::allocateParams() {
    if (built) return;
    // converted weights adopted from a cache file: the fp32 copies of the GEMM weights never exist
    const std::vector<char> skip = mastersReleased ? gemmWeightMask() : std::vector<char>(params.size(), 0);
    for (std::size_t i = 0; i < params.size(); ++i) {
        if (skip[i]) continue;
        params[i].value = DeviceTensor::zeros(localShape(params[i].fullShape, meta[i].shard));
    }
    built = true;
    if (randomInit) {
        for (std::size_t i = 0; i < params.size(); ++i) {
            if (skip[i]) continue;
            HostTensor t = randomTensor(params[i].fullShape, seedFor(seed, meta[i].valueId, meta[i].salt));
            setParam(i, t.data.data());
        }
    }
}

void Model::Impl::setParam(std::size_t index, const float* hostFull) {
    allocateParams();
    require(index < params.size(), "Model: parameter index out of range");
    require(hostFull != nullptr, "Model: null parameter data");
    Parameter& prm = params[index];
    if (mastersReleased && prm.value.data() == nullptr) {
        fail(BFB_UNSUPPORTED, "Model: the fp32 copy of '" + prm.name + "' was released; it can no longer be set");
    }
    const Shard s = tpWorld > 1 ? meta[index].shard : Shard::None;
    const std::size_t n = prm.value.elementCount();
    const std::size_t w = static_cast<std::size_t>(tpWorld), r = static_cast<std::size_t>(tpRank);
    if (s == Shard::None) {
        BFB_CUDA(cudaMemcpy(prm.value.data(), hostFull, n * sizeof(float), cudaMemcpyHostToDevice));
    } else if (s == Shard::Rows || s == Shard::Vec) {
        BFB_CUDA(cudaMemcpy(prm.value.data(), hostFull + r * n, n * sizeof(float), cudaMemcpyHostToDevice));
    } else {  // column slice of [K, N]
        const std::size_t k = prm.fullShape[0], nFull = prm.fullShape[1], nLoc = nFull / w;
        BFB_CUDA(cudaMemcpy2D(prm.value.data(), nLoc * sizeof(float), hostFull + r * nLoc, nFull * sizeof(float),
                              nLoc * sizeof(float), k, cudaMemcpyHostToDevice));
    }
    if (!mastersReleased) prepared = false;
}

void Model::Impl::getParam(std::size_t index, float* hostFull) {
    allocateParams();
    require(index < params.size(), "Model: parameter index out of range");
    require(hostFull != nullptr, "Model: null parameter buffer");
    if (tpWorld > 1 && meta[index].shard != Shard::None) {
        fail(BFB_UNSUPPORTED, "Model: reading back a tensor-parallel parameter is not supported");
    }
    Parameter& prm = params[index];
    if (mastersReleased && prm.value.data() == nullptr) {
        fail(BFB_UNSUPPORTED, "Model: the fp32 copy of '" + prm.name + "' was released");
    }
    BFB_CUDA(cudaMemcpy(hostFull, prm.value.data(), prm.value.elementCount() * sizeof(float), cudaMemcpyDeviceToHost));
}

// Convert weights once for the planned route.
void Model::Impl::prepare(cudaStream_t stream) {
    allocateParams();
    if (prepared || mode == Mode::Fp32) {
        prepared = true;
        return;
    }
    const int wDtype = mode == Mode::Bf16 ? BFB_BF16 : BFB_FP8_E4M3;
    const std::size_t eb = mode == Mode::Bf16 ? 2 : 1;
    // Transposes `count` fp32 [K, N_i] matrices into consecutive row blocks of dst ([sum N_i, K]); for
    // fp8 one scale is derived from the amax over all of them (the fused Q/K/V matrix counts as one tensor).
    auto convert = [&](DevBuf& dst, std::initializer_list<const DeviceTensor*> srcs, float* scaleSlot) {
        std::size_t k = (*srcs.begin())->dim(0), totalN = 0;
        for (const DeviceTensor* t : srcs) totalN += t->dim(1);
        dst.ensure(totalN * k * eb);
        const float* dScale = nullptr;
        if (mode == Mode::Fp8) {
            BFB_CUDA(cudaMemsetAsync(scaleSlot, 0, 2 * sizeof(float), stream));
            // amax lands in scaleSlot[0], then is replaced by {scale, inverse}
            for (const DeviceTensor* t : srcs) {
                bfb::amax(t->data(), BFB_F32, static_cast<int64_t>(t->elementCount()), scaleSlot, stream);
            }
            bfb::fp8ScaleFromAmax(scaleSlot, scaleSlot, stream);
            dScale = scaleSlot;
        }
        std::size_t rowOff = 0;
        for (const DeviceTensor* t : srcs) {
            bfb::weightPrepare(t->data(), static_cast<char*>(dst.ptr) + rowOff * k * eb, wDtype,
                               static_cast<int64_t>(k), static_cast<int64_t>(t->dim(1)), 1.0f, dScale, stream);
            rowOff += t->dim(1);
        }
    };
    for (Layer& l : layers) {
        if (l.kind != BFB_OP_ATTENTION && l.kind != BFB_OP_FEEDFORWARD && l.kind != BFB_OP_LINEAR) continue;
        l.scales.ensure(4 * sizeof(float));
        float* sc = static_cast<float*>(l.scales.ptr);
        if (l.kind == BFB_OP_ATTENTION) {
            convert(l.w0, {&params[l.p[0]].value, &params[l.p[1]].value, &params[l.p[2]].value}, sc);
            convert(l.w1, {&params[l.p[3]].value}, sc + 2);
        } else if (l.kind == BFB_OP_FEEDFORWARD) {
            convert(l.w0, {&params[l.p[0]].value}, sc);
            convert(l.w1, {&params[l.p[2]].value}, sc + 2);
        } else {
            convert(l.w0, {&params[l.p[0]].value}, sc);
        }
    }
    prepared = true;
}

void Model::Impl::checkStatus(cudaStream_t stream, bool checkIds, std::size_t vocab) {
    int host[2] = {0, 0};
    BFB_CUDA(cudaMemcpyAsync(host, status.ptr, sizeof(host), cudaMemcpyDeviceToHost, stream));
    if (tpWorld > 1) tpSynchronize(stream);   // with a deadline: a collective may wait for a rank that never comes
    else BFB_CUDA(cudaStreamSynchronize(stream));
    if (checkIds && host[1] != 0) {
        throw std::invalid_argument("embeddingLookup: " + std::to_string(host[1]) +
                                    " token id(s) outside the vocabulary [0, " + std::to_string(vocab) + ")");
    }
    bfb::failOnDeviceStatus(host[0]);
}

// ---- exactness route: op by op on fp32 tensors ----------------------------------------------------------
void Model::Impl::resetGeneration() {
    genPosition = 0;
    genBatch = 0;
    for (Layer& l : layers) {
        l.kCache.reset();
        l.vCache.reset();
        l.cacheRows = 0;
        l.opCache = KVCache{};
    }
}

// Room for `rowsNeeded` positions per batch entry in the layer's caches; `rowsHint` (the positional table's
// length, 0 when the pipeline has none) sizes them once, otherwise they double. Growing copies the filled rows.
void Model::Impl::ensureCache(Layer& l, std::size_t batch, std::size_t width, std::size_t rowsNeeded,
                              std::size_t rowsHint, cudaStream_t stream) {
    if (l.cacheRows >= rowsNeeded) return;
    std::size_t rows = std::max<std::size_t>(rowsHint, 256);
    while (rows < rowsNeeded) rows *= 2;
    DevBuf nk, nv;
    nk.ensure(batch * rows * width * 2);
    nv.ensure(batch * rows * width * 2);
    if (l.cacheRows > 0 && genPosition > 0) {
        const std::size_t filled = genPosition * width * 2;
        BFB_CUDA(cudaMemcpy2DAsync(nk.ptr, rows * width * 2, l.kCache.ptr, l.cacheRows * width * 2, filled, batch,
                                   cudaMemcpyDeviceToDevice, stream));
        BFB_CUDA(cudaMemcpy2DAsync(nv.ptr, rows * width * 2, l.vCache.ptr, l.cacheRows * width * 2, filled, batch,
                                   cudaMemcpyDeviceToDevice, stream));
        BFB_CUDA(cudaStreamSynchronize(stream));   // the old buffers go back to the pool below
    }
    l.kCache.reset();
    l.vCache.reset();
    l.kCache = nk;
    l.vCache = nv;
    l.cacheRows = rows;
}

DeviceTensor Model::Impl::forwardFp32(const DeviceTensor& input, bool trusted, bool incremental) {
    require(tpWorld == 1, "Model: tensor parallelism needs compute bf16 or fp8.e4m3");
    DeviceTensor current = input.clone();
    auto roundStorage = [&](DeviceTensor& t) {
        if (storageBf16) bfb::roundBf16InPlace(t.data(), static_cast<int64_t>(t.elementCount()), nullptr);
    };
    for (std::size_t i = 0; i < layers.size(); ++i) {
        Layer& l = layers[i];
        if (marks != nullptr) marks->mark(i, nullptr);
        switch (l.kind) {
            case BFB_OP_LINEAR: current = linear(current, params[l.p[0]].value, params[l.p[1]].value); break;
            case BFB_OP_SILU: current = silu(current); break;
            case BFB_OP_RELU: current = relu(current); break;
            case BFB_OP_GELU: current = gelu(current); break;
            case BFB_OP_RMSNORM: current = rmsnorm(current); break;
            case BFB_OP_SOFTMAX: current = softmax(current); break;
            case BFB_OP_EMBEDDING:
                current = (trusted && i == 0) ? embeddingLookupPreValidated(current, params[l.p[0]].value)
                                              : embeddingLookup(current, params[l.p[0]].value);
                break;
            case BFB_OP_POSITIONAL_EMBEDDING:
                current = addPositionalEmbeddingAt(current, params[l.p[0]].value, incremental ? genPosition : 0);
                break;
            case BFB_OP_ATTENTION:
                current = incremental
                              ? selfAttentionIncremental(current, params[l.p[0]].value, params[l.p[1]].value,
                                                         params[l.p[2]].value, params[l.p[3]].value, l.heads, l.opCache)
                              : selfAttention(current, params[l.p[0]].value, params[l.p[1]].value, params[l.p[2]].value,
                                              params[l.p[3]].value, l.heads);
                break;
            case BFB_OP_FEEDFORWARD:
                current = feedForward(current, params[l.p[0]].value, params[l.p[1]].value, params[l.p[2]].value,
                                      params[l.p[3]].value);
                break;
            default: fail(BFB_UNSUPPORTED, "Model: operation not available on the device");
        }
        roundStorage(current);
    }
    if (marks != nullptr) marks->mark(layers.size(), nullptr);
    if (incremental) genPosition += input.rank() >= 2 ? input.dim(1) : 0;
    return current;
}

// ---- planned route: tensor-core GEMMs + flash attention -------------------------------------------------
DeviceTensor Model::Impl::forwardPlanned(const DeviceTensor& input, bool trusted, cudaStream_t stream, void* out16,
                                          bool incremental) {
    prepare(stream);
    status.ensure(2 * sizeof(int));
    BFB_CUDA(cudaMemsetAsync(status.ptr, 0, 2 * sizeof(int), stream));
    int* dStatus = static_cast<int*>(status.ptr);
    int* dOob = dStatus + 1;
    const int S = streamDtype;
    const std::size_t sb = S == BFB_F32 ? 4 : 2;
    const int ab = mode == Mode::Bf16 ? BFB_BF16 : BFB_FP8_E4M3;
    const bool fp8 = mode == Mode::Fp8;

    // running activation: pointer + shape; dtype S except straight after a non-planned op
    std::vector<std::size_t> shape = input.shape();
    void* x = nullptr;  // [tokens, feat] in S
    std::size_t feat = shape.empty() ? 0 : shape.back();
    auto tokensOf = [&]() {
        std::size_t n = 1;
        for (std::size_t i = 0; i + 1 < shape.size(); ++i) n *= shape[i];
        return n;
    };
    bool idsChecked = false;
    std::size_t vocabForCheck = 0;
    const std::size_t oldLen = incremental ? genPosition : 0;   // positions already cached
    std::size_t cacheHint = 0;                                 // the positional table's length, when there is one
    // e4m3 operands: one block of four floats [amax/scale, inverse, alpha, -] per quantised GEMM input. An attention
    // or feed-forward layer quantises two inputs per group of sequences, any other layer at most one; the group count
    // is at most tpChunks (and 1 outside tensor-parallel prompt passes).
    int fp8Slot = 0;
    int fp8SlotLimit = 0;
    if (fp8) {
        const std::size_t maxGroups = (tpWorld > 1 && !incremental) ? static_cast<std::size_t>(std::max(tpChunks, 1)) : 1;
        fp8SlotLimit = static_cast<int>((layers.size() * 2 + 1) * maxGroups);
        fp8Stats.ensure(static_cast<std::size_t>(fp8SlotLimit) * 4 * sizeof(float));
        BFB_CUDA(cudaMemsetAsync(fp8Stats.ptr, 0, fp8Stats.bytes, stream));
    }
    // Row statistics of the current x from the epilogue of the GEMM that wrote it: sums of squares (`ss`) and, on the
    // e4m3 route, largest magnitudes (`mx`), as [parts][tokens]; ssParts == 0 means they do not describe the current x.
    float* ss = nullptr;
    float* mx = nullptr;
    int ssParts = 0;
    auto nextFp8Stats = [&]() -> float* {
        require(fp8Slot < fp8SlotLimit, "Model: more quantised GEMM inputs than scale slots");
        return static_cast<float*>(fp8Stats.ptr) + 4 * (fp8Slot++);
    };

    // A-operand of a GEMM from a bf16 activation: the buffer itself (bf16) or an e4m3 copy with a fresh
    // per-tensor scale; returns the device alpha pointer for fp8 (1 / (scale_a * scale_w)).
    auto gemmInput = [&](const void* act16, std::size_t count, const std::string& name, const float* wScales,
                         const float** dAlpha) -> const void* {
        if (!fp8) {
            *dAlpha = nullptr;
            return act16;
        }
        float* st = nextFp8Stats();  // [0]=scale [1]=inverse [2]=alpha
        void* a8 = buf(name, count);
        const int64_t n = static_cast<int64_t>(count);
        float* scratch = static_cast<float*>(
            buf("partial_" + name, static_cast<std::size_t>(bfb::quantizeScratchFloats(n)) * sizeof(float)));
        bfb::quantizeE4m3(act16, BFB_BF16, n, a8, st, wScales + 1, scratch, stream);
        *dAlpha = st + 2;
        return a8;
    };
    // e4m3 A-operand of the GEMM that follows an rmsnorm, straight from the bf16 residual stream: the norm and
    // the quantisation in two passes over x, without a normalised copy in between
    auto normedFp8Input = [&](std::size_t tokens, std::size_t d, const float* wScales, const float** dAlpha) -> const void* {
        float* st = nextFp8Stats();
        void* a8 = buf("act8_d", tokens * d);
        float* scratch = static_cast<float*>(
            buf("norm_quant", static_cast<std::size_t>(bfb::rmsnormQuantizeScratchFloats(static_cast<int64_t>(tokens))) *
                                  sizeof(float)));
        // with the producer's row statistics the first pass (1 / rms per row, the tensor's maximum) reads those
        // instead of x
        const bool fromStats = ssParts > 0 && mx != nullptr;
        bfb::rmsnormQuantizeE4m3(x, static_cast<int64_t>(tokens), static_cast<int64_t>(d), 1e-6f, a8, st, wScales + 1,
                                 scratch, stream, fromStats ? ss : nullptr, fromStats ? mx : nullptr, fromStats ? ssParts : 0);
        *dAlpha = st + 2;
        return a8;
    };
    auto runGemm = [&](const void* a, const void* w, void* c, std::size_t m, std::size_t n, std::size_t k, int cDtype,
                       int epilogue, const float* bias, const void* residual, const float* dAlpha, int roundC,
                       const float* rowSumSq = nullptr, int rowSumSqParts = 1, float* outSumSq = nullptr,
                       float* outMaxAbs = nullptr) {
        bfb::GemmArgs g;
        g.a = a;
        g.b = w;
        g.c = c;
        g.m = static_cast<int64_t>(m);
        g.n = static_cast<int64_t>(n);
        g.k = static_cast<int64_t>(k);
        g.abDtype = ab;
        g.bLayout = BFB_B_NK;
        g.cDtype = cDtype;
        g.epilogue = epilogue;
        g.bias = bias;
        g.residual = residual;
        g.dAlpha = dAlpha;
        g.roundCBf16 = roundC;
        g.dStatus = dStatus;
        g.rowSumSq = rowSumSq;
        g.rowSumSqParts = rowSumSqParts;
        g.rowInvDim = k > 0 ? 1.0f / static_cast<float>(k) : 0.0f;
        g.rowEps = 1e-6f;
        g.outSumSq = outSumSq;
        g.outMaxAbs = outMaxAbs;
        // a generation step has a handful of rows: stream the weights through every SM instead of tiling C
        g.preferSkinny = incremental && m <= 128 ? 1 : 0;
        bfb::gemm(g, stream);
    };

    // rmsnorm folded into the GEMM that follows it (bf16 residual stream, bf16 operands): an rmsnorm without
    // weights scales rows, which commutes with the product, so the GEMM reads x itself and its epilogue divides
    // row i by sqrt(mean(x_i^2) + eps). The sums of squares come from the epilogue of the GEMM that wrote x
    // (out-projection, feed-forward down-projection) or, where x has another origin (the embedding, a
    // tensor-parallel all-reduce), from one read-only pass. No normalised copy of x is written or read.
    // e4m3 operands keep the separate norm: their per-tensor scale is taken from the normalised values.
    auto fusedNormOk = [&](std::size_t tokens, std::size_t n, std::size_t d, const void* w) {
        if (fp8 || S != BFB_BF16) return false;
        bfb::GemmArgs probe;
        probe.a = x;
        probe.b = w;
        probe.c = x;
        probe.m = static_cast<int64_t>(tokens);
        probe.n = static_cast<int64_t>(n);
        probe.k = static_cast<int64_t>(d);
        probe.abDtype = ab;
        probe.bLayout = BFB_B_NK;
        probe.cDtype = BFB_BF16;
        return bfb::gemmSupportsRowStats(probe);
    };
    // Sums of squares of the rows of x as [parts][tokens]: one part from the read-only pass, one per 128 columns
    // from the epilogue of the GEMM that wrote x. One buffer is enough: by the time a GEMM writes the sums of the
    // next x, the GEMM that read the previous ones has finished (same stream).
    auto sumSqBuffer = [&](std::size_t tokens, std::size_t d) {
        return static_cast<float*>(buf("row_sumsq", ((d + 127) / 128) * tokens * sizeof(float)));
    };
    auto needSumSq = [&](std::size_t tokens, std::size_t d) {
        if (ssParts == 0) {
            ss = sumSqBuffer(tokens, d);
            bfb::rowSumSquares(x, S, ss, static_cast<int64_t>(tokens), static_cast<int64_t>(d), stream);
            ssParts = 1;
        }
        return ss;
    };
    // where the GEMM that writes the next x puts the next sums (null: it cannot deliver them)
    auto nextSumSq = [&](std::size_t tokens, std::size_t d) -> float* {
        if (tpWorld > 1) return nullptr;   // x is completed by an all-reduce: the epilogue only sees a partial sum
        return sumSqBuffer(tokens, d);
    };
    auto producedSumSq = [&](float* produced, std::size_t d, float* producedMax = nullptr) {
        ss = produced;
        mx = produced != nullptr ? producedMax : nullptr;
        ssParts = produced != nullptr ? static_cast<int>((d + 127) / 128) : 0;
    };
    // e4m3 route: can the GEMM that writes the next x (tokens x d from a reduction over k) leave the row statistics
    // the next norm + quantisation needs?
    auto fp8StatsOk = [&](const void* a, std::size_t tokens, std::size_t d, std::size_t k, const void* wt) {
        if (!fp8 || S != BFB_BF16 || incremental || tpWorld > 1) return false;
        bfb::GemmArgs probe;
        probe.a = a;
        probe.b = wt;
        probe.c = x;
        probe.m = static_cast<int64_t>(tokens);
        probe.n = static_cast<int64_t>(d);
        probe.k = static_cast<int64_t>(k);
        probe.abDtype = ab;
        probe.bLayout = BFB_B_NK;
        probe.cDtype = BFB_BF16;
        return bfb::gemmSupportsRowStats(probe);
    };
    auto maxBuffer = [&](std::size_t tokens, std::size_t d) {
        return static_cast<float*>(buf("row_max", ((d + 127) / 128) * tokens * sizeof(float)));
    };

    DeviceTensor result;
    bool haveResult = false;
    const std::size_t w = static_cast<std::size_t>(tpWorld);

    // Tensor parallelism, prompt pass: sequences are independent, so an attention or feed-forward layer runs over
    // one group of sequences after the other, and the all-reduce that completes a group's rows of x runs on a second
    // stream while the next group (then the next layer of the first group) computes. All groups share the scratch
    // buffers (the compute stream is in order); only their rows of x differ.
    std::size_t groups = 1;
    std::vector<char> inFlight;   // group g's rows of x are being reduced on the second stream
    auto planGroups = [&](std::size_t batch) {
        std::size_t want = (tpWorld > 1 && !incremental) ? static_cast<std::size_t>(tpChunks) : 1;
        while (want > 1 && (batch % want != 0)) --want;
        if (want != groups) {
            require(std::find(inFlight.begin(), inFlight.end(), 1) == inFlight.end(), "Model: group count changed mid-flight");
            groups = want;
        }
        if (groups > 1) ensureOverlapStreams(groups);
        inFlight.resize(groups, 0);
    };
    auto awaitGroup = [&](std::size_t g) {
        if (g < inFlight.size() && inFlight[g]) {
            BFB_CUDA(cudaStreamWaitEvent(stream, reduced[g], 0));
            inFlight[g] = 0;
        }
    };
    auto awaitAllGroups = [&]() {
        for (std::size_t g = 0; g < inFlight.size(); ++g) awaitGroup(g);
    };
    // the sum over ranks of `count` values at `rows`, which group g's GEMM has just written on `stream`
    auto reduceGroup = [&](std::size_t g, void* rows, std::size_t count) {
        if (tpWorld == 1) return;
        if (groups == 1) {
            tpAllReduceSum(rows, static_cast<int64_t>(count), S, stream);
            return;
        }
        BFB_CUDA(cudaEventRecord(computed[g], stream));
        BFB_CUDA(cudaStreamWaitEvent(commStream, computed[g], 0));
        tpAllReduceSum(rows, static_cast<int64_t>(count), S, commStream);
        BFB_CUDA(cudaEventRecord(reduced[g], commStream));
        inFlight[g] = 1;
    };
    // while a collective may hold some SMs, the GEMMs draw their tiles dynamically (and may leave SMs free)
    struct SharedSmGuard {
        int reservedBefore;
        bool dynamicBefore;
        SharedSmGuard(bool on, int reserve) : reservedBefore(bfb::reservedSms()), dynamicBefore(bfb::dynamicTiles()) {
            if (on) {
                bfb::setReservedSms(reserve);
                bfb::setDynamicTiles(true);
            }
        }
        ~SharedSmGuard() {
            bfb::setReservedSms(reservedBefore);
            bfb::setDynamicTiles(dynamicBefore);
        }
    };
    SharedSmGuard sharedSms(tpWorld > 1 && !incremental && tpChunks > 1, tpReserveSms);

    for (std::size_t i = 0; i < layers.size(); ++i) {
        Layer& l = layers[i];
        const std::size_t allTokens = tokensOf();
        std::size_t tokens = allTokens;
        if (marks != nullptr) marks->mark(i, stream);
        switch (l.kind) {
            case BFB_OP_EMBEDDING: {
                require(i == 0, "Model: embedding must be the first operation of the planned route");
                if (input.rank() != 2) throw std::invalid_argument("embeddingLookup: token ids must be [batch, seq]");
                const std::size_t batch = shape[0], seq = shape[1];
                const float* pos = nullptr;
                std::size_t maxSeq = 0;
                bool fused = i + 1 < layers.size() && layers[i + 1].kind == BFB_OP_POSITIONAL_EMBEDDING;
                if (fused) {
                    maxSeq = layers[i + 1].maxSeq;
                    if (oldLen + seq > maxSeq) {
                        throw std::invalid_argument("addPositionalEmbedding: sequence (" + std::to_string(oldLen + seq) +
                                                    ") exceeds maxSeqLen (" + std::to_string(maxSeq) + ")");
                    }
                    cacheHint = maxSeq;
                    pos = params[layers[i + 1].p[0]].value.data();
                }
                x = buf("x", batch * seq * l.outFeat * sb);
                bfb::embedPos(input.data(), params[l.p[0]].value.data(), pos, x, S, static_cast<int64_t>(batch),
                              static_cast<int64_t>(seq), static_cast<int64_t>(l.vocab), static_cast<int64_t>(l.outFeat),
                              static_cast<int64_t>(maxSeq), static_cast<int64_t>(oldLen), trusted ? nullptr : dOob, stream);
                idsChecked = !trusted;
                vocabForCheck = l.vocab;
                shape = {batch, seq, l.outFeat};
                feat = l.outFeat;
                if (fused) ++i;
                break;
            }
            case BFB_OP_ATTENTION: {
                require(x != nullptr, "Model: the planned route must start with an embedding");
                if (shape.size() != 3) throw std::invalid_argument("selfAttention: input [batch, seq, dim] required");
                const std::size_t seq = shape[1], d = feat, dl = d / w, hl = l.heads / w;
                const std::size_t hd = d / l.heads;
                planGroups(shape[0]);
                const std::size_t batch = shape[0] / groups;
                tokens = batch * seq;
                void* const xAll = x;
                for (std::size_t g = 0; g < groups; ++g) {
                x = static_cast<char*>(xAll) + g * tokens * d * sb;
                awaitGroup(g);
                if (groups > 1) ssParts = 0;
                const float* sc = static_cast<const float*>(l.scales.ptr);
                const float* dAlpha = nullptr;
                void* qkv = buf("qkv", tokens * 3 * dl * 2);
                const bool fuse = fusedNormOk(tokens, 3 * dl, d, l.w0.ptr);
                if (fuse) {
                    const float* sums = needSumSq(tokens, d);
                    runGemm(x, l.w0.ptr, qkv, tokens, 3 * dl, d, BFB_BF16, BFB_EPI_NONE, nullptr, nullptr, nullptr, 0, sums,
                            ssParts, nullptr);
                } else if (fp8 && S == BFB_BF16) {
                    const void* aQkv = normedFp8Input(tokens, d, sc, &dAlpha);
                    runGemm(aQkv, l.w0.ptr, qkv, tokens, 3 * dl, d, BFB_BF16, BFB_EPI_NONE, nullptr, nullptr, dAlpha, 0);
                } else {
                    void* normed = buf("normed", tokens * d * 2);
                    bfb::rmsnorm(x, S, normed, BFB_BF16, static_cast<int64_t>(tokens), static_cast<int64_t>(d), 1e-6f, stream);
                    const void* aQkv = gemmInput(normed, tokens * d, "act8_d", sc, &dAlpha);
                    runGemm(aQkv, l.w0.ptr, qkv, tokens, 3 * dl, d, BFB_BF16, BFB_EPI_NONE, nullptr, nullptr, dAlpha, 0);
                }
                void* ctx = buf("ctx", tokens * dl * 2);
                bfb::AttentionArgs a;
                a.q = qkv;
                a.out = ctx;
                a.dtype = BFB_BF16;
                a.batch = static_cast<int64_t>(batch);
                a.newLen = static_cast<int64_t>(seq);
                a.numHeads = static_cast<int64_t>(hl);
                a.headDim = static_cast<int64_t>(hd);
                a.ldQ = static_cast<int64_t>(3 * dl);
                a.ldO = static_cast<int64_t>(dl);
                a.scale = 1.0f / std::sqrt(static_cast<float>(hd));
                if (incremental) {
                    // the new keys and values join the layer's cache; attention reads the cache
                    ensureCache(l, batch, dl, oldLen + seq, cacheHint, stream);
                    bfb::appendKv(qkv, BFB_BF16, static_cast<int64_t>(3 * dl), static_cast<int64_t>(dl),
                                  static_cast<int64_t>(2 * dl), l.kCache.ptr, l.vCache.ptr, static_cast<int64_t>(batch),
                                  static_cast<int64_t>(seq), static_cast<int64_t>(dl), static_cast<int64_t>(l.cacheRows),
                                  static_cast<int64_t>(oldLen), stream);
                    a.k = l.kCache.ptr;
                    a.v = l.vCache.ptr;
                    a.ldK = a.ldV = static_cast<int64_t>(dl);
                    a.kvBatchRows = static_cast<int64_t>(l.cacheRows);
                    a.totalLen = static_cast<int64_t>(oldLen + seq);
                } else {
                    a.k = static_cast<char*>(qkv) + dl * 2;
                    a.v = static_cast<char*>(qkv) + 2 * dl * 2;
                    a.ldK = a.ldV = static_cast<int64_t>(3 * dl);
                    a.totalLen = static_cast<int64_t>(seq);
                }
                a.oldLen = static_cast<int64_t>(oldLen);
                a.causal = 1;
                a.dStatus = dStatus;
                // e4m3 route: the attention epilogue also reports the largest magnitudes of what it stores, so the
                // quantisation of its output needs no pass of its own to find the scale
                int64_t ctxMaximaCount = 0;
                if (fp8 && !incremental && bfb::attentionUsesTensorCores(a)) {
                    ctxMaximaCount = bfb::attentionMaximaCount(a);
                    a.outMaxima = static_cast<float*>(buf("ctx_maxima", static_cast<std::size_t>(ctxMaximaCount) * sizeof(float)));
                }
                bfb::attentionForward(a, stream);
                const void* aOut = nullptr;
                if (a.outMaxima != nullptr) {
                    float* st = nextFp8Stats();
                    void* a8 = buf("act8_dl", tokens * dl);
                    float* scratch = static_cast<float*>(
                        buf("partial_ctx_maxima", static_cast<std::size_t>(bfb::quantizeScratchFloats(ctxMaximaCount)) * sizeof(float)));
                    bfb::quantizeE4m3FromMaxima(ctx, BFB_BF16, static_cast<int64_t>(tokens * dl), a8, st, sc + 3, a.outMaxima,
                                                ctxMaximaCount, scratch, stream);
                    dAlpha = st + 2;
                    aOut = a8;
                } else {
                    aOut = gemmInput(ctx, tokens * dl, "act8_dl", sc + 2, &dAlpha);
                }
                // x = x + ctx * Wout (in place); under tensor parallelism rank 0 carries the residual
                const int epi = (tpWorld == 1 || tpRank == 0) ? BFB_EPI_RESIDUAL : BFB_EPI_NONE;
                float* produced = fuse && fusedNormOk(tokens, d, dl, l.w1.ptr) ? nextSumSq(tokens, d) : nullptr;
                float* producedMax = nullptr;
                if (fp8StatsOk(aOut, tokens, d, dl, l.w1.ptr)) {
                    produced = nextSumSq(tokens, d);
                    producedMax = maxBuffer(tokens, d);
                }
                runGemm(aOut, l.w1.ptr, x, tokens, d, dl, S, epi, nullptr, x, dAlpha, 0, nullptr, 1, produced, producedMax);
                producedSumSq(produced, d, producedMax);
                reduceGroup(g, x, tokens * d);
                }
                x = xAll;
                break;
            }
            case BFB_OP_FEEDFORWARD: {
                require(x != nullptr, "Model: the planned route must start with an embedding");
                const std::size_t d = feat, fl = l.hidden / w;
                planGroups(shape.size() == 3 ? shape[0] : 1);
                tokens = allTokens / groups;
                void* const xAll = x;
                for (std::size_t g = 0; g < groups; ++g) {
                x = static_cast<char*>(xAll) + g * tokens * d * sb;
                awaitGroup(g);
                if (groups > 1) ssParts = 0;
                const float* sc = static_cast<const float*>(l.scales.ptr);
                const float* dAlpha = nullptr;
                void* hidden = buf("hidden", tokens * fl * 2);
                float* hiddenMaxima = nullptr;
                const bool fuse = fusedNormOk(tokens, fl, d, l.w0.ptr);
                if (fuse) {
                    const float* sums = needSumSq(tokens, d);
                    runGemm(x, l.w0.ptr, hidden, tokens, fl, d, BFB_BF16, BFB_EPI_BIAS_SILU, params[l.p[1]].value.data(),
                            nullptr, nullptr, 0, sums, ssParts, nullptr);
                } else if (fp8 && S == BFB_BF16) {
                    const void* a1 = normedFp8Input(tokens, d, sc, &dAlpha);
                    // the epilogue that writes `hidden` also reports its largest magnitudes (one per row and 128
                    // columns): the quantisation below then needs no pass over `hidden` to find its scale
                    bfb::GemmArgs probe;
                    probe.a = a1;
                    probe.b = l.w0.ptr;
                    probe.c = hidden;
                    probe.m = static_cast<int64_t>(tokens);
                    probe.n = static_cast<int64_t>(fl);
                    probe.k = static_cast<int64_t>(d);
                    probe.abDtype = ab;
                    probe.bLayout = BFB_B_NK;
                    probe.cDtype = BFB_BF16;
                    if (!incremental && bfb::gemmSupportsRowStats(probe)) {
                        hiddenMaxima = static_cast<float*>(buf("hidden_maxima", ((fl + 127) / 128) * tokens * sizeof(float)));
                    }
                    runGemm(a1, l.w0.ptr, hidden, tokens, fl, d, BFB_BF16, BFB_EPI_BIAS_SILU, params[l.p[1]].value.data(),
                            nullptr, dAlpha, 0, nullptr, 1, nullptr, hiddenMaxima);
                } else {
                    void* normed = buf("normed", tokens * d * 2);
                    bfb::rmsnorm(x, S, normed, BFB_BF16, static_cast<int64_t>(tokens), static_cast<int64_t>(d), 1e-6f, stream);
                    const void* a1 = gemmInput(normed, tokens * d, "act8_d", sc, &dAlpha);
                    runGemm(a1, l.w0.ptr, hidden, tokens, fl, d, BFB_BF16, BFB_EPI_BIAS_SILU, params[l.p[1]].value.data(),
                            nullptr, dAlpha, 0);
                }
                const void* a2 = nullptr;
                if (hiddenMaxima != nullptr) {
                    float* st = nextFp8Stats();
                    void* a8 = buf("act8_f", tokens * fl);
                    const int64_t count = static_cast<int64_t>(((fl + 127) / 128) * tokens);
                    float* scratch = static_cast<float*>(
                        buf("partial_maxima", static_cast<std::size_t>(bfb::quantizeScratchFloats(count)) * sizeof(float)));
                    bfb::quantizeE4m3FromMaxima(hidden, BFB_BF16, static_cast<int64_t>(tokens * fl), a8, st, sc + 3, hiddenMaxima,
                                                count, scratch, stream);
                    dAlpha = st + 2;
                    a2 = a8;
                } else {
                    a2 = gemmInput(hidden, tokens * fl, "act8_f", sc + 2, &dAlpha);
                }
                const bool lead = tpWorld == 1 || tpRank == 0;
                float* produced = fuse && fusedNormOk(tokens, d, fl, l.w1.ptr) ? nextSumSq(tokens, d) : nullptr;
                float* producedMax = nullptr;
                if (fp8StatsOk(a2, tokens, d, fl, l.w1.ptr)) {
                    produced = nextSumSq(tokens, d);
                    producedMax = maxBuffer(tokens, d);
                }
                runGemm(a2, l.w1.ptr, x, tokens, d, fl, S, lead ? BFB_EPI_BIAS_RESIDUAL : BFB_EPI_NONE,
                        lead ? params[l.p[3]].value.data() : nullptr, lead ? x : nullptr, dAlpha, 0, nullptr, 1, produced,
                        producedMax);
                producedSumSq(produced, d, producedMax);
                reduceGroup(g, x, tokens * d);
                }
                x = xAll;
                break;
            }
            case BFB_OP_LINEAR: {
                require(x != nullptr, "Model: the planned route must start with an embedding");
                awaitAllGroups();
                const std::size_t d = feat, outL = l.shardedLinear ? l.outFeat / w : l.outFeat;
                const void* a16 = x;
                if (S == BFB_F32) {
                    void* t = buf("lin16", tokens * d * 2);
                    bfb::castScaled(x, BFB_F32, t, BFB_BF16, static_cast<int64_t>(tokens * d), 1.0f, nullptr, stream);
                    a16 = t;
                }
                const float* sc = static_cast<const float*>(l.scales.ptr);
                const float* dAlpha = nullptr;
                const void* a = gemmInput(a16, tokens * d, "act8_d", sc, &dAlpha);
                std::vector<std::size_t> outShape = shape;
                outShape.back() = outL;
                const bool last = i + 1 == layers.size();
                if (last && out16 != nullptr) {
                    // the caller takes the bf16 values themselves: same rounding as below, half the bytes
                    runGemm(a, l.w0.ptr, out16, tokens, outL, d, BFB_BF16, BFB_EPI_BIAS, params[l.p[1]].value.data(),
                            nullptr, dAlpha, 0);
                    haveResult = true;
                } else if (last) {
                    result = DeviceTensor(outShape);
                    runGemm(a, l.w0.ptr, result.data(), tokens, outL, d, BFB_F32, BFB_EPI_BIAS,
                            params[l.p[1]].value.data(), nullptr, dAlpha, storageBf16 ? 1 : 0);
                    haveResult = true;
                } else {
                    void* nx = buf("x_alt", tokens * outL * sb);
                    runGemm(a, l.w0.ptr, nx, tokens, outL, d, S, BFB_EPI_BIAS, params[l.p[1]].value.data(), nullptr,
                            dAlpha, 0);
                    std::swap(arena["x"], arena["x_alt"]);
                    x = arena["x"].ptr;
                    ssParts = 0;
                }
                shape = outShape;
                feat = outL;
                break;
            }
            default: {
                // elementwise / norm / softmax / standalone positions: run on an fp32 copy
                require(x != nullptr, "Model: the planned route must start with an embedding");
                awaitAllGroups();
                const std::size_t count = tokens * feat;
                DeviceTensor tmp(shape);
                bfb::castScaled(x, S, tmp.data(), BFB_F32, static_cast<int64_t>(count), 1.0f, nullptr, stream);
                BFB_CUDA(cudaStreamSynchronize(stream));  // the fp32 operator API runs on the default stream
                DeviceTensor out;
                switch (l.kind) {
                    case BFB_OP_SILU: out = silu(tmp); break;
                    case BFB_OP_RELU: out = relu(tmp); break;
                    case BFB_OP_GELU: out = gelu(tmp); break;
                    case BFB_OP_RMSNORM: out = rmsnorm(tmp); break;
                    case BFB_OP_SOFTMAX: out = softmax(tmp); break;
                    case BFB_OP_POSITIONAL_EMBEDDING:
                        // positions continue after the cached ones (the reference's forwardIncremental uses
                        // addPositionalEmbeddingAt with its generation position); the call checks the table's length
                        out = addPositionalEmbeddingAt(tmp, params[l.p[0]].value, oldLen);
                        cacheHint = params[l.p[0]].value.dim(0);
                        break;
                    default: fail(BFB_UNSUPPORTED, "Model: operation not available on the device");
                }
                BFB_CUDA(cudaStreamSynchronize(nullptr));
                bfb::castScaled(out.data(), BFB_F32, x, S, static_cast<int64_t>(count), 1.0f, nullptr, stream);
                ssParts = 0;
                break;
            }
        }
    }
    awaitAllGroups();
    if (!haveResult) {
        require(x != nullptr, "Model: empty pipeline");
        result = DeviceTensor(shape);
        bfb::castScaled(x, S, result.data(), BFB_F32, static_cast<int64_t>(tokensOf() * feat), 1.0f, nullptr, stream);
    }
    if (marks != nullptr) marks->mark(layers.size(), stream);
    checkStatus(stream, idsChecked, vocabForCheck);
    if (incremental) genPosition += shape.size() >= 2 ? shape[1] : 0;
    return result;
}

// ---- Model ------------------------------------------------------------------------------------------------

Model::Model(const std::vector<OpDesc>& ops, std::int64_t inputLastDim, unsigned int seed,
             std::optional<PrecisionPolicy> precision, bool randomInit, std::string name)
    : impl_(std::make_unique<Impl>()), name_(std::move(name)) {
    if (ops.empty()) throw std::invalid_argument("Model: the model '" + name_ + "' has no pipeline");
    impl_->ops = ops;
    impl_->inputLastDim = inputLastDim;
    impl_->seed = seed;
    impl_->precision = precision;
    impl_->randomInit = randomInit;
    if (precision.has_value()) {
        if (precision->compute == BFB_DT_BF16) impl_->mode = Mode::Bf16;
        else if (precision->compute == BFB_DT_FP8_E4M3) impl_->mode = Mode::Fp8;
        impl_->storageBf16 = precision->storage == BFB_DT_BF16;
    }
    impl_->streamDtype = (impl_->mode != Mode::Fp32 && impl_->storageBf16) ? BFB_BF16 : BFB_F32;
    impl_->buildStructure();
}

Model::~Model() = default;

void Model::setTensorParallelOverlap(int groups, int reservedSms) {
    if (groups < 1 || reservedSms < 0) throw std::invalid_argument("Model: bad tensor-parallel overlap setting");
    impl_->tpChunks = groups;
    impl_->tpReserveSms = reservedSms;
}

void Model::setTensorParallel(int rank, int world) {
    if (world < 1 || rank < 0 || rank >= world) throw std::invalid_argument("Model: bad tensor-parallel rank/size");
    if (impl_->built) throw std::invalid_argument("Model: tensor parallelism must be set before parameters exist");
    impl_->tpRank = rank;
    impl_->tpWorld = world;
    impl_->params.clear();
    impl_->meta.clear();
    impl_->layers.clear();
    impl_->buildStructure();
}

DeviceTensor Model::forward(const DeviceTensor& input, bool inputRangeTrusted, void* stream) {
    impl_->allocateParams();
    // the planned route needs the pipeline to open with an embedding; everything else is interpreted
    bool planned = impl_->mode != Mode::Fp32 && !impl_->layers.empty() && impl_->layers.front().kind == BFB_OP_EMBEDDING;
    if (!planned) {
        if (impl_->mode != Mode::Fp32) {
            fail(BFB_UNSUPPORTED, "Model: compute bf16 / fp8.e4m3 needs a pipeline that starts with an embedding");
        }
        if (stream != nullptr) BFB_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
        return impl_->forwardFp32(input, inputRangeTrusted, false);
    }
    return impl_->forwardPlanned(input, inputRangeTrusted, static_cast<cudaStream_t>(stream), nullptr, false);
}

DeviceTensor Model::forwardIncremental(const DeviceTensor& newTokenIds, bool inputRangeTrusted, void* stream) {
    impl_->allocateParams();
    if (newTokenIds.rank() < 2) throw std::invalid_argument("forwardIncremental: input [batch, newLen, ...] required");
    if (impl_->genPosition > 0 && newTokenIds.dim(0) != impl_->genBatch) {
        throw std::invalid_argument("forwardIncremental: the batch size changed since the caches were opened (" +
                                    std::to_string(impl_->genBatch) + " -> " + std::to_string(newTokenIds.dim(0)) + ")");
    }
    if (impl_->genPosition == 0) impl_->genBatch = newTokenIds.dim(0);
    bool planned = impl_->mode != Mode::Fp32 && !impl_->layers.empty() && impl_->layers.front().kind == BFB_OP_EMBEDDING;
    if (!planned) {
        if (impl_->mode != Mode::Fp32) {
            fail(BFB_UNSUPPORTED, "Model: compute bf16 / fp8.e4m3 needs a pipeline that starts with an embedding");
        }
        if (stream != nullptr) BFB_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
        return impl_->forwardFp32(newTokenIds, inputRangeTrusted, true);
    }
    return impl_->forwardPlanned(newTokenIds, inputRangeTrusted, static_cast<cudaStream_t>(stream), nullptr, true);
}

namespace {
const char* opKindName(int kind) {   // src/ir/operation.cpp:36-50
    switch (kind) {
        case BFB_OP_LINEAR: return "linear";
        case BFB_OP_SILU: return "silu";
        case BFB_OP_RELU: return "relu";
        case BFB_OP_GELU: return "gelu";
        case BFB_OP_RMSNORM: return "rmsnorm";
        case BFB_OP_SOFTMAX: return "softmax";
        case BFB_OP_EMBEDDING: return "embedding";
        case BFB_OP_POSITIONAL_EMBEDDING: return "positional_embedding";
        case BFB_OP_ATTENTION: return "attention";
        case BFB_OP_FEEDFORWARD: return "feedforward";
        case BFB_OP_BIDIRECTIONAL_ATTENTION: return "bidirectional_attention";
        default: return "?";
    }
}
}  // namespace

BenchmarkResult Model::benchmark(const DeviceTensor& input, std::size_t warmupIterations, std::size_t measuredIterations,
                                 void* stream) {
    if (impl_->layers.empty()) throw std::invalid_argument("runBenchmark: the model '" + name_ + "' has no pipeline to run");
    if (measuredIterations == 0) throw std::invalid_argument("runBenchmark: measuredIterations must be positive");
    BenchmarkResult r;
    r.inputShape = input.shape();
    r.warmupIterations = warmupIterations;
    r.measuredIterations = measuredIterations;
    for (std::size_t i = 0; i < warmupIterations; ++i) (void)forward(input, false, stream);

    const std::size_t nOps = impl_->layers.size();
    std::vector<double> perOp(nOps, 0.0);
    double total = 0.0;
    Impl::OpMarks marks;
    struct Unset {
        Impl* impl;
        ~Unset() { impl->marks = nullptr; }
    } unset{impl_.get()};
    for (std::size_t it = 0; it < measuredIterations; ++it) {
        marks.used = 0;
        impl_->marks = &marks;
        DeviceTensor out = forward(input, false, stream);
        impl_->marks = nullptr;
        BFB_CUDA(cudaEventSynchronize(marks.events[marks.used - 1]));
        for (std::size_t m = 0; m + 1 < marks.used; ++m) {
            float ms = 0.0f;
            BFB_CUDA(cudaEventElapsedTime(&ms, marks.events[m], marks.events[m + 1]));
            if (marks.opIndex[m] < nOps) perOp[marks.opIndex[m]] += static_cast<double>(ms);
            total += static_cast<double>(ms);
        }
    }
    const double n = static_cast<double>(measuredIterations);
    r.meanMilliseconds = total / n;
    const double batch = input.rank() >= 1 ? static_cast<double>(input.dim(0)) : 1.0;
    r.throughputSamplesPerSecond = r.meanMilliseconds > 0.0 ? batch * 1000.0 / r.meanMilliseconds : 0.0;
    for (std::size_t i = 0; i < nOps; ++i) {
        r.perOperation.push_back(OperationBenchmark{opKindName(impl_->layers[i].kind), i, perOp[i] / n});
    }
    // the reference's estimate (elements x 4 bytes of the input, every operation's output and the parameters;
    // src/backend/cpu/benchmark.cpp:117-137), with every parameter counted, not only those of `linear`
    std::size_t elements = input.elementCount();
    std::vector<std::size_t> shape = input.shape();
    for (const Layer& l : impl_->layers) {
        if (l.kind == BFB_OP_EMBEDDING) shape.push_back(l.outFeat);
        else if (l.kind == BFB_OP_LINEAR && !shape.empty()) shape.back() = l.outFeat;
        std::size_t count = 1;
        for (std::size_t d : shape) count *= d;
        elements += count;
    }
    for (const Parameter& p : impl_->params) {
        std::size_t count = 1;
        for (std::size_t d : p.fullShape) count *= d;
        elements += count;
    }
    r.estimatedMemoryBytes = elements * sizeof(float);
    return r;
}

void Model::resetGenerationState() { impl_->resetGeneration(); }
std::size_t Model::generationPosition() const { return impl_->genPosition; }

bool Model::resultIsBf16Exact() const {
    const bool planned = impl_->mode != Mode::Fp32 && !impl_->layers.empty() && impl_->layers.front().kind == BFB_OP_EMBEDDING;
    return planned && impl_->storageBf16 && impl_->layers.back().kind == BFB_OP_LINEAR;
}

void Model::forwardBf16(const DeviceTensor& input, void* deviceOut16, bool inputRangeTrusted, void* stream) {
    require(deviceOut16 != nullptr, "Model::forwardBf16: null output");
    require(resultIsBf16Exact(), "Model::forwardBf16: needs storage bf16 and a pipeline from an embedding to a linear");
    impl_->allocateParams();
    impl_->forwardPlanned(input, inputRangeTrusted, static_cast<cudaStream_t>(stream), deviceOut16, false);
}

std::vector<Parameter*> Model::parameters() {
    impl_->allocateParams();
    std::vector<Parameter*> out;
    for (Parameter& p : impl_->params) out.push_back(&p);
    return out;
}

std::vector<std::size_t> Model::outputShape(const std::vector<std::size_t>& inputShape) const {
    std::vector<std::size_t> shape = inputShape;
    for (const Layer& l : impl_->layers) {
        if (l.kind == BFB_OP_EMBEDDING) shape.push_back(l.outFeat);
        else if (l.kind == BFB_OP_LINEAR && !shape.empty()) {
            shape.back() = l.shardedLinear ? l.outFeat / static_cast<std::size_t>(impl_->tpWorld) : l.outFeat;
        }
    }
    return shape;
}

std::size_t Model::parameterCount() const { return impl_->params.size(); }
const std::string& Model::parameterName(std::size_t index) const { return impl_->params.at(index).name; }
const std::vector<std::size_t>& Model::parameterShape(std::size_t index) const {
    return impl_->params.at(index).fullShape;
}

void Model::fillParameterNormal(std::size_t index, std::uint64_t seed, float sigma) {
    impl_->allocateParams();
    require(index < impl_->params.size(), "Model: parameter index out of range");
    Parameter& prm = impl_->params[index];
    const Shard s = impl_->tpWorld > 1 ? impl_->meta[index].shard : Shard::None;
    const std::size_t r = static_cast<std::size_t>(impl_->tpRank);
    const std::size_t rows = prm.value.rank() == 2 ? prm.value.dim(0) : 1;
    const std::size_t colsLocal = prm.value.rank() == 2 ? prm.value.dim(1) : prm.value.dim(0);
    const std::size_t colsFull = prm.fullShape.size() == 2 ? prm.fullShape[1] : prm.fullShape[0];
    std::size_t rowOff = 0, colOff = 0;
    if (s == Shard::Rows) rowOff = r * rows;
    if (s == Shard::Cols || s == Shard::Vec) colOff = r * colsLocal;
    bfb::fillNormal(prm.value.data(), static_cast<int64_t>(rows), static_cast<int64_t>(colsLocal),
                    static_cast<int64_t>(colsFull), static_cast<int64_t>(rowOff), static_cast<int64_t>(colOff), seed,
                    sigma, nullptr);
    if (!impl_->mastersReleased) impl_->prepared = false;
}

void Model::releaseMasterWeights() {
    impl_->prepare(nullptr);
    BFB_CUDA(cudaStreamSynchronize(nullptr));
    if (impl_->mode == Mode::Fp32) return;  // the fp32 route computes from the masters
    for (Layer& l : impl_->layers) {
        if (l.kind != BFB_OP_ATTENTION && l.kind != BFB_OP_FEEDFORWARD && l.kind != BFB_OP_LINEAR) continue;
        const int weightSlots[3][4] = {{0, 1, 2, 3}, {0, 2, -1, -1}, {0, -1, -1, -1}};
        const int* slots = l.kind == BFB_OP_ATTENTION ? weightSlots[0] : l.kind == BFB_OP_FEEDFORWARD ? weightSlots[1] : weightSlots[2];
        for (int i = 0; i < 4; ++i) {
            if (slots[i] < 0) continue;
            impl_->params[l.p[slots[i]]].value = DeviceTensor();  // biases and tables stay
        }
    }
    impl_->mastersReleased = true;
    bfb::poolTrim();
}

bool Model::parameterIsGemmWeight(std::size_t index) const {
    require(index < impl_->params.size(), "Model: parameter index out of range");
    return impl_->mode != Mode::Fp32 && impl_->gemmWeightMask()[index] != 0;
}

std::string Model::preparedWeightsTag() const {
    if (impl_->mode == Mode::Fp32) return "";
    return std::string(impl_->mode == Mode::Bf16 ? "bf16" : "e4m3") + ".tp" + std::to_string(impl_->tpRank) + "of" +
           std::to_string(impl_->tpWorld);
}

// FNV-1a over the compute format, the tensor-parallel split and every parameter's name and full shape
std::uint64_t Model::structureFingerprint() const {
    std::uint64_t h = 1469598103934665603ull;
    auto mix = [&](const void* data, std::size_t bytes) {
        const unsigned char* p = static_cast<const unsigned char*>(data);
        for (std::size_t i = 0; i < bytes; ++i) {
            h ^= p[i];
            h *= 1099511628211ull;
        }
    };
    const std::string tag = preparedWeightsTag();
    mix(tag.data(), tag.size());
    for (const Parameter& p : impl_->params) {
        mix(p.name.data(), p.name.size());
        for (std::size_t d : p.fullShape) {
            const std::uint64_t v = d;
            mix(&v, sizeof(v));
        }
    }
    return h;
}

// The converted weights of the planned route, layer by layer: w0, w1 (when the layer has one) and the four scale
// floats. allocate == false: after a conversion, for saving. allocate == true: buffers of the right sizes are created
// to be filled from a file; adoptPreparedWeights() then makes them the model's weights.
std::vector<Model::PreparedPiece> Model::preparedWeightPieces(bool allocate) {
    std::vector<PreparedPiece> pieces;
    if (impl_->mode == Mode::Fp32) return pieces;
    if (!allocate) {
        impl_->prepare(nullptr);
        BFB_CUDA(cudaStreamSynchronize(nullptr));
    }
    const std::size_t eb = impl_->mode == Mode::Bf16 ? 2 : 1;
    auto elems = [&](int paramIndex) {
        std::size_t n = 1;
        for (std::size_t d : impl_->localShape(impl_->params[paramIndex].fullShape, impl_->meta[paramIndex].shard)) n *= d;
        return n;
    };
    for (Layer& l : impl_->layers) {
        if (l.kind != BFB_OP_ATTENTION && l.kind != BFB_OP_FEEDFORWARD && l.kind != BFB_OP_LINEAR) continue;
        std::size_t b0 = 0, b1 = 0;
        if (l.kind == BFB_OP_ATTENTION) {
            b0 = (elems(l.p[0]) + elems(l.p[1]) + elems(l.p[2])) * eb;
            b1 = elems(l.p[3]) * eb;
        } else if (l.kind == BFB_OP_FEEDFORWARD) {
            b0 = elems(l.p[0]) * eb;
            b1 = elems(l.p[2]) * eb;
        } else {
            b0 = elems(l.p[0]) * eb;
        }
        if (allocate) {
            l.w0.ensure(b0);
            if (b1 > 0) l.w1.ensure(b1);
            l.scales.ensure(4 * sizeof(float));
        }
        pieces.push_back({l.w0.ptr, b0});
        if (b1 > 0) pieces.push_back({l.w1.ptr, b1});
        pieces.push_back({l.scales.ptr, 4 * sizeof(float)});
    }
    return pieces;
}

void Model::adoptPreparedWeights() {
    if (impl_->mode == Mode::Fp32) return;
    if (impl_->built) {   // fp32 copies exist already: drop those of the GEMM weights
        const std::vector<char> mask = impl_->gemmWeightMask();
        for (std::size_t i = 0; i < impl_->params.size(); ++i) {
            if (mask[i]) impl_->params[i].value = DeviceTensor();
        }
        bfb::poolTrim();
    }
    impl_->mastersReleased = true;
    impl_->prepared = true;
}

// A parameter as rows of the full (unsharded) tensor: [rows, cols] for rank 2, one element per row for vectors (so
// that a vector's slice is a row range), one row otherwise.
Model::RowView Model::parameterRowView(std::size_t index) const {
    require(index < impl_->params.size(), "Model: parameter index out of range");
    const std::vector<std::size_t>& full = impl_->params[index].fullShape;
    RowView v;
    if (full.size() == 2) {
        v.rows = full[0];
        v.rowElems = full[1];
    } else if (full.size() == 1) {
        v.rows = full[0];
        v.rowElems = 1;
    } else {
        v.rows = 1;
        v.rowElems = 1;
        for (std::size_t d : full) v.rowElems *= d;
    }
    v.firstNeededRow = 0;
    v.neededRows = v.rows;
    const Shard s = impl_->tpWorld > 1 ? impl_->meta[index].shard : Shard::None;
    if (s == Shard::Rows || s == Shard::Vec) {
        v.neededRows = v.rows / static_cast<std::size_t>(impl_->tpWorld);
        v.firstNeededRow = static_cast<std::size_t>(impl_->tpRank) * v.neededRows;
    }
    return v;
}

std::size_t Model::uploadParameterRows(std::size_t index, std::size_t firstRow, std::size_t rowCount,
                                       const float* hostRows, void* stream) {
    impl_->allocateParams();
    require(index < impl_->params.size(), "Model: parameter index out of range");
    require(hostRows != nullptr, "Model: null parameter data");
    Parameter& prm = impl_->params[index];
    if (impl_->mastersReleased && prm.value.data() == nullptr) {
        fail(BFB_UNSUPPORTED, "Model: the fp32 copy of '" + prm.name + "' was released; it can no longer be set");
    }
    const RowView v = parameterRowView(index);
    if (firstRow < v.firstNeededRow || firstRow + rowCount > v.firstNeededRow + v.neededRows) {
        fail(BFB_INVALID_ARGUMENT, "Model: rows outside this rank's part of '" + prm.name + "'");
    }
    const Shard s = impl_->tpWorld > 1 ? impl_->meta[index].shard : Shard::None;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    std::size_t bytes = 0;
    if (s == Shard::Cols) {   // this rank's columns out of full rows
        const std::size_t nLoc = v.rowElems / static_cast<std::size_t>(impl_->tpWorld);
        bytes = rowCount * nLoc * sizeof(float);
        BFB_CUDA(cudaMemcpy2DAsync(prm.value.data() + firstRow * nLoc, nLoc * sizeof(float),
                                   hostRows + static_cast<std::size_t>(impl_->tpRank) * nLoc, v.rowElems * sizeof(float),
                                   nLoc * sizeof(float), rowCount, cudaMemcpyHostToDevice, st));
    } else {
        bytes = rowCount * v.rowElems * sizeof(float);
        BFB_CUDA(cudaMemcpyAsync(prm.value.data() + (firstRow - v.firstNeededRow) * v.rowElems, hostRows, bytes,
                                 cudaMemcpyHostToDevice, st));
    }
    if (!impl_->mastersReleased) impl_->prepared = false;
    return bytes;
}

void Model::setParameter(std::size_t index, const float* hostFullValues) { impl_->setParam(index, hostFullValues); }
void Model::getParameter(std::size_t index, float* hostFullValues) { impl_->getParam(index, hostFullValues); }
void Model::invalidatePreparedWeights() {
    if (!impl_->mastersReleased) impl_->prepared = false;   // without fp32 copies there is nothing to convert again
}

std::optional<std::size_t> Model::firstLayerEmbeddingVocabSize() const {
    if (impl_->layers.empty() || impl_->layers.front().kind != BFB_OP_EMBEDDING) return std::nullopt;
    return impl_->layers.front().vocab;
}

// ---- Executor -----------------------------------------------------------------------------------------------

HostTensor Executor::makeSyntheticInput(const std::vector<OpDesc>& ops, const std::vector<std::int64_t>& inputShape,
                                        std::size_t batchSize) const {
    std::vector<std::size_t> shape;
    for (std::int64_t d : inputShape) shape.push_back(d < 0 ? batchSize : static_cast<std::size_t>(d));
    if (!ops.empty() && ops.front().kind == BFB_OP_EMBEDDING) {
        return randomTokenIdTensor(std::move(shape), static_cast<std::size_t>(ops.front().embedding_vocab_size),
                                   seedFor(seed_, 0, kInputSalt));
    }
    return randomTensor(std::move(shape), seedFor(seed_, 0, kInputSalt));
}

HostTensor Executor::run(const std::vector<OpDesc>& ops, std::int64_t inputLastDim, const HostTensor& input,
                         const std::optional<PrecisionPolicy>& precision) const {
    if (ops.empty()) throw std::invalid_argument("the model has no pipeline to run");
    Model model(ops, inputLastDim, seed_, precision, true, "executor");
    DeviceTensor out = model.forward(DeviceTensor::fromHost(input));
    return out.toHost();
}

}  // namespace bfb200
