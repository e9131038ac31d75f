// TEST INFRASTRUCTURE — not part of the product path.
//
// A C-ABI window onto the UNMODIFIED BlackForge CPU backend, compiled from the reference's own
// sources where they lie (see oracle/Makefile). It exists so that the parity tests, the golden
// fixture generator and the CPU baseline leg of the benchmark can call the reference's
// blackforge::backend::cpu::{ops, Model, Executor, quantize, checkpoint} and its front end
// (Lexer -> Parser -> SemanticAnalyzer -> IRBuilder) from Python through ctypes.
// Nothing here re-implements reference behaviour: every entry point forwards to a reference
// function and copies the result out.
//
// Conventions: every function returns 0 on success, 1 for std::invalid_argument, 2 for any other
// std::exception (message kept in refLastError()). Tensor results are left in a per-thread result
// slot and fetched with refResultRank/Shape/Copy.

#include <cstdint>
#include <cstring>
#include <exception>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

#include "blackforge/backend/cpu/checkpoint.hpp"
#include "blackforge/backend/cpu/executor.hpp"
#include "blackforge/backend/cpu/model.hpp"
#include "blackforge/backend/cpu/ops.hpp"
#include "blackforge/backend/cpu/quantize.hpp"
#include "blackforge/backend/cpu/random_init.hpp"
#include "blackforge/diagnostics/diagnostic.hpp"
#include "blackforge/frontend/lexer.hpp"
#include "blackforge/frontend/parser.hpp"
#include "blackforge/ir/ir_builder.hpp"
#include "blackforge/ir/module.hpp"
#include "blackforge/sema/semantic_analyzer.hpp"

namespace bf = blackforge;
namespace cpu = blackforge::backend::cpu;
using bf::runtime::Tensor;

namespace {

thread_local std::string gLastError;
thread_local Tensor gResult;

template <typename Fn>
int guarded(Fn&& fn) {
    try {
        fn();
        return 0;
    } catch (const std::invalid_argument& e) {
        gLastError = e.what();
        return 1;
    } catch (const std::exception& e) {
        gLastError = e.what();
        return 2;
    }
}

Tensor makeTensor(const float* data, const int64_t* shape, int rank) {
    std::vector<std::size_t> dims(static_cast<std::size_t>(rank));
    std::size_t count = 1;
    for (int i = 0; i < rank; ++i) {
        dims[static_cast<std::size_t>(i)] = static_cast<std::size_t>(shape[i]);
        count *= dims[static_cast<std::size_t>(i)];
    }
    return Tensor(std::move(dims), std::vector<float>(data, data + count));
}

struct Compiled {
    bf::ir::Module module;
};

bf::sema::DType dtypeFromCode(int code) {
    switch (code) {
        case 0: return bf::sema::DType::FP8_E4M3;
        case 1: return bf::sema::DType::FP8_E5M2;
        case 2: return bf::sema::DType::FP16;
        case 3: return bf::sema::DType::BF16;
        case 4: return bf::sema::DType::TF32;
        default: return bf::sema::DType::FP32;
    }
}

int dtypeToCode(bf::sema::DType d) {
    switch (d) {
        case bf::sema::DType::FP8_E4M3: return 0;
        case bf::sema::DType::FP8_E5M2: return 1;
        case bf::sema::DType::FP16: return 2;
        case bf::sema::DType::BF16: return 3;
        case bf::sema::DType::TF32: return 4;
        case bf::sema::DType::FP32: return 5;
    }
    return 5;
}

}  // namespace

extern "C" {

const char* refLastError() { return gLastError.c_str(); }

int refResultRank() { return static_cast<int>(gResult.rank()); }
void refResultShape(int64_t* out) {
    for (std::size_t i = 0; i < gResult.rank(); ++i) out[i] = static_cast<int64_t>(gResult.dim(i));
}
int64_t refResultCount() { return static_cast<int64_t>(gResult.elementCount()); }
void refResultCopy(float* out) {
    std::memcpy(out, gResult.data().data(), gResult.elementCount() * sizeof(float));
}

// ---- front end: .bf source text -> ir::Module (the reference's own compile pipeline) ----------

int refCompile(const char* source, void** outHandle) {
    return guarded([&] {
        bf::Lexer lexer(source, "<memory>");
        std::vector<bf::Token> tokens = lexer.tokenize();
        bf::Parser parser(tokens);
        bf::ast::Program program = parser.parseProgram();
        bf::sema::SemanticAnalyzer analyzer;
        analyzer.analyze(program);
        std::string errors;
        auto collect = [&](const bf::DiagnosticList& list) {
            if (list.hasErrors()) {
                for (const auto& d : list.all()) errors += bf::formatDiagnostic(d) + "\n";
            }
        };
        collect(lexer.diagnostics());
        collect(parser.diagnostics());
        collect(analyzer.diagnostics());
        if (!errors.empty()) throw std::invalid_argument(errors);
        bf::ir::IRBuilder builder;
        auto compiled = std::make_unique<Compiled>();
        compiled->module = builder.build(program);
        collect(builder.diagnostics());
        if (!errors.empty()) throw std::invalid_argument(errors);
        if (compiled->module.models.empty()) throw std::invalid_argument("no model in program");
        *outHandle = compiled.release();
    });
}

void refCompiledFree(void* handle) { delete static_cast<Compiled*>(handle); }

// The first model's IR of a compiled program, for ref_cuda_shim.cu (which builds the reference's cuda::Model from it).
const void* refCompiledModelIR(void* handle) { return &static_cast<Compiled*>(handle)->module.models.front(); }

// precision block: returns 1 if present and fills storage/compute/accumulate dtype codes.
int refCompiledPrecision(void* handle, int* storage, int* compute, int* accumulate) {
    auto* c = static_cast<Compiled*>(handle);
    if (!c->module.precision.has_value()) return 0;
    *storage = dtypeToCode(c->module.precision->storage);
    *compute = dtypeToCode(c->module.precision->compute);
    *accumulate = dtypeToCode(c->module.precision->accumulate);
    return 1;
}

int refCompiledOpCount(void* handle) {
    auto* c = static_cast<Compiled*>(handle);
    const auto& model = c->module.models.front();
    return model.pipelines.empty() ? 0 : static_cast<int>(model.pipelines.front().operations.size());
}

// fields: kind, input id, output id, linearOut, vocab, embDim, maxSeq, heads, hidden
void refCompiledOp(void* handle, int index, int64_t* fields) {
    auto* c = static_cast<Compiled*>(handle);
    const auto& op = c->module.models.front().pipelines.front().operations.at(static_cast<std::size_t>(index));
    fields[0] = static_cast<int64_t>(op.kind);
    fields[1] = static_cast<int64_t>(op.input);
    fields[2] = static_cast<int64_t>(op.output);
    fields[3] = op.linearOutFeatures;
    fields[4] = op.embeddingVocabSize;
    fields[5] = op.embeddingDim;
    fields[6] = op.positionalMaxSeqLen;
    fields[7] = op.attentionNumHeads;
    fields[8] = op.feedForwardHiddenDim;
}

// input value shape: literal dims, -1 for a symbolic dim.
int refCompiledInputRank(void* handle) {
    auto* c = static_cast<Compiled*>(handle);
    const auto& model = c->module.models.front();
    return static_cast<int>(model.valueById(model.inputValue).shape.size());
}
void refCompiledInputShape(void* handle, int64_t* out) {
    auto* c = static_cast<Compiled*>(handle);
    const auto& model = c->module.models.front();
    const auto& shape = model.valueById(model.inputValue).shape;
    for (std::size_t i = 0; i < shape.size(); ++i) out[i] = shape[i].isSymbolic ? -1 : shape[i].literalValue;
}

// ---- Executor (weights regenerated from the seed on every call) -------------------------------

int refExecutorSyntheticInput(void* handle, unsigned int seed, int64_t batch) {
    return guarded([&] {
        auto* c = static_cast<Compiled*>(handle);
        gResult = cpu::Executor(seed).makeSyntheticInput(c->module.models.front(), static_cast<std::size_t>(batch));
    });
}

int refExecutorRun(void* handle, unsigned int seed, const float* data, const int64_t* shape, int rank,
                   int usePrecision) {
    return guarded([&] {
        auto* c = static_cast<Compiled*>(handle);
        std::optional<bf::ir::PrecisionPolicy> precision;
        if (usePrecision != 0) precision = c->module.precision;
        gResult = cpu::Executor(seed).run(c->module.models.front(), makeTensor(data, shape, rank), precision);
    });
}

// ---- Model (owns parameters; checkpoints) ------------------------------------------------------

int refModelNew(void* handle, unsigned int seed, int usePrecision, void** outModel) {
    return guarded([&] {
        auto* c = static_cast<Compiled*>(handle);
        std::optional<bf::ir::PrecisionPolicy> precision;
        if (usePrecision != 0) precision = c->module.precision;
        *outModel = new cpu::Model(c->module.models.front(), seed, std::nullopt, precision);
    });
}

// Same, with an explicit precision policy given as dtype codes.
int refModelNewWithPrecision(void* handle, unsigned int seed, int storage, int compute, int accumulate,
                             void** outModel) {
    return guarded([&] {
        auto* c = static_cast<Compiled*>(handle);
        bf::ir::PrecisionPolicy policy;
        policy.storage = dtypeFromCode(storage);
        policy.compute = dtypeFromCode(compute);
        policy.accumulate = dtypeFromCode(accumulate);
        *outModel = new cpu::Model(c->module.models.front(), seed, std::nullopt, policy);
    });
}

void refModelFree(void* model) { delete static_cast<cpu::Model*>(model); }

int refModelForward(void* model, const float* data, const int64_t* shape, int rank) {
    return guarded([&] { gResult = static_cast<cpu::Model*>(model)->forward(makeTensor(data, shape, rank)); });
}

int refModelLoadCheckpoint(void* model, const char* path) {
    return guarded([&] { cpu::loadCheckpoint(*static_cast<cpu::Model*>(model), path); });
}

int refModelSaveCheckpoint(void* model, const char* path) {
    return guarded([&] { cpu::saveCheckpoint(*static_cast<cpu::Model*>(model), path); });
}

int refModelParamCount(void* model) {
    return static_cast<int>(static_cast<cpu::Model*>(model)->allParameters().size());
}

const char* refModelParamName(void* model, int index) {
    return static_cast<cpu::Model*>(model)->allParameters().at(static_cast<std::size_t>(index))->name.c_str();
}

int refModelParamFetch(void* model, int index) {
    return guarded([&] {
        gResult = static_cast<cpu::Model*>(model)->allParameters().at(static_cast<std::size_t>(index))->value;
    });
}

int refModelParamSet(void* model, int index, const float* data, const int64_t* shape, int rank) {
    return guarded([&] {
        auto* p = static_cast<cpu::Model*>(model)->allParameters().at(static_cast<std::size_t>(index));
        Tensor t = makeTensor(data, shape, rank);
        if (t.shape() != p->value.shape()) throw std::invalid_argument("refModelParamSet: shape mismatch");
        p->value = std::move(t);
    });
}

// ---- single operators ---------------------------------------------------------------------------

#define REF_T(name) makeTensor(name, name##Shape, name##Rank)

int refOpUnary(int which, const float* x, const int64_t* xShape, int xRank) {
    return guarded([&] {
        Tensor in = REF_T(x);
        switch (which) {
            case 0: gResult = cpu::silu(in); break;
            case 1: gResult = cpu::relu(in); break;
            case 2: gResult = cpu::gelu(in); break;
            case 3: gResult = cpu::rmsnorm(in); break;
            case 4: gResult = cpu::softmax(in); break;
            default: throw std::invalid_argument("refOpUnary: unknown op");
        }
    });
}

int refOpBinary(int which, const float* a, const int64_t* aShape, int aRank, const float* b, const int64_t* bShape,
                int bRank, int64_t extra) {
    return guarded([&] {
        Tensor ta = REF_T(a);
        Tensor tb = REF_T(b);
        switch (which) {
            case 0: gResult = cpu::add(ta, tb); break;
            case 1: gResult = cpu::addBias(ta, tb); break;
            case 2: gResult = cpu::matmul(ta, tb); break;
            case 3: gResult = cpu::matmulTransposeB(ta, tb); break;
            case 4: gResult = cpu::embeddingLookup(ta, tb); break;
            case 5: gResult = cpu::addPositionalEmbedding(ta, tb); break;
            case 6: gResult = cpu::addPositionalEmbeddingAt(ta, tb, static_cast<std::size_t>(extra)); break;
            default: throw std::invalid_argument("refOpBinary: unknown op");
        }
    });
}

int refOpLinear(const float* x, const int64_t* xShape, int xRank, const float* w, const int64_t* wShape, int wRank,
                const float* b, const int64_t* bShape, int bRank) {
    return guarded([&] { gResult = cpu::linear(REF_T(x), REF_T(w), REF_T(b)); });
}

int refOpFeedForward(const float* x, const int64_t* xShape, int xRank, const float* w1, const int64_t* w1Shape,
                     int w1Rank, const float* b1, const int64_t* b1Shape, int b1Rank, const float* w2,
                     const int64_t* w2Shape, int w2Rank, const float* b2, const int64_t* b2Shape, int b2Rank) {
    return guarded([&] { gResult = cpu::feedForward(REF_T(x), REF_T(w1), REF_T(b1), REF_T(w2), REF_T(b2)); });
}

int refOpSelfAttention(const float* x, const int64_t* xShape, int xRank, const float* wq, const int64_t* wqShape,
                       int wqRank, const float* wk, const int64_t* wkShape, int wkRank, const float* wv,
                       const int64_t* wvShape, int wvRank, const float* wo, const int64_t* woShape, int woRank,
                       int64_t numHeads) {
    return guarded([&] {
        gResult = cpu::selfAttention(REF_T(x), REF_T(wq), REF_T(wk), REF_T(wv), REF_T(wo),
                                     static_cast<std::size_t>(numHeads));
    });
}

int refOpQuantize(const float* x, const int64_t* xShape, int xRank, int dtypeCode) {
    return guarded([&] { gResult = cpu::quantize(REF_T(x), dtypeFromCode(dtypeCode)); });
}

int refRandomTensor(const int64_t* shape, int rank, unsigned int seed) {
    return guarded([&] {
        std::vector<std::size_t> dims(shape, shape + rank);
        gResult = cpu::randomTensor(std::move(dims), seed);
    });
}

unsigned int refSeedFor(unsigned int base, uint64_t valueId, unsigned int salt) {
    return cpu::seedFor(base, static_cast<std::size_t>(valueId), salt);
}

}  // extern "C"
