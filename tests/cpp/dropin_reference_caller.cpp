// TEST INFRASTRUCTURE. Caller code written against the REFERENCE's headers only (blackforge/backend/cuda/*.hpp,
// its front end, its CPU backend), the way the reference's own tests are (tests/backend/cuda/model_tests.cu:25-38,
// 56-74, 380-395; tests/backend/cuda/ops_tests.cu), linked against the drop-in translation unit
// blackforge_b200/dropin/blackforge_backend_cuda.cpp + libbfb200.so instead of the reference's CUDA sources, and
// against the reference's own front end and CPU backend (compiled in place by oracle/Makefile) for the values to
// compare with. It shows that such caller code compiles and runs unchanged. Exit code 0 = every check passed.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>
#include <vector>

#include "blackforge/backend/cpu/checkpoint.hpp"
#include "blackforge/backend/cpu/executor.hpp"
#include "blackforge/backend/cpu/model.hpp"
#include "blackforge/backend/cpu/ops.hpp"
#include "blackforge/backend/cuda/checkpoint.hpp"
#include "blackforge/backend/cuda/device_query.hpp"
#include "blackforge/backend/cuda/device_tensor.hpp"
#include "blackforge/backend/cuda/executor.hpp"
#include "blackforge/backend/cuda/fused_attention.hpp"
#include "blackforge/backend/cuda/model.hpp"
#include "blackforge/backend/cuda/ops.hpp"
#include "blackforge/frontend/lexer.hpp"
#include "blackforge/frontend/parser.hpp"
#include "blackforge/ir/ir_builder.hpp"

using namespace blackforge;
using blackforge::runtime::Tensor;
namespace cpu = blackforge::backend::cpu;
namespace cuda = blackforge::backend::cuda;

namespace {

int failures = 0;

void expect(bool ok, const std::string& what) {
    if (!ok) {
        ++failures;
        std::printf("FAILED: %s\n", what.c_str());
    }
}

void expectNear(const Tensor& want, const Tensor& got, float tol, const std::string& what) {
    if (want.shape() != got.shape()) {
        expect(false, what + ": shapes differ");
        return;
    }
    float worst = 0.0f;
    for (std::size_t i = 0; i < want.elementCount(); ++i) worst = std::fmax(worst, std::fabs(want.at(i) - got.at(i)));
    std::printf("%-58s max abs diff %.3g (bar %.1g)\n", what.c_str(), worst, tol);
    expect(worst <= tol, what);
}

ir::Module buildModule(const std::string& source) {
    Lexer lexer(source, "test.bf");
    auto tokens = lexer.tokenize();
    expect(!lexer.diagnostics().hasErrors(), "lexer");
    Parser parser(std::move(tokens));
    ast::Program program = parser.parseProgram();
    expect(!parser.diagnostics().hasErrors(), "parser");
    ir::IRBuilder builder;
    ir::Module module = builder.build(program);
    expect(!builder.diagnostics().hasErrors(), "ir builder");
    return module;
}

Tensor ramp(std::vector<std::size_t> shape, float scale, float shift) {
    std::size_t n = 1;
    for (std::size_t d : shape) n *= d;
    std::vector<float> v(n);
    for (std::size_t i = 0; i < n; ++i) v[i] = scale * static_cast<float>((i * 37 + 11) % 23) / 23.0f + shift;
    return Tensor(std::move(shape), std::move(v));
}

const char* kTinyLm =
    "model TinyLM {\n"
    "    input bf16[batch, 3]\n"
    "    input |> embedding(6, 4) |> positional_embedding(4) |> attention(2) |> feedforward(8) |> linear(6)\n"
    "}\n";

}  // namespace

int main(int argc, char** argv) {
    const std::string scratch = argc > 1 ? argv[1] : "/tmp";
    expect(!cuda::enumerateDevices().empty(), "a CUDA device is visible");
    cuda::setActiveDevice(0);

    // model_tests.cu:56-74 — rmsnorm / linear / silu pipeline, CPU and CUDA with the same seed
    {
        ir::Module module = buildModule(
            "model M {\n    input bf16[batch, 4]\n    input |> rmsnorm |> linear(3) |> silu |> linear(2)\n}\n");
        cpu::Model cpuModel(module.models.front(), 7);
        cuda::Model cudaModel(module.models.front(), 7);
        Tensor input({2, 4}, {0.1F, -0.2F, 0.3F, 0.4F, -0.5F, 0.1F, 0.2F, -0.3F});
        expectNear(cpuModel.forward(input), cudaModel.forward(cuda::DeviceTensor::fromHost(input)).toHost(), 1e-4F,
                   "rmsnorm |> linear |> silu |> linear, CPU vs CUDA");
        expect(cudaModel.parameters().size() == 4 && cudaModel.name() == "M", "parameters() and name()");
    }
    // model_tests.cu:76-82 — a symbolic feature width is refused
    {
        ir::Module module = buildModule("model M {\n    input bf16[batch, batch2]\n    input |> linear(2)\n}\n");
        bool threw = false;
        try {
            cuda::Model model(module.models.front());
        } catch (const std::invalid_argument&) {
            threw = true;
        }
        expect(threw, "symbolic feature width throws std::invalid_argument");
    }
    // model_tests.cu:380-395 — TinyLM forward, CPU vs CUDA at 1e-3; then generation, a replaced parameter, checkpoints
    {
        ir::Module module = buildModule(kTinyLm);
        cpu::Model cpuModel(module.models.front(), 11);
        cuda::Model cudaModel(module.models.front(), 11);
        Tensor tokenIds({2, 3}, {0.0F, 1.0F, 2.0F, 3.0F, 4.0F, 5.0F});
        Tensor cpuOut = cpuModel.forward(tokenIds);
        Tensor cudaOut = cudaModel.forward(cuda::DeviceTensor::fromHost(tokenIds)).toHost();
        expect(cpuOut.shape() == std::vector<std::size_t>({2, 3, 6}), "TinyLM output shape");
        expectNear(cpuOut, cudaOut, 1e-3F, "TinyLM forward, CPU vs CUDA");
        expect(cudaModel.firstLayerEmbeddingVocabSize().value_or(0) == 6, "firstLayerEmbeddingVocabSize");

        // forwardIncremental: two tokens, then the third, equal the full forward on those positions
        cudaModel.resetGenerationState();
        Tensor firstTwo({2, 2}, {0.0F, 1.0F, 3.0F, 4.0F}), third({2, 1}, {2.0F, 5.0F});
        Tensor a = cudaModel.forwardIncremental(cuda::DeviceTensor::fromHost(firstTwo)).toHost();
        Tensor b = cudaModel.forwardIncremental(cuda::DeviceTensor::fromHost(third)).toHost();
        float worst = 0.0f;
        for (std::size_t s = 0; s < 2; ++s)
            for (std::size_t t = 0; t < 3; ++t)
                for (std::size_t v = 0; v < 6; ++v) {
                    const float inc = t < 2 ? a.at((s * 2 + t) * 6 + v) : b.at(s * 6 + v);
                    worst = std::fmax(worst, std::fabs(inc - cudaOut.at((s * 3 + t) * 6 + v)));
                }
        std::printf("%-58s max abs diff %.3g (bar 1e-4)\n", "forwardIncremental vs forward", worst);
        expect(worst <= 1e-4F, "forwardIncremental equals forward");
        cudaModel.resetGenerationState();

        // a parameter replaced through parameters() is what the next forward uses (both sides get the same values)
        std::vector<cuda::Parameter*> cudaParams = cudaModel.parameters();
        std::vector<cpu::Parameter*> cpuParams = cpuModel.parameters();
        expect(cudaParams.size() == cpuParams.size(), "same parameter count on both sides");
        for (std::size_t i = 0; i < cudaParams.size() && i < cpuParams.size(); ++i) {
            expect(cudaParams[i]->name == cpuParams[i]->name, "parameter name " + cpuParams[i]->name);
            Tensor fresh = ramp(cpuParams[i]->value.shape(), 0.4f, -0.2f);
            cpuParams[i]->value = fresh;
            cudaParams[i]->value = cuda::DeviceTensor::fromHost(fresh);
        }
        expectNear(cpuModel.forward(tokenIds), cudaModel.forward(cuda::DeviceTensor::fromHost(tokenIds)).toHost(), 1e-3F,
                   "TinyLM after replacing every parameter");

        // checkpoints cross the two back ends both ways (checkpoint.cu:60-130, cpu/checkpoint.hpp:15-24)
        const std::string fromCuda = scratch + "/dropin_cuda.bfckpt", fromCpu = scratch + "/dropin_cpu.bfckpt";
        cuda::saveCheckpoint(cudaModel, fromCuda);
        cpu::Model cpuLoaded(module.models.front(), 99);
        cpu::loadCheckpoint(cpuLoaded, fromCuda);
        expectNear(cpuModel.forward(tokenIds), cpuLoaded.forward(tokenIds), 1e-6F, "CUDA-written checkpoint read by the CPU side");
        cpu::saveCheckpoint(cpuModel, fromCpu);
        cuda::Model cudaLoaded(module.models.front(), 123);
        cuda::loadCheckpoint(cudaLoaded, fromCpu);
        expectNear(cpuModel.forward(tokenIds), cudaLoaded.forward(cuda::DeviceTensor::fromHost(tokenIds)).toHost(), 1e-3F,
                   "CPU-written checkpoint read by the CUDA side");
        expectNear(cpuParams[0]->value, cudaLoaded.parameters()[0]->value.toHost(), 0.0F, "loaded parameter visible through parameters()");

        // compute bf16 (the tensor-core path) stays within the bf16 bar of the CPU result
        ir::PrecisionPolicy policy;
        policy.compute = sema::DType::BF16;
        cuda::Model cudaBf16(module.models.front(), 11, policy);
        cpu::Model cpuSame(module.models.front(), 11);
        expectNear(cpuSame.forward(tokenIds), cudaBf16.forward(cuda::DeviceTensor::fromHost(tokenIds)).toHost(), 2e-2F,
                   "TinyLM with compute bf16 vs CPU fp32");

        // training is refused, clearly
        bool threw = false;
        try {
            cudaModel.zeroGrad();
        } catch (const std::runtime_error&) {
            threw = true;
        }
        expect(threw, "zeroGrad throws std::runtime_error");
    }
    // executor.hpp:26-29 — Executor::run / makeSyntheticInput, CPU vs CUDA (src/main.cpp:356-370)
    {
        ir::Module module = buildModule(kTinyLm);
        cpu::Executor cpuExec(42);
        cuda::Executor cudaExec(42);
        Tensor in = cpuExec.makeSyntheticInput(module.models.front(), 3);
        expectNear(in, cudaExec.makeSyntheticInput(module.models.front(), 3), 0.0F, "makeSyntheticInput");
        expectNear(cpuExec.run(module.models.front(), in), cudaExec.run(module.models.front(), in), 1e-3F, "Executor::run");
    }
    // src/main.cpp:803-849 — the `benchmark` command's device part as the reference wrote it: warm-up and measured
    // Executor::run calls timed on the host clock, then the speed-up and the largest difference against the CPU
    // executor's result for the same seed (same input, same initial weights)
    {
        ir::Module module = buildModule(kTinyLm);
        const ir::ModelIR& model = module.models.front();
        const std::size_t batchSize = 4, warmupIterations = 2, measuredIterations = 5;
        cpu::Executor cpuExecutor;
        Tensor cpuInput = cpuExecutor.makeSyntheticInput(model, batchSize);
        auto cpuStart = std::chrono::steady_clock::now();
        Tensor cpuOutput = cpuExecutor.run(model, cpuInput);
        const double cpuMillis = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - cpuStart).count();
        std::string gpuName = "unknown GPU";
        for (const auto& d : cuda::enumerateDevices()) {
            if (d.index == 0) gpuName = d.name;
        }
        cuda::Executor cudaExecutor;
        Tensor cudaInput = cudaExecutor.makeSyntheticInput(model, batchSize);
        for (std::size_t i = 0; i < warmupIterations; ++i) (void)cudaExecutor.run(model, cudaInput);
        Tensor gpuOutput;
        auto start = std::chrono::steady_clock::now();
        for (std::size_t i = 0; i < measuredIterations; ++i) gpuOutput = cudaExecutor.run(model, cudaInput);
        const double gpuMeanMillis = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - start).count() /
                                     static_cast<double>(measuredIterations);
        float maxAbsDiff = 0.0F;
        for (std::size_t i = 0; i < cpuOutput.elementCount() && i < gpuOutput.elementCount(); ++i) {
            maxAbsDiff = std::max(maxAbsDiff, std::fabs(cpuOutput.at(i) - gpuOutput.at(i)));
        }
        std::printf("benchmark report: %s, mean GPU time %.3f ms, throughput %.1f samples/s, speed-up vs CPU %.2fx, "
                    "largest difference vs CPU (reference) %.3g\n",
                    gpuName.c_str(), gpuMeanMillis, gpuMeanMillis > 0.0 ? batchSize * 1000.0 / gpuMeanMillis : 0.0,
                    cpuMillis / gpuMeanMillis, maxAbsDiff);
        expect(gpuOutput.shape() == cpuOutput.shape() && maxAbsDiff <= 1e-3F, "benchmark report: CPU and GPU agree for the same seed");
    }
    // ops.hpp — operator level against the CPU backend's operators (ops_tests.cu compares the same pairs)
    {
        Tensor a = ramp({5, 7}, 1.0f, -0.5f), b = ramp({7, 3}, 0.8f, -0.3f), bias = ramp({3}, 0.5f, 0.0f);
        cuda::DeviceTensor da = cuda::DeviceTensor::fromHost(a), db = cuda::DeviceTensor::fromHost(b),
                           dbias = cuda::DeviceTensor::fromHost(bias);
        expectNear(cpu::matmul(a, b), cuda::matmul(da, db).toHost(), 1e-5F, "matmul");
        expectNear(cpu::matmul(a, b), cuda::matmulBf16(da, db).toHost(), 3e-2F, "matmulBf16 (bf16 operands)");
        expectNear(cpu::matmul(a, b), cuda::matmulBf16CachedWeight(da, db).toHost(), 3e-2F, "matmulBf16CachedWeight");
        expectNear(cpu::linear(a, b, bias), cuda::linear(da, db, dbias).toHost(), 1e-5F, "linear");
        expectNear(cpu::linear(a, b, bias), cuda::linearBf16(da, db, dbias).toHost(), 3e-2F, "linearBf16");
        expectNear(cpu::silu(a), cuda::silu(da).toHost(), 1e-6F, "silu");
        expectNear(cpu::gelu(a), cuda::gelu(da).toHost(), 1e-5F, "gelu");
        expectNear(cpu::relu(a), cuda::relu(da).toHost(), 0.0F, "relu");
        expectNear(cpu::rmsnorm(a), cuda::rmsnorm(da).toHost(), 1e-5F, "rmsnorm");
        expectNear(cpu::softmax(a), cuda::softmax(da).toHost(), 1e-6F, "softmax");
        expectNear(cpu::add(a, a), cuda::add(da, da).toHost(), 0.0F, "add");
        Tensor bt = ramp({4, 7}, 0.6f, -0.2f);
        expectNear(cpu::matmulTransposeB(a, bt), cuda::matmulTransposeB(da, cuda::DeviceTensor::fromHost(bt)).toHost(), 1e-5F,
                   "matmulTransposeB");

        // DeviceTensor: clone, reshape by move, move construction and assignment
        cuda::DeviceTensor c = da.clone();
        expectNear(a, c.toHost(), 0.0F, "DeviceTensor::clone");
        cuda::DeviceTensor r = std::move(c).reshaped({7, 5});
        expect(r.shape() == std::vector<std::size_t>({7, 5}) && c.data() == nullptr && c.elementCount() == 0, "reshaped() && consumes its source");
        cuda::DeviceTensor moved(std::move(r));
        expect(r.data() == nullptr && moved.elementCount() == 35, "move construction");
        cuda::DeviceTensor assigned = cuda::DeviceTensor::zeros({2, 2});
        assigned = std::move(moved);
        expect(moved.data() == nullptr && assigned.dim(0) == 7, "move assignment");
        expect(cuda::DeviceTensor::zeros({3, 2}).toHost().max() == 0.0F, "zeros");
        bool threw = false;
        try {
            (void)std::move(assigned).reshaped({6, 6});
        } catch (const std::invalid_argument&) {
            threw = true;
        }
        expect(threw, "reshaped() to another element count throws");

        // blocks: dim 8, 2 heads
        Tensor x = ramp({2, 5, 8}, 1.0f, -0.5f), wq = ramp({8, 8}, 0.5f, -0.25f), wk = ramp({8, 8}, 0.4f, -0.1f),
               wv = ramp({8, 8}, 0.3f, -0.2f), wo = ramp({8, 8}, 0.6f, -0.3f), w1 = ramp({8, 16}, 0.5f, -0.25f),
               b1 = ramp({16}, 0.2f, -0.1f), w2 = ramp({16, 8}, 0.4f, -0.2f), b2 = ramp({8}, 0.1f, 0.0f);
        auto dev = [](const Tensor& t) { return cuda::DeviceTensor::fromHost(t); };
        cuda::DeviceTensor dx = dev(x), dwq = dev(wq), dwk = dev(wk), dwv = dev(wv), dwo = dev(wo), dw1 = dev(w1), db1 = dev(b1),
                           dw2 = dev(w2), db2 = dev(b2);
        Tensor wantAttn = cpu::selfAttention(x, wq, wk, wv, wo, 2), wantFf = cpu::feedForward(x, w1, b1, w2, b2);
        expectNear(wantAttn, cuda::selfAttention(dx, dwq, dwk, dwv, dwo, 2).toHost(), 1e-4F, "selfAttention");
        expectNear(wantAttn, cuda::selfAttentionBf16(dx, dwq, dwk, dwv, dwo, 2).toHost(), 5e-2F, "selfAttentionBf16");
        expectNear(wantFf, cuda::feedForward(dx, dw1, db1, dw2, db2).toHost(), 1e-4F, "feedForward");
        expectNear(wantFf, cuda::feedForwardBf16(dx, dw1, db1, dw2, db2).toHost(), 5e-2F, "feedForwardBf16");
        // incremental attention: three positions, then two, equal the full result
        cuda::KVCache cache, cache16;
        Tensor head({2, 3, 8}, std::vector<float>(48)), tail({2, 2, 8}, std::vector<float>(32));
        for (std::size_t s = 0; s < 2; ++s)
            for (std::size_t t = 0; t < 5; ++t)
                for (std::size_t d = 0; d < 8; ++d)
                    (t < 3 ? head.at((s * 3 + t) * 8 + d) : tail.at((s * 2 + t - 3) * 8 + d)) = x.at((s * 5 + t) * 8 + d);
        Tensor i1 = cuda::selfAttentionIncremental(dev(head), dwq, dwk, dwv, dwo, 2, cache).toHost();
        Tensor i2 = cuda::selfAttentionIncremental(dev(tail), dwq, dwk, dwv, dwo, 2, cache).toHost();
        Tensor j1 = cuda::selfAttentionIncrementalBf16(dev(head), dwq, dwk, dwv, dwo, 2, cache16).toHost();
        Tensor j2 = cuda::selfAttentionIncrementalBf16(dev(tail), dwq, dwk, dwv, dwo, 2, cache16).toHost();
        float worst = 0.0f, worst16 = 0.0f;
        for (std::size_t s = 0; s < 2; ++s)
            for (std::size_t t = 0; t < 5; ++t)
                for (std::size_t d = 0; d < 8; ++d) {
                    const float want = wantAttn.at((s * 5 + t) * 8 + d);
                    worst = std::fmax(worst, std::fabs(want - (t < 3 ? i1.at((s * 3 + t) * 8 + d) : i2.at((s * 2 + t - 3) * 8 + d))));
                    worst16 = std::fmax(worst16, std::fabs(want - (t < 3 ? j1.at((s * 3 + t) * 8 + d) : j2.at((s * 2 + t - 3) * 8 + d))));
                }
        std::printf("%-58s max abs diff %.3g / bf16 %.3g\n", "selfAttentionIncremental vs selfAttention", worst, worst16);
        expect(worst <= 1e-4F && cache.length == 5, "selfAttentionIncremental");
        expect(worst16 <= 5e-2F && cache16.length == 5, "selfAttentionIncrementalBf16");

        // fusedAttentionForward: row statistics and output against a direct evaluation (fused_attention.hpp:42-57)
        Tensor q = ramp({1, 4, 8}, 1.0f, -0.5f), k = ramp({1, 4, 8}, 0.9f, -0.4f), v = ramp({1, 4, 8}, 0.7f, -0.3f);
        cuda::FusedAttentionForwardResult fr = cuda::fusedAttentionForward(dev(q), dev(k), dev(v), 2, 0.5f, 0);
        Tensor fo = fr.output.toHost(), fm = fr.m.toHost(), fl = fr.l.toHost();
        float worstO = 0.0f, worstM = 0.0f;
        for (std::size_t h = 0; h < 2; ++h)
            for (std::size_t i = 0; i < 4; ++i) {
                double m = -1e30, l = 0.0, o[4] = {0, 0, 0, 0};
                std::vector<double> sc(i + 1);
                for (std::size_t j = 0; j <= i; ++j) {
                    double dot = 0.0;
                    for (std::size_t d = 0; d < 4; ++d) dot += q.at(i * 8 + h * 4 + d) * k.at(j * 8 + h * 4 + d);
                    sc[j] = dot * 0.5;
                    m = std::fmax(m, sc[j]);
                }
                for (std::size_t j = 0; j <= i; ++j) {
                    const double p = std::exp(sc[j] - m);
                    l += p;
                    for (std::size_t d = 0; d < 4; ++d) o[d] += p * v.at(j * 8 + h * 4 + d);
                }
                for (std::size_t d = 0; d < 4; ++d) worstO = std::fmax(worstO, std::fabs(static_cast<float>(o[d] / l) - fo.at(i * 8 + h * 4 + d)));
                worstM = std::fmax(worstM, std::fabs(static_cast<float>(m) - fm.at(h * 4 + i)));
                worstM = std::fmax(worstM, std::fabs(static_cast<float>(l) - fl.at(h * 4 + i)));
            }
        std::printf("%-58s max abs diff %.3g (output) %.3g (m, l)\n", "fusedAttentionForward vs direct evaluation", worstO, worstM);
        expect(worstO <= 1e-5F && worstM <= 1e-5F, "fusedAttentionForward");

        // fusedAttentionBackward (fused_attention.hpp:59-76) against central differences of the forward above:
        // loss = sum(g * output), one element of q, k or v moved by +-0.01 at a time
        Tensor g = ramp({1, 4, 8}, 0.6f, -0.2f);
        cuda::FusedAttentionGrad grad = cuda::fusedAttentionBackward(dev(g), dev(q), dev(k), dev(v), fr.output, fr.m, fr.l, 2, 0.5f, 0);
        Tensor gq = grad.dQ.toHost(), gk = grad.dK.toHost(), gv = grad.dV.toHost();
        auto loss = [&](const Tensor& qq, const Tensor& kk, const Tensor& vv) {
            Tensor o = cuda::fusedAttentionForward(dev(qq), dev(kk), dev(vv), 2, 0.5f, 0).output.toHost();
            double acc = 0.0;
            for (std::size_t i = 0; i < 32; ++i) acc += static_cast<double>(o.at(i)) * g.at(i);
            return acc;
        };
        float worstG = 0.0f;
        for (int which = 0; which < 3; ++which) {
            const Tensor& analytic = which == 0 ? gq : (which == 1 ? gk : gv);
            for (std::size_t i = 0; i < 32; ++i) {
                std::vector<float> up = (which == 0 ? q : (which == 1 ? k : v)).data(), down = up;
                up[i] += 0.01f;
                down[i] -= 0.01f;
                Tensor tu({1, 4, 8}, up), td({1, 4, 8}, down);
                const double numeric = which == 0   ? (loss(tu, k, v) - loss(td, k, v)) / 0.02
                                       : which == 1 ? (loss(q, tu, v) - loss(q, td, v)) / 0.02
                                                    : (loss(q, k, tu) - loss(q, k, td)) / 0.02;
                worstG = std::fmax(worstG, std::fabs(static_cast<float>(numeric) - analytic.at(i)));
            }
        }
        std::printf("%-58s max abs diff %.3g\n", "fusedAttentionBackward vs differences of the forward", worstG);
        expect(worstG <= 2e-3F, "fusedAttentionBackward");
    }
    std::printf(failures == 0 ? "dropin: all checks passed\n" : "dropin: %d check(s) FAILED\n", failures);
    return failures == 0 ? 0 : 1;
}
