// TEST INFRASTRUCTURE — not part of the product path.
//
// A C-ABI window onto the UNMODIFIED BlackForge CUDA backend (blackforge::backend::cuda::Model with its cuBLASLt
// bf16 path, fusedAttentionForward), compiled from the reference's own sources where they lie (oracle/Makefile,
// target cuda). It lets the GPU parity tests compare this repository's kernels with the reference's own device
// results on the same inputs. Nothing here re-implements reference behaviour: every entry point forwards to a
// reference function and copies the result out. Handles of compiled programs come from refCompile (ref_shim.cpp).
//
// Conventions as in ref_shim.cpp: 0 on success, 1 for std::invalid_argument, 2 for any other std::exception
// (message in refCudaLastError()); tensor results are left in a per-thread slot (refCudaResult*).

#include <cublasLt.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <exception>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

#include "blackforge/backend/cuda/autodiff.hpp"
#include "blackforge/backend/cuda/device_query.hpp"
#include "blackforge/backend/cuda/device_tensor.hpp"
#include "blackforge/backend/cuda/fused_attention.hpp"
#include "blackforge/backend/cuda/model.hpp"
#include "blackforge/ir/module.hpp"

namespace bf = blackforge;
namespace cuda = blackforge::backend::cuda;
using bf::runtime::Tensor;

extern "C" const void* refCompiledModelIR(void* handle);   // ref_shim.cpp

namespace {

thread_local std::string gError;
thread_local Tensor gOut;

template <typename Fn>
int guarded(Fn&& fn) {
    try {
        fn();
        return 0;
    } catch (const std::invalid_argument& e) {
        gError = e.what();
        return 1;
    } catch (const std::exception& e) {
        gError = e.what();
        return 2;
    }
}

Tensor hostTensor(const float* data, const int64_t* shape, int rank) {
    std::vector<std::size_t> dims(static_cast<std::size_t>(rank));
    std::size_t count = 1;
    for (int i = 0; i < rank; ++i) {
        dims[static_cast<std::size_t>(i)] = static_cast<std::size_t>(shape[i]);
        count *= dims[static_cast<std::size_t>(i)];
    }
    return Tensor(std::move(dims), std::vector<float>(data, data + count));
}

bf::sema::DType dtypeFromCode(int code) {   // the codes of ref_shim.cpp
    switch (code) {
        case 0: return bf::sema::DType::FP8_E4M3;
        case 1: return bf::sema::DType::FP8_E5M2;
        case 2: return bf::sema::DType::FP16;
        case 3: return bf::sema::DType::BF16;
        case 4: return bf::sema::DType::TF32;
        default: return bf::sema::DType::FP32;
    }
}

}  // namespace

extern "C" {

const char* refCudaLastError() { return gError.c_str(); }
int refCudaResultRank() { return static_cast<int>(gOut.rank()); }
void refCudaResultShape(int64_t* out) {
    for (std::size_t i = 0; i < gOut.rank(); ++i) out[i] = static_cast<int64_t>(gOut.shape()[i]);
}
int64_t refCudaResultCount() { return static_cast<int64_t>(gOut.elementCount()); }
void refCudaResultCopy(float* out) {
    for (std::size_t i = 0; i < gOut.elementCount(); ++i) out[i] = gOut.at(i);
}

int refCudaDeviceCount() {
    try {
        return static_cast<int>(cuda::enumerateDevices().size());
    } catch (...) {
        return 0;
    }
}

int refCudaSetDevice(int index) {
    return guarded([&] { cuda::setActiveDevice(index); });
}

// cuda::Model of a compiled program's first model; compute < 0 means no precision policy (fp32 path).
int refCudaModelNew(void* compiled, unsigned int seed, int storage, int compute, int accumulate, void** outModel) {
    return guarded([&] {
        const auto* ir = static_cast<const bf::ir::ModelIR*>(refCompiledModelIR(compiled));
        std::optional<bf::ir::PrecisionPolicy> policy;
        if (compute >= 0) {
            bf::ir::PrecisionPolicy p;
            p.storage = dtypeFromCode(storage);
            p.compute = dtypeFromCode(compute);
            p.accumulate = dtypeFromCode(accumulate);
            policy = p;
        }
        *outModel = new cuda::Model(*ir, seed, policy);
    });
}

void refCudaModelFree(void* model) { delete static_cast<cuda::Model*>(model); }

int refCudaModelParamCount(void* model) {
    return static_cast<int>(static_cast<cuda::Model*>(model)->parameters().size());
}

const char* refCudaModelParamName(void* model, int index) {
    return static_cast<cuda::Model*>(model)->parameters().at(static_cast<std::size_t>(index))->name.c_str();
}

int refCudaModelParamSet(void* model, int index, const float* data, const int64_t* shape, int rank) {
    return guarded([&] {
        cuda::Parameter* p = static_cast<cuda::Model*>(model)->parameters().at(static_cast<std::size_t>(index));
        Tensor t = hostTensor(data, shape, rank);
        if (t.shape() != p->value.shape()) throw std::invalid_argument("refCudaModelParamSet: shape mismatch");
        p->value = cuda::DeviceTensor::fromHost(t);
    });
}

int refCudaModelForward(void* model, const float* data, const int64_t* shape, int rank) {
    return guarded([&] {
        cuda::DeviceTensor in = cuda::DeviceTensor::fromHost(hostTensor(data, shape, rank));
        gOut = static_cast<cuda::Model*>(model)->forward(in).toHost();
    });
}

// Generation with the reference's key/value caches: `data` holds only the new token ids.
int refCudaModelForwardIncremental(void* model, const float* data, const int64_t* shape, int rank) {
    return guarded([&] {
        cuda::DeviceTensor in = cuda::DeviceTensor::fromHost(hostTensor(data, shape, rank));
        gOut = static_cast<cuda::Model*>(model)->forwardIncremental(in).toHost();
    });
}

int refCudaModelResetGeneration(void* model) {
    return guarded([&] { static_cast<cuda::Model*>(model)->resetGenerationState(); });
}

// Device time of `iters` forward passes (CUDA events around them, input uploaded once, results dropped on the
// device), after `warmup` untimed ones: the reference's own GPU path as a timing baseline.
int refCudaModelForwardTimed(void* model, const float* data, const int64_t* shape, int rank, int warmup, int iters,
                             double* msPerPass) {
    return guarded([&] {
        cuda::DeviceTensor in = cuda::DeviceTensor::fromHost(hostTensor(data, shape, rank));
        auto* m = static_cast<cuda::Model*>(model);
        for (int i = 0; i < warmup; ++i) (void)m->forward(in);
        cudaEvent_t a = nullptr, b = nullptr;
        if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) throw std::runtime_error("cudaEventCreate failed");
        cudaDeviceSynchronize();
        cudaEventRecord(a, nullptr);
        for (int i = 0; i < iters; ++i) (void)m->forward(in);
        cudaEventRecord(b, nullptr);
        if (cudaEventSynchronize(b) != cudaSuccess) throw std::runtime_error("the reference's forward failed on the device");
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, a, b);
        cudaEventDestroy(a);
        cudaEventDestroy(b);
        *msPerPass = static_cast<double>(ms) / (iters > 0 ? iters : 1);
    });
}

// Device time per generation step: the caches are reset, the prompt [batch, context] goes through forwardIncremental
// untimed, then `steps` single-token calls (columns of `stepIds` [batch, steps]) are timed with CUDA events.
int refCudaModelGenerationTimed(void* model, const float* prompt, int64_t batch, int64_t context, const float* stepIds,
                                int64_t steps, double* msPerStep) {
    return guarded([&] {
        auto* m = static_cast<cuda::Model*>(model);
        m->resetGenerationState();
        const int64_t promptShape[2] = {batch, context};
        (void)m->forwardIncremental(cuda::DeviceTensor::fromHost(hostTensor(prompt, promptShape, 2)));
        std::vector<cuda::DeviceTensor> columns;
        for (int64_t s = 0; s < steps; ++s) {
            std::vector<float> col(static_cast<std::size_t>(batch));
            for (int64_t b = 0; b < batch; ++b) col[static_cast<std::size_t>(b)] = stepIds[b * steps + s];
            const int64_t shape[2] = {batch, 1};
            columns.push_back(cuda::DeviceTensor::fromHost(hostTensor(col.data(), shape, 2)));
        }
        cudaEvent_t a = nullptr, b = nullptr;
        if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) throw std::runtime_error("cudaEventCreate failed");
        cudaDeviceSynchronize();
        cudaEventRecord(a, nullptr);
        for (int64_t s = 0; s < steps; ++s) (void)m->forwardIncremental(columns[static_cast<std::size_t>(s)]);
        cudaEventRecord(b, nullptr);
        if (cudaEventSynchronize(b) != cudaSuccess) throw std::runtime_error("the reference's generation step failed on the device");
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, a, b);
        cudaEventDestroy(a);
        cudaEventDestroy(b);
        *msPerStep = static_cast<double>(ms) / static_cast<double>(steps > 0 ? steps : 1);
    });
}

// fusedAttentionForward on fp32 q [batch, newLen, dim], k / v [batch, totalLen, dim]; the output lands in the result slot.
int refCudaFusedAttention(const float* q, const int64_t* qShape, const float* k, const int64_t* kShape, const float* v,
                          int64_t numHeads, float scale, int64_t oldLen) {
    return guarded([&] {
        cuda::DeviceTensor dq = cuda::DeviceTensor::fromHost(hostTensor(q, qShape, 3));
        cuda::DeviceTensor dk = cuda::DeviceTensor::fromHost(hostTensor(k, kShape, 3));
        cuda::DeviceTensor dv = cuda::DeviceTensor::fromHost(hostTensor(v, kShape, 3));
        cuda::FusedAttentionForwardResult r = cuda::fusedAttentionForward(dq, dk, dv, static_cast<std::size_t>(numHeads),
                                                                          scale, static_cast<std::size_t>(oldLen));
        gOut = r.output.toHost();
    });
}

// The same call timed on the device (CUDA events, operands uploaded once, `iters` calls after one warm-up); the last
// output lands in the result slot.
int refCudaFusedAttentionTimed(const float* q, const int64_t* qShape, const float* k, const int64_t* kShape,
                               const float* v, int64_t numHeads, float scale, int64_t oldLen, int iters, double* msPerCall) {
    return guarded([&] {
        cuda::DeviceTensor dq = cuda::DeviceTensor::fromHost(hostTensor(q, qShape, 3));
        cuda::DeviceTensor dk = cuda::DeviceTensor::fromHost(hostTensor(k, kShape, 3));
        cuda::DeviceTensor dv = cuda::DeviceTensor::fromHost(hostTensor(v, kShape, 3));
        const std::size_t heads = static_cast<std::size_t>(numHeads), old = static_cast<std::size_t>(oldLen);
        cuda::FusedAttentionForwardResult r = cuda::fusedAttentionForward(dq, dk, dv, heads, scale, old);
        cudaEvent_t a = nullptr, b = nullptr;
        if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) throw std::runtime_error("cudaEventCreate failed");
        cudaDeviceSynchronize();
        cudaEventRecord(a, nullptr);
        for (int i = 0; i < iters; ++i) r = cuda::fusedAttentionForward(dq, dk, dv, heads, scale, old);
        cudaEventRecord(b, nullptr);
        if (cudaEventSynchronize(b) != cudaSuccess) throw std::runtime_error("the reference's attention kernel failed on the device");
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, a, b);
        cudaEventDestroy(a);
        cudaEventDestroy(b);
        *msPerCall = static_cast<double>(ms) / (iters > 0 ? iters : 1);
        gOut = r.output.toHost();
    });
}

// fusedAttentionForward followed by fusedAttentionBackward of the reference (src/backend/cuda/fused_attention.cu:
// 305-380) on fp32 host operands; every result is copied to the caller's host buffers: out [batch, newLen, dim],
// m and l [batch, heads, newLen], dQ [batch, newLen, dim], dK and dV [batch, totalLen, dim]. `iters` > 0 also times
// the backward call alone on the device.
int refCudaFusedAttentionBackward(const float* dOut, const float* q, const int64_t* qShape, const float* k,
                                  const int64_t* kShape, const float* v, int64_t numHeads, float scale, int64_t oldLen,
                                  float* out, float* m, float* l, float* dQ, float* dK, float* dV, int iters,
                                  double* msPerCall) {
    return guarded([&] {
        cuda::DeviceTensor dq = cuda::DeviceTensor::fromHost(hostTensor(q, qShape, 3));
        cuda::DeviceTensor dk = cuda::DeviceTensor::fromHost(hostTensor(k, kShape, 3));
        cuda::DeviceTensor dv = cuda::DeviceTensor::fromHost(hostTensor(v, kShape, 3));
        cuda::DeviceTensor dg = cuda::DeviceTensor::fromHost(hostTensor(dOut, qShape, 3));
        const std::size_t heads = static_cast<std::size_t>(numHeads), old = static_cast<std::size_t>(oldLen);
        cuda::FusedAttentionForwardResult f = cuda::fusedAttentionForward(dq, dk, dv, heads, scale, old);
        cuda::FusedAttentionGrad g = cuda::fusedAttentionBackward(dg, dq, dk, dv, f.output, f.m, f.l, heads, scale, old);
        if (iters > 0 && msPerCall != nullptr) {
            cudaEvent_t a = nullptr, b = nullptr;
            if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) throw std::runtime_error("cudaEventCreate failed");
            cudaDeviceSynchronize();
            cudaEventRecord(a, nullptr);
            for (int i = 0; i < iters; ++i) g = cuda::fusedAttentionBackward(dg, dq, dk, dv, f.output, f.m, f.l, heads, scale, old);
            cudaEventRecord(b, nullptr);
            if (cudaEventSynchronize(b) != cudaSuccess) throw std::runtime_error("the reference's attention backward failed on the device");
            float ms = 0.0f;
            cudaEventElapsedTime(&ms, a, b);
            cudaEventDestroy(a);
            cudaEventDestroy(b);
            *msPerCall = static_cast<double>(ms) / iters;
        }
        auto copyOut = [](const cuda::DeviceTensor& t, float* dst) {
            if (dst == nullptr) return;
            Tensor h = t.toHost();
            std::copy(h.data().begin(), h.data().end(), dst);
        };
        copyOut(f.output, out);
        copyOut(f.m, m);
        copyOut(f.l, l);
        copyOut(g.dQ, dQ);
        copyOut(g.dK, dK);
        copyOut(g.dV, dV);
    });
}

// matmulBf16Backward of the reference (src/backend/cuda/ops_tensorcore.cu:389-417) on fp32 host operands a [m,k],
// b [k,n], grad [m,n]; dA [m,k] and dB [k,n] are copied to the caller's host buffers.
int refCudaMatmulBf16Backward(const float* a, const float* b, const float* grad, int64_t m, int64_t k, int64_t n, float* dA,
                              float* dB) {
    return guarded([&] {
        const int64_t sa[2] = {m, k}, sb[2] = {k, n}, sg[2] = {m, n};
        cuda::DeviceTensor da = cuda::DeviceTensor::fromHost(hostTensor(a, sa, 2));
        cuda::DeviceTensor db = cuda::DeviceTensor::fromHost(hostTensor(b, sb, 2));
        cuda::DeviceTensor dg = cuda::DeviceTensor::fromHost(hostTensor(grad, sg, 2));
        cuda::MatmulGrad r = cuda::matmulBf16Backward(da, db, dg);
        Tensor ha = r.dA.toHost(), hb = r.dB.toHost();
        std::copy(ha.data().begin(), ha.data().end(), dA);
        std::copy(hb.data().begin(), hb.data().end(), dB);
    });
}

// cublasLtMatmul configured the way the reference's bf16Gemm configures it (src/backend/cuda/ops_tensorcore.cu:
// 156-304: row-major layouts, A [m, k] and B [k, n] in bf16, fp32 compute, the top result of the heuristic search with
// at most 4 MiB of workspace, alpha 1, beta 0) and timed on the device. bf16Gemm itself sits in an unnamed namespace
// of the reference, so the library call it makes is made here with its settings; `cIsBf16` = 0 gives the fp32 result
// the reference writes, 1 a bf16 result (what a bf16 activation stream wants). Operands are the caller's device
// buffers. The calls run back to back for `iters` launches after `warmup`, so a long run settles at the clocks the
// power cap allows, like a kernel inside a long step.
int refCudaLtGemmTimed(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int cIsBf16, int warmup,
                       int iters, double* msPerCall) {
    return guarded([&] {
        auto ok = [](cublasStatus_t st, const char* what) {
            if (st != CUBLAS_STATUS_SUCCESS) throw std::runtime_error(std::string("cuBLASLt ") + what + " failed");
        };
        cublasLtHandle_t handle = nullptr;
        ok(cublasLtCreate(&handle), "create");
        cublasLtMatmulDesc_t op = nullptr;
        ok(cublasLtMatmulDescCreate(&op, CUBLAS_COMPUTE_32F, CUDA_R_32F), "desc");
        cublasOperation_t none = CUBLAS_OP_N;
        ok(cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_TRANSA, &none, sizeof(none)), "transa");
        ok(cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_TRANSB, &none, sizeof(none)), "transb");
        cublasLtOrder_t row = CUBLASLT_ORDER_ROW;
        cublasLtMatrixLayout_t la = nullptr, lb = nullptr, lc = nullptr;
        ok(cublasLtMatrixLayoutCreate(&la, CUDA_R_16BF, static_cast<uint64_t>(m), static_cast<uint64_t>(k), k), "layout a");
        ok(cublasLtMatrixLayoutCreate(&lb, CUDA_R_16BF, static_cast<uint64_t>(k), static_cast<uint64_t>(n), n), "layout b");
        ok(cublasLtMatrixLayoutCreate(&lc, cIsBf16 ? CUDA_R_16BF : CUDA_R_32F, static_cast<uint64_t>(m),
                                      static_cast<uint64_t>(n), n), "layout c");
        for (cublasLtMatrixLayout_t l : {la, lb, lc})
            ok(cublasLtMatrixLayoutSetAttribute(l, CUBLASLT_MATRIX_LAYOUT_ORDER, &row, sizeof(row)), "order");
        cublasLtMatmulPreference_t pref = nullptr;
        ok(cublasLtMatmulPreferenceCreate(&pref), "preference");
        std::size_t maxWorkspace = 4 * 1024 * 1024;
        ok(cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &maxWorkspace,
                                                sizeof(maxWorkspace)), "workspace preference");
        cublasLtMatmulHeuristicResult_t heur = {};
        int found = 0;
        ok(cublasLtMatmulAlgoGetHeuristic(handle, op, la, lb, lc, lc, pref, 1, &heur, &found), "heuristic");
        if (found == 0) throw std::runtime_error("cuBLASLt: no algorithm for this shape");
        void* workspace = nullptr;
        if (heur.workspaceSize > 0 && cudaMalloc(&workspace, heur.workspaceSize) != cudaSuccess)
            throw std::runtime_error("workspace allocation failed");
        const float alpha = 1.0f, beta = 0.0f;
        auto launch = [&] {
            ok(cublasLtMatmul(handle, op, &alpha, a, la, b, lb, &beta, c, lc, c, lc, &heur.algo, workspace,
                              heur.workspaceSize, nullptr), "matmul");
        };
        for (int i = 0; i < warmup; ++i) launch();
        cudaEvent_t e0 = nullptr, e1 = nullptr;
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        cudaDeviceSynchronize();
        cudaEventRecord(e0, nullptr);
        for (int i = 0; i < iters; ++i) launch();
        cudaEventRecord(e1, nullptr);
        if (cudaEventSynchronize(e1) != cudaSuccess) throw std::runtime_error("cublasLtMatmul failed on the device");
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, e0, e1);
        *msPerCall = static_cast<double>(ms) / (iters > 0 ? iters : 1);
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        if (workspace != nullptr) cudaFree(workspace);
        cublasLtMatmulPreferenceDestroy(pref);
        cublasLtMatrixLayoutDestroy(la);
        cublasLtMatrixLayoutDestroy(lb);
        cublasLtMatrixLayoutDestroy(lc);
        cublasLtMatmulDescDestroy(op);
        cublasLtDestroy(handle);
    });
}

}  // extern "C"
