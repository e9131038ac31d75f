// extern "C" surface declared in include/bfb200.h: argument checks, exception -> status mapping,
// and nothing else. All work happens in the kernel layer (kernels.hpp) and the host layer (host/).
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <thread>
#include <vector>

#include "common.cuh"
#include "host/bfb200.hpp"
#include "host/tp.hpp"
#include "host/watchdog.hpp"
#include "host/widen.hpp"
#include "kernels.hpp"
#include "pool.hpp"

using bfb::asStream;
using bfb::guarded;
using bfb::require;

struct bfb_model {
    std::unique_ptr<bfb200::Model> model;
    std::vector<bfb200::Parameter*> params;  // refreshed lazily
    void refresh() {
        if (params.empty()) params = model->parameters();
    }
};

namespace {

std::optional<bfb200::PrecisionPolicy> toPolicy(const bfb_precision* p) {
    if (p == nullptr || p->present == 0) return std::nullopt;
    bfb200::PrecisionPolicy policy;
    policy.storage = p->storage;
    policy.compute = p->compute;
    policy.accumulate = p->accumulate;
    return policy;
}

void requireDevice() {
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        bfb::fail(BFB_CUDA_ERROR, "no usable CUDA device (this library has no CPU fallback)");
    }
}

}  // namespace

extern "C" {

const char* bfb_last_error(void) { return bfb::lastErrorSlot().c_str(); }

int32_t bfb_version(void) { return 100; }

bfb_status bfb_device_count(int32_t* count) {
    return guarded([&] {
        require(count != nullptr, "device_count: null pointer");
        *count = 0;
        int n = 0;
        cudaError_t e = cudaGetDeviceCount(&n);
        if (e != cudaSuccess || n == 0) {
            cudaGetLastError();
            bfb::fail(BFB_CUDA_ERROR, "no usable CUDA device");
        }
        *count = n;
    });
}

bfb_status bfb_set_device(int32_t index) {
    return guarded([&] {
        int n = 0;
        cudaError_t e = cudaGetDeviceCount(&n);
        if (e != cudaSuccess) {
            cudaGetLastError();
            bfb::fail(BFB_CUDA_ERROR, "no usable CUDA device");
        }
        require(index >= 0 && index < n, "set_device: device index out of range");
        BFB_CUDA(cudaSetDevice(index));
    });
}

bfb_status bfb_pool_acquire(size_t bytes, void** d_out) {
    return guarded([&] {
        require(d_out != nullptr, "pool_acquire: null result pointer");
        *d_out = nullptr;
        if (bytes == 0) return;
        requireDevice();
        *d_out = bfb::poolAcquire(bytes);
    });
}

bfb_status bfb_pool_release(void* d_ptr, size_t bytes) {
    bfb::poolRelease(d_ptr, bytes);
    return BFB_OK;
}

bfb_status bfb_pool_trim(void) {
    return guarded([&] { bfb::poolTrim(); });
}

bfb_status bfb_pool_stats(size_t* cached_bytes, size_t* live_bytes) {
    return guarded([&] { bfb::poolStats(cached_bytes, live_bytes); });
}

bfb_status bfb_copy_h2d(void* d_dst, const void* h_src, size_t bytes, void* stream) {
    return guarded([&] {
        if (bytes == 0) return;
        require(d_dst != nullptr && h_src != nullptr, "copy_h2d: null pointer");
        BFB_CUDA(cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, asStream(stream)));
        BFB_CUDA(cudaStreamSynchronize(asStream(stream)));
    });
}

bfb_status bfb_copy_d2h(void* h_dst, const void* d_src, size_t bytes, void* stream) {
    return guarded([&] {
        if (bytes == 0) return;
        require(h_dst != nullptr && d_src != nullptr, "copy_d2h: null pointer");
        BFB_CUDA(cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, asStream(stream)));
        BFB_CUDA(cudaStreamSynchronize(asStream(stream)));
    });
}

bfb_status bfb_copy_d2d(void* d_dst, const void* d_src, size_t bytes, void* stream) {
    return guarded([&] {
        if (bytes == 0) return;
        require(d_dst != nullptr && d_src != nullptr, "copy_d2d: null pointer");
        BFB_CUDA(cudaMemcpyAsync(d_dst, d_src, bytes, cudaMemcpyDeviceToDevice, asStream(stream)));
    });
}

bfb_status bfb_memset_zero(void* d_dst, size_t bytes, void* stream) {
    return guarded([&] {
        if (bytes == 0) return;
        require(d_dst != nullptr, "memset_zero: null pointer");
        BFB_CUDA(cudaMemsetAsync(d_dst, 0, bytes, asStream(stream)));
    });
}

bfb_status bfb_stream_synchronize(void* stream) {
    return guarded([&] { BFB_CUDA(cudaStreamSynchronize(asStream(stream))); });
}

bfb_status bfb_embed_pos(const float* d_ids, const float* d_table, const float* d_pos, void* d_out, int32_t out_dtype,
                         int64_t batch, int64_t seq, int64_t vocab, int64_t dim, int64_t max_seq, int64_t pos_offset,
                         int32_t* d_oob_count, void* stream) {
    return guarded([&] {
        bfb::embedPos(d_ids, d_table, d_pos, d_out, out_dtype, batch, seq, vocab, dim, max_seq, pos_offset, d_oob_count,
                      asStream(stream));
    });
}

bfb_status bfb_add_positional(const float* d_in, const float* d_pos, float* d_out, int64_t batch, int64_t seq,
                              int64_t dim, int64_t max_seq, int64_t pos_offset, void* stream) {
    return guarded([&] { bfb::addPositional(d_in, d_pos, d_out, batch, seq, dim, max_seq, pos_offset, asStream(stream)); });
}

bfb_status bfb_rmsnorm(const void* d_x, int32_t x_dtype, void* d_out, int32_t out_dtype, int64_t rows, int64_t dim,
                       float eps, void* stream) {
    return guarded([&] { bfb::rmsnorm(d_x, x_dtype, d_out, out_dtype, rows, dim, eps, asStream(stream)); });
}

bfb_status bfb_softmax(const float* d_x, float* d_out, int64_t rows, int64_t cols, void* stream) {
    return guarded([&] { bfb::softmaxRows(d_x, d_out, rows, cols, asStream(stream)); });
}

bfb_status bfb_elementwise(int32_t op, const float* d_a, const float* d_b, const float* d_c, float* d_out, int64_t n,
                           int64_t cols, void* stream) {
    return guarded([&] { bfb::elementwise(op, d_a, d_b, d_c, d_out, n, cols, asStream(stream)); });
}

bfb_status bfb_cast(const void* d_in, int32_t in_dtype, void* d_out, int32_t out_dtype, int64_t n, float scale,
                    const float* d_scale, void* stream) {
    return guarded([&] { bfb::castScaled(d_in, in_dtype, d_out, out_dtype, n, scale, d_scale, asStream(stream)); });
}

bfb_status bfb_amax(const void* d_in, int32_t in_dtype, int64_t n, float* d_amax, void* stream) {
    return guarded([&] { bfb::amax(d_in, in_dtype, n, d_amax, asStream(stream)); });
}

bfb_status bfb_fp8_scale_from_amax(const float* d_amax, float* d_scales, void* stream) {
    return guarded([&] { bfb::fp8ScaleFromAmax(d_amax, d_scales, asStream(stream)); });
}

bfb_status bfb_quantize_e4m3(const void* d_in, int32_t in_dtype, int64_t n, void* d_out, float* d_scales,
                             const float* d_weight_inverse, void* stream) {
    return guarded([&] {
        require(n >= 0, "quantize_e4m3: negative size");
        requireDevice();
        const size_t bytes = static_cast<size_t>(bfb::quantizeScratchFloats(n)) * sizeof(float);
        float* scratch = static_cast<float*>(bfb::poolAcquire(bytes));
        try {
            bfb::quantizeE4m3(d_in, in_dtype, n, d_out, d_scales, d_weight_inverse, scratch, asStream(stream));
        } catch (...) {
            bfb::poolRelease(scratch, bytes);
            throw;
        }
        // work on `stream` is ordered before any later use of the buffer on the same stream
        bfb::poolRelease(scratch, bytes);
    });
}

bfb_status bfb_rmsnorm_quantize_e4m3(const void* d_x, int64_t rows, int64_t dim, float eps, void* d_out, float* d_scales,
                                     const float* d_weight_inverse, void* stream) {
    return guarded([&] {
        require(rows >= 0, "rmsnorm_quantize_e4m3: negative size");
        requireDevice();
        const size_t bytes = static_cast<size_t>(bfb::rmsnormQuantizeScratchFloats(rows)) * sizeof(float);
        float* scratch = static_cast<float*>(bfb::poolAcquire(bytes));
        try {
            bfb::rmsnormQuantizeE4m3(d_x, rows, dim, eps, d_out, d_scales, d_weight_inverse, scratch, asStream(stream));
        } catch (...) {
            bfb::poolRelease(scratch, bytes);
            throw;
        }
        // work on `stream` is ordered before any later use of the buffer on the same stream
        bfb::poolRelease(scratch, bytes);
    });
}

bfb_status bfb_rmsnorm_quantize_e4m3_from_stats(const void* d_x, int64_t rows, int64_t dim, float eps, void* d_out,
                                                float* d_scales, const float* d_weight_inverse, const float* d_sum_sq_parts,
                                                const float* d_max_parts, int32_t parts, void* stream) {
    return guarded([&] {
        require(rows >= 0, "rmsnorm_quantize_e4m3_from_stats: negative size");
        require(parts >= 1 && d_sum_sq_parts != nullptr && d_max_parts != nullptr,
                "rmsnorm_quantize_e4m3_from_stats: the row statistics are missing");
        requireDevice();
        const size_t bytes = static_cast<size_t>(bfb::rmsnormQuantizeScratchFloats(rows)) * sizeof(float);
        float* scratch = static_cast<float*>(bfb::poolAcquire(bytes));
        try {
            bfb::rmsnormQuantizeE4m3(d_x, rows, dim, eps, d_out, d_scales, d_weight_inverse, scratch, asStream(stream),
                                     d_sum_sq_parts, d_max_parts, parts);
        } catch (...) {
            bfb::poolRelease(scratch, bytes);
            throw;
        }
        bfb::poolRelease(scratch, bytes);
    });
}

bfb_status bfb_weight_prepare(const float* d_w, void* d_out, int32_t out_dtype, int64_t k, int64_t n, float scale,
                              const float* d_scale, void* stream) {
    return guarded([&] { bfb::weightPrepare(d_w, d_out, out_dtype, k, n, scale, d_scale, asStream(stream)); });
}

bfb_status bfb_gemm(const void* d_a, const void* d_b, void* d_c, int64_t m, int64_t n, int64_t k, int32_t ab_dtype,
                    int32_t b_layout, int32_t c_dtype, int32_t epilogue, const float* d_bias, const void* d_residual,
                    float alpha, const float* d_alpha, int32_t round_c_bf16, int32_t* d_status, void* stream) {
    return guarded([&] {
        bfb::GemmArgs g;
        g.a = d_a;
        g.b = d_b;
        g.c = d_c;
        g.m = m;
        g.n = n;
        g.k = k;
        g.abDtype = ab_dtype;
        g.bLayout = b_layout;
        g.cDtype = c_dtype;
        g.epilogue = epilogue;
        g.bias = d_bias;
        g.residual = d_residual;
        g.alpha = alpha;
        g.dAlpha = d_alpha;
        g.roundCBf16 = round_c_bf16;
        g.dStatus = d_status;
        bfb::gemm(g, asStream(stream));
    });
}

bfb_status bfb_row_sum_squares(const void* d_x, int32_t dtype, float* d_out, int64_t rows, int64_t dim, void* stream) {
    return guarded([&] { bfb::rowSumSquares(d_x, dtype, d_out, rows, dim, asStream(stream)); });
}

bfb_status bfb_gemm_rmsnorm(const void* d_a, const void* d_w, void* d_c, int64_t m, int64_t n, int64_t k,
                            int32_t ab_dtype, int32_t c_dtype, int32_t epilogue, const float* d_bias,
                            const void* d_residual, const float* d_row_sum_sq, int32_t row_sum_sq_parts, float eps,
                            float* d_out_sum_sq, float* d_out_max_abs, int32_t* d_status, void* stream) {
    return guarded([&] {
        bfb::GemmArgs g;
        g.a = d_a;
        g.b = d_w;
        g.c = d_c;
        g.m = m;
        g.n = n;
        g.k = k;
        g.abDtype = ab_dtype;
        g.bLayout = BFB_B_NK;
        g.cDtype = c_dtype;
        g.epilogue = epilogue;
        g.bias = d_bias;
        g.residual = d_residual;
        g.rowSumSq = d_row_sum_sq;
        g.rowSumSqParts = row_sum_sq_parts;
        g.rowInvDim = k > 0 ? 1.0f / static_cast<float>(k) : 0.0f;
        g.rowEps = eps;
        g.outSumSq = d_out_sum_sq;
        g.outMaxAbs = d_out_max_abs;
        g.dStatus = d_status;
        bfb::gemm(g, asStream(stream));
    });
}

bfb_status bfb_gemm_few_rows(const void* d_a, const void* d_w, void* d_c, int64_t m, int64_t n, int64_t k, int32_t ab_dtype,
                             int32_t c_dtype, int32_t epilogue, const float* d_bias, const void* d_residual, float alpha,
                             const float* d_row_sum_sq, int32_t row_sum_sq_parts, float eps, float* d_out_sum_sq,
                             int32_t* d_status, void* stream) {
    return guarded([&] {
        bfb::GemmArgs g;
        g.a = d_a;
        g.b = d_w;
        g.c = d_c;
        g.m = m;
        g.n = n;
        g.k = k;
        g.abDtype = ab_dtype;
        g.bLayout = BFB_B_NK;
        g.cDtype = c_dtype;
        g.epilogue = epilogue;
        g.bias = d_bias;
        g.residual = d_residual;
        g.alpha = alpha;
        g.rowSumSq = d_row_sum_sq;
        g.rowSumSqParts = row_sum_sq_parts;
        g.rowInvDim = k > 0 ? 1.0f / static_cast<float>(k) : 0.0f;
        g.rowEps = eps;
        g.outSumSq = d_out_sum_sq;
        g.dStatus = d_status;
        g.preferSkinny = 1;
        bfb::require(bfb::gemmSkinnyEligible(g) || m == 0 || n == 0,
                     "gemm_few_rows: needs 1..128 rows, k > 0, tensor-core formats and 16-byte aligned rows");
        bfb::gemm(g, asStream(stream));
    });
}

bfb_status bfb_matmul_transpose_b(const float* d_a, const float* d_b, float* d_c, int64_t m, int64_t n, int64_t k,
                                  void* stream) {
    return guarded([&] { bfb::matmulTransposeB(d_a, d_b, d_c, m, n, k, asStream(stream)); });
}

bfb_status bfb_matmul_bf16_backward(const float* d_a, const float* d_b, const float* d_grad, float* d_da, float* d_db,
                                    int64_t m, int64_t k, int64_t n, void* stream) {
    return guarded([&] { bfb::matmulBf16Backward(d_a, d_b, d_grad, d_da, d_db, m, k, n, nullptr, asStream(stream)); });
}

bfb_status bfb_attention_fwd(const void* d_q, const void* d_k, const void* d_v, void* d_out, float* d_m, float* d_l,
                             int32_t dtype, int64_t batch, int64_t new_len, int64_t total_len, int64_t num_heads,
                             int64_t head_dim, int64_t ld_q, int64_t ld_k, int64_t ld_v, int64_t ld_o, float scale,
                             int64_t old_len, int32_t causal, int32_t* d_status, void* stream) {
    return guarded([&] {
        bfb::AttentionArgs a;
        a.q = d_q;
        a.k = d_k;
        a.v = d_v;
        a.out = d_out;
        a.m = d_m;
        a.l = d_l;
        a.dtype = dtype;
        a.batch = batch;
        a.newLen = new_len;
        a.totalLen = total_len;
        a.numHeads = num_heads;
        a.headDim = head_dim;
        a.ldQ = ld_q;
        a.ldK = ld_k;
        a.ldV = ld_v;
        a.ldO = ld_o;
        a.scale = scale;
        a.oldLen = old_len;
        a.causal = causal;
        a.dStatus = d_status;
        bfb::attentionForward(a, asStream(stream));
    });
}

bfb_status bfb_attention_fwd_maxima(const void* d_q, const void* d_k, const void* d_v, void* d_out, float* d_maxima,
                                    int64_t maxima_count, int64_t batch, int64_t new_len, int64_t total_len, int64_t num_heads,
                                    int64_t ld_q, int64_t ld_k, int64_t ld_v, int64_t ld_o, float scale, int64_t old_len,
                                    int32_t* d_status, void* stream) {
    return guarded([&] {
        bfb::AttentionArgs a;
        a.q = d_q;
        a.k = d_k;
        a.v = d_v;
        a.out = d_out;
        a.dtype = BFB_BF16;
        a.batch = batch;
        a.newLen = new_len;
        a.totalLen = total_len;
        a.numHeads = num_heads;
        a.headDim = 128;
        a.ldQ = ld_q;
        a.ldK = ld_k;
        a.ldV = ld_v;
        a.ldO = ld_o;
        a.scale = scale;
        a.oldLen = old_len;
        a.causal = 1;
        a.dStatus = d_status;
        a.outMaxima = d_maxima;
        require(d_maxima != nullptr, "attention_fwd_maxima: null maxima pointer");
        require(maxima_count == bfb::attentionMaximaCount(a), "attention_fwd_maxima: maxima_count must be batch * heads * ceil(new_len / 128) * 4");
        bfb::attentionForward(a, asStream(stream));
    });
}

bfb_status bfb_attention_bwd(const void* d_dout, const void* d_q, const void* d_k, const void* d_v, const void* d_out,
                             const float* d_m, const float* d_l, float* d_dq, float* d_dk, float* d_dv, float* d_scratch,
                             int32_t dtype, int64_t batch, int64_t new_len, int64_t total_len, int64_t num_heads,
                             int64_t head_dim, int64_t ld_in, int64_t ld_kv, int64_t ld_grad_q, int64_t ld_grad_kv,
                             float scale, int64_t old_len, int32_t causal, int32_t* d_status, void* stream) {
    return guarded([&] {
        bfb::AttentionBackwardArgs a;
        a.dOut = d_dout;
        a.q = d_q;
        a.k = d_k;
        a.v = d_v;
        a.out = d_out;
        a.m = d_m;
        a.l = d_l;
        a.dQ = d_dq;
        a.dK = d_dk;
        a.dV = d_dv;
        require(batch >= 0 && new_len >= 0 && num_heads > 0, "attention_bwd: bad sizes");
        require(d_scratch != nullptr || batch * new_len == 0, "attention_bwd: scratch of 2 * batch * heads * new_len floats required");
        a.lse2Scratch = d_scratch;
        a.dTermScratch = d_scratch == nullptr ? nullptr : d_scratch + batch * num_heads * new_len;
        a.dtype = dtype;
        a.batch = batch;
        a.newLen = new_len;
        a.totalLen = total_len;
        a.numHeads = num_heads;
        a.headDim = head_dim;
        a.ldQ = a.ldO = a.ldDo = ld_in;
        a.ldK = a.ldV = ld_kv;
        a.ldDq = ld_grad_q;
        a.ldDk = a.ldDv = ld_grad_kv;
        a.scale = scale;
        a.oldLen = old_len;
        a.causal = causal;
        a.dStatus = d_status;
        bfb::attentionBackward(a, asStream(stream));
    });
}

// ---- model ----------------------------------------------------------------------------------------------

static bfb_status createModel(const bfb_op_desc* ops, int32_t n_ops, int64_t input_last_dim, uint32_t seed,
                              const bfb_precision* precision, bool randomInit, bfb_model** out) {
    return guarded([&] {
        require(out != nullptr, "model_create: null result pointer");
        *out = nullptr;
        require(ops != nullptr && n_ops > 0, "model_create: the model has no pipeline");
        std::vector<bfb_op_desc> v(ops, ops + n_ops);
        auto holder = std::make_unique<bfb_model>();
        holder->model = std::make_unique<bfb200::Model>(v, input_last_dim, seed, toPolicy(precision), randomInit);
        *out = holder.release();
    });
}

bfb_status bfb_model_create(const bfb_op_desc* ops, int32_t n_ops, int64_t input_last_dim, uint32_t seed,
                            const bfb_precision* precision, bfb_model** out) {
    return createModel(ops, n_ops, input_last_dim, seed, precision, true, out);
}

bfb_status bfb_model_create_uninitialised(const bfb_op_desc* ops, int32_t n_ops, int64_t input_last_dim,
                                          const bfb_precision* precision, bfb_model** out) {
    return createModel(ops, n_ops, input_last_dim, 0, precision, false, out);
}

void bfb_model_destroy(bfb_model* model) { delete model; }

bfb_status bfb_model_set_tensor_parallel(bfb_model* model, int32_t rank, int32_t world) {
    return guarded([&] {
        require(model != nullptr, "model: null handle");
        model->model->setTensorParallel(rank, world);
        model->params.clear();
    });
}

bfb_status bfb_set_shared_sm_mode(int32_t dynamic_tiles, int32_t reserved_sms) {
    return guarded([&] {
        require(reserved_sms >= 0, "shared_sm_mode: reserved_sms must not be negative");
        bfb::setDynamicTiles(dynamic_tiles != 0);
        bfb::setReservedSms(reserved_sms);
    });
}

bfb_status bfb_model_set_tensor_parallel_overlap(bfb_model* model, int32_t groups, int32_t reserved_sms) {
    return guarded([&] {
        require(model != nullptr, "model: null handle");
        model->model->setTensorParallelOverlap(groups, reserved_sms);
    });
}

// Parameter metadata comes from the structure alone: no device memory is touched, so these work
// without a GPU.
int32_t bfb_model_param_count(const bfb_model* model) {
    if (model == nullptr) return 0;
    return static_cast<int32_t>(model->model->parameterCount());
}

const char* bfb_model_param_name(const bfb_model* model, int32_t index) {
    if (model == nullptr || index < 0 || index >= bfb_model_param_count(model)) return "";
    return model->model->parameterName(static_cast<std::size_t>(index)).c_str();
}

int32_t bfb_model_param_rank(const bfb_model* model, int32_t index) {
    if (model == nullptr || index < 0 || index >= bfb_model_param_count(model)) return 0;
    return static_cast<int32_t>(model->model->parameterShape(static_cast<std::size_t>(index)).size());
}

void bfb_model_param_shape(const bfb_model* model, int32_t index, int64_t* shape_out) {
    if (model == nullptr || shape_out == nullptr || index < 0 || index >= bfb_model_param_count(model)) return;
    const auto& s = model->model->parameterShape(static_cast<std::size_t>(index));
    for (std::size_t i = 0; i < s.size(); ++i) shape_out[i] = static_cast<int64_t>(s[i]);
}

bfb_status bfb_model_param_set(bfb_model* model, int32_t index, const float* h_values) {
    return guarded([&] {
        require(model != nullptr, "model: null handle");
        require(index >= 0, "model: negative parameter index");
        requireDevice();
        model->model->setParameter(static_cast<std::size_t>(index), h_values);
    });
}

bfb_status bfb_model_param_get(bfb_model* model, int32_t index, float* h_values) {
    return guarded([&] {
        require(model != nullptr, "model: null handle");
        require(index >= 0, "model: negative parameter index");
        requireDevice();
        model->model->getParameter(static_cast<std::size_t>(index), h_values);
    });
}

bfb_status bfb_model_param_fill_normal(bfb_model* model, int32_t index, uint64_t seed, float sigma) {
    return guarded([&] {
        require(model != nullptr, "model: null handle");
        require(index >= 0, "model: negative parameter index");
        requireDevice();
        model->model->fillParameterNormal(static_cast<std::size_t>(index), seed, sigma);
    });
}

bfb_status bfb_model_release_master_weights(bfb_model* model) {
    return guarded([&] {
        require(model != nullptr, "model: null handle");
        requireDevice();
        model->model->releaseMasterWeights();
    });
}

bfb_status bfb_model_load_checkpoint(bfb_model* model, const char* path) {
    return guarded([&] {
        require(model != nullptr && path != nullptr, "model: null argument");
        bfb200::loadCheckpoint(*model->model, path);
    });
}

namespace {
void copyLoadStats(const bfb200::CheckpointLoadStats& s, bfb_checkpoint_load_stats* stats) {
    if (stats == nullptr) return;
    stats->tensors = static_cast<int64_t>(s.tensors);
    stats->file_bytes = s.fileBytes;
    stats->read_bytes = s.readBytes;
    stats->uploaded_bytes = s.uploadedBytes;
    stats->seconds = s.seconds;
    stats->cache_hit = s.cacheHit ? 1 : 0;
    stats->cache_bytes = s.cacheBytes;
}
}  // namespace

bfb_status bfb_model_load_checkpoint_streaming(bfb_model* model, const char* path, uint64_t chunk_bytes,
                                               bfb_checkpoint_load_stats* stats) {
    return guarded([&] {
        require(model != nullptr && path != nullptr, "model: null argument");
        copyLoadStats(bfb200::loadCheckpoint(*model->model, path, static_cast<std::size_t>(chunk_bytes)), stats);
    });
}

bfb_status bfb_model_load_checkpoint_cached(bfb_model* model, const char* path, uint64_t chunk_bytes,
                                            bfb_checkpoint_load_stats* stats) {
    return guarded([&] {
        require(model != nullptr && path != nullptr, "model: null argument");
        copyLoadStats(bfb200::loadCheckpointCached(*model->model, path, static_cast<std::size_t>(chunk_bytes)), stats);
    });
}

bfb_status bfb_checkpoint_index(const char* path, int32_t index, char* name_buf, int32_t name_capacity, int32_t* rank,
                                int64_t* dims8, uint64_t* data_offset, uint64_t* data_bytes, int32_t* count) {
    return guarded([&] {
        require(path != nullptr, "checkpoint_index: null path");
        const std::vector<bfb200::CheckpointEntry> entries = bfb200::indexCheckpoint(path);
        if (count != nullptr) *count = static_cast<int32_t>(entries.size());
        if (index < 0) return;
        require(static_cast<std::size_t>(index) < entries.size(), "checkpoint_index: no such entry");
        const bfb200::CheckpointEntry& e = entries[static_cast<std::size_t>(index)];
        if (name_buf != nullptr && name_capacity > 0) {
            const std::size_t n = std::min<std::size_t>(e.name.size(), static_cast<std::size_t>(name_capacity) - 1);
            std::memcpy(name_buf, e.name.data(), n);
            name_buf[n] = '\0';
        }
        if (rank != nullptr) *rank = static_cast<int32_t>(e.shape.size());
        if (dims8 != nullptr) {
            for (std::size_t d = 0; d < e.shape.size() && d < 8; ++d) dims8[d] = static_cast<int64_t>(e.shape[d]);
        }
        if (data_offset != nullptr) *data_offset = e.dataOffset;
        if (data_bytes != nullptr) *data_bytes = e.dataBytes;
    });
}

bfb_status bfb_model_save_checkpoint(bfb_model* model, const char* path) {
    return guarded([&] {
        require(model != nullptr && path != nullptr, "model: null argument");
        requireDevice();
        bfb200::saveCheckpoint(*model->model, path);
    });
}

bfb_status bfb_model_forward(bfb_model* model, const float* d_input, const int64_t* shape, int32_t rank,
                             int32_t input_range_trusted, float** d_out, int64_t* out_shape, int32_t* out_rank,
                             void* stream) {
    return guarded([&] {
        require(model != nullptr && d_out != nullptr && out_shape != nullptr && out_rank != nullptr && shape != nullptr,
                "model_forward: null argument");
        require(rank >= 1 && rank <= 8, "model_forward: bad rank");
        requireDevice();
        std::vector<std::size_t> dims(shape, shape + rank);
        // borrow the caller's buffer as a DeviceTensor without owning it
        bfb200::DeviceTensor borrowed = bfb200::DeviceTensor::borrow(const_cast<float*>(d_input), dims);
        bfb200::DeviceTensor result;
        try {
            result = model->model->forward(borrowed, input_range_trusted != 0, stream);
        } catch (...) {
            borrowed.releaseOwnership();
            throw;
        }
        borrowed.releaseOwnership();
        *out_rank = static_cast<int32_t>(result.rank());
        for (std::size_t i = 0; i < result.rank(); ++i) out_shape[i] = static_cast<int64_t>(result.dim(i));
        *d_out = result.releaseOwnership();
    });
}

bfb_status bfb_model_benchmark(bfb_model* model, const float* d_input, const int64_t* shape, int32_t rank, int64_t warmup,
                               int64_t measured, bfb_benchmark_result* out, bfb_op_benchmark* per_op,
                               int32_t per_op_capacity, void* stream) {
    return guarded([&] {
        require(model != nullptr && shape != nullptr && out != nullptr, "model_benchmark: null argument");
        require(rank >= 1 && rank <= 8, "model_benchmark: bad rank");
        require(warmup >= 0 && measured >= 0, "model_benchmark: negative iteration count");
        if (measured == 0) throw std::invalid_argument("runBenchmark: measuredIterations must be positive");
        requireDevice();
        std::vector<std::size_t> dims(shape, shape + rank);
        bfb200::DeviceTensor borrowed = bfb200::DeviceTensor::borrow(const_cast<float*>(d_input), dims);
        bfb200::BenchmarkResult r;
        try {
            r = model->model->benchmark(borrowed, static_cast<std::size_t>(warmup), static_cast<std::size_t>(measured), stream);
        } catch (...) {
            borrowed.releaseOwnership();
            throw;
        }
        borrowed.releaseOwnership();
        out->warmup_iterations = static_cast<int64_t>(r.warmupIterations);
        out->measured_iterations = static_cast<int64_t>(r.measuredIterations);
        out->mean_ms = r.meanMilliseconds;
        out->samples_per_second = r.throughputSamplesPerSecond;
        out->estimated_memory_bytes = r.estimatedMemoryBytes;
        out->op_count = static_cast<int32_t>(r.perOperation.size());
        for (std::size_t i = 0; per_op != nullptr && i < r.perOperation.size() && i < static_cast<std::size_t>(std::max(0, per_op_capacity)); ++i) {
            std::memset(per_op[i].name, 0, sizeof(per_op[i].name));
            std::strncpy(per_op[i].name, r.perOperation[i].operationName.c_str(), sizeof(per_op[i].name) - 1);
            per_op[i].index = static_cast<int32_t>(r.perOperation[i].operationIndex);
            per_op[i].mean_ms = r.perOperation[i].meanMilliseconds;
        }
    });
}

bfb_status bfb_model_forward_incremental(bfb_model* model, const float* d_new_ids, const int64_t* shape, int32_t rank,
                                         int32_t input_range_trusted, float** d_out, int64_t* out_shape,
                                         int32_t* out_rank, void* stream) {
    return guarded([&] {
        require(model != nullptr && d_out != nullptr && out_shape != nullptr && out_rank != nullptr && shape != nullptr,
                "model_forward_incremental: null argument");
        require(rank >= 2 && rank <= 8, "model_forward_incremental: bad rank");
        requireDevice();
        std::vector<std::size_t> dims(shape, shape + rank);
        bfb200::DeviceTensor borrowed = bfb200::DeviceTensor::borrow(const_cast<float*>(d_new_ids), dims);
        bfb200::DeviceTensor result;
        try {
            result = model->model->forwardIncremental(borrowed, input_range_trusted != 0, stream);
        } catch (...) {
            borrowed.releaseOwnership();
            throw;
        }
        borrowed.releaseOwnership();
        *out_rank = static_cast<int32_t>(result.rank());
        for (std::size_t i = 0; i < result.rank(); ++i) out_shape[i] = static_cast<int64_t>(result.dim(i));
        *d_out = result.releaseOwnership();
    });
}

bfb_status bfb_model_reset_generation(bfb_model* model) {
    return guarded([&] {
        require(model != nullptr, "model_reset_generation: null model");
        model->model->resetGenerationState();
    });
}

bfb_status bfb_model_generation_position(bfb_model* model, int64_t* position) {
    return guarded([&] {
        require(model != nullptr && position != nullptr, "model_generation_position: null argument");
        *position = static_cast<int64_t>(model->model->generationPosition());
    });
}

namespace {
// slice size of the bf16 result path for small batches: a quarter of the batch
std::size_t step4(std::size_t batch) { return (batch + 3) / 4; }

// Host-link bytes of the calling thread's latest host-buffer forward.
struct HostTransfer {
    int64_t h2d = 0;
    int64_t d2h = 0;
};
HostTransfer& hostTransfer() {
    thread_local HostTransfer t;
    return t;
}

// Share (percent) of the result slices that the host-buffer path moves as bf16 and widens on host threads when
// the result is bf16-exact; the rest is copied as fp32. The 2-byte way halves the link time but costs host
// cores and twice the host memory traffic (the fp32 words are written by the CPU on top of the incoming copy).
// Measured with 2 G logits per call: one process on a 16-core host with a PCIe 5 x16 link, all slices narrow
// 127-138 ms, three quarters 148 ms, half 158 ms, none 168-182 ms (bound by the link); four processes on a 32-core
// host, half narrow 487 ms per step, because they share the host's memory bandwidth, which is then the limit and
// which the plain copies load least. (One host of the same kind took 176 ms with all slices narrow and 147 ms with
// seven of eight; there seven of eight cost 143 against 138 ms on a host that keeps up. The default stays with the
// common case.) So: everything when this process has the host to itself and 12 or more
// threads, half with 6 or more, none below or when a launcher reports several processes on the host
// (LOCAL_WORLD_SIZE > 1). BFB_HOST_NARROW_PCT overrides (0..100).
int narrowSharePercent() {
    if (const char* e = std::getenv("BFB_HOST_NARROW_PCT")) return std::max(0, std::min(100, std::atoi(e)));
    if (const char* e = std::getenv("LOCAL_WORLD_SIZE")) {
        if (std::atoi(e) > 1) return 0;
    }
    const int threads = bfb200::defaultWidenThreads();
    return threads >= 12 ? 100 : (threads >= 6 ? 50 : 0);
}

// Two non-blocking streams per device for the host-buffer path: compute and device-to-host copies.
struct HostPathStreams {
    cudaStream_t compute = nullptr;
    cudaStream_t copy = nullptr;
    // bf16 result path: a ring of device slices, pinned host slices and their copy-finished events, kept between
    // calls (pinning host memory is slow) and grown when a larger slice comes along. Four slots: a slot is busy
    // from the start of its slice's compute to the end of its widening, about three slice times.
    static constexpr int kSlots = 4;
    void* dev16[kSlots] = {};
    void* pinned16[kSlots] = {};
    cudaEvent_t copied[kSlots] = {};
    std::size_t sliceBytes = 0;

    void ensureStaging(std::size_t bytes) {
        if (bytes <= sliceBytes) return;
        for (int i = 0; i < kSlots; ++i) {
            if (dev16[i] != nullptr) BFB_CUDA(cudaFree(dev16[i]));
            if (pinned16[i] != nullptr) BFB_CUDA(cudaFreeHost(pinned16[i]));
            dev16[i] = pinned16[i] = nullptr;
        }
        sliceBytes = 0;
        for (int i = 0; i < kSlots; ++i) {
            BFB_CUDA(cudaMalloc(&dev16[i], bytes));
            BFB_CUDA(cudaMallocHost(&pinned16[i], bytes));
            if (copied[i] == nullptr) BFB_CUDA(cudaEventCreateWithFlags(&copied[i], cudaEventDisableTiming));
        }
        sliceBytes = bytes;
    }
};
// One host-buffer forward at a time per device: the calls of several host threads share the two streams and the
// staging ring above, so the second caller waits for the first (held for the whole sliced pass).
std::mutex& hostPathMutex() {
    static std::mutex perDevice[64];
    int dev = 0;
    BFB_CUDA(cudaGetDevice(&dev));
    return perDevice[dev & 63];
}

HostPathStreams& hostPathStreams() {
    static std::mutex mu;
    static std::map<int, HostPathStreams> perDevice;
    int dev = 0;
    BFB_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    HostPathStreams& s = perDevice[dev];
    if (s.compute == nullptr) {
        BFB_CUDA(cudaStreamCreateWithFlags(&s.compute, cudaStreamNonBlocking));
        BFB_CUDA(cudaStreamCreateWithFlags(&s.copy, cudaStreamNonBlocking));
    }
    return s;
}
}  // namespace

// Sequences are independent, so a batch is run in slices: while slice i+1 computes, the logits of slice i
// travel to the host on a second stream. With pinned host memory the copy (the larger cost for wide
// vocabularies) hides the compute; with pageable memory the result is the same, only without the overlap.
bfb_status bfb_model_forward_host(bfb_model* model, const float* h_input, const int64_t* shape, int32_t rank,
                                  float* h_out, int64_t* out_shape, int32_t* out_rank) {
    return guarded([&] {
        require(model != nullptr && h_input != nullptr && shape != nullptr && out_shape != nullptr && out_rank != nullptr,
                "model_forward_host: null argument");
        require(rank >= 1 && rank <= 8, "model_forward_host: bad rank");
        std::vector<std::size_t> dims(shape, shape + rank);
        std::vector<std::size_t> outDims = model->model->outputShape(dims);
        *out_rank = static_cast<int32_t>(outDims.size());
        for (std::size_t i = 0; i < outDims.size(); ++i) out_shape[i] = static_cast<int64_t>(outDims[i]);
        if (h_out == nullptr) return;  // shape query only
        requireDevice();
        std::size_t count = 1;
        for (std::size_t d : dims) count *= d;
        bfb200::DeviceTensor in(dims);
        if (count > 0) BFB_CUDA(cudaMemcpy(in.data(), h_input, count * sizeof(float), cudaMemcpyHostToDevice));
        hostTransfer().h2d = static_cast<int64_t>(count * sizeof(float));
        hostTransfer().d2h = 0;

        const std::size_t batch = dims[0];
        const std::size_t slices = (rank == 2 && batch >= 8) ? 4 : 1;
        if (slices == 1) {
            bfb200::DeviceTensor result = model->model->forward(in, false, nullptr);
            if (result.elementCount() > 0) {
                BFB_CUDA(cudaMemcpy(h_out, result.data(), result.elementCount() * sizeof(float), cudaMemcpyDeviceToHost));
                hostTransfer().d2h = static_cast<int64_t>(result.elementCount() * sizeof(float));
            }
            return;
        }
        std::lock_guard<std::mutex> hostPathLock(hostPathMutex());
        HostPathStreams& st = hostPathStreams();
        const std::size_t perSeqIn = count / batch;
        std::size_t outCount = 1;
        for (std::size_t d : outDims) outCount *= d;
        const std::size_t perSeqOut = outCount / batch;
        const int narrowPct = model->model->resultIsBf16Exact() ? narrowSharePercent() : 0;
        if (narrowPct > 0) {
            // Under `storage bf16` the logits are bf16 numbers. A share of the slices crosses PCIe as 2-byte values
            // and is widened to the caller's fp32 words by host threads; the rest is copied as fp32 straight into
            // the caller's buffer. The first kind costs half the PCIe time but host memory bandwidth and cores,
            // the second only PCIe time, so mixing them keeps both busy. Every slice's copy overlaps the next
            // slice's compute. The result is bit-identical to copying the fp32 result whole.
            const std::size_t seqs = batch >= 16 ? std::max<std::size_t>(1, batch / 8) : step4(batch);
            st.ensureStaging(seqs * perSeqOut * 2);
            int dev = 0;
            BFB_CUDA(cudaGetDevice(&dev));
            bfb200::WidenQueue queue(dev, bfb200::defaultWidenThreads());
            std::vector<bfb200::DeviceTensor> wide;  // fp32 slices, kept alive until their copies have finished
            std::size_t slice = 0, narrowCount = 0;
            std::size_t jobOfSlot[HostPathStreams::kSlots] = {};
            bool slotUsed[HostPathStreams::kSlots] = {};
            for (std::size_t b0 = 0; b0 < batch; b0 += seqs, ++slice) {
                const std::size_t nb = std::min(seqs, batch - b0);
                // slice s goes the 2-byte way when the running share falls behind the target
                const bool narrow = (slice + 1) * static_cast<std::size_t>(narrowPct) / 100 > narrowCount;
                std::vector<std::size_t> sliceDims = dims;
                sliceDims[0] = nb;
                bfb200::DeviceTensor view = bfb200::DeviceTensor::borrow(in.data() + b0 * perSeqIn, sliceDims);
                const int k = static_cast<int>(narrowCount % HostPathStreams::kSlots);
                try {
                    // both calls return after their own work on the compute stream is complete (status read-back)
                    if (narrow) {
                        if (slotUsed[k]) queue.wait(jobOfSlot[k]);  // the slot has been copied out and widened
                        model->model->forwardBf16(view, st.dev16[k], false, st.compute);
                    } else {
                        wide.push_back(model->model->forward(view, false, st.compute));
                    }
                } catch (...) {
                    view.releaseOwnership();
                    cudaStreamSynchronize(st.copy);
                    throw;
                }
                view.releaseOwnership();
                if (narrow) {
                    BFB_CUDA(cudaMemcpyAsync(st.pinned16[k], st.dev16[k], nb * perSeqOut * 2, cudaMemcpyDeviceToHost, st.copy));
                    BFB_CUDA(cudaEventRecord(st.copied[k], st.copy));
                    jobOfSlot[k] = queue.submit(st.copied[k], static_cast<const std::uint16_t*>(st.pinned16[k]),
                                                h_out + b0 * perSeqOut, nb * perSeqOut);
                    slotUsed[k] = true;
                    ++narrowCount;
                    hostTransfer().d2h += static_cast<int64_t>(nb * perSeqOut * 2);
                } else {
                    BFB_CUDA(cudaMemcpyAsync(h_out + b0 * perSeqOut, wide.back().data(), nb * perSeqOut * sizeof(float),
                                             cudaMemcpyDeviceToHost, st.copy));
                    hostTransfer().d2h += static_cast<int64_t>(nb * perSeqOut * sizeof(float));
                }
            }
            queue.waitAll();
            BFB_CUDA(cudaStreamSynchronize(st.copy));
            return;
        }
        std::vector<bfb200::DeviceTensor> results;  // kept alive until their copies have finished
        results.reserve(slices);
        const std::size_t step = (batch + slices - 1) / slices;
        for (std::size_t b0 = 0; b0 < batch; b0 += step) {
            const std::size_t nb = std::min(step, batch - b0);
            std::vector<std::size_t> sliceDims = dims;
            sliceDims[0] = nb;
            bfb200::DeviceTensor view = bfb200::DeviceTensor::borrow(in.data() + b0 * perSeqIn, sliceDims);
            try {
                // forward returns after its own work on the compute stream is complete (status read-back)
                results.push_back(model->model->forward(view, false, st.compute));
            } catch (...) {
                view.releaseOwnership();
                cudaStreamSynchronize(st.copy);
                throw;
            }
            view.releaseOwnership();
            // the fp32 route works on the default stream, which the non-blocking copy stream does not wait for
            BFB_CUDA(cudaStreamSynchronize(nullptr));
            BFB_CUDA(cudaMemcpyAsync(h_out + b0 * perSeqOut, results.back().data(), nb * perSeqOut * sizeof(float),
                                     cudaMemcpyDeviceToHost, st.copy));
            hostTransfer().d2h += static_cast<int64_t>(nb * perSeqOut * sizeof(float));
        }
        BFB_CUDA(cudaStreamSynchronize(st.copy));
    });
}

bfb_status bfb_host_widen_bf16(const uint16_t* h_src, float* h_dst, int64_t count, int32_t threads) {
    return guarded([&] {
        require(count >= 0 && threads >= 1 && threads <= 256, "host_widen_bf16: bad count or thread number");
        if (count == 0) return;
        require(h_src != nullptr && h_dst != nullptr, "host_widen_bf16: null pointer");
        const std::size_t n = static_cast<std::size_t>(count), parts = static_cast<std::size_t>(threads);
        const std::size_t chunk = ((n + parts - 1) / parts + 7) / 8 * 8;
        std::vector<std::thread> helpers;
        for (std::size_t t = 1; t < parts && t * chunk < n; ++t) {
            helpers.emplace_back([=] { bfb200::widenBf16(h_src + t * chunk, h_dst + t * chunk, std::min(chunk, n - t * chunk)); });
        }
        bfb200::widenBf16(h_src, h_dst, std::min(chunk, n));
        for (std::thread& h : helpers) h.join();
    });
}

bfb_status bfb_host_transfer_bytes(int64_t* h2d_bytes, int64_t* d2h_bytes) {
    return guarded([&] {
        require(h2d_bytes != nullptr && d2h_bytes != nullptr, "host_transfer_bytes: null argument");
        *h2d_bytes = hostTransfer().h2d;
        *d2h_bytes = hostTransfer().d2h;
    });
}

// The same pipeline with the result left as it crossed the link: bf16. No host thread touches the data.
bfb_status bfb_model_forward_host_bf16(bfb_model* model, const float* h_input, const int64_t* shape, int32_t rank,
                                       uint16_t* h_out16, int64_t* out_shape, int32_t* out_rank) {
    return guarded([&] {
        require(model != nullptr && h_input != nullptr && shape != nullptr && out_shape != nullptr && out_rank != nullptr,
                "model_forward_host_bf16: null argument");
        require(rank >= 1 && rank <= 8, "model_forward_host_bf16: bad rank");
        std::vector<std::size_t> dims(shape, shape + rank);
        std::vector<std::size_t> outDims = model->model->outputShape(dims);
        *out_rank = static_cast<int32_t>(outDims.size());
        for (std::size_t i = 0; i < outDims.size(); ++i) out_shape[i] = static_cast<int64_t>(outDims[i]);
        if (h_out16 == nullptr) return;  // shape query only
        if (!model->model->resultIsBf16Exact()) {
            bfb::fail(BFB_UNSUPPORTED, "model_forward_host_bf16: needs storage bf16 and a pipeline from an embedding to a linear");
        }
        requireDevice();
        std::size_t count = 1;
        for (std::size_t d : dims) count *= d;
        const std::size_t batch = dims[0];
        if (count == 0 || batch == 0) return;
        bfb200::DeviceTensor in(dims);
        BFB_CUDA(cudaMemcpy(in.data(), h_input, count * sizeof(float), cudaMemcpyHostToDevice));
        hostTransfer().h2d = static_cast<int64_t>(count * sizeof(float));
        hostTransfer().d2h = 0;
        std::lock_guard<std::mutex> hostPathLock(hostPathMutex());
        HostPathStreams& st = hostPathStreams();
        const std::size_t perSeqIn = count / batch;
        std::size_t outCount = 1;
        for (std::size_t d : outDims) outCount *= d;
        const std::size_t perSeqOut = outCount / batch;
        const std::size_t seqs = batch >= 16 ? std::max<std::size_t>(1, batch / 8) : step4(batch);
        st.ensureStaging(seqs * perSeqOut * 2);   // only the device slots of the ring are used here
        std::size_t slice = 0;
        for (std::size_t b0 = 0; b0 < batch; b0 += seqs, ++slice) {
            const std::size_t nb = std::min(seqs, batch - b0);
            const int k = static_cast<int>(slice % HostPathStreams::kSlots);
            // the copy that last read this device slot (four slices ago) must have finished
            if (slice >= HostPathStreams::kSlots) BFB_CUDA(cudaEventSynchronize(st.copied[k]));
            std::vector<std::size_t> sliceDims = dims;
            sliceDims[0] = nb;
            bfb200::DeviceTensor view = bfb200::DeviceTensor::borrow(in.data() + b0 * perSeqIn, sliceDims);
            try {
                model->model->forwardBf16(view, st.dev16[k], false, st.compute);
            } catch (...) {
                view.releaseOwnership();
                cudaStreamSynchronize(st.copy);
                throw;
            }
            view.releaseOwnership();
            BFB_CUDA(cudaMemcpyAsync(h_out16 + b0 * perSeqOut, st.dev16[k], nb * perSeqOut * 2, cudaMemcpyDeviceToHost, st.copy));
            BFB_CUDA(cudaEventRecord(st.copied[k], st.copy));
            hostTransfer().d2h += static_cast<int64_t>(nb * perSeqOut * 2);
        }
        BFB_CUDA(cudaStreamSynchronize(st.copy));
    });
}

int64_t bfb_launch_count(int32_t reset) {
    int64_t v = bfb::launchCounter();
    if (reset != 0) bfb::launchCounter() = 0;
    return v;
}

bfb_status bfb_profile_enable(int32_t on) {
    return guarded([&] { bfb::profileEnable(on != 0); });
}

bfb_status bfb_profile_reset(void) {
    return guarded([&] { bfb::profileReset(); });
}

bfb_status bfb_profile_read(int32_t kind, double* milliseconds, int64_t* launches, double* work) {
    return guarded([&] {
        require(kind >= 0 && kind < bfb::kProfKindCount, "profile_read: unknown kind");
        bfb::profileRead(kind, milliseconds, launches, work);
    });
}

bfb_status bfb_synthetic_input(const bfb_op_desc* ops, int32_t n_ops, const int64_t* input_shape, int32_t rank,
                               int64_t batch, uint32_t seed, float* h_out) {
    return guarded([&] {
        require(ops != nullptr && n_ops > 0 && input_shape != nullptr && h_out != nullptr, "synthetic_input: null argument");
        require(rank >= 1 && rank <= 8 && batch >= 0, "synthetic_input: bad rank or batch");
        std::vector<bfb_op_desc> v(ops, ops + n_ops);
        std::vector<int64_t> shape(input_shape, input_shape + rank);
        bfb200::HostTensor t = bfb200::Executor(seed).makeSyntheticInput(v, shape, static_cast<std::size_t>(batch));
        std::memcpy(h_out, t.data.data(), t.data.size() * sizeof(float));
    });
}

// ---- tensor parallel ------------------------------------------------------------------------------------

bfb_status bfb_selftest_bounded_wait(uint64_t limit_ns, int32_t* h_observed, void* stream) {
    return guarded([&] {
        int observed[3] = {0, 0, 0};
        const int code = bfb::selfTestBoundedWait(limit_ns, observed, asStream(stream));
        if (h_observed != nullptr) {
            for (int i = 0; i < 3; ++i) h_observed[i] = observed[i];
        }
        bfb::failOnDeviceStatus(code);
    });
}

bfb_status bfb_pool_fail_after(int64_t nth) {
    return guarded([&] { bfb::poolFailAfter(nth); });
}

bfb_status bfb_selftest_collective_watchdog(int32_t ranks, int32_t skip_rank, int64_t timeout_ms, int32_t* timed_out,
                                            int32_t* sum_ok) {
    return guarded([&] {
        require(ranks >= 1 && ranks <= 16 && skip_rank < ranks && timeout_ms >= 0, "selftest_collective_watchdog: bad arguments");
        bool ok = false;
        const int n = bfb200::watchdogSelfTest(ranks, skip_rank, timeout_ms, &ok);
        if (timed_out != nullptr) *timed_out = n;
        if (sum_ok != nullptr) *sum_ok = ok ? 1 : 0;
    });
}

bfb_status bfb_tp_unique_id(void* h_id_128) {
    return guarded([&] { bfb200::tpUniqueId(h_id_128); });
}

bfb_status bfb_tp_init(const void* h_id_128, int32_t rank, int32_t world) {
    return guarded([&] {
        requireDevice();
        bfb200::tpInit(h_id_128, rank, world);
    });
}

bfb_status bfb_tp_allreduce_sum(void* d_buf, int64_t count, int32_t dtype, void* stream) {
    return guarded([&] { bfb200::tpAllReduceSum(d_buf, count, dtype, stream); });
}

bfb_status bfb_gradients_average(void* const* d_grads, const int64_t* counts, int32_t n_tensors, void* stream) {
    return guarded([&] { bfb200::tpAverageGradients(d_grads, counts, n_tensors, stream); });
}

bfb_status bfb_tp_destroy(void) {
    return guarded([&] { bfb200::tpDestroy(); });
}

}  // extern "C"
