/*
 * bfb200 — C ABI of the B200 (sm_100a) backend for BlackForge's decoder-only forward path.
 *
 * BlackForge has no FFI layer of its own: its boundary is the C++ operator API in namespace
 * blackforge::backend::cuda (DeviceTensor + free functions + Model/Executor). This header is the
 * flat C surface a drop-in for that API binds to; each entry point names the reference interface
 * (path:line inside the BlackForge project) whose work it takes over.
 *
 * Conventions
 *  - Every function returns a bfb_status. On failure bfb_last_error() (per host thread) explains.
 *    BFB_INVALID_ARGUMENT corresponds to the reference's std::invalid_argument, BFB_CUDA_ERROR and
 *    BFB_IO_ERROR to its std::runtime_error. Nothing is launched when arguments are rejected.
 *  - Pointers named d_* are device pointers on the CURRENT device (cudaSetDevice is ambient state,
 *    as in the reference, src/backend/cuda/device_query.cu:34-40); h_* are host pointers.
 *  - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream the reference
 *    uses everywhere).
 *  - Row-major everywhere. A tensor [batch, seq, dim] keeps attention heads contiguous inside dim
 *    (include/blackforge/backend/cuda/fused_attention.hpp:48-57).
 *  - There is no CPU fallback: if no CUDA device/driver is usable the compute entry points fail with
 *    BFB_CUDA_ERROR.
 */
#ifndef BFB200_H
#define BFB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t bfb_status;
enum {
    BFB_OK = 0,
    BFB_INVALID_ARGUMENT = 1, /* shape / rank / range violations */
    BFB_CUDA_ERROR = 2,       /* CUDA runtime or driver failure */
    BFB_TIMEOUT = 3,          /* a bounded device-side wait ran out (kernel unwound cleanly) */
    BFB_UNSUPPORTED = 4,      /* valid request this build has no kernel for */
    BFB_IO_ERROR = 5          /* checkpoint file problems */
};

/* Element formats of device buffers. */
enum { BFB_F32 = 0, BFB_BF16 = 1, BFB_FP8_E4M3 = 2 };

/* sema::DType codes (include/blackforge/sema/dtype.hpp:12-19), used by precision policies. */
enum { BFB_DT_FP8_E4M3 = 0, BFB_DT_FP8_E5M2 = 1, BFB_DT_FP16 = 2, BFB_DT_BF16 = 3, BFB_DT_TF32 = 4, BFB_DT_FP32 = 5 };

/* ir::OpKind (include/blackforge/ir/operation.hpp:11-12), same order. */
enum {
    BFB_OP_LINEAR = 0, BFB_OP_SILU, BFB_OP_RELU, BFB_OP_GELU, BFB_OP_RMSNORM, BFB_OP_SOFTMAX, BFB_OP_EMBEDDING,
    BFB_OP_POSITIONAL_EMBEDDING, BFB_OP_ATTENTION, BFB_OP_FEEDFORWARD, BFB_OP_BIDIRECTIONAL_ATTENTION
};

/* Mirror of ir::Operation (include/blackforge/ir/operation.hpp:23-33). */
typedef struct bfb_op_desc {
    int32_t kind;
    int64_t input;   /* value id of the input */
    int64_t output;  /* value id of the output: the integer in parameter names */
    int64_t linear_out_features;
    int64_t embedding_vocab_size;
    int64_t embedding_dim;
    int64_t positional_max_seq_len;
    int64_t attention_num_heads;
    int64_t feedforward_hidden_dim;
} bfb_op_desc;

/* Mirror of ir::PrecisionPolicy (include/blackforge/ir/module.hpp:44-48); BFB_DT_* codes. */
typedef struct bfb_precision {
    int32_t present; /* 0 = the program has no precision block */
    int32_t storage;
    int32_t compute;
    int32_t accumulate;
} bfb_precision;

/* GEMM epilogues: C = epilogue(alpha * A*B). */
enum {
    BFB_EPI_NONE = 0,
    BFB_EPI_BIAS = 1,          /* + bias[col]                 addBias,          ops_elementwise.cu:158-176 */
    BFB_EPI_BIAS_SILU = 2,     /* silu(. + bias[col])         addBiasSilu,      ops_elementwise.cu:178-193 */
    BFB_EPI_BIAS_RESIDUAL = 3, /* . + bias[col] + residual    addBiasResidual,  ops_elementwise.cu:195-213 */
    BFB_EPI_RESIDUAL = 4       /* . + residual                add,              ops_elementwise.cu:147-156 */
};

/* Layout of the second GEMM operand. */
enum {
    BFB_B_KN = 0, /* B[K,N] row-major: the reference's weight layout (src/backend/cuda/model.cu:172-175) */
    BFB_B_NK = 1  /* B^T[N,K] row-major: produced once by bfb_weight_prepare */
};

/* Unary / binary elementwise selectors for bfb_elementwise. */
enum {
    BFB_EW_ADD = 0,           /* add              ops_elementwise.cu:147-156 */
    BFB_EW_ADD_BIAS = 1,      /* addBias          ops_elementwise.cu:158-176 */
    BFB_EW_ADD_BIAS_SILU = 2, /* addBiasSilu      ops_elementwise.cu:178-193 */
    BFB_EW_ADD_BIAS_RESIDUAL = 3, /* addBiasResidual ops_elementwise.cu:195-213 */
    BFB_EW_SILU = 4,          /* silu             ops_elementwise.cu:215-223 */
    BFB_EW_RELU = 5,          /* relu             ops_elementwise.cu:500-507 */
    BFB_EW_GELU = 6           /* gelu             ops_elementwise.cu:509-515 */
};

const char* bfb_last_error(void);
/* Library version (major*10000 + minor*100 + patch). */
int32_t bfb_version(void);
/* Number of usable CUDA devices; 0 devices is reported as BFB_CUDA_ERROR.
 * Replaces enumerateDevices (src/backend/cuda/device_query.cu:9-32). */
bfb_status bfb_device_count(int32_t* count);
/* Replaces setActiveDevice (src/backend/cuda/device_query.cu:34-40). */
bfb_status bfb_set_device(int32_t index);

/* ---- device memory pool ----------------------------------------------------------------------
 * Replaces devicePoolAcquire / devicePoolRelease (src/backend/cuda/device_pool.cu:29-65): per-device
 * free lists keyed by exact byte size, buffers are never returned to the driver unless trimmed,
 * release never fails loudly. bytes == 0 yields a NULL pointer. */
bfb_status bfb_pool_acquire(size_t bytes, void** d_out);
bfb_status bfb_pool_release(void* d_ptr, size_t bytes);
/* Extension: give cached buffers of the current device back to the driver. */
bfb_status bfb_pool_trim(void);
/* Extension: bytes currently cached / handed out on the current device. */
bfb_status bfb_pool_stats(size_t* cached_bytes, size_t* live_bytes);

/* ---- host <-> device copies (DeviceTensor::fromHost / toHost / clone, device_tensor.cu:68-115) */
bfb_status bfb_copy_h2d(void* d_dst, const void* h_src, size_t bytes, void* stream);
bfb_status bfb_copy_d2h(void* h_dst, const void* d_src, size_t bytes, void* stream);
bfb_status bfb_copy_d2d(void* d_dst, const void* d_src, size_t bytes, void* stream);
bfb_status bfb_memset_zero(void* d_dst, size_t bytes, void* stream);
bfb_status bfb_stream_synchronize(void* stream);

/* ---- gather + positions -----------------------------------------------------------------------
 * out[t, :] = table[lround(ids[t]), :] (+ pos[(pos_offset + t % seq), :] when d_pos != NULL).
 * Replaces embeddingLookup / embeddingLookupPreValidated (ops_elementwise.cu:372-441, kernel :305-326)
 * fused with addPositionalEmbedding / addPositionalEmbeddingAt (ops_elementwise.cu:443-498).
 * ids are float32 holding integers. Rows whose id is outside [0, vocab) are zero-filled, as the
 * reference kernel does, and *d_oob_count (optional, int32 on device) is incremented per bad row:
 * the host layer turns a non-zero count into BFB_INVALID_ARGUMENT without a D2H copy of the ids.
 * out_dtype: BFB_F32 (bit-exact with the reference) or BFB_BF16 (storage bf16: rounded once). */
bfb_status bfb_embed_pos(const float* d_ids, const float* d_table, const float* d_pos, void* d_out, int32_t out_dtype,
                         int64_t batch, int64_t seq, int64_t vocab, int64_t dim, int64_t max_seq, int64_t pos_offset,
                         int32_t* d_oob_count, void* stream);

/* out = in + pos[(pos_offset + s), :] on an existing [batch, seq, dim] f32 tensor.
 * Replaces addPositionalEmbedding(+At) (ops_elementwise.cu:443-498). */
bfb_status bfb_add_positional(const float* d_in, const float* d_pos, float* d_out, int64_t batch, int64_t seq,
                              int64_t dim, int64_t max_seq, int64_t pos_offset, void* stream);

/* ---- rmsnorm: y = x / sqrt(mean(x^2) + eps), no gamma ------------------------------------------
 * Replaces rmsnorm (ops_elementwise.cu:355-370, kernel :102-137); eps is an argument, the reference's
 * value is 1e-6. x_dtype / out_dtype in {BFB_F32, BFB_BF16}; the row is read once. */
bfb_status bfb_rmsnorm(const void* d_x, int32_t x_dtype, void* d_out, int32_t out_dtype, int64_t rows, int64_t dim,
                       float eps, void* stream);

/* Row softmax on f32 (softmax, ops_elementwise.cu:225-243, kernel :249-300). */
bfb_status bfb_softmax(const float* d_x, float* d_out, int64_t rows, int64_t cols, void* stream);

/* f32 elementwise ops (BFB_EW_*). `cols` is the bias length for the bias forms; d_b is the second
 * operand (add) or the bias; d_c the residual of BFB_EW_ADD_BIAS_RESIDUAL. */
bfb_status bfb_elementwise(int32_t op, const float* d_a, const float* d_b, const float* d_c, float* d_out, int64_t n,
                           int64_t cols, void* stream);

/* ---- format conversion -------------------------------------------------------------------------
 * out = convert(in * scale). scale comes from *d_scale when non-NULL, else `scale`.
 * Replaces floatToBf16Kernel (ops_tensorcore.cu:21-26) and adds the fp8 e4m3 (saturating) forms. */
bfb_status bfb_cast(const void* d_in, int32_t in_dtype, void* d_out, int32_t out_dtype, int64_t n, float scale,
                    const float* d_scale, void* stream);
/* *d_amax = max(*d_amax, max|in|) (f32 word on device; zero it first for a fresh maximum).
 * No counterpart in the reference (its fp8 path is declared only, README.md:68). */
bfb_status bfb_amax(const void* d_in, int32_t in_dtype, int64_t n, float* d_amax, void* stream);
/* d_scales[0] = 448 / amax (1 when amax == 0), d_scales[1] = 1 / d_scales[0]; reads *d_amax on device. */
bfb_status bfb_fp8_scale_from_amax(const float* d_amax, float* d_scales, void* stream);
/* Per-tensor e4m3 quantisation of an activation in one call: d_scales[0] = 448 / max|in| (1 for an all-zero
 * tensor), d_scales[1] = 1 / d_scales[0], d_scales[2] = d_scales[1] * *d_weight_inverse (1 when NULL: the alpha
 * of the following GEMM); d_out = e4m3(in * d_scales[0]), saturating. in_dtype BFB_F32 or BFB_BF16. The partial
 * maxima (one float per 8192 elements) go through scratch memory taken from the device pool for the duration
 * of the call. Deterministic (no atomics). No counterpart in the reference (fp8 is declared only). */
bfb_status bfb_quantize_e4m3(const void* d_in, int32_t in_dtype, int64_t n, void* d_out, float* d_scales,
                             const float* d_weight_inverse, void* stream);
/* rmsnorm (ops_elementwise.cu:102-137, no weights) of bf16 rows and the per-tensor e4m3 quantisation of the result
 * in one call, without storing the normalised rows: d_out = e4m3(bf16(x * r_row) * d_scales[0]) with
 * r_row = 1 / sqrt(mean(x_row^2) + eps) and d_scales as for bfb_quantize_e4m3 (the maximum is taken over the
 * normalised bf16 values). Two passes over x instead of a norm, a maximum pass and a conversion. Scratch
 * (one float per row and per block) comes from the device pool for the duration of the call. */
bfb_status bfb_rmsnorm_quantize_e4m3(const void* d_x, int64_t rows, int64_t dim, float eps, void* d_out, float* d_scales,
                                     const float* d_weight_inverse, void* stream);
/* The same result when the GEMM that wrote x also left its row statistics (d_out_sum_sq and d_out_max_abs of
 * bfb_gemm_rmsnorm, both [parts][rows] with parts = ceil(dim / 128)): the first pass (1 / rms per row, the largest
 * normalised magnitude) reads those figures instead of x, so x is read once. The sums are added in part order, so a
 * row's 1 / rms may differ in its last bit from the plain call's. No reference counterpart. */
bfb_status bfb_rmsnorm_quantize_e4m3_from_stats(const void* d_x, int64_t rows, int64_t dim, float eps, void* d_out,
                                                float* d_scales, const float* d_weight_inverse, const float* d_sum_sq_parts,
                                                const float* d_max_parts, int32_t parts, void* stream);
/* Same operation and results as bfb_quantize_e4m3, for callers that must not allocate device memory while
 * they run: a host engine that gave the whole GPU to its own arena at start-up, or a latency-critical
 * serving loop where a trip into the device allocator can stall every stream. This entry point has no
 * counterpart in the reference. It calls no allocator at all (not cudaMalloc, not the device pool): the partial
 * maxima go to a fixed 256 KiB array inside the library, which every GPU that uses the library holds until the
 * process exits. Limits and rules:
 *  - n <= 536 870 912 elements (65 536 partial maxima of 8192 elements each); larger n is refused with
 *    BFB_INVALID_ARGUMENT and nothing is launched.
 *  - The first call on each device looks up the array's device address (once, with that device current), and if
 *    the CUDA runtime loads modules lazily it is also the call that loads this library's kernels onto the device,
 *    which the driver may back with memory of its own. So make one warm-up call per device at start-up, before the
 *    phase in which nothing may allocate and before starting any stream capture.
 *  - The looked-up address is kept for the life of the process: after cudaDeviceReset() on a device this entry
 *    point must not be used on it again.
 *  - All calls on a device share the one array. It keeps the previous call's values, which is harmless because
 *    each call overwrites every slot it later reads; but two calls whose kernels overlap on the GPU (different
 *    streams) race on it. Keep calls to this entry point on one stream, or order them yourself. */
bfb_status bfb_quantize_e4m3_static(const void* d_in, int32_t in_dtype, int64_t n, void* d_out, float* d_scales,
                                    const float* d_weight_inverse, void* stream);
/* Weight preparation, done once per weight: W[K,N] f32 (reference layout) -> W^T[N,K] in out_dtype,
 * multiplied by scale (*d_scale when non-NULL). Takes over the per-call weight cast of
 * matmulBf16 (ops_tensorcore.cu:316-317) and the cached-weight variant (:98-131). */
bfb_status bfb_weight_prepare(const float* d_w, void* d_out, int32_t out_dtype, int64_t k, int64_t n, float scale,
                              const float* d_scale, void* stream);

/* ---- GEMM: C[M,N] = epilogue(alpha * A[M,K] * B) ------------------------------------------------
 * Replaces matmul (cublasSgemm, ops_gemm.cu:64-93), matmulBf16 / bf16Gemm (cublasLtMatmul,
 * ops_tensorcore.cu:293-327), linear / linearBf16 (+ addBias) and the fused bias/silu/residual
 * passes listed at BFB_EPI_*.
 *  ab_dtype  BFB_F32      fp32 FFMA kernel, fp32 accumulate in k order (the exactness path)
 *            BFB_BF16     tcgen05 kind::f16 on TMA-fed tiles, fp32 accumulate in TMEM
 *            BFB_FP8_E4M3 tcgen05 kind::f8f6f4 (B must be BFB_B_NK), fp32 accumulate
 *  b_layout  BFB_B_KN or BFB_B_NK
 *  c_dtype   BFB_F32 or BFB_BF16; bias is f32[N]; residual has c_dtype and shape [M,N]
 *  alpha     multiplies the accumulator; *d_alpha (device f32) is used instead when non-NULL
 *  round_c_bf16  non-zero: round an f32 result to bf16 precision before storing (`storage bf16`)
 * Shapes the tensor-core kernel cannot take (K or N not a multiple of 8 for bf16 / 16 for fp8, or
 * misaligned pointers) run a CUDA-core kernel that rounds operands to ab_dtype: same arithmetic
 * contract, no alignment demands. d_status (optional int32 on device) receives a non-zero code if a
 * bounded wait inside the tensor-core kernel ran out. */
bfb_status bfb_gemm(const void* d_a, const void* d_b, void* d_c, int64_t m, int64_t n, int64_t k, int32_t ab_dtype,
                    int32_t b_layout, int32_t c_dtype, int32_t epilogue, const float* d_bias, const void* d_residual,
                    float alpha, const float* d_alpha, int32_t round_c_bf16, int32_t* d_status, void* stream);

/* rmsnorm fused into the adjacent linear (no reference counterpart as one call: it stands for
 * rmsnorm, src/backend/cuda/ops_elementwise.cu:102-137, followed by linearBf16, ops_tensorcore.cu:329-387).
 * An rmsnorm without weights scales each row by 1 / sqrt(mean(x^2) + eps), which commutes with the matrix
 * product: C[i,:] = epilogue(A[i,:] W^T / sqrt(s_i / k + eps)) with A the UN-normalised activation and s_i the
 * sum over p < row_sum_sq_parts of d_row_sum_sq[p * m + i]. bfb_row_sum_squares computes s (one part); a
 * producing GEMM can also deliver it: with d_out_sum_sq set, the sums of squares of every stored row of C are
 * written there per 128-column part, d_out_sum_sq[p * m + i] for p < ceil(n / 128) (no atomics: the same bits on
 * every run); d_out_max_abs, same layout, receives the largest magnitude of each part instead (the per-tensor
 * maximum an e4m3 quantisation of C needs, without another pass over C). d_row_sum_sq, d_out_sum_sq and
 * d_out_max_abs may be NULL. Weights are [n,k] (BFB_B_NK); needs the tensor-core
 * formats and 16-byte aligned rows, else BFB_UNSUPPORTED. */
bfb_status bfb_row_sum_squares(const void* d_x, int32_t dtype, float* d_out, int64_t rows, int64_t dim, void* stream);
bfb_status bfb_gemm_rmsnorm(const void* d_a, const void* d_w, void* d_c, int64_t m, int64_t n, int64_t k,
                            int32_t ab_dtype, int32_t c_dtype, int32_t epilogue, const float* d_bias,
                            const void* d_residual, const float* d_row_sum_sq, int32_t row_sum_sq_parts, float eps,
                            float* d_out_sum_sq, float* d_out_max_abs, int32_t* d_status, void* stream);
/* The linear of a generation step (few rows, all of W): C[m,n] = epilogue(alpha * A[m,k] W^T [* row scale]) for
 * 1 <= m <= 128, W [n,k], bf16 or e4m3 operands. It stands for the same reference calls as bfb_gemm
 * (matmulBf16 / linearBf16, ops_tensorcore.cu:308-387) in the shape Model::forwardIncremental produces. The weight
 * rows take the MMA's M side and K is split over CTAs so that every SM streams part of W; the partial products are
 * added in a fixed order (same bits on every run). Row statistics as for bfb_gemm_rmsnorm (d_row_sum_sq and
 * d_out_sum_sq may be NULL). */
bfb_status bfb_gemm_few_rows(const void* d_a, const void* d_w, void* d_c, int64_t m, int64_t n, int64_t k, int32_t ab_dtype,
                             int32_t c_dtype, int32_t epilogue, const float* d_bias, const void* d_residual, float alpha,
                             const float* d_row_sum_sq, int32_t row_sum_sq_parts, float eps, float* d_out_sum_sq,
                             int32_t* d_status, void* stream);
/* A * B^T on f32: a[M,K], b[N,K] (matmulTransposeB, ops_gemm.cu:95-110, kernel :20-34). */
bfb_status bfb_matmul_transpose_b(const float* d_a, const float* d_b, float* d_c, int64_t m, int64_t n, int64_t k,
                                  void* stream);

/* Gradients of C = A B with bf16 operands (matmulBf16Backward, src/backend/cuda/ops_tensorcore.cu:389-417):
 * d_da[M,K] = grad[M,N] * b^T and d_db[K,N] = a^T * grad from fp32 a [M,K], b [K,N], grad [M,N]; operands are
 * rounded to bf16, accumulation and results are fp32. A zero dimension zero-fills both results, as there.
 * The bf16 copies live in pool buffers that go back to the pool when the call returns, while the kernels may
 * still be running on `stream`: as with the reference's pool (which knows no streams either), a buffer handed
 * out again is safe for work queued on the SAME stream; a caller that uses several streams synchronises first. */
bfb_status bfb_matmul_bf16_backward(const float* d_a, const float* d_b, const float* d_grad, float* d_da, float* d_db,
                                    int64_t m, int64_t k, int64_t n, void* stream);

/* ---- causal attention core ---------------------------------------------------------------------
 * Replaces fusedAttentionForward (src/backend/cuda/fused_attention.cu:315-341, kernel :60-157).
 * q [batch, new_len, H*D] with row stride ld_q elements; k, v [batch, total_len, H*D] with strides
 * ld_k, ld_v (strides let Q, K, V live interleaved in one [tokens, 3*dim] projection output).
 * Query row i attends keys j <= old_len + i. out [batch, new_len, H*D] (row stride ld_o); optional
 * d_m, d_l f32 [batch, H, new_len] receive the online-softmax statistics (row max of scaled scores,
 * sum of exp) as the reference returns them.
 *  dtype BFB_BF16: tcgen05 flash kernel for D == 128 (TMA tiles, fp32 online softmax in registers,
 *                  no materialised scores); other D run the CUDA-core kernel on bf16 data
 *  dtype BFB_F32 : CUDA-core online-softmax kernel, D <= 256 (the reference's limit, :305-311)
 * out has the same dtype as the inputs. causal == 0 gives the bidirectional form. */
bfb_status bfb_attention_fwd(const void* d_q, const void* d_k, const void* d_v, void* d_out, float* d_m, float* d_l,
                             int32_t dtype, int64_t batch, int64_t new_len, int64_t total_len, int64_t num_heads,
                             int64_t head_dim, int64_t ld_q, int64_t ld_k, int64_t ld_v, int64_t ld_o, float scale,
                             int64_t old_len, int32_t causal, int32_t* d_status, void* stream);

/* The causal attention core on bf16 data with head_dim 128 (the tensor-core kernel), which also reports the largest
 * magnitude of the output it stores per 32 rows of a (batch, head): d_maxima[((b * heads + h) * ceil(new_len / 128)
 * + row / 128) * 4 + (row % 128) / 32], maxima_count floats, all written. A per-tensor e4m3 quantisation of the
 * output then needs no pass of its own to find its scale. BFB_UNSUPPORTED where the tensor-core kernel does not
 * apply (one query row, unaligned strides). No reference counterpart (fp8 is declared only). */
bfb_status bfb_attention_fwd_maxima(const void* d_q, const void* d_k, const void* d_v, void* d_out, float* d_maxima,
                                    int64_t maxima_count, int64_t batch, int64_t new_len, int64_t total_len, int64_t num_heads,
                                    int64_t ld_q, int64_t ld_k, int64_t ld_v, int64_t ld_o, float scale, int64_t old_len,
                                    int32_t* d_status, void* stream);

/* Backward of the attention core. Replaces cuda::fusedAttentionBackward
 * (src/backend/cuda/fused_attention.cu:343-380; kernels computeDKernel :166-190 and
 * tiledFusedAttentionBackwardKernel :200-303). d_dout, d_q, d_out are [batch, new_len, ld_in] and d_k, d_v
 * [batch, total_len, ld_kv], all of `dtype` (BFB_F32 or BFB_BF16); d_m, d_l are the forward's row statistics
 * [batch, num_heads, new_len]. Results are fp32: d_dq [batch, new_len, ld_grad_q], d_dk and d_dv
 * [batch, total_len, ld_grad_kv] (every element written: keys no query sees get zero). d_scratch holds
 * 2 * batch * num_heads * new_len floats. head_dim 128 in bf16 runs on the tensor cores (operands rounded to
 * bf16, fp32 accumulation); other shapes on a CUDA-core kernel that keeps the reference's arithmetic. */
bfb_status bfb_attention_bwd(const void* d_dout, const void* d_q, const void* d_k, const void* d_v, const void* d_out,
                             const float* d_m, const float* d_l, float* d_dq, float* d_dk, float* d_dv, float* d_scratch,
                             int32_t dtype, int64_t batch, int64_t new_len, int64_t total_len, int64_t num_heads,
                             int64_t head_dim, int64_t ld_in, int64_t ld_kv, int64_t ld_grad_q, int64_t ld_grad_kv,
                             float scale, int64_t old_len, int32_t causal, int32_t* d_status, void* stream);

/* ---- model: the IR executor's device side ------------------------------------------------------
 * Replaces cuda::Model (src/backend/cuda/model.cu:139-306: constructor, forward, parameters),
 * cuda::Executor::run / makeSyntheticInput (src/backend/cuda/executor.cu:26-132) and
 * cuda::loadCheckpoint / saveCheckpoint (src/backend/cuda/checkpoint.cu:60-130).
 * A model is built from the pipeline of an ir::ModelIR; default parameters reproduce the
 * reference's seeded uniform(-0.1, 0.1) initialisation so that `run` without a checkpoint gives the
 * reference's numbers. */
typedef struct bfb_model bfb_model;

/* input_last_dim: literal size of the input value's last dimension (0 if symbolic). */
bfb_status bfb_model_create(const bfb_op_desc* ops, int32_t n_ops, int64_t input_last_dim, uint32_t seed,
                            const bfb_precision* precision, bfb_model** out);
void bfb_model_destroy(bfb_model* model);
/* Skip the default random initialisation (parameters start at zero) — for models that are always
 * loaded from a checkpoint; call before any parameter access. */
bfb_status bfb_model_create_uninitialised(const bfb_op_desc* ops, int32_t n_ops, int64_t input_last_dim,
                                          const bfb_precision* precision, bfb_model** out);
/* Tensor parallelism over `world` ranks (heads and feed-forward columns sharded, logits columns
 * sharded); the all-reduce is done by the communicator installed with bfb_tp_init. world == 1 is
 * the default. Must be called before parameters are set. */
bfb_status bfb_model_set_tensor_parallel(bfb_model* model, int32_t rank, int32_t world);
/* Overlap of the all-reduces with compute in a tensor-parallel prompt pass (the reference has no tensor
 * parallelism; its data-parallel runner averages on the host, multi_gpu_train_runner.cu:275-297): the batch is
 * cut into `groups` groups of sequences, and while one group's rows are summed over the ranks on a second stream
 * the next group computes. The CTA-pair GEMMs of such a pass draw their tiles from a device counter, so that pairs
 * kept waiting by the collective's CTAs leave no tail; the persistent kernels can also leave `reserved_sms` SMs
 * free altogether. groups == 1 runs everything on the caller's stream. Defaults 2 and 0 (environment BFB_TP_CHUNKS,
 * BFB_TP_RESERVE_SMS). May be changed between forward calls; results do not depend on it. */
bfb_status bfb_model_set_tensor_parallel_overlap(bfb_model* model, int32_t groups, int32_t reserved_sms);

/* Process-wide mode of the persistent tensor-core kernels for callers that run a kernel of their own beside them
 * on another stream: dynamic_tiles != 0 makes the CTA-pair GEMM draw tiles from a device counter instead of the
 * static round-robin (same tiles, same values); reserved_sms sizes the persistent grids for that many fewer SMs.
 * Both default to 0. A tensor-parallel model sets and restores them around its own passes. */
bfb_status bfb_set_shared_sm_mode(int32_t dynamic_tiles, int32_t reserved_sms);

int32_t bfb_model_param_count(const bfb_model* model);
const char* bfb_model_param_name(const bfb_model* model, int32_t index);
int32_t bfb_model_param_rank(const bfb_model* model, int32_t index);
void bfb_model_param_shape(const bfb_model* model, int32_t index, int64_t* shape_out);
/* Full (unsharded) f32 values, host side. */
bfb_status bfb_model_param_set(bfb_model* model, int32_t index, const float* h_values);
bfb_status bfb_model_param_get(bfb_model* model, int32_t index, float* h_values);

/* Synthetic weights for benchmarks, generated on the device: parameter `index` becomes seeded N(0, sigma). A value
 * depends only on (seed, position in the full tensor), so every tensor-parallel rank fills just its slice and
 * all ranks still agree. No counterpart in the reference (its Executor draws uniform weights on the host). */
bfb_status bfb_model_param_fill_normal(bfb_model* model, int32_t index, uint64_t seed, float sigma);
/* Inference-only memory saver: convert the weights now and drop the fp32 copies of the GEMM weights (the
 * reference keeps fp32 values and gradients for every parameter, model.cu:139-250). Those parameters can no
 * longer be read, set or saved afterwards. No effect on an fp32-compute model. */
bfb_status bfb_model_release_master_weights(bfb_model* model);

/* BFCKPT1 (include/blackforge/backend/cpu/checkpoint.hpp:15-24). Load matches by name and shape; an
 * unknown name, a shape mismatch, a bad magic or a truncated file give BFB_IO_ERROR. */
bfb_status bfb_model_load_checkpoint(bfb_model* model, const char* path);
bfb_status bfb_model_save_checkpoint(bfb_model* model, const char* path);

/* cpu::runBenchmark (include/blackforge/backend/cpu/benchmark.hpp:14-62) on the device, on the caller's input:
 * `warmup` discarded passes, `measured` timed ones (0 gives BFB_INVALID_ARGUMENT, as the reference throws). mean_ms is
 * device time between CUDA events on the forward's stream; per_op[i] is the mean device time of pipeline operation
 * i inside the full pass, the per-operation breakdown the reference's header says its CUDA side lacks
 * (benchmark.hpp:34-43). An operation fused into its predecessor reports 0. estimated_memory_bytes is the
 * reference's estimate: 4 bytes per element of the input, every operation's output and every parameter. At most
 * per_op_capacity entries are written; op_count is the pipeline's length. */
typedef struct bfb_op_benchmark {
    char name[32];
    int32_t index;
    double mean_ms;
} bfb_op_benchmark;
typedef struct bfb_benchmark_result {
    int64_t warmup_iterations;
    int64_t measured_iterations;
    double mean_ms;
    double samples_per_second;
    uint64_t estimated_memory_bytes;
    int32_t op_count;
} bfb_benchmark_result;
bfb_status bfb_model_benchmark(bfb_model* model, const float* d_input, const int64_t* shape, int32_t rank, int64_t warmup,
                               int64_t measured, bfb_benchmark_result* out, bfb_op_benchmark* per_op,
                               int32_t per_op_capacity, void* stream);

/* The same load with its figures. The reference (src/backend/cuda/checkpoint.cu:82-130) reads each tensor whole
 * into a host vector and uploads it synchronously; this loader reads the headers first, checks every name and
 * shape, then streams whole rows through a few pinned buffers of about chunk_bytes (0: 4 MiB), filled by up to four
 * reader threads, while earlier rows upload, and a tensor-parallel rank reads only the rows it holds of row-sharded tensors (column-sharded ones are
 * read in full rows and sliced by the copy). bfb_model_load_checkpoint is this call without the figures. */
typedef struct bfb_checkpoint_load_stats {
    int64_t tensors;
    uint64_t file_bytes;     /* fp32 payload of the file */
    uint64_t read_bytes;     /* read from the file by this rank */
    uint64_t uploaded_bytes; /* sent to the device */
    double seconds;
    int32_t cache_hit;       /* bfb_model_load_checkpoint_cached: the converted weights came from the cache file */
    uint64_t cache_bytes;    /* read from (hit) or written to (miss) the cache file */
} bfb_checkpoint_load_stats;
bfb_status bfb_model_load_checkpoint_streaming(bfb_model* model, const char* path, uint64_t chunk_bytes,
                                               bfb_checkpoint_load_stats* stats);

/* The streaming load with a cache of the CONVERTED GEMM weights (bf16 or e4m3, transposed, with their scales) beside
 * the checkpoint, `<path>.bfb200cache.<format>.tp<rank>of<world>`: written after the first load and read instead of
 * the fp32 GEMM weights on later ones while the checkpoint's size and modification time and the model's structure are
 * unchanged. A hit reads half (bf16) or a quarter (e4m3) of the bytes, skips the conversion pass and never creates the
 * fp32 copies of the GEMM weights (as after bfb_model_release_master_weights they can then not be read, set or
 * saved). A cache that cannot be written is not an error. An fp32-compute model loads as bfb_model_load_checkpoint. */
bfb_status bfb_model_load_checkpoint_cached(bfb_model* model, const char* path, uint64_t chunk_bytes,
                                            bfb_checkpoint_load_stats* stats);

/* Header pass over a BFCKPT1 file, no device needed: entry `index` (name copied into name_buf, up to 8 dims, the
 * byte offset and size of its fp32 data) and the number of entries. index == -1 only counts. The whole file's
 * extent is checked: a truncated or corrupt file gives BFB_IO_ERROR. */
bfb_status bfb_checkpoint_index(const char* path, int32_t index, char* name_buf, int32_t name_capacity, int32_t* rank,
                                int64_t* dims8, uint64_t* data_offset, uint64_t* data_bytes, int32_t* count);

/* forward on device buffers: d_input f32 with `rank` dims (token ids as float for a model that starts
 * with an embedding). The result is acquired from the pool (f32); release it with bfb_pool_release
 * (bytes = 4 * product(out_shape)). input_range_trusted != 0 skips the id range check
 * (Model::forward(input, inputRangeTrusted), model.cu:252). */
bfb_status bfb_model_forward(bfb_model* model, const float* d_input, const int64_t* shape, int32_t rank,
                             int32_t input_range_trusted, float** d_out, int64_t* out_shape, int32_t* out_rank,
                             void* stream);
/* Autoregressive generation (Model::forwardIncremental / resetGenerationState, model.cu:385-431; caller
 * runGenerate, src/main.cpp:524-627). d_new_ids holds the ids of the NEW positions only, [batch, new_len] as f32;
 * the result (pool memory, f32, release with bfb_pool_release) is their output, equal to what bfb_model_forward
 * gives for those positions on the whole sequence so far. Keys and values of earlier positions stay in per-layer
 * caches; the batch size is fixed by the first call after a reset. Where the reference re-copies the whole cache
 * for every token (concatSeq, ops_transformer.cu:159-167), the bf16 / e4m3 routes keep preallocated bf16 caches
 * sized for the positional table and append in place. */
bfb_status bfb_model_forward_incremental(bfb_model* model, const float* d_new_ids, const int64_t* shape, int32_t rank,
                                         int32_t input_range_trusted, float** d_out, int64_t* out_shape,
                                         int32_t* out_rank, void* stream);
bfb_status bfb_model_reset_generation(bfb_model* model);
bfb_status bfb_model_generation_position(bfb_model* model, int64_t* position);
/* The `blackforge run` path (src/main.cpp:356-388): host ids in, host logits out, synchronous.
 * h_out must hold product(out_shape) floats; call once with h_out == NULL to learn the shape.
 * Host threads may call the host-buffer entry points on one device concurrently: the calls are serialised per
 * device (they share the library's copy streams and staging buffers). */
bfb_status bfb_model_forward_host(bfb_model* model, const float* h_input, const int64_t* shape, int32_t rank,
                                  float* h_out, int64_t* out_shape, int32_t* out_rank);
/* The same call for a host that takes the logits as bf16 (no reference counterpart: its tensors are fp32). Needs
 * `storage bf16` and a pipeline from an embedding to a final linear, where every logit IS a bf16 number, so
 * h_out16[i] holds the upper 16 bits of the fp32 word bfb_model_forward_host would deliver. Half the bytes over the
 * link and into host memory, and no host thread touches them: what to use when several GPUs return logits to one
 * host, whose memory bandwidth is then the limit. BFB_UNSUPPORTED for other models. */
bfb_status bfb_model_forward_host_bf16(bfb_model* model, const float* h_input, const int64_t* shape, int32_t rank,
                                       uint16_t* h_out16, int64_t* out_shape, int32_t* out_rank);
/* Bytes the calling thread's most recent bfb_model_forward_host moved over the host link: ids host to device,
 * result device to host. Under `storage bf16` part of the result travels as 2-byte bf16 and is widened to the
 * caller's fp32 words by host threads, so d2h can be below 4 * product(out_shape).
 * No reference counterpart: its run path does not report transfers. */
bfb_status bfb_host_transfer_bytes(int64_t* h2d_bytes, int64_t* d2h_bytes);
/* The host half of that path on its own (no device needed): h_dst[i] = the fp32 value of bf16 h_src[i], exact,
 * with `threads` host threads and streaming stores. No reference counterpart. */
bfb_status bfb_host_widen_bf16(const uint16_t* h_src, float* h_dst, int64_t count, int32_t threads);
/* Number of kernels this library launched on the calling thread since the counter was last reset. */
int64_t bfb_launch_count(int32_t reset);

/* Per-kernel device timing with CUDA events on the launching stream — the per-operation breakdown
 * the reference's benchmark only has for its CPU backend (include/blackforge/backend/cpu/benchmark.hpp:34-43).
 * Off by default; state is per host thread. `work` is the algorithmic FLOPs (GEMM, attention) or bytes
 * (the rest) of the launches booked under a kind. Reading synchronises on the recorded events. */
enum { BFB_PROF_GEMM_TC = 0, BFB_PROF_ATTENTION_TC = 1, BFB_PROF_RMSNORM = 2, BFB_PROF_EMBED = 3, BFB_PROF_CAST = 4 };
bfb_status bfb_profile_enable(int32_t on);
bfb_status bfb_profile_reset(void);
bfb_status bfb_profile_read(int32_t kind, double* milliseconds, int64_t* launches, double* work);

/* Executor::makeSyntheticInput (executor.cu:26-42): seeded ids/values, host side. */
bfb_status bfb_synthetic_input(const bfb_op_desc* ops, int32_t n_ops, const int64_t* input_shape, int32_t rank,
                               int64_t batch, uint32_t seed, float* h_out);

/* ---- failure paths, exercised without harming a device --------------------------------------------
 * The reference turns every failed CUDA / cuBLAS call into std::runtime_error
 * (include/blackforge/backend/cuda/cuda_check.hpp:14-53) and has no waits that can time out. This library's
 * tensor-core kernels wait on barriers with a time limit and report through a status word, its device pool can
 * run out, and its collectives can lose a rank; these entry points let a test take each of those paths on purpose.
 *
 * bfb_selftest_bounded_wait: launches a one-CTA kernel in which one role waits on a barrier nobody arrives on,
 * through the same bounded wait the kernels use but with `limit_ns` (1 us .. 1 s) as its limit; it gives up, flags
 * the other role (which then leaves long before its own, ordinary limit), the CTA frees its tensor memory and
 * returns. Nothing traps and the context stays usable. Returns BFB_TIMEOUT, as Model::forward does for a kernel
 * whose wait ran out (BFB_OK would mean the wait did not expire). h_observed (3 ints, may be null) receives
 * {first wait succeeded, second wait succeeded, microseconds the second role waited}.
 * bfb_pool_fail_after: host-only fault injection; the nth bfb_pool_acquire / internal pool acquisition from now on
 * (1 = the next) fails with BFB_CUDA_ERROR as an exhausted device would; 0 disarms. One shot.
 * bfb_selftest_collective_watchdog: host only, no device. `ranks` threads run a stand-in all-reduce of host values
 * guarded by the watchdog that also guards the tensor-parallel step (poll, look for an asynchronous error, abort at
 * the deadline); rank `skip_rank` never joins (-1: all join). *timed_out = ranks that gave up and aborted,
 * *sum_ok = 1 when every rank that completed saw the right sum. */
bfb_status bfb_selftest_bounded_wait(uint64_t limit_ns, int32_t* h_observed, void* stream);
bfb_status bfb_pool_fail_after(int64_t nth);
bfb_status bfb_selftest_collective_watchdog(int32_t ranks, int32_t skip_rank, int64_t timeout_ms, int32_t* timed_out,
                                            int32_t* sum_ok);

/* ---- tensor-parallel communicator (NCCL over NVLink) -------------------------------------------
 * No counterpart in the reference (its only multi-GPU code is host-staged gradient averaging,
 * src/backend/cuda/multi_gpu_train_runner.cu:275-297). unique_id is the 128-byte ncclUniqueId made
 * by rank 0 with bfb_tp_unique_id and distributed by the launcher. */
bfb_status bfb_tp_unique_id(void* h_id_128);
bfb_status bfb_tp_init(const void* h_id_128, int32_t rank, int32_t world);
bfb_status bfb_tp_allreduce_sum(void* d_buf, int64_t count, int32_t dtype, void* stream);
/* In-place average over all ranks of n_tensors fp32 gradient buffers (d_grads[i] holds counts[i] elements; both
 * tables are host arrays), one grouped NCCL all-reduce on `stream`. Replaces the host-staged gradient average of the
 * data-parallel train runner (src/backend/cuda/multi_gpu_train_runner.cu:275-297: every replica's gradient copied to
 * the host, added, scaled by 1/replicas and copied back to every replica). */
bfb_status bfb_gradients_average(void* const* d_grads, const int64_t* counts, int32_t n_tensors, void* stream);
bfb_status bfb_tp_destroy(void);

#ifdef __cplusplus
}
#endif
#endif /* BFB200_H */
