/*
 * ruda_b200.h — C ABI of libruda_b200.so, the NVIDIA B200 (sm_100a) backend for the dense-transformer
 * hot path of rust-ascend.
 *
 * Every entry point names the reference interface it stands in for (file:line inside the
 * rust-ascend repository).  A Rust FFI crate binds these symbols one to one; the signatures use only
 * plain pointers, integers and the POD structs below.
 *
 * Conventions (kept from the reference):
 *   - every function returns an rb_status; 0 is success.  The message of the last failure on the
 *     calling thread is returned by rb_last_error().  Status codes mirror the variants of
 *     CannError (rust-ascend-driver/src/lib.rs:18-40); validation failures are RB_INVALID_TENSOR.
 *   - one context per process and device (rust-ascend-driver/src/tensor/runtime/mod.rs:424-435).
 *   - launches are enqueue-only on the context's stream; a failed launch is pushed on a sticky list
 *     that the next rb_read / rb_sync reports as RB_SERVER_UNHEALTHY (runtime/mod.rs:645-661).
 *     rb_options.synchronous = 1 restores the reference's launch-then-synchronise behaviour.
 *   - tensors must be contiguous row-major unless a function says otherwise; outputs may not overlap
 *     inputs (rust-ascend-driver/src/tensor/runtime/worker.rs:418-453).
 *   - there is no CPU fallback: an unsupported dtype, layout or shape is an error (src/backend.rs:43-45).
 */
#ifndef RUDA_B200_H
#define RUDA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define RB_API
#else
#define RB_API __attribute__((visibility("default")))
#endif

/* CannError variants, rust-ascend-driver/src/lib.rs:18-40. */
typedef enum rb_status {
    RB_OK = 0,
    RB_LIBRARY = 1,          /* CannError::Library: a shared library could not be loaded        */
    RB_SYMBOL = 2,           /* CannError::Symbol                                               */
    RB_STATUS = 3,           /* CannError::Status{operation,code}: a CUDA / NCCL call failed    */
    RB_INVALID_DEVICE = 4,   /* CannError::InvalidDevice                                        */
    RB_INVALID_TENSOR = 5,   /* CannError::InvalidTensor(message)                               */
    RB_NULL_HANDLE = 6,      /* CannError::NullHandle                                           */
    RB_COMPLETION = 7,       /* CannError::Completion{operation,launch_code,sync_code}          */
    RB_SERVER_UNHEALTHY = 8  /* ServerError::ServerUnhealthy{errors}, runtime/mod.rs:645-661    */
} rb_status;

/* ruda_core::tensor::DType values used on this path (runtime/hccl.rs:97-111 lists the same set). */
typedef enum rb_dtype { RB_F32 = 0, RB_F16 = 1, RB_BF16 = 2, RB_I32 = 3, RB_I64 = 4, RB_U8 = 5 } rb_dtype;

/* Transpose, rust-ascend-driver/src/tensor/deepgemm/plan.rs. */
typedef enum rb_transpose { RB_NO_TRANSPOSE = 0, RB_TRANSPOSE = 1 } rb_transpose;

/* RotaryLayout, rust-ascend-compiler/src/ascend/rotary_programs.rs:5-6. */
typedef enum rb_rotary_layout { RB_ROTARY_INTERLEAVED = 0, RB_ROTARY_SPLIT_HALF = 1 } rb_rotary_layout;

/* Epilogue fused into the GEMM store.  The reference GEMM stores the identity only
 * (rust-ascend-kernels/src/kernel.rs:2); bias and SiLU*up are separate passes there
 * (affine_programs.rs:31-36, programs.rs:25,41). */
typedef enum rb_epilogue { RB_EPILOGUE_NONE = 0, RB_EPILOGUE_BIAS = 1, RB_EPILOGUE_SWIGLU = 2 } rb_epilogue;

/* HcclReduceOp, rust-ascend-driver/src/tensor/runtime/hccl.rs. */
typedef enum rb_reduce_op { RB_SUM = 0, RB_PROD = 1, RB_MAX = 2, RB_MIN = 3 } rb_reduce_op;

/* Attention output layout: [B,H,M,Dv] is the reference's (src/nn/attention.rs:49-67); [B,M,H,Dv]
 * feeds the output projection without a transpose. */
typedef enum rb_attention_layout { RB_LAYOUT_BHMD = 0, RB_LAYOUT_BMHD = 1 } rb_attention_layout;

/* RuntimeOptions, rust-ascend-driver/src/tensor/runtime/mod.rs:93-115. */
typedef struct rb_options {
    int32_t device;        /* CUDA ordinal (RuntimeOptions::device)                              */
    int32_t synchronous;   /* 1: synchronise the stream after every launch, as the reference does */
    uint64_t reserved[4];
} rb_options;

/* TensorBuffer{handle,shape,strides,dtype} (ruda_runtime; used throughout runtime/mod.rs:147-436).
 * handle is a storage id from rb_alloc / rb_import; offset is the byte offset of element 0
 * (Binding offset_start, runtime/mod.rs:629-644); strides are in elements. */
typedef struct rb_tensor {
    uint64_t handle;
    uint64_t offset;
    uint32_t dtype;
    uint32_t rank;
    uint64_t shape[8];
    uint64_t strides[8];
} rb_tensor;

/* KernelStats / ProgramStats, deepgemm/mod.rs:16 and common_ir/mod.rs:12. */
typedef struct rb_stats {
    uint64_t launches;
    uint64_t synchronizations;
    uint64_t empty_calls;
    uint64_t bytes_in_use;
    uint64_t allocations;
} rb_stats;

typedef struct rb_ctx rb_ctx;

/* ---- context, storage, server ------------------------------------------------------------------ */
/* AscendRuntime::initialize_exclusive, runtime/mod.rs:424-435: once per process; a second call fails. */
RB_API int32_t rb_init_exclusive(const rb_options* options, rb_ctx** out);
/* Drops the process context (the reference keeps its worker for the process lifetime; tests need this). */
RB_API int32_t rb_shutdown(rb_ctx* ctx);
RB_API const char* rb_last_error(void);
/* Device properties, runtime/mod.rs:544-595: name, SM count, memory bytes. */
RB_API int32_t rb_device_properties(rb_ctx* ctx, char* name, size_t name_bytes, int32_t* sm_count, uint64_t* memory_bytes);

/* AscendStorage::alloc / dealloc, runtime/mod.rs:501-515.  Alignment is 256 B (the reference's is 32);
 * zero-byte requests still own a minimal allocation (tensor/mod.rs:106-111).  rb_free synchronises first. */
RB_API int32_t rb_alloc(rb_ctx* ctx, uint64_t bytes, uint64_t* handle);
RB_API int32_t rb_free(rb_ctx* ctx, uint64_t handle);
/* Debug option (environment RUDA_GUARD_BANDS=1 at rb_init_exclusive): every rb_alloc is surrounded by 256-byte guard bands
 * and starts filled with all-ones bytes (NaN in every float format).  rb_check_guards drains the stream and counts the
 * live allocations whose guard bands a kernel has written into; rb_free checks its allocation too and reports damage as a
 * sticky error.  Stands in for a memory checker where none can run (the reference's test VM poisons local memory in the
 * same spirit, rust-ascend-kernels/src/tests.rs:20-88). */
RB_API int32_t rb_check_guards(rb_ctx* ctx, uint64_t* damaged);
/* Registers caller-owned device memory (for example a torch tensor) as a non-owning storage handle. */
RB_API int32_t rb_import(rb_ctx* ctx, void* device_pointer, uint64_t bytes, uint64_t* handle);
/* AscendStorage::get, runtime/mod.rs:494-500: resolves a handle to its device address and size. */
RB_API int32_t rb_resource(rb_ctx* ctx, uint64_t handle, void** device_pointer, uint64_t* bytes);
/* AscendServer::write / read, runtime/mod.rs:767-845.  write is asynchronous from pinned memory;
 * read synchronises and raises the sticky errors first. */
RB_API int32_t rb_write(rb_ctx* ctx, uint64_t handle, uint64_t offset, const void* host, uint64_t bytes);
RB_API int32_t rb_read(rb_ctx* ctx, uint64_t handle, uint64_t offset, void* host, uint64_t bytes);
RB_API int32_t rb_memset(rb_ctx* ctx, uint64_t handle, uint64_t offset, int32_t value, uint64_t bytes);
/* AscendServer::sync / flush, runtime/mod.rs:840-856. */
RB_API int32_t rb_sync(rb_ctx* ctx);
/* Drains the sticky error list into buf (newline separated); *count receives how many were pending. */
RB_API int32_t rb_take_errors(rb_ctx* ctx, char* buf, size_t buf_bytes, uint32_t* count);
/* AscendServer::memory_usage and the launch counters. */
RB_API int32_t rb_get_stats(rb_ctx* ctx, rb_stats* out);
/* Pinned host staging memory for rb_write / rb_read. */
RB_API int32_t rb_host_alloc(rb_ctx* ctx, uint64_t bytes, void** host);
RB_API int32_t rb_host_free(rb_ctx* ctx, void* host);
/* AscendServer::start_profile / end_profile, runtime/mod.rs:857-873, on CUDA events of the context's
 * stream.  rb_profile_end synchronises and returns the elapsed device milliseconds. */
RB_API int32_t rb_profile_begin(rb_ctx* ctx);
RB_API int32_t rb_profile_end(rb_ctx* ctx, float* milliseconds);
/* Caps the number of SMs the persistent GEMM occupies (0 = all), leaving the rest to a collective that runs beside
 * it.  No counterpart in the reference, whose collectives and kernels never overlap (runtime/hccl.rs:290-305). */
RB_API int32_t rb_set_sm_limit(rb_ctx* ctx, int32_t sm_limit);
/* Records everything enqueued on the context between begin and end (kernels, copies, collectives with their
 * cross-stream fences) into a CUDA graph, and replays it with one launch.  The reference launches and synchronises
 * kernel by kernel (worker.rs:92-103); replay removes the per-launch host cost of a fixed step.  No entry point that
 * synchronises or allocates (rb_read, rb_sync, rb_alloc, first use of a kernel) may be called while recording. */
RB_API int32_t rb_graph_begin(rb_ctx* ctx);
RB_API int32_t rb_graph_end(rb_ctx* ctx, uint64_t* graph);
RB_API int32_t rb_graph_launch(rb_ctx* ctx, uint64_t graph);
RB_API int32_t rb_graph_destroy(rb_ctx* ctx, uint64_t graph);
/* The context's CUDA stream as a cudaStream_t, for callers that share it with other libraries. */
RB_API int32_t rb_stream(rb_ctx* ctx, void** stream);

/* ---- row programs (FP32 math; storage F32 or BF16) --------------------------------------------- */
/* AscendRuntime::rms_norm, runtime/mod.rs:405-408 -> normalization.rs:153-166, IR row_programs.rs:144-151.
 * y = (x * rsqrt(mean(x^2) + eps)) * w over the last axis; rstd [rows] FP32 may be NULL. */
RB_API int32_t rb_rms_norm(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* weight, double epsilon,
                           const rb_tensor* y, const rb_tensor* rstd);
/* Residual update fused into the norm that follows it: x_out = x + delta (rounded to x's storage type; x_out may be
 * x itself), y = rms_norm(x_out).  Equals bias_add's residual sum (affine_programs.rs:31-36, MapProgram::Add
 * programs.rs:34) followed by AscendRuntime::rms_norm (runtime/mod.rs:405-408) with one pass over memory less. */
RB_API int32_t rb_add_rms_norm(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* delta, const rb_tensor* weight, double epsilon,
                               const rb_tensor* x_out, const rb_tensor* y);
/* Runtime::layer_norm, runtime/mod.rs:442-448 -> normalization.rs:116-132, IR row_programs.rs:164-177.
 * bias may be NULL (zeros); mean / rstd [rows] FP32 may be NULL. */
RB_API int32_t rb_layer_norm(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* weight, const rb_tensor* bias,
                             double epsilon, const rb_tensor* y, const rb_tensor* mean, const rb_tensor* rstd);
/* AscendRuntime::softmax / log_softmax, runtime/mod.rs:322-329 -> rows.rs:52-64, IR row_programs.rs:135-143. */
RB_API int32_t rb_softmax(rb_ctx* ctx, const rb_tensor* x, int32_t logarithmic, const rb_tensor* y);
/* AscendRuntime::sum_last / mean_last / max_last, runtime/mod.rs:286-303 (op: 0 sum, 1 mean, 2 max). */
RB_API int32_t rb_reduce_last(rb_ctx* ctx, const rb_tensor* x, int32_t op, const rb_tensor* y);

/* ---- element maps ------------------------------------------------------------------------------- */
/* AscendRuntime::silu_mul, runtime/mod.rs:282-284 -> elementwise.rs:13-19, IR programs.rs:25,41. */
RB_API int32_t rb_silu_mul(rb_ctx* ctx, const rb_tensor* gate, const rb_tensor* up, const rb_tensor* y);
/* AscendRuntime::bias_add, runtime/mod.rs:179-181 -> affine.rs:10-22, IR affine_programs.rs:16-38.
 * y = (x [+ residual]) + bias[col], in that order; residual may be NULL. */
RB_API int32_t rb_bias_add(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* bias, const rb_tensor* residual,
                           const rb_tensor* y);
/* Plain element-wise sum of two equal-shaped tensors (MapProgram::Add, programs.rs:34). */
RB_API int32_t rb_add(rb_ctx* ctx, const rb_tensor* a, const rb_tensor* b, const rb_tensor* y);
/* Division by a scalar, in place allowed: the Mean step after a Sum collective (src/distributed.rs:150-154,267-271). */
RB_API int32_t rb_div_scalar(rb_ctx* ctx, const rb_tensor* x, float divisor, const rb_tensor* y);
/* Multiplication by a scalar, in place allowed: the `matmul(q, k^T) * scale` of the composed attention
 * (src/nn/padded_attention.rs:43, src/nn/attention.rs:10-29).  One FP32 multiply per element, so any finite scale
 * (zero and non-powers of two included) gives the reference's bits. */
RB_API int32_t rb_mul_scalar(rb_ctx* ctx, const rb_tensor* x, float factor, const rb_tensor* y);
/* AscendRuntime::rotary / rotary_backward, runtime/mod.rs:259-268 -> rotary.rs:15-30, IR rotary_programs.rs:47-97. */
RB_API int32_t rb_rotary(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* cos, const rb_tensor* sin,
                         int32_t layout, int32_t backward, const rb_tensor* y);
/* AscendRuntime::rotary_prefix, runtime/mod.rs:215-221 -> rotary.rs:31-48, IR rotary_programs.rs:101-156.
 * Tables have the rank of x, last axis width/2, other axes 1 or equal; columns >= width keep their bits. */
RB_API int32_t rb_rotary_prefix(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* cos, const rb_tensor* sin,
                                uint32_t width, int32_t layout, int32_t backward, const rb_tensor* y);
/* AscendRuntime::repeat_kv_heads, runtime/mod.rs:209 -> heads.rs:21-28, IR heads_programs.rs:43-55. */
RB_API int32_t rb_repeat_kv_heads(rb_ctx* ctx, const rb_tensor* x, uint32_t query_heads, const rb_tensor* y);
/* AscendRuntime::causal_mask, runtime/mod.rs:206 -> mask.rs:5-15, IR mask_programs.rs:19-39.
 * out is FP32 [batch, queries, keys]. */
RB_API int32_t rb_causal_mask(rb_ctx* ctx, uint64_t query_start, uint64_t key_start, const rb_tensor* out);
/* AscendRuntime::cast / cast_into, runtime/mod.rs:271-279 -> conversion.rs:21-45 (F32 <-> BF16 <-> F16, RNE). */
RB_API int32_t rb_cast(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* y);
/* AscendRuntime::embedding, runtime/mod.rs:231-233 -> indexing.rs:33-37: out[i,:] = table[ids[i],:]. */
RB_API int32_t rb_embedding(rb_ctx* ctx, const rb_tensor* table, const rb_tensor* ids, const rb_tensor* out);
/* AscendRuntime::embedding_backward, runtime/mod.rs:253-256 -> indexing.rs:60-64 -> tensor/embedding.rs:60-78: dense weight
 * gradient out[num_weights, W] (the row count is out's) from grad ids.shape + [W]; repeated ids accumulate in FP32,
 * padding_idx (UINT64_MAX = none, else < num_weights) suppresses that row's derivative, scale_grad_by_freq divides each
 * touched row by its number of occurrences. */
RB_API int32_t rb_embedding_backward(rb_ctx* ctx, const rb_tensor* grad, const rb_tensor* ids, uint64_t padding_idx,
                                     int32_t scale_grad_by_freq, const rb_tensor* out);
/* AscendRuntime::copy_contiguous, runtime/mod.rs:223-225 -> indexing.rs:46-59: a private device copy of a contiguous tensor of
 * any storage dtype (the saved indices of embedding_with_saved_indices, runtime/mod.rs:249-251). */
RB_API int32_t rb_copy(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* y);
/* resize_prefix of runtime/padded_matrix.rs:6-16,24-37 (the worker's zero pad / crop that gemm_padded_bf16_fp32,
 * runtime/mod.rs:188-204, is built from): y holds x's values wherever the index lies inside x and +0 elsewhere; equal rank
 * 1..8, positive axes, FP32 or BF16, values moved as bits. */
RB_API int32_t rb_resize_prefix(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* y);

/* ---- first-order backward programs (FP32) -------------------------------------------------------------- */
/* AscendRuntime::rms_norm_backward, runtime/mod.rs:411-414 -> normalization.rs:168-186, IR row_programs.rs:189-217:
 * [input gradient, weight gradient] from the saved rstd; the weight gradient sums all leading rows on the device. */
RB_API int32_t rb_rms_norm_backward(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* weight, const rb_tensor* grad,
                                    const rb_tensor* rstd, const rb_tensor* dx, const rb_tensor* dweight);
/* AscendRuntime::softmax_backward / log_softmax_backward, runtime/mod.rs:332-343 -> rows.rs, IR row_programs.rs:152-163. */
RB_API int32_t rb_softmax_backward(rb_ctx* ctx, const rb_tensor* output, const rb_tensor* grad, int32_t logarithmic, const rb_tensor* dx);
/* AscendRuntime::silu_mul_backward, runtime/mod.rs:287-290 -> elementwise.rs:21-28, IR programs.rs:29,43. */
RB_API int32_t rb_silu_mul_backward(rb_ctx* ctx, const rb_tensor* gate, const rb_tensor* up, const rb_tensor* grad,
                                    const rb_tensor* dgate, const rb_tensor* dup);
/* AscendRuntime::repeat_kv_heads_backward, runtime/mod.rs:211-213 -> heads.rs:30-51, IR heads_programs.rs:59-86. */
RB_API int32_t rb_repeat_kv_heads_backward(rb_ctx* ctx, const rb_tensor* grad, uint32_t kv_heads, const rb_tensor* dx);
/* AscendRuntime::bias_add_backward, runtime/mod.rs:183-185 -> affine.rs:24-26: sum of dY over all leading axes. */
RB_API int32_t rb_bias_add_backward(rb_ctx* ctx, const rb_tensor* grad, const rb_tensor* dbias);

/* Runtime::layer_norm_backward, runtime/mod.rs:449-455 -> normalization.rs:134-152, IR row_programs.rs (LayerNormInputBackward,
 * LayerNormWeightContributions): [input gradient, weight gradient, bias gradient] from the saved mean and rstd. */
RB_API int32_t rb_layer_norm_backward(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* weight, const rb_tensor* grad,
                                      const rb_tensor* mean, const rb_tensor* rstd, const rb_tensor* dx,
                                      const rb_tensor* dweight, const rb_tensor* dbias);
/* nn::CausalCrossEntropyConfig::forward_hidden, src/nn/causal_lm.rs:118-196, which chunks tokens through log_softmax
 * (runtime/mod.rs:327-329) and nll_loss (runtime/mod.rs:222-230, ignore index, sum reduction).  logits FP32 [B,T,V],
 * labels I32/I64 [B,T]; with shift != 0 position t is scored against label t+1 and the last position of every sequence is
 * dropped.  loss_sum and valid_tokens are FP32 [1].  dlogits (NULL or FP32 [B,T,V]) receives the gradient of the mean
 * loss times `upstream`: (softmax - onehot) * upstream / max(valid, 1), zero for rows that are not scored.  A label
 * outside [0, V) other than ignore_index is never used as an index: its row is left unscored, and a synchronous context
 * returns RB_INVALID_TENSOR for the call. */
RB_API int32_t rb_causal_cross_entropy(rb_ctx* ctx, const rb_tensor* logits, const rb_tensor* labels, int64_t ignore_index,
                                       int32_t shift, float upstream, const rb_tensor* loss_sum,
                                       const rb_tensor* valid_tokens, const rb_tensor* dlogits);

/* ---- BF16 matrix programs (tcgen05 tensor cores, FP32 accumulation) ------------------------------ */
/* AscendRuntime::gemm / gemm_into, runtime/mod.rs:346-355 -> matrix.rs:47-59 -> GemmSpec deepgemm/plan.rs:49-80;
 * device program rust-ascend-kernels/src/kernel.rs:11-76.  out = op(A) op(B): contiguous BF16 operands, rank 2
 * or equal-batch rank 3, M/N/K positive multiples of 16, out BF16 or FP32.  With transpose_b = 1 and B = W[N,K]
 * this is Linear, Y = X W^T (src/nn.rs:77-79).  The epilogue runs in FP32 before the output rounding:
 *   RB_EPILOGUE_BIAS   + bias[N] (FP32 or BF16)                      (bias_add, affine_programs.rs:31-36)
 *   RB_EPILOGUE_SWIGLU out = SiLU(op(A) op(B)) * (op(A) op(b_up))    (swiglu, src/nn/feed_forward.rs:39-41)
 * bias / b_up are NULL unless their epilogue is selected. */
RB_API int32_t rb_gemm(rb_ctx* ctx, const rb_tensor* a, const rb_tensor* b, int32_t transpose_a, int32_t transpose_b,
                       const rb_tensor* bias, const rb_tensor* b_up, int32_t epilogue, const rb_tensor* out);

/* AscendRuntime::linear_bf16_fp32, runtime/mod.rs:367-370 -> matrix.rs:84-93,129-133 (tensor level src/nn.rs:73-88,375-413):
 * Y = bf16(X) bf16(W)^T for FP32 X [M,K] and W [N,K], FP32 Y [M,N]; x_bf16 / w_bf16 receive the BF16 operands the
 * reference returns beside Y for the backward pass.  One conversion launch covers both operands, then one GEMM. */
RB_API int32_t rb_linear_bf16_fp32(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* w, const rb_tensor* y,
                                   const rb_tensor* x_bf16, const rb_tensor* w_bf16);
/* Frozen-weight linear, runtime/mod.rs:383-385 -> matrix.rs:147-159 (src/nn/frozen.rs:44-59): Y = bf16(X) W^T with the
 * BF16 weight used in place.  x_bf16 (BF16 [M,K]) receives the converted input, or may be NULL. */
RB_API int32_t rb_linear_frozen_bf16(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* w, const rb_tensor* y, const rb_tensor* x_bf16);
/* RudaAscend::float_matmul, src/backend.rs:692-703 -> generic_matrix::matmul, runtime/generic_matrix.rs:17-54 (the vendor
 * aclnnMatmul with KEEP_DTYPE, worker.rs:128-162): A [.., M, K] @ B [.., K, N] in the operands' own dtype (FP32, FP16 or
 * BF16), ranks 2..6, singleton batch axes broadcast, any sizes (an empty contraction gives zeros).  `out` has the
 * broadcast shape and the operands' dtype.  One pass packs each operand K-major and 16-aligned; one tensor-core launch
 * multiplies: BF16 and FP16 operands in their own format, FP32 operands as three BF16 parts whose six leading cross
 * products accumulate in one FP32 accumulator, smallest first (relative error about 2^-24 per product term). */
RB_API int32_t rb_tensor_matmul(rb_ctx* ctx, const rb_tensor* a, const rb_tensor* b, const rb_tensor* out);
/* M-grouped GEMM, GemmSpec::grouped_nt, deepgemm/plan.rs:61-67 with GroupEnds (plan.rs:15-29) and the tile walk of
 * rust-ascend-kernels/src/scheduler.rs:21-33: A [M,K] BF16, weights [G,N,K] BF16, `ends` = G nondecreasing row prefix sums
 * (host array, multiples of 256, last = M); rows [ends[g-1], ends[g]) meet weight g; out [M,N] BF16 or FP32.  One
 * persistent launch covers all groups, empty ones included. */
RB_API int32_t rb_gemm_grouped_nt(rb_ctx* ctx, const rb_tensor* a, const rb_tensor* weights, const int64_t* ends, uint32_t groups,
                                  const rb_tensor* out);
/* gemm_padded_bf16_fp32, runtime/mod.rs:188-191 -> padded_matrix.rs:40-50, PaddedGemmSpec deepgemm/padded.rs:12-50: FP32 (or
 * BF16) A and B of any positive sizes, rank 2 or equal-batch rank 3, all four transposes; `out` is FP32 with the logical
 * M x N; a_bf16 / b_bf16 receive the zero-padded BF16 operands (both matrix axes rounded up to multiples of 16) that the
 * reference saves for the backward pass. */
RB_API int32_t rb_gemm_padded(rb_ctx* ctx, const rb_tensor* a, const rb_tensor* b, int32_t transpose_a, int32_t transpose_b,
                              const rb_tensor* out, const rb_tensor* a_bf16, const rb_tensor* b_bf16);
/* Backward of the composed attention (the autodiff graph of src/nn/attention.rs:10-29,49-67) with the reference's rounding
 * points (examples/grouped_attention_tensor.rs:14-44): P = softmax(scale bf16(Q) bf16(K)^T + mask), dP = bf16(dY) bf16(V)^T,
 * dS = P (dP - sum(P dP)) in FP32, bf16(scale dS) feeds dQ and dK, bf16(P) feeds dV, and a KV head's gradients sum over
 * its query heads (heads_programs.rs:59-86).  FP32 q [B,Hq,M,D], k [B,Hkv,N,D], v [B,Hkv,N,Dv], grad [B,Hq,M,Dv]; mask
 * (nullable) FP32 [B,Hq,M,N]; the causal rule uses the absolute positions as rb_causal_mask does; dmask (nullable)
 * receives dS.  Scores are materialised, as in the reference. */
RB_API int32_t rb_attention_backward(rb_ctx* ctx, const rb_tensor* q, const rb_tensor* k, const rb_tensor* v, const rb_tensor* grad,
                                     const rb_tensor* mask, float scale, int32_t causal, uint64_t query_start, uint64_t key_start,
                                     const rb_tensor* dq, const rb_tensor* dk, const rb_tensor* dv, const rb_tensor* dmask);

/* Linear on host buffers: Y_host = X_host W^T (+ bias), the reference's write -> launch -> read sequence for one call
 * (AscendServer::write / read, runtime/mod.rs:767-845; launch + stream sync, worker.rs:404-415) as ONE call whose three
 * steps overlap: X is cut into `row_chunks` groups of rows, and while one group multiplies on the tensor cores the next
 * one uploads and the previous one downloads on two copy streams.  host_x [M,K] BF16 and host_y [M,N] (dtype of y)
 * should be pinned (rb_host_alloc); x and y are device staging tensors of those shapes, w [N,K] BF16 and bias [N]
 * (nullable) stay resident.  Returns when host_y is complete (it synchronises, like rb_read).  The result is
 * bit-identical to rb_write + rb_gemm + rb_read on the same operands. */
RB_API int32_t rb_linear_host(rb_ctx* ctx, const void* host_x, const rb_tensor* x, const rb_tensor* w, const rb_tensor* bias,
                              const rb_tensor* y, void* host_y, uint32_t row_chunks);

/* rb_gemm without any device allocation.  It has no counterpart in the reference (whose GEMM provider allocates
 * through ComputeStorage); it exists for hosts that must not call cudaMalloc once they are running: servers with a
 * memory budget fixed at start-up, real-time loops that cannot take the device-wide synchronisation cudaMalloc and
 * cudaFree imply, processes that have handed the rest of the device memory to another pool.
 * Same operand contract as rb_gemm with the identity epilogue.  The scratch rb_gemm would allocate (the K-major
 * rewrite of an operand given as A[K,M] or B[K,N], and the kernel's status word) lives in a 16 MiB + 256 B array
 * inside the library image, held by every GPU that loads the library until the process exits.  Limit: the operands
 * that need a rewrite may take at most 16 MiB together (A[M,K] with B[N,K] needs none); larger ones are rejected with
 * RB_INVALID_TENSOR.  The context's device must be current on the calling thread.  The first call on a device
 * resolves the array's address (cudaGetSymbolAddress); make that first call before any stream capture begins.
 * Every call shares the one array: calls that overlap on the GPU (other streams, other threads) race on it.  The
 * call drains the context's stream before it returns, so that an expired kernel wait is reported by this call; for
 * that reason it returns RB_INVALID_TENSOR between rb_graph_begin and rb_graph_end. */
RB_API int32_t rb_gemm_no_alloc(rb_ctx* ctx, const rb_tensor* a, const rb_tensor* b, int32_t transpose_a, int32_t transpose_b,
                                const rb_tensor* out);

/* ---- attention --------------------------------------------------------------------------------------- */
/* nn::scaled_dot_product_attention_bf16_fp32 / causal_attention / grouped_query_attention /
 * causal_grouped_query_attention, src/nn/attention.rs:10,33,49,69 (domain checks :81-104); the reference composes
 * them from causal_mask (runtime/mod.rs:206), repeat_kv_heads (:209), two BF16 GEMMs and softmax.
 * q [B,Hq,M,D], k [B,Hkv,N,D], v [B,Hkv,N,Dv] as rank-4 tensors whose last axis is contiguous (other strides may
 * describe a [B,S,H,D] buffer); out is contiguous [B,Hq,M,Dv] (RB_LAYOUT_BHMD) or [B,M,Hq,Dv] (RB_LAYOUT_BMHD).
 * O = softmax(scale * bf16(Q) bf16(K)^T + mask) bf16(V); with causal != 0 key k of the block is hidden from query q
 * iff key_start + k > query_start + q (mask_programs.rs:30-37).  additive_mask is NULL or FP32 [B,Hq,M,N].
 * cos / sin (NULL, or FP32 [positions, 64]) apply the rotary encoding of rotary_programs.rs:63-93 to Q and K before
 * the product: key n uses table row n, query i uses row i + (query_start - key_start).
 * BF16 tensors with D = Dv = 128, no additive mask and a positive scale run on the tensor-core kernel (nothing is
 * materialised); other shapes run a general kernel that follows the reference's materialised algorithm. */
RB_API int32_t rb_attention(rb_ctx* ctx, const rb_tensor* q, const rb_tensor* k, const rb_tensor* v, const rb_tensor* additive_mask,
                            float scale, int32_t causal, uint64_t query_start, uint64_t key_start,
                            const rb_tensor* cos, const rb_tensor* sin, int32_t rotary_layout, int32_t out_layout,
                            const rb_tensor* out);
/* How many rb_attention calls of this context ran on the tensor-core kernel and how many on the general row kernel
 * (introspection for tests and profiling, in the spirit of KernelStats, deepgemm/mod.rs:16). */
RB_API int32_t rb_attention_launch_counts(rb_ctx* ctx, uint64_t* tensor_core, uint64_t* general);

/* ---- a side stream beside the compute stream (no counterpart in the reference, where every operation is a launch followed
 * by a stream synchronisation, runtime/worker.rs:404-415) ------------------------------------------------------------ */
/* This entry has no counterpart in the reference.  Forks: until rb_aux_end, everything enqueued on the context goes to a
 * higher-priority side stream, ordered after what the compute stream held at this call. */
RB_API int32_t rb_aux_begin(rb_ctx* ctx);
/* This entry has no counterpart in the reference.  Ends the fork and records the side stream's position in `slot` (0..31). */
RB_API int32_t rb_aux_end(rb_ctx* ctx, uint32_t slot);
/* This entry has no counterpart in the reference.  Joins: later work on the compute stream waits for what `slot` recorded. */
RB_API int32_t rb_aux_wait(rb_ctx* ctx, uint32_t slot);

/* ---- peer memory and the fused tensor-parallel exchange (no counterpart in the reference: its row-parallel projection is a
 * GEMM followed by a vendor all-reduce, runtime/hccl.rs:386-548; src/distributed.rs:139-156) ------------------------- */
#define RB_MAX_PEERS 8
#define RB_PEER_TOKEN_BYTES 80 /* 64-byte CUDA IPC handle of the allocation + 8-byte offset of the storage inside it + 8-byte length of the storage */
/* This entry has no counterpart in the reference.  Exports a storage of this process as a token (CUDA IPC) that another process of
 * the node passes to rb_peer_open; tokens travel over the control plane that carries the communicator's root id
 * (src/distributed.rs:74-110). */
RB_API int32_t rb_peer_export(rb_ctx* ctx, uint64_t handle, uint8_t token[RB_PEER_TOKEN_BYTES]);
/* This entry has no counterpart in the reference.  Opens a peer's token as a storage handle of `bytes` bytes whose device address is the
 * peer's memory; the handle is used like any other in rb_tensor descriptors.  Close it with rb_peer_close, not rb_free. */
RB_API int32_t rb_peer_open(rb_ctx* ctx, const uint8_t token[RB_PEER_TOKEN_BYTES], uint64_t bytes, uint64_t* handle);
/* This entry has no counterpart in the reference.  Drains the stream, forgets the handle and unmaps the peer's memory. */
RB_API int32_t rb_peer_close(rb_ctx* ctx, uint64_t handle);
/* Row-parallel Linear with the reduce-scatter half of its all-reduce fused into the epilogue; stands where the reference runs
 * gemm (runtime/mod.rs:346-349) and then HcclCommunicator::reduce_scatter (src/distributed.rs:139-156).  a BF16 [T, K],
 * b BF16 [H, K] (this rank's K shard); T a multiple of 128 * world, H of 64.  Rows [o*T/world, (o+1)*T/world) of the partial
 * product are stored into staging[o] (BF16 [world, T/world, H], rank o's memory) at slot [rank], and every 32-row slice is
 * announced (in batches, once the storing CTA is done) by adding to word [rank] of flags[o] (INT32 [world + 1], rank o's memory).  rb_gemm_scatter_signals gives the
 * number of announcements one call makes per owner. */
RB_API int32_t rb_gemm_scatter(rb_ctx* ctx, const rb_tensor* a, const rb_tensor* b, uint32_t rank, uint32_t world,
                               const rb_tensor* const* staging, const rb_tensor* const* flags);
/* The same with an FP32 bias [H] folded into this rank's partial product (NULL: none).  A row-parallel Linear adds its bias
 * once, so exactly one rank of the group passes it (src/nn.rs:77-79 adds the bias after the product). */
RB_API int32_t rb_gemm_scatter_bias(rb_ctx* ctx, const rb_tensor* a, const rb_tensor* b, const rb_tensor* bias, uint32_t rank, uint32_t world,
                                    const rb_tensor* const* staging, const rb_tensor* const* flags);
/* This entry has no counterpart in the reference.  Announcements per owner of one rb_gemm_scatter call with T tokens and H columns (0 when
 * the shape is not accepted). */
RB_API uint32_t rb_gemm_scatter_signals(uint64_t tokens, uint64_t hidden, uint32_t world);
/* This entry has no counterpart in the reference.  Waits on this GPU, with a limit of RUDA_PEER_WAIT_MS milliseconds (default 5000), until words [0, world) of `flags` (INT32
 * [world + 1], local memory that peers add to) have each grown by `count` beyond the running target kept in word [world],
 * then advances the target.  On expiry the next rb_sync reports RB_SERVER_UNHEALTHY; nothing faults. */
RB_API int32_t rb_peer_wait(rb_ctx* ctx, const rb_tensor* flags, uint32_t world, uint32_t count);
/* This entry has no counterpart in the reference.  Adds 1 to word [rank] of every flags[d] (INT32 [world + 1], rank d's memory) once
 * everything enqueued before it on this context has finished; with rb_peer_wait(count = 1) on every rank this is a barrier
 * between the GPUs that never leaves the stream. */
RB_API int32_t rb_peer_signal(rb_ctx* ctx, uint32_t rank, uint32_t world, const rb_tensor* const* flags);
/* The rest of the fused all-reduce, on the rows this rank owns; stands where the reference runs the all-reduce's second half
 * (all_gather, src/distributed.rs:121-138) and then rms_norm (runtime/mod.rs:405-408) on the full tensor.  Sums the `world`
 * staged partials (staging BF16 [world, rows, width], may be NULL) in rank order in FP32, rounds once to BF16, adds the residual
 * x_in (BF16 [rows, width], may be NULL) with the rounding of rb_add_rms_norm, stores the new residual to x_out (may be NULL),
 * applies RMSNorm with `weight` (NULL: no normalisation, which makes scatter + this call a plain all-reduce), and stores the rows into every destinations[d] (BF16 [world * rows, width], rank
 * d's memory) at row offset rank * rows; then adds 1 to word [rank] of flags[d].  `done` is one zeroed INT32 word of local
 * scratch. */
RB_API int32_t rb_reduce_norm_push(rb_ctx* ctx, const rb_tensor* staging, const rb_tensor* x_in, const rb_tensor* weight,
                                   double epsilon, const rb_tensor* x_out, uint32_t rank, uint32_t world,
                                   const rb_tensor* const* destinations, const rb_tensor* const* flags,
                                   const rb_tensor* done);
/* The same owner-side step in its pull form, for a row-parallel Linear that ran as a plain rb_gemm: partials[s] is rank s's
 * whole partial product (BF16 [world * rows, width], rank s's memory mapped here), and this rank fetches rows
 * [rank * rows, (rank + 1) * rows) of every one of them itself (asynchronous bulk copies into shared memory, several rows in
 * flight per SM), sums them in rank order and continues exactly as rb_reduce_norm_push does, with the same bits.  The caller
 * orders the step behind every rank's GEMM (rb_peer_signal after the GEMM, rb_peer_wait before this call); a rank may
 * overwrite its partial product again once it has seen every owner's announcement in `flags`.  Stands where the reference runs
 * all_reduce (src/distributed.rs:139-156) and rms_norm (runtime/mod.rs:405-408) after the Linear. */
RB_API int32_t rb_reduce_norm_push_pull(rb_ctx* ctx, const rb_tensor* const* partials, const rb_tensor* x_in, const rb_tensor* weight,
                                        double epsilon, const rb_tensor* x_out, uint32_t rank, uint32_t world,
                                        const rb_tensor* const* destinations, const rb_tensor* const* flags, const rb_tensor* done);
/* The owner-side arithmetic alone, for an exchange whose transfers are device-to-device copies (rb_copy between mapped peer
 * buffers: copy engines, no SM): sums the `world` partial products gathered in `staging` (BF16 [world, rows, width], local) in
 * rank order in FP32, rounds once to BF16, adds the residual x_in, stores the new residual to x_out, applies RMSNorm with
 * `weight` (NULL: none) and writes the rows to `out` (BF16 [rows, width], local), with the bits rb_reduce_norm_push produces.
 * `done` is two zeroed INT32 words of local scratch.  Stands where the reference runs rms_norm (runtime/mod.rs:405-408) on the
 * result of all_reduce (src/distributed.rs:139-156). */
RB_API int32_t rb_reduce_norm_rows(rb_ctx* ctx, const rb_tensor* staging, const rb_tensor* x_in, const rb_tensor* weight, double epsilon,
                                   const rb_tensor* x_out, const rb_tensor* out, const rb_tensor* done);
/* The reduce-scatter half of the exchange as a kernel of its own, for a row-parallel Linear that ran as a plain rb_gemm: every
 * row of `partial` (BF16 [world * rows, width], local) is stored into slot [rank] of the staging area of the rank that owns
 * it (staging[o]: BF16 [world, rows, width], rank o's memory), then 1 is added to word [rank] of every flags[o].  Only posted
 * stores cross the link.  Followed by rb_peer_wait(count 1) and rb_reduce_norm_push it is the scatter form with the transfer
 * moved out of the GEMM, e.g. onto the side stream; same bits.  `done` is one zeroed INT32 word of local scratch.  Stands where
 * the reference runs reduce_scatter (src/distributed.rs:139-156 splits all_reduce the same way). */
RB_API int32_t rb_scatter_rows(rb_ctx* ctx, const rb_tensor* partial, uint32_t rank, uint32_t world, const rb_tensor* const* staging,
                               const rb_tensor* const* flags, const rb_tensor* done);

/* ---- collectives: NCCL over NVLink 5 / NVSwitch in place of HCCL ----------------------------------------------- */
typedef struct rb_comm rb_comm;
/* HcclGetRootInfo, runtime/hccl.rs:340-357: rank 0 creates the 128-byte id (ncclUniqueId) that the control plane
 * hands to every rank (src/distributed.rs:74-110).  The NCCL library is loaded with dlopen (RUDA_NCCL_LIBRARY or
 * libnccl.so.2), as the reference loads libhccl.so (runtime/hccl.rs:79-85). */
RB_API int32_t rb_comm_unique_id(uint8_t* id_128_bytes);
/* HcclCommInitRootInfo, runtime/hccl.rs:133-197: one communicator per process and device. */
RB_API int32_t rb_comm_init(rb_ctx* ctx, const uint8_t* id_128_bytes, uint32_t rank, uint32_t world_size, rb_comm** out);
/* Entry drop, runtime/hccl.rs:119-131: drains, destroys; aborts and leaks if the work cannot be drained. */
RB_API int32_t rb_comm_destroy(rb_comm* comm);
/* HcclCommunicator::rank / world_size, runtime/hccl.rs:435-443. */
RB_API int32_t rb_comm_info(rb_comm* comm, uint32_t* rank, uint32_t* world_size, int32_t* nccl_version);
/* HcclCommunicator::all_reduce, runtime/hccl.rs:452-460 (sum/prod/max/min over F32/F16/BF16/I32/I64).  in == out is
 * allowed.  deferred_fence != 0 lets later compute on the context's stream run while the collective is in flight;
 * rb_comm_fence then orders the compute stream after every collective issued so far. */
RB_API int32_t rb_all_reduce(rb_comm* comm, const rb_tensor* in, int32_t op, const rb_tensor* out, int32_t deferred_fence);
RB_API int32_t rb_comm_fence(rb_comm* comm);
/* Finer fences for deferred collectives: rb_comm_ticket returns the sequence number of the latest collective issued
 * on this communicator, rb_comm_wait_ticket orders the compute stream after that one collective only (the reference
 * synchronises after every collective, runtime/hccl.rs:290-305; these calls let independent row blocks overlap). */
RB_API int32_t rb_comm_ticket(rb_comm* comm, uint64_t* ticket);
RB_API int32_t rb_comm_wait_ticket(rb_comm* comm, uint64_t ticket);
/* HcclCommunicator::broadcast, runtime/hccl.rs:444-451. */
RB_API int32_t rb_broadcast(rb_comm* comm, const rb_tensor* in, uint32_t root, const rb_tensor* out);
/* HcclCommunicator::all_gather, runtime/hccl.rs:461-466: rank-ordered concatenation along the leading axis. */
RB_API int32_t rb_all_gather(rb_comm* comm, const rb_tensor* in, const rb_tensor* out);
/* HcclCommunicator::reduce_scatter, runtime/hccl.rs:467-473: this rank's equal leading-axis shard of the reduction. */
RB_API int32_t rb_reduce_scatter(rb_comm* comm, const rb_tensor* in, int32_t op, const rb_tensor* out);
/* Row-parallel Linear and its all-reduce in one call: what a tensor-parallel caller writes as gemm (runtime/mod.rs:346-349) on its
 * K shard followed by HcclCommunicator::all_reduce(sum) (runtime/hccl.rs:452-460).  x BF16 [T, K/world], w_shard BF16
 * [H, K/world], out BF16 or FP32 [T, H], complete on every rank.  overlap_mode 0: one GEMM then one all-reduce; 1: up to four
 * row chunks whose all-reduces run on the communicator's stream under the next chunk's GEMM. */
RB_API int32_t rb_row_parallel_linear_allreduce(rb_comm* comm, const rb_tensor* x, const rb_tensor* w_shard,
                                                const rb_tensor* out, int32_t overlap_mode);

#ifdef __cplusplus
}
#endif
#endif /* RUDA_B200_H */
