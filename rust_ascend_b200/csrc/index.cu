// Index-driven programs beside the dense path: the dense embedding weight gradient and the prefix resize (zero pad / crop)
// that the padded matrix wrappers are built from.
//
// Embedding backward (tensor/embedding.rs:60-78, runtime/indexing.rs:60-64): out[num_weights, W] starts at zero; every
// position p adds grad[p, :] to row ids[p] unless that row is the padding row; with scale_grad_by_freq each touched row is
// then divided by its number of occurrences (examples/embedding_tensor.rs:44-53).  Accumulation is FP32 (atomic adds into the
// output for FP32 storage, into an FP32 scratch image for half storage), so repeated ids sum in an unspecified order exactly
// as the vendor operator the reference calls leaves it unspecified.
//
// Prefix resize (runtime/padded_matrix.rs:6-16, "resize_prefix"): y[i0..ir] = x[i0..ir] where the index lies inside x, +0
// elsewhere; shrinking an axis crops, growing it pads at the end.  Values are copied as bits.
#include "common.cuh"

namespace {

using bf = __nv_bfloat16;

__device__ __forceinline__ float ldf(const float* p, uint64_t i) { return p[i]; }
__device__ __forceinline__ float ldf(const bf* p, uint64_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ float ldf(const __half* p, uint64_t i) { return __half2float(p[i]); }
__device__ __forceinline__ void stf(float* p, uint64_t i, float v) { p[i] = v; }
__device__ __forceinline__ void stf(bf* p, uint64_t i, float v) { p[i] = __float2bfloat16_rn(v); }
__device__ __forceinline__ void stf(__half* p, uint64_t i, float v) { p[i] = __float2half_rn(v); }

unsigned grid_for(rb_ctx* ctx, uint64_t work_items) {
    uint64_t blocks = (work_items + 255) / 256, cap = (uint64_t)ctx->sm_count * 16;
    return (unsigned)(blocks < cap ? (blocks ? blocks : 1) : cap);
}

template <typename I>
__global__ void __launch_bounds__(256) embedding_count_kernel(const I* ids, uint64_t count, uint64_t rows, uint64_t padding, int* freq, int* bad) {
    uint64_t stride = (uint64_t)gridDim.x * 256;
    for (uint64_t p = (uint64_t)blockIdx.x * 256 + threadIdx.x; p < count; p += stride) {
        int64_t id = (int64_t)ids[p];
        if (id < 0 || (uint64_t)id >= rows) { atomicExch(bad, 1); continue; }
        if ((uint64_t)id != padding) atomicAdd(freq + id, 1);
    }
}

template <typename T, typename I>
__global__ void __launch_bounds__(256) embedding_scatter_kernel(const T* grad, const I* ids, float* acc, uint64_t count, uint32_t width,
                                                               uint64_t rows, uint64_t padding) {
    uint64_t total = count * width, stride = (uint64_t)gridDim.x * 256;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += stride) {
        uint64_t p = i / width; uint32_t c = (uint32_t)(i % width);
        int64_t id = (int64_t)ids[p];
        if (id < 0 || (uint64_t)id >= rows || (uint64_t)id == padding) continue;
        atomicAdd(acc + (uint64_t)id * width + c, ldf(grad, i));
    }
}

// out = acc (/ freq[row] when scaling and the row was touched); acc may alias out for FP32 storage.
template <typename T>
__global__ void __launch_bounds__(256) embedding_finish_kernel(const float* acc, const int* freq, T* out, uint64_t rows, uint32_t width, bool scale) {
    uint64_t total = rows * width, stride = (uint64_t)gridDim.x * 256;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += stride) {
        float v = acc[i];
        if (scale) { int f = freq[i / width]; if (f > 1) v = __fdiv_rn(v, (float)f); }
        stf(out, i, v);
    }
}

struct ResizeDims { uint32_t rank; uint64_t src[8]; uint64_t dst[8]; };

template <typename T>
__global__ void __launch_bounds__(256) resize_prefix_kernel(const T* x, T* y, uint64_t total, ResizeDims d) {
    uint64_t stride = (uint64_t)gridDim.x * 256;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += stride) {
        uint64_t rest = i, src = 0, mul = 1; bool inside = true;
        for (int a = (int)d.rank - 1; a >= 0; --a) {
            uint64_t c = rest % d.dst[a]; rest /= d.dst[a];
            inside = inside && c < d.src[a];
            src += c * mul; mul *= d.src[a];
        }
        y[i] = inside ? x[src] : T(0);
    }
}

}  // namespace

using namespace rb;

extern "C" {

int32_t rb_embedding_backward(rb_ctx* ctx, const rb_tensor* grad, const rb_tensor* ids, uint64_t padding_idx, int32_t scale_grad_by_freq,
                              const rb_tensor* out) {
    RB_TRY(check_ctx(ctx));
    void *pg, *pi, *po;
    RB_TRY(resolve(ctx, grad, "embedding gradient", &pg)); RB_TRY(resolve(ctx, ids, "embedding ids", &pi)); RB_TRY(resolve(ctx, out, "embedding weight gradient", &po));
    if (ids->dtype != RB_I32 && ids->dtype != RB_I64) return fail(RB_INVALID_TENSOR, "embedding indices must be INT32 or INT64");
    bool shape_ok = grad->rank == ids->rank + 1 && out->rank == 2 && grad->dtype == out->dtype &&
                    (grad->dtype == RB_F32 || grad->dtype == RB_F16 || grad->dtype == RB_BF16);
    for (uint32_t a = 0; shape_ok && a < ids->rank; ++a) shape_ok = grad->shape[a] == ids->shape[a];
    if (shape_ok) shape_ok = out->shape[1] == grad->shape[grad->rank - 1];
    const uint64_t count = elements(ids);
    if (!shape_ok || (out->shape[0] == 0 && count != 0))
        return fail(RB_INVALID_TENSOR, "embedding gradient must have the index shape followed by the embedding width and floating dtype");
    const uint64_t rows = out->shape[0], width = out->shape[1];
    if (padding_idx != UINT64_MAX && padding_idx >= rows) return fail(RB_INVALID_TENSOR, "embedding padding index must be within the weight rows");
    if (rows * width > 0xffffffffull || width > 0xffffffffull || rows > 0x7fffffffull) return fail(RB_INVALID_TENSOR, "embedding weight gradient exceeds u32 elements");
    const uint64_t out_elems = rows * width;
    if (out_elems == 0) return empty_call(ctx);
    const bool f32 = out->dtype == RB_F32;
    // Workspace: [0,256) flags, then int freq[rows], then (half storage only) the FP32 accumulation image.
    const uint64_t freq_bytes = (rows * 4 + 255) / 256 * 256;
    RB_TRY(ensure_workspace(ctx, 256 + freq_bytes + (f32 ? 0 : out_elems * 4)));
    uint8_t* ws = static_cast<uint8_t*>(ctx->workspace);
    int* bad = reinterpret_cast<int*>(ws);
    int* freq = reinterpret_cast<int*>(ws + 256);
    float* acc = f32 ? static_cast<float*>(po) : reinterpret_cast<float*>(ws + 256 + freq_bytes);
    RB_CUDA(ctx, "cudaMemsetAsync", cudaMemsetAsync(ws, 0, 256 + freq_bytes, ctx->stream));
    RB_CUDA(ctx, "cudaMemsetAsync", cudaMemsetAsync(acc, 0, out_elems * 4, ctx->stream));
    if (count == 0 || width == 0) {
        if (!f32) RB_CUDA(ctx, "cudaMemsetAsync", cudaMemsetAsync(po, 0, out_elems * 2, ctx->stream));
        return empty_call(ctx);
    }
    const bool i32 = ids->dtype == RB_I32;
    if (i32) embedding_count_kernel<int32_t><<<grid_for(ctx, count), 256, 0, ctx->stream>>>((const int32_t*)pi, count, rows, padding_idx, freq, bad);
    else embedding_count_kernel<int64_t><<<grid_for(ctx, count), 256, 0, ctx->stream>>>((const int64_t*)pi, count, rows, padding_idx, freq, bad);
    RB_TRY(after_launch(ctx, "embedding_backward (count)"));
    const unsigned g = grid_for(ctx, count * width);
#define RB_SCATTER(T, D) if (grad->dtype == D) { \
        if (i32) embedding_scatter_kernel<T, int32_t><<<g, 256, 0, ctx->stream>>>((const T*)pg, (const int32_t*)pi, acc, count, (uint32_t)width, rows, padding_idx); \
        else embedding_scatter_kernel<T, int64_t><<<g, 256, 0, ctx->stream>>>((const T*)pg, (const int64_t*)pi, acc, count, (uint32_t)width, rows, padding_idx); }
    RB_SCATTER(float, RB_F32) RB_SCATTER(bf, RB_BF16) RB_SCATTER(__half, RB_F16)
#undef RB_SCATTER
    RB_TRY(after_launch(ctx, "embedding_backward (scatter)"));
    const bool scale = scale_grad_by_freq != 0;
    if (!f32 || scale) {
        const unsigned gf = grid_for(ctx, out_elems);
        if (f32) embedding_finish_kernel<float><<<gf, 256, 0, ctx->stream>>>(acc, freq, (float*)po, rows, (uint32_t)width, scale);
        else if (out->dtype == RB_BF16) embedding_finish_kernel<bf><<<gf, 256, 0, ctx->stream>>>(acc, freq, (bf*)po, rows, (uint32_t)width, scale);
        else embedding_finish_kernel<__half><<<gf, 256, 0, ctx->stream>>>(acc, freq, (__half*)po, rows, (uint32_t)width, scale);
        RB_TRY(after_launch(ctx, "embedding_backward (finish)"));
    }
    if (ctx->synchronous) {
        int h = 0; cudaMemcpy(&h, bad, sizeof(int), cudaMemcpyDeviceToHost);
        if (h) return fail(RB_INVALID_TENSOR, "embedding id outside [0, weight rows)");
    }
    return RB_OK;
}

int32_t rb_copy(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* y) {
    RB_TRY(check_ctx(ctx));
    void *px, *py;
    RB_TRY(resolve(ctx, x, "copy input", &px)); RB_TRY(resolve(ctx, y, "copy output", &py));
    if (!same_shape(x, y) || x->dtype != y->dtype) return fail(RB_INVALID_TENSOR, "copy keeps shape and dtype");
    const uint64_t bytes = elements(x) * dtype_size(x->dtype);
    RB_TRY(no_overlap(py, bytes, px, bytes, "copy"));
    if (bytes == 0) return empty_call(ctx);
    RB_CUDA(ctx, "cudaMemcpyAsync", cudaMemcpyAsync(py, px, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return empty_call(ctx);
}

int32_t rb_resize_prefix(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* y) {
    RB_TRY(check_ctx(ctx));
    void *px, *py;
    RB_TRY(resolve(ctx, x, "prefix resize input", &px)); RB_TRY(resolve(ctx, y, "prefix resize output", &py));
    bool ok = x->rank == y->rank && x->rank >= 1 && x->rank <= 8 && x->dtype == y->dtype && (x->dtype == RB_F32 || x->dtype == RB_BF16);
    for (uint32_t a = 0; ok && a < x->rank; ++a) ok = x->shape[a] > 0 && y->shape[a] > 0;
    if (!ok) return fail(RB_INVALID_TENSOR, "prefix resize requires positive matching-rank FP32/BF16 layouts of the same dtype");
    const uint64_t total = elements(y), es = dtype_size(x->dtype);
    RB_TRY(no_overlap(py, total * es, px, elements(x) * es, "prefix resize"));
    ResizeDims d{}; d.rank = x->rank;
    for (uint32_t a = 0; a < x->rank; ++a) { d.src[a] = x->shape[a]; d.dst[a] = y->shape[a]; }
    if (x->dtype == RB_F32) resize_prefix_kernel<float><<<grid_for(ctx, total), 256, 0, ctx->stream>>>((const float*)px, (float*)py, total, d);
    else resize_prefix_kernel<uint16_t><<<grid_for(ctx, total), 256, 0, ctx->stream>>>((const uint16_t*)px, (uint16_t*)py, total, d);
    return after_launch(ctx, "resize_prefix");
}

}  // extern "C"
