// First-order backward programs of the row and map operators (FP32 storage, as in the reference).
//
// Formulas follow the reference IR builders operation by operation: RMSNorm input gradient and weight
// contributions (rust-ascend-compiler/src/ascend/row_programs.rs:189-217, driver loop
// rust-ascend-driver/src/tensor/runtime/normalization.rs:168-186 with the column sum :95-114), Softmax /
// LogSoftmax gradient (row_programs.rs:152-163), SiLU*up gradient (programs.rs:29,43), KV-head gradient
// reduction (heads_programs.rs:59-86) and the bias gradient (runtime/affine.rs).  The kernels are bandwidth
// bound: one block per row with the row statistics reduced in shared memory, and a two-stage column sum
// (row-block partials in the context workspace, then one pass over the partials) in place of the
// reference's log2(rows) pairwise Add launches.
#include "common.cuh"

namespace {

__device__ __forceinline__ float block_sum(float v, float* smem) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) r += smem[w];
    return r;
}

__global__ void __launch_bounds__(256) rms_backward_kernel(const float* x, const float* w, const float* dy, const float* rstd,
                                                          float* dx, float* contrib, uint64_t rows, uint32_t width) {
    __shared__ float smem[8];
    for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float* xr = x + row * width; const float* gr = dy + row * width;
        const float r = rstd[row];
        float acc = 0.f;
        for (uint32_t c = threadIdx.x; c < width; c += 256) acc = acc + __fmul_rn(__fmul_rn(gr[c], w[c]), xr[c]);
        const float mean = __fdiv_rn(block_sum(acc, smem), (float)width);
        const float corr = __fmul_rn(mean, __fmul_rn(r, r));
        for (uint32_t c = threadIdx.x; c < width; c += 256) {
            const float g = __fmul_rn(gr[c], w[c]);
            dx[row * width + c] = __fmul_rn(__fsub_rn(g, __fmul_rn(xr[c], corr)), r);
            contrib[row * width + c] = __fmul_rn(__fmul_rn(xr[c], r), gr[c]);
        }
    }
}

template <bool LOG>
__global__ void __launch_bounds__(256) softmax_backward_kernel(const float* y, const float* dy, float* dx, uint64_t rows, uint32_t width) {
    __shared__ float smem[8];
    for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float* yr = y + row * width; const float* gr = dy + row * width;
        float acc = 0.f;
        for (uint32_t c = threadIdx.x; c < width; c += 256) acc = acc + (LOG ? gr[c] : __fmul_rn(yr[c], gr[c]));
        const float dot = block_sum(acc, smem);
        for (uint32_t c = threadIdx.x; c < width; c += 256)
            dx[row * width + c] = LOG ? __fsub_rn(gr[c], __fmul_rn(expf(yr[c]), dot)) : __fmul_rn(yr[c], __fsub_rn(gr[c], dot));
    }
}

__global__ void __launch_bounds__(256) silu_mul_backward_kernel(const float* gate, const float* up, const float* dy, float* dgate, float* dup, uint64_t n) {
    uint64_t stride = (uint64_t)gridDim.x * 256;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
        const float x = gate[i];
        const float s = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x)));
        const float h = __fmul_rn(x, s);
        const float ds = __fmul_rn(s, __fadd_rn(1.0f, __fmul_rn(x, __fsub_rn(1.0f, s))));
        dgate[i] = __fmul_rn(__fmul_rn(dy[i], up[i]), ds);
        dup[i] = __fmul_rn(dy[i], h);
    }
}

__global__ void __launch_bounds__(256) repeat_kv_backward_kernel(const float* dy, float* dx, uint64_t in_elems, uint64_t plane, uint32_t kv_heads, uint32_t group) {
    uint64_t stride = (uint64_t)gridDim.x * 256;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < in_elems; i += stride) {
        const uint64_t head = i / plane, col = i % plane, b = head / kv_heads, kv = head % kv_heads;
        const float* src = dy + ((b * kv_heads + kv) * group) * plane + col;
        float acc = src[0];
        for (uint32_t r = 1; r < group; ++r) acc = acc + src[(uint64_t)r * plane];
        dx[i] = acc;
    }
}

// Column sum, stage 1: block (x: 32-column tile, y: row slab) adds its rows; stage 2 adds the slabs.
constexpr int COL_SLAB = 256;   // rows per partial
__global__ void __launch_bounds__(256) column_partial_kernel(const float* x, float* partial, uint64_t rows, uint32_t width) {
    __shared__ float tile[8][33];
    const uint32_t col = blockIdx.x * 32 + (threadIdx.x & 31), lane_row = threadIdx.x >> 5;
    const uint64_t r0 = (uint64_t)blockIdx.y * COL_SLAB, r1 = r0 + COL_SLAB < rows ? r0 + COL_SLAB : rows;
    float acc = 0.f;
    if (col < width) for (uint64_t r = r0 + lane_row; r < r1; r += 8) acc = acc + x[r * width + col];
    tile[lane_row][threadIdx.x & 31] = acc;
    __syncthreads();
    if (lane_row == 0 && col < width) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) s += tile[i][threadIdx.x & 31];
        partial[(uint64_t)blockIdx.y * width + col] = s;
    }
}
__global__ void __launch_bounds__(256) column_final_kernel(const float* partial, float* out, uint32_t slabs, uint32_t width) {
    const uint32_t col = blockIdx.x * 256 + threadIdx.x;
    if (col >= width) return;
    float s = 0.f;
    for (uint32_t i = 0; i < slabs; ++i) s += partial[(uint64_t)i * width + col];
    out[col] = s;
}

int32_t column_sum(rb_ctx* ctx, const float* x, uint64_t rows, uint32_t width, float* out, uint8_t* scratch) {
    const uint32_t slabs = (uint32_t)((rows + COL_SLAB - 1) / COL_SLAB);
    float* partial = reinterpret_cast<float*>(scratch);
    dim3 grid((width + 31) / 32, slabs);
    column_partial_kernel<<<grid, 256, 0, ctx->stream>>>(x, partial, rows, width);
    RB_TRY(rb::after_launch(ctx, "column sum (partials)"));
    column_final_kernel<<<(width + 255) / 256, 256, 0, ctx->stream>>>(partial, out, slabs, width);
    return rb::after_launch(ctx, "column sum");
}

int32_t f32_pair(rb_ctx* ctx, const rb_tensor* a, const rb_tensor* b, const char* what, void** pa, void** pb) {
    RB_TRY(rb::resolve(ctx, a, what, pa)); RB_TRY(rb::resolve(ctx, b, what, pb));
    if (a->dtype != RB_F32 || b->dtype != RB_F32 || !rb::same_shape(a, b)) return rb::fail(RB_INVALID_TENSOR, "%s requires equal-shaped contiguous FP32 tensors", what);
    return RB_OK;
}

unsigned row_grid(rb_ctx* ctx, uint64_t rows) { uint64_t cap = (uint64_t)ctx->sm_count * 16; return (unsigned)(rows < cap ? rows : cap); }

}  // namespace

using namespace rb;

extern "C" {

int32_t rb_rms_norm_backward(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* weight, const rb_tensor* grad, const rb_tensor* rstd,
                             const rb_tensor* dx, const rb_tensor* dweight) {
    RB_TRY(check_ctx(ctx));
    void *px, *pg, *pw, *pr, *pdx, *pdw;
    RB_TRY(f32_pair(ctx, x, grad, "RMSNorm backward", &px, &pg)); RB_TRY(f32_pair(ctx, x, dx, "RMSNorm backward", &px, &pdx));
    RB_TRY(f32_pair(ctx, weight, dweight, "RMSNorm backward weight", &pw, &pdw)); RB_TRY(resolve(ctx, rstd, "RMSNorm backward rstd", &pr));
    uint64_t rows, width; rows_width(x, &rows, &width);
    if (width == 0 || elements(weight) != width || rstd->dtype != RB_F32 || elements(rstd) != rows || rows * width > 0xffffffffull)
        return fail(RB_INVALID_TENSOR, "RMSNorm backward buffer shape, stride, dtype or byte length mismatch");
    RB_TRY(no_overlap(pdx, rows * width * 4, px, rows * width * 4, "RMSNorm backward")); RB_TRY(no_overlap(pdx, rows * width * 4, pg, rows * width * 4, "RMSNorm backward"));
    if (rows == 0) {  // empty batches yield a zero weight gradient (runtime/mod.rs:411-413)
        RB_CUDA(ctx, "cudaMemsetAsync", cudaMemsetAsync(pdw, 0, width * 4, ctx->stream));
        return empty_call(ctx);
    }
    const uint64_t slabs = (rows + COL_SLAB - 1) / COL_SLAB;
    RB_TRY(ensure_workspace(ctx, 1024 + (rows + slabs) * width * 4));
    uint8_t* ws = static_cast<uint8_t*>(ctx->workspace) + 1024;
    float* contrib = reinterpret_cast<float*>(ws);
    rms_backward_kernel<<<row_grid(ctx, rows), 256, 0, ctx->stream>>>((const float*)px, (const float*)pw, (const float*)pg, (const float*)pr,
                                                                   (float*)pdx, contrib, rows, (uint32_t)width);
    RB_TRY(after_launch(ctx, "rms_norm_backward"));
    return column_sum(ctx, contrib, rows, (uint32_t)width, (float*)pdw, ws + rows * width * 4);
}

int32_t rb_softmax_backward(rb_ctx* ctx, const rb_tensor* output, const rb_tensor* grad, int32_t logarithmic, const rb_tensor* dx) {
    RB_TRY(check_ctx(ctx));
    void *py, *pg, *pdx;
    RB_TRY(f32_pair(ctx, output, grad, "Softmax backward", &py, &pg)); RB_TRY(f32_pair(ctx, output, dx, "Softmax backward", &py, &pdx));
    uint64_t rows, width; rows_width(output, &rows, &width);
    if (width == 0 || rows * width > 0xffffffffull) return fail(RB_INVALID_TENSOR, "Softmax backward requires a positive last dimension and elements within u32");
    RB_TRY(no_overlap(pdx, rows * width * 4, py, rows * width * 4, "Softmax backward")); RB_TRY(no_overlap(pdx, rows * width * 4, pg, rows * width * 4, "Softmax backward"));
    if (rows == 0) return empty_call(ctx);
    if (logarithmic) softmax_backward_kernel<true><<<row_grid(ctx, rows), 256, 0, ctx->stream>>>((const float*)py, (const float*)pg, (float*)pdx, rows, (uint32_t)width);
    else softmax_backward_kernel<false><<<row_grid(ctx, rows), 256, 0, ctx->stream>>>((const float*)py, (const float*)pg, (float*)pdx, rows, (uint32_t)width);
    return after_launch(ctx, logarithmic ? "log_softmax_backward" : "softmax_backward");
}

int32_t rb_silu_mul_backward(rb_ctx* ctx, const rb_tensor* gate, const rb_tensor* up, const rb_tensor* grad, const rb_tensor* dgate, const rb_tensor* dup) {
    RB_TRY(check_ctx(ctx));
    void *pg, *pu, *pd, *pdg, *pdu;
    RB_TRY(f32_pair(ctx, gate, up, "SiLU*up backward", &pg, &pu)); RB_TRY(f32_pair(ctx, gate, grad, "SiLU*up backward", &pg, &pd));
    RB_TRY(f32_pair(ctx, gate, dgate, "SiLU*up backward", &pg, &pdg)); RB_TRY(f32_pair(ctx, gate, dup, "SiLU*up backward", &pg, &pdu));
    const uint64_t n = elements(gate);
    if (n > 0xffffffffull) return fail(RB_INVALID_TENSOR, "SiLU*up backward element count exceeds u32");
    for (void* o : {pdg, pdu}) for (void* i : {pg, pu, pd}) RB_TRY(no_overlap(o, n * 4, i, n * 4, "SiLU*up backward"));
    RB_TRY(no_overlap(pdg, n * 4, pdu, n * 4, "SiLU*up backward"));
    if (n == 0) return empty_call(ctx);
    uint64_t blocks = (n + 255) / 256, cap = (uint64_t)ctx->sm_count * 16;
    silu_mul_backward_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, ctx->stream>>>((const float*)pg, (const float*)pu, (const float*)pd, (float*)pdg, (float*)pdu, n);
    return after_launch(ctx, "silu_mul_backward");
}

int32_t rb_repeat_kv_heads_backward(rb_ctx* ctx, const rb_tensor* grad, uint32_t kv_heads, const rb_tensor* dx) {
    RB_TRY(check_ctx(ctx));
    void *pg, *pdx;
    RB_TRY(resolve(ctx, grad, "KV repetition backward grad", &pg)); RB_TRY(resolve(ctx, dx, "KV repetition backward output", &pdx));
    if (grad->rank != 4 || dx->rank != 4 || grad->dtype != RB_F32 || dx->dtype != RB_F32) return fail(RB_INVALID_TENSOR, "KV repetition backward requires rank-4 FP32 tensors");
    const uint64_t hq = grad->shape[1];
    if (kv_heads == 0 || hq == 0 || hq % kv_heads != 0) return fail(RB_INVALID_TENSOR, "KV repetition requires positive heads and query_heads divisible by kv_heads");
    if (dx->shape[0] != grad->shape[0] || dx->shape[1] != kv_heads || dx->shape[2] != grad->shape[2] || dx->shape[3] != grad->shape[3])
        return fail(RB_INVALID_TENSOR, "KV repetition backward output must be [B,Hkv,N,D]");
    const uint64_t n = elements(dx);
    if (elements(grad) > 0xffffffffull) return fail(RB_INVALID_TENSOR, "KV repetition complete domain exceeds u32");
    RB_TRY(no_overlap(pdx, n * 4, pg, elements(grad) * 4, "KV repetition backward"));
    if (n == 0) return empty_call(ctx);
    uint64_t blocks = (n + 255) / 256, cap = (uint64_t)ctx->sm_count * 16;
    repeat_kv_backward_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, ctx->stream>>>((const float*)pg, (float*)pdx, n, grad->shape[2] * grad->shape[3],
                                                                                                  kv_heads, (uint32_t)(hq / kv_heads));
    return after_launch(ctx, "repeat_kv_heads_backward");
}

int32_t rb_bias_add_backward(rb_ctx* ctx, const rb_tensor* grad, const rb_tensor* dbias) {
    RB_TRY(check_ctx(ctx));
    void *pg, *pb;
    RB_TRY(resolve(ctx, grad, "bias backward grad", &pg)); RB_TRY(resolve(ctx, dbias, "bias backward output", &pb));
    uint64_t rows, width; rows_width(grad, &rows, &width);
    if (grad->dtype != RB_F32 || dbias->dtype != RB_F32 || width == 0 || elements(dbias) != width || rows * width > 0xffffffffull)
        return fail(RB_INVALID_TENSOR, "bias backward requires FP32 dY[...,H] and dBias[H]");
    if (rows == 0) { RB_CUDA(ctx, "cudaMemsetAsync", cudaMemsetAsync(pb, 0, width * 4, ctx->stream)); return empty_call(ctx); }
    const uint64_t slabs = (rows + COL_SLAB - 1) / COL_SLAB;
    RB_TRY(ensure_workspace(ctx, 1024 + slabs * width * 4));
    return column_sum(ctx, (const float*)pg, rows, (uint32_t)width, (float*)pb, static_cast<uint8_t*>(ctx->workspace) + 1024);
}

}  // extern "C"

// ---- LayerNorm backward and the causal-LM loss edge ---------------------------------------------------------
namespace {

// row_programs.rs (LayerNormInputBackward / LayerNormWeightContributions): n=(x-mean)*r; g=dy*w;
// dx=((g-mean(g)) - n*mean(g*n))*r; the weight gradient is the column sum of n*dy, the bias gradient that of dy.
__global__ void __launch_bounds__(256) layer_norm_backward_kernel(const float* x, const float* w, const float* dy, const float* mean, const float* rstd,
                                                                 float* dx, float* contrib, uint64_t rows, uint32_t width) {
    __shared__ float smem[8];
    for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float* xr = x + row * width; const float* gr = dy + row * width;
        const float mu = mean[row], r = rstd[row];
        float acc_g = 0.f, acc_gy = 0.f;
        for (uint32_t c = threadIdx.x; c < width; c += 256) {
            const float n = __fmul_rn(__fsub_rn(xr[c], mu), r), g = __fmul_rn(gr[c], w[c]);
            acc_g = acc_g + g; acc_gy = acc_gy + __fmul_rn(g, n);
        }
        const float mean_g = __fdiv_rn(block_sum(acc_g, smem), (float)width);
        const float mean_gy = __fdiv_rn(block_sum(acc_gy, smem), (float)width);
        for (uint32_t c = threadIdx.x; c < width; c += 256) {
            const float n = __fmul_rn(__fsub_rn(xr[c], mu), r), g = __fmul_rn(gr[c], w[c]);
            dx[row * width + c] = __fmul_rn(__fsub_rn(__fsub_rn(g, mean_g), __fmul_rn(n, mean_gy)), r);
            contrib[row * width + c] = __fmul_rn(n, gr[c]);
        }
    }
}

__device__ __forceinline__ float block_max(float v, float* smem) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = smem[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) r = fmaxf(r, smem[w]);
    return r;
}

// One block per (batch, position).  Scored rows (label present and not ignored) get their log-softmax NLL in
// row_loss and their max / denominator in stats; unscored rows get a zero loss and a zero flag.  A label outside
// [0, vocab) that is not the ignore index raises *bad and is skipped (no out-of-bounds read).
template <typename L>
__global__ void __launch_bounds__(256) cross_entropy_rows_kernel(const float* logits, const L* labels, float* row_loss, float* row_valid, float2* stats,
                                                                uint32_t time, uint32_t vocab, int64_t ignore_index, int shift, int* bad) {
    __shared__ float smem[8];
    const uint64_t row = blockIdx.x;                      // b * time + t
    const uint32_t t = (uint32_t)(row % time);
    bool scored = !(shift && t + 1 == time);
    int64_t label = 0;
    if (scored) {
        label = (int64_t)labels[row + (shift ? 1 : 0)];
        if (label == ignore_index) scored = false;
        else if (label < 0 || label >= (int64_t)vocab) { scored = false; if (threadIdx.x == 0) atomicExch(bad, 1); }
    }
    if (!scored) {                                        // uniform per block
        if (threadIdx.x == 0) { row_loss[row] = 0.f; row_valid[row] = 0.f; stats[row] = make_float2(0.f, 1.f); }
        return;
    }
    const float* x = logits + row * vocab;
    float m = -INFINITY;
    for (uint32_t c = threadIdx.x; c < vocab; c += 256) m = fmaxf(m, x[c]);
    m = block_max(m, smem);
    float acc = 0.f;
    for (uint32_t c = threadIdx.x; c < vocab; c += 256) acc = acc + expf(__fsub_rn(x[c], m));
    const float d = block_sum(acc, smem);
    if (threadIdx.x == 0) {
        row_loss[row] = -__fsub_rn(__fsub_rn(x[label], m), logf(d));   // -(log-softmax at the label)
        row_valid[row] = 1.f;
        stats[row] = make_float2(m, d);
    }
}
// Deterministic sum of the per-row losses and flags by one block.
__global__ void __launch_bounds__(256) cross_entropy_reduce_kernel(const float* row_loss, const float* row_valid, uint64_t rows, float* loss_sum, float* valid) {
    __shared__ float smem[8];
    float a = 0.f, b = 0.f;
    for (uint64_t r = threadIdx.x; r < rows; r += 256) { a += row_loss[r]; b += row_valid[r]; }
    a = block_sum(a, smem); b = block_sum(b, smem);
    if (threadIdx.x == 0) { *loss_sum = a; *valid = b; }
}
template <typename L>
__global__ void __launch_bounds__(256) cross_entropy_grad_kernel(const float* logits, const L* labels, const float* row_valid, const float2* stats,
                                                                const float* valid, float upstream, float* dlogits, uint32_t vocab, int shift) {
    const uint64_t row = blockIdx.x;
    float* d = dlogits + row * vocab;
    if (row_valid[row] == 0.f) { for (uint32_t c = threadIdx.x; c < vocab; c += 256) d[c] = 0.f; return; }
    const float count = fmaxf(*valid, 1.f);
    const float k = __fdiv_rn(upstream, count);
    const float2 st = stats[row];
    const int64_t label = (int64_t)labels[row + (shift ? 1 : 0)];
    const float* x = logits + row * vocab;
    for (uint32_t c = threadIdx.x; c < vocab; c += 256) {
        const float p = __fdiv_rn(expf(__fsub_rn(x[c], st.x)), st.y);
        d[c] = __fmul_rn(__fsub_rn(p, (int64_t)c == label ? 1.f : 0.f), k);
    }
}

}  // namespace

extern "C" {

int32_t rb_layer_norm_backward(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* weight, const rb_tensor* grad, const rb_tensor* mean,
                               const rb_tensor* rstd, const rb_tensor* dx, const rb_tensor* dweight, const rb_tensor* dbias) {
    RB_TRY(check_ctx(ctx));
    void *px, *pg, *pw, *pm, *pr, *pdx, *pdw, *pdb;
    RB_TRY(f32_pair(ctx, x, grad, "LayerNorm backward", &px, &pg)); RB_TRY(f32_pair(ctx, x, dx, "LayerNorm backward", &px, &pdx));
    RB_TRY(f32_pair(ctx, weight, dweight, "LayerNorm backward weight", &pw, &pdw)); RB_TRY(f32_pair(ctx, weight, dbias, "LayerNorm backward bias", &pw, &pdb));
    RB_TRY(f32_pair(ctx, mean, rstd, "LayerNorm backward statistics", &pm, &pr));
    uint64_t rows, width; rows_width(x, &rows, &width);
    if (width == 0 || elements(weight) != width || elements(mean) != rows || rows * width > 0xffffffffull)
        return fail(RB_INVALID_TENSOR, "LayerNorm backward buffer shape, stride, dtype or byte length mismatch");
    RB_TRY(no_overlap(pdx, rows * width * 4, px, rows * width * 4, "LayerNorm backward")); RB_TRY(no_overlap(pdx, rows * width * 4, pg, rows * width * 4, "LayerNorm backward"));
    if (rows == 0) {
        RB_CUDA(ctx, "cudaMemsetAsync", cudaMemsetAsync(pdw, 0, width * 4, ctx->stream));
        RB_CUDA(ctx, "cudaMemsetAsync", cudaMemsetAsync(pdb, 0, width * 4, ctx->stream));
        return empty_call(ctx);
    }
    const uint64_t slabs = (rows + COL_SLAB - 1) / COL_SLAB;
    RB_TRY(ensure_workspace(ctx, 1024 + (rows + slabs) * width * 4));
    uint8_t* ws = static_cast<uint8_t*>(ctx->workspace) + 1024;
    float* contrib = reinterpret_cast<float*>(ws);
    layer_norm_backward_kernel<<<row_grid(ctx, rows), 256, 0, ctx->stream>>>((const float*)px, (const float*)pw, (const float*)pg, (const float*)pm,
                                                                           (const float*)pr, (float*)pdx, contrib, rows, (uint32_t)width);
    RB_TRY(after_launch(ctx, "layer_norm_backward"));
    RB_TRY(column_sum(ctx, contrib, rows, (uint32_t)width, (float*)pdw, ws + rows * width * 4));
    return column_sum(ctx, (const float*)pg, rows, (uint32_t)width, (float*)pdb, ws + rows * width * 4);
}

int32_t rb_causal_cross_entropy(rb_ctx* ctx, const rb_tensor* logits, const rb_tensor* labels, int64_t ignore_index, int32_t shift,
                                float upstream, const rb_tensor* loss_sum, const rb_tensor* valid_tokens, const rb_tensor* dlogits) {
    RB_TRY(check_ctx(ctx));
    void *pl, *plab, *ps, *pv, *pd = nullptr;
    RB_TRY(resolve(ctx, logits, "causal loss logits", &pl)); RB_TRY(resolve(ctx, labels, "causal loss labels", &plab));
    RB_TRY(resolve(ctx, loss_sum, "causal loss sum", &ps)); RB_TRY(resolve(ctx, valid_tokens, "causal loss valid count", &pv));
    RB_TRY(resolve(ctx, dlogits, "causal loss gradient", &pd, true));
    if (logits->rank != 3 || labels->rank != 2 || logits->dtype != RB_F32 || (labels->dtype != RB_I32 && labels->dtype != RB_I64) ||
        labels->shape[0] != logits->shape[0] || labels->shape[1] != logits->shape[1])
        return fail(RB_INVALID_TENSOR, "causal loss requires same-device FP32 hidden and I32/I64 labels with matching batch and sequence");
    if (loss_sum->dtype != RB_F32 || valid_tokens->dtype != RB_F32 || elements(loss_sum) != 1 || elements(valid_tokens) != 1)
        return fail(RB_INVALID_TENSOR, "causal loss sum and valid count are FP32 [1]");
    if (dlogits && (dlogits->dtype != RB_F32 || !same_shape(dlogits, logits))) return fail(RB_INVALID_TENSOR, "causal loss gradient must match the logits");
    const uint64_t batch = logits->shape[0], time = logits->shape[1], vocab = logits->shape[2], rows = batch * time;
    if (vocab == 0 || vocab > 0xffffffffull || rows * vocab > 0xffffffffull || rows > 0x7fffffffull)
        return fail(RB_INVALID_TENSOR, "causal projection requires a positive vocabulary and logits within u32");
    if (pd) RB_TRY(no_overlap(pd, rows * vocab * 4, pl, rows * vocab * 4, "causal loss"));
    if (rows == 0) {
        RB_CUDA(ctx, "cudaMemsetAsync", cudaMemsetAsync(ps, 0, 4, ctx->stream)); RB_CUDA(ctx, "cudaMemsetAsync", cudaMemsetAsync(pv, 0, 4, ctx->stream));
        return empty_call(ctx);
    }
    RB_TRY(ensure_workspace(ctx, 1024 + rows * 16));
    uint8_t* ws = static_cast<uint8_t*>(ctx->workspace);
    int* bad = reinterpret_cast<int*>(ws);
    float* row_loss = reinterpret_cast<float*>(ws + 1024);
    float* row_valid = row_loss + rows;
    float2* stats = reinterpret_cast<float2*>(row_valid + rows);
    RB_CUDA(ctx, "cudaMemsetAsync", cudaMemsetAsync(bad, 0, sizeof(int), ctx->stream));
    const bool wide = labels->dtype == RB_I64;
    if (wide) cross_entropy_rows_kernel<int64_t><<<(unsigned)rows, 256, 0, ctx->stream>>>((const float*)pl, (const int64_t*)plab, row_loss, row_valid, stats, (uint32_t)time, (uint32_t)vocab, ignore_index, shift, bad);
    else cross_entropy_rows_kernel<int32_t><<<(unsigned)rows, 256, 0, ctx->stream>>>((const float*)pl, (const int32_t*)plab, row_loss, row_valid, stats, (uint32_t)time, (uint32_t)vocab, ignore_index, shift, bad);
    RB_TRY(after_launch(ctx, "causal_cross_entropy (rows)"));
    cross_entropy_reduce_kernel<<<1, 256, 0, ctx->stream>>>(row_loss, row_valid, rows, (float*)ps, (float*)pv);
    RB_TRY(after_launch(ctx, "causal_cross_entropy (sum)"));
    if (pd) {
        if (wide) cross_entropy_grad_kernel<int64_t><<<(unsigned)rows, 256, 0, ctx->stream>>>((const float*)pl, (const int64_t*)plab, row_valid, stats, (const float*)pv, upstream, (float*)pd, (uint32_t)vocab, shift);
        else cross_entropy_grad_kernel<int32_t><<<(unsigned)rows, 256, 0, ctx->stream>>>((const float*)pl, (const int32_t*)plab, row_valid, stats, (const float*)pv, upstream, (float*)pd, (uint32_t)vocab, shift);
        RB_TRY(after_launch(ctx, "causal_cross_entropy (gradient)"));
    }
    if (ctx->synchronous) {
        int h = 0; cudaMemcpy(&h, bad, sizeof(int), cudaMemcpyDeviceToHost);
        if (h) return fail(RB_INVALID_TENSOR, "causal loss label outside [0, vocabulary) and not the ignore index");
    }
    return RB_OK;
}

}  // extern "C"
