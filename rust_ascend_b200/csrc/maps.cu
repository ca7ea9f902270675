// Element maps of the dense-transformer path: SiLU*up, bias/residual add, rotary encodings, KV-head
// repetition, causal mask, dtype casts and embedding lookup.
//
// Each kernel restates the per-element formula of the reference IR builders (cited per kernel) with
// separately rounded FP32 operations.  All of them are pure streaming kernels: 16-byte loads/stores
// where the shapes allow it, a grid sized to a multiple of the SM count and a grid-stride loop.
#include "common.cuh"

namespace {

using bf = __nv_bfloat16;

__device__ __forceinline__ float ld(const float* p, uint64_t i) { return p[i]; }
__device__ __forceinline__ float ld(const bf* p, uint64_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ float ld(const __half* p, uint64_t i) { return __half2float(p[i]); }
__device__ __forceinline__ void st(float* p, uint64_t i, float v) { p[i] = v; }
__device__ __forceinline__ void st(bf* p, uint64_t i, float v) { p[i] = __float2bfloat16_rn(v); }
__device__ __forceinline__ void st(__half* p, uint64_t i, float v) { p[i] = __float2half_rn(v); }

// programs.rs:25,41: s = 1/(1+exp(-x)); h = x*s; y = h*up.
__device__ __forceinline__ float silu_mul_f(float g, float u) {
    float s = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g)));
    return __fmul_rn(__fmul_rn(g, s), u);
}

template <typename T, int VEC>
struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };

template <typename T>
__global__ void __launch_bounds__(256) silu_mul_kernel(const T* g, const T* u, T* y, uint64_t n, bool vec) {
    constexpr int V = 16 / sizeof(T);
    uint64_t tid = (uint64_t)blockIdx.x * 256 + threadIdx.x, stride = (uint64_t)gridDim.x * 256;
    if (vec) {
        for (uint64_t i = tid; i < n / V; i += stride) {
            Pack<T, V> a = reinterpret_cast<const Pack<T, V>*>(g)[i], b = reinterpret_cast<const Pack<T, V>*>(u)[i], o;
#pragma unroll
            for (int j = 0; j < V; ++j) st(o.v, j, silu_mul_f(ld(a.v, j), ld(b.v, j)));
            reinterpret_cast<Pack<T, V>*>(y)[i] = o;
        }
        for (uint64_t i = (n / V) * V + tid; i < n; i += stride) st(y, i, silu_mul_f(ld(g, i), ld(u, i)));
    } else {
        for (uint64_t i = tid; i < n; i += stride) st(y, i, silu_mul_f(ld(g, i), ld(u, i)));
    }
}

// affine_programs.rs:31-36: value = x; value += residual (optional); value += bias[col].
template <typename T>
__global__ void __launch_bounds__(256) bias_add_kernel(const T* x, const T* bias, const T* res, T* y, uint64_t n, uint32_t width) {
    uint64_t stride = (uint64_t)gridDim.x * 256;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
        float v = ld(x, i);
        if (res) v = __fadd_rn(v, ld(res, i));
        st(y, i, __fadd_rn(v, ld(bias, i % width)));
    }
}
template <typename T>
__global__ void __launch_bounds__(256) add_kernel(const T* a, const T* b, T* y, uint64_t n, bool vec) {
    constexpr int V = 16 / sizeof(T);
    uint64_t tid = (uint64_t)blockIdx.x * 256 + threadIdx.x, stride = (uint64_t)gridDim.x * 256;
    uint64_t done = 0;
    if (vec) {
        for (uint64_t i = tid; i < n / V; i += stride) {
            Pack<T, V> p = reinterpret_cast<const Pack<T, V>*>(a)[i], q = reinterpret_cast<const Pack<T, V>*>(b)[i], o;
#pragma unroll
            for (int j = 0; j < V; ++j) st(o.v, j, __fadd_rn(ld(p.v, j), ld(q.v, j)));
            reinterpret_cast<Pack<T, V>*>(y)[i] = o;
        }
        done = (n / V) * V;
    }
    for (uint64_t i = done + tid; i < n; i += stride) st(y, i, __fadd_rn(ld(a, i), ld(b, i)));
}

// rotary_programs.rs:63-93 and :101-156.  y = x*cos + ((x_pair*sin)*sign), sign = 2*side-1; the
// transpose Jacobian subtracts.  Columns >= p copy the input bits.  Table rows broadcast over the
// leading axes whose table extent is one.
struct RotaryArgs {
    uint64_t n; uint32_t width, p, rank; int layout, backward;
    uint32_t in_shape[8]; uint32_t table_shape[8];
};
template <typename T>
__global__ void __launch_bounds__(256) rotary_kernel(const T* x, const float* cs, const float* sn, T* y, RotaryArgs a) {
    const uint32_t half = a.p / 2;
    uint64_t stride = (uint64_t)gridDim.x * 256;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < a.n; i += stride) {
        uint64_t row = i / a.width; uint32_t col = (uint32_t)(i % a.width);
        if (col >= a.p) { y[i] = x[i]; continue; }
        uint64_t trow = 0, tstride = 1, rem = row;
        for (int axis = (int)a.rank - 2; axis >= 0; --axis) {
            uint64_t coord = rem % a.in_shape[axis]; rem /= a.in_shape[axis];
            if (a.table_shape[axis] != 1) trow += coord * tstride;
            tstride *= a.table_shape[axis];
        }
        uint32_t pc, pair, side;
        if (a.layout == RB_ROTARY_INTERLEAVED) { pair = col / 2; pc = pair * 2 + ((col + 1) & 1); side = col & 1; }
        else { pc = (col + half) % a.p; pair = col % half; side = col / half; }
        float sign = __fsub_rn(__fmul_rn((float)side, 2.0f), 1.0f);
        float c = cs[trow * half + pair], s = sn[trow * half + pair];
        float direct = __fmul_rn(ld(x, i), c);
        float rot = __fmul_rn(__fmul_rn(ld(x, row * a.width + pc), s), sign);
        st(y, i, a.backward ? __fsub_rn(direct, rot) : __fadd_rn(direct, rot));
    }
}

// heads_programs.rs:43-55: Y[b,h,n,d] = X[b, h/(Hq/Hkv), n, d]; words are copied, never interpreted.
template <typename W>
__global__ void __launch_bounds__(256) repeat_kv_kernel(const W* x, W* y, uint64_t out_words, uint64_t plane_words,
                                                       uint32_t q_heads, uint32_t kv_heads) {
    const uint32_t group = q_heads / kv_heads;
    uint64_t stride = (uint64_t)gridDim.x * 256;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < out_words; i += stride) {
        uint64_t head = i / plane_words, col = i % plane_words;
        uint64_t b = head / q_heads, h = head % q_heads;
        y[i] = x[(b * kv_heads + h / group) * plane_words + col];
    }
}

// mask_programs.rs:19-39: -inf iff key_start+k > query_start+q on u64 positions, else +0.
__global__ void __launch_bounds__(256) causal_mask_kernel(uint32_t* out, uint64_t n, uint32_t queries, uint32_t keys,
                                                         uint64_t query_start, uint64_t key_start) {
    uint64_t stride = (uint64_t)gridDim.x * 256;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
        uint64_t q = query_start + (i / keys) % queries, k = key_start + i % keys;
        out[i] = k > q ? 0xff800000u : 0u;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) div_scalar_kernel(const T* x, T* y, uint64_t n, float divisor) {
    uint64_t stride = (uint64_t)gridDim.x * 256;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) st(y, i, __fdiv_rn(ld(x, i), divisor));
}

template <typename T>
__global__ void __launch_bounds__(256) mul_scalar_kernel(const T* x, T* y, uint64_t n, float factor) {
    uint64_t stride = (uint64_t)gridDim.x * 256;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) st(y, i, __fmul_rn(ld(x, i), factor));
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(256) cast_kernel(const TI* x, TO* y, uint64_t n) {
    uint64_t stride = (uint64_t)gridDim.x * 256;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) st(y, i, ld(x, i));
}

// indexing.rs:33-37: out[i,:] = table[ids[i],:]; rows move as 16-byte words.  An id outside the table
// sets *bad and writes zeros (no fault, no out-of-bounds read); the host reports it.
template <typename I>
__global__ void __launch_bounds__(256) embedding_kernel(const uint4* table, const I* ids, uint4* out, uint64_t count,
                                                       uint32_t row_vecs, uint64_t vocab, int* bad) {
    uint64_t total = count * row_vecs, stride = (uint64_t)gridDim.x * 256;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += stride) {
        uint64_t r = i / row_vecs; uint32_t c = (uint32_t)(i % row_vecs);
        int64_t id = (int64_t)ids[r];
        if (id < 0 || (uint64_t)id >= vocab) { if (c == 0) atomicExch(bad, 1); out[i] = make_uint4(0, 0, 0, 0); continue; }
        out[i] = __ldg(table + (uint64_t)id * row_vecs + c);
    }
}

// The same lookup for rows that are not a multiple of 16 bytes (width 65 FP32 in examples/embedding_tensor.rs:22): rows move
// as 4- or 2-byte words.
template <typename I, typename W>
__global__ void __launch_bounds__(256) embedding_words_kernel(const W* table, const I* ids, W* out, uint64_t count, uint32_t row_words,
                                                             uint64_t vocab, int* bad) {
    uint64_t total = count * row_words, stride = (uint64_t)gridDim.x * 256;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += stride) {
        uint64_t r = i / row_words; uint32_t c = (uint32_t)(i % row_words);
        int64_t id = (int64_t)ids[r];
        if (id < 0 || (uint64_t)id >= vocab) { if (c == 0) atomicExch(bad, 1); out[i] = W(0); continue; }
        out[i] = table[(uint64_t)id * row_words + c];
    }
}

unsigned grid_for(rb_ctx* ctx, uint64_t work_items) {
    uint64_t blocks = (work_items + 255) / 256, cap = (uint64_t)ctx->sm_count * 16;
    return (unsigned)(blocks < cap ? (blocks ? blocks : 1) : cap);
}

}  // namespace

using namespace rb;

extern "C" {

int32_t rb_silu_mul(rb_ctx* ctx, const rb_tensor* gate, const rb_tensor* up, const rb_tensor* y) {
    RB_TRY(check_ctx(ctx));
    void *pg, *pu, *py;
    RB_TRY(resolve(ctx, gate, "SiLU*up gate", &pg)); RB_TRY(resolve(ctx, up, "SiLU*up up", &pu)); RB_TRY(resolve(ctx, y, "SiLU*up output", &py));
    if (!same_shape(gate, up) || !same_shape(gate, y) || gate->dtype != up->dtype || gate->dtype != y->dtype)
        return fail(RB_INVALID_TENSOR, "SiLU*up requires equal-shaped tensors of one dtype");
    uint64_t n = elements(gate);
    if (n > 0xffffffffull) return fail(RB_INVALID_TENSOR, "SiLU*up element count exceeds u32");
    uint64_t bytes = n * dtype_size(gate->dtype);
    RB_TRY(no_overlap(py, bytes, pg, bytes, "SiLU*up")); RB_TRY(no_overlap(py, bytes, pu, bytes, "SiLU*up"));
    if (n == 0) return empty_call(ctx);
    if (gate->dtype == RB_F32) silu_mul_kernel<float><<<grid_for(ctx, n / 4 + 1), 256, 0, ctx->stream>>>((const float*)pg, (const float*)pu, (float*)py, n, true);
    else if (gate->dtype == RB_BF16) silu_mul_kernel<bf><<<grid_for(ctx, n / 8 + 1), 256, 0, ctx->stream>>>((const bf*)pg, (const bf*)pu, (bf*)py, n, true);
    else return fail(RB_INVALID_TENSOR, "SiLU*up supports F32 and BF16 storage");
    return after_launch(ctx, "silu_mul");
}

int32_t rb_bias_add(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* bias, const rb_tensor* residual, const rb_tensor* y) {
    RB_TRY(check_ctx(ctx));
    void *px, *pb, *pr, *py;
    RB_TRY(resolve(ctx, x, "bias add input", &px)); RB_TRY(resolve(ctx, bias, "bias add bias", &pb));
    RB_TRY(resolve(ctx, residual, "bias add residual", &pr, true)); RB_TRY(resolve(ctx, y, "bias add output", &py));
    uint64_t rows, width; rows_width(x, &rows, &width);
    if (width == 0) return fail(RB_INVALID_TENSOR, "bias add requires a positive last-axis width");
    if (!same_shape(x, y) || elements(bias) != width || (residual && !same_shape(x, residual)) || x->dtype != y->dtype ||
        x->dtype != bias->dtype || (residual && residual->dtype != x->dtype))
        return fail(RB_INVALID_TENSOR, "bias add requires X[...,H], bias[H], an optional residual of X's shape and one dtype");
    uint64_t n = rows * width;
    if (n > 0xffffffffull) return fail(RB_INVALID_TENSOR, "bias add complete domain exceeds u32");
    if (n == 0) return empty_call(ctx);
    if (x->dtype == RB_F32) bias_add_kernel<float><<<grid_for(ctx, n), 256, 0, ctx->stream>>>((const float*)px, (const float*)pb, (const float*)pr, (float*)py, n, (uint32_t)width);
    else if (x->dtype == RB_BF16) bias_add_kernel<bf><<<grid_for(ctx, n), 256, 0, ctx->stream>>>((const bf*)px, (const bf*)pb, (const bf*)pr, (bf*)py, n, (uint32_t)width);
    else return fail(RB_INVALID_TENSOR, "bias add supports F32 and BF16 storage");
    return after_launch(ctx, "bias_add");
}

int32_t rb_add(rb_ctx* ctx, const rb_tensor* a, const rb_tensor* b, const rb_tensor* y) {
    RB_TRY(check_ctx(ctx));
    void *pa, *pb, *py;
    RB_TRY(resolve(ctx, a, "add lhs", &pa)); RB_TRY(resolve(ctx, b, "add rhs", &pb)); RB_TRY(resolve(ctx, y, "add output", &py));
    if (!same_shape(a, b) || !same_shape(a, y) || a->dtype != b->dtype || a->dtype != y->dtype)
        return fail(RB_INVALID_TENSOR, "add requires equal-shaped tensors of one dtype");
    uint64_t n = elements(a);
    if (n == 0) return empty_call(ctx);
    // In-place accumulation (y aliasing a or b exactly) is allowed: each element is read before it is written.
    if (a->dtype == RB_F32) add_kernel<float><<<grid_for(ctx, n / 4 + 1), 256, 0, ctx->stream>>>((const float*)pa, (const float*)pb, (float*)py, n, true);
    else if (a->dtype == RB_BF16) add_kernel<bf><<<grid_for(ctx, n / 8 + 1), 256, 0, ctx->stream>>>((const bf*)pa, (const bf*)pb, (bf*)py, n, true);
    else return fail(RB_INVALID_TENSOR, "add supports F32 and BF16 storage");
    return after_launch(ctx, "add");
}

static int32_t rotary_common(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* cos, const rb_tensor* sin, uint32_t p,
                             bool prefix, int32_t layout, int32_t backward, const rb_tensor* y) {
    RB_TRY(check_ctx(ctx));
    void *px, *pc, *ps, *py;
    RB_TRY(resolve(ctx, x, "rotary input", &px)); RB_TRY(resolve(ctx, cos, "rotary cos", &pc));
    RB_TRY(resolve(ctx, sin, "rotary sin", &ps)); RB_TRY(resolve(ctx, y, "rotary output", &py));
    if (layout != RB_ROTARY_INTERLEAVED && layout != RB_ROTARY_SPLIT_HALF) return fail(RB_INVALID_TENSOR, "unknown rotary layout");
    if (cos->dtype != RB_F32 || sin->dtype != RB_F32 || !same_shape(cos, sin)) return fail(RB_INVALID_TENSOR, "rotary tables must be equal-shaped FP32 tensors");
    if (!same_shape(x, y) || x->dtype != y->dtype) return fail(RB_INVALID_TENSOR, "rotary output must match the input shape and dtype");
    uint32_t rank = x->rank; uint64_t width = x->shape[rank - 1];
    if (!prefix) p = (uint32_t)width;
    if (p == 0 || p % 2 != 0 || p > width)
        return fail(RB_INVALID_TENSOR, prefix ? "rotary prefix requires positive even P<=D, table last axis P/2 and singleton or matching leading axes"
                                              : "rotary requires positive even width, complete rows and elements within u32");
    if (cos->rank != rank || cos->shape[rank - 1] != p / 2) return fail(RB_INVALID_TENSOR, "rotary tables need the input's rank and a last axis of half the rotated width");
    RotaryArgs a{};
    for (uint32_t i = 0; i + 1 < rank; ++i) {
        bool ok = prefix ? (cos->shape[i] == 1 || cos->shape[i] == x->shape[i]) : cos->shape[i] == x->shape[i];
        if (!ok) return fail(RB_INVALID_TENSOR, prefix ? "rotary prefix requires positive even P<=D, table last axis P/2 and singleton or matching leading axes"
                                                        : "rotary tables must have the input shape with the width halved");
        if (x->shape[i] > 0xffffffffull) return fail(RB_INVALID_TENSOR, "rotary axis exceeds u32");
        a.in_shape[i] = (uint32_t)x->shape[i]; a.table_shape[i] = (uint32_t)cos->shape[i];
    }
    uint64_t n = elements(x);
    if (n > 0xffffffffull) return fail(RB_INVALID_TENSOR, "rotary complete domain exceeds u32");
    RB_TRY(no_overlap(py, n * dtype_size(x->dtype), px, n * dtype_size(x->dtype), "rotary"));
    if (n == 0) return empty_call(ctx);
    a.n = n; a.width = (uint32_t)width; a.p = p; a.rank = rank; a.layout = layout; a.backward = backward ? 1 : 0;
    if (x->dtype == RB_F32) rotary_kernel<float><<<grid_for(ctx, n), 256, 0, ctx->stream>>>((const float*)px, (const float*)pc, (const float*)ps, (float*)py, a);
    else if (x->dtype == RB_BF16) rotary_kernel<bf><<<grid_for(ctx, n), 256, 0, ctx->stream>>>((const bf*)px, (const float*)pc, (const float*)ps, (bf*)py, a);
    else return fail(RB_INVALID_TENSOR, "rotary supports F32 and BF16 storage");
    return after_launch(ctx, prefix ? "rotary_prefix" : "rotary");
}

int32_t rb_rotary(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* cos, const rb_tensor* sin, int32_t layout, int32_t backward, const rb_tensor* y) {
    return rotary_common(ctx, x, cos, sin, 0, false, layout, backward, y);
}
int32_t rb_rotary_prefix(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* cos, const rb_tensor* sin, uint32_t width, int32_t layout,
                         int32_t backward, const rb_tensor* y) {
    return rotary_common(ctx, x, cos, sin, width, true, layout, backward, y);
}

int32_t rb_repeat_kv_heads(rb_ctx* ctx, const rb_tensor* x, uint32_t query_heads, const rb_tensor* y) {
    RB_TRY(check_ctx(ctx));
    void *px, *py;
    RB_TRY(resolve(ctx, x, "KV repetition input", &px)); RB_TRY(resolve(ctx, y, "KV repetition output", &py));
    if (x->rank != 4 || y->rank != 4 || x->dtype != y->dtype) return fail(RB_INVALID_TENSOR, "KV repetition requires rank-4 tensors of one dtype");
    uint64_t kv = x->shape[1];
    if (kv == 0 || query_heads == 0 || query_heads % kv != 0)
        return fail(RB_INVALID_TENSOR, "KV repetition requires positive heads and query_heads divisible by kv_heads");
    if (y->shape[0] != x->shape[0] || y->shape[1] != query_heads || y->shape[2] != x->shape[2] || y->shape[3] != x->shape[3])
        return fail(RB_INVALID_TENSOR, "KV repetition output must be [B,Hq,N,D]");
    uint64_t out_elems = elements(y);
    if (out_elems > 0xffffffffull) return fail(RB_INVALID_TENSOR, "KV repetition complete domain exceeds u32");
    size_t es = dtype_size(x->dtype);
    RB_TRY(no_overlap(py, out_elems * es, px, elements(x) * es, "KV repetition"));
    if (out_elems == 0) return empty_call(ctx);
    uint64_t plane_bytes = x->shape[2] * x->shape[3] * es;
    if (plane_bytes % 16 == 0)
        repeat_kv_kernel<uint4><<<grid_for(ctx, out_elems * es / 16), 256, 0, ctx->stream>>>((const uint4*)px, (uint4*)py, out_elems * es / 16, plane_bytes / 16, query_heads, (uint32_t)kv);
    else if (es == 4)
        repeat_kv_kernel<uint32_t><<<grid_for(ctx, out_elems), 256, 0, ctx->stream>>>((const uint32_t*)px, (uint32_t*)py, out_elems, plane_bytes / 4, query_heads, (uint32_t)kv);
    else if (es == 2)
        repeat_kv_kernel<uint16_t><<<grid_for(ctx, out_elems), 256, 0, ctx->stream>>>((const uint16_t*)px, (uint16_t*)py, out_elems, plane_bytes / 2, query_heads, (uint32_t)kv);
    else return fail(RB_INVALID_TENSOR, "KV repetition supports 2- and 4-byte element types");
    return after_launch(ctx, "repeat_kv_heads");
}

int32_t rb_causal_mask(rb_ctx* ctx, uint64_t query_start, uint64_t key_start, const rb_tensor* out) {
    RB_TRY(check_ctx(ctx));
    void* po;
    RB_TRY(resolve(ctx, out, "causal mask output", &po));
    if (out->rank != 3 || out->dtype != RB_F32) return fail(RB_INVALID_TENSOR, "causal mask output must be FP32 [B,Q,K]");
    uint64_t queries = out->shape[1], keys = out->shape[2];
    if (queries == 0 || keys == 0) return fail(RB_INVALID_TENSOR, "causal mask requires positive query/key lengths");
    if (query_start + (queries - 1) < query_start || key_start + (keys - 1) < key_start) return fail(RB_INVALID_TENSOR, "causal absolute position overflow");
    uint64_t n = elements(out);
    if (n > 0xffffffffull) return fail(RB_INVALID_TENSOR, "causal mask domain exceeds u32");
    if (n == 0) return empty_call(ctx);
    causal_mask_kernel<<<grid_for(ctx, n), 256, 0, ctx->stream>>>((uint32_t*)po, n, (uint32_t)queries, (uint32_t)keys, query_start, key_start);
    return after_launch(ctx, "causal_mask");
}

int32_t rb_cast(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* y) {
    RB_TRY(check_ctx(ctx));
    void *px, *py;
    RB_TRY(resolve(ctx, x, "cast input", &px)); RB_TRY(resolve(ctx, y, "cast output", &py));
    if (!same_shape(x, y)) return fail(RB_INVALID_TENSOR, "cast keeps the shape");
    uint64_t n = elements(x);
    RB_TRY(no_overlap(py, n * dtype_size(y->dtype), px, n * dtype_size(x->dtype), "cast"));
    if (n == 0) return empty_call(ctx);
    unsigned g = grid_for(ctx, n);
#define RB_CAST(TI, DI, TO, DO) if (x->dtype == DI && y->dtype == DO) { cast_kernel<TI, TO><<<g, 256, 0, ctx->stream>>>((const TI*)px, (TO*)py, n); return after_launch(ctx, "cast"); }
    RB_CAST(float, RB_F32, bf, RB_BF16) RB_CAST(bf, RB_BF16, float, RB_F32) RB_CAST(float, RB_F32, __half, RB_F16)
    RB_CAST(__half, RB_F16, float, RB_F32) RB_CAST(float, RB_F32, float, RB_F32) RB_CAST(bf, RB_BF16, bf, RB_BF16)
    RB_CAST(__half, RB_F16, bf, RB_BF16) RB_CAST(bf, RB_BF16, __half, RB_F16) RB_CAST(__half, RB_F16, __half, RB_F16)
#undef RB_CAST
    return fail(RB_INVALID_TENSOR, "cast supports FP32, FP16 and BF16");
}

int32_t rb_div_scalar(rb_ctx* ctx, const rb_tensor* x, float divisor, const rb_tensor* y) {
    RB_TRY(check_ctx(ctx));
    void *px, *py;
    RB_TRY(resolve(ctx, x, "div_scalar input", &px)); RB_TRY(resolve(ctx, y, "div_scalar output", &py));
    if (!same_shape(x, y) || x->dtype != y->dtype) return fail(RB_INVALID_TENSOR, "div_scalar keeps shape and dtype");
    uint64_t n = elements(x);
    if (n == 0) return empty_call(ctx);
    if (x->dtype == RB_F32) div_scalar_kernel<float><<<grid_for(ctx, n), 256, 0, ctx->stream>>>((const float*)px, (float*)py, n, divisor);
    else if (x->dtype == RB_BF16) div_scalar_kernel<bf><<<grid_for(ctx, n), 256, 0, ctx->stream>>>((const bf*)px, (bf*)py, n, divisor);
    else if (x->dtype == RB_F16) div_scalar_kernel<__half><<<grid_for(ctx, n), 256, 0, ctx->stream>>>((const __half*)px, (__half*)py, n, divisor);
    else return fail(RB_INVALID_TENSOR, "div_scalar supports FP32, FP16 and BF16");
    return after_launch(ctx, "div_scalar");
}

int32_t rb_mul_scalar(rb_ctx* ctx, const rb_tensor* x, float factor, const rb_tensor* y) {
    RB_TRY(check_ctx(ctx));
    void *px, *py;
    RB_TRY(resolve(ctx, x, "mul_scalar input", &px)); RB_TRY(resolve(ctx, y, "mul_scalar output", &py));
    if (!same_shape(x, y) || x->dtype != y->dtype) return fail(RB_INVALID_TENSOR, "mul_scalar keeps shape and dtype");
    uint64_t n = elements(x);
    if (n == 0) return empty_call(ctx);
    if (x->dtype == RB_F32) mul_scalar_kernel<float><<<grid_for(ctx, n), 256, 0, ctx->stream>>>((const float*)px, (float*)py, n, factor);
    else if (x->dtype == RB_BF16) mul_scalar_kernel<bf><<<grid_for(ctx, n), 256, 0, ctx->stream>>>((const bf*)px, (bf*)py, n, factor);
    else if (x->dtype == RB_F16) mul_scalar_kernel<__half><<<grid_for(ctx, n), 256, 0, ctx->stream>>>((const __half*)px, (__half*)py, n, factor);
    else return fail(RB_INVALID_TENSOR, "mul_scalar supports FP32, FP16 and BF16");
    return after_launch(ctx, "mul_scalar");
}

int32_t rb_embedding(rb_ctx* ctx, const rb_tensor* table, const rb_tensor* ids, const rb_tensor* out) {
    RB_TRY(check_ctx(ctx));
    void *pt, *pi, *po;
    RB_TRY(resolve(ctx, table, "embedding table", &pt)); RB_TRY(resolve(ctx, ids, "embedding ids", &pi)); RB_TRY(resolve(ctx, out, "embedding output", &po));
    if (table->rank != 2 || (ids->dtype != RB_I32 && ids->dtype != RB_I64) || out->dtype != table->dtype)
        return fail(RB_INVALID_TENSOR, "embedding requires a rank-2 table, INT32/INT64 ids and an output of the table's dtype");
    uint64_t count = elements(ids), width = table->shape[1];
    if (out->rank != ids->rank + 1 || out->shape[out->rank - 1] != width || elements(out) != count * width)
        return fail(RB_INVALID_TENSOR, "embedding output must be ids.shape + [width]");
    uint64_t row_bytes = width * dtype_size(table->dtype);
    if (row_bytes == 0 || (table->shape[0] == 0 && count != 0)) return fail(RB_INVALID_TENSOR, "embedding needs a positive width and, for any id, at least one table row");
    if (count == 0) return empty_call(ctx);
    RB_TRY(ensure_workspace(ctx, 256));
    int* bad = (int*)ctx->workspace;
    RB_CUDA(ctx, "cudaMemsetAsync", cudaMemsetAsync(bad, 0, sizeof(int), ctx->stream));
    if (row_bytes % 16 != 0) {
        const bool w4 = row_bytes % 4 == 0;
        const uint32_t words = (uint32_t)(row_bytes / (w4 ? 4 : 2));
        unsigned gw = grid_for(ctx, count * words);
        const bool i32 = ids->dtype == RB_I32;
        if (w4 && i32) embedding_words_kernel<int32_t, uint32_t><<<gw, 256, 0, ctx->stream>>>((const uint32_t*)pt, (const int32_t*)pi, (uint32_t*)po, count, words, table->shape[0], bad);
        else if (w4) embedding_words_kernel<int64_t, uint32_t><<<gw, 256, 0, ctx->stream>>>((const uint32_t*)pt, (const int64_t*)pi, (uint32_t*)po, count, words, table->shape[0], bad);
        else if (i32) embedding_words_kernel<int32_t, uint16_t><<<gw, 256, 0, ctx->stream>>>((const uint16_t*)pt, (const int32_t*)pi, (uint16_t*)po, count, words, table->shape[0], bad);
        else embedding_words_kernel<int64_t, uint16_t><<<gw, 256, 0, ctx->stream>>>((const uint16_t*)pt, (const int64_t*)pi, (uint16_t*)po, count, words, table->shape[0], bad);
        RB_TRY(after_launch(ctx, "embedding"));
        if (ctx->synchronous) {
            int h = 0; cudaMemcpy(&h, bad, sizeof(int), cudaMemcpyDeviceToHost);
            if (h) return fail(RB_INVALID_TENSOR, "embedding id outside [0, vocabulary rows)");
        }
        return RB_OK;
    }
    unsigned g = grid_for(ctx, count * (row_bytes / 16));
    if (ids->dtype == RB_I32) embedding_kernel<int32_t><<<g, 256, 0, ctx->stream>>>((const uint4*)pt, (const int32_t*)pi, (uint4*)po, count, (uint32_t)(row_bytes / 16), table->shape[0], bad);
    else embedding_kernel<int64_t><<<g, 256, 0, ctx->stream>>>((const uint4*)pt, (const int64_t*)pi, (uint4*)po, count, (uint32_t)(row_bytes / 16), table->shape[0], bad);
    RB_TRY(after_launch(ctx, "embedding"));
    if (ctx->synchronous) {
        int h = 0; cudaMemcpy(&h, bad, sizeof(int), cudaMemcpyDeviceToHost);
        if (h) return fail(RB_INVALID_TENSOR, "embedding id outside [0, vocabulary rows)");
    }
    return RB_OK;
}

}  // extern "C"
