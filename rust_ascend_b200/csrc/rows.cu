// Last-axis row programs: RMSNorm, LayerNorm, Softmax / LogSoftmax, Sum / Mean / Max.
//
// Arithmetic follows rust-ascend-compiler/src/ascend/row_programs.rs:108-220 operation by operation
// (separately rounded multiply/add, division for the softmax quotient, 1/sqrt for the inverse root);
// only the summation tree differs, which the reference leaves unspecified for its 32-lane reduction.
//
// These kernels are HBM-bound.  The fast path keeps one whole row in registers: each thread owns up to
// four 16-byte vectors at a stride of the row's thread count, so a warp reads 512 contiguous bytes per
// load, the row is read from HBM exactly once and written exactly once.  Rows wider than 16384 elements
// or not a multiple of four fall back to a multi-pass kernel whose re-reads hit L2.
#include "common.cuh"

namespace {

enum RowOp { OP_RMS = 0, OP_LAYER = 1, OP_SOFTMAX = 2, OP_LOGSOFTMAX = 3, OP_SUM = 4, OP_MEAN = 5, OP_MAX = 6, OP_ADD_RMS = 7 };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Four consecutive elements as FP32.
__device__ __forceinline__ void load4(const float* p, float (&v)[4], bool streaming) {
    float4 t = streaming ? __ldcs(reinterpret_cast<const float4*>(p)) : __ldg(reinterpret_cast<const float4*>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4], bool streaming) {
    uint2 t = streaming ? __ldcs(reinterpret_cast<const uint2*>(p)) : __ldg(reinterpret_cast<const uint2*>(p));
    v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
    v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
    __stcs(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3]));
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&v)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 t; t.x = *reinterpret_cast<uint32_t*>(&a); t.y = *reinterpret_cast<uint32_t*>(&b);
    __stcs(reinterpret_cast<uint2*>(p), t);
}

template <bool MAX> __device__ __forceinline__ float combine(float a, float b) { return MAX ? fmaxf(a, b) : a + b; }

// Reduction over the THREADS threads that share threadIdx.y.  THREADS is a multiple of 32.
template <int THREADS, bool MAX>
__device__ __forceinline__ float row_reduce(float v, float* smem /* [rows_per_block][THREADS/32] */) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = combine<MAX>(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (THREADS == 32) return v;
    constexpr int WARPS = THREADS / 32;
    float* s = smem + threadIdx.y * WARPS;
    __syncthreads();  // protect smem against the previous reduction's readers
    if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = s[0];
#pragma unroll
    for (int w = 1; w < WARPS; ++w) r = combine<MAX>(r, s[w]);
    return r;
}

struct RowArgs {
    const void* x; const void* w; const void* b; void* y; float* stat0; float* stat1;
    uint64_t rows; uint32_t width; float eps;
    const void* delta = nullptr;   // fused residual: x <- x + delta (stored to x_out in x's type) before the norm
    void* x_out = nullptr;
};

constexpr int MAXV = 4;  // 16-byte vectors per thread on the register-resident path

template <int OP, typename TIn, typename TOut, typename TW, int THREADS>
__global__ void __launch_bounds__(THREADS * (THREADS >= 256 ? 1 : 256 / THREADS))
row_kernel(RowArgs a) {
    constexpr int ROWS = THREADS >= 256 ? 1 : 256 / THREADS;
    __shared__ float smem[ROWS * (THREADS / 32) + 1];
    const uint32_t width = a.width;
    const uint64_t row0 = (uint64_t)blockIdx.x * ROWS + threadIdx.y;
    const uint64_t stride = (uint64_t)gridDim.x * ROWS;
    const float inv_width = 0.f;  (void)inv_width;
    for (uint64_t row = row0; row - threadIdx.y < a.rows; row += stride) {
        // Every thread of the block must reach the barriers inside row_reduce, so rows past the end
        // are processed with `live == false` instead of leaving the loop early.
        const bool live = row < a.rows;
        const TIn* xr = static_cast<const TIn*>(a.x) + (live ? row : 0) * width;
        float v[MAXV][4];
        bool have[MAXV];
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            uint32_t c = (i * THREADS + threadIdx.x) * 4;
            have[i] = live && c < width;
            if (have[i]) load4(xr + c, v[i], true);
            else { v[i][0] = v[i][1] = v[i][2] = v[i][3] = 0.f; }
        }
        if (OP == OP_ADD_RMS) {
            // residual stream update fused into the norm (its own instantiation, so the plain norm keeps its four
            // loads in flight): the sum is rounded to the storage type first, so the normalised value is computed
            // from exactly what a separate add kernel would have stored
            float d[MAXV][4];
#pragma unroll
            for (int i = 0; i < MAXV; ++i) {
                uint32_t c = (i * THREADS + threadIdx.x) * 4;
                if (have[i]) load4(static_cast<const TIn*>(a.delta) + row * width + c, d[i], true);
            }
#pragma unroll
            for (int i = 0; i < MAXV; ++i) if (have[i]) {
                uint32_t c = (i * THREADS + threadIdx.x) * 4;
#pragma unroll
                for (int j = 0; j < 4; ++j) v[i][j] = to_f32(from_f32<TIn>(__fadd_rn(v[i][j], d[i][j])));
                store4(static_cast<TIn*>(a.x_out) + row * width + c, v[i]);
            }
        }
        if (OP == OP_RMS || OP == OP_ADD_RMS) {
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < MAXV; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc = acc + __fmul_rn(v[i][j], v[i][j]);
            float sum = row_reduce<THREADS, false>(acc, smem);
            float mean = __fdiv_rn(sum, (float)width);
            float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, a.eps)));
            TOut* yr = static_cast<TOut*>(a.y) + row * width;
#pragma unroll
            for (int i = 0; i < MAXV; ++i) if (have[i]) {
                uint32_t c = (i * THREADS + threadIdx.x) * 4;
                float wv[4]; load4(static_cast<const TW*>(a.w) + c, wv, false);
                float o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) o[j] = __fmul_rn(__fmul_rn(v[i][j], r), wv[j]);
                store4(yr + c, o);
            }
            if (live && threadIdx.x == 0 && a.stat0) a.stat0[row] = r;
        } else if (OP == OP_LAYER) {
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < MAXV; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc = acc + v[i][j];
            float mean = __fdiv_rn(row_reduce<THREADS, false>(acc, smem), (float)width);
            acc = 0.f;
#pragma unroll
            for (int i = 0; i < MAXV; ++i) if (have[i])
#pragma unroll
                for (int j = 0; j < 4; ++j) { v[i][j] = __fsub_rn(v[i][j], mean); acc = acc + __fmul_rn(v[i][j], v[i][j]); }
            float var = __fdiv_rn(row_reduce<THREADS, false>(acc, smem), (float)width);
            float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, a.eps)));
            TOut* yr = static_cast<TOut*>(a.y) + row * width;
#pragma unroll
            for (int i = 0; i < MAXV; ++i) if (have[i]) {
                uint32_t c = (i * THREADS + threadIdx.x) * 4;
                float wv[4], bv[4] = {0.f, 0.f, 0.f, 0.f};
                load4(static_cast<const TW*>(a.w) + c, wv, false);
                if (a.b) load4(static_cast<const TW*>(a.b) + c, bv, false);
                float o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) o[j] = __fadd_rn(__fmul_rn(__fmul_rn(v[i][j], r), wv[j]), bv[j]);
                store4(yr + c, o);
            }
            if (live && threadIdx.x == 0) { if (a.stat0) a.stat0[row] = mean; if (a.stat1) a.stat1[row] = r; }
        } else if (OP == OP_SOFTMAX || OP == OP_LOGSOFTMAX) {
            float m = -INFINITY;
#pragma unroll
            for (int i = 0; i < MAXV; ++i) if (have[i])
#pragma unroll
                for (int j = 0; j < 4; ++j) m = fmaxf(m, v[i][j]);
            m = row_reduce<THREADS, true>(m, smem);
            float acc = 0.f;
            float e[MAXV][4];
#pragma unroll
            for (int i = 0; i < MAXV; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    v[i][j] = __fsub_rn(v[i][j], m);
                    e[i][j] = have[i] ? expf(v[i][j]) : 0.f;
                    acc = acc + e[i][j];
                }
            float d = row_reduce<THREADS, false>(acc, smem);
            float ld = logf(d);
            TOut* yr = static_cast<TOut*>(a.y) + row * width;
#pragma unroll
            for (int i = 0; i < MAXV; ++i) if (have[i]) {
                uint32_t c = (i * THREADS + threadIdx.x) * 4;
                float o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) o[j] = OP == OP_SOFTMAX ? __fdiv_rn(e[i][j], d) : __fsub_rn(v[i][j], ld);
                store4(yr + c, o);
            }
        } else {  // OP_SUM / OP_MEAN / OP_MAX
            constexpr bool MX = OP == OP_MAX;
            float acc = MX ? -INFINITY : 0.f;
#pragma unroll
            for (int i = 0; i < MAXV; ++i) if (have[i])
#pragma unroll
                for (int j = 0; j < 4; ++j) acc = combine<MX>(acc, v[i][j]);
            float s = row_reduce<THREADS, MX>(acc, smem);
            if (OP == OP_MEAN) s = __fdiv_rn(s, (float)width);
            if (live && threadIdx.x == 0) static_cast<TOut*>(a.y)[row] = from_f32<TOut>(s);
        }
    }
}

// Any width: one 256-thread block per row, element-wise loads, statistics recomputed from global
// memory (L2-resident for the second and third pass).
template <int OP, typename TIn, typename TOut, typename TW>
__global__ void __launch_bounds__(256) row_kernel_generic(RowArgs a) {
    __shared__ float smem[9];
    const uint32_t width = a.width;
    for (uint64_t row = blockIdx.x; row < a.rows; row += gridDim.x) {
        const TIn* xr = static_cast<const TIn*>(a.x) + row * width;
        TOut* yr = static_cast<TOut*>(a.y) + row * width;
        if (OP == OP_RMS) {
            float acc = 0.f;
            for (uint32_t c = threadIdx.x; c < width; c += 256) { float x = to_f32(xr[c]); acc = acc + __fmul_rn(x, x); }
            float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(row_reduce<256, false>(acc, smem), (float)width), a.eps)));
            for (uint32_t c = threadIdx.x; c < width; c += 256)
                yr[c] = from_f32<TOut>(__fmul_rn(__fmul_rn(to_f32(xr[c]), r), to_f32(static_cast<const TW*>(a.w)[c])));
            if (threadIdx.x == 0 && a.stat0) a.stat0[row] = r;
        } else if (OP == OP_LAYER) {
            float acc = 0.f;
            for (uint32_t c = threadIdx.x; c < width; c += 256) acc = acc + to_f32(xr[c]);
            float mean = __fdiv_rn(row_reduce<256, false>(acc, smem), (float)width);
            acc = 0.f;
            for (uint32_t c = threadIdx.x; c < width; c += 256) { float d = __fsub_rn(to_f32(xr[c]), mean); acc = acc + __fmul_rn(d, d); }
            float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(row_reduce<256, false>(acc, smem), (float)width), a.eps)));
            for (uint32_t c = threadIdx.x; c < width; c += 256) {
                float o = __fmul_rn(__fmul_rn(__fsub_rn(to_f32(xr[c]), mean), r), to_f32(static_cast<const TW*>(a.w)[c]));
                yr[c] = from_f32<TOut>(__fadd_rn(o, a.b ? to_f32(static_cast<const TW*>(a.b)[c]) : 0.f));
            }
            if (threadIdx.x == 0) { if (a.stat0) a.stat0[row] = mean; if (a.stat1) a.stat1[row] = r; }
        } else if (OP == OP_SOFTMAX || OP == OP_LOGSOFTMAX) {
            float m = -INFINITY;
            for (uint32_t c = threadIdx.x; c < width; c += 256) m = fmaxf(m, to_f32(xr[c]));
            m = row_reduce<256, true>(m, smem);
            float acc = 0.f;
            for (uint32_t c = threadIdx.x; c < width; c += 256) acc = acc + expf(__fsub_rn(to_f32(xr[c]), m));
            float d = row_reduce<256, false>(acc, smem);
            float ld = logf(d);
            for (uint32_t c = threadIdx.x; c < width; c += 256) {
                float s = __fsub_rn(to_f32(xr[c]), m);
                yr[c] = from_f32<TOut>(OP == OP_SOFTMAX ? __fdiv_rn(expf(s), d) : __fsub_rn(s, ld));
            }
        } else {
            constexpr bool MX = OP == OP_MAX;
            float acc = MX ? -INFINITY : 0.f;
            for (uint32_t c = threadIdx.x; c < width; c += 256) acc = combine<MX>(acc, to_f32(xr[c]));
            float s = row_reduce<256, MX>(acc, smem);
            if (OP == OP_MEAN) s = __fdiv_rn(s, (float)width);
            if (threadIdx.x == 0) static_cast<TOut*>(a.y)[row] = from_f32<TOut>(s);
        }
    }
}

template <int OP, typename TIn, typename TOut, typename TW, int THREADS>
void launch_fast(rb_ctx* ctx, const RowArgs& a) {
    constexpr int ROWS = THREADS >= 256 ? 1 : 256 / THREADS;
    uint64_t blocks = (a.rows + ROWS - 1) / ROWS;
    uint64_t cap = (uint64_t)ctx->sm_count * 32;  // enough resident bytes per SM; the loop covers the rest
    dim3 grid((unsigned)(blocks < cap ? blocks : cap)), block(THREADS, ROWS);
    row_kernel<OP, TIn, TOut, TW, THREADS><<<grid, block, 0, ctx->stream>>>(a);
}

template <int OP, typename TIn, typename TOut, typename TW>
void launch(rb_ctx* ctx, const RowArgs& a, bool aligned) {
    const uint32_t w = a.width;
    if (aligned && w % 4 == 0 && w <= 1024 * MAXV * 4) {
        uint32_t need = (w / 4 + MAXV - 1) / MAXV;  // threads per row
        if (need <= 32) launch_fast<OP, TIn, TOut, TW, 32>(ctx, a);
        else if (need <= 64) launch_fast<OP, TIn, TOut, TW, 64>(ctx, a);
        else if (need <= 128) launch_fast<OP, TIn, TOut, TW, 128>(ctx, a);
        else if (need <= 256) launch_fast<OP, TIn, TOut, TW, 256>(ctx, a);
        else if (need <= 512) launch_fast<OP, TIn, TOut, TW, 512>(ctx, a);
        else launch_fast<OP, TIn, TOut, TW, 1024>(ctx, a);
    } else {
        uint64_t cap = (uint64_t)ctx->sm_count * 16;
        row_kernel_generic<OP, TIn, TOut, TW><<<(unsigned)(a.rows < cap ? a.rows : cap), 256, 0, ctx->stream>>>(a);
    }
}

template <int OP>
int32_t dispatch(rb_ctx* ctx, const RowArgs& a, uint32_t tin, uint32_t tout, uint32_t tw, bool aligned, const char* what) {
    using bf = __nv_bfloat16;
    if (tin == RB_F32 && tout == RB_F32 && tw == RB_F32) launch<OP, float, float, float>(ctx, a, aligned);
    else if (tin == RB_BF16 && tout == RB_BF16 && tw == RB_BF16) launch<OP, bf, bf, bf>(ctx, a, aligned);
    else if (tin == RB_BF16 && tout == RB_BF16 && tw == RB_F32) launch<OP, bf, bf, float>(ctx, a, aligned);
    else if (tin == RB_F32 && tout == RB_BF16 && tw == RB_F32) launch<OP, float, bf, float>(ctx, a, aligned);
    else if (tin == RB_BF16 && tout == RB_F32 && tw == RB_F32) launch<OP, bf, float, float>(ctx, a, aligned);
    else return rb::fail(RB_INVALID_TENSOR, "%s: unsupported dtype combination x=%s y=%s weight=%s", what,
                         rb::dtype_name(tin), rb::dtype_name(tout), rb::dtype_name(tw));
    return rb::after_launch(ctx, what);
}

int32_t epsilon_f32(double value, const char* what, float* out) {
    // normalization.rs:42-48: finite, positive and representable in FP32.
    float v = (float)value;
    if (!(value == value) || value - value != 0.0 || !(v - v == 0.0f) || v <= 0.0f)
        return rb::fail(RB_INVALID_TENSOR, "%s epsilon must be positive and representable in FP32", what);
    *out = v;
    return RB_OK;
}

int32_t check_stat(rb_ctx* ctx, const rb_tensor* t, uint64_t rows, const char* what, void** p) {
    *p = nullptr;
    if (!t) return RB_OK;
    if (t->dtype != RB_F32 || rb::elements(t) != rows) return rb::fail(RB_INVALID_TENSOR, "%s: statistic must be FP32 with one value per row", what);
    return rb::resolve(ctx, t, what, p);
}

bool vec_aligned(const void* p, uint64_t width, size_t es) {
    return p == nullptr || ((((uintptr_t)p) & 15u) == 0 && (width * es) % (es == 4 ? 16 : 8) == 0);
}

}  // namespace

using namespace rb;

extern "C" {

int32_t rb_rms_norm(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* weight, double epsilon,
                    const rb_tensor* y, const rb_tensor* rstd) {
    RB_TRY(check_ctx(ctx));
    void *px, *pw, *py, *ps; float eps;
    RB_TRY(resolve(ctx, x, "RMSNorm input", &px)); RB_TRY(resolve(ctx, weight, "RMSNorm weight", &pw));
    RB_TRY(resolve(ctx, y, "RMSNorm output", &py)); RB_TRY(epsilon_f32(epsilon, "RMSNorm", &eps));
    uint64_t rows, width; rows_width(x, &rows, &width);
    if (width == 0) return fail(RB_INVALID_TENSOR, "RMSNorm requires a positive last dimension");
    if (rows * width > 0xffffffffull) return fail(RB_INVALID_TENSOR, "RMSNorm element count exceeds u32");
    if (!same_shape(x, y) || elements(weight) != width) return fail(RB_INVALID_TENSOR, "RMSNorm buffer shape, stride, dtype or byte length mismatch");
    RB_TRY(check_stat(ctx, rstd, rows, "RMSNorm rstd", &ps));
    RB_TRY(no_overlap(py, rows * width * dtype_size(y->dtype), px, rows * width * dtype_size(x->dtype), "RMSNorm"));
    if (rows == 0) return empty_call(ctx);
    RowArgs a{px, pw, nullptr, py, (float*)ps, nullptr, rows, (uint32_t)width, eps};
    bool aligned = vec_aligned(px, width, dtype_size(x->dtype)) && vec_aligned(py, width, dtype_size(y->dtype)) && vec_aligned(pw, width, dtype_size(weight->dtype));
    return dispatch<OP_RMS>(ctx, a, x->dtype, y->dtype, weight->dtype, aligned, "RMSNorm");
}

int32_t rb_add_rms_norm(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* delta, const rb_tensor* weight, double epsilon,
                        const rb_tensor* x_out, const rb_tensor* y) {
    RB_TRY(check_ctx(ctx));
    void *px, *pd, *pw, *pxo, *py; float eps;
    RB_TRY(resolve(ctx, x, "add+RMSNorm input", &px)); RB_TRY(resolve(ctx, delta, "add+RMSNorm delta", &pd));
    RB_TRY(resolve(ctx, weight, "add+RMSNorm weight", &pw)); RB_TRY(resolve(ctx, x_out, "add+RMSNorm sum output", &pxo));
    RB_TRY(resolve(ctx, y, "add+RMSNorm output", &py)); RB_TRY(epsilon_f32(epsilon, "RMSNorm", &eps));
    uint64_t rows, width; rows_width(x, &rows, &width);
    if (width == 0 || width % 4 != 0 || width > 1024 * MAXV * 4) return fail(RB_INVALID_TENSOR, "add+RMSNorm needs a last dimension that is a multiple of 4 within 16384");
    if (!same_shape(x, delta) || !same_shape(x, x_out) || !same_shape(x, y) || elements(weight) != width || delta->dtype != x->dtype || x_out->dtype != x->dtype)
        return fail(RB_INVALID_TENSOR, "add+RMSNorm buffer shape, stride, dtype or byte length mismatch");
    const uint64_t bytes = rows * width * dtype_size(x->dtype);
    // x_out may be x itself (the residual stream is updated in place); every other pair must be disjoint
    if (pxo != px) RB_TRY(no_overlap(pxo, bytes, px, bytes, "add+RMSNorm"));
    RB_TRY(no_overlap(pxo, bytes, pd, bytes, "add+RMSNorm")); RB_TRY(no_overlap(py, rows * width * dtype_size(y->dtype), px, bytes, "add+RMSNorm"));
    RB_TRY(no_overlap(py, rows * width * dtype_size(y->dtype), pd, bytes, "add+RMSNorm"));
    if (rows == 0) return empty_call(ctx);
    bool aligned = vec_aligned(px, width, dtype_size(x->dtype)) && vec_aligned(py, width, dtype_size(y->dtype)) && vec_aligned(pw, width, dtype_size(weight->dtype));
    if (!aligned) return fail(RB_INVALID_TENSOR, "add+RMSNorm needs 16-byte aligned rows");
    RowArgs a{px, pw, nullptr, py, nullptr, nullptr, rows, (uint32_t)width, eps};
    a.delta = pd; a.x_out = pxo;
    return dispatch<OP_ADD_RMS>(ctx, a, x->dtype, y->dtype, weight->dtype, true, "add+RMSNorm");
}

int32_t rb_layer_norm(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* weight, const rb_tensor* bias, double epsilon,
                      const rb_tensor* y, const rb_tensor* mean, const rb_tensor* rstd) {
    RB_TRY(check_ctx(ctx));
    void *px, *pw, *pb, *py, *pm, *ps; float eps;
    RB_TRY(resolve(ctx, x, "LayerNorm input", &px)); RB_TRY(resolve(ctx, weight, "LayerNorm weight", &pw));
    RB_TRY(resolve(ctx, bias, "LayerNorm bias", &pb, true)); RB_TRY(resolve(ctx, y, "LayerNorm output", &py));
    RB_TRY(epsilon_f32(epsilon, "LayerNorm", &eps));
    uint64_t rows, width; rows_width(x, &rows, &width);
    if (width == 0) return fail(RB_INVALID_TENSOR, "LayerNorm requires a positive last dimension");
    if (rows * width > 0xffffffffull) return fail(RB_INVALID_TENSOR, "LayerNorm element count exceeds u32");
    if (!same_shape(x, y) || elements(weight) != width || (bias && (elements(bias) != width || bias->dtype != weight->dtype)))
        return fail(RB_INVALID_TENSOR, "LayerNorm buffer shape, stride, dtype or byte length mismatch");
    RB_TRY(check_stat(ctx, mean, rows, "LayerNorm mean", &pm)); RB_TRY(check_stat(ctx, rstd, rows, "LayerNorm rstd", &ps));
    RB_TRY(no_overlap(py, rows * width * dtype_size(y->dtype), px, rows * width * dtype_size(x->dtype), "LayerNorm"));
    if (rows == 0) return empty_call(ctx);
    RowArgs a{px, pw, pb, py, (float*)pm, (float*)ps, rows, (uint32_t)width, eps};
    bool aligned = vec_aligned(px, width, dtype_size(x->dtype)) && vec_aligned(py, width, dtype_size(y->dtype)) &&
                   vec_aligned(pw, width, dtype_size(weight->dtype)) && vec_aligned(pb, width, dtype_size(weight->dtype));
    return dispatch<OP_LAYER>(ctx, a, x->dtype, y->dtype, weight->dtype, aligned, "LayerNorm");
}

int32_t rb_softmax(rb_ctx* ctx, const rb_tensor* x, int32_t logarithmic, const rb_tensor* y) {
    RB_TRY(check_ctx(ctx));
    void *px, *py;
    RB_TRY(resolve(ctx, x, "Softmax input", &px)); RB_TRY(resolve(ctx, y, "Softmax output", &py));
    uint64_t rows, width; rows_width(x, &rows, &width);
    if (width == 0) return fail(RB_INVALID_TENSOR, "Softmax requires a positive last dimension");
    if (rows * width > 0xffffffffull) return fail(RB_INVALID_TENSOR, "Softmax element count exceeds u32");
    if (!same_shape(x, y)) return fail(RB_INVALID_TENSOR, "Softmax buffer shape, stride, dtype or byte length mismatch");
    RB_TRY(no_overlap(py, rows * width * dtype_size(y->dtype), px, rows * width * dtype_size(x->dtype), "Softmax"));
    if (rows == 0) return empty_call(ctx);
    RowArgs a{px, nullptr, nullptr, py, nullptr, nullptr, rows, (uint32_t)width, 0.f};
    bool aligned = vec_aligned(px, width, dtype_size(x->dtype)) && vec_aligned(py, width, dtype_size(y->dtype));
    return logarithmic ? dispatch<OP_LOGSOFTMAX>(ctx, a, x->dtype, y->dtype, RB_F32, aligned, "LogSoftmax")
                       : dispatch<OP_SOFTMAX>(ctx, a, x->dtype, y->dtype, RB_F32, aligned, "Softmax");
}

int32_t rb_reduce_last(rb_ctx* ctx, const rb_tensor* x, int32_t op, const rb_tensor* y) {
    RB_TRY(check_ctx(ctx));
    void *px, *py;
    RB_TRY(resolve(ctx, x, "row reduction input", &px)); RB_TRY(resolve(ctx, y, "row reduction output", &py));
    uint64_t rows, width; rows_width(x, &rows, &width);
    if (width == 0) return fail(RB_INVALID_TENSOR, "row reduction requires a positive last dimension");
    if (op < 0 || op > 2) return fail(RB_INVALID_TENSOR, "row reduction op must be 0 (sum), 1 (mean) or 2 (max)");
    if (elements(y) != rows || y->rank != x->rank || y->shape[y->rank - 1] != 1 || x->dtype != RB_F32 || y->dtype != RB_F32)
        return fail(RB_INVALID_TENSOR, "row reduction needs FP32 tensors and an output that keeps the last axis with size one");
    if (rows == 0) return empty_call(ctx);
    RowArgs a{px, nullptr, nullptr, py, nullptr, nullptr, rows, (uint32_t)width, 0.f};
    bool aligned = vec_aligned(px, width, 4);
    if (op == 0) return dispatch<OP_SUM>(ctx, a, RB_F32, RB_F32, RB_F32, aligned, "sum_last");
    if (op == 1) return dispatch<OP_MEAN>(ctx, a, RB_F32, RB_F32, RB_F32, aligned, "mean_last");
    return dispatch<OP_MAX>(ctx, a, RB_F32, RB_F32, RB_F32, aligned, "max_last");
}

}  // extern "C"
