// Runtime functions of the reference that are sequences of kernels, as single C entry points: a host crate binds one
// symbol per AscendRuntime function and needs no orchestration of its own.
//
//   rb_linear_bf16_fp32 / rb_linear_frozen_bf16   runtime/matrix.rs:84-93,129-133,147-159
//   rb_tensor_matmul                              runtime/generic_matrix.rs:17-54 (the vendor aclnnMatmul(KEEP_DTYPE), worker.rs:128-162)
//   rb_gemm_padded                                runtime/padded_matrix.rs:40-50, deepgemm/padded.rs:12-50
//   rb_gemm_grouped_nt                            deepgemm/plan.rs:15-29,61-67, rust-ascend-kernels/src/scheduler.rs:21-33
//   rb_attention_backward                         the autodiff graph of src/nn/attention.rs:10-29,49-67 with the rounding points
//                                                 of examples/grouped_attention_tensor.rs:14-44 and heads_programs.rs:59-86
//
// Temporaries come from the stream-ordered allocator (cudaMallocAsync / cudaFreeAsync on the context's stream): nothing
// outlives the call, nothing synchronises, and nothing is left behind when a step fails.
#include "common.cuh"

#include <cmath>

namespace {

using namespace rb;
using bf = __nv_bfloat16;

uint64_t up16(uint64_t d) { return (d + 15) / 16 * 16; }

// ---- FP32 -> BF16 of two tensors in one launch (the two Cast calls in front of a trainable Linear) ----------------------
__global__ void __launch_bounds__(256) cast_pair_kernel(const float* x, uint64_t nx, const float* w, uint64_t nw, bf* xo, bf* wo) {
    // both counts are multiples of 4 (rows of at least 16 elements); one thread converts four values
    const uint64_t qx = nx / 4, total = qx + nw / 4;
    const uint64_t stride = (uint64_t)gridDim.x * 256;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += stride) {
        const bool second = i >= qx;
        const uint64_t j = second ? i - qx : i;
        const float4 v = reinterpret_cast<const float4*>(second ? w : x)[j];
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        uint2 o; o.x = *reinterpret_cast<uint32_t*>(&lo); o.y = *reinterpret_cast<uint32_t*>(&hi);
        reinterpret_cast<uint2*>(second ? wo : xo)[j] = o;
    }
}

// ---- operand packing for the dtype-preserving matmul -------------------------------------------------------------------
// in: [batches, rows, cols] of T (rows x cols = M x K for A, K x N for B).  out: [batches * PARTS][R][C] 16-bit, zero padded to
// multiples of 16, where (R, C) = (rows, cols) or, with `transpose`, (cols, rows): both operands leave K-major.  FP32 values
// become PARTS = 3 BF16 values whose sum is the value to 24 bits (each part holds the leading bits of what the parts before
// it left over; every subtraction is exact); FP16 and BF16 values are copied as they are.
template <typename T, int PARTS>
__global__ void __launch_bounds__(256) pack_operand_kernel(const T* in, uint16_t* out, uint32_t rows, uint32_t cols, uint32_t rows_p, uint32_t cols_p, int transpose) {
    __shared__ uint16_t tile[PARTS][32][33];
    const uint32_t batch = blockIdx.z, r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
    const T* src = in + (size_t)batch * rows * cols;
    for (uint32_t i = threadIdx.x; i < 32 * 32; i += 256) {
        const uint32_t r = i / 32, c = i % 32;
        uint16_t parts[PARTS];
#pragma unroll
        for (int q = 0; q < PARTS; ++q) parts[q] = 0;
        if (r0 + r < rows && c0 + c < cols) {
            if constexpr (PARTS == 1) {
                parts[0] = reinterpret_cast<const uint16_t*>(src)[(size_t)(r0 + r) * cols + c0 + c];
            } else {
                float rest = static_cast<float>(src[(size_t)(r0 + r) * cols + c0 + c]);
#pragma unroll
                for (int q = 0; q < PARTS; ++q) {
                    const bf part = __float2bfloat16_rn(rest);
                    parts[q] = *reinterpret_cast<const uint16_t*>(&part);
                    rest = __fsub_rn(rest, __bfloat162float(part));
                }
            }
        }
#pragma unroll
        for (int q = 0; q < PARTS; ++q) tile[q][r][c] = parts[q];
    }
    __syncthreads();
    const uint32_t out_rows = transpose ? cols_p : rows_p, out_cols = transpose ? rows_p : cols_p;
    for (uint32_t i = threadIdx.x; i < 32 * 32; i += 256) {
        const uint32_t a = i / 32, b = i % 32;                      // a: output row inside the tile, b: output column
        const uint32_t orow = (transpose ? c0 : r0) + a, ocol = (transpose ? r0 : c0) + b;
        if (orow < out_rows && ocol < out_cols) {
#pragma unroll
            for (int q = 0; q < PARTS; ++q)
                out[((size_t)(batch * PARTS + q) * out_rows + orow) * out_cols + ocol] = transpose ? tile[q][b][a] : tile[q][a][b];
        }
    }
}

template <typename T, int PARTS>
int32_t pack(rb_ctx* ctx, const void* in, void* out, uint64_t batches, uint64_t rows, uint64_t cols, bool transpose) {
    const uint64_t rp = up16(rows), cp = up16(cols);
    for (uint64_t b0 = 0; b0 < batches; b0 += 65535) {             // grid.z limit
        const uint64_t nb = batches - b0 < 65535 ? batches - b0 : 65535;
        dim3 grid((unsigned)((cp + 31) / 32), (unsigned)((rp + 31) / 32), (unsigned)nb);
        pack_operand_kernel<T, PARTS><<<grid, 256, 0, ctx->stream>>>(static_cast<const T*>(in) + b0 * rows * cols,
            static_cast<uint16_t*>(out) + b0 * PARTS * rp * cp, (uint32_t)rows, (uint32_t)cols, (uint32_t)rp, (uint32_t)cp, transpose ? 1 : 0);
        RB_TRY(after_launch(ctx, "matmul operand packing"));
    }
    return RB_OK;
}

// FP32 or BF16 [.., rows, cols] -> BF16 [.., rows_p, cols_p], zero padded: Cast + resize_prefix of padded_matrix.rs in one pass.
template <typename T>
__global__ void __launch_bounds__(256) pad_cast_kernel(const T* in, bf* out, uint64_t batches, uint32_t rows, uint32_t cols, uint32_t rows_p, uint32_t cols_p) {
    const uint64_t total = batches * rows_p * cols_p, stride = (uint64_t)gridDim.x * 256;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += stride) {
        const uint32_t c = (uint32_t)(i % cols_p); const uint64_t br = i / cols_p; const uint32_t r = (uint32_t)(br % rows_p); const uint64_t b = br / rows_p;
        float v = 0.f;
        if (r < rows && c < cols) {
            if constexpr (sizeof(T) == 4) v = in[(b * rows + r) * cols + c]; else v = __bfloat162float(in[(b * rows + r) * cols + c]);
        }
        out[i] = __float2bfloat16_rn(v);
    }
}

}  // namespace

extern "C" {

int32_t rb_linear_bf16_fp32(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* w, const rb_tensor* y, const rb_tensor* x_bf16, const rb_tensor* w_bf16) {
    RB_TRY(check_ctx(ctx));
    void *px, *pw, *py, *pxo, *pwo;
    RB_TRY(resolve(ctx, x, "linear X", &px)); RB_TRY(resolve(ctx, w, "linear W", &pw)); RB_TRY(resolve(ctx, y, "linear Y", &py));
    RB_TRY(resolve(ctx, x_bf16, "linear saved X", &pxo)); RB_TRY(resolve(ctx, w_bf16, "linear saved W", &pwo));
    if (x->rank != 2 || w->rank != 2) return fail(RB_INVALID_TENSOR, "linear requires rank-2 X[M,K] and W[N,K]");
    if (x->dtype != RB_F32 || w->dtype != RB_F32) return fail(RB_INVALID_TENSOR, "gemm_bf16_fp32 requires FP32 inputs");
    if (!same_shape(x, x_bf16) || !same_shape(w, w_bf16) || x_bf16->dtype != RB_BF16 || w_bf16->dtype != RB_BF16)
        return fail(RB_INVALID_TENSOR, "the saved operands are BF16 tensors of the inputs' shapes");
    const uint64_t nx = elements(x), nw = elements(w);
    if (nx == 0 || nw == 0 || nx % 4 || nw % 4) return fail(RB_INVALID_TENSOR, "GEMM M/N/K must be positive multiples of 16 within INT32_MAX");
    RB_TRY(no_overlap(pxo, nx * 2, px, nx * 4, "linear")); RB_TRY(no_overlap(pwo, nw * 2, pw, nw * 4, "linear"));
    const uint64_t quads = (nx + nw) / 4;
    const uint64_t cap = (uint64_t)ctx->sm_count * 16;
    cast_pair_kernel<<<(unsigned)((quads + 255) / 256 < cap ? (quads + 255) / 256 : cap), 256, 0, ctx->stream>>>((const float*)px, nx, (const float*)pw, nw, (bf*)pxo, (bf*)pwo);
    RB_TRY(after_launch(ctx, "linear operand cast"));
    return rb_gemm(ctx, x_bf16, w_bf16, 0, 1, nullptr, nullptr, RB_EPILOGUE_NONE, y);
}

int32_t rb_linear_frozen_bf16(rb_ctx* ctx, const rb_tensor* x, const rb_tensor* w, const rb_tensor* y, const rb_tensor* x_bf16) {
    RB_TRY(check_ctx(ctx));
    if (!x || !w || !y) return fail(RB_INVALID_TENSOR, "frozen linear: missing tensor");
    if (x->dtype != RB_F32 || w->dtype != RB_BF16) return fail(RB_INVALID_TENSOR, "frozen linear requires FP32 input and BF16 weight storage");
    if (x->rank != 2 || w->rank != 2) return fail(RB_INVALID_TENSOR, "linear requires rank-2 X[M,K] and W[N,K]");
    Scratch scratch(ctx);
    rb_tensor tmp;
    const rb_tensor* xb = x_bf16;
    if (!xb) { RB_TRY(scratch.tensor(RB_BF16, {x->shape[0], x->shape[1]}, &tmp)); xb = &tmp; }
    else if (!same_shape(x, xb) || xb->dtype != RB_BF16) return fail(RB_INVALID_TENSOR, "the saved input is a BF16 tensor of the input's shape");
    RB_TRY(rb_cast(ctx, x, xb));
    return rb_gemm(ctx, xb, w, 0, 1, nullptr, nullptr, RB_EPILOGUE_NONE, y);
}

int32_t rb_tensor_matmul(rb_ctx* ctx, const rb_tensor* a, const rb_tensor* b, const rb_tensor* out) {
    RB_TRY(check_ctx(ctx));
    if (!a || !b || !out) return fail(RB_INVALID_TENSOR, "matmul: missing tensor");
    const bool floats = a->dtype == RB_F32 || a->dtype == RB_F16 || a->dtype == RB_BF16;
    if (!floats || b->dtype != a->dtype || a->rank < 2 || a->rank > 6 || b->rank < 2 || b->rank > 6)
        return fail(RB_INVALID_TENSOR, "generic Ascend matmul requires matching floating dtypes and rank 2..6");
    const uint64_t m = a->shape[a->rank - 2], k = a->shape[a->rank - 1], n = b->shape[b->rank - 1];
    if (b->shape[b->rank - 2] != k) return fail(RB_INVALID_TENSOR, "matmul contraction dimensions differ");
    // batch axes, right aligned; singleton axes broadcast (tensor/layout.rs:123-142)
    const uint32_t ra = a->rank - 2, rbk = b->rank - 2, rank = ra > rbk ? ra : rbk;
    uint64_t da[4], db[4], dout[4], no = 1, na = 1, nb = 1;
    bool same = ra == rbk;
    for (uint32_t i = 0; i < rank; ++i) {
        da[i] = i + ra >= rank ? a->shape[i + ra - rank] : 1;
        db[i] = i + rbk >= rank ? b->shape[i + rbk - rank] : 1;
        if (da[i] != db[i] && da[i] != 1 && db[i] != 1) return fail(RB_INVALID_TENSOR, "matmul batch axes cannot be broadcast");
        dout[i] = da[i] == 1 ? db[i] : da[i];
        no *= dout[i]; na *= da[i]; nb *= db[i];
        same = same && da[i] == db[i];
    }
    if (out->dtype != a->dtype || out->rank != rank + 2 || out->shape[rank] != m || out->shape[rank + 1] != n) return fail(RB_INVALID_TENSOR, "matmul output must keep the dtype and have the broadcast shape");
    for (uint32_t i = 0; i < rank; ++i) if (out->shape[i] != dout[i]) return fail(RB_INVALID_TENSOR, "matmul output must keep the dtype and have the broadcast shape");
    const uint64_t es = dtype_size(a->dtype);
    if (no * m * n == 0) return empty_call(ctx);
    void *pa = nullptr, *pb = nullptr, *po;
    RB_TRY(resolve(ctx, out, "matmul output", &po));
    if (k == 0) {                                      // an empty contraction: zeros (generic_matrix.rs:73-78)
        RB_CUDA(ctx, "cudaMemsetAsync", cudaMemsetAsync(po, 0, no * m * n * es, ctx->stream));
        return RB_OK;
    }
    RB_TRY(resolve(ctx, a, "matmul A", &pa)); RB_TRY(resolve(ctx, b, "matmul B", &pb));
    RB_TRY(no_overlap(po, no * m * n * es, pa, na * m * k * es, "matmul")); RB_TRY(no_overlap(po, no * m * n * es, pb, nb * k * n * es, "matmul"));
    if (m > 0x7fffffffull || n > 0x7fffffffull || up16(k) > 0x7fffffffull || no > 0x7fffffffull) return fail(RB_INVALID_TENSOR, "matmul dimensions exceed INT32_MAX");
    const uint32_t parts = a->dtype == RB_F32 ? 3 : 1;
    const uint64_t mp = up16(m), kp = up16(k), np_ = up16(n);
    Scratch scratch(ctx);
    rb_tensor ta, tb; void *qa, *qb;
    RB_TRY(scratch.tensor(RB_BF16, {na * parts, mp, kp}, &ta, &qa)); RB_TRY(scratch.tensor(RB_BF16, {nb * parts, np_, kp}, &tb, &qb));
    if (a->dtype == RB_F32) { RB_TRY((pack<float, 3>(ctx, pa, qa, na, m, k, false))); RB_TRY((pack<float, 3>(ctx, pb, qb, nb, k, n, true))); }
    else { RB_TRY((pack<uint16_t, 1>(ctx, pa, qa, na, m, k, false))); RB_TRY((pack<uint16_t, 1>(ctx, pb, qb, nb, k, n, true))); }
    GemmCall c;
    c.m = (uint32_t)m; c.n = (uint32_t)n; c.k = (uint32_t)kp; c.a_rows = (uint32_t)mp; c.b_rows = (uint32_t)np_;
    c.out_kind = a->dtype == RB_F32 ? 1 : (a->dtype == RB_F16 ? 2 : 0);
    c.f16_operands = a->dtype == RB_F16;
    c.ragged = (n * es) % 16 != 0;
    c.parts_a = c.parts_b = parts;
    if (parts == 3) {
        // cross products of the parts, smallest first; the three below 2^-24 of the result are left out
        static const uint32_t ia[6] = {0, 1, 2, 0, 1, 0}, ib[6] = {2, 1, 0, 1, 0, 0};
        c.nseg = 6;
        for (int i = 0; i < 6; ++i) { c.seg_a[i] = ia[i]; c.seg_b[i] = ib[i]; }
    }
    const uint64_t a_step = parts * mp * kp * 2, b_step = parts * np_ * kp * 2, o_step = m * n * es;
    if (same || na == 1 || nb == 1) {
        // one batched launch: equal batch shapes, or one operand shared by every output batch
        c.a = qa; c.b = qb; c.out = po; c.batches = (uint32_t)no; c.a_bcast = !same && na == 1 && no != 1; c.b_bcast = !same && nb == 1 && no != 1;
        if (!same && na == 1 && nb == 1) { c.a_bcast = c.b_bcast = false; }
        return gemm_run(ctx, c);
    }
    // general broadcast: one launch per output batch entry
    c.batches = 1;
    for (uint64_t flat = 0; flat < no; ++flat) {
        uint64_t rem = flat, ia_flat = 0, ib_flat = 0, sa = 1, sb = 1;
        for (int i = (int)rank - 1; i >= 0; --i) {
            const uint64_t idx = rem % dout[i]; rem /= dout[i];
            ia_flat += (da[i] == 1 ? 0 : idx) * sa; sa *= da[i];
            ib_flat += (db[i] == 1 ? 0 : idx) * sb; sb *= db[i];
        }
        c.a = static_cast<char*>(qa) + ia_flat * a_step; c.b = static_cast<char*>(qb) + ib_flat * b_step; c.out = static_cast<char*>(po) + flat * o_step;
        RB_TRY(gemm_run(ctx, c));
    }
    return RB_OK;
}

int32_t rb_gemm_grouped_nt(rb_ctx* ctx, const rb_tensor* a, const rb_tensor* weights, const int64_t* ends, uint32_t groups, const rb_tensor* out) {
    RB_TRY(check_ctx(ctx));
    if (!a || !weights || !out || !ends) return fail(RB_INVALID_TENSOR, "grouped NT: missing argument");
    // GroupEnds::new, deepgemm/plan.rs:15-29
    if (groups < 1 || groups > 4096) return fail(RB_INVALID_TENSOR, "group count must be 1..=4096");
    int64_t previous = 0;
    std::vector<int32_t> host(groups);
    for (uint32_t g = 0; g < groups; ++g) {
        if (ends[g] < previous || ends[g] % 256 || ends[g] > 0x7fffffffll) return fail(RB_INVALID_TENSOR, "group ends must be nondecreasing multiples of 256");
        previous = ends[g]; host[g] = (int32_t)ends[g];
    }
    if (previous == 0) return fail(RB_INVALID_TENSOR, "all-empty grouped GEMM is not implemented");
    if (a->rank != 2 || weights->rank != 3) return fail(RB_INVALID_TENSOR, "grouped NT requires [M,K] and [G,N,K]");
    const uint64_t m = a->shape[0], k = a->shape[1], g = weights->shape[0], n = weights->shape[1];
    if (m != (uint64_t)previous || g != groups || weights->shape[2] != k) return fail(RB_INVALID_TENSOR, "grouped NT dimensions do not match the physical prefix sums");
    if (a->dtype != RB_BF16 || weights->dtype != RB_BF16 || (out->dtype != RB_BF16 && out->dtype != RB_F32))
        return fail(RB_INVALID_TENSOR, "native DeepGEMM accepts BF16 inputs and BF16/F32 output only");
    if (m == 0 || n == 0 || k == 0 || m % 16 || n % 16 || k % 16 || m > 0x7fffffffull || n > 0x7fffffffull || k > 0x7fffffffull)
        return fail(RB_INVALID_TENSOR, "M/N/K must be positive multiples of 16 <= INT32_MAX; batches/groups 1..=4096");
    if (out->rank != 2 || out->shape[0] != m || out->shape[1] != n) return fail(RB_INVALID_TENSOR, "grouped NT output is [M,N]");
    void *pa, *pw, *po;
    RB_TRY(resolve(ctx, a, "grouped NT A", &pa)); RB_TRY(resolve(ctx, weights, "grouped NT weights", &pw)); RB_TRY(resolve(ctx, out, "grouped NT output", &po));
    const uint64_t o_bytes = m * n * dtype_size(out->dtype);
    RB_TRY(no_overlap(po, o_bytes, pa, m * k * 2, "grouped NT")); RB_TRY(no_overlap(po, o_bytes, pw, g * n * k * 2, "grouped NT"));
    // One persistent launch over all groups: groups start on 256-row boundaries, so a 128-row tile belongs to one group and
    // the kernel only has to pick that group's weight for the tile (the walk of scheduler.rs:21-33 without its per-group loop).
    Scratch scratch(ctx);
    rb_tensor te; void* pe;
    RB_TRY(scratch.tensor(RB_I32, {groups}, &te, &pe));
    RB_CUDA(ctx, "cudaMemcpyAsync(group ends)", cudaMemcpyAsync(pe, host.data(), groups * 4, cudaMemcpyHostToDevice, ctx->stream));
    GemmCall c;
    c.a = pa; c.b = pw; c.out = po; c.m = (uint32_t)m; c.n = (uint32_t)n; c.k = (uint32_t)k; c.out_kind = out->dtype == RB_F32 ? 1 : 0;
    c.group_ends = static_cast<const int32_t*>(pe); c.groups = groups;
    return gemm_run(ctx, c);
}

int32_t rb_gemm_padded(rb_ctx* ctx, const rb_tensor* a, const rb_tensor* b, int32_t transpose_a, int32_t transpose_b,
                       const rb_tensor* out, const rb_tensor* a_bf16, const rb_tensor* b_bf16) {
    RB_TRY(check_ctx(ctx));
    if (!a || !b || !out || !a_bf16 || !b_bf16) return fail(RB_INVALID_TENSOR, "padded GEMM: missing tensor");
    // PaddedGemmSpec::new, deepgemm/padded.rs:15-41
    const uint32_t rank = a->rank;
    const bool dtypes_ok = (a->dtype == RB_F32 || a->dtype == RB_BF16) && (b->dtype == RB_F32 || b->dtype == RB_BF16);
    if ((rank != 2 && rank != 3) || b->rank != rank || !dtypes_ok) return fail(RB_INVALID_TENSOR, "padded GEMM requires matching rank-2/3 FP32/BF16 inputs");
    if (rank == 3 && a->shape[0] != b->shape[0]) return fail(RB_INVALID_TENSOR, "padded GEMM does not broadcast batches");
    const uint64_t batches = rank == 3 ? a->shape[0] : 1;
    const uint64_t ar = a->shape[rank - 2], ac = a->shape[rank - 1], br = b->shape[rank - 2], bc = b->shape[rank - 1];
    const uint64_t m = transpose_a ? ac : ar, k = transpose_a ? ar : ac, kb = transpose_b ? bc : br, n = transpose_b ? br : bc;
    if (k != kb) return fail(RB_INVALID_TENSOR, "padded GEMM logical contraction mismatch");
    if (ar == 0 || ac == 0 || br == 0 || bc == 0) return fail(RB_INVALID_TENSOR, "padded GEMM matrix axes must be positive");
    if (up16(ar) > 0x7fffffffull || up16(ac) > 0x7fffffffull || up16(br) > 0x7fffffffull || up16(bc) > 0x7fffffffull) return fail(RB_INVALID_TENSOR, "padded GEMM aligned axis exceeds INT32_MAX");
    if (rank == 3 && (batches < 1 || batches > 4096)) return fail(RB_INVALID_TENSOR, "GEMM batch count must be within 1..4096");
    auto padded_like = [&](const rb_tensor* t, uint64_t r, uint64_t c) {
        return t->dtype == RB_BF16 && t->rank == rank && (rank == 2 || t->shape[0] == batches) && t->shape[rank - 2] == up16(r) && t->shape[rank - 1] == up16(c);
    };
    if (!padded_like(a_bf16, ar, ac) || !padded_like(b_bf16, br, bc)) return fail(RB_INVALID_TENSOR, "the saved operands are BF16 tensors with both matrix axes rounded up to multiples of 16");
    if (out->dtype != RB_F32 || out->rank != rank || (rank == 3 && out->shape[0] != batches) || out->shape[rank - 2] != m || out->shape[rank - 1] != n)
        return fail(RB_INVALID_TENSOR, "padded GEMM output is FP32 with the logical M x N");
    void *pa, *pb, *pao, *pbo;
    RB_TRY(resolve(ctx, a, "padded GEMM A", &pa)); RB_TRY(resolve(ctx, b, "padded GEMM B", &pb));
    RB_TRY(resolve(ctx, a_bf16, "padded GEMM saved A", &pao)); RB_TRY(resolve(ctx, b_bf16, "padded GEMM saved B", &pbo));
    auto pad = [&](const rb_tensor* t, const void* src, void* dst, uint64_t r, uint64_t c) -> int32_t {
        const uint64_t total = batches * up16(r) * up16(c), cap = (uint64_t)ctx->sm_count * 16;
        const unsigned grid = (unsigned)((total + 255) / 256 < cap ? (total + 255) / 256 : cap);
        if (t->dtype == RB_F32) pad_cast_kernel<float><<<grid, 256, 0, ctx->stream>>>((const float*)src, (bf*)dst, batches, (uint32_t)r, (uint32_t)c, (uint32_t)up16(r), (uint32_t)up16(c));
        else pad_cast_kernel<bf><<<grid, 256, 0, ctx->stream>>>((const bf*)src, (bf*)dst, batches, (uint32_t)r, (uint32_t)c, (uint32_t)up16(r), (uint32_t)up16(c));
        return after_launch(ctx, "padded GEMM operand");
    };
    RB_TRY(pad(a, pa, pao, ar, ac)); RB_TRY(pad(b, pb, pbo, br, bc));
    Scratch scratch(ctx);
    rb_tensor yp;
    if (rank == 3) RB_TRY(scratch.tensor(RB_F32, {batches, up16(m), up16(n)}, &yp)); else RB_TRY(scratch.tensor(RB_F32, {up16(m), up16(n)}, &yp));
    RB_TRY(rb_gemm(ctx, a_bf16, b_bf16, transpose_a, transpose_b, nullptr, nullptr, RB_EPILOGUE_NONE, &yp));
    return rb_resize_prefix(ctx, &yp, out);
}

int32_t rb_attention_backward(rb_ctx* ctx, const rb_tensor* q, const rb_tensor* k, const rb_tensor* v, const rb_tensor* grad, const rb_tensor* mask,
                              float scale, int32_t causal, uint64_t query_start, uint64_t key_start,
                              const rb_tensor* dq, const rb_tensor* dk, const rb_tensor* dv, const rb_tensor* dmask) {
    RB_TRY(check_ctx(ctx));
    for (const rb_tensor* t : {q, k, v, grad, dq, dk, dv})
        if (!t || t->rank != 4 || t->dtype != RB_F32) return fail(RB_INVALID_TENSOR, "attention backward requires FP32 rank-4 Q/K/V, upstream gradient and gradient outputs");
    const uint64_t b = q->shape[0], hq = q->shape[1], m = q->shape[2], d = q->shape[3];
    const uint64_t hkv = v->shape[1], n = v->shape[2], dvw = v->shape[3];
    if (hkv == 0 || hq % hkv || k->shape[0] != b || k->shape[1] != hkv || k->shape[2] != n || k->shape[3] != d || v->shape[0] != b ||
        grad->shape[0] != b || grad->shape[1] != hq || grad->shape[2] != m || grad->shape[3] != dvw)
        return fail(RB_INVALID_TENSOR, "GQA requires matching batches, positive divisible Q/KV heads and matching K/V lengths and Q/K widths");
    if (!std::isfinite(scale)) return fail(RB_INVALID_TENSOR, "attention backward needs a finite scale");
    if (!same_shape(q, dq) || !same_shape(k, dk) || !same_shape(v, dv)) return fail(RB_INVALID_TENSOR, "gradient outputs have the shapes of Q, K and V");
    const uint64_t flat = b * hq;
    if (mask && (mask->dtype != RB_F32 || elements(mask) != flat * m * n)) return fail(RB_INVALID_TENSOR, "attention additive mask must be FP32 [B,Hq,M,N]");
    if (dmask && (dmask->dtype != RB_F32 || elements(dmask) != flat * m * n)) return fail(RB_INVALID_TENSOR, "the mask gradient is FP32 [B,Hq,M,N]");
    Scratch s(ctx);
    rb_tensor qb, gb, krep, vrep, kb, vb, scores, tri, p, dp, ds, dsb, pb, dk_full, dv_full;
    RB_TRY(s.tensor(RB_BF16, {flat, m, d}, &qb)); RB_TRY(s.tensor(RB_BF16, {flat, m, dvw}, &gb));
    RB_TRY(s.tensor(RB_F32, {b, hq, n, d}, &krep)); RB_TRY(s.tensor(RB_F32, {b, hq, n, dvw}, &vrep));
    RB_TRY(s.tensor(RB_BF16, {flat, n, d}, &kb)); RB_TRY(s.tensor(RB_BF16, {flat, n, dvw}, &vb));
    const rb_tensor q3 = view(*q, {flat, m, d}), g3 = view(*grad, {flat, m, dvw});
    RB_TRY(rb_cast(ctx, &q3, &qb)); RB_TRY(rb_cast(ctx, &g3, &gb));
    RB_TRY(rb_repeat_kv_heads(ctx, k, (uint32_t)hq, &krep)); RB_TRY(rb_repeat_kv_heads(ctx, v, (uint32_t)hq, &vrep));
    const rb_tensor krep3 = view(krep, {flat, n, d}), vrep3 = view(vrep, {flat, n, dvw});
    RB_TRY(rb_cast(ctx, &krep3, &kb)); RB_TRY(rb_cast(ctx, &vrep3, &vb));
    // P = softmax(scale * bf16(Q) bf16(K)^T + mask)
    RB_TRY(s.tensor(RB_F32, {flat, m, n}, &scores));
    RB_TRY(rb_gemm(ctx, &qb, &kb, 0, 1, nullptr, nullptr, RB_EPILOGUE_NONE, &scores));
    RB_TRY(rb_mul_scalar(ctx, &scores, scale, &scores));
    if (mask) { const rb_tensor m3 = view(*mask, {flat, m, n}); RB_TRY(rb_add(ctx, &scores, &m3, &scores)); }
    if (causal) {
        RB_TRY(s.tensor(RB_F32, {flat, m, n}, &tri));
        RB_TRY(rb_causal_mask(ctx, query_start, key_start, &tri));
        RB_TRY(rb_add(ctx, &scores, &tri, &scores));
    }
    RB_TRY(s.tensor(RB_F32, {flat, m, n}, &p)); RB_TRY(rb_softmax(ctx, &scores, 0, &p));
    // dP = bf16(dY) bf16(V)^T ; dS = P (dP - sum(P dP))
    RB_TRY(s.tensor(RB_F32, {flat, m, n}, &dp)); RB_TRY(rb_gemm(ctx, &gb, &vb, 0, 1, nullptr, nullptr, RB_EPILOGUE_NONE, &dp));
    RB_TRY(s.tensor(RB_F32, {flat, m, n}, &ds)); RB_TRY(rb_softmax_backward(ctx, &p, &dp, 0, &ds));
    if (dmask) { const rb_tensor dm3 = view(*dmask, {flat, m, n}); RB_TRY(rb_copy(ctx, &ds, &dm3)); }
    // bf16(scale dS) feeds dQ and dK, bf16(P) feeds dV
    RB_TRY(rb_mul_scalar(ctx, &ds, scale, &ds));
    RB_TRY(s.tensor(RB_BF16, {flat, m, n}, &dsb)); RB_TRY(rb_cast(ctx, &ds, &dsb));
    RB_TRY(s.tensor(RB_BF16, {flat, m, n}, &pb)); RB_TRY(rb_cast(ctx, &p, &pb));
    const rb_tensor dq3 = view(*dq, {flat, m, d});
    RB_TRY(rb_gemm(ctx, &dsb, &kb, 0, 0, nullptr, nullptr, RB_EPILOGUE_NONE, &dq3));
    RB_TRY(s.tensor(RB_F32, {flat, n, d}, &dk_full)); RB_TRY(rb_gemm(ctx, &dsb, &qb, 1, 0, nullptr, nullptr, RB_EPILOGUE_NONE, &dk_full));
    RB_TRY(s.tensor(RB_F32, {flat, n, dvw}, &dv_full)); RB_TRY(rb_gemm(ctx, &pb, &gb, 1, 0, nullptr, nullptr, RB_EPILOGUE_NONE, &dv_full));
    // the gradients of a KV head sum over its query heads (heads_programs.rs:59-86)
    const rb_tensor dk4 = view(dk_full, {b, hq, n, d}), dv4 = view(dv_full, {b, hq, n, dvw});
    RB_TRY(rb_repeat_kv_heads_backward(ctx, &dk4, (uint32_t)hkv, dk));
    return rb_repeat_kv_heads_backward(ctx, &dv4, (uint32_t)hkv, dv);
}

}  // extern "C"
