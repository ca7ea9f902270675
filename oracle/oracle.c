/*
 * TEST INFRASTRUCTURE — CPU restatement of rust-ascend's dense-transformer arithmetic.
 *
 * This file is the checker, not the product.  Only tests, the smoke check and the CPU-baseline /
 * reference leg of the benchmark may call it.  The shipped CUDA path never links or loads it.
 *
 * Every function restates, in plain C, the arithmetic that the reference defines as device IR or
 * as an in-test f64 model; the citation next to each function gives the reference file:line.  The
 * reference has no CPU execution path of its own (src/backend.rs:43-45), so this port is the CPU
 * baseline as well.
 *
 * Pinning status:
 *   - row schedule (reduce / softmax / rms / layer norm): pinned against the reference's own NumPy
 *     statement tools/ascend/tests/test_row_reference.py:7-28 (fixtures under tests/golden/).
 *   - GEMM, RoPE, SiLU*up, KV repeat, causal mask, bias/residual, attention composition: pinned
 *     against the deterministic index-formula vectors of the reference's in-crate tests and device
 *     examples (cited in tests/).
 *   - backward programs, attention backward, LayerNorm backward, causal cross entropy: pinned against the f64
 *     expectations of the reference's device examples (tests/test_backward.py, tests/test_oracle_next.py).
 *   - decoder-stack composition (tests/decoder_reference.py, built from these functions): PARITY UNPINNED — no
 *     reference test fixes a Llama forward value; it is the standard pre-norm block assembled from the pinned ops.
 *
 * Build: see oracle/Makefile (gcc -O3 -fopenmp -ffp-contract=off; contraction is disabled because
 * the reference IR rounds every multiply and add separately).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ---------------------------------------------------------------- BF16 rounding ------------- */
/* rust-ascend-kernels/src/tests.rs:7-11: exponent all ones -> truncate; else RNE on bit 16. */
static inline uint32_t f2u(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static inline float u2f(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }
static inline float bf16r(float x) {
    uint32_t b = f2u(x);
    if ((b & 0x7f800000u) == 0x7f800000u) return u2f(b & 0xffff0000u);
    return u2f((b + 0x7fffu + ((b >> 16) & 1u)) & 0xffff0000u);
}
ORC_API float orc_bf16(float x) { return bf16r(x); }
ORC_API void orc_bf16_array(const float* in, float* out, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = bf16r(in[i]);
}
ORC_API void orc_f32_to_bf16_bits(const float* in, uint16_t* out, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = (uint16_t)(f2u(bf16r(in[i])) >> 16);
}
ORC_API void orc_bf16_bits_to_f32(const uint16_t* in, float* out, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = u2f((uint32_t)in[i] << 16);
}
ORC_API void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
ORC_API int orc_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ---------------------------------------------------------------- 32-lane row schedule ------ */
/* rust-ascend-compiler/src/ascend/row_programs.rs:77-85: lane l owns columns l+32j and folds them
 * in increasing j; then one 32-lane plane reduction.  Rows wider than 4096 or not divisible by 32
 * are cut into <=4096-column tiles whose statistics are merged in tile order, unaligned tiles
 * padded with +0 (sum) or -inf (max) inside the reduction only
 * (rust-ascend-driver/src/tensor/runtime/wide_rows.rs:133-146, wide_programs.rs:158-179).
 * The hardware's 32-lane tree order is unspecified; a fixed pairwise tree is used here. */
#define TILE 4096
static float plane(float* lane, int maximum) {
    for (int s = 16; s >= 1; s >>= 1)
        for (int l = 0; l < s; ++l)
            lane[l] = maximum ? fmaxf(lane[l], lane[l + s]) : lane[l] + lane[l + s];
    return lane[0];
}
static float tile_reduce(const float* x, int64_t n, int maximum) {
    float lane[32];
    for (int l = 0; l < 32; ++l) lane[l] = l < n ? x[l] : (maximum ? -INFINITY : 0.0f);
    for (int64_t j = 32; j < n; j += 32)
        for (int l = 0; l < 32 && j + l < n; ++l)
            lane[l] = maximum ? fmaxf(lane[l], x[j + l]) : lane[l] + x[j + l];
    return plane(lane, maximum);
}
typedef float (*elem_fn)(float, const void*);
/* Reduce f(x[c]) over one row, tile by tile. */
static float row_reduce_map(const float* x, int64_t width, int maximum, elem_fn f, const void* arg,
                            float* scratch) {
    float acc = 0.0f;
    for (int64_t start = 0; start < width; start += TILE) {
        int64_t n = width - start < TILE ? width - start : TILE;
        const float* src = x + start;
        if (f) { for (int64_t c = 0; c < n; ++c) scratch[c] = f(src[c], arg); src = scratch; }
        float t = tile_reduce(src, n, maximum);
        acc = start == 0 ? t : (maximum ? fmaxf(acc, t) : acc + t);
    }
    return acc;
}
static float f_square(float x, const void* a) { (void)a; return x * x; }
static float f_center_square(float x, const void* a) { float c = x - *(const float*)a; return c * c; }
static float f_shift_exp(float x, const void* a) { return expf(x - *(const float*)a); }

/* row_programs.rs:120-134 (Sum / Mean / Max). */
ORC_API void orc_row_reduce(const float* x, int64_t rows, int64_t width, int op, float* out) {
#pragma omp parallel
    {
        float* scratch = (float*)malloc(sizeof(float) * TILE);
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            float s = row_reduce_map(x + r * width, width, op == 2, NULL, NULL, scratch);
            out[r] = op == 1 ? s / (float)width : s;
        }
        free(scratch);
    }
}

/* row_programs.rs:144-151: sq=x*x; mean=sum/W; r=rsqrt(mean+eps); y=(x*r)*w; rstd[row]=r. */
ORC_API void orc_rms_norm(const float* x, const float* w, float eps, int64_t rows, int64_t width,
                          float* y, float* rstd) {
#pragma omp parallel
    {
        float* scratch = (float*)malloc(sizeof(float) * TILE);
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            const float* xr = x + r * width;
            float sum = row_reduce_map(xr, width, 0, f_square, NULL, scratch);
            float mean = sum / (float)width;
            float rs = 1.0f / sqrtf(mean + eps);
            for (int64_t c = 0; c < width; ++c) y[r * width + c] = (xr[c] * rs) * w[c];
            rstd[r] = rs;
        }
        free(scratch);
    }
}

/* row_programs.rs:164-177: mu=sum/W; c=x-mu; var=sum(c*c)/W; r=rsqrt(var+eps); y=((c*r)*w)+b. */
ORC_API void orc_layer_norm(const float* x, const float* w, const float* b, float eps, int64_t rows,
                            int64_t width, float* y, float* mean_out, float* rstd) {
#pragma omp parallel
    {
        float* scratch = (float*)malloc(sizeof(float) * TILE);
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            const float* xr = x + r * width;
            float mean = row_reduce_map(xr, width, 0, NULL, NULL, scratch) / (float)width;
            float var = row_reduce_map(xr, width, 0, f_center_square, &mean, scratch) / (float)width;
            float rs = 1.0f / sqrtf(var + eps);
            for (int64_t c = 0; c < width; ++c) {
                float v = ((xr[c] - mean) * rs) * w[c];
                y[r * width + c] = v + (b ? b[c] : 0.0f);
            }
            mean_out[r] = mean; rstd[r] = rs;
        }
        free(scratch);
    }
}

/* row_programs.rs:135-143: m=max; s=x-m; e=exp(s); d=sum(e); y=e/d (log: y=s-ln d). */
ORC_API void orc_softmax(const float* x, int64_t rows, int64_t width, int logarithmic, float* y) {
#pragma omp parallel
    {
        float* scratch = (float*)malloc(sizeof(float) * TILE);
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            const float* xr = x + r * width;
            float m = row_reduce_map(xr, width, 1, NULL, NULL, scratch);
            float d = row_reduce_map(xr, width, 0, f_shift_exp, &m, scratch);
            float ld = logf(d);
            for (int64_t c = 0; c < width; ++c) {
                float s = xr[c] - m;
                y[r * width + c] = logarithmic ? s - ld : expf(s) / d;
            }
        }
        free(scratch);
    }
}

/* ---------------------------------------------------------------- element maps -------------- */
/* programs.rs:25,41: s=1/(1+exp(-x)); h=x*s; y=h*up. */
ORC_API void orc_silu_mul(const float* gate, const float* up, int64_t n, float* y) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float s = 1.0f / (1.0f + expf(-gate[i]));
        y[i] = (gate[i] * s) * up[i];
    }
}
/* affine_programs.rs:31-36: value=x; if residual value=value+res; value=value+bias[col]. */
ORC_API void orc_bias_add(const float* x, const float* bias, const float* residual, int64_t rows,
                          int64_t width, float* y) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < rows * width; ++i) {
        float v = x[i];
        if (residual) v = v + residual[i];
        y[i] = v + bias[i % width];
    }
}
/* rotary_programs.rs:63-93 (full) and :101-156 (prefix).  layout 0 = Interleaved, 1 = SplitHalf.
 * y = x*cos + ((x_pair*sin)*sign), sign = 2*side-1; backward subtracts.  Columns >= P keep bits.
 * table_row[r] gives the row of the [.., P/2] tables used by input row r. */
static void rotary_rows(const float* x, const float* cs, const float* sn, int64_t rows, int64_t width,
                        int64_t p, int layout, int backward, const int64_t* table_row, float* y) {
    int64_t half = p / 2;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        int64_t tr = table_row ? table_row[r] : r;
        for (int64_t c = 0; c < width; ++c) {
            float v = x[r * width + c];
            if (c < p) {
                int64_t pc, pair, side;
                if (layout == 0) { pair = c / 2; pc = pair * 2 + ((c + 1) % 2); side = c % 2; }
                else { pc = (c + half) % p; pair = c % half; side = c / half; }
                float sign = (float)side * 2.0f - 1.0f;
                float direct = v * cs[tr * half + pair];
                float rot = (x[r * width + pc] * sn[tr * half + pair]) * sign;
                v = backward ? direct - rot : direct + rot;
            }
            y[r * width + c] = v;
        }
    }
}
ORC_API void orc_rotary(const float* x, const float* cs, const float* sn, int64_t rows, int64_t width,
                        int layout, int backward, float* y) {
    rotary_rows(x, cs, sn, rows, width, width, layout, backward, NULL, y);
}
ORC_API void orc_rotary_prefix(const float* x, const float* cs, const float* sn, int32_t rank,
                               const int64_t* in_shape, const int64_t* table_shape, int64_t p,
                               int layout, int backward, float* y) {
    int64_t width = in_shape[rank - 1], rows = 1;
    for (int a = 0; a < rank - 1; ++a) rows *= in_shape[a];
    int64_t* table_row = (int64_t*)malloc(sizeof(int64_t) * (rows > 0 ? rows : 1));
    for (int64_t r = 0; r < rows; ++r) {
        int64_t rem = r, tr = 0, stride = 1;
        for (int a = rank - 2; a >= 0; --a) {
            int64_t coord = rem % in_shape[a]; rem /= in_shape[a];
            if (table_shape[a] != 1) tr += coord * stride;
            stride *= table_shape[a];
        }
        table_row[r] = tr;
    }
    rotary_rows(x, cs, sn, rows, width, p, layout, backward, table_row, y);
    free(table_row);
}
/* heads_programs.rs:43-55: Y[b,h,n,d] = X[b, h/(Hq/Hkv), n, d]; a bit copy. */
ORC_API void orc_repeat_kv_heads(const uint32_t* x, int64_t batch, int64_t kv_heads, int64_t q_heads,
                                 int64_t seq, int64_t width, uint32_t* y) {
    int64_t g = q_heads / kv_heads, plane_n = seq * width;
#pragma omp parallel for schedule(static)
    for (int64_t bh = 0; bh < batch * q_heads; ++bh) {
        int64_t b = bh / q_heads, h = bh % q_heads;
        memcpy(y + bh * plane_n, x + (b * kv_heads + h / g) * plane_n, sizeof(uint32_t) * plane_n);
    }
}
/* mask_programs.rs:19-39: -inf iff key_start+k > query_start+q (u64), else +0. */
ORC_API void orc_causal_mask(int64_t batch, int64_t queries, int64_t keys, uint64_t query_start,
                             uint64_t key_start, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t bq = 0; bq < batch * queries; ++bq) {
        uint64_t q = query_start + (uint64_t)(bq % queries);
        for (int64_t k = 0; k < keys; ++k)
            out[bq * keys + k] = key_start + (uint64_t)k > q ? -INFINITY : 0.0f;
    }
}
/* Embedding gather (rust-ascend-driver/src/tensor/runtime/indexing.rs:33-37): rows of the table. */
ORC_API void orc_embedding(const float* table, const int32_t* ids, int64_t count, int64_t width,
                           float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < count; ++i)
        memcpy(out + i * width, table + (int64_t)ids[i] * width, sizeof(float) * width);
}

/* Dense embedding weight gradient (rust-ascend-driver/src/tensor/embedding.rs:60-78; expectation written out in
 * examples/embedding_tensor.rs:44-53): rows accumulate in position order, the padding row (negative = none) receives
 * nothing, and with scale each touched row is divided by its number of occurrences afterwards. */
ORC_API void orc_embedding_backward(const float* grad, const int64_t* ids, int64_t count, int64_t width, int64_t rows,
                                    int64_t padding, int scale, float* out) {
    int64_t* freq = (int64_t*)calloc((size_t)(rows + 1), sizeof(int64_t));
    memset(out, 0, sizeof(float) * (size_t)(rows * width));
    for (int64_t p = 0; p < count; ++p) {
        int64_t id = ids[p];
        if (id == padding) continue;
        ++freq[id];
        for (int64_t c = 0; c < width; ++c) out[id * width + c] += grad[p * width + c];
    }
    if (scale)
        for (int64_t r = 0; r < rows; ++r)
            if (freq[r] != 0) for (int64_t c = 0; c < width; ++c) out[r * width + c] /= (float)freq[r];
    free(freq);
}

/* ---------------------------------------------------------------- BF16 GEMM ----------------- */
/* rust-ascend-kernels/src/tests.rs:93-103: inputs BF16-representable, f64 accumulation over k in
 * increasing order, result cast to f32 and, for BF16 output, rounded by bf16().  Transposes index
 * as a[t*m+i] / b[j*k+t].  Inputs here are rounded to BF16 first, which is the cast-then-GEMM rule
 * of rust-ascend-driver/src/tensor/runtime/matrix.rs:84-93. */
ORC_API void orc_gemm_bf16(const float* a, const float* b, int64_t batches, int64_t m, int64_t n,
                           int64_t k, int ta, int tb, int out_bf16, float* d) {
    for (int64_t batch = 0; batch < batches; ++batch) {
        const float* A = a + batch * m * k; const float* B = b + batch * n * k;
        float* D = d + batch * m * n;
        /* Pack to row-major [m,k] and [n,k] BF16-rounded copies so the inner loop is contiguous. */
        float* ap = (float*)malloc(sizeof(float) * (size_t)(m * k));
        float* bp = (float*)malloc(sizeof(float) * (size_t)(n * k));
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < m; ++i)
            for (int64_t t = 0; t < k; ++t) ap[i * k + t] = bf16r(ta ? A[t * m + i] : A[i * k + t]);
#pragma omp parallel for schedule(static)
        for (int64_t j = 0; j < n; ++j)
            for (int64_t t = 0; t < k; ++t) bp[j * k + t] = bf16r(tb ? B[j * k + t] : B[t * n + j]);
#pragma omp parallel for schedule(dynamic, 4)
        for (int64_t i = 0; i < m; ++i) {
            for (int64_t j = 0; j < n; ++j) {
                const float* ar = ap + i * k; const float* br = bp + j * k;
                double acc = 0.0;
                for (int64_t t = 0; t < k; ++t) acc += (double)ar[t] * (double)br[t];
                float v = (float)acc;
                D[i * n + j] = out_bf16 ? bf16r(v) : v;
            }
        }
        free(ap); free(bp);
    }
}
/* Linear with an FP32 epilogue as the B200 kernels fuse it: y = X*W^T (f64 accumulate -> f32);
 * mode 0: identity; 1: + bias[n] (affine_programs.rs:31-36); 2: SwiGLU of a gate/up pair
 * (src/nn/feed_forward.rs:39-41 with programs.rs:25,41), w holds gate rows [0,n) and wu the up
 * rows.  Output optionally rounded to BF16. */
ORC_API void orc_linear_epilogue(const float* x, const float* w, const float* wu, const float* bias,
                                 int64_t m, int64_t n, int64_t k, int mode, int out_bf16, float* y) {
    float* xp = (float*)malloc(sizeof(float) * (size_t)(m * k));
    float* wp = (float*)malloc(sizeof(float) * (size_t)(n * k));
    float* up = mode == 2 ? (float*)malloc(sizeof(float) * (size_t)(n * k)) : NULL;
    orc_bf16_array(x, xp, m * k); orc_bf16_array(w, wp, n * k);
    if (up) orc_bf16_array(wu, up, n * k);
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t i = 0; i < m; ++i) {
        for (int64_t j = 0; j < n; ++j) {
            const float* xr = xp + i * k; const float* wr = wp + j * k;
            double acc = 0.0;
            for (int64_t t = 0; t < k; ++t) acc += (double)xr[t] * (double)wr[t];
            float v = (float)acc;
            if (mode == 1) v = v + bias[j];
            if (mode == 2) {
                const float* ur = up + j * k; double au = 0.0;
                for (int64_t t = 0; t < k; ++t) au += (double)xr[t] * (double)ur[t];
                float s = 1.0f / (1.0f + expf(-v));
                v = (v * s) * (float)au;
            }
            y[i * n + j] = out_bf16 ? bf16r(v) : v;
        }
    }
    free(xp); free(wp); free(up);
}

/* ---------------------------------------------------------------- attention ----------------- */
/* src/nn/attention.rs:10-29 with matrix.rs:84-93: S = (sum_d bf16(q)*bf16(k))_f32 * scale (+mask);
 * P = softmax_f32(S) on the row schedule; O = sum_n bf16(P)*bf16(v) in f32.  GQA maps query head h
 * to KV head h/(Hq/Hkv) (src/nn/attention.rs:49-67, heads_programs.rs:48-52) and the causal mask
 * is -inf iff key_start+k > query_start+q (mask_programs.rs:30-37).
 * q [B,Hq,M,D], k [B,Hkv,N,D], v [B,Hkv,N,Dv], mask NULL or [B,Hq,M,N], out [B,Hq,M,Dv].
 * rows_limit > 0 evaluates only the first rows_limit query rows of every head (bounded sample). */
ORC_API void orc_attention(const float* q, const float* k, const float* v, const float* mask,
                           int64_t B, int64_t Hq, int64_t Hkv, int64_t M, int64_t N, int64_t D,
                           int64_t Dv, float scale, int causal, uint64_t query_start,
                           uint64_t key_start, int out_bf16, int64_t rows_limit, float* out) {
    int64_t g = Hq / Hkv, rows = rows_limit > 0 && rows_limit < M ? rows_limit : M;
    float* kb = (float*)malloc(sizeof(float) * (size_t)(B * Hkv * N * D + 1));
    float* vb = (float*)malloc(sizeof(float) * (size_t)(B * Hkv * N * Dv + 1));
    orc_bf16_array(k, kb, B * Hkv * N * D); orc_bf16_array(v, vb, B * Hkv * N * Dv);
#pragma omp parallel
    {
        float* s = (float*)malloc(sizeof(float) * (size_t)N);
        float* p = (float*)malloc(sizeof(float) * (size_t)N);
        float* qb = (float*)malloc(sizeof(float) * (size_t)D);
        double* acc_o = (double*)malloc(sizeof(double) * (size_t)Dv);
        float* scratch = (float*)malloc(sizeof(float) * TILE);
#pragma omp for schedule(dynamic, 8) collapse(2)
        for (int64_t bh = 0; bh < B * Hq; ++bh) {
            for (int64_t i = 0; i < rows; ++i) {
                int64_t b = bh / Hq, h = bh % Hq, kv = h / g;
                const float* kr = kb + (b * Hkv + kv) * N * D;
                const float* vr = vb + (b * Hkv + kv) * N * Dv;
                const float* qr = q + (bh * M + i) * D;
                for (int64_t c = 0; c < D; ++c) qb[c] = bf16r(qr[c]);
                for (int64_t j = 0; j < N; ++j) {
                    double acc = 0.0;
                    for (int64_t c = 0; c < D; ++c) acc += (double)qb[c] * (double)kr[j * D + c];
                    float sc = (float)acc * scale;
                    if (mask) sc = sc + mask[(bh * M + i) * N + j];
                    if (causal && key_start + (uint64_t)j > query_start + (uint64_t)i) sc = sc + -INFINITY;
                    s[j] = sc;
                }
                float mx = row_reduce_map(s, N, 1, NULL, NULL, scratch);
                float dn = row_reduce_map(s, N, 0, f_shift_exp, &mx, scratch);
                for (int64_t j = 0; j < N; ++j) p[j] = bf16r(expf(s[j] - mx) / dn);
                float* o = out + (bh * M + i) * Dv;
                for (int64_t c = 0; c < Dv; ++c) acc_o[c] = 0.0;
                for (int64_t j = 0; j < N; ++j) {
                    if (p[j] == 0.0f) continue; /* adding an exact zero product changes nothing */
                    double pj = (double)p[j];
                    for (int64_t c = 0; c < Dv; ++c) acc_o[c] += pj * (double)vr[j * Dv + c];
                }
                for (int64_t c = 0; c < Dv; ++c) {
                    float val = (float)acc_o[c];
                    o[c] = out_bf16 ? bf16r(val) : val;
                }
            }
        }
        free(acc_o);
        free(s); free(p); free(qb); free(scratch);
    }
    free(kb); free(vb);
}

/* ---------------------------------------------------------------- first-order backward ------ */
/* row_programs.rs:200-217 (RmsNormInputBackward): g=dy*w; mean=sum(g*x)/W; corr=mean*(r*r); dx=(g-x*corr)*r.
 * row_programs.rs:189-199 (RmsNormWeightContributions): (x*r)*dy per element, summed over the rows
 * (rust-ascend-driver/src/tensor/runtime/normalization.rs:95-114,168-186). */
ORC_API void orc_rms_norm_backward(const float* x, const float* w, const float* dy, const float* rstd, int64_t rows,
                                   int64_t width, float* dx, float* dw) {
    float* contrib = (float*)malloc(sizeof(float) * (size_t)(rows * width + 1));
#pragma omp parallel
    {
        float* scratch = (float*)malloc(sizeof(float) * TILE);
        float* gx = (float*)malloc(sizeof(float) * (size_t)(width + 1));
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            const float* xr = x + r * width; const float* gr = dy + r * width; float rs = rstd[r];
            for (int64_t c = 0; c < width; ++c) gx[c] = (gr[c] * w[c]) * xr[c];
            float mean = row_reduce_map(gx, width, 0, NULL, NULL, scratch) / (float)width;
            float corr = mean * (rs * rs);
            for (int64_t c = 0; c < width; ++c) {
                float g = gr[c] * w[c];
                dx[r * width + c] = (g - xr[c] * corr) * rs;
                contrib[r * width + c] = (xr[c] * rs) * gr[c];
            }
        }
        free(scratch); free(gx);
    }
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < width; ++c) {
        double acc = 0.0;   /* the reference sums pairwise in FP32; order is not part of the contract */
        for (int64_t r = 0; r < rows; ++r) acc += (double)contrib[r * width + c];
        dw[c] = (float)acc;
    }
    free(contrib);
}
/* row_programs.rs:152-163: softmax dx = y*(dy - sum(y*dy)); log-softmax dx = dy - exp(y)*sum(dy). */
ORC_API void orc_softmax_backward(const float* y, const float* dy, int64_t rows, int64_t width, int logarithmic, float* dx) {
#pragma omp parallel
    {
        float* scratch = (float*)malloc(sizeof(float) * TILE);
        float* prod = (float*)malloc(sizeof(float) * (size_t)(width + 1));
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            const float* yr = y + r * width; const float* gr = dy + r * width;
            if (logarithmic) {
                float dot = row_reduce_map(gr, width, 0, NULL, NULL, scratch);
                for (int64_t c = 0; c < width; ++c) dx[r * width + c] = gr[c] - expf(yr[c]) * dot;
            } else {
                for (int64_t c = 0; c < width; ++c) prod[c] = yr[c] * gr[c];
                float dot = row_reduce_map(prod, width, 0, NULL, NULL, scratch);
                for (int64_t c = 0; c < width; ++c) dx[r * width + c] = yr[c] * (gr[c] - dot);
            }
        }
        free(scratch); free(prod);
    }
}
/* programs.rs:29,43: s=sigmoid(x); h=x*s; ds=s*(1+x*(1-s)); dgate=(dy*up)*ds; dup=dy*h. */
ORC_API void orc_silu_mul_backward(const float* gate, const float* up, const float* dy, int64_t n, float* dgate, float* dup) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float x = gate[i];
        float s = 1.0f / (1.0f + expf(-x));
        float h = x * s;
        float ds = s * (1.0f + x * (1.0f - s));
        dgate[i] = (dy[i] * up[i]) * ds;
        dup[i] = dy[i] * h;
    }
}
/* heads_programs.rs:59-86: the gradient of a KV head is the sum of its query-head replicas. */
ORC_API void orc_repeat_kv_heads_backward(const float* dy, int64_t batch, int64_t kv_heads, int64_t q_heads, int64_t seq,
                                          int64_t width, float* dx) {
    int64_t g = q_heads / kv_heads, plane_n = seq * width;
#pragma omp parallel for schedule(static)
    for (int64_t bk = 0; bk < batch * kv_heads; ++bk) {
        int64_t b = bk / kv_heads, kv = bk % kv_heads;
        for (int64_t p = 0; p < plane_n; ++p) {
            double acc = 0.0;
            for (int64_t r = 0; r < g; ++r) acc += (double)dy[((b * q_heads + kv * g + r) * plane_n) + p];
            dx[bk * plane_n + p] = (float)acc;
        }
    }
}
/* affine.rs bias_backward: dbias[c] = sum of dY over every leading axis. */
ORC_API void orc_column_sum(const float* x, int64_t rows, int64_t width, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < width; ++c) {
        double acc = 0.0;
        for (int64_t r = 0; r < rows; ++r) acc += (double)x[r * width + c];
        out[c] = (float)acc;
    }
}

/* row_programs.rs (LayerNormInputBackward): n=(x-mean)*r; g=dy*w; dx=((g-mean(g)) - n*mean(g*n))*r;
 * LayerNormWeightContributions: n*dy summed over rows; the bias gradient is the column sum of dy. */
ORC_API void orc_layer_norm_backward(const float* x, const float* w, const float* dy, const float* mean, const float* rstd,
                                     int64_t rows, int64_t width, float* dx, float* dw, float* db) {
    float* contrib = (float*)malloc(sizeof(float) * (size_t)(rows * width + 1));
#pragma omp parallel
    {
        float* scratch = (float*)malloc(sizeof(float) * TILE);
        float* g = (float*)malloc(sizeof(float) * (size_t)(width + 1));
        float* gy = (float*)malloc(sizeof(float) * (size_t)(width + 1));
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            const float* xr = x + r * width; const float* gr = dy + r * width; float mu = mean[r], rs = rstd[r];
            for (int64_t c = 0; c < width; ++c) { float n = (xr[c] - mu) * rs; g[c] = gr[c] * w[c]; gy[c] = g[c] * n; }
            float mean_g = row_reduce_map(g, width, 0, NULL, NULL, scratch) / (float)width;
            float mean_gy = row_reduce_map(gy, width, 0, NULL, NULL, scratch) / (float)width;
            for (int64_t c = 0; c < width; ++c) {
                float n = (xr[c] - mu) * rs;
                dx[r * width + c] = ((g[c] - mean_g) - n * mean_gy) * rs;
                contrib[r * width + c] = n * gr[c];
            }
        }
        free(scratch); free(g); free(gy);
    }
    orc_column_sum(contrib, rows, width, dw);
    orc_column_sum(dy, rows, width, db);
    free(contrib);
}

/* Backward of the composed attention as the reference's autodiff builds it from its BF16 matmuls
 * (examples/grouped_attention_tensor.rs:14-44 states the rounding points): dP = bf16(dY) bf16(V)^T in FP32,
 * dS = P * (dP - sum(P*dP)) in FP32 (this is also the additive-mask gradient), then bf16(scale*dS) feeds
 * dQ = dS_b bf16(K) and dK = dS_b^T bf16(Q), and dV = bf16(P)^T bf16(dY).  K/V gradients of a KV head sum over the
 * query heads of its group (heads_programs.rs:59-86).  Shapes as orc_attention; dmask may be NULL. */
ORC_API void orc_attention_backward(const float* q, const float* k, const float* v, const float* dy, const float* mask,
                                    int64_t B, int64_t Hq, int64_t Hkv, int64_t M, int64_t N, int64_t D, int64_t Dv, float scale,
                                    int causal, uint64_t query_start, uint64_t key_start, float* dq, float* dk, float* dv, float* dmask) {
    int64_t g = Hq / Hkv;
    double* dk_acc = (double*)calloc((size_t)(B * Hkv * N * D + 1), sizeof(double));
    double* dv_acc = (double*)calloc((size_t)(B * Hkv * N * Dv + 1), sizeof(double));
    /* one (batch, kv head) per task so that the K/V accumulators are private to a thread */
#pragma omp parallel
    {
        float* s = (float*)malloc(sizeof(float) * (size_t)N);
        float* p = (float*)malloc(sizeof(float) * (size_t)N);
        float* dp = (float*)malloc(sizeof(float) * (size_t)N);
        float* scratch = (float*)malloc(sizeof(float) * TILE);
#pragma omp for schedule(dynamic, 1)
        for (int64_t bk = 0; bk < B * Hkv; ++bk) {
            int64_t b = bk / Hkv, kv = bk % Hkv;
            const float* kr = k + bk * N * D; const float* vr = v + bk * N * Dv;
            for (int64_t hh = 0; hh < g; ++hh) {
                int64_t bh = b * Hq + kv * g + hh;
                for (int64_t i = 0; i < M; ++i) {
                    const float* qr = q + (bh * M + i) * D; const float* gr = dy + (bh * M + i) * Dv;
                    for (int64_t j = 0; j < N; ++j) {
                        double acc = 0.0, accp = 0.0;
                        for (int64_t c = 0; c < D; ++c) acc += (double)bf16r(qr[c]) * (double)bf16r(kr[j * D + c]);
                        for (int64_t c = 0; c < Dv; ++c) accp += (double)bf16r(gr[c]) * (double)bf16r(vr[j * Dv + c]);
                        float sc = (float)acc * scale;
                        if (mask) sc = sc + mask[(bh * M + i) * N + j];
                        if (causal && key_start + (uint64_t)j > query_start + (uint64_t)i) sc = sc + -INFINITY;
                        s[j] = sc; dp[j] = (float)accp;
                    }
                    float mx = row_reduce_map(s, N, 1, NULL, NULL, scratch);
                    float dn = row_reduce_map(s, N, 0, f_shift_exp, &mx, scratch);
                    for (int64_t j = 0; j < N; ++j) p[j] = expf(s[j] - mx) / dn;
                    for (int64_t j = 0; j < N; ++j) s[j] = p[j] * dp[j];
                    float dot = row_reduce_map(s, N, 0, NULL, NULL, scratch);
                    float* dqr = dq + (bh * M + i) * D;
                    for (int64_t c = 0; c < D; ++c) dqr[c] = 0.0f;
                    double dq_acc[512];
                    for (int64_t c = 0; c < D; ++c) dq_acc[c] = 0.0;
                    for (int64_t j = 0; j < N; ++j) {
                        float ds = p[j] * (dp[j] - dot);
                        if (dmask) dmask[(bh * M + i) * N + j] = ds;
                        double pb = (double)bf16r(p[j]), dsb = (double)bf16r(ds * scale);
                        for (int64_t c = 0; c < Dv; ++c) dv_acc[(bk * N + j) * Dv + c] += pb * (double)bf16r(gr[c]);
                        for (int64_t c = 0; c < D; ++c) {
                            dq_acc[c] += dsb * (double)bf16r(kr[j * D + c]);
                            dk_acc[(bk * N + j) * D + c] += dsb * (double)bf16r(qr[c]);
                        }
                    }
                    for (int64_t c = 0; c < D; ++c) dqr[c] = (float)dq_acc[c];
                }
            }
        }
        free(s); free(p); free(dp); free(scratch);
    }
    for (int64_t i = 0; i < B * Hkv * N * D; ++i) dk[i] = (float)dk_acc[i];
    for (int64_t i = 0; i < B * Hkv * N * Dv; ++i) dv[i] = (float)dv_acc[i];
    free(dk_acc); free(dv_acc);
}

/* Causal cross entropy over logits [B,T,V] (src/nn/causal_lm.rs:118-196; examples/causal_lm_tensor.rs:24-118):
 * with shift, position t is scored against label t+1 and the last position is dropped; labels equal to ignore_index
 * are skipped.  loss_sum = sum(ln sum exp(x-max) + max - x[label]) on the FP32 row schedule, valid = counted tokens,
 * dlogits (may be NULL) = (softmax - onehot) * upstream / max(valid,1) for a mean loss with upstream gradient `upstream`. */
ORC_API void orc_causal_cross_entropy(const float* logits, const int64_t* labels, int64_t batch, int64_t time, int64_t vocab,
                                      int64_t ignore_index, int shift, float upstream, float* loss_sum, float* valid, float* dlogits) {
    int64_t steps = shift ? time - 1 : time, count = 0;
    double total = 0.0;
    float* scratch = (float*)malloc(sizeof(float) * TILE);
    if (dlogits) memset(dlogits, 0, sizeof(float) * (size_t)(batch * time * vocab));
    for (int64_t b = 0; b < batch; ++b)
        for (int64_t t = 0; t < steps; ++t) {
            int64_t label = labels[b * time + t + (shift ? 1 : 0)];
            if (label == ignore_index) continue;
            ++count;
        }
    for (int64_t b = 0; b < batch; ++b)
        for (int64_t t = 0; t < steps; ++t) {
            int64_t label = labels[b * time + t + (shift ? 1 : 0)];
            if (label == ignore_index) continue;
            const float* x = logits + (b * time + t) * vocab;
            float mx = row_reduce_map(x, vocab, 1, NULL, NULL, scratch);
            float dn = row_reduce_map(x, vocab, 0, f_shift_exp, &mx, scratch);
            total += (double)(-((x[label] - mx) - logf(dn)));   /* NLL of the log-softmax row */
            if (dlogits) {
                float* d = dlogits + (b * time + t) * vocab;
                float k = upstream / (float)(count > 0 ? count : 1);
                for (int64_t c = 0; c < vocab; ++c) d[c] = (expf(x[c] - mx) / dn - (c == label ? 1.0f : 0.0f)) * k;
            }
        }
    free(scratch);
    *loss_sum = (float)total; *valid = (float)count;
}
