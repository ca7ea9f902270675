"""Deterministic known-answer cases restated from the reference's own tests and device examples.

Inputs follow the reference's index formulas; expected values are computed here in float64 with the
same formulas the reference's checks use.  Each generator cites the file:line it restates.  Shared by
the CPU oracle tests and the GPU parity tests.
"""
import numpy as np


def bf16_f64(x):
    """BF16 round-to-nearest-even of float32 values, returned as float64
    (examples/causal_attention_tensor.rs:5-7)."""
    b = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    b = (b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFF0000
    return b.astype(np.uint32).view(np.float32).astype(np.float64)


# ---- RMSNorm: examples/rms_norm_runtime.rs:37-73, examples/rms_norm_tensor.rs:27-62 -------------
RMS_RUNTIME_SHAPES = [(0, 32), (1, 32), (3, 96), (7, 256), (33, 4096)]
RMS_TENSOR_SHAPES = RMS_RUNTIME_SHAPES + [(0, 4128), (1, 8192), (3, 8224), (0, 7), (1, 1), (3, 2), (3, 7),
                                          (3, 31), (3, 33), (3, 65), (3, 4095), (3, 4097), (3, 8225)]
RMS_EPS = 1e-3


def rms_case(rows, width):
    i = np.arange(rows * width)
    x = ((i % 31).astype(np.float32) / np.float32(7.0) - np.float32(1.0)).reshape(rows, width)
    w = (np.float32(0.5) + (np.arange(width) % 7).astype(np.float32) / np.float32(9.0))
    xd = x.astype(np.float64)
    r = 1.0 / np.sqrt((xd ** 2).sum(-1) / max(width, 1) + np.float64(np.float32(RMS_EPS)))
    y = xd * r[:, None] * w.astype(np.float64)
    return x, w, y, r


# ---- Softmax: examples/softmax_tensor.rs:25-48 ---------------------------------------------------
SOFTMAX_SHAPES = [(0, 32), (1, 32), (3, 96), (7, 256), (33, 4096), (0, 4128), (1, 4128), (3, 8192), (2, 8224),
                  (0, 7), (1, 1), (3, 2), (3, 7), (3, 31), (3, 33), (3, 65), (3, 4095), (3, 4097), (3, 8225)]


def softmax_case(rows, width, log):
    i = np.arange(rows * width)
    x = ((i % 31).astype(np.float32) / np.float32(4.0) - np.float32(1000.0)).reshape(rows, width)
    xd = x.astype(np.float64)
    if rows == 0:
        return x, xd
    m = xd.max(-1, keepdims=True)
    e = np.exp(xd - m)
    s = e.sum(-1, keepdims=True)
    return x, (xd - m - np.log(s)) if log else e / s


# ---- LayerNorm: rust-ascend-driver/examples/common_rows_validate.rs:60-65 shape set --------------
def layer_norm_case(rows, width, eps=1e-5, bias=True, seed=3):
    rng = np.random.default_rng(width + seed)
    x = rng.normal(size=(rows, width)).astype(np.float32)
    w = rng.normal(size=width).astype(np.float32)
    b = rng.normal(size=width).astype(np.float32) if bias else None
    xd = x.astype(np.float64)
    mean = xd.mean(-1) if width else np.zeros(rows)
    var = ((xd - mean[:, None]) ** 2).mean(-1)
    r = 1.0 / np.sqrt(var + eps)
    y = (xd - mean[:, None]) * r[:, None] * w.astype(np.float64)
    if b is not None:
        y = y + b.astype(np.float64)
    return x, w, b, y, mean, r


# ---- SiLU*up: examples/silu_mul_tensor.rs:25-46 ---------------------------------------------------
SILU_SIZES = [0, 1, 65, 1025]


def silu_mul_case(n):
    i = np.arange(n)
    x = (i % 41).astype(np.float32) * np.float32(0.6) - np.float32(12.0)
    u = (i % 13).astype(np.float32) * np.float32(0.125) - np.float32(0.5)
    a = x.astype(np.float64)
    return x, u, a * (1.0 / (1.0 + np.exp(-a))) * u.astype(np.float64)


# ---- bias / residual: rust-ascend-compiler/src/ascend/affine_programs.rs:47-70 -------------------
def bias_case(rows, width):
    n = rows * width
    i = np.arange(n)
    ordered = rows == 1 and width == 1
    x = np.full(n, 1e20, np.float32) if ordered else ((i % 13).astype(np.float32) / np.float32(8.0) - np.float32(0.5))
    bias = np.full(width, 1.0, np.float32) if ordered else ((np.arange(width) % 7).astype(np.float32) / np.float32(16.0) - np.float32(0.125))
    r = np.full(n, -1e20, np.float32) if ordered else ((i % 5).astype(np.float32) / np.float32(4.0) - np.float32(0.25))
    x, r = x.reshape(rows, width), r.reshape(rows, width)
    return x, bias, r, (x + bias[None, :]).astype(np.float32), ((x + r) + bias[None, :]).astype(np.float32)


# ---- RoPE: rotary_programs.rs:185-205 (host), examples/rotary_tensor.rs:23-45 ---------------------
def rotary_case(rows, width, layout, device_tables=False):
    n, half = rows * width, width // 2
    i = np.arange(n)
    x = (i % 19).astype(np.float32) * np.float32(0.25) - np.float32(2.0)
    t = np.arange(n // 2)
    if device_tables:  # examples/rotary_tensor.rs: angles (i%23)/8
        ang = (t % 23).astype(np.float64) * 0.125
        cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    else:  # rotary_programs.rs:190-191
        cos = np.float32(0.7) + (t % 3).astype(np.float32) * np.float32(0.125)
        sin = np.float32(-0.3) + (t % 5).astype(np.float32) * np.float32(0.0625)
    x = x.reshape(rows, width); cos = cos.reshape(rows, half); sin = sin.reshape(rows, half)
    xd, c, s = x.astype(np.float64), cos.astype(np.float64), sin.astype(np.float64)
    y = np.empty_like(xd)
    if layout == "interleaved":
        a, b = xd[:, 0::2], xd[:, 1::2]
        y[:, 0::2] = a * c - b * s
        y[:, 1::2] = b * c + a * s
    else:
        a, b = xd[:, :half], xd[:, half:]
        y[:, :half] = a * c - b * s
        y[:, half:] = b * c + a * s
    return x, cos, sin, y


# ---- RoPE prefix: rotary_programs.rs:224-260 -----------------------------------------------------
ROTARY_PREFIX_SHAPES = [([11], [3], 6), ([2, 5, 11], [1, 5, 3], 6), ([2, 3, 5, 11], [1, 1, 5, 3], 6),
                        ([2, 3, 5, 11], [2, 1, 5, 3], 6), ([2, 3, 5, 11], [1, 3, 1, 3], 6),
                        ([2, 3, 5, 11], [2, 3, 5, 3], 6), ([2, 1, 1, 1, 1, 3, 5, 11], [1, 1, 1, 1, 1, 1, 5, 3], 6),
                        ([0, 3, 5, 11], [1, 1, 5, 3], 6), ([2, 3, 0, 11], [1, 1, 0, 3], 6), ([2, 3, 5, 6], [1, 1, 5, 3], 6)]
SPECIAL_BITS = [0x80000000, 0x7FC01234, 0x7F800000, 0xFF800000]


def rotary_prefix_case(in_shape, table_shape, p, layout):
    n = int(np.prod(in_shape)); t = int(np.prod(table_shape)); width = in_shape[-1]; half = p // 2
    i = np.arange(n)
    vals = ((i % 17).astype(np.float32) / np.float32(8.0) - np.float32(0.75)).view(np.uint32)
    special = np.array(SPECIAL_BITS, dtype=np.uint32)[i % 4]
    xb = np.where((i % width) >= p, special, vals).astype(np.uint32)
    x = xb.view(np.float32).reshape(in_shape)
    tt = np.arange(t)
    cos = (np.float32(0.7) + (tt % 3).astype(np.float32) / np.float32(8.0)).reshape(table_shape)
    sin = (np.float32(-0.3) + (tt % 5).astype(np.float32) / np.float32(16.0)).reshape(table_shape)
    rows = n // width
    xr = x.reshape(rows, width).astype(np.float64)
    lead_in, lead_t = in_shape[:-1], table_shape[:-1]
    expected = xr.copy()
    cf, sf = cos.reshape(-1, half).astype(np.float64), sin.reshape(-1, half).astype(np.float64)
    for row in range(rows):
        rem, coords = row, []
        for dim in reversed(lead_in):
            coords.append(rem % dim); rem //= dim
        coords = coords[::-1]
        tr = 0
        for dim, c in zip(lead_t, coords):
            tr = tr * dim + (0 if dim == 1 else c)
        for pair in range(half):
            a, b = (2 * pair, 2 * pair + 1) if layout == "interleaved" else (pair, half + pair)
            c, s = cf[tr, pair], sf[tr, pair]
            expected[row, a] = xr[row, a] * c - xr[row, b] * s
            expected[row, b] = xr[row, b] * c + xr[row, a] * s
    return x, cos, sin, expected.reshape(in_shape)


# ---- KV repeat: heads_programs.rs:111-122 --------------------------------------------------------
def repeat_case(batch, heads, group, seq, width):
    n = batch * heads * seq * width
    bits = np.array([0, 0x80000000, 0x7FC01234, 0x7F800000, 0xFF800000, 0x3F800000], dtype=np.uint32)[np.arange(n) % 6]
    x = bits.view(np.float32).reshape(batch, heads, seq, width)
    return x, np.repeat(x.view(np.uint32), group, axis=1)


# ---- Causal mask: mask_programs.rs:47-66 ---------------------------------------------------------
MASK_SHAPES = [(0, 3, 7), (1, 3, 7), (2, 16, 32), (2, 32, 96)]
MASK_STARTS = [(0, 0), (29, 0), (9, 7), (1 << 40, 1 << 40), (2 ** 64 - 1 - 96, 2 ** 64 - 1 - 96)]


def mask_case(batch, queries, keys, qs, ks):
    q = np.array([qs + i for i in range(queries)], dtype=object)[:, None]
    k = np.array([ks + i for i in range(keys)], dtype=object)[None, :]
    bits = np.where((k > q).astype(bool), np.uint32(0xFF800000), np.uint32(0)).astype(np.uint32)
    return np.broadcast_to(bits, (batch, queries, keys)).copy()


# ---- GEMM: rust-ascend-kernels/src/tests.rs:89-117,124-132 ---------------------------------------
def gemm_kernel_case(batches, m, n, k, ta, tb):
    a = ((np.arange(batches * m * k) % 23).astype(np.float32) - np.float32(11.0)) / np.float32(16.0)
    b = ((np.arange(batches * n * k) % 17).astype(np.float32) - np.float32(8.0)) / np.float32(8.0)
    a = a.reshape((batches,) + ((k, m) if ta else (m, k)))
    b = b.reshape((batches,) + ((n, k) if tb else (k, n)))
    A = np.swapaxes(a, 1, 2) if ta else a
    B = np.swapaxes(b, 1, 2) if tb else b
    d = np.matmul(bf16_f64(A), bf16_f64(B))
    return a, b, d


# ---- GEMM via runtime: examples/matrix_runtime.rs:50-77 ------------------------------------------
def gemm_runtime_case(batches, ta, tb, m=32, n=48, k=16):
    a = ((np.arange(batches * m * k) % 17).astype(np.float32) - np.float32(8.0)) * np.float32(0.125)
    b = ((np.arange(batches * k * n) % 13).astype(np.float32) - np.float32(6.0)) * np.float32(0.25)
    a = a.reshape((batches,) + ((k, m) if ta else (m, k)))
    b = b.reshape((batches,) + ((n, k) if tb else (k, n)))
    A = np.swapaxes(a, 1, 2) if ta else a
    B = np.swapaxes(b, 1, 2) if tb else b
    return a, b, np.matmul(A.astype(np.float64), B.astype(np.float64))


# ---- Linear: examples/linear_tensor.rs:24-50 -----------------------------------------------------
def linear_case(m, n, k):
    x = (((np.arange(m * k) % 17).astype(np.float32) - np.float32(8.0)) * np.float32(0.125)).reshape(m, k)
    w = (((np.arange(n * k) % 13).astype(np.float32) - np.float32(6.0)) * np.float32(0.25)).reshape(n, k)
    return x, w, x.astype(np.float64) @ w.astype(np.float64).T


# ---- Attention: examples/attention_tensor.rs:23-68 -----------------------------------------------
def attention_uniform_case(n, masked, batch=2, m=32, d=16, dv=16):
    q = np.zeros((batch, m, d), np.float32); k = np.zeros((batch, n, d), np.float32)
    v = np.zeros((batch, n, dv), np.float32); mask = np.zeros((batch, m, n), np.float32)
    active = n // 2 if masked else n
    q[:, :, 0] = ((np.arange(m) % 3).astype(np.float32) - 1.0) * 0.5
    k[:, :, 1] = ((np.arange(n) % 5).astype(np.float32) - 2.0) * 0.25
    v[:, :, 0] = ((np.arange(n) % 5).astype(np.float32) - 2.0) * 0.125
    if masked:
        mask[:, :, active:] = -np.inf
    y = np.zeros((batch, m, dv)); y[:, :, 0] = v[:, :active, 0].astype(np.float64).sum(-1, keepdims=True) / active
    return q, k, v, (mask if masked else None), y


# ---- Causal attention: examples/causal_attention_tensor.rs:31-55 ----------------------------------
def causal_attention_case(n, cached, batch=2, m=32, d=16, dv=16):
    qs = n - m if cached else 0
    q = np.zeros((batch, m, d), np.float32); k = np.zeros((batch, n, d), np.float32)
    v = ((np.arange(batch * n * dv) % 7).astype(np.float32) / np.float32(8.0) - np.float32(0.375)).reshape(batch, n, dv)
    y = np.zeros((batch, m, dv))
    vb = bf16_f64(v)
    for row in range(m):
        active = min(qs + row + 1, n)
        p = bf16_f64(np.float32(1.0) / np.float32(active))
        y[:, row] = (p * vb[:, :active]).sum(1)
    return q, k, v, qs, y


# ---- GQA: examples/grouped_attention_tensor.rs:14-44,74-99 ----------------------------------------
GQA_CASES = [(3, 1, 32, False), (1, 3, 96, False), (3, 2, 32, False), (3, 5, 96, False), (3, 3, 96, True)]


def gqa_case(kv_heads, group, n, causal, batch=2, m=32, d=16, dv=16):
    heads = kv_heads * group
    q = ((np.arange(batch * heads * m * d) % 13).astype(np.float32) / np.float32(16.0) - np.float32(0.375)).reshape(batch, heads, m, d)
    k = ((np.arange(batch * kv_heads * n * d) % 17).astype(np.float32) / np.float32(16.0) - np.float32(0.5)).reshape(batch, kv_heads, n, d)
    v = ((np.arange(batch * kv_heads * n * dv) % 11).astype(np.float32) / np.float32(8.0) - np.float32(0.5)).reshape(batch, kv_heads, n, dv)
    prefix = n - m
    i = np.arange(batch * heads * m * n)
    if causal:
        mask = np.where((i % n) > prefix + (i // n) % m, np.float32(-np.inf), np.float32(0.0))
    else:
        mask = (i % 5).astype(np.float32) / np.float32(32.0) - np.float32(0.0625)
    mask = mask.astype(np.float32).reshape(batch, heads, m, n)
    qb, kb, vb = bf16_f64(q), bf16_f64(k), bf16_f64(v)
    kb, vb = np.repeat(kb, group, axis=1), np.repeat(vb, group, axis=1)
    s = 0.25 * np.einsum("bhmd,bhnd->bhmn", qb, kb) + mask.astype(np.float64)
    e = np.exp(s - s.max(-1, keepdims=True))
    p = e / e.sum(-1, keepdims=True)
    out = np.einsum("bhmn,bhnd->bhmd", bf16_f64(p.astype(np.float32)), vb)
    return q, k, v, mask, prefix, out


# ---- backward known-answer cases ------------------------------------------------------------------
def rms_backward_case(rows, width):
    """examples/rms_norm_runtime.rs:37-73: dy = (i%11)/5 - 0.7; f64 dX and dWeight."""
    x, w, _, r = rms_case(rows, width)
    dy = ((np.arange(rows * width) % 11).astype(np.float32) / np.float32(5.0) - np.float32(0.7)).reshape(rows, width)
    xd, wd, gd = x.astype(np.float64), w.astype(np.float64), dy.astype(np.float64)
    mean_gx = (gd * wd * xd).sum(-1, keepdims=True) / max(width, 1)
    dx = r[:, None] * (gd * wd - xd * (r ** 2)[:, None] * mean_gx)
    dw = (gd * xd * r[:, None]).sum(0)
    return x, w, dy, r.astype(np.float32), dx, dw


def softmax_backward_case(rows, width, log):
    """examples/softmax_tensor.rs:25-48 with a single upstream gradient (the example doubles it)."""
    x, y = softmax_case(rows, width, log)
    dy = ((np.arange(rows * width) % 11).astype(np.float32) / np.float32(5.0) - np.float32(0.7)).reshape(rows, width)
    g = dy.astype(np.float64)
    p = np.exp(y) if log else y
    dx = (g - p * g.sum(-1, keepdims=True)) if log else p * (g - (p * g).sum(-1, keepdims=True))
    return y.astype(np.float32), dy, dx


def silu_mul_backward_case(n):
    """examples/silu_mul_tensor.rs:25-46."""
    x, u, _ = silu_mul_case(n)
    dy = (np.arange(n) % 7).astype(np.float32) * np.float32(0.25) - np.float32(0.75)
    a = x.astype(np.float64); s = 1.0 / (1.0 + np.exp(-a)); d = s * (1.0 + a * (1.0 - s))
    return x, u, dy, dy.astype(np.float64) * u.astype(np.float64) * d, dy.astype(np.float64) * a * s


def linear_backward_case(m=32, n=48, k=16):
    """examples/matrix_runtime.rs:67-77: dX = dY W, dW = dY^T X with exactly representable values."""
    x = (((np.arange(m * k) % 17).astype(np.float32) - 8.0) * 0.125).reshape(m, k)
    w = (((np.arange(n * k) % 13).astype(np.float32) - 6.0) * 0.25).reshape(n, k)
    dy = (((np.arange(m * n) % 11).astype(np.float32) - 5.0) * 0.0625).reshape(m, n)
    return x, w, dy, dy.astype(np.float64) @ w.astype(np.float64), dy.astype(np.float64).T @ x.astype(np.float64)


# ---- device validation programs of the driver crate -----------------------------------------------
def driver_host(n, seed):
    """rust-ascend-driver/examples/deepgemm_validate.rs:6: ((i*7+seed)%17)/8 - 1, exactly representable in BF16."""
    return ((np.arange(n) * 7 + seed) % 17).astype(np.float32) / np.float32(8.0) - np.float32(1.0)


def driver_gemm_case(batch, ta, tb):
    """deepgemm_validate.rs:32-41: 32 x 64 x 48, batch 1 or 3; returns A, B in their stored shapes and the f64 product."""
    m, n, k = 32, 64, 48
    a = driver_host(batch * m * k, 1).reshape((batch, k, m) if ta else (batch, m, k))
    b = driver_host(batch * k * n, 4).reshape((batch, n, k) if tb else (batch, k, n))
    opa = a.transpose(0, 2, 1) if ta else a
    opb = b.transpose(0, 2, 1) if tb else b
    d = opa.astype(np.float64) @ opb.astype(np.float64)
    if batch == 1:
        return a[0], b[0], d[0]
    return a, b, d


def driver_grouped_case():
    """deepgemm_validate.rs:47-53: 512 x 64 x 48, ends [256, 256, 512] (an empty expert in the middle)."""
    m, n, k = 512, 64, 48
    a = driver_host(m * k, 2).reshape(m, k); w = driver_host(3 * n * k, 5).reshape(3, n, k)
    d = np.concatenate([a[:256].astype(np.float64) @ w[0].astype(np.float64).T, a[256:].astype(np.float64) @ w[2].astype(np.float64).T])
    return a, w, [256, 256, 512], d


def driver_linear_backward_case():
    """deepgemm_validate.rs:55-59: dX = dY W, dW = dY^T X for 32 x 64 x 48."""
    m, n, k = 32, 64, 48
    x = driver_host(m * k, 3).reshape(m, k); w = driver_host(n * k, 2).reshape(n, k); dy = driver_host(m * n, 7).reshape(m, n)
    return x, w, dy, dy.astype(np.float64) @ w.astype(np.float64), dy.astype(np.float64).T @ x.astype(np.float64)


COMMON_IR_SIZES = [1, 7, 256, 257, 1025]


def common_ir_case(n):
    """rust-ascend-driver/examples/common_ir_validate.rs:17-25: SiLU*up and its backward with f64 expectations."""
    i = np.arange(n)
    x = (i % 61).astype(np.float32) / np.float32(7.0) - np.float32(4.0)
    up = (i % 19).astype(np.float32) / np.float32(9.0) - np.float32(1.0)
    dy = (i % 11).astype(np.float32) / np.float32(8.0) - np.float32(0.5)
    a, b, g = x.astype(np.float64), up.astype(np.float64), dy.astype(np.float64)
    s = 1.0 / (1.0 + np.exp(-a)); h = a * s; d = s * (1.0 + a * (1.0 - s))
    return x, up, dy, h * b, g * b * d, g * h


PREFIX_TABLE_SHAPES = [(1, 1, 5, 3), (2, 1, 5, 3), (1, 3, 1, 3), (2, 3, 5, 3)]


def rotary_prefix_tensor_case(table_shape, layout):
    """examples/rotary_prefix_tensor.rs:16-45: x [2,3,5,11], prefix 6, tables with singleton axes; output and the input
    gradient for upstream dy (the example's factor 2 comes from its y*dy + y*dy and is left out here)."""
    batch, heads, seq, width, prefix = 2, 3, 5, 11, 6
    half = prefix // 2
    t = int(np.prod(table_shape)); n = batch * heads * seq * width
    cos = (np.float32(0.75) + (np.arange(t) % 3).astype(np.float32) / np.float32(16.0)).reshape(table_shape)
    sin = (np.float32(0.25) - (np.arange(t) % 5).astype(np.float32) / np.float32(32.0)).reshape(table_shape)
    x = ((np.arange(n) % 19).astype(np.float32) / np.float32(8.0) - np.float32(1.0)).reshape(batch, heads, seq, width)
    dy = ((np.arange(n) % 13).astype(np.float32) / np.float32(8.0) - np.float32(0.5)).reshape(batch, heads, seq, width)
    c = np.broadcast_to(cos, (batch, heads, seq, half)).astype(np.float64); s = np.broadcast_to(sin, (batch, heads, seq, half)).astype(np.float64)
    y = x.astype(np.float64).copy(); dx = dy.astype(np.float64).copy()
    if layout == "interleaved":
        ia, ib = slice(0, prefix, 2), slice(1, prefix, 2)
    else:
        ia, ib = slice(0, half), slice(half, prefix)
    xa, xb = x[..., ia].astype(np.float64), x[..., ib].astype(np.float64)
    ga, gb = dy[..., ia].astype(np.float64), dy[..., ib].astype(np.float64)
    y[..., ia] = xa * c - xb * s; y[..., ib] = xb * c + xa * s
    dx[..., ia] = ga * c + gb * s; dx[..., ib] = gb * c - ga * s
    return x, cos, sin, dy, y, dx


# ---- examples/bias_tensor.rs:11-41 and examples/frozen_bf16_tensor.rs:33-52 -----------------------------------------
BIAS_SHAPES = [(1,), (7,), (3, 31), (2, 3, 33), (5, 4097)]


def bias_tensor_case(shape):
    """Dyadic values, so every expectation is exact in FP32: outputs of the three modes and the bias gradient of dy."""
    count, width = int(np.prod(shape)), shape[-1]
    i = np.arange(count)
    x = ((i % 13).astype(np.float32) / np.float32(8.0) - np.float32(0.5)).reshape(shape)
    r = ((i % 5).astype(np.float32) / np.float32(4.0) - np.float32(0.25)).reshape(shape)
    b = (np.arange(width) % 7).astype(np.float32) / np.float32(16.0) - np.float32(0.125)
    dy = ((i % 11).astype(np.float32) / np.float32(8.0) - np.float32(0.375)).reshape(shape)
    db = dy.reshape(-1, width).astype(np.float64).sum(0).astype(np.float32)
    return x, r, b, dy, x + b, (x + r) + b, (x + x) + b, db


def frozen_linear_case(m, n, k):
    """X FP32 [m,k], fixed W [n,k] stored as BF16, upstream dY; Y = bf16(X) W^T and dX = bf16(dY) W in f64."""
    x = ((np.arange(m * k) % 17).astype(np.float32) * np.float32(0.037) - np.float32(0.25)).reshape(m, k)
    w = ((np.arange(n * k) % 13).astype(np.float32) * np.float32(0.019) - np.float32(0.125)).reshape(n, k)
    dy = ((np.arange(m * n) % 11).astype(np.float32) * np.float32(0.017) - np.float32(0.0625)).reshape(m, n)
    wb = bf16_f64(w)
    return x, w, dy, bf16_f64(x) @ wb.T, bf16_f64(dy) @ wb


# ---- examples/padded_attention_tensor.rs:47-62 ------------------------------------------------------------------------
PADDED_SDPA_SHAPES = [(1, 1, 1, 1, 1), (2, 3, 7, 5, 9), (1, 17, 33, 7, 3)]
PADDED_GQA_SHAPES = [(1, 4, 4, 1, 1, 1, 1), (2, 3, 1, 3, 7, 5, 9), (1, 6, 2, 17, 33, 7, 3), (2, 10, 2, 3, 31, 5, 7), (1, 9, 3, 3, 4097, 7, 9)]


def padded_attention_case(shape, mode):
    """shape = (b, h, kv, m, n, d, dv); mode 0 no mask, 1 additive mask, 2 causal with prefix n - m.  Returns q, k, v, mask."""
    b, h, kv, m, n, d, dv = shape
    q = ((np.arange(b * h * m * d) % 13).astype(np.float32) / np.float32(16.0) - np.float32(0.375)).reshape(b, h, m, d)
    k = ((np.arange(b * kv * n * d) % 17).astype(np.float32) / np.float32(16.0) - np.float32(0.5)).reshape(b, kv, n, d)
    v = ((np.arange(b * kv * n * dv) % 11).astype(np.float32) / np.float32(8.0) - np.float32(0.5)).reshape(b, kv, n, dv)
    i = np.arange(b * h * m * n)
    if mode == 0:
        mask = np.zeros(i.size, np.float32)
    elif mode == 1:
        mask = (i % 5).astype(np.float32) / np.float32(32.0) - np.float32(0.0625)
    else:
        mask = np.where(i % n > n - m + (i // n) % m, np.float32(-np.inf), np.float32(0.0)).astype(np.float32)
    return q, k, v, mask.reshape(b, h, m, n)


def padded_attention_expected(q, k, v, mask, scale=0.25):
    """The f64 reference of padded_attention_tensor.rs:14-36 (forward part): BF16-rounded Q, K, V and probabilities."""
    b, h, m, d = q.shape
    kv = k.shape[1]
    group = h // kv
    qb, kb, vb = bf16_f64(q), np.repeat(bf16_f64(k), group, axis=1), np.repeat(bf16_f64(v), group, axis=1)
    s = scale * np.einsum("bhmd,bhnd->bhmn", qb, kb) + mask.astype(np.float64)
    e = np.exp(s - s.max(-1, keepdims=True)); p = e / e.sum(-1, keepdims=True)
    return np.einsum("bhmn,bhnc->bhmc", bf16_f64(p.astype(np.float32)), vb)
