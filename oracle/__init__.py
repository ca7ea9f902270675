"""TEST INFRASTRUCTURE: ctypes front end of the CPU oracle (oracle.c).

The oracle restates the reference's arithmetic on the host so that the CUDA kernels can be checked
against it.  Only tests, the smoke check and the benchmark's CPU-baseline / reference leg may import
this package; the shipped runtime never does.  Function docstrings cite the reference file:line.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile oracle.c with the committed Makefile (gcc, OpenMP, contraction off)."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_bf16.restype = C.c_float
        _lib.orc_bf16.argtypes = [C.c_float]
        _lib.orc_threads.restype = C.c_int
    return _lib


def threads() -> int:
    return int(lib().orc_threads())


def use_all_cores() -> int:
    """Use every core this process may run on, whatever OMP_NUM_THREADS says (launchers such as torchrun set it to 1)."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().orc_set_threads(C.c_int(n))
    return threads()


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


_i64 = C.c_int64


def bf16(x) -> np.ndarray:
    """Round FP32 to the nearest BF16 value, ties to even, NaN/Inf truncated
    (rust-ascend-kernels/src/tests.rs:7-11)."""
    x = _f32(x)
    out = np.empty_like(x)
    lib().orc_bf16_array(_p(x), _p(out), _i64(x.size))
    return out


def to_bf16_bits(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f32_to_bf16_bits(_p(x), _p(out), _i64(x.size))
    return out


def from_bf16_bits(bits) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, dtype=np.float32)
    lib().orc_bf16_bits_to_f32(_p(bits), _p(out), _i64(bits.size))
    return out


def _rows(x: np.ndarray):
    width = x.shape[-1]
    rows = x.size // width if width else 0
    return rows, width


def row_reduce(x, op: str) -> np.ndarray:
    """Last-axis sum / mean / max on the 32-lane schedule (row_programs.rs:120-134)."""
    x = _f32(x)
    rows, width = _rows(x)
    out = np.empty(x.shape[:-1] + (1,), dtype=np.float32)
    lib().orc_row_reduce(_p(x), _i64(rows), _i64(width), C.c_int({"sum": 0, "mean": 1, "max": 2}[op]), _p(out))
    return out


def rms_norm(x, w, eps: float):
    """[y, rstd] of RMSNorm (row_programs.rs:144-151)."""
    x, w = _f32(x), _f32(w)
    rows, width = _rows(x)
    y = np.empty_like(x)
    rstd = np.empty(rows, dtype=np.float32)
    lib().orc_rms_norm(_p(x), _p(w), C.c_float(eps), _i64(rows), _i64(width), _p(y), _p(rstd))
    return y, rstd


def layer_norm(x, w, b, eps: float):
    """[y, mean, rstd] of LayerNorm (row_programs.rs:164-177); a missing bias is zeros."""
    x, w = _f32(x), _f32(w)
    b = None if b is None else _f32(b)
    rows, width = _rows(x)
    y = np.empty_like(x)
    mean = np.empty(rows, dtype=np.float32)
    rstd = np.empty(rows, dtype=np.float32)
    lib().orc_layer_norm(_p(x), _p(w), _p(b), C.c_float(eps), _i64(rows), _i64(width), _p(y), _p(mean), _p(rstd))
    return y, mean, rstd


def softmax(x, log: bool = False) -> np.ndarray:
    """Last-axis softmax / log-softmax (row_programs.rs:135-143)."""
    x = _f32(x)
    rows, width = _rows(x)
    y = np.empty_like(x)
    lib().orc_softmax(_p(x), _i64(rows), _i64(width), C.c_int(int(log)), _p(y))
    return y


def silu_mul(gate, up) -> np.ndarray:
    """(gate * sigmoid(gate)) * up (programs.rs:25,41)."""
    gate, up = _f32(gate), _f32(up)
    y = np.empty_like(gate)
    lib().orc_silu_mul(_p(gate), _p(up), _i64(gate.size), _p(y))
    return y


def bias_add(x, bias, residual=None) -> np.ndarray:
    """(x [+ residual]) + bias[col] in that order (affine_programs.rs:31-36)."""
    x, bias = _f32(x), _f32(bias)
    residual = None if residual is None else _f32(residual)
    rows, width = _rows(x)
    y = np.empty_like(x)
    lib().orc_bias_add(_p(x), _p(bias), _p(residual), _i64(rows), _i64(width), _p(y))
    return y


LAYOUTS = {"interleaved": 0, "split_half": 1}


def rotary(x, cos, sin, layout: str, backward: bool = False) -> np.ndarray:
    """Full last-axis rotation with same-row tables (rotary_programs.rs:47-97)."""
    x, cos, sin = _f32(x), _f32(cos), _f32(sin)
    rows, width = _rows(x)
    y = np.empty_like(x)
    lib().orc_rotary(_p(x), _p(cos), _p(sin), _i64(rows), _i64(width), C.c_int(LAYOUTS[layout]),
                     C.c_int(int(backward)), _p(y))
    return y


def rotary_prefix(x, cos, sin, width: int, layout: str, backward: bool = False) -> np.ndarray:
    """Rotate the first `width` columns with broadcast tables; the tail keeps its bits
    (rotary_programs.rs:101-156)."""
    x, cos, sin = _f32(x), _f32(cos), _f32(sin)
    rank = x.ndim
    ish = (C.c_int64 * rank)(*x.shape)
    tsh = (C.c_int64 * rank)(*cos.shape)
    y = np.empty_like(x)
    lib().orc_rotary_prefix(_p(x), _p(cos), _p(sin), C.c_int32(rank), ish, tsh, _i64(width),
                            C.c_int(LAYOUTS[layout]), C.c_int(int(backward)), _p(y))
    return y


def repeat_kv_heads(x, query_heads: int) -> np.ndarray:
    """Bit copy X[B,Hkv,N,D] -> Y[B,Hq,N,D] with kv = h // (Hq/Hkv) (heads_programs.rs:43-55)."""
    x = _f32(x)
    b, kv, n, d = x.shape
    y = np.empty((b, query_heads, n, d), dtype=np.float32)
    lib().orc_repeat_kv_heads(_p(x), _i64(b), _i64(kv), _i64(query_heads), _i64(n), _i64(d), _p(y))
    return y


def causal_mask(batch: int, queries: int, keys: int, query_start: int, key_start: int) -> np.ndarray:
    """-inf iff key_start+k > query_start+q with u64 positions (mask_programs.rs:19-39)."""
    out = np.empty((batch, queries, keys), dtype=np.float32)
    lib().orc_causal_mask(_i64(batch), _i64(queries), _i64(keys), C.c_uint64(query_start),
                          C.c_uint64(key_start), _p(out))
    return out


def embedding_backward(grad, ids, num_weights: int, padding_idx=None, scale_grad_by_freq: bool = False) -> np.ndarray:
    """Dense weight gradient [num_weights, W] (rust-ascend-driver/src/tensor/embedding.rs:60-78)."""
    grad = _f32(grad)
    ids = np.ascontiguousarray(ids, dtype=np.int64)
    width = grad.shape[-1]
    out = np.zeros((num_weights, width), dtype=np.float32)
    if out.size:
        lib().orc_embedding_backward(_p(grad), _p(ids), _i64(ids.size), _i64(width), _i64(num_weights),
                                     _i64(-1 if padding_idx is None else padding_idx), C.c_int(int(scale_grad_by_freq)), _p(out))
    return out


def embedding(table, ids) -> np.ndarray:
    """Row gather (rust-ascend-driver/src/tensor/runtime/indexing.rs:33-37)."""
    table = _f32(table)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    out = np.empty(ids.shape + (table.shape[1],), dtype=np.float32)
    lib().orc_embedding(_p(table), _p(ids), _i64(ids.size), _i64(table.shape[1]), _p(out))
    return out


def gemm_bf16(a, b, ta: bool, tb: bool, out_bf16: bool) -> np.ndarray:
    """D = op(A) op(B), BF16-rounded inputs, f64 accumulate, optional BF16 output rounding
    (rust-ascend-kernels/src/tests.rs:93-103; matrix.rs:84-93).  Rank 2 or equal-batch rank 3."""
    a, b = _f32(a), _f32(b)
    batched = a.ndim == 3
    batches = a.shape[0] if batched else 1
    am, bm = a.shape[-2:], b.shape[-2:]
    m, k = (am[1], am[0]) if ta else am
    n = bm[0] if tb else bm[1]
    d = np.empty(((batches,) if batched else ()) + (m, n), dtype=np.float32)
    lib().orc_gemm_bf16(_p(a), _p(b), _i64(batches), _i64(m), _i64(n), _i64(k), C.c_int(int(ta)),
                        C.c_int(int(tb)), C.c_int(int(out_bf16)), _p(d))
    return d


def linear(x, w, bias=None, w_up=None, out_bf16: bool = False) -> np.ndarray:
    """Y = X W^T with the fused FP32 epilogue of the B200 kernels: identity, + bias[n], or
    SwiGLU(gate=X W^T, up=X w_up^T) (src/nn.rs:77-79, affine_programs.rs:31-36,
    src/nn/feed_forward.rs:39-41)."""
    x, w = _f32(x), _f32(w)
    m, k = x.shape
    n = w.shape[0]
    mode = 2 if w_up is not None else (1 if bias is not None else 0)
    bias = None if bias is None else _f32(bias)
    w_up = None if w_up is None else _f32(w_up)
    y = np.empty((m, n), dtype=np.float32)
    lib().orc_linear_epilogue(_p(x), _p(w), _p(w_up), _p(bias), _i64(m), _i64(n), _i64(k), C.c_int(mode),
                              C.c_int(int(out_bf16)), _p(y))
    return y


def attention(q, k, v, scale: float, mask=None, causal: bool = False, query_start: int = 0,
              key_start: int = 0, out_bf16: bool = False, rows_limit: int = 0) -> np.ndarray:
    """Composed attention with the reference's rounding points (src/nn/attention.rs:10-29,49-80).
    q [B,Hq,M,D], k [B,Hkv,N,D], v [B,Hkv,N,Dv] (rank-3 inputs are treated as Hq=Hkv=1)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    squeeze = q.ndim == 3
    if squeeze:
        q, k, v = q[:, None], k[:, None], v[:, None]
        mask = None if mask is None else _f32(mask)[:, None]
    mask = None if mask is None else _f32(mask)
    b, hq, m, d = q.shape
    _, hkv, n, dv = v.shape
    out = np.zeros((b, hq, m, dv), dtype=np.float32)
    lib().orc_attention(_p(q), _p(k), _p(v), _p(mask), _i64(b), _i64(hq), _i64(hkv), _i64(m), _i64(n),
                        _i64(d), _i64(dv), C.c_float(scale), C.c_int(int(causal)), C.c_uint64(query_start),
                        C.c_uint64(key_start), C.c_int(int(out_bf16)), _i64(rows_limit), _p(out))
    return out[:, 0] if squeeze else out


def rms_norm_backward(x, w, dy, rstd):
    """[dx, dw] (row_programs.rs:189-217; normalization.rs:168-186)."""
    x, w, dy, rstd = _f32(x), _f32(w), _f32(dy), _f32(rstd)
    rows, width = _rows(x)
    dx = np.empty_like(x)
    dw = np.empty(width, dtype=np.float32)
    lib().orc_rms_norm_backward(_p(x), _p(w), _p(dy), _p(rstd), _i64(rows), _i64(width), _p(dx), _p(dw))
    return dx, dw


def softmax_backward(y, dy, log: bool = False) -> np.ndarray:
    """Input gradient from the saved forward output (row_programs.rs:152-163)."""
    y, dy = _f32(y), _f32(dy)
    rows, width = _rows(y)
    dx = np.empty_like(y)
    lib().orc_softmax_backward(_p(y), _p(dy), _i64(rows), _i64(width), C.c_int(int(log)), _p(dx))
    return dx


def silu_mul_backward(gate, up, dy):
    """[dgate, dup] (programs.rs:29,43)."""
    gate, up, dy = _f32(gate), _f32(up), _f32(dy)
    dg, du = np.empty_like(gate), np.empty_like(gate)
    lib().orc_silu_mul_backward(_p(gate), _p(up), _p(dy), _i64(gate.size), _p(dg), _p(du))
    return dg, du


def repeat_kv_heads_backward(dy, kv_heads: int) -> np.ndarray:
    """Sum of the replicas' gradients (heads_programs.rs:59-86)."""
    dy = _f32(dy)
    b, hq, n, d = dy.shape
    dx = np.empty((b, kv_heads, n, d), dtype=np.float32)
    lib().orc_repeat_kv_heads_backward(_p(dy), _i64(b), _i64(kv_heads), _i64(hq), _i64(n), _i64(d), _p(dx))
    return dx


def column_sum(x) -> np.ndarray:
    """Sum over every leading axis (bias gradient, affine.rs)."""
    x = _f32(x)
    rows, width = _rows(x)
    out = np.empty(width, dtype=np.float32)
    lib().orc_column_sum(_p(x), _i64(rows), _i64(width), _p(out))
    return out


def layer_norm_backward(x, w, dy, mean, rstd):
    """[dx, dw, db] (row_programs.rs LayerNormInputBackward / LayerNormWeightContributions)."""
    x, w, dy, mean, rstd = _f32(x), _f32(w), _f32(dy), _f32(mean), _f32(rstd)
    rows, width = _rows(x)
    dx = np.empty_like(x)
    dw, db = np.empty(width, dtype=np.float32), np.empty(width, dtype=np.float32)
    lib().orc_layer_norm_backward(_p(x), _p(w), _p(dy), _p(mean), _p(rstd), _i64(rows), _i64(width), _p(dx), _p(dw), _p(db))
    return dx, dw, db


def attention_backward(q, k, v, dy, scale: float, mask=None, causal: bool = False, query_start: int = 0, key_start: int = 0,
                       want_mask_grad: bool = False):
    """[dq, dk, dv(, dmask)] of the composed attention with the reference's rounding points
    (examples/grouped_attention_tensor.rs:14-44).  Rank-4 tensors as in `attention`."""
    q, k, v, dy = _f32(q), _f32(k), _f32(v), _f32(dy)
    mask = None if mask is None else _f32(mask)
    b, hq, m, d = q.shape
    _, hkv, n, dv_ = v.shape
    if d > 512:
        raise ValueError("head dim above 512")
    dq, dk, dv = np.empty_like(q), np.empty_like(k), np.empty_like(v)
    dmask = np.empty((b, hq, m, n), dtype=np.float32) if want_mask_grad else None
    lib().orc_attention_backward(_p(q), _p(k), _p(v), _p(dy), _p(mask), _i64(b), _i64(hq), _i64(hkv), _i64(m), _i64(n), _i64(d), _i64(dv_),
                                 C.c_float(scale), C.c_int(int(causal)), C.c_uint64(query_start), C.c_uint64(key_start), _p(dq), _p(dk), _p(dv), _p(dmask))
    return (dq, dk, dv, dmask) if want_mask_grad else (dq, dk, dv)


def causal_cross_entropy(logits, labels, ignore_index: int = -100, shift: bool = True, upstream: float = 1.0):
    """(loss_sum, valid_tokens, dlogits of the mean loss) (src/nn/causal_lm.rs:118-196)."""
    logits = _f32(logits)
    labels = np.ascontiguousarray(labels, dtype=np.int64)
    b, t, vocab = logits.shape
    loss, valid = C.c_float(), C.c_float()
    d = np.empty_like(logits)
    lib().orc_causal_cross_entropy(_p(logits), _p(labels), _i64(b), _i64(t), _i64(vocab), _i64(ignore_index), C.c_int(int(shift)),
                                   C.c_float(upstream), C.byref(loss), C.byref(valid), _p(d))
    return loss.value, valid.value, d
