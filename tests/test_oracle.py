"""CPU: pin the oracle against the reference's golden vectors and known-answer cases."""
import os

import numpy as np
import pytest

import vectors as V
from golden.make_row_golden import SHAPES, row_case_inputs

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "row_reference.npz"))


def close(actual, expected, atol, rtol):
    actual = np.asarray(actual, dtype=np.float64); expected = np.asarray(expected, dtype=np.float64)
    assert actual.shape == expected.shape
    assert np.all(np.isfinite(actual))
    err = np.abs(actual - expected) - (atol + rtol * np.abs(expected))
    assert err.size == 0 or err.max() <= 0, f"max excess {err.max()}"


@pytest.mark.parametrize("rows,width", SHAPES)
def test_row_schedule_matches_reference_numpy_statement(oracle, rows, width):
    # tools/ascend/tests/test_row_reference.py:7-28 outputs, stored by tests/golden/make_row_golden.py.
    x, big, w = row_case_inputs(rows, width)
    key = f"{rows}x{width}"
    np.testing.assert_array_equal(oracle.row_reduce(x, "max"), GOLDEN[f"max_{key}"])
    close(oracle.row_reduce(x, "sum"), GOLDEN[f"sum_{key}"], 2e-5, 2e-6)
    close(oracle.softmax(big), GOLDEN[f"softmax_{key}"], 1e-7, 2e-6)
    close(oracle.softmax(big, True), GOLDEN[f"logsoftmax_{key}"], 2e-6, 1e-6)
    y, r = oracle.rms_norm(x, w, 1e-5)
    close(y, GOLDEN[f"rms_y_{key}"], 1e-6, 2e-6)
    close(r[:, None], GOLDEN[f"rms_rstd_{key}"], 0, 2e-6)


def test_mean_accumulates_then_divides(oracle):
    # tools/ascend/tests/test_row_reference.py:93-95; row_tests.rs:229-231.
    x = np.full((3, 4096), 1000.0, np.float32)
    np.testing.assert_array_equal(oracle.row_reduce(x, "mean"), np.full((3, 1), 1000.0, np.float32))


def test_bf16_rounding_rule(oracle):
    # rust-ascend-kernels/src/tests.rs:7-11.
    bits = np.array([0x3F800000, 0x3F808000, 0x3F818000, 0x3F807FFF, 0x3F808001, 0x7F800000, 0xFF800000,
                     0x7FC01234, 0x80000000, 0x7F7FFFFF], dtype=np.uint32)
    got = oracle.bf16(bits.view(np.float32)).view(np.uint32)
    want = np.array([0x3F800000, 0x3F800000, 0x3F820000, 0x3F800000, 0x3F810000, 0x7F800000, 0xFF800000,
                     0x7FC00000, 0x80000000, 0x7F800000], dtype=np.uint32)
    np.testing.assert_array_equal(got, want)
    np.testing.assert_array_equal(oracle.from_bf16_bits(oracle.to_bf16_bits(bits.view(np.float32))).view(np.uint32), want)


@pytest.mark.parametrize("rows,width", V.RMS_TENSOR_SHAPES)
def test_rms_norm_examples(oracle, rows, width):
    x, w, y, r = V.rms_case(rows, width)
    got_y, got_r = oracle.rms_norm(x, w, V.RMS_EPS)
    close(got_y, y, 5e-4 * 0.01, 1e-5)  # reference device tolerance is 5e-4; the oracle is held to 1e-5
    close(got_r, r, 0, 1e-5)


@pytest.mark.parametrize("rows,width", V.SOFTMAX_SHAPES)
@pytest.mark.parametrize("log", [False, True])
def test_softmax_examples(oracle, rows, width, log):
    x, y = V.softmax_case(rows, width, log)
    close(oracle.softmax(x, log), y, 2e-6, 2e-6)


@pytest.mark.parametrize("rows,width", [(0, 32), (1, 32), (3, 96), (7, 256), (3, 4096), (3, 4097), (2, 33)])
@pytest.mark.parametrize("bias", [True, False])
def test_layer_norm(oracle, rows, width, bias):
    x, w, b, y, mean, r = V.layer_norm_case(rows, width, bias=bias)
    gy, gm, gr = oracle.layer_norm(x, w, b, 1e-5)
    close(gy, y, 2e-6, 1e-4); close(gm, mean, 1e-6, 1e-5); close(gr, r, 0, 1e-5)


@pytest.mark.parametrize("n", V.SILU_SIZES)
def test_silu_mul(oracle, n):
    x, u, y = V.silu_mul_case(n)
    close(oracle.silu_mul(x, u), y, 2e-6, 1e-6)


@pytest.mark.parametrize("rows", [0, 1, 2, 7])
@pytest.mark.parametrize("width", [1, 7, 31, 32, 33, 4097])
def test_bias_residual_order_is_exact(oracle, rows, width):
    x, bias, r, plain, with_res = V.bias_case(rows, width)
    np.testing.assert_array_equal(oracle.bias_add(x, bias), plain)
    np.testing.assert_array_equal(oracle.bias_add(x, bias, r), with_res)
    if rows == 1 and width == 1:
        assert with_res[0, 0] == 1.0  # (1e20 + -1e20) + 1, not 1e20 + (-1e20 + 1)


@pytest.mark.parametrize("width", [2, 6, 64, 96])
@pytest.mark.parametrize("rows", [0, 1, 3])
@pytest.mark.parametrize("layout", ["interleaved", "split_half"])
@pytest.mark.parametrize("device_tables", [False, True])
def test_rotary(oracle, width, rows, layout, device_tables):
    x, cos, sin, y = V.rotary_case(rows, width, layout, device_tables)
    close(oracle.rotary(x, cos, sin, layout), y, 2e-6, 0)
    # transpose Jacobian: backward(forward(x)) = (cos^2+sin^2) x
    if device_tables and rows:
        close(oracle.rotary(oracle.rotary(x, cos, sin, layout), cos, sin, layout, backward=True), x, 4e-6, 0)


@pytest.mark.parametrize("in_shape,table_shape,p", V.ROTARY_PREFIX_SHAPES)
@pytest.mark.parametrize("layout", ["interleaved", "split_half"])
def test_rotary_prefix_broadcast_and_tail_bits(oracle, in_shape, table_shape, p, layout):
    x, cos, sin, y = V.rotary_prefix_case(in_shape, table_shape, p, layout)
    got = oracle.rotary_prefix(x, cos, sin, p, layout)
    width = in_shape[-1]
    if x.size:
        g2, y2, x2 = got.reshape(-1, width), y.reshape(-1, width), x.reshape(-1, width)
        close(g2[:, :p], y2[:, :p], 3e-6, 3e-6)
        np.testing.assert_array_equal(g2[:, p:].view(np.uint32), x2[:, p:].view(np.uint32))


@pytest.mark.parametrize("batch", [0, 1, 2])
@pytest.mark.parametrize("heads", [1, 3])
@pytest.mark.parametrize("group", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("seq,width", [(0, 7), (3, 0), (3, 7), (2, 32)])
def test_repeat_kv_bits(oracle, batch, heads, group, seq, width):
    x, y = V.repeat_case(batch, heads, group, seq, width)
    np.testing.assert_array_equal(oracle.repeat_kv_heads(x, heads * group).view(np.uint32), y)


@pytest.mark.parametrize("batch,queries,keys", V.MASK_SHAPES)
@pytest.mark.parametrize("qs,ks", V.MASK_STARTS)
def test_causal_mask_bits(oracle, batch, queries, keys, qs, ks):
    np.testing.assert_array_equal(oracle.causal_mask(batch, queries, keys, qs, ks).view(np.uint32),
                                  V.mask_case(batch, queries, keys, qs, ks))


@pytest.mark.parametrize("ta", [False, True])
@pytest.mark.parametrize("tb", [False, True])
@pytest.mark.parametrize("out_bf16", [False, True])
@pytest.mark.parametrize("batches,m,n,k", [(1, 80, 96, 144), (3, 16, 32, 16)])
def test_gemm_kernel_vectors(oracle, ta, tb, out_bf16, batches, m, n, k):
    a, b, d = V.gemm_kernel_case(batches, m, n, k, ta, tb)
    got = oracle.gemm_bf16(a, b, ta, tb, out_bf16)
    want = V.bf16_f64(d.astype(np.float32)) if out_bf16 else d
    close(got, want, 1e-4, 0)  # rust-ascend-kernels/src/tests.rs:117


@pytest.mark.parametrize("batches", [1, 2])
@pytest.mark.parametrize("ta", [False, True])
@pytest.mark.parametrize("tb", [False, True])
def test_gemm_runtime_vectors(oracle, batches, ta, tb):
    a, b, d = V.gemm_runtime_case(batches, ta, tb)
    close(oracle.gemm_bf16(a, b, ta, tb, False), d, 5e-4, 5e-4)
    close(oracle.gemm_bf16(a, b, ta, tb, True), d, 5e-4, 4e-3)


@pytest.mark.parametrize("m,n,k", [(16, 32, 16), (32, 48, 32)])
def test_linear_vectors(oracle, m, n, k):
    x, w, y = V.linear_case(m, n, k)
    close(oracle.linear(x, w), y, 5e-4, 5e-4)
    close(oracle.gemm_bf16(x, w, False, True, False), y, 5e-4, 5e-4)


def test_swiglu_zero_gate_gives_zero(oracle):
    # examples/swiglu_tensor.rs:22-40: zero gate weight -> zero hidden activation.
    width = 16
    x = (((np.arange(width * width) % 7).astype(np.float32) - 3.0) * 0.125).reshape(width, width)
    up = np.eye(width, dtype=np.float32) * 0.5
    h = oracle.linear(x, np.zeros((width, width), np.float32), w_up=up)
    np.testing.assert_array_equal(h, np.zeros_like(h))
    # and a non-trivial gate agrees with the composed definition
    rng = np.random.default_rng(5)
    g = rng.normal(size=(32, 16)).astype(np.float32); u = rng.normal(size=(32, 16)).astype(np.float32)
    composed = oracle.silu_mul(oracle.linear(x, g), oracle.linear(x, u))
    np.testing.assert_array_equal(oracle.linear(x, g, w_up=u), composed)


@pytest.mark.parametrize("n", [32, 8192])
@pytest.mark.parametrize("masked", [False, True])
def test_attention_uniform(oracle, n, masked):
    q, k, v, mask, y = V.attention_uniform_case(n, masked)
    close(oracle.attention(q, k, v, 0.25, mask=mask), y, 5e-4, 5e-4)


@pytest.mark.parametrize("n", [32, 96])
@pytest.mark.parametrize("cached", [False, True])
def test_causal_attention(oracle, n, cached):
    q, k, v, qs, y = V.causal_attention_case(n, cached)
    close(oracle.attention(q, k, v, 0.25, causal=True, query_start=qs, key_start=0), y, 3e-4, 3e-4)
    mask = oracle.causal_mask(q.shape[0], q.shape[1], n, qs, 0)
    np.testing.assert_array_equal(oracle.attention(q, k, v, 0.25, mask=mask),
                                  oracle.attention(q, k, v, 0.25, causal=True, query_start=qs))


@pytest.mark.parametrize("kv_heads,group,n,causal", V.GQA_CASES)
def test_gqa(oracle, kv_heads, group, n, causal):
    q, k, v, mask, prefix, out = V.gqa_case(kv_heads, group, n, causal)
    if causal:
        got = oracle.attention(q, k, v, 0.25, causal=True, query_start=(1 << 40) + prefix, key_start=1 << 40)
    else:
        got = oracle.attention(q, k, v, 0.25, mask=mask)
    close(got, out, 2e-3, 3e-3)
    # GQA equals MHA over explicitly repeated heads (src/nn/attention.rs:61-66)
    rk, rv = oracle.repeat_kv_heads(k, kv_heads * group), oracle.repeat_kv_heads(v, kv_heads * group)
    np.testing.assert_array_equal(oracle.attention(q, rk, rv, 0.25, mask=mask), oracle.attention(q, k, v, 0.25, mask=mask))
