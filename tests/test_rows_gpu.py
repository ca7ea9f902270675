"""GPU parity (through the C ABI): row programs and element maps against the CPU oracle and the
reference's known-answer vectors.  FP32 tolerance: 1e-5 relative (norms), bit-exact for copies/masks."""
import numpy as np
import pytest

import vectors as V
from rust_ascend_b200 import B200Runtime as RT
from rust_ascend_b200 import DType, InvalidTensor, RotaryLayout
from rust_ascend_b200.runtime import bf16_bits_to_f32, f32_to_bf16_bits

pytestmark = pytest.mark.gpu
LAYOUT = {"interleaved": RotaryLayout.Interleaved, "split_half": RotaryLayout.SplitHalf}


def close(actual, expected, atol, rtol):
    actual = np.asarray(actual, dtype=np.float64); expected = np.asarray(expected, dtype=np.float64)
    assert actual.shape == expected.shape
    assert np.all(np.isfinite(actual))
    err = np.abs(actual - expected) - (atol + rtol * np.abs(expected))
    assert err.size == 0 or err.max() <= 0, f"max excess {err.max()}"


@pytest.mark.parametrize("rows,width", V.RMS_TENSOR_SHAPES)
def test_rms_norm_reference_examples(client, oracle, rows, width):
    x, w, y, r = V.rms_case(rows, width)
    out, rstd = RT.rms_norm(client, client.upload(x.reshape(1, rows, width)), client.upload(w), V.RMS_EPS)
    assert out.shape == (1, rows, width) and rstd.shape == (rows,)
    oy, orr = oracle.rms_norm(x, w, V.RMS_EPS)
    close(client.read(out)[0], oy, 1e-7, 1e-5); close(client.read(rstd), orr, 0, 1e-5)
    close(client.read(out)[0], y, 0, 5e-4 * 0.1); close(client.read(rstd), r, 0, 1e-5)


@pytest.mark.parametrize("rows,width,seed", [(4096, 4096, 0), (257, 4096, 1), (64, 8192, 2), (1000, 1024, 3), (33, 128, 4), (5, 16384, 5), (3, 16388, 6)])
def test_rms_norm_random_against_oracle(client, oracle, rows, width, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, width), dtype=np.float32); w = rng.uniform(0.5, 1.5, width).astype(np.float32)
    out, rstd = RT.rms_norm(client, client.upload(x), client.upload(w), 1e-6)
    oy, orr = oracle.rms_norm(x, w, 1e-6)
    close(client.read(out), oy, 1e-7, 1e-5); close(client.read(rstd), orr, 0, 1e-5)


def test_rms_norm_bf16_storage(client, oracle):
    rng = np.random.default_rng(11)
    x = bf16_bits_to_f32(f32_to_bf16_bits(rng.standard_normal((130, 4096), dtype=np.float32)))
    w = bf16_bits_to_f32(f32_to_bf16_bits(rng.uniform(0.5, 1.5, 4096).astype(np.float32)))
    out, _ = RT.rms_norm(client, client.upload(f32_to_bf16_bits(x)), client.upload(f32_to_bf16_bits(w)), 1e-5)
    want = oracle.bf16(oracle.rms_norm(x, w, 1e-5)[0])
    got = bf16_bits_to_f32(client.read(out))
    # identical up to one BF16 ulp where the FP32 value sits on a rounding boundary
    assert np.mean(got != want) < 1e-3 and np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-3)) <= 2 ** -7


@pytest.mark.parametrize("rows,width", V.SOFTMAX_SHAPES)
@pytest.mark.parametrize("log", [False, True])
def test_softmax_reference_examples(client, oracle, rows, width, log):
    x, y = V.softmax_case(rows, width, log)
    t = client.upload(x.reshape(1, rows, width))
    out = RT.log_softmax(client, t) if log else RT.softmax(client, t)
    got = client.read(out)[0]
    close(got, y, 2e-5, 1e-4)                       # examples/softmax_tensor.rs:9
    close(got, oracle.softmax(x, log), 2e-6, 1e-5)  # against the oracle


@pytest.mark.parametrize("rows,width", [(0, 32), (1, 32), (3, 96), (7, 256), (3, 4096), (3, 4097), (2, 33), (600, 1024)])
@pytest.mark.parametrize("bias", [True, False])
def test_layer_norm(client, oracle, rows, width, bias):
    x, w, b, y, mean, r = V.layer_norm_case(rows, width, bias=bias)
    out, m, rs = RT.layer_norm(client, client.upload(x), client.upload(w), client.upload(b) if bias else None, 1e-5)
    oy, om, orr = oracle.layer_norm(x, w, b, 1e-5)
    close(client.read(out), oy, 2e-6, 1e-5); close(client.read(m), om, 1e-6, 1e-5); close(client.read(rs), orr, 0, 1e-5)
    close(client.read(out), y, 2e-6, 1e-4)


@pytest.mark.parametrize("op", ["sum", "mean", "max"])
@pytest.mark.parametrize("rows,width", [(0, 32), (1, 32), (7, 256), (33, 4096), (3, 4097), (3, 7)])
def test_row_reductions(client, oracle, op, rows, width):
    x = np.random.default_rng(40 + rows + width).normal(size=(rows, width)).astype(np.float32)
    t = client.upload(x)
    out = {"sum": RT.sum_last, "mean": RT.mean_last, "max": RT.max_last}[op](client, t)
    assert out.shape == (rows, 1)
    got = client.read(out)
    if op == "max":
        np.testing.assert_array_equal(got, oracle.row_reduce(x, "max"))
    else:
        close(got, oracle.row_reduce(x, op), 3e-5, 3e-5)


def test_mean_of_constant_rows_is_exact(client):
    x = np.full((3, 4096), 1000.0, np.float32)
    np.testing.assert_array_equal(client.read(RT.mean_last(client, client.upload(x))), np.full((3, 1), 1000.0, np.float32))


@pytest.mark.parametrize("n", V.SILU_SIZES + [4096 * 33 + 3])
def test_silu_mul(client, oracle, n):
    if n > 2000:
        rng = np.random.default_rng(n); x = rng.normal(size=n).astype(np.float32) * 4; u = rng.normal(size=n).astype(np.float32)
        y = None
    else:
        x, u, y = V.silu_mul_case(n)
    got = client.read(RT.silu_mul(client, client.upload(x.reshape(1, n)), client.upload(u.reshape(1, n))))[0]
    close(got, oracle.silu_mul(x, u), 1e-6, 1e-5)
    if y is not None:
        close(got, y, 2e-5, 1e-4)


@pytest.mark.parametrize("rows", [0, 1, 2, 7])
@pytest.mark.parametrize("width", [1, 7, 31, 32, 33, 4097])
def test_bias_residual_order_is_exact(client, rows, width):
    x, bias, r, plain, with_res = V.bias_case(rows, width)
    np.testing.assert_array_equal(client.read(RT.bias_add(client, client.upload(x), client.upload(bias))), plain)
    np.testing.assert_array_equal(client.read(RT.bias_add(client, client.upload(x), client.upload(bias), client.upload(r))), with_res)


@pytest.mark.parametrize("width", [2, 6, 64, 96])
@pytest.mark.parametrize("rows", [0, 1, 3])
@pytest.mark.parametrize("layout", ["interleaved", "split_half"])
def test_rotary_full(client, oracle, width, rows, layout):
    x, cos, sin, y = V.rotary_case(rows, width, layout, device_tables=True)
    tx, tc, ts = client.upload(x), client.upload(cos), client.upload(sin)
    got = client.read(RT.rotary(client, tx, tc, ts, LAYOUT[layout]))
    np.testing.assert_array_equal(got, oracle.rotary(x, cos, sin, layout))  # same rounded operations
    close(got, y, 2e-5, 1e-4)
    back = client.read(RT.rotary_backward(client, tx, tc, ts, LAYOUT[layout]))
    np.testing.assert_array_equal(back, oracle.rotary(x, cos, sin, layout, backward=True))


@pytest.mark.parametrize("in_shape,table_shape,p", V.ROTARY_PREFIX_SHAPES)
@pytest.mark.parametrize("layout", ["interleaved", "split_half"])
def test_rotary_prefix_broadcast_and_tail_bits(client, oracle, in_shape, table_shape, p, layout):
    x, cos, sin, y = V.rotary_prefix_case(in_shape, table_shape, p, layout)
    got = client.read(RT.rotary_prefix(client, client.upload(x), client.upload(cos), client.upload(sin), p, LAYOUT[layout]))
    want = oracle.rotary_prefix(x, cos, sin, p, layout)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    width = in_shape[-1]
    if x.size:
        np.testing.assert_array_equal(got.reshape(-1, width)[:, p:].view(np.uint32), x.reshape(-1, width)[:, p:].view(np.uint32))
        close(got.reshape(-1, width)[:, :p], y.reshape(-1, width)[:, :p], 3e-6, 3e-6)


def test_rotary_rejects_bad_shapes(client):
    x = client.upload(np.zeros((2, 3, 5, 11), np.float32))
    for table, p in [((1, 1, 5, 3), 5), ((1, 1, 5, 3), 12), ((1, 2, 5, 3), 6), ((1, 1, 5, 4), 6), ((1, 5, 3), 6)]:
        t = client.upload(np.zeros(table, np.float32))
        with pytest.raises(InvalidTensor):
            RT.rotary_prefix(client, x, t, t, p, RotaryLayout.SplitHalf)
    with pytest.raises(InvalidTensor):
        t = client.upload(np.zeros((3, 1), np.float32))
        RT.rotary(client, client.upload(np.zeros((3, 3), np.float32)), t, t, RotaryLayout.SplitHalf)


@pytest.mark.parametrize("batch", [0, 1, 2])
@pytest.mark.parametrize("heads", [1, 3])
@pytest.mark.parametrize("group", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("seq,width", [(0, 7), (3, 0), (3, 7), (2, 32)])
def test_repeat_kv_bits(client, batch, heads, group, seq, width):
    x, y = V.repeat_case(batch, heads, group, seq, width)
    got = client.read(RT.repeat_kv_heads(client, client.upload(x), heads * group))
    np.testing.assert_array_equal(got.view(np.uint32), y)


def test_repeat_kv_rejects_indivisible_heads(client):
    with pytest.raises(InvalidTensor, match="divisible"):
        RT.repeat_kv_heads(client, client.upload(np.zeros((2, 3, 5, 7), np.float32)), 5)


@pytest.mark.parametrize("batch,queries,keys", V.MASK_SHAPES)
@pytest.mark.parametrize("qs,ks", V.MASK_STARTS)
def test_causal_mask_bits(client, batch, queries, keys, qs, ks):
    got = client.read(RT.causal_mask(client, batch, queries, keys, qs, ks))
    np.testing.assert_array_equal(got.view(np.uint32), V.mask_case(batch, queries, keys, qs, ks))


def test_causal_mask_position_overflow_is_rejected(client):
    with pytest.raises(InvalidTensor, match="overflow"):
        RT.causal_mask(client, 1, 8, 8, 2 ** 64 - 4, 0)


def test_cast_is_round_to_nearest_even(client, oracle):
    x = np.random.default_rng(3).standard_normal(100003).astype(np.float32) * 100
    x[:6] = np.array([0x3F808000, 0x3F818000, 0x7F800000, 0xFF800000, 0x80000000, 0x3F807FFF], dtype=np.uint32).view(np.float32)
    t = RT.cast(client, client.upload(x), DType.BF16)
    np.testing.assert_array_equal(client.read(t), oracle.to_bf16_bits(x))
    back = RT.cast(client, t, DType.F32)
    np.testing.assert_array_equal(client.read(back), oracle.bf16(x))


def test_embedding_lookup(client, oracle):
    rng = np.random.default_rng(9)
    table = rng.standard_normal((1000, 64), dtype=np.float32); ids = rng.integers(0, 1000, size=(3, 17)).astype(np.int32)
    got = client.read(RT.embedding(client, client.upload(table), client.upload(ids)))
    np.testing.assert_array_equal(got, oracle.embedding(table, ids))
    got64 = client.read(RT.embedding(client, client.upload(f32_to_bf16_bits(table)), client.upload(ids.astype(np.int64))))
    np.testing.assert_array_equal(got64, f32_to_bf16_bits(table)[ids])


def test_validation_errors_are_invalid_tensor_not_fallback(client):
    x = client.upload(np.zeros((4, 64), np.float32)); w = client.upload(np.ones(64, np.float32))
    with pytest.raises(InvalidTensor, match="epsilon"):
        RT.rms_norm(client, x, w, 0.0)
    with pytest.raises(InvalidTensor, match="epsilon"):
        RT.rms_norm(client, x, w, float("nan"))
    with pytest.raises(InvalidTensor):
        RT.rms_norm(client, x, client.upload(np.ones(32, np.float32)), 1e-5)
    strided = type(x)(x.handle, (4, 32), DType.F32, (64, 1))
    with pytest.raises(InvalidTensor, match="contiguous"):
        RT.softmax(client, strided)
    with pytest.raises(InvalidTensor):
        RT.softmax(client, client.upload(np.zeros((4, 64), np.int32)))


def test_counters_and_storage(client):
    before = client.stats()
    x = client.upload(np.arange(64, dtype=np.float32).reshape(2, 32))
    y = RT.softmax(client, x); empty = client.upload(np.zeros((0, 32), np.float32)); y_empty = RT.softmax(client, empty)
    client.sync()
    after = client.stats()
    assert after["launches"] == before["launches"] + 1 and after["empty_calls"] == before["empty_calls"] + 1
    assert after["allocations"] >= before["allocations"] + 3      # x, y, empty (a zero-byte tensor still owns storage), y_empty
    del y, y_empty, empty
    assert client.stats()["allocations"] == before["allocations"] + 1   # dropping a tensor releases its storage; x is still held
    assert client.read_one(x.handle) == np.arange(64, dtype=np.float32).tobytes()
    client.free(x.handle)
    from rust_ascend_b200.runtime import NullHandle
    with pytest.raises(NullHandle):
        RT.softmax(client, x)
