"""Operators that are compositions of other entry points.

Attention backward composed from the C ABI's matrix, softmax and head-reduction entry points, against the oracle that
tests/test_oracle_next.py pins to examples/grouped_attention_tensor.rs:14-44,74-99 (tolerance 2e-3 + 3e-3 relative, as
there), plus a larger seeded case with a scale that is not a power of two.  The M-grouped GEMM of deepgemm/plan.rs:61-67 as one
dense launch per expert, against the oracle's GEMM on each group's rows, with the empty-expert case of plan.rs:101.  The file name sorts it near the end of the suite: it
exercises compositions of entry points that the earlier files test one by one."""
import numpy as np
import pytest

import vectors as V
from test_backward import close

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _leave_no_sticky_error_behind(client):
    """A failure here must not follow the shared context into the files collected after this one."""
    yield
    try:
        client.take_errors()
    except Exception:
        pass


@pytest.mark.parametrize("kv_heads,group,n,causal", V.GQA_CASES)
def test_attention_backward_reference_example(client, oracle, kv_heads, group, n, causal):
    from rust_ascend_b200 import B200Runtime as RT
    q, k, v, mask, prefix, _ = V.gqa_case(kv_heads, group, n, causal)
    batch, heads, m, d = q.shape
    dv_ = v.shape[3]
    dy = ((np.arange(batch * heads * m * dv_) % 7).astype(np.float32) / np.float32(8.0) - np.float32(0.25)).reshape(batch, heads, m, dv_)
    up = client.upload
    if causal:
        want = oracle.attention_backward(q, k, v, dy, 0.25, causal=True, query_start=(1 << 40) + prefix, key_start=1 << 40)
        got = RT.attention_backward(client, up(q), up(k), up(v), up(dy), 0.25, causal=True, query_start=(1 << 40) + prefix, key_start=1 << 40)
    else:
        want = oracle.attention_backward(q, k, v, dy, 0.25, mask=mask, want_mask_grad=True)
        got = RT.attention_backward(client, up(q), up(k), up(v), up(dy), 0.25, mask=up(mask), want_mask_grad=True)
        assert got[3].shape == mask.shape
        close(client.read(got[3]), want[3], 2e-3, 3e-3)
    assert got[0].shape == q.shape and got[1].shape == k.shape and got[2].shape == v.shape
    for g, w in zip(got[:3], want[:3]):
        close(client.read(g), w, 2e-3, 3e-3)


def test_attention_backward_seeded_case_and_rejections(client, oracle):
    from rust_ascend_b200 import B200Runtime as RT, InvalidTensor
    rng = np.random.default_rng(33)
    b, hq, hkv, m, n, d, dv_ = 2, 4, 2, 48, 64, 32, 16
    q = rng.standard_normal((b, hq, m, d)).astype(np.float32); k = rng.standard_normal((b, hkv, n, d)).astype(np.float32)
    v = rng.standard_normal((b, hkv, n, dv_)).astype(np.float32); dy = rng.standard_normal((b, hq, m, dv_)).astype(np.float32)
    scale = float(1.0 / np.sqrt(d))
    up = client.upload
    want = oracle.attention_backward(q, k, v, dy, scale, causal=True, query_start=n - m, key_start=0)
    got = RT.attention_backward(client, up(q), up(k), up(v), up(dy), scale, causal=True, query_start=n - m, key_start=0)
    for g, w in zip(got, want):
        g = client.read(g)
        err = np.abs(g - w)
        assert np.all(np.isfinite(g)) and err.max() <= 2e-2 * max(1.0, np.abs(w).max()) and err.mean() <= 1e-2 * np.abs(w).mean() + 1e-5
    with pytest.raises(InvalidTensor):
        RT.attention_backward(client, up(q), up(k[:, :1].repeat(3, axis=1)), up(v), up(dy), scale)          # Hq % Hkv != 0 / KV mismatch
    with pytest.raises(InvalidTensor):
        RT.attention_backward(client, up(q), up(k), up(v), up(dy[:, :, :32]), scale)                           # upstream shape
    with pytest.raises(InvalidTensor):
        RT.attention_backward(client, up(q), up(k), up(v), up(dy), float("nan"))                                # the scale must be finite
    zero = RT.attention_backward(client, up(q), up(k), up(v), up(dy), 0.0)                                       # scale 0: uniform attention, no gradient into Q and K
    assert not client.read(zero[0]).any() and not client.read(zero[1]).any() and np.isfinite(client.read(zero[2])).all()


def test_grouped_gemm_matches_per_group_products(client, oracle):
    from rust_ascend_b200 import B200Runtime as RT, DType, InvalidTensor
    from rust_ascend_b200.runtime import bf16_bits_to_f32, f32_to_bf16_bits
    rng = np.random.default_rng(12)
    ends, n, k = [0, 256, 256, 768], 128, 64                      # plan.rs:101: aligned prefix sums with empty experts
    a = rng.standard_normal((ends[-1], k)).astype(np.float32); w = (rng.standard_normal((len(ends), n, k)) * 0.1).astype(np.float32)
    a16, w16 = f32_to_bf16_bits(a), f32_to_bf16_bits(w)
    want = np.zeros((ends[-1], n), np.float64)
    start = 0
    for g, end in enumerate(ends):
        if end > start:
            want[start:end] = oracle.gemm_bf16(bf16_bits_to_f32(a16[start:end]), bf16_bits_to_f32(w16[g]), False, True, False)
        start = end
    out = RT.gemm_grouped_nt(client, client.upload(a16), client.upload(w16), ends, DType.F32)
    assert out.shape == (768, 128)
    assert np.abs(client.read(out) - want).max() <= 1e-4 * max(1.0, np.abs(want).max())
    out16 = RT.gemm_grouped_nt(client, client.upload(a16), client.upload(w16), ends, DType.BF16)
    assert np.abs(bf16_bits_to_f32(client.read(out16)) - want).max() <= 2.0 ** -8 * np.abs(want).max() + 1e-6
    for bad in ([1, 17], [256, 0], [0, 0], []):                   # plan.rs:102
        with pytest.raises(InvalidTensor):
            RT.group_ends(bad)
    with pytest.raises(InvalidTensor):
        RT.gemm_grouped_nt(client, client.upload(a16), client.upload(w16), [256, 512], DType.F32)


def test_row_parallel_linear_allreduce_on_a_world_of_one(client, oracle):
    # One rank: the all-reduce is the identity, so the call must equal the GEMM, sequentially and in row chunks.
    from rust_ascend_b200 import DType
    from rust_ascend_b200.distributed import NcclCommunicator, SingleControl
    from rust_ascend_b200.runtime import bf16_bits_to_f32, f32_to_bf16_bits
    rng = np.random.default_rng(4)
    x = rng.standard_normal((512, 96)).astype(np.float32); w = (rng.standard_normal((192, 96)) * 0.1).astype(np.float32)
    x16, w16 = f32_to_bf16_bits(x), f32_to_bf16_bits(w)
    want = oracle.gemm_bf16(bf16_bits_to_f32(x16), bf16_bits_to_f32(w16), False, True, False)
    comm = NcclCommunicator.initialize(SingleControl(), client)
    try:
        for overlap in (False, True):
            out = comm.native.row_parallel_linear_allreduce(client.upload(x16), client.upload(w16), DType.F32, overlap)
            assert out.shape == (512, 192)
            assert np.abs(client.read(out) - want).max() <= 1e-4 * max(1.0, np.abs(want).max())
    finally:
        client.sync()
        comm.native.destroy()


# ---- the reference's device validation programs, through the C ABI -------------------------------------------------------
@pytest.mark.parametrize("batch", [1, 3])
@pytest.mark.parametrize("ta", [False, True])
@pytest.mark.parametrize("tb", [False, True])
def test_driver_gemm_validation_cases(client, batch, ta, tb):
    from rust_ascend_b200 import B200Runtime as RT, DType, Transpose
    from rust_ascend_b200.runtime import bf16_bits_to_f32, f32_to_bf16_bits
    a, b, d = V.driver_gemm_case(batch, ta, tb)                    # deepgemm_validate.rs:32-45: gemm, then gemm_into the same output
    da, db = client.upload(f32_to_bf16_bits(a)), client.upload(f32_to_bf16_bits(b))
    T = lambda flag: Transpose.Yes if flag else Transpose.No
    for dtype in (DType.BF16, DType.F32):
        out = RT.gemm(client, da, db, T(ta), T(tb), dtype)
        read = lambda: bf16_bits_to_f32(client.read(out)) if dtype == DType.BF16 else client.read(out)
        close(read(), d, 0.05, 0.01)
        client.memset(out, 0xFF)
        RT.gemm_into(client, da, db, T(ta), T(tb), out)
        close(read(), d, 0.05, 0.01)


def test_driver_grouped_and_linear_backward_cases(client):
    from rust_ascend_b200 import B200Runtime as RT, DType
    from rust_ascend_b200.runtime import bf16_bits_to_f32, f32_to_bf16_bits
    a, w, ends, d = V.driver_grouped_case()                        # deepgemm_validate.rs:47-53
    for dtype in (DType.BF16, DType.F32):
        out = client.read(RT.gemm_grouped_nt(client, client.upload(f32_to_bf16_bits(a)), client.upload(f32_to_bf16_bits(w)), ends, dtype))
        close(bf16_bits_to_f32(out) if dtype == DType.BF16 else out, d, 0.05, 0.01)
    x, w, dy, dx, dw = V.driver_linear_backward_case()             # deepgemm_validate.rs:55-59
    up = lambda v: client.upload(f32_to_bf16_bits(v))
    gdx, gdw = RT.linear_nt_backward(client, up(x), up(w), up(dy))
    close(bf16_bits_to_f32(client.read(gdx)), dx, 0.05, 0.01); close(client.read(gdw), dw, 0.05, 0.01)


@pytest.mark.parametrize("n", V.COMMON_IR_SIZES)
def test_common_ir_silu_programs(client, n):
    from rust_ascend_b200 import B200Runtime as RT
    x, up, dy, y, dgate, dup = V.common_ir_case(n)                 # common_ir_validate.rs:17-31
    dx, dup_, ddy = client.upload(x), client.upload(up), client.upload(dy)
    close(client.read(RT.silu_mul(client, dx, dup_)), y, 5e-4, 5e-4)
    g, u = RT.silu_mul_backward(client, dx, dup_, ddy)
    close(client.read(g), dgate, 5e-4, 5e-4); close(client.read(u), dup, 5e-4, 5e-4)


@pytest.mark.parametrize("table_shape", V.PREFIX_TABLE_SHAPES)
@pytest.mark.parametrize("layout", ["interleaved", "split_half"])
def test_rotary_prefix_tensor_example(client, table_shape, layout):
    from rust_ascend_b200 import B200Runtime as RT, RotaryLayout
    x, cos, sin, dy, y, dx = V.rotary_prefix_tensor_case(table_shape, layout)   # rotary_prefix_tensor.rs:16-45
    lay = RotaryLayout.Interleaved if layout == "interleaved" else RotaryLayout.SplitHalf
    dcos, dsin = client.upload(cos), client.upload(sin)
    got = client.read(RT.rotary_prefix(client, client.upload(x), dcos, dsin, 6, lay))
    close(got, y, 3e-5, 3e-5)
    np.testing.assert_array_equal(got[..., 6:].view(np.uint32), x[..., 6:].view(np.uint32))
    close(client.read(RT.rotary_prefix_backward(client, client.upload(dy), dcos, dsin, 6, lay)), dx, 3e-5, 3e-5)


@pytest.mark.parametrize("shape", V.BIAS_SHAPES)
def test_bias_tensor_example_is_exact(client, shape):
    from rust_ascend_b200 import B200Runtime as RT
    x, r, b, dy, plain, with_res, doubled, db = V.bias_tensor_case(shape)       # examples/bias_tensor.rs:11-41: exact equality
    dx, db_ = client.upload(x), client.upload(b)
    np.testing.assert_array_equal(client.read(RT.bias_add(client, dx, db_)), plain)
    np.testing.assert_array_equal(client.read(RT.bias_add(client, dx, db_, client.upload(r))), with_res)
    np.testing.assert_array_equal(client.read(RT.bias_add(client, dx, db_, client.upload(x))), doubled)
    np.testing.assert_array_equal(client.read(RT.bias_add_backward(client, client.upload(dy), x.shape)), db)


@pytest.mark.parametrize("m,n,k", [(16, 32, 32), (32, 48, 16)])
def test_frozen_linear_example(client, m, n, k):
    from rust_ascend_b200 import B200Runtime as RT
    from rust_ascend_b200.runtime import f32_to_bf16_bits
    x, w, dy, y, dx = V.frozen_linear_case(m, n, k)                # examples/frozen_bf16_tensor.rs:33-52
    stored = f32_to_bf16_bits(w)
    weight = client.upload(stored)
    close(client.read(RT.linear_frozen_bf16_fp32(client, client.upload(x), weight)), y, 5e-4, 5e-4)
    close(client.read(RT.linear_frozen_bf16_fp32_backward(client, x.shape, weight, client.upload(dy))), dx, 5e-4, 5e-4)
    np.testing.assert_array_equal(client.read(weight), stored)     # the fixed weight is never written


def test_nn_affine_and_frozen_wrappers(client, oracle):
    import rust_ascend_b200.nn as nn
    from rust_ascend_b200 import DType, InvalidTensor
    from rust_ascend_b200.runtime import bf16_bits_to_f32, f32_to_bf16_bits
    x, r, b, _, plain, with_res, _, _ = V.bias_tensor_case((3, 31))
    t = lambda a: nn.Tensor.from_data(client, a)
    np.testing.assert_array_equal(nn.bias_add(t(x), t(b)).into_data(), plain)
    np.testing.assert_array_equal(nn.residual_bias_add(t(x), t(r), t(b)).into_data(), with_res)
    xf, w, _, y, _ = V.frozen_linear_case(16, 32, 32)
    close(nn.linear_frozen_bf16_fp32(t(xf), t(f32_to_bf16_bits(w))).into_data(), y, 5e-4, 5e-4)
    rng = np.random.default_rng(2)                                  # SwiGLU with fixed weights against the oracle's fused Linear
    m, k, hidden, n = 32, 48, 64, 16
    xs = rng.standard_normal((m, k)).astype(np.float32)
    g16, u16, d16 = (f32_to_bf16_bits((rng.standard_normal(s) * 0.2).astype(np.float32)) for s in ((hidden, k), (hidden, k), (n, hidden)))
    out = nn.swiglu_frozen_bf16_fp32(t(xs), t(g16), t(u16), t(d16))
    assert out.dims() == [m, n] and out.dtype() == DType.F32
    hid = oracle.linear(xs, bf16_bits_to_f32(g16), w_up=bf16_bits_to_f32(u16))
    want = oracle.gemm_bf16(hid, bf16_bits_to_f32(d16), False, True, False)
    close(out.into_data(), want, 2e-3, 5e-3)
    with pytest.raises(InvalidTensor):
        nn.swiglu_frozen_bf16_fp32(t(xs), t(bf16_bits_to_f32(g16)), t(u16), t(d16))


def _as_dtype(x, dtype):
    from rust_ascend_b200 import DType
    from rust_ascend_b200.runtime import f32_to_bf16_bits
    return x.astype(np.float32) if dtype == DType.F32 else (x.astype(np.float16) if dtype == DType.F16 else f32_to_bf16_bits(x))


def _to_f64(raw, dtype):
    from rust_ascend_b200 import DType
    from rust_ascend_b200.runtime import bf16_bits_to_f32
    return (bf16_bits_to_f32(raw) if dtype == DType.BF16 else raw).astype(np.float64)


@pytest.mark.parametrize("dtype_name,tolerance", [("F32", 2e-6), ("F16", 2.0 ** -10), ("BF16", 2.0 ** -7)])
@pytest.mark.parametrize("a_shape,b_shape", [((2, 1, 3, 5), (1, 4, 5, 7)), ((32, 48), (48, 16)), ((3, 17, 33), (3, 33, 20)), ((2, 2, 16, 64), (64, 32))])
def test_tensor_matmul_keeps_the_dtype_and_broadcasts(client, dtype_name, tolerance, a_shape, b_shape):
    # Shape rules of generic_matrix.rs:60-73 (first case is the reference's own); values against an f64 product of the stored operands.
    from rust_ascend_b200 import B200Runtime as RT, DType
    dtype = DType[dtype_name]
    rng = np.random.default_rng(sum(a_shape) + len(b_shape))
    a = _as_dtype(rng.standard_normal(a_shape).astype(np.float32), dtype); b = _as_dtype(rng.standard_normal(b_shape).astype(np.float32), dtype)
    out = RT.tensor_matmul(client, client.upload(a), client.upload(b))
    want = np.matmul(_to_f64(a, dtype), _to_f64(b, dtype))
    assert out.dtype == dtype and out.shape == want.shape
    got = _to_f64(client.read(out), dtype)
    assert np.abs(got - want).max() <= tolerance * max(1.0, np.abs(want).max())


def test_tensor_matmul_empty_axes_and_rejections(client):
    from rust_ascend_b200 import B200Runtime as RT, DType, InvalidTensor
    z = lambda *shape: client.upload(np.zeros(shape, np.float32))
    assert RT.tensor_matmul(client, z(0, 5), z(5, 7)).shape == (0, 7)              # generic_matrix.rs:67-72
    out = RT.tensor_matmul(client, z(3, 0), z(0, 7))                                # generic_matrix.rs:73-78: empty contraction
    assert out.shape == (3, 7) and not client.read(out).any()
    with pytest.raises(InvalidTensor):
        RT.tensor_matmul(client, z(3, 5), z(4, 7))
    with pytest.raises(InvalidTensor):
        RT.tensor_matmul(client, z(3, 5), client.upload(np.zeros((5, 7), np.uint16)))
    with pytest.raises(InvalidTensor):
        RT.tensor_matmul(client, z(2, 3, 5), z(3, 5, 7))
    with pytest.raises(InvalidTensor):
        RT.matmul_fp32(client, client.upload(np.zeros((3, 5), np.float16)), client.upload(np.zeros((5, 7), np.float16)))


@pytest.mark.parametrize("dtype_name,tolerance", [("F32", 2e-6), ("F16", 2.0 ** -10), ("BF16", 2.0 ** -7)])
@pytest.mark.parametrize("log", [False, True])
def test_tensor_softmax_keeps_half_storage(client, dtype_name, tolerance, log):
    from rust_ascend_b200 import B200Runtime as RT, DType, InvalidTensor
    dtype = DType[dtype_name]
    x = _as_dtype((np.random.default_rng(9).standard_normal((5, 7, 96)) * 3).astype(np.float32), dtype)
    out = RT.tensor_softmax(client, client.upload(x), 2, log)
    assert out.dtype == dtype and out.shape == x.shape
    xf = _to_f64(x, dtype); e = np.exp(xf - xf.max(-1, keepdims=True)); p = e / e.sum(-1, keepdims=True)
    want = np.log(p) if log else p
    assert np.abs(_to_f64(client.read(out), dtype) - want).max() <= tolerance * max(1.0, np.abs(want).max())
    with pytest.raises(InvalidTensor):
        RT.tensor_softmax(client, client.upload(x), 0, log)


@pytest.mark.parametrize("shape", V.PADDED_SDPA_SHAPES)
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_padded_attention_reference_example(client, shape, mode):
    import rust_ascend_b200.nn as nn
    b, m, n, d, dv = shape                                          # examples/padded_attention_tensor.rs:66-77, 2e-3 + 3e-3 |b|
    q, k, v, mask = V.padded_attention_case((b, 1, 1, m, n, d, dv), mode)
    want = V.padded_attention_expected(q, k, v, mask)[:, 0]
    t = lambda a: nn.Tensor.from_data(client, np.ascontiguousarray(a))
    if mode == 2:
        out = nn.causal_attention_padded_bf16_fp32(t(q[:, 0]), t(k[:, 0]), t(v[:, 0]), 0.25, (1 << 40) + (n - m), 1 << 40)
    else:
        out = nn.scaled_dot_product_attention_padded_bf16_fp32(t(q[:, 0]), t(k[:, 0]), t(v[:, 0]), 0.25, t(mask[:, 0]) if mode == 1 else None)
    assert out.dims() == [b, m, dv]
    close(out.into_data(), want, 2e-3, 3e-3)


@pytest.mark.parametrize("shape", V.PADDED_GQA_SHAPES)
@pytest.mark.parametrize("mode", [1, 2])
def test_padded_grouped_attention_reference_example(client, shape, mode):
    import rust_ascend_b200.nn as nn
    b, h, kv, m, n, d, dv = shape                                   # examples/padded_attention_tensor.rs:86-98
    q, k, v, mask = V.padded_attention_case(shape, mode)
    want = V.padded_attention_expected(q, k, v, mask)
    t = lambda a: nn.Tensor.from_data(client, a)
    if mode == 2:
        out = nn.causal_grouped_query_attention_padded_bf16_fp32(t(q), t(k), t(v), 0.25, (1 << 40) + (n - m), 1 << 40)
    else:
        out = nn.grouped_query_attention_padded_bf16_fp32(t(q), t(k), t(v), 0.25, t(mask))
    assert out.dims() == [b, h, m, dv]
    close(out.into_data(), want, 2e-3, 3e-3)


def test_padded_attention_logical_keys_only(client):
    import rust_ascend_b200.nn as nn                                # examples/padded_attention_tensor.rs:99-105
    t = lambda a: nn.Tensor.from_data(client, np.asarray(a, np.float32))
    q, k, v = t(np.ones((1, 1, 1))), t(np.ones((1, 3, 1))), t(np.full((1, 3, 1), 2.0))
    close(nn.scaled_dot_product_attention_padded_bf16_fp32(q, k, v, 0.25).into_data(), [[[2.0]]], 2e-3, 3e-3)   # three equal BF16 probabilities
    masked = nn.scaled_dot_product_attention_padded_bf16_fp32(q, k, v, 0.25, t(np.full((1, 1, 3), -np.inf)))
    assert np.isnan(masked.into_data()).all()                       # every key excluded: no value, as in the reference


def test_composed_operators_reach_a_steady_state_of_device_memory(client):
    """A training loop drops its intermediate tensors every step, as the reference's handles release their storage on drop
    (runtime/mod.rs:501-515).  Fifty calls of the dtype-preserving matmul and of the padded attention must leave the bytes in use
    where they were after the first call."""
    import gc
    import rust_ascend_b200.nn as nn
    from rust_ascend_b200 import B200Runtime as RT
    rng = np.random.default_rng(4)
    a, b = client.upload(rng.standard_normal((3, 17, 33)).astype(np.float32)), client.upload(rng.standard_normal((3, 33, 20)).astype(np.float32))
    t = lambda x: nn.Tensor.from_data(client, x.astype(np.float32))
    q, k, v = t(rng.standard_normal((2, 5, 7))), t(rng.standard_normal((2, 9, 7))), t(rng.standard_normal((2, 9, 3)))

    def step():
        y = RT.tensor_matmul(client, a, b)
        z = nn.scaled_dot_product_attention_padded_bf16_fp32(q, k, v, 0.25)
        return y.shape, z.dims()

    step(); gc.collect(); client.sync()
    in_use = client.stats()["bytes_in_use"]
    for _ in range(50):
        step()
    gc.collect(); client.sync()
    assert client.stats()["bytes_in_use"] == in_use
