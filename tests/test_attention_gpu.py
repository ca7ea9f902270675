"""GPU parity (through the C ABI): attention against the CPU oracle and the reference's attention vectors.
BF16 tolerance on the tensor-core path: max abs error <= 2e-2, mean relative error <= 1e-2 against the oracle
(FP32 softmax, BF16-rounded P, FP32 accumulate)."""
import numpy as np
import pytest

import vectors as V
from rust_ascend_b200 import B200Runtime as RT
from rust_ascend_b200 import DType, InvalidTensor, RotaryLayout, TensorBuffer, nn
from rust_ascend_b200.runtime import bf16_bits_to_f32, f32_to_bf16_bits

pytestmark = pytest.mark.gpu


def r16(x):
    return bf16_bits_to_f32(f32_to_bf16_bits(np.asarray(x, dtype=np.float32)))


def up16(client, x):
    return client.upload(f32_to_bf16_bits(x))


def check_bf16(got, want):
    got = got.astype(np.float64); want = want.astype(np.float64)
    assert np.all(np.isfinite(got))
    err = np.abs(got - want)
    assert err.max() <= 2e-2, f"max abs {err.max()} at {np.unravel_index(err.argmax(), err.shape)}"
    assert err.sum() / max(np.abs(want).sum(), 1e-30) <= 1e-2, f"mean rel {err.sum() / np.abs(want).sum()}"


def close(actual, expected, atol, rtol):
    actual = np.asarray(actual, dtype=np.float64); expected = np.asarray(expected, dtype=np.float64)
    assert actual.shape == expected.shape and np.all(np.isfinite(actual))
    err = np.abs(actual - expected) - (atol + rtol * np.abs(expected))
    assert err.max() <= 0, f"max excess {err.max()}"


# ---- reference vectors through the nn mirror (FP32 storage, general kernel) -------------------------------
@pytest.mark.parametrize("n", [32, 8192])
@pytest.mark.parametrize("masked", [False, True])
def test_reference_uniform_attention(client, n, masked):
    q, k, v, mask, y = V.attention_uniform_case(n, masked)
    T = lambda a: None if a is None else nn.Tensor.from_data(client, a)
    out = nn.scaled_dot_product_attention_bf16_fp32(T(q), T(k), T(v), 0.25, T(mask))
    close(out.into_data(), y, 5e-4, 5e-4)  # examples/attention_tensor.rs:5-12


@pytest.mark.parametrize("n", [32, 96])
@pytest.mark.parametrize("cached", [False, True])
def test_reference_causal_attention(client, oracle, n, cached):
    q, k, v, qs, y = V.causal_attention_case(n, cached)
    T = lambda a: nn.Tensor.from_data(client, a)
    out = nn.causal_attention_bf16_fp32(T(q), T(k), T(v), 0.25, qs, 0).into_data()
    close(out, y, 3e-4, 3e-4)  # examples/causal_attention_tensor.rs:8-13
    close(out, oracle.attention(q, k, v, 0.25, causal=True, query_start=qs), 1e-5, 1e-4)


@pytest.mark.parametrize("kv_heads,group,n,causal", V.GQA_CASES)
def test_reference_grouped_query_attention(client, oracle, kv_heads, group, n, causal):
    q, k, v, mask, prefix, want = V.gqa_case(kv_heads, group, n, causal)
    T = lambda a: nn.Tensor.from_data(client, a)
    if causal:
        out = nn.causal_grouped_query_attention_bf16_fp32(T(q), T(k), T(v), 0.25, (1 << 40) + prefix, 1 << 40)
        ref = oracle.attention(q, k, v, 0.25, causal=True, query_start=(1 << 40) + prefix, key_start=1 << 40)
    else:
        out = nn.grouped_query_attention_bf16_fp32(T(q), T(k), T(v), 0.25, T(mask))
        ref = oracle.attention(q, k, v, 0.25, mask=mask)
    got = out.into_data()
    close(got, want, 2e-3, 3e-3)   # examples/grouped_attention_tensor.rs:6-11
    close(got, ref, 2e-4, 2e-3)    # one BF16 ulp of P where the FP32 exp differs in the last bit


def test_attention_domain_errors(client):
    T = lambda shape: nn.Tensor.from_data(client, np.zeros(shape, np.float32))
    # src/nn/attention.rs:108-132
    for n in (31, 4097):
        with pytest.raises(InvalidTensor):
            nn.scaled_dot_product_attention_bf16_fp32(T((2, 32, 16)), T((2, n, 16)), T((2, n, 32)), 0.25)
    with pytest.raises(InvalidTensor):
        nn.scaled_dot_product_attention_bf16_fp32(T((2, 32, 16)), T((1, 64, 16)), T((2, 64, 32)), 0.25)
    with pytest.raises(InvalidTensor):
        nn.scaled_dot_product_attention_bf16_fp32(T((2, 32, 16)), T((2, 64, 16)), T((2, 64, 32)), float("nan"))
    with pytest.raises(InvalidTensor, match="divisible"):
        nn.grouped_query_attention_bf16_fp32(T((2, 5, 32, 16)), T((2, 3, 96, 16)), T((2, 3, 96, 16)), 0.25)
    with pytest.raises(InvalidTensor):
        nn.grouped_query_attention_bf16_fp32(T((2, 6, 32, 16)), T((2, 3, 96, 16)), T((2, 2, 96, 16)), 0.25)


# ---- tensor-core kernel (BF16, head dim 128) ----------------------------------------------------------------
def rand_qkv(seed, b, hq, hkv, m, n):
    rng = np.random.default_rng(seed)
    return (r16(rng.standard_normal((b, hq, m, 128), dtype=np.float32)), r16(rng.standard_normal((b, hkv, n, 128), dtype=np.float32)),
            r16(rng.standard_normal((b, hkv, n, 128), dtype=np.float32)))


SCALE = 1.0 / np.sqrt(128.0)


@pytest.mark.parametrize("b,hq,hkv,m,n,causal,qs", [
    (1, 1, 1, 128, 128, False, 0), (1, 1, 1, 128, 128, True, 0), (1, 2, 2, 256, 256, True, 0), (2, 4, 4, 384, 384, True, 0),
    (1, 2, 1, 512, 512, True, 0), (2, 8, 2, 256, 640, False, 0), (1, 4, 1, 128, 1024, True, 896), (1, 2, 2, 48, 96, True, 48),
    (1, 3, 3, 400, 416, True, 16), (1, 2, 2, 16, 32, False, 0), (1, 1, 1, 272, 2048, True, 1776)])
def test_tensor_core_attention_against_oracle(client, oracle, b, hq, hkv, m, n, causal, qs):
    q, k, v = rand_qkv(b + hq + m + n, b, hq, hkv, m, n)
    out = RT.attention(client, up16(client, q), up16(client, k), up16(client, v), SCALE, causal=causal, query_start=qs, key_start=0)
    got = bf16_bits_to_f32(client.read(out))
    want = oracle.attention(q, k, v, SCALE, causal=causal, query_start=qs, key_start=0)
    check_bf16(got, want)


def test_large_absolute_positions_and_bmhd_output(client, oracle):
    q, k, v = rand_qkv(77, 2, 4, 2, 256, 384)
    base = (1 << 40)
    out = RT.attention(client, up16(client, q), up16(client, k), up16(client, v), SCALE, causal=True, query_start=base + 128, key_start=base, bmhd_output=True)
    assert out.shape == (2, 256, 4, 128)
    got = bf16_bits_to_f32(client.read(out)).transpose(0, 2, 1, 3)
    check_bf16(got, oracle.attention(q, k, v, SCALE, causal=True, query_start=base + 128, key_start=base))


def test_strided_bshd_inputs(client, oracle):
    # Q/K/V stored [B,S,H,D] (the layout a QKV projection writes) presented as [B,H,S,D] through strides.
    b, hq, hkv, m = 2, 4, 2, 256
    q, k, v = rand_qkv(5, b, hq, hkv, m, m)
    def strided(x):
        phys = np.ascontiguousarray(x.transpose(0, 2, 1, 3))  # [B,S,H,D]
        t = up16(client, phys)
        bb, ss, hh, dd = phys.shape
        return TensorBuffer(t.handle, (bb, hh, ss, dd), DType.BF16, (ss * hh * dd, dd, hh * dd, 1), _owner=t._owner)   # the view keeps the storage alive
    out = RT.attention(client, strided(q), strided(k), strided(v), SCALE, causal=True, bmhd_output=True)
    got = bf16_bits_to_f32(client.read(out)).transpose(0, 2, 1, 3)
    check_bf16(got, oracle.attention(q, k, v, SCALE, causal=True))


@pytest.mark.parametrize("layout", ["split_half", "interleaved"])
def test_fused_rotary(client, oracle, layout):
    b, hq, hkv, m, n, qs = 1, 4, 2, 256, 384, 128
    q, k, v = rand_qkv(9, b, hq, hkv, m, n)
    pos = np.arange(n, dtype=np.float64)[:, None]
    inv = 10000.0 ** (-np.arange(64, dtype=np.float64) * 2 / 128)
    cos, sin = np.cos(pos * inv).astype(np.float32), np.sin(pos * inv).astype(np.float32)
    out = RT.attention(client, up16(client, q), up16(client, k), up16(client, v), SCALE, causal=True, query_start=qs, key_start=0,
                       cos=client.upload(cos), sin=client.upload(sin),
                       rotary_layout=RotaryLayout.SplitHalf if layout == "split_half" else RotaryLayout.Interleaved)
    tq = np.broadcast_to(cos[qs:qs + m], (b, hq, m, 64)), np.broadcast_to(sin[qs:qs + m], (b, hq, m, 64))
    tk = np.broadcast_to(cos[:n], (b, hkv, n, 64)), np.broadcast_to(sin[:n], (b, hkv, n, 64))
    qr = oracle.bf16(oracle.rotary(q, tq[0], tq[1], layout)); kr = oracle.bf16(oracle.rotary(k, tk[0], tk[1], layout))
    check_bf16(bf16_bits_to_f32(client.read(out)), oracle.attention(qr, kr, v, SCALE, causal=True, query_start=qs))


def test_config3_shape_rows_sample(client, oracle):
    # Full configuration-3 size; the oracle checks the first 16 query rows of every head plus the last tile of one head.
    b, h, s = 4, 32, 2048
    q, k, v = rand_qkv(3, b, h, h, s, s)
    out = RT.attention(client, up16(client, q), up16(client, k), up16(client, v), SCALE, causal=True, bmhd_output=True)
    got = bf16_bits_to_f32(client.read(out)).transpose(0, 2, 1, 3)
    want = oracle.attention(q, k, v, SCALE, causal=True, rows_limit=16)
    check_bf16(got[:, :, :16], want[:, :, :16])
    tail = oracle.attention(q[1:2, 5:6, -128:], k[1:2, 5:6], v[1:2, 5:6], SCALE, causal=True, query_start=s - 128)
    check_bf16(got[1:2, 5:6, -128:], tail)
    # size-independent property: a causal row only depends on the keys before it -> output of row 0 equals V row 0
    np.testing.assert_allclose(got[:, :, 0], v[:, :, 0], atol=1e-2)


def test_general_kernel_matches_tensor_core_kernel(client):
    q, k, v = rand_qkv(11, 1, 2, 1, 128, 256)
    fast = bf16_bits_to_f32(client.read(RT.attention(client, up16(client, q), up16(client, k), up16(client, v), SCALE, causal=True, query_start=128)))
    mask = client.upload(np.zeros((1, 2, 128, 256), np.float32))
    slow = bf16_bits_to_f32(client.read(RT.attention(client, up16(client, q), up16(client, k), up16(client, v), SCALE, mask=mask, causal=True, query_start=128)))
    check_bf16(fast, slow)


def test_config4_as_stated_rows_sample(client, oracle):
    """BASELINE configuration 4 as stated: RMSNorm over hidden [2,4096,4096] (w ~ U(0.5,1.5), eps 1e-6) in front, then causal
    grouped-query attention B2, 32 query / 8 KV heads, S 4096, D 128 with RoPE (SplitHalf, theta 1e4) applied to Q and K inside
    the attention call.  The norm is checked on a row sample to 1e-5; the attention output on sampled heads: the first rows,
    rows around a 256-row block boundary and the last rows, against the oracle with the same BF16 rounding of the rotated Q, K."""
    b, hq, hkv, s = 2, 32, 8, 4096
    rng = np.random.default_rng(4)
    hidden = rng.standard_normal((b * s, 4096), dtype=np.float32)
    w = np.random.default_rng(4001).uniform(0.5, 1.5, 4096).astype(np.float32)
    y, _ = RT.rms_norm(client, client.upload(hidden), client.upload(w), 1e-6)
    rows = np.random.default_rng(7).integers(0, b * s, 64)
    want_y, _ = oracle.rms_norm(hidden[rows], w, 1e-6)
    np.testing.assert_allclose(client.read(y)[rows], want_y, rtol=1e-5, atol=1e-7)
    client.free(y.handle)
    q, k, v = rand_qkv(4002, b, hq, hkv, s, s)
    pos = np.arange(s, dtype=np.float64)[:, None]
    inv = 10000.0 ** (-np.arange(64, dtype=np.float64) * 2 / 128)
    cos, sin = np.cos(pos * inv).astype(np.float32), np.sin(pos * inv).astype(np.float32)
    out = RT.attention(client, up16(client, q), up16(client, k), up16(client, v), SCALE, causal=True, cos=client.upload(cos), sin=client.upload(sin),
                       rotary_layout=RotaryLayout.SplitHalf)
    got = bf16_bits_to_f32(client.read(out))
    assert np.all(np.isfinite(got))
    for bi, h in ((0, 0), (1, 13), (1, 31)):
        kvh = h // (hq // hkv)
        tk = np.broadcast_to(cos, (1, 1, s, 64)), np.broadcast_to(sin, (1, 1, s, 64))
        kr = oracle.bf16(oracle.rotary(k[bi:bi + 1, kvh:kvh + 1], tk[0], tk[1], "split_half"))
        for r0, r1 in ((0, 32), (240, 272), (s - 32, s)):
            tq = np.broadcast_to(cos[r0:r1], (1, 1, r1 - r0, 64)), np.broadcast_to(sin[r0:r1], (1, 1, r1 - r0, 64))
            qr = oracle.bf16(oracle.rotary(q[bi:bi + 1, h:h + 1, r0:r1], tq[0], tq[1], "split_half"))
            want = oracle.attention(qr, kr, v[bi:bi + 1, kvh:kvh + 1], SCALE, causal=True, query_start=r0)
            check_bf16(got[bi:bi + 1, h:h + 1, r0:r1], want)


# ---- the reference's own contract (FP32 tensors) on the tensor-core kernel ---------------------------------------
def test_fp32_contract_at_head_dim_128_runs_on_the_tensor_core_kernel(client, oracle):
    """nn.causal_grouped_query_attention_bf16_fp32 (src/nn/attention.rs:69-80) takes FP32 Q/K/V; at head dim 128 the call must
    reach the tcgen05 kernel (launch counter), and its FP32 output must meet the BF16 tolerance against the oracle, which rounds
    the operands and P to BF16 where the reference does."""
    rng = np.random.default_rng(21)
    b, hq, hkv, m, n = 2, 8, 2, 384, 512
    q = rng.standard_normal((b, hq, m, 128), dtype=np.float32); k = rng.standard_normal((b, hkv, n, 128), dtype=np.float32)
    v = rng.standard_normal((b, hkv, n, 128), dtype=np.float32)
    T = lambda a: nn.Tensor.from_data(client, a)
    before = RT.attention_launch_counts(client)
    out = nn.causal_grouped_query_attention_bf16_fp32(T(q), T(k), T(v), float(SCALE), n - m, 0)
    after = RT.attention_launch_counts(client)
    assert after["tensor_core"] == before["tensor_core"] + 1 and after["general"] == before["general"]
    assert out.dtype() == DType.F32 and out.dims() == [b, hq, m, 128]
    check_bf16(out.into_data(), oracle.attention(q, k, v, SCALE, causal=True, query_start=n - m))
    # the plain and the grouped non-causal entry points take the same route
    out2 = nn.grouped_query_attention_bf16_fp32(T(q), T(k), T(v), float(SCALE), None)
    assert RT.attention_launch_counts(client)["tensor_core"] == after["tensor_core"] + 1
    check_bf16(out2.into_data(), oracle.attention(q, k, v, SCALE))


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_additive_mask_tiles_on_the_tensor_core_kernel(client, oracle, dtype):
    """An additive FP32 mask [B,Hq,M,N] (src/nn/attention.rs:10-29) joins the scores inside the tensor-core kernel: finite
    biases, -inf entries, a key block cut by the end of the keys, and one row whose keys are all excluded (no value: NaN, as
    the reference's softmax of a row of -inf gives)."""
    rng = np.random.default_rng(22)
    b, hq, hkv, m, n = 1, 4, 2, 272, 416
    q, k, v = rand_qkv(23, b, hq, hkv, m, n)
    mask = rng.standard_normal((b, hq, m, n)).astype(np.float32)
    mask[rng.random(mask.shape) < 0.3] = -np.inf
    mask[0, 1, 5, :] = -np.inf                                   # a row without any visible key
    mask[0, 2, 100, :300] = -np.inf                              # whole key blocks hidden, the tail visible
    before = RT.attention_launch_counts(client)["tensor_core"]
    if dtype == "bf16":
        out = RT.attention(client, up16(client, q), up16(client, k), up16(client, v), SCALE, mask=client.upload(mask))
        got = bf16_bits_to_f32(client.read(out))
    else:
        out = RT.attention(client, client.upload(q), client.upload(k), client.upload(v), SCALE, mask=client.upload(mask))
        got = client.read(out)
    assert RT.attention_launch_counts(client)["tensor_core"] == before + 1
    want = oracle.attention(q, k, v, SCALE, mask=mask)
    assert np.isnan(got[0, 1, 5]).all() and np.isnan(want[0, 1, 5]).all()
    keep = np.ones((b, hq, m), bool); keep[0, 1, 5] = False
    check_bf16(got[keep], want[keep])


def test_rows_without_visible_keys_have_no_value(client, oracle):
    """Causal attention whose first queries lie before every key (key_start > query_start + row): the reference's mask is -inf
    over the whole row and its softmax gives NaN; the tensor-core kernel and the oracle agree with that, tile by tile and row by row."""
    q, k, v = rand_qkv(31, 1, 2, 2, 384, 256)
    out = RT.attention(client, up16(client, q), up16(client, k), up16(client, v), SCALE, causal=True, query_start=0, key_start=200)
    got = bf16_bits_to_f32(client.read(out))
    want = oracle.attention(q, k, v, SCALE, causal=True, query_start=0, key_start=200)
    assert np.isnan(got[:, :, :200]).all() and np.isnan(want[:, :, :200]).all()      # rows 0..199 see no key (a whole tile and part of the next)
    check_bf16(got[:, :, 200:], want[:, :, 200:])


def test_fp32_contract_with_fused_rotary(client, oracle):
    b, hq, hkv, m, n = 1, 4, 2, 256, 256
    rng = np.random.default_rng(41)
    q = rng.standard_normal((b, hq, m, 128), dtype=np.float32); k = rng.standard_normal((b, hkv, n, 128), dtype=np.float32)
    v = rng.standard_normal((b, hkv, n, 128), dtype=np.float32)
    pos = np.arange(n, dtype=np.float64)[:, None]
    inv = 10000.0 ** (-np.arange(64, dtype=np.float64) * 2 / 128)
    cos, sin = np.cos(pos * inv).astype(np.float32), np.sin(pos * inv).astype(np.float32)
    out = RT.attention(client, client.upload(q), client.upload(k), client.upload(v), SCALE, causal=True, cos=client.upload(cos), sin=client.upload(sin),
                       rotary_layout=RotaryLayout.SplitHalf)
    tq = np.broadcast_to(cos[:m], (b, hq, m, 64)), np.broadcast_to(sin[:m], (b, hq, m, 64))
    tk = np.broadcast_to(cos[:n], (b, hkv, n, 64)), np.broadcast_to(sin[:n], (b, hkv, n, 64))
    qr = oracle.bf16(oracle.rotary(oracle.bf16(q), tq[0], tq[1], "split_half")); kr = oracle.bf16(oracle.rotary(oracle.bf16(k), tk[0], tk[1], "split_half"))
    check_bf16(client.read(out), oracle.attention(qr, kr, v, SCALE, causal=True))


def test_more_steps_per_cta_than_the_item_table_holds(client, oracle):
    """With one SM a single CTA walks every work item: 600 (batch, head) pairs of one 256-row item each are more steps than
    the 512 the kernel tabulates in shared memory, so the last ones are computed by the late-item function.  The result must
    be the one the whole GPU computes (same bits: an item's arithmetic does not depend on which CTA runs it) and match the
    oracle on sampled heads."""
    import ctypes as C
    from rust_ascend_b200.runtime import _check
    rng = np.random.default_rng(23)
    b, h, s = 6, 100, 256
    q, k, v = (r16(rng.standard_normal((b, h, s, 128), dtype=np.float32)) for _ in range(3))
    dq, dk, dv = up16(client, q), up16(client, k), up16(client, v)
    whole = bf16_bits_to_f32(client.read(RT.attention(client, dq, dk, dv, 128 ** -0.5, causal=True)))
    _check(client._lib.rb_set_sm_limit(client._ctx, C.c_int32(1)))
    try:
        one = bf16_bits_to_f32(client.read(RT.attention(client, dq, dk, dv, 128 ** -0.5, causal=True)))
    finally:
        _check(client._lib.rb_set_sm_limit(client._ctx, C.c_int32(0)))
    np.testing.assert_array_equal(one, whole)
    for bi, hi in ((0, 0), (5, 99), (3, 57)):          # (5, 99) is among the last items in any order
        want = oracle.attention(q[bi:bi + 1, hi:hi + 1], k[bi:bi + 1, hi:hi + 1], v[bi:bi + 1, hi:hi + 1], 128 ** -0.5, causal=True)
        check_bf16(one[bi:bi + 1, hi:hi + 1], want)
