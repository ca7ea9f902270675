"""Size-independent properties of the oracle (CPU): identities the domain offers, checked on seeded inputs, so that the
checker itself is checked by something other than the reference's worked examples."""
import numpy as np
import pytest


@pytest.fixture(scope="module")
def rng():
    return np.random.default_rng(2024)


@pytest.mark.parametrize("rows,width", [(5, 33), (3, 4096), (2, 8225)])
def test_softmax_rows_sum_to_one_and_log_softmax_is_its_logarithm(oracle, rng, rows, width):
    x = (rng.standard_normal((rows, width)) * 4).astype(np.float32)
    p = oracle.softmax(x)
    assert np.all(p >= 0) and np.abs(p.sum(-1, dtype=np.float64) - 1).max() < 1e-5
    np.testing.assert_allclose(oracle.softmax(x, log=True), np.log(np.maximum(p.astype(np.float64), 1e-300)), atol=2e-5, rtol=1e-5)
    shifted = oracle.softmax(x + np.float32(3.0))                    # invariant under a common shift of the scores
    np.testing.assert_allclose(shifted, p, atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("width", [32, 96, 4096])
def test_rms_norm_is_scale_invariant_and_unit_rms(oracle, rng, width):
    x = rng.standard_normal((7, width)).astype(np.float32); w = np.ones(width, np.float32)
    y, rstd = oracle.rms_norm(x, w, 1e-12)
    np.testing.assert_allclose(np.sqrt((y.astype(np.float64) ** 2).mean(-1)), 1.0, atol=1e-5)
    y4, rstd4 = oracle.rms_norm(x * np.float32(4.0), w, 1e-12)       # a power of two scales exactly
    np.testing.assert_allclose(y4, y, atol=1e-6, rtol=1e-6)
    np.testing.assert_allclose(rstd4 * 4, rstd, rtol=1e-6)


@pytest.mark.parametrize("layout", ["interleaved", "split_half"])
def test_rotary_is_a_rotation_and_its_backward_is_the_inverse(oracle, rng, layout):
    shape, half = (2, 3, 17, 64), 32
    x = rng.standard_normal(shape).astype(np.float32)
    angle = rng.uniform(0, 6.28, size=shape[:-1] + (half,))
    cos, sin = np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)
    y = oracle.rotary(x, cos, sin, layout)
    np.testing.assert_allclose((y.astype(np.float64) ** 2).sum(-1), (x.astype(np.float64) ** 2).sum(-1), rtol=1e-5)   # norms survive
    back = oracle.rotary(y, cos, sin, layout, backward=True)           # transpose of a rotation = its inverse
    np.testing.assert_allclose(back, x, atol=2e-6, rtol=2e-6)


def test_gemm_is_linear_on_exactly_representable_data(oracle, rng):
    a1 = rng.integers(-8, 9, size=(48, 64)).astype(np.float32); a2 = rng.integers(-8, 9, size=(48, 64)).astype(np.float32)
    b = rng.integers(-8, 9, size=(32, 64)).astype(np.float32)
    whole = oracle.gemm_bf16(a1 + a2, b, False, True, False)
    np.testing.assert_array_equal(whole, oracle.gemm_bf16(a1, b, False, True, False) + oracle.gemm_bf16(a2, b, False, True, False))
    np.testing.assert_array_equal(oracle.gemm_bf16(b, a1, False, True, False), oracle.gemm_bf16(a1, b, False, True, False).T)


def test_attention_rows_are_convex_combinations_and_causal_row_zero_is_the_first_value(oracle, rng):
    q = rng.standard_normal((2, 4, 32, 32)).astype(np.float32); k = rng.standard_normal((2, 2, 64, 32)).astype(np.float32)
    v = rng.standard_normal((2, 2, 64, 16)).astype(np.float32)
    o = oracle.attention(q, k, v, 32 ** -0.5)
    vb = oracle.bf16(v)
    lo, hi = np.repeat(vb.min(2, keepdims=True), 2, axis=1), np.repeat(vb.max(2, keepdims=True), 2, axis=1)
    assert np.all(o >= lo - 2e-2) and np.all(o <= hi + 2e-2)           # inside the hull of the values (BF16 rounding of P)
    causal = oracle.attention(q, k[:, :, :32], v[:, :, :32], 32 ** -0.5, causal=True)
    np.testing.assert_allclose(causal[:, :, 0], np.repeat(vb[:, :, 0], 2, axis=1), atol=1e-6)   # query 0 sees key 0 only
    one_key = oracle.attention(q, k[:, :, :32] * 0, v[:, :, :32], 1.0)
    np.testing.assert_allclose(one_key, np.repeat(vb[:, :, :32].mean(2, keepdims=True), 2, axis=1) * np.ones((1, 1, 32, 1)), atol=2e-2)  # equal scores: the mean


def test_embedding_gradient_conserves_the_upstream_sum(oracle, rng):
    ids = rng.integers(0, 50, size=(4, 37)); grad = rng.standard_normal((4, 37, 24)).astype(np.float32)
    dw = oracle.embedding_backward(grad, ids, 50)
    np.testing.assert_allclose(dw.sum(0, dtype=np.float64), grad.reshape(-1, 24).sum(0, dtype=np.float64), atol=1e-4)
    untouched = np.setdiff1d(np.arange(50), ids)
    assert not dw[untouched].any()
    padded = oracle.embedding_backward(grad, ids, 50, padding_idx=int(ids[0, 0]))
    assert not padded[int(ids[0, 0])].any()


def test_cross_entropy_gradient_rows_sum_to_zero_and_loss_is_positive(oracle, rng):
    logits = (rng.standard_normal((3, 9, 101)) * 2).astype(np.float32); labels = rng.integers(0, 101, size=(3, 9))
    labels[1, 4] = -100
    loss, valid, d = oracle.causal_cross_entropy(logits, labels, -100, True, 1.0)
    assert loss > 0 and valid == 3 * 8 - 1
    assert np.abs(d.sum(-1, dtype=np.float64)).max() < 1e-6            # softmax minus one-hot sums to zero on every scored row
    assert not d[:, -1].any() and not d[1, 3].any()                     # last position and the ignored pair get no gradient
    uniform = np.zeros((1, 2, 64), np.float32)
    loss_u, valid_u, _ = oracle.causal_cross_entropy(uniform, np.array([[3, 5]]), -100, False, 1.0)
    np.testing.assert_allclose(loss_u, valid_u * np.log(64.0), rtol=1e-6)
