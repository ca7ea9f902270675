"""GPU parity (through the C ABI): tcgen05 BF16 GEMM against the CPU oracle and the reference's GEMM vectors.
Tolerance (BF16 path): max abs error <= 2e-2 and mean relative error <= 1e-2 against the FP32-accumulated
oracle; the reference's own small vectors are held to their stated tolerances."""
import numpy as np
import pytest

import vectors as V
from rust_ascend_b200 import B200Runtime as RT
from rust_ascend_b200 import DType, InvalidTensor, Transpose
from rust_ascend_b200.runtime import bf16_bits_to_f32, f32_to_bf16_bits

pytestmark = pytest.mark.gpu
T = {False: Transpose.No, True: Transpose.Yes}


def up16(client, x):
    return client.upload(f32_to_bf16_bits(x))


def read(client, t):
    a = client.read(t)
    return bf16_bits_to_f32(a) if t.dtype == DType.BF16 else a


def bf16_tolerance(got, want):
    got = got.astype(np.float64); want = want.astype(np.float64)
    assert np.all(np.isfinite(got))
    err = np.abs(got - want)
    # 2e-2 absolute covers half a BF16 ulp up to |y| < 8; beyond that the bound is half an ulp, 2^-8 relative.
    assert err.max() <= max(2e-2, 2.0 ** -8 * np.abs(want).max()), f"max abs {err.max()}"
    assert (err.sum() / max(np.abs(want).sum(), 1e-30)) <= 1e-2


@pytest.mark.parametrize("ta", [False, True])
@pytest.mark.parametrize("tb", [False, True])
@pytest.mark.parametrize("out_bf16", [False, True])
@pytest.mark.parametrize("batches,m,n,k", [(1, 80, 96, 144), (3, 16, 32, 16)])
def test_reference_kernel_vectors(client, oracle, ta, tb, out_bf16, batches, m, n, k):
    # rust-ascend-kernels/src/tests.rs:89-132, tolerance 1e-4.
    a, b, d = V.gemm_kernel_case(batches, m, n, k, ta, tb)
    if batches == 1:
        a, b, d = a[0], b[0], d[0]
    out = RT.gemm(client, up16(client, a), up16(client, b), T[ta], T[tb], DType.BF16 if out_bf16 else DType.F32)
    got = read(client, out)
    want = oracle.gemm_bf16(a, b, ta, tb, out_bf16)
    assert np.abs(got.astype(np.float64) - want).max() < 1e-4
    assert np.abs(got.astype(np.float64) - (V.bf16_f64(d.astype(np.float32)) if out_bf16 else d)).max() < 1e-4


@pytest.mark.parametrize("batches", [1, 2])
@pytest.mark.parametrize("ta", [False, True])
@pytest.mark.parametrize("tb", [False, True])
@pytest.mark.parametrize("dtype", [DType.BF16, DType.F32])
def test_reference_runtime_vectors_and_reuse(client, batches, ta, tb, dtype):
    # examples/matrix_runtime.rs:50-77: gemm, then gemm_into the same output.
    a, b, d = V.gemm_runtime_case(batches, ta, tb)
    if batches == 1:
        a, b, d = a[0], b[0], d[0]
    da, db = up16(client, a), up16(client, b)
    out = RT.gemm(client, da, db, T[ta], T[tb], dtype)
    assert out.shape == d.shape
    rel = 4e-3 if dtype == DType.BF16 else 5e-4
    assert np.all(np.abs(read(client, out) - d) <= 5e-4 + rel * np.abs(d))
    client.memset(out, 0xFF)
    RT.gemm_into(client, da, db, T[ta], T[tb], out)
    assert np.all(np.abs(read(client, out) - d) <= 5e-4 + rel * np.abs(d))


@pytest.mark.parametrize("m,n,k", [(16, 32, 16), (32, 48, 32)])
def test_linear_bf16_fp32_contract(client, m, n, k):
    # examples/linear_tensor.rs:24-50: FP32 in, FP32 out, BF16 snapshots returned.
    x, w, y = V.linear_case(m, n, k)
    out, x16, w16 = RT.linear_bf16_fp32(client, client.upload(x), client.upload(w))
    assert out.dtype == DType.F32 and out.shape == (m, n) and x16.dtype == DType.BF16 and w16.shape == (n, k)
    assert np.all(np.abs(client.read(out) - y) <= 5e-4 + 5e-4 * np.abs(y))
    np.testing.assert_array_equal(client.read(x16), f32_to_bf16_bits(x))
    frozen = RT.linear_frozen_bf16_fp32(client, client.upload(x), up16(client, w))
    np.testing.assert_array_equal(client.read(frozen), client.read(out))


@pytest.mark.parametrize("m,n,k,seed", [(128, 256, 64, 0), (256, 512, 512, 1), (384, 1024, 1040, 2), (1024, 4096, 4096, 3),
                                        (144, 272, 208, 4), (2048, 176, 96, 5), (16, 16, 16, 6), (4096, 64, 4096, 7)])
def test_linear_random_against_oracle(client, oracle, m, n, k, seed):
    rng = np.random.default_rng(seed)
    x = bf16_bits_to_f32(f32_to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32)))
    w = bf16_bits_to_f32(f32_to_bf16_bits(rng.standard_normal((n, k), dtype=np.float32) * 0.02))
    got32 = read(client, RT.gemm(client, up16(client, x), up16(client, w), Transpose.No, Transpose.Yes, DType.F32))
    want = oracle.linear(x, w)
    assert np.abs(got32 - want).max() <= 1e-4 * max(1.0, np.abs(want).max())  # FP32 accumulate, order only
    got16 = read(client, RT.gemm(client, up16(client, x), up16(client, w), Transpose.No, Transpose.Yes, DType.BF16))
    bf16_tolerance(got16, want)


def test_batched_random(client, oracle):
    rng = np.random.default_rng(21)
    a = bf16_bits_to_f32(f32_to_bf16_bits(rng.standard_normal((5, 272, 192), dtype=np.float32)))
    b = bf16_bits_to_f32(f32_to_bf16_bits(rng.standard_normal((5, 192, 144), dtype=np.float32)))
    got = read(client, RT.gemm(client, up16(client, a), up16(client, b), Transpose.No, Transpose.No, DType.F32))
    assert np.abs(got - oracle.gemm_bf16(a, b, False, False, False)).max() <= 2e-4


@pytest.mark.parametrize("bias_dtype", [DType.F32, DType.BF16])
def test_bias_epilogue(client, oracle, bias_dtype):
    rng = np.random.default_rng(8)
    m, n, k = 272, 528, 320
    x = bf16_bits_to_f32(f32_to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32)))
    w = bf16_bits_to_f32(f32_to_bf16_bits(rng.standard_normal((n, k), dtype=np.float32) * 0.02))
    bias = (rng.standard_normal(n) * 0.02).astype(np.float32)
    if bias_dtype == DType.BF16:
        bias = bf16_bits_to_f32(f32_to_bf16_bits(bias)); tb = up16(client, bias)
    else:
        tb = client.upload(bias)
    got = read(client, RT.gemm(client, up16(client, x), up16(client, w), Transpose.No, Transpose.Yes, DType.F32, bias=tb))
    assert np.abs(got - oracle.linear(x, w, bias=bias)).max() <= 1e-4
    got16 = read(client, RT.gemm(client, up16(client, x), up16(client, w), Transpose.No, Transpose.Yes, DType.BF16, bias=tb))
    bf16_tolerance(got16, oracle.linear(x, w, bias=bias))


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (272, 528, 320), (512, 11008 // 8, 1024), (16, 16, 16)])
def test_swiglu_epilogue(client, oracle, m, n, k):
    rng = np.random.default_rng(m + n)
    x = bf16_bits_to_f32(f32_to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32)))
    wg = bf16_bits_to_f32(f32_to_bf16_bits(rng.standard_normal((n, k), dtype=np.float32) * 0.05))
    wu = bf16_bits_to_f32(f32_to_bf16_bits(rng.standard_normal((n, k), dtype=np.float32) * 0.05))
    got = read(client, RT.gemm(client, up16(client, x), up16(client, wg), Transpose.No, Transpose.Yes, DType.F32, b_up=up16(client, wu)))
    want = oracle.linear(x, wg, w_up=wu)
    assert np.abs(got - want).max() <= 2e-4 * max(1.0, np.abs(want).max())
    got16 = read(client, RT.gemm(client, up16(client, x), up16(client, wg), Transpose.No, Transpose.Yes, DType.BF16, b_up=up16(client, wu)))
    bf16_tolerance(got16, want)


def test_swiglu_zero_gate_gives_zero(client):
    # examples/swiglu_tensor.rs:22-40.
    width = 16
    x = (((np.arange(width * width) % 7).astype(np.float32) - 3.0) * 0.125).reshape(width, width)
    up = np.eye(width, dtype=np.float32) * 0.5
    got = read(client, RT.gemm(client, up16(client, x), up16(client, np.zeros((width, width), np.float32)), Transpose.No, Transpose.Yes,
                               DType.F32, b_up=up16(client, up)))
    np.testing.assert_array_equal(got, np.zeros((width, width), np.float32))


def test_full_size_linearity_property(client):
    # Config-2 size: (X1+X2) W^T == X1 W^T + X2 W^T when the sums are exact in BF16 (small integers).
    rng = np.random.default_rng(2)
    m = n = k = 4096
    x1 = rng.integers(-4, 5, size=(m, k)).astype(np.float32); x2 = rng.integers(-4, 5, size=(m, k)).astype(np.float32)
    w = rng.integers(-2, 3, size=(n, k)).astype(np.float32)
    tw = up16(client, w)
    y1 = client.read(RT.gemm(client, up16(client, x1), tw, Transpose.No, Transpose.Yes, DType.F32))
    y2 = client.read(RT.gemm(client, up16(client, x2), tw, Transpose.No, Transpose.Yes, DType.F32))
    y12 = client.read(RT.gemm(client, up16(client, x1 + x2), tw, Transpose.No, Transpose.Yes, DType.F32))
    np.testing.assert_array_equal(y12, y1 + y2)  # all values are integers below 2^24: exact in FP32
    rows = rng.integers(0, m, 8)
    np.testing.assert_array_equal(y1[rows], x1[rows].astype(np.float64) @ w.astype(np.float64).T)


def test_domain_errors(client):
    a = up16(client, np.zeros((32, 48), np.float32)); b = up16(client, np.zeros((64, 48), np.float32))
    with pytest.raises(InvalidTensor, match="multiples of 16"):
        RT.gemm(client, up16(client, np.zeros((24, 48), np.float32)), b, Transpose.No, Transpose.Yes, DType.F32)
    with pytest.raises(InvalidTensor, match="agree"):
        RT.gemm(client, a, b, Transpose.No, Transpose.No, DType.F32)
    with pytest.raises(InvalidTensor, match="BF16 operands"):
        RT.gemm(client, client.upload(np.zeros((32, 48), np.float32)), b, Transpose.No, Transpose.Yes, DType.F32)
    out = client.tensor((32, 64), DType.F32)
    alias = type(out)(a.handle, (32, 24), DType.F32)
    with pytest.raises(InvalidTensor):
        RT.gemm_into(client, a, b, Transpose.No, Transpose.Yes, alias)
    with pytest.raises(InvalidTensor, match="FP32 inputs"):
        RT.gemm_bf16_fp32(client, a, b, Transpose.No, Transpose.Yes)


def _normal_bf16(seed, shape, std=1.0):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(shape, dtype=np.float32)
    if std != 1.0:
        x *= np.float32(std)
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


def test_config2a_full_size_on_single_ctas(client, oracle, single_ctas):
    """The same configuration on the single-CTA kernel (512 tiles on 148 CTAs: three rounds of whole tiles and a last round of 136 half tiles)."""
    test_config2a_full_size_against_oracle_rows(client, oracle)


def test_config2a_full_size_against_oracle_rows(client, oracle):
    """BASELINE configuration 2a as stated: X [4096,4096] ~ N(0,1), W [4096,4096] ~ N(0,0.02) stored [N,K], FP32 bias
    ~ N(0,0.02), BF16 output.  The whole output is computed on the GPU; the oracle recomputes 48 sampled rows."""
    m = n = k = 4096
    x, w = _normal_bf16(2, (m, k)), _normal_bf16(2001, (n, k), 0.02)
    bias = (np.random.default_rng(2002).standard_normal(n) * 0.02).astype(np.float32)
    out = RT.gemm(client, up16(client, x), up16(client, w), Transpose.No, Transpose.Yes, DType.BF16, bias=client.upload(bias))
    got = read(client, out)
    rows = np.unique(np.concatenate([[0, 127, 128, m - 1], np.random.default_rng(5).integers(0, m, 44)]))
    bf16_tolerance(got[rows], oracle.linear(x[rows], w, bias=bias))
    assert np.all(np.isfinite(got))


def test_config2b_full_size_swiglu_against_oracle_rows(client, oracle):
    """BASELINE configuration 2b: X [8192,4096], gate and up weights [11008,4096], output bf16(silu(g) * u) [8192,11008]
    from one launch.  The oracle recomputes 24 sampled rows (first/last rows of the first and last row tiles included)."""
    m, n, k = 8192, 11008, 4096
    x = _normal_bf16(2, (m, k))
    wg, wu = _normal_bf16(2003, (n, k), 0.02), _normal_bf16(2004, (n, k), 0.02)
    out = RT.gemm(client, up16(client, x), up16(client, wg), Transpose.No, Transpose.Yes, DType.BF16, b_up=up16(client, wu))
    got = read(client, out)
    rows = np.unique(np.concatenate([[0, 127, m - 128, m - 1], np.random.default_rng(6).integers(0, m, 20)]))
    bf16_tolerance(got[rows], oracle.linear(x[rows], wg, w_up=wu))
    assert np.all(np.isfinite(got))
    client.free(out.handle)


@pytest.mark.parametrize("m,n,k,mode", [(19200, 256, 64, "bias"), (19200, 272, 80, "none"), (19200, 128, 64, "swiglu"), (9600, 400, 48, "swiglu"),
                                        (128, 256, 128, "bias"), (2048, 4096 + 512, 64, "none")])
def test_tail_round_of_half_tiles(client, oracle, single_ctas, m, n, k, mode):
    """Shapes whose last round of the persistent loop is cut into half-width tiles (150 or 300 tiles on 148 SMs, a single tile, and
    a grid with a ragged last column of tiles), with every epilogue: all rows against the oracle."""
    rng = np.random.default_rng(m + n + k)
    x = _normal_bf16(rng.integers(1 << 30), (m, k))
    w = _normal_bf16(rng.integers(1 << 30), (n, k), 0.1)
    if mode == "swiglu":
        wu = _normal_bf16(rng.integers(1 << 30), (n, k), 0.1)
        got = read(client, RT.gemm(client, up16(client, x), up16(client, w), Transpose.No, Transpose.Yes, DType.F32, b_up=up16(client, wu)))
        want = oracle.linear(x, w, w_up=wu)
    elif mode == "bias":
        bias = rng.standard_normal(n).astype(np.float32)
        got = read(client, RT.gemm(client, up16(client, x), up16(client, w), Transpose.No, Transpose.Yes, DType.F32, bias=client.upload(bias)))
        want = oracle.linear(x, w, bias=bias)
    else:
        got = read(client, RT.gemm(client, up16(client, x), up16(client, w), Transpose.No, Transpose.Yes, DType.F32))
        want = oracle.linear(x, w)
    assert np.abs(got - want).max() <= 2e-4 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("m,n,k,chunks,out", [(2048, 768, 512, 8, DType.BF16), (400, 272, 144, 3, DType.F32), (128, 128, 64, 8, DType.BF16)])
def test_linear_on_host_buffers_matches_write_gemm_read(client, oracle, m, n, k, chunks, out):
    """The pipelined host-buffer call gives the bits of rb_write + rb_gemm + rb_read, and meets the oracle."""
    rng = np.random.default_rng(m + chunks)
    x = f32_to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32)); w = f32_to_bf16_bits(rng.standard_normal((n, k), dtype=np.float32) * 0.05)
    bias = rng.standard_normal(n).astype(np.float32)
    hx = client.pinned((m, k), np.uint16); hx[...] = x
    hy = client.pinned((m, n), np.uint16 if out == DType.BF16 else np.float32); hy[...] = 0
    tx, tw, tb, ty = client.tensor((m, k), DType.BF16), client.upload(w), client.upload(bias), client.tensor((m, n), out)
    RT.linear_host(client, hx, tx, tw, ty, hy, bias=tb, row_chunks=chunks)
    want = client.read(RT.gemm(client, client.upload(x), tw, Transpose.No, Transpose.Yes, out, bias=tb))
    np.testing.assert_array_equal(np.array(hy), want)
    got = bf16_bits_to_f32(np.array(hy)) if out == DType.BF16 else np.array(hy)
    ref = oracle.linear(bf16_bits_to_f32(x), bf16_bits_to_f32(w), bias=bias)
    if out == DType.BF16:
        bf16_tolerance(got, ref)
    else:
        assert np.abs(got - ref).max() <= 1e-4 * max(1.0, np.abs(ref).max())


def _with_pairs(value):
    import os
    before = os.environ.get("RUDA_GEMM_PAIRS")
    os.environ["RUDA_GEMM_PAIRS"] = value
    yield
    if before is None:
        del os.environ["RUDA_GEMM_PAIRS"]
    else:
        os.environ["RUDA_GEMM_PAIRS"] = before


@pytest.fixture
def cta_pairs():
    """Wide GEMMs run on pairs of CTAs (clusters of two); this is the default, stated here so that the test says what it covers."""
    yield from _with_pairs("1")


@pytest.fixture
def single_ctas():
    """Keeps every GEMM of the test on the single-CTA kernel, which otherwise only narrow or short shapes reach."""
    yield from _with_pairs("0")


@pytest.mark.parametrize("batches,m,n,k,mode", [(1, 512, 512, 256, "none"), (1, 4096, 1024, 512, "bias"), (1, 1024, 1376, 512, "swiglu"), (1, 400, 272, 144, "bias"),
                                                (1, 19200, 256, 64, "none"), (1, 19200, 128, 64, "swiglu"), (2, 768, 512, 192, "none"), (1, 256, 256, 4096, "none")])
def test_cta_pair_kernel_against_oracle(client, oracle, cta_pairs, batches, m, n, k, mode):
    """The 256-row tiles of the CTA-pair kernel: whole and half-width tiles (75 tiles on 74 pairs), ragged last tiles in both
    directions, every epilogue, batches, a long K: all rows against the oracle, FP32 and BF16 outputs."""
    rng = np.random.default_rng(batches + m + n + k)
    shape = lambda *s: ((batches,) + s) if batches > 1 else s
    x = _normal_bf16(rng.integers(1 << 30), shape(m, k)); w = _normal_bf16(rng.integers(1 << 30), shape(n, k), 0.1)
    flat = lambda a: a.reshape(-1, a.shape[-2], a.shape[-1])
    kwargs, want = {}, None
    if mode == "swiglu":
        wu = _normal_bf16(rng.integers(1 << 30), shape(n, k), 0.1)
        kwargs["b_up"] = up16(client, wu)
        want = np.stack([oracle.linear(a, b, w_up=u) for a, b, u in zip(flat(x), flat(w), flat(wu))])
    elif mode == "bias":
        bias = rng.standard_normal(n).astype(np.float32)
        kwargs["bias"] = client.upload(bias)
        want = np.stack([oracle.linear(a, b, bias=bias) for a, b in zip(flat(x), flat(w))])
    else:
        want = np.stack([oracle.linear(a, b) for a, b in zip(flat(x), flat(w))])
    want = want.reshape(shape(m, n))
    got = read(client, RT.gemm(client, up16(client, x), up16(client, w), Transpose.No, Transpose.Yes, DType.F32, **kwargs))
    assert np.abs(got - want).max() <= 2e-4 * max(1.0, np.abs(want).max())
    got16 = read(client, RT.gemm(client, up16(client, x), up16(client, w), Transpose.No, Transpose.Yes, DType.BF16, **kwargs))
    bf16_tolerance(got16, want)
