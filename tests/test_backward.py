"""First-order backward programs: the oracle against the reference's f64 expectations (CPU), and the CUDA
kernels against the oracle through the C ABI (GPU).  Tolerances are the reference examples' (5e-4 absolute and
relative for norms and matrices, 2e-5 + 1e-4 relative for softmax and SiLU*up)."""
import numpy as np
import pytest

import vectors as V


def close(actual, expected, atol, rtol):
    actual = np.asarray(actual, dtype=np.float64); expected = np.asarray(expected, dtype=np.float64)
    assert actual.shape == expected.shape and np.all(np.isfinite(actual))
    err = np.abs(actual - expected) - (atol + rtol * np.abs(expected))
    assert err.size == 0 or err.max() <= 0, f"max excess {err.max()}"


SHAPES = [(0, 32), (1, 32), (3, 96), (7, 256), (33, 4096), (3, 33), (300, 1000)]


@pytest.mark.parametrize("rows,width", SHAPES)
def test_oracle_rms_norm_backward(oracle, rows, width):
    x, w, dy, r, dx, dw = V.rms_backward_case(rows, width)
    gdx, gdw = oracle.rms_norm_backward(x, w, dy, r)
    close(gdx, dx, 1e-5, 1e-5); close(gdw, dw, 1e-4, 1e-5)


@pytest.mark.parametrize("rows,width", SHAPES)
@pytest.mark.parametrize("log", [False, True])
def test_oracle_softmax_backward(oracle, rows, width, log):
    y, dy, dx = V.softmax_backward_case(rows, width, log)
    close(oracle.softmax_backward(y, dy, log), dx, 2e-5, 1e-4)


@pytest.mark.parametrize("n", V.SILU_SIZES)
def test_oracle_silu_mul_backward(oracle, n):
    x, u, dy, dg, du = V.silu_mul_backward_case(n)
    g, h = oracle.silu_mul_backward(x, u, dy)
    close(g, dg, 2e-5, 1e-4); close(h, du, 2e-5, 1e-4)


def test_oracle_repeat_and_column_sum(oracle):
    dy = ((np.arange(2 * 6 * 5 * 7) % 11).astype(np.float32) / 8 - 0.25).reshape(2, 6, 5, 7)
    want = dy.astype(np.float64).reshape(2, 3, 2, 5, 7).sum(2)   # examples/grouped_attention_tensor.rs:51-68
    close(oracle.repeat_kv_heads_backward(dy, 3), want, 1e-6, 1e-6)
    close(oracle.column_sum(dy), dy.astype(np.float64).reshape(-1, 7).sum(0), 1e-5, 1e-6)


# ---- GPU ---------------------------------------------------------------------------------------------
gpu = pytest.mark.gpu


@gpu
@pytest.mark.parametrize("rows,width", SHAPES)
def test_gpu_rms_norm_backward(client, oracle, rows, width):
    from rust_ascend_b200 import B200Runtime as RT
    x, w, dy, r, dx, dw = V.rms_backward_case(rows, width)
    up = client.upload
    gdx, gdw = RT.rms_norm_backward(client, up(x), up(w), up(dy), up(r))
    odx, odw = oracle.rms_norm_backward(x, w, dy, r)
    close(client.read(gdx), odx, 1e-6, 1e-5); close(client.read(gdw), odw, 1e-4, 2e-5)
    close(client.read(gdx), dx, 5e-4, 5e-4); close(client.read(gdw), dw, 5e-4, 5e-4)   # examples/rms_norm_runtime.rs:20


@gpu
@pytest.mark.parametrize("rows,width", SHAPES)
@pytest.mark.parametrize("log", [False, True])
def test_gpu_softmax_backward(client, oracle, rows, width, log):
    from rust_ascend_b200 import B200Runtime as RT
    y, dy, dx = V.softmax_backward_case(rows, width, log)
    fn = RT.log_softmax_backward if log else RT.softmax_backward
    got = client.read(fn(client, client.upload(y), client.upload(dy)))
    close(got, oracle.softmax_backward(y, dy, log), 2e-6, 2e-5); close(got, dx, 2e-5, 1e-4)


@gpu
@pytest.mark.parametrize("n", V.SILU_SIZES + [100003])
def test_gpu_silu_mul_backward(client, oracle, n):
    from rust_ascend_b200 import B200Runtime as RT
    if n > 5000:
        rng = np.random.default_rng(n); x = rng.normal(size=n).astype(np.float32) * 4; u = rng.normal(size=n).astype(np.float32); dy = rng.normal(size=n).astype(np.float32)
    else:
        x, u, dy, _, _ = V.silu_mul_backward_case(n)
    dg, du = RT.silu_mul_backward(client, client.upload(x.reshape(1, n)), client.upload(u.reshape(1, n)), client.upload(dy.reshape(1, n)))
    og, ou = oracle.silu_mul_backward(x, u, dy)
    close(client.read(dg)[0], og, 1e-6, 1e-5); close(client.read(du)[0], ou, 1e-6, 1e-5)


@gpu
@pytest.mark.parametrize("group", [1, 2, 3, 5, 9])
def test_gpu_repeat_kv_backward_and_bias_backward(client, oracle, group):
    from rust_ascend_b200 import B200Runtime as RT
    b, kv, n, d = 2, 3, 5, 7
    dy = ((np.arange(b * kv * group * n * d) % 11).astype(np.float32) / 8 - 0.25).reshape(b, kv * group, n, d)
    got = client.read(RT.repeat_kv_heads_backward(client, (b, kv, n, d), kv * group, client.upload(dy)))
    close(got, oracle.repeat_kv_heads_backward(dy, kv), 1e-6, 1e-6)
    g2 = np.random.default_rng(group).normal(size=(3, 700, 130)).astype(np.float32)
    close(client.read(RT.bias_add_backward(client, client.upload(g2), g2.shape)), oracle.column_sum(g2), 2e-4, 1e-5)


@gpu
def test_gpu_linear_backward_vectors(client, oracle):
    from rust_ascend_b200 import B200Runtime as RT
    from rust_ascend_b200 import DType
    from rust_ascend_b200.runtime import bf16_bits_to_f32, f32_to_bf16_bits
    x, w, dy, dx, dw = V.linear_backward_case()
    u16 = lambda a: client.upload(f32_to_bf16_bits(a))
    gdx, gdw = RT.linear_nt_backward(client, u16(x), u16(w), u16(dy))
    assert gdx.dtype == DType.BF16 and gdw.dtype == DType.F32 and gdx.shape == x.shape and gdw.shape == w.shape
    close(bf16_bits_to_f32(client.read(gdx)), dx, 5e-4, 4e-3); close(client.read(gdw), dw, 5e-4, 5e-4)   # examples/matrix_runtime.rs:20-24
    # FP32-gradient variant through the saved BF16 snapshots (examples/linear_tensor.rs:24-50)
    out, x16, w16 = RT.linear_bf16_fp32(client, client.upload(x), client.upload(w))
    fdx, fdw = RT.linear_bf16_fp32_backward(client, x16, w16, client.upload(dy))
    close(client.read(fdx), dx, 5e-4, 5e-4); close(client.read(fdw), dw, 5e-4, 5e-4)
    frozen = RT.linear_frozen_bf16_fp32_backward(client, x.shape, w16, client.upload(dy))
    np.testing.assert_array_equal(client.read(frozen), client.read(fdx))
    # all four transpose forms agree with the oracle's GEMM on the same algebra (matrix.rs:95-121)
    rng = np.random.default_rng(4)
    for ta in (False, True):
        for tb in (False, True):
            m, n, k = 48, 32, 64
            a = rng.integers(-4, 5, size=(k, m) if ta else (m, k)).astype(np.float32) / 4
            b = rng.integers(-4, 5, size=(n, k) if tb else (k, n)).astype(np.float32) / 4
            g = rng.integers(-4, 5, size=(m, n)).astype(np.float32) / 8
            from rust_ascend_b200 import Transpose
            da, db = RT.gemm_bf16_fp32_backward(client, u16(a), u16(b), client.upload(g), Transpose(int(ta)), Transpose(int(tb)))
            A = a.T if ta else a; B = b.T if tb else b
            dA, dB = g.astype(np.float64) @ B.T.astype(np.float64), A.T.astype(np.float64) @ g.astype(np.float64)
            close(client.read(da), dA.T if ta else dA, 1e-5, 1e-5); close(client.read(db), dB.T if tb else dB, 1e-5, 1e-5)
