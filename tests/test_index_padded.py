"""Embedding weight gradient, prefix resize and the padded matrix wrappers.

CPU: the oracle's embedding backward against the expectation written out in the reference's device example
(examples/embedding_tensor.rs:22-53) and the padded specification's shape rules (deepgemm/padded.rs:60-80).
GPU: the CUDA kernels through the C ABI against the oracle / NumPy, and the padded matmul against the f64 reference with
explicit BF16 rounding of examples/padded_matrix_tensor.rs:12-47 (tolerance 5e-4 + 5e-4 relative, as there)."""
import itertools

import numpy as np
import pytest

from test_backward import close

gpu = pytest.mark.gpu


def bf16(x):
    bits = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).astype(np.float64)


# ---- embedding ------------------------------------------------------------------------------------------------------
def embedding_example():
    vocab, width = 7, 65
    weights = (np.arange(vocab * width, dtype=np.float32) / 8 - 2).reshape(vocab, width)
    ids = np.array([2, 0, 2, 5, 0, 2], dtype=np.int32).reshape(2, 3)
    upstream = ((np.arange(ids.size * width) % 17).astype(np.float32) / 8 - 0.5).reshape(2, 3, width)
    return weights, ids, upstream


def embedding_expected(ids, grad, vocab, padding_idx, scale):
    """examples/embedding_tensor.rs:44-53 with the factor 2 of its (y*dy + y*dy) already inside `grad`."""
    flat = ids.reshape(-1); g = grad.reshape(flat.size, -1).astype(np.float64)
    dw = np.zeros((vocab, g.shape[1]))
    for p, row in enumerate(flat):
        if padding_idx is not None and row == padding_idx:
            continue
        dw[row] += g[p]
    if scale:
        for row in range(vocab):
            count = int((flat == row).sum())
            if count:
                dw[row] /= count
    return dw


OPTIONS = list(itertools.product([None, 0], [False, True]))


@pytest.mark.parametrize("padding_idx,scale", OPTIONS)
def test_oracle_embedding_backward_matches_reference_example(oracle, padding_idx, scale):
    weights, ids, upstream = embedding_example()
    got = oracle.embedding_backward(2 * upstream, ids, weights.shape[0], padding_idx, scale)
    close(got, embedding_expected(ids, 2 * upstream, weights.shape[0], padding_idx, scale), 1e-5, 1e-5)
    for shape in [(0, 3), (2, 0)]:                              # examples/embedding_tensor.rs:62-70
        empty = oracle.embedding_backward(np.zeros(shape + (65,), np.float32), np.zeros(shape, np.int32), 7)
        assert empty.shape == (7, 65) and not empty.any()


def test_padded_spec_shapes_follow_reference_cases():
    from rust_ascend_b200 import B200Runtime as RT, DType, InvalidTensor, Transpose
    for batch in (None, 2):                                     # deepgemm/padded.rs:60-74
        for m, n, k in [(1, 1, 1), (3, 17, 7), (17, 33, 65), (16, 32, 48)]:
            for ta, tb in itertools.product([Transpose.No, Transpose.Yes], repeat=2):
                a = [m, k] if ta == Transpose.No else [k, m]
                b = [k, n] if tb == Transpose.No else [n, k]
                out = [m, n]
                if batch:
                    a.insert(0, batch); b.insert(0, batch); out.insert(0, batch)
                shape, pa, pb = RT._padded_spec(tuple(a), tuple(b), DType.F32, DType.BF16, ta, tb)
                up = lambda d: (d + 15) // 16 * 16
                assert shape == tuple(out)
                assert pa[-2:] == tuple(up(d) for d in a[-2:]) and pb[-2:] == tuple(up(d) for d in b[-2:])
    no = Transpose.No                                           # deepgemm/padded.rs:76-83
    bad = [((3, 7), (8, 17), DType.F32), ((0, 7), (7, 17), DType.F32), ((2, 3, 7), (1, 7, 17), DType.F32),
           ((3, 7), (7, 17), DType.F16), ((2**31 - 1, 7), (7, 17), DType.F32), ((4097, 3, 7), (4097, 7, 17), DType.F32)]
    for a, b, dt in bad:
        with pytest.raises(InvalidTensor):
            RT._padded_spec(a, b, dt, DType.F32, no, no)


def test_matmul_shape_follows_the_reference_rules():
    from rust_ascend_b200 import B200Runtime as RT, InvalidTensor
    assert RT.matmul_shape((2, 1, 3, 5), (1, 4, 5, 7)) == (2, 4, 3, 7)        # runtime/generic_matrix.rs:60-66
    assert RT.matmul_shape((0, 5), (5, 7)) == (0, 7) and RT.matmul_shape((3, 0), (0, 7)) == (3, 7)
    assert RT.matmul_shape((6, 3, 5), (5, 7)) == (6, 3, 7)
    for a, b in (((3, 5), (4, 7)), ((2, 3, 5), (3, 5, 7))):
        with pytest.raises(InvalidTensor):
            RT.matmul_shape(a, b)


def test_group_ends_follow_the_reference_rules():
    from rust_ascend_b200 import B200Runtime as RT, InvalidTensor
    assert RT.group_ends([0, 256, 256, 768]) == [0, 256, 256, 768]           # deepgemm/plan.rs:101: empty experts are fine
    for bad in ([1, 17], [256, 0], [0, 0], [], [256] * 4097):               # plan.rs:102 and the 4096-group limit
        with pytest.raises(InvalidTensor):
            RT.group_ends(bad)


@gpu
def test_gpu_embedding_lookup_unaligned_rows(client):
    from rust_ascend_b200 import B200Runtime as RT
    from rust_ascend_b200.runtime import f32_to_bf16_bits
    weights, ids, _ = embedding_example()
    np.testing.assert_array_equal(client.read(RT.embedding(client, client.upload(weights), client.upload(ids))), weights[ids])
    out, saved = RT.embedding_with_saved_indices(client, client.upload(weights), client.upload(ids.astype(np.int64)))
    np.testing.assert_array_equal(client.read(out), weights[ids]); np.testing.assert_array_equal(client.read(saved), ids)
    w16 = f32_to_bf16_bits(weights)                             # 130-byte rows move as 2-byte words
    np.testing.assert_array_equal(client.read(RT.embedding(client, client.upload(w16), client.upload(ids))), w16[ids])
    for shape in [(0, 3), (2, 0)]:
        assert client.read(RT.embedding(client, client.upload(weights), client.upload(np.zeros(shape, np.int32)))).shape == shape + (65,)


@gpu
@pytest.mark.parametrize("padding_idx,scale", OPTIONS)
def test_gpu_embedding_backward_reference_example(client, oracle, padding_idx, scale):
    from rust_ascend_b200 import B200Runtime as RT
    weights, ids, upstream = embedding_example()
    for dev_ids in (ids, ids.astype(np.int64)):
        got = client.read(RT.embedding_backward(client, client.upload(2 * upstream), client.upload(dev_ids), 7, padding_idx, scale))
        close(got, oracle.embedding_backward(2 * upstream, ids, 7, padding_idx, scale), 1e-6, 1e-6)
        close(got, embedding_expected(ids, 2 * upstream, 7, padding_idx, scale), 1e-5, 1e-5)


@gpu
def test_gpu_embedding_backward_sizes_dtypes_and_errors(client, oracle):
    from rust_ascend_b200 import B200Runtime as RT, InvalidTensor
    from rust_ascend_b200.runtime import f32_to_bf16_bits, bf16_bits_to_f32
    rng = np.random.default_rng(3)
    ids = rng.integers(0, 1000, size=(4, 513)).astype(np.int32); ids[0, :64] = 7          # a heavily repeated row
    grad = rng.standard_normal((4, 513, 128)).astype(np.float32)
    want = oracle.embedding_backward(grad, ids, 1000, None, True)
    close(client.read(RT.embedding_backward(client, client.upload(grad), client.upload(ids), 1000, None, True)), want, 1e-5, 1e-5)
    g16 = f32_to_bf16_bits(grad)
    got16 = bf16_bits_to_f32(client.read(RT.embedding_backward(client, client.upload(g16), client.upload(ids), 1000)))
    close(got16, oracle.embedding_backward(bf16_bits_to_f32(g16), ids, 1000), 1e-5, 2.0 ** -8)
    for shape in [(0, 3), (2, 0)]:
        empty = RT.embedding_backward(client, client.upload(np.zeros(shape + (65,), np.float32)), client.upload(np.zeros(shape, np.int32)), 7)
        assert client.read(empty).shape == (7, 65) and not client.read(empty).any()
    with pytest.raises(InvalidTensor):
        RT.embedding_backward(client, client.upload(grad), client.upload(ids), 1000, 1000)
    with pytest.raises(InvalidTensor):
        RT.embedding_backward(client, client.upload(grad[:, :512]), client.upload(ids), 1000)
    with pytest.raises(InvalidTensor):
        RT.embedding_backward(client, client.upload(grad), client.upload(ids.astype(np.float32)), 1000)


# ---- prefix resize and padded matrices --------------------------------------------------------------------------------
def resize_numpy(x, shape):
    out = np.zeros(shape, dtype=x.dtype)
    region = tuple(slice(0, min(a, b)) for a, b in zip(x.shape, shape))
    out[region] = x[region]
    return out


@gpu
def test_gpu_resize_prefix_pads_and_crops_bits(client):
    from rust_ascend_b200 import B200Runtime as RT, InvalidTensor
    from rust_ascend_b200.runtime import f32_to_bf16_bits
    rng = np.random.default_rng(11)
    x = rng.standard_normal((2, 3, 17)).astype(np.float32); x[0, 0, 0] = np.inf; x[1, 2, 16] = -0.0
    for shape in [(2, 16, 32), (2, 3, 17), (1, 2, 5), (4, 1, 40), (2, 3, 16)]:
        got = client.read(RT.resize_prefix(client, client.upload(x), shape))
        np.testing.assert_array_equal(got.view(np.uint32), resize_numpy(x, shape).view(np.uint32))
    x16 = f32_to_bf16_bits(x)
    np.testing.assert_array_equal(client.read(RT.resize_prefix(client, client.upload(x16), (2, 16, 32))), resize_numpy(x16, (2, 16, 32)))
    big = rng.standard_normal((513, 1031)).astype(np.float32)
    np.testing.assert_array_equal(client.read(RT.resize_prefix(client, client.upload(big), (528, 1040))), resize_numpy(big, (528, 1040)))
    same = client.upload(x)
    assert RT.resize_prefix(client, same, x.shape) is same
    with pytest.raises(InvalidTensor):
        RT.resize_prefix(client, client.upload(x), (16, 32))
    with pytest.raises(InvalidTensor):
        RT.resize_prefix(client, client.upload(x), (2, 0, 17))
    with pytest.raises(InvalidTensor):
        RT.resize_prefix(client, client.upload(np.zeros((2, 3, 17), np.int32)), (2, 3, 18))


def padded_case(batch, m, n, k, ta, tb):
    """Inputs and f64 expectations of examples/padded_matrix_tensor.rs:12-33 (dY already carries the factor 2)."""
    batches = batch or 1
    a = ((np.arange(batches * m * k) % 17).astype(np.float32) - 8) / np.float32(59)
    b = ((np.arange(batches * k * n) % 13).astype(np.float32) - 6) / np.float32(43)
    dy = ((np.arange(batches * m * n) % 11).astype(np.float32) - 5) / np.float32(37)
    A = a.reshape(batches, *((m, k) if not ta else (k, m))); B = b.reshape(batches, *((k, n) if not tb else (n, k)))
    opa = bf16(A) if not ta else bf16(A).transpose(0, 2, 1); opb = bf16(B) if not tb else bf16(B).transpose(0, 2, 1)
    g = bf16(dy).reshape(batches, m, n)
    y = opa @ opb
    da = g @ opb.transpose(0, 2, 1); db = opa.transpose(0, 2, 1) @ g
    if ta: da = da.transpose(0, 2, 1)
    if tb: db = db.transpose(0, 2, 1)
    lead = (batch,) if batch else ()
    shape = lambda t: lead + t.shape[1:]
    return (A.reshape(shape(A)), B.reshape(shape(B)), dy.reshape(lead + (m, n)), y.reshape(lead + (m, n)), da.reshape(shape(A)), db.reshape(shape(B)))


@gpu
@pytest.mark.parametrize("batch", [None, 2])
@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (3, 17, 7), (17, 33, 65), (16, 32, 48)])
def test_gpu_padded_matmul_reference_example(client, batch, m, n, k):
    from rust_ascend_b200 import B200Runtime as RT, DType, Transpose
    for ta, tb in itertools.product([Transpose.No, Transpose.Yes], repeat=2):
        A, B, dy, y, da, db = padded_case(batch, m, n, k, bool(ta), bool(tb))
        out, a16, b16 = RT.gemm_padded_bf16_fp32(client, client.upload(A), client.upload(B), ta, tb)
        assert out.shape == y.shape and out.dtype == DType.F32 and a16.dtype == DType.BF16
        assert all(d % 16 == 0 for d in a16.shape[-2:] + b16.shape[-2:])
        close(client.read(out), y, 5e-4, 5e-4)
        gda, gdb = RT.gemm_padded_bf16_fp32_backward(client, a16, b16, client.upload(dy), A.shape, B.shape, ta, tb)
        assert gda.shape == A.shape and gdb.shape == B.shape
        close(client.read(gda), da, 5e-4, 5e-4); close(client.read(gdb), db, 5e-4, 5e-4)


@gpu
def test_gpu_frozen_padded_linear(client):
    from rust_ascend_b200 import B200Runtime as RT, DType, InvalidTensor
    from rust_ascend_b200.runtime import f32_to_bf16_bits, bf16_bits_to_f32
    m, n, k = 3, 19, 35                                         # examples/padded_matrix_tensor.rs:49-52
    x = (((np.arange(m * k) % 7).astype(np.float32) - 3) / 64).reshape(m, k)
    w = (((np.arange(n * k) % 5).astype(np.float32) - 2) / 16).reshape(n, k)
    dy = (((np.arange(m * n) % 7).astype(np.float32) - 3) / 8).reshape(m, n)
    w16 = client.upload(f32_to_bf16_bits(w))
    y, used = RT.linear_frozen_padded_bf16_fp32(client, client.upload(x), w16)
    assert y.shape == (m, n) and used.shape == (32, 48) and used.dtype == DType.BF16
    close(client.read(y), bf16(x) @ bf16(w).T, 5e-4, 5e-4)
    dx = RT.linear_frozen_padded_bf16_fp32_backward(client, used, client.upload(dy), x.shape, w.shape)
    assert dx.shape == x.shape
    close(client.read(dx), bf16(dy) @ bf16(w), 5e-4, 5e-4)
    np.testing.assert_array_equal(client.read(w16), f32_to_bf16_bits(w))          # the weight is never written
    aligned = client.upload(f32_to_bf16_bits(np.ones((32, 48), np.float32)))
    _, reused = RT.linear_frozen_padded_bf16_fp32(client, client.upload(np.ones((5, 48), np.float32)), aligned)
    assert reused is aligned                                                      # aligned weights reuse their handle
    # Inf in a logical activation times the zero padding gives NaN only in artificial channels, which the crop removes
    # (examples/padded_matrix_tensor.rs:80-84).
    out, _, _ = RT.gemm_padded_bf16_fp32(client, client.upload(np.array([[np.inf]], np.float32)), client.upload(np.ones((1, 1), np.float32)),
                                         0, 1)
    assert client.read(out).tolist() == [[np.inf]]
    with pytest.raises(InvalidTensor):
        RT.linear_frozen_padded_bf16_fp32(client, client.upload(x), client.upload(w))
