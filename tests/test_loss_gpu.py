"""LayerNorm backward and the causal-LM loss edge: the CUDA kernels through the C ABI against the oracle, which
tests/test_oracle_next.py pins to the reference's own expectations.  Summation order differs (block tree on the GPU,
the reference's row schedule in the oracle), so comparisons are tolerance-based: 5e-4 absolute and relative for the
norm (examples/layer_norm_tensor.rs), 2e-5 + 1e-4 relative for the loss and its gradient."""
import numpy as np
import pytest

from test_backward import close, SHAPES

pytestmark = pytest.mark.gpu


def layer_case(rows, width, seed=5):
    rng = np.random.default_rng(seed + rows * 131 + width)
    x = rng.standard_normal((rows, width)).astype(np.float32) * 1.5 + 0.25
    w = (1 + 0.1 * rng.standard_normal(width)).astype(np.float32)
    dy = rng.standard_normal((rows, width)).astype(np.float32)
    mean = x.mean(-1, dtype=np.float64).astype(np.float32) if rows else np.zeros(0, np.float32)
    var = x.astype(np.float64).var(-1) if rows else np.zeros(0)
    rstd = (1.0 / np.sqrt(var + 1e-5)).astype(np.float32)
    return x, w, dy, mean, rstd


@pytest.mark.parametrize("rows,width", SHAPES)
def test_layer_norm_backward(client, oracle, rows, width):
    from rust_ascend_b200 import B200Runtime as RT
    x, w, dy, mean, rstd = layer_case(rows, width)
    up = client.upload
    dx, dw, db = RT.layer_norm_backward(client, up(x), up(w), up(dy), up(mean), up(rstd))
    odx, odw, odb = oracle.layer_norm_backward(x, w, dy, mean, rstd)
    if rows == 0:
        odw[:] = 0; odb[:] = 0
    close(client.read(dx), odx, 5e-5, 5e-5); close(client.read(dw), odw, 5e-4, 5e-5); close(client.read(db), odb, 5e-4, 5e-5)


def test_layer_norm_backward_rejects_mismatch(client):
    from rust_ascend_b200 import B200Runtime as RT, InvalidTensor
    x, w, dy, mean, rstd = layer_case(4, 32)
    up = client.upload
    with pytest.raises(InvalidTensor):
        RT.layer_norm_backward(client, up(x), up(w[:16].copy()), up(dy), up(mean), up(rstd))
    with pytest.raises(InvalidTensor):
        RT.layer_norm_backward(client, up(x), up(w), up(dy), up(mean[:3].copy()), up(rstd[:3].copy()))


CE_CASES = [(1, 1, 8, True), (2, 5, 11, True), (2, 5, 11, False), (3, 17, 1000, True), (1, 64, 32000, True), (4, 9, 257, False)]


@pytest.mark.parametrize("batch,time,vocab,shift", CE_CASES)
@pytest.mark.parametrize("wide", [False, True])
def test_causal_cross_entropy(client, oracle, batch, time, vocab, shift, wide):
    from rust_ascend_b200 import B200Runtime as RT
    rng = np.random.default_rng(batch * 7 + time * 3 + vocab)
    logits = (rng.standard_normal((batch, time, vocab)) * 3).astype(np.float32)
    labels = rng.integers(0, vocab, size=(batch, time)).astype(np.int64)
    labels[rng.random((batch, time)) < 0.25] = -100
    want_loss, want_valid, want_d = oracle.causal_cross_entropy(logits, labels, -100, shift, 0.5)
    dev_labels = labels if wide else labels.astype(np.int32)
    loss, valid, d = RT.causal_cross_entropy(client, client.upload(logits), client.upload(dev_labels), -100, shift, 0.5)
    assert client.read(valid)[0] == want_valid
    close(client.read(loss), [want_loss], 2e-5, 1e-5 * max(1.0, want_valid) ** 0.5 + 1e-4)
    close(client.read(d), want_d, 2e-6, 1e-4)
    loss2, valid2, none = RT.causal_cross_entropy(client, client.upload(logits), client.upload(dev_labels), -100, shift, 1.0, with_gradient=False)
    assert none is None and client.read(valid2)[0] == want_valid
    assert client.read(loss2)[0] == client.read(loss)[0]          # deterministic sum


def test_causal_cross_entropy_all_ignored_and_errors(client):
    from rust_ascend_b200 import B200Runtime as RT, InvalidTensor
    logits = np.ones((2, 3, 5), np.float32)
    labels = np.full((2, 3), -100, np.int64)
    loss, valid, d = RT.causal_cross_entropy(client, client.upload(logits), client.upload(labels))
    assert client.read(loss)[0] == 0 and client.read(valid)[0] == 0 and not client.read(d).any()
    # A label beyond the vocabulary is never read through: the row is left unscored (a synchronous context also
    # returns InvalidTensor for it; this context is asynchronous).
    loss, valid, d = RT.causal_cross_entropy(client, client.upload(logits), client.upload(np.full((2, 3), 5, np.int64)))
    assert client.read(valid)[0] == 0 and client.read(loss)[0] == 0 and not client.read(d).any()
    with pytest.raises(InvalidTensor):                              # batch mismatch
        RT.causal_cross_entropy(client, client.upload(logits), client.upload(np.zeros((1, 3), np.int64)))
    with pytest.raises(InvalidTensor):                              # FP32 labels
        RT.causal_cross_entropy(client, client.upload(logits), client.upload(np.zeros((2, 3), np.float32)))
