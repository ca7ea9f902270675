"""The tensor-level mirrors of src/nn/padded.rs, src/nn/embedding.rs, src/nn/frozen.rs and src/nn/causal_lm.rs through the
C ABI: the identity case of examples/causal_lm_tensor.rs:24-118 (with an identity projection, so the loss is the example's),
a projected case against the oracle, and the padded / embedding wrappers against NumPy."""
import numpy as np
import pytest

from test_backward import close
from test_index_padded import bf16, embedding_example, embedding_expected

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shift", [False, True])
@pytest.mark.parametrize("all_ignored", [False, True])
def test_causal_loss_reference_example(client, shift, all_ignored):
    import rust_ascend_b200.nn as nn
    batch, time, vocab = 2, 5, 65
    x = ((np.arange(batch * time * vocab) % 23).astype(np.float32) / np.float32(8.0) - np.float32(7.0)).reshape(batch, time, vocab)
    labels = np.array([-100 if (all_ignored or i % 3 == 0) else (i * 7 % vocab) for i in range(batch * time)], dtype=np.int64).reshape(batch, time)
    total, valid = 0.0, 0
    for b in range(batch):
        for t in range(time - 1 if shift else time):
            label = labels[b, t + (1 if shift else 0)]
            if label == -100:
                continue
            valid += 1
            v = x[b, t].astype(np.float64); mx = v.max()
            total += np.log(np.exp(v - mx).sum()) + mx - v[label]
    for dev_labels in (labels, labels.astype(np.int32)):
        loss = nn.CausalCrossEntropyConfig(shift=shift).forward_hidden(nn.Tensor.from_data(client, x), nn.Tensor.from_data(client, dev_labels), lambda h: h)
        close(loss.loss_sum.into_data(), [total], 2e-4, 2e-4)
        assert loss.valid_tokens.into_data()[0] == valid
        close(loss.mean().into_data(), [total / max(valid, 1)], 2e-4, 2e-4)


def test_causal_loss_with_projection_and_rejections(client, oracle):
    import rust_ascend_b200.nn as nn
    from rust_ascend_b200 import InvalidTensor
    rng = np.random.default_rng(21)
    batch, time, width, vocab = 3, 9, 40, 257
    hidden = rng.standard_normal((batch, time, width)).astype(np.float32)
    weight = (rng.standard_normal((vocab, width)) * 0.2).astype(np.float32)
    labels = rng.integers(0, vocab, size=(batch, time)).astype(np.int64); labels[0, 3] = -100
    w = nn.Tensor.from_data(client, weight)
    loss = nn.CausalCrossEntropyConfig().forward_hidden(nn.Tensor.from_data(client, hidden), nn.Tensor.from_data(client, labels),
                                                        lambda h: nn.linear_padded_bf16_fp32(h, w))
    logits = (bf16(hidden.reshape(-1, width)) @ bf16(weight).T).astype(np.float32).reshape(batch, time, vocab)
    want, count, _ = oracle.causal_cross_entropy(logits, labels, -100, True, 1.0)
    close(loss.loss_sum.into_data(), [want], 1e-3, 1e-4)
    assert loss.valid_tokens.into_data()[0] == count
    h, l = nn.Tensor.from_data(client, hidden), nn.Tensor.from_data(client, labels)
    with pytest.raises(InvalidTensor):
        nn.CausalCrossEntropyConfig(token_chunk_size=0).forward_hidden(h, l, lambda t: t)
    with pytest.raises(InvalidTensor):
        nn.CausalCrossEntropyConfig().forward_hidden(h, nn.Tensor.from_data(client, labels[:, :4]), lambda t: t)
    with pytest.raises(InvalidTensor):
        nn.CausalCrossEntropyConfig().forward_hidden(h, nn.Tensor.from_data(client, labels.astype(np.float32)), lambda t: t)


def test_padded_and_embedding_wrappers(client):
    import rust_ascend_b200.nn as nn
    from rust_ascend_b200 import DType, InvalidTensor, Transpose
    from rust_ascend_b200.runtime import f32_to_bf16_bits
    rng = np.random.default_rng(8)
    a = rng.standard_normal((3, 35)).astype(np.float32); b = rng.standard_normal((19, 35)).astype(np.float32)
    y = nn.linear_padded_bf16_fp32(nn.Tensor.from_data(client, a), nn.Tensor.from_data(client, b))
    assert y.dims() == [3, 19] and y.dtype() == DType.F32
    close(y.into_data(), bf16(a) @ bf16(b).T, 5e-4, 5e-4)
    y2 = nn.matmul_padded_bf16_fp32(nn.Tensor.from_data(client, a.T.copy()), nn.Tensor.from_data(client, b.T.copy()), Transpose.Yes, Transpose.No)
    close(y2.into_data(), bf16(a) @ bf16(b).T, 5e-4, 5e-4)
    frozen = nn.linear_frozen_padded_bf16_fp32(nn.Tensor.from_data(client, a), nn.Tensor.from_data(client, f32_to_bf16_bits(b)))
    close(frozen.into_data(), bf16(a) @ bf16(b).T, 5e-4, 5e-4)
    weights, ids, upstream = embedding_example()
    w = nn.Tensor.from_data(client, weights)
    out = nn.embedding(w, nn.Tensor.from_data(client, ids), nn.EmbeddingOptions(padding_idx=0))
    np.testing.assert_array_equal(out.into_data(), weights[ids])           # padding affects the derivative only
    dw = nn.embedding_backward(nn.Tensor.from_data(client, upstream), nn.Tensor.from_data(client, ids), 7, nn.EmbeddingOptions(0, True))
    close(dw.into_data(), embedding_expected(ids, upstream, 7, 0, True), 1e-5, 1e-5)
    frozen_rows = nn.embedding_frozen_bf16_fp32(nn.Tensor.from_data(client, f32_to_bf16_bits(weights)), nn.Tensor.from_data(client, ids.astype(np.int64)))
    assert frozen_rows.dtype() == DType.F32
    np.testing.assert_array_equal(frozen_rows.into_data(), bf16(weights)[ids].astype(np.float32))
    ln = nn.layer_norm(nn.Tensor.from_data(client, a), nn.Tensor.from_data(client, np.ones(35, np.float32)), None, 1e-5)
    ref = (a - a.mean(-1, keepdims=True)) / np.sqrt(a.astype(np.float64).var(-1, keepdims=True) + 1e-5)
    close(ln.into_data(), ref, 1e-4, 1e-4)
    with pytest.raises(InvalidTensor):
        nn.embedding(w, nn.Tensor.from_data(client, ids), nn.EmbeddingOptions(padding_idx=7))
    with pytest.raises(InvalidTensor):
        nn.embedding(nn.Tensor.from_data(client, f32_to_bf16_bits(weights)), nn.Tensor.from_data(client, ids))
