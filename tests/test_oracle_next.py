"""CPU: oracle functions for the operators that come next on the path (attention backward, LayerNorm backward, causal
cross entropy), pinned to the f64 expectations of the reference's device examples.  No CUDA kernel uses them yet; they
are the checker those kernels will be built against."""
import numpy as np
import pytest

import vectors as V


def close(actual, expected, atol, rtol):
    actual = np.asarray(actual, dtype=np.float64); expected = np.asarray(expected, dtype=np.float64)
    assert actual.shape == expected.shape and np.all(np.isfinite(actual))
    err = np.abs(actual - expected) - (atol + rtol * np.abs(expected))
    assert err.size == 0 or err.max() <= 0, f"max excess {err.max()}"


@pytest.mark.parametrize("kv_heads,group,n,causal", V.GQA_CASES)
def test_attention_backward_matches_the_reference_example(oracle, kv_heads, group, n, causal):
    # examples/grouped_attention_tensor.rs:14-44,74-99: f64 reference with BF16 rounding of inputs, P and scale*dS
    q, k, v, mask, prefix, _ = V.gqa_case(kv_heads, group, n, causal)
    batch, heads, m, d = q.shape
    dv_ = v.shape[3]
    dy = ((np.arange(batch * heads * m * dv_) % 7).astype(np.float32) / np.float32(8.0) - np.float32(0.25)).reshape(batch, heads, m, dv_)
    qb, dyb = V.bf16_f64(q), V.bf16_f64(dy)
    kb, vb = np.repeat(V.bf16_f64(k), group, axis=1), np.repeat(V.bf16_f64(v), group, axis=1)
    s = 0.25 * np.einsum("bhmd,bhnd->bhmn", qb, kb) + mask.astype(np.float64)
    e = np.exp(s - s.max(-1, keepdims=True)); p = e / e.sum(-1, keepdims=True)
    dp = np.einsum("bhmc,bhnc->bhmn", dyb, vb)
    ds = p * (dp - (p * dp).sum(-1, keepdims=True))
    p_b, ds_b = V.bf16_f64(p.astype(np.float32)), V.bf16_f64((0.25 * ds).astype(np.float32))
    want_dq = np.einsum("bhmn,bhnd->bhmd", ds_b, kb)
    want_dk = np.einsum("bhmn,bhmd->bhnd", ds_b, qb).reshape(batch, kv_heads, group, n, d).sum(2)
    want_dv = np.einsum("bhmn,bhmc->bhnc", p_b, dyb).reshape(batch, kv_heads, group, n, dv_).sum(2)
    if causal:
        got = oracle.attention_backward(q, k, v, dy, 0.25, causal=True, query_start=(1 << 40) + prefix, key_start=1 << 40)
    else:
        got = oracle.attention_backward(q, k, v, dy, 0.25, mask=mask, want_mask_grad=True)
        close(got[3], ds, 2e-3, 3e-3)
    close(got[0], want_dq, 2e-3, 3e-3); close(got[1], want_dk, 2e-3, 3e-3); close(got[2], want_dv, 2e-3, 3e-3)


@pytest.mark.parametrize("rows,width", [(1, 32), (3, 96), (7, 256), (3, 4096), (5, 33)])
def test_layer_norm_backward_vs_autograd(oracle, rows, width):
    import torch
    rng = np.random.default_rng(width + 3)
    x = rng.normal(size=(rows, width)).astype(np.float32); w = rng.normal(size=width).astype(np.float32)
    b = rng.normal(size=width).astype(np.float32); dy = rng.normal(size=(rows, width)).astype(np.float32)
    _, mean, rstd = oracle.layer_norm(x, w, b, 1e-5)
    dx, dw, db = oracle.layer_norm_backward(x, w, dy, mean, rstd)
    t = torch.tensor(x, dtype=torch.float64, requires_grad=True); tw = torch.tensor(w, dtype=torch.float64, requires_grad=True)
    tb = torch.tensor(b, dtype=torch.float64, requires_grad=True)
    (torch.nn.functional.layer_norm(t, (width,), tw, tb, eps=1e-5) * torch.tensor(dy, dtype=torch.float64)).sum().backward()
    close(dx, t.grad.numpy(), 3e-6, 2e-4)   # tools/ascend/tests/test_row_reference.py:121-123
    close(dw, tw.grad.numpy(), 2e-5, 2e-4); close(db, tb.grad.numpy(), 2e-5, 2e-5)


@pytest.mark.parametrize("shift", [False, True])
@pytest.mark.parametrize("all_ignored", [False, True])
def test_causal_cross_entropy_identity(oracle, shift, all_ignored):
    # examples/causal_lm_tensor.rs:24-118 (upstream gradient 2 = mean + mean)
    batch, time, vocab = 2, 5, 65
    x = ((np.arange(batch * time * vocab) % 23).astype(np.float32) / np.float32(8.0) - np.float32(7.0)).reshape(batch, time, vocab)
    labels = np.array([-100 if (all_ignored or i % 3 == 0) else (i * 7 % vocab) for i in range(batch * time)], dtype=np.int64).reshape(batch, time)
    total, valid, expected = 0.0, 0, np.zeros_like(x, dtype=np.float64)
    for b in range(batch):
        for t in range(time - 1 if shift else time):
            label = labels[b, t + (1 if shift else 0)]
            if label == -100:
                continue
            valid += 1
            v = x[b, t].astype(np.float64); mx = v.max(); e = np.exp(v - mx); den = e.sum()
            total += np.log(den) + mx - v[label]
            expected[b, t] = 2.0 * (e / den - (np.arange(vocab) == label))
    expected /= max(valid, 1)
    loss, count, d = oracle.causal_cross_entropy(x, labels, -100, shift, upstream=2.0)
    close([loss], [total], 2e-4, 2e-4); assert count == valid
    close(d, expected, 2e-4, 2e-4)
