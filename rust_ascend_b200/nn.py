"""Mirror of `rust_ascend::nn` (src/nn.rs and src/nn/*.rs): explicit native operators on tensors.

The reference's functions are generic over RUDA `Tensor<B, D>`; here a `Tensor` is a `TensorBuffer` bound to
its `ComputeClient`.  Names, argument order, shape/dtype rules and error behaviour follow the reference; the
work is done by libruda_b200.so through `B200Runtime`.  Forward contracts only: the reference's autodiff
registration (`Backward` impls, src/nn.rs:209-232) needs RUDA and is outside this package.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .runtime import (B200Runtime as RT, ComputeClient, DType, InvalidTensor, RotaryLayout, TensorBuffer, Transpose)


@dataclass
class Tensor:
    client: ComputeClient
    buffer: TensorBuffer

    @classmethod
    def from_data(cls, client: ComputeClient, data, dtype: DType | None = None) -> "Tensor":
        return cls(client, client.upload(np.asarray(data), dtype))

    def dims(self):
        return list(self.buffer.shape)

    def dtype(self) -> DType:
        return self.buffer.dtype

    def into_data(self) -> np.ndarray:
        return self.client.read(self.buffer)

    def reshape(self, shape) -> "Tensor":
        return Tensor(self.client, self.buffer.reshape(shape))


def _same_client(*tensors):
    client = tensors[0].client
    for t in tensors[1:]:
        if t is not None and t.client is not client:
            raise InvalidTensor("tensors must live on the same device and execution queue")  # src/nn.rs:180-187
    return client


def _wrap(client, buffer):
    return Tensor(client, buffer)


def matmul_bf16_fp32(a: Tensor, b: Tensor, ta: Transpose = Transpose.No, tb: Transpose = Transpose.No) -> Tensor:
    """FP32 operands, BF16 compute, FP32 result (src/nn.rs:55-72)."""
    c = _same_client(a, b)
    return _wrap(c, RT.gemm_bf16_fp32(c, a.buffer, b.buffer, ta, tb)[0])


def linear_bf16_fp32(input: Tensor, weight: Tensor) -> Tensor:
    """Y = X W^T, W stored [N,K] (src/nn.rs:73-88)."""
    c = _same_client(input, weight)
    return _wrap(c, RT.linear_bf16_fp32(c, input.buffer, weight.buffer)[0])


def rms_norm(input: Tensor, weight: Tensor, epsilon: float) -> Tensor:
    """src/nn.rs:165-174."""
    c = _same_client(input, weight)
    return _wrap(c, RT.rms_norm(c, input.buffer, weight.buffer, epsilon)[0])


def softmax(input: Tensor) -> Tensor:
    """src/nn.rs:101-110."""
    return _wrap(input.client, RT.softmax(input.client, input.buffer))


def log_softmax(input: Tensor) -> Tensor:
    """src/nn.rs:111-120."""
    return _wrap(input.client, RT.log_softmax(input.client, input.buffer))


def sum_last(input: Tensor) -> Tensor:
    return _wrap(input.client, RT.sum_last(input.client, input.buffer))


def mean_last(input: Tensor) -> Tensor:
    return _wrap(input.client, RT.mean_last(input.client, input.buffer))


def silu_mul(gate: Tensor, up: Tensor) -> Tensor:
    """src/nn.rs:121-135."""
    c = _same_client(gate, up)
    return _wrap(c, RT.silu_mul(c, gate.buffer, up.buffer))


def swiglu_bf16_fp32(input: Tensor, gate: Tensor, up: Tensor, down: Tensor) -> Tensor:
    """(SiLU(X Wg^T) * (X Wu^T)) Wd^T with FP32 storage (src/nn/feed_forward.rs:28-42).  The gate/up pair runs as
    one tensor-core GEMM whose epilogue applies SiLU*up; the hidden activation is kept in FP32 as in the reference."""
    c = _same_client(input, gate, up, down)
    m, k = input.dims()
    hidden, gk = gate.dims()
    n, dh = down.dims()
    if gk != k or up.dims() != [hidden, k] or dh != hidden or any(s == 0 or s % 16 for s in (m, n, k, hidden)):
        raise InvalidTensor("SwiGLU requires aligned X[M,K], gate/up[H,K] and down[N,H]")
    if any(t.dtype() != DType.F32 for t in (input, gate, up, down)):
        raise InvalidTensor("SwiGLU requires FP32 input and weights on the same device")
    x16 = RT.cast(c, input.buffer, DType.BF16)
    h = RT.gemm(c, x16, RT.cast(c, gate.buffer, DType.BF16), Transpose.No, Transpose.Yes, DType.F32, b_up=RT.cast(c, up.buffer, DType.BF16))
    return _wrap(c, RT.linear_bf16_fp32(c, h, down.buffer)[0])


def rotary(input: Tensor, cos: Tensor, sin: Tensor, layout: RotaryLayout) -> Tensor:
    """src/nn/rotary.rs:19-30."""
    c = _same_client(input, cos, sin)
    return _wrap(c, RT.rotary(c, input.buffer, cos.buffer, sin.buffer, layout))


def rotary_prefix(input: Tensor, cos: Tensor, sin: Tensor, width: int, layout: RotaryLayout) -> Tensor:
    """src/nn/rotary.rs:32-45."""
    c = _same_client(input, cos, sin)
    return _wrap(c, RT.rotary_prefix(c, input.buffer, cos.buffer, sin.buffer, width, layout))


def repeat_kv_heads(input: Tensor, query_heads: int) -> Tensor:
    """src/nn/heads.rs:11-25."""
    return _wrap(input.client, RT.repeat_kv_heads(input.client, input.buffer, query_heads))


def causal_mask(client: ComputeClient, shape, query_start: int, key_start: int) -> Tensor:
    """FP32 [B,Q,K] mask (src/nn/mask.rs:12-25)."""
    b, q, k = shape
    return _wrap(client, RT.causal_mask(client, b, q, k, query_start, key_start))


def _attention(query, key, value, scale, mask, causal, query_start, key_start):
    c = _same_client(query, key, value, mask)
    rank3 = len(query.dims()) == 3
    q, k, v = query.buffer, key.buffer, value.buffer
    m = None if mask is None else mask.buffer
    if rank3:
        q, k, v = (t.reshape((t.shape[0], 1) + t.shape[1:]) for t in (q, k, v))
        m = None if m is None else m.reshape((m.shape[0], 1) + m.shape[1:])
    if any(t.dtype != DType.F32 for t in (q, k, v)):
        raise InvalidTensor("attention requires FP32 Q/K/V on the same device")
    out = RT.attention(c, q, k, v, scale, mask=m, causal=causal, query_start=query_start, key_start=key_start)
    return _wrap(c, out.reshape((out.shape[0],) + out.shape[2:]) if rank3 else out)


def scaled_dot_product_attention_bf16_fp32(query: Tensor, key: Tensor, value: Tensor, scale: float,
                                           additive_mask: Tensor | None = None) -> Tensor:
    """Q[B,M,D], K[B,N,D], V[B,N,Dv] FP32 (src/nn/attention.rs:10-29)."""
    if len(query.dims()) != 3:
        raise InvalidTensor("scaled_dot_product_attention takes rank-3 tensors")
    return _attention(query, key, value, scale, additive_mask, False, 0, 0)


def causal_attention_bf16_fp32(query: Tensor, key: Tensor, value: Tensor, scale: float, query_start: int, key_start: int) -> Tensor:
    """src/nn/attention.rs:33-45."""
    if len(query.dims()) != 3:
        raise InvalidTensor("causal_attention takes rank-3 tensors")
    return _attention(query, key, value, scale, None, True, query_start, key_start)


def grouped_query_attention_bf16_fp32(query: Tensor, key: Tensor, value: Tensor, scale: float,
                                      additive_mask: Tensor | None = None) -> Tensor:
    """Q[B,Hq,M,D], K[B,Hkv,N,D], V[B,Hkv,N,Dv] FP32 (src/nn/attention.rs:49-67)."""
    if len(query.dims()) != 4:
        raise InvalidTensor("grouped_query_attention takes rank-4 tensors")
    return _attention(query, key, value, scale, additive_mask, False, 0, 0)


def causal_grouped_query_attention_bf16_fp32(query: Tensor, key: Tensor, value: Tensor, scale: float, query_start: int,
                                             key_start: int) -> Tensor:
    """src/nn/attention.rs:69-80."""
    if len(query.dims()) != 4:
        raise InvalidTensor("causal_grouped_query_attention takes rank-4 tensors")
    return _attention(query, key, value, scale, None, True, query_start, key_start)


# -- matrices whose axes are not multiples of 16 (src/nn/padded.rs) ----------------------------------------------------
def matmul_padded_bf16_fp32(a: Tensor, b: Tensor, ta: Transpose = Transpose.No, tb: Transpose = Transpose.No) -> Tensor:
    """Positive M/N/K of any size, rank 2 or matching-batch rank 3, all four transposes; X/W rounded to BF16 on the device,
    FP32 result cropped to the logical shape (src/nn/padded.rs:21-27)."""
    c = _same_client(a, b)
    return _wrap(c, RT.gemm_padded_bf16_fp32(c, a.buffer, b.buffer, ta, tb)[0])


def linear_padded_bf16_fp32(input: Tensor, weight: Tensor) -> Tensor:
    """X[M,K] W[N,K]^T with explicit padding (src/nn/padded.rs:28-31)."""
    if len(input.dims()) != 2 or len(weight.dims()) != 2:
        raise InvalidTensor("padded GEMM requires matching rank-2/3 FP32/BF16 inputs")
    return matmul_padded_bf16_fp32(input, weight, Transpose.No, Transpose.Yes)


def linear_frozen_padded_bf16_fp32(input: Tensor, weight: Tensor) -> Tensor:
    """FP32 X times a fixed BF16 W^T of any positive size, FP32 result; the weight is neither copied (when aligned) nor
    written (src/nn/padded.rs:9-11, runtime/padded_matrix.rs:67-79)."""
    c = _same_client(input, weight)
    return _wrap(c, RT.linear_frozen_padded_bf16_fp32(c, input.buffer, weight.buffer)[0])


# -- embedding and the causal-LM loss edge (src/nn/embedding.rs, src/nn/frozen.rs, src/nn/causal_lm.rs) -----------------------
@dataclass
class EmbeddingOptions:
    """runtime::EmbeddingOptions (rust-ascend-driver/src/tensor/embedding.rs:5-8): both fields act on the derivative only."""
    padding_idx: int | None = None
    scale_grad_by_freq: bool = False


def embedding(weight: Tensor, indices: Tensor, options: EmbeddingOptions | None = None) -> Tensor:
    """FP32 weight [V,H] and INT32/INT64 ids of rank 1..7 give output ids.shape + [H] (src/nn/embedding.rs:14-33,35-45)."""
    options = options or EmbeddingOptions()
    c = _same_client(weight, indices)
    if not 1 <= len(indices.dims()) <= 7:
        raise InvalidTensor("embedding output rank must append one axis to rank 1..7 IDs")
    if weight.dtype() != DType.F32 or len(weight.dims()) != 2:
        raise InvalidTensor("RUDA embedding autodiff requires a rank-2 FP32 table")
    if options.padding_idx is not None and options.padding_idx >= weight.dims()[0]:
        raise InvalidTensor("embedding padding row is outside its table")
    return _wrap(c, RT.embedding(c, weight.buffer, indices.buffer))


def embedding_backward(grad: Tensor, indices: Tensor, num_weights: int, options: EmbeddingOptions | None = None) -> Tensor:
    """Dense weight gradient [V,H] that the reference's EmbeddingBackward registers (src/nn/embedding.rs:55-70)."""
    options = options or EmbeddingOptions()
    c = _same_client(grad, indices)
    return _wrap(c, RT.embedding_backward(c, grad.buffer, indices.buffer, num_weights, options.padding_idx, options.scale_grad_by_freq))


def embedding_frozen_bf16_fp32(weight: Tensor, indices: Tensor) -> Tensor:
    """Fixed BF16 table [V,H], ids of rank 1..7, FP32 activations; no table gradient (src/nn/frozen.rs:15-26)."""
    c = _same_client(weight, indices)
    if not 1 <= len(indices.dims()) <= 7:
        raise InvalidTensor("frozen embedding output rank must append one axis to rank 1..7 IDs")
    if weight.dtype() != DType.BF16 or len(weight.dims()) != 2:
        raise InvalidTensor("frozen BF16 embedding requires unquantized BF16 table")
    return _wrap(c, RT.cast(c, RT.embedding(c, weight.buffer, indices.buffer), DType.F32))


def layer_norm(input: Tensor, weight: Tensor, bias: Tensor | None, epsilon: float) -> Tensor:
    """Last-axis LayerNorm, missing bias = zeros (runtime/mod.rs:442-448)."""
    c = _same_client(input, weight, bias)
    return _wrap(c, RT.layer_norm(c, input.buffer, weight.buffer, None if bias is None else bias.buffer, epsilon)[0])


@dataclass
class CausalLoss:
    """Full-vocabulary FP32 loss sum and FP32 count of scored tokens (src/nn/causal_lm.rs:55-66)."""
    loss_sum: Tensor
    valid_tokens: Tensor

    def mean(self) -> Tensor:
        """loss_sum / max(valid_tokens, 1); ignored or empty windows have zero mean.  The two scalars are read back to form
        the quotient (the reference divides on the device)."""
        s = np.float32(self.loss_sum.into_data()[0]); n = np.float32(self.valid_tokens.into_data()[0])
        return Tensor.from_data(self.loss_sum.client, np.array([s / max(n, np.float32(1))], np.float32))


@dataclass
class CausalCrossEntropyConfig:
    """src/nn/causal_lm.rs:38-53.  `token_chunk_size` bounds the reference's per-launch logits; here the whole [B,T,V] block
    goes through one fused kernel, so the field is validated and otherwise unused."""
    token_chunk_size: int = 32
    ignore_index: int = -100
    shift: bool = True

    def forward_hidden(self, hidden: Tensor, labels: Tensor, project) -> CausalLoss:
        """hidden FP32 [B,T,H], labels INT32/INT64 [B,T]; `project` maps FP32 [rows,H] to FP32 logits [rows,V]
        (src/nn/causal_lm.rs:118-196).  With shift, position t is scored against label t+1 of the same sequence."""
        c = _same_client(hidden, labels)
        if len(hidden.dims()) != 3 or len(labels.dims()) != 2:
            raise InvalidTensor("causal loss requires matching [B,T,H]/[B,T], positive H and token chunk size")
        batch, time, width = hidden.dims()
        if self.token_chunk_size <= 0 or labels.dims() != [batch, time] or width == 0:
            raise InvalidTensor("causal loss requires matching [B,T,H]/[B,T], positive H and token chunk size")
        steps = max(time - 1, 0) if self.shift else time
        if batch * steps > 1 << 24:
            raise InvalidTensor("causal loss FP32 token count requires at most 2^24 logical tokens per call")
        if hidden.dtype() != DType.F32 or labels.dtype() not in (DType.I32, DType.I64):
            raise InvalidTensor("causal loss requires same-device FP32 hidden and I32/I64 labels")
        if batch * time == 0:
            zero = lambda: Tensor.from_data(c, np.zeros(1, np.float32))
            return CausalLoss(zero(), zero())
        logits = project(hidden.reshape((batch * time, width)))
        if len(logits.dims()) != 2 or logits.dims()[0] != batch * time or logits.dims()[1] == 0 or logits.dtype() != DType.F32:
            raise InvalidTensor("causal projection must return FP32 [tokens,V] with positive V")
        loss, valid, _ = RT.causal_cross_entropy(c, logits.buffer.reshape((batch, time, logits.dims()[1])), labels.buffer, self.ignore_index,
                                                 self.shift, 1.0, with_gradient=False)
        return CausalLoss(_wrap(c, loss), _wrap(c, valid))


# -- bias / residual (src/nn/affine.rs) and fixed BF16 weights (src/nn/frozen.rs) ---------------------------------------
def bias_add(input: Tensor, bias: Tensor) -> Tensor:
    """X[...,H] + bias[H], contiguous FP32 of rank 1..8 (src/nn/affine.rs:14-19)."""
    c = _same_client(input, bias)
    return _wrap(c, RT.bias_add(c, input.buffer, bias.buffer))


def residual_bias_add(input: Tensor, residual: Tensor, bias: Tensor) -> Tensor:
    """(X + residual) + bias in that FP32 order; the residual must match X exactly (src/nn/affine.rs:20-25)."""
    c = _same_client(input, residual, bias)
    return _wrap(c, RT.bias_add(c, input.buffer, bias.buffer, residual.buffer))


def linear_frozen_bf16_fp32(input: Tensor, weight: Tensor) -> Tensor:
    """FP32 X [M,K] times a fixed BF16-stored W [N,K]^T, FP32 result; the weight is used in place (src/nn/frozen.rs:44-59)."""
    c = _same_client(input, weight)
    return _wrap(c, RT.linear_frozen_bf16_fp32(c, input.buffer, weight.buffer))


def swiglu_frozen_bf16_fp32(input: Tensor, gate: Tensor, up: Tensor, down: Tensor) -> Tensor:
    """SwiGLU with fixed BF16-stored gate/up [H,K] and down [N,H] and FP32 activations (src/nn/frozen.rs:95-107).  Gate and up
    run as one tensor-core GEMM whose epilogue applies SiLU*up on the FP32 accumulators; the hidden activation is FP32."""
    c = _same_client(input, gate, up, down)
    m, k = input.dims()
    hidden, gk = gate.dims()
    n, dh = down.dims()
    if gk != k or up.dims() != [hidden, k] or dh != hidden or any(s == 0 or s % 16 for s in (m, n, k, hidden)):
        raise InvalidTensor("frozen BF16 SwiGLU requires aligned X[M,K], gate/up[H,K], down[N,H]")
    if input.dtype() != DType.F32 or any(w.dtype() != DType.BF16 for w in (gate, up, down)):
        raise InvalidTensor("frozen BF16 SwiGLU requires FP32 input and fixed BF16 weights on the same device")
    x16 = RT.cast(c, input.buffer, DType.BF16)
    h = RT.gemm(c, x16, gate.buffer, Transpose.No, Transpose.Yes, DType.F32, b_up=up.buffer)
    return _wrap(c, RT.linear_frozen_bf16_fp32(c, h, down.buffer))


# -- attention on logical shapes of any size (src/nn/padded_attention.rs) ------------------------------------------------
def _padded_dimensions(query, key, value, scale):
    batch, m, d = query
    kb, n, kd = key
    vb, vn, _ = value
    if kb != batch or vb != batch or kd != d or vn != n or not np.isfinite(scale) or batch * m * n > 0xFFFFFFFF:
        raise InvalidTensor("padded attention requires matching batches/contractions, finite scale and logical scores within u32")
    if min(batch, m, n, d, value[2]) <= 0:
        raise InvalidTensor("padded GEMM matrix axes must be positive")


def scaled_dot_product_attention_padded_bf16_fp32(query: Tensor, key: Tensor, value: Tensor, scale: float,
                                                  additive_mask: Tensor | None = None) -> Tensor:
    """Materialised attention on FP32 Q[B,M,D], K[B,N,D], V[B,N,Dv] with positive axes of any size: each BF16 GEMM pads and
    crops explicitly, softmax and mask see only the logical keys (src/nn/padded_attention.rs:26-45).  The optional additive
    mask is exactly FP32 [B,M,N]."""
    c = _same_client(query, key, value, additive_mask)
    if any(len(t.dims()) != 3 for t in (query, key, value)):
        raise InvalidTensor("padded attention requires matching batches/contractions, finite scale and logical scores within u32")
    _padded_dimensions(query.dims(), key.dims(), value.dims(), scale)
    if any(t.dtype() != DType.F32 for t in (query, key, value)):
        raise InvalidTensor("padded attention requires FP32 Q/K/V on the same device")
    batch, m, _ = query.dims()
    n = key.dims()[1]
    if additive_mask is not None and (additive_mask.dims() != [batch, m, n] or additive_mask.dtype() != DType.F32):
        raise InvalidTensor("padded attention mask must be same-device FP32[B,M,N] without broadcasting")
    if scale == 0.0:
        raise InvalidTensor("padded attention needs a non-zero scale")
    scores = RT.gemm_padded_bf16_fp32(c, query.buffer, key.buffer, Transpose.No, Transpose.Yes)[0]
    RT.scale_in_place(c, scores, scale)
    if additive_mask is not None:
        RT.add(c, scores, additive_mask.buffer, out=scores)
    return _wrap(c, RT.gemm_padded_bf16_fp32(c, RT.softmax(c, scores), value.buffer, Transpose.No, Transpose.No)[0])


def causal_attention_padded_bf16_fp32(query: Tensor, key: Tensor, value: Tensor, scale: float, query_start: int, key_start: int) -> Tensor:
    """The same with the fixed exact-position causal mask; the starts are explicit (src/nn/padded_attention.rs:46-54)."""
    c = _same_client(query, key, value)
    if any(len(t.dims()) != 3 for t in (query, key, value)):
        raise InvalidTensor("padded attention requires matching batches/contractions, finite scale and logical scores within u32")
    _padded_dimensions(query.dims(), key.dims(), value.dims(), scale)
    batch, m, _ = query.dims()
    mask = causal_mask(c, (batch, m, key.dims()[1]), query_start, key_start)
    return scaled_dot_product_attention_padded_bf16_fp32(query, key, value, scale, mask)


def grouped_query_attention_padded_bf16_fp32(query: Tensor, key: Tensor, value: Tensor, scale: float, additive_mask: Tensor | None = None) -> Tensor:
    """Q[B,Hq,M,D], K[B,Hkv,N,D], V[B,Hkv,N,Dv] of any positive sizes: KV heads repeated on the device, then the padded
    materialised path; the optional mask is exactly FP32 [B,Hq,M,N] (src/nn/padded_attention.rs:55-92)."""
    c = _same_client(query, key, value, additive_mask)
    if any(len(t.dims()) != 4 for t in (query, key, value)):
        raise InvalidTensor("padded GQA requires matching batches/KV shapes and positive divisible Q/KV heads")
    batch, heads, m, d = query.dims()
    kb, kv_heads, n, kd = key.dims()
    vb, vh, vn, dv = value.dims()
    if heads == 0 or kv_heads == 0 or heads % kv_heads or kb != batch or vb != batch or vh != kv_heads or vn != n or kd != d:
        raise InvalidTensor("padded GQA requires matching batches/KV shapes and positive divisible Q/KV heads")
    flat = batch * heads
    if additive_mask is not None and (additive_mask.dims() != [batch, heads, m, n] or additive_mask.dtype() != DType.F32):
        raise InvalidTensor("padded GQA additive mask must be FP32 [B,Hq,M,N] on the same device")
    k = repeat_kv_heads(key, heads).reshape((flat, n, d))
    v = repeat_kv_heads(value, heads).reshape((flat, n, dv))
    out = scaled_dot_product_attention_padded_bf16_fp32(query.reshape((flat, m, d)), k, v, scale,
                                                        None if additive_mask is None else additive_mask.reshape((flat, m, n)))
    return out.reshape((batch, heads, m, dv))


def causal_grouped_query_attention_padded_bf16_fp32(query: Tensor, key: Tensor, value: Tensor, scale: float, query_start: int, key_start: int) -> Tensor:
    """Padded GQA with the exact-position causal mask (src/nn/padded_attention.rs:93-104)."""
    c = _same_client(query, key, value)
    if len(query.dims()) != 4 or len(key.dims()) != 4:
        raise InvalidTensor("padded GQA requires matching batches/KV shapes and positive divisible Q/KV heads")
    batch, heads, m, _ = query.dims()
    n = key.dims()[2]
    mask = causal_mask(c, (batch * heads, m, n), query_start, key_start).reshape((batch, heads, m, n))
    return grouped_query_attention_padded_bf16_fp32(query, key, value, scale, mask)
