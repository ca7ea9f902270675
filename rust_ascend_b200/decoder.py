"""Llama-style decoder stack on the B200 operators, tensor-parallel over NCCL.

The reference has no tensor parallelism (README.md:92-106: data parallel plus collective primitives only) and
its Llama model lives in the external RUDA crates, so this composition is new: the standard pre-norm block
(RMSNorm -> QKV -> causal GQA attention with RoPE -> O -> residual; RMSNorm -> SwiGLU -> down -> residual)
assembled from the operators this package provides, sharded Megatron-style:

  column-parallel  Wq/Wk/Wv (packed into one [q_shard; k_shard; v_shard] weight) and Wgate/Wup: rows of [N,K] split
  row-parallel     Wo and Wdown: K split, followed by ONE all-reduce(sum) of the [T, hidden] partial results
  heads            Hq/tp query heads and Hkv/tp KV heads per rank; attention needs no communication
  replicated       embedding lookup, RMSNorm, residual adds;  LM head is vocab-parallel (logits stay sharded)

Activations are BF16 [T, width] row-major; the QKV projection output is consumed by the attention kernel in
place through strides ([B,S,H,D] storage viewed as [B,H,S,D]) and attention writes [B,S,H,D] so the output
projection needs no transpose either.  `chunks > 1` splits T into row chunks so that the all-reduce of chunk i
overlaps the GEMM of chunk i+1 (deferred fences on the communicator's own stream).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .runtime import B200Runtime as RT
from .runtime import ComputeClient, DType, InvalidTensor, RotaryLayout, TensorBuffer, Transpose, f32_to_bf16_bits


@dataclass
class LlamaConfig:
    layers: int = 8
    hidden: int = 4096
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 32000
    eps: float = 1e-5
    theta: float = 500000.0

    def flops(self, tokens: int, seq: int) -> int:
        """Algorithmic forward flops: projections + causal-half attention + LM head."""
        qkv = 2 * tokens * self.hidden * (self.heads + 2 * self.kv_heads) * self.head_dim
        o = 2 * tokens * self.heads * self.head_dim * self.hidden
        ffn = 3 * 2 * tokens * self.hidden * self.ffn
        attn = 2 * tokens * seq * self.heads * self.head_dim  # 4*T*S*H*D halved by the causal mask
        return self.layers * (qkv + o + ffn + attn) + 2 * tokens * self.hidden * self.vocab


def shard_plan(cfg: LlamaConfig, rank: int, world: int) -> dict:
    """Row/column ranges each rank owns.  Pure function: shared by the GPU path and the CPU sharding tests."""
    if cfg.heads % world or cfg.kv_heads % world or cfg.ffn % world or cfg.vocab % world:
        raise InvalidTensor("heads, kv_heads, ffn and vocab must divide by the tensor-parallel world size")
    if cfg.heads % cfg.kv_heads:
        raise InvalidTensor("query heads must be a multiple of KV heads")
    hq, hkv, f, v = cfg.heads // world, cfg.kv_heads // world, cfg.ffn // world, cfg.vocab // world
    d = cfg.head_dim
    return {
        "q_heads": hq, "kv_heads": hkv,
        "q_rows": (rank * hq * d, (rank + 1) * hq * d),          # rows of Wq [Hq*D, hidden]
        "kv_rows": (rank * hkv * d, (rank + 1) * hkv * d),       # rows of Wk / Wv [Hkv*D, hidden]
        "o_cols": (rank * hq * d, (rank + 1) * hq * d),          # columns (K) of Wo [hidden, Hq*D]
        "ffn_rows": (rank * f, (rank + 1) * f),                  # rows of Wgate / Wup [ffn, hidden]
        "down_cols": (rank * f, (rank + 1) * f),                 # columns (K) of Wdown [hidden, ffn]
        "vocab_rows": (rank * v, (rank + 1) * v),                # rows of the LM head [vocab, hidden]
    }


def rope_tables(positions: int, head_dim: int, theta: float):
    """cos/sin FP32 [positions, head_dim/2]: inv_freq_i = theta^(-2i/head_dim), angle = pos * inv_freq_i in f64."""
    inv = theta ** (-np.arange(head_dim // 2, dtype=np.float64) * 2.0 / head_dim)
    ang = np.arange(positions, dtype=np.float64)[:, None] * inv[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


class WeightSource:
    """Seeded N(0, 0.02) BF16 weights.  `exact=True` draws every full matrix from its own seed so that any shard of
    it is identical on every rank and for every world size (parity tests); `exact=False` tiles one random block,
    which is enough for timing and avoids drawing billions of normals on the host."""

    def __init__(self, seed: int, exact: bool):
        self.seed, self.exact = seed, exact
        self._block = None

    def matrix(self, name: str, layer: int, rows: int, cols: int, row_range=None, col_range=None) -> np.ndarray:
        r0, r1 = row_range or (0, rows)
        c0, c1 = col_range or (0, cols)
        if self.exact:
            rng = np.random.default_rng([self.seed, layer, sum(ord(ch) for ch in name), len(name)])
            full = rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(0.02)
            return f32_to_bf16_bits(full[r0:r1, c0:c1])
        if self._block is None:
            rng = np.random.default_rng(self.seed)
            self._block = f32_to_bf16_bits(rng.standard_normal(1 << 24, dtype=np.float32) * np.float32(0.02))
        n = (r1 - r0) * (c1 - c0)
        reps = -(-n // self._block.size)
        start = (layer * 7919 + len(name) * 104729) % 4096
        return np.resize(np.roll(self._block, start), n if reps == 1 else n).reshape(r1 - r0, c1 - c0)


class TensorParallelDecoder:
    def __init__(self, client: ComputeClient, cfg: LlamaConfig, batch: int, seq: int, comm=None, rank: int = 0, world: int = 1,
                 seed: int = 0, exact_weights: bool = False, chunks: int = 1):
        if world > 1 and comm is None:
            raise InvalidTensor("a communicator is required for tensor parallelism")
        if cfg.head_dim != 128:
            raise InvalidTensor("the tensor-core attention kernel needs head_dim 128")
        self.client, self.cfg, self.comm, self.rank, self.world = client, cfg, comm, rank, world
        self.batch, self.seq, self.tokens = batch, seq, batch * seq
        if self.tokens % 16 or seq % 32:
            raise InvalidTensor("batch*seq must be a multiple of 16 and seq a multiple of 32")
        self.chunks = chunks if world > 1 else 1
        if self.tokens % (self.chunks * 128):
            raise InvalidTensor("row chunks must be multiples of 128 tokens")
        self.plan = p = shard_plan(cfg, rank, world)
        src = WeightSource(seed, exact_weights)
        up = lambda a: client.upload(np.ascontiguousarray(a), DType.BF16)
        h, d = cfg.hidden, cfg.head_dim
        self.embedding = up(src.matrix("embedding", 0, cfg.vocab, h))
        self.lm_head = up(src.matrix("lm_head", 0, cfg.vocab, h, row_range=p["vocab_rows"]))
        ones = f32_to_bf16_bits(np.ones(h, np.float32))
        self.final_norm = up(ones)
        self.layers = []
        for li in range(cfg.layers):
            wq = src.matrix("wq", li, cfg.heads * d, h, row_range=p["q_rows"])
            wk = src.matrix("wk", li, cfg.kv_heads * d, h, row_range=p["kv_rows"])
            wv = src.matrix("wv", li, cfg.kv_heads * d, h, row_range=p["kv_rows"])
            self.layers.append({
                "norm1": up(ones), "norm2": up(ones),
                "wqkv": up(np.concatenate([wq, wk, wv], axis=0)),
                "wo": up(src.matrix("wo", li, h, cfg.heads * d, col_range=p["o_cols"])),
                "wg": up(src.matrix("wg", li, cfg.ffn, h, row_range=p["ffn_rows"])),
                "wu": up(src.matrix("wu", li, cfg.ffn, h, row_range=p["ffn_rows"])),
                "wd": up(src.matrix("wd", li, h, cfg.ffn, col_range=p["down_cols"])),
            })
        cos, sin = rope_tables(seq, d, cfg.theta)
        self.cos, self.sin = client.upload(cos), client.upload(sin)
        # activation buffers, allocated once
        t, hq, hkv, f = self.tokens, p["q_heads"], p["kv_heads"], cfg.ffn // world
        self.qkv_width = (hq + 2 * hkv) * d
        T = lambda *shape: client.tensor(shape, DType.BF16)
        self.x, self.h, self.qkv, self.attn = T(t, h), T(t, h), T(t, self.qkv_width), T(batch, seq, hq, d)
        self.proj, self.ffn_act = T(t, h), T(t, f)
        self.logits = T(t, cfg.vocab // world)
        self.tokens_dev = client.tensor((batch, seq), DType.I32)
        self.scale = 1.0 / float(np.sqrt(d))
        self.launches_per_forward = None

    # -- views into the packed QKV buffer: [B,S,H,D] storage presented as [B,H,S,D] -------------------------
    def _head_view(self, first_head: int, heads: int) -> TensorBuffer:
        d, w, s = self.cfg.head_dim, self.qkv_width, self.seq
        return TensorBuffer(self.qkv.handle, (self.batch, heads, s, d), DType.BF16, (s * w, d, w, 1), offset=first_head * d * 2)

    def _rows(self, t: TensorBuffer, chunk: int) -> TensorBuffer:
        rows = self.tokens // self.chunks
        width = t.elements // self.tokens
        return TensorBuffer(t.handle, (rows, width), t.dtype, None, offset=t.offset + chunk * rows * width * t.dtype.size)

    def _row_parallel(self, inp: TensorBuffer, weight: TensorBuffer) -> None:
        """proj = inp @ weight^T summed over ranks, chunked so the all-reduce overlaps the next chunk's GEMM."""
        c = self.client
        inp2 = inp.reshape((self.tokens, inp.elements // self.tokens))
        for ch in range(self.chunks):
            out = self._rows(self.proj, ch)
            RT.gemm_into(c, self._rows(inp2, ch), weight, Transpose.No, Transpose.Yes, out)
            if self.world > 1:
                self.comm.native.all_reduce(out, "sum", out=out, deferred=self.chunks > 1)
        if self.world > 1 and self.chunks > 1:
            self.comm.native.fence()

    def forward(self, tokens: np.ndarray | None = None) -> TensorBuffer:
        """Returns this rank's logits shard [T, vocab/world] (BF16).  `tokens` int32 [B,S]; None reuses the last upload."""
        c, cfg, p = self.client, self.cfg, self.plan
        if tokens is not None:
            c.write(self.tokens_dev.handle, np.ascontiguousarray(tokens, dtype=np.int32))
            c.sync()
        before = c.stats()["launches"]
        hq, hkv = p["q_heads"], p["kv_heads"]
        import ctypes as C
        from .runtime import _check, _ref
        _check(c._lib.rb_embedding(c._ctx, _ref(self.embedding), _ref(self.tokens_dev), _ref(self.x.reshape((self.batch, self.seq, cfg.hidden)))))
        q, k, v = self._head_view(0, hq), self._head_view(hq, hkv), self._head_view(hq + hkv, hkv)
        for lw in self.layers:
            _check(c._lib.rb_rms_norm(c._ctx, _ref(self.x), _ref(lw["norm1"]), C.c_double(cfg.eps), _ref(self.h), None))
            RT.gemm_into(c, self.h, lw["wqkv"], Transpose.No, Transpose.Yes, self.qkv)
            RT.attention(c, q, k, v, self.scale, causal=True, cos=self.cos, sin=self.sin, rotary_layout=RotaryLayout.SplitHalf,
                         bmhd_output=True, out=self.attn)
            self._row_parallel(self.attn, lw["wo"])
            RT.add(c, self.x, self.proj, out=self.x)
            _check(c._lib.rb_rms_norm(c._ctx, _ref(self.x), _ref(lw["norm2"]), C.c_double(cfg.eps), _ref(self.h), None))
            RT.gemm_into(c, self.h, lw["wg"], Transpose.No, Transpose.Yes, self.ffn_act, b_up=lw["wu"])
            self._row_parallel(self.ffn_act, lw["wd"])
            RT.add(c, self.x, self.proj, out=self.x)
        _check(c._lib.rb_rms_norm(c._ctx, _ref(self.x), _ref(self.final_norm), C.c_double(cfg.eps), _ref(self.h), None))
        RT.gemm_into(c, self.h, self.lm_head, Transpose.No, Transpose.Yes, self.logits)
        self.launches_per_forward = c.stats()["launches"] - before
        return self.logits
