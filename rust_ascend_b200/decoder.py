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
projection needs no transpose either.  `micro_batches > 1` splits the batch into groups of sequences so that the
all-reduce of one group overlaps the GEMMs of the other (deferred fences on the communicator's own stream).

`fused=True` replaces the two all-reduces of a layer by the fused exchange of fused.py: the row-parallel GEMMs scatter
their partial rows into the staging area of the rank that owns those rows, the owner sums them, updates its rows of the
residual stream (which is then sharded by rows), normalises and pushes the result into every rank's activation buffer;
`overlap_exchange=True` moves the owner-side step to a side stream under the other micro batch's GEMMs.
`pull_exchange=True` keeps the row-parallel GEMMs plain (each rank writes its partial product locally and announces it) and
lets the owner-side step fetch the partial products itself, so that all link traffic is on the side stream.
`side_scatter=True` keeps the GEMMs plain and scatters their rows to the owners with a kernel of its own (posted stores), on
the side stream when the exchange is overlapped.
`dma_exchange=True` moves the data of the exchange with device-to-device copies (copy engines) and keeps only the owner-side
arithmetic as a kernel, so that the exchange costs the GEMMs beside it no SMs.
"""
from __future__ import annotations

import ctypes as C
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


def fused_schedule(layers: int, micro_batches: int, overlap: bool = False):
    """Order of one forward's steps in fused mode (exchange folded into the kernels, residual stream sharded by rows).
    Pure function: the launch plan is emitted from it and the CPU protocol model replays it.  Steps:
    ("embed", mb) | ("wait_scatter", mb) | ("push", mb, layer, which) | ("wait_gather", mb) | ("attention_block", mb, layer) |
    ("ffn_block", mb, layer) | ("scatter", mb, layer, "wo" or "wd") | ("lm_head", mb) | ("barrier",) and, with `overlap`,
    ("aux_begin", mb) | ("aux_end", mb) | ("aux_wait", mb).
    A push reduces the staged partials of the scatter before it (none for the very first), so its wait comes first; the
    closing barrier keeps a fast rank's next forward from storing into buffers that a slow rank is still reading.
    With `overlap` the exchange that follows a scatter (wait, push, wait) is forked to the side stream right behind the
    scatter and joined just before the micro batch's next block, so that it runs under the other micro batches' GEMMs."""
    steps = [("embed", mb) for mb in range(micro_batches)]
    if not overlap:
        pending = [False] * micro_batches
        for layer in range(layers + 1):
            for mb in range(micro_batches):
                if pending[mb]:
                    steps.append(("wait_scatter", mb))
                steps += [("push", mb, layer, 0), ("wait_gather", mb)]
                if layer == layers:
                    steps.append(("lm_head", mb))
                    continue
                steps += [("attention_block", mb, layer), ("scatter", mb, layer, "wo")]
                pending[mb] = True
            if layer == layers:
                break
            for mb in range(micro_batches):
                steps += [("wait_scatter", mb), ("push", mb, layer, 1), ("wait_gather", mb), ("ffn_block", mb, layer), ("scatter", mb, layer, "wd")]
        steps.append(("barrier",))
        return steps

    def exchange(mb, layer, which):
        return [("aux_begin", mb), ("wait_scatter", mb), ("push", mb, layer, which), ("wait_gather", mb), ("aux_end", mb)]
    for layer in range(layers + 1):
        for mb in range(micro_batches):
            steps += [("push", mb, 0, 0), ("wait_gather", mb)] if layer == 0 else [("aux_wait", mb)]
            if layer == layers:
                steps.append(("lm_head", mb))
                continue
            steps += [("attention_block", mb, layer), ("scatter", mb, layer, "wo")] + exchange(mb, layer, 1)
        if layer == layers:
            break
        for mb in range(micro_batches):
            steps += [("aux_wait", mb), ("ffn_block", mb, layer), ("scatter", mb, layer, "wd")] + exchange(mb, layer + 1, 0)
    steps.append(("barrier",))
    return steps


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
    """Builds the weights, the activation buffers and a flat launch plan once; `forward` replays the plan (or the CUDA
    graph recorded from it).

    micro_batches > 1 splits the batch into groups of sequences that walk through the layers in lock step: while one
    group computes, the all-reduce of the other group's row-parallel projection is in flight on the communicator's
    stream.  `sm_reserve` SMs are then kept free of the persistent GEMM so that the collective can run beside it."""

    def __init__(self, client: ComputeClient, cfg: LlamaConfig, batch: int, seq: int, comm=None, rank: int = 0, world: int = 1,
                 seed: int = 0, exact_weights: bool = False, micro_batches: int = 1, sm_reserve: int = 0, use_graph: bool = False,
                 fused: bool = False, overlap_exchange: bool = False, pull_exchange: bool = False, dma_exchange: bool = False,
                 side_scatter: bool = False):
        if world > 1 and comm is None:
            raise InvalidTensor("a communicator is required for tensor parallelism")
        if cfg.head_dim != 128:
            raise InvalidTensor("the tensor-core attention kernel needs head_dim 128")
        self.client, self.cfg, self.comm, self.rank, self.world = client, cfg, comm, rank, world
        self.batch, self.seq, self.tokens = batch, seq, batch * seq
        if self.tokens % 16 or seq % 32:
            raise InvalidTensor("batch*seq must be a multiple of 16 and seq a multiple of 32")
        self.plan = shard_plan(cfg, rank, world)
        p = self.plan
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
        # activation buffers, allocated once; micro batches are row ranges of them
        t, hq, hkv, f = self.tokens, p["q_heads"], p["kv_heads"], cfg.ffn // world
        self.qkv_width = (hq + 2 * hkv) * d
        T = lambda *shape: client.tensor(shape, DType.BF16)
        self.x, self.h, self.qkv, self.attn = T(t, h), T(t, h), T(t, self.qkv_width), T(t, hq * d)
        self.proj, self.ffn_act = T(t, h), T(t, f)
        self.logits = T(t, cfg.vocab // world)
        self.tokens_dev = client.tensor((batch, seq), DType.I32)
        self.scale = 1.0 / float(np.sqrt(d))
        self._graph = None
        self._exchanges, self._peer_h, self._x_own = [], None, None
        self.configure(comm, micro_batches, sm_reserve, use_graph, fused, overlap_exchange, pull_exchange, dma_exchange, side_scatter)

    def configure(self, comm, micro_batches: int = 1, sm_reserve: int = 0, use_graph: bool = False, fused: bool = False,
                  overlap_exchange: bool = False, pull_exchange: bool = False, dma_exchange: bool = False, side_scatter: bool = False) -> None:
        """(Re)builds the launch plan, and the recorded graph if asked for, on the weights and buffers already resident.
        Lets a caller compare schedules (micro batches, SMs left to NCCL, communicators with different CTA limits)
        without loading the model again."""
        from .runtime import _check
        client = self.client
        if self.batch % micro_batches or (self.batch // micro_batches * self.seq) % 16:
            raise InvalidTensor("micro batches must hold whole sequences")
        if fused and (comm is None or not hasattr(comm, "control") or (self.tokens // micro_batches) % (128 * self.world) or self.cfg.hidden % 64):
            raise InvalidTensor("fused exchange needs a communicator with a control plane and micro batches of a multiple of 128 * world tokens")
        self.close()
        self.comm, self.micro, self.fused, self.overlap_exchange = comm, micro_batches, fused, bool(fused and overlap_exchange)
        self.dma_exchange = bool(fused and dma_exchange)
        self.side_scatter = bool(fused and side_scatter and not pull_exchange and not dma_exchange)
        self.pull_exchange = bool(fused and pull_exchange) or self.dma_exchange     # both keep the row-parallel GEMMs plain
        self._keep = []          # ctypes structures referenced by the plan
        self._steps = []         # (function, argument tuple)
        self.launches_per_forward = 0
        self.collectives_per_forward = 0
        self.fused_exchanges_per_forward = 0     # scatter-GEMM + owner-side reduce pairs that stand where all-reduces stood
        sms = client.properties()["sm_count"]
        _check(client._lib.rb_set_sm_limit(client._ctx, C.c_int32(sms - sm_reserve if sm_reserve else 0)))
        if fused:
            self._build_fused_plan()
        else:
            self._build_plan()
        if use_graph:
            self._run_plan()                     # first use of every kernel and every workspace size happens outside the recording
            client.sync()
            _check(client._lib.rb_graph_begin(client._ctx))
            try:
                self._run_plan()
            finally:
                g = C.c_uint64()
                _check(client._lib.rb_graph_end(client._ctx, C.byref(g)))
            self._graph = g

    # -- plan construction ------------------------------------------------------------------------------------
    def _t(self, t: TensorBuffer | None):
        if t is None:
            return None
        c = t._c()
        self._keep.append(c)
        return C.byref(c)

    def _rows(self, t: TensorBuffer, mb: int) -> TensorBuffer:
        rows = self.tokens // self.micro
        width = t.elements // self.tokens
        return TensorBuffer(t.handle, (rows, width), t.dtype, None, offset=t.offset + mb * rows * width * t.dtype.size)

    def _head_view(self, mb: int, first_head: int, heads: int) -> TensorBuffer:
        """[B,S,H,D] storage of the packed QKV projection presented as [B,H,S,D]."""
        d, w, s = self.cfg.head_dim, self.qkv_width, self.seq
        b = self.batch // self.micro
        return TensorBuffer(self.qkv.handle, (b, heads, s, d), DType.BF16, (s * w, d, w, 1), offset=(mb * b * s * w + first_head * d) * 2)

    def _op(self, name: str, *args, kernel: bool = True):
        self._steps.append((getattr(self.client._lib, name), args))
        if kernel:
            self.launches_per_forward += 1

    def _gemm(self, a, w, out, b_up=None):
        self._op("rb_gemm", self.client._ctx, self._t(a), self._t(w), C.c_int32(0), C.c_int32(1), None, self._t(b_up),
                 C.c_int32(2 if b_up is not None else 0), self._t(out))

    def _build_plan(self):
        cfg, p, c, ctx = self.cfg, self.plan, self.client, self.client._ctx
        hq, hkv, n = p["q_heads"], p["kv_heads"], self.micro
        b = self.batch // n
        eps = C.c_double(cfg.eps)
        comm = self.comm.native._comm if self.world > 1 else None
        self._op("rb_embedding", ctx, self._t(self.embedding), self._t(self.tokens_dev), self._t(self.x.reshape((self.batch, self.seq, cfg.hidden))))
        pending = [False] * n     # a deferred all-reduce of proj[mb] is in flight
        tickets = [0] * n

        def wait(mb):
            if pending[mb]:
                self._op("rb_comm_wait_ticket", comm, C.c_uint64(tickets[mb]), kernel=False)
                pending[mb] = False

        def reduce(mb, view):
            if self.world > 1:
                self._op("rb_all_reduce", comm, self._t(view), C.c_int32(0), self._t(view), C.c_int32(1))
                self.collectives_per_forward += 1
                self._issued += 1
                tickets[mb], pending[mb] = self._issued, True

        self._issued = 0
        first = True
        for lw in self.layers + [None]:
            norm_w = self.final_norm if lw is None else lw["norm1"]
            for mb in range(n):
                x, h, proj = self._rows(self.x, mb), self._rows(self.h, mb), self._rows(self.proj, mb)
                wait(mb)
                if first:
                    self._op("rb_rms_norm", ctx, self._t(x), self._t(norm_w), eps, self._t(h), None)
                else:  # residual of the previous layer's FFN fused into this norm
                    self._op("rb_add_rms_norm", ctx, self._t(x), self._t(proj), self._t(norm_w), eps, self._t(x), self._t(h))
                if lw is None:
                    self._gemm(h, self.lm_head, self._rows(self.logits, mb))
                    continue
                self._gemm(h, lw["wqkv"], self._rows(self.qkv, mb))
                q, k, v = self._head_view(mb, 0, hq), self._head_view(mb, hq, hkv), self._head_view(mb, hq + hkv, hkv)
                attn = self._rows(self.attn, mb)
                self._op("rb_attention", ctx, self._t(q), self._t(k), self._t(v), None, C.c_float(self.scale), C.c_int32(1), C.c_uint64(0), C.c_uint64(0),
                         self._t(self.cos), self._t(self.sin), C.c_int32(int(RotaryLayout.SplitHalf)), C.c_int32(1), self._t(attn.reshape((b, self.seq, hq, cfg.head_dim))))
                self.launches_per_forward += 2   # the Q and K rotations run as two small kernels inside rb_attention
                self._gemm(attn, lw["wo"], proj)
                reduce(mb, proj)
            if lw is None:
                break
            first = False
            for mb in range(n):
                x, h, proj, act = self._rows(self.x, mb), self._rows(self.h, mb), self._rows(self.proj, mb), self._rows(self.ffn_act, mb)
                wait(mb)
                self._op("rb_add_rms_norm", ctx, self._t(x), self._t(proj), self._t(lw["norm2"]), eps, self._t(x), self._t(h))
                self._gemm(h, lw["wg"], act, b_up=lw["wu"])
                self._gemm(act, lw["wd"], proj)
                reduce(mb, proj)

    # -- fused mode: the exchange lives inside the kernels, the residual stream is sharded by rows ------------------
    def _release_fused(self) -> None:
        """Collective: every rank of the group drops its exchange buffers in the same order."""
        for ex in self._exchanges:
            ex.close()
        if self._peer_h is not None:
            self._peer_h.close()
        if self._x_own is not None:
            self.client.free(self._x_own.handle)
        self._exchanges, self._peer_h, self._x_own = [], None, None

    def _build_fused_plan(self):
        from .fused import BARRIER, GATHER, SCATTER, FusedExchange, PeerBuffer
        cfg, p, c, ctx = self.cfg, self.plan, self.client, self.client._ctx
        hq, hkv, n = p["q_heads"], p["kv_heads"], self.micro
        b, hidden = self.batch // n, cfg.hidden
        tm = self.tokens // n                      # tokens of one micro batch
        rows = tm // self.world                    # rows of it this rank owns
        control = self.comm.control
        self._peer_h = PeerBuffer(c, control, self.tokens * hidden * 2)
        self._exchanges = [FusedExchange(c, control, tm, hidden, activations=self._peer_h, activation_offset=mb * tm * hidden * 2, pull=self.pull_exchange, dma=self.dma_exchange, side_scatter=self.side_scatter)
                           for mb in range(n)]
        self._x_own = c.tensor((n, rows, hidden), DType.BF16)
        eps = cfg.eps
        keep = self._keep

        def x_own(mb):
            return TensorBuffer(self._x_own.handle, (rows, hidden), DType.BF16, None, offset=mb * rows * hidden * 2)

        rows_pushed_by_copy = [False] * n        # copy form: the micro batch's last owner-side step left its rows with the owners
        for step in fused_schedule(cfg.layers, n, self.overlap_exchange):
            kind = step[0]
            if kind in ("aux_begin", "aux_end", "aux_wait"):   # fork to / join from the side stream; the slot is the micro batch
                self._op("rb_" + kind, ctx, *(() if kind == "aux_begin" else (C.c_uint32(step[1]),)), kernel=False)
                continue
            if kind == "barrier":
                ex = self._exchanges[0]
                self._op("rb_peer_signal", *ex.signal_args(keep))
                self._op("rb_peer_wait", *ex.wait_args(BARRIER, 1, keep))
                continue
            mb = step[1]
            ex = self._exchanges[mb]
            h = ex.gathered()
            if kind == "embed":
                first = mb * tm + self.rank * rows          # this rank's rows of the micro batch, as flat token positions
                ids = TensorBuffer(self.tokens_dev.handle, (rows,), DType.I32, None, offset=first * 4)
                self._op("rb_embedding", ctx, self._t(self.embedding), self._t(ids), self._t(x_own(mb)))
            elif kind == "wait_scatter":
                if self.side_scatter:        # the transfer of the GEMM's rows starts here: on the side stream when the exchange is forked
                    self._op("rb_scatter_rows", *ex.scatter_rows_args(keep))
                self._op("rb_peer_wait", *ex.wait_args(SCATTER, ex.scatter_count, keep))
            elif kind == "wait_gather":
                self._op("rb_peer_wait", *ex.wait_args(GATHER, 1, keep))
                if self.dma_exchange and rows_pushed_by_copy[mb]:      # the owners announced their rows: fetch them
                    for name, args in ex.dma_gather_calls(keep):
                        self._op(name, *args, kernel=False)
            elif kind == "push":
                _, _, layer, which = step
                lw = self.layers[layer] if layer < cfg.layers else None
                weight = self.final_norm if lw is None else (lw["norm1"] if which == 0 else lw["norm2"])
                very_first = layer == 0 and which == 0     # nothing staged yet: normalise the embedding rows
                rows_pushed_by_copy[mb] = self.dma_exchange and not very_first
                if self.dma_exchange and not very_first:
                    for name, args in ex.dma_reduce_calls(x_own(mb), weight, eps, x_own(mb), keep):
                        self._op(name, *args, kernel=name != "rb_copy")
                elif self.pull_exchange and not very_first:
                    self._op("rb_reduce_norm_push_pull", *ex.pull_args(x_own(mb), weight, eps, x_own(mb), keep))
                else:
                    self._op("rb_reduce_norm_push", *ex.push_args(not very_first, x_own(mb), weight, eps, None if very_first else x_own(mb), keep))
                self.fused_exchanges_per_forward += 0 if very_first else 1
            elif kind == "attention_block":
                lw = self.layers[step[2]]
                self._gemm(h, lw["wqkv"], self._rows(self.qkv, mb))
                q, k, v = self._head_view(mb, 0, hq), self._head_view(mb, hq, hkv), self._head_view(mb, hq + hkv, hkv)
                attn = self._rows(self.attn, mb)
                self._op("rb_attention", ctx, self._t(q), self._t(k), self._t(v), None, C.c_float(self.scale), C.c_int32(1), C.c_uint64(0), C.c_uint64(0),
                         self._t(self.cos), self._t(self.sin), C.c_int32(int(RotaryLayout.SplitHalf)), C.c_int32(1), self._t(attn.reshape((b, self.seq, hq, cfg.head_dim))))
                self.launches_per_forward += 2   # the Q and K rotations run as two small kernels inside rb_attention
            elif kind == "ffn_block":
                lw = self.layers[step[2]]
                self._gemm(h, lw["wg"], self._rows(self.ffn_act, mb), b_up=lw["wu"])
            elif kind == "scatter":
                lw = self.layers[step[2]]
                a = self._rows(self.attn, mb) if step[3] == "wo" else self._rows(self.ffn_act, mb)
                if self.side_scatter:
                    self._gemm(a, lw[step[3]], ex.own_partial())
                elif self.pull_exchange:
                    self._gemm(a, lw[step[3]], ex.own_partial())
                    self._op("rb_peer_signal", *ex.signal_args(keep, SCATTER))
                else:
                    self._op("rb_gemm_scatter", *ex.scatter_args(a, lw[step[3]], keep))
            elif kind == "lm_head":
                self._gemm(h, self.lm_head, self._rows(self.logits, mb))
            else:
                raise AssertionError(kind)

    def _run_plan(self):
        from .runtime import _check
        if self.world > 1 and not self.fused:
            # tickets in the plan count this forward's collectives from one; add the communicator's counter so far
            cur = C.c_uint64()
            _check(self.client._lib.rb_comm_ticket(self.comm.native._comm, C.byref(cur)))
            shift = cur.value
        for fn, args in self._steps:
            if self.world > 1 and not self.fused and fn.__name__ == "rb_comm_wait_ticket":
                rc = fn(args[0], C.c_uint64(args[1].value + shift))
            else:
                rc = fn(*args)
            if rc:
                _check(rc)

    def close(self) -> None:
        """Drops the recorded graph and, in fused mode, the peer buffers (a collective step: every rank of the group calls it
        at the same point).  Call this before destroying the communicator: NCCL does not finish destroying a communicator
        while a graph that holds its collectives exists."""
        if self._graph is not None:
            self.client._lib.rb_graph_destroy(self.client._ctx, self._graph)
            self._graph = None
        self._release_fused()

    def forward(self, tokens: np.ndarray | None = None) -> TensorBuffer:
        """Returns this rank's logits shard [T, vocab/world] (BF16).  `tokens` int32 [B,S]; None reuses the last upload."""
        c = self.client
        if tokens is not None:
            c.write(self.tokens_dev.handle, np.ascontiguousarray(tokens, dtype=np.int32))
            c.sync()
        if self._graph is not None:
            from .runtime import _check
            _check(c._lib.rb_graph_launch(c._ctx, self._graph))
        else:
            self._run_plan()
        return self.logits
