"""The fused tensor-parallel decoder plan, executed on the CPU.

Every rank's launch plan (decoder.py, fused mode) is replayed in one process against a NumPy / oracle stand-in for the
library in which peer buffers really are shared between the simulated ranks: scatter GEMMs store BF16 partial rows into the
owners' staging slots, the owner-side step sums them in rank order, updates its rows of the residual stream, normalises and
stores into every rank's activation buffer, and the blocks in between read those buffers through the descriptors the plan
carries (offsets, strides, slots).  The gathered logits must match the unsharded host reference of the decoder stack, which
checks the plan's data flow end to end: ownership of rows, slot and row offsets, the sharded residual stream, the order of
steps.  What it cannot check is the CUDA code itself and the timing of the flags (tests/test_fused_model.py covers the
latter); because the ranks are stepped in lock step, the stand-in's waits only check that the counts they are given match
what the producers announce.
"""
import ctypes as C
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for _p in (ROOT, os.path.join(ROOT, "tests")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

NP = {0: np.float32, 1: np.float16, 2: np.uint16, 3: np.int32, 4: np.int64, 5: np.uint8}


class World:
    """Storage shared by all simulated ranks, and the registry that makes peer buffers alias."""

    def __init__(self, size):
        self.size, self.store, self.next, self.peer_buffers = size, {}, 0, []

    def alloc(self, nbytes):
        self.next += 1
        self.store[self.next] = bytearray(max(int(nbytes), 1))
        return self.next

    def peer_handles(self, index, nbytes):
        """The i-th peer buffer every rank creates: one allocation per rank, made when the first rank asks."""
        while len(self.peer_buffers) <= index:
            self.peer_buffers.append(None)
        if self.peer_buffers[index] is None:
            self.peer_buffers[index] = [self.alloc(nbytes) for _ in range(self.size)]
        return self.peer_buffers[index]


def bf16r(x):
    from rust_ascend_b200.runtime import bf16_bits_to_f32, f32_to_bf16_bits
    return bf16_bits_to_f32(f32_to_bf16_bits(np.asarray(x, np.float32)))


class EmuLib:
    """NumPy / oracle versions of the entry points the fused plan calls."""

    def __init__(self, world, rank, oracle):
        self.w, self.rank, self.orc = world, rank, oracle
        self.real = C.CDLL(os.path.join(ROOT, "rust_ascend_b200", "libruda_b200.so"))
        self.real.rb_gemm_scatter_signals.restype = C.c_uint32
        self.rb_gemm_scatter_signals = self.real.rb_gemm_scatter_signals

    # -- descriptors -> arrays ------------------------------------------------------------------------------
    def _desc(self, ref):
        t = ref._obj if hasattr(ref, "_obj") else ref.contents
        shape = tuple(int(t.shape[i]) for i in range(t.rank)); strides = tuple(int(t.strides[i]) for i in range(t.rank))
        return int(t.handle), int(t.offset), int(t.dtype), shape, strides

    def _view(self, ref):
        h, off, dt, shape, strides = self._desc(ref)
        item = np.dtype(NP[dt]).itemsize
        base = np.frombuffer(self.w.store[h], dtype=np.uint8)
        span = sum((d - 1) * s for d, s in zip(shape, strides)) * item + item if all(shape) else 0
        assert off + span <= base.size, ("descriptor leaves its storage", h, off, span, base.size)
        flat = base[off:off + span].view(NP[dt]) if span else np.empty(0, NP[dt])
        return np.lib.stride_tricks.as_strided(flat, shape=shape, strides=tuple(s * item for s in strides), writeable=True) if span else flat.reshape(shape)

    def _f32(self, ref):
        from rust_ascend_b200.runtime import bf16_bits_to_f32
        v = self._view(ref)
        return bf16_bits_to_f32(np.ascontiguousarray(v)) if v.dtype == np.uint16 else np.ascontiguousarray(v).astype(np.float32)

    def _store(self, ref, values):
        from rust_ascend_b200.runtime import f32_to_bf16_bits
        v = self._view(ref)
        v[...] = f32_to_bf16_bits(values).reshape(v.shape) if v.dtype == np.uint16 else np.asarray(values).astype(v.dtype).reshape(v.shape)

    # -- entry points -------------------------------------------------------------------------------------------
    def rb_embedding(self, ctx, table, ids, out):
        self._view(out)[...] = self._view(table)[self._view(ids)]
        return 0

    def rb_gemm(self, ctx, a, b, ta, tb, bias, b_up, epilogue, out):
        assert ta.value == 0 and tb.value == 1 and bias is None
        x = self._f32(a).astype(np.float64)
        y = x @ self._f32(b).astype(np.float64).T
        if b_up is not None:
            g = y.astype(np.float32); u = (x @ self._f32(b_up).astype(np.float64).T).astype(np.float32)
            y = (g * (np.float32(1) / (np.float32(1) + np.exp(-g)))) * u
        self._store(out, y.astype(np.float32))
        return 0

    def rb_attention(self, ctx, q, k, v, mask, scale, causal, qs, ks, cos, sin, layout, out_layout, out):
        from rust_ascend_b200.runtime import RotaryLayout
        assert mask is None and causal.value == 1 and out_layout.value == 1 and layout.value == int(RotaryLayout.SplitHalf)
        qf, kf, vf = self._f32(q), self._f32(k), self._f32(v)
        c, s = self._f32(cos), self._f32(sin)
        b, hq, m, d = qf.shape
        hkv = kf.shape[1]
        qr = bf16r(self.orc.rotary(qf, np.broadcast_to(c, (b, hq, m, d // 2)), np.broadcast_to(s, (b, hq, m, d // 2)), "split_half"))
        kr = bf16r(self.orc.rotary(kf, np.broadcast_to(c, (b, hkv, m, d // 2)), np.broadcast_to(s, (b, hkv, m, d // 2)), "split_half"))
        o = self.orc.attention(qr, kr, vf, scale.value, causal=True, out_bf16=True)
        self._store(out, o.transpose(0, 2, 1, 3))
        return 0

    def rb_gemm_scatter(self, ctx, a, b, rank, world, staging, flags):
        assert rank.value == self.rank
        partial = bf16r((self._f32(a).astype(np.float64) @ self._f32(b).astype(np.float64).T).astype(np.float32))
        rows = partial.shape[0] // world.value
        for owner in range(world.value):
            slot = self._view(staging[owner])                     # [world, rows, hidden] in the owner's memory
            assert slot.shape == (world.value, rows, partial.shape[1])
            from rust_ascend_b200.runtime import f32_to_bf16_bits
            slot[rank.value] = f32_to_bf16_bits(partial[owner * rows:(owner + 1) * rows])
            # what the kernel's epilogue warps announce in total for this owner
            self._view(flags[owner])[rank.value] += self.rb_gemm_scatter_signals(C.c_uint64(partial.shape[0]), C.c_uint64(partial.shape[1]), C.c_uint32(world.value))
        return 0

    def rb_peer_signal(self, ctx, rank, world, flags):
        for d in range(world.value):
            self._view(flags[d])[rank.value] += 1
        return 0

    def rb_peer_wait(self, ctx, flags, world, count):
        f = self._view(flags)
        target = f[world.value] + count.value
        assert all(f[i] - target >= 0 for i in range(world.value)), ("a wait would not pass", list(f[:world.value + 1]), count.value)
        assert all(f[i] == target for i in range(world.value)), ("more announcements than the wait consumes", list(f[:world.value + 1]), count.value)
        f[world.value] = target
        return 0

    def rb_reduce_norm_push(self, ctx, staging, x_in, weight, eps, x_out, rank, world, destinations, flags, done):
        value = None
        if staging is not None:
            parts = self._f32(staging)                              # [world, rows, width], summed in rank order in FP32
            acc = np.zeros(parts.shape[1:], np.float32)
            for src in range(world.value):
                acc = acc + parts[src]
            value = bf16r(acc)
        if x_in is not None:
            x = self._f32(x_in)
            value = bf16r(x + (value if value is not None else np.float32(0)))
        if x_out is not None:
            self._store(x_out, value)
        if weight is not None:
            r = np.float32(1) / np.sqrt((value.astype(np.float32) ** 2).mean(-1, keepdims=True, dtype=np.float32) + np.float32(eps.value))
            value = (value * r) * self._f32(weight)
        rows = value.shape[0]
        for d in range(world.value):
            dest = self._view(destinations[d])
            from rust_ascend_b200.runtime import f32_to_bf16_bits
            dest[rank.value * rows:(rank.value + 1) * rows] = f32_to_bf16_bits(value)
            self._view(flags[d])[rank.value] += 1
        return 0

    def rb_scatter_rows(self, ctx, partial, rank, world, staging, flags, done):
        part = self._view(partial)
        rows = part.shape[0] // world.value
        for owner in range(world.value):
            self._view(staging[owner])[rank.value] = part[owner * rows:(owner + 1) * rows]
            self._view(flags[owner])[rank.value] += 1
        return 0

    def rb_copy(self, ctx, x, y):
        self._view(y)[...] = self._view(x)
        return 0

    def rb_reduce_norm_rows(self, ctx, staging, x_in, weight, eps, x_out, out, done):
        """Copy form: the owner-side arithmetic on partial products already gathered locally; rows stay on this rank."""
        parts = self._f32(staging)
        acc = np.zeros(parts.shape[1:], np.float32)
        for src in range(parts.shape[0]):
            acc = acc + parts[src]
        value = bf16r(acc)
        if x_in is not None:
            value = bf16r(self._f32(x_in) + value)
        if x_out is not None:
            self._store(x_out, value)
        if weight is not None:
            r = np.float32(1) / np.sqrt((value.astype(np.float32) ** 2).mean(-1, keepdims=True, dtype=np.float32) + np.float32(eps.value))
            value = (value * r) * self._f32(weight)
        from rust_ascend_b200.runtime import f32_to_bf16_bits
        self._view(out)[...] = f32_to_bf16_bits(value)
        return 0

    def rb_reduce_norm_push_pull(self, ctx, partials, x_in, weight, eps, x_out, rank, world, destinations, flags, done):
        """Pull form: source s is rows [rank * rows, (rank + 1) * rows) of rank s's whole partial product."""
        whole = [self._f32(partials[src]) for src in range(world.value)]
        rows = whole[0].shape[0] // world.value
        acc = np.zeros((rows, whole[0].shape[1]), np.float32)
        for src in range(world.value):        # rank order, FP32, one rounding: the arithmetic of the push form
            acc = acc + whole[src][rank.value * rows:(rank.value + 1) * rows]
        value = bf16r(acc)
        if x_in is not None:
            value = bf16r(self._f32(x_in) + value)
        if x_out is not None:
            self._store(x_out, value)
        if weight is not None:
            r = np.float32(1) / np.sqrt((value.astype(np.float32) ** 2).mean(-1, keepdims=True, dtype=np.float32) + np.float32(eps.value))
            value = (value * r) * self._f32(weight)
        for d in range(world.value):
            dest = self._view(destinations[d])
            from rust_ascend_b200.runtime import f32_to_bf16_bits
            dest[rank.value * rows:(rank.value + 1) * rows] = f32_to_bf16_bits(value)
            self._view(flags[d])[rank.value] += 1
        return 0

    def __getattr__(self, name):          # waits, signals, forks, SM limits: nothing to do when ranks run in lock step
        if name.startswith("rb_"):
            def nothing(*args):
                return 0
            nothing.__name__ = name
            return nothing
        raise AttributeError(name)


class EmuClient:
    def __init__(self, world, rank, oracle):
        self.world, self._lib, self._ctx = world, EmuLib(world, rank, oracle), None

    def empty(self, size):
        return self.world.alloc(size)

    def tensor(self, shape, dtype):
        from rust_ascend_b200.runtime import DType, TensorBuffer
        shape = tuple(int(d) for d in shape)
        return TensorBuffer(self.empty(int(np.prod(shape)) * DType(dtype).size), shape, dtype)

    def upload(self, array, dtype=None):
        from rust_ascend_b200.runtime import DType
        a = np.ascontiguousarray(array)
        dtype = dtype if dtype is not None else {np.dtype(np.float32): DType.F32, np.dtype(np.uint16): DType.BF16, np.dtype(np.int32): DType.I32}[a.dtype]
        t = self.tensor(a.shape, dtype)
        self.world.store[t.handle][:a.nbytes] = a.tobytes()
        return t

    def write(self, handle, host, offset=0):
        raw = np.ascontiguousarray(host).tobytes()
        self.world.store[handle][offset:offset + len(raw)] = raw

    def read(self, t):
        return np.frombuffer(self.world.store[t.handle], dtype=t.dtype.numpy, count=t.elements, offset=t.offset).reshape(t.shape).copy()

    def properties(self):
        return {"sm_count": 148}

    def free(self, handle):
        pass

    def sync(self):
        pass

    def memset(self, t, value=0):
        pass


class EmuControl:
    def __init__(self, rank, world):
        self.rank, self.world_size = rank, world


class EmuComm:
    def __init__(self, rank, world):
        self.control = EmuControl(rank, world)


@pytest.mark.parametrize("world,micro,overlap,pull", [(1, 1, False, False), (1, 2, True, False), (2, 1, False, False), (2, 2, False, False), (2, 2, True, False),
                                                      (4, 1, False, False), (1, 1, False, True), (2, 2, True, True), (4, 1, False, True),
                                                      (1, 1, False, "dma"), (2, 2, True, "dma"), (4, 1, False, "dma"),
                                                      (1, 1, False, "side"), (2, 2, True, "side"), (2, 2, False, "side"), (4, 1, False, "side")])
def test_fused_plan_computes_the_decoder(monkeypatch, oracle, world, micro, overlap, pull):
    import rust_ascend_b200.fused as fused
    from decoder_reference import forward, full_weights
    from rust_ascend_b200.decoder import LlamaConfig, TensorParallelDecoder
    from rust_ascend_b200.runtime import bf16_bits_to_f32
    shared = World(world)
    counters = [0] * world

    class SharedPeerBuffer:
        def __init__(self, client, control, nbytes):
            self.nbytes, self.rank, self.world = int(nbytes), control.rank, control.world_size
            self.handles = shared.peer_handles(counters[self.rank], self.nbytes)
            counters[self.rank] += 1

        def view(self, rank, shape, dtype, byte_offset=0):
            from rust_ascend_b200.runtime import TensorBuffer
            t = TensorBuffer(self.handles[rank], shape, dtype, None, offset=byte_offset)
            assert byte_offset + t.nbytes <= self.nbytes
            return t

        def close(self):
            pass

    monkeypatch.setattr(fused, "PeerBuffer", SharedPeerBuffer)
    cfg = LlamaConfig(layers=2, hidden=256, heads=4, kv_heads=4 if world == 4 else 2, head_dim=128, ffn=512, vocab=1024)
    batch, seq = 2 * micro * (2 if world == 4 else 1), 128
    tokens = np.random.default_rng(0).integers(0, cfg.vocab, size=(batch, seq)).astype(np.int32)
    models = []
    for rank in range(world):
        client = EmuClient(shared, rank, oracle)
        model = TensorParallelDecoder(client, cfg, batch, seq, comm=EmuComm(rank, world), rank=rank, world=world, seed=3, exact_weights=True,
                                      micro_batches=micro, fused=True, overlap_exchange=overlap, pull_exchange=pull is True, dma_exchange=pull == "dma", side_scatter=pull == "side",
                                      sm_reserve=16 if overlap else 0)
        client.write(model.tokens_dev.handle, tokens)
        models.append(model)
    steps = len(models[0]._steps)
    assert all(len(m._steps) == steps for m in models)
    for i in range(steps):                       # lock step: step i on every rank before step i + 1 on any
        for model in models:
            fn, args = model._steps[i]
            assert fn(*args) == 0
    got = np.concatenate([bf16_bits_to_f32(m.client.read(m.logits)) for m in models], axis=1)
    want = forward(oracle, cfg, full_weights(cfg, 3), tokens)
    err = np.abs(got - want)
    assert np.all(np.isfinite(got))
    assert err.max() <= 0.04 * np.abs(want).max() and err.mean() <= 0.015 * np.abs(want).mean() + 1e-4, (err.max(), err.mean(), np.abs(want).max())
    # a second forward on the same buffers gives the same bits (staging, activations and residual rows carry no stale state)
    for model in models:
        model.client.write(model.tokens_dev.handle, tokens)
    for i in range(steps):
        for model in models:
            fn, args = model._steps[i]
            fn(*args)
    again = np.concatenate([bf16_bits_to_f32(m.client.read(m.logits)) for m in models], axis=1)
    np.testing.assert_array_equal(again, got)
