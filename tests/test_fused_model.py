"""CPU models of the fused tensor-parallel exchange (rust_ascend_b200/csrc/fused_tp.cu, fused.py, decoder.py fused mode).

1. Addressing: the scatter GEMM's epilogue, replayed with the kernel's own index functions (csrc/schedule.h), stores every
   16-byte word of every owner's staging slot exactly once, announces as often as rb_gemm_scatter_signals says, and keeps
   the ranks on different owners at any moment.
2. Protocol: the decoder's fused schedule, replayed on N simulated ranks under random interleavings with the counting
   flags and running targets of rb_peer_wait, never reads a buffer before all of its writers have stored the current
   step's data and never overwrites data that a slower rank has not read yet; without the closing barrier it does.
3. Plan: the launch plan the decoder emits in fused mode, built against a recording stand-in for the library, names
   the schedule's steps in order and only describes tensors that lie inside their buffers.
"""
import ctypes as C
import os
import random
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HERE = os.path.join(ROOT, "tests", "host_model")
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


@pytest.fixture(scope="module")
def host():
    so = os.path.join(HERE, "libschedule_host.so")
    src = os.path.join(HERE, "schedule_host.cpp")
    hdr = os.path.join(ROOT, "rust_ascend_b200", "csrc", "schedule.h")
    if not os.path.exists(so) or os.path.getmtime(so) < max(os.path.getmtime(src), os.path.getmtime(hdr)):
        subprocess.run(["g++", "-O2", "-shared", "-fPIC", "-I", os.path.dirname(hdr), "-o", so, src], check=True)
    lib = C.CDLL(so)
    lib.host_scatter_shift.restype = C.c_uint32
    return lib


# ---- 1. addressing ----------------------------------------------------------------------------------------------------
BM, GROUP_M, CHUNK = 128, 8, 64


def replay_scatter(host, rank, world, tokens, hidden):
    """Byte offsets (in 16-byte words) stored per owner, announcements per owner and the owner of each tile in order."""
    bn = 256 if hidden > 128 else 128
    rows = tokens // world
    tiles_m, tiles_n = tokens // BM, -(-hidden // bn)
    shift = host.host_scatter_shift(rank, world, rows, BM)
    out2 = (C.c_uint32 * 2)()
    words = {o: [] for o in range(world)}
    signals = [0] * world
    tile_owner = []
    word_r = np.empty((8, 32), np.int64); word_j = np.empty((8, 32), np.int64)
    for it in range(8):
        for lane in range(32):
            host.host_scatter_word(it, lane, out2)
            word_r[it, lane], word_j[it, lane] = out2[0], out2[1]
    for t in range(tiles_m * tiles_n):
        host.host_scatter_tile(t, tiles_m, tiles_n, GROUP_M, shift, out2)
        tm, tn = out2[0], out2[1]
        for quarter in range(4):
            row0 = tm * BM + quarter * 32
            host.host_scatter_owner(row0, rows, out2)
            owner, local_row0 = out2[0], out2[1]
            col0 = tn * bn
            for c in range(0, bn, CHUNK):
                if col0 + c >= hidden:
                    break
                byte = ((local_row0 + word_r) * hidden + col0 + c) * 2 + word_j * 16
                assert not (byte % 16).any()
                words[owner].append((byte // 16).ravel())
            signals[owner] += 1
            if quarter == 0:
                tile_owner.append(owner)
    return words, signals, tile_owner


@pytest.mark.parametrize("world,tokens,hidden", [(1, 256, 64), (2, 512, 128), (2, 1024, 320), (4, 1024, 4096), (8, 2048, 192), (8, 8192, 512)])
def test_scatter_epilogue_covers_every_staging_word_once(host, world, tokens, hidden):
    lib = C.CDLL(os.path.join(ROOT, "rust_ascend_b200", "libruda_b200.so"))
    lib.rb_gemm_scatter_signals.restype = C.c_uint32
    expected = lib.rb_gemm_scatter_signals(C.c_uint64(tokens), C.c_uint64(hidden), C.c_uint32(world))
    assert expected > 0
    rows = tokens // world
    owners_by_tile = []
    for rank in range(world):
        words, signals, tile_owner = replay_scatter(host, rank, world, tokens, hidden)
        for owner in range(world):
            seen = np.concatenate(words[owner])
            assert seen.size == rows * hidden * 2 // 16 and np.array_equal(np.sort(seen), np.arange(seen.size))
            assert signals[owner] == expected
        assert tile_owner[0] == (rank + 1) % world
        owners_by_tile.append(tile_owner)
    for step in zip(*owners_by_tile):          # the same tile index on every rank: all different owners
        assert len(set(step)) == world
    assert lib.rb_gemm_scatter_signals(C.c_uint64(tokens + 64), C.c_uint64(hidden), C.c_uint32(world)) == 0


# ---- 2. protocol --------------------------------------------------------------------------------------------------------
class Hazard(Exception):
    pass


class Cell:
    """One peer-visible buffer region: which step's data it holds and whether its reader has consumed it."""

    def __init__(self):
        self.version, self.consumed = None, True

    def write(self, version, what):
        if not self.consumed:
            raise Hazard(f"{what}: overwritten before it was read (held {self.version}, new {version})")
        self.version, self.consumed = version, False

    def read(self, version, what):
        if self.version != version:
            raise Hazard(f"{what}: read {self.version}, expected {version}")
        self.consumed = True


class Flags:
    def __init__(self, world):
        self.count, self.target = [0] * world, 0


def simulate(world, layers, micro, forwards, seed, barrier=True, overlap=False, joins=True):
    """Every rank runs the schedule `forwards` times.  Steps between aux_begin and aux_end belong to the rank's side
    stream: they run in order among themselves, not before the compute stream has passed their aux_begin, and an aux_wait
    on the compute stream passes only when the latest segment recorded in its slot has finished."""
    from rust_ascend_b200.decoder import fused_schedule
    main, side = [], []                 # per forward: compute-stream steps and side-stream steps, in program order
    open_segment = None
    for s in fused_schedule(layers, micro, overlap):
        if s[0] == "barrier":
            if barrier:                                           # rb_peer_signal, then rb_peer_wait on the barrier flags
                main += [("barrier_signal",), ("barrier_wait",)]
        elif s[0] == "aux_begin":
            open_segment = len(main)
            main.append(None)                                     # becomes ("fork", end of the segment) at aux_end
        elif s[0] == "aux_end":
            main[open_segment] = ("fork", len(side))              # side steps before this position may start
            main.append(("record", s[1], len(side)))              # slot <- side position after this segment
            open_segment = None
        elif s[0] == "aux_wait" and not joins:
            continue
        elif open_segment is not None:
            side.append(s)
        else:
            main.append(s)
    rng = random.Random(seed)
    signals = 5                                                    # announcements per scatter and owner (any positive count)
    staging = [[[Cell() for _src in range(world)] for _owner in range(world)] for _mb in range(micro)]
    gathered = [[[Cell() for _owner in range(world)] for _dest in range(world)] for _mb in range(micro)]
    flags = {kind: [[Flags(world) for _r in range(world)] for _mb in range(micro)] for kind in ("scatter", "gather", "barrier")}
    pc = {"m": [0] * world, "a": [0] * world}                      # positions over forwards * len(list)
    forked = [0] * world                                           # side position the compute stream has released
    slots = [dict() for _ in range(world)]                         # slot -> side position that must be reached
    scatter_no = [[0] * micro for _ in range(world)]               # per rank and micro batch: scatters / pushes issued so far
    push_no = [[0] * micro for _ in range(world)]
    waits = {"wait_scatter": ("scatter", signals), "wait_gather": ("gather", 1), "barrier_wait": ("barrier", 1)}
    total = {"m": forwards * len(main), "a": forwards * len(side)}
    program = {"m": main, "a": side}

    def ready(rank, kind, mb, count):
        f = flags[kind][mb][rank]
        return all(c - (f.target + count) >= 0 for c in f.count)

    def runnable(r, stream):
        if pc[stream][r] >= total[stream]:
            return False
        step = program[stream][pc[stream][r] % len(program[stream])]
        if stream == "a" and pc["a"][r] >= forked[r]:
            return False                                           # the compute stream has not reached this segment's fork
        if step[0] in waits:
            kind, count = waits[step[0]]
            return ready(r, kind, step[1] if len(step) > 1 else 0, count)
        if step[0] == "aux_wait":
            return pc["a"][r] >= slots[r].get(step[1], 0)
        return True

    steps = 0
    while any(pc[st][r] < total[st] for st in ("m", "a") for r in range(world)):
        steps += 1
        choices = [(r, st) for r in range(world) for st in ("m", "a") if runnable(r, st)]
        if not choices:
            raise Hazard("deadlock: every unfinished stream waits")
        r, st = rng.choice(choices)
        position = pc[st][r]
        step = program[st][position % len(program[st])]
        base = position // len(program[st]) * len(side)            # side positions of earlier forwards
        kind = step[0]
        if kind in waits:
            group, count = waits[kind]
            flags[group][step[1] if len(step) > 1 else 0][r].target += count
        elif kind == "fork":
            forked[r] = base + step[1]
        elif kind == "record":
            slots[r][step[1]] = base + step[2]
        elif kind == "aux_wait":
            pass
        elif kind == "scatter":
            mb = step[1]
            scatter_no[r][mb] += 1
            for owner in range(world):
                staging[mb][owner][r].write(scatter_no[r][mb], f"staging[mb{mb}][owner{owner}][src{r}]")
                flags["scatter"][mb][owner].count[r] += signals
        elif kind == "push":
            mb = step[1]
            very_first = step[2] == 0 and step[3] == 0
            push_no[r][mb] += 1
            if not very_first:
                for src in range(world):
                    staging[mb][r][src].read(scatter_no[r][mb], f"staging[mb{mb}][owner{r}][src{src}]")
            for dest in range(world):
                gathered[mb][dest][r].write(push_no[r][mb], f"gathered[mb{mb}][dest{dest}][rows of {r}]")
                flags["gather"][mb][dest].count[r] += 1
        elif kind in ("attention_block", "ffn_block", "lm_head"):
            mb = step[1]
            for owner in range(world):
                gathered[mb][r][owner].read(push_no[r][mb], f"gathered[mb{mb}][dest{r}][rows of {owner}]")
        elif kind == "barrier_signal":
            for dest in range(world):
                flags["barrier"][0][dest].count[r] += 1
        else:
            assert kind == "embed", kind
        pc[st][r] += 1
    return steps


@pytest.mark.parametrize("world,layers,micro", [(2, 1, 1), (2, 2, 2), (4, 2, 1), (8, 3, 2), (3, 2, 2)])
@pytest.mark.parametrize("overlap", [False, True])
@pytest.mark.parametrize("seed", range(6))
def test_fused_schedule_has_no_buffer_hazard_under_any_interleaving(world, layers, micro, overlap, seed):
    simulate(world, layers, micro, forwards=3, seed=seed, overlap=overlap)


def test_model_detects_a_missing_join_of_the_side_stream():
    # Without aux_wait the compute stream's next block reads activations that the side stream has not gathered yet.
    with pytest.raises(Hazard):
        for seed in range(20):
            simulate(2, 2, 2, forwards=2, seed=seed, overlap=True, joins=False)


def test_model_detects_the_hazard_the_closing_barrier_prevents():
    # Without the barrier a fast rank's next forward pushes its first rows into a buffer the slow rank has not read.
    caught = 0
    for seed in range(40):
        try:
            simulate(4, 1, 1, forwards=3, seed=seed, barrier=False)
        except Hazard:
            caught += 1
    assert caught > 0


# ---- 3. plan ------------------------------------------------------------------------------------------------------------
class Recorder:
    """Stands in for the shared library: every rb_* call is recorded; the one host-only helper is answered by the real one."""

    def __init__(self):
        self.real = C.CDLL(os.path.join(ROOT, "rust_ascend_b200", "libruda_b200.so"))
        self.real.rb_gemm_scatter_signals.restype = C.c_uint32

    def __getattr__(self, name):
        if name == "rb_gemm_scatter_signals":
            return self.real.rb_gemm_scatter_signals

        def call(*args):
            return 0
        call.__name__ = name
        return call


class FakeClient:
    def __init__(self):
        self._lib, self._ctx, self.sizes, self.next = Recorder(), None, {}, 0

    def empty(self, size):
        self.next += 1
        self.sizes[self.next] = size
        return self.next

    def tensor(self, shape, dtype):
        from rust_ascend_b200.runtime import DType, TensorBuffer
        n = int(np.prod(shape)) if len(shape) else 1
        return TensorBuffer(self.empty(n * DType(dtype).size), tuple(int(d) for d in shape), dtype)

    def upload(self, array, dtype=None):
        from rust_ascend_b200.runtime import DType
        a = np.asarray(array)
        return self.tensor(a.shape, dtype if dtype is not None else DType.F32)

    def properties(self):
        return {"sm_count": 148}

    def free(self, handle):
        self.sizes.pop(handle)

    def sync(self):
        pass

    def memset(self, t, value=0):
        pass


class FakePeerBuffer:
    """Peer buffers without a device: handles are fabricated, one per rank."""

    def __init__(self, client, control, nbytes):
        self.client, self.nbytes, self.rank, self.world = client, int(nbytes), control.rank, control.world_size
        self.handles = [client.empty(nbytes) for _ in range(self.world)]

    def view(self, rank, shape, dtype, byte_offset=0):
        from rust_ascend_b200.runtime import TensorBuffer
        t = TensorBuffer(self.handles[rank], shape, dtype, None, offset=byte_offset)
        assert byte_offset + t.nbytes <= self.nbytes
        return t

    def close(self):
        for h in self.handles:
            self.client.free(h)


class FakeControl:
    def __init__(self, rank, world):
        self.rank, self.world_size = rank, world


class FakeComm:
    def __init__(self, rank, world):
        self.control = FakeControl(rank, world)


@pytest.mark.parametrize("world,micro,overlap", [(2, 1, False), (4, 2, False), (8, 1, False), (2, 2, True), (8, 2, True)])
def test_fused_plan_follows_the_schedule_and_stays_inside_its_buffers(monkeypatch, world, micro, overlap):
    import rust_ascend_b200.fused as fused
    from rust_ascend_b200._lib import rb_tensor
    from rust_ascend_b200.decoder import LlamaConfig, TensorParallelDecoder, fused_schedule
    from rust_ascend_b200.runtime import DType
    monkeypatch.setattr(fused, "PeerBuffer", FakePeerBuffer)
    cfg = LlamaConfig(layers=2, hidden=256, heads=8, kv_heads=8, head_dim=128, ffn=1024, vocab=512)
    batch, seq = 2 * micro, 64 * world
    rank = world - 1
    client = FakeClient()
    model = TensorParallelDecoder(client, cfg, batch, seq, comm=FakeComm(rank, world), rank=rank, world=world, micro_batches=micro, fused=True,
                                  overlap_exchange=overlap, sm_reserve=16 if overlap else 0)
    names = [fn.__name__ for fn, _ in model._steps]
    expected = []
    for step in fused_schedule(cfg.layers, micro, overlap):
        expected += {"embed": ["rb_embedding"], "wait_scatter": ["rb_peer_wait"], "wait_gather": ["rb_peer_wait"], "push": ["rb_reduce_norm_push"],
                     "attention_block": ["rb_gemm", "rb_attention"], "ffn_block": ["rb_gemm"], "scatter": ["rb_gemm_scatter"],
                     "lm_head": ["rb_gemm"], "barrier": ["rb_peer_signal", "rb_peer_wait"],
                     "aux_begin": ["rb_aux_begin"], "aux_end": ["rb_aux_end"], "aux_wait": ["rb_aux_wait"]}[step[0]]
    assert names == expected
    assert model.fused_exchanges_per_forward == micro * (2 * cfg.layers) and model.collectives_per_forward == 0
    # every descriptor the plan keeps alive lies inside the storage it names
    checked = 0
    for obj in model._keep:
        if isinstance(obj, rb_tensor):
            n = 1
            for i in range(obj.rank):
                n *= obj.shape[i]
            assert obj.offset + n * DType(obj.dtype).size <= client.sizes[obj.handle], (obj.handle, obj.offset, n)
            assert obj.offset % 16 == 0
            checked += 1
    assert checked > 20
    # the scatter and push calls carry `world` staging / destination / flag descriptors each
    for fn, args in model._steps:
        if fn.__name__ == "rb_gemm_scatter":
            assert len(args[5]) == world and len(args[6]) == world and args[3].value == rank and args[4].value == world
            staging = args[5][0].contents
            assert (staging.shape[0], staging.shape[1], staging.shape[2]) == (world, batch // micro * seq // world, cfg.hidden)
        if fn.__name__ == "rb_reduce_norm_push":
            assert len(args[8]) == world and len(args[9]) == world
            dest = args[8][0].contents
            assert (dest.shape[0], dest.shape[1]) == (batch // micro * seq, cfg.hidden)
    model.close()
    assert not model._exchanges and model._peer_h is None


def test_fused_mode_rejects_shapes_the_kernels_cannot_take():
    from rust_ascend_b200.decoder import LlamaConfig, TensorParallelDecoder
    from rust_ascend_b200.runtime import InvalidTensor
    cfg = LlamaConfig(layers=1, hidden=256, heads=8, kv_heads=8, head_dim=128, ffn=1024, vocab=512)
    with pytest.raises(InvalidTensor):      # 2 * 96 tokens is not a multiple of 128 * world
        TensorParallelDecoder(FakeClient(), cfg, 2, 96, comm=FakeComm(0, 2), rank=0, world=2, fused=True)
    with pytest.raises(InvalidTensor):      # no communicator, no control plane to exchange peer tokens over
        TensorParallelDecoder(FakeClient(), cfg, 2, 128, fused=True)
