"""CPU: host models of the device-side protocols, in the spirit of the reference's test-only VM for its GEMM program
(rust-ascend-kernels/src/tests.rs:20-88: flags may not be signalled twice or waited on unready, local memory is poisoned,
every flag must be drained).

1. The tile raster and the attention block count are compiled from the very header the kernels include.
2. The mbarrier rings of the GEMM and the attention kernel are replayed with randomly interleaved roles on a small
   model of mbarrier phase semantics; the model raises if a stage is overwritten before its consumers are done, if a
   role would wait forever, or if a barrier is left mid-phase at the end.
"""
import ctypes as C
import os
import random
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HERE = os.path.join(ROOT, "tests", "host_model")


@pytest.fixture(scope="module")
def host():
    so = os.path.join(HERE, "libschedule_host.so")
    src = os.path.join(HERE, "schedule_host.cpp")
    hdr = os.path.join(ROOT, "rust_ascend_b200", "csrc", "schedule.h")
    if not os.path.exists(so) or os.path.getmtime(so) < max(os.path.getmtime(src), os.path.getmtime(hdr)):
        subprocess.run(["g++", "-O2", "-shared", "-fPIC", "-I", os.path.dirname(hdr), "-o", so, src], check=True)
    lib = C.CDLL(so)
    lib.host_attention_blocks.restype = C.c_uint32
    lib.host_attention_blocks.argtypes = [C.c_uint32, C.c_uint32, C.c_int, C.c_int64, C.c_uint32, C.c_uint32, C.c_uint32]
    return lib


@pytest.mark.parametrize("tiles_m,tiles_n,batches", [(13, 8, 1), (1, 1, 1), (32, 16, 1), (7, 3, 5), (9, 1, 2), (1, 40, 3)])
def test_tile_raster_is_a_bijection(host, tiles_m, tiles_n, batches):
    # same property the reference checks for its swizzle on 13x8 grids (rust-ascend-kernels/src/tests.rs:140-152)
    seen = set()
    out = (C.c_uint32 * 3)()
    for t in range(batches * tiles_m * tiles_n):
        host.host_tile_coords(t, tiles_m, tiles_n, 8, out)
        b, m, n = out[0], out[1], out[2]
        assert b < batches and m < tiles_m and n < tiles_n
        seen.add((b, m, n))
    assert len(seen) == batches * tiles_m * tiles_n


def test_tile_raster_keeps_a_wave_inside_few_rows(host):
    # 148 consecutive tiles of the 4096^3 problem (32 x 16 tiles) touch at most 16 tile rows and all 16 columns
    out = (C.c_uint32 * 3)()
    rows, cols = set(), set()
    for t in range(148):
        host.host_tile_coords(t, 32, 16, 8, out)
        rows.add(out[1]); cols.add(out[2])
    assert len(rows) <= 16 and len(cols) == 16


@pytest.mark.parametrize("M,N,delta", [(128, 128, 0), (256, 384, 128), (400, 416, 16), (48, 96, 48), (2048, 2048, 0), (128, 1024, 896), (64, 64, -100), (272, 2048, 1776)])
def test_attention_block_count_matches_the_causal_rule(host, M, N, delta):
    for row0 in range(0, M + 256, 128):
        row_end = row0 + 128
        got = host.host_attention_blocks(M, N, 1, delta, row0, row_end, 128)
        # brute force: the last key any valid row of the tile may see
        visible = [k for q in range(row0, min(row_end, M)) for k in range(N) if not (k > q + delta)]
        want = 0 if not visible else max(visible) // 128 + 1
        assert got == want, (row0, got, want)
        assert host.host_attention_blocks(M, N, 0, delta, row0, row_end, 128) == (0 if row0 >= M else -(-N // 128))


# ---- mbarrier model --------------------------------------------------------------------------------------
class Barrier:
    """mbarrier with an arrival count: a phase completes when `count` arrivals have been made; wait(parity) passes
    once the phase with that parity has completed (a fresh barrier passes parity 1)."""

    def __init__(self, count):
        self.count, self.pending, self.phase = count, count, 0

    def arrive(self):
        self.pending -= 1
        assert self.pending >= 0, "more arrivals than the barrier expects"
        if self.pending == 0:
            self.pending, self.phase = self.count, self.phase + 1

    def passed(self, parity):
        return (self.phase & 1) != parity

    def idle(self):
        return self.pending == self.count


def run(roles, seed, limit=200000):
    rng = random.Random(seed)
    live = [r for r in roles]
    steps = 0
    while live:
        progressed = False
        rng.shuffle(live)
        for r in list(live):
            try:
                if next(r):
                    progressed = True
            except StopIteration:
                live.remove(r); progressed = True
        steps += 1
        assert progressed, "every remaining role is blocked: the protocol deadlocks"
        assert steps < limit


def wait(bar, parity):
    while not bar.passed(parity):
        yield False
    yield True


@pytest.mark.parametrize("stages,tiles,kblocks,seed", [(4, 7, 5, 0), (8, 3, 1, 1), (6, 5, 17, 2), (4, 1, 64, 3)])
def test_gemm_ring_and_accumulator_handshake(stages, tiles, kblocks, seed):
    full = [Barrier(1) for _ in range(stages)]; empty = [Barrier(1) for _ in range(stages)]
    tmem_full = [Barrier(1), Barrier(1)]; tmem_empty = [Barrier(128), Barrier(128)]
    smem = [None] * stages            # what a stage holds: (tile, kb) or None when consumed ("poison")
    tmem = [None, None]
    consumed, stored = [], []

    def producer():
        stage = phase = 0
        for t in range(tiles):
            for kb in range(kblocks):
                yield from wait(empty[stage], phase ^ 1)
                assert smem[stage] is None, "stage overwritten before the MMA consumed it"
                smem[stage] = (t, kb); full[stage].arrive(); yield True
                stage += 1
                if stage == stages: stage, phase = 0, phase ^ 1

    def mma():
        stage = phase = 0
        for it in range(tiles):
            acc, acc_phase = it & 1, (it >> 1) & 1
            yield from wait(tmem_empty[acc], acc_phase ^ 1)
            assert tmem[acc] is None, "accumulator overwritten before the epilogue drained it"
            for kb in range(kblocks):
                yield from wait(full[stage], phase)
                assert smem[stage] == (it, kb), "MMA read a stage that does not hold the expected K block"
                consumed.append(smem[stage]); smem[stage] = None
                empty[stage].arrive(); yield True          # tcgen05.commit -> empty
                stage += 1
                if stage == stages: stage, phase = 0, phase ^ 1
            tmem[acc] = it; tmem_full[acc].arrive(); yield True

    def epilogue_thread(tid):
        for it in range(tiles):
            acc, acc_phase = it & 1, (it >> 1) & 1
            yield from wait(tmem_full[acc], acc_phase)
            assert tmem[acc] == it
            if tid == 0:
                stored.append(it)
            yield True
            tmem_empty[acc].arrive()
            if tmem_empty[acc].idle():
                tmem[acc] = None
            yield True

    run([producer(), mma()] + [epilogue_thread(i) for i in range(128)], seed)
    assert consumed == [(t, kb) for t in range(tiles) for kb in range(kblocks)] and stored == list(range(tiles))
    assert all(b.idle() for b in full + empty + tmem_full + tmem_empty) and all(s is None for s in smem)


@pytest.mark.parametrize("n0,n1,seed", [(3, 4, 0), (8, 8, 1), (1, 2, 2), (5, 0, 3), (0, 0, 4), (16, 17, 5)])
def test_attention_barrier_protocol(n0, n1, seed):
    """Two query tiles, K/V rings of two stages, S/P aliased in TMEM (P overwrites the scores it was computed from)."""
    KV = 2
    n = [n0, n1]; n_max = max(n)
    k_full = [Barrier(1) for _ in range(KV)]; k_empty = [Barrier(1) for _ in range(KV)]
    v_full = [Barrier(1) for _ in range(KV)]; v_empty = [Barrier(1) for _ in range(KV)]
    s_full = [Barrier(1), Barrier(1)]; p_full = [Barrier(128), Barrier(128)]; o_full = [Barrier(1), Barrier(1)]
    ksm, vsm = [None] * KV, [None] * KV
    s_tmem = [None, None]            # ("S", j) after the score GEMM, ("P", j) after the softmax
    o_acc = [[], []]
    done = [False, False]

    def producer():
        for j in range(n_max):
            st, ph = j % KV, (j // KV) & 1
            yield from wait(k_empty[st], ph ^ 1)
            assert ksm[st] is None; ksm[st] = j; k_full[st].arrive(); yield True
            yield from wait(v_empty[st], ph ^ 1)
            assert vsm[st] is None; vsm[st] = j; v_full[st].arrive(); yield True

    def issue_s(t, j):
        assert ksm[j % KV] == j, "score GEMM read a K stage that holds another block"
        assert s_tmem[t] is None or s_tmem[t] == ("consumed", j - 1), "scores overwritten while P was still needed"
        s_tmem[t] = ("S", j); s_full[t].arrive()

    def mma():
        if n_max > 0:
            yield from wait(k_full[0], 0)
            for t in range(2):
                if n[t] > 0: issue_s(t, 0)
            ksm[0] = None; k_empty[0].arrive(); yield True
        for j in range(n_max):
            st, ph = j % KV, (j // KV) & 1
            for t in range(2):
                if j >= n[t]: continue
                yield from wait(p_full[t], j & 1)
                yield from wait(v_full[st], ph)
                assert s_tmem[t] == ("P", j) and vsm[st] == j
                o_acc[t].append(j); s_tmem[t] = ("consumed", j)
                if t == 1 or j >= n[1]:
                    vsm[st] = None; v_empty[st].arrive()
                yield True
                if j + 1 < n[t]:
                    st1, ph1 = (j + 1) % KV, ((j + 1) // KV) & 1
                    yield from wait(k_full[st1], ph1)
                    issue_s(t, j + 1)
                    if t == 1 or j + 1 >= n[1]:
                        ksm[st1] = None; k_empty[st1].arrive()
                    yield True
                else:
                    o_full[t].arrive(); yield True

    def softmax_thread(t, tid):
        for j in range(n[t]):
            yield from wait(s_full[t], j & 1)
            assert s_tmem[t] in (("S", j), ("P", j))      # ("P", j): another thread of the tile already finished this block
            yield True
            p_full[t].arrive()
            if p_full[t].idle():
                s_tmem[t] = ("P", j)
            yield True
        if n[t] > 0:
            yield from wait(o_full[t], 0)
            assert o_acc[t] == list(range(n[t]))
        if tid == 0:
            done[t] = True

    run([producer(), mma()] + [softmax_thread(t, i) for t in range(2) for i in range(128)], seed)
    assert done == [True, True] and o_acc == [list(range(n0)), list(range(n1))]
    assert all(b.idle() for b in k_full + k_empty + v_full + v_empty + s_full + p_full + o_full)
    assert all(x is None for x in ksm + vsm)
