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


@pytest.mark.parametrize("tiles,ctas", [(512, 148), (68, 148), (1, 148), (74, 148), (75, 148), (148, 148), (444, 148), (2752, 148), (512, 132), (3, 4), (0, 148)])
def test_gemm_tail_plan_covers_every_tile_once(host, tiles, ctas):
    """The last round of the persistent GEMM becomes half-width tiles when it would fill at most half of the CTAs: every tile is
    then covered either whole or by exactly its two halves, the halves come last, and the number of rounds does not grow."""
    out = (C.c_uint32 * 2)()
    host.host_gemm_plan(tiles, ctas, 1, out)
    split, items = out[0], out[1]
    r = tiles % ctas if ctas else 0
    if 0 < 2 * r <= ctas:
        assert (split, items) == (tiles - r, tiles + r)
    else:
        assert (split, items) == (tiles, tiles)
    cover = {}
    for item in range(items):
        host.host_gemm_item(item, split, out)
        tile, half = out[0], out[1]
        assert tile < tiles and (half == 2) == (item < split)
        cover.setdefault(tile, []).append(half)
    assert sorted(cover) == list(range(tiles))
    assert all(v == [2] or v == [0, 1] for v in cover.values())
    if ctas:
        assert -(-items // ctas) == -(-tiles // ctas)          # same number of rounds; the last one is the cheap one
    host.host_gemm_plan(tiles, ctas, 0, out)
    assert (out[0], out[1]) == (tiles, tiles)                  # shapes whose half tiles would be too narrow keep whole tiles


@pytest.mark.parametrize("q_blocks,batch,heads,ctas", [(8, 4, 32, 148), (16, 2, 32, 148), (32, 1, 32, 148), (1, 1, 1, 1), (3, 2, 5, 7), (8, 8, 4, 132), (1, 3, 7, 148), (40, 1, 2, 148)])
def test_attention_item_order_is_a_balanced_bijection(host, q_blocks, batch, heads, ctas):
    """Every (query block, head, batch) is visited exactly once over the CTAs' rounds; with the causal cost of an item (its number of
    key-block pairs, growing with the query block) no CTA carries much more than the average; and the heads in flight at any
    time are few, so that their K and V stay in L2."""
    host.host_attention_wave_heads.restype = C.c_uint32; host.host_attention_steps.restype = C.c_uint32
    heads_total = batch * heads
    items = q_blocks * heads_total
    grid = min(items, ctas)
    wave = host.host_attention_wave_heads(q_blocks, heads_total, grid)
    assert wave >= 1
    out = (C.c_uint32 * 3)()
    seen, load = set(), [0] * grid
    for step in range(host.host_attention_steps(q_blocks, heads_total, wave, grid)):
        in_flight = set()
        for c in range(grid):
            if not host.host_attention_item(step, c, grid, q_blocks, heads_total, heads, wave, out):
                continue
            qb, h, b = out[0], out[1], out[2]
            assert qb < q_blocks and h < heads and b < batch
            assert (qb, h, b) not in seen
            seen.add((qb, h, b)); load[c] += 2 * qb + 2; in_flight.add((h, b))
        assert len(in_flight) <= wave                    # one step stays inside one wave of heads
    assert len(seen) == items
    if items >= 4 * grid:
        assert max(load) <= 1.10 * (sum(load) / grid) + 2 * q_blocks


def test_group_lookup_matches_the_prefix_sums(host):
    host.host_group_of.restype = C.c_uint32
    ends = [256, 256, 768, 1024, 1024, 1280]
    arr = (C.c_int32 * len(ends))(*ends)
    for row in range(0, 1280, 128):
        want = next(g for g, e in enumerate(ends) if row < e)
        assert host.host_group_of(arr, len(ends), row) == want


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


@pytest.mark.parametrize("items,seed", [([(3, 4)], 0), ([(8, 8), (1, 2), (5, 0)], 1), ([(0, 0), (2, 2), (0, 0), (1, 1)], 2), ([(1, 1)] * 5, 3),
                                        ([(16, 17), (0, 3), (4, 4), (1, 0)], 4), ([(2, 3), (2, 3), (7, 8), (1, 2), (6, 6)], 5)])
def test_attention_barrier_protocol(items, seed):
    """The persistent attention kernel's protocol over a CTA's list of work items (each: key blocks of tile 0 and of tile 1):
    one Q buffer handed back after the item's last score GEMM, K/V rings of two stages that run on across items, S/P aliased
    in TMEM (P overwrites the scores it was computed from) and handed over in two halves, O read out by the softmax warps at
    the end of an item and handed back before the next item's first P V overwrites it."""
    KV = 2
    q_full, q_empty = Barrier(1), Barrier(1)
    k_full = [Barrier(1) for _ in range(KV)]; k_empty = [Barrier(1) for _ in range(KV)]
    v_full = [Barrier(1) for _ in range(KV)]; v_empty = [Barrier(1) for _ in range(KV)]
    s_full = [Barrier(1), Barrier(1)]; p_half = [Barrier(128), Barrier(128)]; p_full = [Barrier(128), Barrier(128)]
    o_full = [Barrier(1), Barrier(1)]; o_free = [Barrier(128), Barrier(128)]
    qsm = [None]                     # item whose Q the shared-memory buffer holds
    ksm, vsm = [None] * KV, [None] * KV
    s_tmem = [None, None]            # ("S", item, j) after the score GEMM, ("P", item, j) after the softmax
    p_state = [0, 0]                 # halves of P the softmax threads have completed for the current block
    o_tmem = [None, None]            # (item, [blocks accumulated]) or None once read out
    stored = [[], []]

    def producer():
        kv_it = q_it = 0
        for i, n in enumerate(items):
            n_max = max(n)
            if n_max == 0: continue
            if q_it > 0:
                yield from wait(q_empty, (q_it - 1) & 1)
            assert qsm[0] is None, "Q overwritten while score GEMMs of the previous item could still read it"
            qsm[0] = i; q_full.arrive(); yield True
            for j in range(n_max):
                st, ph = (kv_it + j) % KV, ((kv_it + j) // KV) & 1
                yield from wait(k_empty[st], ph ^ 1)
                assert ksm[st] is None; ksm[st] = (i, j); k_full[st].arrive(); yield True
                yield from wait(v_empty[st], ph ^ 1)
                assert vsm[st] is None; vsm[st] = (i, j); v_full[st].arrive(); yield True
            kv_it += n_max; q_it += 1

    def mma():
        kv_it = q_it = 0
        blk, used = [0, 0], [0, 0]
        for i, n in enumerate(items):
            n_max = max(n)
            if n_max == 0: continue
            total_s, s_done = n[0] + n[1], 0

            def issue_s(t, j, st):
                assert qsm[0] == i and ksm[st] == (i, j), "score GEMM read a Q or K buffer that holds something else"
                assert s_tmem[t] is None or s_tmem[t][0] == "consumed", "scores overwritten while P was still needed"
                s_tmem[t] = ("S", i, j); p_state[t] = 0; s_full[t].arrive()

            yield from wait(q_full, q_it & 1)
            st, ph = kv_it % KV, (kv_it // KV) & 1
            yield from wait(k_full[st], ph)
            for t in (1, 0):                                   # tile 1 leads: it has the extra key block under a causal mask
                if n[t] > 0: issue_s(t, 0, st); s_done += 1
            ksm[st] = None; k_empty[st].arrive()
            if s_done == total_s: qsm[0] = None; q_empty.arrive()
            yield True
            for j in range(n_max):
                st, ph = (kv_it + j) % KV, ((kv_it + j) // KV) & 1
                for t in (1, 0):
                    if j >= n[t]: continue
                    par = blk[t] & 1
                    yield from wait(p_half[t], par)
                    if j == 0 and used[t] > 0:
                        yield from wait(o_free[t], (used[t] - 1) & 1)
                    yield from wait(v_full[st], ph)
                    assert p_state[t] >= 1 and vsm[st] == (i, j)
                    if j == 0:
                        assert o_tmem[t] is None, "O overwritten before the previous item's rows were read out"
                        o_tmem[t] = (i, [])
                    yield True
                    yield from wait(p_full[t], par)
                    assert s_tmem[t] == ("P", i, j) and p_state[t] == 2
                    o_tmem[t][1].append(j); s_tmem[t] = ("consumed", i, j)
                    blk[t] += 1
                    if t == 0 or j >= n[0]:                    # released by the tile served second, or by the only user
                        vsm[st] = None; v_empty[st].arrive()
                    yield True
                    if j + 1 < n[t]:
                        st1, ph1 = (kv_it + j + 1) % KV, ((kv_it + j + 1) // KV) & 1
                        yield from wait(k_full[st1], ph1)
                        issue_s(t, j + 1, st1); s_done += 1
                        if t == 0 or j + 1 >= n[0]:
                            ksm[st1] = None; k_empty[st1].arrive()
                        if s_done == total_s: qsm[0] = None; q_empty.arrive()
                        yield True
                    else:
                        o_full[t].arrive(); used[t] += 1; yield True
            kv_it += n_max; q_it += 1

    def softmax_thread(t, tid):
        blk = used = 0
        for i, n in enumerate(items):
            if n[t] == 0: continue
            for j in range(n[t]):
                yield from wait(s_full[t], blk & 1)
                assert s_tmem[t][1:] == (i, j) and s_tmem[t][0] in ("S", "P")
                yield True
                p_half[t].arrive()
                if p_half[t].idle(): p_state[t] = 1
                yield True
                p_full[t].arrive()
                if p_full[t].idle(): p_state[t] = 2; s_tmem[t] = ("P", i, j)
                yield True
                blk += 1
            yield from wait(o_full[t], used & 1)
            assert o_tmem[t] == (i, list(range(n[t]))), "epilogue read an accumulator that is not this item's finished O"
            if tid == 0: stored[t].append(i)
            yield True
            o_free[t].arrive()
            if o_free[t].idle(): o_tmem[t] = None
            yield True
            used += 1

    run([producer(), mma()] + [softmax_thread(t, i) for t in range(2) for i in range(128)], seed, limit=2000000)
    for t in range(2):
        assert stored[t] == [i for i, n in enumerate(items) if n[t] > 0]
    assert all(b.idle() for b in [q_full] + k_full + k_empty + v_full + v_empty + s_full + p_half + p_full + o_full)
    assert all(x is None for x in ksm + vsm)
