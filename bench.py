#!/usr/bin/env python
"""Benchmark of the dense-transformer hot path on B200.

Headline (one JSON line on rank 0): BF16 Linear GEMM  Y = bf16(X W^T + bias),  X [4096,4096], W [4096,4096]
(stored [N,K]), FP32 accumulate, bias FP32 — the configuration the reference's metric is quoted on.  One step
is one pass of that GEMM over one synthetic batch.  At N > 1 the same Linear runs as a row-parallel layer: every rank
multiplies its own K shard (one 4096^3 product per rank, so the work per GPU stays that of the one-GPU step: weak
scaling) and the partial products are summed on every rank, which is the exchange step tensor parallelism has.

`--impl reference` times the reference's arithmetic for the same step on the host cores instead (the CPU
oracle port, since the reference has no CPU execution path of its own and its Rust sources do not build here).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M = N = K = 4096
FLOPS_PER_STEP = 2 * M * N * K          # bias adds not counted
METRIC = "BF16 Linear GEMM TFLOP/s (4096x4096x4096, FP32 accumulate, fused bias, BF16 out)"
SETS = 4                                 # rotating operand sets: 4 x 96 MiB > 126 MB L2
NCCL_CTAS = 16                           # SMs left to NCCL while tensor-parallel GEMMs run (decoder extra)


def workload_config(world: int) -> dict:
    """The `config` object both arms print (identical keys and values, so the two lines describe one workload)."""
    parallelism = "one GPU" if world == 1 else (f"row-parallel Linear: K sharded x{world} (one 4096^3 product per GPU and step), the partial products "
                                                "summed on every rank (one exchange of the 32 MiB BF16 result per step)")
    return {"workload": "linear_bf16_4096x4096x4096_bias", "m": M, "n": N, "k": K, "k_total": K * world,
            "l2": f"rotating {SETS} operand sets (384 MiB) > 126 MB L2", "parallelism": parallelism}


PIPELINED = "fused, pipelined: plain GEMM; the owner-side pull kernel of step i runs on the side stream beside the GEMM of step i+1"
PUSHED_PIPELINED = "fused, pipelined: plain GEMM; a scatter kernel (posted stores) and the owner-side sum + push of step i run on the side stream beside the GEMM of step i+1"
PUSH_SIDE_SMS = int(os.environ.get("RUDA_BENCH_PUSH_SIDE_SMS", "16"))
COPIED = "fused: plain GEMM, device-to-device copies (copy engines) gather the partial products and the summed rows, local owner-side kernel"
COPIED_PIPELINED = "fused, pipelined: plain GEMM; the copies and the local owner-side kernel of step i run on the side stream beside the GEMM of step i+1"
SIDE_SMS = int(os.environ.get("RUDA_BENCH_SIDE_SMS", "32"))      # SMs the pipelined form keeps free of the GEMM for the side stream
PIPE_DEPTH = int(os.environ.get("RUDA_BENCH_PIPE_DEPTH", "2"))    # exchanges in flight in the pipelined form (2 or 4: divides the operand sets)


class RowParallelHeadline:
    """The N > 1 headline step: Y = sum_r X_r W_r^T + bias on every rank (rank 0's partial product carries the bias)."""

    def __init__(self, client, RT, dist, rank, world, sets, args):
        import ctypes as C
        from rust_ascend_b200.distributed import NcclCommunicator, TorchControl
        from rust_ascend_b200.fused import GATHER, SCATTER, FusedExchange
        from rust_ascend_b200.runtime import _check
        self.client, self.dist, self.rank, self.world, self.args = client, dist, rank, world, args
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        control = TorchControl()
        lib, keep = client._lib, []
        self._keep = keep
        self.candidates = {}
        try:
            ex = FusedExchange(client, control, M, N)
            self.exchange = ex
            scatter = [ex.scatter_bias_args(st[0], st[1], st[2] if rank == 0 else None, keep) for st in sets]
            wait_s, wait_g = ex.wait_args(SCATTER, ex.signals, keep), ex.wait_args(GATHER, 1, keep)
            push = ex.push_args(True, None, None, 1e-5, None, keep)

            def fused(i):
                _check(lib.rb_gemm_scatter_bias(*scatter[i % SETS])); _check(lib.rb_peer_wait(*wait_s))
                _check(lib.rb_reduce_norm_push(*push)); _check(lib.rb_peer_wait(*wait_g))
            self.candidates["fused scatter-GEMM + owner-side sum + push over peer memory"] = (fused, 4)
            # pull form: the plain GEMM writes this rank's partial product, the owner-side kernel fetches its rows from every rank
            px = FusedExchange(client, control, M, N, activations=ex.activations, pull=True)
            self.pull_exchange = px
            own = px.own_partial()._c()
            keep.append(own)
            pd = [[t._c() for t in st] for st in sets]
            keep.append(pd)
            pull_gemms = [(client._ctx, C.byref(k[0]), C.byref(k[1]), C.c_int32(0), C.c_int32(1), C.byref(k[2]) if rank == 0 else None, None,
                           C.c_int32(1 if rank == 0 else 0), C.byref(own)) for k in pd]
            announce, pull = px.signal_args(keep, SCATTER), px.pull_args(None, None, 1e-5, None, keep)
            pwait_s, pwait_g = px.wait_args(SCATTER, 1, keep), px.wait_args(GATHER, 1, keep)

            def pulled(i):
                _check(lib.rb_gemm(*pull_gemms[i % SETS])); _check(lib.rb_peer_signal(*announce)); _check(lib.rb_peer_wait(*pwait_s))
                _check(lib.rb_reduce_norm_push_pull(*pull)); _check(lib.rb_peer_wait(*pwait_g))
            self.candidates["fused: plain GEMM, owner-side kernel pulls the partial products, sums and pushes over peer memory"] = (pulled, 5)
            # pipelined pull form: consecutive steps are independent products (rotating operand sets), as consecutive micro
            # batches of a layer are, so the exchange of step i (owner-side pull kernel on the side stream, on the SMs the GEMM
            # leaves free) runs beside the GEMM of step i + 1.  Two exchanges alternate: a rank overwrites a partial-product
            # buffer only after the exchange that read it has completed (rb_aux_wait).  Every step's sum is complete on every
            # rank when the timed region ends (drain()).
            self.pipe = [FusedExchange(client, control, M, N, pull=True) for _ in range(PIPE_DEPTH)]
            self.sm_count = client.properties()["sm_count"]
            owns = [e.own_partial()._c() for e in self.pipe]
            keep.append(owns)
            pipe_gemms = [(client._ctx, C.byref(k[0]), C.byref(k[1]), C.c_int32(0), C.c_int32(1), C.byref(k[2]) if rank == 0 else None, None,
                           C.c_int32(1 if rank == 0 else 0), C.byref(owns[i % PIPE_DEPTH])) for i, k in enumerate(pd)]
            pipe_args = [(e.signal_args(keep, SCATTER), e.wait_args(SCATTER, 1, keep), e.pull_args(None, None, 1e-5, None, keep), e.wait_args(GATHER, 1, keep))
                         for e in self.pipe]
            self._slot_used = [False] * PIPE_DEPTH

            def pipelined(i):
                slot = i % PIPE_DEPTH  # the depth divides SETS, so operand set i % SETS always meets the same exchange
                announce_p, wait_sp, pull_p, wait_gp = pipe_args[slot]
                if self._slot_used[slot]:
                    _check(lib.rb_aux_wait(client._ctx, C.c_uint32(slot)))
                _check(lib.rb_gemm(*pipe_gemms[i % SETS])); _check(lib.rb_peer_signal(*announce_p))
                _check(lib.rb_aux_begin(client._ctx))
                _check(lib.rb_peer_wait(*wait_sp)); _check(lib.rb_reduce_norm_push_pull(*pull_p)); _check(lib.rb_peer_wait(*wait_gp))
                _check(lib.rb_aux_end(client._ctx, C.c_uint32(slot)))
                self._slot_used[slot] = True
            self.candidates[PIPELINED] = (pipelined, 5)
            # side-scatter form, pipelined the same way: scatter kernel (posted stores), owner-side sum + push, all on the side stream
            self.push_pipe = [FusedExchange(client, control, M, N, side_scatter=True) for _ in range(PIPE_DEPTH)]
            powns = [e.own_partial()._c() for e in self.push_pipe]
            keep.append(powns)
            push_gemms = [(client._ctx, C.byref(k[0]), C.byref(k[1]), C.c_int32(0), C.c_int32(1), C.byref(k[2]) if rank == 0 else None, None,
                           C.c_int32(1 if rank == 0 else 0), C.byref(powns[i % PIPE_DEPTH])) for i, k in enumerate(pd)]
            push_args = [(e.scatter_rows_args(keep), e.wait_args(SCATTER, 1, keep), e.push_args(True, None, None, 1e-5, None, keep), e.wait_args(GATHER, 1, keep))
                         for e in self.push_pipe]

            def pushed(i):
                slot = i % PIPE_DEPTH
                rows_p, wait_sp, push_p, wait_gp = push_args[slot]
                if self._slot_used[slot]:
                    _check(lib.rb_aux_wait(client._ctx, C.c_uint32(slot)))
                _check(lib.rb_gemm(*push_gemms[i % SETS]))
                _check(lib.rb_aux_begin(client._ctx))
                _check(lib.rb_scatter_rows(*rows_p)); _check(lib.rb_peer_wait(*wait_sp))
                _check(lib.rb_reduce_norm_push(*push_p)); _check(lib.rb_peer_wait(*wait_gp))
                _check(lib.rb_aux_end(client._ctx, C.c_uint32(slot)))
                self._slot_used[slot] = True
            self.candidates[PUSHED_PIPELINED] = (pushed, 5)
            # copy form, pipelined the same way; its transfers use no SM, so the GEMM keeps all of them
            self.copy_pipe = [FusedExchange(client, control, M, N, dma=True) for _ in range(PIPE_DEPTH)]
            cowns = [e.own_partial()._c() for e in self.copy_pipe]
            keep.append(cowns)
            copy_gemms = [(client._ctx, C.byref(k[0]), C.byref(k[1]), C.c_int32(0), C.c_int32(1), C.byref(k[2]) if rank == 0 else None, None,
                           C.c_int32(1 if rank == 0 else 0), C.byref(cowns[i % PIPE_DEPTH])) for i, k in enumerate(pd)]
            copy_args = [(e.signal_args(keep, SCATTER), e.wait_args(SCATTER, 1, keep), e.dma_reduce_calls(None, None, 1e-5, None, keep),
                          e.wait_args(GATHER, 1, keep), e.dma_gather_calls(keep)) for e in self.copy_pipe]
            self.copy_kernels = 4 + 1                    # GEMM, two signals, two waits ... the copies are not kernels

            def copied(i, fork=True):
                slot = i % PIPE_DEPTH
                announce_c, wait_sc, reduce_c, wait_gc, gather_c = copy_args[slot]
                if fork and self._slot_used[slot]:
                    _check(lib.rb_aux_wait(client._ctx, C.c_uint32(slot)))
                _check(lib.rb_gemm(*copy_gemms[i % SETS])); _check(lib.rb_peer_signal(*announce_c))
                if fork:
                    _check(lib.rb_aux_begin(client._ctx))
                _check(lib.rb_peer_wait(*wait_sc))
                for name, a in reduce_c:
                    _check(getattr(lib, name)(*a))
                _check(lib.rb_peer_wait(*wait_gc))
                for name, a in gather_c:
                    _check(getattr(lib, name)(*a))
                if fork:
                    _check(lib.rb_aux_end(client._ctx, C.c_uint32(slot)))
                    self._slot_used[slot] = True
            self.candidates[COPIED] = (lambda i: copied(i, False), 6)
            self.candidates[COPIED_PIPELINED] = (copied, 6)
        except Exception as error:           # peer memory unavailable: the NCCL form still runs
            self.fused_error = f"{type(error).__name__}: {error}"
        comm = NcclCommunicator.initialize(control, client)
        self.comm = comm
        descs = [[t._c() for t in st] for st in sets]
        keep.append(descs)
        gemms = [(client._ctx, C.byref(k[0]), C.byref(k[1]), C.c_int32(0), C.c_int32(1), C.byref(k[2]) if rank == 0 else None, None,
                  C.c_int32(1 if rank == 0 else 0), C.byref(k[3])) for k in descs]
        reduces = [(comm.native._comm, C.byref(k[3]), C.c_int32(0), C.byref(k[3]), C.c_int32(0)) for k in descs]

        def nccl(i):
            _check(lib.rb_gemm(*gemms[i % SETS])); _check(lib.rb_all_reduce(*reduces[i % SETS]))
        self.candidates["GEMM + NCCL all-reduce"] = (nccl, 1)
        self.chosen, self.timings = None, {}

    def prepare(self, name):
        """Per-candidate context state: the pipelined form keeps SIDE_SMS SMs free of the persistent GEMM for the side stream."""
        from rust_ascend_b200.runtime import _check
        import ctypes as C
        limit = self.sm_count - SIDE_SMS if name == PIPELINED else (self.sm_count - PUSH_SIDE_SMS if name == PUSHED_PIPELINED else 0)
        _check(self.client._lib.rb_set_sm_limit(self.client._ctx, C.c_int32(limit)))

    def align(self):
        """Enqueues a barrier between the GPUs on the compute stream (flag words over peer memory, no host involvement), so that
        the timed region starts on every GPU within microseconds: the host-side barrier before it leaves the ranks up to a
        millisecond apart, which a timed region of a few milliseconds whose steps exchange data would count as step time."""
        exchange = getattr(self, "exchange", None)
        if exchange is not None and not getattr(self, "fused_error", None):
            exchange.barrier()

    def drain(self):
        """Joins the side stream: after it, every step enqueued so far is complete in the compute stream's order."""
        from rust_ascend_b200.runtime import _check
        import ctypes as C
        for slot, used in enumerate(getattr(self, "_slot_used", [])):
            if used:
                _check(self.client._lib.rb_aux_wait(self.client._ctx, C.c_uint32(slot)))

    def choose(self):
        self.errors = {}
        for name, (fn, _) in list(self.candidates.items()):
            try:
                self.prepare(name)
                for i in range(max(4, self.args.warmup)):
                    fn(i)
                self.drain()
                self.client.sync()
                failed = 0.0
            except Exception as error:       # a form that does not run on this machine is left out; the others are still timed
                self.errors[name] = f"{type(error).__name__}: {error}"
                self.client.take_errors()
                failed = 1.0
            # every rank must agree on whether the form is timed (the timed loop exchanges data)
            if max_over_ranks(self.dist, failed) > 0:
                self.candidates.pop(name)
                self._slot_used = [False] * PIPE_DEPTH
                continue
            self.dist.barrier()
            self.align()
            self.client.start_profile()
            for i in range(20):
                fn(i)
            self.drain()
            self.timings[name] = max_over_ranks(self.dist, self.client.end_profile() / 20)
        self.chosen = min(self.timings, key=self.timings.get)
        self.prepare(self.chosen)
        return self.candidates[self.chosen]

    def result(self, i):
        """Device tensor that holds Y after step i (and drain())."""
        if self.chosen == PIPELINED:
            return self.pipe[i % PIPE_DEPTH].gathered()
        if self.chosen == PUSHED_PIPELINED:
            return self.push_pipe[i % PIPE_DEPTH].gathered()
        if self.chosen in (COPIED, COPIED_PIPELINED):
            return self.copy_pipe[i % PIPE_DEPTH].gathered()
        return self.exchange.gathered() if self.chosen.startswith("fused") else None


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Reads SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz, self._stop_flag = index, [], set(), None, threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            # built here, not in run(): scanning the module's names takes the interpreter lock for milliseconds, and the thread
            # starts together with the timed region, whose launches come from the main thread
            self.names = {getattr(pynvml, k): k for k in dir(pynvml) if k.startswith("nvmlClocksThrottleReason") or k.startswith("nvmlClocksEventReason")}
            self.ok = True
        except Exception:  # NVML unavailable: the bench still runs, clocks are reported as null
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv, names = self.nv, self.names
        while not self._stop_flag.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if isinstance(bit, int) and bit and bit & (bit - 1) == 0 and mask & bit:
                        short = name.replace("nvmlClocksThrottleReason", "").replace("nvmlClocksEventReason", "")
                        if short not in ("GpuIdle", "None", "All"):
                            self.reasons.add(short)
            except Exception:
                pass
            time.sleep(0.005)

    def stop(self):
        self._stop_flag.set()
        self.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def dist_setup(n):
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist_mod.init_process_group("gloo")  # host control plane only: barrier and max-over-ranks of the timings
        dist = dist_mod
    return rank, world, local, dist


def max_over_ranks(dist, value: float) -> float:
    if dist is None:
        return value
    import torch
    t = torch.tensor([value], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def cpu_linear_rate(orc, rows: int, seconds_target: float | None = None):
    """Time the oracle's Linear on `rows` rows of the workload (all host threads)."""
    rng = np.random.default_rng(1)
    w = (rng.standard_normal((N, K), dtype=np.float32) * 0.02)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float32)
    x = rng.standard_normal((rows, K), dtype=np.float32)
    t0 = time.perf_counter()
    orc.linear(x, w, bias=bias, out_bf16=True)
    dt = time.perf_counter() - t0
    return 2.0 * rows * N * K / dt / 1e12, dt


def run_reference(args):
    """Reference arm: the CPU oracle port of the same step on the host cores, bounded sample per step."""
    if int(os.environ.get("RANK", 0)) != 0:
        return   # rank 0 alone runs the CPU arm; the other ranks leave without work
    import oracle as orc
    orc.build()
    cores = orc.use_all_cores()
    rate, dt = cpu_linear_rate(orc, 16)
    total_seconds = args.reference_seconds  # target for warmup + steps together
    rows = int(max(1, min(M, (rate * 1e12 * total_seconds / (args.steps + args.warmup)) / (2.0 * N * K))))
    rng = np.random.default_rng(1)
    w = (rng.standard_normal((N, K), dtype=np.float32) * 0.02)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float32)
    x = rng.standard_normal((rows, K), dtype=np.float32)
    for _ in range(args.warmup):
        orc.linear(x, w, bias=bias, out_bf16=True)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.linear(x, w, bias=bias, out_bf16=True)
    dt = (time.perf_counter() - t0) / args.steps
    value = 2.0 * rows * N * K / dt / 1e12
    sample = (f"each step multiplies {rows} of the {M} rows of the 4096x4096x4096 Linear (oracle port: unblocked, unvectorised triple loop, "
              f"f64 accumulate, OpenMP over rows); ms_per_step is the time of that sample, value the rate it implies")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(int(os.environ.get("WORLD_SIZE", args.gpus))),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample, "rows_per_step": rows,
                         "full_step_ms_at_this_rate": dt * 1e3 * (M / rows)},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_ours(args):
    rank, world, local, dist = dist_setup(args.gpus)
    from rust_ascend_b200 import B200Runtime as RT
    from rust_ascend_b200 import DType, RuntimeOptions, Transpose
    from rust_ascend_b200.runtime import f32_to_bf16_bits

    device = RT.initialize_exclusive(RuntimeOptions(device=local))
    client = RT.client(device)
    pk = peaks()
    rng = np.random.default_rng(1 + rank)
    sets = []
    for _ in range(SETS):
        x = client.upload(f32_to_bf16_bits(rng.standard_normal((M, K), dtype=np.float32)))
        w = client.upload(f32_to_bf16_bits(rng.standard_normal((N, K), dtype=np.float32) * 0.02))
        b = client.upload((rng.standard_normal(N) * 0.02).astype(np.float32))
        y = client.tensor((M, N), DType.BF16)
        sets.append((x, w, b, y))

    import ctypes as C
    from rust_ascend_b200.runtime import _check
    keep = [[t._c() for t in st] for st in sets]   # descriptors built once, outside the timed region
    calls = [(client._ctx, C.byref(k[0]), C.byref(k[1]), C.c_int32(0), C.c_int32(1), C.byref(k[2]), None, C.c_int32(1), C.byref(k[3])) for k in keep]
    rb_gemm = client._lib.rb_gemm

    def step(i):
        _check(rb_gemm(*calls[i % SETS]))   # Y = X W^T + bias through the C ABI

    exchange, launches_per_step = None, 1
    if world > 1:
        # N > 1: the same Linear as a row-parallel layer.  Every rank holds its own K shard (X_r [4096,4096], W_r [4096,4096]: one
        # 4096^3 product per rank and step, so the work per GPU is that of the one-GPU step) and every rank ends with
        # Y = sum over ranks of X_r W_r^T + bias.  Two ways to make that sum are timed in warm-up and the faster one is kept:
        # the exchange fused into the kernels over peer memory, and the plain GEMM followed by an NCCL all-reduce.
        exchange = RowParallelHeadline(client, RT, dist, rank, world, sets, args)
        step, launches_per_step = exchange.choose()
    for i in range(args.warmup):
        step(i)
    if exchange is not None:
        exchange.drain()
    client.sync()
    if dist is not None:
        dist.barrier()
    sampler = ClockSampler(local)
    sampler.start()
    if exchange is not None:
        exchange.align()
    launches_before = client.stats()["launches"]
    client.start_profile()
    for i in range(args.steps):
        step(i)
    if exchange is not None:
        exchange.drain()
    total_ms = client.end_profile()
    clocks = sampler.stop()
    gpu_launches = client.stats()["launches"] - launches_before
    if dist is not None:
        dist.barrier()
    total_ms = max_over_ranks(dist, total_ms)
    ms_per_step = total_ms / args.steps
    value = world * FLOPS_PER_STEP / (ms_per_step * 1e-3) / 1e12

    # ---- end to end through the C ABI with host buffers: every step uploads X from pinned host memory, multiplies and
    # reads Y back into pinned host memory.  rb_linear_host is the public call for that: it cuts the rows into chunks so that
    # the upload of one chunk, the GEMM of the previous one and the read-back of the one before run at the same time. ----
    e2e_steps = max(3, min(args.steps, 40))
    chunks = 8
    hx = client.pinned((M, K), np.uint16)
    hy = client.pinned((M, N), np.uint16)
    hx[...] = f32_to_bf16_bits(rng.standard_normal((M, K), dtype=np.float32))
    x, w, b, y = sets[0]
    if exchange is None:
        for _ in range(3):
            RT.linear_host(client, hx, x, w, y, hy, bias=b, row_chunks=chunks)
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            x, w, b, y = sets[i % SETS]
            RT.linear_host(client, hx, x, w, y, hy, bias=b, row_chunks=chunks)   # returns when Y is in host memory
        e2e_s = (time.perf_counter() - t0) / e2e_steps
        # the same three steps one after the other (rb_write, rb_gemm, rb_read), for comparison
        t0 = time.perf_counter()
        for i in range(min(e2e_steps, 10)):
            x, w, b, y = sets[i % SETS]
            client.write(x.handle, hx)
            RT.gemm_into(client, x, w, Transpose.No, Transpose.Yes, y, bias=b)
            client.read_into(y.handle, hy)
        serial_s = (time.perf_counter() - t0) / min(e2e_steps, 10)
        e2e_note = (f"rb_linear_host: every byte of X uploaded and of Y read back inside every timed step, in {chunks} row chunks whose H2D copy, GEMM "
                    "and D2H copy overlap on three streams; W and bias stay resident as module parameters")
    else:
        # row-parallel: every rank uploads its K shard of X, the ranks exchange, every rank reads the whole Y back
        def e2e_step(i):
            st = sets[i % SETS]
            client.write(st[0].handle, hx)
            step(i)
            exchange.drain()
            out = exchange.result(i) or st[3]
            client.read_into(out.handle, hy, out.offset)
        for i in range(3):
            e2e_step(i)
        dist.barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            e2e_step(i)
        e2e_s = max_over_ranks(dist, (time.perf_counter() - t0) / e2e_steps)
        serial_s = e2e_s
        e2e_note = ("every rank uploads its K shard of X (rb_write), runs the row-parallel step and reads the whole Y back (rb_read) inside every timed step; "
                    "W and bias stay resident as module parameters")
    e2e_value = world * FLOPS_PER_STEP / e2e_s / 1e12
    if exchange is not None:
        exchange.drain()
        exchange.prepare(None)        # the secondary measurements start from the default context state (all SMs)

    kernel_tflops = FLOPS_PER_STEP / (ms_per_step * 1e-3) / 1e12
    sustained = total_ms > 1000.0
    peak = pk["bf16_tflops_sustained"] if sustained else pk["bf16_tflops"]
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": workload_config(world),
        "clocks": clocks, "gpu_launches": int(gpu_launches),
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": int(hx.nbytes), "d2h_bytes_per_step": int(hy.nbytes),
                "steps": e2e_steps, "ms_per_step": e2e_s * 1e3, "serial_write_gemm_read_ms": serial_s * 1e3, "note": e2e_note},
        "roofline": {"bound": "tensor", "achieved": kernel_tflops, "peak": peak, "unit": "TFLOP/s", "frac": kernel_tflops / peak,
                     "traffic": 99.5e6, "traffic_source": "ncu dram__bytes_read+write per launch of this kernel and shape, mean of two captured launches (profiles/gemm_bf16_pair_linear4096.txt); algorithmic bytes are 100.7e6", "kernel": "gemm_bf16_pair_kernel", "peak_kind": ("sustained" if sustained else "burst") + " of " + pk["source"],
                     "frac_of_burst": kernel_tflops / pk["bf16_tflops"], "frac_of_sustained": kernel_tflops / pk["bf16_tflops_sustained"],
                     "frac_of_nominal_2250": kernel_tflops / 2250.0},
    }
    if exchange is not None:
        line["exchange"] = {"chosen": exchange.chosen, "us_per_step_in_warm_up": {k: v * 1e3 for k, v in exchange.timings.items()},
                            "bytes_per_rank_and_step": M * N * 2, "fused_error": getattr(exchange, "fused_error", None),
                            "forms_left_out": getattr(exchange, "errors", None) or None}
        line["roofline"]["note"] = "the step is one 4096^3 GEMM per GPU plus the exchange of its result; achieved counts the GEMM's flops over the whole step"
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle as orc
        orc.build()
        orc.use_all_cores()
        rate, _ = cpu_linear_rate(orc, 64)
        rows = int(max(16, min(M, rate * 1e12 * 12.0 / (2.0 * N * K))))
        reps, spent, rates = 0, 0.0, []
        while spent < 10.0 and reps < 16:   # bounded: about 10-30 s of CPU work
            rate, dt = cpu_linear_rate(orc, rows)
            rates.append(rate); spent += dt; reps += 1
        line["cpu_baseline"] = {"value": float(np.median(rates)), "unit": "TFLOP/s", "cores": orc.threads(), "kind": "port",
                                "sample": f"{rows} of {M} rows of the same Linear, {reps} repetitions, {spent:.1f} s, oracle port (f64 accumulate, OpenMP)"}
    # The extras (tensor-parallel decoder over NCCL among them) run under a watchdog: if they do not finish, the
    # headline line is still printed and every rank leaves, so one stuck collective cannot take the whole run down.
    line["tp"] = None            # filled from the decoder-stack measurement below; printed before the longer extras
    line["extras"] = {}
    emitted = threading.Event()

    def emit(note=None):
        if emitted.is_set():
            return
        emitted.set()
        if note:
            line["extras"]["note"] = note
        line["tp"] = tp_summary(line["extras"], world, rank)
        if rank == 0:
            print(json.dumps(line), flush=True)

    def give_up():
        note = f"extras did not finish within {args.extras_timeout} s; what had finished by then is reported"
        try:
            # Every device-side wait is bounded (seconds), so the stream drains by itself; leaving before it has would free
            # buffers that the other ranks' kernels may still be storing into.
            client._lib.rb_sync(client._ctx)
        except Exception:
            pass
        try:
            emit(note)
        except Exception:                      # the main thread was writing into the dictionary being printed
            emitted.clear()
            line["extras"] = {}
            emit(note)
        finally:
            os._exit(0)

    if not args.no_extras:
        dog = threading.Timer(args.extras_timeout, give_up)
        dog.daemon = True
        dog.start()
        try:
            extras(client, RT, pk, args, rank, world, dist, line["extras"])
        except Exception as error:  # an extra must never cost the headline
            line["extras"]["error"] = f"{type(error).__name__}: {error}"
        dog.cancel()
    emit()


TP_N1_FILE = os.path.join(ROOT, "gpurun_out", "bench_tp_decoder_n1.json")
TP_N1_RECORDED_MS = 56.5     # one-GPU forward of the decoder stack measured on this pool earlier; used only when no N=1 run left its file


def tp_summary(extras_out: dict, world: int, rank: int):
    """The tensor-parallel decoder-stack figure as a short top-level object: time per forward, whole-job TFLOP/s, and the
    efficiency T1 / (N * TN) against the one-GPU forward (taken from the file an N=1 run of this script leaves behind, else
    from the recorded constant, and labelled accordingly).  The list of all timed schedules goes to a file, not the line."""
    tpd = extras_out.get("tp_decoder")
    if not tpd:
        return None
    schedules = tpd.pop("schedules_timed", None)
    if rank == 0:
        try:
            os.makedirs(os.path.dirname(TP_N1_FILE), exist_ok=True)
            if schedules is not None:
                json.dump(schedules, open(os.path.join(os.path.dirname(TP_N1_FILE), f"bench_tp_schedules_n{world}.json"), "w"), indent=1)
            if world == 1:
                json.dump({"ms_per_forward": tpd["ms_per_forward"]}, open(TP_N1_FILE, "w"))
        except OSError:
            pass
    t1, source = TP_N1_RECORDED_MS, "recorded constant"
    if world == 1:
        t1, source = tpd["ms_per_forward"], "this run"
    elif tpd.get("t1_this_run_ms"):
        t1, source = tpd["t1_this_run_ms"], "every GPU running the whole batch alone, this run"
    elif os.path.exists(TP_N1_FILE):
        try:
            t1, source = float(json.load(open(TP_N1_FILE))["ms_per_forward"]), "N=1 run on this box"
        except (OSError, ValueError, KeyError):
            pass
    sched = tpd.get("schedule", {})
    return {"workload": "llama_decoder_8L_h4096_b8_s2048_bf16", "parallelism": tpd.get("parallelism"), "ms_per_forward": tpd["ms_per_forward"],
            "value": tpd["value"], "unit": "TFLOP/s (whole job)", "efficiency_vs_n1": t1 / (world * tpd["ms_per_forward"]), "t1_ms": t1, "t1_source": source,
            "schedule": sched.get("parallelism"), "exchanges_per_forward": sched.get("all_reduces_per_forward", 0) + sched.get("fused_exchanges_per_forward", 0),
            "exchange_bytes": 16384 * 4096 * 2}


def extras(client, RT, pk, args, rank, world, dist, out):
    """Secondary kernels of the same hot path, each against its own roofline (reported, not the headline).  Results are
    written into `out` as they arrive, so that a run cut short by the watchdog still reports what finished."""
    from rust_ascend_b200 import DType
    if world > 1:
        # NVLS (in-switch reduction) stays off for every communicator of this process: the watchdog may end a rank while
        # collectives are pending, and a rank that leaves while its memory is bound to an NVLS group can fault its peers.
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        # Order: tensor parallelism over all GPUs (the north-star figure) first, then the row-parallel Linear, then the
        # smaller tensor-parallel groups; whatever the watchdog cuts off is the least important part.
        fused = os.environ.get("RUDA_BENCH_FUSED", "1") != "0"   # the exchange fused into the kernels over peer memory is timed beside NCCL
        candidates = decoder_candidates(world, fused=fused)
        results = []
        decoder_extra(client, pk, rank, world, dist, out, [c for c in candidates if c["tp"] == world], results)
        try:
            out["row_parallel_linear"] = row_parallel_extra(client, pk, rank, world, dist)
        except Exception as error:      # the decoder measurements do not depend on this one
            out["row_parallel_linear"] = {"error": f"{type(error).__name__}: {error}"}
        decoder_extra(client, pk, rank, world, dist, out, [c for c in candidates if c["tp"] != world], results)
        try:
            out["sharded_kernels"] = sharded_extras(client, RT, pk, rank, world, dist)
        except Exception as error:
            out["sharded_kernels"] = {"error": f"{type(error).__name__}: {error}"}
        return out
    rows, width = 4096, 4096
    rng = np.random.default_rng(0)
    sets = []
    for _ in range(6):  # 6 x 128 MiB > L2
        x = client.upload(rng.standard_normal((rows, width), dtype=np.float32))
        w = client.upload(rng.uniform(0.5, 1.5, width).astype(np.float32))
        sets.append((x, w, client.tensor((rows, width), DType.F32), client.tensor((rows,), DType.F32)))
    import ctypes as C
    from rust_ascend_b200.runtime import _check, _ref

    # descriptors are built once: a 23 us kernel must not wait for Python to marshal four structs per launch
    keep = [[t._c() for t in st] for st in sets]
    calls = [(client._ctx, C.byref(k[0]), C.byref(k[1]), C.c_double(1e-6), C.byref(k[2]), C.byref(k[3])) for k in keep]
    fn = client._lib.rb_rms_norm

    def rms(i):
        _check(fn(*calls[i % len(calls)]))
    for i in range(10):
        rms(i)
    client.sync()
    blocks = []
    for _ in range(5):   # median of five timed blocks of 100 launches
        client.start_profile()
        for i in range(100):
            rms(i)
        blocks.append(client.end_profile() / 100)
    ms = float(np.median(blocks))
    nbytes = 2 * rows * width * 4 + width * 4 + rows * 4
    gbs = nbytes / (ms * 1e-3) / 1e9
    out["rms_norm_fp32_4096x4096"] = {"value": gbs, "unit": "GB/s", "us": ms * 1e3,
                                      "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s",
                                                   "frac": gbs / pk["hbm_gbs"], "peak_kind": "copy of " + pk["source"]}}
    for s in sets:
        for t in s:
            client.free(t.handle)
    out.update(attention_extra(client, RT, pk))
    try:
        out.update(gemm_extras(client, RT, pk))
    except Exception as error:
        out["gemm_extras_error"] = f"{type(error).__name__}: {error}"
    decoder_extra(client, pk, rank, world, dist, out, decoder_candidates(world), [])
    if not args.no_cpu_baseline:
        try:
            import oracle as orc
            orc.build()
            orc.use_all_cores()
            out["cpu_baselines"] = cpu_side_baselines(orc)
        except Exception as error:
            out["cpu_baselines"] = {"error": f"{type(error).__name__}: {error}"}
    return out


def sharded_extras(client, RT, pk, rank, world, dist):
    """Configs 1, 3 and 4 split over the GPUs without any exchange (strong scaling: the whole-job work is that of one
    config): RMSNorm by rows, attention by heads (query heads and their KV heads stay together).  Time is the slowest
    rank's; value is whole-job work over that time."""
    import ctypes as C
    from rust_ascend_b200 import DType
    from rust_ascend_b200.runtime import _check, f32_to_bf16_bits
    out = {"scaling": "strong", "n_gpus": world}
    rng = np.random.default_rng(50 + rank)
    rows, width = 4096 // world, 4096
    sets = []
    for _ in range(6):
        x = client.upload(rng.standard_normal((rows, width), dtype=np.float32))
        w = client.upload(rng.uniform(0.5, 1.5, width).astype(np.float32))
        sets.append((x, w, client.tensor((rows, width), DType.F32), client.tensor((rows,), DType.F32)))
    keep = [[t._c() for t in st] for st in sets]
    calls = [(client._ctx, C.byref(k[0]), C.byref(k[1]), C.c_double(1e-6), C.byref(k[2]), C.byref(k[3])) for k in keep]
    for i in range(10):
        _check(client._lib.rb_rms_norm(*calls[i % 6]))
    client.sync()
    if dist is not None:
        dist.barrier()
    client.start_profile()
    for i in range(200):
        _check(client._lib.rb_rms_norm(*calls[i % 6]))
    ms = max_over_ranks(dist, client.end_profile() / 200)
    nbytes = 2 * 4096 * width * 4 + width * 4 + 4096 * 4
    out["rms_norm_fp32_4096x4096_by_rows"] = {"value": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s (whole job)", "us": ms * 1e3, "rows_per_gpu": rows}
    for st in sets:
        for t in st:
            client.free(t.handle)
    for name, (b, hq, hkv, s) in {"attention_causal_b4_h32_s2048_d128_by_heads": (4, 32, 32, 2048),
                                   "attention_causal_gqa_b2_h32_kv8_s4096_d128_by_heads": (2, 32, 8, 4096)}.items():
        if hkv % world:
            out[name] = {"skipped": f"{hkv} KV heads do not divide over {world} GPUs"}
            continue
        lq, lkv = hq // world, hkv // world
        mk = lambda h: client.upload(f32_to_bf16_bits(rng.standard_normal((b, h, s, 128), dtype=np.float32)))
        sets = [(mk(lq), mk(lkv), mk(lkv), client.tensor((b, s, lq, 128), DType.BF16)) for _ in range(3)]
        run = lambda i: RT.attention(client, sets[i % 3][0], sets[i % 3][1], sets[i % 3][2], 128 ** -0.5, causal=True, bmhd_output=True, out=sets[i % 3][3])
        for i in range(5):
            run(i)
        client.sync()
        if dist is not None:
            dist.barrier()
        client.start_profile()
        for i in range(30):
            run(i)
        ms = max_over_ranks(dist, client.end_profile() / 30)
        out[name] = {"value": 2 * b * hq * s * s * 128 / (ms * 1e-3) / 1e12, "unit": "TFLOP/s (whole job)", "us": ms * 1e3, "query_heads_per_gpu": lq, "kv_heads_per_gpu": lkv}
        for st in sets:
            for t in st:
                client.free(t.handle)
    return out


def cpu_side_baselines(orc):
    """The oracle port of the secondary kernels on the host cores, beside their GPU numbers: RMSNorm at config 1's full size
    and causal attention on one (batch, head) pair of config 3 (the flops of that pair; the full config is 128 such pairs)."""
    out = {"cores": orc.threads(), "kind": "port"}
    rng = np.random.default_rng(0)
    x = rng.standard_normal((4096, 4096), dtype=np.float32); w = rng.uniform(0.5, 1.5, 4096).astype(np.float32)
    orc.rms_norm(x[:64], w, 1e-6)
    times = []
    for _ in range(3):
        t0 = time.perf_counter(); orc.rms_norm(x, w, 1e-6); times.append(time.perf_counter() - t0)
    dt = float(np.median(times))
    out["rms_norm_fp32_4096x4096"] = {"value": (2 * x.nbytes + w.nbytes + 4096 * 4) / dt / 1e9, "unit": "GB/s", "ms": dt * 1e3, "sample": "full size, median of 3"}
    s, d = 2048, 128
    q, k, v = (rng.standard_normal((1, 1, s, d), dtype=np.float32) for _ in range(3))
    t0 = time.perf_counter(); orc.attention(q, k, v, d ** -0.5, causal=True); dt = time.perf_counter() - t0
    out["attention_causal_s2048_d128"] = {"value": 2 * s * s * d / dt / 1e12, "unit": "TFLOP/s", "ms": dt * 1e3,
                                          "sample": "1 of the 128 (batch, head) pairs of config 3, once"}
    return out


def gemm_extras(client, RT, pk):
    """Configuration 2b (X [8192,4096] against gate and up weights [11008,4096], SiLU(g)*u fused into the store: one launch) and the
    headline GEMM held for more than a second, where the 1 kW power cap sets the clock (compared with the sustained peak)."""
    import ctypes as C
    from rust_ascend_b200 import DType
    from rust_ascend_b200.runtime import _check, f32_to_bf16_bits
    out = {}
    rng = np.random.default_rng(22)
    m, n, k = 8192, 11008, 4096
    block = f32_to_bf16_bits(rng.standard_normal((2048, k), dtype=np.float32))
    x = client.upload(np.tile(block, (m // 2048, 1)))
    wblock = f32_to_bf16_bits(rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
    wg, wu = client.upload(wblock), client.upload(np.roll(wblock, 7, axis=0))
    y = client.tensor((m, n), DType.BF16)
    keep = [t._c() for t in (x, wg, wu, y)]
    call = (client._ctx, C.byref(keep[0]), C.byref(keep[1]), C.c_int32(0), C.c_int32(1), None, C.byref(keep[2]), C.c_int32(2), C.byref(keep[3]))
    for _ in range(3):
        _check(client._lib.rb_gemm(*call))
    client.sync()
    client.start_profile()
    for _ in range(20):
        _check(client._lib.rb_gemm(*call))
    ms = client.end_profile() / 20
    tf = 2 * 2 * m * n * k / (ms * 1e-3) / 1e12
    out["swiglu_gemm_8192x11008x4096"] = {"value": tf, "unit": "TFLOP/s", "us": ms * 1e3, "l2": "operands 408 MiB > 126 MB L2",
                                          "roofline": {"bound": "tensor", "achieved": tf, "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": tf / pk["bf16_tflops"],
                                                       "peak_kind": "burst of " + pk["source"], "frac_of_sustained": tf / pk["bf16_tflops_sustained"]}}
    for t in (x, wg, wu, y):
        client.free(t.handle)
    sets = []
    for _ in range(SETS):
        sets.append((client.upload(f32_to_bf16_bits(rng.standard_normal((M, K), dtype=np.float32))),
                     client.upload(f32_to_bf16_bits(rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02))),
                     client.upload((rng.standard_normal(N) * 0.02).astype(np.float32)), client.tensor((M, N), DType.BF16)))
    keep = [[t._c() for t in st] for st in sets]
    calls = [(client._ctx, C.byref(q[0]), C.byref(q[1]), C.c_int32(0), C.c_int32(1), C.byref(q[2]), None, C.c_int32(1), C.byref(q[3])) for q in keep]
    for i in range(50):
        _check(client._lib.rb_gemm(*calls[i % SETS]))
    client.sync()
    sampler = ClockSampler(0)
    sampler.start()
    launches = 12000                       # more than a second of back-to-back launches
    client.start_profile()
    for i in range(launches):
        _check(client._lib.rb_gemm(*calls[i % SETS]))
    total_ms = client.end_profile()
    clocks = sampler.stop()
    us = total_ms / launches * 1e3
    tf = FLOPS_PER_STEP / (us * 1e-6) / 1e12
    out["linear_gemm_4096_sustained"] = {"value": tf, "unit": "TFLOP/s", "us": us, "seconds": total_ms * 1e-3, "clocks": clocks,
                                         "us_times_sm_ghz": (us * clocks["sm_mhz"] * 1e-3) if clocks.get("sm_mhz") else None,
                                         "roofline": {"bound": "tensor", "achieved": tf, "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                                                      "frac": tf / pk["bf16_tflops_sustained"], "peak_kind": "sustained of " + pk["source"]}}
    for st in sets:
        for t in st:
            client.free(t.handle)
    return out


def attention_extra(client, RT, pk):
    """Causal attention at configs 3 and 4 (flops = the causal half, 2*B*H*S^2*D)."""
    from rust_ascend_b200 import DType
    from rust_ascend_b200.runtime import f32_to_bf16_bits
    out = {}
    rng = np.random.default_rng(3)
    for name, (b, hq, hkv, s) in {"attention_causal_b4_h32_s2048_d128": (4, 32, 32, 2048),
                                   "attention_causal_gqa_b2_h32_kv8_s4096_d128": (2, 32, 8, 4096)}.items():
        sets = []
        for _ in range(3):  # 3 x (Q,K,V,O) > 126 MB L2
            mk = lambda h: client.upload(f32_to_bf16_bits(rng.standard_normal((b, h, s, 128), dtype=np.float32)))
            sets.append((mk(hq), mk(hkv), mk(hkv), client.tensor((b, s, hq, 128), DType.BF16)))
        run = lambda i: RT.attention(client, sets[i % 3][0], sets[i % 3][1], sets[i % 3][2], 128 ** -0.5, causal=True, bmhd_output=True, out=sets[i % 3][3])
        for i in range(5):
            run(i)
        client.sync()
        client.start_profile()
        for i in range(30):
            run(i)
        ms = client.end_profile() / 30
        tf = 2 * b * hq * s * s * 128 / (ms * 1e-3) / 1e12
        out[name] = {"value": tf, "unit": "TFLOP/s", "us": ms * 1e3,
                     "roofline": {"bound": "tensor", "achieved": tf, "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": tf / pk["bf16_tflops"],
                                  "peak_kind": "burst of " + pk["source"]}}
        for st in sets:
            for t in st:
                client.free(t.handle)
    return out


def row_parallel_extra(client, pk, rank, world, dist):
    """Config 2a as a row-parallel Linear: every rank holds K/world columns of X [4096, 4096] and W [4096, 4096] and the
    partial products are summed on every rank: by one NCCL all-reduce of the BF16 [4096, 4096] result, and by the exchange fused
    into the kernels over peer memory.  Strong scaling: whole-job flops are those of the one full product."""
    from rust_ascend_b200 import DType
    from rust_ascend_b200.distributed import NcclCommunicator, TorchControl
    from rust_ascend_b200.runtime import f32_to_bf16_bits
    os.environ.pop("RUDA_NCCL_MAX_CTAS", None)
    comm = NcclCommunicator.initialize(TorchControl(), client)
    rng = np.random.default_rng(100 + rank)
    k = K // world
    x = client.upload(f32_to_bf16_bits(rng.standard_normal((M, k), dtype=np.float32)))
    w = client.upload(f32_to_bf16_bits(rng.standard_normal((N, k), dtype=np.float32) * np.float32(0.02)))
    result = {"config": f"X [{M}, {K}/{world}] . W [{N}, {K}/{world}]^T summed over {world} ranks, BF16 result on every rank", "unit": "TFLOP/s (whole job)"}
    import ctypes as C
    from rust_ascend_b200.runtime import _check
    y = client.tensor((M, N), DType.BF16)
    keep = [x._c(), w._c(), y._c()]

    def call(overlap):
        _check(client._lib.rb_row_parallel_linear_allreduce(comm.native._comm, C.byref(keep[0]), C.byref(keep[1]), C.byref(keep[2]), C.c_int32(int(overlap))))
    variants = {"gemm_then_nccl_all_reduce": lambda: call(False)}
    try:
        from rust_ascend_b200.fused import FusedExchange, row_parallel_linear_allreduce
        ex = FusedExchange(client, TorchControl(), M, N)
        variants["fused_scatter_reduce_push"] = lambda: row_parallel_linear_allreduce(ex, x, w)
        px = FusedExchange(client, TorchControl(), M, N, activations=ex.activations, pull=True)
        variants["gemm_then_pull_reduce_push"] = lambda: row_parallel_linear_allreduce(px, x, w)
    except Exception as error:
        result["fused_error"] = f"{type(error).__name__}: {error}"
    for name, fn in variants.items():
        for _ in range(5):
            fn()
        client.sync()
        if dist is not None:
            dist.barrier()
        steps = 20
        client.start_profile()
        for _ in range(steps):
            fn()
        ms = max_over_ranks(dist, client.end_profile() / steps)
        result[name] = {"us": ms * 1e3, "value": 2.0 * M * N * K / (ms * 1e-3) / 1e12}
    return result


def decoder_candidates(world: int, sequences: int = 8, fused: bool = False):
    """What the decoder extra times at `world` GPUs: pure tensor parallelism first (three schedules), then tensor-parallel
    groups of world/2, world/4, ... GPUs that each take their own share of the sequences, and last plain replicas (every GPU
    runs whole sequences, no exchange).  Every entry names its tensor-parallel degree `tp`; the others split the batch."""
    overlap = {"micro_batches": 2, "sms_left_to_nccl": NCCL_CTAS, "nccl_max_ctas": NCCL_CTAS}   # all-reduce under the other group's GEMMs
    plain = {"micro_batches": 1, "sms_left_to_nccl": 0, "nccl_max_ctas": 0}                      # sequential, NCCL at full width
    if world == 1:
        # one GPU: the whole batch at once, and in groups of sequences one after the other (smaller activations stay in L2
        # between the kernels of a layer)
        return [dict(plain, tp=1)] + [dict(plain, tp=1, micro_batches=n) for n in (2, 4) if sequences % n == 0]
    out = [dict(overlap, tp=world), dict(plain, tp=world), dict(plain, tp=world, micro_batches=2)]
    if fused:   # exchange fused into the kernels over peer memory: on one stream, and with the owner-side step on the side stream
        out += [dict(plain, tp=world, fused=True), dict(overlap, tp=world, fused=True, overlap_exchange=True, nccl_max_ctas=0)]
        # pull form: plain GEMMs, the owner-side kernel fetches the partial products (all link traffic on the side stream)
        out += [dict(plain, tp=world, fused=True, pull_exchange=True),
                dict(overlap, tp=world, fused=True, overlap_exchange=True, pull_exchange=True, nccl_max_ctas=0)]
        if sequences % 4 == 0 and (sequences // 4 * 2048) % (128 * world) == 0:
            out.append(dict(overlap, tp=world, fused=True, overlap_exchange=True, pull_exchange=True, nccl_max_ctas=0, micro_batches=4))
        for sms in (NCCL_CTAS // 2, NCCL_CTAS * 5 // 4, NCCL_CTAS * 3 // 2, NCCL_CTAS * 7 // 4, 2 * NCCL_CTAS):
            out.append(dict(overlap, tp=world, fused=True, overlap_exchange=True, pull_exchange=True, nccl_max_ctas=0, sms_left_to_nccl=sms))
        if sequences % 4 == 0 and (sequences // 4 * 2048) % (128 * world) == 0:
            out.append(dict(overlap, tp=world, fused=True, overlap_exchange=True, pull_exchange=True, nccl_max_ctas=0, micro_batches=4,
                            sms_left_to_nccl=NCCL_CTAS * 3 // 2))
        # side-scatter form: plain GEMMs, the rows go to their owners by a kernel of posted stores (on the side stream when overlapped)
        out.append(dict(plain, tp=world, fused=True, side_scatter=True))
        for sms in (NCCL_CTAS // 2, NCCL_CTAS, NCCL_CTAS * 3 // 2):
            out.append(dict(overlap, tp=world, fused=True, overlap_exchange=True, side_scatter=True, nccl_max_ctas=0, sms_left_to_nccl=sms))
        # copy form: device-to-device copies move the data (copy engines), only the owner-side arithmetic is a kernel, and the
        # GEMMs beside it keep every SM
        out.append(dict(plain, tp=world, fused=True, dma_exchange=True))
        for n in (2, 4):
            if sequences % n == 0 and (sequences // n * 2048) % (128 * world) == 0:
                out.append(dict(plain, tp=world, fused=True, dma_exchange=True, overlap_exchange=True, micro_batches=n))
    tp = world // 2
    while tp >= 1:
        per_group = sequences * tp // world
        if per_group >= 1 and sequences * tp % world == 0:
            if tp > 1 and per_group >= 2:
                out.append(dict(overlap, tp=tp))
            out.append(dict(plain, tp=tp))
        tp //= 2
    # T1 of the same run: every GPU runs the whole batch alone (what the efficiency of tensor parallelism is measured against)
    out += [dict(plain, tp=1, whole_batch=True), dict(plain, tp=1, whole_batch=True, micro_batches=4)]
    return out


def decoder_extra(client, pk, rank, world, dist, sink, candidates, results):
    """Config 5: Llama-style stack, 8 layers, T = 8 x 2048.  The reported value is tensor parallelism over all `world` GPUs
    with NCCL all-reduces (fastest of three schedules); the same forward with smaller tensor-parallel groups that split the
    sequences between them is timed too and reported beside it, labelled with its parallelism."""
    from rust_ascend_b200.decoder import LlamaConfig, TensorParallelDecoder
    cfg = LlamaConfig()
    sequences, seq = 8, 2048
    tokens = np.random.default_rng(5).integers(0, cfg.vocab, size=(sequences, seq)).astype(np.int32)
    if world > 1:
        from rust_ascend_b200.distributed import GroupControl, NcclCommunicator, TorchControl, tensor_parallel_groups
        # NVLS (in-switch reduction) stays off: the watchdog may end a rank while collectives are pending, and a rank that
        # leaves while its memory is bound to an NVLS group can fault its peers.  Ring/tree all-reduce is used instead.
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    comms, models = {}, {}
    total_flops = cfg.flops(sequences * seq, seq)

    def summary():
        pure = [r for r in results if r["tp"] == world]
        best = min(pure, key=lambda r: r["ms_per_forward"])
        tf = total_flops / (best["ms_per_forward"] * 1e-3) / 1e12
        out = {"value": tf, "unit": "TFLOP/s (whole job)", "ms_per_forward": best["ms_per_forward"], "n_gpus": world, "cuda_graph": True,
               "parallelism": f"tp{world}", "schedule": best, "schedules_timed": list(results),
               "config": "8 layers, hidden 4096, 32q/8kv heads, ffn 14336, vocab 32000, batch 8 x seq 2048, BF16",
               "frac_of_sustained_peak_per_gpu": tf / world / pk["bf16_tflops_sustained"]}
        whole = [r for r in results if r.get("whole_batch")]
        if whole:
            out["t1_this_run_ms"] = min(r["ms_per_forward"] for r in whole)
        mixed = [r for r in results if r["tp"] != world and not r.get("whole_batch")]
        if mixed:
            b = min(mixed, key=lambda r: r["ms_per_forward"])
            out["smaller_groups_best"] = {"parallelism": b["parallelism"], "ms_per_forward": b["ms_per_forward"],
                                          "value": total_flops / (b["ms_per_forward"] * 1e-3) / 1e12, "unit": "TFLOP/s (whole job)"}
        return out

    for cand in candidates:
        tp = cand["tp"]
        groups = world // tp
        group, tp_rank = rank // tp, rank % tp
        comm = None
        if tp > 1:
            cap = cand["nccl_max_ctas"]
            if (tp, cap) not in comms:
                if cap:
                    os.environ["RUDA_NCCL_MAX_CTAS"] = str(cap)
                else:
                    os.environ.pop("RUDA_NCCL_MAX_CTAS", None)
                control = TorchControl() if tp == world else GroupControl(TorchControl(), tensor_parallel_groups(world, tp)[group])
                comms[(tp, cap)] = NcclCommunicator.initialize(control, client)
            comm = comms[(tp, cap)]
        per_group = sequences if cand.get("whole_batch") else sequences // groups
        first = 0 if cand.get("whole_batch") else group * per_group
        key = (tp, per_group)
        if key not in models:
            for other in models.values():
                other.close()
            models.clear()
            models[key] = TensorParallelDecoder(client, cfg, per_group, seq, comm=comm, rank=tp_rank, world=tp, micro_batches=cand["micro_batches"],
                                               sm_reserve=cand["sms_left_to_nccl"], use_graph=True, fused=cand.get("fused", False),
                                               overlap_exchange=cand.get("overlap_exchange", False), pull_exchange=cand.get("pull_exchange", False),
                                               dma_exchange=cand.get("dma_exchange", False), side_scatter=cand.get("side_scatter", False))
        else:
            models[key].configure(comm, cand["micro_batches"], cand["sms_left_to_nccl"], True, cand.get("fused", False), cand.get("overlap_exchange", False),
                                 cand.get("pull_exchange", False), cand.get("dma_exchange", False), cand.get("side_scatter", False))
        model = models[key]
        model.forward(tokens[first:first + per_group])
        for _ in range(2):
            model.forward()
        client.sync()
        if dist is not None:
            dist.barrier()
        steps = 6
        if getattr(model, "_exchanges", None):      # fused forms: the GPUs start the timed forwards together (see RowParallelHeadline.align)
            model._exchanges[0].barrier()
        client.start_profile()
        for _ in range(steps):
            model.forward()
        ms = max_over_ranks(dist, client.end_profile() / steps)
        label = "every GPU runs the whole batch alone (T1 of this run)" if cand.get("whole_batch") else f"tp{tp}" if groups == 1 else (f"tp{tp} x {groups} groups of {per_group} sequences" if tp > 1 else f"{groups} replicas of {per_group} sequences, no exchange")
        if tp == 1 and cand["micro_batches"] > 1:
            label += f", in {cand['micro_batches']} groups of sequences one after the other"
        if cand.get("fused"):
            label += (", exchange by device-to-device copies and a local owner-side kernel" if cand.get("dma_exchange") else
                      ", rows scattered to their owners by a kernel of posted stores" if cand.get("side_scatter") else
                      ", partial products pulled by the owner-side kernel" if cand.get("pull_exchange") else ", exchange fused into the kernels") \
                + (" and overlapped on the side stream" if cand.get("overlap_exchange") else "")
            if cand["micro_batches"] > 2:
                label += f", {cand['micro_batches']} micro batches"
            if cand.get("overlap_exchange") and cand["sms_left_to_nccl"] != NCCL_CTAS and not cand.get("dma_exchange"):
                label += f", {cand['sms_left_to_nccl']} SMs left to the side stream"
        results.append(dict(cand, parallelism=label, ms_per_forward=ms, launches_per_forward=model.launches_per_forward,
                            all_reduces_per_forward=model.collectives_per_forward, fused_exchanges_per_forward=model.fused_exchanges_per_forward))
        sink["tp_decoder"] = summary()
    for model in models.values():
        model.close()
    return sink.get("tp_decoder")


def run_single_kernel(args):
    """`--kernel NAME`: W + K launches of one kernel of the path on its bench workload and a one-line JSON with the
    CUDA-event time per launch.  This is the command the ncu captures under profiles/ run."""
    from rust_ascend_b200 import B200Runtime as RT
    from rust_ascend_b200 import DType, RuntimeOptions, Transpose
    from rust_ascend_b200.runtime import f32_to_bf16_bits
    import ctypes as C
    from rust_ascend_b200.runtime import _check, _ref
    client = RT.client(RT.initialize_exclusive(RuntimeOptions(device=0)))
    rng = np.random.default_rng(0)
    bf = lambda *shape, scale=1.0: client.upload(f32_to_bf16_bits(rng.standard_normal(shape, dtype=np.float32) * np.float32(scale)))
    if args.kernel == "gemm":
        sets = [(bf(M, K), bf(N, K, scale=0.02), client.upload((rng.standard_normal(N) * 0.02).astype(np.float32)), client.tensor((M, N), DType.BF16)) for _ in range(SETS)]
        run = lambda i: RT.gemm_into(client, sets[i % SETS][0], sets[i % SETS][1], Transpose.No, Transpose.Yes, sets[i % SETS][3], bias=sets[i % SETS][2])
        work, unit = FLOPS_PER_STEP, "TFLOP/s"
    elif args.kernel == "attention":
        b, h, s = 4, 32, 2048
        sets = [(bf(b, h, s, 128), bf(b, h, s, 128), bf(b, h, s, 128), client.tensor((b, s, h, 128), DType.BF16)) for _ in range(3)]
        run = lambda i: RT.attention(client, sets[i % 3][0], sets[i % 3][1], sets[i % 3][2], 128 ** -0.5, causal=True, bmhd_output=True, out=sets[i % 3][3])
        work, unit = 2 * b * h * s * s * 128, "TFLOP/s"
    else:
        rows = width = 4096
        sets = [(client.upload(rng.standard_normal((rows, width), dtype=np.float32)), client.upload(rng.uniform(0.5, 1.5, width).astype(np.float32)),
                 client.tensor((rows, width), DType.F32), client.tensor((rows,), DType.F32)) for _ in range(6)]
        run = lambda i: _check(client._lib.rb_rms_norm(client._ctx, _ref(sets[i % 6][0]), _ref(sets[i % 6][1]), C.c_double(1e-6), _ref(sets[i % 6][2]), _ref(sets[i % 6][3])))
        work, unit = 2 * rows * width * 4 + width * 4 + rows * 4, "GB/s"
    for i in range(args.warmup):
        run(i)
    client.sync()
    client.start_profile()
    for i in range(args.steps):
        run(i)
    ms = client.end_profile() / args.steps
    rate = work / (ms * 1e-3) / (1e12 if unit == "TFLOP/s" else 1e9)
    print(json.dumps({"kernel": args.kernel, "us_per_launch": ms * 1e3, "value": rate, "unit": unit, "steps": args.steps, "warmup": args.warmup}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--extras-timeout", type=float, default=200.0, help="seconds before the secondary measurements are abandoned")
    ap.add_argument("--reference-seconds", type=float, default=90.0, help="CPU time the reference arm aims to spend over warm-up and steps together")
    ap.add_argument("--kernel", default=None, choices=["gemm", "attention", "rms_norm"], help="time one kernel alone (profiling helper)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.kernel:
        run_single_kernel(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
