"""Two GPUs: peer buffers, the fused row-parallel projection (scatter GEMM + owner-side reduce + push) against a host
reference and against the NCCL path, and the decoder in fused mode against the same host reference the NCCL decoder meets.

These kernels store into another GPU's memory and wait on flags that another GPU sets; every wait in the kernels is bounded
(a few seconds) and the workers are joined with a deadline, so a protocol error ends as a failed test, not as a hang.  The
single-GPU test runs the same kernels as a world of one, where every store, flag and wait stays in local memory."""
import os
import socket
import sys
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cfg():
    from rust_ascend_b200.decoder import LlamaConfig
    return LlamaConfig(layers=2, hidden=256, heads=4, kv_heads=2, head_dim=128, ffn=512, vocab=1024)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(world, tokens=512, hidden=320, k=192):
    rng = np.random.default_rng(17)
    x = rng.standard_normal((tokens, k * world)).astype(np.float32)
    w = (rng.standard_normal((hidden, k * world)) * 0.05).astype(np.float32)
    return x, w


def _worker(rank, world, port, results):
    for p in (ROOT, os.path.join(ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from rust_ascend_b200 import B200Runtime as RT
    from rust_ascend_b200 import DType, RuntimeOptions
    from rust_ascend_b200.decoder import TensorParallelDecoder
    from rust_ascend_b200.distributed import NcclCommunicator, TorchControl
    from rust_ascend_b200.fused import FusedExchange, PeerBuffer, row_parallel_linear_allreduce
    from rust_ascend_b200.runtime import TensorBuffer, bf16_bits_to_f32, f32_to_bf16_bits
    client = RT.client(RT.initialize_exclusive(RuntimeOptions(device=rank)))
    control = TorchControl()
    out = {}
    # 1. peer buffer: every rank writes its own buffer, then reads everybody's through the mapping
    buf = PeerBuffer(client, control, 4096)
    mine = np.full(1024, 1000 + rank, np.int32)
    client.write(buf.handles[rank], mine); client.sync()
    control.all_gather_bytes(b"written")
    out["peer"] = [int(client.read(buf.view(r, (1024,), DType.I32))[5]) for r in range(world)]
    control.all_gather_bytes(b"read")
    buf.close()
    # 2. fused row-parallel Linear + all-reduce, twice on the same exchange (buffer reuse), against NumPy
    x, w = _inputs(world)
    k = x.shape[1] // world
    xs = client.upload(f32_to_bf16_bits(x[:, rank * k:(rank + 1) * k]))
    ws = client.upload(f32_to_bf16_bits(w[:, rank * k:(rank + 1) * k]))
    ex = FusedExchange(client, control, x.shape[0], w.shape[0])
    y1 = bf16_bits_to_f32(client.read(row_parallel_linear_allreduce(ex, xs, ws)))
    y2 = bf16_bits_to_f32(client.read(row_parallel_linear_allreduce(ex, xs, ws)))
    out["fused_linear"], out["fused_linear_again_equal"] = y1, bool(np.array_equal(y1, y2))
    # pull form: plain GEMM into this rank's own buffer, the owner-side kernel fetches its rows from every rank; the second call
    # runs on other inputs, so a stale read of a peer's buffer cannot go unnoticed
    px = FusedExchange(client, control, x.shape[0], w.shape[0], pull=True)
    out["pull_linear"] = bf16_bits_to_f32(client.read(row_parallel_linear_allreduce(px, xs, ws)))
    xs2 = client.upload(f32_to_bf16_bits(-2.0 * x[:, rank * k:(rank + 1) * k]))
    out["pull_linear_scaled"] = bf16_bits_to_f32(client.read(row_parallel_linear_allreduce(px, xs2, ws)))
    client.sync()
    px.close()
    # side-scatter form: plain GEMM, then a kernel of posted stores takes the rows to their owners
    sx = FusedExchange(client, control, x.shape[0], w.shape[0], side_scatter=True)
    out["side_linear"] = bf16_bits_to_f32(client.read(row_parallel_linear_allreduce(sx, xs, ws)))
    out["side_linear_scaled"] = bf16_bits_to_f32(client.read(row_parallel_linear_allreduce(sx, xs2, ws)))
    client.sync()
    sx.close()
    # copy form: device-to-device copies between the mapped buffers move the data, the owner-side arithmetic runs locally
    cx = FusedExchange(client, control, x.shape[0], w.shape[0], dma=True)
    out["copy_linear"] = bf16_bits_to_f32(client.read(row_parallel_linear_allreduce(cx, xs, ws)))
    out["copy_linear_scaled"] = bf16_bits_to_f32(client.read(row_parallel_linear_allreduce(cx, xs2, ws)))
    client.sync()
    cx.close()
    # residual + RMSNorm folded into the owner-side step
    rows = x.shape[0] // world
    resid = np.random.default_rng(5).standard_normal((x.shape[0], w.shape[0])).astype(np.float32)
    weight = np.random.default_rng(6).uniform(0.5, 1.5, w.shape[0]).astype(np.float32)
    x_own = client.upload(f32_to_bf16_bits(resid[rank * rows:(rank + 1) * rows]))
    ex.gemm_scatter(xs, ws); ex.wait_scatter()
    ex.reduce_norm_push(x_in=x_own, weight=client.upload(f32_to_bf16_bits(weight)), eps=1e-5, x_out=x_own)
    ex.wait_gather(); ex.barrier()
    out["normed"] = bf16_bits_to_f32(client.read(ex.gathered()))
    out["residual_rows"] = bf16_bits_to_f32(client.read(x_own))
    client.sync()
    ex.close()
    # 3. the decoder: fused mode against the NCCL mode on the same weights and tokens
    comm = NcclCommunicator.initialize(control, client)
    for overlap in (False, True):   # the NCCL form of the same projection, sequential and in row chunks
        y = comm.native.row_parallel_linear_allreduce(xs, ws, DType.BF16, overlap)
        out[f"nccl_linear_{int(overlap)}"] = bf16_bits_to_f32(client.read(y))
    cfg = _cfg()
    tokens = np.random.default_rng(0).integers(0, cfg.vocab, size=(2, 128)).astype(np.int32)
    for name, kwargs in (("nccl", {}), ("fused", {"fused": True}), ("fused_graph", {"fused": True, "use_graph": True}),
                         ("pull_graph", {"fused": True, "use_graph": True, "pull_exchange": True}),
                         ("copy_graph", {"fused": True, "use_graph": True, "dma_exchange": True})):
        model = TensorParallelDecoder(client, cfg, 2, 128, comm=comm, rank=rank, world=world, seed=3, exact_weights=True, **kwargs)
        model.forward(tokens)
        out[name] = bf16_bits_to_f32(client.read(model.forward()))
        model.close()
    # overlapped exchange: two micro batches, the owner-side step on the side stream under the other batch's GEMMs
    tokens4 = np.random.default_rng(1).integers(0, cfg.vocab, size=(4, 128)).astype(np.int32)
    for name, kwargs in (("fused4", {"fused": True}), ("fused4_overlap", {"fused": True, "micro_batches": 2, "overlap_exchange": True, "sm_reserve": 16, "use_graph": True}),
                         ("pull4_overlap", {"fused": True, "micro_batches": 2, "overlap_exchange": True, "pull_exchange": True, "sm_reserve": 16, "use_graph": True}),
                         ("copy4_overlap", {"fused": True, "micro_batches": 2, "overlap_exchange": True, "dma_exchange": True, "use_graph": True}),
                         ("side4_overlap", {"fused": True, "micro_batches": 2, "overlap_exchange": True, "side_scatter": True, "sm_reserve": 16, "use_graph": True})):
        model = TensorParallelDecoder(client, cfg, 4, 128, comm=comm, rank=rank, world=world, seed=3, exact_weights=True, **kwargs)
        model.forward(tokens4)
        out[name] = bf16_bits_to_f32(client.read(model.forward()))
        model.close()
    results[rank] = out
    comm.native.destroy()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_gpu_fused_exchange(oracle):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from decoder_reference import forward, full_weights
    from test_index_padded import bf16
    world, port = 2, _free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        ctx = mp.spawn(_worker, args=(world, port, results), nprocs=world, join=False)
        deadline = time.time() + 240
        while not ctx.join(timeout=5):
            if time.time() > deadline:   # a rank is stuck: end exactly the processes this test started
                for proc in ctx.processes:
                    if proc.is_alive():
                        proc.terminate()
                pytest.fail("two-GPU workers did not finish within 240 s")
        r = {k: dict(v) for k, v in results.items()}
    x, w = _inputs(world)
    k = x.shape[1] // world
    partial = [bf16(bf16(x[:, i * k:(i + 1) * k]) @ bf16(w[:, i * k:(i + 1) * k]).T) for i in range(world)]   # each rank's BF16 partial tile
    total = bf16(sum(partial))
    for rank in range(world):
        assert r[rank]["peer"] == [1000, 1001]
        assert r[rank]["fused_linear_again_equal"]
        got = r[rank]["fused_linear"]
        assert got.shape == total.shape
        err = np.abs(got - total)
        assert err.max() <= 2.0 ** -7 * np.abs(total).max() and err.mean() <= 1e-3 * np.abs(total).mean() + 1e-6, (err.max(), err.mean())
        np.testing.assert_array_equal(got, r[0]["fused_linear"])          # every rank holds the same bits
        np.testing.assert_array_equal(r[rank]["pull_linear"], got)        # the pull form sums the same partial products in the same order
        np.testing.assert_array_equal(r[rank]["pull_linear_scaled"], -2.0 * got)   # exact: a power of two scales every BF16 value exactly
        np.testing.assert_array_equal(r[rank]["side_linear"], got)
        np.testing.assert_array_equal(r[rank]["side_linear_scaled"], -2.0 * got)
        np.testing.assert_array_equal(r[rank]["copy_linear"], got)
        np.testing.assert_array_equal(r[rank]["copy_linear_scaled"], -2.0 * got)
        for key in ("nccl_linear_0", "nccl_linear_1"):
            assert np.abs(r[rank][key] - total).max() <= 2.0 ** -7 * np.abs(total).max()
    rows = x.shape[0] // world
    resid = np.random.default_rng(5).standard_normal(total.shape).astype(np.float32)
    weight = bf16(np.random.default_rng(6).uniform(0.5, 1.5, total.shape[1]).astype(np.float32))
    xn = bf16(bf16(resid) + r[0]["fused_linear"])                          # residual update with the sums the GPUs produced
    want = bf16(xn / np.sqrt((xn ** 2).mean(-1, keepdims=True) + 1e-5) * weight)
    for rank in range(world):
        got_x = r[rank]["residual_rows"]; want_x = xn[rank * rows:(rank + 1) * rows]
        assert np.abs(got_x - want_x).max() <= 2.0 ** -8 * np.abs(want_x).max()   # FP32 add then BF16 rounding against f64: at most one ulp
        err = np.abs(r[rank]["normed"] - want)
        assert err.max() <= 2.0 ** -7 * np.abs(want).max(), err.max()
    cfg = _cfg()
    tokens = np.random.default_rng(0).integers(0, cfg.vocab, size=(2, 128)).astype(np.int32)
    want = forward(oracle, cfg, full_weights(cfg, 3), tokens)
    for name in ("nccl", "fused", "fused_graph", "pull_graph", "copy_graph"):
        got = np.concatenate([r[0][name], r[1][name]], axis=1)
        err = np.abs(got - want)
        assert err.max() <= 0.04 * np.abs(want).max() and err.mean() <= 0.015 * np.abs(want).mean() + 1e-4, (name, err.max(), err.mean())
    np.testing.assert_array_equal(r[0]["fused"], r[0]["fused_graph"])
    np.testing.assert_array_equal(r[0]["fused"], r[0]["pull_graph"])
    np.testing.assert_array_equal(r[0]["fused"], r[0]["copy_graph"])
    for rank in range(world):      # the schedule changes, the arithmetic does not
        assert np.abs(r[rank]["fused4"] - r[rank]["fused4_overlap"]).max() <= 2.0 ** -7 * np.abs(r[rank]["fused4"]).max()
        assert np.abs(r[rank]["fused4"] - r[rank]["pull4_overlap"]).max() <= 2.0 ** -7 * np.abs(r[rank]["fused4"]).max()
        assert np.abs(r[rank]["fused4"] - r[rank]["copy4_overlap"]).max() <= 2.0 ** -7 * np.abs(r[rank]["fused4"]).max()
        assert np.abs(r[rank]["fused4"] - r[rank]["side4_overlap"]).max() <= 2.0 ** -7 * np.abs(r[rank]["fused4"]).max()


def test_single_gpu_fused_exchange(client, oracle):
    """The same kernels on one GPU (a world of one): every store, announcement and wait stays in local memory, which makes
    this the cheapest first check of the scatter GEMM, the owner-side step, the waits and the side stream."""
    from decoder_reference import forward, full_weights
    from rust_ascend_b200.decoder import TensorParallelDecoder
    from rust_ascend_b200.distributed import SingleControl
    from rust_ascend_b200.fused import FusedExchange, LocalGroup, row_parallel_linear_allreduce
    from rust_ascend_b200.runtime import bf16_bits_to_f32, f32_to_bf16_bits
    from test_index_padded import bf16
    try:
        x, w = _inputs(1)
        xs, ws = client.upload(f32_to_bf16_bits(x)), client.upload(f32_to_bf16_bits(w))
        ex = FusedExchange(client, SingleControl(), x.shape[0], w.shape[0])
        want = bf16(bf16(bf16(x) @ bf16(w).T))
        for _ in range(2):                                           # twice: flags only count up, buffers are reused
            got = bf16_bits_to_f32(client.read(row_parallel_linear_allreduce(ex, xs, ws)))
            assert np.abs(got - want).max() <= 2.0 ** -7 * np.abs(want).max()
        # pull form in a world of one: bulk copies from local memory, same bits
        px = FusedExchange(client, SingleControl(), x.shape[0], w.shape[0], pull=True)
        for _ in range(2):
            np.testing.assert_array_equal(bf16_bits_to_f32(client.read(row_parallel_linear_allreduce(px, xs, ws))), got)
        px.close()
        sx = FusedExchange(client, SingleControl(), x.shape[0], w.shape[0], side_scatter=True)
        for _ in range(2):
            np.testing.assert_array_equal(bf16_bits_to_f32(client.read(row_parallel_linear_allreduce(sx, xs, ws))), got)
        sx.close()
        cx = FusedExchange(client, SingleControl(), x.shape[0], w.shape[0], dma=True)
        for _ in range(2):
            np.testing.assert_array_equal(bf16_bits_to_f32(client.read(row_parallel_linear_allreduce(cx, xs, ws))), got)
        cx.close()
        # the scatter GEMM runs on CTA pairs for these sizes; single CTAs must give the same bits
        os.environ["RUDA_GEMM_PAIRS"] = "0"
        try:
            single = bf16_bits_to_f32(client.read(row_parallel_linear_allreduce(ex, xs, ws)))
        finally:
            del os.environ["RUDA_GEMM_PAIRS"]
        np.testing.assert_array_equal(single, got)
        resid = np.random.default_rng(5).standard_normal(want.shape).astype(np.float32)
        weight = np.random.default_rng(6).uniform(0.5, 1.5, want.shape[1]).astype(np.float32)
        x_own = client.upload(f32_to_bf16_bits(resid))
        ex.gemm_scatter(xs, ws); ex.wait_scatter()
        ex.reduce_norm_push(x_in=x_own, weight=client.upload(f32_to_bf16_bits(weight)), eps=1e-5, x_out=x_own)
        ex.wait_gather(); ex.barrier()
        xn = bf16(bf16(resid) + got)
        normed = bf16(xn / np.sqrt((xn ** 2).mean(-1, keepdims=True) + 1e-5) * bf16(weight))
        assert np.abs(bf16_bits_to_f32(client.read(x_own)) - xn).max() <= 2.0 ** -8 * np.abs(xn).max()
        assert np.abs(bf16_bits_to_f32(client.read(ex.gathered())) - normed).max() <= 2.0 ** -7 * np.abs(normed).max()
        ex.close()
        cfg = _cfg()
        tokens = np.random.default_rng(0).integers(0, cfg.vocab, size=(4, 128)).astype(np.int32)
        want_logits = forward(oracle, cfg, full_weights(cfg, 3), tokens)
        for kwargs in ({}, {"use_graph": True}, {"micro_batches": 2, "overlap_exchange": True, "sm_reserve": 16, "use_graph": True},
                       {"pull_exchange": True, "use_graph": True}, {"micro_batches": 2, "overlap_exchange": True, "pull_exchange": True, "sm_reserve": 16, "use_graph": True},
                       {"dma_exchange": True, "use_graph": True}, {"micro_batches": 2, "overlap_exchange": True, "dma_exchange": True, "use_graph": True},
                       {"side_scatter": True, "use_graph": True}, {"micro_batches": 2, "overlap_exchange": True, "side_scatter": True, "sm_reserve": 16, "use_graph": True}):
            model = TensorParallelDecoder(client, cfg, 4, 128, comm=LocalGroup(), seed=3, exact_weights=True, fused=True, **kwargs)
            model.forward(tokens)
            got = bf16_bits_to_f32(client.read(model.forward()))
            model.close()
            err = np.abs(got - want_logits)
            assert err.max() <= 0.04 * np.abs(want_logits).max() and err.mean() <= 0.015 * np.abs(want_logits).mean() + 1e-4, (kwargs, err.max(), err.mean())
    finally:
        client.take_errors()          # an expired wait is a sticky error; it must not follow the context into other tests


def test_bounded_peer_wait_runs_out_and_the_context_survives(client, oracle):
    """Failure detection on the device without a fault: a peer wait on a flag that nobody signals gives up after its time
    limit (50 ms here), raises the device status word, the next sync reports ServerUnhealthy, the waits queued behind it return
    at once, and after take_errors the same context still multiplies matrices correctly."""
    import ctypes as C
    from rust_ascend_b200 import B200Runtime as RT
    from rust_ascend_b200 import DType, ServerUnhealthy
    from rust_ascend_b200.runtime import _check, f32_to_bf16_bits
    flags = client.tensor((16,), DType.I32)
    client.memset(flags, 0)
    client.sync()
    before = os.environ.get("RUDA_PEER_WAIT_MS")
    os.environ["RUDA_PEER_WAIT_MS"] = "50"
    try:
        desc = flags._c()
        started = time.time()
        for _ in range(20):                                    # 20 queued waits: only the first may spend its limit
            _check(client._lib.rb_peer_wait(client._ctx, C.byref(desc), C.c_uint32(1), C.c_uint32(1)))
        with pytest.raises(ServerUnhealthy):
            client.sync()
        assert time.time() - started < 0.8                     # far below 20 x 50 ms plus launch overheads
    finally:
        if before is None:
            del os.environ["RUDA_PEER_WAIT_MS"]
        else:
            os.environ["RUDA_PEER_WAIT_MS"] = before
        errors = client.take_errors()
    assert any("bounded wait" in e for e in errors), errors
    rng = np.random.default_rng(2)
    a = rng.standard_normal((128, 64)).astype(np.float32); b = rng.standard_normal((96, 64)).astype(np.float32)
    from rust_ascend_b200 import Transpose
    got = client.read(RT.gemm(client, client.upload(f32_to_bf16_bits(a)), client.upload(f32_to_bf16_bits(b)), Transpose.No, Transpose.Yes, DType.F32))
    client.sync()                                              # raises if the context were still unhealthy
    want = oracle.gemm_bf16(a, b, False, True, False)
    np.testing.assert_allclose(got, want, rtol=0, atol=1e-4 * np.abs(want).max())
