"""GPU: the decoder-stack composition against the host reference built from the oracle's operators (small
configuration; the composition itself is unpinned in the reference), and the NCCL path on two GPUs when present."""
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cfg():
    from rust_ascend_b200.decoder import LlamaConfig
    return LlamaConfig(layers=2, hidden=256, heads=4, kv_heads=2, head_dim=128, ffn=512, vocab=1024)


def test_single_gpu_decoder_matches_host_reference(client, oracle):
    from decoder_reference import forward, full_weights
    from rust_ascend_b200.decoder import TensorParallelDecoder
    from rust_ascend_b200.runtime import bf16_bits_to_f32
    cfg = _cfg()
    tokens = np.random.default_rng(0).integers(0, cfg.vocab, size=(2, 128)).astype(np.int32)
    model = TensorParallelDecoder(client, cfg, 2, 128, seed=3, exact_weights=True)
    got = bf16_bits_to_f32(client.read(model.forward(tokens)))
    want = forward(oracle, cfg, full_weights(cfg, 3), tokens)
    assert np.all(np.isfinite(got))
    err = np.abs(got - want)
    assert err.max() <= 0.03 * np.abs(want).max() and err.mean() <= 0.01 * np.abs(want).mean() + 1e-4, (err.max(), err.mean(), np.abs(want).max())
    assert model.launches_per_forward == 3 + cfg.layers * 9
    # a second forward on the same buffers gives the same bits (no stale state between steps)
    np.testing.assert_array_equal(client.read(model.forward()), f32_bits(got))
    # micro batches and graph replay change the schedule, not the arithmetic
    for kwargs in ({"micro_batches": 2}, {"use_graph": True}, {"micro_batches": 2, "use_graph": True}):
        other = TensorParallelDecoder(client, cfg, 2, 128, seed=3, exact_weights=True, **kwargs)
        np.testing.assert_array_equal(client.read(other.forward(tokens)), f32_bits(got))
        np.testing.assert_array_equal(client.read(other.forward()), f32_bits(got))


def f32_bits(x):
    from rust_ascend_b200.runtime import f32_to_bf16_bits
    return f32_to_bf16_bits(x)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _two_gpu_worker(rank, world, port, results):
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
    from rust_ascend_b200.runtime import bf16_bits_to_f32
    client = RT.client(RT.initialize_exclusive(RuntimeOptions(device=rank)))
    comm = NcclCommunicator.initialize(TorchControl(), client)
    out = {}
    # collectives against numpy (hccl.rs:398-473 shapes)
    x = (np.arange(4 * 6, dtype=np.float32).reshape(4, 6) + 100 * rank)
    t = client.upload(x)
    out["all_reduce"] = client.read(comm.all_reduce_float(t, "sum")).tolist()
    out["mean"] = client.read(comm.all_reduce_float(t, "mean")).tolist()
    out["all_gather"] = client.read(comm.all_gather_float(t)).tolist()
    out["reduce_scatter"] = client.read(comm.reduce_scatter_float(t, "sum")).tolist()
    out["broadcast"] = client.read(comm.broadcast_float(t, 1)).tolist()
    out["gather_int"] = client.read(comm.all_gather_int(client.upload(np.array([rank, rank + 7], np.int64)))).tolist()
    cfg = _cfg()
    tokens = np.random.default_rng(0).integers(0, cfg.vocab, size=(2, 128)).astype(np.int32)
    for chunks, kwargs in ((1, {}), (2, {"micro_batches": 2, "use_graph": True})):
        model = TensorParallelDecoder(client, cfg, 2, 128, comm=comm, rank=rank, world=world, seed=3, exact_weights=True, **kwargs)
        model.forward(tokens)
        out[f"logits{chunks}"] = bf16_bits_to_f32(client.read(model.forward()))
        model.close()
    results[rank] = out
    comm.native.destroy()
    dist.destroy_process_group()


@pytest.mark.timeout(240)
def test_two_gpu_collectives_and_tensor_parallel_decoder(oracle):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from decoder_reference import forward, full_weights
    world, port = 2, _free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        ctx = mp.spawn(_two_gpu_worker, args=(world, port, results), nprocs=world, join=False)
        deadline = __import__("time").time() + 180
        while not ctx.join(timeout=5):
            if __import__("time").time() > deadline:   # a rank is stuck: end exactly the processes this test started
                for proc in ctx.processes:
                    if proc.is_alive():
                        proc.terminate()
                pytest.fail("two-GPU workers did not finish within 180 s")
        r = {k: dict(v) for k, v in results.items()}
    x = [np.arange(24, dtype=np.float32).reshape(4, 6) + 100 * k for k in range(2)]
    for k in range(2):
        np.testing.assert_array_equal(r[k]["all_reduce"], x[0] + x[1])
        np.testing.assert_array_equal(r[k]["mean"], (x[0] + x[1]) / 2)
        np.testing.assert_array_equal(r[k]["all_gather"], np.concatenate(x, 0))
        np.testing.assert_array_equal(r[k]["reduce_scatter"], (x[0] + x[1])[2 * k:2 * k + 2])
        np.testing.assert_array_equal(r[k]["broadcast"], x[1])
        np.testing.assert_array_equal(r[k]["gather_int"], [0, 7, 1, 8])
    cfg = _cfg()
    tokens = np.random.default_rng(0).integers(0, cfg.vocab, size=(2, 128)).astype(np.int32)
    want = forward(oracle, cfg, full_weights(cfg, 3), tokens)
    for chunks in (1, 2):
        got = np.concatenate([r[0][f"logits{chunks}"], r[1][f"logits{chunks}"]], axis=1)
        err = np.abs(got - want)
        assert err.max() <= 0.04 * np.abs(want).max() and err.mean() <= 0.015 * np.abs(want).mean() + 1e-4, (chunks, err.max(), err.mean())
