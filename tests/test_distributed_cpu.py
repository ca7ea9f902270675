"""CPU (gloo, world size 2): the control-plane handshake of the communicator, failure propagation to every rank,
and the tensor-parallel sharding plan checked by running the sharded composition on the CPU oracle."""
import os
import socket
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for _p in (ROOT, os.path.join(ROOT, "tests")):
    if _p not in sys.path:
        sys.path.insert(0, _p)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init(rank, world, port):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    return dist


class FakeNative:
    """Stands in for the NCCL object on CPU ranks: same method surface, no device."""
    fail_root = None       # rank whose root_info() raises
    fail_init = None       # rank whose initialize() raises

    def __init__(self, client):
        self.rank, self.world_size = 0, 1
        self.my_rank = client

    def root_info(self):
        if FakeNative.fail_root == self.my_rank:
            raise RuntimeError("cannot load the NCCL library 'libnccl.so.2'")
        return bytes(range(128))

    def initialize(self, root, rank, world_size):
        assert root == bytes(range(128))
        if FakeNative.fail_init == rank:
            raise RuntimeError("ncclCommInitRank failed with NCCL status 2")
        self.rank, self.world_size = rank, world_size
        return self


def _handshake_worker(rank, world, port, fail_root, fail_init, results):
    dist = _init(rank, world, port)
    from rust_ascend_b200.distributed import CollectiveError, NcclCommunicator, TorchControl
    FakeNative.fail_root, FakeNative.fail_init = fail_root, fail_init
    try:
        comm = NcclCommunicator.initialize(TorchControl(), rank, native_factory=FakeNative)
        results[rank] = ("ok", comm.rank, comm.world_size)
    except CollectiveError as e:
        results[rank] = ("error", str(e))
    dist.destroy_process_group()


@pytest.mark.parametrize("fail_root,fail_init", [(None, None), (0, None), (None, 1)])
def test_handshake_and_failure_reaches_every_rank(fail_root, fail_init):
    # src/distributed.rs:74-110,196-213: any rank's failure text becomes an error on every rank.
    world, port = 2, _free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_handshake_worker, args=(world, port, fail_root, fail_init, results), nprocs=world, join=True)
        results = dict(results)
    if fail_root is None and fail_init is None:
        assert results == {0: ("ok", 0, 2), 1: ("ok", 1, 2)}
    else:
        bad = fail_root if fail_root is not None else fail_init
        for rank in range(world):
            assert results[rank][0] == "error" and f"NCCL rank {bad}:" in results[rank][1]


def test_reply_checks():
    from rust_ascend_b200.distributed import CollectiveError, ContractError, check_replies, failure_bytes
    check_replies([b"\x00abc", b"\x00"], 2)
    with pytest.raises(ContractError):
        check_replies([b"\x00"], 2)
    with pytest.raises(CollectiveError, match="rank 1: boom"):
        check_replies([b"\x00", failure_bytes("boom")], 2)


def test_shard_plan_partitions_every_weight_exactly_once():
    from rust_ascend_b200.decoder import LlamaConfig, shard_plan
    from rust_ascend_b200.runtime import InvalidTensor
    cfg = LlamaConfig()
    for world in (1, 2, 4, 8):
        for key, total in [("q_rows", cfg.heads * 128), ("kv_rows", cfg.kv_heads * 128), ("o_cols", cfg.heads * 128),
                           ("ffn_rows", cfg.ffn), ("down_cols", cfg.ffn), ("vocab_rows", cfg.vocab)]:
            covered = []
            for rank in range(world):
                a, b = shard_plan(cfg, rank, world)[key]
                covered += list(range(a, b))
            assert covered == list(range(total))
        p = shard_plan(cfg, 0, world)
        assert p["q_heads"] // p["kv_heads"] == cfg.heads // cfg.kv_heads   # the GQA group survives sharding
    with pytest.raises(InvalidTensor):
        shard_plan(cfg, 0, 16)
    assert cfg.flops(8 * 2048, 2048) == 63_668_595_195_904


def _tp_worker(rank, world, port, results):
    dist = _init(rank, world, port)
    import torch
    import oracle as orc
    from decoder_reference import forward, full_weights
    from rust_ascend_b200.decoder import LlamaConfig
    cfg = LlamaConfig(layers=2, hidden=128, heads=4, kv_heads=2, head_dim=128, ffn=256, vocab=256)
    w = full_weights(cfg, 3)
    tokens = np.random.default_rng(0).integers(0, cfg.vocab, size=(2, 32)).astype(np.int32)

    def all_reduce(a):
        t = torch.from_numpy(np.ascontiguousarray(a)); dist.all_reduce(t); return t.numpy()
    shard = forward(orc, cfg, w, tokens, rank, world, all_reduce)
    gathered = [torch.zeros_like(torch.from_numpy(shard)) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(np.ascontiguousarray(shard)))
    if rank == 0:
        full = forward(orc, cfg, w, tokens)
        results["err"] = float(np.abs(np.concatenate([g.numpy() for g in gathered], axis=1) - full).max())
        results["scale"] = float(np.abs(full).max())
    dist.destroy_process_group()


def test_tensor_parallel_sharding_equals_unsharded_model_on_cpu_ranks():
    world, port = 2, _free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_tp_worker, args=(world, port, results), nprocs=world, join=True)
        err, scale = results["err"], results["scale"]
    assert err <= 0.03 * scale + 1e-3, (err, scale)   # BF16 partial sums round differently from the unsharded sum


class GroupFake:
    """Records which root id each rank was initialised with; the id names the global rank that made it."""

    def __init__(self, client):
        self.global_rank = client
        self.rank, self.world_size, self.root = 0, 1, None

    def root_info(self):
        return bytes([self.global_rank]) * 128

    def initialize(self, root, rank, world_size):
        self.rank, self.world_size, self.root = rank, world_size, root[0]
        return self


def _group_worker(rank, world, port, tp, results):
    dist = _init(rank, world, port)
    from rust_ascend_b200.distributed import GroupControl, NcclCommunicator, TorchControl, tensor_parallel_groups
    groups = tensor_parallel_groups(world, tp)
    mine = next(g for g in groups if rank in g)
    control = GroupControl(TorchControl(), mine)
    comm = NcclCommunicator.initialize(control, rank, native_factory=GroupFake)
    gathered = control.all_gather_bytes(bytes([rank]))
    results[rank] = (comm.rank, comm.world_size, comm.native.root, [b[0] for b in gathered])
    dist.destroy_process_group()


def test_one_communicator_per_tensor_parallel_group():
    # Four ranks, two tensor-parallel groups of two: each group's communicator is rooted at its own first rank and the
    # group-local control plane sees only its members.
    world, tp, port = 4, 2, _free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_group_worker, args=(world, port, tp, results), nprocs=world, join=True)
        results = dict(results)
    assert results == {0: (0, 2, 0, [0, 1]), 1: (1, 2, 0, [0, 1]), 2: (0, 2, 2, [2, 3]), 3: (1, 2, 2, [2, 3])}


def test_group_rules():
    from rust_ascend_b200.distributed import ContractError, GroupControl, SingleControl, tensor_parallel_groups
    assert tensor_parallel_groups(8, 2) == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert tensor_parallel_groups(8, 8) == [list(range(8))] and tensor_parallel_groups(4, 1) == [[0], [1], [2], [3]]
    with pytest.raises(ContractError):
        tensor_parallel_groups(8, 3)
    with pytest.raises(ContractError):
        GroupControl(SingleControl(), [1])
    with pytest.raises(ContractError):
        GroupControl(SingleControl(), [0, 0])
    assert GroupControl(SingleControl(), [0]).all_gather_bytes(b"x") == [b"x"]


class _FakePeerLib:
    """rb_peer_* without a device: a token names the exporting rank, opening it yields handle 100 + that rank."""

    def __init__(self, rank, fail_export):
        self.rank, self.fail_export, self.closed = rank, fail_export, []

    def rb_peer_export(self, ctx, handle, token):
        if self.fail_export:
            return 5
        token[0] = self.rank
        return 0

    def rb_peer_open(self, ctx, token, nbytes, out):
        out._obj.value = 100 + token[0]
        return 0

    def rb_peer_close(self, ctx, handle):
        self.closed.append(handle.value)
        return 0

    def rb_last_error(self):
        return b"cudaIpcGetMemHandle failed with CUDA status 1"


class _FakePeerClient:
    def __init__(self, rank, fail_export):
        self._lib, self._ctx, self.freed = _FakePeerLib(rank, fail_export), None, []

    def empty(self, size):
        return 7

    def memset(self, t, value=0):
        pass

    def sync(self):
        pass

    def free(self, handle):
        self.freed.append(handle)


def _peer_worker(rank, world, port, fail_rank, results):
    dist = _init(rank, world, port)
    import rust_ascend_b200.fused as fused
    from rust_ascend_b200.distributed import CollectiveError, TorchControl
    from rust_ascend_b200.runtime import B200Error
    fused._check = lambda code: (_ for _ in ()).throw(B200Error("cudaIpcGetMemHandle failed with CUDA status 1")) if code else None
    client = _FakePeerClient(rank, fail_rank == rank)
    try:
        buf = fused.PeerBuffer(client, TorchControl(), 4096)
        handles = list(buf.handles)
        buf.close()
        results[rank] = ("ok", handles, client._lib.closed, client.freed)
    except CollectiveError as e:
        results[rank] = ("error", str(e))
    dist.destroy_process_group()


@pytest.mark.parametrize("fail_rank", [None, 1])
def test_peer_buffer_exchange_orders_handles_by_rank_and_fails_on_every_rank(fail_rank):
    world, port = 3, _free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_peer_worker, args=(world, port, fail_rank, results), nprocs=world, join=True)
        results = dict(results)
    for rank in range(world):
        if fail_rank is None:
            status, handles, closed, freed = results[rank]
            assert status == "ok"
            assert handles == [7 if r == rank else 100 + r for r in range(world)]       # own allocation, peers' mappings by rank
            assert sorted(closed) == [100 + r for r in range(world) if r != rank] and freed == [7]
        else:
            assert results[rank][0] == "error" and f"NCCL rank {fail_rank}:" in results[rank][1]


# ---- TCP rendezvous, RUDA_* process configuration and the data-parallel layer, on host-side stand-ins -------------------------
class HostTensor:
    """A tensor of a CPU rank: the shape / dtype surface of TensorBuffer over a NumPy array."""

    def __init__(self, array):
        from rust_ascend_b200 import DType
        self.array = np.ascontiguousarray(array)
        self.shape = self.array.shape
        self.dtype = {np.dtype(np.float32): DType.F32, np.dtype(np.float16): DType.F16, np.dtype(np.int64): DType.I64,
                      np.dtype(np.int32): DType.I32, np.dtype(np.uint8): DType.U8}[self.array.dtype]


class HostCommunicator:
    """The NcclCommunicator surface with the tensor payloads carried by the control plane (a CPU rank has no NCCL)."""

    def __init__(self, control):
        self.control, self.rank, self.world_size = control, control.rank, control.world_size

    def all_gather_bytes(self, payload):
        return self.control.all_gather_bytes(payload)

    def _everyone(self, value):
        return [np.frombuffer(b, dtype=value.array.dtype).reshape(value.shape) for b in self.control.all_gather_bytes(value.array.tobytes())]

    def broadcast_float(self, value, root): return HostTensor(self._everyone(value)[root].copy())
    broadcast_int = broadcast_bool = broadcast_float

    def all_reduce_float(self, value, operation="sum"):
        total = sum(self._everyone(value))
        return HostTensor((total / self.world_size if operation == "mean" else total).astype(value.array.dtype))

    def zeros_fp32(self, shape): return HostTensor(np.zeros(shape, np.float32))
    def to_fp32(self, value): return HostTensor(value.array.astype(np.float32))
    def divide(self, value, divisor): return HostTensor((value.array / np.float32(divisor)).astype(np.float32))


def _data_parallel_worker(rank, world, port, results):
    from rust_ascend_b200.distributed import ContractError, DataParallel, TcpControl, process_configuration
    env = {"RUDA_RANK": str(rank), "RUDA_WORLD_SIZE": str(world), "RUDA_RENDEZVOUS": f"127.0.0.1:{port}",
           "RUDA_RENDEZVOUS_ID": "00000000000000000000000000002077"}
    cfg = process_configuration(env)
    assert cfg["device"] == rank and cfg["rendezvous_id"] == bytes.fromhex(env["RUDA_RENDEZVOUS_ID"])
    control = TcpControl(cfg["rank"], cfg["world_size"], cfg["address"], cfg["rendezvous_id"], timeout=30)
    out = {"gather": control.all_gather_bytes(bytes([rank]) * (rank + 1))}
    comm = HostCommunicator(control)
    root = world - 1
    ddp = DataParallel(comm, root)
    # examples/hccl_data_parallel.rs:77-104: float weight, an I64 counter beyond 2^53 and Bool flags leave with the root's values
    synced = ddp.initialize_with_buffers({"weight": HostTensor(np.full(4, rank + 1, np.float32)),
                                          "counter": HostTensor(np.array([9_007_199_254_740_993 + rank], np.int64)),
                                          "flags": HostTensor(np.array([rank == root, rank != root], np.uint8))})
    out["weight"], out["counter"], out["flags"] = synced["weight"].array.tolist(), synced["counter"].array.tolist(), synced["flags"].array.tolist()
    # :105-124: local loss weight^2 * sum(w) -> local gradient (rank+1)^2, local weight rank+1 -> (2 world + 1) / 3
    local_weight = rank + 1
    grads, global_weight = ddp.reduce_fp32({"weight": HostTensor(np.full(4, local_weight * local_weight, np.float16))}, local_weight)
    out["reduced"], out["global_weight"], out["dtype"] = grads["weight"].array.tolist(), global_weight, str(grads["weight"].array.dtype)
    # a rank without the gradient: an error under the strict policy (on every rank), zeros under the lenient one
    mine = {} if rank == 0 else {"weight": HostTensor(np.ones(4, np.float32))}
    try:
        ddp.reduce_fp32(mine, 1)
        out["strict"] = "passed"
    except ContractError as error:
        out["strict"] = str(error)
    lenient, _ = ddp.reduce_fp32(mine, 1, missing="zero")
    out["lenient"] = lenient["weight"].array.tolist()
    control.close()
    results[rank] = out


@pytest.mark.parametrize("world", [2, 3])
def test_tcp_rendezvous_and_data_parallel_reduction(world):
    port = _free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_data_parallel_worker, args=(world, port, results), nprocs=world, join=True)
        r = {k: dict(v) for k, v in results.items()}
    root = world - 1
    for rank in range(world):
        assert r[rank]["gather"] == [bytes([i]) * (i + 1) for i in range(world)]
        assert r[rank]["weight"] == [float(root + 1)] * 4
        assert r[rank]["counter"] == [9_007_199_254_740_993 + root] and r[rank]["flags"] == [1, 0]
        assert r[rank]["global_weight"] == world * (world + 1) // 2 and r[rank]["dtype"] == "float32"
        assert np.allclose(r[rank]["reduced"], (2 * world + 1) / 3, atol=1e-2)
        assert "missing" in r[rank]["strict"]
        assert np.allclose(r[rank]["lenient"], (world - 1) / world)


def test_process_configuration_rejects_bad_settings():
    from rust_ascend_b200.distributed import ContractError, process_configuration
    good = {"RUDA_RANK": "1", "RUDA_WORLD_SIZE": "2", "RUDA_RENDEZVOUS": "127.0.0.1:29500", "RUDA_RENDEZVOUS_ID": "0" * 32, "RUDA_CUDA_DEVICE": "5"}
    assert process_configuration(good)["device"] == 5
    for key, value in (("RUDA_RENDEZVOUS_ID", "abc"), ("RUDA_RENDEZVOUS_ID", "g" * 32), ("RUDA_RANK", "2"), ("RUDA_RENDEZVOUS", "nowhere"), ("RUDA_WORLD_SIZE", "x")):
        with pytest.raises(ContractError):
            process_configuration(dict(good, **{key: value}))
    with pytest.raises(ContractError, match="RUDA_RANK"):
        process_configuration({k: v for k, v in good.items() if k != "RUDA_RANK"})
