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
