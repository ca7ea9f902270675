"""Mirror of `rust_ascend::distributed` (src/distributed.rs) with NCCL in place of HCCL.

`NcclCommunicator` keeps the reference's two planes: a control communicator that moves small byte payloads
between ranks (RUDA's TCP `RankCommunicator` there; any object with `rank`, `world_size` and
`all_gather_bytes` here, e.g. `TorchControl` over a gloo process group) and a native communicator that moves
tensor payloads device to device (`rb_comm_*` / `rb_all_reduce` ... in libruda_b200.so).  Initialisation follows
src/distributed.rs:74-110: rank 0 creates the id, every rank all-gathers `[status byte || payload]`, any rank's
failure text becomes an error on every rank, then a second status round after the native init.
"""
from __future__ import annotations

import ctypes as C

from . import _lib
from .runtime import B200Error, ComputeClient, DType, InvalidTensor, TensorBuffer, _check, _ref

REDUCE_OPS = {"sum": 0, "prod": 1, "max": 2, "min": 3}


class CollectiveError(B200Error):
    """DataParallelError::Collective / TensorDeviceError::Data (src/distributed.rs:196-216)."""


class ContractError(B200Error):
    """DataParallelError::Contract."""


class TorchControl:
    """Control plane over an initialised torch.distributed process group (gloo is enough: bytes only)."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self._dist, self._group = dist, group
        self.rank, self.world_size = dist.get_rank(group), dist.get_world_size(group)

    def all_gather_bytes(self, payload: bytes) -> list[bytes]:
        out = [None] * self.world_size
        self._dist.all_gather_object(out, bytes(payload), group=self._group)
        return [bytes(b) for b in out]


class SingleControl:
    """World of one: no exchange."""
    rank, world_size = 0, 1

    def all_gather_bytes(self, payload: bytes) -> list[bytes]:
        return [bytes(payload)]


class GroupControl:
    """A subset of a parent control plane's ranks seen as a world of its own (group-local `rank`, `world_size`), for one
    communicator per tensor-parallel group when the job also splits its batch across groups.  Every rank of the parent
    must enter the same number of `all_gather_bytes` rounds, which holds when all groups run the same initialisation at
    the same time; each group reads only its members' replies."""

    def __init__(self, parent, members):
        self._parent, self._members = parent, [int(m) for m in members]
        if len(set(self._members)) != len(self._members) or any(not 0 <= m < parent.world_size for m in self._members):
            raise ContractError("group members must be distinct ranks of the parent world")
        if parent.rank not in self._members:
            raise ContractError(f"rank {parent.rank} is not a member of the group {self._members}")
        self.rank, self.world_size = self._members.index(parent.rank), len(self._members)

    def all_gather_bytes(self, payload: bytes) -> list[bytes]:
        replies = self._parent.all_gather_bytes(payload)
        return [replies[m] for m in self._members]


def tensor_parallel_groups(world_size: int, tensor_parallel: int) -> list[list[int]]:
    """Ranks [g*tp, (g+1)*tp) form tensor-parallel group g; the world_size/tp groups each take their own sequences."""
    if tensor_parallel < 1 or world_size % tensor_parallel:
        raise ContractError("the tensor-parallel degree must divide the world size")
    return [list(range(g * tensor_parallel, (g + 1) * tensor_parallel)) for g in range(world_size // tensor_parallel)]


def failure_bytes(error) -> bytes:
    return b"\x01" + str(error).encode()


def check_replies(replies, world_size: int) -> None:
    """src/distributed.rs:196-213."""
    if len(replies) != world_size:
        raise ContractError("NCCL rank metadata count mismatch")
    for rank, reply in enumerate(replies):
        if reply[:1] != b"\x00":
            raise CollectiveError(f"NCCL rank {rank}: {reply[1:].decode('utf-8', 'replace')}")


class NativeNccl:
    """runtime::HcclCommunicator (runtime/hccl.rs:386-548) over rb_comm."""

    def __init__(self, client: ComputeClient):
        self.client, self._lib, self._comm = client, _lib.load(), None
        self.rank, self.world_size = 0, 1

    @staticmethod
    def root_info() -> bytes:
        buf = (C.c_uint8 * 128)()
        _check(_lib.load().rb_comm_unique_id(buf))
        return bytes(buf)

    def initialize(self, root: bytes, rank: int, world_size: int) -> "NativeNccl":
        if len(root) != 128:
            raise InvalidTensor("NCCL root info must be 128 bytes")
        comm = C.c_void_p()
        _check(self._lib.rb_comm_init(self.client._ctx, (C.c_uint8 * 128)(*root), C.c_uint32(rank), C.c_uint32(world_size), C.byref(comm)))
        self._comm, self.rank, self.world_size = comm, rank, world_size
        return self

    def destroy(self) -> None:
        if self._comm is not None:
            _check(self._lib.rb_comm_destroy(self._comm))
            self._comm = None

    def all_reduce(self, value: TensorBuffer, op: str = "sum", out: TensorBuffer | None = None, deferred: bool = False) -> TensorBuffer:
        out = out or self.client.tensor(value.shape, value.dtype)
        _check(self._lib.rb_all_reduce(self._comm, _ref(value), C.c_int32(REDUCE_OPS[op]), _ref(out), C.c_int32(int(deferred))))
        return out

    def fence(self) -> None:
        _check(self._lib.rb_comm_fence(self._comm))

    def broadcast(self, value: TensorBuffer, root: int) -> TensorBuffer:
        if root >= self.world_size:
            raise InvalidTensor("NCCL broadcast root is outside the world")
        out = self.client.tensor(value.shape, value.dtype)
        _check(self._lib.rb_broadcast(self._comm, _ref(value), C.c_uint32(root), _ref(out)))
        return out

    def all_gather(self, value: TensorBuffer) -> TensorBuffer:
        out = self.client.tensor((value.shape[0] * self.world_size,) + value.shape[1:], value.dtype)
        _check(self._lib.rb_all_gather(self._comm, _ref(value), _ref(out)))
        return out

    def row_parallel_linear_allreduce(self, x: TensorBuffer, w_shard: TensorBuffer, dtype: DType = DType.BF16, overlap: bool = False) -> TensorBuffer:
        """out [T, H] = sum over ranks of x_r [T, K/world] w_r [H, K/world]^T on every rank: GEMM and all-reduce(sum) in one call,
        optionally in row chunks so that a chunk's all-reduce runs under the next chunk's GEMM."""
        if len(x.shape) != 2 or len(w_shard.shape) != 2:
            raise InvalidTensor("row-parallel linear takes x [T, K/world], w [H, K/world] and out [T, H]")
        out = self.client.tensor((x.shape[0], w_shard.shape[0]), dtype)
        _check(self._lib.rb_row_parallel_linear_allreduce(self._comm, _ref(x), _ref(w_shard), _ref(out), C.c_int32(int(overlap))))
        return out

    def reduce_scatter(self, value: TensorBuffer, op: str = "sum") -> TensorBuffer:
        if value.shape[0] % self.world_size:
            raise InvalidTensor("reduce_scatter needs a leading axis divisible by the world size")
        out = self.client.tensor((value.shape[0] // self.world_size,) + value.shape[1:], value.dtype)
        _check(self._lib.rb_reduce_scatter(self._comm, _ref(value), C.c_int32(REDUCE_OPS[op]), _ref(out)))
        return out


FLOATS = (DType.F32, DType.F16, DType.BF16)
INTS = (DType.I32, DType.I64)


class NcclCommunicator:
    """distributed::HcclCommunicator (src/distributed.rs:63-190,218-273): control plane + native payload transport."""

    def __init__(self, control, native):
        self.control, self.native = control, native

    @classmethod
    def initialize(cls, control, client: ComputeClient, native_factory=NativeNccl) -> "NcclCommunicator":
        prepared, payload = None, None
        try:
            prepared = native_factory(client)
            root = prepared.root_info() if control.rank == 0 else b""
            payload = b"\x00" + root
        except Exception as error:  # every rank must still answer the round
            payload = failure_bytes(error)
        replies = control.all_gather_bytes(payload)
        check_replies(replies, control.world_size)
        root = replies[0][1:]
        native, failure = None, None
        try:
            native = prepared.initialize(root, control.rank, control.world_size)
            payload = b"\x00"
        except Exception as error:
            failure, payload = error, failure_bytes(error)
        replies = control.all_gather_bytes(payload)
        check_replies(replies, control.world_size)
        if failure is not None:
            raise CollectiveError(str(failure))
        return cls(control, native)

    @property
    def rank(self) -> int:
        return self.native.rank

    @property
    def world_size(self) -> int:
        return self.native.world_size

    def all_gather_bytes(self, payload: bytes) -> list[bytes]:
        return self.control.all_gather_bytes(payload)

    @staticmethod
    def _check(value: TensorBuffer, kinds) -> None:
        if value.dtype not in kinds:
            raise InvalidTensor(f"UnsupportedDType({value.dtype.name})")

    def _mean(self, out: TensorBuffer, operation: str) -> TensorBuffer:
        if operation == "mean":  # Mean = Sum then divide by the world size (src/distributed.rs:150-154)
            client = self.native.client
            _check(client._lib.rb_div_scalar(client._ctx, _ref(out), C.c_float(float(self.world_size)), _ref(out)))
        return out

    def all_reduce_float(self, value: TensorBuffer, operation: str = "sum") -> TensorBuffer:
        self._check(value, FLOATS)
        return self._mean(self.native.all_reduce(value, "sum"), operation)

    def all_gather_float(self, value: TensorBuffer) -> TensorBuffer:
        self._check(value, FLOATS)
        return self.native.all_gather(value)

    def all_gather_int(self, value: TensorBuffer) -> TensorBuffer:
        self._check(value, INTS)
        return self.native.all_gather(value)

    def reduce_scatter_float(self, value: TensorBuffer, operation: str = "sum") -> TensorBuffer:
        self._check(value, FLOATS)
        return self._mean(self.native.reduce_scatter(value, "sum"), operation)

    def reduce_scatter_int(self, value: TensorBuffer, operation: str = "sum") -> TensorBuffer:
        self._check(value, INTS)
        return self.native.reduce_scatter(value, operation)

    def broadcast_float(self, value: TensorBuffer, root: int) -> TensorBuffer:
        self._check(value, FLOATS)
        return self.native.broadcast(value, root)

    def broadcast_int(self, value: TensorBuffer, root: int) -> TensorBuffer:
        self._check(value, INTS)
        return self.native.broadcast(value, root)
