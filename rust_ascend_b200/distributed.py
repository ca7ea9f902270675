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

    # -- small device helpers the data-parallel layer needs beside the collectives ----------------------------------
    def zeros_fp32(self, shape) -> TensorBuffer:
        client = self.native.client
        t = client.tensor(shape, DType.F32)
        client.memset(t, 0)
        return t

    def to_fp32(self, value: TensorBuffer) -> TensorBuffer:
        from .runtime import B200Runtime
        return B200Runtime.cast(self.native.client, value, DType.F32)

    def divide(self, value: TensorBuffer, divisor: float) -> TensorBuffer:
        client = self.native.client
        _check(client._lib.rb_div_scalar(client._ctx, _ref(value), C.c_float(divisor), _ref(value)))
        return value

    def broadcast_bool(self, value: TensorBuffer, root: int) -> TensorBuffer:
        """Bool buffers travel as bytes; they are broadcast, never reduced (README.md:104)."""
        self._check(value, (DType.U8,))
        return self.native.broadcast(value, root)


class TcpControl:
    """Control plane over TCP in the shape of RUDA's `RankCommunicator` rendezvous (examples/hccl_data_parallel.rs:32-47): rank 0
    listens on `address` ("host:port"), the other ranks connect and identify themselves with the 16-byte rendezvous id and their
    rank.  `all_gather_bytes` sends one length-prefixed payload to rank 0 and receives everybody's back, in rank order."""

    def __init__(self, rank: int, world_size: int, address: str, rendezvous_id: bytes, timeout: float = 60.0):
        import socket
        import struct
        import time
        if world_size < 1 or not 0 <= rank < world_size or len(rendezvous_id) != 16:
            raise ContractError("rendezvous needs 0 <= rank < world_size and a 16-byte id")
        self.rank, self.world_size, self._struct = rank, world_size, struct
        host, _, port = address.rpartition(":")
        self._peers, self._sock = {}, None
        if world_size == 1:
            return
        if rank == 0:
            server = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
            server.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            server.bind((host, int(port))); server.listen(world_size); server.settimeout(timeout)
            try:
                while len(self._peers) < world_size - 1:
                    conn, _ = server.accept()
                    conn.settimeout(timeout)
                    hello = self._read(conn, 20)
                    peer = struct.unpack("<I", hello[16:])[0]
                    if hello[:16] != rendezvous_id or not 0 < peer < world_size or peer in self._peers:
                        conn.close()
                        raise ContractError("a peer presented another rendezvous id or an invalid rank")
                    self._peers[peer] = conn
            finally:
                server.close()
        else:
            deadline = time.time() + timeout
            while True:
                try:
                    self._sock = socket.create_connection((host, int(port)), timeout=timeout)
                    break
                except OSError:
                    if time.time() > deadline:
                        raise CollectiveError(f"rank {rank} could not reach the rendezvous at {address}")
                    time.sleep(0.05)
            self._sock.sendall(rendezvous_id + struct.pack("<I", rank))

    @staticmethod
    def _read(conn, n: int) -> bytes:
        chunks = []
        while n:
            part = conn.recv(n)
            if not part:
                raise CollectiveError("a rank closed the control connection")
            chunks.append(part); n -= len(part)
        return b"".join(chunks)

    def _send(self, conn, payload: bytes) -> None:
        conn.sendall(self._struct.pack("<Q", len(payload)) + payload)

    def _recv(self, conn) -> bytes:
        return self._read(conn, self._struct.unpack("<Q", self._read(conn, 8))[0])

    def all_gather_bytes(self, payload: bytes) -> list[bytes]:
        payload = bytes(payload)
        if self.world_size == 1:
            return [payload]
        if self.rank == 0:
            replies = [payload] + [self._recv(self._peers[r]) for r in range(1, self.world_size)]
            packed = b"".join(self._struct.pack("<Q", len(r)) + r for r in replies)
            for r in range(1, self.world_size):
                self._send(self._peers[r], packed)
            return replies
        self._send(self._sock, payload)
        packed, out, at = self._recv(self._sock), [], 0
        for _ in range(self.world_size):
            n = self._struct.unpack("<Q", packed[at:at + 8])[0]
            out.append(packed[at + 8:at + 8 + n]); at += 8 + n
        return out

    def close(self) -> None:
        for conn in list(self._peers.values()) + ([self._sock] if self._sock else []):
            conn.close()
        self._peers, self._sock = {}, None


def process_configuration(environ=None) -> dict:
    """The per-process settings of the reference's multi-rank launch (README.md:108-116, examples/hccl_data_parallel.rs:32-47):
    RUDA_RANK, RUDA_WORLD_SIZE, RUDA_RENDEZVOUS (rank-zero host:port), RUDA_RENDEZVOUS_ID (32 hex digits, the same on every rank)
    and the device ordinal, RUDA_CUDA_DEVICE here where the reference reads RUDA_NPU_DEVICE (default: the rank)."""
    import os
    env = os.environ if environ is None else environ
    try:
        rank, world = int(env["RUDA_RANK"]), int(env["RUDA_WORLD_SIZE"])
        address, hex_id = env["RUDA_RENDEZVOUS"], env["RUDA_RENDEZVOUS_ID"]
    except KeyError as missing:
        raise ContractError(f"{missing.args[0]} is not set") from None
    except ValueError:
        raise ContractError("RUDA_RANK and RUDA_WORLD_SIZE must be integers") from None
    if len(hex_id) != 32 or any(ch not in "0123456789abcdefABCDEF" for ch in hex_id):
        raise ContractError("RUDA_RENDEZVOUS_ID must contain 32 hex digits")
    if world < 1 or not 0 <= rank < world or ":" not in address:
        raise ContractError("RUDA_RANK must lie in 0..RUDA_WORLD_SIZE and RUDA_RENDEZVOUS must be host:port")
    return {"rank": rank, "world_size": world, "address": address, "rendezvous_id": bytes.fromhex(hex_id),
            "device": int(env.get("RUDA_CUDA_DEVICE", env.get("RUDA_NPU_DEVICE", rank)))}


def communicator_from_environment(environ=None, native_factory=NativeNccl):
    """One process per GPU configured by the RUDA_* variables: initialises the runtime on the configured device, joins the TCP
    rendezvous and returns (client, NcclCommunicator)."""
    from .runtime import B200Runtime, RuntimeOptions
    cfg = process_configuration(environ)
    client = B200Runtime.client(B200Runtime.initialize_exclusive(RuntimeOptions(device=cfg["device"])))
    control = TcpControl(cfg["rank"], cfg["world_size"], cfg["address"], cfg["rendezvous_id"])
    return client, NcclCommunicator.initialize(control, client, native_factory)


class DataParallel:
    """What RUDA's `DataParallel<B, HcclCommunicator>` does with the communicator (README.md:94, examples/hccl_data_parallel.rs:97-140):
    one-off synchronisation of parameters and buffers from a root rank, and the reduction of local gradients normalised by the
    global weight (the total number of valid tokens or samples), returned in FP32."""

    def __init__(self, communicator: NcclCommunicator, root: int = 0):
        if not 0 <= root < communicator.world_size:
            raise ContractError("the initialisation root is outside the world")
        self.communicator, self.root = communicator, root

    def _agree(self, what: str, payload: bytes) -> list[bytes]:
        replies = self.communicator.all_gather_bytes(payload)
        if any(r != replies[0] for r in replies):
            raise ContractError(f"the ranks disagree on {what}")
        return replies

    def initialize_with_buffers(self, tensors: dict) -> dict:
        """Every rank leaves with the root's values: float parameters, I32/I64 buffers and Bool (U8) buffers, each by one broadcast
        (`initialize_with_buffers` synchronises the integer and Bool buffers once; nothing is re-broadcast before later forwards)."""
        names = sorted(tensors)
        self._agree("the replica structure", repr([(n, tuple(tensors[n].shape), int(tensors[n].dtype)) for n in names]).encode())
        out = {}
        for name in names:
            t = tensors[name]
            if t.dtype in FLOATS:
                out[name] = self.communicator.broadcast_float(t, self.root)
            elif t.dtype in INTS:
                out[name] = self.communicator.broadcast_int(t, self.root)
            elif t.dtype == DType.U8:
                out[name] = self.communicator.broadcast_bool(t, self.root)
            else:
                raise InvalidTensor(f"UnsupportedDType({t.dtype.name})")
        return out

    def reduce_fp32(self, gradients: dict, local_weight: int, missing: str = "error"):
        """(reduced gradients in FP32, global weight).  Each rank passes the gradients of its local loss, which it scaled by its
        own weight (valid tokens or samples); the result is the sum over ranks divided by the sum of the weights.  Half-precision
        gradients are widened first.  `missing`: "error" demands the same gradient names on every rank, "zero" lets a rank that
        lacks one contribute zeros (it still takes part in the collective)."""
        import struct
        if missing not in ("error", "zero") or local_weight < 0:
            raise ContractError("missing-gradient policy is 'error' or 'zero' and the local weight is not negative")
        self._agree("the missing-gradient policy", missing.encode())
        replies = self.communicator.all_gather_bytes(struct.pack("<Q", int(local_weight)) + repr(sorted((n, tuple(g.shape)) for n, g in gradients.items())).encode())
        global_weight = sum(struct.unpack("<Q", r[:8])[0] for r in replies)
        if global_weight == 0:
            raise ContractError("the global weight of a gradient reduction must be positive")
        import ast
        listings = [ast.literal_eval(r[8:].decode()) for r in replies]             # lists of (name, shape) written by repr above
        everything = {}
        for listing in listings:
            for name, shape in listing:
                if everything.setdefault(name, shape) != shape:
                    raise ContractError(f"gradient {name} has different shapes on different ranks")
        if missing == "error" and any(sorted(listing) != sorted(everything.items()) for listing in listings):
            raise ContractError("a gradient is missing on some rank")
        comm = self.communicator
        reduced = {}
        for name in sorted(everything):
            g = gradients.get(name)
            if g is None:
                g = comm.zeros_fp32(everything[name])
            elif g.dtype not in FLOATS:
                raise InvalidTensor(f"UnsupportedDType({g.dtype.name})")
            elif g.dtype != DType.F32:
                g = comm.to_fp32(g)
            reduced[name] = comm.divide(comm.all_reduce_float(g, "sum"), float(global_weight))
        return reduced, global_weight
