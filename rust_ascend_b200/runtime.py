"""Host-side mirror of rust-ascend's runtime boundary (rust-ascend-driver/src/tensor/runtime/mod.rs).

`B200Runtime` keeps the associated-function style of `AscendRuntime` (runtime/mod.rs:146-436): every
operator takes the `ComputeClient` first, `TensorBuffer` arguments after it, and returns new
`TensorBuffer`s or raises a `B200Error` whose subclass mirrors the `CannError` variant
(rust-ascend-driver/src/lib.rs:18-40).  All arithmetic happens in libruda_b200.so; nothing here
computes on the host.
"""
from __future__ import annotations

import ctypes as C
import weakref
import enum
from dataclasses import dataclass, field

import numpy as np

from . import _lib
from ._lib import rb_options, rb_stats, rb_tensor


class DType(enum.IntEnum):
    F32 = 0
    F16 = 1
    BF16 = 2
    I32 = 3
    I64 = 4
    U8 = 5

    @property
    def size(self) -> int:
        return {0: 4, 1: 2, 2: 2, 3: 4, 4: 8, 5: 1}[int(self)]

    @property
    def numpy(self):
        """Host carrier type: BF16 travels as its 16-bit pattern."""
        return {0: np.float32, 1: np.float16, 2: np.uint16, 3: np.int32, 4: np.int64, 5: np.uint8}[int(self)]


class Transpose(enum.IntEnum):
    No = 0
    Yes = 1


class RotaryLayout(enum.IntEnum):
    Interleaved = 0
    SplitHalf = 1


class B200Error(RuntimeError):
    """Base of the CannError mirror; `.status` is the rb_status code."""
    status = 0


class LibraryError(B200Error): status = 1
class SymbolError(B200Error): status = 2
class StatusError(B200Error): status = 3
class InvalidDevice(B200Error): status = 4
class InvalidTensor(B200Error): status = 5
class NullHandle(B200Error): status = 6
class CompletionError(B200Error): status = 7
class ServerUnhealthy(B200Error): status = 8


class CompilationError(B200Error):
    """LaunchError::CompilationError of the reference's server (runtime/mod.rs:723-751)."""
    status = 5


_ERRORS = {c.status: c for c in (LibraryError, SymbolError, StatusError, InvalidDevice, InvalidTensor, NullHandle,
                                 CompletionError, ServerUnhealthy)}


def _check(code: int) -> None:
    if code != 0:
        message = _lib.load().rb_last_error().decode("utf-8", "replace")
        raise _ERRORS.get(code, B200Error)(message)


@dataclass
class RuntimeOptions:
    """RuntimeOptions (runtime/mod.rs:93-115) reduced to what a CUDA device needs."""
    device: int = 0
    synchronous: bool = False


@dataclass(frozen=True)
class B200Device:
    """AscendDevice (runtime/mod.rs:117-140)."""
    ordinal: int = 0


def _contiguous_strides(shape) -> tuple:
    strides, s = [], 1
    for d in reversed(shape):
        strides.append(s)
        s *= d
    return tuple(reversed(strides))


class _Owner:
    """Stands for one device allocation.  Tensors made by `ComputeClient.tensor` / `upload` and every view derived from them
    share one owner; when the last of them is dropped the storage is released, as ComputeStorage::dealloc does when the
    reference drops a handle (runtime/mod.rs:501-515).  Storages taken with `ComputeClient.empty` have no owner and are
    released with `free` only."""
    __slots__ = ("__weakref__",)


def _release(lib, ctx_value: int, handle: int) -> None:
    rt = B200Runtime
    if rt._ctx is None or rt._ctx.value != ctx_value:
        return                                   # the context this storage belonged to is gone, and its memory with it
    lib.rb_free(rt._ctx, C.c_uint64(handle))     # an explicit free may have come first: the status is not an error here


@dataclass
class TensorBuffer:
    """TensorBuffer{handle, shape, strides, dtype} (ruda_runtime); strides in elements.  A tensor built by hand over another
    tensor's handle is a non-owning view: pass `_owner=base._owner` (as `reshape` does) or keep the base alive while it is used."""
    handle: int
    shape: tuple
    dtype: DType
    strides: tuple = field(default=None)
    offset: int = 0
    _owner: object = field(default=None, repr=False, compare=False)

    def __post_init__(self):
        self.shape = tuple(int(d) for d in self.shape)
        if self.strides is None:
            self.strides = _contiguous_strides(self.shape)
        self.dtype = DType(self.dtype)

    @property
    def elements(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    @property
    def nbytes(self) -> int:
        return self.elements * self.dtype.size

    def reshape(self, shape) -> "TensorBuffer":
        shape = tuple(int(d) for d in shape)
        n = 1
        for d in shape:
            n *= d
        if n != self.elements:
            raise InvalidTensor("reshape must keep the element count")
        return TensorBuffer(self.handle, shape, self.dtype, None, self.offset, self._owner)

    def _c(self) -> rb_tensor:
        if not 1 <= len(self.shape) <= 8:
            raise InvalidTensor("tensor rank must be within 1..8")
        t = rb_tensor()
        t.handle, t.offset, t.dtype, t.rank = self.handle, self.offset, int(self.dtype), len(self.shape)
        for i, (d, s) in enumerate(zip(self.shape, self.strides)):
            t.shape[i], t.strides[i] = d, s
        return t


def _ref(t: TensorBuffer | None):
    return None if t is None else C.byref(t._c())


class ComputeClient:
    """ComputeClient<AscendRuntime> as the operators see it: storage, transfers, sync and counters
    (AscendStorage runtime/mod.rs:485-517, AscendServer runtime/mod.rs:767-877)."""

    def __init__(self, ctx, device: B200Device):
        self._ctx = ctx
        self.device = device
        self._lib = _lib.load()

    # -- storage ---------------------------------------------------------------------------------
    def empty(self, size: int) -> int:
        h = C.c_uint64()
        _check(self._lib.rb_alloc(self._ctx, C.c_uint64(size), C.byref(h)))
        return h.value

    def create_from_slice(self, data) -> int:
        """Allocate and upload bytes (or any C-contiguous array)."""
        arr = np.ascontiguousarray(data) if not isinstance(data, (bytes, bytearray, memoryview)) else np.frombuffer(data, dtype=np.uint8)
        h = self.empty(arr.nbytes)
        if arr.nbytes:
            _check(self._lib.rb_write(self._ctx, C.c_uint64(h), C.c_uint64(0), arr.ctypes.data_as(C.c_void_p), C.c_uint64(arr.nbytes)))
            _check(self._lib.rb_sync(self._ctx))  # the source array may be pageable and short-lived
        return h

    def free(self, handle: int) -> None:
        _check(self._lib.rb_free(self._ctx, C.c_uint64(handle)))

    def import_pointer(self, device_pointer: int, size: int) -> int:
        h = C.c_uint64()
        _check(self._lib.rb_import(self._ctx, C.c_void_p(device_pointer), C.c_uint64(size), C.byref(h)))
        return h.value

    def resource(self, handle: int):
        p, n = C.c_void_p(), C.c_uint64()
        _check(self._lib.rb_resource(self._ctx, C.c_uint64(handle), C.byref(p), C.byref(n)))
        return p.value, n.value

    # -- transfers -------------------------------------------------------------------------------
    def write(self, handle: int, host: np.ndarray, offset: int = 0) -> None:
        """Asynchronous upload; `host` should be pinned (see `pinned`) and must outlive the copy."""
        _check(self._lib.rb_write(self._ctx, C.c_uint64(handle), C.c_uint64(offset), host.ctypes.data_as(C.c_void_p), C.c_uint64(host.nbytes)))

    def read_into(self, handle: int, host: np.ndarray, offset: int = 0) -> None:
        _check(self._lib.rb_read(self._ctx, C.c_uint64(handle), C.c_uint64(offset), host.ctypes.data_as(C.c_void_p), C.c_uint64(host.nbytes)))

    def read_one(self, handle: int) -> bytes:
        _, size = self.resource(handle)
        out = np.empty(size, dtype=np.uint8)
        self.read_into(handle, out)
        return out.tobytes()

    def read(self, t: TensorBuffer) -> np.ndarray:
        """Contiguous tensors only, like AscendServer::read (runtime/mod.rs:926-943)."""
        if tuple(t.strides) != _contiguous_strides(t.shape) and t.elements > 1:
            raise InvalidTensor("UnsupportedStrides: read requires a contiguous tensor")
        out = np.empty(t.shape, dtype=t.dtype.numpy)
        self.read_into(t.handle, out, t.offset)
        return out

    def upload(self, array, dtype: DType | None = None) -> TensorBuffer:
        """Upload a host array as a new contiguous tensor.  BF16 takes uint16 bit patterns."""
        arr = np.ascontiguousarray(array)
        if dtype is None:
            dtype = {np.dtype(np.float32): DType.F32, np.dtype(np.float16): DType.F16, np.dtype(np.uint16): DType.BF16,
                     np.dtype(np.int32): DType.I32, np.dtype(np.int64): DType.I64, np.dtype(np.uint8): DType.U8}[arr.dtype]
        if arr.dtype != np.dtype(DType(dtype).numpy):
            raise InvalidTensor(f"host array dtype {arr.dtype} does not carry {DType(dtype).name}")
        return self._owned(self.create_from_slice(arr), arr.shape if arr.ndim else (1,), dtype)

    def tensor(self, shape, dtype: DType) -> TensorBuffer:
        shape = tuple(int(d) for d in shape)
        n = 1
        for d in shape:
            n *= d
        return self._owned(self.empty(n * DType(dtype).size), shape, dtype)

    def _owned(self, handle: int, shape, dtype) -> TensorBuffer:
        owner = _Owner()
        weakref.finalize(owner, _release, self._lib, self._ctx.value, handle).atexit = False
        return TensorBuffer(handle, shape, dtype, None, 0, owner)

    def pinned(self, shape, dtype) -> np.ndarray:
        """Page-locked host array for asynchronous rb_write / rb_read."""
        dt = np.dtype(dtype)
        n = int(np.prod(shape)) * dt.itemsize
        p = C.c_void_p()
        _check(self._lib.rb_host_alloc(self._ctx, C.c_uint64(n), C.byref(p)))
        buf = (C.c_uint8 * max(n, 1)).from_address(p.value)
        arr = np.frombuffer(buf, dtype=dt, count=int(np.prod(shape))).reshape(shape)
        return arr

    def memset(self, t: TensorBuffer, value: int = 0) -> None:
        _check(self._lib.rb_memset(self._ctx, C.c_uint64(t.handle), C.c_uint64(t.offset), C.c_int32(value), C.c_uint64(t.nbytes)))

    # -- server ----------------------------------------------------------------------------------
    def sync(self) -> None:
        _check(self._lib.rb_sync(self._ctx))

    flush = sync

    def check_guards(self) -> int:
        """With RUDA_GUARD_BANDS=1: drains the stream and returns how many live allocations had a kernel write outside them."""
        n = C.c_uint64()
        _check(self._lib.rb_check_guards(self._ctx, C.byref(n)))
        return n.value

    def take_errors(self) -> list[str]:
        buf = C.create_string_buffer(4096)
        n = C.c_uint32()
        _check(self._lib.rb_take_errors(self._ctx, buf, C.c_size_t(4096), C.byref(n)))
        return [s for s in buf.value.decode().split("\n") if s]

    def stats(self) -> dict:
        s = rb_stats()
        _check(self._lib.rb_get_stats(self._ctx, C.byref(s)))
        return {k: getattr(s, k) for k, _ in rb_stats._fields_}

    memory_usage = stats

    def memory_cleanup(self) -> None:
        """AscendServer::memory_cleanup (runtime/mod.rs:854-856).  Storage here is returned to the driver by `free`, so there is
        no pool to trim; the call drains the stream so that everything freed so far is really released."""
        self.sync()

    def allocation_mode(self, mode) -> None:
        """AscendServer::allocation_mode (runtime/mod.rs:874-876): accepted for interface parity; there is one allocation mode."""

    def launch(self, kernel, count=None, arguments=None, mode=None) -> None:
        """AscendServer::launch (runtime/mod.rs:832-845) compiles RUDA IR for the device.  This backend ships named operators
        only: any IR kernel is refused the way the reference refuses unsupported IR (a compilation error, never a fallback,
        runtime/mod.rs:723-751)."""
        raise CompilationError(f"LaunchError::CompilationError: no IR compiler in the B200 backend (kernel {kernel!r}); use the named operators")

    def start_profile(self) -> None:
        _check(self._lib.rb_profile_begin(self._ctx))

    def end_profile(self) -> float:
        ms = C.c_float()
        _check(self._lib.rb_profile_end(self._ctx, C.byref(ms)))
        return ms.value

    def properties(self) -> dict:
        name = C.create_string_buffer(128)
        sm, mem = C.c_int32(), C.c_uint64()
        _check(self._lib.rb_device_properties(self._ctx, name, C.c_size_t(128), C.byref(sm), C.byref(mem)))
        return {"name": name.value.decode(), "sm_count": sm.value, "memory_bytes": mem.value}


class B200Runtime:
    """Mirror of AscendRuntime's associated functions (runtime/mod.rs:146-436)."""

    _ctx = None
    _device: B200Device | None = None

    # -- lifetime --------------------------------------------------------------------------------
    @classmethod
    def initialize_exclusive(cls, options: RuntimeOptions | None = None) -> B200Device:
        """Once per process; a second call is an error (runtime/mod.rs:424-435)."""
        options = options or RuntimeOptions()
        o = rb_options(device=options.device, synchronous=int(options.synchronous))
        ctx = C.c_void_p()
        _check(_lib.load().rb_init_exclusive(C.byref(o), C.byref(ctx)))
        cls._ctx, cls._device = ctx, B200Device(options.device)
        return cls._device

    @classmethod
    def client(cls, device: B200Device) -> ComputeClient:
        if cls._ctx is None or device != cls._device:
            raise InvalidDevice("call B200Runtime.initialize_exclusive before B200Runtime.client")
        return ComputeClient(cls._ctx, device)

    @classmethod
    def shutdown(cls) -> None:
        if cls._ctx is not None:
            _check(_lib.load().rb_shutdown(cls._ctx))
            cls._ctx = cls._device = None

    # -- helpers ---------------------------------------------------------------------------------
    @staticmethod
    def _rows(t: TensorBuffer) -> int:
        n = 1
        for d in t.shape[:-1]:
            n *= d
        return n

    # -- row programs ----------------------------------------------------------------------------
    @staticmethod
    def rms_norm(client: ComputeClient, input: TensorBuffer, weight: TensorBuffer, epsilon: float, out_dtype: DType | None = None):
        """[output, rstd] (runtime/mod.rs:405-408)."""
        out = client.tensor(input.shape, out_dtype if out_dtype is not None else input.dtype)
        rstd = client.tensor((B200Runtime._rows(input),), DType.F32)
        _check(client._lib.rb_rms_norm(client._ctx, _ref(input), _ref(weight), C.c_double(epsilon), _ref(out), _ref(rstd)))
        return [out, rstd]

    @staticmethod
    def layer_norm(client: ComputeClient, input: TensorBuffer, weight: TensorBuffer, bias: TensorBuffer | None, epsilon: float):
        """[output, mean, rstd] (runtime/mod.rs:442-448)."""
        out = client.tensor(input.shape, input.dtype)
        rows = B200Runtime._rows(input)
        mean, rstd = client.tensor((rows,), DType.F32), client.tensor((rows,), DType.F32)
        _check(client._lib.rb_layer_norm(client._ctx, _ref(input), _ref(weight), _ref(bias), C.c_double(epsilon), _ref(out), _ref(mean), _ref(rstd)))
        return [out, mean, rstd]

    @staticmethod
    def softmax(client: ComputeClient, input: TensorBuffer) -> TensorBuffer:
        """runtime/mod.rs:322-324."""
        out = client.tensor(input.shape, input.dtype)
        _check(client._lib.rb_softmax(client._ctx, _ref(input), C.c_int32(0), _ref(out)))
        return out

    @staticmethod
    def log_softmax(client: ComputeClient, input: TensorBuffer) -> TensorBuffer:
        """runtime/mod.rs:327-329."""
        out = client.tensor(input.shape, input.dtype)
        _check(client._lib.rb_softmax(client._ctx, _ref(input), C.c_int32(1), _ref(out)))
        return out

    @staticmethod
    def scale_in_place(client, t: TensorBuffer, scale: float) -> TensorBuffer:
        """t *= scale: one FP32 multiply per element, as the reference's `matmul(...) * scale` (src/nn/padded_attention.rs:43)."""
        _check(client._lib.rb_mul_scalar(client._ctx, _ref(t), C.c_float(scale), _ref(t)))
        return t

    @staticmethod
    def tensor_softmax(client: ComputeClient, input: TensorBuffer, dim: int, log: bool = False) -> TensorBuffer:
        """Softmax / log-softmax that keeps a half storage dtype (runtime/typed.rs:769-776, the vendor softmax in the
        reference): FP32 goes straight to the row kernel; FP16 and BF16 are widened to FP32, normalised there and rounded
        back once.  Only the last axis is supported (the one the dense-transformer path uses)."""
        if dim != len(input.shape) - 1:
            raise InvalidTensor("softmax is implemented over the last axis only")
        if input.dtype not in (DType.F32, DType.F16, DType.BF16):
            raise InvalidTensor("softmax requires FP32, FP16 or BF16 storage")
        fn = B200Runtime.log_softmax if log else B200Runtime.softmax
        if input.dtype == DType.F32:
            return fn(client, input)
        return B200Runtime.cast(client, fn(client, B200Runtime.cast(client, input, DType.F32)), input.dtype)

    @staticmethod
    def _reduce(client, input, op):
        out = client.tensor(input.shape[:-1] + (1,), DType.F32)
        _check(client._lib.rb_reduce_last(client._ctx, _ref(input), C.c_int32(op), _ref(out)))
        return out

    @staticmethod
    def sum_last(client, input):
        """runtime/mod.rs:286-289."""
        return B200Runtime._reduce(client, input, 0)

    @staticmethod
    def mean_last(client, input):
        """runtime/mod.rs:292-294."""
        return B200Runtime._reduce(client, input, 1)

    @staticmethod
    def max_last(client, input):
        """runtime/mod.rs:297-299."""
        return B200Runtime._reduce(client, input, 2)

    # -- element maps ----------------------------------------------------------------------------
    @staticmethod
    def silu_mul(client, gate: TensorBuffer, up: TensorBuffer) -> TensorBuffer:
        """runtime/mod.rs:282-284."""
        out = client.tensor(gate.shape, gate.dtype)
        _check(client._lib.rb_silu_mul(client._ctx, _ref(gate), _ref(up), _ref(out)))
        return out

    @staticmethod
    def bias_add(client, input: TensorBuffer, bias: TensorBuffer, residual: TensorBuffer | None = None) -> TensorBuffer:
        """runtime/mod.rs:179-181."""
        out = client.tensor(input.shape, input.dtype)
        _check(client._lib.rb_bias_add(client._ctx, _ref(input), _ref(bias), _ref(residual), _ref(out)))
        return out

    @staticmethod
    def add(client, a: TensorBuffer, b: TensorBuffer, out: TensorBuffer | None = None) -> TensorBuffer:
        out = out or client.tensor(a.shape, a.dtype)
        _check(client._lib.rb_add(client._ctx, _ref(a), _ref(b), _ref(out)))
        return out

    @staticmethod
    def rotary(client, input, cos, sin, layout: RotaryLayout) -> TensorBuffer:
        """runtime/mod.rs:259-262."""
        out = client.tensor(input.shape, input.dtype)
        _check(client._lib.rb_rotary(client._ctx, _ref(input), _ref(cos), _ref(sin), C.c_int32(int(layout)), C.c_int32(0), _ref(out)))
        return out

    @staticmethod
    def rotary_backward(client, grad, cos, sin, layout: RotaryLayout) -> TensorBuffer:
        """runtime/mod.rs:265-268."""
        out = client.tensor(grad.shape, grad.dtype)
        _check(client._lib.rb_rotary(client._ctx, _ref(grad), _ref(cos), _ref(sin), C.c_int32(int(layout)), C.c_int32(1), _ref(out)))
        return out

    @staticmethod
    def rotary_prefix(client, input, cos, sin, width: int, layout: RotaryLayout) -> TensorBuffer:
        """runtime/mod.rs:215-217."""
        out = client.tensor(input.shape, input.dtype)
        _check(client._lib.rb_rotary_prefix(client._ctx, _ref(input), _ref(cos), _ref(sin), C.c_uint32(width), C.c_int32(int(layout)), C.c_int32(0), _ref(out)))
        return out

    @staticmethod
    def rotary_prefix_backward(client, grad, cos, sin, width: int, layout: RotaryLayout) -> TensorBuffer:
        """runtime/mod.rs:219-221."""
        out = client.tensor(grad.shape, grad.dtype)
        _check(client._lib.rb_rotary_prefix(client._ctx, _ref(grad), _ref(cos), _ref(sin), C.c_uint32(width), C.c_int32(int(layout)), C.c_int32(1), _ref(out)))
        return out

    @staticmethod
    def repeat_kv_heads(client, input: TensorBuffer, query_heads: int) -> TensorBuffer:
        """runtime/mod.rs:209."""
        if len(input.shape) != 4:
            raise InvalidTensor("KV repetition requires [B,Hkv,N,D]")
        b, _, n, d = input.shape
        out = client.tensor((b, query_heads, n, d), input.dtype)
        _check(client._lib.rb_repeat_kv_heads(client._ctx, _ref(input), C.c_uint32(query_heads), _ref(out)))
        return out

    @staticmethod
    def causal_mask(client, batch: int, queries: int, keys: int, query_start: int, key_start: int) -> TensorBuffer:
        """CausalMaskSpec{batch,queries,keys,query_start,key_start} (runtime/mod.rs:206)."""
        out = client.tensor((batch, queries, keys), DType.F32)
        _check(client._lib.rb_causal_mask(client._ctx, C.c_uint64(query_start), C.c_uint64(key_start), _ref(out)))
        return out

    @staticmethod
    def cast(client, input: TensorBuffer, dtype: DType) -> TensorBuffer:
        """runtime/mod.rs:271-274."""
        out = client.tensor(input.shape, dtype)
        _check(client._lib.rb_cast(client._ctx, _ref(input), _ref(out)))
        return out

    @staticmethod
    def cast_into(client, input: TensorBuffer, output: TensorBuffer) -> None:
        """runtime/mod.rs:277-279."""
        _check(client._lib.rb_cast(client._ctx, _ref(input), _ref(output)))

    @staticmethod
    def embedding(client, weight: TensorBuffer, indices: TensorBuffer) -> TensorBuffer:
        """runtime/mod.rs:231-233."""
        out = client.tensor(indices.shape + (weight.shape[1],), weight.dtype)
        _check(client._lib.rb_embedding(client._ctx, _ref(weight), _ref(indices), _ref(out)))
        return out

    @staticmethod
    def embedding_with_saved_indices(client, weight: TensorBuffer, indices: TensorBuffer):
        """[output, private copy of the indices] (runtime/mod.rs:249-251 -> indexing.rs:38-45)."""
        if indices.dtype not in (DType.I32, DType.I64):
            raise InvalidTensor("embedding indices must be INT32 or INT64")
        saved = B200Runtime.copy_contiguous(client, indices)
        return [B200Runtime.embedding(client, weight, saved), saved]

    @staticmethod
    def copy_contiguous(client, input: TensorBuffer) -> TensorBuffer:
        """Private device copy (runtime/mod.rs:223-225)."""
        out = client.tensor(input.shape, input.dtype)
        _check(client._lib.rb_copy(client._ctx, _ref(input), _ref(out)))
        return out

    @staticmethod
    def embedding_backward(client, grad: TensorBuffer, indices: TensorBuffer, num_weights: int, padding_idx: int | None = None,
                           scale_grad_by_freq: bool = False) -> TensorBuffer:
        """Dense weight gradient [num_weights, W] accumulating repeated ids (runtime/mod.rs:253-256 -> indexing.rs:60-64)."""
        if padding_idx is not None and not 0 <= padding_idx < num_weights:
            raise InvalidTensor("embedding padding index must be within the weight rows")
        if not grad.shape:
            raise InvalidTensor("embedding gradient must have the index shape followed by the embedding width and floating dtype")
        out = client.tensor((num_weights, grad.shape[-1]), grad.dtype)
        _check(client._lib.rb_embedding_backward(client._ctx, _ref(grad), _ref(indices), C.c_uint64(2**64 - 1 if padding_idx is None else padding_idx),
                                                 C.c_int32(int(scale_grad_by_freq)), _ref(out)))
        return out

    @staticmethod
    def resize_prefix(client, input: TensorBuffer, shape) -> TensorBuffer:
        """Zero pad / crop to `shape` keeping the common prefix of every axis (runtime/padded_matrix.rs:24-37); returns the
        input itself when nothing changes, as the reference does."""
        shape = tuple(int(d) for d in shape)
        if shape == tuple(input.shape):
            if len(shape) not in range(1, 9) or input.dtype not in (DType.F32, DType.BF16) or any(d <= 0 for d in shape):
                raise InvalidTensor("prefix resize requires positive matching-rank FP32/BF16 layouts of the same dtype")
            return input
        if len(shape) != len(input.shape):
            raise InvalidTensor("prefix resize requires positive matching-rank FP32/BF16 layouts of the same dtype")
        out = client.tensor(shape, input.dtype)
        _check(client._lib.rb_resize_prefix(client._ctx, _ref(input), _ref(out)))
        return out


    # -- BF16 matrix programs --------------------------------------------------------------------
    @staticmethod
    def _gemm_shape(a: TensorBuffer, b: TensorBuffer, ta: Transpose, tb: Transpose):
        if len(a.shape) not in (2, 3) or len(a.shape) != len(b.shape):
            raise InvalidTensor("GEMM operands are rank 2 or equal-batch rank 3")
        m = a.shape[-1] if ta else a.shape[-2]
        n = b.shape[-2] if tb else b.shape[-1]
        return tuple(a.shape[:-2]) + (m, n)

    @staticmethod
    def gemm_into(client, a: TensorBuffer, b: TensorBuffer, ta: Transpose, tb: Transpose, out: TensorBuffer,
                  bias: TensorBuffer | None = None, b_up: TensorBuffer | None = None) -> None:
        """runtime/mod.rs:352-355; `bias` / `b_up` select the fused epilogues of the B200 kernel."""
        epilogue = 2 if b_up is not None else (1 if bias is not None else 0)
        _check(client._lib.rb_gemm(client._ctx, _ref(a), _ref(b), C.c_int32(int(ta)), C.c_int32(int(tb)), _ref(bias), _ref(b_up),
                                   C.c_int32(epilogue), _ref(out)))

    @staticmethod
    def gemm(client, a: TensorBuffer, b: TensorBuffer, ta: Transpose, tb: Transpose, dtype: DType,
             bias: TensorBuffer | None = None, b_up: TensorBuffer | None = None) -> TensorBuffer:
        """runtime/mod.rs:346-349: BF16 operands, BF16 or FP32 result."""
        out = client.tensor(B200Runtime._gemm_shape(a, b, ta, tb), dtype)
        B200Runtime.gemm_into(client, a, b, ta, tb, out, bias, b_up)
        return out

    @staticmethod
    def linear_host(client, host_x: np.ndarray, x: TensorBuffer, w: TensorBuffer, y: TensorBuffer, host_y: np.ndarray,
                    bias: TensorBuffer | None = None, row_chunks: int = 8) -> None:
        """rb_linear_host: host_y = host_x . w^T (+ bias) with upload, GEMM and read-back of row chunks overlapped on three
        streams (the reference's write -> launch -> read, runtime/mod.rs:767-845, as one pipelined call).  `host_x` / `host_y`
        are host arrays (pinned ones from `client.pinned` for full speed) holding BF16 bit patterns (and FP32 for an FP32 `y`);
        `x` and `y` are device staging tensors of the same shapes.  Returns when `host_y` is complete."""
        if host_x.nbytes != x.nbytes or host_y.nbytes != y.nbytes or not host_x.flags.c_contiguous or not host_y.flags.c_contiguous:
            raise InvalidTensor("host buffers must be contiguous and as large as their staging tensors")
        _check(client._lib.rb_linear_host(client._ctx, C.c_void_p(host_x.ctypes.data), _ref(x), _ref(w), _ref(bias), _ref(y),
                                          C.c_void_p(host_y.ctypes.data), C.c_uint32(row_chunks)))

    @staticmethod
    def gemm_no_alloc(client, a: TensorBuffer, b: TensorBuffer, ta: Transpose, tb: Transpose, out: TensorBuffer) -> None:
        """rb_gemm_no_alloc: GEMM into `out` that takes its scratch from a fixed array inside the library instead of
        cudaMalloc, for hosts that may not allocate device memory while running.  Operands stored against the K-major
        layout may need at most 16 MiB of rewrite space; the call returns after the stream has drained."""
        _check(client._lib.rb_gemm_no_alloc(client._ctx, _ref(a), _ref(b), C.c_int32(int(ta)), C.c_int32(int(tb)), _ref(out)))

    @staticmethod
    def gemm_bf16_fp32(client, a: TensorBuffer, b: TensorBuffer, ta: Transpose, tb: Transpose):
        """[FP32 output, saved BF16 A, saved BF16 B] from FP32 operands: Cast, Cast, GEMM
        (runtime/mod.rs:422-425 -> matrix.rs:84-93)."""
        if a.dtype != DType.F32 or b.dtype != DType.F32:
            raise InvalidTensor("gemm_bf16_fp32 requires FP32 inputs")
        a16, b16 = B200Runtime.cast(client, a, DType.BF16), B200Runtime.cast(client, b, DType.BF16)
        return [B200Runtime.gemm(client, a16, b16, ta, tb, DType.F32), a16, b16]

    @staticmethod
    def linear_bf16_fp32(client, input: TensorBuffer, weight: TensorBuffer):
        """Y = bf16(X) bf16(W)^T with FP32 X [M,K], W [N,K]; returns [Y, X_bf16, W_bf16]
        (runtime/mod.rs:367-370 -> matrix.rs:129-133)."""
        if len(input.shape) != 2 or len(weight.shape) != 2:
            raise InvalidTensor("linear requires rank-2 X[M,K] and W[N,K]")
        if input.dtype != DType.F32 or weight.dtype != DType.F32:
            raise InvalidTensor("gemm_bf16_fp32 requires FP32 inputs")
        y = client.tensor((input.shape[0], weight.shape[0]), DType.F32)
        x16, w16 = client.tensor(input.shape, DType.BF16), client.tensor(weight.shape, DType.BF16)
        _check(client._lib.rb_linear_bf16_fp32(client._ctx, _ref(input), _ref(weight), _ref(y), _ref(x16), _ref(w16)))
        return [y, x16, w16]

    @staticmethod
    def linear_frozen_bf16_fp32(client, input: TensorBuffer, weight: TensorBuffer) -> TensorBuffer:
        """FP32 X times a fixed BF16 W^T, FP32 result, no weight copy (runtime/mod.rs:383-385 -> matrix.rs:147-159)."""
        if input.dtype != DType.F32 or weight.dtype != DType.BF16 or len(input.shape) != 2 or len(weight.shape) != 2:
            raise InvalidTensor("frozen linear requires FP32 input and BF16 weight storage")
        y = client.tensor((input.shape[0], weight.shape[0]), DType.F32)
        _check(client._lib.rb_linear_frozen_bf16(client._ctx, _ref(input), _ref(weight), _ref(y), None))
        return y


    # -- dtype-preserving broadcast matmul (runtime/generic_matrix.rs; the vendor aclnnMatmul(KEEP_DTYPE) in the reference) ----
    @staticmethod
    def matmul_shape(a_shape, b_shape) -> tuple:
        """Output shape of A[..., M, K] @ B[..., K, N] with singleton batch axes broadcasting (tensor/layout.rs:123-142)."""
        a_shape, b_shape = tuple(a_shape), tuple(b_shape)
        if a_shape[-1] != b_shape[-2]:
            raise InvalidTensor("matmul contraction dimensions differ")
        ba, bb = a_shape[:-2], b_shape[:-2]
        rank = max(len(ba), len(bb))
        ba, bb = (1,) * (rank - len(ba)) + ba, (1,) * (rank - len(bb)) + bb
        batch = []
        for x, y in zip(ba, bb):
            if x != y and x != 1 and y != 1:
                raise InvalidTensor("matmul batch axes cannot be broadcast")
            batch.append(y if x == 1 else x)
        return tuple(batch) + (a_shape[-2], b_shape[-1])

    @staticmethod
    def tensor_matmul(client, a: TensorBuffer, b: TensorBuffer) -> TensorBuffer:
        """A[..., M, K] @ B[..., K, N] in the operands' own dtype (FP32, FP16 or BF16), ranks 2..6, singleton batch axes
        broadcasting, any non-negative sizes (runtime/mod.rs:156-158 -> generic_matrix.rs:17-54): rb_tensor_matmul.  BF16 and FP16
        operands go to the tensor cores in their own format; FP32 operands as three BF16 parts whose six leading cross products
        accumulate in one FP32 accumulator, smallest first, so the result carries FP32's precision rather than BF16's."""
        floats = (DType.F32, DType.F16, DType.BF16)
        if a.dtype not in floats or b.dtype != a.dtype or not 2 <= len(a.shape) <= 6 or not 2 <= len(b.shape) <= 6:
            raise InvalidTensor("generic Ascend matmul requires matching floating dtypes and rank 2..6")
        out = client.tensor(B200Runtime.matmul_shape(a.shape, b.shape), a.dtype)
        _check(client._lib.rb_tensor_matmul(client._ctx, _ref(a), _ref(b), _ref(out)))
        return out

    @staticmethod
    def matmul_fp32(client, a: TensorBuffer, b: TensorBuffer) -> TensorBuffer:
        """FP32 ND matrix product without a BF16 or TF32 cast of the result's precision (runtime/mod.rs:148-155)."""
        if a.dtype != DType.F32 or b.dtype != DType.F32:
            raise InvalidTensor("matmul_fp32 requires FP32 inputs")
        return B200Runtime.tensor_matmul(client, a, b)

    @staticmethod
    def group_ends(ends) -> list[int]:
        """GroupEnds::new (deepgemm/plan.rs:15-29): 1..4096 nondecreasing physical row prefix sums, each a multiple of 256,
        not all empty."""
        ends = [int(e) for e in ends]
        if not 1 <= len(ends) <= 4096:
            raise InvalidTensor("group count must be 1..=4096")
        previous = 0
        for end in ends:
            if end < previous or end % 256:
                raise InvalidTensor("group ends must be nondecreasing multiples of 256")
            previous = end
        if previous == 0:
            raise InvalidTensor("all-empty grouped GEMM is not implemented")
        return ends

    @staticmethod
    def gemm_grouped_nt(client, a: TensorBuffer, weights: TensorBuffer, ends, dtype: DType) -> TensorBuffer:
        """M-grouped GEMM of GemmSpec::grouped_nt (deepgemm/plan.rs:61-67, tile walk scheduler.rs:21-33): A [M,K], weights
        [G,N,K], rows [ends[g-1], ends[g]) of A meet expert g's weight; output [M,N].  rb_gemm_grouped_nt: one persistent launch
        over all groups (groups start on 256-row boundaries, so every 128-row tile belongs to one group)."""
        ends = B200Runtime.group_ends(ends)
        if len(a.shape) != 2 or len(weights.shape) != 3:
            raise InvalidTensor("grouped NT requires [M,K] and [G,N,K]")
        m, k = a.shape
        g, n, kw = weights.shape
        if m != ends[-1] or g != len(ends) or k != kw:
            raise InvalidTensor("grouped NT dimensions do not match the physical prefix sums")
        if a.dtype != DType.BF16 or weights.dtype != DType.BF16 or dtype not in (DType.BF16, DType.F32):
            raise InvalidTensor("native DeepGEMM accepts BF16 inputs and BF16/F32 output only")
        if any(x <= 0 or x % 16 or x > 2**31 - 1 for x in (m, n, k)):
            raise InvalidTensor("M/N/K must be positive multiples of 16 <= INT32_MAX; batches/groups 1..=4096")
        out = client.tensor((m, n), dtype)
        _check(client._lib.rb_gemm_grouped_nt(client._ctx, _ref(a), _ref(weights), (C.c_int64 * len(ends))(*ends), C.c_uint32(len(ends)), _ref(out)))
        return out

    # -- matrices whose axes are not multiples of 16 (runtime/padded_matrix.rs, deepgemm/padded.rs) --------------
    @staticmethod
    def _padded_spec(a_shape, b_shape, a_dtype, b_dtype, ta: Transpose, tb: Transpose):
        """PaddedGemmSpec::new (deepgemm/padded.rs:15-41): logical output shape and the physical 16-aligned A, B shapes."""
        rank = len(a_shape)
        if rank not in (2, 3) or len(b_shape) != rank or a_dtype not in (DType.F32, DType.BF16) or b_dtype not in (DType.F32, DType.BF16):
            raise InvalidTensor("padded GEMM requires matching rank-2/3 FP32/BF16 inputs")
        if rank == 3 and a_shape[0] != b_shape[0]:
            raise InvalidTensor("padded GEMM does not broadcast batches")
        m, k = (a_shape[-2], a_shape[-1]) if not ta else (a_shape[-1], a_shape[-2])
        kb, n = (b_shape[-2], b_shape[-1]) if not tb else (b_shape[-1], b_shape[-2])
        if k != kb:
            raise InvalidTensor("padded GEMM logical contraction mismatch")

        def pad(shape):
            if any(d <= 0 for d in shape[-2:]):
                raise InvalidTensor("padded GEMM matrix axes must be positive")
            tail = tuple((d + 15) // 16 * 16 for d in shape[-2:])
            if any(d > 2**31 - 1 for d in tail):
                raise InvalidTensor("padded GEMM aligned axis exceeds INT32_MAX")
            return tuple(shape[:-2]) + tail
        pa, pb = pad(tuple(a_shape)), pad(tuple(b_shape))
        if rank == 3 and not 1 <= a_shape[0] <= 4096:
            raise InvalidTensor("GEMM batch count must be within 1..4096")
        out = (tuple(a_shape[:-2]) + (m, n))
        return out, pa, pb

    @staticmethod
    def _rounded(client, t: TensorBuffer, shape) -> TensorBuffer:
        return B200Runtime.resize_prefix(client, t if t.dtype == DType.BF16 else B200Runtime.cast(client, t, DType.BF16), shape)

    @staticmethod
    def gemm_padded_bf16_fp32(client, a: TensorBuffer, b: TensorBuffer, ta: Transpose, tb: Transpose):
        """[FP32 output cropped to the logical M x N, padded BF16 A, padded BF16 B] for positive M/N/K of any size
        (runtime/mod.rs:188-191 -> padded_matrix.rs:42-50)."""
        if a.dtype != DType.F32 or b.dtype != DType.F32:
            raise InvalidTensor("padded trainable matmul requires FP32 inputs")
        out_shape, pa, pb = B200Runtime._padded_spec(a.shape, b.shape, a.dtype, b.dtype, ta, tb)
        y, a16, b16 = client.tensor(out_shape, DType.F32), client.tensor(pa, DType.BF16), client.tensor(pb, DType.BF16)
        _check(client._lib.rb_gemm_padded(client._ctx, _ref(a), _ref(b), C.c_int32(int(ta)), C.c_int32(int(tb)), _ref(y), _ref(a16), _ref(b16)))
        return [y, a16, b16]

    @staticmethod
    def gemm_padded_bf16_fp32_backward(client, a: TensorBuffer, b: TensorBuffer, grad: TensorBuffer, a_shape, b_shape, ta: Transpose, tb: Transpose):
        """[FP32 dA, FP32 dB] cropped to the original physical input shapes, from the saved padded BF16 operands and the
        logical FP32 dY (runtime/mod.rs:192-197 -> padded_matrix.rs:51-66)."""
        out_shape, pa, pb = B200Runtime._padded_spec(tuple(a_shape), tuple(b_shape), DType.F32, DType.F32, ta, tb)
        if (tuple(a.shape), a.dtype) != (pa, DType.BF16) or (tuple(b.shape), b.dtype) != (pb, DType.BF16) or (tuple(grad.shape), grad.dtype) != (out_shape, DType.F32):
            raise InvalidTensor("padded matmul backward saved input or logical dY layout mismatch")
        g = B200Runtime._rounded(client, grad, B200Runtime._gemm_shape(a, b, ta, tb))
        no, yes = Transpose.No, Transpose.Yes
        opposite = lambda t: yes if t == no else no
        da = B200Runtime.gemm(client, g, b, no, opposite(tb), DType.F32) if ta == no else B200Runtime.gemm(client, b, g, tb, yes, DType.F32)
        db = B200Runtime.gemm(client, a, g, opposite(ta), no, DType.F32) if tb == no else B200Runtime.gemm(client, g, a, yes, ta, DType.F32)
        return [B200Runtime.resize_prefix(client, da, a_shape), B200Runtime.resize_prefix(client, db, b_shape)]

    @staticmethod
    def linear_frozen_padded_bf16_fp32(client, input: TensorBuffer, weight: TensorBuffer):
        """[FP32 Y [M,N], BF16 weight as used (the caller's handle when already aligned)] for FP32 X [M,K] and a fixed BF16
        W [N,K] of any positive size (runtime/mod.rs:198-200 -> padded_matrix.rs:67-79)."""
        if len(input.shape) != 2 or len(weight.shape) != 2 or input.dtype != DType.F32 or weight.dtype != DType.BF16:
            raise InvalidTensor("frozen padded linear requires rank-2 FP32 input and fixed BF16 weight")
        out_shape, pa, pb = B200Runtime._padded_spec(input.shape, weight.shape, input.dtype, weight.dtype, Transpose.No, Transpose.Yes)
        x16 = B200Runtime._rounded(client, input, pa)
        w16 = B200Runtime.resize_prefix(client, weight, pb)
        y = B200Runtime.gemm(client, x16, w16, Transpose.No, Transpose.Yes, DType.F32)
        return [B200Runtime.resize_prefix(client, y, out_shape), w16]

    @staticmethod
    def linear_frozen_padded_bf16_fp32_backward(client, weight: TensorBuffer, grad: TensorBuffer, input_shape, weight_shape) -> TensorBuffer:
        """FP32 dX [M,K] from the padded fixed weight and the logical FP32 dY (runtime/mod.rs:201-204 -> padded_matrix.rs:80-90)."""
        if len(input_shape) != 2 or len(weight_shape) != 2:
            raise InvalidTensor("frozen padded linear backward requires rank-2 shapes")
        out_shape, pa, pb = B200Runtime._padded_spec(tuple(input_shape), tuple(weight_shape), DType.F32, DType.BF16, Transpose.No, Transpose.Yes)
        if (tuple(weight.shape), weight.dtype) != (pb, DType.BF16) or (tuple(grad.shape), grad.dtype) != (out_shape, DType.F32):
            raise InvalidTensor("frozen padded linear saved weight or dY layout mismatch")
        g = B200Runtime._rounded(client, grad, (pa[0], pb[0]))
        dx = B200Runtime.gemm(client, g, weight, Transpose.No, Transpose.No, DType.F32)
        return B200Runtime.resize_prefix(client, dx, input_shape)


    # -- first-order backward --------------------------------------------------------------------
    @staticmethod
    def linear_nt_backward(client, input: TensorBuffer, weight: TensorBuffer, grad: TensorBuffer):
        """[BF16 dX, FP32 dWeight] for Y = X W^T with BF16 X, W and dY (runtime/mod.rs:360-363 -> matrix.rs:60-74)."""
        if any(t.dtype != DType.BF16 or len(t.shape) != 2 for t in (input, weight, grad)) or grad.shape != (input.shape[0], weight.shape[0]):
            raise InvalidTensor("linear backward requires rank-2 BF16 dY matching X @ W^T")
        return [B200Runtime.gemm(client, grad, weight, Transpose.No, Transpose.No, DType.BF16),
                B200Runtime.gemm(client, grad, input, Transpose.Yes, Transpose.No, DType.F32)]

    @staticmethod
    def gemm_bf16_fp32_backward(client, a: TensorBuffer, b: TensorBuffer, grad: TensorBuffer, ta: Transpose, tb: Transpose):
        """[FP32 dA, FP32 dB] in the original physical layouts from the saved BF16 operands and FP32 dY, which is
        rounded to BF16 first (runtime/mod.rs:428-431 -> matrix.rs:95-121)."""
        if a.dtype != DType.BF16 or b.dtype != DType.BF16 or grad.dtype != DType.F32 or grad.shape != B200Runtime._gemm_shape(a, b, ta, tb):
            raise InvalidTensor("BF16-compute matmul backward requires saved BF16 inputs and matching FP32 dY")
        g = B200Runtime.cast(client, grad, DType.BF16)
        no, yes = Transpose.No, Transpose.Yes
        opposite = lambda t: yes if t == no else no
        da = B200Runtime.gemm(client, g, b, no, opposite(tb), DType.F32) if ta == no else B200Runtime.gemm(client, b, g, tb, yes, DType.F32)
        db = B200Runtime.gemm(client, a, g, opposite(ta), no, DType.F32) if tb == no else B200Runtime.gemm(client, g, a, yes, ta, DType.F32)
        return [da, db]

    @staticmethod
    def linear_bf16_fp32_backward(client, input: TensorBuffer, weight: TensorBuffer, grad: TensorBuffer):
        """[FP32 dX, FP32 dW] from the saved BF16 X/W of linear_bf16_fp32 (runtime/mod.rs:375-378)."""
        if len(input.shape) != 2 or len(weight.shape) != 2:
            raise InvalidTensor("BF16-compute linear backward requires saved rank-2 inputs")
        return B200Runtime.gemm_bf16_fp32_backward(client, input, weight, grad, Transpose.No, Transpose.Yes)

    @staticmethod
    def linear_frozen_bf16_fp32_backward(client, input_shape, weight: TensorBuffer, grad: TensorBuffer) -> TensorBuffer:
        """Input-only FP32 gradient with the fixed BF16 weight (runtime/mod.rs:387-389 -> matrix.rs:160-173)."""
        if weight.dtype != DType.BF16 or grad.dtype != DType.F32 or tuple(grad.shape) != (input_shape[0], weight.shape[0]) or input_shape[1] != weight.shape[1]:
            raise InvalidTensor("frozen BF16 linear backward requires matching FP32 dY")
        return B200Runtime.gemm(client, B200Runtime.cast(client, grad, DType.BF16), weight, Transpose.No, Transpose.No, DType.F32)

    @staticmethod
    def rms_norm_backward(client, input: TensorBuffer, weight: TensorBuffer, grad: TensorBuffer, rstd: TensorBuffer):
        """[input gradient, weight gradient] (runtime/mod.rs:411-414)."""
        dx, dw = client.tensor(input.shape, DType.F32), client.tensor(weight.shape, DType.F32)
        _check(client._lib.rb_rms_norm_backward(client._ctx, _ref(input), _ref(weight), _ref(grad), _ref(rstd), _ref(dx), _ref(dw)))
        return [dx, dw]

    @staticmethod
    def softmax_backward(client, output: TensorBuffer, grad: TensorBuffer) -> TensorBuffer:
        """runtime/mod.rs:332-336."""
        dx = client.tensor(output.shape, DType.F32)
        _check(client._lib.rb_softmax_backward(client._ctx, _ref(output), _ref(grad), C.c_int32(0), _ref(dx)))
        return dx

    @staticmethod
    def log_softmax_backward(client, output: TensorBuffer, grad: TensorBuffer) -> TensorBuffer:
        """runtime/mod.rs:339-343."""
        dx = client.tensor(output.shape, DType.F32)
        _check(client._lib.rb_softmax_backward(client._ctx, _ref(output), _ref(grad), C.c_int32(1), _ref(dx)))
        return dx

    @staticmethod
    def silu_mul_backward(client, gate: TensorBuffer, up: TensorBuffer, grad: TensorBuffer):
        """[gate gradient, up gradient] (runtime/mod.rs:287-290)."""
        dg, du = client.tensor(gate.shape, DType.F32), client.tensor(gate.shape, DType.F32)
        _check(client._lib.rb_silu_mul_backward(client._ctx, _ref(gate), _ref(up), _ref(grad), _ref(dg), _ref(du)))
        return [dg, du]

    @staticmethod
    def repeat_kv_heads_backward(client, input_shape, query_heads: int, grad: TensorBuffer) -> TensorBuffer:
        """runtime/mod.rs:211-213."""
        if len(input_shape) != 4 or len(grad.shape) != 4 or grad.shape[1] != query_heads:
            raise InvalidTensor("KV repetition backward requires [B,Hkv,N,D] and a [B,Hq,N,D] gradient")
        dx = client.tensor(input_shape, DType.F32)
        _check(client._lib.rb_repeat_kv_heads_backward(client._ctx, _ref(grad), C.c_uint32(input_shape[1]), _ref(dx)))
        return dx

    @staticmethod
    def bias_add_backward(client, grad: TensorBuffer, input_shape) -> TensorBuffer:
        """runtime/mod.rs:183-185."""
        if tuple(grad.shape) != tuple(input_shape):
            raise InvalidTensor("bias backward requires dY of the input's shape")
        db = client.tensor((input_shape[-1],), DType.F32)
        _check(client._lib.rb_bias_add_backward(client._ctx, _ref(grad), _ref(db)))
        return db

    @staticmethod
    def layer_norm_backward(client, input: TensorBuffer, weight: TensorBuffer, grad: TensorBuffer, mean: TensorBuffer, rstd: TensorBuffer):
        """[input gradient, weight gradient, bias gradient] (runtime/mod.rs:449-455)."""
        dx, dw, db = client.tensor(input.shape, DType.F32), client.tensor(weight.shape, DType.F32), client.tensor(weight.shape, DType.F32)
        _check(client._lib.rb_layer_norm_backward(client._ctx, _ref(input), _ref(weight), _ref(grad), _ref(mean), _ref(rstd), _ref(dx), _ref(dw), _ref(db)))
        return [dx, dw, db]

    @staticmethod
    def causal_cross_entropy(client, logits: TensorBuffer, labels: TensorBuffer, ignore_index: int = -100, shift: bool = True,
                             upstream: float = 1.0, with_gradient: bool = True):
        """[loss_sum [1], valid_tokens [1], dlogits or None]: the CausalLoss of src/nn/causal_lm.rs:118-196 in one pass over
        the logits, plus the gradient of the mean loss."""
        loss, valid = client.tensor((1,), DType.F32), client.tensor((1,), DType.F32)
        d = client.tensor(logits.shape, DType.F32) if with_gradient else None
        _check(client._lib.rb_causal_cross_entropy(client._ctx, _ref(logits), _ref(labels), C.c_int64(ignore_index), C.c_int32(int(shift)),
                                                   C.c_float(upstream), _ref(loss), _ref(valid), _ref(d)))
        return [loss, valid, d]

    @staticmethod
    def attention_backward(client, q: TensorBuffer, k: TensorBuffer, v: TensorBuffer, grad: TensorBuffer, scale: float,
                           mask: TensorBuffer | None = None, causal: bool = False, query_start: int = 0, key_start: int = 0,
                           want_mask_grad: bool = False):
        """[dQ, dK, dV(, dMask)] of the composed attention for FP32 q [B,Hq,M,D], k [B,Hkv,N,D], v [B,Hkv,N,Dv] and upstream
        grad [B,Hq,M,Dv], with the rounding points of the reference's autodiff graph (src/nn/attention.rs:10-29,49-67 and
        examples/grouped_attention_tensor.rs:14-44): the probabilities are rebuilt as softmax(scale * bf16(Q) bf16(K)^T + mask),
        dP = bf16(dY) bf16(V)^T, dS = P (dP - sum(P dP)) in FP32, bf16(scale dS) feeds dQ and dK, bf16(P) feeds dV, and the
        K/V gradients of a KV head sum over its query heads (heads_programs.rs:59-86).  Scores are materialised, as in the
        reference; the fused forward kernel keeps nothing to reuse here."""
        RT = B200Runtime
        if any(len(t.shape) != 4 or t.dtype != DType.F32 for t in (q, k, v, grad)):
            raise InvalidTensor("attention backward requires FP32 rank-4 Q/K/V and upstream gradient")
        b, hq, m, d = q.shape
        _, hkv, n, dv = v.shape
        if hkv == 0 or hq % hkv or k.shape != (b, hkv, n, d) or v.shape[0] != b or grad.shape != (b, hq, m, dv):
            raise InvalidTensor("GQA requires matching batches, positive divisible Q/KV heads and matching K/V lengths and Q/K widths")
        if not np.isfinite(scale):
            raise InvalidTensor("attention backward needs a finite scale")
        flat = b * hq
        if mask is not None and (mask.dtype != DType.F32 or mask.elements != flat * m * n):
            raise InvalidTensor("attention additive mask must be FP32 [B,Hq,M,N]")
        dq, dk, dv_ = client.tensor(q.shape, DType.F32), client.tensor(k.shape, DType.F32), client.tensor(v.shape, DType.F32)
        dmask = client.tensor((b, hq, m, n), DType.F32) if want_mask_grad else None
        _check(client._lib.rb_attention_backward(client._ctx, _ref(q), _ref(k), _ref(v), _ref(grad), _ref(mask), C.c_float(scale), C.c_int32(int(causal)),
                                                 C.c_uint64(query_start), C.c_uint64(key_start), _ref(dq), _ref(dk), _ref(dv_), _ref(dmask)))
        return [dq, dk, dv_] + ([dmask] if want_mask_grad else [])

    # -- attention -------------------------------------------------------------------------------
    @staticmethod
    def attention_launch_counts(client) -> dict:
        """How many attention calls of this context ran on the tensor-core kernel and how many on the general row kernel."""
        fast, general = C.c_uint64(), C.c_uint64()
        _check(client._lib.rb_attention_launch_counts(client._ctx, C.byref(fast), C.byref(general)))
        return {"tensor_core": fast.value, "general": general.value}

    @staticmethod
    def attention(client, q: TensorBuffer, k: TensorBuffer, v: TensorBuffer, scale: float, mask: TensorBuffer | None = None,
                  causal: bool = False, query_start: int = 0, key_start: int = 0, cos: TensorBuffer | None = None,
                  sin: TensorBuffer | None = None, rotary_layout: RotaryLayout = RotaryLayout.SplitHalf,
                  bmhd_output: bool = False, out: TensorBuffer | None = None) -> TensorBuffer:
        """Fused attention for q [B,Hq,M,D], k [B,Hkv,N,D], v [B,Hkv,N,Dv] (src/nn/attention.rs:10-80).
        Returns [B,Hq,M,Dv], or [B,M,Hq,Dv] when `bmhd_output`."""
        if len(q.shape) != 4 or len(v.shape) != 4:
            raise InvalidTensor("attention tensors are rank 4 [B,H,S,D]")
        b, hq, m, _ = q.shape
        dv = v.shape[3]
        out = out or client.tensor((b, m, hq, dv) if bmhd_output else (b, hq, m, dv), q.dtype)
        _check(client._lib.rb_attention(client._ctx, _ref(q), _ref(k), _ref(v), _ref(mask), C.c_float(scale), C.c_int32(int(causal)),
                                        C.c_uint64(query_start), C.c_uint64(key_start), _ref(cos), _ref(sin), C.c_int32(int(rotary_layout)),
                                        C.c_int32(1 if bmhd_output else 0), _ref(out)))
        return out


# ---- host-side BF16 carriers (bit patterns in uint16) ---------------------------------------------
def f32_to_bf16_bits(x) -> np.ndarray:
    """Round-to-nearest-even FP32 -> BF16 bit patterns; NaN/Inf keep their upper half."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    special = (u & 0x7F800000) == 0x7F800000
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return np.where(special, u >> 16, r).astype(np.uint16)


def bf16_bits_to_f32(bits) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
