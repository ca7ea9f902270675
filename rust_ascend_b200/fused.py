"""Tensor parallelism with the exchange fused into the kernels, over peer memory.

The reference's row-parallel projection is a GEMM followed by a vendor all-reduce (runtime/hccl.rs:386-548,
src/distributed.rs:139-156).  Here every rank exports a staging area, an activation buffer and a few flag words to the
other ranks of the node (`PeerBuffer`), and the two halves of the all-reduce become parts of the neighbouring kernels:

* `rb_gemm_scatter`   - the GEMM's epilogue stores each finished slice into the staging area of the rank that owns those
                        rows and announces it (reduce-scatter, tile by tile, under the next tile's main loop);
* `rb_reduce_norm_push` - the owner sums the staged partials in rank order, adds the residual stream, normalises and stores
                        the rows into every rank's activation buffer (all-gather folded into the norm);
* `rb_peer_wait`      - a one-warp kernel that waits, with a time limit, for the announcements of the other GPUs.

The pull form (`FusedExchange(..., pull=True)`) keeps the GEMM plain: every rank writes its whole partial product into a
buffer of its own that the others have mapped, announces it (`rb_peer_signal`), and the owner-side step
(`rb_reduce_norm_push_pull`) fetches its rows of every partial product itself.  All link traffic then belongs to the
owner-side kernel, which can run on a few SMs beside another micro batch's GEMMs, and the GEMM is never held up by the link.

The side-scatter form (`FusedExchange(..., side_scatter=True)`) also keeps the GEMM plain, and moves its result to the owners'
staging areas with a kernel of its own (`rb_scatter_rows`: posted stores only, which a few SMs keep flowing); the owner-side
step is then the one of the scatter form.  Every transfer of the exchange can so run on the side stream, and nothing has to be
held in flight on an SM the way remote reads must.

The copy form (`FusedExchange(..., dma=True)`) moves the data with device-to-device copies between the mapped buffers
(`rb_copy`: copy engines, no SM at all): every rank copies its rows of every partial product into a local staging area, runs
the owner-side arithmetic locally (`rb_reduce_norm_rows`), announces its rows, and copies the other ranks' finished rows into
its own activation buffer.  Beside another micro batch's GEMMs it costs them no SMs except for the short local kernel.

`FusedExchange` owns the buffers and flags of one stream of such projections; `row_parallel_linear_allreduce` is the
all-reduce-equivalent composition (the entry the reference-shaped API asks for), and `decoder.TensorParallelDecoder` uses the
pieces directly so that the residual stream stays sharded by rows between projections.
"""
from __future__ import annotations

import ctypes as C

from . import _lib
from ._lib import rb_tensor
from .distributed import check_replies, failure_bytes
from .runtime import ComputeClient, DType, InvalidTensor, TensorBuffer, _check, _ref

MAX_PEERS = 8
TOKEN_BYTES = 80                     # RB_PEER_TOKEN_BYTES
FLAG_WORDS = 16                      # words per flag group: world counters, the running target, padding
SCATTER, GATHER, BARRIER = 0, 1, 2   # flag groups inside one flags buffer; word 48 is the local block counter


def tensor_array(tensors, keep: list):
    """ctypes array of pointers to rb_tensor descriptors; the descriptors are appended to `keep`, which must outlive the call
    (or, for a recorded plan, the plan)."""
    structs = [t._c() for t in tensors]
    keep.extend(structs)
    array = (C.POINTER(rb_tensor) * len(structs))(*[C.pointer(s) for s in structs])
    keep.append(array)
    return array


class PeerBuffer:
    """One device buffer of `nbytes` per rank, zeroed, with every rank holding a storage handle for each of them
    (`handles[r]`: its own allocation for r == rank, the peer's memory mapped over NVLink otherwise).  Creation and `close`
    are collective: every rank of the control plane must call them in the same order."""

    def __init__(self, client: ComputeClient, control, nbytes: int):
        if not 1 <= control.world_size <= MAX_PEERS:
            raise InvalidTensor(f"peer buffers span 1..{MAX_PEERS} ranks")
        self.client, self.control, self.nbytes = client, control, int(nbytes)
        self.rank, self.world = control.rank, control.world_size
        lib = client._lib
        local, payload = None, None
        try:
            # At least 2 MiB per buffer: an allocation of that size is a mapping of its own in the driver, so the exported
            # handle names exactly this buffer and not a block it shares with unrelated small allocations.
            self.allocated = max(self.nbytes, 2 << 20)
            local = client.empty(self.allocated)
            client.memset(TensorBuffer(local, (self.allocated,), DType.U8), 0)
            client.sync()
            token = (C.c_uint8 * TOKEN_BYTES)()
            _check(lib.rb_peer_export(client._ctx, C.c_uint64(local), token))
            payload = b"\x00" + bytes(token)
        except Exception as error:          # every rank must still answer the round
            payload = failure_bytes(error)
        replies = control.all_gather_bytes(payload)
        check_replies(replies, self.world)
        self.handles, failure = [], None
        try:
            for r, reply in enumerate(replies):
                if r == self.rank:
                    self.handles.append(local)
                    continue
                h = C.c_uint64()
                _check(lib.rb_peer_open(client._ctx, (C.c_uint8 * TOKEN_BYTES)(*reply[1:1 + TOKEN_BYTES]), C.c_uint64(self.allocated), C.byref(h)))
                self.handles.append(h.value)
            payload = b"\x00"
        except Exception as error:
            failure, payload = error, failure_bytes(error)
        # second round: everyone has zeroed and mapped before anyone stores or signals
        check_replies(control.all_gather_bytes(payload), self.world)
        if failure is not None:
            raise failure

    def view(self, rank: int, shape, dtype: DType, byte_offset: int = 0) -> TensorBuffer:
        """A tensor inside rank `rank`'s buffer."""
        t = TensorBuffer(self.handles[rank], shape, dtype, None, offset=byte_offset)
        if byte_offset + t.nbytes > self.nbytes:
            raise InvalidTensor("view exceeds the peer buffer")
        return t

    def close(self) -> None:
        lib, client = self.client._lib, self.client
        for r, h in enumerate(self.handles):
            if r != self.rank:
                _check(lib.rb_peer_close(client._ctx, C.c_uint64(h)))
        # nobody frees memory that another rank still has mapped
        check_replies(self.control.all_gather_bytes(b"\x00"), self.world)
        client.free(self.handles[self.rank])
        self.handles = []


class FusedExchange:
    """Staging area and flags for row-parallel projections of `tokens` x `hidden` outputs over the ranks of `control`.
    `activations` (a PeerBuffer holding at least tokens*hidden BF16 at `activation_offset`) receives the gathered rows."""

    def __init__(self, client: ComputeClient, control, tokens: int, hidden: int, activations: PeerBuffer | None = None,
                 activation_offset: int = 0, pull: bool = False, dma: bool = False, side_scatter: bool = False):
        self.client, self.control = client, control
        self.rank, self.world = control.rank, control.world_size
        self.tokens, self.hidden = int(tokens), int(hidden)
        self.signals = int(client._lib.rb_gemm_scatter_signals(C.c_uint64(tokens), C.c_uint64(hidden), C.c_uint32(self.world)))
        if self.signals == 0 or hidden % 64:
            raise InvalidTensor("fused exchange needs tokens a multiple of 128 * world and hidden a multiple of 64")
        self.rows = tokens // self.world
        self.dma = bool(dma)
        self.side_scatter = bool(side_scatter) and not (pull or dma)
        self.local_partial = client.tensor((tokens, hidden), DType.BF16) if self.side_scatter else None
        self.pull = bool(pull) or self.dma
        # push form: a staging area the peers' GEMMs store into; pull and copy forms: this rank's whole partial product, read by
        # the peers; copy form: also a local staging area that the copies fill
        self.staging = None if self.pull else PeerBuffer(client, control, self.world * self.rows * hidden * 2)
        self.partial = PeerBuffer(client, control, tokens * hidden * 2) if self.pull else None
        self.local_staging = client.tensor((self.world, self.rows, hidden), DType.BF16) if self.dma else None
        self.flags = PeerBuffer(client, control, 256)
        self._own_activations = activations is None
        self.activations = activations or PeerBuffer(client, control, tokens * hidden * 2)
        self.activation_offset = activation_offset
        self._keep: list = []

    # -- descriptors -------------------------------------------------------------------------------------------
    def staging_views(self):
        return [self.staging.view(o, (self.world, self.rows, self.hidden), DType.BF16) for o in range(self.world)]

    def partial_views(self):
        return [self.partial.view(r, (self.tokens, self.hidden), DType.BF16) for r in range(self.world)]

    def own_partial(self) -> TensorBuffer:
        """Where this rank's plain row-parallel GEMM writes its partial product [tokens, hidden] (every form but the scatter GEMM)."""
        if self.side_scatter:
            return self.local_partial
        return self.partial.view(self.rank, (self.tokens, self.hidden), DType.BF16)

    def scatter_rows_args(self, keep: list):
        """Arguments of rb_scatter_rows (side-scatter form)."""
        sp, sd = self.local_partial._c(), self.done_word()._c()
        keep.extend([sp, sd])
        return (self.client._ctx, C.byref(sp), C.c_uint32(self.rank), C.c_uint32(self.world), tensor_array(self.staging_views(), keep),
                tensor_array(self.flag_views(SCATTER), keep), C.byref(sd))

    def flag_views(self, group: int):
        return [self.flags.view(d, (FLAG_WORDS,), DType.I32, group * FLAG_WORDS * 4) for d in range(self.world)]

    def local_flags(self, group: int) -> TensorBuffer:
        return self.flags.view(self.rank, (FLAG_WORDS,), DType.I32, group * FLAG_WORDS * 4)

    def done_word(self) -> TensorBuffer:
        return self.flags.view(self.rank, (2,), DType.I32, 3 * FLAG_WORDS * 4)

    # -- copy form: the call list of the owner-side step and of the gather, as (entry point name, argument tuple) ----------
    def _row_bytes(self) -> int:
        return self.rows * self.hidden * 2

    def dma_reduce_calls(self, x_in, weight, eps: float, x_out, keep: list):
        """After the wait for every rank's partial product: fetch this rank's rows of all of them, reduce + normalise locally
        into this rank's rows of its own activation buffer, announce them."""
        ctx, calls = self.client._ctx, []

        def ref(t):
            if t is None:
                return None
            c = t._c()
            keep.append(c)
            return C.byref(c)
        for src in range(self.world):
            theirs = self.partial.view(src, (self.rows, self.hidden), DType.BF16, self.rank * self._row_bytes())
            slot = TensorBuffer(self.local_staging.handle, (self.rows, self.hidden), DType.BF16, None, offset=src * self._row_bytes())
            calls.append(("rb_copy", (ctx, ref(theirs), ref(slot))))
        mine = self.activations.view(self.rank, (self.rows, self.hidden), DType.BF16, self.activation_offset + self.rank * self._row_bytes())
        calls.append(("rb_reduce_norm_rows", (ctx, ref(self.local_staging), ref(x_in), ref(weight), C.c_double(eps), ref(x_out), ref(mine), ref(self.done_word()))))
        calls.append(("rb_peer_signal", self.signal_args(keep, GATHER)))
        return calls

    def dma_gather_calls(self, keep: list):
        """After the wait for every rank's announcement: copy the other ranks' finished rows into this rank's activation buffer."""
        ctx, calls = self.client._ctx, []
        for src in range(self.world):
            if src == self.rank:
                continue
            off = self.activation_offset + src * self._row_bytes()
            a = self.activations.view(src, (self.rows, self.hidden), DType.BF16, off)._c()
            b = self.activations.view(self.rank, (self.rows, self.hidden), DType.BF16, off)._c()
            keep.extend([a, b])
            calls.append(("rb_copy", (ctx, C.byref(a), C.byref(b))))
        return calls

    def activation_views(self):
        return [self.activations.view(d, (self.tokens, self.hidden), DType.BF16, self.activation_offset) for d in range(self.world)]

    def gathered(self) -> TensorBuffer:
        """This rank's copy of the gathered activations [tokens, hidden]."""
        return self.activations.view(self.rank, (self.tokens, self.hidden), DType.BF16, self.activation_offset)

    # -- argument tuples for the C ABI (shared by the eager calls below and by recorded plans) ---------------------
    def scatter_args(self, a: TensorBuffer, w: TensorBuffer, keep: list):
        sa, sw = a._c(), w._c()
        keep.extend([sa, sw])
        return (self.client._ctx, C.byref(sa), C.byref(sw), C.c_uint32(self.rank), C.c_uint32(self.world),
                tensor_array(self.staging_views(), keep), tensor_array(self.flag_views(SCATTER), keep))

    def scatter_bias_args(self, a: TensorBuffer, w: TensorBuffer, bias: TensorBuffer | None, keep: list):
        """Arguments of rb_gemm_scatter_bias; `bias` (FP32 [hidden]) is given by exactly one rank of the group."""
        args = self.scatter_args(a, w, keep)
        sb = None
        if bias is not None:
            sb = bias._c()
            keep.append(sb)
        return args[:3] + (C.byref(sb) if sb is not None else None,) + args[3:]

    def wait_args(self, group: int, count: int, keep: list):
        f = self.local_flags(group)._c()
        keep.append(f)
        return (self.client._ctx, C.byref(f), C.c_uint32(self.world), C.c_uint32(count))

    def push_args(self, use_staging: bool, x_in, weight, eps: float, x_out, keep: list):
        def ref(t):
            if t is None:
                return None
            s = t._c()
            keep.append(s)
            return C.byref(s)
        staging = self.staging.view(self.rank, (self.world, self.rows, self.hidden), DType.BF16) if use_staging else None
        return (self.client._ctx, ref(staging), ref(x_in), ref(weight), C.c_double(eps), ref(x_out), C.c_uint32(self.rank), C.c_uint32(self.world),
                tensor_array(self.activation_views(), keep), tensor_array(self.flag_views(GATHER), keep), ref(self.done_word()))

    def pull_args(self, x_in, weight, eps: float, x_out, keep: list):
        """Arguments of rb_reduce_norm_push_pull."""
        def ref(t):
            if t is None:
                return None
            s = t._c()
            keep.append(s)
            return C.byref(s)
        return (self.client._ctx, tensor_array(self.partial_views(), keep), ref(x_in), ref(weight), C.c_double(eps), ref(x_out),
                C.c_uint32(self.rank), C.c_uint32(self.world), tensor_array(self.activation_views(), keep),
                tensor_array(self.flag_views(GATHER), keep), ref(self.done_word()))

    def signal_args(self, keep: list, group: int = BARRIER):
        return (self.client._ctx, C.c_uint32(self.rank), C.c_uint32(self.world), tensor_array(self.flag_views(group), keep))

    @property
    def scatter_count(self) -> int:
        """What every peer adds to this rank's SCATTER flag words per projection: the slices its scatter GEMM stores here, or one
        announcement of its finished partial product in the pull form."""
        return 1 if self.pull or self.side_scatter else self.signals

    # -- eager calls ---------------------------------------------------------------------------------------------
    def gemm_scatter(self, a: TensorBuffer, w: TensorBuffer) -> None:
        """Partial product a [tokens, K/world] x w [hidden, K/world]^T: scattered to the owners' staging areas, or (pull form)
        written to this rank's partial-product buffer by the plain GEMM and announced to every rank."""
        lib = self.client._lib
        if self.side_scatter:
            sa, sw, so = a._c(), w._c(), self.own_partial()._c()
            self._keep.extend([sa, sw, so])
            _check(lib.rb_gemm(self.client._ctx, C.byref(sa), C.byref(sw), C.c_int32(0), C.c_int32(1), None, None, C.c_int32(0), C.byref(so)))
            _check(lib.rb_scatter_rows(*self.scatter_rows_args(self._keep)))
        elif self.pull:
            sa, sw, so = a._c(), w._c(), self.own_partial()._c()
            self._keep.extend([sa, sw, so])
            _check(lib.rb_gemm(self.client._ctx, C.byref(sa), C.byref(sw), C.c_int32(0), C.c_int32(1), None, None, C.c_int32(0), C.byref(so)))
            _check(lib.rb_peer_signal(*self.signal_args(self._keep, SCATTER)))
        else:
            _check(lib.rb_gemm_scatter(*self.scatter_args(a, w, self._keep)))

    def wait_scatter(self) -> None:
        _check(self.client._lib.rb_peer_wait(*self.wait_args(SCATTER, self.scatter_count, self._keep)))

    def reduce_norm_push(self, x_in=None, weight=None, eps: float = 1e-5, x_out=None, use_staging: bool = True) -> None:
        if self.dma and use_staging:
            for name, args in self.dma_reduce_calls(x_in, weight, eps, x_out, self._keep):
                _check(getattr(self.client._lib, name)(*args))
        elif self.pull and use_staging:
            _check(self.client._lib.rb_reduce_norm_push_pull(*self.pull_args(x_in, weight, eps, x_out, self._keep)))
        else:
            _check(self.client._lib.rb_reduce_norm_push(*self.push_args(use_staging and not self.pull, x_in, weight, eps, x_out, self._keep)))

    def wait_gather(self, after_push_form: bool = False) -> None:
        """Waits for every rank's rows.  In the copy form the rows are then fetched; `after_push_form` says that the step
        before was a plain rb_reduce_norm_push (rows already stored here by their owners)."""
        _check(self.client._lib.rb_peer_wait(*self.wait_args(GATHER, 1, self._keep)))
        if self.dma and not after_push_form:
            for name, args in self.dma_gather_calls(self._keep):
                _check(getattr(self.client._lib, name)(*args))

    def barrier(self) -> None:
        """All ranks have finished everything enqueued before this point (stream-ordered, no host involvement)."""
        _check(self.client._lib.rb_peer_signal(*self.signal_args(self._keep)))
        _check(self.client._lib.rb_peer_wait(*self.wait_args(BARRIER, 1, self._keep)))

    def close(self) -> None:
        self.client.sync()
        self._keep = []
        for buf in ([self.activations] if self._own_activations else []) + [self.flags, self.staging, self.partial]:
            if buf is not None:
                buf.close()
        self.local_staging = self.local_partial = None


class LocalGroup:
    """A world of one with a control plane: lets the fused exchange (and the decoder's fused mode) run on a single GPU, where
    every store, announcement and wait stays inside that GPU's memory."""

    def __init__(self):
        from .distributed import SingleControl
        self.control = SingleControl()


def row_parallel_linear_allreduce(exchange: FusedExchange, x: TensorBuffer, w_shard: TensorBuffer) -> TensorBuffer:
    """Y = sum over ranks of x_r [T, K/world] . w_r [H, K/world]^T, complete on every rank: what the reference computes with a
    row-parallel Linear followed by all_reduce(sum) (src/distributed.rs:139-156), here as scatter-GEMM, owner-side sum in rank
    order and a push of the summed rows to every rank.  Returns this rank's gathered [T, H], valid until the next push on this
    exchange; work enqueued on this context before the next call still reads it safely, because a peer can only push again
    after it has seen this rank's next scatter, which is enqueued behind that work."""
    exchange.gemm_scatter(x, w_shard)
    exchange.wait_scatter()
    exchange.reduce_norm_push(weight=None)
    exchange.wait_gather()
    return exchange.gathered()
