"""N-sharded (tensor-parallel) int8 weight-only linears: one process per GPU.

The quantized-matmul path shards along the output columns of each weight:
rank r of P holds ``w[:, r*N/P:(r+1)*N/P]`` and the matching per-channel
scales, computes ``y[:, shard]`` from the replicated activations with no
reduction across ranks, and an all-gather rebuilds the output.  The reference
has nothing to compare with here: its collectives are identity ops on a single
device (src/pjrt_plugin/ops/collective_ops.mm:34-84,118-146); the semantics
implemented are those of ``stablehlo.all_gather`` over one replica group
(src/pjrt_plugin/ops/collective_ops.mm:88-229).

The gathered output of a linear is held as ``[P, M, N/P]`` (block r = rank r's
columns, which is also what ``ncclAllGather`` builds); :func:`gathered_to_logical`
turns it into the logical ``[M, N]`` result.

:class:`GatherExchange` owns the gathered buffers of a set of linears and fills
them in one of five ways:

``fused``       the buffers live in symmetric memory bound to an NVSwitch multicast
                object and the GEMM's epilogue stores with ``multimem.st``: one store
                reaches block r of every rank's buffer, so the all-gather costs no
                extra kernel, no copy and no SM, and a step is a plain sequence of
                GEMM launches.  Each launch ends by incrementing a per-(slot, linear,
                rank) signal word on every rank (release, system scope), which a
                consumer waits for with a bounded wait.
``mcast``       the GEMM writes its block locally; a small kernel on a side stream
                (``qmm_multicast_copy``, a few CTAs that the GEMM leaves free) copies the
                finished block to the multicast address in 512-byte runs and publishes
                the same signal word.  The GEMM epilogue's stores reach the switch as
                64-byte runs; where the links are the bound this uses them better.
``peer``        the same with plain peer stores (``qmm_peer_copy``): P-1 stores per load,
                but nothing is sent to the sender's own buffer, 1/P of what a multicast
                store delivers.
``copy``        symmetric memory without multicast: the GEMM writes its block locally
                and copy-engine peer copies on side streams put it into every peer's
                buffer.
``collective``  ``all_gather_into_tensor`` of the process group on a second stream
                (NCCL on GPUs; gloo on CPU ranks in the host-logic tests).

No TMA multicast load is involved anywhere.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch
import torch.distributed as dist


def shard_bounds(n: int, world: int, rank: int) -> tuple[int, int]:
    """Columns ``[start, stop)`` of an N-wide weight held by ``rank`` of ``world`` ranks."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if n % world:
        raise ValueError(f"N ({n}) must be divisible by the number of ranks ({world})")
    per = n // world
    return rank * per, (rank + 1) * per


def gathered_view(gathered: torch.Tensor) -> torch.Tensor:
    """The gathered ``[P, M, N/P]`` buffer addressed as ``[M, P, N/P]`` (a strided view, no copy):
    element ``[m, p, j]`` is column ``p * N/P + j`` of row ``m`` of the logical output."""
    if gathered.ndim != 3:
        raise ValueError("expected a [P, M, N/P] buffer")
    return gathered.permute(1, 0, 2)


def gathered_to_logical(gathered: torch.Tensor) -> torch.Tensor:
    """The logical ``[M, N]`` output of a gathered ``[P, M, N/P]`` buffer.

    For P > 1 this materialises a copy (the rank and column dimensions of the buffer cannot be
    merged into one stride); consumers on a hot path should index :func:`gathered_view` instead.
    """
    p, m, ns = gathered.shape
    return gathered_view(gathered).reshape(m, p * ns)


class ColumnShardedLinear:
    """One rank's shard of an int8 per-channel weight-only linear."""

    def __init__(self, w_shard: torch.Tensor, scale_shard: torch.Tensor, n_total: int, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        start, stop = shard_bounds(n_total, self.world, self.rank)
        if w_shard.shape[1] != stop - start or scale_shard.shape != (stop - start,):
            raise ValueError("shard shapes do not match this rank's column range")
        self.w, self.scale, self.n_total = w_shard, scale_shard, n_total
        self.columns = (start, stop)

    def local(self, x: torch.Tensor, out: torch.Tensor | None = None, matmul=None) -> torch.Tensor:
        """``x @ dequant(w_shard)`` -> ``[M, N/P]``.  ``matmul`` replaces the CUDA kernel in host-logic tests."""
        if matmul is None:
            from . import ops

            return ops.w8a16_perchannel(x, self.w, self.scale, out=out)
        y = matmul(x, self.w, self.scale)
        if out is not None:
            out.copy_(y)
            return out
        return y

    def forward(self, x: torch.Tensor, matmul=None) -> torch.Tensor:
        """Local matmul followed by a blocking all-gather; returns the ``[P, M, N/P]`` buffer."""
        y = self.local(x, matmul=matmul)
        if self.world == 1:
            return y.unsqueeze(0)
        gathered = torch.empty((self.world,) + tuple(y.shape), dtype=y.dtype, device=y.device)
        dist.all_gather_into_tensor(gathered.view(-1), y.contiguous().view(-1), group=self.group)
        return gathered


# ----------------------------------------------------------------------------
# Gathered output buffers and their exchange
# ----------------------------------------------------------------------------
@dataclass(frozen=True)
class BlockLayout:
    """Where the gathered buffer of (slot, linear) lives inside one allocation (byte offsets)."""

    offset: int      # of the [P, M, N/P] buffer
    block_bytes: int  # of one rank's [M, N/P] block
    m: int
    n: int


def plan_layout(shapes: dict, world: int, depth: int, elem_bytes: int = 2, align: int = 256):
    """Byte layout of ``depth`` slots of gathered buffers for ``shapes = {name: (M, N)}``.

    Returns ``(blocks, signal_offset, total_bytes)``: ``blocks[(slot, name)]`` is a
    :class:`BlockLayout`; behind the buffers sit ``depth * len(shapes) * world`` 32-bit signal
    words, word ``(slot * len(shapes) + index_of(name)) * world + rank``.
    """
    if depth < 1:
        raise ValueError("depth must be >= 1")
    blocks = {}
    off = 0
    for slot in range(depth):
        for name, (m, n) in shapes.items():
            if n % world:
                raise ValueError(f"{name}: N ({n}) must be divisible by the number of ranks ({world})")
            size = m * n * elem_bytes
            blocks[(slot, name)] = BlockLayout(off, size // world, m, n)
            off += (size + align - 1) // align * align
    signal_offset = off
    off += (depth * len(shapes) * world * 4 + align - 1) // align * align
    return blocks, signal_offset, off


class GatherExchange:
    """Gathered ``[P, M, N/P]`` outputs of a set of column-sharded linears, ``depth`` slots each.

    A caller alternates slots between consecutive uses of the same linear (layer parity), so that
    the exchange of one use may still be in flight while the next use computes.  Every rank must
    issue the same sequence of :meth:`linear` calls.  Nothing here orders a producer behind the
    *readers* of a slot it overwrites: a model that consumes the gathered outputs has to wait for
    its own reads before the slot comes round again (after ``depth`` uses).
    """

    def __init__(self, shapes: dict, device, group=None, depth: int = 2, mode: str = "auto",
                 dtype: torch.dtype = torch.bfloat16, reserve_ctas: int = 32):
        self.shapes = dict(shapes)
        self.names = list(self.shapes)
        self.device = torch.device(device)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.depth = depth
        self.dtype = dtype
        self._elem = torch.empty((), dtype=dtype).element_size()
        self.blocks, self._sig_off, self._total = plan_layout(self.shapes, self.world, depth, self._elem)
        self._counts = {(s, n): 0 for s in range(depth) for n in self.names}
        self._hdl = None
        self._mc_ptr = 0
        self._comm = None
        self._peer_streams = {}
        self._pending = {}
        self._peer_views = {}
        self._set_cta_limit = False
        self.why_not_fused = ""
        if mode not in ("auto", "fused", "mcast", "peer", "copy", "collective", "local"):
            raise ValueError(f"unknown exchange mode {mode!r}")
        if self.world == 1:
            mode = "local"
        elif self.device.type != "cuda":
            if mode in ("fused", "mcast", "peer", "copy"):
                raise ValueError("symmetric-memory exchange modes need CUDA devices")
            mode = "collective"
        self._buf = None
        if mode in ("auto", "fused", "mcast", "peer", "copy"):
            mode = self._setup_symmetric(mode)
        if self._buf is None:
            self._buf = torch.zeros(self._total, dtype=torch.uint8, device=self.device)
        self.mode = mode
        if mode in ("copy", "collective", "mcast", "peer"):
            self._comm = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        if mode == "copy":
            self._peer_streams = {p: torch.cuda.Stream(device=self.device) for p in range(self.world) if p != self.rank}
            self._sync_word = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._copy_ctas = 0
        if mode in ("mcast", "peer"):
            reserve_ctas = max(1, min(reserve_ctas, 32))
            self._copy_ctas = reserve_ctas
        if mode in ("collective", "mcast", "peer") and self.device.type == "cuda":
            # the persistent GEMM keeps one CTA per SM resident; leave the all-gather kernel its own SMs
            from . import _lib

            sms = torch.cuda.get_device_properties(self.device).multi_processor_count
            _lib.check(_lib.load().qmm_set_cta_limit(max(1, sms - reserve_ctas)))
            self._set_cta_limit = True
        if mode == "collective" and self.device.type == "cuda":
            self._shards = {n: torch.empty((m, nn // self.world), dtype=dtype, device=self.device)
                            for n, (m, nn) in self.shapes.items()}
        if mode in ("fused", "mcast", "peer"):
            self._arrive = torch.zeros(len(self._counts), dtype=torch.int32, device=self.device)
        self._peer_args = {}
        self._signals = self._buf[self._sig_off:self._sig_off + 4 * depth * len(self.names) * self.world].view(torch.int32)

    # -- set-up ---------------------------------------------------------------
    def _setup_symmetric(self, mode: str) -> str:
        """Allocate the buffers in symmetric memory; agree across ranks on what is available."""
        ok, mc = 1, 1
        try:
            import torch.distributed._symmetric_memory as symm_mem

            buf = symm_mem.empty((self._total,), dtype=torch.uint8, device=self.device)
            hdl = symm_mem.rendezvous(buf, self.group if self.group is not None else dist.group.WORLD)
            mc_ptr = int(getattr(hdl, "multicast_ptr", 0) or 0)
            if mc_ptr == 0:
                mc = 0
        except Exception as exc:  # noqa: BLE001 - any failure means "not available on this system"
            ok, mc = 0, 0
            self.why_not_fused = f"symmetric memory unavailable: {exc!r}"
        flags = torch.tensor([ok, mc], dtype=torch.int32, device=self.device)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN, group=self.group)
        ok, mc = int(flags[0].item()), int(flags[1].item())
        if not ok:
            if mode in ("fused", "mcast", "peer", "copy"):
                raise RuntimeError(f"exchange mode {mode!r} needs symmetric memory ({self.why_not_fused})")
            return "collective"
        buf.zero_()
        self._buf, self._hdl = buf, hdl
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)  # every rank's signal words are zero before anyone signals
        if mode in ("copy", "peer"):
            return mode
        if not mc:
            self.why_not_fused = self.why_not_fused or "no NVSwitch multicast address for the symmetric allocation"
            if mode in ("fused", "mcast"):
                raise RuntimeError(f"exchange mode {mode!r} unavailable: {self.why_not_fused}")
            return "copy"
        self._mc_ptr = mc_ptr
        return "mcast" if mode == "mcast" else "fused"

    def close(self) -> None:
        """Give back what the exchange changed process-wide (the CTA limit of ``collective`` mode)."""
        if self._set_cta_limit:
            from . import _lib

            _lib.load().qmm_set_cta_limit(0)
            self._set_cta_limit = False

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass

    # -- views ----------------------------------------------------------------
    def out(self, name: str, slot: int) -> torch.Tensor:
        """This rank's copy of the gathered ``[P, M, N/P]`` buffer of (``name``, ``slot``)."""
        b = self.blocks[(slot, name)]
        return self._buf[b.offset:b.offset + b.block_bytes * self.world].view(self.dtype).view(
            self.world, b.m, b.n // self.world)

    def logical(self, name: str, slot: int) -> torch.Tensor:
        return gathered_to_logical(self.out(name, slot))

    def signal_words(self, name: str, slot: int) -> torch.Tensor:
        """The ``P`` signal words of (``name``, ``slot``): word r counts rank r's finished launches."""
        i = (slot * len(self.names) + self.names.index(name)) * self.world
        return self._signals[i:i + self.world]

    # -- the exchange ---------------------------------------------------------
    def linear(self, name: str, slot: int, x: torch.Tensor, w_shard: torch.Tensor, scale_shard: torch.Tensor,
               independent: bool = False, matmul=None) -> torch.Tensor:
        """Compute this rank's columns of linear ``name`` into slot ``slot`` and start its exchange.

        ``independent=True`` states that nothing still running on the stream writes ``x`` / the
        weights or touches the slot (see ``QMM_GEMM_INDEPENDENT``).  ``matmul`` replaces the CUDA
        kernel in host-logic tests on CPU ranks.
        """
        b = self.blocks[(slot, name)]
        out = self.out(name, slot)
        mine = out[self.rank]
        self._counts[(slot, name)] += 1
        if matmul is not None:
            y = matmul(x, w_shard, scale_shard)
            if self.mode == "collective":
                dist.all_gather_into_tensor(out.view(-1), y.contiguous().view(-1), group=self.group)
            else:
                mine.copy_(y)
            return out
        from . import _lib

        lib = _lib.load()
        m, k = x.shape
        ns = w_shard.shape[1]
        if (m, ns * self.world) != (b.m, b.n) or scale_shard.shape != (ns,):
            raise ValueError(f"{name}: operand shapes do not match the planned [{b.m}, {b.n}] output")
        stream = torch.cuda.current_stream(self.device)
        flags = _lib.QMM_GEMM_INDEPENDENT if independent else 0
        if self.mode == "fused":
            idx = (slot * len(self.names) + self.names.index(name))
            ext = _lib.GemmExt(flags | _lib.QMM_GEMM_STORE_MULTIMEM,
                               self._mc_ptr + self._sig_off + 4 * (idx * self.world + self.rank),
                               self._arrive.data_ptr() + 4 * idx)
            y_mc = self._mc_ptr + b.offset + self.rank * b.block_bytes
            _lib.check(lib.qmm_w8a16_perchannel_ex(x.data_ptr(), w_shard.data_ptr(), scale_shard.data_ptr(), y_mc, m, ns,
                                                   k, ns, ctypes.byref(ext), stream.cuda_stream))
            return out
        if self.mode == "local":
            ext = _lib.GemmExt(flags)
            _lib.check(lib.qmm_w8a16_perchannel_ex(x.data_ptr(), w_shard.data_ptr(), scale_shard.data_ptr(),
                                                   mine.data_ptr(), m, ns, k, ns, ctypes.byref(ext), stream.cuda_stream))
            return out
        if self.mode == "peer":
            # the GEMM stores its block locally; a small kernel on the side stream then stores it into every
            # peer's buffer over NVLink and bumps this rank's word in every buffer
            prev = self._pending.pop((slot, name), None)
            if prev is not None:
                stream.wait_event(prev)
            ext = _lib.GemmExt(flags)
            _lib.check(lib.qmm_w8a16_perchannel_ex(x.data_ptr(), w_shard.data_ptr(), scale_shard.data_ptr(),
                                                   mine.data_ptr(), m, ns, k, ns, ctypes.byref(ext), stream.cuda_stream))
            ready = torch.cuda.Event()
            ready.record(stream)
            self._comm.wait_event(ready)
            idx = (slot * len(self.names) + self.names.index(name))
            args = self._peer_args.get((slot, name))
            if args is None:
                peers = [p for p in range(self.world) if p != self.rank]
                dst = (ctypes.c_void_p * len(peers))()
                sig = (ctypes.c_void_p * len(peers))()
                for i, p in enumerate(peers):
                    base = self._hdl.get_buffer(p, (self._total,), torch.uint8, 0).data_ptr()
                    dst[i] = base + b.offset + self.rank * b.block_bytes
                    sig[i] = base + self._sig_off + 4 * (idx * self.world + self.rank)
                args = (dst, sig, len(peers))
                self._peer_args[(slot, name)] = args
            _lib.check(lib.qmm_peer_copy(mine.data_ptr(), args[0], args[1], args[2], b.block_bytes,
                                         self._signals.data_ptr() + 4 * (idx * self.world + self.rank),
                                         self._arrive.data_ptr() + 4 * idx, self._copy_ctas, self._comm.cuda_stream))
            done = torch.cuda.Event()
            done.record(self._comm)
            self._pending[(slot, name)] = done
            return out
        if self.mode == "mcast":
            # the GEMM stores its block locally; a small kernel on the side stream then copies it to the
            # multicast address in 512-byte runs and publishes the completion count on every rank
            prev = self._pending.pop((slot, name), None)
            if prev is not None:
                stream.wait_event(prev)   # the previous copy out of this block has read it
            ext = _lib.GemmExt(flags)
            _lib.check(lib.qmm_w8a16_perchannel_ex(x.data_ptr(), w_shard.data_ptr(), scale_shard.data_ptr(),
                                                   mine.data_ptr(), m, ns, k, ns, ctypes.byref(ext), stream.cuda_stream))
            ready = torch.cuda.Event()
            ready.record(stream)
            self._comm.wait_event(ready)
            idx = (slot * len(self.names) + self.names.index(name))
            _lib.check(lib.qmm_multicast_copy(mine.data_ptr(), self._mc_ptr + b.offset + self.rank * b.block_bytes,
                                              b.block_bytes,
                                              self._mc_ptr + self._sig_off + 4 * (idx * self.world + self.rank),
                                              self._arrive.data_ptr() + 4 * idx, self._copy_ctas,
                                              self._comm.cuda_stream))
            done = torch.cuda.Event()
            done.record(self._comm)
            self._pending[(slot, name)] = done
            return out
        # copy / collective: the exchange of this slot's previous use must have finished
        prev = self._pending.pop((slot, name), None)
        if prev is not None:
            stream.wait_event(prev)
        target = mine if self.mode == "copy" else self._shards[name]
        _lib.check(lib.qmm_w8a16_perchannel(x.data_ptr(), w_shard.data_ptr(), scale_shard.data_ptr(), target.data_ptr(),
                                            m, ns, k, ns, stream.cuda_stream))
        ready = torch.cuda.Event()
        ready.record(stream)
        self._comm.wait_event(ready)
        if self.mode == "copy":
            # one contiguous [M, N/P] block per peer, each on its own stream (copy engines)
            for p, st in self._peer_streams.items():
                st.wait_event(ready)
                peer = self._peer_views.get((p, slot, name))
                if peer is None:
                    peer = self._hdl.get_buffer(p, (self.world, b.m, b.n // self.world), self.dtype,
                                                b.offset // self._elem)
                    self._peer_views[(p, slot, name)] = peer
                with torch.cuda.stream(st):
                    peer[self.rank].copy_(mine, non_blocking=True)
                self._comm.wait_stream(st)
        else:
            with torch.cuda.stream(self._comm):
                dist.all_gather_into_tensor(out.view(-1), target.view(-1), group=self.group)
        done = torch.cuda.Event()
        done.record(self._comm)
        self._pending[(slot, name)] = done
        return out

    def finish(self, timeout_ns: int = 0) -> None:
        """Make the current stream wait until every block issued so far, by every rank, has arrived
        in this rank's buffers.  In ``fused`` mode that is a bounded wait on the signal words (a
        wait that runs out shows in ``qmm_device_status()``); in ``copy`` mode a 4-byte all-reduce
        ordered behind each rank's copies is the rendezvous."""
        if self.mode == "local" or self.device.type != "cuda":
            return
        stream = torch.cuda.current_stream(self.device)
        if self.mode in ("fused", "mcast", "peer"):
            from . import _lib

            lib = _lib.load()
            if self.mode != "fused":
                stream.wait_stream(self._comm)
            for (slot, name), count in self._counts.items():
                if count:
                    words = self.signal_words(name, slot)
                    _lib.check(lib.qmm_wait_signals(words.data_ptr(), self.world, count & 0xFFFFFFFF, timeout_ns,
                                                    stream.cuda_stream))
            return
        stream.wait_stream(self._comm)
        if self.mode == "copy":
            dist.all_reduce(self._sync_word, group=self.group)
