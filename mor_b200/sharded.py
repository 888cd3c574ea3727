"""Row-sharded tensor-scaled fake-quantize: one process per GPU, each holding a
contiguous slab of rows whose height is a multiple of the block height, so that no
block, row or group straddles two GPUs.

The reference (boryiings/mor) is single-GPU; this is the multi-GPU form of its
``fake_quantize_block_scaling`` / ``fake_quantize_channel_scaling`` pipeline
(mor/csrc/cuda/fake_quantize.cu:2013-2102, 2431-2526).  Per call:

    phase 1  slab amax + non-zero count                     (kernel, local)
             all-reduce amax (MAX, float32, exact), non-zero count (SUM, int64)
    phase 2  scale, cast, store, per-CTA error sums          (kernel, local)
             all-gather the per-CTA error sums (rank order = row order)
    phase 3  ordered sum of ALL error sums, error / nnz vs threshold -> meta
             (every rank repeats the reference's single-CTA summation order on the
             gathered array, so meta and global_error are bit-identical on every
             rank and equal to the single-GPU result; a float all-reduce would not be)
    phase 4  if meta == 3 copy the slab's input over its output

The collectives are two scalars and a few hundred KiB: latency-bound over NVLink.
Operators without a tensor-wide quantity (per-block MoR, per-row, 1 x 32 MX) need no
communication at all: call them on the slab.

``backend`` supplies the four phases.  The product backend is :class:`CudaBackend`
(C ABI of libmor_b200 on the current CUDA stream).  Tests of the host logic pass a CPU
stand-in over gloo; nothing in this module falls back to one on its own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from . import cabi

KIND_BLOCK = cabi.OP_BLOCK_SCALING
KIND_CHANNEL = cabi.OP_CHANNEL_SCALING


def shard_rows(rows: int, world_size: int, rank: int, multiple: int):
    """Contiguous row range of `rank`: slabs are multiples of `multiple` rows, sizes differ by at most one unit."""
    if rows % multiple:
        raise ValueError(f"rows ({rows}) must be a multiple of the block height ({multiple})")
    units = rows // multiple
    base, extra = divmod(units, world_size)
    start = rank * base + min(rank, extra)
    n = base + (1 if rank < extra else 0)
    return start * multiple, (start + n) * multiple


@dataclass
class ScalingResult:
    meta: torch.Tensor          # int32[1]: 1 = E4M3 kept, 3 = tensor left as it was, -1 = a bounded wait ran out
    global_amax: torch.Tensor   # float32[1]
    global_nnz: torch.Tensor    # int64[1]
    global_error: torch.Tensor  # float32[1]
    ready: Optional[torch.cuda.Event] = None   # set by a pipelined operator: see ShardedScaling(overlap=True)

    def wait(self) -> "ScalingResult":
        """Makes the current stream wait until the output tensor and these scalars are final (a no-op unless the
        operator was built with ``overlap=True``)."""
        if self.ready is not None:
            torch.cuda.current_stream().wait_event(self.ready)
        return self


class CudaBackend:
    """The four phases on the GPU through the C ABI (include/mor_b200.h)."""

    def __init__(self, kind: int, rows: int, cols: int, brows: int, bcols: int, dtype: torch.dtype,
                 device: torch.device):
        if dtype not in (torch.bfloat16, torch.float32):
            raise TypeError("bfloat16 or float32 tensors only")
        self.kind, self.rows, self.cols, self.brows, self.bcols = kind, rows, cols, brows, bcols
        self.dt = cabi.FP32 if dtype == torch.float32 else cabi.BF16
        self.device = device
        self.ws_bytes = cabi.workspace_bytes(kind, rows, cols, brows, bcols)
        if self.ws_bytes == 0:
            raise ValueError(f"unsupported slab/block shape {rows}x{cols} / {brows}x{bcols}")
        self.ws = torch.empty(self.ws_bytes, dtype=torch.uint8, device=device)
        self.n_err = int(cabi.lib().mor_b200_scaling_num_errors(kind, rows, cols, brows, bcols))
        self.stride = int(cabi.lib().mor_b200_scaling_error_stride(kind, brows, bcols))
        self.launches = 0

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def amax_nnz(self, x, amax_out, nnz_out):
        cabi.call("mor_b200_scaling_amax", self.kind, x.data_ptr(), self.dt, self.rows, self.cols, self.brows,
                  self.bcols, amax_out.data_ptr(), nnz_out.data_ptr(), self.ws.data_ptr(), self.ws_bytes,
                  self._stream())
        self.launches += 3

    def cast(self, x, out, ss_mode, global_amax, block_err):
        cabi.call("mor_b200_scaling_cast", self.kind, x.data_ptr(), out.data_ptr(), self.dt, self.rows, self.cols,
                  self.brows, self.bcols, ss_mode, global_amax.data_ptr(), block_err.data_ptr(), self.ws.data_ptr(),
                  self.ws_bytes, self._stream())
        self.launches += 1

    def finalize(self, all_err, global_nnz, threshold, meta, global_error):
        cabi.call("mor_b200_scaling_finalize", all_err.data_ptr(), all_err.numel(), self.stride,
                  global_nnz.data_ptr(), float(threshold), meta.data_ptr(), global_error.data_ptr(),
                  self.ws.data_ptr(), self.ws_bytes, self._stream())
        self.launches += 2 if all_err.numel() > 65536 else 1  # long arrays: partial sums over several CTAs first

    def amax_nnz_local(self, x):
        """phase 1 without the copy of the slab's own amax / count to tensors (the peer exchange reads the workspace)"""
        cabi.call("mor_b200_scaling_amax", self.kind, x.data_ptr(), self.dt, self.rows, self.cols, self.brows,
                  self.bcols, None, None, self.ws.data_ptr(), self.ws_bytes, self._stream())
        self.launches += 2

    def amax_nnz_exchange(self, x, ex: "PeerExchange", epoch: int, amax_out, nnz_out) -> bool:
        """phase 1 with the exchange of the slab's amax and count built into the amax kernel (its last CTA stores
        to the peers and waits for theirs); False, with nothing launched, for block shapes whose kernel has none"""
        try:
            cabi.call("mor_b200_scaling_amax_p2p", self.kind, x.data_ptr(), self.dt, self.rows, self.cols, self.brows,
                      self.bcols, self.ws.data_ptr(), self.ws_bytes, ex.mine, ex.peer_array, ex.rank, ex.world, epoch,
                      amax_out.data_ptr(), nnz_out.data_ptr(), self._stream())
        except cabi.MorB200Error as e:
            if e.status == cabi.ERR_UNSUPPORTED_SHAPE:
                return False
            raise
        self.launches += 2
        return True

    def exchange_scalars(self, ex: "PeerExchange", epoch: int, amax_out, nnz_out):
        cabi.call("mor_b200_p2p_exchange_scalars", self.ws.data_ptr(), ex.mine, ex.peer_array, ex.rank, ex.world, epoch,
                  amax_out.data_ptr(), nnz_out.data_ptr(), self._stream())
        self.launches += 1

    def exchange_errors(self, ex: "PeerExchange", epoch: int, local_err):
        cabi.call("mor_b200_p2p_exchange_errors", local_err.data_ptr(), local_err.numel(), ex.mine, ex.peer_array, ex.rank,
                  ex.world, epoch, self.ws.data_ptr(), self._stream())
        self.launches += 2

    def finalize_ptr(self, err_ptr: int, n: int, global_nnz, threshold, meta, global_error):
        cabi.call("mor_b200_scaling_finalize", err_ptr, n, self.stride, global_nnz.data_ptr(), float(threshold),
                  meta.data_ptr(), global_error.data_ptr(), self.ws.data_ptr(), self.ws_bytes, self._stream())
        self.launches += 2 if n > 65536 else 1

    def fallback(self, x, out, meta):
        cabi.call("mor_b200_scaling_fallback", x.data_ptr(), out.data_ptr(), x.numel() * x.element_size(),
                  meta.data_ptr(), self._stream())
        self.launches += 1


def check_same_on_every_rank(values, what: str, group: Optional[dist.ProcessGroup] = None) -> None:
    """Collective: raises ``ValueError`` on EVERY rank if the ranks do not all hold the same ``values``.

    The row-sharded pipeline gathers fixed-size arrays (every rank computes its offsets into the peers'
    buffers from its OWN slab height), so slabs of different heights would write outside a peer's
    buffer; :func:`shard_rows` gives uneven slabs when the block rows do not divide by the world size."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    world = dist.get_world_size(group)
    seen = [None] * world
    dist.all_gather_object(seen, tuple(values), group=group)
    if any(v != seen[0] for v in seen):
        raise ValueError(f"every rank must hold the same {what}; ranks report {seen}")


class PeerExchange:
    """Buffers of all ranks mapped into every rank (CUDA IPC over NVLink), for the peer exchange of
    include/mor_b200.h: every rank allocates one zero-filled buffer through the library, the 64-byte
    handles travel through the process group once, and kernels store into the peers' buffers
    directly.  Construction is a collective call; it raises if a peer's buffer cannot be opened."""

    def __init__(self, n_err: int, device: torch.device, group: Optional[dist.ProcessGroup] = None):
        import ctypes
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.n_err = n_err
        self.group = group
        self.device_index = device.index if device.index is not None else torch.cuda.current_device()
        self.mine = 0
        self.opened = []
        # every rank runs the same collectives whatever happens locally: a failure is exchanged, not raised early
        err = None
        handle = (ctypes.c_ubyte * 64)()
        try:
            nbytes = int(cabi.lib().mor_b200_p2p_bytes(self.world, n_err))
            if nbytes == 0:
                raise ValueError(f"peer exchange supports up to 16 ranks (world = {self.world})")
            ptr = ctypes.c_void_p()
            cabi.call("mor_b200_p2p_alloc", self.device_index, nbytes, ctypes.byref(ptr), handle)
            self.mine = int(ptr.value)
        except Exception as e:  # noqa: BLE001
            err = e
        handles = [None] * self.world
        dist.all_gather_object(handles, (err is None, bytes(handle)), group=group)
        ptrs = []
        if all(ok for ok, _ in handles):
            try:
                for r in range(self.world):
                    if r == self.rank:
                        ptrs.append(self.mine)
                        continue
                    q = ctypes.c_void_p()
                    cabi.call("mor_b200_p2p_open", self.device_index,
                              (ctypes.c_ubyte * 64).from_buffer_copy(handles[r][1]), ctypes.byref(q))
                    self.opened.append(int(q.value))
                    ptrs.append(int(q.value))
            except Exception as e:  # noqa: BLE001
                err = e
        elif err is None:
            err = RuntimeError("another rank could not allocate its exchange buffer")
        oks = [None] * self.world
        dist.all_gather_object(oks, err is None, group=group)   # also: nobody stores before every buffer is mapped
        if not all(oks):
            self.close(collective=False)
            raise RuntimeError(f"peer exchange could not be set up on every rank ({err})")
        self.peer_ptrs = ptrs
        self.peer_array = (ctypes.c_void_p * self.world)(*ptrs)
        self.epoch = 0

    def error_ptr(self, epoch: int) -> int:
        return self.mine + int(cabi.lib().mor_b200_p2p_error_offset(self.world, self.n_err, epoch))

    def close(self, collective: bool = True):
        """Unmaps the peers' buffers, then (after a barrier, if ``collective``) frees the own one."""
        if self.mine or self.opened:
            torch.cuda.synchronize(self.device_index)
        for q in self.opened:
            cabi.lib().mor_b200_p2p_close(self.device_index, q)
        self.opened = []
        if collective and dist.is_initialized():
            dist.barrier(group=self.group)
        if self.mine:
            cabi.lib().mor_b200_p2p_free(self.device_index, self.mine)
        self.mine = 0


class ShardedScaling:
    """Row-sharded ``fake_quantize_block_scaling`` / ``fake_quantize_channel_scaling``.

    All ranks must call with slabs of the SAME height (the gathered arrays are fixed-size);
    :func:`shard_rows` gives such a partition when the row count divides evenly.  The constructor is a
    collective call and raises ``ValueError`` on every rank when the slabs differ.

    ``overlap=True`` pipelines consecutive calls: everything after the cast kernel (error exchange, ordered
    sum, decision, conditional copy -- a chain of small latency-bound kernels) is enqueued on a second
    stream, so that it runs under the amax pass of the NEXT call; two sets of scratch and scalar tensors
    alternate between calls.  The output and the scalars of a call are then final once ``result.wait()``
    (or a device synchronisation) has been passed, and the next call's cast waits for them by itself
    before it writes ``out`` again.

    A call whose peer wait ran out reports ``meta == -1`` (its output is not valid): see :meth:`timed_out`.
    After that the ranks are no longer in step -- drop the object (``close()``) and build a new one on
    every rank before the next call.
    """

    def __init__(self, rows_local: int, cols: int, brows: int, bcols: int, dtype: torch.dtype,
                 device: torch.device, kind: int = KIND_BLOCK, group: Optional[dist.ProcessGroup] = None,
                 backend=None, exchange: str = "auto", overlap: bool = False, fused_exchange: bool = False):
        """``exchange``: "nccl" (two all-reduces and an all-gather), "p2p" (stores into peer-mapped
        buffers, :class:`PeerExchange`), or "auto": p2p with the CUDA backend on more than one rank when
        the peer buffers can be set up, NCCL otherwise.  The choice is made once, here, by all ranks
        together; both give the same bits.  ``fused_exchange``: with p2p, let the amax kernel's last CTA do
        the exchange of the amax and the count itself where its block shape allows (no launch in between).
        Off by default: every CTA then has to count itself in with a release, which keeps it resident a
        microsecond longer, and on slabs of a GiB and more that costs more than the launch it saves."""
        self.fused_exchange = fused_exchange
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.device = device
        if overlap and backend is not None:
            raise ValueError("overlap=True builds its own two CUDA backends")
        n_sets = 2 if overlap else 1
        self.backends = [backend if backend is not None else CudaBackend(kind, rows_local, cols, brows, bcols, dtype, device)
                         for _ in range(n_sets)]
        self.backend = self.backends[0]
        n_err = self.backend.n_err
        # both exchanges move fixed-size arrays: refuse slabs of different shapes before anything is stored
        check_same_on_every_rank((rows_local, cols, brows, bcols, n_err), "slab shape (rows, cols, block, error entries)", group)
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.collectives = 0
        self.calls = 0
        self.peer = None
        if exchange not in ("auto", "nccl", "p2p"):
            raise ValueError("exchange must be 'auto', 'nccl' or 'p2p'")
        if self.world > 1 and exchange != "nccl" and isinstance(self.backend, CudaBackend):
            try:   # raises on every rank or on none
                self.peer = PeerExchange(n_err, device, group)
            except RuntimeError:
                self.peer = None
                if exchange == "p2p":
                    raise
        self.sets = []
        for _ in range(n_sets):
            all_err = torch.zeros(n_err * self.world, dtype=torch.float32, device=device)
            local = (torch.zeros(n_err, dtype=torch.float32, device=device) if self.peer is not None
                     else all_err[self.rank * n_err:(self.rank + 1) * n_err])
            self.sets.append({"amax": torch.zeros(1, dtype=torch.float32, device=device),
                              "nnz": torch.zeros(1, dtype=torch.int64, device=device),
                              "meta": torch.zeros(1, dtype=torch.int32, device=device),
                              "gerr": torch.zeros(1, dtype=torch.float32, device=device),
                              "all_err": all_err, "local_err": local})
        self.overlap = overlap
        if overlap:
            self.side = torch.cuda.Stream(device)
            self.cast_done = [torch.cuda.Event() for _ in range(2)]
            self.finished = [torch.cuda.Event() for _ in range(2)]

    # the scalars and error sums of the most recent call
    @property
    def local_err(self):
        return self.sets[(self.calls - 1) & (len(self.sets) - 1)]["local_err"] if self.calls else self.sets[0]["local_err"]

    def timed_out(self, result: ScalingResult) -> bool:
        """True if a bounded wait of the call that produced ``result`` ran out (synchronises on one int)."""
        result.wait()
        return int(result.meta.item()) == -1

    def close(self) -> None:
        """Collective: releases the peer-exchange buffers (a no-op for the NCCL exchange)."""
        if self.peer is not None:
            self.peer.close()
            self.peer = None

    def _finish(self, b, s, x, out, threshold, ep):
        """everything after the cast: error exchange, ordered sum and decision, conditional copy"""
        if self.peer is not None:
            ex = self.peer
            b.exchange_errors(ex, ep, s["local_err"])
            b.finalize_ptr(ex.error_ptr(ep), ex.world * ex.n_err, s["nnz"], threshold, s["meta"], s["gerr"])
        else:
            if self.world > 1:
                dist.all_gather_into_tensor(s["all_err"], s["local_err"].clone(), group=self.group)
                self._nnz_done.wait()
                self.collectives += 1
            b.finalize(s["all_err"], s["nnz"], threshold, s["meta"], s["gerr"])
        b.fallback(x, out, s["meta"])

    def __call__(self, x: torch.Tensor, out: torch.Tensor, ss_mode: int, threshold: float) -> ScalingResult:
        i = self.calls & (len(self.sets) - 1)
        b, s = self.backends[i], self.sets[i]
        self.calls += 1
        ep = 0
        if self.peer is not None:
            ex = self.peer
            ex.epoch += 1
            ep = ex.epoch
            if not (self.fused_exchange and b.amax_nnz_exchange(x, ex, ep, s["amax"], s["nnz"])):
                b.amax_nnz_local(x)
                b.exchange_scalars(ex, ep, s["amax"], s["nnz"])
        else:
            b.amax_nnz(x, s["amax"], s["nnz"])
            if self.world > 1:
                # the cast needs the global amax only: the non-zero count is summed while the cast runs
                amax_done = dist.all_reduce(s["amax"], op=dist.ReduceOp.MAX, group=self.group, async_op=True)
                self._nnz_done = dist.all_reduce(s["nnz"], op=dist.ReduceOp.SUM, group=self.group, async_op=True)
                amax_done.wait()
                self.collectives += 2
        if not self.overlap:
            b.cast(x, out, ss_mode, s["amax"], s["local_err"])
            self._finish(b, s, x, out, threshold, ep)
            return ScalingResult(s["meta"], s["amax"], s["nnz"], s["gerr"])
        main = torch.cuda.current_stream(self.device)
        if self.calls >= 2:
            main.wait_event(self.finished[1 - i])    # the previous call's decision and conditional copy, before `out` is written again
        b.cast(x, out, ss_mode, s["amax"], s["local_err"])
        self.cast_done[i].record(main)
        self.side.wait_event(self.cast_done[i])
        with torch.cuda.stream(self.side):
            self._finish(b, s, x, out, threshold, ep)
            self.finished[i].record(self.side)
        return ScalingResult(s["meta"], s["amax"], s["nnz"], s["gerr"], ready=self.finished[i])


class HostScaling:
    """:class:`ShardedScaling` for tensors that live in PINNED HOST memory.

    A call enqueues, and returns without waiting: the host-to-device copy of the slab on a copy
    stream, the four phases on the compute stream, the device-to-host copy of the result and of
    the scalars on a second copy stream.  Two sets of device buffers alternate between calls, so
    the upload of call k+1 runs while call k is being read back -- PCIe carries both directions
    at once -- and the kernels (about 2 % of a call at PCIe speeds) disappear behind the copies.
    ``synchronize()`` waits for everything enqueued; the host result of a call is complete after
    it, or once a later call has reused that call's buffer set (every second call).
    """

    def __init__(self, rows_local: int, cols: int, brows: int, bcols: int, dtype: torch.dtype, device: torch.device,
                 kind: int = KIND_BLOCK, group: Optional[dist.ProcessGroup] = None, backend_factory=None,
                 exchange: str = "auto"):
        self.device = device
        make = backend_factory or (lambda: None)
        self.ops = [ShardedScaling(rows_local, cols, brows, bcols, dtype, device, kind, group, make(), exchange)
                    for _ in range(2)]
        self.x = [torch.empty(rows_local, cols, dtype=dtype, device=device) for _ in range(2)]
        self.out = [torch.empty(rows_local, cols, dtype=dtype, device=device) for _ in range(2)]
        self.s_in, self.s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        self.uploaded = [torch.cuda.Event() for _ in range(2)]
        self.computed = [torch.cuda.Event() for _ in range(2)]
        self.read_back = [torch.cuda.Event() for _ in range(2)]
        self.calls = 0

    def __call__(self, x_host: torch.Tensor, out_host: torch.Tensor, scalars_host: torch.Tensor, ss_mode: int,
                 threshold: float) -> ScalingResult:
        """``x_host`` / ``out_host``: pinned tensors of the slab's shape; ``scalars_host``: pinned float32[2]
        that receives (global_amax, global_error).  Returns the device-side scalars of this call."""
        if not (x_host.is_pinned() and out_host.is_pinned() and scalars_host.is_pinned()):
            raise ValueError("HostScaling needs pinned host tensors (torch.empty(..., pin_memory=True))")
        b = self.calls & 1
        main = torch.cuda.current_stream(self.device)
        if self.calls >= 2:
            self.s_in.wait_event(self.computed[b])     # the kernels that read this input buffer two calls ago
        with torch.cuda.stream(self.s_in):
            self.x[b].copy_(x_host, non_blocking=True)
            self.uploaded[b].record()
        main.wait_event(self.uploaded[b])
        if self.calls >= 2:
            main.wait_event(self.read_back[b])         # the read-back that still used this output buffer
        res = self.ops[b](self.x[b], self.out[b], ss_mode, threshold)
        self.computed[b].record(main)
        self.s_out.wait_event(self.computed[b])
        with torch.cuda.stream(self.s_out):
            out_host.copy_(self.out[b], non_blocking=True)
            scalars_host[0:1].copy_(res.global_amax, non_blocking=True)
            scalars_host[1:2].copy_(res.global_error, non_blocking=True)
            self.read_back[b].record()
        self.calls += 1
        return res

    def synchronize(self):
        self.s_out.synchronize()
        torch.cuda.current_stream(self.device).synchronize()
