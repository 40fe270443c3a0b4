"""Column / row partitioning of quantized linears over the GPUs of one node (NCCL over NVLink).

xqt has no multi-device execution; it only declares where a shard would be recorded
(``PackedWeightMetadata.local_shape / shard_axis``, xqt/kernels/ops/gemm/contracts.py:379-402).  This
module fills and consumes those fields:

* column-parallel (``shard_axis=0``): rank r owns output channels ``[r N/g, (r+1) N/g)`` -- contiguous
  row slices of ``qweight``, ``scales`` and ``zero_points``; the activation is replicated; outputs
  are concatenated with an all-gather (or left sharded when the next layer is row-parallel);
* row-parallel (``shard_axis=1``): rank r owns input features ``[r K/g, (r+1) K/g)`` -- the byte
  columns ``[r K/2g, ...)`` of ``qweight`` and the group columns of the scales; every rank produces
  an fp32 partial ``[M, N]`` which is summed with an all-reduce and rounded once.

One process per GPU, ``torch.distributed`` for the plumbing; collectives run on the current stream
after the kernels that feed them.  The local computation is injected (``local_linear``), so the
partition arithmetic and the collective wiring are tested on CPU ranks with the gloo backend.
The GEMM / GEMV kernels read only their own GPU's memory; the one kernel that reads peers' memory is the
decode-size reduction of ``PeerAllReduce`` (plain peer loads over NVLink, no cluster-wide TMA loads).
"""

from __future__ import annotations

from dataclasses import fields
from typing import Callable

import torch
import torch.distributed as dist

from .contracts import PackedWeight, PackedWeightMetadata
from .errors import XQTBackendError


def shard_packed_weight(weight: PackedWeight, *, world: int, rank: int, axis: int) -> PackedWeight:
    """Slice a canonical W4 ``PackedWeight`` for ``rank`` of ``world``.  ``axis`` 0 = over N
    (column-parallel), 1 = over K (row-parallel).  Shards keep the canonical byte layout."""

    meta = weight.metadata
    n, k = meta.logical_shape
    group = int(meta.group_size)
    if not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    if meta.padded_k != k:
        raise XQTBackendError("sharding needs K == padded_K")
    if axis == 0:
        if n % world:
            raise XQTBackendError(f"N={n} is not divisible by {world} ranks")
        rows = n // world
        sl = slice(rank * rows, (rank + 1) * rows)
        q, s = weight.qweight[sl], weight.scales[sl]
        z = None if weight.zero_points is None else weight.zero_points[sl]
        local = (rows, k)
    elif axis == 1:
        if k % (world * group) or (k // world) % 2:
            raise XQTBackendError(f"K={k} must split into {world} whole groups of {group}")
        cols = k // world
        q = weight.qweight[:, rank * cols // 2:(rank + 1) * cols // 2]
        gs = slice(rank * cols // group, (rank + 1) * cols // group)
        s = weight.scales[:, gs]
        z = None if weight.zero_points is None else weight.zero_points[:, gs]
        local = (n, cols)
    else:
        raise ValueError("axis must be 0 (N) or 1 (K)")
    values = {f.name: getattr(meta, f.name) for f in fields(PackedWeightMetadata)}
    values.update(logical_shape=local, padded_k=local[1], local_shape=local, shard_axis=axis)
    return PackedWeight(
        qweight=q.contiguous(), scales=s.contiguous(), zero_points=None if z is None else z.contiguous(),
        metadata=PackedWeightMetadata(**values))


LocalLinear = Callable[..., torch.Tensor]


def _default_local_linear(x, weight: PackedWeight, *, out_dtype=None, bias=None):
    from .ops.w4a16 import w4a16_linear

    meta = weight.metadata
    return w4a16_linear(x, weight.qweight, weight.scales, weight.zero_points, bias, group_size=int(meta.group_size),
                        nibble_signed=bool(meta.nibble_signed), k=meta.logical_shape[1], out_dtype=out_dtype)


class ColumnParallelLinear:
    """``y = x W^T`` with W split over N.  ``gather_output=False`` leaves ``[M, N/g]`` on each rank."""

    def __init__(self, shard: PackedWeight, *, group=None, gather_output: bool = True, bias: torch.Tensor | None = None,
                 local_linear: LocalLinear | None = None) -> None:
        if shard.metadata.shard_axis != 0:
            raise XQTBackendError("ColumnParallelLinear needs a shard over N (shard_axis=0)")
        self.shard, self.group, self.gather_output, self.bias = shard, group, gather_output, bias
        self.local_linear = local_linear or _default_local_linear
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        local = self.local_linear(x, self.shard, bias=self.bias)
        if not self.gather_output or self.world == 1:
            return local
        m, n_local = local.shape
        # all_gather_into_tensor concatenates the ranks' [m, n_local] blocks along dim 0
        gathered = torch.empty((self.world * m, n_local), device=local.device, dtype=local.dtype)
        dist.all_gather_into_tensor(gathered, local.contiguous(), group=self.group)
        return gathered.reshape(self.world, m, n_local).permute(1, 0, 2).reshape(m, self.world * n_local)


class RowParallelLinear:
    """``y = x W^T`` with W split over K; ``x`` is the rank's slice ``[M, K/g]``.  Partials are fp32,
    summed with an all-reduce, bias added once, result rounded once to the activation dtype."""

    def __init__(self, shard: PackedWeight, *, group=None, bias: torch.Tensor | None = None,
                 local_linear: LocalLinear | None = None) -> None:
        if shard.metadata.shard_axis != 1:
            raise XQTBackendError("RowParallelLinear needs a shard over K (shard_axis=1)")
        self.shard, self.group, self.bias = shard, group, bias
        self.local_linear = local_linear or _default_local_linear
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return self.local_linear(x, self.shard, bias=self.bias)
        partial = self.local_linear(x, self.shard, out_dtype=torch.float32)
        dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.group)
        if self.bias is not None:
            partial = partial + self.bias.to(partial.dtype)
        return partial.to(x.dtype)


class PeerAllReduce:
    """Sum of the ranks' fp32 partials over NVLink peer memory, epilogue (bias, rounding) fused in.

    One instance per (process group, device).  ``partial(call_rows, n)`` hands out this rank's slot of
    the shared buffer for the next call (the row-parallel GEMV writes its fp32 result straight into
    it), ``reduce(rows, n, bias, dtype)`` launches the kernel that waits for the peers, adds the
    partials in rank order and returns the rank's own full ``[rows, n]`` output.  Buffers come from
    torch's symmetric memory (plain peer pointers).  Meant for decode sizes (a few hundred KiB): every
    rank reads every partial once; larger reductions stay with NCCL.
    """

    MAX_WORLD = 8

    def __init__(self, device: torch.device, max_elements: int, group=None, counted: bool = False) -> None:
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem

        from . import native

        group = dist.group.WORLD if group is None else group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if not 2 <= self.world <= self.MAX_WORLD:
            raise XQTBackendError(f"PeerAllReduce serves 2..{self.MAX_WORLD} ranks")
        self.device, self.max_elements = device, int(-(-max_elements // 4) * 4)
        # two alternating slots of fp32 partials, then the flag words
        self._buffer = symm_mem.empty(2 * self.max_elements + 64, dtype=torch.float32, device=device)
        self._buffer.zero_()
        handle = symm_mem.rendezvous(self._buffer, group)
        self._handle = handle
        base = [int(ptr) for ptr in handle.buffer_ptrs]
        self._slot_ptrs = [[b + slot * self.max_elements * 4 for b in base] for slot in (0, 1)]
        flag_ptrs = [b + 2 * self.max_elements * 4 for b in base]
        array = ctypes.c_void_p * self.world
        self._partials = [array(*ptrs) for ptrs in self._slot_ptrs]
        self._flags = array(*flag_ptrs)
        self._call = 0
        self._native = native
        # counted form: the call number lives in device memory ([0] finished calls, [1] block tickets), the kernels pick
        # the slot from it, and a launch may be captured into a CUDA graph (see reduce)
        self.counted = bool(counted)
        self._counter = torch.zeros(4, dtype=torch.int32, device=device) if counted else None
        # the kernel reports a peer that never signalled here; pinned, so the host reads it without a sync
        self._host_status = torch.zeros(16, dtype=torch.int32).pin_memory()
        self.spin_limit = 0          # 0 = the kernel's default bound (2^22 polls)
        torch.cuda.synchronize(device)
        dist.barrier(group)          # every rank's zeros are in place before anybody signals

    @property
    def out_select(self) -> tuple[int, int]:
        """``(address of the finished-call counter, bytes between the two slots)`` for the kernel that writes this rank's
        partial (counted form): it then stores at ``partial(...) + ((counter + 1) & 1) * stride``."""

        if not self.counted:
            raise XQTBackendError("PeerAllReduce: out_select belongs to the counted form")
        return self._counter.data_ptr(), self.max_elements * 4

    def partial(self, rows: int, n: int) -> torch.Tensor:
        """This rank's fp32 ``[rows, n]`` slot for the NEXT call of ``reduce`` (counted form: slot 0, from which the
        writing kernel steps to the slot in use through ``out_select``)."""

        count = rows * n
        if count > self.max_elements:
            raise XQTBackendError("PeerAllReduce: partial larger than the buffer it was built with")
        slot = 0 if self.counted else (self._call + 1) & 1
        return self._buffer[slot * self.max_elements: slot * self.max_elements + count].view(rows, n)

    def reduce(self, rows: int, n: int, *, bias: torch.Tensor | None = None, dtype: torch.dtype = torch.bfloat16,
               out: torch.Tensor | None = None) -> torch.Tensor:
        native = self._native
        if n % 4 or dtype not in (torch.float16, torch.bfloat16):
            raise XQTBackendError("PeerAllReduce: N must be a multiple of 4 and the output fp16 or bf16")
        if self.counted:
            # nothing in this launch changes from call to call: it may be captured and replayed
            if not torch.cuda.is_current_stream_capturing():
                self.check()
            if out is None:
                out = torch.empty((rows, n), device=self.device, dtype=dtype)
            with torch.cuda.device(self.device):
                code = native.library().xqt_b200_peer_allreduce_counted(
                    self._partials[0], self._flags, self.rank, self.world, self._counter.data_ptr(), self.max_elements, rows * n, n,
                    native.ptr(bias), out.data_ptr(), native.DTYPE_CODE[dtype], int(self.spin_limit),
                    self._host_status.data_ptr(), native.stream_handle(self.device))
            native.check(code, "xqt_b200_peer_allreduce_counted")
            return out
        if torch.cuda.is_current_stream_capturing():
            # the call number is a host-side counter passed by value: a replayed graph would repeat it,
            # its wait would pass at once and it would sum partials that are still being written
            raise XQTBackendError("PeerAllReduce.reduce with a host call number cannot be captured into a CUDA graph (build it with counted=True)")
        self.check()
        self._call += 1
        if out is None:
            out = torch.empty((rows, n), device=self.device, dtype=dtype)
        with torch.cuda.device(self.device):
            code = native.library().xqt_b200_peer_allreduce(
                self._partials[self._call & 1], self._flags, self.rank, self.world, self._call & 0xFFFFFFFF or 1, rows * n, n,
                native.ptr(bias), out.data_ptr(), native.DTYPE_CODE[dtype], int(self.spin_limit),
                self._host_status.data_ptr(), native.stream_handle(self.device))
        native.check(code, "xqt_b200_peer_allreduce")
        return out

    def check(self) -> None:
        """Raise if a finished ``reduce`` gave up waiting for a peer (its output was not the sum).
        Called at the start of every ``reduce``; call it after a synchronisation to check the last one."""

        if int(self._host_status[0]) != 0:
            code = int(self._host_status[0])
            self._host_status.zero_()
            raise XQTBackendError(f"PeerAllReduce: a rank did not signal within the wait bound (status {code}); "
                                  "the affected outputs are not valid")


class PeerAllGather:
    """Concatenation of the ranks' output bytes over NVLink peer memory, graph-safe (the counted form of
    :class:`PeerAllReduce`: the call number lives in device memory).

    Every rank's kernels write their ``nbytes`` of output into ``slot0`` stepped by ``out_select`` (the decode kernel
    selects the slot of this two-slot buffer on the device); ``gather(out)`` launches the kernel that signals the
    peers, waits for them (bounded) and copies every rank's slot into ``out[rank]``.  All launches have fixed
    arguments, so a step of local kernels followed by ``gather`` can be captured into one CUDA graph; every rank must
    make the same sequence of calls."""

    def __init__(self, device: torch.device, nbytes: int, group=None) -> None:
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem

        from . import native

        group = dist.group.WORLD if group is None else group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if not 2 <= self.world <= PeerAllReduce.MAX_WORLD:
            raise XQTBackendError(f"PeerAllGather serves 2..{PeerAllReduce.MAX_WORLD} ranks")
        self.device, self.nbytes = device, int(-(-int(nbytes) // 256) * 256)
        self._buffer = symm_mem.empty(2 * self.nbytes + 256, dtype=torch.uint8, device=device)
        self._buffer.zero_()
        handle = symm_mem.rendezvous(self._buffer, group)
        self._handle = handle
        base = [int(ptr) for ptr in handle.buffer_ptrs]
        array = ctypes.c_void_p * self.world
        self._sources = array(*base)
        self._flags = array(*[b + 2 * self.nbytes for b in base])
        self._counter = torch.zeros(4, dtype=torch.int32, device=device)
        self._host_status = torch.zeros(16, dtype=torch.int32).pin_memory()
        self._native = native
        self.spin_limit = 0
        torch.cuda.synchronize(device)
        dist.barrier(group)

    @property
    def slot0(self) -> torch.Tensor:
        """This rank's slot 0 as uint8 ``[nbytes]``: the address the writing kernels are given (with ``out_select``)."""

        return self._buffer[: self.nbytes]

    @property
    def out_select(self) -> tuple[int, int]:
        return self._counter.data_ptr(), self.nbytes

    def gather(self, out: torch.Tensor, nbytes: int | None = None) -> torch.Tensor:
        """``out`` (contiguous, ``world * nbytes`` bytes): rank r's bytes at ``[r * nbytes, (r + 1) * nbytes)``."""

        native = self._native
        count = self.nbytes if nbytes is None else int(nbytes)
        if count % 16 or count > self.nbytes or out.numel() * out.element_size() != self.world * count or not out.is_contiguous():
            raise XQTBackendError("PeerAllGather: out must hold world * nbytes contiguous bytes, nbytes a multiple of 16")
        if not torch.cuda.is_current_stream_capturing():
            self.check()
        with torch.cuda.device(self.device):
            code = native.library().xqt_b200_peer_allgather_counted(
                self._sources, self._flags, self.rank, self.world, self._counter.data_ptr(), self.nbytes, count, out.data_ptr(),
                int(self.spin_limit), self._host_status.data_ptr(), native.stream_handle(self.device))
        native.check(code, "xqt_b200_peer_allgather_counted")
        return out

    def check(self) -> None:
        if int(self._host_status[0]) != 0:
            code = int(self._host_status[0])
            self._host_status.zero_()
            raise XQTBackendError(f"PeerAllGather: a rank did not signal within the wait bound (status {code}); "
                                  "the gathered outputs are not valid")


__all__ = ["ColumnParallelLinear", "PeerAllGather", "PeerAllReduce", "RowParallelLinear", "shard_packed_weight"]
