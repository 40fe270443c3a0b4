"""W4A16 SwiGLU MLP block on B200: ``y = down(silu(gate x) * up x)``.

The block shape is xqt's toy SwiGLU MLP (xqt/kernels/nn/fixtures/toy_models.py:87-121); the fusion
choices follow its ConvRot W8A8 backend, which fuses gate and up horizontally into one linear and
gates with one vectorised kernel (xqt/kernels/ops/_impl/cute/convrot_w8a8_sm89.py:664-917,
convrot_w8a8_sm89_kernel.cu:756-837).

Per call and rank: one linear for the concatenated ``[gate; up]`` shard, one SwiGLU kernel, one
linear for the down shard; at M <= 16 the linears are the cluster split-K decode kernel, above it
the tcgen05 GEMM.  With more than one rank gate/up are split over N, down over K, and the fp32 partial
sums of down are added with one NCCL all-reduce and rounded once.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .. import native
from ..contracts import PackedWeight, PackedWeightMetadata
from ..errors import XQTBackendError
from ..parallel import shard_packed_weight
from .w4a16 import bind_w4a16_decode, glu_row_order, prepare_decode, w4a16_linear


def swiglu(gate_up: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``[M, 2I] -> [M, I]``: ``silu(gate_up[:, :I]) * gate_up[:, I:]`` in fp32, rounded once."""

    if gate_up.ndim != 2 or gate_up.shape[1] % 16 or gate_up.dtype not in (torch.float16, torch.bfloat16):
        raise XQTBackendError("swiglu expects a rank-2 fp16/bf16 tensor [M, 2*inter] with inter % 8 == 0")
    if not gate_up.is_cuda or not gate_up.is_contiguous():
        raise XQTBackendError("swiglu expects a contiguous CUDA tensor")
    m, inter = int(gate_up.shape[0]), int(gate_up.shape[1]) // 2
    if out is None:
        out = torch.empty((m, inter), device=gate_up.device, dtype=gate_up.dtype)
    if m:
        with torch.cuda.device(gate_up.device):
            native.check(native.library().xqt_b200_swiglu(
                gate_up.data_ptr(), out.data_ptr(), m, inter, native.DTYPE_CODE[gate_up.dtype],
                native.stream_handle(gate_up.device)), "xqt_b200_swiglu")
    return out


def _concat_rows(a: PackedWeight, b: PackedWeight) -> PackedWeight:
    ma, mb = a.metadata, b.metadata
    if (ma.logical_shape[1], ma.group_size, ma.nibble_signed) != (mb.logical_shape[1], mb.group_size, mb.nibble_signed):
        raise XQTBackendError("gate and up must share K, group size and signedness to be fused")
    if (a.zero_points is None) != (b.zero_points is None):
        raise XQTBackendError("gate and up must both carry zero points or neither")
    n = ma.logical_shape[0] + mb.logical_shape[0]
    values = {f: getattr(ma, f) for f in PackedWeightMetadata.__dataclass_fields__}
    values.update(logical_shape=(n, ma.logical_shape[1]), local_shape=None if ma.local_shape is None else (n, ma.logical_shape[1]))
    return PackedWeight(
        qweight=torch.cat((a.qweight, b.qweight)), scales=torch.cat((a.scales, b.scales)),
        zero_points=None if a.zero_points is None else torch.cat((a.zero_points, b.zero_points)),
        metadata=PackedWeightMetadata(**values))


CHUNKED_DECODE_MAX_ROWS = 32


class _Linear:
    """One W4A16 layer on a device with both execution forms: decode layout and canonical bytes."""

    def __init__(self, weight: PackedWeight, device: torch.device, dtype: torch.dtype, glu: bool = False) -> None:
        meta = weight.metadata
        self.n, self.k = meta.logical_shape
        self.group, self.signed, self.dtype = int(meta.group_size), bool(meta.nibble_signed), dtype
        self.qweight = weight.qweight.to(device).contiguous()
        self.scales = weight.scales.to(device).contiguous()
        self.zeros = None if weight.zero_points is None else weight.zero_points.to(device).contiguous()
        self._bound: dict[tuple[int, torch.dtype], object] = {}
        self._gated: dict[int, object] = {}
        # glu: this is a fused [gate; up] layer.  Where the decode layout is the lanes one its tiles are built from the
        # rows in glu_row_order, and `gated` runs linear + SwiGLU as one decode launch; `tiled` then serves only that.
        self.glu, self.tiled = False, None
        if glu and self.n % 128 == 0:
            order = glu_row_order(self.n // 2).to(device)
            tiled = prepare_decode(self.qweight[order], self.scales[order], None if self.zeros is None else self.zeros[order],
                                   group_size=self.group, nibble_signed=self.signed)
            if tiled.layout == "lanes":
                self.glu, self.tiled = True, tiled
        if self.tiled is None:
            self.tiled = prepare_decode(self.qweight, self.scales, self.zeros, group_size=self.group, nibble_signed=self.signed)

    def gated(self, x: torch.Tensor) -> torch.Tensor | None:
        """``silu(gate) * up`` of a fused gate/up layer in one decode launch per 16 rows, or None where that form does
        not apply (not a glu layer, too many rows)."""

        m = int(x.shape[0])
        if not self.glu or m > CHUNKED_DECODE_MAX_ROWS:
            return None
        out = torch.empty((m, self.n // 2), device=x.device, dtype=self.dtype)
        for r0 in range(0, m, 16):
            rows = min(16, m - r0)
            run = self._gated.get(rows)
            if run is None:
                run = bind_w4a16_decode(self.tiled, rows=rows, dtype=self.dtype, glu=True)
                self._gated[rows] = run
            run(x if rows == m else x[r0:r0 + rows], out if rows == m else out[r0:r0 + rows])
        return out

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
        m = int(x.shape[0])
        odt = self.dtype if out_dtype is None else out_dtype
        if self.glu and m <= CHUNKED_DECODE_MAX_ROWS:
            raise XQTBackendError("a glu layer's decode tiles are interleaved: call gated()")
        if m <= 16 and (odt == self.dtype or self.tiled.layout in ("rows128", "lanes")):
            run = self._bound.get((m, odt))
            if run is None:
                run = bind_w4a16_decode(self.tiled, rows=m, dtype=self.dtype, out_dtype=odt)
                self._bound[(m, odt)] = run
            return run(x, out) if out is not None else run(x)
        if m <= CHUNKED_DECODE_MAX_ROWS and self.tiled.layout == "lanes":
            # a few decode passes over 16-row chunks: the packed weights of a layer (tens of MB) stay in the 126 MB
            # L2 between passes, and each pass runs at the decode kernel's rate -- measured ahead of the GEMM forms
            # up to two passes (from 33 rows the fused tcgen05 GEMM is ahead)
            if out is None:
                out = torch.empty((m, self.n), device=x.device, dtype=odt)
            for r0 in range(0, m, 16):
                rows = min(16, m - r0)
                run = self._bound.get((rows, odt))
                if run is None:
                    run = bind_w4a16_decode(self.tiled, rows=rows, dtype=self.dtype, out_dtype=odt)
                    self._bound[(rows, odt)] = run
                run(x[r0:r0 + rows], out[r0:r0 + rows])
            return out
        return w4a16_linear(x, self.qweight, self.scales, self.zeros, group_size=self.group,
                            nibble_signed=self.signed, k=self.k, out_dtype=odt, out=out)

    def partial_into(self, x: torch.Tensor, peer) -> None:
        """Decode-size fp32 partial sums of a K-sharded layer, written into the slot of ``peer`` (a counted
        :class:`xqt_b200.parallel.PeerAllReduce`) that its next reduction reads; the kernel picks the slot on the device."""

        m = int(x.shape[0])
        run = self._bound.get((m, "peer"))
        if run is None:
            run = bind_w4a16_decode(self.tiled, rows=m, dtype=self.dtype, out_dtype=torch.float32, out_select=peer.out_select)
            self._bound[(m, "peer")] = run
        run(x, peer.partial(m, self.n))

    def rows(self, x: torch.Tensor, n0: int, n1: int, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """The output channels [n0, n1) only: ``x @ W[n0:n1]^T`` (a row block of the canonical weight is contiguous)."""

        return w4a16_linear(x, self.qweight[n0:n1], self.scales[n0:n1], None if self.zeros is None else self.zeros[n0:n1],
                            group_size=self.group, nibble_signed=self.signed, k=self.k,
                            out_dtype=self.dtype if out_dtype is None else out_dtype)


class _InjectedLinear:
    """One layer served by a caller-supplied ``local_linear(x, weight, out_dtype=...)`` (the gloo tests run the
    block's sharding and reduction logic on the CPU with the oracle in this seat)."""

    def __init__(self, weight: PackedWeight, local_linear) -> None:
        self.weight, self.local_linear = weight, local_linear
        self.n, self.k = weight.metadata.logical_shape
        self.tiled = None

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
        y = self.local_linear(x, self.weight) if out_dtype is None else self.local_linear(x, self.weight, out_dtype=out_dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y


class W4A16SwiGLUMLP:
    """The MLP block of one rank.  ``gate`` / ``up`` are canonical ``[inter, hidden]`` weights,
    ``down`` is ``[hidden, inter]``; they are sharded here for ``rank`` of ``world``.  ``local_linear`` /
    ``swiglu_fn`` replace the CUDA kernels (tests of the multi-rank logic on CPU ranks)."""

    def __init__(self, gate: PackedWeight, up: PackedWeight, down: PackedWeight, *, device: torch.device,
                 dtype: torch.dtype = torch.bfloat16, rank: int = 0, world: int = 1, group=None,
                 peer_reduce: bool | None = None, local_linear=None, swiglu_fn=None) -> None:
        if world > 1:
            gate = shard_packed_weight(gate, world=world, rank=rank, axis=0)
            up = shard_packed_weight(up, world=world, rank=rank, axis=0)
            down = shard_packed_weight(down, world=world, rank=rank, axis=1)
        self.world, self.group, self.dtype = world, group, dtype
        self._swiglu = swiglu_fn or swiglu
        if local_linear is not None:
            self.gate_up = _InjectedLinear(_concat_rows(gate, up), local_linear)
            self.down = _InjectedLinear(down, local_linear)
            peer_reduce = False
        else:
            self.gate_up = _Linear(_concat_rows(gate, up), device, dtype, glu=swiglu_fn is None and os.environ.get("XQT_B200_FUSED_SWIGLU", "1") not in {"0", ""})
            self.down = _Linear(down, device, dtype)
        self.hidden, self.inter_local = self.down.n, self.down.k
        # decode sizes (M <= 16): the partial sums of down are added by our own kernel over NVLink peer
        # memory instead of an NCCL all-reduce (XQT_B200_PEER_REDUCE=0 or peer_reduce=False: NCCL)
        if peer_reduce is None:
            peer_reduce = os.environ.get("XQT_B200_PEER_REDUCE", "1") not in {"0", ""}
        self._peer = None
        if world > 1 and peer_reduce and self.down.tiled is not None and self.down.tiled.layout in ("rows128", "lanes"):
            from ..parallel import PeerAllReduce

            # on the lanes layout the reduction is the counted (graph-safe) form: the call number lives on the device
            self._peer = PeerAllReduce(device, 16 * self.hidden, group, counted=self.down.tiled.layout == "lanes")

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        h = self.gate_up.gated(x) if isinstance(self.gate_up, _Linear) else None     # decode sizes: one launch
        if h is None:
            h = self._swiglu(self.gate_up(x))
        if self.world == 1:
            return self.down(h)
        m = int(h.shape[0])
        if self._peer is not None and m <= 16:
            if self._peer.counted:
                self.down.partial_into(h, self._peer)
            else:
                self.down(h, out_dtype=torch.float32, out=self._peer.partial(m, self.hidden))
            return self._peer.reduce(m, self.hidden, dtype=self.dtype)
        blocks = self._reduce_blocks(m)
        if blocks == 1 or not isinstance(self.down, _Linear):
            partial = self.down(h, out_dtype=torch.float32)
            dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.group)
            return partial.to(self.dtype)
        # The down projection in column blocks of the output: block j's fp32 partial sums are all-reduced (NCCL, its
        # own stream) while block j + 1 is computed, so only the last block's reduction is exposed.  Blocks cut the
        # weight's rows, every packed weight is still dequantised once.
        width = self.hidden // blocks
        parts, works = [], []
        for j in range(blocks):
            part = self.down.rows(h, j * width, (j + 1) * width, out_dtype=torch.float32)
            works.append(dist.all_reduce(part, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
            parts.append(part)
        out = torch.empty((m, self.hidden), device=h.device, dtype=self.dtype)
        for j, (part, work) in enumerate(zip(parts, works)):
            work.wait()
            out[:, j * width:(j + 1) * width].copy_(part)       # the cast to the activation dtype
        return out

    def capture(self, rows: int):
        """The block for a fixed row count as one CUDA graph (the decode kernels chain through programmatic dependent
        launch inside the graph, so the launches run without host gaps -- what xqt's graph decode runtime does around
        its modules, xqt/runtime/graph_decode.py).  Single-GPU blocks at any row count; with more ranks the decode
        sizes, whose reduction is the counted peer-memory kernel (every rank must then capture and replay in step: the
        same number of calls on every rank).  Returns ``replay`` with
        ``replay.input`` (``[rows, hidden]``, written by the caller, e.g. the target of its host-to-device copy) and
        ``replay.output``; ``replay()`` launches the graph on the current stream and returns ``replay.output``."""

        rows = int(rows)
        if self.world != 1 and not (self._peer is not None and self._peer.counted and rows <= 16):
            raise XQTBackendError("capture: with more than one rank only the decode sizes (rows <= 16) on the counted "
                                  "peer-memory reduction can be captured (NCCL collectives stay outside graphs here)")
        device = self.gate_up.qweight.device
        static_in = torch.zeros((rows, self.hidden), device=device, dtype=self.dtype)
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            for _ in range(2):                      # bind the callables and load the kernels outside the capture
                self(static_in)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                static_out = self(static_in)
        torch.cuda.current_stream(device).wait_stream(side)

        def replay() -> torch.Tensor:
            graph.replay()
            return static_out

        replay.input, replay.output, replay.graph = static_in, static_out, graph
        return replay

    def _reduce_blocks(self, m: int) -> int:
        """Column blocks of the row-parallel reduction.  One block (the whole partial in one all-reduce) unless
        ``XQT_B200_REDUCE_BLOCKS`` asks for more: measured on two GPUs the blocked form is slower at every M (M = 4096:
        850 / 867 / 950 us with 1 / 2 / 4 blocks; M = 512: 242 / 293 / 460 us) -- the narrower GEMMs lose more than the
        overlapped part of a two-rank all-reduce gains.  More ranks shift that balance; it is a knob, not a default."""

        forced = os.environ.get("XQT_B200_REDUCE_BLOCKS")
        if forced and m >= 256 and self.hidden % (128 * max(1, int(forced))) == 0:
            return max(1, int(forced))
        return 1

    def execution_metadata(self) -> dict:
        """Which kernels serve this block (the report xqt's runtime modules expose,
        xqt/runtime/modules/composite_add_w4a4.py:304-318)."""

        return {
            "implementation": "b200_w4a16_swiglu_mlp", "world": self.world,
            "reduction": "none" if self.world == 1 else ("peer_allreduce_kernel (M <= 16) / " if self._peer else "") +
                         "NCCL all-reduce of fp32 partial sums (XQT_B200_REDUCE_BLOCKS: in column blocks overlapped with the down projection)",
            "decode_layout": None if self.gate_up.tiled is None else self.gate_up.tiled.layout, "hidden": self.hidden,
            "inter_local": self.inter_local,
            "kernels": {"m<=16": {"lanes": "w4a16_decode_cl_kernel", "rows128": "w4a16_decode_tc_kernel"}.get(
                            None if self.gate_up.tiled is None else self.gate_up.tiled.layout, "w4a16_decode_kernel"),
                        "17<=m<=128": "gemm_w4a16_fused_kernel (where it fills the SMs) else dequant_w4_f16_kernel + gemm_f16_kernel",
                        "m>128": "dequant_w4_f16_kernel + gemm_f16_kernel",
                        "gating": "w4a16_decode_cl_kernel epilogue (m <= 32) / swiglu_kernel" if getattr(self.gate_up, "glu", False) else "swiglu_kernel"},
        }


__all__ = ["W4A16SwiGLUMLP", "swiglu"]
