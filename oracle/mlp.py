"""Oracle for the W4A16 SwiGLU MLP block.  Test infrastructure only.

``y = down(silu(gate(x)) * up(x))`` with three W4A16 linears, the block shape of
xqt's toy SwiGLU MLP (xqt/kernels/nn/fixtures/toy_models.py:87-121).  Each
linear is the contract reference (fp32 dequant + fp32 matmul, one cast to the
activation dtype, xqt/kernels/ops/gemm/reference.py:469-577); the gating product
is evaluated in fp32 from the two rounded projections and rounded once, which is
what a fused ``silu(g) * u`` elementwise kernel produces
(convrot_w8a8_sm89_kernel.cu:756-837).
"""

from __future__ import annotations

import torch

from . import w4a16


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    g = gate.to(torch.float32)
    return (torch.nn.functional.silu(g) * up.to(torch.float32)).to(gate.dtype)


def forward(x, gate_w, up_w, down_w, *, group_size: int, signed: bool = False):
    """Each ``*_w`` is ``(qweight, scales, zero_points)``."""

    g = w4a16.gemm(x, *gate_w, group_size=group_size, signed=signed)
    u = w4a16.gemm(x, *up_w, group_size=group_size, signed=signed)
    return w4a16.gemm(swiglu(g, u), *down_w, group_size=group_size, signed=signed)


def forward_sharded(x, gate_w, up_w, down_w, *, group_size: int, world: int, signed: bool = False):
    """Tensor-parallel evaluation order: gate/up split over N, down split over K,
    fp32 partial sums added in rank order, one final cast."""

    inter = gate_w[0].shape[0]
    step = inter // world
    gstep = step // group_size
    total = None
    for r in range(world):
        rows = slice(r * step, (r + 1) * step)
        g = w4a16.gemm(x, gate_w[0][rows], gate_w[1][rows], None if gate_w[2] is None else gate_w[2][rows],
                       group_size=group_size, signed=signed)
        u = w4a16.gemm(x, up_w[0][rows], up_w[1][rows], None if up_w[2] is None else up_w[2][rows],
                       group_size=group_size, signed=signed)
        h = swiglu(g, u)
        cols = slice(r * step // 2, (r + 1) * step // 2)
        gcols = slice(r * gstep, (r + 1) * gstep)
        part = w4a16.gemm(h, down_w[0][:, cols].contiguous(), down_w[1][:, gcols],
                          None if down_w[2] is None else down_w[2][:, gcols],
                          group_size=group_size, signed=signed, out_dtype=torch.float32)
        total = part if total is None else total + part
    return total.to(x.dtype)
