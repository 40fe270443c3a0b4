"""SVDQuant W8A8 (int8 x int8 GEMM + low-rank branch) against its CPU oracle."""

from __future__ import annotations

import pytest
import torch

from conftest import seeded
from oracle import svdq_w8a8 as oracle
from oracle import w4a16 as o16

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _layer(n, k, rank, seed, dtype):
    w = (torch.randn((n, k), generator=seeded(seed)) * 0.02).to(dtype)
    w[3] = 0                                                  # a zero row: scale 1, codes 0
    down = (torch.randn((rank, k), generator=seeded(seed + 1)) * 0.05).to(dtype) if rank else None
    up = (torch.randn((n, rank), generator=seeded(seed + 2)) * 0.05).to(dtype) if rank else None
    return w, down, up


@pytest.mark.parametrize("m,n,k,rank,dtype", [(1, 256, 512, 16, torch.bfloat16), (130, 264, 1024, 32, torch.bfloat16),
                                              (300, 512, 4096, 8, torch.float16), (64, 128, 256, 0, torch.bfloat16)])
def test_svdq_w8a8_forward(m, n, k, rank, dtype):
    from xqt_b200 import native
    from xqt_b200.ops.svdq_w8a8 import pack_svdq_w8a8_linear, svdq_w8a8_linear, w8a8_linear
    w, down, up = _layer(n, k, rank, 40 + n, dtype)
    bias = torch.randn((n,), generator=seeded(5))
    x = torch.randn((m, k), generator=seeded(m)).to(dtype)
    x[m // 2] = 0                                             # an all-zero token: scale 0, codes 0, output = bias
    packed = pack_svdq_w8a8_linear(w.to(DEV), None if down is None else down.to(DEV), None if up is None else up.to(DEV), bias.to(DEV))
    q_w, s_w = oracle.quantize_weight(w)
    assert torch.equal(packed.qweight.cpu(), q_w) and torch.equal(packed.weight_scales.cpu(), s_w)
    out, parts = svdq_w8a8_linear(x.to(DEV), packed, lora_scale=0.5, return_parts=True)
    ref, rparts = oracle.forward(x, q_w, s_w, down, up, bias, lora_scale=0.5, return_parts=True)
    assert torch.equal(parts["codes"].cpu(), rparts["q_a"])          # bit-exact codes and scales
    assert torch.equal(parts["scales"].cpu(), rparts["s_a"])
    assert o16.rel_l2(out.cpu(), ref) <= 1e-3
    plain = w8a8_linear(x.to(DEV), packed)
    assert o16.rel_l2(plain.cpu(), oracle.forward(x, q_w, s_w, None, None, bias)) <= 1e-3
    assert native.workspace_status(DEV) == 0


def test_bound_call_reuses_its_workspace():
    from xqt_b200.ops.svdq_w8a8 import allocate_svdq_w8a8_workspace, bind_svdq_w8a8_linear, pack_svdq_w8a8_linear, svdq_w8a8_linear
    m, n, k, rank = 96, 384, 768, 32
    w, down, up = _layer(n, k, rank, 9, torch.bfloat16)
    packed = pack_svdq_w8a8_linear(w.to(DEV), down.to(DEV), up.to(DEV))
    x = torch.randn((m, k), generator=seeded(2)).to(torch.bfloat16).to(DEV)
    ws = allocate_svdq_w8a8_workspace(m, packed)
    bound = bind_svdq_w8a8_linear(packed, ws, rows=m)
    assert torch.equal(bound(x), svdq_w8a8_linear(x, packed))
    with pytest.raises(Exception):
        bound(x[:10])
