"""ConvRot W8A8 on the GPU against the CPU oracle: activation codes and scales bit-exact, output
rel-L2 <= 1e-3 against the reference's dequantise-then-matmul form."""

from __future__ import annotations

import pytest
import torch

from conftest import seeded
from oracle import rotation as orot
from oracle import w4a16 as o16
from oracle import w8a8 as oracle
from xqt_b200 import native, quantize
from xqt_b200.errors import XQTBackendError
from xqt_b200.ops.activation import rotate_quantize
from xqt_b200.ops.w8a8 import convrot_w8a8_linear, pack_convrot_w8a8_linear, w8a8_gemm

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _layer(n, k, seed, rot):
    w = torch.randn((n, k), generator=seeded(seed)) * 0.02
    q, s = quantize.quantize_w8_per_channel(rot.apply(w))
    return q, s


@pytest.mark.parametrize("kind,block", [("regular", 256), ("regular", 64), ("regular", 16), ("sylvester", 128),
                                        ("sylvester", 32), (None, 0)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_rotation_and_int8_codes_bit_exact(kind, block, dtype):
    m, k = 37, 1024
    x = (torch.randn((m, k), generator=seeded(3)) * 1.7).to(dtype)
    if kind is None:
        rot, x_rot = None, x
    else:
        rot = quantize.Rotation(kind, block, orot.random_signs(block, 5) if kind == "sylvester" else None)
        x_rot = orot.rotate_fht(x, kind=kind, block=block, signs=rot.signs)
    q_ref, s_ref = oracle.quantize_act_per_token(x_rot)
    codes, scales, rotated = rotate_quantize(x.to(DEV), rot, bits=8, return_rotated=True)
    torch.cuda.synchronize()
    assert torch.equal(rotated.cpu(), x_rot)
    assert torch.equal(scales.cpu(), s_ref.reshape(-1))
    assert torch.equal(codes.cpu(), q_ref)


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (256, 256, 512), (100, 136, 272), (2048, 4096, 4096),
                                   (1, 64, 128), (300, 384, 1040)])
def test_w8a8_gemm_integer_exact(m, n, k):
    # random int8 operands, unit scales: the tensor-core accumulation must be exact
    a = torch.randint(-128, 128, (m, k), generator=seeded(m + n), dtype=torch.int64).to(torch.int8)
    w = torch.randint(-127, 128, (n, k), generator=seeded(k), dtype=torch.int64).to(torch.int8)
    sa = torch.rand((m,), generator=seeded(1)) * 1e-2 + 1e-3
    sw = torch.rand((n,), generator=seeded(2)) * 1e-3 + 1e-4
    packed = pack_convrot_w8a8_linear(w.t().contiguous().to(DEV), sw.to(DEV), None, dtype=torch.bfloat16)
    out = w8a8_gemm(a.to(DEV), sa.to(DEV), packed)
    torch.cuda.synchronize()
    assert native.workspace_status(DEV) == 0
    ref = oracle.gemm_integer(a, sa, w, sw)
    assert o16.rel_l2(out.cpu(), ref) <= 1e-3
    mismatch = (out.cpu() != ref).float().mean().item()
    assert mismatch < 0.01          # same fp32 value rounded once to bf16; isolated ulp flips only


def test_config4_full_forward():
    # x [2048,4096] ~ N(0,1) bf16, regular Hadamard 256, W [4096,4096] ~ N(0,0.02) per-channel int8
    m, n, k = 2048, 4096, 4096
    rot = quantize.regular_rotation(256)
    x = torch.randn((m, k), generator=seeded(5)).to(torch.bfloat16)
    q, s = _layer(n, k, 6, rot)
    bias = torch.randn((n,), generator=seeded(7))
    packed = pack_convrot_w8a8_linear(q.t().contiguous().to(DEV), s.to(DEV), bias.to(DEV), dtype=torch.bfloat16)
    out = convrot_w8a8_linear(x.to(DEV), packed, rot_size=256)
    torch.cuda.synchronize()
    ref = oracle.linear(x, q, s, rot_block=256, rot_kind="regular", bias=bias)
    assert o16.rel_l2(out.cpu(), ref) <= 1e-3
    assert native.workspace_status(DEV) == 0


def test_batched_input_and_fp16():
    rot = quantize.regular_rotation(64)
    x = torch.randn((3, 5, 256), generator=seeded(11)).to(torch.float16)
    q, s = _layer(72, 256, 12, rot)
    packed = pack_convrot_w8a8_linear(q.t().contiguous().to(DEV), s.to(DEV), None, dtype=torch.float16)
    out = convrot_w8a8_linear(x.to(DEV), packed, rot_size=64)
    assert tuple(out.shape) == (3, 5, 72)
    ref = oracle.linear(x.reshape(15, 256), q, s, rot_block=64, rot_kind="regular")
    assert o16.rel_l2(out.cpu().reshape(15, 72), ref) <= 1e-3


@pytest.mark.gpu
@pytest.mark.parametrize("prequantized", [True, False])
def test_registry_executor_through_dispatch(prequantized):
    """The GEMM-registry row `sm100_w8a8_int8_b200`: int8 codes + per-token scales, or a floating
    activation quantised per token by the prologue kernel."""

    from xqt_b200.contracts import EpilogueSpec, GemmProblem, GemmSpec, QuantSpec
    from xqt_b200.dispatch import dispatch_gemm
    from xqt_b200.executors import install_b200_executors
    from xqt_b200.registry import B200_W8A8, GemmKernelRegistry, b200_rows

    m, n, k = 96, 264, 512
    dev = torch.device("cuda", 0)
    w = torch.randn((n, k), generator=seeded(21)) * 0.02
    q_w, s_w = quantize.quantize_w8_per_channel(w)
    x = torch.randn((m, k), generator=seeded(22)).to(torch.bfloat16)
    bias = torch.randn((n,), generator=seeded(23))
    q_a, s_a = oracle.quantize_act_per_token(x)
    ref = oracle.gemm_integer(q_a, s_a, q_w, s_w, bias=bias, out_dtype=torch.bfloat16)
    reg = GemmKernelRegistry(b200_rows())
    assert B200_W8A8 in install_b200_executors(reg)
    spec = GemmSpec(
        problem=GemmProblem(m=m, n=n, k=k, sm=100),
        quant=QuantSpec(weight_dtype="int8", activation_dtype="int8", output_dtype="bf16", weight_granularity="per_channel",
                        activation_granularity="per_token", weight_scale_source="weight_offline",
                        activation_scale_source="activation_dynamic"),
        epilogue=EpilogueSpec(has_bias=True, output_dtype="bf16"))
    if prequantized:
        result = dispatch_gemm(q_a.to(dev), q_w.to(dev), spec=spec, registry=reg, weight_scales=s_w.to(dev),
                               activation_scales=s_a.to(dev), bias=bias.to(dev))
    else:
        result = dispatch_gemm(x.to(dev), q_w.to(dev), spec=spec, registry=reg, weight_scales=s_w.to(dev), bias=bias.to(dev))
    torch.cuda.synchronize()
    assert result.report.selected_kernel == B200_W8A8 and result.report.native
    assert o16.rel_l2(result.output.cpu(), ref) <= 1e-3


@pytest.mark.gpu
def test_shared_and_fused_projection_groups():
    """Gate/up style groups: one prologue for all projections; the fused group is one horizontal GEMM whose
    column slices equal the separate projections bit for bit, and feeds the SwiGLU kernel."""

    from oracle import mlp as omlp
    from xqt_b200.ops.w8a8 import FusedConvRotW8A8LinearGroup, SharedConvRotW8A8Group

    dev = torch.device("cuda", 0)
    m, k, inter = 70, 512, 384
    rot = quantize.regular_rotation(256)
    x = torch.randn((m, k), generator=seeded(31)).to(torch.bfloat16)
    packeds, refs = [], []
    for i in range(2):
        w = torch.randn((inter, k), generator=seeded(32 + i)) * 0.02
        q, s = quantize.quantize_w8_per_channel(rot.apply(w))
        bias = torch.randn((inter,), generator=seeded(34 + i)) if i == 0 else None
        packeds.append(pack_convrot_w8a8_linear(q.t().contiguous().to(dev), s.to(dev), None if bias is None else bias.to(dev),
                                                dtype=torch.bfloat16))
        refs.append(oracle.linear(x, q, s, rot_block=256, bias=bias))
    shared = SharedConvRotW8A8Group(packeds, rot_size=256)(x.to(dev))
    fused_group = FusedConvRotW8A8LinearGroup(packeds, rot_size=256)
    fused = fused_group(x.to(dev))
    for got_s, got_f, ref in zip(shared, fused, refs):
        assert o16.rel_l2(got_s.cpu(), ref) <= 1e-3
        assert torch.equal(got_s, got_f)
    gated = fused_group.forward_swiglu(x.to(dev))
    assert torch.equal(gated.cpu(), omlp.swiglu(fused[0].cpu(), fused[1].cpu()))
    x3 = x.reshape(2, 35, k).to(dev)
    assert tuple(fused_group(x3)[1].shape) == (2, 35, inter)
    with pytest.raises(XQTBackendError):
        FusedConvRotW8A8LinearGroup(packeds + packeds[:1], rot_size=256).forward_swiglu(x.to(dev))
