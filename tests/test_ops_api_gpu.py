"""The reference-named op surfaces on the GPU: AWQ decode (prepack -> parameters -> decode / bind),
ConvRot W8A8 and SVDQuant W4A4 with caller-owned workspaces and bound callables, and the SVD dual-path
registry executor.  Every result is checked against the CPU oracle."""

from __future__ import annotations

import pytest
import torch

from conftest import seeded
from oracle import w4a16 as o16
from oracle import w4a4 as o44
from oracle import w8a8 as o88
from xqt_b200 import native, quantize
from xqt_b200.errors import XQTBackendError

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _on_device(pw):
    return type(pw)(qweight=pw.qweight.to(DEV), scales=pw.scales.to(DEV),
                    zero_points=None if pw.zero_points is None else pw.zero_points.to(DEV), metadata=pw.metadata)


@pytest.mark.parametrize("symmetric,group,param_dtype", [(False, 128, torch.bfloat16), (False, 64, torch.float32),
                                                         (True, 128, torch.float32)])
def test_awq_decode_three_step_path(symmetric, group, param_dtype):
    from xqt_b200.contracts import EpilogueSpec, GemmProblem, GemmSpec
    from xqt_b200.ops import awq

    n, k, m = 392, 1024, 7
    w = torch.randn((n, k), generator=seeded(3)) * 0.02
    pw = quantize.quantize_w4_symmetric(w, group_size=group) if symmetric else \
        quantize.quantize_w4_asymmetric(w, group_size=group, param_dtype=param_dtype)
    x = torch.randn((m, k), generator=seeded(4)).to(torch.bfloat16)
    bias = torch.randn((n,), generator=seeded(5))
    ref = o16.gemm(x, pw.qweight, pw.scales, pw.zero_points, group_size=group, signed=symmetric)
    ref_b = o16.gemm(x, pw.qweight, pw.scales, pw.zero_points, group_size=group, signed=symmetric, bias=bias)
    assert awq.native_awq_w4a16_available(build=True) and awq.native_awq_w4a16_shape_supported(m, k, n, group)
    execution = awq.prepack_b200_awq_w4a16_decode(_on_device(pw))
    assert execution.metadata.storage_layout == awq.LANES_LAYOUT and execution.canonical_qweight is not None
    spec = GemmSpec(problem=GemmProblem(m=m, n=n, k=k, phase="decode", sm=100),
                    quant=quantize.w4_spec(group_size=group, symmetric=symmetric), epilogue=EpilogueSpec(output_dtype="bf16"))
    qweight, scales, zeros = awq.prepare_b200_awq_w4a16_decode_parameters(execution, spec=spec, dtype=torch.bfloat16)
    out = torch.empty((m, n), device=DEV, dtype=torch.bfloat16)
    assert awq.awq_w4a16_decode(x.to(DEV), qweight, scales, zeros, output=out) is out
    assert o16.rel_l2(out.cpu(), ref) <= 1e-3
    bound = awq.bind_awq_w4a16_decode(qweight, scales, zeros, rows=m, input_features=k, output_features=n,
                                      dtype=torch.bfloat16, device=DEV, bias=bias.to(DEV))
    assert o16.rel_l2(bound(x.to(DEV)).cpu(), ref_b) <= 1e-3
    out_exec = awq.b200_awq_w4a16_decode_executor(x.to(DEV), execution, spec=spec, bias=bias.to(DEV))
    assert torch.equal(out_exec, bound(x.to(DEV)))
    with pytest.raises(XQTBackendError):
        awq.prepare_b200_awq_w4a16_decode_parameters(_on_device(pw), dtype=torch.bfloat16)     # not prepacked
    with pytest.raises(XQTBackendError):
        awq.bind_awq_w4a16_decode(qweight, scales, zeros, rows=17, input_features=k, output_features=n,
                                  dtype=torch.bfloat16, device=DEV)
    assert native.workspace_status(DEV) == 0


def test_registry_decode_path_caches_the_layout_per_weight_tensor():
    from xqt_b200 import executors
    from xqt_b200.contracts import EpilogueSpec, GemmProblem, GemmSpec

    n, k, m = 256, 512, 3
    pw = _on_device(quantize.quantize_w4_asymmetric(torch.randn((n, k), generator=seeded(7)) * 0.02, group_size=128))
    x = torch.randn((m, k), generator=seeded(8)).to(torch.bfloat16)
    spec = GemmSpec(problem=GemmProblem(m=m, n=n, k=k, phase="decode", sm=100),
                    quant=quantize.w4_spec(group_size=128, symmetric=False), epilogue=EpilogueSpec(output_dtype="bf16"))
    first = executors.b200_w4a16_executor(x.to(DEV), pw, spec=spec)
    entry = executors._decode_layouts.get(pw.qweight)
    assert entry is not None and entry["tiled"].layout == "lanes"
    second = executors.b200_w4a16_executor(x.to(DEV), pw, spec=spec)          # second call: cache hit, same callable
    assert executors._decode_layouts.get(pw.qweight) is entry and torch.equal(first, second)
    ref = o16.gemm(x, pw.qweight.cpu(), pw.scales.cpu(), pw.zero_points.cpu(), group_size=128, signed=False)
    assert o16.rel_l2(first.cpu(), ref) <= 1e-3
    pw.qweight.add_(0)                                                         # an in-place write bumps the version
    executors.b200_w4a16_executor(x.to(DEV), pw, spec=spec)
    assert executors._decode_layouts.get(pw.qweight) is not entry


def test_convrot_w8a8_workspace_bind_and_prerotated_input():
    from xqt_b200.ops import w8a8

    m, n, k = 48, 264, 512
    rot = quantize.regular_rotation(256)
    w = torch.randn((n, k), generator=seeded(11)) * 0.02
    q, s = quantize.quantize_w8_per_channel(rot.apply(w))
    packed = w8a8.pack_convrot_w8a8_linear(q.t().contiguous().to(DEV), s.to(DEV), None, dtype=torch.bfloat16)
    x = torch.randn((m, k), generator=seeded(12)).to(torch.bfloat16)
    ref = o88.linear(x, q, s, rot_block=256)
    assert w8a8.native_convrot_w8a8_available(torch.bfloat16, build=True)
    assert w8a8.native_convrot_w8a8_shape_supported(k, k, n, 256) and not w8a8.native_convrot_w8a8_shape_supported(k, k, n, 100)
    workspace = w8a8.allocate_convrot_w8a8_workspace(64, packed)
    out = w8a8.convrot_w8a8_linear(x.to(DEV), packed, rotated_input_features=k, rot_size=256, workspace=workspace)
    assert o16.rel_l2(out.cpu(), ref) <= 1e-3
    bound = w8a8.bind_convrot_w8a8_linear(packed, workspace, rows=m, rotated_input_features=k, rot_size=256)
    assert torch.equal(bound(x.to(DEV)), out)
    # rot_size == 1: the caller rotated already
    x_rot = rot.apply(x.float()).to(torch.bfloat16)
    pre = w8a8.convrot_w8a8_linear(x_rot.to(DEV), packed, rotated_input_features=k, rot_size=1)
    ref_pre = o88.gemm_reference(*o88.quantize_act_per_token(x_rot), q, s)
    assert o16.rel_l2(pre.cpu(), ref_pre) <= 1e-3
    with pytest.raises(XQTBackendError):
        w8a8.convrot_w8a8_linear(x.to(DEV), packed, rotated_input_features=True, rot_size=256)   # xqt's argument is the padded K
    with pytest.raises(XQTBackendError):
        w8a8.convrot_w8a8_linear(x.to(DEV), packed, rotated_input_features=k + 256, rot_size=256)


def test_svdq_w4a4_workspace_bind_and_registry_executor():
    from xqt_b200.contracts import EpilogueSpec, GemmProblem, GemmSpec, QuantSpec
    from xqt_b200.dispatch import dispatch_gemm
    from xqt_b200.executors import SVDGemmContract, install_b200_executors
    from xqt_b200.layout import W4_LAYOUT, build_packed_weight
    from xqt_b200.ops import w4a4
    from xqt_b200.registry import B200_SVD_W4A4, GemmKernelRegistry, b200_rows

    m, n, k, rank = 80, 264, 512, 8
    rot = quantize.randomized_rotation(128, seed=5)
    w_rot = rot.apply(torch.randn((n, k), generator=seeded(21)) * 0.02)
    down, up, residual = quantize.svd_split(w_rot, rank)
    down, up = down.to(torch.bfloat16), up.to(torch.bfloat16)
    packed_r, scale_r, _ = quantize.quantize_residual_int4(residual, group_size=64)
    bias = torch.randn((n,), generator=seeded(22))
    x = torch.randn((m, k), generator=seeded(23)).to(torch.bfloat16)
    ref = o44.w4a4_forward(x, packed_r, scale_r, down, up, group_size=64, rot_kind=rot.kind, rot_block=128, signs=rot.signs, bias=bias)
    layer = w4a4.pack_svdq_w4a4_linear(None, down.to(DEV), up.to(DEV), bias.to(DEV), packed_residual=packed_r.to(DEV),
                                       residual_scale=scale_r.to(DEV), rotation=rot)
    assert w4a4.native_w4a4_available(build=True) and w4a4.native_w4a4_shape_supported(k, n)
    workspace = w4a4.allocate_w4a4_workspace(128, layer, with_lora_rank=rank)
    out = w4a4.svdq_w4a4_linear(x.to(DEV), layer, workspace=workspace)
    assert o16.rel_l2(out.cpu(), ref) <= 1e-3
    bound = w4a4.bind_svdq_w4a4_linear(layer, workspace, rows=m)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated(DEV)
    again = bound(x.to(DEV))
    torch.cuda.synchronize()
    assert torch.equal(again, out)
    # the bound call allocated its input copy and its output, nothing else survives it
    del again
    assert torch.cuda.memory_allocated(DEV) <= before
    # the registry executor: rotation applied by the caller, low-rank pair as executor kwargs
    quant = QuantSpec(weight_dtype="int4", activation_dtype="bf16", output_dtype="bf16", weight_granularity="groupwise",
                      group_size=64, symmetric=True, weight_zero_point=False, weight_scale_source="weight_offline",
                      storage_layout=W4_LAYOUT)
    weight = build_packed_weight(packed_r.to(DEV), logical_shape=(n, k), spec=quant, scales=scale_r.to(DEV), padded_k=k)
    spec = GemmSpec(problem=GemmProblem(m=m, n=n, k=k, sm=100), quant=quant, epilogue=EpilogueSpec(has_bias=True, output_dtype="bf16"))
    reg = GemmKernelRegistry(b200_rows())
    assert B200_SVD_W4A4 in install_b200_executors(reg)
    contract = SVDGemmContract(main_spec=spec, rank=rank, fusion_boundary="fuse_up")
    result = dispatch_gemm(x.to(DEV), weight, spec=spec, registry=reg, requested_kernel=B200_SVD_W4A4, bias=bias.to(DEV),
                           executor_kwargs={"low_rank_down": down.to(DEV), "low_rank_up": up.to(DEV), "contract": contract,
                                            "rotation": rot})
    torch.cuda.synchronize()
    assert result.report.selected_kernel == B200_SVD_W4A4 and result.report.native
    assert o16.rel_l2(result.output.cpu(), ref) <= 1e-3
    # against the reference's floating dual path the only difference is the int4 activation rounding
    dual = o44.composite_forward(rot.apply(x.float()), packed_r, scale_r, down, up, group_size=64, bias=bias)
    assert o16.rel_l2(result.output.float().cpu(), dual) < 0.25
    assert native.workspace_status(DEV) == 0


@pytest.mark.parametrize("symmetric,scalar_scale", [(True, True), (False, False)])
def test_awq_w4a8_decode(symmetric, scalar_scale):
    """int8 activation codes with one scale against the W4 execution layout: exact integer group sums, fp32
    scaling -- checked against the integer arithmetic of the reference's DP4A kernel restated on the CPU."""

    from xqt_b200.layout import unpack_int4
    from xqt_b200.ops import awq

    n, k, m, group = 264, 1024, 3, 128
    w = torch.randn((n, k), generator=seeded(40)) * 0.02
    pw = quantize.quantize_w4_symmetric(w, group_size=group) if symmetric else quantize.quantize_w4_asymmetric(w, group_size=group)
    codes = torch.randint(-127, 128, (m, k), generator=seeded(41), dtype=torch.int8)
    scale_a = 0.0173
    q = unpack_int4(pw.qweight, logical_k=k, signed=symmetric).to(torch.float64)
    if not symmetric:
        q = q - pw.zero_points.to(torch.float64).repeat_interleave(group, dim=1)
    sums = torch.einsum("mgk,ngk->mng", codes.to(torch.float64).reshape(m, k // group, group), q.reshape(n, k // group, group))
    ref = ((sums * pw.scales.to(torch.float64).unsqueeze(0)).sum(dim=2) * scale_a).to(torch.float32).to(torch.bfloat16)
    execution = awq.prepack_b200_awq_w4a16_decode(_on_device(pw))
    qweight, scales, zeros = awq.prepare_b200_awq_w4a16_decode_parameters(execution, dtype=torch.bfloat16)
    out = torch.empty((m, n), device=DEV, dtype=torch.bfloat16)
    sa = scale_a if scalar_scale else torch.tensor(scale_a, device=DEV)
    got = awq.awq_w4a8_decode(codes.to(DEV), qweight, scales, sa, scaled_zeros=zeros, dtype=torch.bfloat16, output=out)
    assert got is out and o16.rel_l2(out.cpu(), ref) <= 1e-3
    run = awq.bind_awq_w4a8_decode(qweight, scales, zeros, rows=m, input_features=k, output_features=n, dtype=torch.bfloat16,
                                   device=DEV, residual=True)
    res = torch.randn((m, n), generator=seeded(42)).to(torch.bfloat16)
    assert torch.equal(run(codes.to(DEV), sa, res.to(DEV)).cpu(), out.cpu() + res)
    with pytest.raises(XQTBackendError):
        awq.awq_w4a8_decode(codes.to(DEV).to(torch.bfloat16), qweight, scales, sa)
    assert native.workspace_status(DEV) == 0
