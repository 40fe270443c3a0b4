"""Runtime modules, the operator-stage pattern and the per-tensor / per-token activation forms on the GPU,
each checked against the CPU oracle or the reference-generated golden vectors."""

from __future__ import annotations

import pytest
import torch
from torch import nn

from conftest import seeded
from oracle import pattern as opat
from oracle import w4a16 as o16
from oracle import w4a4 as o44
from oracle import w8a8 as o88
from xqt_b200 import engine, native, quantize
from xqt_b200.errors import XQTBackendError
from xqt_b200.modules import AWQW4A16Linear, B200PackedDequantLinear, Int8MmaLinear

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _on_device(pw):
    return type(pw)(qweight=pw.qweight.to(DEV), scales=pw.scales.to(DEV),
                    zero_points=None if pw.zero_points is None else pw.zero_points.to(DEV), metadata=pw.metadata)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_awq_module_forward_bind_and_residual(dtype):
    n, k = 640, 1024
    w = torch.randn((n, k), generator=seeded(11)) * 0.02
    pw = quantize.quantize_w4_asymmetric(w, group_size=128)
    bias = torch.randn((n,), generator=seeded(12)) * 0.1
    with_bias = AWQW4A16Linear(_on_device(pw), bias=bias.to(DEV)).eval()
    plain = AWQW4A16Linear(_on_device(pw)).eval()
    for m in (1, 5, 16, 40):
        x = torch.randn((m, k), generator=seeded(13 + m)).to(dtype)
        want = o16.gemm(x, pw.qweight, pw.scales, pw.zero_points, group_size=128, signed=False, bias=bias)
        got = with_bias(x.to(DEV))
        assert got.dtype == dtype and o16.rel_l2(got.cpu(), want) <= 1e-3
        meta = with_bias.execution_metadata()
        assert meta["native"] and meta["rows"] == m and meta["kernel"] == ("w4a16_decode_cl_kernel" if m <= 16 else "w4a16 tcgen05 GEMM")
    x3 = torch.randn((2, 3, k), generator=seeded(20)).to(dtype)
    assert tuple(plain(x3.to(DEV)).shape) == (2, 3, n)
    # the fused residual epilogue keeps the numerics of the unfused add bit for bit
    for m in (1, 4):
        x = torch.randn((m, k), generator=seeded(30 + m)).to(dtype).to(DEV)
        residual = torch.randn((m, n), generator=seeded(40 + m)).to(dtype).to(DEV)
        unfused = residual + plain.bind(rows=m, dtype=dtype)(x)
        fused = residual.clone()
        assert plain.bind_residual(rows=m, dtype=dtype)(x, fused) is None
        assert torch.equal(fused, unfused)
    with pytest.raises(XQTBackendError):
        with_bias.bind_residual(rows=1, dtype=dtype)
    with pytest.raises(XQTBackendError):
        plain.bind(rows=2, dtype=dtype)(torch.zeros((3, k), device=DEV, dtype=dtype))
    assert native.workspace_status(DEV) == 0


def test_awq_module_freeze_and_signed_storage_import():
    n, k, group = 256, 512, 64

    class Storage:          # the attribute surface of xqt's signed group-wise artifact
        pass

    w = torch.randn((n, k), generator=seeded(50)) * 0.02
    pw = quantize.quantize_w4_symmetric(w, group_size=group)
    st = Storage()
    st.bits, st.group_size, st.output_features, st.input_features, st.padded_input_features = 4, group, n, k, k
    st.quantized_weight, st.weight_scale, st.bias = pw.qweight, pw.scales.unsqueeze(-1), torch.randn((n,), generator=seeded(51))
    module = AWQW4A16Linear.from_signed_groupwise_storage(st, device=DEV).eval()
    x = torch.randn((2, k), generator=seeded(52)).to(torch.bfloat16)
    want = o16.gemm(x, pw.qweight, pw.scales, None, group_size=group, signed=True, bias=st.bias)
    assert o16.rel_l2(module(x.to(DEV)).cpu(), want) <= 1e-3
    st.group_size = 32
    with pytest.raises(XQTBackendError):
        AWQW4A16Linear.from_signed_groupwise_storage(st, device=DEV)
    before = module(x.to(DEV)).clone()
    released = module.freeze_native_inference(device=DEV, dtype=torch.bfloat16, rows=(1, 2))
    assert released == n * k // 2 and module.native_only and module.canonical_qweight is None
    assert torch.equal(module(x.to(DEV)), before)
    with pytest.raises(RuntimeError):
        module(torch.zeros((3, k), device=DEV, dtype=torch.bfloat16))           # rows 3 were not frozen
    with pytest.raises(RuntimeError):
        module(torch.zeros((2, k), device=DEV, dtype=torch.float16))
    with pytest.raises(RuntimeError):
        module.freeze_native_inference(device=DEV, dtype=torch.bfloat16)
    meta = module.execution_metadata()
    assert meta["native_only"] and meta["native_only_rows"] == [1, 2] and meta["native_only_released_bytes"] == released


@pytest.mark.parametrize("m,group,with_zero,activation", [(1, 128, False, None), (4, 64, True, None), (16, 128, True, None),
                                                          (48, 128, True, "silu"), (300, 64, False, "gelu"), (33, 32, True, "relu")])
def test_gemm_int4_dequant_pattern(m, group, with_zero, activation):
    from xqt_b200.ops.pattern import gemm_int4_dequant

    n, k = 384, 1024
    w = torch.randn((n, k), generator=seeded(60)) * 0.02
    pw = quantize.quantize_w4_symmetric(w, group_size=group)
    scale = pw.scales.unsqueeze(-1)                                          # the artifact's [N, G, 1] form
    zero = (torch.randn((n, k // group), generator=seeded(61)) * 0.01) if with_zero else None
    bias = torch.randn((n,), generator=seeded(62)) * 0.1
    x = torch.randn((m, k), generator=seeded(63)).to(torch.bfloat16)
    want = opat.gemm_int4_dequant(x, pw.qweight, scale, zero, bias, group_size=group, activation=activation)
    got = gemm_int4_dequant(x.to(DEV), pw.qweight.to(DEV), scale.to(DEV), None if zero is None else zero.to(DEV), bias.to(DEV),
                            group_size=group, activation=activation)
    assert got.dtype == torch.bfloat16 and o16.rel_l2(got.cpu(), want) <= 1e-3
    with pytest.raises(XQTBackendError):
        gemm_int4_dequant(x.to(DEV), pw.qweight.to(DEV), scale.to(DEV), group_size=group, activation="tanh")
    assert native.workspace_status(DEV) == 0


def test_operator_stage_candidate_is_validated_and_timed():
    from test_engine_cpu import _PackedInt4Linear

    eager = _PackedInt4Linear(n=512, k=1024).to(DEV)
    target = engine.OperatorOptimizationTargetPlan(name="proj", patterns=["gemm_int4_dequant"], validate={"atol": 2e-2, "rtol": 2e-2},
                                                   min_speedup=0.0)
    candidate, _ = engine.materialize_operator_candidate_model(eager, target)
    assert isinstance(candidate, B200PackedDequantLinear)
    sample = torch.randn((4, 1024), generator=seeded(70)).to(torch.bfloat16).to(DEV)
    report = engine.accept_candidate(eager, candidate, sample, target, reps=3)
    assert report["numerics_ok"] and report["accepted"] and report["speedup"] > 0
    assert report["execution_metadata"][0]["execution_mode"] == "b200_cuda_entry"
    strict = engine.OperatorOptimizationTargetPlan(name="proj", validate={"atol": 0.0, "rtol": 0.0}, min_speedup=1e9)
    assert not engine.accept_candidate(eager, candidate, sample, strict, reps=1)["accepted"]


def test_int8_mma_linear_matches_the_reference_vectors(golden):
    g = golden("int8_mma")
    module = Int8MmaLinear(g["qweight_t"], g["weight_scale"], g["bias"], eps=float(g["eps"])).to(DEV)
    out = module(g["x"].to(DEV))
    assert out.dtype == torch.bfloat16
    torch.testing.assert_close(out.float().cpu(), g["out"].to(torch.bfloat16).float(), atol=0, rtol=2 ** -7)
    from xqt_b200.ops.activation import quantize_int8_per_tensor
    codes, rows, scale = quantize_int8_per_tensor(g["x"].to(DEV), eps=float(g["eps"]))
    assert torch.equal(codes.cpu(), g["act_codes"]) and torch.equal(scale.cpu().reshape(()), g["act_scale"])
    assert torch.equal(rows.cpu(), g["act_scale"].expand(rows.numel()))
    meta = module.execution_metadata()
    assert meta["activation_granularity"] == "per_tensor" and meta["true_int8_mma"]
    # a larger, seeded case against the oracle, bias-free, fp16
    n, k, m = 320, 768, 200
    lin = nn.Linear(k, n, bias=False)
    big = Int8MmaLinear.from_linear(lin).to(DEV)
    x = torch.randn((m, k), generator=seeded(80)).to(torch.float16)
    q, s = o88.quantize_act_per_tensor(x, eps=1e-6)
    want = o88.gemm_integer(q, s.expand(m), big.qweight_t.cpu().t().contiguous(), big.weight_scale.cpu(), out_dtype=torch.float16)
    assert o16.rel_l2(big(x.to(DEV)).cpu(), want) <= 1e-3


def test_registry_executor_serves_per_tensor_activations():
    from xqt_b200.contracts import EpilogueSpec, GemmProblem, GemmSpec, QuantSpec
    from xqt_b200.dispatch import dispatch_gemm
    from xqt_b200.executors import install_b200_executors

    install_b200_executors()
    n, k, m = 256, 512, 64
    w = torch.randn((n, k), generator=seeded(81)) * 0.02
    q8, s8 = quantize.quantize_w8_per_channel(w)
    spec = GemmSpec(problem=GemmProblem(m=m, n=n, k=k, sm=100),
                    quant=QuantSpec(weight_dtype="int8", activation_dtype="int8", output_dtype="bf16", weight_granularity="per_channel",
                                    activation_granularity="per_tensor", weight_scale_source="weight_offline",
                                    activation_scale_source="activation_dynamic"),
                    epilogue=EpilogueSpec(output_dtype="bf16"))
    x = torch.randn((m, k), generator=seeded(82)).to(torch.bfloat16)
    result = dispatch_gemm(x.to(DEV), q8.to(DEV), spec=spec, weight_scales=s8.to(DEV))
    assert result.report.native and result.report.selected_kernel == "sm100_w8a8_int8_b200"
    q, s = o88.quantize_act_per_tensor(x, eps=1e-6)
    want = o88.gemm_integer(q, s.expand(m), q8, s8, out_dtype=torch.bfloat16)
    assert o16.rel_l2(result.output.cpu(), want) <= 1e-3


def test_w4a4_per_token_activation_form():
    from xqt_b200.ops.activation import rotate_quantize
    from xqt_b200.ops.w4a4 import pack_svdq_w4a4_linear, svdq_w4a4_linear

    n, k, m, rank = 256, 512, 70, 16
    rot = quantize.regular_rotation(256)
    w = rot.apply(torch.randn((n, k), generator=seeded(90)) * 0.02)
    down, up, residual = quantize.svd_split(w, rank)
    down, up = down.to(torch.bfloat16), up.to(torch.bfloat16)
    packed, scale, _ = quantize.quantize_residual_int4(residual, group_size=64)
    layer = pack_svdq_w4a4_linear(None, down.to(DEV), up.to(DEV), None, packed_residual=packed.to(DEV), residual_scale=scale.to(DEV),
                                  rotation=rot, act_granularity="token")
    x = torch.randn((m, k), generator=seeded(91)).to(torch.bfloat16)
    want, parts = o44.w4a4_forward(x, packed, scale, down, up, group_size=64, rot_kind=rot.kind, rot_block=256, signs=rot.signs,
                                   act_group_size=k, return_parts=True)
    codes, scales = rotate_quantize(x.to(DEV), rot, bits=4, group_size=0)
    assert tuple(scales.shape) == (m, k // 64)
    assert torch.equal(scales.cpu(), parts["s_a"]) and torch.equal(codes.cpu(), parts["q_a"])
    assert o16.rel_l2(svdq_w4a4_linear(x.to(DEV), layer).cpu(), want) <= 1e-3


def test_decode_lanes_symmetric_weights_without_a_zero_plane():
    from xqt_b200.ops.w4a16 import bind_w4a16_decode, prepare_decode

    n, k = 264, 1536
    w = torch.randn((n, k), generator=seeded(95)) * 0.02
    pw = quantize.quantize_w4_symmetric(w, group_size=128)
    tiled = prepare_decode(pw.qweight.to(DEV), pw.scales.to(DEV), None, group_size=128, nibble_signed=True, layout="lanes")
    for m in (1, 9):
        x = torch.randn((m, k), generator=seeded(96 + m)).to(torch.float16)
        want = o16.gemm(x, pw.qweight, pw.scales, None, group_size=128, signed=True)
        assert o16.rel_l2(bind_w4a16_decode(tiled, rows=m, dtype=torch.float16)(x.to(DEV)).cpu(), want) <= 1e-3
