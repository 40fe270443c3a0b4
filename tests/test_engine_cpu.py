"""Operator-stage integration on the CPU: engine registration, materializer, fallbacks, and -- when an
xqt checkout is importable (``XQT_REFERENCE_PATH``) -- the hand-off to xqt's own engine table and artifact."""

from __future__ import annotations

import os
import sys

import pytest
import torch
from torch import nn

from conftest import seeded
from oracle import w8a8 as oracle_w8a8
from xqt_b200 import engine, quantize
from xqt_b200.errors import XQTBackendError
from xqt_b200.modules import B200PackedDequantLinear, Int8MmaLinear


class _PackedInt4Linear(nn.Module):
    """Stand-in for xqt's weight-only artifact: holds signed-nibble bytes and exposes the bridge."""

    def __init__(self, n=8, k=256, group=128):
        super().__init__()
        pw = quantize.quantize_w4_symmetric(torch.randn((n, k), generator=seeded(1)) * 0.02, group_size=group)
        self.register_buffer("quantized_weight", pw.qweight)
        self.register_buffer("weight_scale", pw.scales.unsqueeze(-1))
        self.input_features, self.group_size = k, group

    def triton_packed_dequant_gemm_args(self, *, dtype, device):
        return self.quantized_weight.to(device), self.weight_scale.to(device=device, dtype=dtype), None, None, self.input_features, self.group_size

    def forward(self, x):
        from oracle import pattern
        return pattern.gemm_int4_dequant(x, self.quantized_weight, self.weight_scale, group_size=self.group_size)


def test_engine_registration_schema():
    reg = engine.register_b200_engine()
    assert reg.name == "b200_cuda" and reg.materializer == "b200_cuda" and reg.min_capability == 100
    assert {"gemm_int4_dequant", "dequant_gemm_epilogue", "int8_mma"} <= set(reg.provides)
    assert reg.operator_visible and reg.requires_cuda


def test_materializer_replaces_bridged_modules_and_keeps_the_rest():
    model = nn.Sequential(nn.LayerNorm(256), _PackedInt4Linear(), nn.ReLU())
    target = engine.OperatorOptimizationTargetPlan(name="proj", target_path=None, patterns=["gemm_int4_dequant"])
    candidate, compile_ms = engine.materialize_operator_candidate_model(model, target)
    assert compile_ms is None and candidate is not model
    assert isinstance(candidate[1], B200PackedDequantLinear) and isinstance(model[1], _PackedInt4Linear)   # the original is untouched
    assert isinstance(candidate[0], nn.LayerNorm)
    single, _ = engine.materialize_operator_candidate_model(model, engine.OperatorOptimizationTargetPlan(name="p", target_path="1"))
    assert isinstance(single[1], B200PackedDequantLinear)
    with pytest.raises(XQTBackendError, match="does not serve patterns"):
        engine.build_b200_candidate_model(_PackedInt4Linear(), engine.OperatorOptimizationTargetPlan(name="p", patterns=["attention"]))
    with pytest.raises(XQTBackendError, match="found no packed int4 linear"):
        engine.build_b200_candidate_model(nn.Sequential(nn.Linear(4, 4)), engine.OperatorOptimizationTargetPlan(name="p"))


def test_wrapper_fallback_policy_on_cpu_inputs():
    wrapped = B200PackedDequantLinear(_PackedInt4Linear(), fallback="eager")
    x = torch.randn((3, 256), generator=seeded(2)).to(torch.bfloat16)
    out = wrapped(x)                                   # CPU tensor: the stage's declared fallback is the eager module
    assert torch.equal(out, wrapped.module(x))
    meta = wrapped.execution_metadata()
    assert meta["execution_mode"] == "eager_fallback" and meta["kernel_pattern"] == "gemm_int4_dequant" and meta["engine"] == "b200_cuda"
    with pytest.raises(XQTBackendError):
        B200PackedDequantLinear(_PackedInt4Linear(), fallback="none")(x)
    with pytest.raises(XQTBackendError):
        B200PackedDequantLinear(nn.Linear(4, 4))


def test_per_tensor_int8_oracle_and_module_quantiser_match_the_reference(golden):
    g = golden("int8_mma")
    q, scale = oracle_w8a8.quantize_act_per_tensor(g["x"], eps=float(g["eps"]))
    assert torch.equal(scale, g["act_scale"]) and torch.equal(q, g["act_codes"])
    torch.set_num_threads(1)
    out = oracle_w8a8.gemm_integer(q, scale.expand(q.shape[0]), g["qweight_t"].t().contiguous(), g["weight_scale"], bias=g["bias"],
                                   out_dtype=torch.float32)
    torch.testing.assert_close(out, g["out"], atol=1e-6, rtol=1e-6)
    lin = nn.Linear(256, 24)
    with torch.no_grad():
        lin.weight.copy_(torch.randn((24, 256), generator=seeded(90)) * 0.02)
    mod = Int8MmaLinear.from_linear(lin)
    assert torch.equal(mod.qweight_t, g["qweight_t"]) and torch.equal(mod.weight_scale, g["weight_scale"])


def test_materializer_accepts_the_reference_artifact_and_engine_table():
    path = os.environ.get("XQT_REFERENCE_PATH")
    if path and path not in sys.path:
        sys.path.insert(0, path)
    weight_only = pytest.importorskip("xqt.contracts.weight_only")
    xer = pytest.importorskip("xqt.kernels.engine_resolve")
    lin = nn.Linear(256, 16, bias=True)
    artifact = weight_only.AWQGPTQWeightOnlyLinear.from_linear(lin, bits=4, group_size=128, method="awq")
    candidate = engine.build_b200_candidate_model(artifact, engine.OperatorOptimizationTargetPlan(name="p", patterns=["gemm_int4_dequant"]))
    assert isinstance(candidate, B200PackedDequantLinear)
    assert "gemm_int4_dequant" in xer.operator_contract_patterns("linear")
    registered = engine.register_b200_engine()
    assert type(registered) is xer.EngineRegistration and xer.get_engine_registration("b200_cuda") is registered
    x = torch.randn((2, 256), generator=seeded(3))
    assert torch.equal(candidate(x), artifact(x))          # CPU input: eager fallback, the artifact's own forward
