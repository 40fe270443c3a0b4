"""Host-side mirror of xqt's operator API: contracts, canonical layouts, registry/dispatch with fake
executors, kernel namespace.  Written after the reference's CPU tier (tests/gemm/test_w4_pack.py,
test_registry.py:113-226, tests/kernels/test_registry_cpu.py:21-190): no GPU, no native code run."""

from __future__ import annotations

from dataclasses import replace

import pytest
import torch

from conftest import seeded
from xqt_b200 import kernel_spec as ks
from xqt_b200 import layout, quantize
from xqt_b200.contracts import EpilogueSpec, GemmProblem, GemmSpec, QuantSpec
from xqt_b200.dispatch import dispatch_gemm
from xqt_b200.errors import XQTBackendError
from xqt_b200.registry import B200_W4A16, GemmKernelRegistry, b200_rows


def test_pack_unpack_matches_reference_vectors(golden):
    g = golden("pack")
    assert torch.equal(layout.pack_int4_unsigned(g["codes_u"]), g["packed_u"])
    assert torch.equal(layout.pack_int4_signed(g["codes_s"]), g["packed_s"])
    assert torch.equal(layout.unpack_int4(g["packed_u"], logical_k=37, signed=False), g["unpacked_u"])
    assert torch.equal(layout.unpack_int4(g["packed_s"], logical_k=40, signed=True), g["unpacked_s"])
    with pytest.raises(ValueError):
        layout.pack_int4_signed(torch.tensor([[8]], dtype=torch.int8))
    with pytest.raises(ValueError):
        layout.pack_int4_unsigned(torch.tensor([[16]], dtype=torch.int16))


def test_awq_and_gptq_repack_match_reference(golden):
    g = golden("pack")
    awq = layout.repack_awq_int4(
        g["awq_words"], logical_shape=(32, 24), scales=torch.rand((1, 32), generator=seeded(4)) + 0.5,
        zero_points=torch.randint(0, 16, (1, 32), generator=seeded(5)).to(torch.float32), group_size=32)
    assert torch.equal(awq.qweight, g["awq_qweight"])
    assert torch.equal(awq.scales, g["awq_scales"]) and torch.equal(awq.zero_points, g["awq_zeros"])
    assert awq.metadata.padded_k == int(g["awq_padded_k"]) and not awq.metadata.nibble_signed
    gptq = layout.repack_gptq_int4(g["gptq_words"], logical_shape=(16, 64),
                                   scales=torch.rand((2, 16), generator=seeded(7)) + 0.5, group_size=32)
    assert torch.equal(gptq.qweight, g["gptq_qweight"]) and torch.equal(gptq.scales, g["gptq_scales"])
    assert gptq.metadata.nibble_signed and gptq.zero_points is None
    with pytest.raises(ValueError):
        layout.repack_gptq_int4(g["gptq_words"], logical_shape=(16, 64), scales=torch.ones((2, 16)), group_size=32,
                                g_idx=torch.arange(64).flip(0))      # act-order is not supported


def test_signed_to_unsigned_bridge():
    codes = torch.randint(-8, 8, (4, 16), generator=seeded(1), dtype=torch.int64)
    packed = layout.pack_int4_signed(codes)
    assert torch.equal(layout.unpack_int4(layout.signed_storage_to_unsigned(packed), logical_k=16, signed=False).long() - 8,
                       codes)


def test_contract_validation():
    with pytest.raises(ValueError):
        GemmProblem(m=1, n=0, k=4)
    assert GemmProblem(m=0, n=4, k=4).shape == (0, 4, 4)          # only M may be zero
    assert GemmProblem(m=1, n=1, k=1, sm=100).arch == "sm_100"
    with pytest.raises(ValueError):
        QuantSpec(weight_dtype="int4", weight_granularity="groupwise", group_size=128)      # needs a scale source
    with pytest.raises(ValueError):
        QuantSpec(weight_dtype="int4", weight_scale_source="weight_offline", group_size=128)  # group only if groupwise
    with pytest.raises(ValueError):
        GemmSpec(problem=GemmProblem(m=1, n=1, k=1), quant=QuantSpec(output_dtype="bf16"))    # epilogue dtype mismatch
    spec = quantize.w4_spec(group_size=128, symmetric=False)
    assert spec.scale_mode == "w:groupwise/a:per_tensor" and spec.is_weight_only
    assert QuantSpec.from_dict(spec.to_dict()) == spec


def test_w4a16_validator_rejects_what_the_reference_rejects():
    pw = quantize.quantize_w4_asymmetric(torch.randn((8, 256), generator=seeded(1)), group_size=128)
    spec = quantize.w4_spec(group_size=128, symmetric=False)
    layout.validate_w4a16_packed_weight(pw, spec=spec, logical_shape=(8, 256))
    with pytest.raises(ValueError):
        layout.validate_w4a16_packed_weight(pw, spec=spec, logical_shape=(8, 128))
    with pytest.raises(ValueError):
        layout.validate_w4a16_packed_weight(pw, spec=quantize.w4_spec(group_size=64, symmetric=False), logical_shape=(8, 256))
    with pytest.raises(ValueError):
        layout.validate_w4a16_packed_weight(pw, spec=quantize.w4_spec(group_size=128, symmetric=True), logical_shape=(8, 256))
    bad = replace(pw, metadata=replace(pw.metadata, storage_layout="something_else"))
    with pytest.raises(ValueError):
        layout.validate_w4a16_packed_weight(bad, spec=spec, logical_shape=(8, 256))


def _spec(m=4, n=8, k=256):
    return GemmSpec(problem=GemmProblem(m=m, n=n, k=k, sm=100, device="cuda:0"),
                    quant=quantize.w4_spec(group_size=128, symmetric=False), epilogue=EpilogueSpec(output_dtype="bf16"))


def test_registry_conflicts_and_replace():
    reg = GemmKernelRegistry(b200_rows())
    reg.register(b200_rows()[0])                                   # identical entry: no-op
    with pytest.raises(ValueError):
        reg.register(replace(b200_rows()[0], backend="triton"))
    with pytest.raises(KeyError):
        reg.replace(replace(b200_rows()[0], name="unknown_row"))
    with pytest.raises(ValueError):
        replace(b200_rows()[0], maturity="executable")             # executable needs an executor
    # the SVD dual-path row serves the same request shape (it needs a low-rank pair) and ranks below W4A16
    assert [e.name for e in reg.matching(_spec().problem, _spec().quant, _spec().epilogue)] == [B200_W4A16, "sm100_svd_w4a4_b200"]
    other_arch = GemmProblem(m=4, n=8, k=256, sm=89)
    assert reg.matching(other_arch, _spec().quant, _spec().epilogue) == ()


def test_dispatch_runs_fake_executor_and_reports():
    reg = GemmKernelRegistry(b200_rows())
    pw = quantize.quantize_w4_asymmetric(torch.randn((8, 256), generator=seeded(1)), group_size=128)
    calls = []

    def fake(activation, weight, *, spec, **kwargs):
        calls.append(kwargs)
        return torch.full((spec.problem.m, spec.problem.n), 7.0)

    reg.replace(replace(reg.get(B200_W4A16), maturity="executable", executor=fake))
    result = dispatch_gemm(torch.zeros((4, 256), dtype=torch.bfloat16), pw, spec=_spec(), registry=reg,
                           executor_kwargs={"variant": "gemv"})
    assert result.report.native and result.report.selected_kernel == B200_W4A16
    assert result.report.shape_variant == "gemv_m_le_16" and result.report.group_size == 128
    assert calls[0]["variant"] == "gemv" and float(result.output[0, 0]) == 7.0
    assert result.report.to_dict()["fallback_chain"] == [B200_W4A16, "sm100_svd_w4a4_b200"]


def test_dispatch_without_executable_row_raises_and_never_falls_back_to_cpu():
    reg = GemmKernelRegistry(b200_rows())
    pw = quantize.quantize_w4_asymmetric(torch.randn((8, 256), generator=seeded(1)), group_size=128)
    x = torch.zeros((4, 256), dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="maturity=metadata_only"):
        dispatch_gemm(x, pw, spec=_spec(), registry=reg)

    def failing(*args, **kwargs):
        raise XQTBackendError("artifact missing")

    reg.replace(replace(reg.get(B200_W4A16), maturity="executable", executor=failing))
    with pytest.raises(RuntimeError, match="artifact missing"):
        dispatch_gemm(x, pw, spec=_spec(), registry=reg)
    with pytest.raises(XQTBackendError):
        dispatch_gemm(x, pw, spec=_spec(), registry=reg, allow_reference=True)
    with pytest.raises(ValueError):
        dispatch_gemm(x, pw, spec=_spec(), registry=reg, requested_kernel="sm100_w8a8_int8_b200")


def test_executor_rejects_cpu_tensors_with_backend_error():
    from xqt_b200.executors import b200_w4a16_executor
    pw = quantize.quantize_w4_asymmetric(torch.randn((8, 256), generator=seeded(1)), group_size=128)
    with pytest.raises(XQTBackendError):
        b200_w4a16_executor(torch.zeros((4, 256), dtype=torch.bfloat16), pw, spec=_spec())
    with pytest.raises(XQTBackendError):
        b200_w4a16_executor(torch.zeros((4, 256), dtype=torch.bfloat16), pw.qweight, spec=_spec())


def test_kernel_namespace_selection_and_conflicts(monkeypatch):
    table = ks.KernelRegistry()
    sm89 = frozenset({ks.CapabilityRequirement.cuda(min_sm=(8, 9), max_sm=(8, 9))})
    theirs = ks.KernelSpec("quantization.awq_w4a16_decode", ks.KernelBackend.TVM_FFI, "xqt.somewhere:fn", sm89)
    ours = ks.B200_KERNELS[0]
    table.register(theirs)
    table.register(ours)
    table.register(ours)                                           # same spec twice is fine
    with pytest.raises(ValueError):
        table.register(replace(ours, target="xqt_b200.ops.w4a16:w4a16_linear"))
    b200 = ks.PlatformInfo("cuda", 10, 0)
    ada = ks.PlatformInfo("cuda", 8, 9)
    assert ks.select_kernel(ours.op, platform=b200, table=table) is ours
    assert ks.select_kernel(ours.op, platform=ada, table=table) is theirs
    with pytest.raises(ValueError):
        ks.select_kernel(ours.op, platform=ks.PlatformInfo("cpu"), table=table)
    monkeypatch.setenv("XQT_FORCE_BACKEND", "tvm_ffi")
    assert ks.select_kernel(ours.op, platform=b200, table=table) is theirs
    monkeypatch.delenv("XQT_FORCE_BACKEND")
    assert callable(ours.load())
    with pytest.raises(XQTBackendError):
        replace(ours, target="xqt_b200.ops.w4a16:missing").load()
    with pytest.raises(KeyError):
        ks.select_kernel("quantization.nothing", table=table)
    assert "quantization.svdq_w4a4_linear" in ks.registry.ops() and "quantization.gemm_int4_dequant" in ks.registry.ops()


def _w8a8_spec(m=4, n=8, k=64, out="bf16"):
    from xqt_b200.contracts import EpilogueSpec, GemmSpec

    return GemmSpec(
        problem=GemmProblem(m=m, n=n, k=k, sm=100),
        quant=QuantSpec(weight_dtype="int8", activation_dtype="int8", output_dtype=out, weight_granularity="per_channel",
                        activation_granularity="per_token", weight_scale_source="weight_offline",
                        activation_scale_source="activation_dynamic"),
        epilogue=EpilogueSpec(output_dtype=out))


def test_w8a8_executor_validates_before_touching_the_gpu():
    from xqt_b200.executors import b200_w8a8_executor

    w = torch.zeros((8, 64), dtype=torch.int8)
    ws = torch.ones(8)
    x = torch.zeros((4, 64), dtype=torch.bfloat16)
    with pytest.raises(XQTBackendError, match="CUDA"):
        b200_w8a8_executor(x, w, spec=_w8a8_spec(), weight_scales=ws)
    with pytest.raises(XQTBackendError, match="int8 \\[N, K\\]"):
        b200_w8a8_executor(x, w.to(torch.float32), spec=_w8a8_spec(), weight_scales=ws)
    with pytest.raises(XQTBackendError, match="weight_scales"):
        b200_w8a8_executor(x, w, spec=_w8a8_spec())
    with pytest.raises(XQTBackendError, match="zero points"):
        b200_w8a8_executor(x, w, spec=_w8a8_spec(), weight_scales=ws, weight_zero_points=torch.zeros(8))
    with pytest.raises(XQTBackendError, match="bias only"):
        b200_w8a8_executor(x, w, spec=_w8a8_spec(), weight_scales=ws, residual=torch.zeros((4, 8)))


def test_svd_contract_and_executor_reject_what_they_cannot_serve():
    from xqt_b200.executors import SVDGemmContract, b200_svd_w4a4_executor

    spec = _spec()
    with pytest.raises(ValueError):
        SVDGemmContract(main_spec=spec, rank=0)
    with pytest.raises(ValueError):
        SVDGemmContract(main_spec=spec, rank=4, fusion_boundary="somewhere")
    with pytest.raises(ValueError):
        SVDGemmContract(main_spec=spec, rank=4, outlier_channels=(1, 1))
    contract = SVDGemmContract(main_spec=spec, rank=4, fusion_boundary="fuse_up")
    assert contract.to_dict()["fusion_boundary"] == "fuse_up" and contract.to_dict()["rank"] == 4
    pw = quantize.quantize_w4_asymmetric(torch.randn((8, 256), generator=seeded(1)), group_size=128)
    x = torch.zeros((4, 256), dtype=torch.bfloat16)
    with pytest.raises(XQTBackendError, match="low_rank_down"):
        b200_svd_w4a4_executor(x, pw, spec=spec)                       # a plain W4A16 request: next candidate
    with pytest.raises(XQTBackendError, match="symmetric signed residual"):
        b200_svd_w4a4_executor(x, pw, spec=spec, low_rank_down=torch.zeros((4, 256)), low_rank_up=torch.zeros((8, 4)))


def test_reference_named_ops_resolve_through_the_kernel_namespace():
    from xqt_b200 import kernel_spec
    from xqt_b200.ops import awq, w4a4, w8a8

    platform = kernel_spec.PlatformInfo("cuda", 10, 0)
    assert kernel_spec.select_kernel("quantization.awq_w4a16_decode", platform=platform).load() is awq.awq_w4a16_decode
    assert kernel_spec.select_kernel("quantization.convrot_w8a8_linear", platform=platform).load() is w8a8.convrot_w8a8_linear
    assert kernel_spec.select_kernel("quantization.svdq_w4a4_linear", platform=platform).load() is w4a4.svdq_w4a4_linear
    assert not kernel_spec.select_kernel("quantization.awq_w4a16_decode", platform=platform).is_available(
        kernel_spec.PlatformInfo("cuda", 8, 9))
    # argument names and order of xqt's ops (awq_w4a16_sm89.py:152-302, convrot_w8a8_sm89.py:365-448,
    # svdq_w4a4_sm89.py:471-479,963-969,1203-1270)
    import inspect

    assert list(inspect.signature(awq.awq_w4a16_decode).parameters) == ["inputs", "qweight", "scales", "scaled_zeros", "output"]
    assert list(inspect.signature(awq.bind_awq_w4a16_decode).parameters) == [
        "qweight", "scales", "scaled_zeros", "rows", "input_features", "output_features", "dtype", "device", "bias"]
    assert list(inspect.signature(w8a8.convrot_w8a8_linear).parameters)[:5] == [
        "inputs", "packed", "rotated_input_features", "rot_size", "workspace"]
    assert list(inspect.signature(w8a8.bind_convrot_w8a8_linear).parameters)[:5] == [
        "packed", "workspace", "rows", "rotated_input_features", "rot_size"]
    assert list(inspect.signature(w4a4.pack_svdq_w4a4_linear).parameters)[:6] == [
        "residual_weight", "down_weight", "up_weight", "bias", "smooth", "norm_weight"]
    assert list(inspect.signature(w4a4.allocate_w4a4_workspace).parameters) == ["rows", "packed", "with_lora_rank", "with_row_scales"]
    assert list(inspect.signature(w4a4.bind_svdq_w4a4_linear).parameters)[:4] == ["packed", "workspace", "rows", "lora_scale"]
    with pytest.raises(XQTBackendError):
        w4a4.pack_svdq_w4a4_linear(torch.zeros((8, 128)), None, None, smooth=torch.ones(128))


def test_install_into_the_reference_registry_and_dispatch_with_its_own_dispatcher():
    """With an xqt checkout importable (``XQT_REFERENCE_PATH`` or an installed package): the B200 rows go
    into xqt's own default registry as xqt's own row class, and xqt's ``dispatch_gemm`` reaches a (fake)
    executor swapped into the B200 row when asked for ``GemmProblem(sm=100)``."""

    import os
    import sys

    path = os.environ.get("XQT_REFERENCE_PATH")
    if path and path not in sys.path:
        sys.path.insert(0, path)
    xreg = pytest.importorskip("xqt.kernels.ops.gemm.registry")
    from xqt.kernels.ops.gemm import contracts as xc
    from xqt.kernels.ops.gemm import dispatch as xd
    from xqt.kernels.ops.gemm import layout as xl

    from xqt_b200.executors import install_b200_executors

    registry = xreg.default_registry()
    promoted = install_b200_executors(registry, require_native=False) or ()
    from xqt_b200 import native

    if not native.available():
        pytest.skip("the shared library is not built here")
    assert B200_W4A16 in promoted
    row = registry.get(B200_W4A16)
    assert type(row) is xreg.GemmKernelRegistration and row.executable
    calls = []

    def fake(activation, weight, *, spec, **kwargs):
        calls.append((type(weight).__module__, spec.problem.arch))
        return torch.full((spec.problem.m, spec.problem.n), 3.0, dtype=torch.bfloat16)

    registry.replace(replace(row, executor=fake))
    try:
        codes = torch.randint(0, 16, (8, 256), generator=seeded(2), dtype=torch.int64).to(torch.uint8)
        quant = xc.QuantSpec(weight_dtype="int4", activation_dtype="bf16", output_dtype="bf16", weight_granularity="groupwise",
                             group_size=128, symmetric=False, weight_zero_point=True, weight_scale_source="weight_offline",
                             storage_layout="xqt_int4_nk_v1")
        weight = xl.build_packed_weight(xl.pack_int4_unsigned(codes), logical_shape=(8, 256), spec=quant,
                                        scales=torch.ones((8, 2)), zero_points=torch.full((8, 2), 8.0), padded_k=256)
        spec = xc.GemmSpec(problem=xc.GemmProblem(m=4, n=8, k=256, sm=100), quant=quant,
                           epilogue=xc.EpilogueSpec(output_dtype="bf16"))
        result = xd.dispatch_gemm(torch.zeros((4, 256), dtype=torch.bfloat16), weight, spec=spec, registry=registry)
        assert result.report.selected_kernel == B200_W4A16 and float(result.output[0, 0]) == 3.0
        assert calls == [("xqt.kernels.ops.gemm.contracts", "sm_100")]
    finally:
        registry.replace(row)
