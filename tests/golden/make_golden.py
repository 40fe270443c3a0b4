"""Regenerate the golden vectors by running the reference itself on seeded inputs.

Run where the reference checkout is importable (it needs nothing but torch; the
quantiser modules also import ``omegaconf``, for which a minimal stand-in is
installed below when the real package is absent):

    python tests/golden/make_golden.py --reference /path/to/xqt-checkout

Outputs ``tests/golden/*.pt`` (torch.save of small tensors).  The tests only read
those files; they never import the reference.
"""

from __future__ import annotations

import argparse
import importlib.util
import pathlib
import sys
import types

import torch

HERE = pathlib.Path(__file__).resolve().parent


def _install_omegaconf_stub() -> None:
    try:
        import omegaconf  # noqa: F401
        return
    except Exception:  # noqa: BLE001
        pass
    module = types.ModuleType("omegaconf")

    class OmegaConf:  # the quantiser modules only touch resolver registration at import
        @staticmethod
        def has_resolver(name):
            return True

        @staticmethod
        def register_new_resolver(*args, **kwargs):
            return None

    class _Any:
        def __getattr__(self, name):
            return _Any()

        def __call__(self, *args, **kwargs):
            return _Any()

    module.OmegaConf = OmegaConf
    module.MISSING = "???"
    module.DictConfig = dict
    module.ListConfig = list
    def _module_getattr(name):
        if name.startswith("__"):          # inspect / importlib probe dunder attributes of every module
            raise AttributeError(name)
        return _Any()

    module.__getattr__ = _module_getattr
    errors = types.ModuleType("omegaconf.errors")
    errors.OmegaConfBaseException = Exception
    module.errors = errors
    sys.modules["omegaconf"] = module
    sys.modules["omegaconf.errors"] = errors


def gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(seed)


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True)
    args = parser.parse_args()
    sys.path.insert(0, args.reference)
    _install_omegaconf_stub()
    torch.set_num_threads(1)  # fixed summation order for the stored matmul outputs

    from xqt.kernels.ops.gemm import contracts as C
    from xqt.kernels.ops.gemm import layout as L
    from xqt.kernels.ops.gemm import quantize as Q
    from xqt.kernels.ops.gemm import reference as R
    from xqt.contracts import weight_only as WO

    # ------------------------------------------------------------------ packing
    codes_u = torch.randint(0, 16, (6, 37), generator=gen(1), dtype=torch.int64)
    codes_s = torch.randint(-8, 8, (5, 40), generator=gen(2), dtype=torch.int64)
    words = torch.randint(-(2**31), 2**31 - 1, (24, 4), generator=gen(3), dtype=torch.int64).to(torch.int32)
    awq = L.repack_awq_int4(
        words[:, :], logical_shape=(32, 24), scales=torch.rand((1, 32), generator=gen(4)) + 0.5,
        zero_points=torch.randint(0, 16, (1, 32), generator=gen(5)).to(torch.float32), group_size=32,
    )
    gptq_words = torch.randint(-(2**31), 2**31 - 1, (8, 16), generator=gen(6), dtype=torch.int64).to(torch.int32)
    gptq = L.repack_gptq_int4(
        gptq_words, logical_shape=(16, 64), scales=torch.rand((2, 16), generator=gen(7)) + 0.5, group_size=32
    )
    torch.save(
        {
            "codes_u": codes_u, "packed_u": L.pack_int4_unsigned(codes_u),
            "codes_s": codes_s, "packed_s": L.pack_int4_signed(codes_s),
            "unpacked_u": L.unpack_int4(L.pack_int4_unsigned(codes_u), logical_k=37, signed=False),
            "unpacked_s": L.unpack_int4(L.pack_int4_signed(codes_s), logical_k=40, signed=True),
            "awq_words": words, "awq_qweight": awq.qweight, "awq_scales": awq.scales, "awq_zeros": awq.zero_points,
            "awq_padded_k": torch.tensor(awq.metadata.padded_k),
            "gptq_words": gptq_words, "gptq_qweight": gptq.qweight, "gptq_scales": gptq.scales,
        },
        HERE / "pack.pt",
    )

    # ------------------------------------------------------------------ W4A16
    def w4a16_case(seed, m, n, k, group, signed, dtype, param_dtype, with_bias):
        w = torch.randn((n, k), generator=gen(seed)) * 0.02
        x = torch.randn((m, k), generator=gen(seed + 1)).to(dtype)
        padded_k = -(-k // group) * group
        wp = torch.nn.functional.pad(w, (0, padded_k - k))
        grouped = wp.reshape(n, padded_k // group, group)
        if signed:
            # the reference's own symmetric RTN (xqt/contracts/weight_only.py:40-71): packed signed
            # nibbles, fp32 scale [N, G, 1]
            packed, scale, padded_ref = WO._quantize_grouped_weight(
                w, bits=4, group_size=group, input_features=k, output_features=n)
            assert padded_ref == padded_k and param_dtype == torch.float32
            zeros = None
        else:
            lo, hi = grouped.amin(2, keepdim=True), grouped.amax(2, keepdim=True)
            scale = ((hi - lo) / 15.0).to(param_dtype)
            zeros = torch.clamp(torch.round(-lo / scale.float()), 0, 15)
            codes = torch.clamp(torch.round(grouped / scale.float() + zeros), 0, 15).to(torch.uint8).reshape(n, padded_k)
            packed = L.pack_int4_unsigned(codes)
            zeros = zeros.squeeze(-1).to(param_dtype)
        scale = scale.squeeze(-1)
        name = {torch.bfloat16: "bf16", torch.float16: "fp16", torch.float32: "fp32"}[dtype]
        quant = C.QuantSpec(
            weight_dtype="int4", activation_dtype=name, output_dtype=name, weight_granularity="groupwise",
            group_size=group, symmetric=signed, weight_zero_point=not signed,
            weight_scale_source="weight_offline", storage_layout="xqt_int4_nk_v1",
        )
        weight = L.build_packed_weight(packed, logical_shape=(n, k), spec=quant, scales=scale,
                                       zero_points=zeros, padded_k=padded_k)
        bias = torch.randn((n,), generator=gen(seed + 2)) if with_bias else None
        spec = C.GemmSpec(
            problem=C.GemmProblem(m=m, n=n, k=k), quant=quant,
            epilogue=C.EpilogueSpec(output_dtype=name, has_bias=with_bias),
        )
        out = R.reference_w4a16_gemm(x, weight, spec=spec, bias=bias)
        deq = R.dequantize_weight_reference(weight, spec=quant)
        return {"x": x, "qweight": packed, "scales": scale, "zeros": zeros, "bias": bias, "out": out,
                "dequant": deq, "group": torch.tensor(group), "signed": torch.tensor(signed),
                "k": torch.tensor(k), "padded_k": torch.tensor(padded_k)}

    torch.save(
        {
            "u4_g128_bf16": w4a16_case(10, 5, 64, 256, 128, False, torch.bfloat16, torch.bfloat16, False),
            "u4_g64_fp16_bias": w4a16_case(20, 3, 48, 192, 64, False, torch.float16, torch.float32, True),
            "s4_g32_bf16": w4a16_case(30, 16, 40, 96, 32, True, torch.bfloat16, torch.float32, True),
            "s4_g128_padk": w4a16_case(40, 2, 24, 200, 128, True, torch.bfloat16, torch.float32, False),
        },
        HERE / "w4a16.pt",
    )

    # ------------------------------------------------------------------ int8 activations / W8A8 contract
    act = torch.randn((6, 512), generator=gen(50)).to(torch.bfloat16)
    res = Q.quantize_int8_activation(act, granularity="per_token", source="activation_dynamic")
    qw = torch.randint(-127, 128, (20, 512), generator=gen(51), dtype=torch.int64).to(torch.int8)
    ws = torch.rand((20, 1), generator=gen(52)) * 1e-3 + 1e-4
    quant8 = C.QuantSpec(
        weight_dtype="int8", activation_dtype="int8", output_dtype="bf16", weight_granularity="per_channel",
        activation_granularity="per_token", weight_scale_source="weight_offline",
        activation_scale_source="activation_dynamic",
    )
    spec8 = C.GemmSpec(problem=C.GemmProblem(m=6, n=20, k=512), quant=quant8,
                       epilogue=C.EpilogueSpec(output_dtype="bf16"))
    out8 = R.reference_gemm(act, qw, spec=spec8, weight_scales=ws)
    golden8 = {"act": act, "q": res.values, "scale": res.scales, "qw": qw, "ws": ws, "out": out8}

    # ------------------------------------------------------------------ rotations and quantisers
    from xqt.compression.quant.quantizers import convrot_4bit as C4
    from xqt.compression.quant.quantizers import convrot_int8 as C8
    from xqt.compression.quant.quantizers import svd as SV
    from xqt.analysis.svd_analysis import decompose_weight_svd
    from xqt.contracts.composite import CompositeAddLinear

    quarot = importlib.util.spec_from_file_location(
        "_quarot", pathlib.Path(args.reference) / "xqt/model/minicpm5_quarot.py")
    try:
        quarot_mod = importlib.util.module_from_spec(quarot)
        sys.modules["_quarot"] = quarot_mod
        quarot.loader.exec_module(quarot_mod)
        r128 = quarot_mod.build_quarot_rotation(128, seed=7).to(torch.float32)
        r64 = quarot_mod.build_quarot_rotation(64, seed=9).to(torch.float32)
    except Exception as exc:  # noqa: BLE001
        print("quarot module not importable:", exc)
        r128 = r64 = None

    xr = torch.randn((3, 512), generator=gen(60))
    wrot = torch.randn((12, 512), generator=gen(61)) * 0.02
    q8, s8 = C8._quantize_int8_per_row(C4._apply_groupwise_rotation(wrot, rot_size=256, return_padded=True),
                                       eps=1e-6, mse_clip=False, mse_clip_grid=80)
    lin = torch.nn.Linear(512, 12, bias=True)
    with torch.no_grad():
        lin.weight.copy_(wrot)
        lin.bias.copy_(torch.randn((12,), generator=gen(62)))
    art = C8.ConvRotInt8Linear.from_linear(lin, rot_size=256)
    golden_rot = {
        "h16": C4.build_regular_hadamard_matrix(16),
        "h256_rowsum": C4.build_regular_hadamard_matrix(256).sum(dim=1),
        "x": xr,
        "x_rot256": C4._apply_groupwise_rotation(xr, rot_size=256),
        "x_rot16": C4._apply_groupwise_rotation(xr, rot_size=16),
        "x_bf16_rot256": C4._apply_groupwise_rotation(xr.to(torch.bfloat16), rot_size=256),
        "quarot128_seed7": r128,
        "quarot64_seed9": r64,
        "w": wrot, "w_q8": q8, "w_s8": s8,
        "artifact_qweight_t": art.int8_compute.qweight_t, "artifact_scale": art.int8_compute.weight_scale,
    }
    golden8.update({f"rot_{k}": v for k, v in golden_rot.items() if v is not None})
    torch.save(golden8, HERE / "w8a8_rotation.pt")

    # ------------------------------------------------------------------ SVD composite artifact
    wsvd = torch.randn((24, 128), generator=gen(70)) * 0.02
    dec = decompose_weight_svd(wsvd, rank=4)
    down, up = dec.low_rank_components()
    residual = dec.residual_weight(wsvd).to(torch.float32)
    packed, rscale, padded = SV._quantize_residual_int4(residual, group_size=64)
    bias = torch.randn((24,), generator=gen(71))
    module = CompositeAddLinear.from_packed_parts(
        down_weight=down, up_weight=up, packed_residual=packed, residual_scale=rscale, bias=bias,
        input_features=128, output_features=24, group_size=64, padded_input_features=padded, quant_dtype="int4",
    )
    xs = torch.randn((7, 128), generator=gen(72))
    # per-token fake-quant of ConvRot W4A4: the artifact's own methods (convrot_4bit.py:669-679)
    lin4 = torch.nn.Linear(128, 24, bias=False)
    with torch.no_grad():
        lin4.weight.copy_(wsvd)
    art4 = C4.ConvRotMixedPrecisionLinear.from_linear(lin4, rot_size=16, group_size=64)
    a_scale = art4._activation_scale(xs)
    a_fake = art4._quantize_rotated_activation(xs)
    a_codes = torch.round(a_fake / a_scale)
    torch.save(
        {
            "w": wsvd, "down": down, "up": up, "residual": residual, "packed": packed, "scale": rscale,
            "bias": bias, "x": xs, "out_fp32": module(xs),
            "dequant": module.dequantize_residual(),
            "act_scale_per_token": a_scale, "act_codes_per_token": a_codes, "act_fake_quant_per_token": a_fake,
        },
        HERE / "svd_w4a4.pt",
    )

    # ------------------------------------------------------------------ the reference's own quantisers, called
    wq1 = torch.randn((20, 200), generator=gen(80)) * 0.02
    wq2 = torch.randn((16, 256), generator=gen(81)) * 0.02
    wq2[3, 128:] = 0.0                                   # an all-zero group: scale 1
    p1, s1, k1 = WO._quantize_grouped_weight(wq1, bits=4, group_size=64, input_features=200, output_features=20)
    p2, s2, k2 = WO._quantize_grouped_weight(wq2, bits=4, group_size=128, input_features=256, output_features=16)
    xa = torch.randn((5, 128), generator=gen(82))
    rotated = art4._rotate_inputs(xa)
    torch.save(
        {
            "wo_w1": wq1, "wo_packed1": p1, "wo_scale1": s1, "wo_padded1": torch.tensor(k1),
            "wo_w2": wq2, "wo_packed2": p2, "wo_scale2": s2, "wo_padded2": torch.tensor(k2),
            "convrot4_w": wsvd, "convrot4_packed_weight": art4.packed_weight, "convrot4_weight_scale": art4.weight_scale,
            "convrot4_x": xa, "convrot4_x_rot16": rotated,
            "convrot4_act_scale": art4._activation_scale(rotated),
            "convrot4_act_fake_quant": art4._quantize_rotated_activation(rotated),
        },
        HERE / "quantizers.pt",
    )
    # ------------------------------------------------------------------ Int8MmaLinear (per-tensor W8A8)
    from xqt.contracts.int8_mma import Int8MmaLinear

    lin8 = torch.nn.Linear(256, 24, bias=True)
    with torch.no_grad():
        lin8.weight.copy_(torch.randn((24, 256), generator=gen(90)) * 0.02)
        lin8.bias.copy_(torch.randn((24,), generator=gen(91)))
    mod8 = Int8MmaLinear.from_linear(lin8)
    x8 = torch.randn((5, 256), generator=gen(92)).to(torch.bfloat16)
    a_scale8 = Int8MmaLinear.activation_scale_from_inputs(x8, eps=mod8.eps)
    torch.save(
        {
            "x": x8, "qweight_t": mod8.qweight_t, "weight_scale": mod8.weight_scale, "bias": mod8.bias,
            "act_scale": a_scale8, "act_codes": torch.round(x8.to(torch.float32) / a_scale8).clamp(-127, 127).to(torch.int8),
            "out": mod8(x8), "eps": torch.tensor(mod8.eps),
        },
        HERE / "int8_mma.pt",
    )
    for path in sorted(HERE.glob("*.pt")):
        print(path.name, path.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
