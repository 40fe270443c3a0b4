"""The CPU oracle against vectors produced by the reference itself (tests/golden/make_golden.py)
and against the literal known-answer cases of the reference's own unit tests."""

from __future__ import annotations

import pytest
import torch

from oracle import rotation, w4a16, w4a4, w8a8


def test_pack_unpack_bit_exact(golden):
    g = golden("pack")
    assert torch.equal(w4a16.pack_nibbles(g["codes_u"], signed=False), g["packed_u"])
    assert torch.equal(w4a16.pack_nibbles(g["codes_s"], signed=True), g["packed_s"])
    assert torch.equal(w4a16.unpack_nibbles(g["packed_u"], 37, signed=False), g["unpacked_u"].float())
    assert torch.equal(w4a16.unpack_nibbles(g["packed_s"], 40, signed=True), g["unpacked_s"].float())


def test_literal_signed_group_scale_case():
    # tests/gemm/test_reference.py:53-78 of the reference
    values = torch.tensor([[-8, -4, 0, 4, 7], [7, 3, -1, -5, -8]], dtype=torch.int8)
    packed = w4a16.pack_nibbles(values, signed=True)
    scales = torch.tensor([[0.5, 1.0, 2.0], [1.0, 0.5, 0.25]])
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0, 5.0]])
    out = w4a16.gemm(x, packed, scales, None, group_size=2, signed=True, k=5, out_dtype=torch.float32)
    decoded = values.float() * torch.tensor([[0.5, 0.5, 1.0, 1.0, 2.0], [1.0, 1.0, 0.5, 0.5, 0.25]])
    torch.testing.assert_close(out, x @ decoded.t())


def test_literal_unsigned_zero_point_case():
    # tests/gemm/test_reference.py:81-105 of the reference: expected value 13
    packed = w4a16.pack_nibbles(torch.tensor([[0, 4, 8, 15]]), signed=False)
    out = w4a16.gemm(torch.ones(1, 4), packed, torch.ones(1, 2), torch.tensor([[1.0, 7.0]]),
                     group_size=2, signed=False, out_dtype=torch.float32)
    assert out.item() == pytest.approx((0 - 1) + (4 - 1) + (8 - 7) + (15 - 7))


@pytest.mark.parametrize("case", ["u4_g128_bf16", "u4_g64_fp16_bias", "s4_g32_bf16", "s4_g128_padk"])
def test_w4a16_matches_reference(golden, case):
    g = golden("w4a16")[case]
    group, signed, k, padded_k = int(g["group"]), bool(g["signed"]), int(g["k"]), int(g["padded_k"])
    deq = w4a16.dequantize(g["qweight"], g["scales"], g["zeros"], k=k, padded_k=padded_k,
                           group_size=group, signed=signed)
    assert torch.equal(deq, g["dequant"])          # dequantised values bit-exact
    torch.set_num_threads(1)
    out = w4a16.gemm(g["x"], g["qweight"], g["scales"], g["zeros"], group_size=group, signed=signed,
                     k=k, bias=g["bias"])
    assert out.dtype == g["out"].dtype
    assert w4a16.rel_l2(out, g["out"]) < 1e-6


def test_hadamard_literals(golden):
    g = golden("w8a8_rotation")
    h4 = rotation.regular_hadamard(4)
    # tests/quant/test_convrot_4bit_quantizer.py:29-41 of the reference
    assert torch.equal(h4, torch.tensor([[1, 1, 1, -1], [1, 1, -1, 1], [1, -1, 1, 1], [-1, 1, 1, 1]]).float())
    assert torch.equal(rotation.regular_hadamard(16), g["rot_h16"])
    assert torch.equal(rotation.regular_hadamard(256).sum(dim=1), g["rot_h256_rowsum"])
    r = rotation.rotation_matrix("regular", 256)
    torch.testing.assert_close(r @ r, torch.eye(256), atol=1e-5, rtol=0)       # self-inverse
    assert torch.equal(r, r.t())                                                # symmetric


def test_randomized_hadamard_matches_quarot(golden):
    g = golden("w8a8_rotation")
    for order, seed, key in ((128, 7, "rot_quarot128_seed7"), (64, 9, "rot_quarot64_seed9")):
        kind = "regular" if rotation.is_power_of(order, 4) else "sylvester"
        mine = rotation.rotation_matrix(kind, order, rotation.random_signs(order, seed))
        torch.testing.assert_close(mine, g[key], atol=1e-7, rtol=0)


def test_rotation_fht_equals_reference_matmul(golden):
    g = golden("w8a8_rotation")
    x = g["rot_x"]
    for block, key in ((256, "rot_x_rot256"), (16, "rot_x_rot16")):
        mat = rotation.rotate_matmul(x, rotation.rotation_matrix("regular", block))
        torch.testing.assert_close(mat, g[key], atol=1e-6, rtol=1e-6)
        fht = rotation.rotate_fht(x, kind="regular", block=block)
        torch.testing.assert_close(fht, g[key], atol=2e-6, rtol=1e-5)
    # bf16 activation: the fht result rounded once must agree with the reference's bf16 matmul
    # except for isolated one-ulp rounding flips
    fht16 = rotation.rotate_fht(x.to(torch.bfloat16), kind="regular", block=256)
    ref16 = g["rot_x_bf16_rot256"]
    assert fht16.dtype == torch.bfloat16
    mismatch = (fht16 != ref16).float().mean().item()
    assert mismatch < 0.02
    torch.testing.assert_close(fht16.float(), ref16.float(), atol=0.04, rtol=0.01)
    # sylvester family: fht == matmul with the matrix
    signs = rotation.random_signs(128, 11)
    xs = x[:, :384]
    torch.testing.assert_close(
        rotation.rotate_fht(xs, kind="sylvester", block=128, signs=signs),
        rotation.rotate_matmul(xs, rotation.rotation_matrix("sylvester", 128, signs)), atol=2e-6, rtol=1e-5)


def test_int8_activation_and_contract_gemm(golden):
    g = golden("w8a8_rotation")
    q, s = w8a8.quantize_act_per_token(g["act"])
    assert torch.equal(q, g["q"])
    assert torch.equal(s, g["scale"])
    torch.set_num_threads(1)
    ref = w8a8.gemm_reference(q, s, g["qw"], g["ws"])
    assert w4a16.rel_l2(ref, g["out"]) < 1e-6
    integer = w8a8.gemm_integer(q, s, g["qw"], g["ws"])
    assert w4a16.rel_l2(integer, g["out"]) < 2e-3      # both rounded to bf16; differ by isolated ulps
    assert w4a16.rel_l2(w8a8.gemm_integer(q, s, g["qw"], g["ws"], out_dtype=torch.float32),
                        w8a8.gemm_reference(q, s, g["qw"], g["ws"], out_dtype=torch.float32)) < 1e-6


def test_int8_weight_quantiser_matches_artifact(golden):
    g = golden("w8a8_rotation")
    w_rot = rotation.rotate_matmul(g["rot_w"], rotation.rotation_matrix("regular", 256))
    q, s = w8a8.quantize_weight_per_channel(w_rot)
    assert torch.equal(q, g["rot_w_q8"])
    assert torch.equal(s, g["rot_w_s8"])
    assert torch.equal(q.t().contiguous(), g["rot_artifact_qweight_t"])
    assert torch.equal(s, g["rot_artifact_scale"])


def test_svd_residual_and_composite_forward(golden):
    g = golden("svd_w4a4")
    packed, scale = w4a4.quantize_residual(g["residual"], group_size=64)
    assert torch.equal(packed, g["packed"])
    assert torch.equal(scale, g["scale"])
    assert torch.equal(w4a4.dequantize_residual(packed, scale, group_size=64), g["dequant"])
    down, up, residual = w4a4.svd_split(g["w"], 4)
    # singular vectors are defined up to sign: compare the products
    torch.testing.assert_close(up @ down, g["up"] @ g["down"], atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(residual, g["residual"], atol=1e-5, rtol=1e-4)
    torch.set_num_threads(1)
    out = w4a4.composite_forward(g["x"], packed, scale, g["down"], g["up"], group_size=64, bias=g["bias"])
    torch.testing.assert_close(out, g["out_fp32"], atol=1e-6, rtol=1e-6)


def test_group_activation_quant_reduces_to_reference_per_token_formula(golden):
    g = golden("svd_w4a4")
    codes, scale = w4a4.quantize_act_groups(g["x"], group_size=g["x"].shape[1])
    assert torch.equal(scale, g["act_scale_per_token"])
    assert torch.equal(codes.float(), g["act_codes_per_token"])
    # the artifact's own fake-quantised activation (ConvRotMixedPrecisionLinear._quantize_rotated_activation)
    assert torch.equal(codes.float() * scale, g["act_fake_quant_per_token"])


def test_w4a4_two_forms_agree(golden):
    g = golden("svd_w4a4")
    x = g["x"].to(torch.bfloat16)
    signs = rotation.random_signs(128, 3)
    kw = dict(group_size=64, rot_kind="sylvester", rot_block=128, signs=signs, bias=g["bias"])
    a = w4a4.w4a4_forward(x, g["packed"], g["scale"], g["down"], g["up"], **kw)
    b = w4a4.w4a4_forward_dequant(x, g["packed"], g["scale"], g["down"], g["up"], **kw)
    assert w4a16.rel_l2(a, b) < 2e-3
    # with activations left unquantised the W4A4 oracle degenerates to the composite artifact forward
    ref = w4a4.composite_forward(x.float(), g["packed"], g["scale"], g["down"], g["up"], group_size=64,
                                 bias=g["bias"])
    no_rot = w4a4.w4a4_forward(x, g["packed"], g["scale"], g["down"], g["up"], group_size=64,
                               rot_kind=None, bias=g["bias"])
    assert w4a16.rel_l2(no_rot, ref) < 0.25     # int4 activation noise only
