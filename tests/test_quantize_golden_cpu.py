"""The package's own offline functions (quantisers, SVD split, rotations) against vectors produced by
running the reference's functions (tests/golden/make_golden.py).  The oracle's twins are pinned in
test_oracle_golden.py; these are the functions a user of the package actually calls."""

from __future__ import annotations

import torch

from xqt_b200 import quantize
from xqt_b200.layout import unpack_int4


def test_symmetric_w4_quantiser_matches_the_reference_quantiser(golden):
    # reference: AWQGPTQWeightOnlyLinear's _quantize_grouped_weight (xqt/contracts/weight_only.py:40-71)
    g = golden("quantizers")
    for tag, group in (("1", 64), ("2", 128)):
        w = g[f"wo_w{tag}"]
        pw = quantize.quantize_w4_symmetric(w, group_size=group)
        assert pw.metadata.padded_k == int(g[f"wo_padded{tag}"])
        assert torch.equal(pw.qweight, g[f"wo_packed{tag}"])
        assert torch.equal(pw.scales, g[f"wo_scale{tag}"].squeeze(-1))
        assert pw.zero_points is None and pw.metadata.nibble_signed
    assert float(g["wo_scale2"][3, 1, 0]) == 1.0          # the all-zero group keeps scale 1


def test_svd_split_and_residual_quantiser_match_the_reference(golden):
    # reference: decompose_weight_svd (xqt/analysis/svd_analysis.py:46-120), _quantize_residual_int4
    # (xqt/compression/quant/quantizers/svd.py:92-128)
    g = golden("svd_w4a4")
    down, up, residual = quantize.svd_split(g["w"], 4)
    assert tuple(down.shape) == tuple(g["down"].shape) and tuple(up.shape) == tuple(g["up"].shape)
    # singular vectors are defined up to a sign per component: compare what the layer uses, the product
    torch.testing.assert_close(up @ down, g["up"] @ g["down"], atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(residual, g["residual"], atol=1e-5, rtol=1e-4)
    packed, scale, padded = quantize.quantize_residual_int4(g["residual"], group_size=64)
    assert padded == 128
    assert torch.equal(packed, g["packed"])
    assert torch.equal(scale, g["scale"])


def test_rotation_matrices_match_the_reference_builders(golden):
    # reference: build_regular_hadamard_matrix / _apply_groupwise_rotation (convrot_4bit.py:85-229),
    # build_quarot_rotation (xqt/model/minicpm5_quarot.py:54-93)
    g = golden("w8a8_rotation")
    h16 = quantize.regular_rotation(16).matrix()
    ref16 = g["rot_h16"]
    scale = 1.0 if float(ref16.abs().max()) < 0.5 else 4.0      # the builder returns the +-1 matrix or the normalised one
    torch.testing.assert_close(h16 * scale, ref16, atol=1e-7, rtol=0)
    torch.testing.assert_close(quantize.regular_rotation(256).matrix().sum(dim=1) * (16.0 if scale == 4.0 else 1.0),
                               g["rot_h256_rowsum"], atol=1e-5, rtol=0)
    torch.testing.assert_close(quantize.randomized_rotation(128, 7).matrix(), g["rot_quarot128_seed7"], atol=1e-7, rtol=0)
    torch.testing.assert_close(quantize.randomized_rotation(64, 9).matrix(), g["rot_quarot64_seed9"], atol=1e-7, rtol=0)
    torch.set_num_threads(1)
    torch.testing.assert_close(quantize.regular_rotation(256).apply(g["rot_x"]), g["rot_x_rot256"], atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(quantize.regular_rotation(16).apply(g["rot_x"]), g["rot_x_rot16"], atol=1e-6, rtol=1e-6)


def test_int8_per_channel_quantiser_matches_the_artifact(golden):
    # reference: ConvRotInt8Linear.from_linear / _quantize_int8_per_row (convrot_int8.py:361-400,1528-1556)
    g = golden("w8a8_rotation")
    torch.set_num_threads(1)
    w_rot = quantize.regular_rotation(256).apply(g["rot_w"])
    q, s = quantize.quantize_w8_per_channel(w_rot)
    assert torch.equal(q, g["rot_w_q8"])
    assert torch.equal(s, g["rot_w_s8"].reshape(-1))
    assert torch.equal(q.t().contiguous(), g["rot_artifact_qweight_t"])
    assert torch.equal(s, g["rot_artifact_scale"].reshape(-1))


def test_convrot_w4a4_artifact_weight_and_per_token_activation(golden):
    # reference: ConvRotMixedPrecisionLinear.from_linear (rotate, signed int4 per group) and its per-token
    # activation fake-quantisation (convrot_4bit.py:418-520,669-679)
    from oracle import w4a4 as oracle_w4a4

    g = golden("quantizers")
    torch.set_num_threads(1)
    w_rot = quantize.regular_rotation(16).apply(g["convrot4_w"])
    pw = quantize.quantize_w4_symmetric(w_rot, group_size=64)
    ref_codes = unpack_int4(g["convrot4_packed_weight"], logical_k=128, signed=True)
    assert torch.equal(unpack_int4(pw.qweight, logical_k=128, signed=True), ref_codes)
    torch.testing.assert_close(pw.scales, g["convrot4_weight_scale"].reshape(pw.scales.shape).float(), atol=0, rtol=0)
    x_rot = quantize.regular_rotation(16).apply(g["convrot4_x"])
    torch.testing.assert_close(x_rot, g["convrot4_x_rot16"], atol=1e-6, rtol=1e-6)
    codes, scale = oracle_w4a4.quantize_act_groups(g["convrot4_x_rot16"], group_size=128)     # one group = per token
    assert torch.equal(scale.reshape(-1, 1), g["convrot4_act_scale"])
    assert torch.equal(codes.float() * scale.reshape(-1, 1), g["convrot4_act_fake_quant"])
