"""SVDQuant / ConvRot W4A4 on the GPU against the CPU oracle: rotated activation, integer codes
and scales bit-exact; output rel-L2 <= 1e-3 against fp32((q_a s_a) @ (q_w s_w)^T + (x_rot L1^T) L2^T + b)."""

from __future__ import annotations

import pytest
import torch

from conftest import seeded
from oracle import rotation as orot
from oracle import w4a16 as o16
from oracle import w4a4 as oracle
from xqt_b200 import native, quantize
from xqt_b200.ops.activation import rotate_quantize
from xqt_b200.ops.w4a4 import convrot_w4a4_linear, pack_svdq_w4a4_linear, svdq_w4a4_linear

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _layer(n, k, rank, seed, rot):
    w = torch.randn((n, k), generator=seeded(seed)) * 0.02
    w_rot = rot.apply(w) if rot is not None else w
    if rank:
        down, up, residual = oracle.svd_split(w_rot, rank)
        down, up = down.to(torch.bfloat16), up.to(torch.bfloat16)
    else:
        down, up, residual = None, None, w_rot
    packed, scale = oracle.quantize_residual(residual, group_size=64)
    return packed, scale, down, up


def _outliers(x, seed):
    k = x.shape[1]
    idx = torch.randperm(k, generator=seeded(seed))[: max(1, k // 100)]
    x = x.clone()
    x[:, idx] *= 20.0
    return x


@pytest.mark.parametrize("kind,block", [("sylvester", 128), ("regular", 256), ("regular", 64), (None, 0)])
def test_group_int4_codes_bit_exact(kind, block):
    m, k = 45, 1024
    x = _outliers(torch.randn((m, k), generator=seeded(3)), 4).to(torch.bfloat16)
    rot = None if kind is None else quantize.Rotation(kind, block, orot.random_signs(block, 5) if kind == "sylvester" else None)
    x_rot = x if rot is None else orot.rotate_fht(x, kind=kind, block=block, signs=rot.signs)
    q_ref, s_ref = oracle.quantize_act_groups(x_rot, group_size=64)
    codes, scales, rotated = rotate_quantize(x.to(DEV), rot, bits=4, group_size=64, return_rotated=True)
    torch.cuda.synchronize()
    assert torch.equal(rotated.cpu(), x_rot)
    assert torch.equal(scales.cpu(), s_ref)
    assert torch.equal(codes.cpu(), q_ref)


@pytest.mark.parametrize("form", ["integer", "dense"])
@pytest.mark.parametrize("m,n,k,rank", [(128, 128, 128, 32), (200, 264, 512, 16), (33, 136, 256, 4), (512, 1024, 3072, 32),
                                        (1, 128, 128, 32)])
def test_svdq_forward(m, n, k, rank, form):
    rot = quantize.randomized_rotation(128, seed=7)
    x = _outliers(torch.randn((m, k), generator=seeded(m)), 9).to(torch.bfloat16)
    packed_w, scale, down, up = _layer(n, k, rank, 100 + n, rot)
    bias = torch.randn((n,), generator=seeded(2))
    layer = pack_svdq_w4a4_linear(None, down.to(DEV), up.to(DEV), bias.to(DEV), packed_residual=packed_w.to(DEV),
                                  residual_scale=scale.to(DEV), rotation=rot)
    out, parts = svdq_w4a4_linear(x.to(DEV), layer, return_parts=True, form=form)
    torch.cuda.synchronize()
    assert native.workspace_status(DEV) == 0
    ref, rparts = oracle.w4a4_forward(x, packed_w, scale, down, up, group_size=64, rot_kind=rot.kind, rot_block=128,
                                      signs=rot.signs, bias=bias, return_parts=True)
    assert torch.equal(parts["codes"].cpu(), rparts["q_a"])
    assert torch.equal(parts["scales"].cpu(), rparts["s_a"])
    assert o16.rel_l2(parts["la"].cpu()[:, :rank], rparts["low"]) <= 1e-5
    assert not parts["la"].cpu()[:, rank:].any()
    assert o16.rel_l2(out.cpu(), ref) <= 1e-3


def test_convrot_w4a4_without_low_rank_and_fp16():
    m, n, k = 96, 256, 512
    rot = quantize.regular_rotation(256)
    x = torch.randn((m, k), generator=seeded(1)).to(torch.float16)
    packed_w, scale, _, _ = _layer(n, k, 0, 55, rot)
    layer = pack_svdq_w4a4_linear(None, None, None, None, packed_residual=packed_w.to(DEV), residual_scale=scale.to(DEV),
                                  rotation=rot, dtype=torch.float16)
    out = convrot_w4a4_linear(x.to(DEV), layer, rot_size=256)
    zeros_d, zeros_u = torch.zeros((1, k)), torch.zeros((n, 1))
    ref = oracle.w4a4_forward(x, packed_w, scale, zeros_d, zeros_u, group_size=64, rot_kind="regular", rot_block=256)
    assert o16.rel_l2(out.cpu(), ref) <= 1e-3


def test_operand_cache_gives_the_same_bits():
    """Weights held in operand form (one byte each) by the layer: same output as widening them on every call."""

    from xqt_b200.ops.w4a4 import bind_svdq_w4a4_linear, with_operand_cache
    m, n, k, rank = 200, 384, 1024, 16
    rot = quantize.randomized_rotation(128, seed=6)
    x = _outliers(torch.randn((m, k), generator=seeded(3)), 5).to(torch.bfloat16).to(DEV)
    packed_w, scale, down, up = _layer(n, k, rank, 31, rot)
    layer = pack_svdq_w4a4_linear(None, down.to(DEV), up.to(DEV), None, packed_residual=packed_w.to(DEV),
                                  residual_scale=scale.to(DEV), rotation=rot)
    plain = svdq_w4a4_linear(x, layer)
    cached = with_operand_cache(layer)
    assert cached.weight_bytes.shape == (n, k) and layer.weight_bytes is None
    assert torch.equal(svdq_w4a4_linear(x, cached), plain)
    assert torch.equal(bind_svdq_w4a4_linear(layer, rows=m, operand_cache=True)(x), plain)
    assert native.workspace_status(DEV) == 0


def test_dense_form_is_opt_in_and_close_to_the_integer_form():
    m, n, k, rank = 300, 264, 512, 8
    assert native.library().xqt_b200_w4a4_dense_preferred(m, n, k) == 1      # faster here, but never chosen silently
    assert native.library().xqt_b200_w4a4_dense_preferred(255, n, k) == 0
    rot = quantize.randomized_rotation(128, seed=5)
    x = _outliers(torch.randn((m, k), generator=seeded(12)), 4).to(torch.bfloat16)
    packed_w, scale, down, up = _layer(n, k, rank, 77, rot)
    layer = pack_svdq_w4a4_linear(None, down.to(DEV), up.to(DEV), None, packed_residual=packed_w.to(DEV),
                                  residual_scale=scale.to(DEV), rotation=rot)
    auto = svdq_w4a4_linear(x.to(DEV), layer)
    dense = svdq_w4a4_linear(x.to(DEV), layer, form="dense")
    integer = svdq_w4a4_linear(x.to(DEV), layer, form="integer")
    torch.cuda.synchronize()
    assert native.workspace_status(DEV) == 0
    assert torch.equal(auto, integer)
    # each form is within 1e-3 of the reference (test_svdq_forward); against each other two bf16 roundings add up
    assert o16.rel_l2(dense.cpu(), integer.cpu()) <= 2e-3


@pytest.mark.parametrize("factors", ["svd", "random"])
def test_config3_full_size(factors):
    # x [4096,3072] with 1% outlier channels x20, randomized block-Hadamard 128, W [12288,3072], rank 32
    m, n, k, rank = 4096, 12288, 3072, 32
    rot = quantize.randomized_rotation(128, seed=3)
    x = _outliers(torch.randn((m, k), generator=seeded(3)), 33).to(torch.bfloat16)
    w = torch.randn((n, k), generator=seeded(4)) * 0.02
    w_rot = rot.apply(w)
    if factors == "svd":
        # as the configuration states: rank-32 factors from a truncated SVD of W (the package's own
        # svd_split, run on the GPU to keep the test short), residual = W - up @ down in fp32
        down32, up32, residual = (t.cpu() for t in quantize.svd_split(w_rot.to(DEV), rank))
        down, up = down32.to(torch.bfloat16), up32.to(torch.bfloat16)
    else:
        # a seeded random rank-32 pair: larger low-rank term than a Gaussian matrix's SVD gives
        down = (torch.randn((rank, k), generator=seeded(5)) * 0.05).to(torch.bfloat16)
        up = (torch.randn((n, rank), generator=seeded(6)) * 0.05).to(torch.bfloat16)
        residual = w_rot - up.float() @ down.float()
    packed_w, scale = oracle.quantize_residual(residual, group_size=64)
    packed_p, scale_p, _ = quantize.quantize_residual_int4(residual, group_size=64)
    assert torch.equal(packed_p, packed_w) and torch.equal(scale_p, scale)      # product quantiser == oracle's
    layer = pack_svdq_w4a4_linear(None, down.to(DEV), up.to(DEV), None, packed_residual=packed_w.to(DEV),
                                  residual_scale=scale.to(DEV), rotation=rot)
    out = svdq_w4a4_linear(x.to(DEV), layer)
    torch.cuda.synchronize()
    assert native.workspace_status(DEV) == 0
    torch.set_num_threads(16)
    ref = oracle.w4a4_forward_dequant(x, packed_w, scale, down, up, group_size=64, rot_kind=rot.kind, rot_block=128,
                                      signs=rot.signs)
    assert o16.rel_l2(out.cpu(), ref) <= 1e-3
    # the opt-in dense form: fp16 rounding of both operands, measured 1.2e-3 at this K
    dense = svdq_w4a4_linear(x.to(DEV), layer, form="dense")
    torch.cuda.synchronize()
    assert native.workspace_status(DEV) == 0
    assert o16.rel_l2(dense.cpu(), ref) <= 1.5e-3
