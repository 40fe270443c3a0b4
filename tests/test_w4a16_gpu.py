"""W4A16 CUDA kernels against the CPU oracle, through the C ABI.  Bar: rel-L2 <= 1e-3 (bf16/fp16
output, fp32 accumulation); the golden cases additionally compare with the reference's own output."""

from __future__ import annotations

import pytest
import torch

from conftest import seeded
from oracle import w4a16 as oracle
from xqt_b200.ops.w4a16 import select_variant, w4a16_linear
from xqt_b200 import quantize

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _run(case_x, qw, s, z, *, group, signed, k=None, bias=None, residual=None, activation="none", variant="auto"):
    dev = torch.device("cuda", 0)
    mv = lambda t: None if t is None else t.to(dev)
    out = w4a16_linear(mv(case_x), mv(qw), mv(s), mv(z), mv(bias), mv(residual), group_size=group,
                       nibble_signed=signed, k=k, activation=activation, variant=variant)
    torch.cuda.synchronize()
    return out.cpu()


@pytest.mark.parametrize("case", ["u4_g128_bf16", "u4_g64_fp16_bias", "s4_g32_bf16", "s4_g128_padk"])
def test_golden_cases_simt(golden, case):
    g = golden("w4a16")[case]
    out = _run(g["x"], g["qweight"], g["scales"], g["zeros"], group=int(g["group"]), signed=bool(g["signed"]),
               k=int(g["k"]), bias=g["bias"], variant="simt")
    assert out.dtype == g["out"].dtype
    assert oracle.rel_l2(out, g["out"]) <= TOL


def test_golden_case_gemv(golden):
    g = golden("w4a16")["u4_g128_bf16"]
    assert select_variant(5, 64, 256, 256, 128) == "gemv"
    out = _run(g["x"], g["qweight"], g["scales"], g["zeros"], group=128, signed=False, variant="gemv")
    assert oracle.rel_l2(out, g["out"]) <= TOL


def _synthetic(n, k, m, *, seed, dtype=torch.bfloat16, symmetric=False, param_dtype=torch.bfloat16, group=128):
    w = torch.randn((n, k), generator=seeded(seed)) * 0.02
    x = torch.randn((m, k), generator=seeded(seed + 1)).to(dtype)
    if symmetric:
        pw = quantize.quantize_w4_symmetric(w, group_size=group)
    else:
        pw = quantize.quantize_w4_asymmetric(w, group_size=group, param_dtype=param_dtype)
    return x, pw


@pytest.mark.parametrize("m", [1, 4, 8, 16])
@pytest.mark.parametrize("n,k", [(4096, 4096), (1024, 4096), (4096, 14336), (14336, 4096), (200, 512), (64, 128)])
def test_gemv_decode_shapes(m, n, k):
    if (n, k) in {(4096, 14336), (14336, 4096)} and m not in (1, 16):
        pytest.skip("large shapes: first and last M only")
    x, pw = _synthetic(n, k, m, seed=100 + m)
    out = _run(x, pw.qweight, pw.scales, pw.zero_points, group=128, signed=False, variant="gemv")
    ref = oracle.gemm(x, pw.qweight, pw.scales, pw.zero_points, group_size=128, signed=False)
    assert oracle.rel_l2(out, ref) <= TOL
    # split-K is reduced in a fixed order: a second launch is bit-identical
    again = _run(x, pw.qweight, pw.scales, pw.zero_points, group=128, signed=False, variant="gemv")
    assert torch.equal(out, again)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("symmetric", [False, True])
def test_gemv_dtypes_signedness_bias_residual(dtype, symmetric):
    n, k, m = 384, 1024, 7
    x, pw = _synthetic(n, k, m, seed=7, dtype=dtype, symmetric=symmetric, param_dtype=torch.float32)
    bias = torch.randn((n,), generator=seeded(8))
    residual = torch.randn((m, n), generator=seeded(9)).to(dtype)
    out = _run(x, pw.qweight, pw.scales, pw.zero_points, group=128, signed=symmetric, bias=bias,
               residual=residual, variant="gemv")
    ref = oracle.gemm(x, pw.qweight, pw.scales, pw.zero_points, group_size=128, signed=symmetric, bias=bias,
                      residual=residual)
    assert oracle.rel_l2(out, ref) <= TOL


def test_simt_and_gemv_agree_and_config1():
    # configuration 1 of the benchmark: x [16,4096], W [4096,4096], uint4 g128, bf16 scale/zero
    x = torch.randn((16, 4096), generator=seeded(1)).to(torch.bfloat16)
    w = torch.randn((4096, 4096), generator=seeded(2)) * 0.02
    pw = quantize.quantize_w4_asymmetric(w, group_size=128)
    ref = oracle.gemm(x, pw.qweight, pw.scales, pw.zero_points, group_size=128, signed=False)
    fast = _run(x, pw.qweight, pw.scales, pw.zero_points, group=128, signed=False)
    slow = _run(x, pw.qweight, pw.scales, pw.zero_points, group=128, signed=False, variant="simt")
    assert oracle.rel_l2(fast, ref) <= TOL
    assert oracle.rel_l2(slow, ref) <= TOL


@pytest.mark.parametrize("activation", ["relu", "gelu", "silu"])
def test_simt_epilogue_activations(activation):
    x, pw = _synthetic(96, 256, 5, seed=21, group=64)
    bias = torch.randn((96,), generator=seeded(22))
    out = _run(x, pw.qweight, pw.scales, pw.zero_points, group=64, signed=False, bias=bias, activation=activation)
    ref = oracle.gemm(x, pw.qweight, pw.scales, pw.zero_points, group_size=64, signed=False, bias=bias,
                      activation=activation)
    assert oracle.rel_l2(out, ref) <= 2e-3   # bf16 output of a gated value: one extra rounding step


def test_empty_batch_and_bad_arguments():
    from xqt_b200.errors import XQTBackendError
    x, pw = _synthetic(64, 128, 0, seed=3)
    out = _run(x, pw.qweight, pw.scales, pw.zero_points, group=128, signed=False)
    assert tuple(out.shape) == (0, 64)
    x1, _ = _synthetic(64, 256, 2, seed=3)
    with pytest.raises(XQTBackendError):
        _run(x1, pw.qweight, pw.scales, pw.zero_points, group=128, signed=False)       # K mismatch
    with pytest.raises(XQTBackendError):
        _run(x1[:, :128].float(), pw.qweight, pw.scales, pw.zero_points, group=128, signed=False)   # fp32 act


# ---------------------------------------------------------------------------- tiled decode kernel


def _tiled_run(x, pw, *, bias=None, residual=None):
    from xqt_b200 import native, prepack
    from xqt_b200.ops.w4a16 import w4a16_decode_tiled

    dev = torch.device("cuda", 0)
    mv = lambda t: None if t is None else t.to(dev)
    tiled = prepack.tile_w4(mv(pw.qweight), mv(pw.scales), mv(pw.zero_points), group_size=pw.metadata.group_size,
                            nibble_signed=pw.metadata.nibble_signed)
    out = w4a16_decode_tiled(mv(x), tiled, bias=mv(bias), residual=mv(residual))
    torch.cuda.synchronize()
    assert native.workspace_status(dev) == 0
    return out.cpu()


@pytest.mark.parametrize("m", [1, 4, 8, 16])
@pytest.mark.parametrize("n,k", [(4096, 4096), (1024, 4096), (4096, 14336), (14336, 4096), (200, 512), (128, 256),
                                 (72, 768)])
def test_decode_tiled_shapes(m, n, k):
    if (n, k) in {(4096, 14336), (14336, 4096)} and m not in (1, 16):
        pytest.skip("large shapes: first and last M only")
    x, pw = _synthetic(n, k, m, seed=300 + m)
    ref = oracle.gemm(x, pw.qweight, pw.scales, pw.zero_points, group_size=128, signed=False)
    out = _tiled_run(x, pw)
    assert oracle.rel_l2(out, ref) <= TOL
    assert torch.equal(out, _tiled_run(x, pw))          # fixed reduction order: bit-reproducible


@pytest.mark.parametrize("group", [32, 64, 128])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("symmetric", [False, True])
def test_decode_tiled_groups_dtypes_epilogue(group, dtype, symmetric):
    n, k, m = 392, 1280, 13
    x, pw = _synthetic(n, k, m, seed=40 + group, dtype=dtype, symmetric=symmetric, group=group,
                       param_dtype=torch.float32 if group == 64 else torch.bfloat16)
    bias = torch.randn((n,), generator=seeded(8))
    residual = torch.randn((m, n), generator=seeded(9)).to(dtype)
    ref = oracle.gemm(x, pw.qweight, pw.scales, pw.zero_points, group_size=group, signed=symmetric, bias=bias,
                      residual=residual)
    out = _tiled_run(x, pw, bias=bias, residual=residual)
    assert oracle.rel_l2(out, ref) <= TOL


def test_decode_tiled_prepack_round_trip_on_device():
    from xqt_b200 import prepack
    x, pw = _synthetic(200, 512, 1, seed=5)
    dev = torch.device("cuda", 0)
    tiled = prepack.tile_w4(pw.qweight.to(dev), pw.scales.to(dev), pw.zero_points.to(dev), group_size=128,
                            nibble_signed=False)
    q, s, z = prepack.untile_w4(tiled)
    assert torch.equal(q.cpu(), pw.qweight) and torch.equal(s.cpu(), pw.scales) and torch.equal(z.cpu(), pw.zero_points)


# ---------------------------------------------------------------------------- tcgen05 decode kernel


def _tc_run(x, pw, *, bias=None, residual=None):
    from xqt_b200 import native, prepack
    from xqt_b200.ops.w4a16 import w4a16_decode_tiled

    dev = torch.device("cuda", 0)
    mv = lambda t: None if t is None else t.to(dev)
    tiled = prepack.rows_w4(mv(pw.qweight), mv(pw.scales), mv(pw.zero_points), group_size=pw.metadata.group_size,
                            nibble_signed=pw.metadata.nibble_signed)
    assert tiled.layout == "rows128" and tiled.integer_zero_points
    out = w4a16_decode_tiled(mv(x), tiled, bias=mv(bias), residual=mv(residual))
    torch.cuda.synchronize()
    assert native.workspace_status(dev) == 0
    return out.cpu()


@pytest.mark.parametrize("m", [1, 4, 8, 16])
@pytest.mark.parametrize("n,k", [(128, 256), (4096, 4096), (1024, 4096), (4096, 14336), (14336, 4096), (200, 512),
                                 (72, 768)])
def test_decode_tc_shapes(m, n, k):
    if (n, k) in {(4096, 14336), (14336, 4096)} and m not in (1, 16):
        pytest.skip("large shapes: first and last M only")
    x, pw = _synthetic(n, k, m, seed=500 + m)
    ref = oracle.gemm(x, pw.qweight, pw.scales, pw.zero_points, group_size=128, signed=False)
    out = _tc_run(x, pw)
    assert oracle.rel_l2(out, ref) <= TOL
    assert torch.equal(out, _tc_run(x, pw))


@pytest.mark.parametrize("group", [64, 128])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("symmetric", [False, True])
def test_decode_tc_groups_dtypes_epilogue(group, dtype, symmetric):
    n, k, m = 392, 1280, 13
    x, pw = _synthetic(n, k, m, seed=60 + group, dtype=dtype, symmetric=symmetric, group=group,
                       param_dtype=torch.float32 if group == 64 else torch.bfloat16)
    bias = torch.randn((n,), generator=seeded(8))
    residual = torch.randn((m, n), generator=seeded(9)).to(dtype)
    ref = oracle.gemm(x, pw.qweight, pw.scales, pw.zero_points, group_size=group, signed=symmetric, bias=bias,
                      residual=residual)
    out = _tc_run(x, pw, bias=bias, residual=residual)
    assert oracle.rel_l2(out, ref) <= TOL


# ---------------------------------------------------------------------------- cluster split-K decode kernel


def _lanes_run(x, pw, *, bias=None, residual=None, out_dtype=None):
    from xqt_b200 import native, prepack
    from xqt_b200.ops.w4a16 import bind_w4a16_decode

    dev = torch.device("cuda", 0)
    mv = lambda t: None if t is None else t.to(dev)
    tiled = prepack.lanes_w4(mv(pw.qweight), mv(pw.scales), mv(pw.zero_points), group_size=pw.metadata.group_size,
                             nibble_signed=pw.metadata.nibble_signed)
    run = bind_w4a16_decode(tiled, rows=int(x.shape[0]), dtype=x.dtype, bias=mv(bias), out_dtype=out_dtype)
    out = run(mv(x), None, mv(residual))
    torch.cuda.synchronize()
    assert native.workspace_status(dev) == 0
    return out.cpu()


@pytest.mark.parametrize("m", [1, 4, 8, 16])
@pytest.mark.parametrize("n,k", [(128, 128), (128, 256), (4096, 4096), (1024, 4096), (4096, 14336), (14336, 4096),
                                 (200, 512), (72, 768), (512, 1792), (1792, 4096)])
def test_decode_lanes_shapes(m, n, k):
    if (n, k) in {(4096, 14336), (14336, 4096)} and m not in (1, 16):
        pytest.skip("large shapes: first and last M only")
    x, pw = _synthetic(n, k, m, seed=800 + m)
    ref = oracle.gemm(x, pw.qweight, pw.scales, pw.zero_points, group_size=128, signed=False)
    out = _lanes_run(x, pw)
    assert oracle.rel_l2(out, ref) <= TOL
    assert torch.equal(out, _lanes_run(x, pw))          # fixed reduction order: bit-reproducible


@pytest.mark.parametrize("m", [3, 9, 13])
def test_decode_lanes_ragged_m(m):
    x, pw = _synthetic(392, 1280, m, seed=820 + m)
    ref = oracle.gemm(x, pw.qweight, pw.scales, pw.zero_points, group_size=128, signed=False)
    assert oracle.rel_l2(_lanes_run(x, pw), ref) <= TOL


@pytest.mark.parametrize("group", [64, 128])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("symmetric", [False, True])
def test_decode_lanes_groups_dtypes_epilogue(group, dtype, symmetric):
    n, k, m = 392, 1280, 13
    x, pw = _synthetic(n, k, m, seed=60 + group, dtype=dtype, symmetric=symmetric, group=group,
                       param_dtype=torch.float32 if group == 64 else torch.bfloat16)
    bias = torch.randn((n,), generator=seeded(8))
    residual = torch.randn((m, n), generator=seeded(9)).to(dtype)
    ref = oracle.gemm(x, pw.qweight, pw.scales, pw.zero_points, group_size=group, signed=symmetric, bias=bias,
                      residual=residual)
    out = _lanes_run(x, pw, bias=bias, residual=residual)
    assert oracle.rel_l2(out, ref) <= TOL


@pytest.mark.parametrize("param_dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_decode_lanes_fractional_zero_points_and_fp32_output(param_dtype):
    """Zero points need not be integers here (the zero point only enters the fp32 fold), and the
    unrounded fp32 sums of a K-sharded layer come from the same kernel."""

    from xqt_b200.contracts import PackedWeight

    n, k, m = 264, 768, 5
    x, pw = _synthetic(n, k, m, seed=77, param_dtype=param_dtype)
    zeros = (pw.zero_points.float() + 0.25).to(param_dtype)
    pw2 = PackedWeight(qweight=pw.qweight, scales=pw.scales, zero_points=zeros, metadata=pw.metadata)
    ref = oracle.gemm(x, pw.qweight, pw.scales, zeros, group_size=128, signed=False)
    assert oracle.rel_l2(_lanes_run(x, pw2), ref) <= TOL
    out32 = _lanes_run(x, pw2, out_dtype=torch.float32)
    assert out32.dtype == torch.float32
    ref32 = oracle.gemm(x.float(), pw.qweight, pw.scales, zeros, group_size=128, signed=False)
    assert oracle.rel_l2(out32, ref32.float()) <= 1e-4


def test_decode_lanes_is_the_default_decode_layout():
    from xqt_b200.ops.w4a16 import prepare_decode

    x, pw = _synthetic(256, 512, 2, seed=5)
    dev = torch.device("cuda", 0)
    tiled = prepare_decode(pw.qweight.to(dev), pw.scales.to(dev), pw.zero_points.to(dev), group_size=128,
                           nibble_signed=False)
    assert tiled.layout == "lanes"
    forced = prepare_decode(pw.qweight.to(dev), pw.scales.to(dev), pw.zero_points.to(dev), group_size=128,
                            nibble_signed=False, layout="rows128")
    assert forced.layout == "rows128"


@pytest.mark.parametrize("source", ["awq", "gptq"])
def test_decode_of_an_imported_checkpoint_layer(source):
    """HF AWQ / GPTQ int32 words -> canonical xqt_int4_nk_v1 (repack pinned bit for bit by the CPU golden
    test) -> decode execution layout -> cluster decode kernel, against the oracle on the canonical form."""

    from xqt_b200 import layout
    from xqt_b200.ops.w4a16 import bind_w4a16_decode, prepare_decode

    n, k, g, m = 256, 512, 128, 5
    x = torch.randn((m, k), generator=seeded(91)).to(torch.bfloat16)
    if source == "awq":      # words [K, N/8], scales / zero points [K/g, N]
        words = torch.randint(-(2**31), 2**31 - 1, (k, n // 8), generator=seeded(92), dtype=torch.int64).to(torch.int32)
        pw = layout.repack_awq_int4(words, logical_shape=(n, k), scales=torch.rand((k // g, n), generator=seeded(93)) * 0.01 + 0.002,
                                    zero_points=torch.randint(0, 16, (k // g, n), generator=seeded(94)).to(torch.float32), group_size=g)
        assert not pw.metadata.nibble_signed and pw.zero_points is not None
    else:                    # words [K/8, N], scales [K/g, N], symmetric
        words = torch.randint(-(2**31), 2**31 - 1, (k // 8, n), generator=seeded(95), dtype=torch.int64).to(torch.int32)
        pw = layout.repack_gptq_int4(words, logical_shape=(n, k), scales=torch.rand((k // g, n), generator=seeded(96)) * 0.01 + 0.002,
                                     group_size=g)
        assert pw.metadata.nibble_signed and pw.zero_points is None
    dev = torch.device("cuda", 0)
    mv = lambda v: None if v is None else v.to(dev)
    tiled = prepare_decode(mv(pw.qweight), mv(pw.scales), mv(pw.zero_points), group_size=g,
                           nibble_signed=pw.metadata.nibble_signed)
    assert tiled.layout == "lanes"
    out = bind_w4a16_decode(tiled, rows=m, dtype=torch.bfloat16)(mv(x)).cpu()
    ref = oracle.gemm(x, pw.qweight, pw.scales, pw.zero_points, group_size=g, signed=pw.metadata.nibble_signed)
    assert oracle.rel_l2(out, ref) <= TOL


# ---------------------------------------------------------------------------- tcgen05 GEMM (M > 16)


@pytest.mark.parametrize("m,n,k", [(17, 128, 128), (128, 256, 256), (300, 392, 1280), (512, 4096, 4096),
                                   (1000, 14336, 4096), (4096, 4096, 14336)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_tcgen05_shapes(m, n, k, dtype):
    if m >= 1000 and dtype == torch.float16:
        pytest.skip("large shapes in bf16 only")
    x, pw = _synthetic(n, k, m, seed=700 + m, dtype=dtype)
    assert select_variant(m, n, k, k, 128) == "tcgen05"
    out = _run(x, pw.qweight, pw.scales, pw.zero_points, group=128, signed=False)      # auto -> tcgen05
    torch.set_num_threads(16)
    ref = oracle.gemm(x, pw.qweight, pw.scales, pw.zero_points, group_size=128, signed=False)
    assert oracle.rel_l2(out, ref) <= TOL


@pytest.mark.parametrize("group,symmetric", [(64, False), (64, True), (128, True)])
def test_gemm_tcgen05_groups_signed_epilogue(group, symmetric):
    m, n, k = 200, 264, 768
    x, pw = _synthetic(n, k, m, seed=33, symmetric=symmetric, group=group, param_dtype=torch.float32)
    bias = torch.randn((n,), generator=seeded(8))
    residual = torch.randn((m, n), generator=seeded(9)).to(torch.bfloat16)
    out = _run(x, pw.qweight, pw.scales, pw.zero_points, group=group, signed=symmetric, bias=bias,
               residual=residual, variant="tcgen05_fused")
    ref = oracle.gemm(x, pw.qweight, pw.scales, pw.zero_points, group_size=group, signed=symmetric, bias=bias,
                      residual=residual)
    assert oracle.rel_l2(out, ref) <= TOL


@pytest.mark.parametrize("m,n,k", [(17, 128, 128), (128, 256, 256), (300, 392, 1280), (512, 4096, 4096)])
def test_gemm_single_pass_variant_shapes(m, n, k):
    """The single-pass kernel (dequantisation inside the GEMM, no weight scratch) on its own variant code."""

    x, pw = _synthetic(n, k, m, seed=900 + m)
    out = _run(x, pw.qweight, pw.scales, pw.zero_points, group=128, signed=False, variant="tcgen05_fused")
    ref = oracle.gemm(x, pw.qweight, pw.scales, pw.zero_points, group_size=128, signed=False)
    assert oracle.rel_l2(out, ref) <= TOL


@pytest.mark.parametrize("m,n,k", [(64, 512, 1792), (200, 4096, 3584), (300, 392, 1280)])
def test_fused_gemm_writes_fp32_partial_sums(m, n, k):
    """Unrounded fp32 output (the partial sums of a K-sharded layer) from the fused kernel, with and without a K split."""

    dev = torch.device("cuda", 0)
    x, pw = _synthetic(n, k, m, seed=950 + m)
    out = w4a16_linear(x.to(dev), pw.qweight.to(dev), pw.scales.to(dev), pw.zero_points.to(dev), group_size=128,
                       nibble_signed=False, out_dtype=torch.float32, variant="tcgen05_fused")
    assert out.dtype == torch.float32
    ref = oracle.gemm(x, pw.qweight, pw.scales, pw.zero_points, group_size=128, signed=False, out_dtype=torch.float32)
    assert oracle.rel_l2(out.cpu(), ref) <= TOL


@pytest.mark.parametrize("group,symmetric", [(64, False), (128, True), (128, False)])
def test_gemm_two_pass_groups_signed_epilogue(group, symmetric):
    """M >= 256: weights dequantised once into an fp16 scratch, then the dense tcgen05 GEMM."""

    from xqt_b200 import native

    m, n, k = 300, 264, 768
    assert native.library().xqt_b200_w4a16_two_pass(m) == 1 and native.library().xqt_b200_w4a16_two_pass(16) == 0
    x, pw = _synthetic(n, k, m, seed=35, symmetric=symmetric, group=group, param_dtype=torch.float32)
    bias = torch.randn((n,), generator=seeded(8))
    residual = torch.randn((m, n), generator=seeded(9)).to(torch.bfloat16)
    out = _run(x, pw.qweight, pw.scales, pw.zero_points, group=group, signed=symmetric, bias=bias,
               residual=residual, variant="tcgen05")
    ref = oracle.gemm(x, pw.qweight, pw.scales, pw.zero_points, group_size=group, signed=symmetric, bias=bias,
                      residual=residual)
    assert oracle.rel_l2(out, ref) <= TOL


def test_gemm_two_pass_serves_non_integer_zero_points():
    m, n, k = 320, 128, 256
    x, pw = _synthetic(n, k, m, seed=45, param_dtype=torch.float32)
    zeros = pw.zero_points + 0.25
    out = _run(x, pw.qweight, pw.scales, zeros, group=128, signed=False, variant="tcgen05")
    ref = oracle.gemm(x, pw.qweight, pw.scales, zeros, group_size=128, signed=False)
    assert oracle.rel_l2(out, ref) <= TOL
    auto = _run(x, pw.qweight, pw.scales, zeros, group=128, signed=False)
    assert torch.equal(auto, out)          # auto takes the same two-pass kernel at this M


def test_gemm_non_integer_zero_points_take_the_exact_path():
    m, n, k = 64, 128, 256
    x, pw = _synthetic(n, k, m, seed=44, param_dtype=torch.float32)
    zeros = pw.zero_points + 0.25
    out = _run(x, pw.qweight, pw.scales, zeros, group=128, signed=False)     # auto: two-pass GEMM (fp32 dequantisation)
    ref = oracle.gemm(x, pw.qweight, pw.scales, zeros, group_size=128, signed=False)
    assert oracle.rel_l2(out, ref) <= TOL
    from xqt_b200.errors import XQTBackendError
    with pytest.raises(XQTBackendError):     # the single-pass kernel folds the zero point into an integer subtraction
        _run(x, pw.qweight, pw.scales, zeros, group=128, signed=False, variant="tcgen05_fused")
