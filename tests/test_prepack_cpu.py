"""Host logic of the execution layouts: bit-exact round trips, no GPU needed."""

from __future__ import annotations

import pytest
import torch

from conftest import seeded
from xqt_b200 import prepack, quantize
from xqt_b200.errors import XQTBackendError


@pytest.mark.parametrize("n,k,group,symmetric", [(200, 512, 128, False), (256, 256, 32, True), (64, 128, 64, False),
                                                 (129, 384, 64, True)])
def test_tile_w4_round_trip(n, k, group, symmetric):
    w = torch.randn((n, k), generator=seeded(n + k)) * 0.02
    pw = quantize.quantize_w4_symmetric(w, group_size=group) if symmetric else quantize.quantize_w4_asymmetric(w, group_size=group)
    tiled = prepack.tile_w4(pw.qweight, pw.scales, pw.zero_points, group_size=group, nibble_signed=symmetric)
    assert tuple(tiled.weights.shape) == (-(-n // 128), k // 128, 16, 32, 16)
    q, s, z = prepack.untile_w4(tiled)
    assert torch.equal(q, pw.qweight) and torch.equal(s, pw.scales)
    assert (z is None) == (pw.zero_points is None)
    if z is not None:
        assert torch.equal(z, pw.zero_points)


def test_tile_w4_word_semantics():
    # (word >> 4i) & 0x000f000f must give the adjacent pair (k+2i, k+2i+1) of the lane's 8-K run
    n, k = 128, 256
    codes = torch.randint(0, 16, (n, k), generator=seeded(1), dtype=torch.int64).to(torch.uint8)
    qweight = codes[:, 0::2] | (codes[:, 1::2] << 4)
    scales = torch.ones((n, k // 128), dtype=torch.bfloat16)
    tiled = prepack.tile_w4(qweight, scales, None, group_size=128, nibble_signed=False)
    words = tiled.weights.reshape(1, 2, 16, 32, 4, 4).to(torch.int64)
    words = words[..., 0] | (words[..., 1] << 8) | (words[..., 2] << 16) | (words[..., 3] << 24)
    for (kb, j, g, t, w) in [(0, 0, 0, 0, 0), (1, 5, 3, 2, 1), (1, 15, 7, 3, 3)]:
        word = int(words[0, kb, j, 4 * g + t, w])
        row, k0 = 8 * j + g, 128 * kb + 32 * w + 8 * t
        for i in range(4):
            assert (word >> (4 * i)) & 0xF == int(codes[row, k0 + 2 * i])
            assert (word >> (4 * i + 16)) & 0xF == int(codes[row, k0 + 2 * i + 1])


def test_tile_w4_rejects_ragged_k():
    q = torch.zeros((8, 100), dtype=torch.uint8)
    with pytest.raises(XQTBackendError):
        prepack.tile_w4(q, torch.ones((8, 2)), None, group_size=128, nibble_signed=True, k=200)


@pytest.mark.parametrize("n,k,group,symmetric", [(200, 512, 128, False), (128, 256, 64, True), (72, 768, 64, False)])
def test_lanes_w4_round_trip(n, k, group, symmetric):
    w = torch.randn((n, k), generator=seeded(n + k)) * 0.02
    pw = quantize.quantize_w4_symmetric(w, group_size=group) if symmetric else quantize.quantize_w4_asymmetric(w, group_size=group)
    tiled = prepack.lanes_w4(pw.qweight, pw.scales, pw.zero_points, group_size=group, nibble_signed=symmetric)
    assert tiled.layout == "lanes"
    assert tuple(tiled.weights.shape) == (-(-n // 128), k // 128, 4, 2, 2, 32, 16)
    assert tuple(tiled.params.shape) == (1 if symmetric else 2, -(-n // 128), k // 128, 128 // group, 4, 8, 4)
    assert tiled.nbytes == tiled.weights.numel() + tiled.params.numel() * tiled.params.element_size()
    q, s, z = prepack.untile_w4(tiled)
    assert torch.equal(q, pw.qweight) and torch.equal(s, pw.scales)
    assert (z is None) == (pw.zero_points is None)
    if z is not None:
        assert torch.equal(z, pw.zero_points)


def test_lanes_w4_fragment_semantics():
    """Walk the layout the way the decode kernel's lanes do (mma.m16n8k16 fragment positions,
    16 contiguous activation bytes per two K-steps) and rebuild W @ x from it."""

    n, k, m = 128, 256, 8
    codes = torch.randint(0, 16, (n, k), generator=seeded(3), dtype=torch.int64)
    qweight = (codes[:, 0::2] | (codes[:, 1::2] << 4)).to(torch.uint8)
    scales = torch.ones((n, k // 128), dtype=torch.bfloat16)
    tiled = prepack.lanes_w4(qweight, scales, None, group_size=128, nibble_signed=False)
    x = torch.randint(-3, 4, (m, k), generator=seeded(4), dtype=torch.int64)
    b = tiled.weights.permute(0, 1, 2, 3, 5, 4, 6).reshape(1, k // 128, 4, 2, 32, 8, 4).to(torch.int64)   # lane-major view
    words = b[..., 0] | (b[..., 1] << 8) | (b[..., 2] << 16) | (b[..., 3] << 24)
    out = torch.zeros((n, m), dtype=torch.int64)
    for kb in range(k // 128):
        for w in range(4):
            for t in range(2):
                for j in range(8):
                    a = torch.zeros((16, 16), dtype=torch.int64)       # A fragment, row-major 16 x 16
                    bm = torch.zeros((16, 8), dtype=torch.int64)       # B fragment, 16 x 8
                    for lane in range(32):
                        r, c = lane >> 2, lane & 3
                        word = int(words[0, kb, w, t, lane, j])
                        regs = [((word >> (4 * i)) & 0xF, (word >> (4 * i + 16)) & 0xF) for i in range(4)]
                        a[r, 2 * c], a[r, 2 * c + 1] = regs[0]
                        a[r + 8, 2 * c], a[r + 8, 2 * c + 1] = regs[1]
                        a[r, 2 * c + 8], a[r, 2 * c + 9] = regs[2]
                        a[r + 8, 2 * c + 8], a[r + 8, 2 * c + 9] = regs[3]
                        v = x[r, 128 * kb + 32 * (j // 2) + 8 * c: 128 * kb + 32 * (j // 2) + 8 * c + 8]
                        jj = j % 2
                        bm[2 * c, r], bm[2 * c + 1, r] = v[4 * jj], v[4 * jj + 1]
                        bm[2 * c + 8, r], bm[2 * c + 9, r] = v[4 * jj + 2], v[4 * jj + 3]
                    base = 32 * w + 16 * t
                    out[base:base + 16] += a @ bm
    assert torch.equal(out, codes @ x.T)
    # the four (scale, zero) pairs of lane (w, r): channels 32w + 16t + 8h + r at index 2t + h
    s2 = torch.arange(n * 2, dtype=torch.float32).reshape(n, 2)
    t2 = prepack.lanes_w4(qweight, s2, s2 + 0.5, group_size=128, nibble_signed=False)
    for (kb, w, r, t, h) in [(0, 0, 0, 0, 0), (1, 3, 7, 1, 1), (1, 2, 5, 0, 1)]:
        ch = 32 * w + 16 * t + 8 * h + r
        assert float(t2.params[0, 0, kb, 0, w, r, 2 * t + h]) == float(s2[ch, kb])
        assert float(t2.params[1, 0, kb, 0, w, r, 2 * t + h]) == float(s2[ch, kb]) + 0.5
