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
