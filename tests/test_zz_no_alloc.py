"""The allocation-free decode entry point (scratch built into the library) against the regular one.

Some callers of this library may launch kernels but cannot allocate device memory where they call
it: a server that distributed its whole memory pool at start-up, a plugin inside an application that
owns the allocator, a latency-critical loop where allocator calls are banned.  For them
``xqt_b200_w4a16_decode_tiled_static`` takes only inputs and outputs.  The test drives it through
the C ABI with buffers created beforehand and checks, on two calls in a row (the second finds the
scratch as the first left it), that it returns exactly what ``xqt_b200_w4a16_decode_tiled`` returns
with a caller-provided workspace: both run the same kernel with the same fixed summation order, so
the comparison is bit for bit, well inside the rel-L2 <= 1e-3 bar of the other W4A16 tests.
The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""

from __future__ import annotations

import pytest
import torch

from conftest import seeded
from xqt_b200 import native, prepack, quantize

pytestmark = pytest.mark.gpu


def _case(n, k, m, seed, device):
    w = torch.randn((n, k), generator=seeded(seed)) * 0.02
    x = torch.randn((m, k), generator=seeded(seed + 1)).to(torch.bfloat16).to(device)
    pw = quantize.quantize_w4_asymmetric(w, group_size=128)
    tiled = prepack.tile_w4(pw.qweight.to(device), pw.scales.to(device), pw.zero_points.to(device),
                            group_size=128, nibble_signed=False)
    bias = torch.randn((n,), generator=seeded(seed + 2)).to(device)
    return x, tiled, bias


@pytest.mark.parametrize("n,k,m", [(4096, 4096, 16), (1000, 1024, 3), (14336, 4096, 1)])
def test_static_scratch_entry_matches_workspace_entry(n, k, m):
    device = torch.device("cuda", 0)
    lib = native.library()
    x, tiled, bias = _case(n, k, m, 400 + m, device)
    stream = native.stream_handle(device)
    # everything the calls need exists before them; the entry point under test allocates nothing
    expected = torch.empty((m, n), device=device, dtype=torch.bfloat16)
    outputs = [torch.full((m, n), float("nan"), device=device, dtype=torch.bfloat16) for _ in range(2)]
    scratch = torch.zeros(lib.xqt_b200_w4a16_decode_workspace_bytes(), dtype=torch.uint8, device=device)
    common = (tiled.weights.data_ptr(), tiled.params.data_ptr(), bias.data_ptr(), 0)
    dims = (m, n, k, 128, 0, 1, native.BF16, native.BF16)
    native.check(lib.xqt_b200_w4a16_decode_tiled(x.data_ptr(), *common, expected.data_ptr(), *dims,
                                                 scratch.data_ptr(), scratch.numel(), stream),
                 "xqt_b200_w4a16_decode_tiled")
    torch.cuda.synchronize()
    reserved = torch.cuda.memory_reserved(device)
    for out in outputs:          # two calls in a row share the built-in scratch
        native.check(lib.xqt_b200_w4a16_decode_tiled_static(x.data_ptr(), *common, out.data_ptr(), *dims, stream),
                     "xqt_b200_w4a16_decode_tiled_static")
    torch.cuda.synchronize()
    assert torch.cuda.memory_reserved(device) == reserved
    for out in outputs:
        assert not torch.isnan(out.float()).any()
        assert torch.equal(out, expected)


def test_static_scratch_entry_rejects_sizes_beyond_its_limit():
    lib = native.library()
    limit = lib.xqt_b200_w4a16_decode_static_max_n()
    assert limit == 131072 and lib.xqt_b200_w4a16_decode_static_scratch_bytes() < 4 * 1024 * 1024
    device = torch.device("cuda", 0)
    dummy = torch.zeros(4096, dtype=torch.uint8, device=device)
    code = lib.xqt_b200_w4a16_decode_tiled_static(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), 0, 0,
                                                  dummy.data_ptr(), 1, limit + 128, 256, 128, 0, 1, native.BF16,
                                                  native.BF16, native.stream_handle(device))
    assert code == 1          # cudaErrorInvalidValue, nothing launched
    with pytest.raises(native.CudaCallError):
        native.check(code, "xqt_b200_w4a16_decode_tiled_static")
