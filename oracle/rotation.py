"""Oracle for the block-diagonal Hadamard rotations.  Test infrastructure only.

Two matrix families, as in the reference:

* regular Hadamard of order 4^k: ``H4 = [[1,1,1,-1],[1,1,-1,1],[1,-1,1,1],[-1,1,1,1]]``,
  ``H_{4^k} = kron(H4, H_{4^(k-1)})``, normalised by ``1/sqrt(n)``; symmetric and
  self-inverse (xqt/compression/quant/quantizers/convrot_4bit.py:85-123,191-193);
* Sylvester Hadamard of order 2^k times a seeded diagonal of +-1 ("randomized
  Hadamard", ``H @ diag(signs)``, xqt/model/minicpm5_quarot.py:54-93).

The rotation is applied per block of the last dimension as ``x_block @ R``
(convrot_4bit.py:197-229).  :func:`rotate_matmul` is that statement verbatim.
:func:`rotate_fht` is the same product evaluated as a fast Hadamard transform
with a FIXED butterfly order in fp32; it is the bit-exact specification the CUDA
prologue follows (additions and subtractions only, then one multiply by
``sign/sqrt(n)``, then one rounding to the activation dtype), so integer
activation codes can be compared bit for bit.  The two agree to fp32 rounding.
"""

from __future__ import annotations

import math

import torch

H4 = ((1.0, 1.0, 1.0, -1.0), (1.0, 1.0, -1.0, 1.0), (1.0, -1.0, 1.0, 1.0), (-1.0, 1.0, 1.0, 1.0))


def is_power_of(value: int, base: int) -> bool:
    value = int(value)
    if value < 1:
        return False
    while value % base == 0:
        value //= base
    return value == 1


def regular_hadamard(order: int) -> torch.Tensor:
    """Unnormalised regular Hadamard matrix, order a power of four (convrot_4bit.py:98-123)."""

    if not is_power_of(order, 4):
        raise ValueError("regular Hadamard order must be a power of four")
    base = torch.tensor(H4, dtype=torch.float32)
    matrix = torch.ones((1, 1), dtype=torch.float32)
    while matrix.shape[0] < order:
        matrix = torch.kron(matrix, base) if matrix.shape[0] > 1 else base.clone()
    return matrix.contiguous()


def sylvester_hadamard(order: int) -> torch.Tensor:
    """Unnormalised Sylvester matrix, order a power of two (minicpm5_quarot.py:54-71)."""

    if not is_power_of(order, 2):
        raise ValueError("Sylvester Hadamard order must be a power of two")
    matrix = torch.ones((1, 1), dtype=torch.float32)
    while matrix.shape[0] < order:
        matrix = torch.cat((torch.cat((matrix, matrix), 1), torch.cat((matrix, -matrix), 1)), 0)
    return matrix


def random_signs(order: int, seed: int) -> torch.Tensor:
    """+-1 diagonal drawn like ``build_quarot_rotation`` (minicpm5_quarot.py:82-89)."""

    generator = torch.Generator(device="cpu").manual_seed(int(seed))
    bits = torch.randint(0, 2, (order,), generator=generator, dtype=torch.float64)
    return bits.mul(2.0).sub(1.0).to(torch.float32)


def rotation_matrix(kind: str, order: int, signs: torch.Tensor | None = None) -> torch.Tensor:
    """Normalised ``[order, order]`` fp32 rotation ``H / sqrt(n) * signs[None, :]``."""

    if kind == "regular":
        matrix = regular_hadamard(order)
    elif kind == "sylvester":
        matrix = sylvester_hadamard(order)
    else:
        raise ValueError(f"unknown rotation kind {kind!r}")
    matrix = (matrix.to(torch.float64) / math.sqrt(float(order))).to(torch.float32)
    if signs is not None:
        matrix = matrix * signs.to(torch.float32).reshape(1, order)
    return matrix


def rotate_matmul(x: torch.Tensor, matrix: torch.Tensor) -> torch.Tensor:
    """``_apply_groupwise_rotation`` for a last dim that is a multiple of the block
    (convrot_4bit.py:197-229): matmul in the dtype of ``x``."""

    block = int(matrix.shape[0])
    assert x.shape[-1] % block == 0
    blocks = x.reshape(-1, x.shape[-1] // block, block)
    return torch.matmul(blocks, matrix.to(x.dtype)).reshape(x.shape)


def _radix4_stage(v: torch.Tensor, stride: int) -> torch.Tensor:
    """One digit of the regular transform.  With (a,b,c,d) the four inputs at
    distance ``stride``: p=a+b, q=a-b, r=c+d, t=c-d; outputs p+t, p-t, q+r, r-q."""

    rows, n = v.shape
    g = v.reshape(rows, n // (4 * stride), 4, stride)
    a, b, c, d = g[:, :, 0], g[:, :, 1], g[:, :, 2], g[:, :, 3]
    p, q, r, t = a + b, a - b, c + d, c - d
    return torch.stack((p + t, p - t, q + r, r - q), dim=2).reshape(rows, n)


def _radix2_stage(v: torch.Tensor, stride: int) -> torch.Tensor:
    rows, n = v.shape
    g = v.reshape(rows, n // (2 * stride), 2, stride)
    a, b = g[:, :, 0], g[:, :, 1]
    return torch.stack((a + b, a - b), dim=2).reshape(rows, n)


def rotate_fht(
    x: torch.Tensor,
    *,
    kind: str,
    block: int,
    signs: torch.Tensor | None = None,
    out_dtype: torch.dtype | None = None,
) -> torch.Tensor:
    """Block-diagonal rotation with the fixed butterfly order the CUDA prologue uses.

    Stages run from the smallest stride to the largest (stride 1, 4, 16, ... for
    the regular family; 1, 2, 4, ... for Sylvester), all in fp32; then each
    element is multiplied once by ``signs[j] / sqrt(block)`` (an fp32 constant
    per column) and rounded once to ``out_dtype`` (default: dtype of ``x``).
    """

    k = int(x.shape[-1])
    assert k % block == 0
    v = x.to(torch.float32).reshape(-1, block)
    stride = 1
    if kind == "regular":
        assert is_power_of(block, 4)
        while stride < block:
            v = _radix4_stage(v, stride)
            stride *= 4
    elif kind == "sylvester":
        assert is_power_of(block, 2)
        while stride < block:
            v = _radix2_stage(v, stride)
            stride *= 2
    else:
        raise ValueError(f"unknown rotation kind {kind!r}")
    norm = torch.full((block,), 1.0 / math.sqrt(float(block)), dtype=torch.float64)
    if signs is not None:
        norm = norm * signs.to(torch.float64)
    v = v * norm.to(torch.float32)
    return v.reshape(x.shape).to(out_dtype or x.dtype)
