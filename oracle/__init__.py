"""CPU oracle of the quantized-linear path.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Every function here restates, on the CPU, the arithmetic of xqt's own reference
implementation of the path (the file:line each one follows is in its docstring).
Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this package, and only as the checker or as the timed CPU baseline; the
shipped package never imports it and has no CPU fallback.

Arithmetic is done with torch CPU tensors because the reference itself is torch
CPU code: using the same elementwise primitives (IEEE fp32 division,
round-half-to-even, fp32 matmul) is what makes integer codes reproducible bit
for bit.  Nothing here touches CUDA.

Pinning: the oracle is checked against golden vectors produced by importing the
reference in place and running its functions on seeded inputs
(tests/golden/make_golden.py, outputs committed under tests/golden/), and
against the literal known-answer cases of the reference's own tests
(tests/gemm/test_reference.py:53-105, tests/gemm/test_w4_pack.py:19-41,
tests/quant/test_convrot_4bit_quantizer.py:29-41).  The one piece with no
reference CPU counterpart is the per-(token, 64-K group) int4 activation
quantisation of the W4A4 path, which exists in the reference only as CUDA
(gemm_w4a4.cuh:534-624): for that piece parity is unpinned; it is restated from
the reference's per-token CPU formula (convrot_4bit.py:669-679) applied at the
CUDA kernel's group granularity.
"""

from . import mlp, pattern, rotation, w4a16, w4a4, w8a8  # noqa: F401
