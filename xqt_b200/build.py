"""Ahead-of-time build of the C-ABI library for sm_100a: ``python -m xqt_b200.build``.

One ``nvcc -shared`` over every ``csrc/*.cu`` into ``xqt_b200/libxqt_b200.so`` (in-tree, so the
binary travels with the checkout).  xqt compiles its sm_89 sources just in time with a cache key
of flags + source hash (xqt/kernels/jit/utils/compile/spec.py:14-58, compile/cache.py:15-52);
the same key decides here whether a rebuild is needed, but the build itself happens once, offline.
nvcc cross-compiles, so no GPU is needed to build.
"""

from __future__ import annotations

import hashlib
import pathlib
import shutil
import subprocess
import sys

PACKAGE = pathlib.Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
INCLUDE = PACKAGE.parent / "include"
OUTPUT = PACKAGE / "libxqt_b200.so"
STAMP = PACKAGE / "libxqt_b200.so.key"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
# -fmad=false: no implicit multiply-add contraction, so fp32 results that the tests compare bit for
# bit (rotation, quantisation) do not depend on the compiler; the kernels spell out fmaf where they want it
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-fmad=false", "--threads", "8", "-Xcompiler", "-fPIC", "-shared"]


def sources() -> list[pathlib.Path]:
    return sorted(CSRC.glob("*.cu"))


def cache_key() -> str:
    digest = hashlib.sha256()
    digest.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    for path in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()


def up_to_date() -> bool:
    return OUTPUT.exists() and STAMP.exists() and STAMP.read_text().strip() == cache_key()


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    if not force and up_to_date():
        return OUTPUT
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not pathlib.Path(nvcc).exists():
        raise RuntimeError("nvcc not found; the sm_100a library cannot be built on this machine")
    command = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(INCLUDE), "-o", str(OUTPUT)]
    if verbose:
        command += ["-Xptxas", "-v"]
    command += [str(path) for path in sources()]
    result = subprocess.run(command, capture_output=True, text=True)
    if verbose or result.returncode != 0:
        sys.stderr.write(result.stdout + result.stderr)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed with exit code {result.returncode}")
    STAMP.write_text(cache_key() + "\n")
    return OUTPUT


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
