"""Builds the sm_100a kernel library in-tree with nvcc.

The library is plain CUDA C++ with a C interface (no PyTorch headers), so each
translation unit compiles in seconds and the result is loaded with ctypes.  A
stamp file holding the hash of all sources makes rebuilds a no-op; the built
``libsfl_b200.so`` sits next to this package so it travels with the source tree.

The reference builds its only CUDA file with ``torch.utils.cpp_extension.load``
at first use (attention_lab/cuda_decode/kernel.py:14-24); here the build is an
explicit step (``python -m systems_for_llms_b200.ops.build``) that also works
on machines without a GPU because nvcc cross-compiles.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
LIB_DIR = Path(__file__).resolve().parent
LIB_PATH = LIB_DIR / "libsfl_b200.so"
STAMP_PATH = LIB_DIR / "libsfl_b200.stamp"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
]


def _nvcc() -> str | None:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).exists():
            return candidate
    return None


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def source_hash() -> str:
    digest = hashlib.sha256()
    for path in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update(" ".join(NVCC_FLAGS).encode())
    return digest.hexdigest()


def is_current() -> bool:
    return (LIB_PATH.exists() and STAMP_PATH.exists()
            and STAMP_PATH.read_text().strip() == source_hash())


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link ``libsfl_b200.so``."""
    if not force and is_current():
        return LIB_PATH
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernel library")
    build_dir = LIB_DIR / "build"
    build_dir.mkdir(exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src: Path) -> Path:
        obj = build_dir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        result = subprocess.run(cmd, capture_output=True, text=True)
        if verbose:
            sys.stderr.write(result.stderr)
        if result.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{result.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objects = list(pool.map(compile_one, sources()))
    temporary = LIB_PATH.with_suffix(".so.tmp")
    link = [nvcc, "-shared", "-o", str(temporary), *map(str, objects)]
    result = subprocess.run(link, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"link failed:\n{result.stderr}")
    os.replace(temporary, LIB_PATH)
    STAMP_PATH.write_text(source_hash() + "\n")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
