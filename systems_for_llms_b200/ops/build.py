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


def build(force: bool = False, verbose: bool = False, *, defines: tuple[str, ...] = (),
          output: Path | None = None) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link ``libsfl_b200.so``.

    ``defines`` (e.g. ``("SFL_DEBUG_BOUNDS",)``) builds an instrumented variant; it must be
    given its own ``output`` path and is loaded by setting ``SFL_LIBRARY`` to that path
    before the first kernel call (``ops/lib.py``).  Concurrent callers (the ranks of one
    job started on a fresh checkout) serialise on a lock file and re-check the stamp once
    they hold it, so only the first one compiles.
    """
    if defines:
        if output is None:
            raise ValueError("an instrumented build needs its own output path")
        return _compile(Path(output), Path(output).with_suffix(".objects"), verbose, defines)
    if not force and is_current():
        return LIB_PATH
    import fcntl
    with open(LIB_DIR / "libsfl_b200.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and is_current():      # another process built it meanwhile
                return LIB_PATH
            _compile(LIB_PATH, LIB_DIR / "build", verbose, ())
            STAMP_PATH.write_text(source_hash() + "\n")
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB_PATH


def _compile(target: Path, build_dir: Path, verbose: bool, defines: tuple[str, ...]) -> Path:
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernel library")
    build_dir.mkdir(parents=True, exist_ok=True)
    extra = (["-Xptxas", "-v"] if verbose else []) + [f"-D{name}" for name in defines]

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
    temporary = target.with_suffix(f".tmp{os.getpid()}")
    link = [nvcc, "-shared", "-o", str(temporary), *map(str, objects)]
    result = subprocess.run(link, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"link failed:\n{result.stderr}")
    os.replace(temporary, target)
    return target


if __name__ == "__main__":
    # python -m systems_for_llms_b200.ops.build [--force] [--verbose] [-DNAME ... --output PATH]
    names = tuple(arg[2:] for arg in sys.argv[1:] if arg.startswith("-D"))
    out = Path(sys.argv[sys.argv.index("--output") + 1]) if "--output" in sys.argv else None
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, defines=names,
                 output=out)
    print(path)
