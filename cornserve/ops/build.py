"""Builds the sm_100a kernel library in-tree.

Every ``csrc/*.cu`` file is compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a`` and the
objects are linked into ``cornserve/ops/libcornserve.so``.  nvcc cross-compiles, so this
works on a machine without a GPU.  The library exposes a plain C ABI (see ``csrc/*.h``) that
``cornserve.ops`` binds with ctypes, so neither pybind11 nor the torch headers are needed.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

REPO = Path(__file__).resolve().parents[2]
CSRC = REPO / "csrc"
OUT_DIR = Path(__file__).resolve().parent
LIB_PATH = OUT_DIR / "libcornserve.so"
BUILD_DIR = REPO / "build" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; the kernel library cannot be built")
    return cand


def _digest(path: Path, extra: bytes) -> str:
    h = hashlib.sha256()
    h.update(path.read_bytes())
    h.update(extra)
    return h.hexdigest()


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile (only what changed) and link; returns the path of the shared library."""
    nvcc = _nvcc()
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    headers = b"".join(p.read_bytes() for p in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")))
    flags_blob = " ".join(NVCC_FLAGS).encode()
    todo: list[tuple[Path, Path, Path, str]] = []
    objs: list[Path] = []
    for src in sources():
        obj = BUILD_DIR / (src.stem + ".o")
        stamp = BUILD_DIR / (src.stem + ".sha")
        dig = _digest(src, headers + flags_blob)
        objs.append(obj)
        if force or not obj.exists() or not stamp.exists() or stamp.read_text() != dig:
            todo.append((src, obj, stamp, dig))

    def compile_one(item: tuple[Path, Path, Path, str]) -> None:
        src, obj, stamp, dig = item
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            sys.stderr.write(res.stderr)
        stamp.write_text(dig)

    if todo:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
            list(ex.map(compile_one, todo))
    if todo or not LIB_PATH.exists():
        tmp = LIB_PATH.with_suffix(".so.tmp")
        cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-lpthread"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(p)
