"""Builds ``libmircuda_b200.so`` in-tree with nvcc for sm_100a.

``python -m mircuda_b200.build`` (or ``build_library()``) compiles every ``csrc/*.cu``
into one shared library next to this file. Objects are rebuilt only when their source
or a header is newer. nvcc cross-compiles, so no GPU is needed.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
SOURCE_DIR = PACKAGE_DIR / "csrc"
OBJECT_DIR = PACKAGE_DIR / "_obj"
LIBRARY = PACKAGE_DIR / "libmircuda_b200.so"
INCLUDE_DIR = PACKAGE_DIR.parent / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    f"-I{INCLUDE_DIR}", f"-I{SOURCE_DIR}",
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; cannot build libmircuda_b200.so")
    return found


def _stale(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(source.stat().st_mtime > stamp for source in sources)


def _compile(source: Path, headers: list[Path], verbose: bool) -> Path:
    obj = OBJECT_DIR / (source.stem + ".o")
    if _stale(obj, [source, *headers]):
        command = [_nvcc(), *NVCC_FLAGS, "-c", str(source), "-o", str(obj)]
        if verbose:
            command.insert(1, "-Xptxas=-v")
        result = subprocess.run(command, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"nvcc failed for {source.name}:\n{result.stdout}{result.stderr}")
        if verbose:
            sys.stderr.write(result.stderr)
    return obj


def build_library(force: bool = False, verbose: bool = False) -> Path:
    sources = sorted(SOURCE_DIR.glob("*.cu"))
    headers = sorted(SOURCE_DIR.glob("*.cuh")) + sorted(SOURCE_DIR.glob("*.hpp")) \
        + sorted(INCLUDE_DIR.glob("*.h"))
    if not sources:
        raise RuntimeError("no CUDA sources found")
    if shutil.which("nvcc") is None and not Path("/usr/local/cuda/bin/nvcc").exists():
        if LIBRARY.exists():
            return LIBRARY
        raise RuntimeError("nvcc not found and no prebuilt libmircuda_b200.so")
    OBJECT_DIR.mkdir(exist_ok=True)
    if force:
        for stale in OBJECT_DIR.glob("*.o"):
            stale.unlink()
    workers = min(len(sources), os.cpu_count() or 4)
    with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as pool:
        objects = list(pool.map(lambda source: _compile(source, headers, verbose), sources))
    if force or _stale(LIBRARY, objects):
        command = [_nvcc(), "-shared", "-o", str(LIBRARY), *map(str, objects),
                   "-gencode", "arch=compute_100a,code=sm_100a"]
        result = subprocess.run(command, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"link failed:\n{result.stdout}{result.stderr}")
    return LIBRARY


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
