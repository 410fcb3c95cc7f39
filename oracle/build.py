"""Build recipe for the test oracle and for the reference-derived checkers.

TEST INFRASTRUCTURE ONLY. Nothing here is imported by the product package.

* ``build_oracle()`` compiles ``mircuda_oracle.c`` (the C restatement) into
  ``oracle/_build/libmircuda_oracle.so``.
* ``build_ref()`` compiles, from the sources where they lie in a reference checkout,
  - ``kernels/mxfp8.cu`` for the host (helper functions only) -> ``_ref/libref_host.so``
  - ``kernels/mxfp8.cu`` for sm_100a with launchers          -> ``_ref/libref_device.so``
  - ``sys/native/{fp4_vector,dense_vector}_sm120.cu``        -> ``_ref/libref_vector.so``
  Outputs go only into ``oracle/_ref/`` (git-ignored). No reference source is copied.
  Without a reference checkout this is a no-op and prebuilt files are used as they are.

Run ``python oracle/build.py`` to build both.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
BUILD_DIR = HERE / "_build"
REF_DIR = HERE / "_ref"
ORACLE_LIB = BUILD_DIR / "libmircuda_oracle.so"
# The reference checkout: MIRCUDA_REFERENCE_ROOT, else a directory named `reference` beside this
# repository. When neither exists the prebuilt files in `_ref/` are used as they are.
REFERENCE_ROOT = Path(os.environ.get("MIRCUDA_REFERENCE_ROOT", HERE.parent.parent / "reference"))
GENCODE = "arch=compute_100a,code=sm_100a"


def _newer(target: Path, *sources: Path) -> bool:
    if not target.exists():
        return False
    stamp = target.stat().st_mtime
    return all(source.exists() and source.stat().st_mtime <= stamp for source in sources)


def _run(command: list[str]) -> None:
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(
            "command failed: " + " ".join(command) + "\n" + result.stdout + result.stderr
        )


def build_oracle(force: bool = False) -> Path:
    source = HERE / "mircuda_oracle.c"
    if not force and _newer(ORACLE_LIB, source):
        return ORACLE_LIB
    compiler = shutil.which("gcc")
    if compiler is None:
        if ORACLE_LIB.exists():
            return ORACLE_LIB
        raise RuntimeError("gcc not found and no prebuilt oracle library")
    BUILD_DIR.mkdir(exist_ok=True)
    _run([
        compiler, "-O3", "-mavx2", "-mfma", "-fopenmp", "-fPIC", "-shared", "-std=c11",
        "-fvisibility=hidden", "-o", str(ORACLE_LIB), str(source), "-lm",
    ])
    return ORACLE_LIB


def _cutlass_include() -> list[str]:
    """Header-only CUTLASS tree the reference's vector kernels include (bfloat16.h, float8.h):
    MIRCUDA_CUTLASS_ROOT (a checkout with `include/` and `tools/util/include/`), else the tree an
    installed flashinfer wheel carries."""
    override = os.environ.get("MIRCUDA_CUTLASS_ROOT")
    if override:
        paths = [Path(override) / "include", Path(override) / "tools" / "util" / "include"]
        return [f"-I{path}" for path in paths if path.exists()]
    try:
        import flashinfer  # noqa: F401  (only for its vendored header tree)
        root = Path(flashinfer.__file__).resolve().parent / "data" / "cutlass"
    except Exception:
        return []
    paths = [root / "include", root / "tools" / "util" / "include"]
    return [f"-I{path}" for path in paths if path.exists()]


def build_ref(force: bool = False) -> dict[str, Path]:
    outputs = {
        "host": REF_DIR / "libref_host.so",
        "device": REF_DIR / "libref_device.so",
        "vector": REF_DIR / "libref_vector.so",
    }
    mxfp8 = REFERENCE_ROOT / "kernels" / "mxfp8.cu"
    if not mxfp8.exists():
        return {name: path for name, path in outputs.items() if path.exists()}
    REF_DIR.mkdir(exist_ok=True)
    define = f'-DREF_MXFP8_CU="{mxfp8}"'

    host_shim = HERE / "ref_host_shim.cpp"
    if force or not _newer(outputs["host"], host_shim, mxfp8):
        # -x c++ : the .cu file is plain C++ once the CUDA qualifiers are defined away.
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-x", "c++", define,
              "-o", str(outputs["host"]), str(host_shim)])

    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    common = [nvcc, "-O3", "-std=c++17", "--expt-relaxed-constexpr", "-gencode", GENCODE,
              "-Xcompiler", "-fPIC", "-shared", "-cudart", "shared"]
    device_shim = HERE / "ref_device.cu"
    if force or not _newer(outputs["device"], device_shim, mxfp8):
        _run(common + [define, "-o", str(outputs["device"]), str(device_shim)])

    native = REFERENCE_ROOT / "sys" / "native"
    vector_sources = [native / "fp4_vector_sm120.cu", native / "dense_vector_sm120.cu"]
    if force or not _newer(outputs["vector"], *vector_sources):
        include = _cutlass_include()
        if include:
            _run(common + include + [f"-I{native}", "-o", str(outputs["vector"])]
                 + [str(source) for source in vector_sources])
    return {name: path for name, path in outputs.items() if path.exists()}


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    for name, path in build_ref(force="--force" in sys.argv).items():
        print(name, path)
