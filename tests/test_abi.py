"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def library():
    from mircuda_b200 import build, _lib
    build.build_library()
    return _lib.load()


def declared_symbols():
    text = (ROOT / "include" / "mircuda_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mircuda_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(library):
    from mircuda_b200 import _lib
    names = declared_symbols()
    assert len(names) >= 15
    for name in names:
        assert hasattr(library, name), name
    assert sorted(_lib.SIGNATURES) == names


def test_version(library):
    assert library.mircuda_b200_version() == (2 << 8)
    # sys/native/cutlass_probe.cu:16 with the pin of sys/build/sources.rs:8 (v4.4.2)
    assert library.mircuda_cutlass_version() == 40402


def test_argument_validation_needs_no_gpu(library):
    """-1 for bad arguments is decided before any CUDA call (sys/native/mxfp8_sm120.cu:113-114)."""
    raw = ctypes.c_void_p()
    fake_stream = ctypes.c_void_p(0x10)
    assert library.mircuda_mxfp8_tc_create(128, 128, 128, None, ctypes.byref(raw)) == -1
    assert library.mircuda_mxfp8_tc_create(128, 128, 100, fake_stream, ctypes.byref(raw)) == -1
    assert library.mircuda_mxfp8_tc_create(0, 128, 128, fake_stream, ctypes.byref(raw)) == -1
    assert library.mircuda_mxfp8_tc_create(128, 128, 128, fake_stream, None) == -1
    assert library.mircuda_fp4_vector_create(16, 100, fake_stream, ctypes.byref(raw)) == -1
    assert library.mircuda_fp4_vector_create(16, 128, None, ctypes.byref(raw)) == -1
    assert library.mircuda_dense_vector_create(2, 16, 16, fake_stream, ctypes.byref(raw)) == -1
    assert library.mircuda_dense_vector_create(1, 0, 16, fake_stream, ctypes.byref(raw)) == -1
    assert library.mircuda_b200_nvfp4_vector_create(9, 16, 64, fake_stream, ctypes.byref(raw)) == -1
    assert library.mircuda_b200_mxfp8_quantize_bf16(None, None, None, 1, 32, fake_stream) == -1
    assert library.mircuda_mxfp8_tc_execute(None, fake_stream, None, None, None, None, None) == -1
    fake = ctypes.c_void_p(0x1000)
    assert library.mircuda_b200_mxfp8_quantize_bf16_blocks(fake, fake, fake, 4, 128, 0, fake_stream) == -1
    assert library.mircuda_b200_mxfp8_quantize_bf16_blocks(fake, fake, fake, 4, 128, 48, fake_stream) == -1
    assert library.mircuda_b200_mxfp8_quantize_bf16_blocks(fake, fake, fake, 4, 128, 12, fake_stream) == -1
    assert library.mircuda_b200_column_gather_create(1, 0, ctypes.byref(raw)) == -1
    assert library.mircuda_b200_column_gather_create(9, 0, ctypes.byref(raw)) == -1
    assert library.mircuda_b200_column_gather_create(4, 4, ctypes.byref(raw)) == -1
    assert library.mircuda_b200_column_gather_create(4, 0, None) == -1
    assert library.mircuda_b200_column_gather_send(None, None, 8, 0, 8, 1, fake_stream) == -1
    assert library.mircuda_b200_column_gather_join(None, fake_stream) == -1
    library.mircuda_b200_column_gather_destroy(None)
    assert library.mircuda_mxfp8_tc_workspace_bytes(None) == 0
    library.mircuda_mxfp8_tc_destroy(None)
    library.mircuda_fp4_vector_destroy(None)
    library.mircuda_dense_vector_destroy(None)


def test_host_mirror_validates_shapes():
    from mircuda_b200 import plans
    assert plans.BlockScaledMxFp8Spec(4, 128, 128).scale_bytes(4) == 512
    with pytest.raises(plans.InvalidMatmulShape):
        plans.BlockScaledMxFp8Spec(4, 128, 96)
    with pytest.raises(plans.InvalidMatmulShape):
        plans.MxFp8Spec(1, 31, 1)                       # tests/mxfp8/main.rs:22
    spec = plans.MxFp8Spec(2, 32, 3)                    # tests/mxfp8/main.rs:16-21
    assert spec.weight_words() == 24 and spec.scale_elements() == 3
    with pytest.raises(plans.InvalidMatmulShape):
        plans.BlockScaledFp4VectorSpec(16, 100)
    assert plans.BlockScaledFp4VectorSpec(704, 2816).scale_bytes(704) == 6 * 44 * 512
