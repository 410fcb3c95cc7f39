"""Host-side mirrors added after the first milestone: spec validation, buffer-size rules and
the int4 weight quantiser, all on CPU; argument validation of the newer C entry points."""
import ctypes

import pytest
import torch


@pytest.fixture(scope="module")
def library():
    from mircuda_b200 import build, _lib
    build.build_library()
    return _lib.load()


def test_variable_grouped_fp4_spec_sizes():
    """sys/src/platform/cutlass/variable_grouped/fp4/mod.rs:150-223: scale capacity and bytes."""
    from mircuda_b200 import plans, plans_fp4
    spec = plans_fp4.VariableGroupedFp4Spec(4, 3, 4, 128, 128, 6)
    assert spec.scale_capacity_rows() == (6 + 127 * 4) // 128 * 128 == 512
    assert spec.a_scale_bytes() == 4 * (128 // 64) * 512          # tests/cutlass/grouped/fp4.rs:47-48
    assert spec.b_scale_bytes() == 3 * (128 // 64) * 512
    with pytest.raises(plans.InvalidMatmulShape):
        plans_fp4.VariableGroupedFp4Spec(4, 3, 4, 128, 96, 6)      # k % 64
    with pytest.raises(plans.InvalidMatmulShape):
        plans_fp4.VariableGroupedFp4Spec(0, 3, 4, 128, 128, 6)


def test_indexed_grouped_fp4_spec():
    from mircuda_b200 import plans, plans_fp4
    spec = plans_fp4.IndexedGroupedFp4Spec(64, 33, 1, 128, 128)
    assert spec.inputs() == 64 and spec.with_broadcast_input().inputs() == 1
    with pytest.raises(plans.InvalidMatmulShape):
        plans_fp4.IndexedGroupedFp4Spec(64, 33, 1, 128, 100)


def test_dense_and_w4a16_specs():
    from mircuda_b200 import dense, plans
    assert dense.DenseMatmulSpec(2, 4, 3).output() == torch.bfloat16
    assert dense.DenseMatmulSpec(1, 128, 128, torch.bfloat16, torch.float32).output() == torch.float32
    with pytest.raises(plans.InvalidMatmulShape):
        dense.DenseMatmulSpec(1, 128, 128, torch.float32)
    with pytest.raises(plans.InvalidMatmulShape):
        dense.DenseMatmulSpec(1, 128, 128, torch.float16, torch.bfloat16)
    with pytest.raises(plans.InvalidMatmulShape):
        dense.W4A16Spec(1, 128, 100)
    with pytest.raises(plans.InvalidMatmulShape):
        dense.BlockwiseFp8VectorSpec(100, 128)
    assert dense.BlockwiseFp8VectorSpec(256, 512).weight_scale_elements() == 8


def test_quantize_int4_round_trip():
    """max|w| / 7 per 128 elements, zero point 8, even k in the low nibble."""
    from mircuda_b200 import dense
    generator = torch.Generator().manual_seed(3)
    weight = torch.randn(16, 256, generator=generator) * 0.02
    packed, scales = dense.quantize_int4(weight)
    assert packed.shape == (16, 128) and scales.shape == (16, 2) and scales.dtype == torch.float16
    codes = torch.stack([packed & 15, packed >> 4], dim=-1).reshape(16, 256).float()
    restored = (codes - 8.0) * scales.float().repeat_interleave(128, dim=1)
    step = scales.float().repeat_interleave(128, dim=1)
    assert ((restored - weight).abs() <= 0.5 * step + 1e-6).all()
    assert codes.max() <= 15 and codes.min() >= 1          # symmetric: -7..7 around 8
    zero_packed, zero_scales = dense.quantize_int4(torch.zeros(8, 128))
    assert (zero_packed == 0x88).all() and (zero_scales == 0).all()


def test_new_entry_points_validate_without_a_gpu(library):
    raw = ctypes.c_void_p()
    fake = ctypes.c_void_p(0x10)
    assert library.mircuda_variable_grouped_fp4_create(4, 3, 4, 128, 100, fake, ctypes.byref(raw)) == -1
    assert library.mircuda_grouped_fp4_create(4, 3, 4, 128, 128, False, None, ctypes.byref(raw)) == -1
    assert library.mircuda_dense_create(2, 2, 4, 4, 4, fake, ctypes.byref(raw)) == -1     # f32 inputs
    assert library.mircuda_dense_create(0, 1, 4, 4, 4, fake, ctypes.byref(raw)) == -1     # f16 -> bf16
    assert library.mircuda_b200_w4a16_create(1, 128, 100, fake, ctypes.byref(raw)) == -1
    assert library.mircuda_fp8_vector_create(100, 128, fake, ctypes.byref(raw)) == -1
    assert library.mircuda_b200_moe_swiglu_bf16(None, None, 1, None, 8, fake) == -1
    assert library.mircuda_b200_moe_expert_layout(None, 2, 0, 8, 1, None, None, None, None, 64, None, fake) == -1
    assert library.mircuda_b200_mxfp8_bf16_gathered(None, None, None, None, None, None, 1, 1, 1, 32, 1, fake) == -1
    assert library.mircuda_marlin_nvfp4_moe_execute(fake, None, None, None, None, None, None, None, None,
                                                    None, None, 1, False, 1, 64, 64, 0, None, False) == -1
    assert library.mircuda_scaled_fp8_create(1, 24, 16, 0, 0, 0, 0, fake, ctypes.byref(raw)) == -1   # n % 16
    assert library.mircuda_scaled_fp8_create(1, 16, 16, 2, 0, 0, 0, fake, ctypes.byref(raw)) == -1   # scale type
    assert library.mircuda_scaled_fp8_create(1, 16, 16, 0, 0, 0, 2, fake, ctypes.byref(raw)) == -1   # tile
    assert library.mircuda_scaled_fp8_workspace_bytes(None) == 0
    assert library.mircuda_dense_workspace_bytes(None) == 0
    assert library.mircuda_fp8_vector_workspace_bytes(None) == 0
    library.mircuda_variable_grouped_fp4_destroy(None)
    library.mircuda_grouped_fp4_destroy(None)
    library.mircuda_dense_destroy(None)
    library.mircuda_b200_w4a16_destroy(None)
    library.mircuda_fp8_vector_destroy(None)
    library.mircuda_scaled_fp8_destroy(None)


def test_scaled_fp8_spec_validation():
    import torch
    from mircuda_b200 import dense, plans
    spec = dense.ScaledFp8Spec(3, 32, 48, torch.bfloat16, "output_channel", True)
    assert spec.weight_scale_elements() == 48
    assert dense.ScaledFp8Spec(1, 16, 16).weight_scale_elements() == 1
    for bad in ((0, 16, 16), (1, 24, 16), (1, 16, 8)):
        with pytest.raises(plans.InvalidMatmulShape):
            dense.ScaledFp8Spec(*bad)
    with pytest.raises(plans.InvalidMatmulShape):
        dense.ScaledFp8Spec(1, 16, 16, torch.float16)
    with pytest.raises(plans.InvalidMatmulShape):
        dense.ScaledFp8Spec(1, 16, 16, torch.float32, "row")


def test_output_alignment_rule_of_the_gemm_plans():
    """The GEMM epilogues store 16-byte vectors when n % 8 == 0; an output that starts
    elsewhere (a sub-buffer of a pool) is refused on the host, as the C ABI refuses it (-1)."""
    from mircuda_b200 import plans
    pool = torch.zeros(64, dtype=torch.bfloat16)
    base = pool.data_ptr() % 16 // 2                 # elements past a 16-byte boundary
    aligned = pool[(8 - base) % 8:][:16]
    shifted = pool[(8 - base) % 8 + 1:][:16]
    plans._require_vector_output("C", 8, aligned)
    plans._require_vector_output("C", 12, shifted)   # scalar store path: no rule
    with pytest.raises(plans.MisalignedOperand):
        plans._require_vector_output("C", 8, shifted)


def test_blocked_quantizer_input_is_validated_on_the_host():
    """The blocked form of the activation quantizer takes [blocks, rows, columns / blocks]; shape
    errors and buffer lengths are reported before anything is launched."""
    from mircuda_b200 import plans

    class NoStream:
        cuda_stream = 0x10

    blocked = torch.zeros(4, 8, 64, dtype=torch.bfloat16)
    codes = torch.zeros(8 * 256, dtype=torch.uint8)
    scales = torch.zeros(plans.scale_bytes(8, 256 // 32), dtype=torch.uint8)
    with pytest.raises(plans.InvalidMatmulShape):
        plans.mxfp8_quantize_bf16(NoStream(), blocked, codes, scales, blocks=2)        # 4 blocks stored
    with pytest.raises(plans.InvalidMatmulShape):
        plans.mxfp8_quantize_bf16(NoStream(), torch.zeros(2, 8, 12, dtype=torch.bfloat16), codes, scales, blocks=2)
    with pytest.raises(plans.MatmulLengthMismatch):
        plans.mxfp8_quantize_bf16(NoStream(), blocked, codes[:-1], scales, blocks=4)
    with pytest.raises(ValueError):                                                    # not device memory
        plans.mxfp8_quantize_bf16(NoStream(), blocked, codes, scales, blocks=4)
