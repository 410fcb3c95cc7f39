"""GPU parity: MXFP8 quantizer (bit-exact) and block-scaled GEMM (tolerance) through the C ABI."""
import ctypes
import os

import numpy as np
import pytest
import torch

import oracle
from helpers import assert_close_bf16, bf16_bits, from_bf16_bits, seeded_bf16, u8

pytestmark = pytest.mark.gpu


def quantize_on_gpu(stream, values: torch.Tensor):
    from mircuda_b200 import plans
    rows, columns = values.shape
    codes = torch.empty(rows * columns, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(plans.scale_bytes(rows, columns // 32), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    plans.mxfp8_quantize_bf16(stream, values, codes, scales)
    stream.synchronize()
    return codes.cpu().numpy().reshape(rows, columns), scales.cpu().numpy()


def reference_quantize_on_gpu(stream, values: torch.Tensor):
    """The reference's own kernel (built from its source into oracle/_ref), reference geometry."""
    path = oracle.ref_library("device")
    if path is None:
        return None
    library = ctypes.CDLL(str(path))
    rows, columns = values.shape
    from mircuda_b200 import plans
    codes = torch.empty(rows * columns, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(plans.scale_bytes(rows, columns // 32), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    status = library.ref_mxfp8_quantize_bf16(
        ctypes.c_void_p(values.data_ptr()), ctypes.c_void_p(codes.data_ptr()),
        ctypes.c_void_p(scales.data_ptr()), ctypes.c_uint32(rows), ctypes.c_uint32(columns),
        ctypes.c_void_p(stream.cuda_stream))
    assert status == 0
    stream.synchronize()
    return codes.cpu().numpy().reshape(rows, columns), scales.cpu().numpy()


def test_quantizer_golden_ones(cuda_stream):
    """tests/mxfp8/quantize.rs:18-46."""
    codes, scales = quantize_on_gpu(cuda_stream, torch.ones(1, 32, dtype=torch.bfloat16, device="cuda"))
    assert (codes == 0x78).all()
    assert scales[0] == 119 and not scales[1:].any()


@pytest.mark.parametrize("shape", [(128, 1024), (4, 128), (77, 96), (1, 32), (300, 4096), (5, 160)])
def test_quantizer_bit_exact_random(cuda_stream, shape):
    values = seeded_bf16(shape, 1.0, 1000 + shape[0])
    codes, scales = quantize_on_gpu(cuda_stream, values)
    expected_codes, expected_scales = oracle.mxfp8_quantize(bf16_bits(values))
    assert np.array_equal(codes, expected_codes)
    assert np.array_equal(scales, expected_scales)
    reference = reference_quantize_on_gpu(cuda_stream, values)
    if reference is not None:
        assert np.array_equal(codes, reference[0])
        assert np.array_equal(scales, reference[1])


@pytest.mark.parametrize("shape,blocks", [((128, 1024), 8), ((300, 4096), 4), ((77, 96), 2), ((5, 160), 5),
                                          ((64, 768), 3)])
def test_quantizer_blocked_input(cuda_stream, shape, blocks):
    """Column blocks stored one after another (the layout an all-gather of column shards leaves)
    give the codes and scales of the row-major matrix, bit for bit."""
    from mircuda_b200 import plans
    rows, columns = shape
    values = seeded_bf16(shape, 1.0, 1700 + rows)
    blocked = values.view(rows, blocks, columns // blocks).permute(1, 0, 2).contiguous()
    codes = torch.empty(rows * columns, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(plans.scale_bytes(rows, columns // 32), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    plans.mxfp8_quantize_bf16(cuda_stream, blocked, codes, scales, blocks=blocks)
    cuda_stream.synchronize()
    expected_codes, expected_scales = oracle.mxfp8_quantize(bf16_bits(values))
    assert np.array_equal(codes.cpu().numpy().reshape(rows, columns), expected_codes)
    assert np.array_equal(scales.cpu().numpy(), expected_scales)


def test_quantizer_bit_exact_every_finite_bf16(cuda_stream):
    """Every finite bf16 value as the block maximum and as a non-maximal element.

    Row r holds value bits r in column 0 (plus smaller companions) so that each bf16 pattern
    sets a block scale; a second block of the same row holds the pattern next to a fixed
    larger maximum so that each pattern is also encoded under foreign scales.
    """
    bits = np.arange(65536, dtype=np.uint16)
    finite = bits[(bits & 0x7F80) != 0x7F80]
    rows = finite.size
    data = np.zeros((rows, 128), dtype=np.uint16)
    data[:, 0] = finite
    data[:, 1] = finite & 0x7FFF                       # same magnitude, positive
    data[:, 2] = (finite & 0x7F80) | 0x0040            # same binade, different mantissa
    for block, maximum in enumerate((1.0, 3.0e-3, 5.0e4), start=1):
        data[:, 32 * block] = oracle.f32_to_bf16(np.float32(maximum))
        data[:, 32 * block + 1] = finite
        # keep the fixed value the maximum: clear entries that would exceed it
        too_big = np.abs(oracle.bf16_to_f32(finite)) > maximum
        data[too_big, 32 * block + 1] = 0
    values = from_bf16_bits(data)
    codes, scales = quantize_on_gpu(cuda_stream, values)
    expected_codes, expected_scales = oracle.mxfp8_quantize(data)
    assert np.array_equal(scales, expected_scales)
    assert np.array_equal(codes, expected_codes)
    reference = reference_quantize_on_gpu(cuda_stream, values)
    if reference is not None:
        assert np.array_equal(scales, reference[1])
        assert np.array_equal(codes, reference[0])


def test_swizzle_scales(cuda_stream):
    from mircuda_b200 import plans
    rng = np.random.default_rng(5)
    source = rng.integers(0, 255, size=(300, 24), dtype=np.uint8)
    device_source = u8(source)
    output = torch.zeros(plans.scale_bytes(300, 24), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    plans.mxfp8_swizzle_scales(cuda_stream, device_source, output)
    cuda_stream.synchronize()
    assert np.array_equal(output.cpu().numpy(), oracle.swizzle_scales(source))


def run_gemm(stream, a_codes, a_scales, b_codes, b_scales, m, n, k):
    from mircuda_b200 import plans
    plan = plans.BlockScaledMxFp8Plan(stream, plans.BlockScaledMxFp8Spec(m, n, k))
    a, sa, b, sb = u8(a_codes), u8(a_scales), u8(b_codes), u8(b_scales)
    output = torch.full((m * n,), float("nan"), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    plan.execute(stream, a, sa, b, sb, output)
    stream.synchronize()
    plan.close()
    return bf16_bits(output).reshape(m, n)


def test_tensor_core_golden_ones(cuda_stream):
    """tests/mxfp8/matmul.rs:35-63 — ones [4,128] (device-quantized) x 1.0 [128,128] -> 128."""
    from mircuda_b200 import plans
    spec = plans.MxFp8Spec(4, 128, 128)
    operation = plans.MxFp8TensorCore(cuda_stream, spec)
    x = torch.ones(4 * 128, dtype=torch.bfloat16, device="cuda")
    weight = torch.full((128 * 128,), 0x38, dtype=torch.uint8, device="cuda")
    scales = torch.full((128 * 4,), 127, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    swizzled = operation.swizzle_weight_scales(cuda_stream, scales)
    output = torch.zeros(4 * 128, dtype=torch.bfloat16, device="cuda")
    cuda_stream.synchronize()
    operation.execute(cuda_stream, x, weight, swizzled, output)
    cuda_stream.synchronize()
    assert (output.float() == 128.0).all()


@pytest.mark.parametrize("block_n", ["128", "192", "256"])
@pytest.mark.parametrize("m,n,k", [(128, 1024, 1024), (4, 128, 128), (200, 328, 256), (129, 704, 384)])
def test_gemm_matches_oracle(cuda_stream, monkeypatch, m, n, k, block_n):
    """BASELINE config 1 (128x1024x1024) and ragged shapes, every tile width."""
    monkeypatch.setenv("MIRCUDA_B200_GEMM_BN", block_n)
    a = seeded_bf16((m, k), 1.0, 1000)
    b = seeded_bf16((n, k), 1.0, 1001)
    a_codes, a_scales = oracle.mxfp8_quantize(bf16_bits(a))
    b_codes, b_scales = oracle.mxfp8_quantize(bf16_bits(b))
    expected = oracle.mxfp8_gemm(a_codes, a_scales, b_codes, b_scales)
    actual = run_gemm(cuda_stream, a_codes, a_scales, b_codes, b_scales, m, n, k)
    assert not np.isnan(oracle.bf16_to_f32(actual)).any()
    assert_close_bf16(actual, expected, f"{m}x{n}x{k} bn={block_n}")


def test_gemm_uses_block_scales(cuda_stream):
    """Exact small-integer case where every K-block carries a different power-of-two scale."""
    m, n, k = 128, 256, 512
    rng = np.random.default_rng(9)
    a_codes = np.full((m, k), 0x38, dtype=np.uint8)            # 1.0
    b_codes = np.full((n, k), 0x38, dtype=np.uint8)
    a_exp = rng.integers(124, 130, size=(m, k // 32)).astype(np.uint8)
    b_exp = rng.integers(124, 130, size=(n, k // 32)).astype(np.uint8)
    a_scales, b_scales = oracle.swizzle_scales(a_exp), oracle.swizzle_scales(b_exp)
    expected = oracle.mxfp8_gemm(a_codes, a_scales, b_codes, b_scales)
    actual = run_gemm(cuda_stream, a_codes, a_scales, b_codes, b_scales, m, n, k)
    assert np.array_equal(actual, expected)


def test_gemm_rejects_other_stream_and_bad_lengths(cuda_stream):
    from mircuda_b200 import plans
    plan = plans.BlockScaledMxFp8Plan(cuda_stream, plans.BlockScaledMxFp8Spec(128, 128, 128))
    good = torch.zeros(128 * 128, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(512, dtype=torch.uint8, device="cuda")
    out = torch.zeros(128 * 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(plans.StreamMismatch):
        plan.execute(torch.cuda.Stream(), good, scales, good, scales, out)
    with pytest.raises(plans.MatmulLengthMismatch):
        plan.execute(cuda_stream, good[:100], scales, good, scales, out)
    other = torch.cuda.Stream()
    status = plan._lib.mircuda_mxfp8_tc_execute(
        plan._raw, ctypes.c_void_p(other.cuda_stream), ctypes.c_void_p(good.data_ptr()),
        ctypes.c_void_p(scales.data_ptr()), ctypes.c_void_p(good.data_ptr()),
        ctypes.c_void_p(scales.data_ptr()), ctypes.c_void_p(out.data_ptr()))
    assert status == -1                                        # sys/native/mxfp8_sm120.cu:146
    plan.close()


@pytest.mark.parametrize("name,n,k", [("qkv", 6144, 4096), ("o", 4096, 4096),
                                      ("gate_up", 24576, 4096), ("down", 4096, 12288)])
def test_prefill_shape_rows_against_oracle(cuda_stream, name, n, k):
    """The four Qwen3-8B prefill linears at M = 4096 (the shapes the throughput is quoted on),
    activations quantized on the device as src/mxfp8/tensor_core.rs:127-162 does, checked on
    output rows taken from the first, a middle and the last 256-row tile against the oracle.
    Whole rows are compared, so every column tile (first to last) of those rows is covered;
    each output row depends on one A row only."""
    from mircuda_b200 import plans
    m = 4096
    x = seeded_bf16((m, k), 1.0, 2000)
    w = seeded_bf16((n, k), 0.02, 2001)
    spec = plans.MxFp8Spec(m, k, n)
    operation = plans.MxFp8TensorCore(cuda_stream, spec)
    w_codes = torch.empty(n * k, dtype=torch.uint8, device="cuda")
    w_scales = torch.zeros(plans.scale_bytes(n, k // 32), dtype=torch.uint8, device="cuda")
    output = torch.zeros(m * n, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    plans.mxfp8_quantize_bf16(cuda_stream, w, w_codes, w_scales)
    operation.execute(cuda_stream, x.view(-1), w_codes, w_scales, output)
    cuda_stream.synchronize()
    rows = np.array([0, 1, 127, 128, 255, 2047, 2048, 2177, 3840, 3967, 3968, 4095])
    a_codes, a_scales = oracle.mxfp8_quantize(bf16_bits(x)[rows])
    # quantization is per row block, so quantizing the sampled rows alone gives the same codes
    device_codes = operation.scratch.quantized_input.view(m, k)[torch.from_numpy(rows).cuda()].cpu().numpy()
    assert np.array_equal(device_codes, a_codes)
    b_dequantized = oracle.mxfp8_dequantize(w_codes.cpu().numpy().reshape(n, k), w_scales.cpu().numpy())
    expected = oracle.f32_to_bf16(oracle.mxfp8_dequantize(a_codes, a_scales) @ b_dequantized.T)
    actual = bf16_bits(output).reshape(m, n)[rows]
    assert_close_bf16(actual, expected, f"prefill {name} rows")


def test_gemm_refuses_an_output_that_cannot_take_vector_stores(cuda_stream):
    """n % 8 == 0 selects 16-byte stores in the epilogue: an output that is only 2-byte aligned
    gets status -1 from the C ABI instead of a misaligned-address fault, and the host mirror
    names the operand."""
    from mircuda_b200 import plans
    plan = plans.BlockScaledMxFp8Plan(cuda_stream, plans.BlockScaledMxFp8Spec(128, 128, 128))
    codes = torch.zeros(128 * 128, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(512, dtype=torch.uint8, device="cuda")
    pool = torch.zeros(128 * 128 + 8, dtype=torch.bfloat16, device="cuda")
    shifted = pool[1:1 + 128 * 128]
    with pytest.raises(plans.MisalignedOperand):
        plan.execute(cuda_stream, codes, scales, codes, scales, shifted)
    pointer = lambda tensor: ctypes.c_void_p(tensor.data_ptr())
    status = plan._lib.mircuda_mxfp8_tc_execute(
        plan._raw, ctypes.c_void_p(cuda_stream.cuda_stream), pointer(codes), pointer(scales),
        pointer(codes), pointer(scales), pointer(shifted))
    assert status == -1
    plan.close()


def test_a_wait_that_runs_out_reports_minus_three(cuda_stream):
    """Failure path of the bounded waits: a kernel waits (2 ms budget) on a barrier nothing
    arrives at, gives up by itself and raises the plan's status word; the context stays usable,
    the plan's next execute answers -3 and other plans keep working."""
    import time
    from mircuda_b200 import plans
    plan = plans.BlockScaledMxFp8Plan(cuda_stream, plans.BlockScaledMxFp8Spec(128, 128, 128))
    codes = torch.full((128 * 128,), 0x38, dtype=torch.uint8, device="cuda")
    scales = torch.full((512,), 127, dtype=torch.uint8, device="cuda")
    out = torch.zeros(128 * 128, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    plan.execute(cuda_stream, codes, scales, codes, scales, out)      # healthy first
    cuda_stream.synchronize()
    assert (out.float() == 128.0).all()
    begin = time.perf_counter()
    assert plan._lib.mircuda_b200_mxfp8_tc_wait_probe(plan._raw, ctypes.c_void_p(cuda_stream.cuda_stream)) == 0
    cuda_stream.synchronize()                                          # the kernel returned by itself
    assert time.perf_counter() - begin < 5.0
    with pytest.raises(plans.NativeError) as failure:
        plan.execute(cuda_stream, codes, scales, codes, scales, out)
    assert failure.value.status == -3
    plan.close()
    healthy = plans.BlockScaledMxFp8Plan(cuda_stream, plans.BlockScaledMxFp8Spec(128, 128, 128))
    out.zero_()
    torch.cuda.synchronize()
    healthy.execute(cuda_stream, codes, scales, codes, scales, out)
    cuda_stream.synchronize()
    assert (out.float() == 128.0).all()
    healthy.close()
