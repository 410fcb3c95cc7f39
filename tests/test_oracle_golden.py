"""Pins the CPU oracle: against the reference's own helper functions compiled for the
host (oracle/_ref, built from the reference checkout) and against the constant-valued
golden vectors of the reference's tests. No GPU needed."""
import numpy as np
import pytest

import oracle


def bf16(value: float) -> int:
    return int(oracle.f32_to_bf16(np.array([value], dtype=np.float32))[0])


def test_codec_matches_reference_helpers_exhaustively():
    ref = oracle.ref_host()
    if ref is None:
        pytest.skip("reference checkout not available at build time")
    lib = oracle.lib()
    for code in range(256):
        a, b = lib.oracle_e4m3(code), ref.ref_e4m3(code)
        assert (np.isnan(a) and np.isnan(b)) or a == b
        a, b = lib.oracle_e8m0(code), ref.ref_e8m0(code)
        assert (np.isnan(a) and np.isnan(b)) or a == b
    # Every finite bf16 value, at the scalings a 32-block can apply (powers of two).
    bits = np.arange(65536, dtype=np.uint16)
    values = oracle.bf16_to_f32(bits)
    finite = values[np.isfinite(values)]
    rng = np.random.default_rng(7)
    samples = np.concatenate([
        finite[np.abs(finite) < 1024.0],
        (rng.standard_normal(20000) * 100).astype(np.float32),
        np.array([448.0, 447.99, 464.0, 1e9, -1e9, 0.015625, 0.0156, 2.0 ** -10, 2.0 ** -9,
                  0.0009765, 0.00097, -0.0, 0.0], dtype=np.float32),
    ])
    for value in samples.tolist():
        assert lib.oracle_encode_e4m3(value) == ref.ref_encode_e4m3(value), value
    floats = rng.standard_normal(50000).astype(np.float32) * np.float32(3.0)
    ours = oracle.f32_to_bf16(floats)
    for index in range(0, floats.size, 7):
        assert int(ours[index]) == ref.ref_float_to_bf16(float(floats[index]))
        assert lib.oracle_float_to_bf16(float(floats[index])) == int(ours[index])
    for bit in range(0, 65536, 13):
        a, b = lib.oracle_bf16_to_float(bit), ref.ref_bf16_to_float(bit)
        assert (np.isnan(a) and np.isnan(b)) or a == b


def test_scale_offset_matches_reference_and_vector_index():
    ref = oracle.ref_host()
    lib = oracle.lib()
    rows, columns = 300, 24
    table = oracle.scale_offsets(rows, columns)
    for row in range(0, rows, 7):
        for column in range(columns):
            ours = lib.oracle_scale_offset(row, column, columns)
            assert ours == table[row, column]
            if ref is not None:
                assert ours == ref.ref_scale_offset(row, column, rows, columns)
            # sys/native/fp4_vector_sm120.cu:32-39 is the same layout for K = 16 * columns.
            if columns % 4 == 0:
                assert ours == lib.oracle_fp4_scale_index(row, column, columns * 16)
    assert sorted(oracle.scale_offsets(256, 8).reshape(-1).tolist()) == list(range(256 * 8))


def test_quantizer_golden_ones():
    """tests/mxfp8/quantize.rs:18-46 — 32 x 1.0 -> codes 0x78, scale byte 119 at offset 0."""
    codes, scales = oracle.mxfp8_quantize(np.full((1, 32), bf16(1.0), dtype=np.uint16))
    assert codes.tolist() == [[0x78] * 32]
    assert scales.size == 512 and scales[0] == 119 and not scales[1:].any()


def test_quantizer_edge_cases():
    row = np.zeros((4, 64), dtype=np.uint16)
    row[0, :32] = bf16(0.0)                       # all-zero block -> scale byte 0, codes 0
    row[0, 32:] = bf16(-0.0)                      # negative zero keeps its sign bit
    row[1, :32] = bf16(448.0)                     # amax / 448 is exactly 1 -> 127, code 0x7e
    row[1, 32:] = bf16(449.0)                     # bf16(449) = 448 as well
    row[2, :] = bf16(1e-40)                       # subnormal input -> clamped exponent 0
    row[3, :32] = bf16(3.0e38)                    # near bf16 max
    row[3, 32] = bf16(1.75)
    row[3, 33] = bf16(-0.4375)
    codes, scales = oracle.mxfp8_quantize(row)
    offsets = oracle.scale_offsets(4, 2)
    assert scales[offsets[0, 0]] == 0 and not codes[0, :32].any()
    assert (codes[0, 32:] == 0x80).all()
    assert scales[offsets[1, 0]] == 127 and (codes[1, :32] == 0x7E).all()
    assert scales[offsets[2, 0]] == 0
    assert scales[offsets[3, 0]] == 247 and (codes[3, :32] == 0x76).all()  # 3e38 / 2^120 = 225.7 -> 224
    # amax 1.75 = 448 * 2^-8 exactly -> exponent 119; 1.75/2^-8 = 448 -> 0x7e; -0.4375 -> -112 -> 0xee
    assert scales[offsets[3, 1]] == 119 and codes[3, 32] == 0x7E and codes[3, 33] == 0xEE


def test_weight_only_golden():
    """tests/mxfp8/matmul.rs:7-33 — tokens 1..5, weights 1.0 / -0.5 with scales 1 / 2 -> +-32 t."""
    x = np.repeat(np.array([bf16(float(t)) for t in range(1, 6)], dtype=np.uint16), 32).reshape(5, 32)
    words = np.array([0x38383838] * 8 + [0xB0B0B0B0] * 8, dtype=np.uint32).reshape(2, 8)
    scales = np.array([[127], [128]], dtype=np.uint8)
    result = oracle.mxfp8_bf16_matmul(x, words, scales)
    expected = [[bf16(32.0 * t), bf16(-32.0 * t)] for t in range(1, 6)]
    assert result.tolist() == expected


def test_tensor_core_golden_ones():
    """tests/mxfp8/matmul.rs:35-63 — quantized ones [4,128] x weights 1.0 [128,128] -> 128."""
    codes, a_scales = oracle.mxfp8_quantize(np.full((4, 128), bf16(1.0), dtype=np.uint16))
    weight = np.full((128, 128), 0x38, dtype=np.uint8)
    b_scales = oracle.swizzle_scales(np.full((128, 4), 127, dtype=np.uint8))
    for use_c in (True, False):
        result = oracle.mxfp8_gemm(codes, a_scales, weight, b_scales, use_c=use_c)
        assert (result == bf16(128.0)).all()


def test_gathered_golden():
    """tests/mxfp8/gathered.rs:5-69."""
    x = np.full((1, 32), bf16(1.0), dtype=np.uint16)
    words = np.array([0x38383838] * 8 + [0xB0B0B0B0] * 8 + [0x38383838] * 8 + [0xB0B0B0B0] * 8,
                     dtype=np.uint32)
    scales = np.array([127, 127, 128, 128], dtype=np.uint8)
    selected = np.array([1, 0], dtype=np.uint32)
    bias = np.array([bf16(v) for v in (1.0, 2.0, 3.0, 4.0)], dtype=np.uint16)
    plain = oracle.mxfp8_bf16_gathered(x, words, scales, None, selected, 2, 2, 32, 2)
    assert plain.reshape(-1).tolist() == [bf16(v) for v in (64.0, -32.0, 32.0, -16.0)]
    biased = oracle.mxfp8_bf16_gathered(x, words, scales, bias, selected, 2, 2, 32, 2)
    assert biased.reshape(-1).tolist() == [bf16(v) for v in (67.0, -28.0, 33.0, -14.0)]
    out_of_range = oracle.mxfp8_bf16_gathered(x, words, scales, None,
                                              np.array([5, 0], dtype=np.uint32), 2, 2, 32, 2)
    assert out_of_range[0].tolist() == [0, 0]


def test_embedding_golden():
    """tests/mxfp8/quantize.rs:48-79 — rows selected [1, 0] -> -1.0 then 1.0."""
    words = np.array([0x38383838] * 8 + [0xB0B0B0B0] * 8, dtype=np.uint32)
    scales = np.array([127, 128], dtype=np.uint8)
    result = oracle.mxfp8_embedding(words, scales, np.array([1, 0], dtype=np.uint32), 0, 2, 2, 32, 1.0)
    assert (result[0] == bf16(-1.0)).all() and (result[1] == bf16(1.0)).all()


def test_fp4_vector_golden():
    """tests/cutlass/fp4/vector.rs:11-30 — 0x22 codes, 0x38 scales, N=704, K=2816 -> 2816.0."""
    n, k = 704, 2816
    x = np.full(k // 2, 0x22, dtype=np.uint8)
    xs = np.full(oracle.fp4_scale_bytes(1, k), 0x38, dtype=np.uint8)
    w = np.full(n * k // 2, 0x22, dtype=np.uint8)
    ws = np.full(oracle.fp4_scale_bytes(n, k), 0x38, dtype=np.uint8)
    assert xs.size == 1 * k // 64 * 512 and ws.size == 6 * k // 64 * 512
    result = oracle.fp4_vector(x, xs, w, ws, n, k, 1.0)
    assert (result == bf16(2816.0)).all()
    half = oracle.fp4_vector(x, xs, w, ws, n, k, 0.5)
    assert (half == bf16(1408.0)).all()
    dequantized = oracle.nvfp4_dequantize(w.reshape(n, k // 2), ws, k)
    assert (dequantized == 1.0).all()


def test_grouped_bf16_golden():
    """tests/cutlass/grouped/bf16.rs:12-36 — rows [3,0,2,1], offsets [0,3,3,5], NaN-prefilled C."""
    n = k = 128
    a = np.full((6, k), bf16(1.0), dtype=np.uint16)
    weights = np.concatenate([np.full((n * k,), bf16(float(e + 1)), dtype=np.uint16) for e in range(4)])
    rows = np.array([3, 0, 2, 1], dtype=np.uint32)
    offsets = np.array([0, 3, 3, 5], dtype=np.uint32)
    c = np.full((6, n), 0x7FC0, dtype=np.uint16)
    for use_c in (True, False):
        result = oracle.variable_grouped_bf16(a, weights, rows, offsets, c, 4, n, k, 0.0, use_c=use_c)
        expected = [128.0, 128.0, 128.0, 384.0, 384.0, 512.0]
        for row, value in enumerate(expected):
            assert (result.reshape(6, n)[row] == bf16(value)).all(), row


def test_dense_vector_matches_numpy():
    rng = np.random.default_rng(3)
    n, k = 37, 264
    x = oracle.f32_to_bf16(rng.standard_normal(k).astype(np.float32))
    w = oracle.f32_to_bf16((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    y = oracle.f32_to_bf16(rng.standard_normal(n).astype(np.float32))
    result = oracle.dense_vector(1, x, w, y, n, k, 1.5, 0.25)
    expected = 1.5 * (oracle.bf16_to_f32(w) @ oracle.bf16_to_f32(x)) + 0.25 * oracle.bf16_to_f32(y)
    assert np.allclose(oracle.bf16_to_f32(result), expected, rtol=1e-2, atol=1e-3)
    # f16 path: exact small integers
    ones = np.full(k, 0x3C00, dtype=np.uint16)
    result = oracle.dense_vector(0, ones, np.full((n, k), 0x3C00, dtype=np.uint16),
                                 np.zeros(n, dtype=np.uint16), n, k, 1.0, 0.0)
    assert (result == 0x5C20).all()  # 264.0 in f16


def test_nvfp4_quantizer_spec_round_trip():
    """The NVFP4 quantizer is this repo's own spec (parity unpinned): check its invariants."""
    rng = np.random.default_rng(11)
    values = oracle.f32_to_bf16((rng.standard_normal((8, 128)) * 0.02).astype(np.float32))
    codes, scales, global_scale = oracle.nvfp4_quantize(values)
    original = oracle.bf16_to_f32(values)
    assert np.isclose(global_scale, np.abs(original).max() / 2688.0)
    restored = oracle.nvfp4_dequantize(codes, scales, 128) * global_scale
    block_max = np.abs(original).reshape(8, 8, 16).max(axis=2, keepdims=True)
    error = np.abs(restored - original).reshape(8, 8, 16)
    assert (error <= block_max * 0.26 + 1e-12).all()      # half an E2M1 step of the largest value
    ones = np.full((1, 64), bf16(1.0), dtype=np.uint16)
    codes, scales, global_scale = oracle.nvfp4_quantize(ones)
    assert np.isclose(global_scale, 1.0 / 2688.0)
    assert (codes == 0x77).all() and scales[oracle.fp4_scale_offsets(1, 64)].tolist() == [[0x7E] * 4]


def test_variable_grouped_fp4_golden_rows():
    """tests/cutlass/grouped/fp4.rs:38-87: both executions of the reference's variable-row test."""
    n = k = 128
    weights = np.full((3, n, k // 2), 0x22, np.uint8)
    weights[0] = 0
    bank_scales = np.full(3 * oracle.fp4_scale_bytes(n, k), 0x38, np.uint8)
    a = np.full((6, k // 2), 0x22, np.uint8)
    a_scales = np.full(4 * (k // 64) * 512, 0x38, np.uint8)
    ones = np.full((6, n), 0x3F80, np.uint16)
    first = oracle.variable_grouped_fp4(a, a_scales, weights, bank_scales, [1.0, 0.5, 0.25], [1, 0, 2, 1],
                                        [3, 0, 2, 1], [0, 3, 3, 5], [0, 128, 128, 256], ones, 3, 4, n, k)
    assert oracle.bf16_to_f32(first)[:, 0].tolist() == [64.0, 64.0, 64.0, 32.0, 32.0, 64.0]
    second = oracle.variable_grouped_fp4(a, a_scales, weights, bank_scales, [1.0, 0.5, 0.25],
                                         [1, 0, 2, 1], [0, 1, 1, 4], [0, 0, 1, 2], [0, 0, 128, 256],
                                         first, 3, 4, n, k)
    assert oracle.bf16_to_f32(second)[:, 0].tolist() == [0.0, 32.0, 64.0, 64.0, 64.0, 64.0]
    assert (second == second[:, :1]).all()


def test_indexed_grouped_fp4_golden_rows():
    """tests/cutlass/grouped/fp4.rs:173-217 with broadcast input (run_case(2, 2, true))."""
    n = k = 128
    matrices = 33
    weights = np.full((matrices, n, k // 2), 0x22, np.uint8)
    weights[0] = 0
    bank_scales = np.full(matrices * oracle.fp4_scale_bytes(n, k), 0x38, np.uint8)
    alphas = [0.5 if matrix % 2 == 0 else 1.0 for matrix in range(matrices)]
    a = np.full((2, k // 2), 0x22, np.uint8)
    a_scales = np.full(oracle.fp4_scale_bytes(2, k), 0x38, np.uint8)
    out = oracle.indexed_grouped_fp4(a, a_scales, weights, bank_scales, alphas, [0, 1],
                                     np.full((4, n), 0x3F80, np.uint16), matrices, 2, n, k, True)
    assert oracle.bf16_to_f32(out)[:, 0].tolist() == [0.0, 0.0, 128.0, 128.0]


def test_scaled_fp8_golden():
    """per_token_and_channel_scales_with_bias and per_token_and_tensor_scale
    (tests/cutlass/scaled_fp8.rs:9-71): ones, token scale 0.5, channel scales j/16 and bias 1
    -> 8 * j/16 + 1; tensor scale 0.25 -> 2."""
    ones_x = np.full(16, 0x38, dtype=np.uint8)
    ones_w = np.full(256, 0x38, dtype=np.uint8)
    channel = np.arange(1, 17, dtype=np.float32) / 16.0
    bias = oracle.f32_to_bf16(np.ones(16, dtype=np.float32))
    out = oracle.scaled_fp8(ones_x, ones_w, [0.5], channel, bias, 1, 16, 16)
    expected = oracle.f32_to_bf16((8.0 * channel + 1.0).astype(np.float32))
    assert (out.reshape(-1) == expected).all()
    out = oracle.scaled_fp8(ones_x, ones_w, [0.5], [0.25], None, 1, 16, 16)
    assert (oracle.bf16_to_f32(out) == 2.0).all()


def test_int4_g128_known_answers():
    """int4 with symmetric zero point 8 (sys/native/marlin/vendor/dequant.h:107-216: the
    dequantiser subtracts 8, weight = (q - 8) * scale): a group whose largest magnitude is 7
    gets scale 1 and codes value + 8, packed with the even k in the low nibble; the product is
    the plain dot product of the dequantised weights."""
    values = np.tile(np.arange(-7, 8, dtype=np.float32), 9)[:128]
    weights = np.stack([values, -values * 0.5])
    packed, scales = oracle.int4_g128_quantize(weights)
    assert scales.dtype == np.float16 and scales.tolist() == [[1.0], [0.5]]
    assert packed[0, 0] == ((-7 + 8) | ((-6 + 8) << 4)) and packed[0, 7] == (15 | (1 << 4))
    assert np.array_equal(oracle.int4_g128_dequantize(packed, scales), weights)
    x = np.arange(128, dtype=np.float32).astype(np.float16).reshape(1, 128) / 64
    out = oracle.w4a16_int4(x, packed, scales)
    expected = (x.astype(np.float32) @ weights.T).astype(np.float16)
    assert np.array_equal(out, expected)
    zero_packed, zero_scales = oracle.int4_g128_quantize(np.zeros((1, 128), np.float32))
    assert zero_scales[0, 0] == 0 and (zero_packed == 0x88).all()
