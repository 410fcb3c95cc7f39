"""CPU oracle for the quantized-matmul hot path — TEST INFRASTRUCTURE ONLY.

numpy-facing wrappers around ``mircuda_oracle.c`` (the C restatement of the reference's
kernel arithmetic; each C function cites the reference file:line it follows) plus, where a
reference checkout was available at build time, the reference's own functions compiled
from its sources (``oracle/_ref``).

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline / reference
legs may import this package. The product package ``mircuda_b200`` never does.

Pin status: codec, scale layout and MXFP8 quantizer are pinned against the reference's
host-compiled helpers and its tests' golden vectors; the NVFP4 quantizer is this repo's
own written spec ("parity unpinned").
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np

from . import build as _build

_u8p = ctypes.POINTER(ctypes.c_uint8)
_u16p = ctypes.POINTER(ctypes.c_uint16)
_u32p = ctypes.POINTER(ctypes.c_uint32)
_f32p = ctypes.POINTER(ctypes.c_float)

_lib = None
_ref_host = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(_build.build_oracle()))
        _lib.oracle_bf16_to_float.restype = ctypes.c_float
        _lib.oracle_bf16_to_float.argtypes = [ctypes.c_uint16]
        _lib.oracle_float_to_bf16.restype = ctypes.c_uint16
        _lib.oracle_float_to_bf16.argtypes = [ctypes.c_float]
        _lib.oracle_f16_to_float.restype = ctypes.c_float
        _lib.oracle_f16_to_float.argtypes = [ctypes.c_uint16]
        _lib.oracle_float_to_f16.restype = ctypes.c_uint16
        _lib.oracle_float_to_f16.argtypes = [ctypes.c_float]
        _lib.oracle_e4m3.restype = ctypes.c_float
        _lib.oracle_e4m3.argtypes = [ctypes.c_uint8]
        _lib.oracle_e8m0.restype = ctypes.c_float
        _lib.oracle_e8m0.argtypes = [ctypes.c_uint8]
        _lib.oracle_e2m1.restype = ctypes.c_float
        _lib.oracle_e2m1.argtypes = [ctypes.c_uint8]
        _lib.oracle_ue4m3.restype = ctypes.c_float
        _lib.oracle_ue4m3.argtypes = [ctypes.c_uint8]
        _lib.oracle_encode_e4m3.restype = ctypes.c_uint8
        _lib.oracle_encode_e4m3.argtypes = [ctypes.c_float]
        _lib.oracle_encode_ue4m3.restype = ctypes.c_uint8
        _lib.oracle_encode_ue4m3.argtypes = [ctypes.c_float]
        _lib.oracle_encode_e2m1.restype = ctypes.c_uint8
        _lib.oracle_encode_e2m1.argtypes = [ctypes.c_float]
        _lib.oracle_scale_offset.restype = ctypes.c_uint32
        _lib.oracle_scale_offset.argtypes = [ctypes.c_uint32] * 3
        _lib.oracle_fp4_scale_index.restype = ctypes.c_uint32
        _lib.oracle_fp4_scale_index.argtypes = [ctypes.c_uint32] * 3
        _lib.oracle_scale_bytes.restype = ctypes.c_size_t
        _lib.oracle_scale_bytes.argtypes = [ctypes.c_size_t] * 2
        _lib.oracle_threads.restype = ctypes.c_int
    return _lib


def ref_host() -> ctypes.CDLL | None:
    """The reference's own helper functions compiled for the host, or None if not built."""
    global _ref_host
    if _ref_host is None:
        path = _build.build_ref().get("host")
        if path is None:
            return None
        handle = ctypes.CDLL(str(path))
        handle.ref_bf16_to_float.restype = ctypes.c_float
        handle.ref_bf16_to_float.argtypes = [ctypes.c_uint16]
        handle.ref_float_to_bf16.restype = ctypes.c_uint16
        handle.ref_float_to_bf16.argtypes = [ctypes.c_float]
        handle.ref_e4m3.restype = ctypes.c_float
        handle.ref_e4m3.argtypes = [ctypes.c_uint8]
        handle.ref_e8m0.restype = ctypes.c_float
        handle.ref_e8m0.argtypes = [ctypes.c_uint8]
        handle.ref_encode_e4m3.restype = ctypes.c_uint8
        handle.ref_encode_e4m3.argtypes = [ctypes.c_float]
        handle.ref_scale_offset.restype = ctypes.c_uint32
        handle.ref_scale_offset.argtypes = [ctypes.c_uint32] * 4
        _ref_host = handle
    return _ref_host


def ref_library(name: str) -> Path | None:
    """Path of a prebuilt reference-derived library ('device' or 'vector'), if present."""
    return _build.build_ref().get(name)


def threads() -> int:
    return int(lib().oracle_threads())


def _ptr(array: np.ndarray, kind):
    assert array.flags["C_CONTIGUOUS"]
    return array.ctypes.data_as(kind)


def _c(array, dtype) -> np.ndarray:
    return np.ascontiguousarray(array, dtype=dtype)


# ----------------------------------------------------------------------------- conversions

def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    """kernels/mxfp8.cu:1-3."""
    return (_c(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(values: np.ndarray) -> np.ndarray:
    """kernels/mxfp8.cu:5-9 (nearest even by bias add; no NaN special case)."""
    bits = _c(values, np.float32).view(np.uint32).astype(np.uint64)
    bits = bits + 0x7FFF + ((bits >> 16) & 1)
    return ((bits >> 16) & 0xFFFF).astype(np.uint16)


def e4m3_table() -> np.ndarray:
    """All 256 decoded E4M3 values (kernels/mxfp8.cu:11-23)."""
    return np.array([lib().oracle_e4m3(code) for code in range(256)], dtype=np.float32)


def e2m1_table() -> np.ndarray:
    return np.array([lib().oracle_e2m1(code) for code in range(16)], dtype=np.float32)


def scale_bytes(rows: int, columns: int) -> int:
    """Padded size of a swizzled scale buffer (src/cutlass/mxfp8.rs:45-50)."""
    return int(lib().oracle_scale_bytes(rows, columns))


def scale_offsets(rows: int, columns: int) -> np.ndarray:
    """Byte offset of every (row, column) scale in the swizzled layout (kernels/mxfp8.cu:55-67)."""
    row = np.arange(rows, dtype=np.int64)[:, None]
    column = np.arange(columns, dtype=np.int64)[None, :]
    column_tiles = (columns + 3) // 4
    return ((((row // 128) * column_tiles + column // 4) * 32 + row % 32) * 4
            + (row % 128) // 32) * 4 + column % 4


# -------------------------------------------------------------------------------- MXFP8

def mxfp8_quantize(values_bf16: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """bf16 bits [rows, K] -> (codes [rows, K] u8, swizzled E8M0 scales) — kernels/mxfp8.cu:69-96."""
    values = _c(values_bf16, np.uint16)
    rows, columns = values.shape
    codes = np.zeros((rows, columns), dtype=np.uint8)
    scales = np.zeros(scale_bytes(rows, columns // 32), dtype=np.uint8)
    lib().oracle_mxfp8_quantize_bf16(_ptr(values, _u16p), _ptr(codes, _u8p), _ptr(scales, _u8p),
                                     ctypes.c_uint32(rows), ctypes.c_uint32(columns))
    return codes, scales


def swizzle_scales(scales_row_major: np.ndarray) -> np.ndarray:
    """kernels/mxfp8.cu:98-109."""
    source = _c(scales_row_major, np.uint8)
    rows, columns = source.shape
    output = np.zeros(scale_bytes(rows, columns), dtype=np.uint8)
    lib().oracle_swizzle_scales(_ptr(source, _u8p), _ptr(output, _u8p), ctypes.c_uint32(rows),
                                ctypes.c_uint32(columns))
    return output


def mxfp8_dequantize(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """codes [rows, K] + swizzled E8M0 -> fp32 [rows, K] (code * 2^(s-127))."""
    codes = _c(codes, np.uint8)
    rows, k = codes.shape
    offsets = scale_offsets(rows, k // 32)
    exponents = _c(scales, np.uint8)[offsets].astype(np.int32) - 127
    decoded = e4m3_table()[codes]
    return (decoded.reshape(rows, k // 32, 32) * np.ldexp(np.float32(1.0), exponents)[:, :, None]
            ).astype(np.float32).reshape(rows, k)


def mxfp8_gemm(a, a_scales, b, b_scales, use_c: bool = False) -> np.ndarray:
    """C = bf16(dequant(A) . dequant(B)^T), fp32 accumulation — sys/native/mxfp8_sm120.cu:17-48.

    ``use_c`` runs the C restatement end to end (slow; small shapes); otherwise the
    dequantised operands are multiplied with numpy's fp32 matmul.
    """
    a = _c(a, np.uint8)
    b = _c(b, np.uint8)
    m, k = a.shape
    n = b.shape[0]
    if use_c:
        output = np.zeros((m, n), dtype=np.uint16)
        status = lib().oracle_mxfp8_gemm(_ptr(a, _u8p), _ptr(_c(a_scales, np.uint8), _u8p),
                                         _ptr(b, _u8p), _ptr(_c(b_scales, np.uint8), _u8p),
                                         _ptr(output, _u16p), ctypes.c_uint32(m),
                                         ctypes.c_uint32(n), ctypes.c_uint32(k))
        assert status == 0
        return output
    product = mxfp8_dequantize(a, a_scales) @ mxfp8_dequantize(b, b_scales).T
    return f32_to_bf16(product)


def mxfp8_bf16_matmul(x_bf16, weight_words, scales_row_major) -> np.ndarray:
    """Weight-only MXFP8 (kernels/mxfp8.cu:111-153): bf16 bits [tokens, N]."""
    x = _c(x_bf16, np.uint16)
    words = _c(weight_words, np.uint32)
    scales = _c(scales_row_major, np.uint8)
    tokens, features = x.shape
    outputs = scales.shape[0]
    result = np.zeros((tokens, outputs), dtype=np.uint16)
    lib().oracle_mxfp8_bf16_matmul(_ptr(x, _u16p), _ptr(words, _u32p), _ptr(scales, _u8p),
                                   _ptr(result, _u16p), ctypes.c_uint32(tokens),
                                   ctypes.c_uint32(features), ctypes.c_uint32(outputs))
    return result


def mxfp8_bf16_gathered(x_bf16, weight_words, scales, bias, selected, matrices, rows, columns,
                        selections_per_input) -> np.ndarray:
    """kernels/mxfp8.cu:219-271."""
    x = _c(x_bf16, np.uint16)
    words = _c(weight_words, np.uint32)
    scales = _c(scales, np.uint8)
    selected = _c(selected, np.uint32)
    assignments = selected.shape[0]
    result = np.zeros((assignments, rows), dtype=np.uint16)
    has_bias = bias is not None
    bias_array = _c(bias if has_bias else np.zeros(1), np.uint16)
    lib().oracle_mxfp8_bf16_gathered(
        _ptr(x, _u16p), _ptr(words, _u32p), _ptr(scales, _u8p), _ptr(bias_array, _u16p),
        _ptr(selected, _u32p), _ptr(result, _u16p), ctypes.c_uint32(assignments),
        ctypes.c_uint32(matrices), ctypes.c_uint32(rows), ctypes.c_uint32(columns),
        ctypes.c_uint32(selections_per_input), ctypes.c_uint32(1 if has_bias else 0))
    return result


def mxfp8_embedding(weight_words, scales, selected, selected_start, tokens, vocab, hidden,
                    output_scale, output=None) -> np.ndarray:
    """kernels/mxfp8.cu:273-296."""
    words = _c(weight_words, np.uint32)
    scales = _c(scales, np.uint8)
    selected = _c(selected, np.uint32)
    result = np.zeros((tokens, hidden), dtype=np.uint16) if output is None else output
    lib().oracle_mxfp8_embedding_bf16(
        _ptr(words, _u32p), _ptr(scales, _u8p), _ptr(selected, _u32p), _ptr(result, _u16p),
        ctypes.c_uint32(selected_start), ctypes.c_uint32(tokens), ctypes.c_uint32(vocab),
        ctypes.c_uint32(hidden), ctypes.c_float(output_scale))
    return result


# -------------------------------------------------------------------------------- NVFP4

def fp4_scale_offsets(rows: int, k: int) -> np.ndarray:
    """sys/native/fp4_vector_sm120.cu:32-39 for every (row, 16-wide block)."""
    row = np.arange(rows, dtype=np.int64)[:, None]
    column = np.arange(k // 16, dtype=np.int64)[None, :]
    blocks_k = k // 64
    return (((row >> 7) * blocks_k) << 9) + ((row & 31) << 4) + (((row & 127) >> 5) << 2) \
        + ((column >> 2) << 9) + (column & 3)


def fp4_scale_bytes(rows: int, k: int) -> int:
    """tests/cutlass/fp4/mod.rs:35-37: ceil(rows/128) * (K/64) * 512."""
    return ((rows + 127) // 128) * (k // 64) * 512


def nvfp4_dequantize(codes: np.ndarray, scales: np.ndarray, k: int) -> np.ndarray:
    """packed codes [rows, K/2] + swizzled UE4M3 per 16 -> fp32 [rows, K] (no global scale)."""
    codes = _c(codes, np.uint8)
    rows = codes.shape[0]
    nibbles = np.empty((rows, k), dtype=np.uint8)
    nibbles[:, 0::2] = codes & 0xF
    nibbles[:, 1::2] = codes >> 4
    values = e2m1_table()[nibbles]
    decoded_scales = e4m3_table()[_c(scales, np.uint8)[fp4_scale_offsets(rows, k)] & 0x7F]
    return (values.reshape(rows, k // 16, 16) * decoded_scales[:, :, None]).reshape(rows, k)


def nvfp4_quantize(values_bf16: np.ndarray, global_scale: float | None = None
                   ) -> tuple[np.ndarray, np.ndarray, float]:
    """bf16 bits [rows, K] -> (packed codes, swizzled UE4M3 scales, global). Parity unpinned.
    With `global_scale` given, the tensor scale is that value instead of amax / (448 * 6)."""
    values = _c(values_bf16, np.uint16)
    rows, k = values.shape
    codes = np.zeros((rows, k // 2), dtype=np.uint8)
    scales = np.zeros(fp4_scale_bytes(rows, k), dtype=np.uint8)
    if global_scale is not None:
        lib().oracle_nvfp4_quantize_bf16_scaled(_ptr(values, _u16p), _ptr(codes, _u8p),
                                                _ptr(scales, _u8p), ctypes.c_float(global_scale),
                                                ctypes.c_uint32(rows), ctypes.c_uint32(k))
        return codes, scales, float(np.float32(global_scale))
    global_scale = ctypes.c_float(0.0)
    lib().oracle_nvfp4_quantize_bf16(_ptr(values, _u16p), _ptr(codes, _u8p), _ptr(scales, _u8p),
                                     ctypes.byref(global_scale), ctypes.c_uint32(rows),
                                     ctypes.c_uint32(k))
    return codes, scales, float(global_scale.value)


def fp4_vector(x_codes, x_scales, w_codes, w_scales, n: int, k: int, alpha: float) -> np.ndarray:
    """FP4 x FP4 GEMV, M = 1 (sys/native/fp4_vector_sm120.cu:85-125): bf16 bits [n]."""
    output = np.zeros(n, dtype=np.uint16)
    lib().oracle_fp4_vector(_ptr(_c(x_codes, np.uint8), _u8p), _ptr(_c(x_scales, np.uint8), _u8p),
                            _ptr(_c(w_codes, np.uint8), _u8p), _ptr(_c(w_scales, np.uint8), _u8p),
                            _ptr(output, _u16p), ctypes.c_uint32(n), ctypes.c_uint32(k),
                            ctypes.c_float(alpha))
    return output


def nvfp4_gemv_bf16(x_bf16, w_codes, w_scales, n: int, k: int, global_scale: float,
                    use_c: bool = False) -> np.ndarray:
    """bf16 activations [M, K] x NVFP4 weights -> bf16 bits [M, n]."""
    x = _c(x_bf16, np.uint16)
    m = x.shape[0]
    if use_c:
        output = np.zeros((m, n), dtype=np.uint16)
        lib().oracle_nvfp4_gemv_bf16(_ptr(x, _u16p), _ptr(_c(w_codes, np.uint8), _u8p),
                                     _ptr(_c(w_scales, np.uint8), _u8p), _ptr(output, _u16p),
                                     ctypes.c_uint32(m), ctypes.c_uint32(n), ctypes.c_uint32(k),
                                     ctypes.c_float(global_scale))
        return output
    weights = nvfp4_dequantize(np.asarray(w_codes).reshape(n, k // 2), w_scales, k)
    product = (bf16_to_f32(x) @ weights.T) * np.float32(global_scale)
    return f32_to_bf16(product.astype(np.float32))


# ------------------------------------------------------------------ int4-g128 W4A16
# No reference entry point executes this format; the numerics restated here are the ones the
# reference's (unused) int4 dequantiser defines, sys/native/marlin/vendor/dequant.h:107-216:
# unsigned 4-bit codes with the symmetric zero point 8 folded in, weight = (q - 8) * scale, f16
# group scales, one per 128 K-elements. Parity unpinned: no reference test or kernel runs it.

INT4_GROUP = 128


def int4_g128_quantize(weights_f32: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """fp32 [n, k] -> (packed codes u8 [n, k/2], even k in the low nibble; f16 scales [n, k/128]),
    scale = max|w| / 7 per group rounded to f16, code = clamp(rne(w / scale) + 8, 0, 15)."""
    weights = np.asarray(weights_f32, dtype=np.float32)
    n, k = weights.shape
    groups = weights.reshape(n, k // INT4_GROUP, INT4_GROUP)
    scales = (np.max(np.abs(groups), axis=-1) / np.float32(7.0)).astype(np.float16)
    safe = np.where(scales == 0, np.float16(1.0), scales).astype(np.float32)
    codes = np.clip(np.rint(groups / safe[..., None]) + 8, 0, 15).astype(np.uint8).reshape(n, k)
    packed = np.ascontiguousarray(codes[:, 0::2] | (codes[:, 1::2] << 4))
    return packed, np.ascontiguousarray(scales)


def int4_g128_dequantize(packed: np.ndarray, scales_f16: np.ndarray) -> np.ndarray:
    """(q - 8) * scale as fp32 [n, k]; exact (a 4-bit integer times an f16 fits fp32)."""
    packed = _c(packed, np.uint8)
    n = packed.shape[0]
    codes = np.empty((n, packed.shape[1] * 2), dtype=np.float32)
    codes[:, 0::2] = packed & 0xF
    codes[:, 1::2] = packed >> 4
    scales = np.asarray(scales_f16, dtype=np.float16).astype(np.float32)
    return ((codes - np.float32(8.0)).reshape(n, -1, INT4_GROUP) * scales[:, :, None]).reshape(n, -1)


def w4a16_int4(x_f16: np.ndarray, packed: np.ndarray, scales_f16: np.ndarray) -> np.ndarray:
    """f16 activations [m, k] x int4-g128 weights [n, k] -> f16 [m, n], fp32 accumulation."""
    x = np.asarray(x_f16, dtype=np.float16).astype(np.float32)
    return (x @ int4_g128_dequantize(packed, scales_f16).T).astype(np.float16)


# ------------------------------------------------------------------ dense GEMV and grouped

def dense_vector(data_type: int, x, weight, y, n: int, k: int, alpha: float, beta: float):
    """sys/native/dense_vector_sm120.cu:50-132; ``y`` is updated in place and returned."""
    output = _c(y, np.uint16).copy()
    lib().oracle_dense_vector(ctypes.c_int(data_type), _ptr(_c(x, np.uint16), _u16p),
                              _ptr(_c(weight, np.uint16), _u16p), _ptr(output, _u16p),
                              ctypes.c_uint32(n), ctypes.c_uint32(k), ctypes.c_float(alpha),
                              ctypes.c_float(beta))
    return output


def variable_grouped_bf16(a, weights, rows, offsets, c, max_rows: int, n: int, k: int,
                          beta: float, use_c: bool = False) -> np.ndarray:
    """sys/native/variable_grouped_bf16_sm120.cu:18-33; returns the updated copy of ``c``."""
    a = _c(a, np.uint16)
    weights = _c(weights, np.uint16)
    rows = _c(rows, np.uint32)
    offsets = _c(offsets, np.uint32)
    output = _c(c, np.uint16).copy()
    groups = rows.shape[0]
    if use_c:
        lib().oracle_variable_grouped_bf16(
            _ptr(a, _u16p), _ptr(weights, _u16p), _ptr(rows, _u32p), _ptr(offsets, _u32p),
            _ptr(output, _u16p), ctypes.c_uint32(groups), ctypes.c_uint32(max_rows),
            ctypes.c_uint32(n), ctypes.c_uint32(k), ctypes.c_float(beta))
        return output
    a_f = bf16_to_f32(a).reshape(-1, k)
    out_view = output.reshape(-1, n)
    for group in range(groups):
        count = min(int(rows[group]), max_rows)
        if count == 0:
            continue
        start = int(offsets[group])
        w = bf16_to_f32(weights.reshape(groups, n, k)[group])
        product = a_f[start:start + count] @ w.T
        if beta != 0.0:
            product = product + np.float32(beta) * bf16_to_f32(out_view[start:start + count])
        out_view[start:start + count] = f32_to_bf16(product.astype(np.float32))
    return output


# ------------------------------------------------------------------------------- metrics

def variable_grouped_fp4(a, a_scales, b, b_scales, alphas, indices, rows, offsets, scale_offsets,
                         c_bits, matrices: int, max_rows: int, n: int, k: int) -> np.ndarray:
    """Variable-row grouped NVFP4 product (sys/native/variable_grouped_fp4_sm120.cu:31-62 for
    the operand addressing; the arithmetic is CUTLASS's block-scaled MMA: exact E2M1 x UE4M3
    products, fp32 accumulation, alpha, bf16 round). `c_bits` [capacity, n] is returned with
    each group's rows replaced; a group whose index is out of range leaves its rows alone."""
    a = _c(a, np.uint8).reshape(-1, k // 2)
    b = _c(b, np.uint8).reshape(matrices, n, k // 2)
    a_scales = _c(a_scales, np.uint8)
    b_scales = _c(b_scales, np.uint8).reshape(matrices, -1)
    output = np.array(c_bits, dtype=np.uint16).reshape(-1, n).copy()
    atom_row_bytes = (k // 64) * 512
    for group in range(len(indices)):
        matrix = int(indices[group])
        if matrix >= matrices:
            continue
        count = min(int(rows[group]), max_rows)
        if count == 0:
            continue
        first = int(offsets[group])
        scale_begin = (int(scale_offsets[group]) // 128) * atom_row_bytes
        group_scales = a_scales[scale_begin:scale_begin + fp4_scale_bytes(count, k)]
        left = nvfp4_dequantize(a[first:first + count], group_scales, k)
        right = nvfp4_dequantize(b[matrix], b_scales[matrix], k)
        product = (left @ right.T).astype(np.float32) * np.float32(alphas[matrix])
        output[first:first + count] = f32_to_bf16(product.astype(np.float32))
    return output


def indexed_grouped_fp4(a, a_scales, b, b_scales, alphas, selected, c_bits, experts: int, m: int,
                        n: int, k: int, broadcast_input: bool) -> np.ndarray:
    """Fixed-m grouped NVFP4 product (sys/native/grouped_fp4_sm120.cu:29-57): group g reads
    input group g (0 when broadcast), matrix selected[g], writes C rows [g*m, g*m + m)."""
    groups = len(selected)
    stride_rows = (m + 127) // 128 * 128
    inputs = 1 if broadcast_input else groups
    source = np.arange(groups) * 0 if broadcast_input else np.arange(groups)
    padded = np.zeros((groups * m, k // 2), dtype=np.uint8)
    a = _c(a, np.uint8).reshape(inputs, m, k // 2)
    for group in range(groups):
        padded[group * m:(group + 1) * m] = a[source[group]]
    # Re-express as the variable problem: A rows copied per group, scales addressed per input.
    output = np.array(c_bits, dtype=np.uint16).reshape(groups * m, n).copy()
    a_scales = _c(a_scales, np.uint8).reshape(inputs, -1)
    b = _c(b, np.uint8).reshape(experts, n, k // 2)
    b_scales = _c(b_scales, np.uint8).reshape(experts, -1)
    for group in range(groups):
        expert = int(selected[group])
        if expert >= experts:
            continue
        left = nvfp4_dequantize(padded[group * m:(group + 1) * m], a_scales[source[group]], k)
        right = nvfp4_dequantize(b[expert], b_scales[expert], k)
        product = (left @ right.T).astype(np.float32) * np.float32(alphas[expert])
        output[group * m:(group + 1) * m] = f32_to_bf16(product.astype(np.float32))
    del stride_rows
    return output


def scaled_fp8(x_codes, w_codes, input_scales, weight_scales, bias_bits, m: int, n: int,
               k: int) -> np.ndarray:
    """FP8 matmul with epilogue scales (sys/native/scaled_fp8_sm120.cuh:21-50): the fp32
    accumulator is multiplied by the weight scale (one value, or one per output channel; fp32
    or bf16 already widened to fp32 by the caller) and rounded to fp32, then multiplied by the
    token's fp32 scale and, with a bias, added to the bf16 bias in one fused multiply-add,
    and rounded to bf16. Returns bf16 bits [m, n]."""
    table = e4m3_table().astype(np.float64)
    x = table[_c(x_codes, np.uint8).reshape(m, k)]
    w = table[_c(w_codes, np.uint8).reshape(n, k)]
    accumulator = (x @ w.T).astype(np.float32)
    channel = np.broadcast_to(_c(weight_scales, np.float32).reshape(1, -1), (1, n))
    scaled = (channel * accumulator).astype(np.float32)
    tokens = _c(input_scales, np.float32).reshape(m, 1).astype(np.float64)
    result = tokens * scaled.astype(np.float64)          # exact in f64: two 24-bit factors
    if bias_bits is not None:
        result = result + bf16_to_f32(bias_bits).reshape(1, n).astype(np.float64)
    return f32_to_bf16(result.astype(np.float32))


def compare_bf16(actual_bits, expected_bits) -> dict:
    """max|d|/max|ref| and relative Frobenius error between two bf16 bit arrays."""
    actual = bf16_to_f32(np.asarray(actual_bits).reshape(-1)).astype(np.float64)
    expected = bf16_to_f32(np.asarray(expected_bits).reshape(-1)).astype(np.float64)
    scale = max(float(np.max(np.abs(expected))), 1e-30)
    delta = actual - expected
    return {
        "max_rel_to_max": float(np.max(np.abs(delta)) / scale),
        "rel_frobenius": float(np.linalg.norm(delta) / max(np.linalg.norm(expected), 1e-30)),
    }
