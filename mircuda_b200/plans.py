"""Host-side mirror of the reference's Spec / Plan interface for the quantized-matmul path.

The reference's host layer is Rust (``src/cutlass/*.rs``, ``src/mxfp8/*.rs``); no Rust
toolchain exists where this is built, so the same classes, argument meaning and error
behaviour are provided here over the C ABI (``include/mircuda_b200.h``) with torch tensors
as device buffers. PyTorch only supplies device memory and streams. Every class cites the
reference type it mirrors. Errors mirror the reference's enum as exceptions:

* ``InvalidMatmulShape``    — ``Error::InvalidMatmulShape`` (spec constructors)
* ``MatmulLengthMismatch``  — ``Error::MatmulLengthMismatch`` (buffer length checks)
* ``StreamMismatch``        — ``Error::StreamMismatch`` (plan used on another stream)
* ``NativeError``           — ``Error::Cutlass(i32)`` (non-zero status from the C ABI)
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib


class InvalidMatmulShape(ValueError):
    pass


class MatmulLengthMismatch(ValueError):
    def __init__(self, operand: str, expected: int, actual: int):
        super().__init__(f"{operand}: expected {expected} elements, got {actual}")
        self.operand, self.expected, self.actual = operand, expected, actual


class StreamMismatch(RuntimeError):
    pass


class MisalignedOperand(ValueError):
    """An operand's address does not allow the 16-byte accesses the kernel makes (the C ABI
    answers -1 for it; the host mirror names the operand instead)."""


class NativeError(RuntimeError):
    def __init__(self, status: int):
        super().__init__(f"native call failed with status {status}")
        self.status = status


def _check(status: int) -> None:
    if status != 0:
        raise NativeError(int(status))


def _exact(operand: str, expected: int, tensor: torch.Tensor) -> None:
    if tensor.numel() != expected:
        raise MatmulLengthMismatch(operand, expected, tensor.numel())


def _require_vector_output(operand: str, n: int, tensor: torch.Tensor) -> None:
    """With n a multiple of 8 the GEMM epilogues store 16-byte vectors, so the output must
    start on a 16-byte boundary (a sub-buffer of a pool might not)."""
    if n % 8 == 0 and tensor.data_ptr() % 16 != 0:
        raise MisalignedOperand(f"{operand} must be 16-byte aligned when n % 8 == 0")


def _device_pointer(tensor: torch.Tensor, dtypes) -> ctypes.c_void_p:
    if not tensor.is_cuda or not tensor.is_contiguous():
        raise ValueError("operands must be contiguous CUDA tensors")
    if tensor.dtype not in dtypes:
        raise TypeError(f"expected one of {dtypes}, got {tensor.dtype}")
    return ctypes.c_void_p(tensor.data_ptr())


def _stream_handle(stream: torch.cuda.Stream) -> ctypes.c_void_p:
    if stream.cuda_stream == 0:
        raise ValueError("the null stream is not accepted; create a torch.cuda.Stream()")
    return ctypes.c_void_p(stream.cuda_stream)


_BYTES = (torch.uint8, torch.int8)
_WORDS = (torch.uint8, torch.int32, torch.uint32)
_BF16 = (torch.bfloat16,)


def scale_bytes(rows: int, columns: int) -> int:
    """Padded bytes of the 128x4-swizzled scale layout (src/cutlass/mxfp8.rs:45-50)."""
    return (rows + 127) // 128 * 128 * ((columns + 3) // 4 * 4)


# ------------------------------------------------------------------------------ MXFP8

@dataclass(frozen=True)
class BlockScaledMxFp8Spec:
    """``BlockScaledMxFp8Spec`` (src/cutlass/mxfp8.rs:4-57): E4M3[M,K] x E4M3[N,K]^T -> BF16[M,N]."""
    m: int
    n: int
    k: int

    def __post_init__(self):
        if self.m <= 0 or self.n <= 0 or self.k <= 0 or self.k % 128 != 0:
            raise InvalidMatmulShape(f"invalid MXFP8 shape {self.m}x{self.n}x{self.k}")
        if max(self.m, self.n, self.k) > 2**31 - 1:
            raise InvalidMatmulShape("dimension does not fit i32")

    def scale_bytes(self, rows: int) -> int:
        return scale_bytes(rows, self.k // 32)


class BlockScaledMxFp8Plan:
    """``BlockScaledMxFp8Plan`` (src/cutlass/mxfp8.rs:59-106) over ``mircuda_mxfp8_tc_*``."""

    def __init__(self, stream: torch.cuda.Stream, spec: BlockScaledMxFp8Spec):
        self._lib = _lib.load()
        self.spec = spec
        self._stream = stream
        raw = ctypes.c_void_p()
        _check(self._lib.mircuda_mxfp8_tc_create(spec.m, spec.n, spec.k, _stream_handle(stream),
                                                 ctypes.byref(raw)))
        self._raw = raw

    def workspace_bytes(self) -> int:
        return int(self._lib.mircuda_mxfp8_tc_workspace_bytes(self._raw))

    def execute(self, stream, a, a_scales, b, b_scales, output) -> None:
        if stream.cuda_stream != self._stream.cuda_stream:
            raise StreamMismatch()
        s = self.spec
        _exact("A", s.m * s.k, a)
        _exact("A scales", s.scale_bytes(s.m), a_scales)
        if b.dtype in (torch.int32, torch.uint32):
            _exact("B", s.n * s.k // 4, b)
        else:
            _exact("B", s.n * s.k, b)
        _exact("B scales", s.scale_bytes(s.n), b_scales)
        _exact("C", s.m * s.n, output)
        _require_vector_output("C", s.n, output)
        _check(self._lib.mircuda_mxfp8_tc_execute(
            self._raw, _stream_handle(stream), _device_pointer(a, _BYTES),
            _device_pointer(a_scales, _BYTES), _device_pointer(b, _WORDS),
            _device_pointer(b_scales, _BYTES), _device_pointer(output, _BF16)))

    def close(self) -> None:
        if getattr(self, "_raw", None):
            self._lib.mircuda_mxfp8_tc_destroy(self._raw)
            self._raw = None

    __del__ = close


def mxfp8_quantize_bf16(stream, values, codes, scales, blocks: int = 1) -> None:
    """Launch of the activation quantizer (src/mxfp8/tensor_core.rs:140-158).

    ``values`` bf16 [rows, columns]; ``codes`` u8 [rows, columns]; ``scales`` a zero-filled
    u8 buffer of ``scale_bytes(rows, columns // 32)``. With ``blocks`` > 1 ``values`` is
    [blocks, rows, columns // blocks]: the column blocks of the matrix one after another, as an
    all-gather of column shards leaves them; the outputs are those of the row-major matrix.
    """
    if blocks > 1:
        stored_blocks, rows, block_columns = values.shape
        if stored_blocks != blocks or block_columns % 8 != 0:
            raise InvalidMatmulShape("blocked input must be [blocks, rows, columns / blocks] with 8-column pieces")
        columns = blocks * block_columns
    else:
        rows, columns = values.shape
    if columns % 32 != 0:
        raise InvalidMatmulShape("columns must be a multiple of 32")
    _exact("MXFP8 codes", rows * columns, codes)
    _exact("MXFP8 scales", scale_bytes(rows, columns // 32), scales)
    library = _lib.load()
    if blocks > 1:
        _check(library.mircuda_b200_mxfp8_quantize_bf16_blocks(
            _device_pointer(values, _BF16), _device_pointer(codes, _BYTES),
            _device_pointer(scales, _BYTES), rows, columns, columns // blocks, _stream_handle(stream)))
        return
    _check(library.mircuda_b200_mxfp8_quantize_bf16(
        _device_pointer(values, _BF16), _device_pointer(codes, _BYTES),
        _device_pointer(scales, _BYTES), rows, columns, _stream_handle(stream)))


def mxfp8_swizzle_scales(stream, scales_row_major, output) -> None:
    """``swizzle_weight_scales`` (src/mxfp8/tensor_core.rs:89-107); ``output`` zero-filled."""
    rows, columns = scales_row_major.shape
    _exact("swizzled MXFP8 weight scales", scale_bytes(rows, columns), output)
    _check(_lib.load().mircuda_b200_mxfp8_swizzle_scales(
        _device_pointer(scales_row_major, _BYTES), _device_pointer(output, _BYTES), rows, columns,
        _stream_handle(stream)))


@dataclass(frozen=True)
class MxFp8Spec:
    """``MxFp8Spec`` (src/mxfp8/matmul.rs): tokens x input_features -> output_features."""
    tokens: int
    input_features: int
    output_features: int

    def __post_init__(self):
        if (self.tokens <= 0 or self.input_features <= 0 or self.output_features <= 0
                or self.input_features % 32 != 0):
            raise InvalidMatmulShape("invalid MXFP8 geometry")

    def weight_words(self) -> int:
        return self.output_features * self.input_features // 4

    def scale_elements(self) -> int:
        return self.output_features * self.input_features // 32


class MxFp8Matmul:
    """``MxFp8Matmul`` (src/mxfp8/matmul.rs:92-159): weight-only MXFP8, bf16 activations."""

    def __init__(self, spec: MxFp8Spec):
        self._lib = _lib.load()
        self.spec = spec

    def execute(self, stream, input, weight, scales, output) -> None:
        s = self.spec
        _exact("MXFP8 input", s.tokens * s.input_features, input)
        if weight.dtype in (torch.int32, torch.uint32):
            _exact("MXFP8 weight", s.weight_words(), weight)
        else:
            _exact("MXFP8 weight", s.weight_words() * 4, weight)
        _exact("MXFP8 scales", s.scale_elements(), scales)
        _exact("MXFP8 output", s.tokens * s.output_features, output)
        _check(self._lib.mircuda_b200_mxfp8_bf16(
            _device_pointer(input, _BF16), _device_pointer(weight, _WORDS),
            _device_pointer(scales, _BYTES), _device_pointer(output, _BF16), s.tokens,
            s.input_features, s.output_features, _stream_handle(stream)))


class MxFp8TensorCoreScratch:
    """``MxFp8TensorCoreScratch`` (src/mxfp8/tensor_core.rs:165-197): codes + scales for (M, K)."""

    def __init__(self, spec: MxFp8Spec, device=None):
        self.tokens, self.input_features = spec.tokens, spec.input_features
        self.quantized_input = torch.empty(spec.tokens * spec.input_features, dtype=torch.uint8,
                                           device=device or "cuda")
        self.input_scales = torch.zeros(scale_bytes(spec.tokens, spec.input_features // 32),
                                        dtype=torch.uint8, device=device or "cuda")

    def validate(self, spec: MxFp8Spec) -> None:
        if self.tokens != spec.tokens or self.input_features != spec.input_features:
            raise InvalidMatmulShape("scratch geometry does not match")


class MxFp8TensorCore:
    """``MxFp8TensorCore`` (src/mxfp8/tensor_core.rs:33-162): quantize bf16 activations on the
    device, then run the block-scaled GEMM against MXFP8 weights."""

    def __init__(self, stream: torch.cuda.Stream, spec: MxFp8Spec,
                 scratch: MxFp8TensorCoreScratch | None = None):
        self.spec = spec
        with torch.cuda.stream(stream):
            self.scratch = scratch or MxFp8TensorCoreScratch(spec)
        self.scratch.validate(spec)
        self.plan = BlockScaledMxFp8Plan(
            stream, BlockScaledMxFp8Spec(spec.tokens, spec.output_features, spec.input_features))

    def swizzle_weight_scales(self, stream, scales: torch.Tensor) -> torch.Tensor:
        rows, columns = self.spec.output_features, self.spec.input_features // 32
        _exact("MXFP8 weight scales", rows * columns, scales)
        with torch.cuda.stream(stream):
            output = torch.zeros(self.plan.spec.scale_bytes(rows), dtype=torch.uint8,
                                 device=scales.device)
        mxfp8_swizzle_scales(stream, scales.view(rows, columns), output)
        return output

    def workspace_bytes(self) -> int:
        return self.plan.workspace_bytes()

    def execute(self, stream, input, weight, weight_scales, output) -> None:
        s = self.spec
        _exact("MXFP8 input", s.tokens * s.input_features, input)
        _exact("MXFP8 output", s.tokens * s.output_features, output)
        mxfp8_quantize_bf16(stream, input.view(s.tokens, s.input_features),
                            self.scratch.quantized_input, self.scratch.input_scales)
        self.plan.execute(stream, self.scratch.quantized_input, self.scratch.input_scales, weight,
                          weight_scales, output)


# ------------------------------------------------------------------------------ GEMV

@dataclass(frozen=True)
class BlockScaledFp4VectorSpec:
    """``BlockScaledFp4VectorSpec`` (src/cutlass/fp4/vector.rs:3-40)."""
    n: int
    k: int

    def __post_init__(self):
        if self.n <= 0 or self.k <= 0 or self.k % 64 != 0:
            raise InvalidMatmulShape("invalid FP4 vector shape")

    def scale_bytes(self, rows: int) -> int:
        return (rows + 127) // 128 * (self.k // 64) * 512


class BlockScaledFp4VectorPlan:
    """``BlockScaledFp4VectorPlan`` (src/cutlass/fp4/vector.rs:42-93) over ``mircuda_fp4_vector_*``."""

    def __init__(self, stream, spec: BlockScaledFp4VectorSpec):
        self._lib = _lib.load()
        self.spec, self._stream = spec, stream
        raw = ctypes.c_void_p()
        _check(self._lib.mircuda_fp4_vector_create(spec.n, spec.k, _stream_handle(stream),
                                                   ctypes.byref(raw)))
        self._raw = raw

    def execute(self, stream, input, input_scales, weight, weight_scales, output, alpha: float):
        if stream.cuda_stream != self._stream.cuda_stream:
            raise StreamMismatch()
        s = self.spec
        _exact("input", s.k // 2, input)
        _exact("input scales", s.scale_bytes(1), input_scales)
        _exact("weight", s.n * s.k // 2, weight)
        _exact("weight scales", s.scale_bytes(s.n), weight_scales)
        _exact("output", s.n, output)
        _check(self._lib.mircuda_fp4_vector_execute(
            self._raw, _stream_handle(stream), _device_pointer(input, _BYTES),
            _device_pointer(input_scales, _BYTES), _device_pointer(weight, _BYTES),
            _device_pointer(weight_scales, _BYTES), _device_pointer(output, _BF16), float(alpha)))

    def close(self):
        if getattr(self, "_raw", None):
            self._lib.mircuda_fp4_vector_destroy(self._raw)
            self._raw = None

    __del__ = close


@dataclass(frozen=True)
class DenseVectorSpec:
    """``DenseVectorSpec`` (src/cutlass/vector.rs): data_type 0 = f16, 1 = bf16."""
    n: int
    k: int
    data_type: int = 1

    def __post_init__(self):
        if self.n <= 0 or self.k <= 0 or self.data_type not in (0, 1):
            raise InvalidMatmulShape("invalid dense vector shape")


class DenseVectorPlan:
    """``DenseVectorPlan<T>`` (src/cutlass/vector.rs:41-86) over ``mircuda_dense_vector_*``."""

    def __init__(self, stream, spec: DenseVectorSpec):
        self._lib = _lib.load()
        self.spec, self._stream = spec, stream
        raw = ctypes.c_void_p()
        _check(self._lib.mircuda_dense_vector_create(spec.data_type, spec.n, spec.k,
                                                     _stream_handle(stream), ctypes.byref(raw)))
        self._raw = raw

    def execute(self, stream, input, weight, output, alpha: float = 1.0, beta: float = 0.0):
        if stream.cuda_stream != self._stream.cuda_stream:
            raise StreamMismatch()
        s = self.spec
        dtypes = (torch.bfloat16,) if s.data_type == 1 else (torch.float16,)
        _exact("input", s.k, input)
        _exact("weight", s.n * s.k, weight)
        _exact("output", s.n, output)
        _check(self._lib.mircuda_dense_vector_execute(
            self._raw, _stream_handle(stream), _device_pointer(input, dtypes),
            _device_pointer(weight, dtypes), _device_pointer(output, dtypes), float(alpha),
            float(beta)))

    def close(self):
        if getattr(self, "_raw", None):
            self._lib.mircuda_dense_vector_destroy(self._raw)
            self._raw = None

    __del__ = close


@dataclass(frozen=True)
class NvFp4VectorSpec:
    """bf16 activations [m <= 8, k] x NVFP4 weights [n, k] (no reference counterpart)."""
    m: int
    n: int
    k: int

    def __post_init__(self):
        if not (1 <= self.m <= 8) or self.n <= 0 or self.k <= 0 or self.k % 64 != 0:
            raise InvalidMatmulShape("invalid NVFP4 vector shape")

    def scale_bytes(self) -> int:
        return (self.n + 127) // 128 * (self.k // 64) * 512


class NvFp4VectorPlan:
    """Decode GEMV / skinny GEMM over ``mircuda_b200_nvfp4_vector_*``."""

    def __init__(self, stream, spec: NvFp4VectorSpec):
        self._lib = _lib.load()
        self.spec, self._stream = spec, stream
        raw = ctypes.c_void_p()
        _check(self._lib.mircuda_b200_nvfp4_vector_create(spec.m, spec.n, spec.k,
                                                          _stream_handle(stream), ctypes.byref(raw)))
        self._raw = raw

    def execute(self, stream, input, weight, weight_scales, output, global_scale: float):
        if stream.cuda_stream != self._stream.cuda_stream:
            raise StreamMismatch()
        s = self.spec
        _exact("input", s.m * s.k, input)
        _exact("weight", s.n * s.k // 2, weight)
        _exact("weight scales", s.scale_bytes(), weight_scales)
        _exact("output", s.m * s.n, output)
        _check(self._lib.mircuda_b200_nvfp4_vector_execute(
            self._raw, _stream_handle(stream), _device_pointer(input, _BF16),
            _device_pointer(weight, _BYTES), _device_pointer(weight_scales, _BYTES),
            _device_pointer(output, _BF16), float(global_scale)))

    def close(self):
        if getattr(self, "_raw", None):
            self._lib.mircuda_b200_nvfp4_vector_destroy(self._raw)
            self._raw = None

    __del__ = close


def nvfp4_quantize_bf16(stream, values: torch.Tensor):
    """bf16 [rows, k] -> (codes u8 [rows, k/2], swizzled UE4M3 scales, device float global)."""
    rows, k = values.shape
    if k % 64 != 0:
        raise InvalidMatmulShape("k must be a multiple of 64")
    library = _lib.load()
    with torch.cuda.stream(stream):
        codes = torch.empty(rows * k // 2, dtype=torch.uint8, device=values.device)
        scales = torch.zeros((rows + 127) // 128 * (k // 64) * 512, dtype=torch.uint8,
                             device=values.device)
        global_scale = torch.zeros(1, dtype=torch.float32, device=values.device)
    handle = _stream_handle(stream)
    _check(library.mircuda_b200_nvfp4_global_scale(_device_pointer(values, _BF16), rows * k,
                                                   ctypes.c_void_p(global_scale.data_ptr()), handle))
    _check(library.mircuda_b200_nvfp4_quantize_bf16(
        _device_pointer(values, _BF16), ctypes.c_void_p(global_scale.data_ptr()),
        _device_pointer(codes, _BYTES), _device_pointer(scales, _BYTES), rows, k, handle))
    return codes.view(rows, k // 2), scales, global_scale


# --------------------------------------------------------------------------- grouped MoE

@dataclass(frozen=True)
class VariableGroupedBf16Spec:
    """``VariableGroupedBf16Spec`` (src/cutlass/variable_grouped/bf16.rs:4-81)."""
    groups: int
    max_rows: int
    n: int
    k: int
    capacity_rows: int
    # Not in the reference: size of a weight bank the groups index into (expert-parallel MoE
    # has one group per (source GPU, local expert)); None = one matrix per group.
    matrices: int | None = None

    def __post_init__(self):
        values = (self.groups, self.max_rows, self.n, self.k, self.capacity_rows,
                  self.matrices if self.matrices is not None else 1)
        if any(v <= 0 for v in values) or self.n % 8 != 0 or self.k % 8 != 0:
            raise InvalidMatmulShape("invalid grouped bf16 shape")
        if max(values) > 2**32 - 1:
            raise InvalidMatmulShape("dimension does not fit u32")


class VariableGroupedBf16Plan:
    """``VariableGroupedBf16Plan`` (src/cutlass/variable_grouped/bf16.rs:83-124): all products
    are enqueued without the host ever reading ``rows`` / ``offsets``."""

    def __init__(self, stream, spec: VariableGroupedBf16Spec):
        self._lib = _lib.load()
        self.spec, self._stream = spec, stream
        raw = ctypes.c_void_p()
        if spec.matrices is None:
            _check(self._lib.mircuda_variable_grouped_bf16_create(
                spec.groups, spec.max_rows, spec.n, spec.k, _stream_handle(stream),
                ctypes.byref(raw)))
        else:
            _check(self._lib.mircuda_b200_variable_grouped_bf16_create_indexed(
                spec.groups, spec.matrices, spec.max_rows, spec.n, spec.k, _stream_handle(stream),
                ctypes.byref(raw)))
        self._raw = raw

    def execute(self, stream, input, weights, rows, offsets, output, beta: float = 0.0,
                indices=None):
        if stream.cuda_stream != self._stream.cuda_stream:
            raise StreamMismatch()
        s = self.spec
        _exact("input", s.capacity_rows * s.k, input)
        _exact("weights", (s.matrices or s.groups) * s.n * s.k, weights)
        _exact("rows", s.groups, rows)
        _exact("offsets", s.groups, offsets)
        _exact("output", s.capacity_rows * s.n, output)
        words = (torch.int32, torch.uint32)
        if s.matrices is None:
            if indices is not None:
                raise ValueError("indices need a spec with `matrices`")
            _check(self._lib.mircuda_variable_grouped_bf16_execute(
                self._raw, _stream_handle(stream), _device_pointer(input, _BF16),
                _device_pointer(weights, _BF16), _device_pointer(rows, words),
                _device_pointer(offsets, words), _device_pointer(output, _BF16), float(beta)))
            return
        _exact("indices", s.groups, indices)
        _check(self._lib.mircuda_b200_variable_grouped_bf16_execute_indexed(
            self._raw, _stream_handle(stream), _device_pointer(input, _BF16),
            _device_pointer(weights, _BF16), _device_pointer(indices, words),
            _device_pointer(rows, words), _device_pointer(offsets, words),
            _device_pointer(output, _BF16), float(beta)))

    def close(self):
        if getattr(self, "_raw", None):
            self._lib.mircuda_variable_grouped_bf16_destroy(self._raw)
            self._raw = None

    __del__ = close
