"""Host-side mirrors of the reference's dense GEMM plan (src/cutlass/dense.rs,
sys/src/platform/cutlass/dense/mod.rs) and of the int4 W4A16 plan this library adds."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib
from .plans import (InvalidMatmulShape, StreamMismatch, _check, _device_pointer, _exact,
                    _stream_handle)

_TYPES = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


@dataclass(frozen=True)
class DenseMatmulSpec:
    """``DenseMatmulSpec`` (sys/src/platform/cutlass/dense/mod.rs:55-62): C[m,n] = alpha A B^T + beta C."""
    m: int
    n: int
    k: int
    input_type: torch.dtype = torch.bfloat16
    output_type: torch.dtype | None = None

    def __post_init__(self):
        if self.m <= 0 or self.n <= 0 or self.k <= 0:
            raise InvalidMatmulShape("invalid dense shape")
        if self.input_type not in (torch.float16, torch.bfloat16):
            raise InvalidMatmulShape("inputs are f16 or bf16")
        if self.output() not in (self.input_type, torch.float32):
            raise InvalidMatmulShape("output is the input type or f32")

    def output(self) -> torch.dtype:
        return self.output_type or self.input_type


class DenseMatmulPlan:
    """``DenseMatmulPlan`` over ``mircuda_dense_*``."""

    def __init__(self, stream, spec: DenseMatmulSpec):
        self._lib = _lib.load()
        self.spec, self._stream = spec, stream
        raw = ctypes.c_void_p()
        _check(self._lib.mircuda_dense_create(_TYPES[spec.input_type], _TYPES[spec.output()], spec.m,
                                              spec.n, spec.k, _stream_handle(stream), ctypes.byref(raw)))
        self._raw = raw

    def execute(self, stream, a, b, c, alpha: float = 1.0, beta: float = 0.0) -> None:
        if stream.cuda_stream != self._stream.cuda_stream:
            raise StreamMismatch()
        s = self.spec
        _exact("A", s.m * s.k, a)
        _exact("B", s.n * s.k, b)
        _exact("C", s.m * s.n, c)
        _check(self._lib.mircuda_dense_execute(
            self._raw, _stream_handle(stream), _device_pointer(a, (s.input_type,)),
            _device_pointer(b, (s.input_type,)), _device_pointer(c, (s.output(),)), float(alpha),
            float(beta)))

    def close(self) -> None:
        if getattr(self, "_raw", None):
            self._lib.mircuda_dense_destroy(self._raw)
            self._raw = None

    __del__ = close


GROUP = 128


def quantize_int4(weight: torch.Tensor):
    """Symmetric int4 with zero point 8, one f16 scale = max|w| / 7 per 128 K-elements:
    returns (packed codes u8 [n, k/2], even k in the low nibble; scales f16 [n, k/128])."""
    n, k = weight.shape
    if k % GROUP != 0:
        raise InvalidMatmulShape("k must be a multiple of 128")
    groups = weight.float().view(n, k // GROUP, GROUP)
    # A device tensor as divisor: dividing by a Python scalar is evaluated as a multiplication by
    # the rounded reciprocal on CUDA, which is not the IEEE quotient the format is defined with.
    seven = torch.full((), 7.0, dtype=torch.float32, device=weight.device)
    scales = torch.div(groups.abs().amax(dim=-1), seven).to(torch.float16)
    safe = torch.where(scales == 0, torch.ones_like(scales), scales).float()
    codes = torch.clamp(torch.round(groups / safe[..., None]) + 8, 0, 15).to(torch.uint8).view(n, k)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
    return packed, scales.contiguous()


@dataclass(frozen=True)
class W4A16Spec:
    m: int
    n: int
    k: int

    def __post_init__(self):
        if self.m <= 0 or self.n <= 0 or self.k <= 0 or self.k % GROUP != 0 or self.n % 8 != 0:
            raise InvalidMatmulShape("invalid int4 W4A16 shape")


class W4A16Plan:
    """f16 activations x int4-g128 weights over ``mircuda_b200_w4a16_*`` (no reference plan)."""

    def __init__(self, stream, spec: W4A16Spec):
        self._lib = _lib.load()
        self.spec, self._stream = spec, stream
        raw = ctypes.c_void_p()
        _check(self._lib.mircuda_b200_w4a16_create(spec.m, spec.n, spec.k, _stream_handle(stream),
                                                   ctypes.byref(raw)))
        self._raw = raw

    def workspace_bytes(self) -> int:
        return int(self._lib.mircuda_b200_w4a16_workspace_bytes(self._raw))

    def execute(self, stream, input, weight, scales, output) -> None:
        if stream.cuda_stream != self._stream.cuda_stream:
            raise StreamMismatch()
        s = self.spec
        _exact("input", s.m * s.k, input)
        _exact("weight", s.n * s.k // 2, weight)
        _exact("scales", s.n * s.k // GROUP, scales)
        _exact("output", s.m * s.n, output)
        _check(self._lib.mircuda_b200_w4a16_execute(
            self._raw, _stream_handle(stream), _device_pointer(input, (torch.float16,)),
            _device_pointer(weight, (torch.uint8, torch.int8)), _device_pointer(scales, (torch.float16,)),
            _device_pointer(output, (torch.float16,))))

    def close(self) -> None:
        if getattr(self, "_raw", None):
            self._lib.mircuda_b200_w4a16_destroy(self._raw)
            self._raw = None

    __del__ = close


@dataclass(frozen=True)
class BlockwiseFp8VectorSpec:
    """``BlockwiseFp8VectorSpec`` (src/cutlass/fp8_vector.rs): E4M3 vector x E4M3 [n, k] matrix
    with one fp32 scale per 128 input elements and per 128 x 128 weight block."""
    n: int
    k: int

    def __post_init__(self):
        if self.n <= 0 or self.k <= 0 or self.n % 128 != 0 or self.k % 128 != 0:
            raise InvalidMatmulShape("n and k must be positive multiples of 128")

    def input_scale_elements(self) -> int:
        return self.k // 128

    def weight_scale_elements(self) -> int:
        return (self.n // 128) * (self.k // 128)


class BlockwiseFp8VectorPlan:
    """``BlockwiseFp8VectorPlan`` over ``mircuda_fp8_vector_*``."""

    def __init__(self, stream, spec: BlockwiseFp8VectorSpec):
        self._lib = _lib.load()
        self.spec, self._stream = spec, stream
        raw = ctypes.c_void_p()
        _check(self._lib.mircuda_fp8_vector_create(spec.n, spec.k, _stream_handle(stream),
                                                   ctypes.byref(raw)))
        self._raw = raw

    def execute(self, stream, input, input_scales, weight, weight_scales, output) -> None:
        if stream.cuda_stream != self._stream.cuda_stream:
            raise StreamMismatch()
        s = self.spec
        _exact("input", s.k, input)
        _exact("input scales", s.input_scale_elements(), input_scales)
        _exact("weight", s.n * s.k, weight)
        _exact("weight scales", s.weight_scale_elements(), weight_scales)
        _exact("output", s.n, output)
        bytes_ = (torch.uint8, torch.int8)
        _check(self._lib.mircuda_fp8_vector_execute(
            self._raw, _stream_handle(stream), _device_pointer(input, bytes_),
            _device_pointer(input_scales, (torch.float32,)), _device_pointer(weight, bytes_),
            _device_pointer(weight_scales, (torch.float32,)), _device_pointer(output, (torch.bfloat16,))))

    def close(self) -> None:
        if getattr(self, "_raw", None):
            self._lib.mircuda_fp8_vector_destroy(self._raw)
            self._raw = None

    __del__ = close


@dataclass(frozen=True)
class ScaledFp8Spec:
    """``ScaledFp8Spec`` (src/cutlass/scaled_fp8.rs:29-87): E4M3 [tokens, input_features] x E4M3
    [output_features, input_features] with one fp32 scale per token, one weight scale for the
    tensor (``weight_scale="tensor"``) or per output channel (``"output_channel"``) in fp32 or
    bf16 (``scale``), and an optional bf16 bias. Both feature counts are multiples of 16.
    ``tile`` (0 or 1) is the reference's decode-tile choice; it has no meaning here."""
    tokens: int
    input_features: int
    output_features: int
    scale: torch.dtype = torch.float32
    weight_scale: str = "tensor"
    has_bias: bool = False
    tile: int = 0

    def __post_init__(self):
        if (self.tokens <= 0 or self.input_features <= 0 or self.output_features <= 0
                or self.input_features % 16 != 0 or self.output_features % 16 != 0):
            raise InvalidMatmulShape("feature counts must be positive multiples of 16")
        if self.scale not in (torch.float32, torch.bfloat16):
            raise InvalidMatmulShape("weight scales are fp32 or bf16")
        if self.weight_scale not in ("tensor", "output_channel") or self.tile not in (0, 1):
            raise InvalidMatmulShape("unknown weight scale geometry or tile")

    def weight_scale_elements(self) -> int:
        return 1 if self.weight_scale == "tensor" else self.output_features


class ScaledFp8Plan:
    """``ScaledFp8Plan`` over ``mircuda_scaled_fp8_*``."""

    def __init__(self, stream, spec: ScaledFp8Spec):
        self._lib = _lib.load()
        self.spec, self._stream = spec, stream
        raw = ctypes.c_void_p()
        _check(self._lib.mircuda_scaled_fp8_create(
            spec.tokens, spec.output_features, spec.input_features,
            0 if spec.scale == torch.float32 else 1, 0 if spec.weight_scale == "tensor" else 1,
            int(spec.has_bias), spec.tile, _stream_handle(stream), ctypes.byref(raw)))
        self._raw = raw

    def workspace_bytes(self) -> int:
        return int(self._lib.mircuda_scaled_fp8_workspace_bytes(self._raw))

    def execute_f32_scales(self, stream, input, weight, input_scales, weight_scales, bias, output):
        if self.spec.scale != torch.float32:
            raise InvalidMatmulShape("plan was built for bf16 weight scales")
        self._execute(stream, input, weight, input_scales, weight_scales, bias, output)

    def execute_bf16_scales(self, stream, input, weight, input_scales, weight_scales, bias, output):
        if self.spec.scale != torch.bfloat16:
            raise InvalidMatmulShape("plan was built for fp32 weight scales")
        self._execute(stream, input, weight, input_scales, weight_scales, bias, output)

    def _execute(self, stream, input, weight, input_scales, weight_scales, bias, output) -> None:
        if stream.cuda_stream != self._stream.cuda_stream:
            raise StreamMismatch()
        s = self.spec
        if (bias is not None) != s.has_bias:
            raise InvalidMatmulShape("bias does not match the plan")
        _exact("input", s.tokens * s.input_features, input)
        _exact("weight", s.output_features * s.input_features, weight)
        _exact("input scales", s.tokens, input_scales)
        _exact("weight scales", s.weight_scale_elements(), weight_scales)
        _exact("output", s.tokens * s.output_features, output)
        if bias is not None:
            _exact("bias", s.output_features, bias)
        bytes_ = (torch.uint8, torch.int8)
        _check(self._lib.mircuda_scaled_fp8_execute(
            self._raw, _stream_handle(stream), _device_pointer(input, bytes_),
            _device_pointer(weight, bytes_), _device_pointer(input_scales, (torch.float32,)),
            _device_pointer(weight_scales, (s.scale,)),
            None if bias is None else _device_pointer(bias, (torch.bfloat16,)),
            _device_pointer(output, (torch.bfloat16,))))

    def close(self) -> None:
        if getattr(self, "_raw", None):
            self._lib.mircuda_scaled_fp8_destroy(self._raw)
            self._raw = None

    __del__ = close
