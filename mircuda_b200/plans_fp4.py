"""Host-side mirror of the reference's NVFP4 GEMM plan (src/cutlass/fp4/mod.rs)."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib
from .plans import (InvalidMatmulShape, StreamMismatch, _BF16, _BYTES, _check, _device_pointer,
                    _exact, _require_vector_output, _stream_handle)


@dataclass(frozen=True)
class BlockScaledFp4Spec:
    """``BlockScaledFp4Spec`` (src/cutlass/fp4/mod.rs): E2M1[M,K] x E2M1[N,K]^T -> BF16[M,N]."""
    m: int
    n: int
    k: int

    def __post_init__(self):
        if self.m <= 0 or self.n <= 0 or self.k <= 0 or self.k % 64 != 0:
            raise InvalidMatmulShape(f"invalid NVFP4 shape {self.m}x{self.n}x{self.k}")

    def scale_bytes(self, rows: int) -> int:
        """rows.div_ceil(128) * 128 * (k/16).div_ceil(4) * 4 (src/cutlass/fp4/mod.rs:106-111)."""
        return (rows + 127) // 128 * 128 * ((self.k // 16 + 3) // 4 * 4)


class BlockScaledFp4Plan:
    """``BlockScaledFp4Plan`` over ``mircuda_fp4_*``; ``alpha`` carries the global scales."""

    def __init__(self, stream, spec: BlockScaledFp4Spec):
        self._lib = _lib.load()
        self.spec, self._stream = spec, stream
        raw = ctypes.c_void_p()
        _check(self._lib.mircuda_fp4_create(spec.m, spec.n, spec.k, _stream_handle(stream),
                                            ctypes.byref(raw)))
        self._raw = raw

    def workspace_bytes(self) -> int:
        return int(self._lib.mircuda_fp4_workspace_bytes(self._raw))

    def execute(self, stream, a, a_scales, b, b_scales, output, alpha: float = 1.0) -> None:
        if stream.cuda_stream != self._stream.cuda_stream:
            raise StreamMismatch()
        s = self.spec
        _exact("A", s.m * s.k // 2, a)
        _exact("A scales", s.scale_bytes(s.m), a_scales)
        _exact("B", s.n * s.k // 2, b)
        _exact("B scales", s.scale_bytes(s.n), b_scales)
        _exact("C", s.m * s.n, output)
        _require_vector_output("C", s.n, output)
        _check(self._lib.mircuda_fp4_execute(
            self._raw, _stream_handle(stream), _device_pointer(a, _BYTES),
            _device_pointer(a_scales, _BYTES), _device_pointer(b, _BYTES),
            _device_pointer(b_scales, _BYTES), _device_pointer(output, _BF16), float(alpha)))

    def close(self) -> None:
        if getattr(self, "_raw", None):
            self._lib.mircuda_fp4_destroy(self._raw)
            self._raw = None

    __del__ = close


# ----------------------------------------------------------------- grouped NVFP4 (MoE)

def _scale_bytes(rows: int, k: int) -> int:
    """rows.div_ceil(128) * k.div_ceil(64) * 512
    (sys/src/platform/cutlass/variable_grouped/fp4/mod.rs:208-214)."""
    return (rows + 127) // 128 * ((k + 63) // 64) * 512


_U32 = (torch.int32, torch.uint32)
_F32 = (torch.float32,)


@dataclass(frozen=True)
class VariableGroupedFp4Spec:
    """``VariableGroupedFp4Spec`` (src/cutlass/variable_grouped/fp4/mod.rs:9-47)."""
    groups: int
    matrices: int
    max_rows: int
    n: int
    k: int
    capacity_rows: int

    def __post_init__(self):
        values = (self.groups, self.matrices, self.max_rows, self.n, self.k, self.capacity_rows)
        if any(v <= 0 for v in values) or self.k % 64 != 0:
            raise InvalidMatmulShape("invalid grouped NVFP4 shape")
        if max(values) > 2**32 - 1:
            raise InvalidMatmulShape("dimension does not fit u32")

    def scale_capacity_rows(self) -> int:
        """(capacity_rows + 127 * groups) / 128 * 128: every group's scales start on a
        128-row tile (sys/src/platform/cutlass/variable_grouped/fp4/mod.rs:216-223)."""
        return (self.capacity_rows + 127 * self.groups) // 128 * 128

    def a_scale_bytes(self) -> int:
        return _scale_bytes(self.scale_capacity_rows(), self.k)

    def b_scale_bytes(self) -> int:
        return _scale_bytes(self.n, self.k) * self.matrices


def _check_variable_operands(s: VariableGroupedFp4Spec, a, a_scales, b, b_scales, alphas, output):
    _exact("A", s.capacity_rows * s.k // 2, a)
    _exact("A scales", s.a_scale_bytes(), a_scales)
    _exact("B", s.matrices * s.n * s.k // 2, b)
    _exact("B scales", s.b_scale_bytes(), b_scales)
    _exact("alphas", s.matrices, alphas)
    _exact("C", s.capacity_rows * s.n, output)


def _check_metadata(s: VariableGroupedFp4Spec, indices, rows, offsets, scale_offsets):
    for name, tensor in (("indices", indices), ("rows", rows), ("offsets", offsets),
                         ("scale offsets", scale_offsets)):
        _exact(name, s.groups, tensor)


class VariableGroupedFp4Plan:
    """``VariableGroupedFp4Plan`` (src/cutlass/variable_grouped/fp4/mod.rs:106-161): all
    products are enqueued without the host reading any routing array."""

    def __init__(self, stream, spec: VariableGroupedFp4Spec):
        self._lib = _lib.load()
        self.spec, self._stream = spec, stream
        raw = ctypes.c_void_p()
        _check(self._lib.mircuda_variable_grouped_fp4_create(
            spec.groups, spec.matrices, spec.max_rows, spec.n, spec.k, _stream_handle(stream),
            ctypes.byref(raw)))
        self._raw = raw

    def execute(self, stream, a, a_scales, b, b_scales, alphas, indices, rows, offsets,
                scale_offsets, output) -> None:
        if stream.cuda_stream != self._stream.cuda_stream:
            raise StreamMismatch()
        s = self.spec
        _check_variable_operands(s, a, a_scales, b, b_scales, alphas, output)
        _check_metadata(s, indices, rows, offsets, scale_offsets)
        _check(self._lib.mircuda_variable_grouped_fp4_execute(
            self._raw, _stream_handle(stream), _device_pointer(a, _BYTES),
            _device_pointer(a_scales, _BYTES), _device_pointer(b, _BYTES),
            _device_pointer(b_scales, _BYTES), _device_pointer(alphas, _F32),
            _device_pointer(indices, _U32), _device_pointer(rows, _U32),
            _device_pointer(offsets, _U32), _device_pointer(scale_offsets, _U32),
            _device_pointer(output, _BF16)))

    def close(self) -> None:
        if getattr(self, "_raw", None):
            self._lib.mircuda_variable_grouped_fp4_destroy(self._raw)
            self._raw = None

    __del__ = close


class PairedVariableGroupedFp4Plan:
    """``PairedVariableGroupedFp4Plan`` (src/cutlass/variable_grouped/fp4/paired.rs:46-94): two
    products per group (e.g. gate and up) that share only the device-resident routing.
    ``left`` / ``right`` are (a, a_scales, b, b_scales, alphas, output) tuples."""

    def __init__(self, stream, spec: VariableGroupedFp4Spec):
        self._lib = _lib.load()
        self.spec, self._stream = spec, stream
        raw = ctypes.c_void_p()
        _check(self._lib.mircuda_paired_variable_grouped_fp4_create(
            spec.groups, spec.matrices, spec.max_rows, spec.n, spec.k, _stream_handle(stream),
            ctypes.byref(raw)))
        self._raw = raw

    def execute(self, stream, left, right, indices, rows, offsets, scale_offsets) -> None:
        if stream.cuda_stream != self._stream.cuda_stream:
            raise StreamMismatch()
        s = self.spec
        pointers = []
        outputs = []
        for side in (left, right):
            a, a_scales, b, b_scales, alphas, output = side
            _check_variable_operands(s, a, a_scales, b, b_scales, alphas, output)
            pointers += [_device_pointer(a, _BYTES), _device_pointer(a_scales, _BYTES),
                         _device_pointer(b, _BYTES), _device_pointer(b_scales, _BYTES),
                         _device_pointer(alphas, _F32)]
            outputs.append(_device_pointer(output, _BF16))
        _check_metadata(s, indices, rows, offsets, scale_offsets)
        _check(self._lib.mircuda_paired_variable_grouped_fp4_execute(
            self._raw, _stream_handle(stream), *pointers, _device_pointer(indices, _U32),
            _device_pointer(rows, _U32), _device_pointer(offsets, _U32),
            _device_pointer(scale_offsets, _U32), *outputs))

    def close(self) -> None:
        if getattr(self, "_raw", None):
            self._lib.mircuda_paired_variable_grouped_fp4_destroy(self._raw)
            self._raw = None

    __del__ = close


@dataclass(frozen=True)
class IndexedGroupedFp4Spec:
    """``IndexedGroupedFp4Spec`` (src/cutlass/grouped_fp4.rs): ``groups`` products of ``m`` rows
    each against the matrix ``selected[group]`` picks; one shared input when broadcast."""
    groups: int
    experts: int
    m: int
    n: int
    k: int
    broadcast_input: bool = False

    def __post_init__(self):
        values = (self.groups, self.experts, self.m, self.n, self.k)
        if any(v <= 0 for v in values) or self.k % 64 != 0:
            raise InvalidMatmulShape("invalid indexed grouped NVFP4 shape")

    def with_broadcast_input(self) -> "IndexedGroupedFp4Spec":
        return IndexedGroupedFp4Spec(self.groups, self.experts, self.m, self.n, self.k, True)

    def inputs(self) -> int:
        return 1 if self.broadcast_input else self.groups


class IndexedGroupedFp4Plan:
    """``IndexedGroupedFp4Plan`` (src/cutlass/grouped_fp4.rs:84-123) over ``mircuda_grouped_fp4_*``."""

    def __init__(self, stream, spec: IndexedGroupedFp4Spec):
        self._lib = _lib.load()
        self.spec, self._stream = spec, stream
        raw = ctypes.c_void_p()
        _check(self._lib.mircuda_grouped_fp4_create(
            spec.groups, spec.experts, spec.m, spec.n, spec.k, bool(spec.broadcast_input),
            _stream_handle(stream), ctypes.byref(raw)))
        self._raw = raw

    def execute(self, stream, a, a_scales, b, b_scales, alphas, selected, output) -> None:
        if stream.cuda_stream != self._stream.cuda_stream:
            raise StreamMismatch()
        s = self.spec
        _exact("A", s.inputs() * s.m * s.k // 2, a)
        _exact("A scales", s.inputs() * _scale_bytes(s.m, s.k), a_scales)
        _exact("B", s.experts * s.n * s.k // 2, b)
        _exact("B scales", s.experts * _scale_bytes(s.n, s.k), b_scales)
        _exact("alphas", s.experts, alphas)
        _exact("selected", s.groups, selected)
        _exact("C", s.groups * s.m * s.n, output)
        _check(self._lib.mircuda_grouped_fp4_execute(
            self._raw, _stream_handle(stream), _device_pointer(a, _BYTES),
            _device_pointer(a_scales, _BYTES), _device_pointer(b, _BYTES),
            _device_pointer(b_scales, _BYTES), _device_pointer(alphas, _F32),
            _device_pointer(selected, _U32), _device_pointer(output, _BF16)))

    def close(self) -> None:
        if getattr(self, "_raw", None):
            self._lib.mircuda_grouped_fp4_destroy(self._raw)
            self._raw = None

    __del__ = close
