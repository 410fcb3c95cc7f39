"""Host-side mirror of the reference's NVFP4 GEMM plan (src/cutlass/fp4/mod.rs)."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

from . import _lib
from .plans import (InvalidMatmulShape, StreamMismatch, _BF16, _BYTES, _check, _device_pointer,
                    _exact, _stream_handle)


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
        _check(self._lib.mircuda_fp4_execute(
            self._raw, _stream_handle(stream), _device_pointer(a, _BYTES),
            _device_pointer(a_scales, _BYTES), _device_pointer(b, _BYTES),
            _device_pointer(b_scales, _BYTES), _device_pointer(output, _BF16), float(alpha)))

    def close(self) -> None:
        if getattr(self, "_raw", None):
            self._lib.mircuda_fp4_destroy(self._raw)
            self._raw = None

    __del__ = close
