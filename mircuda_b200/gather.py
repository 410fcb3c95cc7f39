"""Column-sharded linears across the GPUs of one box, with the all-gather of the outputs either
fused into the GEMM or carried by the copy engines beside it.

Each rank owns a contiguous block of weight rows (`sharding.column_shard`) and quantizes the
replicated activations itself. `execute_gather`: the GEMM epilogue stores every output tile
straight into the full-width output buffer of every rank over NVLink
(`mircuda_b200_mxfp8_tc_execute_gather`). `ColumnCopier`: the GEMM writes only the rank's own
full-width buffer and one strided device-to-device copy per peer moves the finished column block
while the next layer computes (`mircuda_b200_column_gather_*`), which needs no store slots of the
SMs. The full-width buffers live in symmetric memory (`torch.distributed._symmetric_memory`),
which is only used to obtain the peers' device pointers and a stream-ordered cross-GPU barrier.
The reference has no multi-GPU path; the partitioning follows its operand layouts.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib
from .plans import NativeError, StreamMismatch


class SymmetricOutput:
    """A [rows, columns] bf16 buffer with the same address layout on every rank."""

    def __init__(self, rows: int, columns: int, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symmetric_memory

        self.rows, self.columns = rows, columns
        self.group = group if group is not None else dist.group.WORLD
        self.local = symmetric_memory.empty(rows * columns, dtype=torch.bfloat16, device=device)
        self.handle = symmetric_memory.rendezvous(self.local, self.group)
        self.world = dist.get_world_size(self.group)
        pointers = [int(pointer) for pointer in self.handle.buffer_ptrs]
        if len(pointers) != self.world:
            raise RuntimeError("symmetric memory returned an unexpected number of peers")
        self.pointers = (ctypes.c_void_p * self.world)(*pointers)
        # NVSwitch multicast address of the same buffers (0 when the fabric or the allocation
        # has none): one multimem store to it reaches every rank's copy.
        self.multicast = int(getattr(self.handle, "multicast_ptr", 0) or 0)

    def barrier(self) -> None:
        """Stream-ordered barrier over all ranks: after it, every rank's stores have landed."""
        self.handle.barrier(channel=0)

    def matrix(self) -> torch.Tensor:
        return self.local.view(self.rows, self.columns)


def execute_gather(plan, stream: torch.cuda.Stream, a, a_scales, b, b_scales,
                   output: SymmetricOutput, column_offset: int, multicast: bool = False) -> None:
    """Run `plan` (a BlockScaledMxFp8Plan over this rank's shard) and scatter its output
    columns into every rank's `output` at `column_offset`: through the buffers' multicast
    address when there is one and `multicast` is set, else with one store per rank."""
    if stream.cuda_stream != plan._stream.cuda_stream:
        raise StreamMismatch()
    status = _lib.load().mircuda_b200_mxfp8_tc_execute_gather(
        plan._raw, ctypes.c_void_p(stream.cuda_stream), ctypes.c_void_p(a.data_ptr()),
        ctypes.c_void_p(a_scales.data_ptr()), ctypes.c_void_p(b.data_ptr()),
        ctypes.c_void_p(b_scales.data_ptr()),
        ctypes.cast(output.pointers, ctypes.POINTER(ctypes.c_void_p)), output.world,
        output.columns, column_offset,
        ctypes.c_void_p(output.multicast if multicast and output.multicast else None))
    if status != 0:
        raise NativeError(int(status))


class ColumnCopier:
    """Sends column blocks of `SymmetricOutput` buffers to every peer with the copy engines."""

    def __init__(self, world: int, rank: int):
        self._lib = _lib.load()
        self.world, self.rank = world, rank
        raw = ctypes.c_void_p()
        status = self._lib.mircuda_b200_column_gather_create(world, rank, ctypes.byref(raw))
        if status != 0:
            raise NativeError(int(status))
        self._raw = raw

    def execute(self, plan, stream: torch.cuda.Stream, a, a_scales, b, b_scales,
                output: SymmetricOutput, begin: int, end: int) -> None:
        """Run `plan` into columns [begin, end) of this rank's own `output`, then start the
        copies of that block to the peers; `stream` does not wait for them."""
        if stream.cuda_stream != plan._stream.cuda_stream:
            raise StreamMismatch()
        own = (ctypes.c_void_p * 1)(output.pointers[self.rank])
        handle = ctypes.c_void_p(stream.cuda_stream)
        status = self._lib.mircuda_b200_mxfp8_tc_execute_gather(
            plan._raw, handle, ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(a_scales.data_ptr()),
            ctypes.c_void_p(b.data_ptr()), ctypes.c_void_p(b_scales.data_ptr()),
            ctypes.cast(own, ctypes.POINTER(ctypes.c_void_p)), 1, output.columns, begin, None)
        if status == 0:
            status = self._lib.mircuda_b200_column_gather_send(
                self._raw, ctypes.cast(output.pointers, ctypes.POINTER(ctypes.c_void_p)),
                output.columns * 2, begin * 2, (end - begin) * 2, output.rows, handle)
        if status != 0:
            raise NativeError(int(status))

    def execute_blocks(self, plan, stream: torch.cuda.Stream, a, a_scales, b, b_scales,
                       output: SymmetricOutput) -> None:
        """The rank-major layout of an all-gather: `output` is [world * m, n_local] and rank r's
        [m, n_local] result is its block r on every rank. Run `plan` into this rank's block of
        its own `output`, then start one contiguous copy of that block per peer."""
        if stream.cuda_stream != plan._stream.cuda_stream:
            raise StreamMismatch()
        block_rows = output.rows // self.world
        block_bytes = block_rows * output.columns * 2
        own = output.matrix()[self.rank * block_rows:(self.rank + 1) * block_rows]
        plan.execute(stream, a, a_scales, b, b_scales, own.reshape(-1))
        status = self._lib.mircuda_b200_column_gather_send(
            self._raw, ctypes.cast(output.pointers, ctypes.POINTER(ctypes.c_void_p)),
            block_bytes, self.rank * block_bytes, block_bytes, 1, ctypes.c_void_p(stream.cuda_stream))
        if status != 0:
            raise NativeError(int(status))

    def join(self, stream: torch.cuda.Stream) -> None:
        """`stream` waits for every copy started so far. Follow it with `SymmetricOutput.barrier()`
        before the gathered outputs are read or a block is computed again."""
        status = self._lib.mircuda_b200_column_gather_join(self._raw, ctypes.c_void_p(stream.cuda_stream))
        if status != 0:
            raise NativeError(int(status))

    def close(self) -> None:
        if getattr(self, "_raw", None):
            self._lib.mircuda_b200_column_gather_destroy(self._raw)
            self._raw = ctypes.c_void_p()

    __del__ = close
