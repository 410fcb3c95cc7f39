"""The allocation-free FP4 x FP4 GEMV entry point against the plan-based one.

Some hosts forbid this library from calling the CUDA allocator (their own arena owns all
device memory); for them ``mircuda_b200_fp4_vector_execute_static`` keeps its scratch in a
fixed device array inside the library. It computes what ``mircuda_fp4_vector_execute``
computes (whichever kernel the plan picks for the shape), so the two must agree; the check is
made on several calls in a row, a large shape before and after smaller ones and one that needs
no scratch at all (k <= 512), because the static scratch keeps the previous call's contents. Collected last on
purpose (file name), and written to pass both alone in a fresh process and after the rest
of the suite.
"""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from helpers import assert_close_bf16, bf16_bits, u8

pytestmark = pytest.mark.gpu


def random_fp4(rows, k, seed):
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 256, size=(rows, k // 2), dtype=np.uint8)
    values = rng.integers(0x20, 0x48, size=(rows, k // 16), dtype=np.uint8)
    scales = np.zeros(oracle.fp4_scale_bytes(rows, k), dtype=np.uint8)
    scales[oracle.fp4_scale_offsets(rows, k)] = values
    return codes, scales


def test_static_entry_point_matches_plan_entry_point(cuda_stream):
    from mircuda_b200 import _lib, plans
    library = _lib.load()
    stream = ctypes.c_void_p(cuda_stream.cuda_stream)
    for call, (n, k) in enumerate([(4096, 4096), (200, 1088), (256, 512), (4096, 4096)]):   # calls in a row
        x, xs = random_fp4(1, k, 31 + call)
        w, ws = random_fp4(n, k, 41 + call)
        tensors = [u8(x.reshape(-1)), u8(xs), u8(w.reshape(-1)), u8(ws)]
        from_plan = torch.full((n,), float("nan"), dtype=torch.bfloat16, device="cuda")
        from_static = torch.full((n,), float("nan"), dtype=torch.bfloat16, device="cuda")
        plan = plans.BlockScaledFp4VectorPlan(cuda_stream, plans.BlockScaledFp4VectorSpec(n, k))
        torch.cuda.synchronize()
        plan.execute(cuda_stream, *tensors, from_plan, 0.5)
        status = library.mircuda_b200_fp4_vector_execute_static(
            n, k, stream, *[ctypes.c_void_p(t.data_ptr()) for t in tensors],
            ctypes.c_void_p(from_static.data_ptr()), 0.5)
        assert status == 0
        cuda_stream.synchronize()
        plan.close()
        assert not torch.isnan(from_static).any()
        assert_close_bf16(bf16_bits(from_static), bf16_bits(from_plan), f"static vs plan call {call}")
        assert_close_bf16(bf16_bits(from_static), oracle.fp4_vector(x, xs, w, ws, n, k, 0.5),
                          f"static vs oracle call {call}")


def test_static_entry_point_rejects_shapes_beyond_its_scratch(cuda_stream):
    from mircuda_b200 import _lib
    library = _lib.load()
    stream = ctypes.c_void_p(cuda_stream.cuda_stream)
    dummy = torch.zeros(64, dtype=torch.uint8, device="cuda")
    pointer = ctypes.c_void_p(dummy.data_ptr())
    # 131072 rows x 16384 columns would need 32 * 131072 partial sums: far beyond 262144.
    status = library.mircuda_b200_fp4_vector_execute_static(
        131072, 16384, stream, pointer, pointer, pointer, pointer, pointer, 1.0)
    assert status == -4
    cuda_stream.synchronize()
