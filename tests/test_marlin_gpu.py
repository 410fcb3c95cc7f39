"""GPU parity (bit-exact) for the Marlin-layout preparation entry points, against the numpy
restatement of the host references inside the reference's own tests."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from oracle import marlin
from helpers import u8

pytestmark = pytest.mark.gpu

EXPERTS, N, K = 2, 64, 64


def canonical_weights(experts=EXPERTS, n=N, k=K):
    """tests/marlin/main.rs:124-137."""
    e = np.arange(experts)[:, None, None]
    row = np.arange(n)[None, :, None]
    col = np.arange(0, k, 2)[None, None, :]
    low = (e * 7 + row * 3 + col) & 15
    high = (e * 7 + row * 3 + col + 1) & 15
    return (low | (high << 4)).astype(np.uint8).reshape(-1)


def library():
    from mircuda_b200 import _lib
    return _lib.load()


def pointer(tensor):
    return ctypes.c_void_p(tensor.data_ptr())


def test_nvfp4_repack_matches_marlin_tile_layout(cuda_stream):
    """tests/marlin/main.rs:15-31."""
    raw = canonical_weights()
    source = u8(raw)
    output = torch.zeros(raw.size, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    assert library().mircuda_marlin_nvfp4_repack(
        ctypes.c_void_p(cuda_stream.cuda_stream), pointer(source), pointer(output), EXPERTS, N, K) == 0
    cuda_stream.synchronize()
    expected = marlin.repack(raw, EXPERTS, N, K)
    assert np.array_equal(output.cpu().numpy().view(np.uint32), expected)


def test_nvfp4_repack_pair_and_large(cuda_stream):
    rng = np.random.default_rng(3)
    experts, n, k = 3, 256, 128
    left = rng.integers(0, 256, experts * (n // 2) * k // 2, dtype=np.uint8)
    right = rng.integers(0, 256, experts * (n // 2) * k // 2, dtype=np.uint8)
    l, r = u8(left), u8(right)
    output = torch.zeros(experts * n * k // 2, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    assert library().mircuda_marlin_nvfp4_repack_pair(
        ctypes.c_void_p(cuda_stream.cuda_stream), pointer(l), pointer(r), pointer(output), experts, n, k) == 0
    cuda_stream.synchronize()
    expected = marlin.repack(left, experts, n, k, right=right)
    assert np.array_equal(output.cpu().numpy().view(np.uint32), expected)


@pytest.mark.parametrize("padded_n,padded_k", [(64, 64), (128, 128)])
def test_mxfp4_interleaved_weights_and_scales(cuda_stream, padded_n, padded_k):
    """tests/marlin/main.rs:33-58 (unpadded) and tests/marlin/padded.rs:11-34 (zero padding)."""
    raw = canonical_weights()
    source = u8(raw)
    output = torch.zeros(EXPERTS * padded_n * padded_k // 2, dtype=torch.uint8, device="cuda")
    stream = ctypes.c_void_p(cuda_stream.cuda_stream)
    torch.cuda.synchronize()
    assert library().mircuda_marlin_mxfp4_repack(
        stream, pointer(source), pointer(output), EXPERTS, padded_n, padded_k, N, K, True) == 0
    cuda_stream.synchronize()
    expected = marlin.repack(raw, EXPERTS, padded_n, padded_k, N, K, interleaved=True)
    assert np.array_equal(output.cpu().numpy().view(np.uint32), expected)

    scales = (np.arange(EXPERTS * N * K // 32) % 251).astype(np.uint8)
    scale_source = u8(scales)
    scale_output = torch.zeros(EXPERTS * padded_n * padded_k // 32, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    assert library().mircuda_marlin_mxfp4_prepare_scales(
        stream, pointer(scale_source), pointer(scale_output), EXPERTS, padded_n, padded_k, N, K, True) == 0
    cuda_stream.synchronize()
    expected = marlin.mxfp4_scales(scales, EXPERTS, padded_n, padded_k, N, K, True)
    assert np.array_equal(scale_output.cpu().numpy(), expected)


@pytest.mark.parametrize("paired", [False, True])
def test_nvfp4_prepare_scales(cuda_stream, paired):
    """sys/native/marlin/repack.cu:88-140 (no reference test covers the re-encoding)."""
    rng = np.random.default_rng(5)
    experts, n, k = 3, 128, 256
    source_n = n // 2 if paired else n
    left = rng.integers(0x10, 0x60, experts * source_n * k // 16, dtype=np.uint8)
    right = rng.integers(0x10, 0x60, experts * source_n * k // 16, dtype=np.uint8) if paired else None
    globals_ = rng.random(experts, dtype=np.float32) + np.float32(0.5)
    l = u8(left)
    r = u8(right) if paired else None
    g = torch.from_numpy(globals_).cuda()
    output = torch.zeros(experts * n * k // 16, dtype=torch.uint8, device="cuda")
    out_globals = torch.zeros(experts, dtype=torch.float32, device="cuda")
    maximum = torch.zeros(1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    assert library().mircuda_marlin_nvfp4_prepare_scales(
        ctypes.c_void_p(cuda_stream.cuda_stream), pointer(l), pointer(r) if paired else None,
        pointer(g), pointer(output), pointer(out_globals), pointer(maximum), experts, n, k) == 0
    cuda_stream.synchronize()
    expected, expected_globals, _ = marlin.nvfp4_scales(left, right, globals_, experts, n, k)
    assert np.array_equal(output.cpu().numpy(), expected)
    assert np.array_equal(out_globals.cpu().numpy(), expected_globals)


@pytest.mark.parametrize("block", [8, 64])
def test_routes_order_each_experts_rows_by_assignment(cuda_stream, block):
    """tests/marlin/routes.rs:8-54."""
    tokens, top_k, experts = 2400, 8, 16
    assignments = tokens * top_k
    index = np.arange(assignments)
    choices = ((index * 7 + index // 5) % experts).astype(np.uint32)
    choices[17] = 99                                    # an out-of-range expert is skipped
    selected = torch.from_numpy(choices.view(np.int32)).cuda()
    routing = torch.full((assignments,), 0.5, dtype=torch.bfloat16, device="cuda")
    capacity = assignments + experts * (block - 1)
    sorted_rows = torch.zeros(capacity, dtype=torch.int32, device="cuda")
    expert_ids = torch.full(((capacity + block - 1) // block,), -1, dtype=torch.int32, device="cuda")
    padded = torch.zeros(1, dtype=torch.int32, device="cuda")
    offsets = torch.zeros(experts, dtype=torch.int32, device="cuda")
    routing_f32 = torch.zeros(assignments, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    assert library().mircuda_marlin_prepare_moe_routes(
        ctypes.c_void_p(cuda_stream.cuda_stream), pointer(selected), pointer(routing),
        pointer(sorted_rows), pointer(expert_ids), pointer(padded), pointer(offsets),
        pointer(routing_f32), assignments, experts, block) == 0
    cuda_stream.synchronize()
    expected_sorted, expected_ids, expected_total, expected_offsets = marlin.routes(choices, experts, block)
    assert int(padded.item()) == expected_total
    assert np.array_equal(offsets.cpu().numpy(), expected_offsets)
    assert np.array_equal(sorted_rows.cpu().numpy(), expected_sorted)
    blocks = expected_total // block
    assert np.array_equal(expert_ids.cpu().numpy()[:blocks], expected_ids[:blocks])
    assert (routing_f32.cpu().numpy() == 0.5).all()
