"""GPU parity for the routed (MoE) Marlin W4A16 projections through the C ABI: canonical
weights -> repack + scale preparation + route bucketing on the device -> execute."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from helpers import assert_close_bf16, bf16_bits, seeded_bf16, u8

pytestmark = pytest.mark.gpu

N64K128, N128K128, M64N64K128 = 2, 0, 5       # sys/src/platform/marlin/spec.rs:28-37


def pointer(tensor):
    return ctypes.c_void_p(tensor.data_ptr())


def prepare_routes(library, stream, selected, experts, block_size):
    assignments = len(selected)
    capacity = assignments + experts * (block_size - 1)
    device = dict(device="cuda")
    buffers = dict(
        selected=torch.from_numpy(np.asarray(selected, np.int32)).cuda(),
        routing=torch.ones(assignments, dtype=torch.bfloat16, **device),
        sorted=torch.zeros(capacity, dtype=torch.int32, **device),
        expert_ids=torch.zeros((capacity + block_size - 1) // block_size, dtype=torch.int32, **device),
        padded=torch.zeros(1, dtype=torch.int32, **device),
        offsets=torch.zeros(experts, dtype=torch.int32, **device),
        routing_f32=torch.zeros(assignments, dtype=torch.float32, **device))
    return buffers


def route(library, stream, buffers, experts, block_size):
    assert library.mircuda_marlin_prepare_moe_routes(
        stream, pointer(buffers["selected"]), pointer(buffers["routing"]), pointer(buffers["sorted"]),
        pointer(buffers["expert_ids"]), pointer(buffers["padded"]), pointer(buffers["offsets"]),
        pointer(buffers["routing_f32"]), buffers["selected"].numel(), experts, block_size) == 0


def test_mxfp4_moe_unit_projection_golden(cuda_stream):
    """mxfp4_moe_executes_unit_projection (tests/marlin/main.rs:60-122): one expert, codes 0x22
    (1.0), scales 127 (2^0), logical K = 64 zero-padded to 128 -> every output 64."""
    from mircuda_b200 import _lib
    library = _lib.load()
    stream = ctypes.c_void_p(cuda_stream.cuda_stream)
    tokens, outputs, k, padded_k = 8, 64, 64, 128
    weights = u8(np.full(outputs * k // 2, 0x22, np.uint8))
    packed = torch.zeros(outputs * padded_k // 2, dtype=torch.uint8, device="cuda")
    scales = u8(np.full(outputs * k // 32, 127, np.uint8))
    prepared = torch.zeros(outputs * padded_k // 32, dtype=torch.uint8, device="cuda")
    x = torch.zeros(tokens, padded_k, dtype=torch.bfloat16, device="cuda")
    x[:, :k] = 1.0
    out = torch.zeros(tokens * outputs, dtype=torch.bfloat16, device="cuda")
    buffers = prepare_routes(library, stream, [0] * tokens, 1, 8)
    torch.cuda.synchronize()
    assert library.mircuda_marlin_mxfp4_repack(stream, pointer(weights), pointer(packed), 1, outputs,
                                               padded_k, outputs, k, False) == 0
    assert library.mircuda_marlin_mxfp4_prepare_scales(stream, pointer(scales), pointer(prepared), 1,
                                                       outputs, padded_k, outputs, k, False) == 0
    route(library, stream, buffers, 1, 8)
    assert library.mircuda_marlin_mxfp4_moe_execute(
        stream, pointer(x), pointer(packed), pointer(out), None, pointer(prepared),
        pointer(buffers["sorted"]), pointer(buffers["expert_ids"]), pointer(buffers["padded"]),
        pointer(buffers["routing_f32"]), 1, False, tokens, outputs, padded_k, N64K128, None, False) == 0
    cuda_stream.synchronize()
    assert ((out.float() - 64.0).abs() <= 0.5).all()


def test_mxfp4_moe_padded_projections_golden(cuda_stream):
    """mxfp4_sequential_padded_projections_reset_workspace (tests/marlin/padded.rs:37-125): four
    experts, logical 64x64 weights padded to N = 256 and K = 256 then 128; logical columns read
    64, padded columns 0, in both projections."""
    from mircuda_b200 import _lib
    library = _lib.load()
    stream = ctypes.c_void_p(cuda_stream.cuda_stream)
    tokens, top_k, experts, n, k, physical_n = 2, 2, 4, 64, 64, 256
    routed = tokens * top_k
    buffers = prepare_routes(library, stream, [0, 1, 2, 3], experts, 8)
    for projection, physical_k in enumerate([256, 128]):
        raw = u8(np.full(experts * n * k // 2, 0x22, np.uint8))
        weight = torch.zeros(experts * physical_n * physical_k // 2, dtype=torch.uint8, device="cuda")
        scales = u8(np.full(experts * n * k // 32, 127, np.uint8))
        prepared = torch.zeros(experts * physical_n * physical_k // 32, dtype=torch.uint8, device="cuda")
        rows = tokens if projection == 0 else routed
        x = torch.zeros(rows, physical_k, dtype=torch.bfloat16, device="cuda")
        x[:, :k] = 1.0
        out = torch.zeros(routed * physical_n, dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        assert library.mircuda_marlin_mxfp4_repack(stream, pointer(raw), pointer(weight), experts,
                                                   physical_n, physical_k, n, k, False) == 0
        assert library.mircuda_marlin_mxfp4_prepare_scales(stream, pointer(scales), pointer(prepared),
                                                           experts, physical_n, physical_k, n, k, False) == 0
        if projection == 0:
            route(library, stream, buffers, experts, 8)
        assert library.mircuda_marlin_mxfp4_moe_execute(
            stream, pointer(x), pointer(weight), pointer(out), None, pointer(prepared),
            pointer(buffers["sorted"]), pointer(buffers["expert_ids"]), pointer(buffers["padded"]),
            pointer(buffers["routing_f32"]), top_k if projection == 0 else 1, False, rows, physical_n,
            physical_k, N128K128, None, False) == 0
        cuda_stream.synchronize()
        values = out.float().view(routed, physical_n)
        assert ((values[:, :n] - 64.0).abs() <= 0.5).all(), projection
        assert (values[:, n:].abs() <= 0.5).all(), projection


def expected_outputs(x, weights, selected, top_k, routing):
    """weights fp64 [experts, n, k]; one output row per assignment."""
    x = oracle.bf16_to_f32(bf16_bits(x)).astype(np.float64)
    rows = []
    for assignment, expert in enumerate(selected):
        row = x[assignment // top_k] @ weights[expert].T
        rows.append(row * (routing[assignment] if routing is not None else 1.0))
    return oracle.f32_to_bf16(np.asarray(rows, dtype=np.float32))


@pytest.fixture(params=["stream", "tiles"])
def moe_kernel(request, monkeypatch):
    """Both kernels behind the routed entry points: the streaming one (k % 256 == 0, k <= 2048;
    other shapes fall to the tile kernel) and the tile kernel."""
    monkeypatch.setenv("MIRCUDA_B200_MARLIN_MOE", request.param)
    return request.param


@pytest.mark.parametrize("thread_config,block_size", [(N64K128, 8), (M64N64K128, 64)])
@pytest.mark.parametrize("multiply", [False, True])
@pytest.mark.parametrize("n,k", [(192, 272), (256, 768), (192, 2048), (64, 256)])
def test_nvfp4_moe_random(cuda_stream, moe_kernel, thread_config, block_size, multiply, n, k):
    from mircuda_b200 import _lib
    library = _lib.load()
    stream = ctypes.c_void_p(cuda_stream.cuda_stream)
    experts, tokens, top_k = 5, 37, 2
    rng = np.random.default_rng(41 + block_size)
    codes = rng.integers(0, 256, size=experts * n * k // 2, dtype=np.uint8)
    scales = rng.integers(0x28, 0x48, size=experts * n * k // 16, dtype=np.uint8)
    globals_ = rng.uniform(0.005, 0.02, size=experts).astype(np.float32)
    selected = rng.integers(0, experts, size=tokens * top_k)
    selected[selected == 3] = 4                                   # expert 3 gets no rows
    routing = rng.uniform(0.1, 1.0, size=tokens * top_k).astype(np.float32)
    x = seeded_bf16((tokens, k), 1.0, 8300)

    packed = torch.zeros(experts * n * k // 2, dtype=torch.uint8, device="cuda")
    prepared = torch.zeros(experts * n * k // 16, dtype=torch.uint8, device="cuda")
    prepared_globals = torch.zeros(experts, dtype=torch.float32, device="cuda")
    maximum = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.full((tokens * top_k * n,), float("nan"), dtype=torch.bfloat16, device="cuda")
    buffers = prepare_routes(library, stream, selected, experts, block_size)
    buffers["routing"] = torch.from_numpy(routing).cuda().to(torch.bfloat16)
    routing = buffers["routing"].float().cpu().numpy()            # what the kernel will multiply by
    d_codes, d_scales, d_globals = u8(codes), u8(scales), torch.from_numpy(globals_).cuda()
    torch.cuda.synchronize()
    assert library.mircuda_marlin_nvfp4_repack(stream, pointer(d_codes), pointer(packed), experts, n, k) == 0
    assert library.mircuda_marlin_nvfp4_prepare_scales(
        stream, pointer(d_scales), None, pointer(d_globals), pointer(prepared),
        pointer(prepared_globals), pointer(maximum), experts, n, k) == 0
    route(library, stream, buffers, experts, block_size)
    for _ in range(2):
        assert library.mircuda_marlin_nvfp4_moe_execute(
            stream, pointer(x), pointer(packed), pointer(out), None, pointer(prepared),
            pointer(prepared_globals), pointer(buffers["sorted"]), pointer(buffers["expert_ids"]),
            pointer(buffers["padded"]), pointer(buffers["routing_f32"]), top_k, multiply, tokens, n, k,
            thread_config, None, False) == 0
    cuda_stream.synchronize()
    nibbles = np.stack([codes & 15, codes >> 4], axis=-1).reshape(experts, n, k)
    values = oracle.e2m1_table()[nibbles].astype(np.float64)
    decoded = oracle.e4m3_table()[scales.reshape(experts, n, k // 16)].astype(np.float64)
    weights = values * np.repeat(decoded, 16, axis=2) * globals_[:, None, None].astype(np.float64)
    expected = expected_outputs(x, weights, selected, top_k, routing if multiply else None)
    assert_close_bf16(bf16_bits(out).reshape(tokens * top_k, n), expected,
                      f"marlin nvfp4 moe block={block_size} multiply={multiply}")


@pytest.mark.parametrize("thread_config,block_size", [(N128K128, 8), (M64N64K128, 64)])
@pytest.mark.parametrize("n,k", [(128, 320), (128, 512), (192, 2048), (256, 768)])
def test_mxfp4_moe_random(cuda_stream, moe_kernel, thread_config, block_size, n, k):
    from mircuda_b200 import _lib
    library = _lib.load()
    stream = ctypes.c_void_p(cuda_stream.cuda_stream)
    experts, tokens, top_k = 3, 21, 3
    rng = np.random.default_rng(43 + block_size)
    codes = rng.integers(0, 256, size=experts * n * k // 2, dtype=np.uint8)
    scales = rng.integers(118, 132, size=experts * n * k // 32, dtype=np.uint8)
    selected = rng.integers(0, experts, size=tokens * top_k)
    x = seeded_bf16((tokens, k), 1.0, 8400)
    packed = torch.zeros(experts * n * k // 2, dtype=torch.uint8, device="cuda")
    prepared = torch.zeros(experts * n * k // 32, dtype=torch.uint8, device="cuda")
    out = torch.full((tokens * top_k * n,), float("nan"), dtype=torch.bfloat16, device="cuda")
    buffers = prepare_routes(library, stream, selected, experts, block_size)
    d_codes, d_scales = u8(codes), u8(scales)
    torch.cuda.synchronize()
    assert library.mircuda_marlin_mxfp4_repack(stream, pointer(d_codes), pointer(packed), experts, n, k,
                                               n, k, False) == 0
    assert library.mircuda_marlin_mxfp4_prepare_scales(stream, pointer(d_scales), pointer(prepared),
                                                       experts, n, k, n, k, False) == 0
    route(library, stream, buffers, experts, block_size)
    assert library.mircuda_marlin_mxfp4_moe_execute(
        stream, pointer(x), pointer(packed), pointer(out), None, pointer(prepared),
        pointer(buffers["sorted"]), pointer(buffers["expert_ids"]), pointer(buffers["padded"]),
        pointer(buffers["routing_f32"]), top_k, False, tokens, n, k, thread_config, None, False) == 0
    cuda_stream.synchronize()
    nibbles = np.stack([codes & 15, codes >> 4], axis=-1).reshape(experts, n, k)
    values = oracle.e2m1_table()[nibbles].astype(np.float64)
    decoded = np.exp2(scales.reshape(experts, n, k // 32).astype(np.float64) - 127.0)
    weights = values * np.repeat(decoded, 32, axis=2)
    expected = expected_outputs(x, weights, selected, top_k, None)
    assert_close_bf16(bf16_bits(out).reshape(tokens * top_k, n), expected, f"marlin mxfp4 moe block={block_size}")
