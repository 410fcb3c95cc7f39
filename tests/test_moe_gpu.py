"""MoE feed-forward over the grouped plans: single-GPU layer against a torch fp32 restatement,
and the expert-parallel layer on two GPUs against the single-GPU result."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

HIDDEN, INTERMEDIATE, EXPERTS, TOP_K, TOKENS = 256, 128, 8, 2, 96


def make_inputs(device):
    generator = torch.Generator().manual_seed(4100)
    x = torch.randn(TOKENS, HIDDEN, generator=generator).to(torch.bfloat16).to(device)
    gate_up = (torch.randn(EXPERTS, 2 * INTERMEDIATE, HIDDEN, generator=generator) * 0.05).to(torch.bfloat16).to(device)
    down = (torch.randn(EXPERTS, HIDDEN, INTERMEDIATE, generator=generator) * 0.05).to(torch.bfloat16).to(device)
    logits = torch.randn(TOKENS, EXPERTS, generator=generator).to(device)
    return x, gate_up, down, logits


def reference_layer(x, gate_up, down, chosen, weights):
    """fp32 math with bf16 roundings where the kernels round (GEMM outputs, activation)."""
    output = torch.zeros(x.shape[0], x.shape[1], dtype=torch.float32, device=x.device)
    for token in range(x.shape[0]):
        for choice in range(chosen.shape[1]):
            expert = int(chosen[token, choice])
            hidden = (x[token].float() @ gate_up[expert].float().T).to(torch.bfloat16).float()
            gate, up = hidden[:INTERMEDIATE], hidden[INTERMEDIATE:]
            activated = (torch.nn.functional.silu(gate) * up).to(torch.bfloat16).float()
            expert_out = (activated @ down[expert].float().T).to(torch.bfloat16).float()
            output[token] += weights[token, choice] * expert_out
    return output


def run_single(stream, nvfp4, transport="peer"):
    from mircuda_b200 import moe
    device = torch.device("cuda", torch.cuda.current_device())
    x, gate_up, down, logits = make_inputs(device)
    chosen, weights = moe.route(logits, TOP_K)
    align = 128 if nvfp4 else 1
    dispatch = moe.plan_dispatch(chosen, EXPERTS, 1, None, align)
    capacity = (dispatch.largest_block + 127) // 128 * 128
    dispatch = moe.plan_dispatch(chosen, EXPERTS, 1, capacity, align)
    bank = moe.ExpertWeights(stream, gate_up, down, nvfp4)
    if transport == "peer":
        capacity = (TOKENS * TOP_K + 128 * EXPERTS) // 128 * 128
    layer = moe.ExpertParallelMoe(stream, HIDDEN, INTERMEDIATE, EXPERTS, TOP_K, TOKENS, capacity, bank,
                                  transport=transport)
    if nvfp4:
        layer.calibrate(x, dispatch if transport == "peer" else None, weights)
    torch.cuda.synchronize()
    for _ in range(2):
        out = layer.forward(x, dispatch, weights)
    stream.synchronize()
    expected = reference_layer(x, gate_up, down, chosen, weights)
    layer.close()
    return out.float(), expected


@pytest.mark.parametrize("transport", ["peer", "nccl"])
def test_moe_layer_bf16_single_gpu(cuda_stream, transport):
    out, expected = run_single(cuda_stream, False, transport)
    error = (out - expected).norm() / expected.norm()
    assert error < 5e-3, error
    assert (out - expected).abs().max() <= 1e-2 * expected.abs().max()


def nvfp4_layer_restatement(x, gate_up, down, chosen, weights, global1, global2):
    """The NVFP4 layer restated with the oracle, step by step as the layer runs it: token rows
    quantised with the calibrated scale `global1` (oracle.nvfp4_quantize), the routed rows
    grouped per expert and multiplied by the NVFP4 gate_up bank (oracle.variable_grouped_fp4,
    sys/native/variable_grouped_fp4_sm120.cu:31-62; alpha = bank global * global1, bf16 out),
    SwiGLU rounded to bf16, requantised with `global2`, multiplied by the down bank the same
    way, and the top_k rows of a token added in choice order with fused multiply-adds."""
    import oracle
    from helpers import bf16_bits
    tokens, hidden = x.shape
    experts, two_i, _ = gate_up.shape
    intermediate = two_i // 2
    top_k = chosen.shape[1]
    flat = chosen.reshape(-1).cpu().numpy()
    order = np.argsort(flat, kind="stable")
    rows = np.bincount(flat, minlength=experts).astype(np.uint32)
    offsets = (np.cumsum(rows) - rows).astype(np.uint32)
    scale_offsets = (np.cumsum((rows + 127) // 128 * 128) - (rows + 127) // 128 * 128).astype(np.uint32)
    capacity = int(rows.sum())
    scale_rows = int(((rows + 127) // 128 * 128).sum())

    def quantize_groups(values_bits, k, global_scale):
        codes = np.zeros((capacity, k // 2), np.uint8)
        scales = np.zeros(scale_rows // 128 * (k // 64) * 512, np.uint8)
        for expert in range(experts):
            count, first = int(rows[expert]), int(offsets[expert])
            if count == 0:
                continue
            group_codes, group_scales, _ = oracle.nvfp4_quantize(values_bits[first:first + count], global_scale)
            codes[first:first + count] = group_codes
            begin = int(scale_offsets[expert]) // 128 * (k // 64) * 512
            scales[begin:begin + group_scales.size] = group_scales
        return codes, scales

    def bank(matrix):
        count, n, k = matrix.shape
        codes, scales, bank_global = oracle.nvfp4_quantize(bf16_bits(matrix.reshape(count * n, k)))
        return codes.reshape(count, n, k // 2), scales, bank_global

    x_rows = bf16_bits(x)[order // top_k]
    a1, a1_scales = quantize_groups(x_rows, hidden, global1)
    b1, b1_scales, b1_global = bank(gate_up)
    indices = np.arange(experts, dtype=np.uint32)
    alphas1 = np.full(experts, np.float32(b1_global) * np.float32(global1), np.float32)
    hidden_bits = oracle.variable_grouped_fp4(
        a1, a1_scales, b1, b1_scales, alphas1, indices, rows, offsets, scale_offsets,
        np.zeros((capacity, two_i), np.uint16), experts, capacity, two_i, hidden)
    hidden_values = oracle.bf16_to_f32(hidden_bits)
    gate, up = hidden_values[:, :intermediate], hidden_values[:, intermediate:]
    activated = oracle.f32_to_bf16((gate / (np.float32(1.0) + np.exp(-gate)) * up).astype(np.float32))
    a2, a2_scales = quantize_groups(activated, intermediate, global2)
    b2, b2_scales, b2_global = bank(down)
    alphas2 = np.full(experts, np.float32(b2_global) * np.float32(global2), np.float32)
    expert_out = oracle.bf16_to_f32(oracle.variable_grouped_fp4(
        a2, a2_scales, b2, b2_scales, alphas2, indices, rows, offsets, scale_offsets,
        np.zeros((capacity, hidden), np.uint16), experts, capacity, hidden, intermediate))
    slot = np.empty_like(order)
    slot[order] = np.arange(order.size)
    routing = weights.cpu().numpy().astype(np.float32)
    output = np.zeros((tokens, hidden), np.float32)
    for choice in range(top_k):
        picked = expert_out[slot.reshape(tokens, top_k)[:, choice]]
        output = (routing[:, choice:choice + 1].astype(np.float64) * picked + output).astype(np.float32)
    return oracle.f32_to_bf16(output), float(np.max(np.abs(oracle.bf16_to_f32(activated)))), a1


@pytest.mark.parametrize("transport", ["peer", "nccl"])
def test_moe_layer_nvfp4_single_gpu(cuda_stream, transport):
    """The NVFP4 layer against its exact restatement (same quantisers, same scales, same grouped
    products), to the GEMM tolerance: max |d| <= 1e-2 max|ref|, relative Frobenius <= 5e-3."""
    import oracle
    from helpers import assert_close_bf16, bf16_bits
    from mircuda_b200 import moe
    device = torch.device("cuda", torch.cuda.current_device())
    x, gate_up, down, logits = make_inputs(device)
    chosen, weights = moe.route(logits, TOP_K)
    dispatch = moe.plan_dispatch(chosen, EXPERTS, 1, None, 128)
    capacity = (dispatch.largest_block + 127) // 128 * 128
    dispatch = moe.plan_dispatch(chosen, EXPERTS, 1, capacity, 128)
    bank = moe.ExpertWeights(cuda_stream, gate_up, down, True)
    if transport == "peer":
        capacity = (TOKENS * TOP_K + 128 * EXPERTS) // 128 * 128
    layer = moe.ExpertParallelMoe(cuda_stream, HIDDEN, INTERMEDIATE, EXPERTS, TOP_K, TOKENS, capacity,
                                  bank, transport=transport)
    layer.calibrate(x, dispatch if transport == "peer" else None, weights)
    torch.cuda.synchronize()
    for _ in range(2):
        out = layer.forward(x, dispatch, weights)
    cuda_stream.synchronize()
    global1 = float(x.abs().max().float()) / 2688.0
    if transport == "peer":
        assert float(layer.dispatch_global) == np.float32(global1)
    else:
        assert float(layer.global1) == np.float32(global1)
    global2 = float(layer.global2)          # calibrated (peer) or measured this step (nccl)
    expected, activated_amax, token_codes = nvfp4_layer_restatement(
        x, gate_up, down, chosen, weights, np.float32(global1), np.float32(global2))
    # The intermediate scale the layer settled on is the oracle's, up to the calibration margin.
    margin = 2.0 if transport == "peer" else 1.0
    assert abs(global2 / (margin * activated_amax / 2688.0) - 1.0) < 0.02
    if transport == "peer":
        # codes of the dispatched token rows, bit for bit (row-major on the device, before travel)
        device_codes = layer.token_codes.cpu().numpy().reshape(TOKENS, HIDDEN // 2)
        order = np.argsort(chosen.reshape(-1).cpu().numpy(), kind="stable")
        assert np.array_equal(device_codes[order // TOP_K], token_codes)
    assert torch.isfinite(out.float()).all()
    assert_close_bf16(bf16_bits(out), expected, f"nvfp4 moe layer ({transport})")
    layer.close()


def _worker(rank, world, port, transport, nvfp4, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from mircuda_b200 import moe
        device = torch.device("cuda", rank)
        stream = torch.cuda.Stream()
        x, gate_up, down, logits = make_inputs(device)
        chosen, weights = moe.route(logits, TOP_K)
        local_tokens = TOKENS // world
        local = slice(rank * local_tokens, (rank + 1) * local_tokens)
        local_experts = EXPERTS // world
        experts = slice(rank * local_experts, (rank + 1) * local_experts)
        dispatch = moe.plan_dispatch(chosen[local], EXPERTS, world, None)
        largest = torch.tensor([dispatch.largest_block], device=device)
        dist.all_reduce(largest, op=dist.ReduceOp.MAX)
        capacity = (int(largest.item()) + 15) // 16 * 16
        dispatch = moe.plan_dispatch(chosen[local], EXPERTS, world, capacity)
        bank = moe.ExpertWeights(stream, gate_up[experts], down[experts], nvfp4)
        if transport == "peer":
            # A rank can never receive more rows than exist (plus 128-row alignment per expert).
            capacity = (TOKENS * TOP_K + 128 * local_experts + 127) // 128 * 128
        layer = moe.ExpertParallelMoe(stream, HIDDEN, INTERMEDIATE, EXPERTS, TOP_K, local_tokens,
                                      capacity, bank, transport=transport)
        if nvfp4:
            layer.calibrate(x[local], dispatch, weights[local].contiguous())
        torch.cuda.synchronize()
        dist.barrier()
        for _ in range(2):
            out = layer.forward(x[local].contiguous(), dispatch, weights[local].contiguous())
        stream.synchronize()
        expected = reference_layer(x[local], gate_up, down, chosen[local], weights[local])
        error = float((out.float() - expected).norm() / expected.norm())
        results[rank] = error
        layer.close()
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("transport,nvfp4", [("peer", False), ("nccl", False), ("peer", True)])
def test_moe_layer_expert_parallel_two_gpus(transport, nvfp4):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, port, transport, nvfp4, results), nprocs=2, join=True)
    assert set(results.keys()) == {0, 1}
    bound = 0.25 if nvfp4 else 5e-3        # NVFP4: plausibility bound, as on one GPU
    assert all(error < bound for error in results.values()), dict(results)


def test_fused_swiglu_quantiser_matches_two_passes(cuda_stream):
    """SwiGLU fused with the NVFP4 quantiser must give the codes and scales of SwiGLU followed by
    the stand-alone quantiser, bit for bit, and respect the device-side row bound."""
    import ctypes
    from mircuda_b200 import _lib
    library = _lib.load()
    rows, intermediate, bound_rows = 300, 192, 257
    generator = torch.Generator(device="cuda").manual_seed(99)
    hidden = torch.randn(rows, 2 * intermediate, generator=generator, device="cuda").to(torch.bfloat16)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    handle = ctypes.c_void_p(cuda_stream.cuda_stream)
    activated = torch.zeros(rows, intermediate, dtype=torch.bfloat16, device="cuda")
    global_scale = torch.full((1,), 0.0031, dtype=torch.float32, device="cuda")
    scale_bytes = (rows + 127) // 128 * (intermediate // 64) * 512
    codes = [torch.zeros(rows * intermediate // 2, dtype=torch.uint8, device="cuda") for _ in range(2)]
    scales = [torch.zeros(scale_bytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
    bound = torch.tensor([bound_rows], dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    assert library.mircuda_b200_moe_swiglu_bf16(p(hidden), p(activated), rows, p(bound), intermediate, handle) == 0
    assert library.mircuda_b200_nvfp4_quantize_bf16(p(activated), p(global_scale), p(codes[0]), p(scales[0]),
                                                    bound_rows, intermediate, handle) == 0
    assert library.mircuda_b200_moe_swiglu_nvfp4(p(hidden), p(global_scale), p(codes[1]), p(scales[1]), rows,
                                                 p(bound), intermediate, handle) == 0
    cuda_stream.synchronize()
    assert torch.equal(codes[0], codes[1]) and torch.equal(scales[0], scales[1])
    assert codes[1][bound_rows * intermediate // 2:].eq(0).all() and codes[1].any()


def test_scale_atoms_matches_swizzle(cuda_stream):
    import ctypes
    from mircuda_b200 import _lib
    library = _lib.load()
    rows, columns = 300, 128
    source = torch.randint(0, 256, (rows * columns,), dtype=torch.uint8, device="cuda")
    size = (rows + 127) // 128 * 128 * columns
    expected = torch.zeros(size, dtype=torch.uint8, device="cuda")
    actual = torch.zeros(size, dtype=torch.uint8, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    handle = ctypes.c_void_p(cuda_stream.cuda_stream)
    torch.cuda.synchronize()
    assert library.mircuda_b200_mxfp8_swizzle_scales(p(source), p(expected), rows, columns, handle) == 0
    assert library.mircuda_b200_moe_scale_atoms(p(source), p(actual), rows, None, columns, handle) == 0
    cuda_stream.synchronize()
    assert torch.equal(actual, expected)


def test_dispatch_respects_the_receive_capacity(cuda_stream):
    """A routing more skewed than the buffers were sized for: the layout kernel clamps the
    owner's rows / offsets to the capacity and raises the overflow word, the dispatch kernel
    skips the rows that do not fit (recorded as -1), the rows behind the capacity keep their
    contents, and the way back adds nothing for a skipped row."""
    import ctypes
    from mircuda_b200 import _lib
    library = _lib.load()
    experts, columns, capacity, guard = 4, 64, 24, 8
    counts = [10, 9, 8, 5]                                   # 32 rows wanted, 24 fit
    assignments = sum(counts)
    p = lambda tensor: ctypes.c_void_p(tensor.data_ptr())
    handle = ctypes.c_void_p(cuda_stream.cuda_stream)
    i32 = lambda values: torch.tensor(values, dtype=torch.int32, device="cuda")
    all_counts = i32(counts)
    sorted_expert = i32([e for e, c in enumerate(counts) for _ in range(c)])
    position = i32([j for c in counts for j in range(c)])
    source_index = torch.arange(assignments, dtype=torch.int32, device="cuda")
    source = torch.arange(assignments * columns, dtype=torch.float32, device="cuda").view(assignments, columns)
    source = (source % 251 + 1).to(torch.bfloat16)
    receive = torch.full((capacity + guard, columns), -7.0, dtype=torch.bfloat16, device="cuda")
    base_for_me, remote_row = i32([0] * experts), i32([0] * assignments)
    rows, offsets, received = i32([0] * experts), i32([0] * experts), i32([0])
    overflow = torch.zeros(1, dtype=torch.int32, device="cuda")
    pointers = (ctypes.c_void_p * 1)(receive.data_ptr())
    torch.cuda.synchronize()
    assert library.mircuda_b200_moe_expert_layout(p(all_counts), 1, 0, experts, 1, p(base_for_me), p(rows),
                                                  p(offsets), p(received), capacity, p(overflow), handle) == 0
    assert library.mircuda_b200_moe_dispatch_rows_bf16(
        p(source), p(source_index), p(sorted_expert), p(position), p(base_for_me),
        ctypes.cast(pointers, ctypes.POINTER(ctypes.c_void_p)), 1, p(remote_row), assignments, experts,
        columns, capacity, handle) == 0
    cuda_stream.synchronize()
    assert int(overflow) == 1
    assert rows.tolist() == [10, 9, 5, 0] and offsets.tolist() == [0, 10, 19, 24] and int(received) == 24
    expected_rows = [r if r < capacity else -1 for r in range(assignments)]
    assert remote_row.tolist() == expected_rows
    assert torch.equal(receive[:capacity], source[:capacity])
    assert (receive[capacity:] == -7.0).all()                # nothing was written past the capacity
    # The way back: token t owns assignments 2t and 2t + 1; skipped rows contribute nothing.
    tokens, top_k = assignments // 2, 2
    slot = torch.arange(assignments, dtype=torch.int32, device="cuda")
    weights = torch.full((tokens, top_k), 0.5, dtype=torch.float32, device="cuda")
    output = torch.full((tokens, columns), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert library.mircuda_b200_moe_collect_rows_bf16(
        ctypes.cast(pointers, ctypes.POINTER(ctypes.c_void_p)), 1, p(slot), p(sorted_expert), p(remote_row),
        p(weights), p(output), tokens, top_k, experts, columns, handle) == 0
    cuda_stream.synchronize()
    kept = source.float().clone()
    kept[capacity:] = 0.0
    expected = 0.5 * (kept[0::2] + kept[1::2])
    assert torch.equal(output.float(), expected.to(torch.bfloat16).float())
    # No overflow: the word stays clear.
    overflow.zero_()
    assert library.mircuda_b200_moe_expert_layout(p(all_counts), 1, 0, experts, 1, p(base_for_me), p(rows),
                                                  p(offsets), p(received), 32, p(overflow), handle) == 0
    cuda_stream.synchronize()
    assert int(overflow) == 0 and rows.tolist() == counts


def test_dispatch_and_collect_skip_indices_outside_the_job(cuda_stream):
    """An expert index with no owner, a negative one and a slot past the assignments are treated
    like rows that did not fit: nothing is stored or loaded for them. The row width (40 pieces of
    16 bytes) is not a whole number of 32-lane rounds, so the last round of the collection has
    idle lanes."""
    import ctypes
    from mircuda_b200 import _lib
    library = _lib.load()
    experts, columns, capacity = 4, 320, 16
    p = lambda tensor: ctypes.c_void_p(tensor.data_ptr())
    handle = ctypes.c_void_p(cuda_stream.cuda_stream)
    i32 = lambda values: torch.tensor(values, dtype=torch.int32, device="cuda")
    sorted_expert = i32([0, 1, 99, -3, 2, 3])                 # 99: owner 24 of 1; -3: no expert
    position = i32([0, 0, 0, 0, 0, 0])
    base_for_me = i32([0, 1, 2, 3])
    assignments = 6
    source_index = torch.arange(assignments, dtype=torch.int32, device="cuda")
    source = (torch.arange(assignments * columns, dtype=torch.float32, device="cuda") % 199 + 1)
    source = source.view(assignments, columns).to(torch.bfloat16)
    receive = torch.full((capacity, columns), -7.0, dtype=torch.bfloat16, device="cuda")
    remote_row = i32([0] * assignments)
    pointers = (ctypes.c_void_p * 1)(receive.data_ptr())
    torch.cuda.synchronize()
    assert library.mircuda_b200_moe_dispatch_rows_bf16(
        p(source), p(source_index), p(sorted_expert), p(position), p(base_for_me),
        ctypes.cast(pointers, ctypes.POINTER(ctypes.c_void_p)), 1, p(remote_row), assignments, experts,
        columns, capacity, handle) == 0
    cuda_stream.synchronize()
    assert remote_row.tolist() == [0, 1, -1, -1, 2, 3]
    assert torch.equal(receive[:4], source[[0, 1, 4, 5]])
    assert (receive[4:] == -7.0).all()
    # The way back: three tokens of two choices; token 1 owns the two skipped rows, token 2's second
    # slot points past the assignments.
    tokens, top_k = 3, 2
    slot = i32([0, 1, 2, 3, 4, 1000])
    weights = torch.full((tokens, top_k), 0.5, dtype=torch.float32, device="cuda")
    output = torch.full((tokens, columns), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert library.mircuda_b200_moe_collect_rows_bf16(
        ctypes.cast(pointers, ctypes.POINTER(ctypes.c_void_p)), 1, p(slot), p(sorted_expert), p(remote_row),
        p(weights), p(output), tokens, top_k, experts, columns, handle) == 0
    cuda_stream.synchronize()
    rows = source.float()
    expected = torch.stack([0.5 * (rows[0] + rows[1]), torch.zeros(columns, device="cuda"), 0.5 * rows[4]])
    assert torch.equal(output.float(), expected.to(torch.bfloat16).float())


def test_layer_reports_an_exceeded_capacity(cuda_stream):
    """The layer turns the device-side overflow word into CapacityExceeded and stays usable."""
    from mircuda_b200 import moe
    device = torch.device("cuda", torch.cuda.current_device())
    x, gate_up, down, logits = make_inputs(device)
    chosen, weights = moe.route(logits, TOP_K)
    dispatch = moe.plan_dispatch(chosen, EXPERTS, 1, None, 1)
    bank = moe.ExpertWeights(cuda_stream, gate_up, down, False)
    layer = moe.ExpertParallelMoe(cuda_stream, HIDDEN, INTERMEDIATE, EXPERTS, TOP_K, TOKENS, 128, bank)
    torch.cuda.synchronize()
    out = layer.forward(x, dispatch, weights)                 # 192 routed rows, room for 128
    with pytest.raises(moe.CapacityExceeded):
        layer.check()
    assert torch.isfinite(out.float()).all()
    layer.close()


def test_gate_up_epilogue_fusion_matches_two_passes(cuda_stream):
    """gate_up with SwiGLU and the NVFP4 requantisation in its epilogue (gate and up rows of the
    bank interleaved in runs of 16) against the plain grouped product on the [gate | up] bank
    followed by the fused SwiGLU quantiser: same codes and scales, bit for bit, for every row a
    group owns; rows no group owns are left alone."""
    import ctypes
    from mircuda_b200 import _lib, plans, plans_fp4
    library = _lib.load()
    experts, intermediate, hidden = 5, 192, 256
    rows = [130, 0, 77, 128, 1]
    offsets = [0, 256, 256, 384, 512]                 # every group starts on a 128-row tile
    capacity = 640
    generator = torch.Generator(device="cuda").manual_seed(321)
    bank = (torch.randn(experts, 2 * intermediate, hidden, generator=generator, device="cuda") * 0.05).to(torch.bfloat16)
    gate = bank[:, :intermediate].reshape(experts, intermediate // 16, 16, hidden)
    up = bank[:, intermediate:].reshape(experts, intermediate // 16, 16, hidden)
    interleaved = torch.cat([gate, up], dim=2).reshape(experts * 2 * intermediate, hidden).contiguous()
    x = torch.randn(capacity, hidden, generator=generator, device="cuda").to(torch.bfloat16)
    torch.cuda.synchronize()
    a_codes, a_scales, a_global = plans.nvfp4_quantize_bf16(cuda_stream, x)
    plain_codes, plain_scales, bank_global = plans.nvfp4_quantize_bf16(cuda_stream, bank.view(-1, hidden))
    fused_codes, fused_scales, fused_global = plans.nvfp4_quantize_bf16(cuda_stream, interleaved)
    cuda_stream.synchronize()
    assert float(bank_global) == float(fused_global)
    alphas = (bank_global * a_global).expand(experts).contiguous()
    words = lambda values: torch.tensor(values, dtype=torch.int32, device="cuda")
    indices, rows_d, offsets_d = words(list(range(experts))), words(rows), words(offsets)
    p = lambda tensor: ctypes.c_void_p(tensor.data_ptr())
    handle = ctypes.c_void_p(cuda_stream.cuda_stream)
    raw = ctypes.c_void_p()
    assert library.mircuda_variable_grouped_fp4_create(experts, experts, capacity, 2 * intermediate, hidden,
                                                       handle, ctypes.byref(raw)) == 0
    hidden_states = torch.zeros(capacity, 2 * intermediate, dtype=torch.bfloat16, device="cuda")
    out_global = torch.full((1,), 0.0042, dtype=torch.float32, device="cuda")
    scale_bytes = capacity // 128 * (intermediate // 64) * 512
    expected_codes = torch.zeros(capacity * intermediate // 2, dtype=torch.uint8, device="cuda")
    expected_scales = torch.zeros(scale_bytes, dtype=torch.uint8, device="cuda")
    actual_codes = torch.full((capacity * intermediate // 2,), 0xEE, dtype=torch.uint8, device="cuda")
    actual_scales = torch.full((scale_bytes,), 0xEE, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    assert library.mircuda_variable_grouped_fp4_execute(
        raw, handle, p(a_codes), p(a_scales), p(plain_codes), p(plain_scales), p(alphas), p(indices),
        p(rows_d), p(offsets_d), p(offsets_d), p(hidden_states)) == 0
    assert library.mircuda_b200_moe_swiglu_nvfp4(p(hidden_states), p(out_global), p(expected_codes),
                                                 p(expected_scales), capacity, None, intermediate, handle) == 0
    for _ in range(2):
        assert library.mircuda_b200_variable_grouped_fp4_execute_swiglu(
            raw, handle, p(a_codes), p(a_scales), p(fused_codes), p(fused_scales), p(alphas), p(indices),
            p(rows_d), p(offsets_d), p(offsets_d), p(out_global), p(actual_codes), p(actual_scales)) == 0
    cuda_stream.synchronize()
    library.mircuda_variable_grouped_fp4_destroy(raw)
    import oracle
    owned = np.zeros(capacity, bool)
    for count, first in zip(rows, offsets):
        owned[first:first + count] = True
    expected = expected_codes.cpu().numpy().reshape(capacity, intermediate // 2)
    actual = actual_codes.cpu().numpy().reshape(capacity, intermediate // 2)
    assert np.array_equal(actual[owned], expected[owned])
    assert (actual[~owned] == 0xEE).all()
    assert actual[owned].any()
    positions = oracle.fp4_scale_offsets(capacity, intermediate)          # [capacity, intermediate / 16]
    expected_bytes, actual_bytes = expected_scales.cpu().numpy(), actual_scales.cpu().numpy()
    assert np.array_equal(actual_bytes[positions[owned]], expected_bytes[positions[owned]])
    assert (actual_bytes[positions[~owned]] == 0xEE).all()


def test_layer_with_and_without_epilogue_fusion(cuda_stream):
    """The NVFP4 layer gives the same output, bit for bit, with the fused gate_up epilogue and
    with the separate SwiGLU quantiser."""
    from mircuda_b200 import moe
    device = torch.device("cuda", torch.cuda.current_device())
    x, gate_up, down, logits = make_inputs(device)
    chosen, weights = moe.route(logits, TOP_K)
    dispatch = moe.plan_dispatch(chosen, EXPERTS, 1, None, 128)
    capacity = (TOKENS * TOP_K + 128 * EXPERTS) // 128 * 128
    bank = moe.ExpertWeights(cuda_stream, gate_up, down, True)
    assert bank.fused
    layer = moe.ExpertParallelMoe(cuda_stream, HIDDEN, INTERMEDIATE, EXPERTS, TOP_K, TOKENS, capacity, bank)
    layer.calibrate(x, dispatch, weights)
    torch.cuda.synchronize()
    outputs = []
    for fuse in (True, False):
        layer.fuse_swiglu = fuse
        outputs.append(layer.forward(x, dispatch, weights).clone())
        cuda_stream.synchronize()
    assert torch.equal(outputs[0], outputs[1])
    layer.close()
