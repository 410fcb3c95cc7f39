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
        layer.calibrate(x)
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


@pytest.mark.parametrize("transport", ["peer", "nccl"])
def test_moe_layer_nvfp4_single_gpu(cuda_stream, transport):
    """Two NVFP4 quantisations (activations and weights, twice) sit between this result and the
    unquantised restatement, so this is a plausibility bound; the grouped NVFP4 kernel itself
    is checked against the oracle elsewhere."""
    out, expected = run_single(cuda_stream, True, transport)
    assert torch.isfinite(out).all()
    error = (out - expected).norm() / expected.norm()
    assert error < 0.25, error


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
            layer.calibrate(x[local])
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
