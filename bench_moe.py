"""Grouped MoE benchmark: Qwen3-30B-A3B-shaped feed-forward (128 experts, top-8, hidden 2048,
expert intermediate 768, 4096 tokens) as bf16 and as NVFP4, experts sharded over the GPUs.

    python bench_moe.py [--mode bf16|nvfp4|both] [--steps K] [--warmup W]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        bench_moe.py --mode bf16

Inputs are synthetic and seeded (seed 5000 + index): activations N(0,1), expert weights
N(0,0.02), router logits N(0,1) -> softmax -> top-8 -> renormalised. The total token count is
fixed (strong scaling): each of N ranks routes 4096/N tokens and owns 128/N experts. A step is
the whole layer of `mircuda_b200.moe` (count exchange, dispatch of the routed rows to the
experts' owners, two grouped GEMMs with SwiGLU between them, weighted collection of the
results); the router's output is prepared once, outside the timed region. One JSON line per
mode: `value` = 2*assignments*(gate_up + down) flop of all ranks over the step time (max over
ranks, CUDA events, no other instrumentation in that loop); `gemm` = the same flop over the
summed durations of the two grouped GEMM launches on rank 0 (the grouped kernel alone, from a
second loop with an event pair around every stage); the bytes a rank moves over NVLink each way are
reported beside them.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

from mircuda_b200 import moe  # noqa: E402

EXPERTS, TOP_K, HIDDEN, INTERMEDIATE, TOKENS = 128, 8, 2048, 768, 4096


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--mode", default="both", choices=["bf16", "nvfp4", "both"])
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--transport", default="peer", choices=["peer", "nccl"],
                        help="peer: this library's dispatch/collect kernels over NVLink peer memory; "
                             "nccl: all_to_all_single of padded blocks")
    parser.add_argument("--graph", action="store_true",
                        help="replay the step from a CUDA graph (no host launch cost; the grouped "
                             "GEMMs are then not timed separately)")
    args = parser.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.graph and world > 1:
        # Capturing the cross-GPU barrier and the count all-gather did not complete when tried
        # on two GPUs; the graph option is for the single-GPU layer only.
        raise SystemExit("--graph is only supported on one GPU")
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    stream = torch.cuda.Stream()
    local_tokens, local_experts = TOKENS // world, EXPERTS // world

    with torch.cuda.stream(stream):
        generator = torch.Generator(device=device).manual_seed(5000)
        # Every rank draws the full token batch and router so that the shards agree; the expert
        # banks are drawn per expert from their own seeds and only the local ones are kept.
        x_all = torch.randn(TOKENS, HIDDEN, generator=generator, device=device).to(torch.bfloat16)
        logits = torch.randn(TOKENS, EXPERTS, generator=generator, device=device)
        x = x_all[rank * local_tokens:(rank + 1) * local_tokens].contiguous()
        gate_up = torch.empty(local_experts, 2 * INTERMEDIATE, HIDDEN, dtype=torch.bfloat16, device=device)
        down = torch.empty(local_experts, HIDDEN, INTERMEDIATE, dtype=torch.bfloat16, device=device)
        for index in range(local_experts):
            expert = rank * local_experts + index
            local_generator = torch.Generator(device=device).manual_seed(5001 + expert)
            gate_up[index] = (torch.randn(2 * INTERMEDIATE, HIDDEN, generator=local_generator, device=device) * 0.02).to(torch.bfloat16)
            down[index] = (torch.randn(HIDDEN, INTERMEDIATE, generator=local_generator, device=device) * 0.02).to(torch.bfloat16)
        chosen, weights = moe.route(logits[rank * local_tokens:(rank + 1) * local_tokens], TOP_K)
    stream.synchronize()

    modes = ["bf16", "nvfp4"] if args.mode == "both" else [args.mode]
    for mode in modes:
        nvfp4 = mode == "nvfp4"
        if nvfp4 and world > 1 and args.transport != "peer":
            if rank == 0:
                print(json.dumps({"metric": "moe_grouped_gemm_tflops", "mode": mode, "n_gpus": world,
                                  "unavailable": "NVFP4 expert parallelism uses the peer transport"}),
                      flush=True)
            continue
        align = 128 if nvfp4 else 1
        dispatch = moe.plan_dispatch(chosen, EXPERTS, world, None, align)
        largest = torch.tensor([dispatch.largest_block], device=device)
        if world > 1:
            dist.all_reduce(largest, op=dist.ReduceOp.MAX)
        capacity = (int(largest.item()) + 127) // 128 * 128
        dispatch = moe.plan_dispatch(chosen, EXPERTS, world, capacity, align)
        peer = args.transport == "peer"
        if peer:
            # Rows this rank will receive = everyone's counts for its experts, every expert
            # rounded up to `align` rows (set-up time read).
            totals = dispatch.counts.clone()
            if world > 1:
                dist.all_reduce(totals)
            totals = (totals + align - 1) // align * align
            received = totals.view(world, local_experts).sum(dim=1).max()
            capacity = (int(received.item()) + 127) // 128 * 128
        bank = moe.ExpertWeights(stream, gate_up, down, nvfp4)
        layer = moe.ExpertParallelMoe(stream, HIDDEN, INTERMEDIATE, EXPERTS, TOP_K, local_tokens,
                                      capacity, bank, transport=args.transport)
        if nvfp4:
            layer.calibrate(x, dispatch, weights)

        def barrier():
            stream.synchronize()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        for _ in range(args.warmup):
            layer.forward(x, dispatch, weights)
        barrier()
        graph = None
        if args.graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                layer.forward(x, dispatch, weights)
            with torch.cuda.stream(stream):
                graph.replay()
            barrier()
        # The layer is timed without instrumentation; a second loop of the same length records an
        # event pair around every stage for the per-stage and per-GEMM figures.
        layer.gemm_events = None
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            begin.record(stream)
            for _ in range(args.steps):
                if graph is not None:
                    graph.replay()
                else:
                    layer.forward(x, dispatch, weights)
            end.record(stream)
        barrier()
        elapsed_ms = begin.elapsed_time(end)
        if graph is None:
            layer.gemm_events = []
            with torch.cuda.stream(stream):
                for _ in range(args.steps):
                    layer.forward(x, dispatch, weights)
            barrier()
        if world > 1:
            tensor = torch.tensor([elapsed_ms], device=device)
            dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
            elapsed_ms = float(tensor.item())
        ms_per_step = elapsed_ms / args.steps
        assignments = TOKENS * TOP_K
        flops = {"gate_up": 2.0 * assignments * 2 * INTERMEDIATE * HIDDEN,
                 "down": 2.0 * assignments * HIDDEN * INTERMEDIATE}
        per_kernel = {}
        for name, start, stop in (layer.gemm_events or []):
            per_kernel.setdefault(name, []).append(start.elapsed_time(stop))
        # Rank 0's launches cover 1/world of the flop (experts and rows are balanced on average).
        gemm_ms = {name: sum(times) / len(times) for name, times in per_kernel.items()}
        line = {
            "metric": "moe_grouped_gemm_tflops", "mode": mode, "n_gpus": world,
            "transport": "peer" if peer else ("nccl" if world > 1 else "local"), "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step,
            "value": sum(flops.values()) / (ms_per_step * 1e-3) / 1e12, "unit": "TFLOP/s",
            "scaling": "strong", "data": "synthetic",
            "gemm": {name: {"ms": gemm_ms[name],
                            "tflops_per_gpu": flops[name] / world / (gemm_ms[name] * 1e-3) / 1e12}
                     for name in gemm_ms if name in flops},
            "gemm_tflops_all_gpus": (sum(flops.values()) / (sum(gemm_ms[name] for name in flops) * 1e-3) / 1e12
                                     if gemm_ms else None),
            "stage_ms_rank0": {name: round(value, 4) for name, value in gemm_ms.items() if name not in flops},
            "cuda_graph": bool(args.graph),
            # NVFP4: SwiGLU and the requantisation run inside the gate_up epilogue (its time then
            # includes them and no separate stage exists)
            "fused_gate_up_epilogue": bool(nvfp4 and layer.static_scales and bank.fused and layer.fuse_swiglu),
            "config": {"workload": "qwen3-30b-a3b moe feed-forward", "experts": EXPERTS, "top_k": TOP_K,
                       "hidden": HIDDEN, "intermediate": INTERMEDIATE, "tokens": TOKENS,
                       "capacity_rows": capacity,
                       "remote_bytes_per_rank_dispatch":
                           (world - 1) * (TOKENS * TOP_K // world // world if peer else capacity)
                           * (HIDDEN * 9 // 16 if nvfp4 else HIDDEN * 2),
                       "remote_bytes_per_rank_collect":
                           (world - 1) * (TOKENS * TOP_K // world // world if peer else capacity) * HIDDEN * 2},
        }
        if rank == 0:
            print(json.dumps(line), flush=True)
        layer.close()
        del layer, bank
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
