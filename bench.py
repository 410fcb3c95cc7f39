"""Benchmark of the MXFP8 prefill hot path on B200.

Workload (the configuration the headline metric is quoted on): the four Qwen3-8B-shaped
prefill linears at M = 4096 tokens — QKV (N=6144, K=4096), O (4096, 4096), gate_up
(24576, 4096), down (4096, 12288) — each as "quantize bf16 activations to MXFP8 on the fly,
then block-scaled GEMM against MXFP8 weights" (``MxFp8TensorCore.execute``). One step is one
pass over all four: 4 quantizer launches + 4 GEMM launches, 1580.5 GFLOP. Synthetic seeded
data: activations ~N(0,1), weights ~N(0,0.02), bf16, weights quantized once up front.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Prints one JSON line. ``value`` is device-resident throughput (GEMM flops of a step over
the step time, quantizers included). The ``--steps`` loop is timed as one region and repeated
until about two seconds of timed work have run, so that the clocks settle under the power cap
and dozens of clock samples land inside; ``ms_per_step`` is the median repeat (min and max are
printed beside it). ``e2e`` is the same through the public API with host buffers (pinned), H2D
of every activation and D2H of every output inside the timed region. At one GPU the line also
carries ``decode`` (the bf16 x NVFP4 decode GEMV at the same four weight shapes, M in {1,4,8},
HBM GB/s: the other half of the headline metric) and ``reference_kernels`` (the reference's own
sm_100a-runnable kernels timed beside this library's for the same op).
With N > 1 the weight N dimension is column-sharded across ranks and outputs are
all-gathered (strong scaling). ``--impl reference`` times the CPU restatement of the
reference's dequantize-then-matmul on the host cores (the reference has no CPU
implementation of this path and its GPU kernels are sm_120-only).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

NOMINAL_FP8_TFLOPS = 4500.0        # dense FP8 of one B200, vendor figure
NVLINK_GBS_PER_DIRECTION = 900.0   # NVLink 5, per GPU and direction, vendor figure
TIMED_REGION_SECONDS = 2.0         # the --steps loop is repeated until this much has been timed

SHAPES = [  # name, N, K
    ("qkv", 6144, 4096),
    ("o", 4096, 4096),
    ("gate_up", 24576, 4096),
    ("down", 4096, 12288),
]
TOKENS = 4096
METRIC = "mxfp8_prefill_gemm_tflops"
UNIT = "TFLOP/s"
WORKLOAD = "qwen3-8b prefill linears, MXFP8 W8A8 with on-the-fly activation quantization"


def step_flops(tokens: int = TOKENS) -> float:
    return sum(2.0 * tokens * n * k for _, n, k in SHAPES)


def measured_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text())
    return {}


# ----------------------------------------------------------------------------- reference arm

def run_reference(args) -> None:
    """CPU dequantize-then-matmul (the oracle port) on a bounded sample of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    import oracle

    sample_rows = 128
    rng = np.random.default_rng(1000)
    weights = []
    for _, n, k in SHAPES:      # weights dequantized once (one-time prep, not timed)
        w = oracle.f32_to_bf16((rng.standard_normal((n, k), dtype=np.float32) * 0.02))
        codes, scales = oracle.mxfp8_quantize(w)
        weights.append(oracle.mxfp8_dequantize(codes, scales))
    activations = [oracle.f32_to_bf16(rng.standard_normal((sample_rows, k), dtype=np.float32))
                   for _, _, k in SHAPES]
    flops = step_flops(sample_rows)

    def one_step():
        for x, w in zip(activations, weights):
            codes, scales = oracle.mxfp8_quantize(x)
            oracle.f32_to_bf16(oracle.mxfp8_dequantize(codes, scales) @ w.T)

    for _ in range(min(args.warmup, 1)):
        one_step()
    steps = max(1, args.steps)
    begin = time.perf_counter()
    for _ in range(steps):
        one_step()
    elapsed = (time.perf_counter() - begin) / steps
    value = flops / elapsed / 1e12
    cores = os.cpu_count() or 1
    sample = f"first {sample_rows} of {TOKENS} token rows of all four linears per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT,
        "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 1),
        "ms_per_step": elapsed * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "tokens": TOKENS, "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def cpu_baseline_leg() -> dict:
    """The oracle port timed on the host cores on a bounded sample (rank 0, N = 1 only)."""
    import numpy as np
    import oracle

    sample_rows = 128
    rng = np.random.default_rng(1000)
    total_time = 0.0
    for _, n, k in SHAPES:
        w = oracle.f32_to_bf16((rng.standard_normal((n, k), dtype=np.float32) * 0.02))
        codes, scales = oracle.mxfp8_quantize(w)
        w_f32 = oracle.mxfp8_dequantize(codes, scales)
        x = oracle.f32_to_bf16(rng.standard_normal((sample_rows, k), dtype=np.float32))
        best = None
        for _ in range(3):
            begin = time.perf_counter()
            x_codes, x_scales = oracle.mxfp8_quantize(x)
            oracle.f32_to_bf16(oracle.mxfp8_dequantize(x_codes, x_scales) @ w_f32.T)
            elapsed = time.perf_counter() - begin
            best = elapsed if best is None else min(best, elapsed)
        total_time += best
    return {
        "value": step_flops(sample_rows) / total_time / 1e12, "unit": UNIT,
        "cores": os.cpu_count() or 1, "kind": "port",
        "sample": (f"first {sample_rows} of {TOKENS} token rows of all four linears, weights "
                   "dequantized once outside the timed region, best of 3"),
    }


# ------------------------------------------------------------------------------- GPU arm

def fp8_peak_probe(torch, stream) -> dict | None:
    """Measured dense FP8 tensor peak of this GPU: cuBLASLt E4M3 x E4M3 -> bf16 at 8192^3 through
    `torch._scaled_mm` with per-tensor scales (a library GEMM, used only as the roofline's
    denominator, outside every timed region of the benchmark). `burst` is the best single call
    after a pause, `sustained` the rate of a loop about two seconds long under the power cap.
    Returns None when the call is not available."""
    try:
        size = 8192
        with torch.cuda.stream(stream):
            a = (torch.randn(size, size, device="cuda") * 0.5).to(torch.float8_e4m3fn)
            b = (torch.randn(size, size, device="cuda") * 0.5).to(torch.float8_e4m3fn).t()
            one = torch.ones((), device="cuda")
            flops = 2.0 * size ** 3
            for _ in range(3):
                torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            stream.synchronize()
            best = None
            for _ in range(10):
                time.sleep(0.02)
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record(stream)
                torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
                stop.record(stream)
                stream.synchronize()
                elapsed = start.elapsed_time(stop)
                best = elapsed if best is None else min(best, elapsed)
            calls = max(20, int(2000.0 / best))
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(stream)
            for _ in range(calls):
                torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            stop.record(stream)
            stream.synchronize()
            sustained_ms = start.elapsed_time(stop) / calls
        return {"burst": flops / (best * 1e-3) / 1e12, "sustained": flops / (sustained_ms * 1e-3) / 1e12,
                "how": f"torch._scaled_mm (cuBLASLt) e4m3 x e4m3 -> bf16, {size}^3, per-tensor scales: "
                       f"best of 10 single calls (burst), {calls} calls back to back (sustained)"}
    except Exception as error:  # noqa: BLE001 - the probe is optional
        print(f"fp8 peak probe unavailable: {error}", file=sys.stderr, flush=True)
        return None


def run_gpu(args) -> None:
    import torch
    import torch.distributed as dist

    from mircuda_b200 import gather, plans, sharding

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    distributed = world > 1
    if distributed:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    stream = torch.cuda.Stream()
    device = torch.device("cuda", local_rank)

    # N > 1: the all-gather is fused into the GEMM epilogue, which stores every tile into each
    # rank's full-width [TOKENS, N] buffer over NVLink (peer pointers from symmetric memory);
    # no separate collective kernel competes with the persistent GEMM for SMs. If symmetric
    # memory cannot be set up on any rank, every rank falls back to an NCCL all-gather after
    # the GEMM, and the JSON line says so.
    fused = distributed
    if distributed:
        try:
            probe = gather.SymmetricOutput(8, 8, device)
            probe.barrier()
            torch.cuda.synchronize()
            ok = 1
        except Exception as error:  # noqa: BLE001 - any set-up failure selects the NCCL path
            print(f"rank {rank}: symmetric memory unavailable ({error}); using NCCL all-gather",
                  file=sys.stderr, flush=True)
            ok = 0
        flag = torch.tensor([ok], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        fused = bool(flag.item())

    layers = []
    with torch.cuda.stream(stream):
        for index, (name, n, k) in enumerate(SHAPES):
            begin, end = sharding.column_shard(n, world, rank)
            local_n = end - begin
            generator = torch.Generator(device=device).manual_seed(2000 + index)
            # Only this rank's weight rows are materialised; the seed makes the full matrix
            # well defined (rows are drawn shard by shard in rank order).
            weight = (torch.randn(local_n, k, generator=generator, device=device) * 0.02).to(torch.bfloat16)
            codes = torch.empty(local_n * k, dtype=torch.uint8, device=device)
            scales = torch.zeros(plans.scale_bytes(local_n, k // 32), dtype=torch.uint8, device=device)
            plans.mxfp8_quantize_bf16(stream, weight, codes, scales)
            del weight
            generator = torch.Generator(device=device).manual_seed(1000 + index)
            x = torch.randn(TOKENS, k, generator=generator, device=device).to(torch.bfloat16)
            spec = plans.MxFp8Spec(TOKENS, k, local_n)
            operation = plans.MxFp8TensorCore(stream, spec)
            out = torch.empty(TOKENS * local_n, dtype=torch.bfloat16, device=device)
            full = gather.SymmetricOutput(TOKENS, n, device) if fused else None
            gathered = (torch.empty(world * TOKENS * local_n, dtype=torch.bfloat16, device=device)
                        if distributed and not fused else None)
            layers.append(dict(name=name, n=n, k=k, local_n=local_n, begin=begin, end=end, x=x,
                               codes=codes, scales=scales, op=operation, out=out, full=full,
                               gathered=gathered))
    stream.synchronize()

    gemm_events: list[tuple] = []
    # MIRCUDA_B200_GATHER=multimem writes every piece once through the buffers' NVSwitch
    # multicast address instead of once per rank. Measured at 4 GPUs it is 5 % slower than the
    # per-rank stores (the receiving side, not this GPU's egress, is the limit), so it is opt-in.
    use_multicast = os.environ.get("MIRCUDA_B200_GATHER", "peer") == "multimem"
    # MIRCUDA_B200_GATHER=copy: the GEMM writes the rank's own full-width buffer only and the copy
    # engines send each finished column block to the peers while the next layer computes.
    # MIRCUDA_B200_GATHER=blocks: the copy engines again, with the gathered result in rank-major
    # blocks ([world, TOKENS, N / world], what an all-gather call returns) so that every copy is
    # contiguous; the quantizer of a following layer reads that layout in place.
    gather_mode = os.environ.get("MIRCUDA_B200_GATHER", "peer")
    copier = gather.ColumnCopier(world, rank) if fused and gather_mode in ("copy", "blocks") else None
    blocked = copier is not None and gather_mode == "blocks"
    if blocked:
        for layer in layers:
            if layer["local_n"] * world != layer["n"]:
                raise SystemExit("MIRCUDA_B200_GATHER=blocks needs equal shards")
            layer["full"] = gather.SymmetricOutput(world * TOKENS, layer["local_n"], device)
        torch.cuda.synchronize()
    multicast_active = bool(fused and use_multicast and all(layer["full"].multicast for layer in layers))

    def one_step(record: bool):
        for layer in layers:
            op = layer["op"]
            plans.mxfp8_quantize_bf16(stream, layer["x"], op.scratch.quantized_input,
                                      op.scratch.input_scales)
            if record:
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record(stream)
            if blocked:
                copier.execute_blocks(op.plan, stream, op.scratch.quantized_input, op.scratch.input_scales,
                                      layer["codes"], layer["scales"], layer["full"])
            elif copier is not None:
                copier.execute(op.plan, stream, op.scratch.quantized_input, op.scratch.input_scales,
                               layer["codes"], layer["scales"], layer["full"], layer["begin"], layer["end"])
            elif fused:
                gather.execute_gather(op.plan, stream, op.scratch.quantized_input,
                                      op.scratch.input_scales, layer["codes"], layer["scales"],
                                      layer["full"], layer["begin"], use_multicast)
            else:
                op.plan.execute(stream, op.scratch.quantized_input, op.scratch.input_scales,
                                layer["codes"], layer["scales"], layer["out"])
            if record:
                stop.record(stream)
                gemm_events.append((layer["name"], start, stop))
            if distributed and not fused:
                with torch.cuda.stream(stream):
                    dist.all_gather_into_tensor(layer["gathered"], layer["out"])
        if fused:
            # The step ends when every rank's stores (or copies) have landed everywhere.
            if copier is not None:
                copier.join(stream)
            with torch.cuda.stream(stream):
                layers[-1]["full"].barrier()

    def barrier():
        stream.synchronize()
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    from bench_decode import ClockSampler

    warm_begin, warm_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    one_step(False)
    barrier()
    warm_begin.record(stream)
    for _ in range(max(args.warmup - 1, 2)):
        one_step(False)
    warm_end.record(stream)
    barrier()
    estimate_ms = warm_begin.elapsed_time(warm_end) / max(args.warmup - 1, 2)
    # Repeats of the K-step loop: enough for TIMED_REGION_SECONDS of timed work in total, the same
    # count on every rank.
    repeats = max(1, min(2000, math.ceil(TIMED_REGION_SECONDS * 1e3 / max(estimate_ms * args.steps, 1e-3))))
    if args.repeats > 0:
        repeats = args.repeats
    if distributed:
        tensor = torch.tensor([repeats], device=device)
        dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
        repeats = int(tensor.item())
    # Plain repeats give `value`; after every fourth one an extra repeat carries an event pair
    # around every GEMM launch (the roofline's per-kernel durations), so that those events do not
    # sit inside the regions `value` is taken from.
    regions, instrumented = [], 0
    with ClockSampler(local_rank) as sampler:
        for repeat in range(repeats):
            begin_event, end_event = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            begin_event.record(stream)
            for _ in range(args.steps):
                one_step(False)
            end_event.record(stream)
            barrier()
            regions.append((begin_event, end_event))
            if repeat % 4 == 0:
                for _ in range(args.steps):
                    one_step(True)
                barrier()
                instrumented += 1
    region_ms = torch.tensor([begin.elapsed_time(end) for begin, end in regions], device=device)
    if distributed:
        dist.all_reduce(region_ms, op=dist.ReduceOp.MAX)      # each repeat: the slowest rank
    region_ms = region_ms.tolist()
    ms_per_step = statistics.median(region_ms) / args.steps
    value = step_flops() / (ms_per_step * 1e-3) / 1e12
    clocks = sampler.summary()

    gemm_ms = sum(start.elapsed_time(stop) for _, start, stop in gemm_events)
    per_layer = {}
    for name, start, stop in gemm_events:
        per_layer.setdefault(name, []).append(start.elapsed_time(stop))
    local_flops = sum(2.0 * TOKENS * layer["local_n"] * layer["k"] for layer in layers)
    achieved = local_flops * args.steps * instrumented / (gemm_ms * 1e-3) / 1e12
    peaks = measured_peaks()
    probe = fp8_peak_probe(torch, stream) if (world == 1 and not args.no_peak_probe) else None
    begin_event, end_event = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    # ------------------------------------------------------------------ end-to-end leg
    e2e_steps = max(1, min(args.steps, 10))
    host_in = [torch.empty(TOKENS, layer["k"], dtype=torch.bfloat16).pin_memory() for layer in layers]
    for host, layer in zip(host_in, layers):
        host.copy_(layer["x"])
    host_out = [torch.empty(TOKENS * layer["local_n"], dtype=torch.bfloat16).pin_memory()
                for layer in layers]
    h2d = sum(t.numel() * 2 for t in host_in)
    d2h = sum(t.numel() * 2 for t in host_out)

    # Three streams: the copies in, the quantizer + GEMM, the copies out. PCIe carries both
    # directions at once, so a layer's result leaves while the next layer's input arrives and
    # the GEMMs run under both; events order each buffer's reuse (x is free once its layer has
    # run, a result buffer once its copy out has finished).
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    arrived = [torch.cuda.Event() for _ in layers]
    x_free = [torch.cuda.Event() for _ in layers]
    computed = [torch.cuda.Event() for _ in layers]
    out_free = [torch.cuda.Event() for _ in layers]
    for index in range(len(layers)):
        x_free[index].record(stream)
        out_free[index].record(stream)

    def e2e_step():
        for index, (host, out_host, layer) in enumerate(zip(host_in, host_out, layers)):
            op = layer["op"]
            with torch.cuda.stream(copy_in):
                copy_in.wait_event(x_free[index])
                layer["x"].copy_(host, non_blocking=True)
                arrived[index].record(copy_in)
            with torch.cuda.stream(stream):
                stream.wait_event(arrived[index])
                stream.wait_event(out_free[index])
                if fused:
                    plans.mxfp8_quantize_bf16(stream, layer["x"], op.scratch.quantized_input,
                                              op.scratch.input_scales)
                    if blocked:
                        copier.execute_blocks(op.plan, stream, op.scratch.quantized_input,
                                              op.scratch.input_scales, layer["codes"], layer["scales"],
                                              layer["full"])
                        copier.join(stream)
                    elif copier is not None:
                        copier.execute(op.plan, stream, op.scratch.quantized_input, op.scratch.input_scales,
                                       layer["codes"], layer["scales"], layer["full"], layer["begin"],
                                       layer["end"])
                        copier.join(stream)
                    else:
                        gather.execute_gather(op.plan, stream, op.scratch.quantized_input,
                                              op.scratch.input_scales, layer["codes"], layer["scales"],
                                              layer["full"], layer["begin"], use_multicast)
                    layer["full"].barrier()
                else:
                    # MxFp8TensorCore.execute: the quantizer and the GEMM, the call a user makes.
                    op.execute(stream, layer["x"].view(-1), layer["codes"], layer["scales"], layer["out"])
                    if distributed:
                        dist.all_gather_into_tensor(layer["gathered"], layer["out"])
                x_free[index].record(stream)
                computed[index].record(stream)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(computed[index])
                if fused:
                    # Each rank reads back its own column block of the gathered result; only
                    # this rank's GEMM writes those columns.
                    own = (layer["full"].matrix()[rank * TOKENS:(rank + 1) * TOKENS] if blocked
                           else layer["full"].matrix()[:, layer["begin"]:layer["end"]])
                    out_host.view(TOKENS, layer["local_n"]).copy_(own, non_blocking=True)
                else:
                    out_host.copy_(layer["out"], non_blocking=True)
                out_free[index].record(copy_out)

    def e2e_join():
        # The timed region ends when the last copy out has landed.
        for event in out_free:
            stream.wait_event(event)

    if args.no_e2e:
        e2e_steps = 0
    else:
        e2e_step()
        e2e_join()
    barrier()
    begin_event.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    e2e_join()
    end_event.record(stream)
    barrier()
    e2e_ms = max(begin_event.elapsed_time(end_event), 1e-9)
    e2e_steps = max(e2e_steps, 1)
    if distributed:
        tensor = torch.tensor([e2e_ms], device=device)
        dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
        e2e_ms = float(tensor.item())
    e2e_value = step_flops() / (e2e_ms / e2e_steps * 1e-3) / 1e12

    # ------------------------------------------------ decode GEMV and reference-kernel legs
    decode_record, reference_records = None, None
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    hbm_source = ("measured copy bandwidth (MEASURED_PEAKS.json)" if "hbm_gbs" in peaks
                  else "fallback 6650 GB/s (an earlier measurement on this pool)")
    if world == 1 and not args.no_decode:
        import bench_decode
        with ClockSampler(local_rank) as decode_sampler:
            everything = bench_decode.run(["nvfp4", "fp4", "marlin", "w4a16", "mxfp8_wo", "fp4_gemm"], 200, 5, hbm_peak,
                                          sampler=decode_sampler, echo=False)["results"]
        results = [record for record in everything if record["op"] == "nvfp4"]
        fp4_results = [record for record in everything if record["op"] == "fp4"]
        fractions = [record["frac_of_measured_hbm"] for record in results]
        decode_record = {
            "op": "bf16 x NVFP4 GEMV (mircuda_b200_nvfp4_vector_*), Qwen3-8B weight shapes, M in {1,4,8}",
            "method": ("weights rotate through banks larger than 768 MiB, 200 back-to-back launches from a "
                       "CUDA graph between two events, median of 5 (examples/dense-vector.rs:9,133-141)"),
            "unit": "GB/s of algorithmic bytes (N*K*0.5625 + M*K*2 + M*N*2)",
            "peak_gbs": hbm_peak, "peak_source": hbm_source,
            "min_frac": min(fractions), "mean_frac": sum(fractions) / len(fractions),
            "clocks": decode_sampler.summary(),
            "launches": ("overlapped (programmatic dependent launch, the plans' default): a launch fetches "
                         "weights while the previous one finishes; activations and outputs stay ordered"),
            "results": [{key: record[key] for key in ("shape", "m", "us", "gbs", "frac_of_measured_hbm",
                                                      "banks", "sm_mhz", "clock_samples")}
                        for record in results],
            # the reference's own decode op, FP4 x FP4 at M = 1 (mircuda_fp4_vector_*), same method
            "fp4_vector_results": [{key: record[key] for key in ("shape", "m", "us", "gbs",
                                                                 "frac_of_measured_hbm", "banks", "sm_mhz")}
                                   for record in fp4_results],
            # the W4A16 decode paths: Marlin-layout NVFP4 (mircuda_marlin_nvfp4_dense_execute, M in
            # {1,4,8}) and int4-g128 (mircuda_b200_w4a16_*, M in {1,16}; M = 256 is a GEMM, in TFLOP/s)
            "marlin_results": [{key: record[key] for key in ("shape", "m", "us", "gbs",
                                                             "frac_of_measured_hbm", "banks", "sm_mhz")}
                               for record in everything if record["op"] == "marlin"],
            "w4a16_results": [{key: record[key] for key in ("shape", "m", "us", "gbs", "frac_of_measured_hbm",
                                                            "banks", "sm_mhz", "tflops") if key in record}
                              for record in everything if record["op"] == "w4a16"],
            # the weight-only MXFP8 projection (mircuda_b200_mxfp8_bf16; kernels/mxfp8.cu:111-217), M in {1,4,8}
            "mxfp8_weight_only_results": [{key: record[key] for key in ("shape", "m", "us", "gbs",
                                                                        "frac_of_measured_hbm", "banks", "sm_mhz")}
                                          for record in everything if record["op"] == "mxfp8_wo"],
            # the NVFP4 x NVFP4 prefill GEMM (mircuda_fp4_*) at M = 4096 and the same four weight shapes:
            # 20 launches from a graph per repeat, i.e. a burst figure (nominal dense FP4: 9000 TFLOP/s)
            "nvfp4_gemm_results": [{key: record[key] for key in ("shape", "m", "us", "tflops", "sm_mhz")
                                    if key in record}
                                   for record in everything if record["op"] == "fp4_gemm"],
        }
    if world == 1 and not args.no_reference_kernels:
        import bench_decode
        reference_records = bench_decode.reference_kernel_records(100, 3, hbm_peak)

    if rank == 0:
        timed_ms = sum(region_ms)
        sustained_regime = timed_ms >= 1000.0
        candidates = {}
        if probe is not None:
            candidates["fp8_probe_burst"] = probe["burst"]
            candidates["fp8_probe_sustained"] = probe["sustained"]
        if "bf16_tflops" in peaks:
            candidates["2x_bf16_burst"] = 2.0 * float(peaks["bf16_tflops"])
            candidates["2x_bf16_sustained"] = 2.0 * float(peaks["bf16_tflops_sustained"])
        if probe is not None:
            peak = probe["sustained"] if sustained_regime else probe["burst"]
            peak_note = ("measured FP8 tensor peak of this GPU, " + ("sustained" if sustained_regime else "burst")
                         + f" figure because the timed regions sum to {timed_ms:.0f} ms: " + probe["how"])
        elif "bf16_tflops" in peaks:
            peak = candidates["2x_bf16_sustained" if sustained_regime else "2x_bf16_burst"]
            peak_note = ("2 x measured " + ("sustained" if sustained_regime else "burst")
                         + " bf16 cuBLAS TFLOP/s of MEASURED_PEAKS.json (no FP8 probe in this run)")
        else:
            peak = NOMINAL_FP8_TFLOPS
            peak_note = "nominal dense FP8 (no measured peak available)"
        mhz = clocks["sm_mhz"]
        layer_table = {}
        for name, times in per_layer.items():
            layer = next(l for l in layers if l["name"] == name)
            mean_ms = statistics.mean(times)
            layer_table[name] = {
                "us": mean_ms * 1e3,
                "tflops": 2.0 * TOKENS * layer["local_n"] * layer["k"] / (mean_ms * 1e-3) / 1e12,
                # time x clock: a kernel change moves it, a clock change does not
                "us_x_mhz": mean_ms * 1e3 * mhz if mhz else None,
            }
        if distributed:
            received = (world - 1) / world * TOKENS * sum(n for _, n, _ in SHAPES) * 2.0
            roofline = {
                "bound": "nvlink", "achieved": received / (ms_per_step * 1e-3) / 1e9,
                "peak": NVLINK_GBS_PER_DIRECTION, "unit": "GB/s",
                "frac": received / (ms_per_step * 1e-3) / 1e9 / NVLINK_GBS_PER_DIRECTION,
                "traffic": None,
                "kernel": ("block_scaled_pair_gemm_kernel + one contiguous copy-engine copy per peer and layer"
                           if blocked else
                           "block_scaled_pair_gemm_kernel + one copy-engine 2-D copy per peer and layer"
                           if copier is not None else "block_scaled_pair_gemm_kernel (gather epilogue)"),
                "peak_source": ("nominal NVLink 5 ingress per GPU; measured on this pool: 770 GB/s peer copy, "
                                "555 GB/s for SM-issued peer stores"),
                "bytes_received_per_rank_per_step": received,
                "why": ("every rank must receive the other ranks' columns of all four outputs; with K = 4096 "
                        "that is one received byte per 4096 flop, so from 2 GPUs up the step is bound by "
                        "NVLink ingress, not by the tensor pipe"),
                "gemm_tflops_this_rank": achieved, "per_layer": layer_table,
            }
        else:
            roofline = {
                "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak,
                # dram__bytes_read.sum + dram__bytes_write.sum of the gate_up launch from the ncu
                # capture summarised under profiles/ (algorithmic 322.5 MB; 33 MB of C were still
                # dirty in L2 when the kernel ended). Not measured by this run.
                "traffic": 289.6e6, "traffic_launch": "gate_up (M=4096, N=24576, K=4096)",
                "traffic_source": "profiles/block_scaled_pair_gemm_kernel_gate_up_4096x24576x4096.md",
                "kernel": "block_scaled_pair_gemm_kernel",
                "peak_source": peak_note,
                "frac_of": {name: achieved / figure for name, figure in candidates.items()},
                "peaks_tflops": candidates,
                "frac_of_nominal_fp8_4500": achieved / NOMINAL_FP8_TFLOPS,
                "value_frac_of_nominal_fp8_4500": value / NOMINAL_FP8_TFLOPS,
                "per_layer": layer_table,
                "per_layer_tflops": {name: entry["tflops"] for name, entry in layer_table.items()},
            }
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step,
            "ms_per_step_min": min(region_ms) / args.steps, "ms_per_step_max": max(region_ms) / args.steps,
            "repeats": repeats, "timed_ms_total": timed_ms,
            "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)",
            "data": "synthetic",
            "config": {
                "workload": WORKLOAD, "tokens": TOKENS,
                "shapes": {name: [n, k] for name, n, k in SHAPES},
                "parallelism": (f"weight N column-sharded x{world}, outputs all-gathered into rank-major blocks "
                                f"[{world}, tokens, N/{world}]: each rank's finished block goes to the peers as "
                                "one contiguous copy-engine copy per peer while the next layer computes"
                                if blocked else
                                f"weight N column-sharded x{world}, each finished column block sent to the "
                                "peers by the copy engines while the next layer computes"
                                if copier is not None else
                                f"weight N column-sharded x{world}, all-gather fused into the GEMM "
                                "epilogue (" + ("multimem stores through NVSwitch multicast"
                                                if multicast_active else "peer stores over NVLink") + ")"
                                if fused else
                                f"weight N column-sharded x{world}, NCCL all-gather of outputs"
                                if distributed else "single GPU"),
                "l2": "per-step operands (193 MB of weights + activations + 318 MB of outputs) exceed the 126 MB L2",
                "timing": (f"the {args.steps}-step loop timed {repeats} times back to back (barrier + synchronize "
                           "around each), ms_per_step = median repeat / steps, max over ranks per repeat"),
            },
            "roofline": roofline,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e2e_steps},
            # launches of this library's kernels inside one timed region of `steps` steps
            "gpu_launches": args.steps * 2 * len(layers),
            "clocks": clocks,
        }
        if decode_record is not None:
            line["decode"] = decode_record
        if reference_records is not None:
            line["reference_kernels"] = {
                "what": ("the reference's own kernels that run on sm_100a (built from its sources into "
                         "oracle/_ref, reference launch geometry) timed beside this library's kernel for the "
                         "same op and inputs; rotating banks, CUDA-graph launches, median of 3"),
                "results": reference_records,
            }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_leg()
        print(json.dumps(line), flush=True)
    if distributed:
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    global SHAPES
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    parser.add_argument("--no-decode", action="store_true", help="skip the decode GEMV record")
    parser.add_argument("--no-reference-kernels", action="store_true",
                        help="skip timing the reference's own kernels from oracle/_ref")
    parser.add_argument("--no-peak-probe", action="store_true", help="skip the cuBLASLt FP8 peak probe")
    parser.add_argument("--repeats", type=int, default=0,
                        help="repeats of the timed --steps loop (default: enough for about 2 s)")
    parser.add_argument("--layers", default=",".join(name for name, _, _ in SHAPES),
                        help="comma-separated subset of the four linears (profiling runs)")
    args = parser.parse_args()
    chosen = args.layers.split(",")
    SHAPES = [shape for shape in SHAPES if shape[0] in chosen]
    if not SHAPES:
        raise SystemExit("--layers selected nothing")
    if args.impl == "reference":
        run_reference(args)
    else:
        args.warmup = max(args.warmup, 3)
        run_gpu(args)


if __name__ == "__main__":
    main()
