"""Benchmark of the MXFP8 prefill hot path on B200.

Workload (the configuration the headline metric is quoted on): the four Qwen3-8B-shaped
prefill linears at M = 4096 tokens — QKV (N=6144, K=4096), O (4096, 4096), gate_up
(24576, 4096), down (4096, 12288) — each as "quantize bf16 activations to MXFP8 on the fly,
then block-scaled GEMM against MXFP8 weights" (``MxFp8TensorCore.execute``). One step is one
pass over all four: 4 quantizer launches + 4 GEMM launches, 1580.5 GFLOP. Synthetic seeded
data: activations ~N(0,1), weights ~N(0,0.02), bf16, weights quantized once up front.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Prints one JSON line. ``value`` is device-resident throughput (GEMM flops of a step over
the step time, quantizers included); ``e2e`` is the same through the public API with host
buffers (pinned), H2D of every activation and D2H of every output inside the timed region.
With N > 1 the weight N dimension is column-sharded across ranks and outputs are
all-gathered (strong scaling). ``--impl reference`` times the CPU restatement of the
reference's dequantize-then-matmul on the host cores (the reference has no CPU
implementation of this path and its GPU kernels are sm_120-only).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

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


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML while the timed region runs
    (read-only queries, one every few milliseconds; `nvidia-smi` would take ~100 ms a call)."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.index = index
        self.clocks: list[int] = []
        self.maximum = None
        self.reasons: set[str] = set()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = self.index
            if visible:
                entry = visible.split(",")[self.index].strip()
                index = int(entry) if entry.isdigit() else self.index
            handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.maximum = int(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            return
        while not self._stop.is_set():
            try:
                self.clocks.append(int(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                mask = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.004)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self) -> dict:
        return {
            "sm_mhz": statistics.median(self.clocks) if self.clocks else None,
            "sm_min_mhz": min(self.clocks) if self.clocks else None,
            "sm_max_mhz": self.maximum,
            "reasons": sorted(self.reasons),
            "samples": len(self.clocks),
        }


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
    multicast_active = bool(fused and use_multicast and all(layer["full"].multicast for layer in layers))

    def one_step(record: bool):
        for layer in layers:
            op = layer["op"]
            plans.mxfp8_quantize_bf16(stream, layer["x"], op.scratch.quantized_input,
                                      op.scratch.input_scales)
            if record:
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record(stream)
            if fused:
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
            # The step ends when every rank's stores have landed everywhere.
            with torch.cuda.stream(stream):
                layers[-1]["full"].barrier()

    def barrier():
        stream.synchronize()
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        one_step(False)
    barrier()
    begin_event, end_event = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as sampler:
        barrier()
        begin_event.record(stream)
        for _ in range(args.steps):
            one_step(True)
        end_event.record(stream)
        barrier()
    elapsed_ms = begin_event.elapsed_time(end_event)
    if distributed:
        tensor = torch.tensor([elapsed_ms], device=device)
        dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
        elapsed_ms = float(tensor.item())
    ms_per_step = elapsed_ms / args.steps
    value = step_flops() / (ms_per_step * 1e-3) / 1e12

    gemm_ms = sum(start.elapsed_time(stop) for _, start, stop in gemm_events)
    per_layer = {}
    for name, start, stop in gemm_events:
        per_layer.setdefault(name, []).append(start.elapsed_time(stop))
    local_flops = sum(2.0 * TOKENS * layer["local_n"] * layer["k"] for layer in layers)
    achieved = local_flops * args.steps / (gemm_ms * 1e-3) / 1e12
    peaks = measured_peaks()
    if "bf16_tflops_sustained" in peaks:
        peak = 2.0 * float(peaks["bf16_tflops_sustained"])
        peak_note = "2 x measured sustained bf16 cuBLAS TFLOP/s (FP8 issues at twice the bf16 rate)"
    else:
        peak = 2.0 * 1400.0
        peak_note = "2 x fallback sustained bf16 1.4 PFLOP/s"

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
                    out_host.view(TOKENS, layer["local_n"]).copy_(
                        layer["full"].matrix()[:, layer["begin"]:layer["end"]], non_blocking=True)
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

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)",
            "data": "synthetic",
            "config": {
                "workload": WORKLOAD, "tokens": TOKENS,
                "shapes": {name: [n, k] for name, n, k in SHAPES},
                "parallelism": (f"weight N column-sharded x{world}, all-gather fused into the GEMM "
                                "epilogue (" + ("multimem stores through NVSwitch multicast"
                                                if multicast_active else "peer stores over NVLink") + ")"
                                if fused else
                                f"weight N column-sharded x{world}, NCCL all-gather of outputs"
                                if distributed else "single GPU"),
                "l2": "per-step operands (193 MB of weights + activations + 318 MB of outputs) exceed the 126 MB L2",
            },
            "roofline": {
                "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak,
                # dram__bytes_read.sum + dram__bytes_write.sum of the gate_up launch from the ncu
                # capture summarised under profiles/ (algorithmic 322.5 MB; 33 MB of C were still
                # dirty in L2 when the kernel ended). Not measured by this run.
                "traffic": 289.6e6, "traffic_launch": "gate_up (M=4096, N=24576, K=4096)",
                "kernel": "block_scaled_pair_gemm_kernel",
                "peak_source": peak_note, "frac_of_nominal_fp8_4500": achieved / 4500.0,
                "per_layer_tflops": {
                    name: 2.0 * TOKENS * next(l for l in layers if l["name"] == name)["local_n"]
                    * next(l for l in layers if l["name"] == name)["k"] / (statistics.mean(times) * 1e-3) / 1e12
                    for name, times in per_layer.items()},
            },
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e2e_steps},
            "gpu_launches": args.steps * 2 * len(layers),
            "clocks": sampler.summary(),
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
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
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
