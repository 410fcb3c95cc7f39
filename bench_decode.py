"""Decode-path micro-benchmarks (bandwidth-bound GEMVs) on one B200.

    python bench_decode.py [--cycles 200] [--repeats 5] [--ops nvfp4,fp4,dense,marlin,w4a16,scaled_fp8,marlin_moe,fp4_gemm]

Method follows the reference's examples (examples/dense-vector.rs:9,133-141,172-194 and
examples/fp4-vector.rs:9-11,102-116): for every shape the weights live in enough rotating
banks that their total exceeds 768 MiB (at least 8 banks), so no launch finds its matrix in
the 126 MB L2; `cycles` back-to-back launches are timed between two CUDA events on the
launching stream after a warm-up pass; the median of `repeats` timings is reported.
Bytes counted per launch are the algorithmic ones: weights + scales + activations + outputs.
Shapes: the four Qwen3-8B linears (N, K) at M in {1, 4, 8}; for the int4-g128 W4A16 op,
K=4096 x N=14336 and K=14336 x N=4096 at M in {1, 16, 256} (TFLOP/s reported beside GB/s). Prints one JSON line per op and
a final summary line.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import statistics
import threading

import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))

from mircuda_b200 import _lib, plans  # noqa: E402

SHAPES = [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 24576, 4096), ("down", 4096, 12288)]
BANK_BYTES = 768 << 20


def _banks(bytes_per_bank: int) -> int:
    return max(8, math.ceil(BANK_BYTES / bytes_per_bank))


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML while a timed region runs (read-only
    queries every few milliseconds; `nvidia-smi` would take ~100 ms a call). NVML is initialised
    and the device handle fetched before the region starts, so the first sample lands inside."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap"}

    def __init__(self, index: int, interval: float = 0.004):
        self.index, self.interval = index, interval
        self.clocks: list[int] = []
        self.power: list[float] = []
        self.maximum = None
        self.reasons: set[str] = set()
        self._handle = None
        self._nvml = None
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            if visible:
                entry = visible.split(",")[index].strip()
                index = int(entry) if entry.isdigit() else index
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.maximum = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml
        except Exception:  # noqa: BLE001 - no NVML: the record says so (samples 0)
            self._handle = None

    def sample(self) -> None:
        if self._handle is None:
            return
        nvml = self._nvml
        try:
            self.clocks.append(int(nvml.nvmlDeviceGetClockInfo(self._handle, nvml.NVML_CLOCK_SM)))
            mask = int(nvml.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
            for bit, name in self.REASONS.items():
                if mask & bit:
                    self.reasons.add(name)
            self.power.append(nvml.nvmlDeviceGetPowerUsage(self._handle) / 1000.0)
        except Exception:  # noqa: BLE001
            pass

    def _run(self):
        while not self._stop.is_set():
            self.sample()
            self._stop.wait(self.interval)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def mark(self) -> int:
        """Index of the next sample: `summary(start=mark)` then covers what follows."""
        return len(self.clocks)

    def summary(self, start: int = 0) -> dict:
        clocks, power = self.clocks[start:], self.power[start:]
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_min_mhz": min(clocks) if clocks else None,
            "sm_max_mhz": self.maximum,
            "power_w": statistics.median(power) if power else None,
            "reasons": sorted(self.reasons),
            "samples": len(clocks),
        }


def _time(stream, launch, banks: int, cycles: int, repeats: int) -> float:
    """Median seconds per launch."""
    for index in range(banks):
        launch(index)
    stream.synchronize()
    # The launches are microseconds long: issue them from a CUDA graph (as the reference's
    # callers do, examples/graph.rs) so that host launch cost is not what gets measured.
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        for cycle in range(cycles):
            launch(cycle % banks)
    # Keep the GPU busy for a while first: these kernels are so short that a cold start would
    # be timed at idle clocks.
    warm = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    warm[0].record()
    for _ in range(2000):
        graph.replay()
        warm[1].record()
        warm[1].synchronize()
        if warm[0].elapsed_time(warm[1]) > 150.0:
            break
    torch.cuda.synchronize()
    samples = []
    for _ in range(repeats):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        stop.record()
        torch.cuda.synchronize()
        samples.append(start.elapsed_time(stop) * 1e-3 / cycles)
    return statistics.median(samples)


def _random_bytes(count: int, low: int, high: int) -> torch.Tensor:
    return torch.randint(low, high, (count,), dtype=torch.uint8, device="cuda")


def bench_nvfp4(stream, n, k, m, cycles, repeats):
    scale_bytes = (n + 127) // 128 * (k // 64) * 512
    banks = _banks(n * k // 2 + scale_bytes)
    weights = [_random_bytes(n * k // 2, 0, 256) for _ in range(banks)]
    scales = [_random_bytes(scale_bytes, 0x28, 0x48) for _ in range(banks)]
    x = torch.randn(m * k, device="cuda").to(torch.bfloat16)
    out = torch.empty(m * n, dtype=torch.bfloat16, device="cuda")
    plan = plans.NvFp4VectorPlan(stream, plans.NvFp4VectorSpec(m, n, k))
    torch.cuda.synchronize()
    seconds = _time(stream, lambda i: plan.execute(stream, x, weights[i], scales[i], out, 0.5),
                    banks, cycles, repeats)
    plan.close()
    return seconds, n * k * 0.5625 + m * k * 2 + m * n * 2, banks


def bench_fp4(stream, n, k, cycles, repeats):
    scale_bytes = (n + 127) // 128 * (k // 64) * 512
    banks = _banks(n * k // 2 + scale_bytes)
    weights = [_random_bytes(n * k // 2, 0, 256) for _ in range(banks)]
    scales = [_random_bytes(scale_bytes, 0x28, 0x48) for _ in range(banks)]
    x = _random_bytes(k // 2, 0, 256)
    xs = _random_bytes((k // 64) * 512, 0x28, 0x48)
    out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    plan = plans.BlockScaledFp4VectorPlan(stream, plans.BlockScaledFp4VectorSpec(n, k))
    torch.cuda.synchronize()
    seconds = _time(stream, lambda i: plan.execute(stream, x, xs, weights[i], scales[i], out, 0.5),
                    banks, cycles, repeats)
    plan.close()
    return seconds, n * k * 0.5625 + k * 0.5625 + n * 2, banks


def bench_dense(stream, n, k, cycles, repeats):
    banks = _banks(n * k * 2)
    weights = [(torch.randn(n * k, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(banks)]
    x = torch.randn(k, device="cuda").to(torch.bfloat16)
    out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    plan = plans.DenseVectorPlan(stream, plans.DenseVectorSpec(n, k, 1))
    torch.cuda.synchronize()
    seconds = _time(stream, lambda i: plan.execute(stream, x, weights[i], out, 1.0, 0.0),
                    banks, cycles, repeats)
    plan.close()
    return seconds, 2.0 * n * k + 2 * k + 2 * n, banks


def bench_mxfp8_weight_only(stream, n, k, m, cycles, repeats):
    """Weight-only MXFP8 projection (bf16 activations, E4M3 weights, row-major E8M0 scales)."""
    banks = _banks(n * k + n * k // 32)
    weights = [_random_bytes(n * k, 0x20, 0x48) for _ in range(banks)]
    row_scales = [_random_bytes(n * k // 32, 120, 130) for _ in range(banks)]
    x = torch.randn(m * k, device="cuda").to(torch.bfloat16)
    out = torch.empty(m * n, dtype=torch.bfloat16, device="cuda")
    operation = plans.MxFp8Matmul(plans.MxFp8Spec(m, k, n))
    torch.cuda.synchronize()
    seconds = _time(stream, lambda i: operation.execute(stream, x, weights[i], row_scales[i], out),
                    banks, cycles, repeats)
    return seconds, n * k * (1 + 1 / 32) + m * k * 2 + m * n * 2, banks


def bench_marlin(stream, n, k, m, cycles, repeats):
    library = _lib.load()
    banks = _banks(n * k // 2 + n * k // 16)
    weights = [_random_bytes(n * k // 2, 0, 256) for _ in range(banks)]
    scales = [_random_bytes(n * k // 16, 0x90, 0xF0) for _ in range(banks)]   # prepared codes
    x = torch.randn(m * k, device="cuda").to(torch.bfloat16)
    out = torch.empty(m * n, dtype=torch.bfloat16, device="cuda")
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    temporary = torch.zeros(sms * 4096, dtype=torch.float32, device="cuda")
    locks = torch.zeros(sms, dtype=torch.int32, device="cuda")
    global_scale = torch.full((1,), 2.0 ** 100, dtype=torch.float32, device="cuda")
    handle = ctypes.c_void_p(stream.cuda_stream)
    torch.cuda.synchronize()

    def launch(index):
        status = library.mircuda_marlin_nvfp4_dense_execute(
            handle, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(weights[index].data_ptr()),
            ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(temporary.data_ptr()),
            ctypes.c_void_p(scales[index].data_ptr()), ctypes.c_void_p(global_scale.data_ptr()),
            m, n, k, 0, ctypes.c_void_p(locks.data_ptr()), False)
        if status != 0:
            raise RuntimeError(f"marlin dense status {status}")

    seconds = _time(stream, launch, banks, cycles, repeats)
    return seconds, n * k * 0.5625 + m * k * 2 + m * n * 2, banks


W4A16_SHAPES = [("k4096_n14336", 14336, 4096), ("k14336_n4096", 4096, 14336)]


def bench_w4a16(stream, n, k, m, cycles, repeats):
    """int4-g128 weights, f16 activations (the Marlin-style W4A16 shapes of the benchmark)."""
    from mircuda_b200 import dense
    banks = _banks(n * k // 2 + n * k // 128 * 2)
    weights = [_random_bytes(n * k // 2, 0, 256) for _ in range(banks)]
    scales = [(torch.rand(n * k // 128, device="cuda") * 0.01 + 0.002).to(torch.float16)
              for _ in range(banks)]
    x = torch.randn(m * k, device="cuda").to(torch.float16)
    out = torch.empty(m * n, dtype=torch.float16, device="cuda")
    plan = dense.W4A16Plan(stream, dense.W4A16Spec(m, n, k))
    torch.cuda.synchronize()
    seconds = _time(stream, lambda i: plan.execute(stream, x, weights[i], scales[i], out),
                    banks, cycles, repeats)
    plan.close()
    return seconds, n * k * 0.5 + n * k / 128 * 2 + m * k * 2 + m * n * 2, banks


MARLIN_MOE_SHAPES = [("moe_gate_up", 1536, 2048), ("moe_down", 2048, 768)]
MOE_EXPERTS, MOE_TOP_K = 128, 8


def bench_marlin_moe(stream, n, k, m, cycles, repeats):
    """Routed Marlin NVFP4 projection, 128 experts, 8 choices per token (Qwen3-30B-A3B sizes).
    Sixteen route sets are rotated so that consecutive launches touch different experts; the
    byte count is the weights of the experts a launch touches plus its rows in and out."""
    library = _lib.load()
    experts, top_k, block = MOE_EXPERTS, MOE_TOP_K, 8
    weights = _random_bytes(experts * n * k // 2, 0, 256)
    scales = _random_bytes(experts * n * k // 16, 0x90, 0xF0)          # prepared codes
    global_scales = torch.full((experts,), 2.0 ** 100, dtype=torch.float32, device="cuda")
    x = torch.randn(m * k, device="cuda").to(torch.bfloat16)
    out = torch.empty(m * top_k * n, dtype=torch.bfloat16, device="cuda")
    handle = ctypes.c_void_p(stream.cuda_stream)
    pointer = lambda tensor: ctypes.c_void_p(tensor.data_ptr())
    assignments = m * top_k
    capacity = assignments + experts * (block - 1)
    routes, touched = [], 0.0
    for rotation in range(16):
        token, choice = torch.arange(m).view(-1, 1), torch.arange(top_k).view(1, -1)
        selected = ((rotation + 16 * choice + 3 * token) % experts).to(torch.int32).reshape(-1)
        touched += len(torch.unique(selected)) / 16.0
        buffers = dict(selected=selected.cuda(),
                       routing=torch.ones(assignments, dtype=torch.bfloat16, device="cuda"),
                       sorted=torch.zeros(capacity, dtype=torch.int32, device="cuda"),
                       expert_ids=torch.zeros((capacity + block - 1) // block, dtype=torch.int32, device="cuda"),
                       padded=torch.zeros(1, dtype=torch.int32, device="cuda"),
                       offsets=torch.zeros(experts, dtype=torch.int32, device="cuda"),
                       routing_f32=torch.zeros(assignments, dtype=torch.float32, device="cuda"))
        status = library.mircuda_marlin_prepare_moe_routes(
            handle, pointer(buffers["selected"]), pointer(buffers["routing"]), pointer(buffers["sorted"]),
            pointer(buffers["expert_ids"]), pointer(buffers["padded"]), pointer(buffers["offsets"]),
            pointer(buffers["routing_f32"]), assignments, experts, block)
        if status != 0:
            raise RuntimeError(f"marlin route preparation status {status}")
        routes.append(buffers)
    torch.cuda.synchronize()

    def launch(index):
        route = routes[index]
        status = library.mircuda_marlin_nvfp4_moe_execute(
            handle, pointer(x), pointer(weights), pointer(out), None, pointer(scales),
            pointer(global_scales), pointer(route["sorted"]), pointer(route["expert_ids"]),
            pointer(route["padded"]), pointer(route["routing_f32"]), top_k, False, m, n, k, 0, None, False)
        if status != 0:
            raise RuntimeError(f"marlin moe status {status}")

    seconds = _time(stream, launch, len(routes), cycles, repeats)
    return seconds, touched * n * k * 0.5625 + m * k * 2 + assignments * n * 2, len(routes)


def bench_scaled_fp8(stream, n, k, m, cycles, repeats):
    """E4M3 weights and activations, fp32 token scales, fp32 channel scales, bf16 bias."""
    from mircuda_b200 import dense
    banks = _banks(n * k)
    weights = [_random_bytes(n * k, 0x20, 0x48) for _ in range(banks)]
    x = _random_bytes(m * k, 0x20, 0x48)
    token_scales = torch.rand(m, device="cuda") + 0.5
    channel_scales = torch.rand(n, device="cuda") * 0.04 + 0.01
    bias = torch.randn(n, device="cuda").to(torch.bfloat16)
    out = torch.empty(m * n, dtype=torch.bfloat16, device="cuda")
    plan = dense.ScaledFp8Plan(stream, dense.ScaledFp8Spec(m, k, n, torch.float32, "output_channel", True))
    torch.cuda.synchronize()
    seconds = _time(stream, lambda i: plan.execute_f32_scales(stream, x, weights[i], token_scales,
                                                              channel_scales, bias, out),
                    banks, cycles, repeats)
    plan.close()
    return seconds, n * k + m * k + m * n * 2 + n * 6 + m * 4, banks


def bench_fp4_gemm(stream, n, k, m, cycles, repeats):
    """NVFP4 x NVFP4 prefill GEMM (mircuda_fp4_*): E2M1 codes and UE4M3 block scales for both
    operands (random bytes with scales in [2^-2, 4]), bf16 output."""
    from mircuda_b200 import plans_fp4
    spec = plans_fp4.BlockScaledFp4Spec(m, n, k)
    banks = max(2, min(8, _banks(n * k // 2)))
    weights = [_random_bytes(n * k // 2, 0, 256) for _ in range(banks)]
    weight_scales = [_random_bytes(spec.scale_bytes(n), 0x28, 0x48) for _ in range(banks)]
    a = _random_bytes(m * k // 2, 0, 256)
    a_scales = _random_bytes(spec.scale_bytes(m), 0x28, 0x48)
    out = torch.empty(m * n, dtype=torch.bfloat16, device="cuda")
    plan = plans_fp4.BlockScaledFp4Plan(stream, spec)
    torch.cuda.synchronize()
    seconds = _time(stream, lambda i: plan.execute(stream, a, a_scales, weights[i], weight_scales[i], out, 1.0),
                    banks, cycles, repeats)
    plan.close()
    return seconds, (n * k + m * k) // 2 + spec.scale_bytes(n) + spec.scale_bytes(m) + m * n * 2, banks


def run(ops, cycles: int, repeats: int, peak_gbs: float, shapes=None, tokens=None, sampler=None,
        echo: bool = True) -> dict:
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream()
    results = []
    for op in ops:
        for name, n, k in (W4A16_SHAPES if op == "w4a16" else MARLIN_MOE_SHAPES if op == "marlin_moe"
                           else SHAPES):
            if shapes and name not in shapes:
                continue
            for m in ([1, 4, 8] if op in ("nvfp4", "marlin", "mxfp8_wo") else [1, 16, 256] if op == "w4a16" else
                      [1, 16, 512, 4096] if op == "scaled_fp8" else [4096] if op == "fp4_gemm" else
                      [1, 8, 64] if op == "marlin_moe" else [1]):
                if tokens and m not in tokens:
                    continue
                mark = sampler.mark() if sampler is not None else 0
                with torch.cuda.stream(stream):
                    if op == "nvfp4":
                        seconds, byte_count, banks = bench_nvfp4(stream, n, k, m, cycles, repeats)
                    elif op == "fp4":
                        seconds, byte_count, banks = bench_fp4(stream, n, k, cycles, repeats)
                    elif op == "dense":
                        seconds, byte_count, banks = bench_dense(stream, n, k, cycles, repeats)
                    elif op == "w4a16":
                        seconds, byte_count, banks = bench_w4a16(stream, n, k, m, cycles, repeats)
                    elif op == "marlin_moe":
                        seconds, byte_count, banks = bench_marlin_moe(stream, n, k, m, cycles, repeats)
                    elif op == "scaled_fp8":
                        seconds, byte_count, banks = bench_scaled_fp8(stream, n, k, m, cycles, repeats)
                    elif op == "fp4_gemm":
                        seconds, byte_count, banks = bench_fp4_gemm(stream, n, k, m, max(8, cycles // 10), repeats)
                    elif op == "mxfp8_wo":
                        seconds, byte_count, banks = bench_mxfp8_weight_only(stream, n, k, m, cycles, repeats)
                    else:
                        seconds, byte_count, banks = bench_marlin(stream, n, k, m, cycles, repeats)
                torch.cuda.empty_cache()
                record = {"op": op, "shape": name, "n": n, "k": k, "m": m, "us": seconds * 1e6,
                          "gbs": byte_count / seconds / 1e9, "frac_of_measured_hbm":
                          byte_count / seconds / 1e9 / peak_gbs, "banks": banks}
                if op in ("w4a16", "scaled_fp8", "fp4_gemm"):
                    record["tflops"] = 2.0 * m * n * k / seconds / 1e12
                if sampler is not None:
                    clocks = sampler.summary(mark)
                    record["sm_mhz"] = clocks["sm_mhz"]
                    record["clock_samples"] = clocks["samples"]
                results.append(record)
                if echo:
                    print(json.dumps(record), flush=True)
    return {"results": results}


# --------------------------------------------------------------- the reference's own kernels
# The reference kernels that compile for sm_100a (plain SIMT, no waits): FP4 x FP4 GEMV and dense
# GEMV (sys/native/{fp4_vector,dense_vector}_sm120.cu), the MXFP8 activation quantizer and the
# weight-only MXFP8 product (kernels/mxfp8.cu:69-96,111-217), built from the reference's sources
# into oracle/_ref by oracle/build.py and launched with the reference's own geometry. They are
# timed beside this library's kernels for the same op, same inputs, same rotating banks.

REF_DIR = Path(__file__).resolve().parent / "oracle" / "_ref"


def _reference_library(name: str):
    path = REF_DIR / f"libref_{name}.so"
    return ctypes.CDLL(str(path)) if path.exists() else None


def reference_kernel_records(cycles: int, repeats: int, peak_gbs: float) -> list[dict]:
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream()
    handle = ctypes.c_void_p(stream.cuda_stream)
    pointer = lambda tensor: ctypes.c_void_p(tensor.data_ptr())
    records = []
    vector, device = _reference_library("vector"), _reference_library("device")

    def add(op, shape, byte_count, ours, reference):
        records.append({"op": op, "shape": shape, "us": ours * 1e6, "reference_us": reference * 1e6,
                        "speedup_over_reference_kernel": reference / ours,
                        "frac_of_measured_hbm": byte_count / ours / 1e9 / peak_gbs,
                        "reference_frac_of_measured_hbm": byte_count / reference / 1e9 / peak_gbs})

    with torch.cuda.stream(stream):
        if vector is not None:
            vector.mircuda_fp4_vector_execute.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_float]
            vector.mircuda_fp4_vector_destroy.argtypes = [ctypes.c_void_p]
            vector.mircuda_dense_vector_execute.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_float] * 2
            vector.mircuda_dense_vector_destroy.argtypes = [ctypes.c_void_p]
            for name, n, k in SHAPES:
                # FP4 x FP4 GEMV
                scale_bytes = (n + 127) // 128 * (k // 64) * 512
                banks = _banks(n * k // 2 + scale_bytes)
                weights = [_random_bytes(n * k // 2, 0, 256) for _ in range(banks)]
                scales = [_random_bytes(scale_bytes, 0x28, 0x48) for _ in range(banks)]
                x, xs = _random_bytes(k // 2, 0, 256), _random_bytes((k // 64) * 512, 0x28, 0x48)
                out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
                plan = plans.BlockScaledFp4VectorPlan(stream, plans.BlockScaledFp4VectorSpec(n, k))
                raw = ctypes.c_void_p()
                if vector.mircuda_fp4_vector_create(n, k, handle, ctypes.byref(raw)) != 0:
                    raise RuntimeError("reference fp4_vector plan")
                torch.cuda.synchronize()
                ours = _time(stream, lambda i: plan.execute(stream, x, xs, weights[i], scales[i], out, 0.5),
                             banks, cycles, repeats)

                def reference_fp4(i):
                    if vector.mircuda_fp4_vector_execute(raw, handle, pointer(x), pointer(xs), pointer(weights[i]),
                                                         pointer(scales[i]), pointer(out), 0.5) != 0:
                        raise RuntimeError("reference fp4_vector execute")

                reference = _time(stream, reference_fp4, banks, cycles, repeats)
                plan.close()
                vector.mircuda_fp4_vector_destroy(raw)
                add("fp4_vector", name, n * k * 0.5625 + k * 0.5625 + n * 2, ours, reference)
                del weights, scales
                torch.cuda.empty_cache()
                # dense bf16 GEMV
                banks = _banks(n * k * 2)
                weights = [(torch.randn(n * k, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(banks)]
                xd = torch.randn(k, device="cuda").to(torch.bfloat16)
                plan = plans.DenseVectorPlan(stream, plans.DenseVectorSpec(n, k, 1))
                raw = ctypes.c_void_p()
                if vector.mircuda_dense_vector_create(1, n, k, handle, ctypes.byref(raw)) != 0:
                    raise RuntimeError("reference dense_vector plan")
                torch.cuda.synchronize()
                ours = _time(stream, lambda i: plan.execute(stream, xd, weights[i], out, 1.0, 0.0),
                             banks, cycles, repeats)

                def reference_dense(i):
                    if vector.mircuda_dense_vector_execute(raw, handle, pointer(xd), pointer(weights[i]),
                                                           pointer(out), 1.0, 0.0) != 0:
                        raise RuntimeError("reference dense_vector execute")

                reference = _time(stream, reference_dense, banks, cycles, repeats)
                plan.close()
                vector.mircuda_dense_vector_destroy(raw)
                add("dense_vector_bf16", name, 2.0 * n * k + 2 * k + 2 * n, ours, reference)
                del weights
                torch.cuda.empty_cache()
        if device is not None:
            u32 = ctypes.c_uint32
            device.ref_mxfp8_quantize_bf16.argtypes = [ctypes.c_void_p] * 3 + [u32, u32, ctypes.c_void_p]
            device.ref_mxfp8_bf16.argtypes = [ctypes.c_void_p] * 4 + [u32, u32, u32, ctypes.c_int, ctypes.c_void_p]
            for rows, columns in ((4096, 4096), (4096, 12288)):
                # activation quantizer: inputs rotate through banks larger than L2
                byte_count = rows * columns * (2 + 1 + 1 / 32)
                banks = max(8, math.ceil((256 << 20) / (rows * columns * 2)))
                values = [torch.randn(rows, columns, device="cuda").to(torch.bfloat16) for _ in range(banks)]
                codes = torch.empty(rows * columns, dtype=torch.uint8, device="cuda")
                scales = torch.zeros(plans.scale_bytes(rows, columns // 32), dtype=torch.uint8, device="cuda")
                torch.cuda.synchronize()
                ours = _time(stream, lambda i: plans.mxfp8_quantize_bf16(stream, values[i], codes, scales),
                             banks, min(cycles, 50), repeats)

                def reference_quantize(i):
                    if device.ref_mxfp8_quantize_bf16(pointer(values[i]), pointer(codes), pointer(scales), rows,
                                                      columns, handle) != 0:
                        raise RuntimeError("reference quantizer launch")

                reference = _time(stream, reference_quantize, banks, min(cycles, 50), repeats)
                add("mxfp8_quantize_bf16", f"{rows}x{columns}", byte_count, ours, reference)
                del values
                torch.cuda.empty_cache()
            for name, n, k in SHAPES:
                # weight-only MXFP8 product, one token (kernels/mxfp8.cu:111-153)
                banks = _banks(n * k + n * k // 32)
                weights = [_random_bytes(n * k, 0x20, 0x48) for _ in range(banks)]
                row_scales = [_random_bytes(n * k // 32, 120, 130) for _ in range(banks)]
                xd = torch.randn(k, device="cuda").to(torch.bfloat16)
                out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
                operation = plans.MxFp8Matmul(plans.MxFp8Spec(1, k, n))
                torch.cuda.synchronize()
                ours = _time(stream, lambda i: operation.execute(stream, xd, weights[i], row_scales[i], out),
                             banks, cycles, repeats)

                def reference_matmul(i):
                    if device.ref_mxfp8_bf16(pointer(xd), pointer(weights[i]), pointer(row_scales[i]), pointer(out),
                                             1, k, n, 0, handle) != 0:
                        raise RuntimeError("reference weight-only launch")

                reference = _time(stream, reference_matmul, banks, cycles, repeats)
                add("mxfp8_bf16_weight_only", name, n * k * (1 + 1 / 32) + 2 * k + 2 * n, ours, reference)
                del weights, row_scales
                torch.cuda.empty_cache()
    return records


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--cycles", type=int, default=200)
    parser.add_argument("--repeats", type=int, default=5)
    parser.add_argument("--ops", default="nvfp4,fp4,dense,marlin,w4a16")
    parser.add_argument("--peak-gbs", type=float, default=6551.4)
    parser.add_argument("--shapes", default="", help="subset of qkv,o,gate_up,down (profiling runs)")
    parser.add_argument("--tokens", default="", help="subset of 1,4,8 (profiling runs)")
    parser.add_argument("--reference-kernels", action="store_true",
                        help="also time the reference's own sm_100a-runnable kernels (oracle/_ref)")
    args = parser.parse_args()
    if args.reference_kernels:
        for record in reference_kernel_records(args.cycles, args.repeats, args.peak_gbs):
            print(json.dumps(record), flush=True)
    summary = run(args.ops.split(","), args.cycles, args.repeats, args.peak_gbs,
                  set(filter(None, args.shapes.split(","))),
                  {int(t) for t in args.tokens.split(",") if t})
    by_op = {}
    for record in summary["results"]:
        by_op.setdefault(record["op"], []).append(record["frac_of_measured_hbm"])
    print(json.dumps({"summary": {op: {"min_frac": min(v), "mean_frac": sum(v) / len(v)}
                                  for op, v in by_op.items()}}), flush=True)


if __name__ == "__main__":
    main()
