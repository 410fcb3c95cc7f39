"""Expert-parallel MoE feed-forward over the grouped GEMM plans.

Experts are sharded contiguously over the GPUs of one box (`experts / world` per GPU), tokens
are data-parallel. Two transports move the routed rows:

`peer` (default): the dispatch and combine are this library's own kernels over NVLink peer
memory; no collective kernel sits on the data path.
  1. every rank's per-expert counts are all-gathered (a few hundred bytes);
  2. `mircuda_b200_moe_expert_layout` turns them, on the device, into where this rank's rows go
     on each owner (an owner keeps each expert's rows from all sources contiguous, so a group
     of the grouped plan is a whole expert, as on one GPU) and into the owner's own
     `rows` / `offsets`;
  3. `mircuda_b200_moe_dispatch_rows_bf16` stores each routed token row straight into the
     owner's receive buffer (symmetric memory); a stream-ordered barrier follows;
  4. gate_up grouped GEMM, SwiGLU (bounded by the device-side row count), down grouped GEMM;
  5. a barrier, then `mircuda_b200_moe_collect_rows_bf16` loads each token's `top_k` result rows
     from the owners' buffers and adds them with the routing weights.

`nccl`: rows are packed into `world` blocks of `capacity` rows and exchanged with
`all_to_all_single` (equal splits, so the host never reads a count); the received blocks are
used as they arrive, one group per (source GPU, local expert) with the matrix picked by an
index array; results return through a second all-to-all.

With one GPU the collectives drop out and the same code is the single-GPU MoE layer. The
reference has no multi-GPU path and leaves routing and activation to its callers; the grouped
plans are the reference's (src/cutlass/variable_grouped/*).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import _lib, plans, plans_fp4


class CapacityExceeded(RuntimeError):
    """The routing sent a rank more rows than its receive buffers were sized for."""


def route(logits: torch.Tensor, top_k: int):
    """Router: softmax over experts, top-k, renormalised weights. Returns (experts [T, k] int64,
    weights [T, k] float32)."""
    probabilities = torch.softmax(logits.float(), dim=-1)
    weights, chosen = torch.topk(probabilities, top_k, dim=-1)
    return chosen, (weights / weights.sum(dim=-1, keepdim=True)).contiguous()


@dataclass
class Dispatch:
    """Where every (token, choice) of this rank goes. All tensors live on the device."""
    source_rows: torch.Tensor      # [assignments] i32: token row of the i-th sorted assignment
    send_rows: torch.Tensor        # [assignments] i32: its row in the send buffer
    token_rows: torch.Tensor       # [tokens * top_k] i32: send-buffer row of (token, choice)
    counts: torch.Tensor           # [world * local_experts] i32: rows per (destination, expert)
    largest_block: int             # most rows this rank sends to one destination (incl. padding)
    sorted_experts: torch.Tensor   # [assignments] i32: global expert of the i-th sorted assignment
    position: torch.Tensor         # [assignments] i32: its index among this rank's rows of that expert
    slots: torch.Tensor            # [tokens * top_k] i32: sorted position of (token, choice)


def plan_dispatch(chosen: torch.Tensor, experts: int, world: int, capacity: int | None,
                  align: int = 1) -> Dispatch:
    """Sorts the rank's assignments by (destination GPU, local expert) and lays them out in
    `world` blocks of `capacity` rows; inside a block every expert's rows start on a multiple
    of `align` rows (128 keeps NVFP4 scale tiles per group). Pure index arithmetic on the
    device; `largest_block` is the only value read back (set-up time, to size buffers)."""
    tokens, top_k = chosen.shape
    local_experts = experts // world
    flat = chosen.reshape(-1)
    order = torch.argsort(flat, stable=True)
    sorted_experts = flat[order]
    counts = torch.bincount(flat, minlength=experts)
    padded = (counts + align - 1) // align * align
    per_block = padded.view(world, local_experts)
    start_in_block = (torch.cumsum(per_block, dim=1) - per_block).reshape(-1)
    first_of_expert = torch.cumsum(counts, 0) - counts
    position = torch.arange(flat.numel(), device=flat.device) - first_of_expert[sorted_experts]
    largest_block = int(per_block.sum(dim=1).max().item())
    block_rows = capacity if capacity is not None else largest_block
    send_rows = ((sorted_experts // local_experts) * block_rows + start_in_block[sorted_experts]
                 + position)
    token_rows = torch.empty_like(send_rows)
    token_rows[order] = send_rows
    slots = torch.empty_like(order)
    slots[order] = torch.arange(flat.numel(), device=flat.device)
    return Dispatch((order // top_k).to(torch.int32), send_rows.to(torch.int32),
                    token_rows.to(torch.int32), counts.to(torch.int32), largest_block,
                    sorted_experts.to(torch.int32), position.to(torch.int32), slots.to(torch.int32))


class ExpertWeights:
    """The rank's expert banks: gate_up [local_experts, 2*intermediate, hidden] and
    down [local_experts, hidden, intermediate] in bf16, quantised to NVFP4 on request."""

    def __init__(self, stream, gate_up: torch.Tensor, down: torch.Tensor, nvfp4: bool,
                 fuse_swiglu: bool = True):
        """`fuse_swiglu` (NVFP4 only): also keep a gate_up bank whose rows interleave gate and up
        in runs of 16, the layout `mircuda_b200_variable_grouped_fp4_execute_swiglu` reads; the
        layer then runs SwiGLU and the requantisation inside the gate_up epilogue."""
        self.gate_up, self.down = gate_up.contiguous(), down.contiguous()
        self.nvfp4 = nvfp4
        self.fused = False
        if nvfp4:
            # The banks were produced on the caller's current stream; the quantiser runs on `stream`.
            stream.wait_stream(torch.cuda.current_stream(self.gate_up.device))
            # One quantiser pass per bank: every matrix has a whole number of 128-row scale
            # tiles, so the bank's scale layout is the concatenation of the matrices' layouts.
            for name, bank in (("gate_up", self.gate_up), ("down", self.down)):
                local_experts, n, k = bank.shape
                if n % 128 != 0:
                    raise plans.InvalidMatmulShape("NVFP4 banks need n % 128 == 0")
                codes, scales, global_scale = plans.nvfp4_quantize_bf16(stream, bank.view(local_experts * n, k))
                setattr(self, f"{name}_codes", codes.reshape(-1))
                setattr(self, f"{name}_scales", scales)
                setattr(self, f"{name}_global", global_scale)
            local_experts, two_i, k = self.gate_up.shape
            intermediate = two_i // 2
            if fuse_swiglu and intermediate % 16 == 0:
                # rows [gate 16 b .. | up 16 b ..] per block b; quantisation is per row, so the
                # bank's codes and scales are those of the plain bank, permuted
                gate = self.gate_up[:, :intermediate].reshape(local_experts, intermediate // 16, 16, k)
                up = self.gate_up[:, intermediate:].reshape(local_experts, intermediate // 16, 16, k)
                # built on the quantiser's stream, after whatever produced the bank, so that the
                # temporary's memory is not handed out again while the quantiser still reads it
                stream.wait_stream(torch.cuda.current_stream(self.gate_up.device))
                with torch.cuda.stream(stream):
                    interleaved = torch.cat([gate, up], dim=2).reshape(local_experts * two_i, k).contiguous()
                codes, scales, global_scale = plans.nvfp4_quantize_bf16(stream, interleaved)
                self.gate_up_fused_codes, self.gate_up_fused_scales = codes.reshape(-1), scales
                self.gate_up_fused_global = global_scale
                self.fused = True


class ExpertParallelMoe:
    """Buffers and plans for one MoE layer on this rank; `forward` enqueues one step."""

    def __init__(self, stream, hidden: int, intermediate: int, experts: int, top_k: int,
                 tokens: int, capacity: int, weights: ExpertWeights, group=None,
                 transport: str = "peer"):
        """`capacity`: rows per peer block (`nccl`) or rows this rank can receive in total
        (`peer`; the sum over all ranks' assignments is always enough)."""
        self._lib = _lib.load()
        if transport not in ("peer", "nccl"):
            raise ValueError("transport must be 'peer' or 'nccl'")
        self.stream, self.weights = stream, weights
        self.hidden, self.intermediate, self.top_k, self.tokens = hidden, intermediate, top_k, tokens
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.group = group
        self.local_experts = experts // self.world
        self.capacity = capacity
        self.nvfp4 = weights.nvfp4
        if self.nvfp4 and self.world > 1 and transport != "peer":
            raise NotImplementedError("NVFP4 expert parallelism uses the peer transport")
        self.align = 128 if self.nvfp4 else 1
        self.experts = experts
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        # One GPU: both transports degenerate to local copies.
        self.peer = transport == "peer"
        device = weights.gate_up.device
        rows = capacity if self.peer else self.world * capacity
        groups = self.local_experts if self.peer else self.world * self.local_experts
        self.buffer_rows = rows
        bf16 = dict(dtype=torch.bfloat16, device=device)
        with torch.cuda.stream(stream):
            # NVFP4 over the peer transport dispatches quantised rows: packed codes (hidden / 2
            # bytes) and their row-major scales (hidden / 16 bytes), as rows of 2-byte units.
            self._code_units = hidden // 4
            self._scale_units = hidden // 32
            if self.peer and self.nvfp4:
                if hidden % 256 != 0 or capacity % 128 != 0:
                    raise plans.InvalidMatmulShape("NVFP4 dispatch needs hidden % 256 == 0 and capacity % 128 == 0")
                if self.world > 1:
                    from . import gather
                    self._codes_symmetric = gather.SymmetricOutput(rows, self._code_units, device, group)
                    self._scales_symmetric = gather.SymmetricOutput(rows, self._scale_units, device, group)
                    self._result_symmetric = gather.SymmetricOutput(rows, hidden, device, group)
                    self.received_codes = self._codes_symmetric.local
                    self.received_scales = self._scales_symmetric.local
                    self.expert_out = self._result_symmetric.matrix()
                    self._code_pointers = self._codes_symmetric.pointers
                    self._scale_pointers = self._scales_symmetric.pointers
                    self._result_pointers = self._result_symmetric.pointers
                else:
                    self.received_codes = torch.zeros(rows * self._code_units, **bf16)
                    self.received_scales = torch.zeros(rows * self._scale_units, **bf16)
                    self.expert_out = torch.zeros(rows, hidden, **bf16)
                    self._code_pointers = (ctypes.c_void_p * 1)(self.received_codes.data_ptr())
                    self._scale_pointers = (ctypes.c_void_p * 1)(self.received_scales.data_ptr())
                    self._result_pointers = (ctypes.c_void_p * 1)(self.expert_out.data_ptr())
                self.token_codes = torch.zeros(tokens * hidden // 2, dtype=torch.uint8, device=device)
                self.token_scales = torch.zeros(tokens * hidden // 16, dtype=torch.uint8, device=device)
                self.all_counts = torch.zeros(self.world * experts, dtype=torch.int32, device=device)
                self.base_for_me = torch.zeros(experts, dtype=torch.int32, device=device)
                self.remote_rows = torch.zeros(tokens * top_k, dtype=torch.int32, device=device)
                self.received_rows = torch.zeros(1, dtype=torch.int32, device=device)
            elif self.peer:
                # Buffers peers write into / read from live in symmetric memory, which is only
                # used to obtain their peer-mapped addresses and a stream-ordered barrier.
                if self.world > 1:
                    from . import gather
                    self._received_symmetric = gather.SymmetricOutput(rows, hidden, device, group)
                    self._result_symmetric = gather.SymmetricOutput(rows, hidden, device, group)
                    self.received = self._received_symmetric.matrix()
                    self.expert_out = self._result_symmetric.matrix()
                    self._receive_pointers = self._received_symmetric.pointers
                    self._result_pointers = self._result_symmetric.pointers
                else:
                    self.received = torch.zeros(rows, hidden, **bf16)
                    self.expert_out = torch.zeros(rows, hidden, **bf16)
                    self._receive_pointers = (ctypes.c_void_p * 1)(self.received.data_ptr())
                    self._result_pointers = (ctypes.c_void_p * 1)(self.expert_out.data_ptr())
                self.all_counts = torch.zeros(self.world * experts, dtype=torch.int32, device=device)
                self.base_for_me = torch.zeros(experts, dtype=torch.int32, device=device)
                self.remote_rows = torch.zeros(tokens * top_k, dtype=torch.int32, device=device)
                self.received_rows = torch.zeros(1, dtype=torch.int32, device=device)
            else:
                self.send = torch.zeros(rows, hidden, **bf16)
                self.received = self.send if self.world == 1 else torch.zeros(rows, hidden, **bf16)
                self.expert_out = torch.zeros(rows, hidden, **bf16)
                self.returned = self.expert_out if self.world == 1 else torch.zeros(rows, hidden, **bf16)
            self.hidden_states = torch.zeros(rows, 2 * intermediate, **bf16)
            self.activated = torch.zeros(rows, intermediate, **bf16)
            self.output = torch.zeros(tokens, hidden, **bf16)
            self.counts = torch.zeros(groups, dtype=torch.int32, device=device)
            self.rows = torch.zeros(groups, dtype=torch.int32, device=device)
            self.offsets = torch.zeros(groups, dtype=torch.int32, device=device)
            self.indices = torch.arange(self.local_experts, dtype=torch.int32, device=device).repeat(self.world)
            if self.nvfp4:
                k1, k2 = hidden, intermediate
                # Activation scale of the dispatched rows when they are quantised before they
                # travel: every rank must use the same value (the plans take one alpha per
                # matrix), so it is fixed at set-up time (`calibrate`) instead of per step.
                self.dispatch_global = torch.ones(1, dtype=torch.float32, device=device)
                self.codes1 = torch.zeros(rows * k1 // 2, dtype=torch.uint8, device=device)
                self.scales1 = torch.zeros(rows // 128 * (k1 // 64) * 512, dtype=torch.uint8, device=device)
                self.codes2 = torch.zeros(rows * k2 // 2, dtype=torch.uint8, device=device)
                self.scales2 = torch.zeros(rows // 128 * (k2 // 64) * 512, dtype=torch.uint8, device=device)
                self.global1 = torch.zeros(1, dtype=torch.float32, device=device)
                self.global2 = torch.zeros(1, dtype=torch.float32, device=device)
                self.alphas1 = torch.zeros(self.local_experts, dtype=torch.float32, device=device)
                self.alphas2 = torch.zeros(self.local_experts, dtype=torch.float32, device=device)
        if self.nvfp4:
            if capacity % 128 != 0:
                raise plans.InvalidMatmulShape("NVFP4 capacity must be a multiple of 128 rows")
            self.plan1 = _RawGroupedFp4(stream, groups, self.local_experts, capacity, 2 * intermediate, hidden)
            self.plan2 = _RawGroupedFp4(stream, groups, self.local_experts, capacity, hidden, intermediate)
            if self.peer:
                self.indices = torch.arange(self.local_experts, dtype=torch.int32, device=device)
        elif self.peer:
            self.plan1 = plans.VariableGroupedBf16Plan(stream, plans.VariableGroupedBf16Spec(
                groups, capacity, 2 * intermediate, hidden, rows))
            self.plan2 = plans.VariableGroupedBf16Plan(stream, plans.VariableGroupedBf16Spec(
                groups, capacity, hidden, intermediate, rows))
        else:
            self.plan1 = plans.VariableGroupedBf16Plan(stream, plans.VariableGroupedBf16Spec(
                groups, capacity, 2 * intermediate, hidden, rows, self.local_experts))
            self.plan2 = plans.VariableGroupedBf16Plan(stream, plans.VariableGroupedBf16Spec(
                groups, capacity, hidden, intermediate, rows, self.local_experts))
        self.gemm_events = None   # set to a list to record (name, start, stop) CUDA events
        self.static_scales = False
        self.fuse_swiglu = True   # use the fused gate_up epilogue once the scales are frozen
        # Raised by the layout kernel when the routing sends an owner more rows than its buffers
        # hold. Pinned host memory: kernels write it through its device-visible address and the
        # host reads it without touching the stream.
        self._overflow = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._overflow_pointer = ctypes.c_void_p(self._overflow.data_ptr())

    # ------------------------------------------------------------------ helpers
    def _handle(self):
        return ctypes.c_void_p(self.stream.cuda_stream)

    @staticmethod
    def _p(tensor):
        return ctypes.c_void_p(tensor.data_ptr())

    def _timed(self, name, launch):
        if self.gemm_events is None:
            launch()
            return
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(self.stream)
        launch()
        stop.record(self.stream)
        self.gemm_events.append((name, start, stop))

    def _quantize(self, values, rows, k, global_scale, codes, scales):
        plans._check(self._lib.mircuda_b200_nvfp4_global_scale(self._p(values), rows * k,
                                                               self._p(global_scale), self._handle()))
        plans._check(self._lib.mircuda_b200_nvfp4_quantize_bf16(
            self._p(values), self._p(global_scale), self._p(codes), self._p(scales), rows, k,
            self._handle()))

    # ------------------------------------------------------------------- one step
    def check(self, synchronize: bool = True) -> None:
        """Raises `CapacityExceeded` if a step since the last check routed more rows to an
        owner than `capacity` (the overflowing rows were skipped, nothing was written out of
        bounds, and the outputs of the affected tokens lack those experts' contributions).
        With `synchronize` the layer's stream is drained first, so the answer covers every
        enqueued step; without it only steps that have already run are seen."""
        if synchronize:
            self.stream.synchronize()
        if int(self._overflow[0]) != 0:
            self._overflow[0] = 0
            raise CapacityExceeded(
                f"an expert-parallel MoE step needed more than {self.buffer_rows} receive rows on a rank")

    def forward(self, x: torch.Tensor, dispatch: Dispatch, routing_weights: torch.Tensor) -> torch.Tensor:
        """x [tokens, hidden] bf16 on this rank -> output [tokens, hidden] bf16. An overflow of
        the receive capacity seen on an earlier step raises `CapacityExceeded` here; `check()`
        reports the current one. Everything is enqueued on the layer's stream and nothing waits
        for other streams: inputs produced elsewhere must be ordered before this call by the
        caller (`stream.wait_stream(...)`), as with the plans."""
        self.check(synchronize=False)
        if self.peer:
            return self._forward_peer(x, dispatch, routing_weights)
        if dispatch.largest_block > self.capacity:
            raise CapacityExceeded(
                f"a destination block needs {dispatch.largest_block} rows, capacity is {self.capacity}")
        lib, handle = self._lib, self._handle()
        assignments = dispatch.source_rows.numel()
        rows = self.world * self.capacity
        with torch.cuda.stream(self.stream):
            plans._check(lib.mircuda_b200_moe_scatter_rows_bf16(
                self._p(x), self._p(dispatch.source_rows), self._p(dispatch.send_rows),
                self._p(self.send), assignments, self.hidden, handle))
            if self.world > 1:
                dist.all_to_all_single(self.counts, dispatch.counts, group=self.group)
                dist.all_to_all_single(self.received, self.send, group=self.group)
                counts = self.counts
            else:
                counts = dispatch.counts
            plans._check(lib.mircuda_b200_moe_group_offsets(
                self._p(counts), self._p(self.rows), self._p(self.offsets), self.world,
                self.local_experts, self.capacity, self.align, handle))
            w = self.weights
            if self.nvfp4:
                self._quantize(self.received, rows, self.hidden, self.global1, self.codes1, self.scales1)
                torch.mul(w.gate_up_global, self.global1, out=self.alphas1[:1])
                self.alphas1.copy_(self.alphas1[:1].expand_as(self.alphas1))
                self._timed("gate_up", lambda: self.plan1.execute(
                    self.codes1, self.scales1, w.gate_up_codes, w.gate_up_scales, self.alphas1,
                    self.indices, self.rows, self.offsets, self.offsets, self.hidden_states))
            else:
                self._timed("gate_up", lambda: self.plan1.execute(
                    self.stream, self.received.view(-1), w.gate_up.view(-1), self.rows, self.offsets,
                    self.hidden_states.view(-1), 0.0, indices=self.indices))
            plans._check(lib.mircuda_b200_moe_swiglu_bf16(
                self._p(self.hidden_states), self._p(self.activated), rows, None, self.intermediate,
                handle))
            if self.nvfp4:
                self._quantize(self.activated, rows, self.intermediate, self.global2, self.codes2, self.scales2)
                torch.mul(w.down_global, self.global2, out=self.alphas2[:1])
                self.alphas2.copy_(self.alphas2[:1].expand_as(self.alphas2))
                self._timed("down", lambda: self.plan2.execute(
                    self.codes2, self.scales2, w.down_codes, w.down_scales, self.alphas2,
                    self.indices, self.rows, self.offsets, self.offsets, self.expert_out))
            else:
                self._timed("down", lambda: self.plan2.execute(
                    self.stream, self.activated.view(-1), w.down.view(-1), self.rows, self.offsets,
                    self.expert_out.view(-1), 0.0, indices=self.indices))
            if self.world > 1:
                dist.all_to_all_single(self.returned, self.expert_out, group=self.group)
            plans._check(lib.mircuda_b200_moe_combine_rows_bf16(
                self._p(self.returned), self._p(dispatch.token_rows), self._p(routing_weights),
                self._p(self.output), self.tokens, self.top_k, self.hidden, handle))
        return self.output

    def calibrate(self, x: torch.Tensor, dispatch: Dispatch | None = None,
                  routing_weights: torch.Tensor | None = None, margin: float = 2.0) -> None:
        """Fixes the NVFP4 activation scales at set-up time (call again when the activation range
        changes). The scale of the dispatched rows is amax of `x` over all ranks / (448 * 6):
        every rank must use the same value because the plans take one alpha per matrix. When a
        routing is given, one step is run with the intermediate activations' scale measured
        from the data; that scale times `margin` is then frozen too, which lets later steps fuse
        SwiGLU with the quantiser and skip the amax pass."""
        # set-up time: order the layer's stream after the stream that produced x and the routing
        self.stream.wait_stream(torch.cuda.current_stream(x.device))
        with torch.cuda.stream(self.stream):
            amax = x.abs().max().float().reshape(1)
            if self.world > 1:
                dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=self.group)
            self.dispatch_global.copy_(torch.where(amax > 0, amax / 2688.0, torch.ones_like(amax)))
            self.alphas1.copy_((self.weights.gate_up_global * self.dispatch_global).expand_as(self.alphas1))
        self.static_scales = False
        if dispatch is None or not self.peer:
            return
        self.forward(x, dispatch, routing_weights)
        with torch.cuda.stream(self.stream):
            frozen = self.global2 * margin
            if self.world > 1:
                dist.all_reduce(frozen, op=dist.ReduceOp.MAX, group=self.group)
            self.global2.copy_(frozen)
            self.alphas2.copy_((self.weights.down_global * self.global2).expand_as(self.alphas2))
        self.static_scales = True

    def _forward_peer_fp4(self, x, dispatch: Dispatch, routing_weights):
        lib, handle = self._lib, self._handle()
        assignments = dispatch.source_rows.numel()
        pointer_array = ctypes.POINTER(ctypes.c_void_p)
        rows = self.buffer_rows
        w = self.weights
        with torch.cuda.stream(self.stream):
            # Quantise the rank's token rows once (each is dispatched top_k times), scales
            # row-major so that codes and scales travel as rows.
            self._timed("quantize tokens", lambda: plans._check(lib.mircuda_b200_nvfp4_quantize_rows_bf16(
                self._p(x), self._p(self.dispatch_global), self._p(self.token_codes),
                self._p(self.token_scales), self.tokens, self.hidden, handle)))
            if self.world > 1:
                self._timed("count exchange", lambda: dist.all_gather_into_tensor(
                    self.all_counts, dispatch.counts, group=self.group))
                all_counts = self.all_counts
            else:
                all_counts = dispatch.counts
            self._timed("layout", lambda: plans._check(lib.mircuda_b200_moe_expert_layout(
                self._p(all_counts), self.world, self.rank, self.experts, 128, self._p(self.base_for_me),
                self._p(self.rows), self._p(self.offsets), self._p(self.received_rows), self.buffer_rows,
                self._overflow_pointer, handle)))

            def dispatch_rows():
                for source, pointers, units in ((self.token_codes, self._code_pointers, self._code_units),
                                                (self.token_scales, self._scale_pointers, self._scale_units)):
                    plans._check(lib.mircuda_b200_moe_dispatch_rows_bf16(
                        self._p(source), self._p(dispatch.source_rows), self._p(dispatch.sorted_experts),
                        self._p(dispatch.position), self._p(self.base_for_me),
                        ctypes.cast(pointers, pointer_array), self.world, self._p(self.remote_rows),
                        assignments, self.local_experts, units, self.buffer_rows, handle))
                if self.world > 1:
                    self._codes_symmetric.barrier()

            self._timed("dispatch", dispatch_rows)

            # Row-major scales of the received rows -> 128-row atoms (every expert starts on a
            # 128-row tile, so the whole buffer is one plain scale matrix). alphas1 was fixed by
            # `calibrate`.
            self._timed("scale atoms", lambda: plans._check(lib.mircuda_b200_moe_scale_atoms(
                self._p(self.received_scales), self._p(self.scales1), rows, self._p(self.received_rows),
                self.hidden // 16, handle)))
            if self.static_scales and w.fused and self.fuse_swiglu:
                # gate_up with SwiGLU and the requantisation in its epilogue: the bf16 intermediate
                # never exists
                self._timed("gate_up", lambda: self.plan1.execute_swiglu(
                    self.received_codes, self.scales1, w.gate_up_fused_codes, w.gate_up_fused_scales,
                    self.alphas1, self.indices, self.rows, self.offsets, self.offsets, self.global2,
                    self.codes2, self.scales2))
            else:
                self._timed("gate_up", lambda: self.plan1.execute(
                    self.received_codes, self.scales1, w.gate_up_codes, w.gate_up_scales, self.alphas1,
                    self.indices, self.rows, self.offsets, self.offsets, self.hidden_states))
            if self.static_scales and w.fused and self.fuse_swiglu:
                pass
            elif self.static_scales:
                self._timed("swiglu + quantize", lambda: plans._check(lib.mircuda_b200_moe_swiglu_nvfp4(
                    self._p(self.hidden_states), self._p(self.global2), self._p(self.codes2),
                    self._p(self.scales2), rows, self._p(self.received_rows), self.intermediate, handle)))
            else:
                self._timed("swiglu", lambda: plans._check(lib.mircuda_b200_moe_swiglu_bf16(
                    self._p(self.hidden_states), self._p(self.activated), rows, self._p(self.received_rows),
                    self.intermediate, handle)))

                def requantize():
                    self._quantize(self.activated, rows, self.intermediate, self.global2, self.codes2,
                                   self.scales2)
                    torch.mul(w.down_global, self.global2, out=self.alphas2[:1])
                    self.alphas2.copy_(self.alphas2[:1].expand_as(self.alphas2))

                self._timed("quantize activations", requantize)
            self._timed("down", lambda: self.plan2.execute(
                self.codes2, self.scales2, w.down_codes, w.down_scales, self.alphas2,
                self.indices, self.rows, self.offsets, self.offsets, self.expert_out))

            def collect():
                if self.world > 1:
                    self._result_symmetric.barrier()
                plans._check(lib.mircuda_b200_moe_collect_rows_bf16(
                    ctypes.cast(self._result_pointers, pointer_array), self.world, self._p(dispatch.slots),
                    self._p(dispatch.sorted_experts), self._p(self.remote_rows), self._p(routing_weights),
                    self._p(self.output), self.tokens, self.top_k, self.local_experts, self.hidden, handle))

            self._timed("collect", collect)
        return self.output

    def _forward_peer(self, x, dispatch: Dispatch, routing_weights):
        if self.nvfp4:
            return self._forward_peer_fp4(x, dispatch, routing_weights)
        lib, handle = self._lib, self._handle()
        assignments = dispatch.source_rows.numel()
        pointer_array = ctypes.POINTER(ctypes.c_void_p)
        with torch.cuda.stream(self.stream):
            if self.world > 1:
                dist.all_gather_into_tensor(self.all_counts, dispatch.counts, group=self.group)
                all_counts = self.all_counts
            else:
                all_counts = dispatch.counts
            plans._check(lib.mircuda_b200_moe_expert_layout(
                self._p(all_counts), self.world, self.rank, self.experts, 1, self._p(self.base_for_me),
                self._p(self.rows), self._p(self.offsets), self._p(self.received_rows), self.buffer_rows,
                self._overflow_pointer, handle))
            plans._check(lib.mircuda_b200_moe_dispatch_rows_bf16(
                self._p(x), self._p(dispatch.source_rows), self._p(dispatch.sorted_experts),
                self._p(dispatch.position), self._p(self.base_for_me),
                ctypes.cast(self._receive_pointers, pointer_array), self.world,
                self._p(self.remote_rows), assignments, self.local_experts, self.hidden,
                self.buffer_rows, handle))
            if self.world > 1:
                self._received_symmetric.barrier()     # every peer's rows have landed here
            w = self.weights
            self._timed("gate_up", lambda: self.plan1.execute(
                self.stream, self.received.reshape(-1), w.gate_up.view(-1), self.rows, self.offsets,
                self.hidden_states.view(-1), 0.0))
            plans._check(lib.mircuda_b200_moe_swiglu_bf16(
                self._p(self.hidden_states), self._p(self.activated), self.buffer_rows,
                self._p(self.received_rows), self.intermediate, handle))
            self._timed("down", lambda: self.plan2.execute(
                self.stream, self.activated.view(-1), w.down.view(-1), self.rows, self.offsets,
                self.expert_out.reshape(-1), 0.0))
            if self.world > 1:
                self._result_symmetric.barrier()       # every owner's results are complete
            plans._check(lib.mircuda_b200_moe_collect_rows_bf16(
                ctypes.cast(self._result_pointers, pointer_array), self.world, self._p(dispatch.slots),
                self._p(dispatch.sorted_experts), self._p(self.remote_rows), self._p(routing_weights),
                self._p(self.output), self.tokens, self.top_k, self.local_experts, self.hidden, handle))
        return self.output

    def close(self):
        self.plan1.close()
        self.plan2.close()


class _RawGroupedFp4:
    """`mircuda_variable_grouped_fp4_*` without the buffer-length checks of the public plan: the
    MoE layer sizes its activation-scale buffer by its own padded capacity."""

    def __init__(self, stream, groups, matrices, max_rows, n, k):
        self._lib, self._stream = _lib.load(), stream
        raw = ctypes.c_void_p()
        plans._check(self._lib.mircuda_variable_grouped_fp4_create(
            groups, matrices, max_rows, n, k, ctypes.c_void_p(stream.cuda_stream), ctypes.byref(raw)))
        self._raw = raw

    def execute(self, a, a_scales, b, b_scales, alphas, indices, rows, offsets, scale_offsets, c):
        p = lambda tensor: ctypes.c_void_p(tensor.data_ptr())
        plans._check(self._lib.mircuda_variable_grouped_fp4_execute(
            self._raw, ctypes.c_void_p(self._stream.cuda_stream), p(a), p(a_scales), p(b), p(b_scales),
            p(alphas), p(indices), p(rows), p(offsets), p(scale_offsets), p(c)))

    def execute_swiglu(self, a, a_scales, b, b_scales, alphas, indices, rows, offsets, scale_offsets,
                       global_scale, codes, scales):
        p = lambda tensor: ctypes.c_void_p(tensor.data_ptr())
        plans._check(self._lib.mircuda_b200_variable_grouped_fp4_execute_swiglu(
            self._raw, ctypes.c_void_p(self._stream.cuda_stream), p(a), p(a_scales), p(b), p(b_scales),
            p(alphas), p(indices), p(rows), p(offsets), p(scale_offsets), p(global_scale), p(codes),
            p(scales)))

    def close(self):
        if getattr(self, "_raw", None):
            self._lib.mircuda_variable_grouped_fp4_destroy(self._raw)
            self._raw = None

    __del__ = close
