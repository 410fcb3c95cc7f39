"""Grouped MoE GEMMs at the full Qwen3-30B-A3B-shaped configuration the throughput is quoted
on: 128 experts, top-8 routing of 4096 tokens (32768 routed rows), hidden 2048, expert
intermediate 768; gate_up is [2*768, 2048] and down [2048, 768] per expert, run once as bf16
and once as NVFP4. The oracle is evaluated on a sample of experts that always includes the
smallest and the largest group (sys/native/variable_grouped_bf16_sm120.cu:18-33,
variable_grouped_fp4_sm120.cu:31-62 define which rows a group reads and writes); every other
row is checked for having been written (NaN pre-fill) and for finiteness."""
import numpy as np
import pytest
import torch

import oracle
from helpers import assert_close_bf16, bf16_bits

pytestmark = pytest.mark.gpu

EXPERTS, TOP_K, TOKENS, HIDDEN, INTERMEDIATE = 128, 8, 4096, 2048, 768
PROJECTIONS = [("gate_up", 2 * INTERMEDIATE, HIDDEN), ("down", HIDDEN, INTERMEDIATE)]


def routing(seed):
    """Router logits ~N(0,1) -> softmax -> top-8; rows per expert and their compact offsets
    (assignments sorted by expert)."""
    generator = torch.Generator().manual_seed(seed)
    logits = torch.randn(TOKENS, EXPERTS, generator=generator)
    chosen = torch.topk(torch.softmax(logits, dim=-1), TOP_K, dim=-1).indices.reshape(-1)
    rows = torch.bincount(chosen, minlength=EXPERTS).numpy().astype(np.uint32)
    offsets = (np.cumsum(rows) - rows).astype(np.uint32)
    return rows, offsets


def sampled_experts(rows):
    picked = {int(np.argmin(rows)), int(np.argmax(rows)), 0, 63, EXPERTS - 1}
    return sorted(picked)


def words(values):
    return torch.from_numpy(np.asarray(values, dtype=np.uint32).view(np.int32)).cuda()


@pytest.mark.parametrize("name,n,k", PROJECTIONS)
def test_grouped_bf16_full_configuration(cuda_stream, name, n, k):
    from mircuda_b200 import plans
    rows, offsets = routing(5000)
    capacity = TOKENS * TOP_K
    assert int(rows.sum()) == capacity
    generator = torch.Generator(device="cuda").manual_seed(5001)
    a = torch.randn(capacity, k, generator=generator, device="cuda").to(torch.bfloat16)
    weights = (torch.randn(EXPERTS * n, k, generator=generator, device="cuda") * 0.02).to(torch.bfloat16)
    out = torch.full((capacity, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    plan = plans.VariableGroupedBf16Plan(
        cuda_stream, plans.VariableGroupedBf16Spec(EXPERTS, capacity, n, k, capacity))
    torch.cuda.synchronize()
    plan.execute(cuda_stream, a.view(-1), weights.view(-1), words(rows), words(offsets), out.view(-1), 0.0)
    cuda_stream.synchronize()
    plan.close()
    assert torch.isfinite(out.float()).all()                    # every routed row was written
    for expert in sampled_experts(rows):
        first, count = int(offsets[expert]), int(rows[expert])
        left = oracle.bf16_to_f32(bf16_bits(a[first:first + count]))
        right = oracle.bf16_to_f32(bf16_bits(weights.view(EXPERTS, n, k)[expert]))
        expected = oracle.f32_to_bf16((left @ right.T).astype(np.float32))
        assert_close_bf16(bf16_bits(out[first:first + count]), expected,
                          f"grouped bf16 {name} expert {expert} ({count} rows)")


@pytest.mark.parametrize("name,n,k", PROJECTIONS)
def test_grouped_nvfp4_full_configuration(cuda_stream, name, n, k):
    from mircuda_b200 import plans_fp4
    rows, offsets = routing(5100)
    capacity = TOKENS * TOP_K
    padded = (rows + 127) // 128 * 128
    scale_offsets = (np.cumsum(padded) - padded).astype(np.uint32)
    spec = plans_fp4.VariableGroupedFp4Spec(EXPERTS, EXPERTS, capacity, n, k, capacity)
    generator = torch.Generator(device="cuda").manual_seed(5101)

    def random_bytes(count, low, high):
        return torch.randint(low, high, (count,), dtype=torch.uint8, device="cuda", generator=generator)

    # Every code and every scale byte of both operands is random (scales 2^-2 .. 1.875), so any
    # group layout reads defined values.
    a = random_bytes(capacity * k // 2, 0, 256)
    a_scales = random_bytes(spec.a_scale_bytes(), 0x28, 0x40)
    b = random_bytes(EXPERTS * n * k // 2, 0, 256)
    b_scales = random_bytes(spec.b_scale_bytes(), 0x28, 0x40)
    alphas = (torch.rand(EXPERTS, generator=generator, device="cuda") * 0.5 + 0.1).float()
    indices = np.arange(EXPERTS, dtype=np.uint32)
    out = torch.full((capacity * n,), float("nan"), dtype=torch.bfloat16, device="cuda")
    plan = plans_fp4.VariableGroupedFp4Plan(cuda_stream, spec)
    torch.cuda.synchronize()
    plan.execute(cuda_stream, a, a_scales, b, b_scales, alphas, words(indices), words(rows),
                 words(offsets), words(scale_offsets), out)
    cuda_stream.synchronize()
    plan.close()
    assert torch.isfinite(out.float()).all()
    sample = sampled_experts(rows)
    sample_rows = np.zeros_like(rows)
    sample_rows[sample] = rows[sample]                          # the oracle skips empty groups
    before = np.zeros((capacity, n), np.uint16)
    expected = oracle.variable_grouped_fp4(
        a.cpu().numpy(), a_scales.cpu().numpy(), b.cpu().numpy(), b_scales.cpu().numpy(),
        alphas.cpu().numpy(), indices, sample_rows, offsets, scale_offsets, before, EXPERTS,
        capacity, n, k)
    actual = bf16_bits(out).reshape(capacity, n)
    for expert in sample:
        first, count = int(offsets[expert]), int(rows[expert])
        assert_close_bf16(actual[first:first + count], expected[first:first + count],
                          f"grouped nvfp4 {name} expert {expert} ({count} rows)")
