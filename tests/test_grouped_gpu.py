"""GPU parity for the variable-row grouped bf16 GEMM (MoE) through the C ABI."""
import numpy as np
import pytest
import torch

import oracle
from helpers import assert_close_bf16, bf16_bits, seeded_bf16

pytestmark = pytest.mark.gpu


def run_grouped(stream, a, weights, rows, offsets, c, groups, max_rows, n, k, capacity, beta):
    from mircuda_b200 import plans
    plan = plans.VariableGroupedBf16Plan(
        stream, plans.VariableGroupedBf16Spec(groups, max_rows, n, k, capacity))
    rows_d = torch.tensor(rows, dtype=torch.int32, device="cuda")
    offsets_d = torch.tensor(offsets, dtype=torch.int32, device="cuda")
    out = c.clone()
    torch.cuda.synchronize()
    plan.execute(stream, a.view(-1), weights.view(-1), rows_d, offsets_d, out.view(-1), beta)
    stream.synchronize()
    plan.close()
    return out


@pytest.mark.parametrize("block_n", ["128", "256"])
def test_grouped_bf16_golden(cuda_stream, monkeypatch, block_n):
    """tests/cutlass/grouped/bf16.rs:12-36 — rows [3,0,2,1], offsets [0,3,3,5], expert e filled
    with e+1, output pre-filled with NaN to catch unwritten rows."""
    monkeypatch.setenv("MIRCUDA_B200_GROUPED_BN", block_n)
    n = k = 128
    a = torch.ones(6, k, dtype=torch.bfloat16, device="cuda")
    weights = torch.cat([torch.full((n, k), float(e + 1), dtype=torch.bfloat16, device="cuda")
                         for e in range(4)])
    c = torch.full((6, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    out = run_grouped(cuda_stream, a, weights, [3, 0, 2, 1], [0, 3, 3, 5], c, 4, 4, n, k, 6, 0.0)
    expected = torch.tensor([128.0, 128.0, 128.0, 384.0, 384.0, 512.0], device="cuda")
    assert (out.float() == expected[:, None]).all()


@pytest.mark.parametrize("block_n", ["128", "256"])
@pytest.mark.parametrize("beta", [0.0, 0.5])
def test_grouped_bf16_random_ragged(cuda_stream, monkeypatch, block_n, beta):
    """Ragged groups: empty ones, one row, exactly 128, 129, 255 and 300 rows; rows clamped to
    max_rows; untouched rows of C must keep their contents."""
    monkeypatch.setenv("MIRCUDA_B200_GROUPED_BN", block_n)
    groups, n, k, max_rows = 9, 328, 200, 280
    rows = [0, 1, 128, 129, 255, 0, 300, 7, 64]
    clamped = [min(r, max_rows) for r in rows]
    offsets, cursor = [], 5                      # leave rows 0..4 unowned
    for r in rows:
        offsets.append(cursor)
        cursor += r + 3                          # gaps between groups are unowned too
    capacity = cursor + 10
    a = seeded_bf16((capacity, k), 1.0, 6000)
    weights = seeded_bf16((groups * n, k), 0.05, 6001)
    c = seeded_bf16((capacity, n), 1.0, 6002)
    out = run_grouped(cuda_stream, a, weights, rows, offsets, c, groups, max_rows, n, k, capacity, beta)
    expected = oracle.variable_grouped_bf16(bf16_bits(a), bf16_bits(weights), rows, offsets,
                                            bf16_bits(c), max_rows, n, k, beta)
    actual = bf16_bits(out)
    owned = np.zeros(capacity, dtype=bool)
    for offset, count in zip(offsets, clamped):
        owned[offset:offset + count] = True
    assert np.array_equal(actual.reshape(capacity, n)[~owned], bf16_bits(c).reshape(capacity, n)[~owned])
    assert_close_bf16(actual.reshape(capacity, n)[owned], expected.reshape(capacity, n)[owned],
                      f"grouped ragged bn={block_n} beta={beta}")


def test_grouped_bf16_moe_shape_sample(cuda_stream):
    """Qwen3-30B-A3B-like routing at reduced expert count: 16 experts, hidden 2048,
    intermediate 2x768, 4096 routed rows drawn from a softmax/top-k router; re-executed with
    new routing metadata on the same plan (tests/cutlass/grouped/fp4.rs:36-80 idiom)."""
    from mircuda_b200 import plans
    groups, n, k, tokens, top_k = 16, 1536, 2048, 512, 8
    capacity = tokens * top_k
    generator = torch.Generator().manual_seed(7000)
    weights = seeded_bf16((groups * n, k), 0.02, 7001)
    a = seeded_bf16((capacity, k), 1.0, 7002)
    plan = plans.VariableGroupedBf16Plan(
        cuda_stream, plans.VariableGroupedBf16Spec(groups, capacity, n, k, capacity))
    for attempt in range(2):
        logits = torch.randn(tokens, groups, generator=generator)
        chosen = torch.topk(torch.softmax(logits, dim=-1), top_k, dim=-1).indices.reshape(-1)
        counts = torch.bincount(chosen, minlength=groups)
        rows = counts.tolist()
        offsets = (torch.cumsum(counts, 0) - counts).tolist()
        out = torch.full((capacity, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        rows_d = torch.tensor(rows, dtype=torch.int32, device="cuda")
        offsets_d = torch.tensor(offsets, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        plan.execute(cuda_stream, a.view(-1), weights.view(-1), rows_d, offsets_d, out.view(-1), 0.0)
        cuda_stream.synchronize()
        assert not torch.isnan(out).any()
        expected = oracle.variable_grouped_bf16(bf16_bits(a), bf16_bits(weights), rows, offsets,
                                                np.zeros((capacity, n), np.uint16), capacity, n, k, 0.0)
        assert_close_bf16(bf16_bits(out), expected, f"moe sample attempt {attempt}")
    plan.close()


def test_grouped_bf16_indexed_bank(cuda_stream):
    """Groups pick their matrix out of a smaller bank through a device index array (one group
    per (source GPU, local expert) in expert-parallel MoE); an out-of-range index skips the
    group. Expected values come from the plain oracle on the gathered weights."""
    from mircuda_b200 import plans
    groups, matrices, n, k, max_rows = 10, 3, 264, 136, 200
    rows = [5, 130, 0, 64, 200, 1, 33, 128, 90, 17]
    indices = [2, 0, 1, 1, 2, 7, 0, 1, 2, 0]            # group 5 is out of range
    offsets = np.concatenate([[0], np.cumsum(rows)[:-1]]).tolist()
    capacity = sum(rows) + 4
    a = seeded_bf16((capacity, k), 1.0, 6100)
    bank = seeded_bf16((matrices * n, k), 0.05, 6101)
    c = seeded_bf16((capacity, n), 1.0, 6102)
    gathered = torch.cat([bank.view(matrices, n, k)[min(i, matrices - 1)] for i in indices])
    effective_rows = [0 if i >= matrices else r for r, i in zip(rows, indices)]
    expected = oracle.variable_grouped_bf16(bf16_bits(a), bf16_bits(gathered), effective_rows, offsets,
                                            bf16_bits(c), max_rows, n, k, 0.0)
    plan = plans.VariableGroupedBf16Plan(
        cuda_stream, plans.VariableGroupedBf16Spec(groups, max_rows, n, k, capacity, matrices))
    as_words = lambda values: torch.tensor(values, dtype=torch.int32, device="cuda")
    out = c.clone()
    torch.cuda.synchronize()
    plan.execute(cuda_stream, a.view(-1), bank.view(-1), as_words(rows), as_words(offsets),
                 out.view(-1), 0.0, indices=as_words(indices))
    cuda_stream.synchronize()
    plan.close()
    assert_close_bf16(bf16_bits(out).reshape(capacity, n), expected, "indexed grouped bf16")
    begin = offsets[5]
    assert (bf16_bits(out).reshape(capacity, n)[begin:begin + rows[5]] ==
            bf16_bits(c).reshape(capacity, n)[begin:begin + rows[5]]).all()
