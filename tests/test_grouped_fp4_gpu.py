"""GPU parity for the grouped NVFP4 GEMMs (variable, paired, indexed) through the C ABI."""
import numpy as np
import pytest
import torch

import oracle
from helpers import assert_close_bf16, bf16_bits, u8

pytestmark = pytest.mark.gpu

N, K = 128, 128


def u32(values):
    return torch.from_numpy(np.asarray(values, dtype=np.uint32).view(np.int32)).cuda()


def f32(values):
    return torch.from_numpy(np.asarray(values, dtype=np.float32)).cuda()


def ones_bf16(count):
    return torch.ones(count, dtype=torch.bfloat16, device="cuda")


def golden_bank():
    """tests/cutlass/grouped/fp4.rs: three matrices of 0x22 codes (1.0), the first all zero;
    every scale 0x38 (1.0)."""
    weights = np.full((3, N, K // 2), 0x22, np.uint8)
    weights[0] = 0
    scales = np.full(3 * oracle.fp4_scale_bytes(N, K), 0x38, np.uint8)
    return weights, scales


def rows_of(output, columns):
    values = output.float().view(-1, columns)
    assert (values == values[:, :1]).all()
    return values[:, 0].tolist()


def test_variable_grouped_fp4_golden(cuda_stream):
    """variable_grouped_fp4_uses_device_rows_and_compact_offsets
    (tests/cutlass/grouped/fp4.rs:38-87), both executions of the same plan."""
    from mircuda_b200 import plans_fp4
    capacity = 6
    spec = plans_fp4.VariableGroupedFp4Spec(4, 3, 4, N, K, capacity)
    a = u8(np.full(capacity * K // 2, 0x22, np.uint8))
    a_scales = u8(np.full(4 * (K // 64) * 512, 0x38, np.uint8))
    weights, bank_scales = golden_bank()
    b, b_scales = u8(weights.reshape(-1)), u8(bank_scales)
    alphas = f32([1.0, 0.5, 0.25])
    indices = u32([1, 0, 2, 1])
    output = ones_bf16(capacity * N)
    plan = plans_fp4.VariableGroupedFp4Plan(cuda_stream, spec)
    torch.cuda.synchronize()
    plan.execute(cuda_stream, a, a_scales, b, b_scales, alphas, indices, u32([3, 0, 2, 1]),
                 u32([0, 3, 3, 5]), u32([0, 128, 128, 256]), output)
    cuda_stream.synchronize()
    assert rows_of(output, N) == [64.0, 64.0, 64.0, 32.0, 32.0, 64.0]
    plan.execute(cuda_stream, a, a_scales, b, b_scales, alphas, indices, u32([0, 1, 1, 4]),
                 u32([0, 0, 1, 2]), u32([0, 0, 128, 256]), output)
    cuda_stream.synchronize()
    plan.close()
    assert rows_of(output, N) == [0.0, 32.0, 64.0, 64.0, 64.0, 64.0]


def test_paired_variable_grouped_fp4_golden(cuda_stream):
    """paired_variable_grouped_fp4_shares_only_device_metadata (tests/cutlass/grouped/fp4.rs:89-163)."""
    from mircuda_b200 import plans_fp4
    capacity = 6
    spec = plans_fp4.VariableGroupedFp4Spec(4, 3, 4, N, K, capacity)
    weights, bank_scales = golden_bank()

    def side(alpha_values):
        return (u8(np.full(capacity * K // 2, 0x22, np.uint8)),
                u8(np.full(4 * (K // 64) * 512, 0x38, np.uint8)), u8(weights.reshape(-1)),
                u8(bank_scales), f32(alpha_values), ones_bf16(capacity * N))

    left, right = side([1.0, 0.5, 0.25]), side([2.0, 1.0, 0.5])
    plan = plans_fp4.PairedVariableGroupedFp4Plan(cuda_stream, spec)
    torch.cuda.synchronize()
    plan.execute(cuda_stream, left, right, u32([1, 0, 2, 1]), u32([3, 0, 2, 1]), u32([0, 3, 3, 5]),
                 u32([0, 128, 128, 256]))
    cuda_stream.synchronize()
    plan.close()
    assert rows_of(left[5], N) == [64.0, 64.0, 64.0, 32.0, 32.0, 64.0]
    assert rows_of(right[5], N) == [128.0, 128.0, 128.0, 64.0, 64.0, 128.0]


@pytest.mark.parametrize("groups,m,broadcast", [(64, 128, False), (64, 1, False), (1025, 1, False),
                                                (2, 2, True)])
def test_indexed_grouped_fp4_golden(cuda_stream, groups, m, broadcast):
    """run_case (tests/cutlass/grouped/fp4.rs:173-217): 33 matrices, the first zero, alpha 0.5
    for even matrices and 1.0 for odd ones; every group must read K * alpha."""
    from mircuda_b200 import plans_fp4
    matrices = 33
    spec = plans_fp4.IndexedGroupedFp4Spec(groups, matrices, m, N, K, broadcast)
    inputs = spec.inputs()
    a = u8(np.full(inputs * m * K // 2, 0x22, np.uint8))
    a_scales = u8(np.full(inputs * oracle.fp4_scale_bytes(m, K), 0x38, np.uint8))
    weights = np.full((matrices, N, K // 2), 0x22, np.uint8)
    weights[0] = 0
    b = u8(weights.reshape(-1))
    b_scales = u8(np.full(matrices * oracle.fp4_scale_bytes(N, K), 0x38, np.uint8))
    alpha_values = [0.5 if matrix % 2 == 0 else 1.0 for matrix in range(matrices)]
    selected = [group % matrices for group in range(groups)]
    output = ones_bf16(groups * m * N)
    plan = plans_fp4.IndexedGroupedFp4Plan(cuda_stream, spec)
    torch.cuda.synchronize()
    plan.execute(cuda_stream, a, a_scales, b, b_scales, f32(alpha_values), u32(selected), output)
    cuda_stream.synchronize()
    plan.close()
    values = output.float().view(groups, m * N)
    for group in range(groups):
        expert = group % matrices
        expected = 0.0 if expert == 0 else K * alpha_values[expert]
        assert (values[group] == expected).all(), f"group {group}"


def random_fp4(rows, k, rng):
    codes = rng.integers(0, 256, size=(rows, k // 2), dtype=np.uint8)
    values = rng.integers(0x28, 0x40, size=(rows, k // 16), dtype=np.uint8)
    scales = np.zeros(oracle.fp4_scale_bytes(rows, k), dtype=np.uint8)
    scales[oracle.fp4_scale_offsets(rows, k)] = values
    return codes, scales


def routed_problem(groups, matrices, max_rows, n, k, seed, empty_every=5):
    """Random ragged groups packed back to back; scales of each group start on a 128-row tile."""
    rng = np.random.default_rng(seed)
    rows = rng.integers(1, max_rows + 1, size=groups).astype(np.uint32)
    rows[::empty_every] = 0
    offsets = np.concatenate([[0], np.cumsum(rows)[:-1]]).astype(np.uint32)
    scale_offsets = np.concatenate([[0], np.cumsum((rows + 127) // 128 * 128)[:-1]]).astype(np.uint32)
    capacity = int(rows.sum()) + 3
    indices = rng.integers(0, matrices, size=groups).astype(np.uint32)
    indices[1] = matrices + 7                      # out of range: the group must be skipped
    return rows, offsets, scale_offsets, capacity, indices


def build_side(spec, rows, scale_offsets, offsets, rng):
    a = rng.integers(0, 256, size=(spec.capacity_rows, spec.k // 2), dtype=np.uint8)
    a_scales = np.zeros(spec.a_scale_bytes(), np.uint8)
    for group in range(spec.groups):
        count = int(rows[group])
        if count == 0:
            continue
        _, group_scales = random_fp4(count, spec.k, rng)
        begin = int(scale_offsets[group]) // 128 * (spec.k // 64) * 512
        a_scales[begin:begin + group_scales.size] = group_scales
    bank = [random_fp4(spec.n, spec.k, rng) for _ in range(spec.matrices)]
    b = np.stack([codes for codes, _ in bank])
    b_scales = np.concatenate([scales for _, scales in bank])
    alphas = rng.uniform(0.1, 0.6, size=spec.matrices).astype(np.float32)
    return a, a_scales, b, b_scales, alphas


@pytest.mark.parametrize("groups,matrices,max_rows,n,k", [
    (12, 5, 300, 256, 256), (9, 4, 130, 200, 448), (128, 16, 80, 1536, 512), (7, 3, 700, 384, 768)])
def test_variable_grouped_fp4_random(cuda_stream, groups, matrices, max_rows, n, k):
    from mircuda_b200 import plans_fp4
    rows, offsets, scale_offsets, capacity, indices = routed_problem(groups, matrices, max_rows, n, k, 77)
    spec = plans_fp4.VariableGroupedFp4Spec(groups, matrices, max_rows, n, k, capacity)
    rng = np.random.default_rng(78)
    a, a_scales, b, b_scales, alphas = build_side(spec, rows, scale_offsets, offsets, rng)
    before = np.full((capacity, n), 0x3F80, np.uint16)
    expected = oracle.variable_grouped_fp4(a, a_scales, b, b_scales, alphas, indices, rows, offsets,
                                           scale_offsets, before, matrices, max_rows, n, k)
    output = ones_bf16(capacity * n)
    plan = plans_fp4.VariableGroupedFp4Plan(cuda_stream, spec)
    torch.cuda.synchronize()
    for _ in range(2):
        plan.execute(cuda_stream, u8(a.reshape(-1)), u8(a_scales), u8(b.reshape(-1)), u8(b_scales),
                     f32(alphas), u32(indices), u32(rows), u32(offsets), u32(scale_offsets), output)
    cuda_stream.synchronize()
    plan.close()
    actual = bf16_bits(output).reshape(capacity, n)
    # Rows no group owns (skipped group, slack at the end) must be untouched.
    owned = np.zeros(capacity, bool)
    for group in range(groups):
        if indices[group] < matrices:
            owned[offsets[group]:offsets[group] + rows[group]] = True
    assert (actual[~owned] == 0x3F80).all()
    assert_close_bf16(actual, expected, f"variable grouped nvfp4 {groups}x{n}x{k}")


def test_paired_variable_grouped_fp4_random(cuda_stream):
    from mircuda_b200 import plans_fp4
    groups, matrices, max_rows, n, k = 20, 6, 200, 512, 256
    rows, offsets, scale_offsets, capacity, indices = routed_problem(groups, matrices, max_rows, n, k, 91)
    spec = plans_fp4.VariableGroupedFp4Spec(groups, matrices, max_rows, n, k, capacity)
    rng = np.random.default_rng(92)
    sides, expected, outputs = [], [], []
    before = np.full((capacity, n), 0x3F80, np.uint16)
    for _ in range(2):
        a, a_scales, b, b_scales, alphas = build_side(spec, rows, scale_offsets, offsets, rng)
        expected.append(oracle.variable_grouped_fp4(a, a_scales, b, b_scales, alphas, indices, rows,
                                                    offsets, scale_offsets, before, matrices,
                                                    max_rows, n, k))
        output = ones_bf16(capacity * n)
        outputs.append(output)
        sides.append((u8(a.reshape(-1)), u8(a_scales), u8(b.reshape(-1)), u8(b_scales), f32(alphas),
                      output))
    plan = plans_fp4.PairedVariableGroupedFp4Plan(cuda_stream, spec)
    torch.cuda.synchronize()
    plan.execute(cuda_stream, sides[0], sides[1], u32(indices), u32(rows), u32(offsets),
                 u32(scale_offsets))
    cuda_stream.synchronize()
    plan.close()
    for name, output, reference in zip(("left", "right"), outputs, expected):
        assert_close_bf16(bf16_bits(output).reshape(capacity, n), reference, f"paired {name}")


def test_indexed_grouped_fp4_random(cuda_stream):
    from mircuda_b200 import plans_fp4
    groups, experts, m, n, k = 24, 7, 5, 320, 192
    rng = np.random.default_rng(93)
    spec = plans_fp4.IndexedGroupedFp4Spec(groups, experts, m, n, k)
    inputs = [random_fp4(m, k, rng) for _ in range(groups)]
    a = np.stack([codes for codes, _ in inputs])
    a_scales = np.concatenate([scales for _, scales in inputs])
    bank = [random_fp4(n, k, rng) for _ in range(experts)]
    b = np.stack([codes for codes, _ in bank])
    b_scales = np.concatenate([scales for _, scales in bank])
    alphas = rng.uniform(0.1, 0.6, size=experts).astype(np.float32)
    selected = rng.integers(0, experts, size=groups).astype(np.uint32)
    selected[3] = experts                               # skipped
    before = np.full((groups * m, n), 0x3F80, np.uint16)
    expected = oracle.indexed_grouped_fp4(a, a_scales, b, b_scales, alphas, selected, before, experts,
                                          m, n, k, False)
    output = ones_bf16(groups * m * n)
    plan = plans_fp4.IndexedGroupedFp4Plan(cuda_stream, spec)
    torch.cuda.synchronize()
    plan.execute(cuda_stream, u8(a.reshape(-1)), u8(a_scales), u8(b.reshape(-1)), u8(b_scales),
                 f32(alphas), u32(selected), output)
    cuda_stream.synchronize()
    plan.close()
    actual = bf16_bits(output).reshape(groups * m, n)
    assert (actual[3 * m:4 * m] == 0x3F80).all()
    assert_close_bf16(actual, expected, "indexed grouped nvfp4")
