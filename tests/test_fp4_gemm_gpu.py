"""GPU parity for the NVFP4 block-scaled GEMM (CTA-pair tcgen05 kernel) through the C ABI."""
import numpy as np
import pytest
import torch

import oracle
from helpers import assert_close_bf16, bf16_bits, u8

pytestmark = pytest.mark.gpu


def random_fp4(rows, k, seed):
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 256, size=(rows, k // 2), dtype=np.uint8)
    values = rng.integers(0x28, 0x40, size=(rows, k // 16), dtype=np.uint8)
    scales = np.zeros(oracle.fp4_scale_bytes(rows, k), dtype=np.uint8)
    scales[oracle.fp4_scale_offsets(rows, k)] = values
    return codes, scales


def run(stream, a, sa, b, sb, m, n, k, alpha):
    from mircuda_b200 import plans_fp4
    plan = plans_fp4.BlockScaledFp4Plan(stream, plans_fp4.BlockScaledFp4Spec(m, n, k))
    tensors = [u8(a.reshape(-1)), u8(sa), u8(b.reshape(-1)), u8(sb)]
    out = torch.full((m * n,), float("nan"), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    plan.execute(stream, *tensors, out, alpha)
    stream.synchronize()
    plan.close()
    return bf16_bits(out).reshape(m, n)


def test_fp4_gemm_golden(cuda_stream):
    """tests/cutlass/fp4/mod.rs:14-33 — 0x22 codes, 0x38 scales, M=1, N=704, K=2816 -> 2816.0."""
    m, n, k = 1, 704, 2816
    a = np.full((m, k // 2), 0x22, np.uint8)
    sa = np.full(oracle.fp4_scale_bytes(m, k), 0x38, np.uint8)
    b = np.full((n, k // 2), 0x22, np.uint8)
    sb = np.full(oracle.fp4_scale_bytes(n, k), 0x38, np.uint8)
    out = run(cuda_stream, a, sa, b, sb, m, n, k, 1.0)
    assert (oracle.bf16_to_f32(out) == 2816.0).all()


@pytest.mark.parametrize("block_n", ["128", "192", "256"])
@pytest.mark.parametrize("m,n,k", [(256, 512, 1024), (300, 328, 448), (5, 1000, 64), (512, 1536, 2048)])
def test_fp4_gemm_random(cuda_stream, monkeypatch, m, n, k, block_n):
    monkeypatch.setenv("MIRCUDA_B200_FP4_GEMM_BN", block_n)
    a, sa = random_fp4(m, k, 51)
    b, sb = random_fp4(n, k, 52)
    expected = oracle.f32_to_bf16(
        (oracle.nvfp4_dequantize(a, sa, k) @ oracle.nvfp4_dequantize(b, sb, k).T * np.float32(0.25))
        .astype(np.float32))
    actual = run(cuda_stream, a, sa, b, sb, m, n, k, 0.25)
    assert not np.isnan(oracle.bf16_to_f32(actual)).any()
    assert_close_bf16(actual, expected, f"nvfp4 gemm {m}x{n}x{k} bn={block_n}")
