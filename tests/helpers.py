"""Shared helpers for the GPU parity tests."""
import numpy as np
import torch

import oracle

TOLERANCE_MAX = 1e-2      # max |delta| <= 1e-2 * max |ref|
TOLERANCE_FROBENIUS = 5e-3


def bf16_bits(tensor: torch.Tensor) -> np.ndarray:
    """bf16 torch tensor -> numpy uint16 bit patterns."""
    return tensor.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def from_bf16_bits(bits: np.ndarray, device="cuda") -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(device).view(torch.bfloat16)


def u8(array: np.ndarray, device="cuda") -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(array, dtype=np.uint8)).to(device)


def assert_close_bf16(actual_bits, expected_bits, what=""):
    stats = oracle.compare_bf16(actual_bits, expected_bits)
    assert stats["max_rel_to_max"] <= TOLERANCE_MAX, (what, stats)
    assert stats["rel_frobenius"] <= TOLERANCE_FROBENIUS, (what, stats)
    return stats


def seeded_bf16(shape, std, seed, device="cuda") -> torch.Tensor:
    generator = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=generator, dtype=torch.float32) * std).to(torch.bfloat16).to(device)
