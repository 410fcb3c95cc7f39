"""CPU restatement of the Marlin W4A16 layouts — TEST INFRASTRUCTURE ONLY.

The reference pins these layouts bit for bit with host code inside its own tests; the
functions here follow those host references (tests/marlin/main.rs:139-217 for the packed
tiles and the scale permutation, tests/marlin/padded.rs:127-203 for zero padding and the
gate/up de-interleave, tests/marlin/routes.rs:8-54 for route ordering) and, for the NVFP4
scale re-encoding that no reference test covers, the kernel sys/native/marlin/repack.cu:105-140.
"""
from __future__ import annotations

import numpy as np

from . import e4m3_table


def scale_destination(linear: np.ndarray) -> np.ndarray:
    """tests/marlin/main.rs:208-214."""
    linear = np.asarray(linear, dtype=np.int64)
    chunk, local = linear // 64, linear % 64
    permuted = chunk * 64 + 8 * (local % 8) + local // 8
    reorder = np.array([0, 2, 1, 3])
    return permuted // 4 * 4 + reorder[permuted % 4]


def source_rows(size_n: int, logical_n: int, interleaved: bool) -> np.ndarray:
    """Canonical row feeding packed row n, or -1 for padding (tests/marlin/padded.rs:194-203)."""
    n = np.arange(size_n)
    if interleaved:
        physical, logical = size_n // 2, logical_n // 2
        up = n >= physical
        unit = np.where(up, n - physical, n)
        return np.where(unit < logical, unit * 2 + up, -1)
    return np.where(n < logical_n, n, -1)


def unpack_nibbles(raw: np.ndarray, experts: int, rows: int, k: int) -> np.ndarray:
    """[experts, rows, k/2] bytes -> [experts, rows, k] nibbles (even k in the low nibble)."""
    raw = np.asarray(raw, dtype=np.uint8).reshape(experts, rows, k // 2)
    out = np.empty((experts, rows, k), dtype=np.uint8)
    out[:, :, 0::2] = raw & 0xF
    out[:, :, 1::2] = raw >> 4
    return out


def repack(raw, experts, size_n, size_k, logical_n=None, logical_k=None, interleaved=False,
           right=None) -> np.ndarray:
    """Packed u32 words [experts * size_n * size_k / 8] (tests/marlin/main.rs:139-169,
    tests/marlin/padded.rs:127-161). `right` = second buffer of the paired variant."""
    logical_n = size_n if logical_n is None else logical_n
    logical_k = size_k if logical_k is None else logical_k
    canonical = np.zeros((experts, size_n, size_k), dtype=np.uint32)
    if right is not None:
        half = size_n // 2
        canonical[:, :half, :] = unpack_nibbles(raw, experts, half, size_k)
        canonical[:, half:, :] = unpack_nibbles(right, experts, half, size_k)
    else:
        nibbles = unpack_nibbles(raw, experts, logical_n, logical_k)
        rows = source_rows(size_n, logical_n, interleaved)
        valid = rows >= 0
        canonical[:, valid, :logical_k] = nibbles[:, rows[valid], :]
    tiles_n, tiles_k = size_n // 64, size_k // 16
    output = np.zeros((experts, tiles_k, tiles_n, 32, 4), dtype=np.uint32)
    lane = np.arange(32)[:, None]
    quarter = np.arange(4)[None, :]
    order = [0, 2, 4, 6, 1, 3, 5, 7]
    k_offsets = [0, 1, 8, 9, 0, 1, 8, 9]
    n_offsets = [0, 0, 0, 0, 8, 8, 8, 8]
    for tile_k in range(tiles_k):
        for tile_n in range(tiles_n):
            n = tile_n * 64 + quarter * 16 + lane // 4
            k = tile_k * 16 + (lane % 4) * 2
            word = np.zeros((experts, 32, 4), dtype=np.uint32)
            for shift, index in enumerate(order):
                word |= canonical[:, n + n_offsets[index], k + k_offsets[index]] << np.uint32(shift * 4)
            output[:, tile_k, tile_n] = word
    return output.reshape(-1)


def mxfp4_scales(raw, experts, size_n, size_k, logical_n, logical_k, interleaved) -> np.ndarray:
    """tests/marlin/main.rs:190-206 and tests/marlin/padded.rs:163-181: permute, pad with 127."""
    groups, source_groups = size_k // 32, logical_k // 32
    per_expert = size_n * groups
    raw = np.asarray(raw, dtype=np.uint8).reshape(experts, logical_n, source_groups)
    output = np.full(experts * per_expert, 127, dtype=np.uint8)
    rows = source_rows(size_n, logical_n, interleaved)
    for group in range(source_groups):
        n = np.arange(size_n)[rows >= 0]
        destination = scale_destination(group * size_n + n)
        for expert in range(experts):
            output[expert * per_expert + destination] = raw[expert, rows[rows >= 0], group]
    return output


def nvfp4_scales(left, right, globals_, experts, size_n, size_k):
    """sys/native/marlin/repack.cu:88-140: (codes, output_globals, factor)."""
    groups = size_k // 16
    per_expert = size_n * groups
    table = e4m3_table()
    if right is None:
        source = np.asarray(left, dtype=np.uint8).reshape(experts, size_n, groups)
    else:
        half = size_n // 2
        source = np.concatenate([np.asarray(left, np.uint8).reshape(experts, half, groups),
                                 np.asarray(right, np.uint8).reshape(experts, half, groups)], axis=1)
    values = table[source]
    maximum = np.float32(values.max())
    scaled_maximum = np.float32(maximum * np.float32(128.0))
    if 0.0 < scaled_maximum < 57344.0:
        factor = np.float32(2.0) ** np.floor(np.log2(np.float32(57344.0) / scaled_maximum))
    else:
        factor = np.float32(1.0)
    halves = (values * np.float32(factor)).astype(np.float16) * np.float16(128.0)
    bits = halves.view(np.uint16)
    codes = np.where(halves.astype(np.float32) < 2.0, 0, (bits >> 7) & 0xFF).astype(np.uint8)
    output = np.zeros(experts * per_expert, dtype=np.uint8)
    group = np.arange(groups)[None, :]
    n = np.arange(size_n)[:, None]
    destination = scale_destination(group * size_n + n)
    for expert in range(experts):
        output[expert * per_expert + destination] = codes[expert]
    output_globals = (np.asarray(globals_, np.float32) * np.float32(2.0 ** 119) / np.float32(factor)
                      ).astype(np.float32)
    return output, output_globals, float(factor)


def routes(selected, experts: int, block_size: int):
    """tests/marlin/routes.rs:8-54: (sorted, expert_ids, padded_total, offsets)."""
    selected = np.asarray(selected, dtype=np.int64)
    assignments = selected.shape[0]
    capacity = assignments + experts * (block_size - 1)
    sorted_rows = np.full(capacity, assignments, dtype=np.int32)
    expert_ids = np.full((capacity + block_size - 1) // block_size, -1, dtype=np.int32)
    offsets = np.zeros(experts, dtype=np.int32)
    cursor = 0
    for expert in range(experts):
        rows = np.nonzero(selected == expert)[0]
        offsets[expert] = cursor
        sorted_rows[cursor:cursor + rows.size] = rows
        blocks = (rows.size + block_size - 1) // block_size
        expert_ids[cursor // block_size:cursor // block_size + blocks] = expert
        cursor += blocks * block_size
    return sorted_rows, expert_ids, cursor, offsets


def dequantize_packed_nvfp4(packed_words, codes, experts, size_n, size_k):
    """Inverse of `repack` + `nvfp4_scales` for checking kernels: fp32 [experts, N, K] holding
    e2m1(w) * (decoded prepared scale), where the prepared scale byte is the upper 8 bits
    (without sign) of an f16."""
    from . import e2m1_table
    words = np.asarray(packed_words, dtype=np.uint32).reshape(experts, size_k // 16, size_n // 64, 32, 4)
    weights = np.zeros((experts, size_n, size_k), dtype=np.float32)
    e2m1 = e2m1_table()
    lane = np.arange(32)[:, None]
    quarter = np.arange(4)[None, :]
    order = [0, 2, 4, 6, 1, 3, 5, 7]
    k_offsets = [0, 1, 8, 9, 0, 1, 8, 9]
    n_offsets = [0, 0, 0, 0, 8, 8, 8, 8]
    for tile_k in range(size_k // 16):
        for tile_n in range(size_n // 64):
            n = tile_n * 64 + quarter * 16 + lane // 4
            k = tile_k * 16 + (lane % 4) * 2
            word = words[:, tile_k, tile_n]
            for shift, index in enumerate(order):
                nibble = (word >> np.uint32(shift * 4)) & 0xF
                weights[:, n + n_offsets[index], k + k_offsets[index]] = e2m1[nibble]
    groups = size_k // 16
    per_expert = size_n * groups
    group = np.arange(groups)[None, :]
    n = np.arange(size_n)[:, None]
    destination = scale_destination(group * size_n + n)
    codes = np.asarray(codes, dtype=np.uint8).reshape(experts, per_expert)
    scale_bits = (codes[:, destination].astype(np.uint16) << 7)
    scales = scale_bits.view(np.float16).astype(np.float32)          # [experts, N, groups]
    return (weights.reshape(experts, size_n, groups, 16) * scales[:, :, :, None]).reshape(
        experts, size_n, size_k)
