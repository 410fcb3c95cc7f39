"""How the path shards over the GPUs of one box.

Linears: the weight N dimension (rows of B[N, K] and their scale row tiles) is split into
contiguous column shards whose boundaries are multiples of 128 rows, so that no 128-row
scale atom is split; activations are replicated and quantized on every rank; the only
exchange is an all-gather of the bf16 outputs. The reference has no multi-GPU path; this
follows the partitioning its operand layouts allow (one scale row tile per 128 weight rows,
src/cutlass/mxfp8.rs:45-50 in the reference).
"""
from __future__ import annotations


def column_shard(n: int, world: int, rank: int, granule: int = 128) -> tuple[int, int]:
    """[begin, end) of rank's rows of an N-row weight; boundaries are multiples of `granule`
    (except the end of the last non-empty shard, which is N)."""
    if world <= 0 or not (0 <= rank < world) or n <= 0:
        raise ValueError("invalid shard request")
    granules = (n + granule - 1) // granule
    base, extra = divmod(granules, world)
    first = rank * base + min(rank, extra)
    count = base + (1 if rank < extra else 0)
    begin = min(first * granule, n)
    end = min((first + count) * granule, n)
    return begin, end


def gather_columns(shards, out=None, group=None):
    """All-gather per-rank outputs [M, N_r] into the full [M, N] (columns in rank order).

    `shards` is this rank's [M, N_r] tensor. Narrower shards are zero-padded to the widest
    one for the collective and cut back afterwards. Works with any torch.distributed
    backend (nccl on GPUs, gloo in the CPU tests).
    """
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    m, local_n = shards.shape
    widths = [torch.zeros(1, dtype=torch.int64, device=shards.device) for _ in range(world)]
    dist.all_gather(widths, torch.tensor([local_n], dtype=torch.int64, device=shards.device), group=group)
    widths = [int(w.item()) for w in widths]
    widest = max(widths)
    padded = shards.contiguous()
    if local_n != widest:                      # collectives want equal sizes on every rank
        padded = torch.zeros(m, widest, dtype=shards.dtype, device=shards.device)
        padded[:, :local_n] = shards
    pieces = [torch.empty(m, widest, dtype=shards.dtype, device=shards.device) for _ in widths]
    dist.all_gather(pieces, padded, group=group)
    full = torch.cat([piece[:, :width] for piece, width in zip(pieces, widths)], dim=1)
    if out is not None:
        out.copy_(full)
        return out
    return full
