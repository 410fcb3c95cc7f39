"""Fused GEMM + all-gather over NVLink peer stores: two ranks, each owning half of the weight
rows, must both end up with the full output, equal to the single-GPU result. Needs 2 GPUs
(skipped otherwise); ranks run as child processes with NVLS off and plain peer stores."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import oracle
        from helpers import bf16_bits
        from mircuda_b200 import gather, plans, sharding
        m, n, k = 512, 1024, 512
        generator = torch.Generator().manual_seed(11)
        x = torch.randn(m, k, generator=generator).to(torch.bfloat16).cuda()
        w = (torch.randn(n, k, generator=generator) * 0.05).to(torch.bfloat16).cuda()
        begin, end = sharding.column_shard(n, world, rank)
        stream = torch.cuda.Stream()
        a_codes = torch.empty(m * k, dtype=torch.uint8, device="cuda")
        a_scales = torch.zeros(plans.scale_bytes(m, k // 32), dtype=torch.uint8, device="cuda")
        b_codes = torch.empty((end - begin) * k, dtype=torch.uint8, device="cuda")
        b_scales = torch.zeros(plans.scale_bytes(end - begin, k // 32), dtype=torch.uint8, device="cuda")
        plan = plans.BlockScaledMxFp8Plan(stream, plans.BlockScaledMxFp8Spec(m, end - begin, k))
        full_codes, full_scales = oracle.mxfp8_quantize(bf16_bits(w))
        x_codes, x_scales = oracle.mxfp8_quantize(bf16_bits(x))
        expected = oracle.mxfp8_gemm(x_codes, x_scales, full_codes, full_scales)
        ok = True
        # Once with one store per rank, once through the multicast address (where the fabric has
        # one; otherwise the second pass repeats the first path).
        for multicast in (False, True):
            output = gather.SymmetricOutput(m, n, torch.device("cuda", rank))
            output.local.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            with torch.cuda.stream(stream):
                plans.mxfp8_quantize_bf16(stream, x, a_codes, a_scales)
                plans.mxfp8_quantize_bf16(stream, w[begin:end].contiguous(), b_codes, b_scales)
                gather.execute_gather(plan, stream, a_codes, a_scales, b_codes, b_scales, output,
                                      begin, multicast)
                output.barrier()
            stream.synchronize()
            actual = bf16_bits(output.matrix())
            stats = oracle.compare_bf16(actual, expected)
            ok = ok and (not np.isnan(oracle.bf16_to_f32(actual)).any()
                         and stats["max_rel_to_max"] <= 1e-2 and stats["rel_frobenius"] <= 5e-3)
            dist.barrier()
        # The same gather carried by the copy engines: the GEMM writes the rank's own buffer only
        # and one strided copy per peer moves the finished block.
        copier = gather.ColumnCopier(world, rank)
        for _ in range(2):
            output = gather.SymmetricOutput(m, n, torch.device("cuda", rank))
            output.local.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            with torch.cuda.stream(stream):
                copier.execute(plan, stream, a_codes, a_scales, b_codes, b_scales, output, begin, end)
                copier.join(stream)
                output.barrier()
            stream.synchronize()
            actual = bf16_bits(output.matrix())
            stats = oracle.compare_bf16(actual, expected)
            ok = ok and (not np.isnan(oracle.bf16_to_f32(actual)).any()
                         and stats["max_rel_to_max"] <= 1e-2 and stats["rel_frobenius"] <= 5e-3)
            dist.barrier()
        # Rank-major blocks (what an all-gather call returns): rank r's [m, n / world] result is
        # block r everywhere, sent as one contiguous copy per peer; the quantizer of a following
        # layer reads that layout in place.
        local_n = end - begin
        blocks = gather.SymmetricOutput(world * m, local_n, torch.device("cuda", rank))
        blocks.local.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
        with torch.cuda.stream(stream):
            copier.execute_blocks(plan, stream, a_codes, a_scales, b_codes, b_scales, blocks)
            copier.join(stream)
            blocks.barrier()
        stream.synchronize()
        gathered = blocks.matrix().view(world, m, local_n).permute(1, 0, 2).reshape(m, n)
        stats = oracle.compare_bf16(bf16_bits(gathered.contiguous()), expected)
        ok = ok and stats["max_rel_to_max"] <= 1e-2 and stats["rel_frobenius"] <= 5e-3
        next_codes = torch.empty(m * n, dtype=torch.uint8, device="cuda")
        next_scales = torch.zeros(plans.scale_bytes(m, n // 32), dtype=torch.uint8, device="cuda")
        plans.mxfp8_quantize_bf16(stream, blocks.matrix().view(world, m, local_n), next_codes, next_scales,
                                  blocks=world)
        stream.synchronize()
        want_codes, want_scales = oracle.mxfp8_quantize(bf16_bits(gathered.contiguous()))
        ok = ok and np.array_equal(next_codes.cpu().numpy().reshape(m, n), want_codes)
        ok = ok and np.array_equal(next_scales.cpu().numpy(), want_scales)
        dist.barrier()
        copier.close()
        results[rank] = (ok, bool(output.multicast))
    finally:
        dist.destroy_process_group()


def test_fused_gather_two_ranks():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    assert all(ok for ok, _ in results.values()) and set(results.keys()) == {0, 1}, dict(results)
    print("multicast address available:", [has for _, has in results.values()])
