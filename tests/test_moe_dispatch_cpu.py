"""Host-side logic of the expert-parallel MoE dispatch on CPU: the send layout, counts and
token->row maps of two `gloo` ranks must reassemble, after the all-to-all, into one group per
(source rank, local expert) holding exactly the rows routed to that expert."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mircuda_b200 import moe

EXPERTS, TOP_K, TOKENS, HIDDEN = 8, 2, 40, 4


def _inputs():
    generator = torch.Generator().manual_seed(515)
    x = torch.randn(TOKENS, HIDDEN, generator=generator)
    logits = torch.randn(TOKENS, EXPERTS, generator=generator)
    return x, logits


def test_route_renormalises():
    _, logits = _inputs()
    chosen, weights = moe.route(logits, TOP_K)
    assert chosen.shape == (TOKENS, TOP_K) and weights.shape == (TOKENS, TOP_K)
    assert torch.allclose(weights.sum(dim=-1), torch.ones(TOKENS))
    probabilities = torch.softmax(logits, dim=-1)
    assert torch.equal(chosen, torch.topk(probabilities, TOP_K, dim=-1).indices)


def test_plan_dispatch_single_rank_aligned():
    _, logits = _inputs()
    chosen, _ = moe.route(logits, TOP_K)
    dispatch = moe.plan_dispatch(chosen, EXPERTS, 1, None, align=128)
    counts = torch.bincount(chosen.reshape(-1), minlength=EXPERTS)
    assert torch.equal(dispatch.counts.long(), counts)
    assert dispatch.largest_block == int(((counts + 127) // 128 * 128).sum())
    starts = torch.cumsum((counts + 127) // 128 * 128, 0) - (counts + 127) // 128 * 128
    for token in range(TOKENS):
        for choice in range(TOP_K):
            expert = int(chosen[token, choice])
            row = int(dispatch.token_rows[token * TOP_K + choice])
            assert starts[expert] <= row < starts[expert] + counts[expert]
    assert len(set(dispatch.send_rows.tolist())) == TOKENS * TOP_K


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x, logits = _inputs()
        chosen, _ = moe.route(logits, TOP_K)
        local_tokens = TOKENS // world
        local = slice(rank * local_tokens, (rank + 1) * local_tokens)
        local_experts = EXPERTS // world
        dispatch = moe.plan_dispatch(chosen[local], EXPERTS, world, None)
        largest = torch.tensor([dispatch.largest_block])
        dist.all_reduce(largest, op=dist.ReduceOp.MAX)
        capacity = int(largest.item())
        dispatch = moe.plan_dispatch(chosen[local], EXPERTS, world, capacity)
        send = torch.zeros(world * capacity, HIDDEN)
        send[dispatch.send_rows.long()] = x[local][dispatch.source_rows.long()]
        received = torch.zeros_like(send)
        counts = torch.zeros_like(dispatch.counts)
        dist.all_to_all_single(counts, dispatch.counts)
        dist.all_to_all_single(received, send)
        # Group (source s, local expert e) starts at s * capacity + the counts before e.
        ok = True
        per_source = counts.view(world, local_experts)
        for source in range(world):
            cursor = source * capacity
            source_tokens = slice(source * local_tokens, (source + 1) * local_tokens)
            for expert in range(local_experts):
                global_expert = rank * local_experts + expert
                expected_tokens = [t for t in range(local_tokens) for c in range(TOP_K)
                                   if int(chosen[source_tokens][t, c]) == global_expert]
                count = int(per_source[source, expert])
                ok &= count == len(expected_tokens)
                rows = received[cursor:cursor + count]
                expected_rows = x[source_tokens][expected_tokens]
                ok &= bool(torch.equal(rows, expected_rows))
                cursor += count
        # Combine side: the row a (token, choice) was sent to is where its result comes back.
        returned = torch.zeros_like(send)
        dist.all_to_all_single(returned, received)
        back = returned[dispatch.token_rows.long()].view(local_tokens, TOP_K, HIDDEN)
        ok &= bool(torch.equal(back, x[local][:, None, :].expand(-1, TOP_K, -1)))
        results[rank] = ok
    finally:
        dist.destroy_process_group()


def test_dispatch_round_trip_two_gloo_ranks():
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    assert dict(results) == {0: True, 1: True}
