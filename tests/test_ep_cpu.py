"""CPU tests (gloo, world_size 2 and 3) of the expert-parallel row exchange: counts, split
sizes, permutations and their inverses, with a stand-in for the expert computation so that no
GPU is needed."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, E, tokens, top_k, width, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torch_ggml_ops_b200.expert_parallel import ExpertParallel

        ep = ExpertParallel(E)
        g = torch.Generator().manual_seed(100 + rank)
        logits = torch.randn(tokens, E, generator=g)
        ids = torch.topk(logits, top_k, dim=1).indices
        x = torch.randn(tokens, width, generator=g)
        plan = ep.plan(ids)
        # every rank agrees on how many rows cross each pair
        sent = torch.tensor(plan.send_splits)
        got = torch.tensor(plan.recv_splits)
        all_sent = [torch.zeros_like(sent) for _ in range(world)]
        dist.all_gather(all_sent, sent)
        assert [int(all_sent[s][rank]) for s in range(world)] == got.tolist()
        rows = ep.dispatch_tokens(plan, x)
        assert rows.shape == (plan.rows_recv, width)
        assert int(plan.expert_offsets[-1]) == plan.rows_recv
        assert plan.expert_indices.tolist() == list(range(E // world))
        # stand-in expert: multiply by (global expert id + 1); rows are expert-major
        out = torch.empty_like(rows)
        begin = 0
        for le, end in enumerate(plan.expert_offsets.tolist()):
            out[begin:end] = rows[begin:end] * float(rank * ep.experts_per_rank + le + 1)
            begin = end
        back = ep.combine_rows(plan, out)
        want = x.repeat_interleave(top_k, 0) * (ids.reshape(-1, 1).float() + 1.0)
        assert torch.equal(back, want)
        w = torch.rand(tokens, top_k, generator=g)
        summed = ep.combine_tokens(plan, out, w)
        want_sum = (want.reshape(tokens, top_k, width) * w.unsqueeze(-1)).sum(1)
        assert torch.allclose(summed, want_sum, rtol=1e-5, atol=1e-5)
        # dispatch_rows moves per-routed-row data (the backward cotangent) with the same plan
        dy = torch.randn(tokens * top_k, 3, generator=g)
        assert torch.equal(ep.combine_rows(plan, ep.dispatch_rows(plan, dy)), dy)
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_dispatch_and_combine_round_trip(world):
    mgr = mp.Manager()
    results = mgr.dict()
    port = _free_port()
    mp.spawn(_worker, args=(world, port, 12, 37, 4, 8, results), nprocs=world, join=True)
    assert dict(results) == {r: "ok" for r in range(world)}


def test_single_rank_plan_is_a_plain_sort():
    from torch_ggml_ops_b200.expert_parallel import ExpertParallel

    ep = ExpertParallel(8)
    ids = torch.tensor([[3, 1], [0, 3], [7, 1]])
    plan = ep.plan(ids)
    assert plan.send_splits == [6] and plan.recv_splits == [6]
    assert plan.expert_offsets.tolist() == [1, 3, 3, 5, 5, 5, 5, 6]
    x = torch.arange(3.0).reshape(3, 1)
    rows = ep.dispatch_tokens(plan, x)
    assert rows.reshape(-1).tolist() == [1.0, 0.0, 2.0, 0.0, 1.0, 2.0]
    assert torch.equal(ep.combine_rows(plan, rows), x.repeat_interleave(2, 0))


def test_uneven_expert_split_is_refused():
    from torch_ggml_ops_b200.expert_parallel import ExpertParallel

    assert ExpertParallel(7).experts_per_rank == 7  # one rank: anything divides
