"""GPU tests of the peer-memory expert-parallel exchange.  Several virtual ranks are emulated on
one GPU (their receive buffers are ordinary allocations on the same device and every phase is a
separate stream-ordered launch, so nothing ever waits on another kernel): plan, dispatch, grouped
matmul and pull are checked against the host oracle.  A real multi-GPU run is the benchmark's job."""
import numpy as np
import pytest
import torch

from oracle import blocks, ref
from helpers import DX_TOL, FWD_TOL, bits, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_virtual_ranks_dispatch_matmul_pull(cuda, world):
    from torch_ggml_ops_b200 import native

    qt, E, N, K, tokens, top_k, cap = ref.Q4_K, 16, 64, 256, 150, 4, 1024
    EL = E // world
    w = blocks.expert_weights(qt, E, N, K, 3)
    W = torch.from_numpy(ref.expert_weights_fp32(w, qt, N, K))
    ids = [blocks.topk_routing(tokens, E, top_k, seed=10 + r) for r in range(world)]
    xs = [blocks.gaussian_bf16((tokens, K), 20 + r) for r in range(world)]
    dys = [blocks.gaussian_bf16((tokens * top_k, N), 30 + r) for r in range(world)]
    flat = [to_dev(i.reshape(-1).astype(np.int32)) for i in ids]
    sorts = [native.route_sort(f, E) for f in flat]
    counts_all = torch.stack([torch.diff(s[3], prepend=s[3].new_zeros(1)) for s in sorts]).contiguous()
    plans = [native.ep_plan(counts_all, r, flat[r], sorts[r][1], cap) for r in range(world)]
    assert all(int(p[4].item()) == 0 for p in plans)
    x_in = [torch.full((cap, K), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    y_out = [torch.full((cap, N), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    dy_in = [torch.zeros((cap, N), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    dx_out = [torch.zeros((cap, K), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    ptrs = lambda bufs: [b.data_ptr() for b in bufs]  # noqa: E731
    for r in range(world):
        native.ep_dispatch(to_dev(xs[r]), top_k, plans[r][0], plans[r][1], ptrs(x_in))
        native.ep_dispatch(to_dev(dys[r]), 1, plans[r][0], plans[r][1], ptrs(dy_in))
    torch.cuda.synchronize()
    # layout of every owner's buffer: (local expert, source rank, order of the source's stable sort)
    for o in range(world):
        want_rows = []
        for le in range(EL):
            e = o * EL + le
            for s in range(world):
                f = ids[s].reshape(-1)
                for i in np.nonzero(f == e)[0]:
                    want_rows.append(xs[s][i // top_k])
        want = torch.stack(want_rows) if want_rows else torch.empty(0, K, dtype=torch.bfloat16)
        assert np.array_equal(bits(x_in[o][: len(want_rows)]), bits(want))
        offs = plans[o][3].cpu().numpy()
        assert offs[-1] == len(want_rows)
        assert plans[o][2].tolist() == list(range(EL))
    # owners run the grouped operators over their whole buffer; group offsets say which rows exist
    wdev = to_dev(w)
    for o in range(world):
        ws = torch.empty(native.grouped_workspace_bytes(cap, EL), dtype=torch.uint8, device="cuda")
        wl = wdev[o * EL:(o + 1) * EL].contiguous()
        native.grouped_fwd(x_in[o], wl, None, y_out[o], None, plans[o][2], plans[o][3], EL, cap, N, K, qt, ws)
        native.grouped_dx(dy_in[o], None, wl, None, dx_out[o], plans[o][2], plans[o][3], EL, cap, N, K, qt, ws)
    # token-level exchange: one row per (token, destination GPU); the owner replicates / reduces
    slots = world * tokens
    tok_in = [torch.full((slots, K), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    dx_part = [torch.full((slots, K), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    row_slot = [torch.full((cap,), -7, dtype=torch.int32, device="cuda") for _ in range(world)]
    slot_rows = [torch.full((slots, top_k), -1, dtype=torch.int32, device="cuda") for _ in range(world)]
    for r in range(world):
        native.ep_token_maps(plans[r][0], plans[r][1], tokens, top_k, r, tokens, ptrs(row_slot), ptrs(slot_rows))
        native.ep_dispatch_tokens(to_dev(xs[r]), plans[r][0], top_k, r, tokens, ptrs(tok_in))
    for o in range(world):
        n = int(plans[o][3][-1].item())
        x2 = torch.full((cap, K), float("nan"), dtype=torch.bfloat16, device="cuda")
        native.ep_expand(tok_in[o], row_slot[o], plans[o][3][EL - 1:], x2)
        torch.cuda.synchronize()
        assert np.array_equal(bits(x2[:n]), bits(x_in[o][:n]))          # same rows as the pair-level dispatch
        assert torch.isnan(x2[n:]).all()                                 # nothing written past the rows that exist
        native.ep_reduce(dx_out[o], slot_rows[o], top_k, dx_part[o])
    for r in range(world):
        dx_tok = torch.empty(tokens, K, dtype=torch.bfloat16, device="cuda")
        native.ep_pull_tokens(ptrs(dx_part), plans[r][0], top_k, r, tokens, dx_tok)
        f = ids[r].reshape(-1)
        want_dx = torch.zeros(tokens, K)
        for i in range(f.size):
            want_dx[i // top_k] += dys[r][i].float() @ W[f[i]]
        assert ref.rel_frobenius(dx_tok.float().cpu(), want_dx) < DX_TOL
    gate = torch.rand(tokens, top_k)
    for r in range(world):
        y = torch.empty(tokens * top_k, N, dtype=torch.bfloat16, device="cuda")
        native.ep_pull(ptrs(y_out), plans[r][0], plans[r][1], y, 1)
        dx = torch.empty(tokens, K, dtype=torch.bfloat16, device="cuda")
        native.ep_pull(ptrs(dx_out), plans[r][0], plans[r][1], dx, top_k, to_dev(gate.reshape(-1).contiguous()))
        f = ids[r].reshape(-1)
        xf = xs[r].float()
        want_y = torch.stack([xf[i // top_k] @ W[f[i]].t() for i in range(f.size)])
        want_dx = torch.zeros(tokens, K)
        for i in range(f.size):
            want_dx[i // top_k] += gate.reshape(-1)[i] * (dys[r][i].float() @ W[f[i]])
        assert ref.rel_frobenius(y.float().cpu(), want_y) < FWD_TOL
        assert ref.rel_frobenius(dx.float().cpu(), want_dx) < DX_TOL
    # forward with scattered output rows: every owner's matmul epilogue stores each row straight into
    # the result buffer of the rank that owns the token; bit-identical to compute-then-pull
    y_tok = [torch.full((tokens * top_k, N), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    for o in range(world):
        row_ptrs = torch.full((cap,), -1, dtype=torch.int64, device="cuda")
        native.ep_row_pointers(row_slot[o], slot_rows[o], plans[o][3][EL - 1:], top_k, tokens, ptrs(y_tok), N, row_ptrs)
        ws = torch.empty(native.grouped_workspace_bytes(cap, EL), dtype=torch.uint8, device="cuda")
        wl = wdev[o * EL:(o + 1) * EL].contiguous()
        native.grouped_fwd_rows(x_in[o], wl, row_ptrs, plans[o][2], plans[o][3], EL, cap, N, K, qt, ws)
    for r in range(world):
        y = torch.empty(tokens * top_k, N, dtype=torch.bfloat16, device="cuda")
        native.ep_pull(ptrs(y_out), plans[r][0], plans[r][1], y, 1)
        torch.cuda.synchronize()
        assert np.array_equal(bits(y_tok[r]), bits(y))
    assert native.device_status() == 0


@pytest.mark.parametrize("N", [64, 72, 200])
def test_scattered_rows_null_pointers_and_odd_widths(cuda, N):
    """tgo_grouped_fwd_rows on its own: rows go to a permuted destination, a null entry drops its row,
    out-feature counts that leave a partial last tile of weight rows take the element-wise path."""
    from torch_ggml_ops_b200 import native

    qt, E, K, sizes = ref.Q4_K, 3, 256, [70, 0, 300]
    w = blocks.expert_weights(qt, E, N, K, 8)
    R = sum(sizes)
    eo = to_dev(torch.tensor(np.cumsum(sizes), dtype=torch.int32))
    ei = to_dev(torch.arange(E, dtype=torch.int64))
    x = to_dev(blocks.gaussian_bf16((R, K), 9))
    ws = torch.empty(native.grouped_workspace_bytes(R, E), dtype=torch.uint8, device="cuda")
    y = torch.empty(R, N, dtype=torch.bfloat16, device="cuda")
    native.grouped_fwd(x, to_dev(w), None, y, None, ei, eo, E, R, N, K, qt, ws)
    perm = torch.randperm(R, generator=torch.Generator().manual_seed(3))
    dst = torch.full((R, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ptr = dst.data_ptr() + perm.to(torch.int64) * (N * 2)
    dropped = torch.arange(R) % 7 == 3
    ptr[dropped] = 0
    native.grouped_fwd_rows(x, to_dev(w), to_dev(ptr), ei, eo, E, R, N, K, qt, ws)
    torch.cuda.synchronize()
    got = dst.cpu()
    keep = ~dropped
    assert np.array_equal(bits(got[perm[keep]]), bits(y.cpu()[keep]))
    assert torch.isnan(got[perm[dropped]]).all()
    assert native.device_status() == 0


def test_token_maps_rows_zeroes_the_rows_of_dropped_pairs(cuda):
    from torch_ggml_ops_b200 import native

    tokens, top_k, cap, N = 6, 2, 16, 64
    dst_rank = torch.tensor([0, -1, 0, 0, -1, 0, 0, 0, 0, -1, 0, 0], dtype=torch.int32, device="cuda")
    dst_row = torch.tensor([0, -1, 1, 2, -1, 3, 4, 5, 6, -1, 7, 8], dtype=torch.int32, device="cuda")
    row_slot = torch.full((cap,), -1, dtype=torch.int32, device="cuda")
    slot_rows = torch.full((tokens, top_k), -9, dtype=torch.int32, device="cuda")
    result = torch.full((tokens * top_k, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    native.ep_token_maps_rows(dst_rank, dst_row, tokens, top_k, 0, tokens, [row_slot.data_ptr()], [slot_rows.data_ptr()], result)
    torch.cuda.synchronize()
    dropped = (dst_rank < 0).cpu()
    assert int(torch.count_nonzero(result.cpu()[dropped].float())) == 0 and not torch.isnan(result.cpu()[dropped]).any()
    assert torch.isnan(result.cpu()[~dropped]).all()
    assert slot_rows.reshape(-1).cpu().tolist() == dst_row.cpu().tolist()
    assert row_slot[:9].cpu().tolist() == [0, 1, 1, 2, 3, 3, 4, 5, 5]


def test_wrapper_push_forward_equals_pull_forward(cuda):
    from torch_ggml_ops_b200.peer_parallel import PeerExpertParallel

    qt, E, N, K, tokens, top_k = ref.Q4_K, 8, 128, 256, 96, 4
    w = to_dev(blocks.expert_weights(qt, E, N, K, 4))
    ids = to_dev(torch.from_numpy(blocks.topk_routing(tokens, E, top_k, seed=2)))
    x = to_dev(blocks.gaussian_bf16((tokens, K), 5))
    outs = []
    for push in (True, False):
        pep = PeerExpertParallel(w, qt, E, N, K, capacity_rows=tokens * top_k, tokens_per_rank=tokens, top_k=top_k,
                                 push_forward=push)
        assert pep.push == push
        plan = pep.plan(ids)
        outs.append(pep.forward(plan, x).clone())
        pep.check_overflow()
    torch.cuda.synchronize()
    assert np.array_equal(bits(outs[0]), bits(outs[1]))


def test_capacity_overflow_is_flagged_not_written(cuda):
    from torch_ggml_ops_b200 import native

    E, tokens, top_k, cap = 4, 64, 2, 16
    ids = blocks.topk_routing(tokens, E, top_k, seed=1)
    flat = to_dev(ids.reshape(-1).astype(np.int32))
    _, p2s, _, ends = native.route_sort(flat, E)
    counts = torch.diff(ends, prepend=ends.new_zeros(1)).reshape(1, E).contiguous()
    dst_rank, dst_row, _, _, overflow = native.ep_plan(counts, 0, flat, p2s, cap)
    assert int(overflow.item()) == 1
    kept = dst_rank.cpu().numpy() >= 0
    assert kept.sum() == cap and int(dst_row.max().item()) == cap - 1


@pytest.mark.parametrize("token_level", [False, True])
def test_single_rank_wrapper(cuda, token_level):
    from torch_ggml_ops_b200.peer_parallel import PeerExpertParallel

    qt, E, N, K, tokens, top_k = ref.Q5_K, 8, 128, 512, 100, 2
    w = blocks.expert_weights(qt, E, N, K, 4)
    W = torch.from_numpy(ref.expert_weights_fp32(w, qt, N, K))
    ids = blocks.topk_routing(tokens, E, top_k, seed=2)
    x = blocks.gaussian_bf16((tokens, K), 5)
    dy = blocks.gaussian_bf16((tokens * top_k, N), 6)
    pep = PeerExpertParallel(to_dev(w), qt, E, N, K, capacity_rows=512, tokens_per_rank=tokens if token_level else None,
                             top_k=top_k)
    plan = pep.plan(to_dev(torch.from_numpy(ids)))
    assert plan["token_level"] == token_level
    y = pep.forward(plan, to_dev(x))
    dx = pep.grad_input(plan, to_dev(dy))
    f = ids.reshape(-1)
    want_y = torch.stack([x[i // top_k].float() @ W[f[i]].t() for i in range(f.size)])
    want_dx = torch.zeros(tokens, K)
    for i in range(f.size):
        want_dx[i // top_k] += dy[i].float() @ W[f[i]]
    assert ref.rel_frobenius(y.float().cpu(), want_y) < FWD_TOL
    assert ref.rel_frobenius(dx.float().cpu(), want_dx) < DX_TOL
    assert int(pep.overflow.item()) == 0
    pep.check_overflow()
    if token_level:
        with pytest.raises(ValueError, match="top_k"):   # every rank must take the same exchange form
            pep.plan(to_dev(torch.from_numpy(ids[:, :1].copy())))


def test_overflow_is_surfaced_by_the_wrapper(cuda):
    from torch_ggml_ops_b200.peer_parallel import PeerExpertParallel

    qt, E, N, K, tokens, top_k = ref.Q4_K, 4, 64, 256, 64, 2
    w = blocks.expert_weights(qt, E, N, K, 4)
    W = torch.from_numpy(ref.expert_weights_fp32(w, qt, N, K))
    ids = blocks.topk_routing(tokens, E, top_k, seed=1)
    x = blocks.gaussian_bf16((tokens, K), 5)
    pep = PeerExpertParallel(to_dev(w), qt, E, N, K, capacity_rows=48)      # 128 routed pairs do not fit
    plan = pep.plan(to_dev(torch.from_numpy(ids)))
    y = pep.forward(plan, to_dev(x))
    with pytest.raises(RuntimeError, match="overflow"):
        pep.check_overflow()
    # the pairs that fitted are computed (also those of the expert that straddles the capacity), the rest are zeros
    kept = plan["dst_rank"].cpu().numpy() >= 0
    assert kept.sum() == 48
    f = ids.reshape(-1)
    want = torch.stack([x[i // top_k].float() @ W[f[i]].t() for i in range(f.size)])
    got = y.float().cpu()
    assert ref.rel_frobenius(got[kept], want[kept]) < FWD_TOL
    assert int(torch.count_nonzero(got[~kept])) == 0
    # the flag describes the last plan only
    pep2_ids = to_dev(torch.from_numpy(ids[:20].copy()))
    pep.plan(pep2_ids)
    pep.check_overflow()


def test_rank_barrier_and_count_exchange_kernels(cuda):
    """The peer-memory rank barrier on one GPU: with every flag already set it passes at once; with
    a peer that never arrives its bounded wait runs out, the status word records code 11 and the
    context stays usable (no kernel ever waits on another launch here: rank 1 simply never calls)."""
    from torch_ggml_ops_b200 import native

    world, E = 2, 8
    flags = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(world)]
    tables = [torch.full((world, E), -1, dtype=torch.int32, device="cuda") for _ in range(world)]
    ptrs = lambda bufs: [b.data_ptr() for b in bufs]  # noqa: E731
    for r in range(world):
        native.ep_share_counts(torch.arange(E, dtype=torch.int32, device="cuda") + 10 * r, r, ptrs(tables))
    torch.cuda.synchronize()
    for t in tables:
        assert t.cpu().tolist() == [list(range(E)), list(range(10, 10 + E))]
    # rank 1 "arrived" already (its slot holds the epoch everywhere): rank 0 passes
    for f in flags:
        f[1] = 1
    assert native.device_status() == 0
    native.ep_barrier(ptrs(flags), 0, 1, limit_cycles=2_000_000)
    torch.cuda.synchronize()
    assert native.device_status() == 0
    assert flags[0].cpu().tolist()[:2] == [1, 1] and flags[1].cpu().tolist()[:2] == [1, 1]
    # epoch 2: rank 1 never signals; the wait gives up after about a millisecond
    native.ep_barrier(ptrs(flags), 0, 2, limit_cycles=2_000_000)
    torch.cuda.synchronize()
    status = native.device_status()
    assert status & 0xFF == 11 and status >> 8 == 1          # code, and the rank that was missing
    assert native.device_status() == 0
    x = torch.ones(8, device="cuda") * 2                      # the context still works
    assert float(x.sum()) == 16.0


def test_phase_times_reports_every_phase_of_a_step(cuda):
    from torch_ggml_ops_b200.peer_parallel import PeerExpertParallel

    qt, E, N, K, tokens, top_k = ref.Q4_K, 8, 128, 256, 64, 4
    w = to_dev(blocks.expert_weights(qt, E, N, K, 4))
    ids = to_dev(torch.from_numpy(blocks.topk_routing(tokens, E, top_k, seed=2)))
    x = to_dev(blocks.gaussian_bf16((tokens, K), 5))
    dy = to_dev(blocks.gaussian_bf16((tokens * top_k, N), 6))
    pep = PeerExpertParallel(w, qt, E, N, K, capacity_rows=tokens * top_k, tokens_per_rank=tokens, top_k=top_k)

    def step():
        plan = pep.plan(ids)
        pep.forward(plan, x)
        pep.grad_input(plan, dy)

    ph = pep.phase_times(step)
    assert set(ph) == {"plan", "dispatch_tokens", "barriers", "expand", "forward_matmul_and_return", "dispatch_dy",
                       "dx_matmul", "reduce", "pull_partial_sums"}
    assert all(v >= 0.0 for v in ph.values()) and pep.marks is None
