"""GPU tests of the expert-parallel MoE feed-forward step (gate/up pair -> silu(gate) * up -> down
projection -> weighted top-k combine, forward and input gradient) with the quant types of the
expert-parallel benchmark configuration: IQ2_S gate/up, Q6_K down.

Several virtual ranks are stepped in lockstep on one GPU: their "peer" buffers are ordinary
allocations on the same device and every phase is a separate stream-ordered launch, so nothing ever
waits on another kernel.  Checked against the fp32 oracle chain end to end, and stage by stage with
the per-operator tolerances (each grouped matmul against the oracle applied to that stage's own
device inputs).  The reference defines the per-operator semantics only
(tests/test_grouped_mmq.py:108-170); the block around them is this library's."""
import numpy as np
import pytest
import torch

from oracle import blocks, ref
from helpers import DX_TOL, FWD_TOL, to_dev

pytestmark = pytest.mark.gpu

CHAIN_TOL = 1e-2   # three bf16 roundings in a row (gate/up, activation, down) plus the partial sums


def _silu(x):
    return x * torch.sigmoid(x)


def _dsilu(x):
    s = torch.sigmoid(x)
    return s * (1 + x * (1 - s))


@pytest.mark.parametrize("scaled", [False, True])
def test_swiglu_kernels(cuda, scaled):
    from torch_ggml_ops_b200 import native

    rows, width, live = 300, 264, 257
    g, u, dh = (to_dev(blocks.gaussian_bf16((rows, width), s)) for s in (1, 2, 3))
    scale = to_dev(torch.rand(rows) + 0.5) if scaled else None
    n = torch.tensor([live], dtype=torch.int32, device="cuda")
    h = torch.full((rows, width), 7.0, dtype=torch.bfloat16, device="cuda")
    dg, du = torch.full_like(h, 7.0), torch.full_like(h, 7.0)
    native.swiglu_fwd(g, u, h, row_scale=scale, n_rows_device=n)
    native.swiglu_bwd(dh, g, u, dg, du, row_scale=scale, n_rows_device=n)
    gf, uf, df = g.float(), u.float(), dh.float()
    s = scale[:, None] if scaled else 1.0
    for got, want in ((h, s * _silu(gf) * uf), (dg, df * s * uf * _dsilu(gf)), (du, df * s * _silu(gf))):
        assert bool((got[live:] == 7.0).all())          # rows past the device-side count are not touched
        err = (got[:live].float() - want[:live]).abs()
        assert bool((err <= want[:live].abs() * 2.0 ** -7 + 1e-6).all())   # one bf16 rounding of the fp32 value


def _make_world(world, E, H, F, tokens, top_k, cap, qt_gu, qt_d, weighted):
    from torch_ggml_ops_b200.moe_parallel import PEER_BUFFERS, MoEMLPRank

    EL = E // world
    wg, wu = blocks.expert_weights(qt_gu, E, F, H, 3), blocks.expert_weights(qt_gu, E, F, H, 4)
    wd = blocks.expert_weights(qt_d, E, H, F, 5)
    W = {k: torch.from_numpy(ref.expert_weights_fp32(w, qt, n, kk))
         for k, (w, qt, n, kk) in dict(g=(wg, qt_gu, F, H), u=(wu, qt_gu, F, H), d=(wd, qt_d, H, F)).items()}
    ranks = [MoEMLPRank(r, world, to_dev(wg[r * EL:(r + 1) * EL]), to_dev(wu[r * EL:(r + 1) * EL]),
                        to_dev(wd[r * EL:(r + 1) * EL]), qt_gu, qt_d, E, H, F, cap, tokens, top_k) for r in range(world)]
    peers = {name: [rk.buf[name].data_ptr() for rk in ranks] for name in PEER_BUFFERS}
    for rk in ranks:
        rk.connect(peers)
    ids = [blocks.topk_routing(tokens, E, top_k, seed=10 + r) for r in range(world)]
    gate_w = [torch.rand(tokens, top_k) + 0.25 if weighted else None for _ in range(world)]
    xs = [blocks.gaussian_bf16((tokens, H), 20 + r) for r in range(world)]
    dys = [blocks.gaussian_bf16((tokens, H), 30 + r) for r in range(world)]
    return ranks, W, ids, gate_w, xs, dys


def _oracle(W, ids, gate_w, x, dy):
    """fp32 chain for one rank's tokens: (y [tokens, H], dx [tokens, H])."""
    tokens, top_k = ids.shape
    xf, dyf = x.float(), dy.float()
    y, dx = torch.zeros_like(xf), torch.zeros_like(xf)
    for t in range(tokens):
        for s in range(top_k):
            e = int(ids[t, s])
            w = float(gate_w[t, s]) if gate_w is not None else 1.0
            g, u = W["g"][e] @ xf[t], W["u"][e] @ xf[t]
            y[t] += w * (W["d"][e] @ (_silu(g) * u))
            dh = w * (dyf[t] @ W["d"][e])
            dx[t] += (dh * u * _dsilu(g)) @ W["g"][e] + (dh * _silu(g)) @ W["u"][e]
    return y, dx


@pytest.mark.parametrize("world,weighted", [(1, False), (2, True), (4, True), (8, False)])
def test_virtual_ranks_moe_mlp_step(cuda, world, weighted):
    from torch_ggml_ops_b200 import native

    E, H, F, tokens, top_k, cap = 16, 512, 256, 96, 4, 1024
    qt_gu, qt_d = ref.IQ2_S, ref.Q6_K
    ranks, W, ids, gate_w, xs, dys = _make_world(world, E, H, F, tokens, top_k, cap, qt_gu, qt_d, weighted)
    counts = torch.stack([rk.route(to_dev(torch.from_numpy(ids[r]))) for r, rk in enumerate(ranks)]).contiguous()
    for r, rk in enumerate(ranks):
        rk.make_plan(counts, None if gate_w[r] is None else to_dev(gate_w[r]))
    for r, rk in enumerate(ranks):
        rk.fwd_send(to_dev(xs[r]))
    for rk in ranks:
        rk.fwd_compute()
    ys = [rk.fwd_recv() for rk in ranks]
    for r, rk in enumerate(ranks):
        rk.bwd_send(to_dev(dys[r]))
    for rk in ranks:
        rk.bwd_compute()
    dxs = [rk.bwd_recv() for rk in ranks]
    torch.cuda.synchronize()
    for r, rk in enumerate(ranks):
        rk.check_overflow()
        want_y, want_dx = _oracle(W, ids[r], gate_w[r], xs[r], dys[r])
        assert ref.rel_frobenius(ys[r].float().cpu(), want_y) < CHAIN_TOL
        assert ref.rel_frobenius(dxs[r].float().cpu(), want_dx) < CHAIN_TOL
        assert ref.max_row_error(ys[r].float().cpu(), want_y) < 2 * CHAIN_TOL
        assert ref.max_row_error(dxs[r].float().cpu(), want_dx) < 2 * CHAIN_TOL
    assert native.device_status() == 0


def test_moe_mlp_stage_by_stage(cuda):
    """Every grouped matmul of the step against the oracle applied to that stage's own device
    inputs, with the per-operator tolerances (forward 1e-2, input gradient 5e-3)."""
    world, E, H, F, tokens, top_k, cap = 2, 8, 512, 256, 120, 2, 512
    qt_gu, qt_d = ref.IQ2_S, ref.Q6_K
    ranks, W, ids, gate_w, xs, dys = _make_world(world, E, H, F, tokens, top_k, cap, qt_gu, qt_d, True)
    EL = E // world
    counts = torch.stack([rk.route(to_dev(torch.from_numpy(ids[r]))) for r, rk in enumerate(ranks)]).contiguous()
    for r, rk in enumerate(ranks):
        rk.make_plan(counts, to_dev(gate_w[r]))
    for r, rk in enumerate(ranks):
        rk.fwd_send(to_dev(xs[r]))
    snap = []
    for rk in ranks:
        rk.fwd_compute()
        torch.cuda.synchronize()
        snap.append({k: getattr(rk, k).clone() for k in ("rows_a", "gate", "up", "h", "rows_b")})
    for r, rk in enumerate(ranks):
        rk.fwd_recv()
        rk.bwd_send(to_dev(dys[r]))
    for o, rk in enumerate(ranks):
        rk.bwd_compute()
        torch.cuda.synchronize()
        offs = rk.plan["offsets"].cpu().numpy()
        n = int(offs[-1])
        scale = rk.buf["row_weight"].reshape(-1)[:n].cpu()
        le = list(range(EL))
        Wg, Wu, Wd = (W[k][o * EL:(o + 1) * EL].numpy() for k in ("g", "u", "d"))
        f = snap[o]
        x_rows, g, u, h, y_rows = (f[k][:n].cpu() for k in ("rows_a", "gate", "up", "h", "rows_b"))
        assert ref.rel_frobenius(g.float(), ref.grouped_forward(x_rows, Wg, le, offs)) < FWD_TOL
        assert ref.rel_frobenius(u.float(), ref.grouped_forward(x_rows, Wu, le, offs)) < FWD_TOL
        want_h = scale[:, None] * _silu(g.float()) * u.float()
        assert ref.rel_frobenius(h.float(), want_h) < 5e-3
        assert ref.rel_frobenius(y_rows.float(), ref.grouped_forward(h, Wd, le, offs)) < FWD_TOL
        dy_rows, dh, dg, du, dx_rows = (t[:n].cpu() for t in (rk.rows_a, rk.h, rk.dgate, rk.dup, rk.rows_b))
        assert ref.rel_frobenius(dh.float(), ref.grouped_grad_input(dy_rows, Wd, le, offs)) < DX_TOL
        assert ref.rel_frobenius(dg.float(), dh.float() * scale[:, None] * u.float() * _dsilu(g.float())) < 5e-3
        assert ref.rel_frobenius(du.float(), dh.float() * scale[:, None] * _silu(g.float())) < 5e-3
        assert ref.rel_frobenius(dx_rows.float(), ref.grouped_grad_input(dg, Wg, le, offs, second=(du, Wu))) < DX_TOL


def test_single_process_wrapper(cuda):
    from torch_ggml_ops_b200.moe_parallel import PeerMoEMLP

    E, H, F, tokens, top_k = 8, 256, 256, 64, 2
    qt_gu, qt_d = ref.Q5_K, ref.Q6_K
    wg, wu, wd = blocks.expert_weights(qt_gu, E, F, H, 3), blocks.expert_weights(qt_gu, E, F, H, 4), blocks.expert_weights(qt_d, E, H, F, 5)
    W = {"g": torch.from_numpy(ref.expert_weights_fp32(wg, qt_gu, F, H)), "u": torch.from_numpy(ref.expert_weights_fp32(wu, qt_gu, F, H)),
         "d": torch.from_numpy(ref.expert_weights_fp32(wd, qt_d, H, F))}
    mlp = PeerMoEMLP(to_dev(wg), to_dev(wu), to_dev(wd), qt_gu, qt_d, E, H, F, capacity_rows=tokens * top_k,
                     tokens_per_rank=tokens, top_k=top_k)
    ids = blocks.topk_routing(tokens, E, top_k, seed=2)
    gw = torch.rand(tokens, top_k)
    x, dy = blocks.gaussian_bf16((tokens, H), 5), blocks.gaussian_bf16((tokens, H), 6)
    for _ in range(2):   # a second step reuses every buffer
        mlp.plan(to_dev(torch.from_numpy(ids)), to_dev(gw))
        y = mlp.forward(to_dev(x))
        dx = mlp.grad_input(to_dev(dy))
    mlp.check_overflow()
    want_y, want_dx = _oracle(W, ids, gw, x, dy)
    assert ref.rel_frobenius(y.float().cpu(), want_y) < CHAIN_TOL
    assert ref.rel_frobenius(dx.float().cpu(), want_dx) < CHAIN_TOL
    with pytest.raises(ValueError, match="top_k"):
        mlp.plan(to_dev(torch.from_numpy(ids[:, :1].copy())))
