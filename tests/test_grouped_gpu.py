"""GPU parity of the grouped and paired operators (reference properties:
tests/test_grouped_mmq.py:173-668) on seeded synthetic experts and routing."""
import numpy as np
import pytest
import torch

from oracle import blocks, ref
from helpers import ALL_TYPES, DX_TOL, FWD_TOL, bits, expert_case, routing_from_sizes, to_dev

pytestmark = pytest.mark.gpu


def run_grouped(qt, E, N, K, sizes, ids, seed=0, pair=False):
    """Forward + backward through the torch operators; returns device results and oracle values."""
    import torch_ggml_ops_b200 as tgo

    w0, W0 = expert_case(qt, E, N, K, seed + 1)
    R = int(sum(sizes))
    ei, eo = routing_from_sizes(sizes, ids)
    x = blocks.gaussian_bf16((R, K), seed + 2)
    dy0 = blocks.gaussian_bf16((R, N), seed + 3)
    xd = to_dev(x).requires_grad_(True)
    if not pair:
        y = tgo.grouped_mmq(xd, to_dev(w0), to_dev(ei), to_dev(eo), qt, N)
        y.backward(to_dev(dy0))
        return {"y": (y.detach(), ref.grouped_forward(x, W0, ids, eo)),
                "dx": (xd.grad, ref.grouped_grad_input(dy0, W0, ids, eo))}
    w1, W1 = expert_case(qt, E, N, K, seed + 4)
    dy1 = blocks.gaussian_bf16((R, N), seed + 5)
    y0, y1 = tgo.grouped_mmq_pair(xd, to_dev(w0), to_dev(w1), to_dev(ei), to_dev(eo), qt, N)
    torch.autograd.backward([y0, y1], [to_dev(dy0), to_dev(dy1)])
    return {"y0": (y0.detach(), ref.grouped_forward(x, W0, ids, eo)),
            "y1": (y1.detach(), ref.grouped_forward(x, W1, ids, eo)),
            "dx": (xd.grad, ref.grouped_grad_input(dy0, W0, ids, eo, second=(dy1, W1)))}


@pytest.mark.parametrize("name,qt", ALL_TYPES)
def test_grouped_forward_and_grad_input(cuda, name, qt):
    # the reference's group layout: experts [0,2,5,7], ends [1,128,257,262]
    res = run_grouped(qt, 8, 96, 512, [1, 127, 129, 5], [0, 2, 5, 7], seed=qt)
    assert ref.rel_frobenius(res["y"][0].float().cpu(), res["y"][1]) < FWD_TOL
    assert ref.rel_frobenius(res["dx"][0].float().cpu(), res["dx"][1]) < DX_TOL


@pytest.mark.parametrize("name,qt", ALL_TYPES)
def test_pair_forward_and_fused_grad_input(cuda, name, qt):
    res = run_grouped(qt, 6, 128, 512, [65, 129, 129, 189], [4, 1, 0, 3], seed=10 + qt, pair=True)
    assert ref.rel_frobenius(res["y0"][0].float().cpu(), res["y0"][1]) < FWD_TOL
    assert ref.rel_frobenius(res["y1"][0].float().cpu(), res["y1"][1]) < FWD_TOL
    assert ref.rel_frobenius(res["dx"][0].float().cpu(), res["dx"][1]) < DX_TOL


@pytest.mark.parametrize("name,qt", ALL_TYPES)
def test_pair_equals_two_singles_bit_for_bit(cuda, name, qt):
    import torch_ggml_ops_b200 as tgo

    E, N, K = 5, 512, 2048 if qt != ref.Q6_K else 512
    sizes, ids = [65, 129, 129, 189], [0, 4, 2, 3]
    w0, _ = expert_case(qt, E, N, K, 1)
    w1, _ = expert_case(qt, E, N, K, 2)
    ei, eo = routing_from_sizes(sizes, ids)
    x = to_dev(blocks.gaussian_bf16((sum(sizes), K), 3))
    args = (to_dev(ei), to_dev(eo), qt, N)
    y0, y1 = tgo.grouped_mmq_pair(x, to_dev(w0), to_dev(w1), *args)
    s0 = tgo.grouped_mmq(x, to_dev(w0), *args)
    s1 = tgo.grouped_mmq(x, to_dev(w1), *args)
    assert np.array_equal(bits(y0), bits(s0)) and np.array_equal(bits(y1), bits(s1))


@pytest.mark.parametrize("name,qt", ALL_TYPES)
def test_grouped_equals_per_group_dense_bit_for_bit(cuda, name, qt):
    """Each group's rows equal the dense operator run on that expert alone, forward and backward
    (reference: tests/test_grouped_mmq.py:233-280, 283-320)."""
    import torch_ggml_ops_b200 as tgo

    E, N, K = 4, 512, 2048
    sizes, ids = [65, 129, 129, 189], [3, 0, 2, 1]
    w, _ = expert_case(qt, E, N, K, 5)
    wd = to_dev(w)
    ei, eo = routing_from_sizes(sizes, ids)
    x = to_dev(blocks.gaussian_bf16((sum(sizes), K), 6))
    dy = to_dev(blocks.gaussian_bf16((sum(sizes), N), 7))
    y = tgo.grouped_mmq(x, wd, to_dev(ei), to_dev(eo), qt, N)
    dx = torch.ops.torch_ggml_ops.grouped_mmq_grad_input(dy, wd, to_dev(ei), to_dev(eo), qt, K)
    b = 0
    for e, n in zip(ids, sizes):
        flat = wd[e].reshape(-1).clone()
        assert np.array_equal(bits(y[b:b + n]), bits(tgo.mmq(x[b:b + n].clone(), flat, qt, N)))
        assert np.array_equal(bits(dx[b:b + n]),
                              bits(torch.ops.torch_ggml_ops.mmq_grad_input(dy[b:b + n].clone(), flat, qt, K)))
        b += n


@pytest.mark.parametrize("qt", [ref.Q4_K, ref.Q3_K])
@pytest.mark.parametrize("size", [1, 15, 16, 17, 63, 64, 65, 127, 128, 129, 255, 256, 257, 600])
def test_group_size_boundaries(cuda, qt, size):
    res = run_grouped(qt, 3, 64, 256, [size, 3, size], [2, 0, 1], seed=size)
    assert ref.rel_frobenius(res["y"][0].float().cpu(), res["y"][1]) < FWD_TOL
    assert ref.rel_frobenius(res["dx"][0].float().cpu(), res["dx"][1]) < DX_TOL


def test_invalid_and_empty_groups_are_skipped_and_leave_rows_untouched(cuda):
    from torch_ggml_ops_b200 import native

    qt, E, N, K = ref.Q4_K, 6, 64, 256
    w, W = expert_case(qt, E, N, K, 1)
    # groups: valid, empty, expert id out of range, valid, span past the end
    ids = [1, 2, 9, 0, 3]
    ends = [10, 10, 20, 30, 50]
    R = 40
    x = blocks.gaussian_bf16((R, K), 2)
    ei, eo = torch.tensor(ids, dtype=torch.int64), torch.tensor(ends, dtype=torch.int32)
    y = torch.full((R, N), 7.0, dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(native.grouped_workspace_bytes(R, len(ids)), dtype=torch.uint8, device="cuda")
    native.grouped_fwd(to_dev(x), to_dev(w), None, y, None, to_dev(ei), to_dev(eo), E, R, N, K, qt, ws)
    want = ref.grouped_forward(x, W, ids, ends)
    got = y.float().cpu()
    valid = torch.isfinite(want[:, 0])
    assert valid.sum() == 20
    assert ref.rel_frobenius(got[valid], want[valid]) < FWD_TOL
    assert bool((got[~valid] == 7.0).all())
    assert int(ws[:4].view(torch.int32).item()) == 2 and native.device_status() == 0


def test_third_benchmark_configuration_full_size(cuda):
    """256 experts of Q4_K 512 x 2048, 8192 tokens top-8 (65536 routed rows), forward + dX.
    Checked against the oracle on a sample of groups, and over all groups through the
    size-independent property grouped == dense per group."""
    import torch_ggml_ops_b200 as tgo

    qt, E, N, K, tokens, top_k = ref.Q4_K, 256, 512, 2048, 8192, 8
    ids = blocks.topk_routing(tokens, E, top_k, seed=3)
    perm, ei, eo = blocks.sort_by_expert(ids, E)
    R = tokens * top_k
    w = blocks.expert_weights(qt, E, N, K, 5)
    wd = to_dev(w)
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn((R, K), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16).requires_grad_(True)
    dy = torch.randn((R, N), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    y = tgo.grouped_mmq(x, wd, to_dev(ei), to_dev(eo), qt, N)
    y.backward(dy)
    starts = np.concatenate([[0], eo[:-1]])
    order = np.argsort(-(eo - starts))
    for e in list(order[:3]) + list(order[-3:]) + [17, 101]:
        b, end = int(starts[e]), int(eo[e])
        if end == b:
            continue
        We = ref.weight_fp32(w[e].reshape(-1), qt, N, K)
        want_y, want_dx = ref.mmq_forward(x[b:end].detach().cpu(), We), ref.mmq_grad_input(dy[b:end].cpu(), We)
        assert ref.rel_frobenius(y[b:end].detach().float().cpu(), want_y) < FWD_TOL
        assert ref.rel_frobenius(x.grad[b:end].float().cpu(), want_dx) < DX_TOL
        assert ref.max_row_error(y[b:end].detach().float().cpu(), want_y) < 1e-2
        assert ref.max_row_error(x.grad[b:end].float().cpu(), want_dx) < 1e-2
        flat = wd[e].reshape(-1).clone()
        assert np.array_equal(bits(y[b:end]), bits(tgo.mmq(x[b:end].detach().clone(), flat, qt, N)))
    assert not torch.isnan(y).any() and not torch.isnan(x.grad).any()


def _sampled_groups(eo, extra=(17, 101)):
    """Three largest, three smallest and two fixed groups: (start, end, expert) with end > start."""
    starts = np.concatenate([[0], eo[:-1]])
    order = np.argsort(-(eo - starts))
    picks = []
    for e in list(order[:3]) + list(order[-3:]) + list(extra):
        b, end = int(starts[e]), int(eo[e])
        if end > b and (b, end, int(e)) not in picks:
            picks.append((b, end, int(e)))
    return picks


def test_fourth_benchmark_configuration_full_size(cuda):
    """Gate/up pair Q5_K 512 x 2048 and down Q6_K 2048 x 512 over 256 experts, top-8 routing of
    16384 tokens (131072 routed rows), forward + dX.  The fp32 oracle over everything would take
    minutes, so: sampled groups against the oracle (norm over the group and worst row), and every
    group against the dense operator on that expert alone, bit for bit (the dense calls use
    256-token tiles, the grouped ones 512-token tiles: the tiling must not change a bit)."""
    import torch_ggml_ops_b200 as tgo

    E, tokens, top_k = 256, 16384, 8
    ids = blocks.topk_routing(tokens, E, top_k, seed=4)
    _, ei, eo = blocks.sort_by_expert(ids, E)
    R = tokens * top_k
    wg = blocks.expert_weights(ref.Q5_K, E, 512, 2048, 1)
    wu = blocks.expert_weights(ref.Q5_K, E, 512, 2048, 2)
    wdn = blocks.expert_weights(ref.Q6_K, E, 2048, 512, 3)
    gen = torch.Generator(device="cuda").manual_seed(7)
    rnd = lambda cols: torch.randn((R, cols), generator=gen, device="cuda", dtype=torch.float32).to(torch.bfloat16)  # noqa: E731
    xd, hd = rnd(2048).requires_grad_(True), rnd(512).requires_grad_(True)
    d0, d1, dd = rnd(512), rnd(512), rnd(2048)
    wgd, wud, wdnd = to_dev(wg), to_dev(wu), to_dev(wdn)
    eid, eod = to_dev(ei), to_dev(eo)
    y0, y1 = tgo.grouped_mmq_pair(xd, wgd, wud, eid, eod, ref.Q5_K, 512)
    torch.autograd.backward([y0, y1], [d0, d1])
    yd = tgo.grouped_mmq(hd, wdnd, eid, eod, ref.Q6_K, 2048)
    yd.backward(dd)
    for t in (y0, y1, xd.grad, yd, hd.grad):
        assert not torch.isnan(t).any()
    for b, end, e in _sampled_groups(np.asarray(eo)):
        Wg = ref.weight_fp32(wg[e].reshape(-1), ref.Q5_K, 512, 2048)
        Wu = ref.weight_fp32(wu[e].reshape(-1), ref.Q5_K, 512, 2048)
        Wd = ref.weight_fp32(wdn[e].reshape(-1), ref.Q6_K, 2048, 512)
        xs, hs = xd[b:end].detach().cpu(), hd[b:end].detach().cpu()
        checks = [
            (y0[b:end], ref.mmq_forward(xs, Wg), FWD_TOL), (y1[b:end], ref.mmq_forward(xs, Wu), FWD_TOL),
            (xd.grad[b:end], ref.mmq_grad_input(d0[b:end].cpu(), Wg) + ref.mmq_grad_input(d1[b:end].cpu(), Wu), DX_TOL),
            (yd[b:end], ref.mmq_forward(hs, Wd), FWD_TOL), (hd.grad[b:end], ref.mmq_grad_input(dd[b:end].cpu(), Wd), DX_TOL)]
        for got, want, tol in checks:
            got = got.detach().float().cpu()
            assert ref.rel_frobenius(got, want) < tol
            assert ref.max_row_error(got, want) < 1e-2
    # every group == the dense operator on that expert alone, bit for bit
    starts = np.concatenate([[0], np.asarray(eo)[:-1]])
    for e in range(E):
        b, end = int(starts[e]), int(eo[e])
        if end == b:
            continue
        fg, fd = wgd[e].reshape(-1).clone(), wdnd[e].reshape(-1).clone()
        assert np.array_equal(bits(y0[b:end]), bits(tgo.mmq(xd[b:end].detach().clone(), fg, ref.Q5_K, 512))), e
        assert np.array_equal(bits(yd[b:end]), bits(tgo.mmq(hd[b:end].detach().clone(), fd, ref.Q6_K, 2048))), e
        assert np.array_equal(bits(hd.grad[b:end]),
                              bits(torch.ops.torch_ggml_ops.mmq_grad_input(dd[b:end].clone(), fd, ref.Q6_K, 512))), e


def test_third_benchmark_configuration_both_tile_widths(cuda, monkeypatch):
    """The benchmark workload with 256-token tiles and with 512-token tiles: every CTA pair walks
    through about ten tiles, narrow and wide ones mixed, and not a bit may differ."""
    from torch_ggml_ops_b200 import native

    qt, E, N, K, tokens, top_k = ref.Q4_K, 256, 512, 2048, 8192, 8
    ids = blocks.topk_routing(tokens, E, top_k, seed=3)
    _, ei, eo = blocks.sort_by_expert(ids, E)
    R = tokens * top_k
    wd = to_dev(blocks.expert_weights(qt, E, N, K, 5))
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn((R, K), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    dy = torch.randn((R, N), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    eid, eod = to_dev(ei), to_dev(eo)
    ws = torch.empty(native.grouped_workspace_bytes(R, E), dtype=torch.uint8, device="cuda")
    outs = []
    for mode in ("0", "1"):
        monkeypatch.setenv("TGO_WIDE_TILES", mode)
        y = torch.full((R, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        dx = torch.full((R, K), float("nan"), dtype=torch.bfloat16, device="cuda")
        for _ in range(3):   # back to back: the next launch's first tiles meet the previous launch's tail
            native.grouped_fwd(x, wd, None, y, None, eid, eod, E, R, N, K, qt, ws)
            native.grouped_dx(dy, None, wd, None, dx, eid, eod, E, R, N, K, qt, ws)
        torch.cuda.synchronize()
        outs.append((y, dx))
    monkeypatch.delenv("TGO_WIDE_TILES")
    assert np.array_equal(bits(outs[0][0]), bits(outs[1][0])) and np.array_equal(bits(outs[0][1]), bits(outs[1][1]))
    assert not torch.isnan(outs[1][0]).any() and not torch.isnan(outs[1][1]).any()
    assert native.device_status() == 0


def test_pair_backward_with_one_cotangent_uses_that_projection(cuda):
    import torch_ggml_ops_b200 as tgo

    qt, E, N, K = ref.Q4_K, 3, 64, 256
    sizes, ids = [20, 30], [2, 0]
    w0, W0 = expert_case(qt, E, N, K, 1)
    w1, W1 = expert_case(qt, E, N, K, 2)
    ei, eo = routing_from_sizes(sizes, ids)
    x = blocks.gaussian_bf16((50, K), 3)
    dy = blocks.gaussian_bf16((50, N), 4)
    xd = to_dev(x).requires_grad_(True)
    y0, y1 = tgo.grouped_mmq_pair(xd, to_dev(w0), to_dev(w1), to_dev(ei), to_dev(eo), qt, N)
    y1.backward(to_dev(dy))
    assert ref.rel_frobenius(xd.grad.float().cpu(), ref.grouped_grad_input(dy, W1, ids, eo)) < DX_TOL


def test_grouped_opcheck_compile_and_errors(cuda):
    import torch_ggml_ops_b200 as tgo

    qt, E, N, K = ref.Q4_K, 3, 64, 256
    sizes, ids = [20, 30], [2, 0]
    w0 = to_dev(expert_case(qt, E, N, K, 1)[0])
    ei, eo = (to_dev(t) for t in routing_from_sizes(sizes, ids))
    x = to_dev(blocks.gaussian_bf16((50, K), 3))
    torch.library.opcheck(torch.ops.torch_ggml_ops.grouped_mmq.default,
                          (x.clone().requires_grad_(True), w0, ei, eo, qt, N),
                          test_utils=("test_schema", "test_autograd_registration", "test_faketensor"))
    torch.library.opcheck(torch.ops.torch_ggml_ops.grouped_mmq_pair.default,
                          (x.clone().requires_grad_(True), w0, w0, ei, eo, qt, N),
                          test_utils=("test_schema", "test_autograd_registration", "test_faketensor"))
    eager = tgo.grouped_mmq(x, w0, ei, eo, qt, N)
    compiled = torch.compile(lambda a: tgo.grouped_mmq(a, w0, ei, eo, qt, N), fullgraph=True, backend="aot_eager")
    assert np.array_equal(bits(compiled(x)), bits(eager))
    with pytest.raises(RuntimeError, match="torch.int32"):
        tgo.grouped_mmq(x, w0, ei, eo.long(), qt, N)
    with pytest.raises(RuntimeError, match="bytes per row"):
        tgo.grouped_mmq(x, w0[:, :, :-16].contiguous(), ei, eo, qt, N)
    with pytest.raises(RuntimeError, match="contiguous"):
        tgo.grouped_mmq(to_dev(blocks.gaussian_bf16((K, 50), 3)).t(), w0, ei, eo, qt, N)
    with pytest.raises(RuntimeError, match="zero-row"):
        tgo.grouped_mmq(x[:0], w0, ei, eo, qt, N)
    with pytest.raises(RuntimeError, match="unsupported quant_type"):
        tgo.grouped_mmq(x, w0, ei, eo, 1, N)
    dxg = torch.ops.torch_ggml_ops.grouped_mmq_grad_input(
        to_dev(blocks.gaussian_bf16((50, N), 1)).requires_grad_(True), w0, ei, eo, qt, K)
    with pytest.raises(RuntimeError, match="does not support higher-order"):
        dxg.sum().backward()
