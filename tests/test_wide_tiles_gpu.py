"""Wide tiles: a token tile of more than 256 (up to 512) rows uses both accumulators of the GEMM
kernel at once and shares every decoded weight step between them.  The tiling must not change a
single bit of any result (the reduction order of an output element never depends on it), so every
case here runs with 256-token tiles and with 512-token tiles (TGO_WIDE_TILES, read at every call)
and compares bit patterns, besides the oracle check.  Reference properties mirrored:
tests/test_grouped_mmq.py:233-280 (grouped == dense), 385-431 (group-size boundaries)."""
import numpy as np
import pytest
import torch

from oracle import blocks, ref
from helpers import ALL_TYPES, DX_TOL, FWD_TOL, bits, dense_case, expert_case, routing_from_sizes, to_dev

pytestmark = pytest.mark.gpu


def _both_modes(monkeypatch, fn):
    out = []
    for mode in ("0", "1"):
        monkeypatch.setenv("TGO_WIDE_TILES", mode)
        out.append(fn())
    monkeypatch.delenv("TGO_WIDE_TILES")
    return out


@pytest.mark.parametrize("name,qt", ALL_TYPES)
@pytest.mark.parametrize("M", [257, 300, 511, 512, 513, 1100])
def test_dense_wide_equals_narrow_bit_for_bit(cuda, monkeypatch, name, qt, M):
    from torch_ggml_ops_b200 import native

    N, K = 384, 512
    w, W, _ = dense_case(qt, N, K, 40 + qt)
    x, dy = blocks.gaussian_bf16((M, K), M), blocks.gaussian_bf16((M, N), M + 1)
    xd, dyd, wd = to_dev(x), to_dev(dy), to_dev(w)

    def run():
        y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        dx = torch.full((M, K), float("nan"), dtype=torch.bfloat16, device="cuda")
        native.mmq_fwd(xd, wd, y, M, N, K, qt)
        native.mmq_dx(dyd, wd, dx, M, N, K, qt)
        torch.cuda.synchronize()
        return y, dx

    (y_n, dx_n), (y_w, dx_w) = _both_modes(monkeypatch, run)
    assert np.array_equal(bits(y_n), bits(y_w)) and np.array_equal(bits(dx_n), bits(dx_w))
    assert ref.rel_frobenius(y_w.float().cpu(), ref.mmq_forward(x, W)) < FWD_TOL
    assert ref.rel_frobenius(dx_w.float().cpu(), ref.mmq_grad_input(dy, W)) < DX_TOL
    assert ref.max_row_error(y_w.float().cpu(), ref.mmq_forward(x, W)) < 2 * FWD_TOL
    assert native.device_status() == 0


@pytest.mark.parametrize("name,qt", ALL_TYPES)
@pytest.mark.parametrize("pair", [False, True])
def test_grouped_wide_equals_narrow_bit_for_bit(cuda, monkeypatch, name, qt, pair):
    from torch_ggml_ops_b200 import native

    E, N, K = 9, 320, 768
    sizes = [1, 255, 256, 257, 1000, 16, 512, 511, 300]
    ids = [8, 7, 6, 5, 4, 3, 2, 1, 0]
    w0, W0 = expert_case(qt, E, N, K, 3)
    w1, W1 = expert_case(qt, E, N, K, 4)
    ei, eo = routing_from_sizes(sizes, ids)
    R = sum(sizes)
    x = blocks.gaussian_bf16((R, K), 5)
    dy0, dy1 = blocks.gaussian_bf16((R, N), 6), blocks.gaussian_bf16((R, N), 7)
    d = {k: to_dev(v) for k, v in dict(x=x, dy0=dy0, dy1=dy1, w0=w0, w1=w1, ei=ei, eo=eo).items()}
    ws = torch.empty(native.grouped_workspace_bytes(R, len(ids)), dtype=torch.uint8, device="cuda")

    def run():
        y0 = torch.full((R, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        y1 = torch.full((R, N), float("nan"), dtype=torch.bfloat16, device="cuda") if pair else None
        dx = torch.full((R, K), float("nan"), dtype=torch.bfloat16, device="cuda")
        native.grouped_fwd(d["x"], d["w0"], d["w1"] if pair else None, y0, y1, d["ei"], d["eo"], E, R, N, K, qt, ws)
        native.grouped_dx(d["dy0"], d["dy1"] if pair else None, d["w0"], d["w1"] if pair else None, dx,
                          d["ei"], d["eo"], E, R, N, K, qt, ws)
        torch.cuda.synchronize()
        return y0, y1, dx

    narrow, wide = _both_modes(monkeypatch, run)
    for a, b in zip(narrow, wide):
        assert (a is None and b is None) or np.array_equal(bits(a), bits(b))
    y0, y1, dx = wide
    assert ref.rel_frobenius(y0.float().cpu(), ref.grouped_forward(x, W0, ids, eo)) < FWD_TOL
    if pair:
        assert ref.rel_frobenius(y1.float().cpu(), ref.grouped_forward(x, W1, ids, eo)) < FWD_TOL
    want_dx = ref.grouped_grad_input(dy0, W0, ids, eo, second=(dy1, W1) if pair else None)
    assert ref.rel_frobenius(dx.float().cpu(), want_dx) < DX_TOL
    assert ref.max_row_error(dx.float().cpu(), want_dx) < 2 * DX_TOL
    assert native.device_status() == 0


@pytest.mark.parametrize("max_tok", [256, 512])
def test_tile_list_builder_both_tile_sizes(cuda, max_tok):
    from torch_ggml_ops_b200 import native

    sizes = [1, 255, 256, 257, 1000, 0, 16, 512, 513, 2049]
    ids = list(range(len(sizes) - 1, -1, -1))
    ei, eo = routing_from_sizes(sizes, ids)
    R = sum(sizes)
    ws = torch.zeros(native.grouped_workspace_bytes(R, len(ids)), dtype=torch.uint8, device="cuda")
    native.build_tiles(to_dev(ei), to_dev(eo), len(sizes), R, ws, max_tile_tokens=max_tok)
    torch.cuda.synchronize()
    count = int(ws[:4].view(torch.int32).item())
    tasks = ws[16:16 + 16 * count].view(torch.int32).reshape(count, 4).cpu().numpy()
    covered = np.zeros(R, dtype=np.int32)
    ends = np.cumsum(sizes)
    for e, r0, n, g in tasks:
        assert 0 < n <= max_tok and e == ids[g]
        assert ends[g] - sizes[g] <= r0 and r0 + n <= ends[g]
        covered[r0:r0 + n] += 1
    assert (covered == 1).all()
    assert count == sum((s + max_tok - 1) // max_tok for s in sizes)


def test_short_reductions_and_wide_tiles(cuda, monkeypatch):
    """Backward tiles with one or two 64-element steps (N <= 128) make decoded-weight slots wrap
    across several tiles, wide and narrow mixed: the hardest case for the slot bookkeeping."""
    from torch_ggml_ops_b200 import native

    qt, E, K = ref.Q4_K, 6, 512
    for N in (8, 64, 68, 72, 128, 200):   # 68: rows of 136 bytes take the plain-load activation producer
        sizes, ids = [300, 20, 512, 257, 40, 700], [0, 1, 2, 3, 4, 5]
        w, W = expert_case(qt, E, N, K, N)
        ei, eo = routing_from_sizes(sizes, ids)
        R = sum(sizes)
        dy = blocks.gaussian_bf16((R, N), 9)
        ws = torch.empty(native.grouped_workspace_bytes(R, E), dtype=torch.uint8, device="cuda")
        dyd, wd, eid, eod = to_dev(dy), to_dev(w), to_dev(ei), to_dev(eo)

        def run():
            dx = torch.full((R, K), float("nan"), dtype=torch.bfloat16, device="cuda")
            native.grouped_dx(dyd, None, wd, None, dx, eid, eod, E, R, N, K, qt, ws)
            torch.cuda.synchronize()
            return dx

        narrow, wide = _both_modes(monkeypatch, run)
        assert np.array_equal(bits(narrow), bits(wide)), N
        assert ref.rel_frobenius(wide.float().cpu(), ref.grouped_grad_input(dy, W, ids, eo)) < DX_TOL
    assert native.device_status() == 0
