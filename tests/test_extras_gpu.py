"""GPU tests of the operators either side of the reference's surface (``extras.py``): the dense
multi-projection call, silu(gate) * up, the single-GPU MoE feed-forward block and the chunked
LM-head loss loop (reference context: docs/mmq_fwd_optimization.md:299-307,
docs/mmq_bwd_optimization.md:502-524, README.md:3)."""
import numpy as np
import pytest
import torch

from oracle import blocks, ref
from helpers import ALL_TYPES, DX_TOL, FWD_TOL, bits, dense_case, expert_case, routing_from_sizes, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,qt", ALL_TYPES)
@pytest.mark.parametrize("count", [1, 2, 3, 4])
def test_multi_projection_equals_separate_calls_bit_for_bit(cuda, name, qt, count):
    import torch_ggml_ops_b200 as tgo

    M, N, K = 333, 200, 512
    cases = [dense_case(qt, N, K, 60 + i) for i in range(count)]
    ws = [to_dev(c[0]) for c in cases]
    x = blocks.gaussian_bf16((M, K), 1)
    xd = to_dev(x).requires_grad_(True)
    ys = tgo.mmq_multi(xd, ws, qt, N)
    assert len(ys) == count
    for y, w in zip(ys, ws):
        assert np.array_equal(bits(y), bits(tgo.mmq(xd.detach(), w, qt, N)))
    dys = [blocks.gaussian_bf16((M, N), 10 + i) for i in range(count)]
    torch.autograd.backward(list(ys), [to_dev(d) for d in dys])
    want = sum(ref.mmq_grad_input(d, c[1]) for d, c in zip(dys, cases))
    assert ref.rel_frobenius(xd.grad.float().cpu(), want) < 2 * DX_TOL   # the per-weight gradients are summed in bf16


def test_multi_projection_checks_and_compile(cuda):
    import torch_ggml_ops_b200 as tgo

    qt, M, N, K = ref.Q4_K, 40, 64, 256
    ws = [to_dev(blocks.dense_weight(qt, N, K, s)) for s in (1, 2)]
    x = to_dev(blocks.gaussian_bf16((M, K), 3))
    eager = tgo.mmq_multi(x, ws, qt, N)
    compiled = torch.compile(lambda a: tgo.mmq_multi(a, ws, qt, N), fullgraph=True, backend="aot_eager")(x)
    for a, b in zip(eager, compiled):
        assert np.array_equal(bits(a), bits(b))
    torch.library.opcheck(torch.ops.torch_ggml_ops_b200.mmq_multi.default, (x.clone().requires_grad_(True), ws, qt, N),
                          test_utils=("test_schema", "test_autograd_registration", "test_faketensor"))
    with pytest.raises(RuntimeError, match="1 to 4"):
        tgo.mmq_multi(x, ws * 3, qt, N)
    with pytest.raises(RuntimeError, match="bytes"):
        tgo.mmq_multi(x, [ws[0][:-144].contiguous()], qt, N)
    with pytest.raises(RuntimeError, match="hidden copy"):
        tgo.mmq_multi(to_dev(blocks.gaussian_bf16((K, M), 3)).t(), ws, qt, N)


def test_swiglu_operator_and_its_gradient(cuda):
    import torch_ggml_ops_b200 as tgo

    g = to_dev(blocks.gaussian_bf16((3, 50, 72), 1)).requires_grad_(True)
    u = to_dev(blocks.gaussian_bf16((3, 50, 72), 2)).requires_grad_(True)
    d = to_dev(blocks.gaussian_bf16((3, 50, 72), 3))
    h = tgo.swiglu(g, u)
    h.backward(d)
    gf, uf = g.detach().float().requires_grad_(True), u.detach().float().requires_grad_(True)
    hf = torch.nn.functional.silu(gf) * uf
    hf.backward(d.float())
    assert ref.rel_frobenius(h.detach().float().cpu(), hf.detach().cpu()) < 3e-3
    assert ref.rel_frobenius(g.grad.float().cpu(), gf.grad.cpu()) < 3e-3
    assert ref.rel_frobenius(u.grad.float().cpu(), uf.grad.cpu()) < 3e-3


def test_single_gpu_moe_block(cuda):
    import torch_ggml_ops_b200 as tgo

    E, H, F = 6, 512, 256
    qt_gu, qt_d = ref.IQ2_S, ref.Q6_K
    sizes, ids = [70, 1, 300, 129], [5, 0, 2, 3]
    wg, Wg = expert_case(qt_gu, E, F, H, 1)
    wu, Wu = expert_case(qt_gu, E, F, H, 2)
    wd, Wd = expert_case(qt_d, E, H, F, 3)
    ei, eo = routing_from_sizes(sizes, ids)
    R = sum(sizes)
    x, dy = blocks.gaussian_bf16((R, H), 4), blocks.gaussian_bf16((R, H), 5)
    xd = to_dev(x).requires_grad_(True)
    y = tgo.moe_mlp(xd, to_dev(wg), to_dev(wu), to_dev(wd), to_dev(ei), to_dev(eo), qt_gu, qt_d, F)
    y.backward(to_dev(dy))
    xf = x.float().requires_grad_(True)
    want = torch.zeros(R, H)
    b = 0
    parts = []
    for e, n in zip(ids, sizes):
        xe = xf[b:b + n]
        ge, ue = xe @ torch.from_numpy(Wg[e]).t(), xe @ torch.from_numpy(Wu[e]).t()
        parts.append((torch.nn.functional.silu(ge) * ue) @ torch.from_numpy(Wd[e]).t())
        b += n
    want = torch.cat(parts)
    want.backward(dy.float())
    assert ref.rel_frobenius(y.detach().float().cpu(), want.detach()) < 1e-2
    assert ref.rel_frobenius(xd.grad.float().cpu(), xf.grad) < 1e-2


def test_chunked_lm_head_loss(cuda):
    """A vocabulary that is not a multiple of the 128-row weight tile, rows that do not fill the
    last chunk: loss and hidden-state gradient against the fp64 computation on the dequantised weight."""
    import torch_ggml_ops_b200 as tgo

    qt, V, K, T = ref.Q6_K, 1000, 512, 600
    w, W, _ = dense_case(qt, V, K, 8)
    # hidden states scaled so that the logits have a spread of about one (with a spread of 60 the
    # softmax is so peaked that the bf16 rounding of the logits alone moves the gradient by 3 %)
    hidden = (blocks.gaussian_bf16((T, K), 9).float() * 0.02).to(torch.bfloat16)
    targets = torch.from_numpy(np.random.default_rng(1).integers(0, V, size=T))
    loss, dh = tgo.lm_head_loss(to_dev(hidden), to_dev(w), qt, V, to_dev(targets), chunk_rows=256)
    hf = hidden.double().requires_grad_(True)
    logits = hf @ torch.from_numpy(W).double().t() * 1.0
    want = torch.nn.functional.cross_entropy(logits, targets, reduction="sum")
    want.backward()
    assert abs(float(loss) - float(want.detach())) / float(want.detach()) < 2e-3, (float(loss), float(want.detach()))
    assert ref.rel_frobenius(dh.float().cpu(), hf.grad.float()) < 1e-2
    # the chunk size changes the launches (and the order of torch's fp32 softmax sums), not the result
    loss64, dh64 = tgo.lm_head_loss(to_dev(hidden), to_dev(w), qt, V, to_dev(targets), chunk_rows=64)
    assert abs(float(loss64) - float(loss)) / float(want) < 1e-4
    assert ref.rel_frobenius(dh64.float().cpu(), dh.float().cpu()) < 1e-3


@pytest.mark.parametrize("name,qt", ALL_TYPES)
@pytest.mark.parametrize("M,N,K", [(100, 8192, 512), (256, 8200, 256), (37, 8201, 512)])
def test_split_reduction_of_the_dense_input_gradient(cuda, name, qt, M, N, K):
    """Few rows against very many out-features: the reduction is cut into ranges with fp32 partial
    sums (the LM-head shape).  Same result as the unsplit launch up to the summation order, within
    the input-gradient tolerance of the oracle, row by row; N = 8200 leaves the last range part
    empty, N = 8201 takes the plain-load activation path (rows of 16402 bytes)."""
    from torch_ggml_ops_b200 import native

    w, W, _ = dense_case(qt, N, K, 90 + qt)
    dy = blocks.gaussian_bf16((M, N), 4)
    dyd, wd = to_dev(dy), to_dev(w)
    plain = torch.full((M, K), float("nan"), dtype=torch.bfloat16, device="cuda")
    split = torch.full((M, K), float("nan"), dtype=torch.bfloat16, device="cuda")
    native.mmq_dx(dyd, wd, plain, M, N, K, qt)
    used = native.mmq_dx_split(dyd, wd, split, M, N, K, qt)
    torch.cuda.synchronize()
    assert used > 0 and used % (M * K * 4) == 0 and used // (M * K * 4) >= 2     # it did split
    want = ref.mmq_grad_input(dy, W)
    assert not torch.isnan(split).any()
    assert ref.rel_frobenius(split.float().cpu(), want) < DX_TOL
    assert ref.max_row_error(split.float().cpu(), want) < 2 * DX_TOL
    assert ref.rel_frobenius(split.float().cpu(), plain.float().cpu()) < 3e-3
    # the torch operator takes the same path on its own
    op = torch.ops.torch_ggml_ops.mmq_grad_input(dyd, wd, qt, K)
    assert np.array_equal(bits(op), bits(split))
    assert native.device_status() == 0
