"""GPU tests of the device-side routing helpers (stable sort by expert with prefix-sum offsets,
row gather, weighted top-k combine) and of the activation quantiser, against host restatements."""
import numpy as np
import pytest
import torch

from oracle import blocks, ref
from helpers import bits, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens,experts,top_k", [(1, 4, 2), (37, 8, 2), (300, 256, 8), (8192, 256, 8), (1000, 1000, 4)])
def test_route_sort_is_a_stable_sort_with_cumulative_offsets(cuda, tokens, experts, top_k):
    from torch_ggml_ops_b200 import native

    ids = blocks.topk_routing(tokens, experts, top_k, seed=tokens)
    perm, ei, eo = blocks.sort_by_expert(ids, experts)
    s2p, p2s, dei, deo = native.route_sort(to_dev(ids.reshape(-1).astype(np.int32)), experts)
    assert np.array_equal(s2p.cpu().numpy(), perm.astype(np.int32))
    assert np.array_equal(deo.cpu().numpy(), eo) and np.array_equal(dei.cpu().numpy(), ei)
    inv = np.empty_like(perm)
    inv[perm] = np.arange(perm.size)
    assert np.array_equal(p2s.cpu().numpy(), inv.astype(np.int32))


def test_out_of_range_expert_ids_are_dropped(cuda):
    from torch_ggml_ops_b200 import native

    ids = torch.tensor([3, -1, 0, 9, 3, 0], dtype=torch.int32, device="cuda")
    s2p, p2s, ei, eo = native.route_sort(ids, 4)
    assert eo.tolist() == [2, 2, 2, 4] and p2s.tolist() == [2, -1, 0, -1, 3, 1]
    assert s2p[:4].tolist() == [2, 5, 0, 4]


def test_gather_combine_and_grouped_op_end_to_end(cuda):
    """top-k ids -> device sort -> gather -> grouped_mmq -> weighted combine, against the oracle."""
    import torch_ggml_ops_b200 as tgo
    from torch_ggml_ops_b200 import native

    qt, E, N, K, tokens, top_k = ref.Q4_K, 16, 64, 256, 200, 4
    ids = blocks.topk_routing(tokens, E, top_k, seed=5)
    w = blocks.expert_weights(qt, E, N, K, 1)
    W = ref.expert_weights_fp32(w, qt, N, K)
    x = blocks.gaussian_bf16((tokens, K), 2)
    g = torch.Generator().manual_seed(3)
    gate = torch.rand(tokens, top_k, generator=g)
    s2p, p2s, ei, eo = native.route_sort(to_dev(ids.reshape(-1).astype(np.int32)), E)
    rows = native.gather_rows(to_dev(x), s2p, top_k)
    perm, _, offs = blocks.sort_by_expert(ids, E)
    assert np.array_equal(bits(rows), bits(x[torch.from_numpy(perm // top_k)]))
    y = tgo.grouped_mmq(rows, to_dev(w), ei, eo, qt, N)
    out = native.combine_rows(y, p2s, top_k, to_dev(gate))
    want = torch.zeros(tokens, N)
    xf = x.float()
    for t in range(tokens):
        for s in range(top_k):
            want[t] += gate[t, s] * (xf[t] @ torch.from_numpy(W[ids[t, s]]).t())
    assert ref.rel_frobenius(out.float().cpu(), want) < 1e-2
    # unweighted combine of the gathered rows themselves reproduces top_k * x
    back = native.combine_rows(rows, p2s, top_k)
    assert ref.rel_frobenius(back.float().cpu(), top_k * xf) < 4e-3


@pytest.mark.parametrize("rows,width", [(1, 32), (7, 256), (300, 2048)])
def test_activation_quantiser(cuda, rows, width):
    from torch_ggml_ops_b200 import native

    x = blocks.gaussian_bf16((rows, width), rows)
    x[0, :32] = 0  # an all-zero block: d = 0, q = 0
    q, d, s = native.quantize_q8(to_dev(x))
    wq, wd, ws = ref.quantize_q8(x)
    assert np.array_equal(q.cpu().numpy(), wq)
    assert np.array_equal(d.cpu().numpy(), wd)
    np.testing.assert_allclose(s.cpu().numpy(), ws, rtol=1e-5, atol=1e-5)
    # dequantised activations are within half a quantisation step
    deq = q.float().cpu().reshape(rows, -1, 32) * d.cpu()[:, :, None]
    assert float((deq - x.float().reshape(rows, -1, 32)).abs().max()) <= float(d.max()) * 0.5 + 1e-6
