"""GPU test of the expert-parallel wrapper on one rank (its CUDA fast paths: device routing sort,
gather and fused top-k combine kernels) against the CPU oracle; the multi-rank bookkeeping is
covered on CPU ranks in test_ep_cpu.py."""
import numpy as np
import pytest
import torch

from oracle import blocks, ref
from helpers import DX_TOL, FWD_TOL, to_dev

pytestmark = pytest.mark.gpu


def test_single_rank_moe_projection_forward_and_backward(cuda):
    import torch_ggml_ops_b200 as tgo
    from torch_ggml_ops_b200.expert_parallel import ExpertParallel

    qt, E, N, K, tokens, top_k = ref.Q4_K, 32, 128, 512, 300, 4
    ids = blocks.topk_routing(tokens, E, top_k, seed=9)
    w = blocks.expert_weights(qt, E, N, K, 1)
    W = torch.from_numpy(ref.expert_weights_fp32(w, qt, N, K))
    x = blocks.gaussian_bf16((tokens, K), 2)
    dy = blocks.gaussian_bf16((tokens * top_k, N), 3)   # cotangent per routed row, token-major
    ep = ExpertParallel(E)
    plan = ep.plan(to_dev(torch.from_numpy(ids)))
    assert plan.send_perm.dtype == torch.int32 and int(plan.expert_offsets[-1]) == tokens * top_k
    rows = ep.dispatch_tokens(plan, to_dev(x)).requires_grad_(True)
    out = tgo.grouped_mmq(rows, to_dev(w), plan.expert_indices, plan.expert_offsets, qt, N)
    y = ep.combine_rows(plan, out.detach())
    out.backward(ep.dispatch_rows(plan, to_dev(dy)))
    dx = ep.combine_tokens(plan, rows.grad)
    xf = x.float()
    flat = ids.reshape(-1)
    want_y = torch.stack([xf[i // top_k] @ W[flat[i]].t() for i in range(flat.size)])
    want_dx = torch.zeros(tokens, K)
    for i in range(flat.size):
        want_dx[i // top_k] += dy[i].float() @ W[flat[i]]
    assert ref.rel_frobenius(y.float().cpu(), want_y) < FWD_TOL
    assert ref.rel_frobenius(dx.float().cpu(), want_dx) < DX_TOL
