"""GPU test of tgo_grouped_fwd_noalloc, the grouped forward for callers that cannot allocate
device memory (a runtime that owns all of it, a serving loop where cudaMalloc would stall every
stream, a bare FFI binding with no allocator): its tile list lives in a fixed array inside the
library.  The results must be identical to tgo_grouped_fwd with a caller workspace, call after
call, although the array still holds the previous call's tile list.

Collected last on purpose (file name), so a failure here cannot hide one elsewhere."""
import numpy as np
import pytest
import torch

from oracle import blocks, ref
from helpers import FWD_TOL, bits, expert_case, routing_from_sizes, to_dev

pytestmark = pytest.mark.gpu


def _both_ways(native, qt, E, N, K, sizes, ids, seed, pair):
    w0, W0 = expert_case(qt, E, N, K, seed)
    w1 = expert_case(qt, E, N, K, seed + 1)[0] if pair else None
    R = int(sum(sizes))
    ei, eo = routing_from_sizes(sizes, ids)
    x = blocks.gaussian_bf16((R, K), seed + 2)
    dev = [to_dev(t) for t in (x, w0, w1, ei, eo)]
    outs = []
    for use_builtin_scratch in (False, True):
        y0 = torch.full((R, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        y1 = torch.full((R, N), float("nan"), dtype=torch.bfloat16, device="cuda") if pair else None
        if use_builtin_scratch:
            native.grouped_fwd_noalloc(dev[0], dev[1], dev[2], y0, y1, dev[3], dev[4], E, R, N, K, qt)
        else:
            ws = torch.empty(native.grouped_workspace_bytes(R, len(sizes)), dtype=torch.uint8, device="cuda")
            native.grouped_fwd(dev[0], dev[1], dev[2], y0, y1, dev[3], dev[4], E, R, N, K, qt, ws)
        torch.cuda.synchronize()
        outs.append((y0, y1))
    (a0, a1), (b0, b1) = outs
    assert np.array_equal(bits(a0), bits(b0))
    if pair:
        assert np.array_equal(bits(a1), bits(b1))
    assert not torch.isnan(b0).any()
    assert ref.rel_frobenius(b0.float().cpu(), ref.grouped_forward(x, W0, ids, eo)) < FWD_TOL


def test_two_calls_in_a_row_match_the_workspace_entry_point(cuda):
    from torch_ggml_ops_b200 import native

    # first call: many small groups (a long tile list); second call: fewer, larger groups and a
    # different type, so stale entries of the first list sit behind the second one
    _both_ways(native, ref.Q4_K, 16, 512, 2048, [3, 70, 129, 256, 257, 1, 40, 600, 31, 5], list(range(15, 5, -1)), 1, False)
    _both_ways(native, ref.Q6_K, 6, 128, 512, [300, 17, 258], [4, 0, 5], 7, True)
    assert native.device_status() == 0


def test_sizes_beyond_the_built_in_scratch_are_rejected(cuda):
    from torch_ggml_ops_b200 import native

    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    rows = (native.NOALLOC_MAX_TILES + 1) * 256
    with pytest.raises(RuntimeError, match="exceeds the built-in limit"):
        native.check(native.lib().tgo_grouped_fwd_noalloc(
            buf.data_ptr(), buf.data_ptr(), None, buf.data_ptr(), None, buf.data_ptr(), buf.data_ptr(),
            1, 1, rows, 8, 256, 12, None), "tgo_grouped_fwd_noalloc")


def test_the_limit_itself_is_accepted(cuda):
    """rows / 256 + groups == TGO_NOALLOC_MAX_TILES exactly: 4000 one-row-tile experts (N = 8,
    K = 256) and 24576 rows; same bits as the workspace entry point."""
    from torch_ggml_ops_b200 import native

    qt, E, N, K, R = ref.Q4_K, 4000, 8, 256, 24576
    assert R // 256 + E == native.NOALLOC_MAX_TILES
    rng = np.random.default_rng(5)
    sizes = rng.multinomial(R, np.full(E, 1.0 / E)).astype(np.int64)
    ei, eo = routing_from_sizes(sizes, range(E))
    w = to_dev(blocks.expert_weights(qt, E, N, K, 11))
    x = to_dev(blocks.gaussian_bf16((R, K), 12))
    eid, eod = to_dev(ei), to_dev(eo)
    y_a = torch.full((R, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    y_b = torch.full((R, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(native.grouped_workspace_bytes(R, E), dtype=torch.uint8, device="cuda")
    native.grouped_fwd(x, w, None, y_a, None, eid, eod, E, R, N, K, qt, ws)
    native.grouped_fwd_noalloc(x, w, None, y_b, None, eid, eod, E, R, N, K, qt)
    torch.cuda.synchronize()
    assert np.array_equal(bits(y_a), bits(y_b)) and not torch.isnan(y_b).any()
    with pytest.raises(RuntimeError, match="exceeds the built-in limit"):
        native.grouped_fwd_noalloc(x, w, None, y_b, None, eid, eod, E, R + 256, N, K, qt)
