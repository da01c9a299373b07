"""The GEMM kernel exists in two forms: CTA pairs (cta_group::2 UMMAs over a cluster of two, the
default) and single CTAs (TGO_CTA_PAIR=0, also the fallback where a pair cannot be co-scheduled).
The choice is read once per process, so the single-CTA form is exercised in a child process; both
forms must give bit-identical results (the reduction order does not depend on the tiling), with
256-token tiles and with 512-token tiles (TGO_WIDE_TILES).
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parents[1]

CHILD = r"""
import hashlib, json, sys
import numpy as np, torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/tests")
from oracle import blocks, ref
from helpers import bits, dense_case, expert_case, routing_from_sizes, to_dev, FWD_TOL, DX_TOL
from torch_ggml_ops_b200 import native

out = {}
def digest(t):
    return hashlib.sha256(bits(t).tobytes()).hexdigest()

for qt, N, K, M in ((12, 384, 512, 300), (14, 200, 256, 77), (22, 256, 768, 513)):
    w, W, _ = dense_case(qt, N, K, 5 + qt)
    x = blocks.gaussian_bf16((M, K), 1); dy = blocks.gaussian_bf16((M, N), 2)
    xd, dyd, wd = to_dev(x), to_dev(dy), to_dev(w)
    y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda"); dx = torch.empty(M, K, dtype=torch.bfloat16, device="cuda")
    native.mmq_fwd(xd, wd, y, M, N, K, qt); native.mmq_dx(dyd, wd, dx, M, N, K, qt)
    torch.cuda.synchronize()
    ef = ref.rel_frobenius(y.float().cpu(), ref.mmq_forward(x, W))
    eb = ref.rel_frobenius(dx.float().cpu(), ref.mmq_grad_input(dy, W))
    assert ef <= FWD_TOL and eb <= DX_TOL, (qt, ef, eb)
    out[f"dense{qt}"] = [digest(y), digest(dx)]

for qt, E, N, K, sizes in ((12, 6, 512, 512, [5, 300, 0, 17, 256, 33]), (13, 4, 136, 256, [40, 1, 270, 9])):
    ids = [e for e, s in enumerate(sizes) if s > 0]; sz = [s for s in sizes if s > 0]
    w0, W0 = expert_case(qt, E, N, K, 31); w1, W1 = expert_case(qt, E, N, K, 32)
    R = sum(sz); ei, eo = routing_from_sizes(sz, ids)
    x = blocks.gaussian_bf16((R, K), 3); dy0 = blocks.gaussian_bf16((R, N), 4); dy1 = blocks.gaussian_bf16((R, N), 6)
    d = [to_dev(t) for t in (x, dy0, dy1, w0, w1, ei, eo)]
    y0 = torch.empty(R, N, dtype=torch.bfloat16, device="cuda"); y1 = torch.empty_like(y0)
    dx = torch.empty(R, K, dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(native.grouped_workspace_bytes(R, len(sz)), dtype=torch.uint8, device="cuda")
    native.grouped_fwd(d[0], d[3], d[4], y0, y1, d[5], d[6], E, R, N, K, qt, ws)
    native.grouped_dx(d[1], d[2], d[3], d[4], dx, d[5], d[6], E, R, N, K, qt, ws)
    torch.cuda.synchronize()
    want = ref.grouped_forward(x, W0, ei.tolist(), eo.tolist())
    assert ref.rel_frobenius(y0.float().cpu(), want) <= FWD_TOL
    out[f"grouped{qt}"] = [digest(y0), digest(y1), digest(dx)]
assert native.device_status() == 0
print("RESULT " + json.dumps(out))
"""


def _run(pair: str, wide: str) -> dict:
    env = dict(os.environ, TGO_CTA_PAIR=pair, TGO_WIDE_TILES=wide)
    p = subprocess.run([sys.executable, "-c", CHILD, str(ROOT)], env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-4000:]
    line = [l for l in p.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


def test_single_cta_and_pair_kernels_agree_bit_for_bit():
    """Also across tile widths: 256-token tiles and 512-token (two-accumulator) tiles."""
    runs = {(pair, wide): _run(pair, wide) for pair in ("0", "1") for wide in ("0", "1")}
    first = runs[("1", "0")]
    for key, got in runs.items():
        assert got.keys() == first.keys()
        for k in first:
            assert got[k] == first[k], (key, k)
