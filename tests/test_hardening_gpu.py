"""GPU tests of the edges around the operators: the reference's remaining test properties
(opcheck with dynamic-shape AOT dispatch, torch.compile with the default backend:
tests/test_mmq.py:140-173, tests/test_grouped_mmq.py:453-470, 581-639), tensors loaded from a GGUF
file fed straight to the operators (bench/mmq_benchmark_common.py:196-200 does the same), and the
time-out path of the kernels' bounded waits."""
import numpy as np
import pytest
import torch

from oracle import blocks, ref
from helpers import DX_TOL, FWD_TOL, bits, dense_case, expert_case, routing_from_sizes, to_dev

pytestmark = pytest.mark.gpu

OPCHECK_UTILS = ("test_schema", "test_autograd_registration", "test_faketensor", "test_aot_dispatch_dynamic")


def test_opcheck_with_dynamic_aot_dispatch(cuda):
    qt, E, N, K = ref.Q4_K, 3, 64, 256
    w = to_dev(blocks.dense_weight(qt, N, K, 3))
    we = to_dev(expert_case(qt, E, N, K, 1)[0])
    ei, eo = (to_dev(t) for t in routing_from_sizes([20, 30], [2, 0]))
    x = to_dev(blocks.gaussian_bf16((50, K), 3))
    dy = to_dev(blocks.gaussian_bf16((50, N), 4))
    ops = torch.ops.torch_ggml_ops
    torch.library.opcheck(ops.mmq.default, (x.clone().requires_grad_(True), w, qt, N), test_utils=OPCHECK_UTILS)
    torch.library.opcheck(ops.mmq_grad_input.default, (dy, w, qt, K),
                          test_utils=("test_schema", "test_faketensor", "test_aot_dispatch_dynamic"))
    torch.library.opcheck(ops.grouped_mmq.default, (x.clone().requires_grad_(True), we, ei, eo, qt, N),
                          test_utils=OPCHECK_UTILS)
    torch.library.opcheck(ops.grouped_mmq_pair.default, (x.clone().requires_grad_(True), we, we, ei, eo, qt, N),
                          test_utils=OPCHECK_UTILS)
    torch.library.opcheck(ops.grouped_mmq_grad_input.default, (dy, we, ei, eo, qt, K),
                          test_utils=("test_schema", "test_faketensor", "test_aot_dispatch_dynamic"))
    torch.library.opcheck(ops.grouped_mmq_pair_grad_input.default, (dy, dy, we, we, ei, eo, qt, K),
                          test_utils=("test_schema", "test_faketensor", "test_aot_dispatch_dynamic"))


def test_compile_with_the_default_backend(cuda):
    """fullgraph=True through the default (inductor) backend, forward and backward, dense and
    grouped pair; the compiled graph must call the same kernels, so results are bit-identical."""
    import torch_ggml_ops_b200 as tgo

    qt, E, N, K = ref.Q5_K, 3, 128, 512
    w = to_dev(blocks.dense_weight(qt, N, K, 3))
    we0, we1 = to_dev(expert_case(qt, E, N, K, 1)[0]), to_dev(expert_case(qt, E, N, K, 2)[0])
    ei, eo = (to_dev(t) for t in routing_from_sizes([40, 70], [2, 0]))
    x = to_dev(blocks.gaussian_bf16((110, K), 3))
    g = to_dev(blocks.gaussian_bf16((110, N), 4))

    def dense(a):
        return tgo.mmq(a, w, qt, N)

    def pair(a):
        y0, y1 = tgo.grouped_mmq_pair(a, we0, we1, ei, eo, qt, N)
        return y0 + y1

    for fn in (dense, pair):
        xe = x.clone().requires_grad_(True)
        ye = fn(xe)
        ye.backward(g)
        xc = x.clone().requires_grad_(True)
        try:
            yc = torch.compile(fn, fullgraph=True)(xc)
            yc.backward(g)
        except Exception as exc:  # the backend needs a working host compiler / Triton on the box
            if "torch_ggml_ops" in str(exc):
                raise
            pytest.skip(f"default torch.compile backend unavailable here: {type(exc).__name__}")
        assert np.array_equal(bits(yc), bits(ye)) and np.array_equal(bits(xc.grad), bits(xe.grad))


def test_tensors_loaded_from_a_gguf_file_feed_the_operators(cuda, tmp_path):
    gguf = pytest.importorskip("gguf")
    import torch_ggml_ops_b200 as tgo
    from torch_ggml_ops_b200 import gguf_loader

    path = tmp_path / "ops.gguf"
    wr = gguf.GGUFWriter(str(path), "llama")
    N, K, E = 96, 512, 5
    dense = {}
    for name, qt in ref.QTYPES.items():
        raw = blocks.dense_weight(qt, N, K, seed=30 + qt).reshape(N, -1)
        dense[name] = (qt, raw)
        wr.add_tensor(f"blk.0.attn_{name}.weight", raw, raw_dtype=gguf.GGMLQuantizationType(qt))
    experts = blocks.expert_weights(ref.Q6_K, E, N, K, seed=9)
    wr.add_tensor("blk.0.ffn_down_exps.weight", experts, raw_dtype=gguf.GGMLQuantizationType.Q6_K)
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()

    loaded = gguf_loader.load_packed(path, device="cuda")
    x = blocks.gaussian_bf16((77, K), 1)
    dy = blocks.gaussian_bf16((77, N), 2)
    for name, (qt, raw) in dense.items():
        p = loaded[f"blk.0.attn_{name}.weight"]
        assert p.data.is_cuda and (p.quant_type, p.out_features, p.in_features) == (qt, N, K)
        W = ref.weight_fp32(raw.reshape(-1), qt, N, K)
        xd = to_dev(x).requires_grad_(True)
        y = tgo.mmq(xd, p.data.reshape(-1), p.quant_type, p.out_features)
        y.backward(to_dev(dy))
        assert ref.rel_frobenius(y.detach().float().cpu(), ref.mmq_forward(x, W)) < FWD_TOL
        assert ref.rel_frobenius(xd.grad.float().cpu(), ref.mmq_grad_input(dy, W)) < DX_TOL
    p = loaded["blk.0.ffn_down_exps.weight"]
    assert (p.experts, p.out_features, p.in_features) == (E, N, K)
    sizes, ids = [30, 0, 47], [4, 1, 2]
    ei, eo = routing_from_sizes(sizes, ids)
    We = ref.expert_weights_fp32(experts, ref.Q6_K, N, K)
    xd = to_dev(x).requires_grad_(True)
    y = tgo.grouped_mmq(xd, p.data, to_dev(ei), to_dev(eo), p.quant_type, p.out_features)
    y.backward(to_dev(dy))
    assert ref.rel_frobenius(y.detach().float().cpu(), ref.grouped_forward(x, We, ids, eo)) < FWD_TOL
    assert ref.rel_frobenius(xd.grad.float().cpu(), ref.grouped_grad_input(dy, We, ids, eo)) < DX_TOL


def test_a_wait_that_runs_out_is_reported_and_the_context_survives(cuda, monkeypatch):
    """A kernel whose only wait can never be satisfied gives up after its (short) limit, records
    its code in the status word and returns; the next operator call works.  With TGO_CHECK_STATUS
    set, the matmul entry points turn a set status word into an error of the call."""
    import torch_ggml_ops_b200 as tgo
    from torch_ggml_ops_b200 import native

    qt, N, K = ref.Q4_K, 32, 256
    w, W, _ = dense_case(qt, N, K, 3)
    x = blocks.gaussian_bf16((8, K), 1)
    assert native.device_status() == 0
    native.selftest_wait_timeout(2_000_000)          # about a millisecond
    torch.cuda.synchronize()
    assert native.device_status() & 0xFF == 10       # the self-test's wait code; reading clears the word
    assert native.device_status() == 0
    y = tgo.mmq(to_dev(x), to_dev(w), qt, N)
    assert ref.rel_frobenius(y.float().cpu(), ref.mmq_forward(x, W)) < FWD_TOL
    # the debug option: the first matmul call after a recorded time-out fails, the one after it works
    native.selftest_wait_timeout(2_000_000)
    monkeypatch.setenv("TGO_CHECK_STATUS", "1")
    with pytest.raises(RuntimeError, match="gave up a bounded wait"):
        tgo.mmq(to_dev(x), to_dev(w), qt, N)
    y = tgo.mmq(to_dev(x), to_dev(w), qt, N)
    monkeypatch.delenv("TGO_CHECK_STATUS")
    assert ref.rel_frobenius(y.float().cpu(), ref.mmq_forward(x, W)) < FWD_TOL
    with pytest.raises(RuntimeError, match="limit_cycles"):
        native.selftest_wait_timeout(10)
