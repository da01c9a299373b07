"""GPU parity of the dense operators against the CPU oracle (fp32 dequantise + matmul).

Mirrors the properties the reference's dense tests assert (tests/test_mmq.py:50-223) on seeded
synthetic super-blocks: forward and input-gradient accuracy, one-hot cotangent returns the bf16
dequantised weight row exactly, zero input gives exact zeros on a non-default stream, opcheck and
torch.compile agree with eager, and the fail-fast error messages."""
import numpy as np
import pytest
import torch

from oracle import blocks, ref
from helpers import ALL_TYPES, DX_TOL, FWD_TOL, bits, dense_case, to_dev, values_equal

pytestmark = pytest.mark.gpu

SMALL_SHAPES = [(1, 8, 256), (16, 128, 256), (43 * 3, 37, 2048), (300, 384, 1024), (257, 130, 512)]


@pytest.mark.parametrize("name,qt", ALL_TYPES)
@pytest.mark.parametrize("M,N,K", SMALL_SHAPES)
def test_forward_and_grad_input_through_the_c_abi(cuda, name, qt, M, N, K):
    from torch_ggml_ops_b200 import native

    w, W, _ = dense_case(qt, N, K, 100 + qt)
    wd = to_dev(w)
    x = blocks.gaussian_bf16((M, K), 1)
    y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    native.mmq_fwd(to_dev(x), wd, y, M, N, K, qt)
    assert ref.rel_frobenius(y.float().cpu(), ref.mmq_forward(x, W)) < FWD_TOL
    dy = blocks.gaussian_bf16((M, N), 2)
    dx = torch.full((M, K), float("nan"), dtype=torch.bfloat16, device="cuda")
    native.mmq_dx(to_dev(dy), wd, dx, M, N, K, qt)
    assert ref.rel_frobenius(dx.float().cpu(), ref.mmq_grad_input(dy, W)) < DX_TOL
    assert not torch.isnan(y).any() and not torch.isnan(dx).any()
    assert native.device_status() == 0


@pytest.mark.parametrize("name,qt", ALL_TYPES)
@pytest.mark.parametrize("wide", ["0", "1"])
def test_identity_activations_return_the_dequantised_weights(cuda, monkeypatch, name, qt, wide):
    """x = I gives y[t, n] = W[n, t] and dy = I gives dx[t, k] = W[t, k], both exactly: every
    output is one product by 1.0 plus zeros.  This pins the decoders inside the matmul kernel
    (all groups, rows and chunks, both operand orientations, both tile widths) against the
    stand-alone dequantiser, which the oracle tests pin bit for bit."""
    from torch_ggml_ops_b200 import native

    monkeypatch.setenv("TGO_WIDE_TILES", wide)
    N, K = 384, 512
    w, _, _ = dense_case(qt, N, K, 300 + qt)
    wd = to_dev(w)
    Wb = native.dequantize_bf16(wd.reshape(-1), qt).reshape(N, K)
    eye_k = torch.eye(K, dtype=torch.bfloat16, device="cuda")
    y = torch.full((K, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    native.mmq_fwd(eye_k, wd, y, K, N, K, qt)
    assert values_equal(y, Wb.t())
    eye_n = torch.eye(N, dtype=torch.bfloat16, device="cuda")
    dx = torch.full((N, K), float("nan"), dtype=torch.bfloat16, device="cuda")
    native.mmq_dx(eye_n, wd, dx, N, N, K, qt)
    assert values_equal(dx, Wb)
    assert native.device_status() == 0


@pytest.mark.parametrize("name,qt", ALL_TYPES)
def test_golden_known_answers(cuda, golden, name, qt):
    import torch_ggml_ops_b200 as tgo

    w = to_dev(golden[f"{name}_mm_w"].reshape(-1))
    x = to_dev(torch.from_numpy(golden[f"{name}_mm_x"]).to(torch.bfloat16))
    dy = to_dev(torch.from_numpy(golden[f"{name}_mm_dy"]).to(torch.bfloat16))
    y = tgo.mmq(x, w, qt, 16)
    dx = torch.ops.torch_ggml_ops.mmq_grad_input(dy, w, qt, 256)
    assert ref.rel_frobenius(y.float().cpu(), torch.from_numpy(golden[f"{name}_mm_y"])) < FWD_TOL
    assert ref.rel_frobenius(dx.float().cpu(), torch.from_numpy(golden[f"{name}_mm_dx"])) < DX_TOL


@pytest.mark.parametrize("name,qt", ALL_TYPES)
@pytest.mark.parametrize("N,K", [(4096, 2048), (2048, 4096)])
def test_benchmark_shapes_full_size(cuda, name, qt, N, K):
    """The dense benchmark configuration at full size (M = 4096), forward + input gradient."""
    import torch_ggml_ops_b200 as tgo

    M = 4096
    w, W, _ = dense_case(qt, N, K, 7 + qt)
    x = blocks.gaussian_bf16((M, K), 11)
    dy = blocks.gaussian_bf16((M, N), 12)
    xd = to_dev(x).requires_grad_(True)
    y = tgo.mmq(xd, to_dev(w), qt, N)
    y.backward(to_dev(dy))
    assert ref.rel_frobenius(y.detach().float().cpu(), ref.mmq_forward(x, W)) < FWD_TOL
    assert ref.rel_frobenius(xd.grad.float().cpu(), ref.mmq_grad_input(dy, W)) < DX_TOL


def test_first_benchmark_configuration(cuda):
    """Q4_K N=2048 x K=2048 (16384 raw blocks), M=512: forward vs fp32 dequantise + matmul."""
    import torch_ggml_ops_b200 as tgo

    qt, M, N, K = ref.Q4_K, 512, 2048, 2048
    w, W, _ = dense_case(qt, N, K, 2024)
    assert w.size == 16384 * 144
    x = blocks.gaussian_bf16((M, K), 5)
    y = tgo.mmq(to_dev(x), to_dev(w), qt, N)
    assert y.shape == (M, N) and y.dtype == torch.bfloat16
    assert ref.rel_frobenius(y.float().cpu(), ref.mmq_forward(x, W)) < FWD_TOL


@pytest.mark.parametrize("name,qt", ALL_TYPES)
def test_one_hot_cotangent_returns_the_bf16_weight_row(cuda, name, qt):
    """dX of a one-hot dY is exactly the dequantised weight row rounded to bf16
    (reference: tests/test_mmq.py:77-92)."""
    N, K = 72, 768
    w, _, Wb = dense_case(qt, N, K, 50 + qt)
    rows = list(range(0, N, 5))
    dy = torch.zeros(len(rows), N, dtype=torch.bfloat16)
    for i, j in enumerate(rows):
        dy[i, j] = 1.0
    dx = torch.ops.torch_ggml_ops.mmq_grad_input(to_dev(dy), to_dev(w), qt, K)
    assert values_equal(dx, Wb[rows])


@pytest.mark.parametrize("name,qt", ALL_TYPES)
def test_grad_input_equals_bf16_matmul_on_a_short_reduction(cuda, name, qt):
    """With a reduction shorter than one UMMA step-chain the fp32 accumulation has no ordering
    freedom left beyond the hardware's, so the result stays within one bf16 ulp of torch.mm on the
    bf16-dequantised weight (reference asserts equality on its hardware: tests/test_mmq.py:95-118)."""
    N, K, M = 37, 512, 129
    w, _, Wb = dense_case(qt, N, K, 70 + qt)
    dy = blocks.gaussian_bf16((M, N), 3)
    dx = torch.ops.torch_ggml_ops.mmq_grad_input(to_dev(dy), to_dev(w), qt, K).float().cpu()
    want = (dy.double() @ Wb.double()).float()
    assert ref.rel_frobenius(dx, want) < 3e-3
    ulp = torch.abs(want) * 2.0 ** -7 + 1e-30
    assert bool((torch.abs(dx - want) <= ulp).all())


def test_zero_input_gives_exact_zeros_on_a_side_stream(cuda):
    import torch_ggml_ops_b200 as tgo

    qt, N, K = ref.Q5_K, 200, 512
    w = to_dev(blocks.dense_weight(qt, N, K, 1))
    x = torch.zeros(3, 5, K, dtype=torch.bfloat16, device="cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        y = tgo.mmq(x, w, qt, N)
    side.synchronize()
    assert y.shape == (3, 5, N) and int(torch.count_nonzero(y)) == 0


def test_results_are_deterministic(cuda):
    import torch_ggml_ops_b200 as tgo

    qt, M, N, K = ref.Q6_K, 777, 640, 1024
    w = to_dev(blocks.dense_weight(qt, N, K, 9))
    x = to_dev(blocks.gaussian_bf16((M, K), 9))
    a = tgo.mmq(x, w, qt, N)
    b = tgo.mmq(x, w, qt, N)
    assert np.array_equal(bits(a), bits(b))


def test_autograd_compile_and_opcheck(cuda):
    import torch_ggml_ops_b200 as tgo

    qt, N, K = ref.Q4_K, 64, 256
    w = to_dev(blocks.dense_weight(qt, N, K, 3))
    x = to_dev(blocks.gaussian_bf16((2, 9, K), 4)).requires_grad_(True)
    y = tgo.mmq(x, w, qt, N)
    g = to_dev(blocks.gaussian_bf16((2, 9, N), 5))
    y.backward(g)
    assert x.grad is not None and x.grad.shape == x.shape and w.grad is None
    torch.library.opcheck(torch.ops.torch_ggml_ops.mmq.default, (x.detach().requires_grad_(True), w, qt, N),
                          test_utils=("test_schema", "test_autograd_registration", "test_faketensor"))
    torch.library.opcheck(torch.ops.torch_ggml_ops.mmq_grad_input.default, (g, w, qt, K),
                          test_utils=("test_schema", "test_faketensor"))

    def f(a):
        return tgo.mmq(a, w, qt, N)

    compiled = torch.compile(f, fullgraph=True, backend="aot_eager")
    assert np.array_equal(bits(compiled(x.detach())), bits(y.detach()))


def test_higher_order_gradients_are_refused(cuda):
    qt, N, K = ref.Q4_K, 16, 256
    w = to_dev(blocks.dense_weight(qt, N, K, 3))
    dy = to_dev(blocks.gaussian_bf16((4, N), 1)).requires_grad_(True)
    dx = torch.ops.torch_ggml_ops.mmq_grad_input(dy, w, qt, K)
    with pytest.raises(RuntimeError, match="does not support higher-order"):
        dx.sum().backward()


def test_fail_fast_error_messages(cuda):
    import torch_ggml_ops_b200 as tgo

    qt, N, K = ref.Q4_K, 8, 256
    w = to_dev(blocks.dense_weight(qt, N, K, 3))
    x = to_dev(blocks.gaussian_bf16((4, K), 1))
    with pytest.raises(RuntimeError, match="contiguous"):
        tgo.mmq(to_dev(blocks.gaussian_bf16((K, 4), 1)).t(), w, qt, N)
    with pytest.raises(RuntimeError, match="zero storage offset"):
        tgo.mmq(to_dev(blocks.gaussian_bf16((5, K), 1))[1:], w, qt, N)
    with pytest.raises(RuntimeError, match="expected"):
        tgo.mmq(x, w[:-144], qt, N)
    with pytest.raises(RuntimeError, match="unsupported quant_type"):
        tgo.mmq(x, w, 2, N)
    with pytest.raises(RuntimeError, match="zero-row"):
        tgo.mmq(x[:0], w, qt, N)
    with pytest.raises(RuntimeError, match="torch.bfloat16"):
        tgo.mmq(x.float(), w, qt, N)
    with pytest.raises(RuntimeError, match="multiple of 256"):
        torch.ops.torch_ggml_ops.mmq_grad_input(to_dev(blocks.gaussian_bf16((4, N), 1)), w, qt, 100)
