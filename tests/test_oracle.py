"""CPU tests: the oracle against the committed golden vectors, gguf-py and its own invariants."""
import numpy as np
import pytest
import torch

from oracle import blocks, ref
from helpers import ALL_TYPES


@pytest.mark.parametrize("name,qt", ALL_TYPES)
def test_dequantize_matches_golden_bit_for_bit(golden, name, qt):
    blk = golden[f"{name}_blocks"]
    want = golden[f"{name}_fp32"]
    got = ref.dequantize(blk, qt)
    assert got.dtype == np.float32
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("name,qt", ALL_TYPES)
def test_dequantize_matches_gguf_py(name, qt):
    gguf = pytest.importorskip("gguf")
    from gguf import quants

    blk = np.concatenate([blocks.random_blocks(qt, 2048, 31 + qt), blocks.extreme_blocks(qt)])
    theirs = quants.dequantize(blk, getattr(gguf.GGMLQuantizationType, name)).astype(np.float32).reshape(-1)
    mine = ref.dequantize(blk, qt)
    assert np.array_equal(mine.view(np.uint32), theirs.view(np.uint32))


@pytest.mark.parametrize("name,qt", ALL_TYPES)
def test_threaded_dequantize_equals_single_thread(name, qt):
    blk = blocks.random_blocks(qt, 5000, 5)
    a = ref.dequantize(blk, qt, threads=1)
    b = ref.dequantize(blk, qt, threads=4)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_block_bytes_table():
    assert {qt: ref.lib().tgo_ref_block_bytes(qt) for qt in ref.BLOCK_BYTES} == ref.BLOCK_BYTES
    assert ref.lib().tgo_ref_block_bytes(2) == -1


def test_bf16_rounding_is_nearest_even_and_matches_torch():
    rng = np.random.Generator(np.random.PCG64(0))
    x = rng.standard_normal(100000).astype(np.float32) * np.float32(37.0)
    x[:6] = [0.0, -0.0, 1.0, 1.00390625, 1.01171875, -3.0e38]  # ties: 1+2^-8 -> 1, 1+3*2^-8 -> 1+2^-6
    got = ref.round_bf16_bits(x)
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(got, want)
    assert got[3] == 0x3F80 and got[4] == 0x3F82


@pytest.mark.parametrize("name,qt", ALL_TYPES)
def test_golden_matmul_known_answers(golden, name, qt):
    W = ref.weight_fp32(golden[f"{name}_mm_w"].reshape(-1), qt, 16, 256)
    x = torch.from_numpy(golden[f"{name}_mm_x"])
    dy = torch.from_numpy(golden[f"{name}_mm_dy"])
    y = ref.mmq_forward(x, W).numpy()
    dx = ref.mmq_grad_input(dy, W).numpy()
    np.testing.assert_allclose(y, golden[f"{name}_mm_y"], rtol=2e-5, atol=1e-5 * np.abs(golden[f"{name}_mm_y"]).max())
    np.testing.assert_allclose(dx, golden[f"{name}_mm_dx"], rtol=2e-5, atol=1e-5 * np.abs(golden[f"{name}_mm_dx"]).max())


def test_random_blocks_are_seeded_and_have_finite_scales():
    for _, qt in ALL_TYPES:
        a = blocks.random_blocks(qt, 64, 9)
        b = blocks.random_blocks(qt, 64, 9)
        c = blocks.random_blocks(qt, 64, 10)
        assert np.array_equal(a, b) and not np.array_equal(a, c)
        assert a.shape == (64, ref.BLOCK_BYTES[qt])
        assert np.isfinite(ref.dequantize(a, qt)).all()


def test_groups_skip_invalid_entries():
    # expert ids out of range, empty and decreasing spans are skipped; begin is always the previous offset
    got = list(ref.groups([0, 9, 2, 1, 3], [4, 6, 6, 5, 12], rows=12, num_experts=4))
    assert got == [(0, 0, 4), (3, 5, 12)]
    assert list(ref.groups([1], [13], rows=12, num_experts=4)) == []


def test_grouped_reference_matches_dense_slices():
    qt = ref.Q4_K
    w = blocks.expert_weights(qt, 3, 32, 256, 1)
    W = ref.expert_weights_fp32(w, qt, 32, 256)
    x = blocks.gaussian_bf16((10, 256), 2)
    y = ref.grouped_forward(x, W, [2, 0], [4, 10])
    assert torch.equal(y[:4], ref.mmq_forward(x[:4], W[2]))
    assert torch.equal(y[4:], ref.mmq_forward(x[4:], W[0]))
    dy = blocks.gaussian_bf16((10, 32), 3)
    dx = ref.grouped_grad_input(dy, W, [2, 0], [4, 10], second=(dy, W))
    assert torch.allclose(dx[:4], 2 * ref.mmq_grad_input(dy[:4], W[2]))


def test_routing_generator_and_sort():
    ids = blocks.topk_routing(512, 32, 8, seed=4)
    assert ids.shape == (512, 8) and ids.min() >= 0 and ids.max() < 32
    assert all(len(set(r)) == 8 for r in ids.tolist())
    perm, ei, eo = blocks.sort_by_expert(ids, 32)
    flat = ids.reshape(-1)
    assert (np.diff(flat[perm]) >= 0).all() and eo[-1] == flat.size and len(ei) == 32
    counts = np.bincount(flat, minlength=32)
    assert np.array_equal(np.diff(np.concatenate([[0], eo])), counts)
    assert counts.max() > 2 * max(1, counts.min())  # skewed, as the benchmark configs ask
