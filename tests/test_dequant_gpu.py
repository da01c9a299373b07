"""GPU parity of the device decoders: bit-exact against the CPU oracle and the golden vectors.
(Property: every dequantised value, all 256 positions of a block, all five types, including
extreme scale / minimum bytes and blocks that start on every 2-byte misalignment.)"""
import numpy as np
import pytest
import torch

from oracle import blocks, ref
from helpers import ALL_TYPES, bits, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,qt", ALL_TYPES)
def test_decode_equals_golden_bits(cuda, golden, name, qt):
    from torch_ggml_ops_b200 import native

    blk = golden[f"{name}_blocks"]
    want = ref.round_bf16_bits(golden[f"{name}_fp32"])
    got = bits(native.dequantize_bf16(to_dev(blk.reshape(-1)), qt))
    assert np.array_equal(got, want)


@pytest.mark.parametrize("name,qt", ALL_TYPES)
@pytest.mark.parametrize("n_blocks", [1, 7, 33, 4099])
def test_decode_equals_oracle_bits(cuda, name, qt, n_blocks):
    from torch_ggml_ops_b200 import native

    blk = np.concatenate([blocks.random_blocks(qt, n_blocks, 17 * n_blocks + qt), blocks.extreme_blocks(qt)])
    want = ref.round_bf16_bits(ref.dequantize(blk, qt))
    got = bits(native.dequantize_bf16(to_dev(blk.reshape(-1)), qt))
    assert np.array_equal(got, want)
    assert native.device_status() == 0


def test_decode_rejects_bad_arguments(cuda):
    from torch_ggml_ops_b200 import native

    buf = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError, match="unsupported quant_type"):
        native.dequantize_bf16(buf, 3)
    out = torch.empty(512, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="16-byte aligned"):
        native.check(native.lib().tgo_dequantize_bf16(buf.data_ptr() + 2, 1, 12, out.data_ptr(), None), "x")
