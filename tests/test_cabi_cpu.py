"""CPU tests of the C-ABI library and the Python operator surface: the library loads, exports
every declared symbol, rejects bad arguments before touching a device, and the operators are
registered with the reference's schemas, fake kernels and autograd guards."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "tgo_mmq.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tgo_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from torch_ggml_ops_b200 import native

    lib = native.lib()
    names = declared_symbols()
    assert len(names) >= 11
    for name in names:
        assert hasattr(lib, name), name
    assert sorted(native.SIGNATURES) == names


def test_host_only_entry_points():
    from torch_ggml_ops_b200 import native

    lib = native.lib()
    assert lib.tgo_version() >= 100
    assert [lib.tgo_block_bytes(q) for q in (11, 12, 13, 14, 22)] == [110, 144, 176, 210, 82]
    assert lib.tgo_block_bytes(2) == -1
    # capacity of the tile list: rows/256 + groups entries of 16 bytes after a 16-byte header
    assert lib.tgo_grouped_workspace_bytes(65536, 256) == 16 + 16 * (256 + 256)
    assert lib.tgo_grouped_workspace_bytes(1, 1) == 32


def test_argument_validation_happens_before_any_device_work():
    from torch_ggml_ops_b200 import native

    lib = native.lib()
    buf = (ctypes.c_char * 64)()
    p = ctypes.addressof(buf) & ~15
    cases = [
        (lambda: lib.tgo_mmq_fwd(p, p, p, 4, 8, 256, 99, None), "unsupported quant_type: 99"),
        (lambda: lib.tgo_mmq_fwd(p, p, p, 0, 8, 256, 12, None), "zero-row"),
        (lambda: lib.tgo_mmq_fwd(p, p, p, 4, 8, 100, 12, None), "multiple of 256"),
        (lambda: lib.tgo_mmq_fwd(p + 2, p, p, 4, 8, 256, 12, None), "16-byte aligned"),
        (lambda: lib.tgo_mmq_dx(None, p, p, 4, 8, 256, 12, None), "null"),
        (lambda: lib.tgo_grouped_fwd(p, p, None, p, None, p, p, 2, 1, 4, 8, 256, 12, p, 4096, None),
         "exceeds packed expert count"),
        (lambda: lib.tgo_grouped_fwd(p, p, p, p, None, p, p, 1, 1, 4, 8, 256, 12, p, 4096, None), "both"),
        (lambda: lib.tgo_grouped_dx(p, None, p, None, p, p, p, 1, 1, 4, 8, 256, 12, p, 8, None), "workspace"),
        (lambda: lib.tgo_build_tiles(p, p, 0, 1, 4, 256, p, 4096, None), "at least one active expert"),
        (lambda: lib.tgo_dequantize_bf16(p, 0, 12, p, None), "n_blocks"),
    ]
    for call, needle in cases:
        assert call() < 0
        assert needle in native.last_error(), (needle, native.last_error())


SCHEMAS = {
    "mmq": "torch_ggml_ops::mmq(Tensor input, Tensor packed_weight, int quant_type, int out_features) -> Tensor",
    "mmq_grad_input": "torch_ggml_ops::mmq_grad_input(Tensor grad_output, Tensor packed_weight, int quant_type, int in_features) -> Tensor",
    "grouped_mmq": "torch_ggml_ops::grouped_mmq(Tensor input, Tensor packed_weight, Tensor expert_indices, Tensor expert_offsets, int quant_type, int out_features) -> Tensor",
    "grouped_mmq_grad_input": "torch_ggml_ops::grouped_mmq_grad_input(Tensor grad_output, Tensor packed_weight, Tensor expert_indices, Tensor expert_offsets, int quant_type, int in_features) -> Tensor",
    "grouped_mmq_pair": "torch_ggml_ops::grouped_mmq_pair(Tensor input, Tensor first_packed_weight, Tensor second_packed_weight, Tensor expert_indices, Tensor expert_offsets, int quant_type, int out_features) -> (Tensor, Tensor)",
    "grouped_mmq_pair_grad_input": "torch_ggml_ops::grouped_mmq_pair_grad_input(Tensor first_grad_output, Tensor second_grad_output, Tensor first_packed_weight, Tensor second_packed_weight, Tensor expert_indices, Tensor expert_offsets, int quant_type, int in_features) -> Tensor",
}


@pytest.mark.parametrize("name", sorted(SCHEMAS))
def test_operator_schemas_match_the_reference(name):
    import torch_ggml_ops_b200  # noqa: F401

    op = getattr(torch.ops.torch_ggml_ops, name).default
    assert str(op._schema) == SCHEMAS[name]


def test_fake_kernels_give_the_reference_shapes():
    import torch_ggml_ops_b200 as tgo

    x = torch.empty(3, 43, 2048, dtype=torch.bfloat16, device="meta")
    w = torch.empty(37 * 8 * 144, dtype=torch.uint8, device="meta")
    assert tgo.mmq(x, w, 12, 37).shape == (3, 43, 37)
    dy = torch.empty(3, 43, 37, dtype=torch.bfloat16, device="meta")
    assert torch.ops.torch_ggml_ops.mmq_grad_input(dy, w, 12, 2048).shape == (3, 43, 2048)
    xr = torch.empty(262, 2048, dtype=torch.bfloat16, device="meta")
    we = torch.empty(8, 512, 8 * 144, dtype=torch.uint8, device="meta")
    ei = torch.empty(4, dtype=torch.int64, device="meta")
    eo = torch.empty(4, dtype=torch.int32, device="meta")
    assert tgo.grouped_mmq(xr, we, ei, eo, 12, 512).shape == (262, 512)
    a, b = tgo.grouped_mmq_pair(xr, we, we, ei, eo, 12, 512)
    assert a.shape == b.shape == (262, 512) and a.dtype == torch.bfloat16
    g = torch.empty(262, 512, dtype=torch.bfloat16, device="meta")
    assert torch.ops.torch_ggml_ops.grouped_mmq_grad_input(g, we, ei, eo, 12, 2048).shape == (262, 2048)
    assert torch.ops.torch_ggml_ops.grouped_mmq_pair_grad_input(g, g, we, we, ei, eo, 12, 2048).shape == (262, 2048)


def test_there_is_no_cpu_implementation():
    import torch_ggml_ops_b200 as tgo

    x = torch.zeros(2, 256, dtype=torch.bfloat16)
    w = torch.zeros(4 * 144, dtype=torch.uint8)
    with pytest.raises((NotImplementedError, RuntimeError)):
        tgo.mmq(x, w, 12, 4)


def test_reference_package_name_is_an_alias():
    import torch_ggml_ops
    import torch_ggml_ops_b200

    assert torch_ggml_ops.mmq is torch_ggml_ops_b200.mmq
    assert torch_ggml_ops.grouped_mmq_pair is torch_ggml_ops_b200.grouped_mmq_pair


def test_product_never_imports_the_oracle():
    pkg = ROOT / "torch_ggml_ops_b200"
    for path in list(pkg.rglob("*.py")) + list(pkg.rglob("*.cu*")) + list(pkg.rglob("*.cpp")) + list(pkg.rglob("*.h")):
        assert "oracle" not in path.read_text().lower(), path
