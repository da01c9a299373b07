"""GGUF ingestion (CPU): a GGUF file written with gguf-py's own writer is read back into the
operators' layouts, and the bytes dequantise (oracle) to what gguf-py dequantises."""
import importlib.util
import sys
from pathlib import Path

import numpy as np
import pytest

from oracle import blocks, ref

gguf = pytest.importorskip("gguf")

ROOT = Path(__file__).resolve().parents[1]


def _loader():
    # the package itself needs the CUDA extension; the loader does not
    pkg = ROOT / "torch_ggml_ops_b200"
    for name in ("quant_types", "gguf_loader"):
        full = f"tgo_loader_test.{name}"
        if full in sys.modules:
            continue
        if "tgo_loader_test" not in sys.modules:
            import types

            m = types.ModuleType("tgo_loader_test")
            m.__path__ = [str(pkg)]
            sys.modules["tgo_loader_test"] = m
        spec = importlib.util.spec_from_file_location(full, pkg / f"{name}.py")
        mod = importlib.util.module_from_spec(spec)
        sys.modules[full] = mod
        spec.loader.exec_module(mod)
    return sys.modules["tgo_loader_test.gguf_loader"]


def test_round_trip_through_a_gguf_file(tmp_path):
    loader = _loader()
    path = tmp_path / "tiny.gguf"
    w = gguf.GGUFWriter(str(path), "llama")
    dense = {}
    for name, qt in ref.QTYPES.items():
        N, K = 24, 512
        raw = blocks.dense_weight(qt, N, K, seed=qt).reshape(N, -1)
        dense[name] = (qt, N, K, raw)
        w.add_tensor(f"blk.0.dense_{name}.weight", raw, raw_dtype=gguf.GGMLQuantizationType(qt))
    E3, N3, K3 = 3, 16, 256
    experts = blocks.expert_weights(ref.Q4_K, E3, N3, K3, seed=9)
    w.add_tensor("blk.0.ffn_gate_exps.weight", experts, raw_dtype=gguf.GGMLQuantizationType.Q4_K)
    w.add_tensor("blk.0.norm.weight", np.ones(8, dtype=np.float32))   # not a supported type: skipped
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()

    got = loader.load_packed(path)
    assert "blk.0.norm.weight" not in got
    for name, (qt, N, K, raw) in dense.items():
        p = got[f"blk.0.dense_{name}.weight"]
        assert (p.quant_type, p.out_features, p.in_features, p.experts) == (qt, N, K, 0)
        assert np.array_equal(p.data.numpy(), raw)
        want = gguf.quants.dequantize(raw, gguf.GGMLQuantizationType(qt))
        assert np.array_equal(ref.weight_fp32(p.data.numpy().reshape(-1), qt, N, K), want)
    p = got["blk.0.ffn_gate_exps.weight"]
    assert (p.quant_type, p.experts, p.out_features, p.in_features) == (ref.Q4_K, E3, N3, K3)
    assert np.array_equal(p.data.numpy(), experts)
    only = loader.load_packed(path, names=["blk.0.ffn_gate_exps.weight"])
    assert list(only) == ["blk.0.ffn_gate_exps.weight"]
    with pytest.raises(KeyError):
        loader.load_packed(path, names=["nope"])
    with pytest.raises(ValueError, match="unsupported quant_type"):
        loader.load_packed(path, names=["blk.0.norm.weight"])
