"""GGUF ingestion: map the quantized tensors of a GGUF file straight into the layouts the
operators take - dense ``[N, row_bytes]`` and grouped ``[E, N, row_bytes]`` uint8, raw super-blocks
exactly as stored, never repacked or dequantised.

The reference reads its benchmark weights the same way (``gguf.GGUFReader`` in
bench/mmq_benchmark_common.py:196-200); its operators then take ``packed_weight`` as an uint8
tensor of raw blocks plus the GGML type id, which is what ``load_packed`` returns.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .quant_types import GGML_TYPE_IDS, row_bytes

SUPPORTED_TYPES = frozenset(GGML_TYPE_IDS.values())


@dataclass
class PackedTensor:
    """A quantized GGUF tensor in operator layout."""

    name: str
    quant_type: int           # GGML type id (11 Q3_K, 12 Q4_K, 13 Q5_K, 14 Q6_K, 22 IQ2_S)
    out_features: int         # N
    in_features: int          # K (a multiple of 256)
    experts: int              # 0 for a dense [N, K] tensor, E for an expert stack [E, N, K]
    data: torch.Tensor        # uint8 [N, row_bytes] or [E, N, row_bytes]


def pack_tensor(name: str, raw: np.ndarray, quant_type: int, logical_shape) -> PackedTensor:
    """``raw``: the tensor's bytes as gguf-py exposes them (uint8, any shape whose last axis runs
    along a row); ``logical_shape``: GGUF order, innermost first: (K, N) or (K, N, E)."""
    if quant_type not in SUPPORTED_TYPES:
        raise ValueError(f"unsupported quant_type: {quant_type}")
    dims = [int(d) for d in logical_shape]
    if len(dims) not in (2, 3):
        raise ValueError(f"{name}: expected a 2-D or 3-D tensor, got shape {dims}")
    k, n = dims[0], dims[1]
    e = dims[2] if len(dims) == 3 else 0
    rb = row_bytes(quant_type, k)
    flat = np.ascontiguousarray(raw).reshape(-1).view(np.uint8)
    want = max(e, 1) * n * rb
    if flat.size != want:
        raise ValueError(f"{name}: {flat.size} bytes, expected {want} ({max(e, 1)} x {n} rows of {rb} bytes per row)")
    shape = (e, n, rb) if e else (n, rb)
    return PackedTensor(name, int(quant_type), n, k, e, torch.from_numpy(flat.reshape(shape).copy()))


def load_packed(path, names=None, device=None) -> dict:
    """All tensors of the GGUF file at ``path`` whose type the operators support (or only
    ``names``), keyed by tensor name.  ``device``: move the bytes there (e.g. "cuda")."""
    from gguf import GGUFReader

    reader = GGUFReader(str(path))
    out = {}
    for t in reader.tensors:
        if names is not None and t.name not in names:
            continue
        qt = int(t.tensor_type)
        if qt not in SUPPORTED_TYPES:
            if names is not None:
                raise ValueError(f"{t.name}: unsupported quant_type: {qt}")
            continue
        p = pack_tensor(t.name, np.asarray(t.data), qt, t.shape)
        if device is not None:
            p.data = p.data.to(device)
        out[t.name] = p
    if names is not None:
        missing = [n for n in names if n not in out]
        if missing:
            raise KeyError(f"tensors not found in {path}: {missing}")
    return out


__all__ = ["PackedTensor", "pack_tensor", "load_packed"]
