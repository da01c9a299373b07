"""Python face of the CPU oracle (test infrastructure, not product code).

What it restates and where the reference states it:

* GGUF super-block decode  -> ``gguf_ref.c`` (csrc/ck/gguf_decode.cuh:13-149),
  called through ctypes; ``dequantize`` returns fp32, ``dequantize_bf16_bits``
  the round-to-nearest-even bf16 image the backward kernels consume
  (csrc/ck/mmq_backward.cuh:44).
* dense forward / input gradient -> fp32 ``x @ W.T`` and ``dy @ W``: the semantics
  the reference's tests assert (tests/test_mmq.py:59-63,110-117).
* grouped and pair variants -> per-group slices, two products and one sum
  (tests/test_grouped_mmq.py:108-170, 323-382).

Parity pin: ``gguf_ref.c`` is compared bit-for-bit with gguf-py 0.19.0
(``gguf.quants.dequantize``, an independent implementation of the same formats)
and with the committed vectors in ``tests/golden``.  The reference's own test
oracle lives in an un-pinned transformers fork and reads a GGUF checkpoint that is
not available, so parity at that boundary is unpinned.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libtgo_oracle.so"

Q3_K, Q4_K, Q5_K, Q6_K, IQ2_S = 11, 12, 13, 14, 22
QTYPES = {"IQ2_S": IQ2_S, "Q3_K": Q3_K, "Q4_K": Q4_K, "Q5_K": Q5_K, "Q6_K": Q6_K}
BLOCK_BYTES = {Q3_K: 110, Q4_K: 144, Q5_K: 176, Q6_K: 210, IQ2_S: 82}
QK_K = 256

IQ2S_GRID_SHA256 = "e1aa1473412b0552c2174c30ef22ab4073f6a181b85a17056e8249bd2932fd88"

_lib = None
_grid = None


def build(force: bool = False) -> Path:
    """Compile ``gguf_ref.c`` into ``libtgo_oracle.so`` next to it (gcc only)."""
    src = _HERE / "gguf_ref.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B", "libtgo_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(_LIB_PATH))
        _lib.tgo_ref_dequantize.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int,
                                            ctypes.c_void_p, ctypes.c_void_p]
        _lib.tgo_ref_dequantize.restype = ctypes.c_int
        _lib.tgo_ref_round_bf16.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
        _lib.tgo_ref_round_bf16.restype = None
        _lib.tgo_ref_block_bytes.argtypes = [ctypes.c_int]
        _lib.tgo_ref_block_bytes.restype = ctypes.c_int64
    return _lib


def iq2s_grid() -> np.ndarray:
    """The IQ2_S codebook as uint64[1024] (byte e of entry i = magnitude of element e).

    Taken at run time from the installed gguf package (the same table the reference
    vendors at csrc/vendor/llama_cpp/iq2_s_grid.cuh:7-263) and hash-checked.
    """
    global _grid
    if _grid is None:
        from gguf import quants

        quants.IQ2_S.init_grid()
        raw = np.ascontiguousarray(quants.IQ2_S.grid.reshape(1024, 8).astype(np.uint8))
        digest = hashlib.sha256(raw.tobytes()).hexdigest()
        if digest != IQ2S_GRID_SHA256:
            raise RuntimeError(f"IQ2_S grid hash mismatch: {digest}")
        _grid = raw.view("<u8").reshape(1024).copy()
    return _grid


def cpu_threads() -> int:
    return max(1, len(os.sched_getaffinity(0)))


def dequantize(packed: np.ndarray, qtype: int, threads: int | None = None) -> np.ndarray:
    """Decode a flat uint8 array of whole super-blocks to fp32 (n_blocks*256 values)."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1)
    bb = BLOCK_BYTES[qtype]
    if packed.size % bb:
        raise ValueError("byte count is not a whole number of blocks")
    n_blocks = packed.size // bb
    out = np.empty(n_blocks * QK_K, dtype=np.float32)
    grid = iq2s_grid() if qtype == IQ2_S else None
    gptr = grid.ctypes.data if grid is not None else None
    L = lib()
    threads = threads or cpu_threads()
    threads = max(1, min(threads, n_blocks // 1024 or 1))
    bounds = np.linspace(0, n_blocks, threads + 1).astype(np.int64)

    def work(i):
        b0, b1 = int(bounds[i]), int(bounds[i + 1])
        if b1 > b0:
            rc = L.tgo_ref_dequantize(packed.ctypes.data + b0 * bb, b1 - b0, qtype, gptr,
                                      out.ctypes.data + b0 * QK_K * 4)
            if rc:
                raise RuntimeError(f"oracle dequantize failed: {rc}")

    if threads == 1:
        work(0)
    else:
        with ThreadPoolExecutor(threads) as ex:
            list(ex.map(work, range(threads)))
    return out


def round_bf16_bits(values: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit patterns (uint16), round to nearest even."""
    values = np.ascontiguousarray(values, dtype=np.float32)
    out = np.empty(values.shape, dtype=np.uint16)
    lib().tgo_ref_round_bf16(values.ctypes.data, values.size, out.ctypes.data)
    return out


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def weight_fp32(packed: np.ndarray, qtype: int, out_features: int, in_features: int,
                threads: int | None = None) -> np.ndarray:
    """Logical weight [N, K] of a dense packed tensor (row n = K/256 consecutive blocks)."""
    return dequantize(packed, qtype, threads).reshape(out_features, in_features)


def expert_weights_fp32(packed: np.ndarray, qtype: int, out_features: int, in_features: int,
                        threads: int | None = None) -> np.ndarray:
    """Logical weights [E, N, K] of a grouped packed tensor [E, N, row_bytes]."""
    e = packed.shape[0]
    return dequantize(packed, qtype, threads).reshape(e, out_features, in_features)


def groups(expert_indices, expert_offsets, rows: int, num_experts: int):
    """Yield (expert, begin, end) of every valid group; invalid ones are skipped exactly
    as the reference kernels skip them (csrc/mmq_core.cuh:468-476)."""
    begin = 0
    for e, end in zip(list(map(int, expert_indices)), list(map(int, expert_offsets))):
        b = begin
        begin = end
        if 0 <= e < num_experts and 0 <= b < end <= rows:
            yield e, b, end


def mmq_forward(x, weight):
    """fp32 ``x @ W.T`` (x: torch tensor [..., K] any float dtype, weight: fp32 [N, K])."""
    import torch

    w = torch.from_numpy(np.asarray(weight))
    return x.to(torch.float32).reshape(-1, w.shape[1]) @ w.t()


def mmq_grad_input(dy, weight):
    import torch

    w = torch.from_numpy(np.asarray(weight))
    return dy.to(torch.float32).reshape(-1, w.shape[0]) @ w


def grouped_forward(x, weights, expert_indices, expert_offsets):
    """Per-group fp32 ``x[b:e] @ W[expert].T``; rows outside every valid group stay NaN."""
    import torch

    w = torch.from_numpy(np.asarray(weights))
    out = torch.full((x.shape[0], w.shape[1]), float("nan"), dtype=torch.float32)
    xf = x.to(torch.float32)
    for e, b, end in groups(expert_indices, expert_offsets, x.shape[0], w.shape[0]):
        out[b:end] = xf[b:end] @ w[e].t()
    return out


def grouped_grad_input(dy, weights, expert_indices, expert_offsets, second=None):
    """Per-group fp32 ``dy[b:e] @ W[expert]``; ``second=(dy2, weights2)`` adds the other
    Jacobian of a gate/up pair before anything is rounded
    (csrc/ck/grouped_mmq_backward.cuh:415-441)."""
    import torch

    w = torch.from_numpy(np.asarray(weights))
    out = torch.full((dy.shape[0], w.shape[2]), float("nan"), dtype=torch.float32)
    dyf = dy.to(torch.float32)
    if second is not None:
        dy2 = second[0].to(torch.float32)
        w2 = torch.from_numpy(np.asarray(second[1]))
    for e, b, end in groups(expert_indices, expert_offsets, dy.shape[0], w.shape[0]):
        acc = dyf[b:end] @ w[e]
        if second is not None:
            acc = acc + dy2[b:end] @ w2[e]
        out[b:end] = acc
    return out


def rel_frobenius(test, ref) -> float:
    """||test - ref||_F / ||ref||_F over finite reference entries (torch tensors)."""
    import torch

    ref = ref.to(torch.float64)
    test = test.to(torch.float64)
    mask = torch.isfinite(ref)
    num = torch.linalg.vector_norm((test - ref)[mask])
    den = torch.linalg.vector_norm(ref[mask])
    return float(num / den) if float(den) > 0 else float(num)


def max_row_error(test, ref) -> float:
    """max over rows of ||test[r] - ref[r]|| / ||ref[r]||, over the rows whose reference is finite.
    A norm over the whole output hides a handful of wrong rows in a large matrix; this does not."""
    import torch

    ref = ref.to(torch.float64)
    test = test.to(torch.float64)
    rows = torch.isfinite(ref).all(dim=1)
    num = torch.linalg.vector_norm((test - ref)[rows], dim=1)
    den = torch.linalg.vector_norm(ref[rows], dim=1)
    err = torch.where(den > 0, num / den.clamp_min(1e-300), num)
    return float(err.max()) if err.numel() else 0.0


def quantize_q8(x):
    """q8_1-style activation blocks of 32 values (csrc/mmq_core.cuh:151-209): returns
    (int8 quants, fp32 d = amax/127, fp32 sum of the unquantised values), numpy arrays.
    ``x``: torch tensor [rows, width] of any float dtype, width a multiple of 32."""
    xf = x.to(__import__("torch").float32).numpy()
    rows, width = xf.shape
    b = xf.reshape(rows, width // 32, 32)
    amax = np.abs(b).max(axis=2)
    with np.errstate(divide="ignore", invalid="ignore"):
        inv = np.where(amax > 0, np.float32(127.0) / amax, np.float32(0)).astype(np.float32)
        d = np.where(amax > 0, amax / np.float32(127.0), np.float32(0)).astype(np.float32)
    scaled = b * inv[:, :, None]
    q = (np.sign(scaled) * np.floor(np.abs(scaled) + np.float32(0.5))).astype(np.int8)  # roundf: half away from zero
    return q.reshape(rows, width), d, b.sum(axis=2, dtype=np.float64).astype(np.float32)
