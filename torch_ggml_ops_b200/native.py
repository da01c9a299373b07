"""ctypes binding of ``lib/libtgo_mmq.so`` (the C ABI declared in ``include/tgo_mmq.h``).

The torch operators reach the same entry points through the stable-ABI module ``_C``; this view
exists for callers that hold raw device pointers (tests that exercise the C boundary directly,
the benchmark's kernel-only timing).  Every wrapper raises ``RuntimeError`` with the library's
message when a call fails; nothing here computes anything.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

NOALLOC_MAX_TILES = 4096  # TGO_NOALLOC_MAX_TILES in include/tgo_mmq.h
_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libtgo_mmq.so"

_vp, _i64, _i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int

# name -> (restype, argtypes); must list every symbol include/tgo_mmq.h declares
SIGNATURES = {
    "tgo_version": (_i32, []),
    "tgo_last_error": (ctypes.c_char_p, []),
    "tgo_block_bytes": (_i64, [_i32]),
    "tgo_device_status": (_i32, [ctypes.POINTER(ctypes.c_int)]),
    "tgo_dequantize_bf16": (_i32, [_vp, _i64, _i32, _vp, _vp]),
    "tgo_mmq_fwd": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i32, _vp]),
    "tgo_mmq_dx": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i32, _vp]),
    "tgo_grouped_workspace_bytes": (_i64, [_i64, _i64]),
    "tgo_build_tiles": (_i32, [_vp, _vp, _i64, _i64, _i64, _vp, _i64, _vp]),
    "tgo_grouped_fwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp, _i64, _vp]),
    "tgo_grouped_dx": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp, _i64, _vp]),
    "tgo_grouped_fwd_noalloc": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """Load the library (once).  Fails loudly if it has not been built."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise ImportError(f"{_LIB_PATH} is missing: run `python torch_ggml_ops_b200/_build.py`")
        import torch  # noqa: F401  loads libcudart.so.12 into the process first

        handle = ctypes.CDLL(str(_LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def last_error() -> str:
    return (lib().tgo_last_error() or b"").decode()


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed ({rc}): {last_error()}")


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream(stream=None) -> int:
    import torch

    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


def device_status() -> int:
    out = ctypes.c_int(0)
    check(lib().tgo_device_status(ctypes.byref(out)), "tgo_device_status")
    return out.value


def dequantize_bf16(packed, quant_type: int, out=None, stream=None):
    import torch

    bb = lib().tgo_block_bytes(quant_type)
    if bb <= 0:
        raise RuntimeError(f"unsupported quant_type: {quant_type}")
    n_blocks = packed.numel() // bb
    if out is None:
        out = torch.empty(n_blocks * 256, dtype=torch.bfloat16, device=packed.device)
    check(lib().tgo_dequantize_bf16(_ptr(packed), n_blocks, quant_type, _ptr(out), _stream(stream)),
          "tgo_dequantize_bf16")
    return out


def mmq_fwd(x, packed, y, rows, out_features, in_features, quant_type, stream=None) -> None:
    check(lib().tgo_mmq_fwd(_ptr(x), _ptr(packed), _ptr(y), rows, out_features, in_features, quant_type,
                            _stream(stream)), "tgo_mmq_fwd")


def mmq_dx(dy, packed, dx, rows, out_features, in_features, quant_type, stream=None) -> None:
    check(lib().tgo_mmq_dx(_ptr(dy), _ptr(packed), _ptr(dx), rows, out_features, in_features, quant_type,
                           _stream(stream)), "tgo_mmq_dx")


def grouped_workspace_bytes(rows: int, groups: int) -> int:
    return int(lib().tgo_grouped_workspace_bytes(rows, groups))


def build_tiles(expert_indices, expert_offsets, num_experts, rows, workspace, stream=None) -> None:
    check(lib().tgo_build_tiles(_ptr(expert_indices), _ptr(expert_offsets), expert_indices.numel(), num_experts, rows,
                                _ptr(workspace), workspace.numel(), _stream(stream)), "tgo_build_tiles")


def grouped_fwd(x, w0, w1, y0, y1, expert_indices, expert_offsets, num_experts, rows, out_features, in_features,
                quant_type, workspace, stream=None) -> None:
    check(lib().tgo_grouped_fwd(_ptr(x), _ptr(w0), _ptr(w1), _ptr(y0), _ptr(y1), _ptr(expert_indices),
                                _ptr(expert_offsets), expert_indices.numel(), num_experts, rows, out_features,
                                in_features, quant_type, _ptr(workspace), workspace.numel(), _stream(stream)),
          "tgo_grouped_fwd")


def grouped_dx(dy0, dy1, w0, w1, dx, expert_indices, expert_offsets, num_experts, rows, out_features, in_features,
               quant_type, workspace, stream=None) -> None:
    check(lib().tgo_grouped_dx(_ptr(dy0), _ptr(dy1), _ptr(w0), _ptr(w1), _ptr(dx), _ptr(expert_indices),
                               _ptr(expert_offsets), expert_indices.numel(), num_experts, rows, out_features,
                               in_features, quant_type, _ptr(workspace), workspace.numel(), _stream(stream)),
          "tgo_grouped_dx")


def grouped_fwd_noalloc(x, w0, w1, y0, y1, expert_indices, expert_offsets, num_experts, rows, out_features,
                        in_features, quant_type, stream=None) -> None:
    """Grouped forward that keeps its tile list in the library's built-in scratch (no workspace
    argument, no device allocation); see ``tgo_grouped_fwd_noalloc`` in ``include/tgo_mmq.h``."""
    check(lib().tgo_grouped_fwd_noalloc(_ptr(x), _ptr(w0), _ptr(w1), _ptr(y0), _ptr(y1), _ptr(expert_indices),
                                        _ptr(expert_offsets), expert_indices.numel(), num_experts, rows,
                                        out_features, in_features, quant_type, _stream(stream)),
          "tgo_grouped_fwd_noalloc")
