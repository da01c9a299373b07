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
    "tgo_selftest_wait_timeout": (_i32, [_i64, _vp]),
    "tgo_dequantize_bf16": (_i32, [_vp, _i64, _i32, _vp, _vp]),
    "tgo_mmq_fwd": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i32, _vp]),
    "tgo_mmq_dx": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i32, _vp]),
    "tgo_mmq_dx_workspace_bytes": (_i64, [_i64, _i64, _i64, _i32]),
    "tgo_mmq_dx_ws": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i32, _vp, _i64, _vp]),
    "tgo_mmq_fwd_multi": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _vp]),
    "tgo_grouped_workspace_bytes": (_i64, [_i64, _i64]),
    "tgo_build_tiles": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _vp]),
    "tgo_grouped_fwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp, _i64, _vp]),
    "tgo_grouped_dx": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp, _i64, _vp]),
    "tgo_route_workspace_bytes": (_i64, [_i64, _i64]),
    "tgo_route_sort": (_i32, [_vp, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp]),
    "tgo_gather_rows": (_i32, [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _vp]),
    "tgo_combine_rows": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "tgo_quantize_q8": (_i32, [_vp, _i64, _i64, _vp, _vp, _vp, _vp]),
    "tgo_ep_plan": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "tgo_ep_barrier": (_i32, [_vp, _i64, _i64, _i64, _i64, _vp]),
    "tgo_ep_share_counts": (_i32, [_vp, _i64, _i64, _vp, _i64, _vp]),
    "tgo_ep_dispatch": (_i32, [_vp, _i64, _vp, _vp, _i64, _i64, _vp, _i64, _vp]),
    "tgo_ep_pull": (_i32, [_vp, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "tgo_ep_token_maps": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _i64, _vp]),
    "tgo_swiglu_fwd": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _vp, _vp]),
    "tgo_swiglu_bwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp, _vp]),
    "tgo_ep_dispatch_tokens": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _i64, _vp]),
    "tgo_ep_expand": (_i32, [_vp, _i64, _vp, _vp, _vp, _i64, _i64, _vp]),
    "tgo_ep_reduce": (_i32, [_vp, _vp, _i64, _i64, _vp, _i64, _vp]),
    "tgo_ep_token_maps_rows": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp, _i64, _vp, _i64, _vp]),
    "tgo_ep_zero_dropped": (_i32, [_vp, _i64, _vp, _i64, _vp]),
    "tgo_ep_row_pointers": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _i64, _vp, _vp]),
    "tgo_grouped_fwd_rows": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp, _i64, _vp]),
    "tgo_ep_pull_tokens": (_i32, [_vp, _i64, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _vp]),
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


def selftest_wait_timeout(limit_cycles: int = 1_000_000, stream=None) -> None:
    """Launches the kernel whose bounded wait runs out on purpose (see ``tgo_selftest_wait_timeout``);
    ``device_status()`` then reports code 10."""
    check(lib().tgo_selftest_wait_timeout(limit_cycles, _stream(stream)), "tgo_selftest_wait_timeout")


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


def mmq_dx_split(dy, packed, dx, rows, out_features, in_features, quant_type, stream=None) -> int:
    """Input gradient with the split reduction where it applies (``tgo_mmq_dx_ws``); allocates the
    workspace with torch.  Returns the workspace bytes used (0: same launch as ``mmq_dx``)."""
    import torch

    need = int(lib().tgo_mmq_dx_workspace_bytes(rows, out_features, in_features, quant_type))
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dy.device)
    check(lib().tgo_mmq_dx_ws(_ptr(dy), _ptr(packed), _ptr(dx), rows, out_features, in_features, quant_type,
                              _ptr(ws) if need else None, need, _stream(stream)), "tgo_mmq_dx_ws")
    return need


def mmq_fwd_multi(x, packed_list, y_list, rows, out_features, in_features, quant_type, stream=None) -> None:
    """ys[i] = x @ W_i.T for up to four packed weights of one type and shape (``tgo_mmq_fwd_multi``)."""
    check(lib().tgo_mmq_fwd_multi(_ptr(x), _ptr_array([w.data_ptr() for w in packed_list]),
                                  _ptr_array([y.data_ptr() for y in y_list]), len(packed_list), rows, out_features,
                                  in_features, quant_type, _stream(stream)), "tgo_mmq_fwd_multi")


def grouped_workspace_bytes(rows: int, groups: int) -> int:
    return int(lib().tgo_grouped_workspace_bytes(rows, groups))


def build_tiles(expert_indices, expert_offsets, num_experts, rows, workspace, stream=None, max_tile_tokens=256) -> None:
    check(lib().tgo_build_tiles(_ptr(expert_indices), _ptr(expert_offsets), expert_indices.numel(), num_experts, rows,
                                max_tile_tokens, _ptr(workspace), workspace.numel(), _stream(stream)), "tgo_build_tiles")


def grouped_fwd(x, w0, w1, y0, y1, expert_indices, expert_offsets, num_experts, rows, out_features, in_features,
                quant_type, workspace, stream=None) -> None:
    check(lib().tgo_grouped_fwd(_ptr(x), _ptr(w0), _ptr(w1), _ptr(y0), _ptr(y1), _ptr(expert_indices),
                                _ptr(expert_offsets), expert_indices.numel(), num_experts, rows, out_features,
                                in_features, quant_type, _ptr(workspace), workspace.numel(), _stream(stream)),
          "tgo_grouped_fwd")


def grouped_fwd_rows(x, w, y_row_ptrs, expert_indices, expert_offsets, num_experts, rows, out_features, in_features,
                     quant_type, workspace, stream=None) -> None:
    """Grouped forward of one projection whose result row r is stored at the address ``y_row_ptrs[r]``
    (int64 device tensor of ``rows`` addresses, 0 = drop the row); see ``tgo_grouped_fwd_rows``."""
    check(lib().tgo_grouped_fwd_rows(_ptr(x), _ptr(w), _ptr(y_row_ptrs), _ptr(expert_indices), _ptr(expert_offsets),
                                     expert_indices.numel(), num_experts, rows, out_features, in_features, quant_type,
                                     _ptr(workspace), workspace.numel(), _stream(stream)), "tgo_grouped_fwd_rows")


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


def route_sort(expert_ids, num_experts, stream=None, out=None):
    """Device counting sort of routed pairs by expert.  ``expert_ids``: int32 [n_pairs] on the GPU.
    Returns (sorted_to_pair, pair_to_sorted, expert_indices int64 [E], expert_offsets int32 [E]).
    ``out``: optional dict of preallocated tensors (keys s2p, p2s, ei, eo, counts, ws); with a
    ``counts`` entry the per-expert pair counts are written there too."""
    import torch

    n = expert_ids.numel()
    dev = expert_ids.device
    out = {} if out is None else out
    s2p = out.get("s2p") if "s2p" in out else torch.empty(n, dtype=torch.int32, device=dev)
    p2s = out.get("p2s") if "p2s" in out else torch.empty(n, dtype=torch.int32, device=dev)
    ei = out.get("ei") if "ei" in out else torch.empty(num_experts, dtype=torch.int64, device=dev)
    eo = out.get("eo") if "eo" in out else torch.empty(num_experts, dtype=torch.int32, device=dev)
    ws = out.get("ws") if "ws" in out else torch.empty(lib().tgo_route_workspace_bytes(n, num_experts),
                                                        dtype=torch.uint8, device=dev)
    check(lib().tgo_route_sort(_ptr(expert_ids), n, num_experts, _ptr(s2p), _ptr(p2s), _ptr(ei), _ptr(eo),
                               _ptr(out.get("counts")), _ptr(ws), ws.numel(), _stream(stream)), "tgo_route_sort")
    return s2p, p2s, ei, eo


def gather_rows(src, index, divisor=1, stream=None):
    import torch

    dst = torch.empty((index.numel(), src.shape[1]), dtype=src.dtype, device=src.device)
    check(lib().tgo_gather_rows(_ptr(src), src.shape[0], _ptr(index), divisor, _ptr(dst), index.numel(), src.shape[1],
                                _stream(stream)), "tgo_gather_rows")
    return dst


def combine_rows(rows, pair_to_sorted, top_k, weights=None, stream=None):
    import torch

    tokens = pair_to_sorted.numel() // top_k
    out = torch.empty((tokens, rows.shape[1]), dtype=rows.dtype, device=rows.device)
    check(lib().tgo_combine_rows(_ptr(rows), _ptr(pair_to_sorted), _ptr(weights), _ptr(out), tokens, top_k,
                                 rows.shape[1], _stream(stream)), "tgo_combine_rows")
    return out


def quantize_q8(x, stream=None):
    """bf16 [rows, width] -> (int8 [rows, width], fp32 d [rows, width/32], fp32 sum [rows, width/32])."""
    import torch

    rows, width = x.shape
    q = torch.empty((rows, width), dtype=torch.int8, device=x.device)
    d = torch.empty((rows, width // 32), dtype=torch.float32, device=x.device)
    s = torch.empty((rows, width // 32), dtype=torch.float32, device=x.device)
    check(lib().tgo_quantize_q8(_ptr(x), rows, width, _ptr(q), _ptr(d), _ptr(s), _stream(stream)), "tgo_quantize_q8")
    return q, d, s


def _ptr_array(ptrs):
    return (ctypes.c_void_p * len(ptrs))(*[int(p) for p in ptrs])


def ep_plan(counts_all, my_rank, expert_ids, pair_to_sorted, capacity, stream=None, out=None):
    """Destination of every routed pair and the local group metadata; see ``tgo_ep_plan``.
    ``counts_all``: int32 [world, E] on the GPU.  Returns (dst_rank, dst_row, local_indices,
    local_offsets, overflow_flag).  ``out``: optional dict of preallocated tensors (keys dst_rank,
    dst_row, li, lo, scratch, overflow; the overflow flag is then sticky)."""
    import torch

    world, E = counts_all.shape
    n, dev = expert_ids.numel(), expert_ids.device
    out = {} if out is None else out
    dst_rank = out["dst_rank"] if "dst_rank" in out else torch.empty(n, dtype=torch.int32, device=dev)
    dst_row = out["dst_row"] if "dst_row" in out else torch.empty(n, dtype=torch.int32, device=dev)
    li = out["li"] if "li" in out else torch.empty(E // world, dtype=torch.int64, device=dev)
    lo = out["lo"] if "lo" in out else torch.empty(E // world, dtype=torch.int32, device=dev)
    scratch = out["scratch"] if "scratch" in out else torch.empty(2 * E, dtype=torch.int32, device=dev)
    overflow = out["overflow"] if "overflow" in out else torch.zeros(1, dtype=torch.int32, device=dev)
    check(lib().tgo_ep_plan(_ptr(counts_all), world, E, my_rank, _ptr(expert_ids), _ptr(pair_to_sorted), n, capacity,
                            _ptr(dst_rank), _ptr(dst_row), _ptr(li), _ptr(lo), _ptr(scratch), _ptr(overflow),
                            _stream(stream)), "tgo_ep_plan")
    return dst_rank, dst_row, li, lo, overflow


def ep_barrier(flag_ptrs, my_rank, epoch, limit_cycles=2_000_000_000, stream=None) -> None:
    """Stream-ordered rank barrier over peer memory with a bounded wait (``tgo_ep_barrier``)."""
    check(lib().tgo_ep_barrier(_ptr_array(flag_ptrs), len(flag_ptrs), my_rank, epoch, limit_cycles, _stream(stream)),
          "tgo_ep_barrier")


def ep_share_counts(counts, my_rank, table_ptrs, stream=None) -> None:
    """Writes this rank's per-expert pair counts into every rank's table (``tgo_ep_share_counts``)."""
    check(lib().tgo_ep_share_counts(_ptr(counts), counts.numel(), my_rank, _ptr_array(table_ptrs), len(table_ptrs),
                                    _stream(stream)), "tgo_ep_share_counts")


def ep_dispatch(src, divisor, dst_rank, dst_row, peer_ptrs, stream=None) -> None:
    check(lib().tgo_ep_dispatch(_ptr(src), divisor, _ptr(dst_rank), _ptr(dst_row), dst_rank.numel(), src.shape[1],
                                _ptr_array(peer_ptrs), len(peer_ptrs), _stream(stream)), "tgo_ep_dispatch")


def ep_pull(peer_ptrs, dst_rank, dst_row, out, group=1, weights=None, stream=None) -> None:
    check(lib().tgo_ep_pull(_ptr_array(peer_ptrs), len(peer_ptrs), _ptr(dst_rank), _ptr(dst_row), _ptr(weights),
                            _ptr(out), out.shape[0], group, out.shape[1], _stream(stream)), "tgo_ep_pull")


def ep_token_maps(dst_rank, dst_row, tokens, top_k, my_rank, tokens_per_rank, row_slot_ptrs, slot_rows_ptrs,
                  stream=None, pair_weights=None, row_weight_ptrs=None) -> None:
    """Token-level exchange, plan time: per-slot row lists on every owner and the row -> slot map on
    each pair's owner (plus, with ``pair_weights`` fp32 [tokens * top_k], each row's routing weight
    on its owner); see ``tgo_ep_token_maps``."""
    check(lib().tgo_ep_token_maps(_ptr(dst_rank), _ptr(dst_row), tokens, top_k, my_rank, tokens_per_rank,
                                  _ptr_array(row_slot_ptrs), _ptr_array(slot_rows_ptrs), _ptr(pair_weights),
                                  None if row_weight_ptrs is None else _ptr_array(row_weight_ptrs),
                                  len(row_slot_ptrs), _stream(stream)), "tgo_ep_token_maps")


def swiglu_fwd(gate, up, out, row_scale=None, n_rows_device=None, stream=None) -> None:
    """out = row_scale * silu(gate) * up on bf16 rows (``tgo_swiglu_fwd``)."""
    check(lib().tgo_swiglu_fwd(_ptr(gate), _ptr(up), _ptr(row_scale), _ptr(out), gate.shape[0], gate.shape[1],
                               _ptr(n_rows_device), _stream(stream)), "tgo_swiglu_fwd")


def swiglu_bwd(dh, gate, up, dgate, dup, row_scale=None, n_rows_device=None, stream=None) -> None:
    """dgate, dup of ``swiglu_fwd`` for the cotangent ``dh`` (``tgo_swiglu_bwd``)."""
    check(lib().tgo_swiglu_bwd(_ptr(dh), _ptr(gate), _ptr(up), _ptr(row_scale), _ptr(dgate), _ptr(dup), gate.shape[0],
                               gate.shape[1], _ptr(n_rows_device), _stream(stream)), "tgo_swiglu_bwd")


def ep_dispatch_tokens(src, dst_rank, top_k, my_rank, tokens_per_rank, token_buffer_ptrs, stream=None) -> None:
    check(lib().tgo_ep_dispatch_tokens(_ptr(src), _ptr(dst_rank), src.shape[0], top_k, src.shape[1], my_rank,
                                       tokens_per_rank, _ptr_array(token_buffer_ptrs), len(token_buffer_ptrs),
                                       _stream(stream)), "tgo_ep_dispatch_tokens")


def ep_expand(token_buffer, row_slot, n_rows_device, rows, stream=None) -> None:
    """rows[r] = token_buffer[row_slot[r]] for r < n_rows_device[0] (a device int32 tensor)."""
    check(lib().tgo_ep_expand(_ptr(token_buffer), token_buffer.shape[0], _ptr(row_slot), _ptr(n_rows_device),
                              _ptr(rows), rows.shape[0], rows.shape[1], _stream(stream)), "tgo_ep_expand")


def ep_token_maps_rows(dst_rank, dst_row, tokens, top_k, my_rank, tokens_per_rank, row_slot_ptrs, slot_rows_ptrs, result,
                       stream=None) -> None:
    """``ep_token_maps`` that also zeroes the rows of ``result`` ([tokens * top_k, width]) whose routed pair was
    dropped (``tgo_ep_token_maps_rows``)."""
    check(lib().tgo_ep_token_maps_rows(_ptr(dst_rank), _ptr(dst_row), tokens, top_k, my_rank, tokens_per_rank,
                                       _ptr_array(row_slot_ptrs), _ptr_array(slot_rows_ptrs), len(row_slot_ptrs),
                                       _ptr(result), result.shape[1], _stream(stream)), "tgo_ep_token_maps_rows")


def ep_zero_dropped(dst_rank, result, stream=None) -> None:
    """result[i] = 0 for the routed pairs with dst_rank[i] < 0 (``tgo_ep_zero_dropped``)."""
    check(lib().tgo_ep_zero_dropped(_ptr(dst_rank), dst_rank.numel(), _ptr(result), result.shape[1], _stream(stream)),
          "tgo_ep_zero_dropped")


def ep_row_pointers(row_slot, slot_rows, n_rows_device, top_k, tokens_per_rank, result_ptrs, width, row_ptrs,
                    stream=None) -> None:
    """row_ptrs[r] (int64 device tensor [capacity]) = address of the result row, at the token's owner, of
    the routed pair that expert-major row r belongs to; ``result_ptrs``: this GPU's addresses of every
    rank's [tokens_per_rank * top_k, width] result buffer.  See ``tgo_ep_row_pointers``."""
    check(lib().tgo_ep_row_pointers(_ptr(row_slot), _ptr(slot_rows), _ptr(n_rows_device), row_ptrs.shape[0],
                                    slot_rows.shape[0], top_k, tokens_per_rank, _ptr_array(result_ptrs),
                                    len(result_ptrs), width, _ptr(row_ptrs), _stream(stream)), "tgo_ep_row_pointers")


def ep_reduce(rows, slot_rows, top_k, partial_sums, stream=None) -> None:
    check(lib().tgo_ep_reduce(_ptr(rows), _ptr(slot_rows), partial_sums.shape[0], top_k, _ptr(partial_sums),
                              rows.shape[1], _stream(stream)), "tgo_ep_reduce")


def ep_pull_tokens(partial_sum_ptrs, dst_rank, top_k, my_rank, tokens_per_rank, out, stream=None) -> None:
    check(lib().tgo_ep_pull_tokens(_ptr_array(partial_sum_ptrs), len(partial_sum_ptrs), _ptr(dst_rank), out.shape[0],
                                   top_k, my_rank, tokens_per_rank, _ptr(out), out.shape[1], _stream(stream)),
          "tgo_ep_pull_tokens")
