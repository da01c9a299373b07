"""Shared helpers of the parity tests: seeded inputs, device transfer, comparisons."""
import numpy as np
import torch

from oracle import blocks, ref

ALL_TYPES = sorted(ref.QTYPES.items(), key=lambda kv: kv[1])  # [(name, id)]
TYPE_IDS = [qt for _, qt in ALL_TYPES]
TYPE_NAMES = [n for n, _ in ALL_TYPES]

FWD_TOL = 1e-2   # relative Frobenius error of forward outputs vs fp32 dequant + matmul
DX_TOL = 5e-3    # same for input gradients


def to_dev(a, device="cuda"):
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        a = torch.from_numpy(a)
    return a.to(device)


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> uint16 bit patterns on the host."""
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def bf16_from_bits(b: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(b.view(np.int16).copy()).view(torch.bfloat16)


def dense_case(qt, N, K, seed):
    """(packed uint8 flat, fp32 weight [N,K], bf16-rounded weight as torch bf16 [N,K])."""
    w = blocks.dense_weight(qt, N, K, seed)
    W = ref.weight_fp32(w, qt, N, K)
    Wb = bf16_from_bits(ref.round_bf16_bits(W))
    return w, W, Wb


def expert_case(qt, E, N, K, seed):
    w = blocks.expert_weights(qt, E, N, K, seed)
    W = ref.expert_weights_fp32(w, qt, N, K)
    return w, W


def routing_from_sizes(sizes, expert_ids):
    ei = torch.tensor(list(expert_ids), dtype=torch.int64)
    eo = torch.tensor(np.cumsum(sizes), dtype=torch.int32)
    return ei, eo


def values_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Exact equality of values (+0 == -0, as torch.equal treats them)."""
    return bool(torch.equal(a.float().cpu(), b.float().cpu()))
