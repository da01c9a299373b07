"""Operators either side of the reference's surface (they have no reference schema, so they are
registered under this package's own namespace ``torch_ggml_ops_b200::``):

* ``mmq_multi``: several dense projections of one activation tensor in one call (the reference's
  own "remaining work" for the dense forward, docs/mmq_fwd_optimization.md:299-307);
* ``swiglu``: ``silu(gate) * up``, the step a caller runs between ``grouped_mmq_pair`` and the down
  projection (README.md:3 leaves it to the caller);
* ``moe_mlp``: the single-GPU MoE feed-forward block built from the grouped operators;
* ``lm_head_loss``: the chunked LM-head loop (forward -> cross entropy -> input gradient over
  chunks of rows) that the reference's other production consumer runs
  (docs/mmq_bwd_optimization.md:502-524), which never materialises the full logits.

Everything here calls the same native kernels as the six reference operators; nothing has a CPU or
eager fallback.
"""
from __future__ import annotations

import torch

from . import native

_NS = "torch_ggml_ops_b200"


# ------------------------------------------------------------------ dense multi-projection
@torch.library.custom_op(f"{_NS}::mmq_multi", mutates_args=(), device_types="cuda")
def _mmq_multi(input: torch.Tensor, packed_weights: list[torch.Tensor], quant_type: int, out_features: int) -> list[torch.Tensor]:
    if not 1 <= len(packed_weights) <= 4:
        raise RuntimeError(f"mmq_multi takes 1 to 4 packed weights; got {len(packed_weights)}")
    if input.dtype != torch.bfloat16 or not input.is_contiguous() or input.storage_offset() != 0:
        raise RuntimeError("input must be a contiguous torch.bfloat16 tensor with zero storage offset; "
                           "torch_ggml_ops will not insert a hidden copy")
    k = input.shape[-1]
    rows = input.numel() // k
    expected = out_features * (k // 256) * native.lib().tgo_block_bytes(int(quant_type))
    for w in packed_weights:
        if w.dtype != torch.uint8 or not w.is_contiguous() or w.numel() != expected or w.device != input.device:
            raise RuntimeError(f"every packed_weight must be a contiguous torch.uint8 tensor of {expected} bytes on the input's device")
    outs = [input.new_empty((*input.shape[:-1], out_features)) for _ in packed_weights]
    with torch.cuda.device(input.device):
        native.mmq_fwd_multi(input, packed_weights, outs, rows, out_features, k, int(quant_type))
    return outs


@_mmq_multi.register_fake
def _(input, packed_weights, quant_type, out_features):
    return [input.new_empty((*input.shape[:-1], out_features)) for _ in packed_weights]


def _multi_setup(ctx, inputs, output):
    activation, packed_weights, quant_type, _ = inputs
    ctx.quant_type, ctx.in_features, ctx.n = quant_type, activation.shape[-1], len(packed_weights)
    if ctx.needs_input_grad[0]:
        ctx.save_for_backward(*packed_weights)


def _multi_dx(ctx, grads):
    no_weight_grads = [None] * ctx.n
    if not ctx.needs_input_grad[0]:
        return None, no_weight_grads, None, None
    total = None
    for g, w in zip(grads, ctx.saved_tensors):
        if g is None:
            continue
        dx = torch.ops.torch_ggml_ops.mmq_grad_input.default(g.contiguous(), w, ctx.quant_type, ctx.in_features)
        total = dx if total is None else total + dx
    return total, no_weight_grads, None, None


_mmq_multi.register_autograd(_multi_dx, setup_context=_multi_setup)


def mmq_multi(input: torch.Tensor, packed_weights, quant_type: int, out_features: int):
    """``[input @ W_i.T for W_i in packed_weights]`` (1 to 4 weights of one quant type and shape
    [out_features, in_features]) with two weight sets per kernel launch; every result is
    bit-identical to ``mmq`` on that weight alone."""
    return tuple(_mmq_multi(input, list(packed_weights), int(quant_type), int(out_features)))


# ------------------------------------------------------------------ silu(gate) * up
@torch.library.custom_op(f"{_NS}::swiglu", mutates_args=(), device_types="cuda")
def _swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    if gate.shape != up.shape or gate.dtype != torch.bfloat16 or up.dtype != torch.bfloat16:
        raise RuntimeError("gate and up must be torch.bfloat16 tensors of the same shape")
    g2, u2 = gate.contiguous().reshape(-1, gate.shape[-1]), up.contiguous().reshape(-1, up.shape[-1])
    out = torch.empty_like(g2)
    with torch.cuda.device(gate.device):
        native.swiglu_fwd(g2, u2, out)
    return out.reshape(gate.shape)


@_swiglu.register_fake
def _(gate, up):
    return torch.empty_like(gate)


@torch.library.custom_op(f"{_NS}::swiglu_grad", mutates_args=(), device_types="cuda")
def _swiglu_grad(grad: torch.Tensor, gate: torch.Tensor, up: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    g2, u2 = gate.contiguous().reshape(-1, gate.shape[-1]), up.contiguous().reshape(-1, up.shape[-1])
    d2 = grad.contiguous().reshape(-1, grad.shape[-1])
    dg, du = torch.empty_like(g2), torch.empty_like(g2)
    with torch.cuda.device(gate.device):
        native.swiglu_bwd(d2, g2, u2, dg, du)
    return dg.reshape(gate.shape), du.reshape(gate.shape)


@_swiglu_grad.register_fake
def _(grad, gate, up):
    return torch.empty_like(gate), torch.empty_like(gate)


def _swiglu_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs)


def _swiglu_backward(ctx, grad):
    gate, up = ctx.saved_tensors
    return _swiglu_grad(grad, gate, up)


_swiglu.register_autograd(_swiglu_backward, setup_context=_swiglu_setup)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` on bf16 tensors (fp32 arithmetic, one rounding), differentiable."""
    return _swiglu(gate, up)


def moe_mlp(input, gate_weight, up_weight, down_weight, expert_indices, expert_offsets, quant_type_gate_up: int,
            quant_type_down: int, ffn_features: int):
    """MoE feed-forward block over expert-sorted rows on one GPU:
    ``grouped_mmq(swiglu(*grouped_mmq_pair(x, Wg, Wu)), Wd)``; differentiable with respect to ``input``.
    ``gate_weight`` / ``up_weight``: [E, ffn, row bytes]; ``down_weight``: [E, hidden, row bytes]."""
    from .grouped_mmq import grouped_mmq, grouped_mmq_pair

    gate, up = grouped_mmq_pair(input, gate_weight, up_weight, expert_indices, expert_offsets, quant_type_gate_up, ffn_features)
    return grouped_mmq(swiglu(gate, up), down_weight, expert_indices, expert_offsets, quant_type_down, input.shape[-1])


# ------------------------------------------------------------------ chunked LM-head loss
def lm_head_loss(hidden: torch.Tensor, packed_weight: torch.Tensor, quant_type: int, vocab: int, targets: torch.Tensor,
                 chunk_rows: int = 256, grad_scale: float = 1.0):
    """Sum of the token cross entropies of ``softmax(hidden @ W.T)`` against ``targets`` and its
    gradient with respect to ``hidden``, computed over chunks of ``chunk_rows`` rows so that only
    one chunk of logits ([chunk_rows, vocab]) exists at a time.  Per chunk: ``mmq`` (bf16 logits)
    -> fp32 log-softmax and loss -> cotangent ``(softmax - onehot) * grad_scale`` in bf16 ->
    ``mmq_grad_input``.  Returns ``(loss_sum fp32 scalar tensor, d_hidden bf16 like hidden)``.

    The reference's production consumer runs this loop with chunk_rows = 256 for a Q6_K head of
    248320 x 2048 (docs/mmq_bwd_optimization.md:502-524); rows = hidden.numel() / K."""
    from .mmq import mmq

    k = hidden.shape[-1]
    h2 = hidden.reshape(-1, k)
    t1 = targets.reshape(-1)
    if t1.numel() != h2.shape[0]:
        raise ValueError("targets must have one entry per row of hidden")
    d_hidden = torch.empty_like(h2)
    loss = torch.zeros((), dtype=torch.float32, device=hidden.device)
    for b in range(0, h2.shape[0], chunk_rows):
        e = min(b + chunk_rows, h2.shape[0])
        # a chunk is a view with a storage offset: the operators take no hidden copies, so make it explicit
        logits = mmq(h2[b:e].clone(), packed_weight, quant_type, vocab).float()
        logp = torch.log_softmax(logits, dim=-1)
        loss += -logp.gather(1, t1[b:e, None].long()).sum()
        dlogits = torch.exp(logp)
        dlogits.scatter_add_(1, t1[b:e, None].long(), torch.full((e - b, 1), -1.0, device=hidden.device))
        if grad_scale != 1.0:
            dlogits *= grad_scale
        d_hidden[b:e] = torch.ops.torch_ggml_ops.mmq_grad_input.default(dlogits.to(torch.bfloat16), packed_weight,
                                                                      int(quant_type), k)
    return loss, d_hidden.reshape(hidden.shape)


__all__ = ["lm_head_loss", "mmq_multi", "moe_mlp", "swiglu"]
