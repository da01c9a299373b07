"""Grouped (mixture-of-experts) packed-weight matmul and the fused gate/up pair: Python surface of
``torch_ggml_ops::grouped_mmq`` and ``torch_ggml_ops::grouped_mmq_pair``.

Same contract as the reference (torch_ggml_ops/grouped_mmq.py:4-250).  Rows are pre-sorted by
expert; ``expert_indices`` (int64) names the expert of each group and ``expert_offsets`` (int32)
the cumulative end row of each group; both stay on the device.  Backward of the pair has three
cases: both cotangents present -> one fused ``grouped_mmq_pair_grad_input`` (the two Jacobian
products are summed in fp32 before one bf16 rounding); only one present -> the single-projection
``grouped_mmq_grad_input`` with that projection's weight.
"""
import torch

from .mmq import _NS, _no_double_backward


def _rows_by(like: torch.Tensor, width: int) -> torch.Tensor:
    return like.new_empty((like.shape[0], width))


@torch.library.register_fake(f"{_NS}::grouped_mmq")
def _(input, packed_weight, expert_indices, expert_offsets, quant_type, out_features):
    return _rows_by(input, out_features)


@torch.library.register_fake(f"{_NS}::grouped_mmq_grad_input")
def _(grad_output, packed_weight, expert_indices, expert_offsets, quant_type, in_features):
    return _rows_by(grad_output, in_features)


@torch.library.register_fake(f"{_NS}::grouped_mmq_pair")
def _(input, first_packed_weight, second_packed_weight, expert_indices, expert_offsets, quant_type, out_features):
    return _rows_by(input, out_features), _rows_by(input, out_features)


@torch.library.register_fake(f"{_NS}::grouped_mmq_pair_grad_input")
def _(first_grad_output, second_grad_output, first_packed_weight, second_packed_weight, expert_indices,
      expert_offsets, quant_type, in_features):
    return _rows_by(first_grad_output, in_features)


def _single_dx(grad_output, packed_weight, expert_indices, expert_offsets, quant_type, in_features):
    return torch.ops.torch_ggml_ops.grouped_mmq_grad_input.default(
        grad_output.contiguous(), packed_weight, expert_indices, expert_offsets, quant_type, in_features)


# ---------------------------------------------------------------- grouped_mmq
def _save_single(ctx, inputs, output) -> None:
    activation, packed_weight, expert_indices, expert_offsets, quant_type, _ = inputs
    ctx.quant_type = quant_type
    ctx.in_features = activation.shape[1]
    if ctx.needs_input_grad[0]:
        ctx.save_for_backward(packed_weight, expert_indices, expert_offsets)


def _single_backward(ctx, grad_output):
    grad_input = None
    if ctx.needs_input_grad[0]:
        grad_input = _single_dx(grad_output, *ctx.saved_tensors, ctx.quant_type, ctx.in_features)
    return (grad_input,) + (None,) * 5


torch.library.register_autograd(f"{_NS}::grouped_mmq", _single_backward, setup_context=_save_single)


# ---------------------------------------------------------------- grouped_mmq_pair
def _save_pair(ctx, inputs, output) -> None:
    activation, first_weight, second_weight, expert_indices, expert_offsets, quant_type, _ = inputs
    ctx.quant_type = quant_type
    ctx.in_features = activation.shape[1]
    if ctx.needs_input_grad[0]:
        ctx.save_for_backward(first_weight, second_weight, expert_indices, expert_offsets)


def _pair_backward(ctx, first_grad, second_grad):
    grad_input = None
    if ctx.needs_input_grad[0]:
        first_weight, second_weight, expert_indices, expert_offsets = ctx.saved_tensors
        routing = (expert_indices, expert_offsets, ctx.quant_type, ctx.in_features)
        if first_grad is not None and second_grad is not None:
            grad_input = torch.ops.torch_ggml_ops.grouped_mmq_pair_grad_input.default(
                first_grad.contiguous(), second_grad.contiguous(), first_weight, second_weight, *routing)
        elif first_grad is not None:
            grad_input = _single_dx(first_grad, first_weight, *routing)
        elif second_grad is not None:
            grad_input = _single_dx(second_grad, second_weight, *routing)
    return (grad_input,) + (None,) * 6


torch.library.register_autograd(f"{_NS}::grouped_mmq_pair", _pair_backward, setup_context=_save_pair)

for _name in ("grouped_mmq_grad_input", "grouped_mmq_pair_grad_input"):
    torch.library.register_autograd(f"{_NS}::{_name}", _no_double_backward(_name))


def grouped_mmq(input, packed_weight, expert_indices, expert_offsets, quant_type: int, out_features: int):
    """Per-group ``input[rows_g] @ W[expert_g].T`` over expert-sorted bf16 rows."""
    return torch.ops.torch_ggml_ops.grouped_mmq.default(
        input, packed_weight, expert_indices, expert_offsets, int(quant_type), int(out_features))


def grouped_mmq_pair(input, first_packed_weight, second_packed_weight, expert_indices, expert_offsets,
                     quant_type: int, out_features: int):
    """Gate and up projections of the same rows in one launch: ``(x @ W1[e].T, x @ W2[e].T)``."""
    return torch.ops.torch_ggml_ops.grouped_mmq_pair.default(
        input, first_packed_weight, second_packed_weight, expert_indices, expert_offsets,
        int(quant_type), int(out_features))


__all__ = ["grouped_mmq", "grouped_mmq_pair"]
