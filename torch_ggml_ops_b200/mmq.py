"""Dense packed-weight matmul: Python surface of ``torch_ggml_ops::mmq``.

Same contract as the reference (torch_ggml_ops/mmq.py:4-80): a fake (meta) kernel per operator so
the ops trace under ``torch.compile``; an autograd formula for ``mmq`` that saves only the packed
weight and calls ``mmq_grad_input`` on a contiguous cotangent; and a guard that makes second-order
differentiation of ``mmq_grad_input`` an error.  The packed weight never receives a gradient.
"""
import torch

_NS = "torch_ggml_ops"


def _swap_last_dim(like: torch.Tensor, width: int) -> torch.Tensor:
    return like.new_empty((*like.shape[:-1], width))


@torch.library.register_fake(f"{_NS}::mmq")
def _(input, packed_weight, quant_type, out_features):
    return _swap_last_dim(input, out_features)


@torch.library.register_fake(f"{_NS}::mmq_grad_input")
def _(grad_output, packed_weight, quant_type, in_features):
    return _swap_last_dim(grad_output, in_features)


def _save_for_dx(ctx, inputs, output) -> None:
    activation, packed_weight, quant_type, _ = inputs
    ctx.quant_type = quant_type
    ctx.in_features = activation.shape[-1]
    if ctx.needs_input_grad[0]:
        ctx.save_for_backward(packed_weight)


def _dx(ctx, grad_output):
    if not ctx.needs_input_grad[0]:
        return None, None, None, None
    (packed_weight,) = ctx.saved_tensors
    # The native operator refuses non-contiguous tensors; a cotangent handed over by autograd
    # may be a transposed view, so only this autograd-owned temporary is normalised.
    grad_input = torch.ops.torch_ggml_ops.mmq_grad_input.default(
        grad_output.contiguous(), packed_weight, ctx.quant_type, ctx.in_features)
    return grad_input, None, None, None


torch.library.register_autograd(f"{_NS}::mmq", _dx, setup_context=_save_for_dx)


def _no_double_backward(name: str):
    def backward(ctx, *grads):
        raise RuntimeError(f"{_NS}::{name} does not support higher-order gradients")

    return backward


torch.library.register_autograd(f"{_NS}::mmq_grad_input", _no_double_backward("mmq_grad_input"))


def mmq(input: torch.Tensor, packed_weight: torch.Tensor, quant_type: int, out_features: int) -> torch.Tensor:
    """``input[..., K] @ W[N, K].T`` with ``W`` given as raw GGUF super-blocks (uint8).

    bf16 in, bf16 out; ``quant_type`` is the GGML type id (IQ2_S, Q3_K, Q4_K, Q5_K, Q6_K)."""
    return torch.ops.torch_ggml_ops.mmq.default(input, packed_weight, int(quant_type), int(out_features))


__all__ = ["mmq"]
