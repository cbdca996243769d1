"""``torch.library`` registration of the three operators.

The reference exposes a raw pybind function (csrc/hadamard_transform.cpp:72-81);
callers that trace or compile their model need real dispatcher ops with
fake-tensor (meta) functions, and training code needs a backward.  Registered
under the ``b200ht`` namespace:

* ``torch.ops.b200ht.hadamard_transform(x, scale)``  — out of place; autograd:
  H is symmetric, so the gradient is the same transform of the incoming gradient.
* ``torch.ops.b200ht.fused_ht_gemm(X, W, scale, token_major, out_bf16)``
* ``torch.ops.b200ht.fused_ht_gemv(W, X, scale, out_bf16)``

All three run the CUDA library; there is no CPU kernel behind them.
"""
from __future__ import annotations

import torch

from . import ops


@torch.library.custom_op("b200ht::hadamard_transform", mutates_args=(), device_types="cuda")
def hadamard_transform_op(x: torch.Tensor, scale: float) -> torch.Tensor:
    return ops.hadamard_transform(x, inplace=False, scale=scale)


@hadamard_transform_op.register_fake
def _(x, scale):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


def _ht_backward(ctx, grad):
    return torch.ops.b200ht.hadamard_transform(grad.contiguous(), ctx.scale), None


def _ht_setup(ctx, inputs, output):
    ctx.scale = inputs[1]


hadamard_transform_op.register_autograd(_ht_backward, setup_context=_ht_setup)


@torch.library.custom_op("b200ht::fused_ht_gemm", mutates_args=(), device_types="cuda")
def fused_ht_gemm_op(X: torch.Tensor, W: torch.Tensor, scale: float, token_major: bool, out_bf16: bool) -> torch.Tensor:
    return ops.fused_ht_gemm(X, W, scale=scale, out_layout="nm" if token_major else "mn",
                             out_dtype=torch.bfloat16 if out_bf16 else torch.float32)


@fused_ht_gemm_op.register_fake
def _(X, W, scale, token_major, out_bf16):
    n, m = X.shape[0], W.shape[0]
    return X.new_empty((n, m) if token_major else (m, n), dtype=torch.bfloat16 if out_bf16 else torch.float32)


@torch.library.custom_op("b200ht::fused_ht_gemv", mutates_args=(), device_types="cuda")
def fused_ht_gemv_op(W: torch.Tensor, X: torch.Tensor, scale: float, out_bf16: bool) -> torch.Tensor:
    return ops.fused_ht_gemv(W, X, scale=scale, out_dtype=torch.bfloat16 if out_bf16 else torch.float32)


@fused_ht_gemv_op.register_fake
def _(W, X, scale, out_bf16):
    return W.new_empty((W.shape[0], X.shape[1]), dtype=torch.bfloat16 if out_bf16 else torch.float32)
