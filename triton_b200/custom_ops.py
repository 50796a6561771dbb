"""PyTorch custom-op registration of the library's entry points.

`torch.ops.triton_b200.matmul`, `.attention_fwd`, `.attention_bwd` and the differentiable
`.attention` are registered with `torch.library.custom_op`: they show up in the dispatcher, have
fake (meta) implementations so that `torch.compile` / export can trace through them without
running a kernel, and `attention` carries its backward formula.  The CUDA implementations are the
functions of `triton_b200.ops`, i.e. the C ABI of include/triton_b200.h through ctypes; there is
no CPU implementation: on CPU tensors the ops raise, like the functions they wrap.
"""
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import ops

_lib_ns = "triton_b200"


@torch.library.custom_op(f"{_lib_ns}::matmul", mutates_args=(), device_types="cuda")
def matmul(a: Tensor, b: Tensor, activation: str = "", out_dtype: Optional[torch.dtype] = None,
           scale_a: Optional[Tensor] = None, scale_b: Optional[Tensor] = None,
           bias: Optional[Tensor] = None) -> Tensor:
    return ops.matmul(a, b, activation, scale_a=scale_a, scale_b=scale_b, out_dtype=out_dtype, bias=bias)


@matmul.register_fake
def _(a, b, activation="", out_dtype=None, scale_a=None, scale_b=None, bias=None):
    torch._check(a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[0], lambda: "Incompatible dimensions")
    if out_dtype is None:
        out_dtype = torch.float16 if a.dtype == torch.float16 else torch.bfloat16
    return a.new_empty((a.shape[0], b.shape[1]), dtype=out_dtype)


@torch.library.custom_op(f"{_lib_ns}::attention_fwd", mutates_args=(), device_types="cuda")
def attention_fwd(q: Tensor, k: Tensor, v: Tensor, causal: bool, sm_scale: float) -> Tuple[Tensor, Tensor]:
    return ops.attention_forward(q, k, v, causal, sm_scale)


@attention_fwd.register_fake
def _(q, k, v, causal, sm_scale):
    return torch.empty_like(q), q.new_empty(q.shape[:3], dtype=torch.float32)


@torch.library.custom_op(f"{_lib_ns}::attention_bwd", mutates_args=(), device_types="cuda")
def attention_bwd(q: Tensor, k: Tensor, v: Tensor, o: Tensor, M: Tensor, do: Tensor, causal: bool,
                  sm_scale: float) -> Tuple[Tensor, Tensor, Tensor]:
    return ops.attention_backward(q, k, v, o, M, do.contiguous(), causal, sm_scale)


@attention_bwd.register_fake
def _(q, k, v, o, M, do, causal, sm_scale):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


@torch.library.custom_op(f"{_lib_ns}::attention", mutates_args=(), device_types="cuda")
def attention(q: Tensor, k: Tensor, v: Tensor, causal: bool, sm_scale: float) -> Tuple[Tensor, Tensor]:
    """(O, M); differentiable with respect to q, k, v through O."""
    return ops.attention_forward(q, k, v, causal, sm_scale)


@attention.register_fake
def _(q, k, v, causal, sm_scale):
    return torch.empty_like(q), q.new_empty(q.shape[:3], dtype=torch.float32)


def _attention_setup(ctx, inputs, output):
    q, k, v, causal, sm_scale = inputs
    o, M = output
    ctx.save_for_backward(q, k, v, o, M)
    ctx.causal, ctx.sm_scale = causal, sm_scale


def _attention_backward(ctx, do, dM):
    q, k, v, o, M = ctx.saved_tensors
    dq, dk, dv = torch.ops.triton_b200.attention_bwd(q, k, v, o, M, do, ctx.causal, ctx.sm_scale)
    return dq, dk, dv, None, None


torch.library.register_autograd(f"{_lib_ns}::attention", _attention_backward, setup_context=_attention_setup)
