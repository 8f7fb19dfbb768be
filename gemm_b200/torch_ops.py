"""`torch.library` registration of the operator: ``torch.ops.neogemm.linear(x, w)`` and the
out-variant ``torch.ops.neogemm.linear_out(x, w, out)``.

The reference exposes one in-place, column-major, default-stream function (nemgemmV03.cu:343,383).
Its layout is already that of ``torch.nn.Linear`` without bias - y = x @ W^T with W stored [N, K]
(benchmark.py:10-11,18) - so the same kernel serves as a module drop-in for the decode-shaped
MLP projections.  Registering it as a custom op gives it a fake (meta) implementation, so shape
inference and tracing tools see through it; the real implementation calls the C ABI on torch's
current stream.  There is no CPU implementation: calling it with CPU tensors raises.
"""
from __future__ import annotations

import torch

from . import ops as _ops

_LIB_NAME = "neogemm"


def _check(x: torch.Tensor, weight: torch.Tensor) -> None:
    if x.dim() < 1 or weight.dim() != 2:
        raise ValueError("linear expects x[..., K] and weight[N, K]")
    if x.shape[-1] != weight.shape[1]:
        raise ValueError(f"K mismatch: x has {x.shape[-1]}, weight has {weight.shape[1]}")
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise TypeError("linear expects bfloat16 tensors")


@torch.library.custom_op(f"{_LIB_NAME}::linear", mutates_args=())
def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    _check(x, weight)
    return _ops.linear(x, weight)


@linear.register_fake
def _(x, weight):
    _check(x, weight)
    return x.new_empty((*x.shape[:-1], weight.shape[0]))


@torch.library.custom_op(f"{_LIB_NAME}::linear_out", mutates_args=("out",))
def linear_out(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    _check(x, weight)
    x2 = x.reshape(-1, x.shape[-1])
    if x2.size(1) > 1 and x2.stride(1) != 1:
        x2 = x2.contiguous()
    out2 = out.view(-1, weight.shape[0])
    _ops.matmul(x2, weight, out=out2)


@linear_out.register_fake
def _(x, weight, out):
    _check(x, weight)
    if tuple(out.shape) != (*x.shape[:-1], weight.shape[0]):
        raise ValueError("out has the wrong shape")
    return None


class NeoLinear(torch.nn.Module):
    """Bias-free ``nn.Linear`` whose forward is the B200 kernel (inference only: no autograd
    formula is registered)."""

    def __init__(self, in_features: int, out_features: int, device=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = torch.nn.Parameter(
            torch.empty(out_features, in_features, dtype=torch.bfloat16, device=device),
            requires_grad=False)
        torch.nn.init.normal_(self.weight, std=in_features ** -0.5)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.ops.neogemm.linear(x, self.weight)
