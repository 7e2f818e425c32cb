"""RMSNorm, fused with the residual addition that precedes it."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Part, register_norm


@dataclass
class Deferred:
    """A sub-layer's output that has not joined the residual stream yet because it is RMS-normed
    first (a norm AFTER the sub-layer): the next norm of the stream does both in one kernel,
    x += weight * value * rsqrt(mean(value^2) + eps), then its own norm of x."""
    value: torch.Tensor
    weight: torch.Tensor
    eps: float


@register_norm("rmsnorm")
class RMSNorm(Part):
    """y = weight * round(x * rsqrt(mean(x^2) + eps)), statistics in 32-bit (layover/model.py:25-36).

    params: dim, eps, weight (tensor name relative to the prefix).
    `forward(x, delta)` first adds `delta` into `x` (the residual sum, in 32-bit, rounded once)
    so that a block never launches a separate addition.

    Two more forms, both for models that keep the residual stream in 32-bit floats whatever the
    run's type: `delta` may be a `Deferred` (what `defer(value)` of the norm that FOLLOWS a sub-layer
    returns: its output is normed, then added), and `extra` is one more 32-bit tensor to add (the
    embedding output, between the passes of layers that run several times). These take the
    32-bit-stream kernel, which rounds once, at the output; `add(x, delta, extra)` is the same
    without a norm of the sum."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("dim", "eps", "weight")
        self.dim, self.eps = int(params["dim"]), float(params["eps"])
        self.weight_name = prefix + params["weight"]
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.dim,), kind="vector", init="ones")]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.weight_name]

    def kernel_libraries(self, dtype):
        return ("elementwise",)

    def defer(self, value: torch.Tensor) -> Deferred:
        """`value` as something this norm is to be applied to when it is added to the stream."""
        return Deferred(value, self.weight, self.eps)

    def forward(self, x: torch.Tensor, delta, rows: torch.Tensor | None = None,
                extra: torch.Tensor | None = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.shape[0]
        wide = x.dtype == torch.float32 and self.runtime.dtype != torch.float32
        if not (wide or isinstance(delta, Deferred) or extra is not None):
            out = torch.empty((n, self.dim), dtype=x.dtype, device=x.device)
            return ops.add_rmsnorm(x, delta, self.weight, self.eps, out, rows)
        out = torch.empty((n, self.dim), dtype=self.runtime.dtype, device=x.device)
        value, weight, eps = (delta.value, delta.weight, delta.eps) if isinstance(delta, Deferred) else (delta, None, 0.0)
        return ops.residual_rmsnorm(x, value, weight, eps, extra, self.weight, self.eps, out, rows)

    @staticmethod
    def add(x: torch.Tensor, delta, extra: torch.Tensor | None = None) -> torch.Tensor:
        """x += delta (normed first if it is a `Deferred`) (+ extra), no norm of the sum: the stream itself."""
        value, weight, eps = (delta.value, delta.weight, delta.eps) if isinstance(delta, Deferred) else (delta, None, 0.0)
        if value is not None or extra is not None:
            ops.residual_rmsnorm(x, value, weight, eps, extra, None, 0.0, None)
        return x
