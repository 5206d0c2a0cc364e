"""Norms of the residual stream: RMS norm with a weight offset, Dynamic Tanh, and the RMS norm in groups.

y = x / sqrt(mean(x^2) + eps) * (offset + w).  Gemma2 stores w and uses 1 + w
(`gemma/gemma.go:22-28`); offset 0 is the usual RMS norm (`qwen/norm.go:10-27`).
eps lies inside the root, added to the mean (`cpu/cpu_ops.go:145-162`).  The
sum of squares, the root and offset + w are float32 whatever the model's dtype.

`DynamicTanh` takes no statistics of the row: y = tanh(alpha x) * w + b with a stored scalar alpha and vectors w
and b, element by element, in float32.

`GroupRMSNorm` cuts the row into `groups` equal runs and divides each by its own sqrt(mean(run^2) + eps) before the
whole is multiplied by w.  It can norm the stream itself after a scaled residual sum (`scaled_add`: h <- N(a h + r)),
which is what a block that norms after the sum needs.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Norm, Runtime, StepContext


class RMSNorm(Norm):
    def __init__(self, width: int, eps: float, weight_name: str, offset: float = 0.0, init_std: float = 0.1,
                 init_mean: float = 0.0):
        self.width = width
        self.eps = float(eps)
        self.offset = float(offset)
        self.weight_name = weight_name
        self.init_std, self.init_mean = init_std, init_mean      # how random weights are drawn
        self.weight = None          # float32: offset + w

    def tensor_specs(self):
        return {self.weight_name: TensorSpec((self.width,), init_std=self.init_std, init_mean=self.init_mean)}

    def load(self, store, rt: Runtime):
        self.weight = (store.get(self.weight_name).to(torch.float32) + self.offset).contiguous()

    def forward(self, x, ctx: StepContext, out, rows=None):
        return ctx.rt.ops.rmsnorm(x, self.weight, self.eps, out, rows)

    def residual_add(self, h, r, ctx: StepContext, next_norm: Norm | None = None, out=None):
        """h += self(r); out = next_norm(h) when a next norm is given."""
        if next_norm is None:
            ctx.rt.ops.add_rmsnorm(h, r, self.weight, self.eps)
            return None
        if isinstance(next_norm, RMSNorm):
            return ctx.rt.ops.add_rmsnorm(h, r, self.weight, self.eps, next_norm.weight, next_norm.eps, out)
        ctx.rt.ops.add_rmsnorm(h, r, self.weight, self.eps)
        return next_norm.forward(h, ctx, out)


class DynamicTanh(Norm):
    """y = tanh(alpha x) * w + b.  Tensors: `weight_name` [width], `<weight_name>.b` [width], `<weight_name>.alpha` []
    (other names through `bias_name` and `alpha_name`)."""

    def __init__(self, width: int, weight_name: str, bias_name: str | None = None, alpha_name: str | None = None,
                 init_std: float = 0.1, init_mean: float = 1.0, init_alpha: float = 0.5):
        self.width = width
        self.weight_name = weight_name
        self.bias_name = bias_name or weight_name + ".b"
        self.alpha_name = alpha_name or weight_name + ".alpha"
        self.init_std, self.init_mean, self.init_alpha = init_std, init_mean, init_alpha
        self.weight = self.bias = None      # float32
        self.alpha = 0.0

    def tensor_specs(self):
        return {self.weight_name: TensorSpec((self.width,), init_std=self.init_std, init_mean=self.init_mean),
                self.bias_name: TensorSpec((self.width,), init_std=self.init_std),
                self.alpha_name: TensorSpec((), init_std=0.1 * self.init_alpha, init_mean=self.init_alpha)}

    def load(self, store, rt: Runtime):
        self.weight = store.get(self.weight_name).to(torch.float32).contiguous()
        self.bias = store.get(self.bias_name).to(torch.float32).contiguous()
        self.alpha = float(store.get(self.alpha_name).to(torch.float32).reshape(()).item())

    def forward(self, x, ctx: StepContext, out, rows=None):
        return ctx.rt.ops.dyt_norm(x, None, self.alpha, self.weight, self.bias, out, rows)

    def after_add(self, h, r, ctx: StepContext, out):
        """h += r and out = self(h) in one pass over the stream."""
        return ctx.rt.ops.dyt_norm(h, r, self.alpha, self.weight, self.bias, out)

    def residual_add(self, h, r, ctx: StepContext, next_norm: Norm | None = None, out=None):
        raise NotImplementedError("Dynamic Tanh stands before a sublayer, not after one")


class GroupRMSNorm(Norm):
    def __init__(self, width: int, eps: float, groups: int, weight_name: str, init_std: float = 0.1, init_mean: float = 1.0):
        if groups < 1 or width % groups:
            raise ValueError(f"{groups} groups do not divide a width of {width}")
        self.width, self.eps, self.groups = width, float(eps), int(groups)
        self.weight_name = weight_name
        self.init_std, self.init_mean = init_std, init_mean
        self.weight = None          # float32

    def tensor_specs(self):
        return {self.weight_name: TensorSpec((self.width,), init_std=self.init_std, init_mean=self.init_mean)}

    def load(self, store, rt: Runtime):
        self.weight = store.get(self.weight_name).to(torch.float32).contiguous()

    def forward(self, x, ctx: StepContext, out, rows=None):
        return ctx.rt.ops.group_norm(x, None, 1.0, self.weight, self.eps, self.groups, out, rows)

    def scaled_add(self, h, r, alpha: float, ctx: StepContext, out=None):
        """h <- self(alpha h + r) on the float32 stream in place; out (when given) = the new h in the activation type."""
        return ctx.rt.ops.group_norm(h, r, alpha, self.weight, self.eps, self.groups, out)

    def residual_add(self, h, r, ctx: StepContext, next_norm: Norm | None = None, out=None):
        raise NotImplementedError("the norm in groups norms the stream itself (scaled_add), not a sublayer's output")


def plain_residual_add(h, r, ctx: StepContext, next_norm: Norm | None = None, out=None):
    """h += r for blocks without a norm after the sublayer; out = next_norm(h) when given."""
    if isinstance(next_norm, RMSNorm):
        return ctx.rt.ops.add_rmsnorm(h, r, None, 0.0, next_norm.weight, next_norm.eps, out)
    if hasattr(next_norm, "after_add"):
        return next_norm.after_add(h, r, ctx, out)
    ctx.rt.ops.add_rmsnorm(h, r, None, 0.0)
    return next_norm.forward(h, ctx, out) if next_norm is not None else None
