"""Hyper-connections: several copies of the residual stream that a layer's sublayers read and write through small
stored maps, in place of the one stream and its plain sum.

With S copies x_1 .. x_S (all equal to the embedding's output at the start; a token's copies lie side by side in the
float32 stream [T, S W]) and, for a sublayer, vectors a, b [S] and a matrix M [S, S] indexed [from, to]:

    u   = sum_s a[s] x_s                      the sublayer's input, before its norm
    y   = sublayer(N(u))                      N: RMS norm with weight offset + w
    x_k <- sum_s M[s, k] x_s + b[k] y         all k at once from the old copies

`HyperRead` is the read with its norm, as a `Norm` (so that the block before can apply it together with its own last
write, and so that the model's final norm, a read with a = 1, sums the copies).  `HyperConnectionBlock` is a layer:
mixer, then optionally a feed-forward, each between its read and its write.  The copies, the maps and the norm are
float32 whatever the activations are.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Block, FeedForward, Mixer, Norm, Runtime, StepContext


class HyperRead(Norm):
    """out = N(sum_s a[s] x_s).  `in_name` None: a = 1, the plain sum of the copies."""

    def __init__(self, width: int, copies: int, eps: float, weight_name: str, in_name: str | None = None,
                 offset: float = 0.0, init_std: float = 0.1, init_mean: float = 0.0):
        if copies < 1:
            raise ValueError(f"a stream has at least one copy, found {copies}")
        self.width, self.copies, self.eps, self.offset = width, int(copies), float(eps), float(offset)
        self.weight_name, self.in_name = weight_name, in_name
        self.init_std, self.init_mean = init_std, init_mean
        self.weight = self.a = None          # float32

    def tensor_specs(self):
        specs = {self.weight_name: TensorSpec((self.width,), init_std=self.init_std, init_mean=self.init_mean)}
        if self.in_name is not None:
            specs[self.in_name] = TensorSpec((self.copies,), init_std=0.1, init_mean=1.0 / self.copies)
        return specs

    def load(self, store, rt: Runtime):
        self.weight = (store.get(self.weight_name).to(torch.float32) + self.offset).contiguous()
        self.a = store.get(self.in_name).to(torch.float32).contiguous() if self.in_name is not None else None

    def forward(self, x, ctx: StepContext, out, rows=None):
        return ctx.rt.ops.hc_read_norm(x, self.copies, self.a, self.weight, self.eps, out, rows)

    def residual_add(self, h, r, ctx: StepContext, next_norm: Norm | None = None, out=None):
        raise NotImplementedError("a read of the copies stands before a sublayer, not after one")


class HyperConnectionBlock(Block):
    """names: "mix1", "out1" (the mixer's write) and, with a feed-forward, "mix2", "out2"."""

    def __init__(self, mixer: Mixer, feed_forward: FeedForward | None, mixer_read: HyperRead, ff_read: HyperRead | None,
                 names: dict[str, str]):
        if feed_forward is not None and ff_read is None:
            raise ValueError("a block with a feed-forward needs the read before it")
        for k in ("mix1", "out1") + (("mix2", "out2") if feed_forward is not None else ()):
            if k not in names:
                raise ValueError(f"a hyper-connection block needs the checkpoint name of its {k!r} tensor")
        self.mixer, self.feed_forward = mixer, feed_forward
        self.first_norm, self.ff_read = mixer_read, ff_read
        self.copies, self.width = mixer_read.copies, mixer_read.width
        self.names = dict(names)
        self.maps: dict[str, torch.Tensor] = {}

    def sub_parts(self):
        if self.feed_forward is None:
            return [self.first_norm, self.mixer]
        return [self.first_norm, self.mixer, self.ff_read, self.feed_forward]

    def tensor_specs(self):
        S = self.copies
        specs = {}
        for q in ("1", "2") if self.feed_forward is not None else ("1",):
            specs[self.names["mix" + q]] = TensorSpec((S, S), init_std=0.1, init_mean=1.0 / S)
            specs[self.names["out" + q]] = TensorSpec((S,), init_std=0.1, init_mean=1.0)
        return specs

    def load(self, store, rt: Runtime):
        for k, name in self.names.items():
            if k in ("mix1", "out1") or self.feed_forward is not None:
                self.maps[k] = store.get(name).to(torch.float32).contiguous()

    def _write(self, h, r, q: str, ctx: StepContext, next_norm: Norm | None):
        """The sublayer's write and, in the same pass where it is a read of the copies, what stands before the next one."""
        ops, M, b = ctx.rt.ops, self.maps["mix" + q], self.maps["out" + q]
        if next_norm is None:
            ops.hc_update(h, r, self.copies, M, b)
            return None
        y = ctx.ws.buf("block.y", (h.shape[0], self.width), ctx.rt.dtype)
        if isinstance(next_norm, HyperRead) and next_norm.copies == self.copies and next_norm.a is not None:
            return ops.hc_update(h, r, self.copies, M, b, next_norm.a, next_norm.weight, next_norm.eps, y)
        ops.hc_update(h, r, self.copies, M, b)
        return next_norm.forward(h, ctx, y)

    def forward(self, h, ctx: StepContext, line, y_in=None, next_norm: Norm | None = None):
        y = y_in if y_in is not None else self.first_norm.forward(
            h, ctx, ctx.ws.buf("block.y", (h.shape[0], self.width), ctx.rt.dtype))
        r = self.mixer.forward(y, ctx, line)
        if self.feed_forward is None:
            return h, self._write(h, r, "1", ctx, next_norm)
        y = self._write(h, r, "1", ctx, self.ff_read)
        r = self.feed_forward.forward(y, ctx)
        return h, self._write(h, r, "2", ctx, next_norm)
