"""Arrangements of a mixer, a feed-forward and norms around the residual stream.

`SandwichBlock` is Gemma2's (`gemma/gemma.go:162-167`): a norm before and a
norm after each sublayer, the second applied to the sublayer's output before it
is added:  r = Mixer(N_in(x)); h = x + N_post_mixer(r); r = FF(N_pre_ff(h));
out = h + N_post_ff(r).  Without a feed-forward (`feed_forward=None`) a layer is the first line alone.

`PreNormBlock` is the usual arrangement without the norms after the sublayers
(`qwen/block.go:58-61`): h = x + Mixer(N_in(x)); out = h + FF(N_pre_ff(h)); without a feed-forward the first
line alone.

`PostNormBlock` norms after the sum, and the stream that goes on is the normed one: x <- N1(a x + Mixer(x));
x <- N2(a x + FF(x)) with a constant a; the sublayers read the stream itself (rounded to the activation type).
Without a feed-forward the first line alone.

The residual stream is float32 and is updated in place.  A block may be handed
its first norm's output (computed by the block before it together with that
block's last residual sum) and may be asked to apply the next block's first
norm to its own result, which saves a pass over the stream per layer.
"""
from __future__ import annotations

from .base import Block, FeedForward, Mixer, Norm, StepContext
from .norm import plain_residual_add

import torch


class SandwichBlock(Block):
    def __init__(self, mixer: Mixer, feed_forward: FeedForward | None, input_norm: Norm, post_mixer_norm: Norm,
                 pre_ff_norm: Norm | None = None, post_ff_norm: Norm | None = None):
        if feed_forward is not None and (pre_ff_norm is None or post_ff_norm is None):
            raise ValueError("a block with a feed-forward needs the norms before and after it")
        self.mixer, self.feed_forward = mixer, feed_forward
        self.first_norm = input_norm
        self.post_mixer_norm, self.pre_ff_norm, self.post_ff_norm = post_mixer_norm, pre_ff_norm, post_ff_norm

    def sub_parts(self):
        if self.feed_forward is None:
            return [self.first_norm, self.mixer, self.post_mixer_norm]
        return [self.first_norm, self.mixer, self.post_mixer_norm, self.pre_ff_norm, self.feed_forward,
                self.post_ff_norm]

    def forward(self, h, ctx: StepContext, line, y_in=None, next_norm: Norm | None = None):
        T, H = h.shape
        dt = ctx.rt.dtype
        y = y_in if y_in is not None else self.first_norm.forward(h, ctx, ctx.ws.buf("block.y", (T, H), dt))
        r = self.mixer.forward(y, ctx, line)
        if self.feed_forward is None:
            return h, self.post_mixer_norm.residual_add(h, r, ctx, next_norm, ctx.ws.buf("block.y", (T, H), dt)
                                                        if next_norm is not None else None)
        y = self.post_mixer_norm.residual_add(h, r, ctx, self.pre_ff_norm, ctx.ws.buf("block.y", (T, H), dt))
        r = self.feed_forward.forward(y, ctx)
        y_next = self.post_ff_norm.residual_add(h, r, ctx, next_norm,
                                                ctx.ws.buf("block.y", (T, H), dt) if next_norm is not None else None)
        return h, y_next


class PreNormBlock(Block):
    def __init__(self, mixer: Mixer, feed_forward: FeedForward | None, input_norm: Norm, pre_ff_norm: Norm | None = None):
        if feed_forward is not None and pre_ff_norm is None:
            raise ValueError("a block with a feed-forward needs the norm before it")
        self.mixer, self.feed_forward = mixer, feed_forward
        self.first_norm = input_norm
        self.pre_ff_norm = pre_ff_norm

    def sub_parts(self):
        if self.feed_forward is None:
            return [self.first_norm, self.mixer]
        return [self.first_norm, self.mixer, self.pre_ff_norm, self.feed_forward]

    def forward(self, h, ctx: StepContext, line, y_in=None, next_norm: Norm | None = None):
        T, H = h.shape
        dt = ctx.rt.dtype
        y = y_in if y_in is not None else self.first_norm.forward(h, ctx, ctx.ws.buf("block.y", (T, H), dt))
        r = self.mixer.forward(y, ctx, line)
        if self.feed_forward is None:
            return h, plain_residual_add(h, r, ctx, next_norm,
                                         ctx.ws.buf("block.y", (T, H), dt) if next_norm is not None else None)
        y = plain_residual_add(h, r, ctx, self.pre_ff_norm, ctx.ws.buf("block.y", (T, H), dt))
        r = self.feed_forward.forward(y, ctx)
        y_next = plain_residual_add(h, r, ctx, next_norm,
                                    ctx.ws.buf("block.y", (T, H), dt) if next_norm is not None else None)
        return h, y_next


class StreamItself(Norm):
    """What stands before a sublayer that reads the stream as it is: the row rounded to the activation type."""

    def forward(self, x, ctx: StepContext, out, rows=None):
        if rows is not None:
            raise NotImplementedError("the stream itself is read row by row, not gathered")
        if out.dtype == torch.float32:
            return x
        return ctx.rt.ops.round_rows(x, out)


class PostNormBlock(Block):
    def __init__(self, mixer: Mixer, feed_forward: FeedForward | None, post_mixer_norm: Norm, post_ff_norm: Norm | None = None,
                 alpha: float = 1.0):
        if feed_forward is not None and post_ff_norm is None:
            raise ValueError("a block with a feed-forward needs the norm after it")
        for n in (post_mixer_norm, post_ff_norm):
            if n is not None and not hasattr(n, "scaled_add"):
                raise ValueError("a block that norms after the sum needs norms that can norm the stream in place")
        self.mixer, self.feed_forward = mixer, feed_forward
        self.first_norm = StreamItself()
        self.post_mixer_norm, self.post_ff_norm = post_mixer_norm, post_ff_norm
        self.alpha = float(alpha)

    def sub_parts(self):
        if self.feed_forward is None:
            return [self.mixer, self.post_mixer_norm]
        return [self.mixer, self.post_mixer_norm, self.feed_forward, self.post_ff_norm]

    def _out(self, h, ctx):
        # (in the 32-bit path the sublayers read the stream's own rows)
        return None if ctx.rt.dtype == torch.float32 else ctx.ws.buf("block.y", tuple(h.shape), ctx.rt.dtype)

    def forward(self, h, ctx: StepContext, line, y_in=None, next_norm: Norm | None = None):
        y = y_in if y_in is not None else self.first_norm.forward(h, ctx, self._out(h, ctx) if self._out(h, ctx) is not None else h)
        r = self.mixer.forward(y, ctx, line)
        y = self.post_mixer_norm.scaled_add(h, r, self.alpha, ctx, self._out(h, ctx))
        if self.feed_forward is not None:
            r = self.feed_forward.forward(y if y is not None else h, ctx)
            y = self.post_ff_norm.scaled_add(h, r, self.alpha, ctx, self._out(h, ctx))
        if next_norm is None:
            return h, None
        if isinstance(next_norm, StreamItself):
            return h, (y if y is not None else h)
        return h, next_norm.forward(h, ctx, ctx.ws.buf("block.y", tuple(h.shape), ctx.rt.dtype))
