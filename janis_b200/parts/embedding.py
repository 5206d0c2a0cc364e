"""Token embedding into the float32 residual stream, and the output head.

Gemma2 scales the embedding by sqrt(hidden), a float32 constant
(`gemma/gemma.go:193`, `:197`), ties the head to the embedding table
(`gemma/gemma.go:210`, `qwen/embed.go:87-89`) and caps the logits with
fc * tanh(logits / fc) (`gemma/gemma.go:211-212`).  Logits are float32.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Part, Runtime, StepContext


class Embedding(Part):
    def __init__(self, vocab: int, hidden: int, table_name: str, scale: float = 1.0, init_std: float = 0.02,
                 round_scale: bool = True, copies: int = 1):
        self.vocab, self.hidden = vocab, hidden
        self.copies = int(copies)               # the stream holds this many copies of every row, side by side
        self.stream_width = hidden * self.copies
        self.table_name = table_name
        self.scale = float(scale)
        self.round_scale = bool(round_scale)    # False: the constant multiplies as a float32 whatever the activations are
        self.init_std = init_std
        self.table = None
        self.scale_used = self.scale

    def tensor_specs(self):
        return {self.table_name: TensorSpec((self.vocab, self.hidden), init_std=self.init_std)}

    def load(self, store, rt: Runtime):
        self.table = store.get(self.table_name, rt.dtype).contiguous()
        # the reference casts the scalar to the activation dtype before the multiply (`mlxc/mlxc.go:587-601`):
        # in bfloat16 sqrt(2304) = 48 stays exact, sqrt(3584) = 59.87 becomes 59.75
        self.scale_used = float(torch.tensor(self.scale, dtype=torch.float32).to(rt.dtype if self.round_scale else torch.float32))

    def forward(self, tokens, ctx: StepContext, out):
        if self.copies == 1:
            return ctx.rt.ops.embed(tokens, self.table, self.scale_used, out)
        x = ctx.rt.ops.embed(tokens, self.table, self.scale_used,
                             ctx.ws.buf("embed.x", (out.shape[0], self.hidden), torch.float32))
        return ctx.rt.ops.hc_spread(x, out, self.copies)


class LMHead(Part):
    """logits = y W^T, then the cap.  `table_name` may be the embedding's (a tied head)."""

    def __init__(self, vocab: int, hidden: int, table_name: str, softcap: float = 0.0, init_std: float = 0.02,
                 scale: float = 1.0):
        self.vocab, self.hidden = vocab, hidden
        self.table_name = table_name
        self.softcap = float(softcap or 0.0)
        self.scale = float(scale)               # a constant on the logits (before the cap, if there is one)
        self.init_std = init_std
        self.table = None

    def tensor_specs(self):
        return {self.table_name: TensorSpec((self.vocab, self.hidden), init_std=self.init_std)}

    def load(self, store, rt: Runtime):
        self.table = store.get(self.table_name, rt.dtype).contiguous()

    def forward(self, y, ctx: StepContext, out):
        """y [R, hidden] in the compute dtype -> out float32 [R, vocab]."""
        if self.scale != 1.0:
            if self.softcap > 0:
                raise NotImplementedError("a constant on the logits together with a cap")
            return ctx.rt.ops.scale_values(self._product(y, ctx, out), self.scale)
        return self._product(y, ctx, out)

    def _product(self, y, ctx: StepContext, out):
        ops = ctx.rt.ops
        R = y.shape[0]
        if ctx.rt.dtype == torch.float32:
            return ops.gemm_f32(y, self.table, out, self.softcap)
        vec = self.hidden % 8 == 0        # the skinny products read 16 bytes at a time; other widths take the library's
        if R <= ops.GEMV_FAST_ROWS and vec:
            return ops.gemv_bf16(y, self.table, out, ops.EPI_SOFTCAP, self.softcap)
        if R <= ops.TC05_MAX_ROWS and vec:
            return ops.gemm_tc05(y, self.table, out, ops.EPI_SOFTCAP, self.softcap)   # float32 logits straight from tensor memory
        # many rows: the library's product with float32 output, then the cap
        ops.matmul_bf16_to_f32(y, self.table, out)
        if self.softcap > 0:
            ops.softcap(out, self.softcap)
        return out
