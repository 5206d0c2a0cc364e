"""Dense feed-forwards: the gated one, down(act(gate(x)) * up(x)) without biases, and the plain one,
down(act(up(x) + b_up)) + b_down (`DenseMLP`, at the end of the file).

Gemma2's is GeGLU with the tanh form of gelu (`gemma/gemma.go:121-123`;
0.5 v (1 + tanh(0.7978845608028654 (v + 0.044715 v^3))), `cpu/cpu.go:417-423`);
with act="silu" it is the SwiGLU of the reference's other models
(`qwen/mlp.go:32-36`).

gate and up are one product: their rows are interleaved at load in groups of 8
(8 gate rows, the 8 matching up rows, ...), which puts each gate value beside
its up value in one tile of the skinny decode kernel, so the activation is
applied to float accumulators before anything is written.  Above 16 rows the
product comes from the library and a separate kernel applies the activation.
"""
from __future__ import annotations

import math

import torch

from ..weights.loader import TensorSpec
from .base import FeedForward, Runtime, StepContext

_ACTS = {"gelu_tanh": 0, "gelu_pytorch_tanh": 0, "silu": 1}


class GatedMLP(FeedForward):
    GROUP = 8

    def __init__(self, hidden: int, intermediate: int, names: dict[str, str], act: str = "gelu_tanh",
                 init_std: float = 0.02):
        if act not in _ACTS:
            raise ValueError(f"unknown activation {act!r} (known: {sorted(_ACTS)})")
        for k in ("gate", "up", "down"):
            if k not in names:
                raise ValueError(f"feed-forward needs the checkpoint name of its {k!r} projection")
        self.hidden, self.intermediate = hidden, intermediate
        # the fused gate/up layout wants whole groups: an intermediate width that is no multiple of the group is
        # padded with zero rows of gate and up (act(0) * 0 = 0) and zero columns of down
        self.padded = -(-intermediate // self.GROUP) * self.GROUP
        self.act = _ACTS[act]
        self.names = dict(names)
        self.init_std = init_std
        self.w_gu = None
        self.w_down = None

    def tensor_specs(self):
        H, I, s = self.hidden, self.intermediate, self.init_std
        return {self.names["gate"]: TensorSpec((I, H), init_std=s),
                self.names["up"]: TensorSpec((I, H), init_std=s),
                self.names["down"]: TensorSpec((H, I), init_std=s)}

    def load(self, store, rt: Runtime):
        g = store.get(self.names["gate"], rt.dtype)
        u = store.get(self.names["up"], rt.dtype)
        I, H, G = self.padded, self.hidden, self.GROUP
        if I != self.intermediate:
            pad = torch.zeros(I - self.intermediate, H, dtype=g.dtype, device=g.device)
            g, u = torch.cat([g, pad]), torch.cat([u, pad])
        fused = torch.stack([g.view(I // G, G, H), u.view(I // G, G, H)], dim=1)   # [I/G, 2, G, H]
        self.w_gu = fused.reshape(2 * I, H).contiguous()
        del g, u, fused
        store.drop(self.names["gate"], self.names["up"])                   # the fused copy is the one that stays
        self.w_down = store.get(self.names["down"], rt.dtype).contiguous()
        if I != self.intermediate:
            self.w_down = torch.cat([self.w_down, torch.zeros(H, I - self.intermediate, dtype=self.w_down.dtype,
                                                              device=self.w_down.device)], dim=1).contiguous()

    def forward(self, x, ctx: StepContext):
        rt, ws, ops = ctx.rt, ctx.ws, ctx.rt.ops
        T, I = ctx.n_tok, self.padded
        a = ws.buf("ffn.act", (T, I), rt.dtype)
        epi = ops.EPI_GATED_GELU if self.act == 0 else ops.EPI_GATED_SILU
        if rt.dtype == torch.bfloat16 and T <= ops.GEMV_FAST_ROWS and self.hidden % 8 == 0:   # (the skinny product reads 16 bytes at a time)
            ops.gemv_bf16(x, self.w_gu, a, epi)
        else:
            # (ops.gemm_tc05 computes this product with the activation fused for 17..64 rows, but at these
            # shapes the library product plus the activation kernel is still the faster pair)
            gu = ws.buf("ffn.gu", (T, 2 * I), rt.dtype)
            rt.linear(x, self.w_gu, gu)
            ops.gated_act(gu, a, self.act, self.GROUP)
        out = ws.buf("ffn.out", (T, self.hidden), rt.dtype)
        return rt.linear(a, self.w_down, out)


def _softplus(v: float) -> float:
    return max(v, 0.0) + math.log1p(math.exp(-abs(v)))


class DenseMLP(FeedForward):
    """down(act(up(x) + b_up)) + b_down, the biases optional.

    act: "gelu_tanh", "silu", "relu2" (the square of relu), or "xielu", a piecewise activation with two learnt numbers (p, q) per layer, stored
    as a tensor of two values under names["act"]:
        z > 0:   softplus(p) z^2 + z/2
        z <= 0:  (1/2 + softplus(q)) (e^z - 1 - z) + z/2
    The two factors are formed once, at load, in double precision."""

    def __init__(self, hidden: int, intermediate: int, names: dict[str, str], act: str = "xielu",
                 init_std: float = 0.02):
        if act not in ("xielu", "gelu_tanh", "silu", "relu2"):
            raise ValueError(f"unknown activation {act!r} (known: gelu_tanh, relu2, silu, xielu)")
        for k in ("up", "down"):
            if k not in names:
                raise ValueError(f"feed-forward needs the checkpoint name of its {k!r} projection")
        if act == "xielu" and "act" not in names:
            raise ValueError("the xielu activation needs the checkpoint name of its two numbers ('act')")
        self.hidden, self.intermediate = hidden, intermediate
        self.act = act
        self.names = dict(names)
        self.init_std = init_std
        self.w_up = self.w_down = self.b_up = self.b_down = None
        self.a_pos = self.a_neg = 0.0

    def tensor_specs(self):
        H, I, s, n = self.hidden, self.intermediate, self.init_std, self.names
        specs = {n["up"]: TensorSpec((I, H), init_std=s), n["down"]: TensorSpec((H, I), init_std=s)}
        if "up_bias" in n:
            specs[n["up_bias"]] = TensorSpec((I,), init_std=s)
        if "down_bias" in n:
            specs[n["down_bias"]] = TensorSpec((H,), init_std=s)
        if self.act == "xielu":
            specs[n["act"]] = TensorSpec((2,), init_std=0.5)
        return specs

    def load(self, store, rt: Runtime):
        n = self.names
        self.w_up = store.get(n["up"], rt.dtype).contiguous()
        self.w_down = store.get(n["down"], rt.dtype).contiguous()
        self.b_up = store.get(n["up_bias"], rt.dtype).contiguous() if "up_bias" in n else None
        self.b_down = store.get(n["down_bias"], rt.dtype).contiguous() if "down_bias" in n else None
        if self.act == "xielu":
            p, q = (float(v) for v in store.get(n["act"]).to(torch.float64).cpu().tolist())
            self.a_pos, self.a_neg = _softplus(p), 0.5 + _softplus(q)

    def forward(self, x, ctx: StepContext):
        rt, ws, ops = ctx.rt, ctx.ws, ctx.rt.ops
        T = ctx.n_tok
        a = ws.buf("ffn.act", (T, self.intermediate), rt.dtype)
        out = ws.buf("ffn.out", (T, self.hidden), rt.dtype)
        kind = {"xielu": ops.ACT_XIELU, "gelu_tanh": ops.ACT_GELU, "silu": ops.ACT_SILU_PLAIN, "relu2": ops.ACT_RELU2}[self.act]
        if (rt.dtype == torch.bfloat16 and T <= ops.GEMV_FAST_ROWS and self.hidden % 8 == 0 and self.intermediate % 8 == 0
                and hasattr(ops, "gemv_bf16_bias_act")):
            # few rows: bias and activation in the epilogue of the skinny products (the same bits as the two kernels)
            ops.gemv_bf16_bias_act(x, self.w_up, a, self.b_up, kind, self.a_pos, self.a_neg)
            return ops.gemv_bf16_bias_act(a, self.w_down, out, self.b_down, ops.ACT_NONE)
        rt.linear(x, self.w_up, a)
        ops.bias_act(a, self.b_up, kind, self.a_pos, self.a_neg)
        rt.linear(a, self.w_down, out)
        if self.b_down is not None:
            ops.bias_act(out, self.b_down, ops.ACT_NONE)
        return out
