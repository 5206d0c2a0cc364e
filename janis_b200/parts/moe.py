"""A mixture of experts as a feed-forward: a router picks `top` of E small gated feed-forwards per token; a shared
expert may run for every token beside them.

Router (all of it float32; its input may be the activations' rounding):

    s = sigmoid(W_r y)                                    one score per expert
    c = s + correction                                    choice scores: they pick, s weighs
    experts form `group_count` equal groups of neighbours; a group's score is the sum of its two largest c;
    only experts of the best `group_keep` groups can be chosen (the others' c count as minus infinity)
    chosen = the `top` experts of largest c;   w_e = s_e / (sum over chosen s + 1e-20) * scale

Expert (no biases):  g = min(W_gate y, limit),  u = clamp(W_up y, -limit, limit),
                     a = g sigmoid(1.702 g) (u + 1),  out = W_down a.

    ff(y) = sum over chosen w_e expert_e(y)  +  sigmoid(w_sg . y) shared(y)

Other forms of the same parts: `score="softmax"` takes s = softmax(W_r y) over all router entries instead of the
logistic function; `act="silu"` is the plain gated expert W_down (silu(W_gate y) * (W_up y)) without limits; and
`n_identity` router entries behind the experts have no tensors and return their input, so that a token's chosen
identity entries add (sum of their w) y to the output.

How it is computed: the gate and up matrices of all experts (and of the shared one) are one matrix, their down
matrices another, concatenated at load.  One product gives every expert's g and u for every token; the activation
kernel multiplies each expert's a by the token's weight for it (0 for experts that were not chosen, the gate's
sigmoid for the shared expert); the product with the concatenated down matrices then is the weighted sum.  An
expert that was not chosen contributes exact zeros.  This does the work of all experts for every token, which at E /
top of a few and steps of many tokens costs less than sorting tokens to experts would save; it is exact in the
choice and independent of what else is in the step.  The router's logits and the shared gate's are one float32
product over the rows W_r | w_sg.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import FeedForward, Runtime, StepContext


class RoutedExperts(FeedForward):
    def __init__(self, hidden: int, n_experts: int, top: int, expert_ff: int, limit: float, scale: float,
                 names: dict[str, str], group_count: int = 1, group_keep: int = 1, shared_ff: int = 0,
                 shared_limit: float = 0.0, gate_alpha: float = 1.702, init_std: float = 0.02, score: str = "sigmoid",
                 act: str = "clamped_swish", n_identity: int = 0):
        """names: "router", "correction", "expert" (a pattern with {e} and {w}: w is gate, up or down), and with a
        shared expert "shared" (a pattern with {w}) and "shared_gate"."""
        for k in ("router", "correction", "expert") + (("shared", "shared_gate") if shared_ff else ()):
            if k not in names:
                raise ValueError(f"the mixture of experts needs the checkpoint name of its {k!r} tensors")
        if score not in ("sigmoid", "softmax"):
            raise ValueError(f"unknown router score {score!r} (known: sigmoid, softmax)")
        if act not in ("clamped_swish", "silu"):
            raise ValueError(f"unknown expert activation {act!r} (known: clamped_swish, silu)")
        self.score, self.act, self.n_identity = score, act, int(n_identity or 0)
        n_route = n_experts + self.n_identity
        if self.n_identity and group_count != 1:
            raise ValueError("identity entries stand in no group")
        if n_route % group_count or group_keep > group_count or top > group_keep * (n_route // group_count):
            raise ValueError(f"{n_route} router entries in {group_count} groups, {group_keep} kept, {top} chosen")
        if n_route > 1024:
            raise ValueError(f"the router kernel takes up to 1024 entries, found {n_route}")
        if act == "silu":                      # no limits, g sigmoid(g) u
            limit, shared_limit, gate_alpha = float("inf"), float("inf"), 1.0
        self.hidden, self.n_experts, self.top, self.expert_ff = hidden, n_experts, top, expert_ff
        self.limit, self.scale = float(limit), float(scale)
        self.group_count, self.group_keep = group_count, group_keep
        self.shared_ff, self.shared_limit = int(shared_ff or 0), float(shared_limit or 0.0)
        self.gate_alpha = float(gate_alpha)
        self.names = dict(names)
        self.init_std = init_std
        self.w_route = self.correction = self.w_gu = self.w_down = None

    def _expert_names(self):
        n = self.names
        out = [{w: n["expert"].format(e=e, w=w) for w in ("gate", "up", "down")} for e in range(self.n_experts)]
        if self.shared_ff:
            out.append({w: n["shared"].format(w=w) for w in ("gate", "up", "down")})
        return out

    def tensor_specs(self):
        W, s, n = self.hidden, self.init_std, self.names
        specs = {n["router"]: TensorSpec((self.n_experts + self.n_identity, W), init_std=s),
                 n["correction"]: TensorSpec((self.n_experts + self.n_identity,), init_std=0.1)}
        for i, en in enumerate(self._expert_names()):
            ff = self.expert_ff if i < self.n_experts else self.shared_ff
            specs[en["gate"]] = TensorSpec((ff, W), init_std=s)
            specs[en["up"]] = TensorSpec((ff, W), init_std=s)
            specs[en["down"]] = TensorSpec((W, ff), init_std=s)
        if self.shared_ff:
            specs[n["shared_gate"]] = TensorSpec((1, W), init_std=s)
        return specs

    @property
    def total_ff(self) -> int:
        return self.n_experts * self.expert_ff + self.shared_ff

    def load(self, store, rt: Runtime):
        n = self.names
        route = [store.get(n["router"], rt.dtype)]
        if self.shared_ff:
            route.append(store.get(n["shared_gate"], rt.dtype).reshape(1, self.hidden))
        self.w_route = torch.cat(route, dim=0).contiguous()
        self.correction = store.get(n["correction"]).to(torch.float32).contiguous()
        gu, down = [], []
        for en in self._expert_names():
            gu += [store.get(en["gate"], rt.dtype), store.get(en["up"], rt.dtype)]      # per expert: gate rows, then up rows
            down.append(store.get(en["down"], rt.dtype))
        self.w_gu = torch.cat(gu, dim=0).contiguous()                                   # [2 total_ff, W]
        self.w_down = torch.cat(down, dim=1).contiguous()                               # [W, total_ff]
        del gu, down
        for en in self._expert_names():
            store.drop(*en.values())

    def forward(self, x, ctx: StepContext):
        rt, ws, ops = ctx.rt, ctx.ws, ctx.rt.ops
        T, E = ctx.n_tok, self.n_experts
        n_route = E + self.n_identity + (1 if self.shared_ff else 0)
        n_weights = E + (1 if self.shared_ff else 0) + (1 if self.n_identity else 0)
        z = ws.buf("moe.logits", (T, n_route), torch.float32)
        if rt.dtype == torch.float32:
            ops.gemm_f32(x, self.w_route, z)
        elif T <= ops.GEMV_FAST_ROWS and self.hidden % 8 == 0:
            ops.gemv_bf16(x, self.w_route, z)
        else:
            ops.matmul_bf16_to_f32(x, self.w_route, z)
        wts = ws.buf("moe.weights", (T, n_weights), torch.float32)
        plain = self.score == "sigmoid" and not self.n_identity and self.act == "clamped_swish"
        ops.moe_route(z, self.correction, E, self.group_count, self.group_keep, self.top, self.scale,
                      bool(self.shared_ff), wts,
                      **({} if plain else {"n_identity": self.n_identity, "softmax": self.score == "softmax"}))
        out = ws.buf("ffn.out", (T, self.hidden), rt.dtype)
        if self.total_ff:
            gu = rt.linear(x, self.w_gu, ws.buf("moe.gu", (T, 2 * self.total_ff), rt.dtype))
            a = ws.buf("moe.act", (T, self.total_ff), rt.dtype)
            ops.moe_expert_act(gu, wts, E, self.expert_ff, self.limit, self.shared_ff, self.shared_limit, self.gate_alpha, a,
                               **({} if plain else {"up_add": 0.0 if self.act == "silu" else 1.0}))
            rt.linear(a, self.w_down, out)
        else:
            out.zero_()
        if self.n_identity:
            ops.moe_identity_add(out, x, wts, n_weights - 1)
        return out
