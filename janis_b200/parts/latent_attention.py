"""Attention over a compressed key/value row: one small vector per position is cached, every head's keys and values
are linear maps of it.

With H heads, a query/key head of d plain and dr turned features, values of dv, a compressed row of R features, and
y the mixer's input:

    q_h          = [a_h | b_h] = rows of Wq y                  a_h: d features, b_h: dr features
    [c | r]      = Wdkv y                                      c: R features, r: dr features shared by all heads
    c            = N(c) * wc                                   RMS norm with a weight
    b_h, r       = turn(b_h, i), turn(r, j)                    `position`: neighbouring pairs, scaled frequencies,
                                                               an amplitude on sine and cosine
    k_h[j]       = [Uk_h c[j] | r[j]],  v_h[j] = Uv_h c[j]
    s_h[i, j]    = scale (a_h[i] . Uk_h c[j] + b_h[i] . r[j])  0 <= i - j < window (window 0: every j <= i)
    p_h[i, j]    = exp(s_h[i, j]) / (exp(z_h) + sum_j' exp(s_h[i, j']))      z: a stored number per head (names["sink"])
    o_h[i]       = sigmoid(Wg y)_h * sum_j p_h[i, j] v_h[j]    one gate per head (names["g"]; absent: none)

The queries may pass a compressed row of their own (names "dq", "dq_norm", "uq" instead of "q"): cq = N(Wdq y) * wq,
q = Wuq cq.  The turned pairs are neighbours (2i, 2i + 1) or, with a position encoding of pairs="halves", (i, i + dr/2)
inside the turned part.  The gate is one number per head (`gate="head"`) or one per feature of the heads side by side
(`gate="element"`, Wg of H dv rows).  Without `sink` the softmax is the ordinary one.

The cache line holds [c | r] per position and nothing per head.  Because a . (Uk c) = (Uk^T a) . c and
sum_j p Uv c[j] = Uv sum_j p c[j], the scores are taken between [Uk_h^T a_h | b_h] and the cached row itself, the
weighted sum runs over the cached c, and Uv_h is applied once per query afterwards: no key or value of a head is
ever formed, in prompts or in decoding.  A step writes its rows first and attends over the line alone.  Norm,
angles, scores, the softmax and the sums are float32 whatever the activations are.
"""
from __future__ import annotations

import torch

from ..cache.cache import KVNeed
from ..weights.loader import TensorSpec
from .base import Mixer, Runtime, StepContext
from .position import RotaryEncoding


class LatentAttention(Mixer):
    def __init__(self, hidden: int, n_heads: int, key_dim: int, rot_dim: int, value_dim: int, rank: int, scale: float,
                 names: dict[str, str], position: RotaryEncoding | None = None, window: int = 0, sink: bool = True,
                 norm_eps: float = 1e-6, init_std: float = 0.02, gate: str = "head", q_rank: int = 0):
        self.q_rank = int(q_rank or 0)          # > 0: the queries pass a compressed row of that size
        need = (["dq", "dq_norm", "uq"] if self.q_rank else ["q"]) + ["dkv", "dkv_norm", "uk", "uv", "o"] + (["sink"] if sink else [])
        if gate not in ("head", "element"):
            raise ValueError(f"unknown gate {gate!r} (known: head, element)")
        self.gate = gate
        for k in need:
            if k not in names:
                raise ValueError(f"latent attention needs the checkpoint name of its {k!r} tensor")
        if rot_dim % 2:
            raise ValueError(f"the turned part of a head has pairs of features, found {rot_dim}")
        if rot_dim and (position is None or position.head_dim != rot_dim or position.amplitude != 1.0 and position.pairs == "halves"):
            raise ValueError("latent attention turns its rot_dim features itself: it needs a position encoding of that size")
        if window < 0:
            raise ValueError(f"a window holds at least one position, found {window}")
        self.hidden, self.n_heads = hidden, n_heads
        self.key_dim, self.rot_dim, self.value_dim, self.rank = key_dim, rot_dim, value_dim, rank
        self.scale, self.eps = float(scale), float(norm_eps)
        self.window = int(window or 0)
        self.sink = bool(sink)
        self.position = position
        self.names = dict(names)
        self.init_std = init_std
        self.w_in = self.w_o = self.uk_t = self.uv = self.wc = self.sink_values = self.inv_freq = None
        self.w_dq = self.w_uq = self.wq = None

    def tensor_specs(self):
        H, d, dr, dv, R, W, s, n = (self.n_heads, self.key_dim, self.rot_dim, self.value_dim, self.rank, self.hidden,
                                    self.init_std, self.names)
        specs = {n["dkv"]: TensorSpec((R + dr, W), init_std=s),
                 n["dkv_norm"]: TensorSpec((R,), init_std=0.1, init_mean=1.0),
                 n["uk"]: TensorSpec((H * d, R), init_std=R ** -0.5), n["uv"]: TensorSpec((H * dv, R), init_std=R ** -0.5),
                 n["o"]: TensorSpec((W, H * dv), init_std=s)}
        if self.sink:
            specs[n["sink"]] = TensorSpec((H,), init_std=1.0)
        if self.q_rank:
            specs[n["dq"]] = TensorSpec((self.q_rank, W), init_std=s)
            specs[n["dq_norm"]] = TensorSpec((self.q_rank,), init_std=0.1, init_mean=1.0)
            specs[n["uq"]] = TensorSpec((H * (d + dr), self.q_rank), init_std=self.q_rank ** -0.5)
        else:
            specs[n["q"]] = TensorSpec((H * (d + dr), W), init_std=s)
        if "g" in n:
            specs[n["g"]] = TensorSpec((H * dv if self.gate == "element" else H, W), init_std=s)
        return specs

    def sub_parts(self):
        return [self.position] if self.position is not None else []

    def cache_needs(self):
        # one "head" whose key is [c | r]; the values are the key's first R features, so the value side is not used
        return {"kv": KVNeed(1, self.rank + self.rot_dim, None, 1)}

    def prompt_flops(self, n_tokens: int) -> float:
        w = min(self.window, n_tokens) if self.window else n_tokens
        seen = w * (w + 1) // 2 + (n_tokens - w) * w
        per_query = 2.0 * self.n_heads * self.rank * (self.key_dim + self.value_dim)       # Uk^T a and Uv (sum p c)
        return seen * 2.0 * self.n_heads * (2 * self.rank + self.rot_dim) + n_tokens * per_query

    def load(self, store, rt: Runtime):
        n, H, d, dv, R = self.names, self.n_heads, self.key_dim, self.value_dim, self.rank
        fused = (() if self.q_rank else ("q",)) + ("dkv",) + (("g",) if "g" in n else ())
        mats = [store.get(n[x], rt.dtype) for x in fused]
        self.w_in = torch.cat(mats, dim=0).contiguous()
        del mats
        store.drop(*(n[x] for x in fused))
        if self.q_rank:
            self.w_dq = store.get(n["dq"], rt.dtype).contiguous()
            self.w_uq = store.get(n["uq"], rt.dtype).contiguous()
            self.wq = store.get(n["dq_norm"]).to(torch.float32).contiguous()
        self.w_o = store.get(n["o"], rt.dtype).contiguous()
        self.uk_t = store.get(n["uk"], rt.dtype).view(H, d, R).transpose(1, 2).contiguous()     # [H, R, d]: Uk_h^T
        self.uv = store.get(n["uv"], rt.dtype).view(H, dv, R).contiguous()
        store.drop(n["uk"], n["uv"])
        self.wc = store.get(n["dkv_norm"]).to(torch.float32).contiguous()
        self.sink_values = store.get(n["sink"]).to(torch.float32).contiguous() if self.sink else None
        table = torch.zeros(max(self.rot_dim // 2, 1), dtype=torch.float32)
        if self.position is not None and self.position.rot:
            table[:self.position.rot // 2] = torch.from_numpy(self.position._inv_host.copy())
        self.inv_freq = table[:self.rot_dim // 2].contiguous().to(rt.device) if self.rot_dim else table.to(rt.device)

    def forward(self, x, ctx: StepContext, line):
        rt, ws, ops = ctx.rt, ctx.ws, ctx.rt.ops
        kv = line["kv"]
        if not kv.write:
            raise ValueError("latent attention keeps a line of its own: the schedule cannot let it only read")
        T, H, d, dr, dv, R = ctx.n_tok, self.n_heads, self.key_dim, self.rot_dim, self.value_dim, self.rank
        D = R + dr
        lat_off = 0 if self.q_rank else H * (d + dr)
        g_off = lat_off + D
        n_gate = 0 if "g" not in self.names else (H * dv if self.gate == "element" else H)
        rows = ws.buf("lattn.rows", (T, g_off + n_gate), rt.dtype)
        rt.linear(x, self.w_in, rows)
        q_rows = None
        if self.q_rank:
            # the queries through their compressed row: product, norm (float32 inside), product
            cq = rt.linear(x, self.w_dq, ws.buf("lattn.cq", (T, self.q_rank), rt.dtype))
            cq = ops.rmsnorm(cq, self.wq, self.eps, ws.buf("lattn.cqn", (T, self.q_rank), rt.dtype))
            q_rows = rt.linear(cq, self.w_uq, ws.buf("lattn.qrows", (T, H * (d + dr)), rt.dtype))
        qfull = ws.buf("lattn.q", (T, H * D), rt.dtype)
        if d:
            ops.head_linear(q_rows if q_rows is not None else rows, d + dr, 0, self.uk_t, qfull, D, 0)          # [Uk_h^T a_h | .]
        else:
            qfull.zero_()
        pos = self.position
        extra = {"q_rows": q_rows} if q_rows is not None else {}
        if pos is not None and pos.pairs == "halves":
            extra["halves"] = True
        ops.latent_rotate_store(rows, lat_off, H, d, dr, R, self.wc, self.eps, self.inv_freq,
                                pos.amplitude if pos is not None else 1.0, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, qfull,
                                kv.k, kv.table, rot=pos.rot if pos is not None else 0, **extra)
        mixed = ws.buf("lattn.mixed", (T, H * R), rt.dtype)                   # sum_j p c[j], head by head
        decode = ctx.mode == "decode"
        max_keys, n_chunks, scratch = 0, 1, None
        rows_floats = 0
        if decode and rt.dtype == torch.bfloat16:
            # a decode step in the serving dtype: the kernels that take single rows and read the cached rows once
            max_keys = min(ctx.len_bound, self.window) if self.window else ctx.len_bound
            rows_floats = ops.talk_attention_rows_floats(rt.dtype, T, H, 1, D, R, max_keys)
        if rows_floats:
            ops.talk_attention_rows(qfull, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, kv.k, None, kv.table, None, mixed, H, 1, D, R,
                                    self.scale, ws.buf("lattn.rows_scratch", (rows_floats,), torch.float32), max_keys,
                                    sink=self.sink, window=self.window, sink_values=self.sink_values, values_in_keys=True)
        elif decode:
            max_keys = min(ctx.len_bound, self.window) if self.window else ctx.len_bound
            n_chunks = max(1, min(rt.sm_count // max(T, 1), -(-max_keys // 128), 64))
            n = ops.talk_attention_scratch_floats(T, n_chunks, H, R)
            scratch = ws.buf("lattn.partial", (n,), torch.float32) if n else None
        if not rows_floats:
            ops.talk_attention(qfull, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, kv.k, None, kv.table, None, None, mixed, H, 1,
                               D, R, self.scale, 0, self.sink, one_row=decode, max_keys=max_keys, n_chunks=n_chunks,
                               scratch=scratch, window=self.window, sink_values=self.sink_values, values_in_keys=True)
        att = ws.buf("lattn.ctx", (T, H * dv), rt.dtype)
        ops.head_linear(mixed, R, 0, self.uv, att, dv, 0)
        if "g" in self.names:
            ops.sigmoid_gate(att, rows, g_off, per=dv if self.gate == "head" else 1)
        return rt.linear(att, self.w_o, ws.buf("mixer.out", (T, self.hidden), rt.dtype))
