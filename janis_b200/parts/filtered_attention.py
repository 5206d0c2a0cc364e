"""Softmax attention without positions, whose projections are filtered over time and normed before they are cached,
and whose heads' weights are mixed after the softmax.

With H query heads over G key/value heads (query head h uses key/value head h // (H/G)), keys of d features and
values of dv, and y the mixer's input:

    q, k, v      = F_q(Wq y), F_k(Wk y), F_v(Wv y)            F: a causal filter of `taps` taps on every channel,
                                                              u'[t] = sum_j f[c, j] u[t - taps + 1 + j], zeros
                                                              before the sequence starts (taps 0: no filter)
    q, k         = N(q) * wq, N(k) * wk                       N: RMS norm over the whole projection, all heads at once
    v_g          = v_g / rms(v_g)                             each value head by itself, no weight
    s_h[i, j]    = cap tanh(scale (q_h[i] . k[j]) / cap)      j <= i; cap 0: the scaled score itself
    p_h[i, :]    = softmax(s_h[i, :])
    p'_h[i, j]   = sum_g M[h, g] p_g[i, j]                    M: a stored H x H matrix (names["talk"]; absent: none)
    o_h[i]       = sum_j p'_h[i, j] v[j]

Positions enter nowhere but through the filter and the causal mask.  Keys and values are cached as normed; the last
taps - 1 projected rows of a sequence (before the filter) are kept per slot as float32 state, so that a step can
reach back before its first token.  A step writes its keys and values first and attends over the line alone, so
a prompt, a prompt that comes in pieces and a decode step are one code path.  Filter, norms, scores, softmax, mixing
and sums are float32 whatever the activations are.
"""
from __future__ import annotations

import torch

from ..cache.cache import KVNeed, StateNeed
from ..weights.loader import TensorSpec
from .base import Mixer, Runtime, StepContext


class FilteredAttention(Mixer):
    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, key_dim: int, value_dim: int, scale: float,
                 names: dict[str, str], taps: int = 0, cap: float = 0.0, norm_eps: float = 1e-6, qk_norm: bool = True,
                 unit_values: bool = True, init_std: float = 0.02):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} query heads do not divide over {n_kv_heads} key/value heads")
        need = ["q", "k", "v", "o"] + (["q_norm", "k_norm"] if qk_norm else []) + \
               (["q_conv", "k_conv", "v_conv"] if taps else [])
        for k in need:
            if k not in names:
                raise ValueError(f"filtered attention needs the checkpoint name of its {k!r} tensor")
        if not 0 <= taps <= 16:
            raise ValueError(f"a filter of {taps} taps (0 to 16 are taken)")
        self.hidden, self.n_heads, self.n_kv_heads = hidden, n_heads, n_kv_heads
        self.key_dim, self.value_dim = key_dim, value_dim
        self.scale, self.cap, self.eps = float(scale), float(cap or 0.0), float(norm_eps)
        self.taps = int(taps or 0)
        self.qk_norm, self.unit_values = bool(qk_norm), bool(unit_values)
        self.names = dict(names)
        self.init_std = init_std
        self.channels = n_heads * key_dim + n_kv_heads * (key_dim + value_dim)
        self.w_qkv = self.w_o = self.talk = self.filt = self.wq = self.wk = None

    def tensor_specs(self):
        H, G, d, dv, W, s, n = self.n_heads, self.n_kv_heads, self.key_dim, self.value_dim, self.hidden, self.init_std, self.names
        specs = {n["q"]: TensorSpec((H * d, W), init_std=s), n["k"]: TensorSpec((G * d, W), init_std=s),
                 n["v"]: TensorSpec((G * dv, W), init_std=s), n["o"]: TensorSpec((W, H * dv), init_std=s)}
        if self.qk_norm:
            specs[n["q_norm"]] = TensorSpec((H * d,), init_std=0.1, init_mean=1.0)
            specs[n["k_norm"]] = TensorSpec((G * d,), init_std=0.1, init_mean=1.0)
        if self.taps:
            for key, rows in (("q_conv", H * d), ("k_conv", G * d), ("v_conv", G * dv)):
                specs[n[key]] = TensorSpec((rows, self.taps), init_std=self.taps ** -0.5)
        if "talk" in n:
            specs[n["talk"]] = TensorSpec((H, H), init_std=H ** -0.5)
        return specs

    def cache_needs(self):
        needs = {"kv": KVNeed(self.n_kv_heads, self.key_dim, None, self.value_dim)}
        if self.taps > 1:
            needs["filter"] = StateNeed((self.taps - 1, self.channels))
        return needs

    def prompt_flops(self, n_tokens: int) -> float:
        seen = n_tokens * (n_tokens + 1) // 2
        return seen * 2.0 * self.n_heads * (self.key_dim + self.value_dim + ("talk" in self.names) * self.n_heads)

    def load(self, store, rt: Runtime):
        n = self.names
        self.w_qkv = torch.cat([store.get(n[x], rt.dtype) for x in ("q", "k", "v")], dim=0).contiguous()
        store.drop(*(n[x] for x in ("q", "k", "v")))
        self.w_o = store.get(n["o"], rt.dtype).contiguous()
        f32 = lambda key: store.get(n[key]).to(torch.float32).contiguous()
        self.talk = f32("talk") if "talk" in n else None
        self.wq, self.wk = (f32("q_norm"), f32("k_norm")) if self.qk_norm else (None, None)
        self.filt = torch.cat([f32("q_conv"), f32("k_conv"), f32("v_conv")], dim=0).contiguous() if self.taps else None

    def forward(self, x, ctx: StepContext, line):
        rt, ws, ops = ctx.rt, ctx.ws, ctx.rt.ops
        kv = line["kv"]
        if not kv.write:
            raise ValueError("filtered attention keeps keys and values of its own: the schedule cannot let it only read")
        T, H, G, d, dv = ctx.n_tok, self.n_heads, self.n_kv_heads, self.key_dim, self.value_dim
        decode = ctx.mode == "decode"
        rows = ws.buf("fattn.rows", (T, self.channels), rt.dtype)
        rt.linear(x, self.w_qkv, rows)
        q = ws.buf("fattn.q", (T, H * d), rt.dtype)
        ops.qkv_conv_norm_store(rows, H, G, d, dv, self.filt, line["filter"].data if self.taps > 1 else None, self.wq,
                                self.wk, self.unit_values, self.eps, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot,
                                ctx.seq_first_row, ctx.seq_start, ctx.seq_end, ctx.n_seq, q, kv.k, kv.v, kv.table,
                                one_token=decode)
        att = ws.buf("fattn.ctx", (T, H * dv), rt.dtype)
        if decode and rt.dtype == torch.bfloat16:
            # a decode step in the serving dtype: the kernels that take single rows and read keys and values once
            n = ops.talk_attention_rows_floats(rt.dtype, T, H, G, d, dv, ctx.len_bound)
            if n:
                ops.talk_attention_rows(q, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, kv.k, kv.v, kv.table, self.talk, att, H, G,
                                        d, dv, self.scale, ws.buf("fattn.rows_scratch", (n,), torch.float32), ctx.len_bound,
                                        cap=self.cap)
                return rt.linear(att, self.w_o, ws.buf("mixer.out", (T, self.hidden), rt.dtype))
        stats = None
        if self.talk is not None:
            stats = ws.buf("fattn.stats", (ops.talk_attention_stats_floats(T, H),), torch.float32)
        max_keys, n_chunks, scratch = 0, 1, None
        if decode:
            max_keys = ctx.len_bound
            n_chunks = max(1, min(rt.sm_count // max(T, 1), -(-max_keys // 128), 64))
            n = ops.talk_attention_scratch_floats(T, n_chunks, H, dv)
            scratch = ws.buf("fattn.partial", (n,), torch.float32) if n else None
        ops.talk_attention(q, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, kv.k, kv.v, kv.table, self.talk, None, att, H, G,
                           d, dv, self.scale, 0, False, one_row=decode, max_keys=max_keys, n_chunks=n_chunks,
                           scratch=scratch, cap=self.cap, mix_after=True, stats=stats)
        return rt.linear(att, self.w_o, ws.buf("mixer.out", (T, self.hidden), rt.dtype))
