"""Softmax attention whose heads are mixed before the softmax, with values of a size of their own.

With H query heads over G key/value heads (query head h uses key/value head h // (H/G)), keys of d features
and values of dv:

    raw_g[i, j] = (q_g[i] . k[j]) * scale                     positions encoded on q and k by `position`
    s_h[i, j]   = sum_g M[h, g] raw_g[i, j]                   M: a stored H x H matrix (names["talk"]; absent: none)
    p_h[i, j]   = exp(s_h[i, j]) / (sink + sum_j' exp(s_h[i, j']))
    o_h[i]      = sum_j p_h[i, j] v[j]

over the keys j <= i that lie in the query's block of `block` positions (block 0: all of them; blocks are counted
from the sequence's first position) and, with a `window`, among the query's last `window` positions (i - j < window:
the query's own and the window - 1 before it).  `sink` adds 1 to the denominator: a key of score 0 that has no value.  With a
`value_position` the values are rotated by their own position before they are cached (over all dv features) and
each head's output is turned back by the query's position, so that o depends on relative positions only.

With a gate (names["g"]) the heads side by side are multiplied, element by element, by sigmoid(Wg y) before the
output projection; Wg's rows stand behind the other projections' in the one product.

Further options.  `values_from_keys`: there is no value projection; a key/value head's values are its keys as
projected, before any turn or norm (so the value size is the key size), cached beside the keys.  `unit_norm_eps`:
after the turn every head of q and k is divided by its own root mean square, sqrt(mean(head^2) + eps), without a
weight.  A position encoding of pairs="neighbours" turns (2i, 2i + 1) instead of (i, i + rot/2).  `keep_first` (with
a window): the sequence's first `keep_first` positions stay seen behind the window, at their true positions.
`gate="head"`: Wg has one row per head and the gate is one number per head.

Keys and values live in a paged cache line with separate head sizes.  A step writes its keys and values first
and then attends over the line alone, so a prompt, a prompt that continues, a decode step and a layer that reads
the line of another layer (`own_kv=False`: queries only, no key/value tensors of its own) are one code path.
Scores, the mixing, the softmax and the sums are float32 whatever the activations are.
"""
from __future__ import annotations

import torch

from ..cache.cache import KVNeed
from ..weights.loader import TensorSpec
from .base import Mixer, Runtime, StepContext
from .position import RotaryEncoding


class TalkingHeadsAttention(Mixer):
    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, key_dim: int, value_dim: int, scale: float,
                 position: RotaryEncoding, names: dict[str, str], value_position: RotaryEncoding | None = None,
                 block: int = 0, sink: bool = False, own_kv: bool = True, init_std: float = 0.02, window: int = 0,
                 keep_first: int = 0, values_from_keys: bool = False, unit_norm_eps: float | None = None,
                 gate: str = "element"):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} query heads do not divide over {n_kv_heads} key/value heads")
        if gate not in ("head", "element"):
            raise ValueError(f"unknown gate {gate!r} (known: head, element)")
        if values_from_keys and (value_dim != key_dim or value_position is not None or not own_kv):
            raise ValueError("values that are the keys as projected have the keys' size, no turn of their own, and a line of their own")
        if keep_first < 0 or (keep_first and (not window or block)):
            raise ValueError("kept first positions need a window and no blocks")
        self.keep_first = int(keep_first or 0)
        self.values_from_keys = bool(values_from_keys)
        self.unit_norm_eps = None if unit_norm_eps is None else float(unit_norm_eps)
        self.gate = gate
        need = (("q", "k", "o") if values_from_keys else ("q", "k", "v", "o")) if own_kv else ("q", "o")
        for k in need:
            if k not in names:
                raise ValueError(f"attention needs the checkpoint name of its {k!r} projection")
        if value_position is not None and (value_position.rot != value_dim or value_dim % 2):
            raise ValueError("rotated values turn all of their features, in pairs")
        self.hidden, self.n_heads, self.n_kv_heads = hidden, n_heads, n_kv_heads
        self.key_dim, self.value_dim = key_dim, value_dim
        self.scale = float(scale)
        self.block = int(block or 0)
        self.window = int(window or 0)
        if self.window < 0:
            raise ValueError(f"a window holds at least one position, found {window}")
        self.sink = bool(sink)
        self.own_kv = bool(own_kv)
        self.position, self.value_position = position, value_position
        self.names = dict(names)
        self.init_std = init_std
        self.w_qkv = self.w_o = self.talk = None

    def tensor_specs(self):
        H, G, d, dv, W, s, n = self.n_heads, self.n_kv_heads, self.key_dim, self.value_dim, self.hidden, self.init_std, self.names
        specs = {n["q"]: TensorSpec((H * d, W), init_std=s), n["o"]: TensorSpec((W, H * dv), init_std=s)}
        if self.own_kv:
            specs[n["k"]] = TensorSpec((G * d, W), init_std=s)
            if not self.values_from_keys:
                specs[n["v"]] = TensorSpec((G * dv, W), init_std=s)
        if "talk" in n:
            specs[n["talk"]] = TensorSpec((H, H), init_std=H ** -0.5)
        if "g" in n:
            specs[n["g"]] = TensorSpec((H * dv if self.gate == "element" else H, W), init_std=s)
        return specs

    def sub_parts(self):
        return [p for p in (self.position, self.value_position) if p is not None]

    def cache_needs(self):
        return {"kv": KVNeed(self.n_kv_heads, self.key_dim, None, self.value_dim)}

    def prompt_flops(self, n_tokens: int) -> float:
        B = self.block or n_tokens
        full, rest = divmod(n_tokens, B)
        seen = full * (B * (B + 1) // 2) + rest * (rest + 1) // 2         # (query, key) pairs
        if self.window and not self.block:
            w = min(self.window, n_tokens)
            seen = w * (w + 1) // 2 + (n_tokens - w) * w
            far = max(0, n_tokens - w - self.keep_first)          # queries whose window has left all the kept positions behind
            seen += self.keep_first * far + sum(range(1, min(self.keep_first, max(0, n_tokens - w)) + 1)) if self.keep_first else 0
        return seen * 2.0 * self.n_heads * (self.key_dim + self.value_dim + ("talk" in self.names) * self.n_heads)

    def load(self, store, rt: Runtime):
        n = self.names
        gated = ("g",) if "g" in n else ()
        if self.own_kv:
            fused = (("q", "k") if self.values_from_keys else ("q", "k", "v")) + gated
            mats = [store.get(n[x], rt.dtype) for x in fused]
            self.w_qkv = torch.cat(mats, dim=0).contiguous()
            del mats
            store.drop(*(n[x] for x in fused))
        elif gated:
            self.w_qkv = torch.cat([store.get(n["q"], rt.dtype), store.get(n["g"], rt.dtype)], dim=0).contiguous()
            store.drop(n["q"], n["g"])
        else:
            self.w_qkv = store.get(n["q"], rt.dtype).contiguous()
        if self.w_qkv.shape[0] % 8:
            # rows of the step in whole 16-byte pieces (a gate per head may leave any number of columns): zero rows behind the last
            pad = torch.zeros(8 - self.w_qkv.shape[0] % 8, self.w_qkv.shape[1], dtype=self.w_qkv.dtype, device=self.w_qkv.device)
            self.w_qkv = torch.cat([self.w_qkv, pad], dim=0).contiguous()
        self.w_o = store.get(n["o"], rt.dtype).contiguous()
        self.talk = store.get(n["talk"]).to(torch.float32).contiguous() if "talk" in n else None

    def forward(self, x, ctx: StepContext, line):
        rt, ws, ops = ctx.rt, ctx.ws, ctx.rt.ops
        kv = line["kv"]
        if kv.write != self.own_kv:
            raise ValueError("the schedule lets a layer with keys and values of its own only read a line, or the reverse")
        T, H, G, d, dv = ctx.n_tok, self.n_heads, self.n_kv_heads, self.key_dim, self.value_dim
        kv_cols = (G * d if self.values_from_keys else G * (d + dv)) if self.own_kv else 0
        g_off = H * d + kv_cols                                        # where the gate's logits start in a row
        rows = ws.buf("tattn.rows", (T, self.w_qkv.shape[0]), rt.dtype)      # (the product's columns: the gate's, and padding, last)
        rt.linear(x, self.w_qkv, rows)
        inv_v = self.value_position.inv_freq if self.value_position is not None else None
        neighbours = self.position.pairs == "neighbours" and self.position.rot > 0
        if self.values_from_keys or self.unit_norm_eps is not None or neighbours:
            if inv_v is not None or not self.own_kv or self.position.amplitude != 1.0:
                raise NotImplementedError("turned values, a borrowed line or an amplitude together with normed or neighbouring pairs")
            if not self.values_from_keys:
                raise NotImplementedError("normed or neighbouring pairs beside a value projection of its own")
            ops.qk_rotate_norm_store(rows, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, self.position.inv_freq, self.position.rot,
                                     not neighbours, self.unit_norm_eps is not None, self.unit_norm_eps or 0.0, H, G, d,
                                     kv.k, kv.v if self.values_from_keys else None, kv.table)
        else:
            ops.qkv_rotate_store(rows, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, self.position.inv_freq, self.position.rot,
                                 inv_v, H, G, d, dv, kv.k if self.own_kv else None, kv.v if self.own_kv else None,
                                 kv.table if self.own_kv else None, store=self.own_kv)
        att = ws.buf("tattn.ctx", (T, H * dv), rt.dtype)
        decode = ctx.mode == "decode"
        max_keys, n_chunks, scratch = 0, 1, None
        rows_floats = 0
        if (decode and rt.dtype == torch.bfloat16 and not self.block and not self.sink and self.talk is None and inv_v is None
                and hasattr(ops, "talk_attention_rows_floats")):
            # a decode step in the serving dtype with nothing the kernels that take single rows leave out: keys and
            # values read once, 16 bytes a lane
            max_keys = min(ctx.len_bound, self.window + self.keep_first) if self.window else ctx.len_bound
            rows_floats = ops.talk_attention_rows_floats(rt.dtype, T, H, G, d, dv, max_keys)
        if rows_floats:
            ops.talk_attention_rows(rows, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, kv.k, kv.v, kv.table, None, att, H, G, d, dv,
                                    self.scale, ws.buf("tattn.rows_scratch", (rows_floats,), torch.float32), max_keys,
                                    window=self.window, **({"keep_first": self.keep_first} if self.keep_first else {}))
            if "g" in self.names:
                ops.sigmoid_gate(att, rows, g_off, per=dv if self.gate == "head" else 1)
            return rt.linear(att, self.w_o, ws.buf("mixer.out", (T, self.hidden), rt.dtype))
        if decode:
            # a decode row's keys over several CTAs when the rows alone would leave most of the GPU idle: about a
            # CTA an SM in all, none with fewer than 128 keys (the bound on the lengths is the host's)
            max_keys = min(self.block, ctx.len_bound) if self.block else ctx.len_bound
            if self.window:
                max_keys = min(max_keys, self.window + self.keep_first)
            n_chunks = max(1, min(rt.sm_count // max(T, 1), -(-max_keys // 128), 64))
            n = ops.talk_attention_scratch_floats(T, n_chunks, H, dv)
            scratch = ws.buf("tattn.partial", (n,), torch.float32) if n else None
        ops.talk_attention(rows, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, kv.k, kv.v, kv.table, self.talk, inv_v, att,
                           H, G, d, dv, self.scale, self.block, self.sink, one_row=decode, max_keys=max_keys,
                           n_chunks=n_chunks, scratch=scratch, window=self.window,
                           **({"keep_first": self.keep_first} if self.keep_first else {}))
        if "g" in self.names:
            ops.sigmoid_gate(att, rows, g_off, per=dv if self.gate == "head" else 1)
        return rt.linear(att, self.w_o, ws.buf("mixer.out", (T, self.hidden), rt.dtype))
