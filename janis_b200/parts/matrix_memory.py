"""Matrix memory with exponential gates (the mLSTM of xLSTM): a recurrent mixer whose state is, per head, a matrix
C [d, dv], a vector n [d] and a running maximum m.

With y the mixer's input, per head (d key channels, dv value channels):

    q = Wq y / sqrt(d),   k = Wk y,   v = Wv y
    i = cap tanh((Wi y + bi) / cap),   f = logsigmoid(cap tanh((Wf y + bf) / cap))        log gates, one each per head
    m' = max(f + m, i)
    C <- e^(f + m - m') C + e^(i - m') k v^T,   n <- e^(f + m - m') n + e^(i - m') k
    o = C^T q / (max(|n . q|, e^(-m')) + 1e-6)

C, n and m start at zero (m at 0, not at minus infinity).  Each head's o is divided by its root mean square, the
heads side by side are multiplied by a weight vector of all heads' size and by sigmoid(Wg y), and projected by Wo.

q | k | v | g are one product over rows concatenated at load; the gates' logits are a product of their own with
float32 results, since everything from there to the state is float32 whatever the activations are: the gates, the
maxima, the exponentials, C, n, m and o.  The state lives in fixed-size parts of the cache line (C transposed as
[heads, dv, d]; n once per group of 8 value columns, so that the CTAs of the recurrence kernel each own a copy; m):
a step loads it, runs its tokens in order and writes it back, so a prompt, a prompt that continues and a decode
step are one code path; sequences without a slot (padding) start from zero and store nothing.
"""
from __future__ import annotations

import torch

from ..cache.cache import StateNeed
from ..weights.loader import TensorSpec
from .base import Mixer, Runtime, StepContext


class MatrixMemory(Mixer):
    NAMES = ("q", "k", "v", "g", "o", "i", "i_bias", "f", "f_bias", "norm")

    def __init__(self, hidden: int, n_heads: int, key_dim: int, value_dim: int, gate_cap: float, norm_eps: float,
                 names: dict[str, str], q_scale: float | None = None, init_std: float = 0.02):
        for k in self.NAMES:
            if k not in names:
                raise ValueError(f"the matrix memory needs the checkpoint name of its {k!r} tensor")
        if key_dim > 256:
            raise ValueError(f"the recurrence kernel takes up to 256 key channels a head, found {key_dim}")
        if not gate_cap > 0:
            raise ValueError("the gates' cap must be positive")
        self.hidden, self.n_heads, self.key_dim, self.value_dim = hidden, n_heads, key_dim, value_dim
        self.gate_cap, self.norm_eps = float(gate_cap), float(norm_eps)
        self.q_scale = float(q_scale) if q_scale is not None else key_dim ** -0.5
        self.names = dict(names)
        self.init_std = init_std
        self.w_in = self.w_gates = self.b_gates = self.w_norm = self.w_o = None

    def tensor_specs(self):
        H, d, dv, W, s, n = self.n_heads, self.key_dim, self.value_dim, self.hidden, self.init_std, self.names
        return {n["q"]: TensorSpec((H * d, W), init_std=s), n["k"]: TensorSpec((H * d, W), init_std=s),
                n["v"]: TensorSpec((H * dv, W), init_std=s), n["g"]: TensorSpec((H * dv, W), init_std=s),
                n["o"]: TensorSpec((W, H * dv), init_std=s),
                n["i"]: TensorSpec((H, W), init_std=s), n["i_bias"]: TensorSpec((H,), init_std=1.0),
                n["f"]: TensorSpec((H, W), init_std=s), n["f_bias"]: TensorSpec((H,), init_std=1.0, init_mean=3.0),
                n["norm"]: TensorSpec((H * dv,), init_std=0.1, init_mean=1.0)}

    def cache_needs(self):
        H, d, dv = self.n_heads, self.key_dim, self.value_dim
        return {"memory": StateNeed((H, dv, d), torch.float32),                 # C^T per head
                "normaliser": StateNeed((H, (dv + 7) // 8, d), torch.float32),  # n, a copy per group of value columns
                "maximum": StateNeed((H,), torch.float32)}

    def prompt_flops(self, n_tokens: int) -> float:
        return 5.0 * self.n_heads * self.key_dim * (self.value_dim + 1) * n_tokens      # decay, outer product, read-out

    def load(self, store, rt: Runtime):
        n = self.names
        parts = [store.get(n[k], rt.dtype) for k in ("q", "k", "v", "g")]
        self.w_in = torch.cat(parts, dim=0).contiguous()
        del parts
        store.drop(*(n[k] for k in ("q", "k", "v", "g")))
        self.w_gates = torch.cat([store.get(n["i"], rt.dtype), store.get(n["f"], rt.dtype)], dim=0).contiguous()
        store.drop(n["i"], n["f"])
        self.b_gates = torch.cat([store.get(n["i_bias"]).to(torch.float32), store.get(n["f_bias"]).to(torch.float32)]).contiguous()
        self.w_norm = store.get(n["norm"]).to(torch.float32).contiguous()
        self.w_o = store.get(n["o"], rt.dtype).contiguous()

    def forward(self, x, ctx: StepContext, line):
        rt, ws, ops = ctx.rt, ctx.ws, ctx.rt.ops
        mem, nrm, mx = line["memory"], line["normaliser"], line["maximum"]
        if not mem.write:
            raise ValueError("a recurrent state has one writer: a matrix-memory layer cannot read another's line")
        T, H, d, dv = ctx.n_tok, self.n_heads, self.key_dim, self.value_dim
        q_off, k_off, v_off, g_off = 0, H * d, 2 * H * d, 2 * H * d + H * dv
        rows = ws.buf("mlstm.rows", (T, g_off + H * dv), rt.dtype)
        rt.linear(x, self.w_in, rows)
        z = ws.buf("mlstm.z", (T, 2 * H), torch.float32)
        if rt.dtype == torch.float32:
            ops.gemm_f32(x, self.w_gates, z)
        elif T <= ops.GEMV_FAST_ROWS and self.hidden % 8 == 0:
            ops.gemv_bf16(x, self.w_gates, z)
        else:
            ops.matmul_bf16_to_f32(x, self.w_gates, z)
        o = ws.buf("mlstm.o", (T, H * dv), torch.float32)
        ops.mlstm_scan(rows, q_off, k_off, v_off, z, self.b_gates, self.gate_cap, ctx.seq_slot, ctx.seq_first_row,
                       ctx.seq_start, ctx.seq_end, mem.data, nrm.data, mx.data, o, ctx.n_seq, H, d, dv, self.q_scale,
                       ws.buf("mlstm.coef", (T, H, 3), torch.float32))
        y = ws.buf("mlstm.y", (T, H * dv), rt.dtype)
        ops.head_norm_gate(o, rows, g_off, self.w_norm, self.norm_eps, y, H, dv, gate="sigmoid")
        return rt.linear(y, self.w_o, ws.buf("mixer.out", (T, self.hidden), rt.dtype))
