"""Plain, slow Vivazen: whole sequences, no cache, one function per mechanism.

It is the oracle of the Vivazen tests and shares no code with the package under
test (the container reader is the other oracle's).  Everything runs in float64
torch operations.

The design, in this file's notation.  r is the residual stream [T, width]; a sublayer reads r itself.

* embedding:     r = E[token]
* layer:         r = N1(a r + mixer(r));  r = N2(a r + ff(r))      a = postln_alpha; the second line only with a feed-forward
* norm:          the row in `groups` equal runs, each divided by sqrt(mean(run^2) + eps); then the whole times w
* 'attention':   q, k, v = conv(W_q r), conv(W_k r), conv(W_v r): a causal filter of `conv` taps per channel;
                 q and k RMS-normed over the whole projection (one mean over all heads) with a weight vector;
                 each value head divided by its root mean square; s = cap tanh(scale q.k / cap), causal;
                 p = softmax(s) per head; p'_h = sum_g M[h, g] p_g; o_h = p'_h v_kv(h); W_o
* 'latent_attention':  q = W_q r, per head [dim plain | rot_dim turned]; [c | kr] = W_dkv r, c RMS-normed with a weight;
                 k_h = [W_uk c | turn(kr)], v_h = W_uv c; turned pairs are neighbours (2i, 2i + 1), frequencies
                 blended between f and f / factor over a ramp, amplitude 0.1 ln(factor) + 1 on sine and cosine;
                 query i sees keys i - size < j <= i; softmax whose denominator also holds exp(sink_h);
                 o_h times sigmoid(W_g r)_h; W_o
* feed-forward:  W_down (gelu_tanh(W_gate r) * (W_up r))
* output:        the same norm with final.norm, then head
A layer with `weights_of: j` runs layer j's tensors.
"""
from __future__ import annotations

import math

import torch

from .gemma2_plain import load_folder  # noqa: F401  (the folder reader: config dict and float64 tensors)

F = torch.float64


def group_norm(x, weight, groups, eps):
    T, W = x.shape
    g = x.reshape(T, groups, W // groups)
    g = g / torch.sqrt((g * g).mean(-1, keepdim=True) + eps)
    return g.reshape(T, W) * weight


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def short_filter(u, taps_w):
    """u [T, C], taps_w [C, taps]: y[t] = sum_j taps_w[:, j] u[t - taps + 1 + j], zeros before the start."""
    T, C = u.shape
    taps = taps_w.shape[1]
    y = torch.zeros(T, C, dtype=F)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += taps_w[:, j] * u[s]
    return y


def mixed_softmax_attention(q, k, v, scale, cap, talk):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; causal; weights mixed over heads after the softmax."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    p = torch.zeros(H, T, T, dtype=F)
    keep = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for h in range(H):
        s = (q[:, h] @ k[:, h // rep].T) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~keep, float("-inf"))
        p[h] = torch.softmax(s, dim=-1)
    if talk is not None:
        p = torch.einsum("hg,gij->hij", talk, p)
    return torch.stack([p[h] @ v[:, h // rep] for h in range(H)], dim=1)        # [T, H, dv]


def attention_mixer(y, w, pre, m, eps):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = y.shape[0]
    q, k, v = y @ w[pre + "q"].T, y @ w[pre + "k"].T, y @ w[pre + "v"].T
    if m.get("conv"):
        q, k, v = (short_filter(u, w[pre + n + ".conv"]) for u, n in ((q, "q"), (k, "k"), (v, "v")))
    q = rms(q, eps) * w[pre + "q.norm"]
    k = rms(k, eps) * w[pre + "k.norm"]
    v = rms(v.reshape(T, G, dv), eps)
    o = mixed_softmax_attention(q.reshape(T, H, d), k.reshape(T, G, d), v, m["scale"], m.get("softcap") or 0.0,
                                w.get(pre + "talk"))
    return o.reshape(T, H * dv) @ w[pre + "o"].T


def ramped_frequencies(rot):
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = sc["factor"], sc["original"]

    def where(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(sc["fast"])), 0)
    hi = min(math.ceil(where(sc["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def turn_neighbours(x, pos, freq, amp):
    """x [T, n, dims]: the pair (2i, 2i + 1) turned by pos * freq[i]; sine and cosine times amp."""
    ang = pos.to(F)[:, None] * torch.tensor(freq, dtype=F)[None, :]
    c, s = (torch.cos(ang) * amp)[:, None, :], (torch.sin(ang) * amp)[:, None, :]
    a, b = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = a * c - b * s
    out[..., 1::2] = b * c + a * s
    return out


def latent_attention_mixer(y, w, pre, m, eps):
    H, d, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = y.shape[0]
    pos = torch.arange(T)
    freq, amp = ramped_frequencies(m["rot"])
    q = (y @ w[pre + "q"].T).reshape(T, H, d + dr)
    lat = y @ w[pre + "dkv"].T
    c = rms(lat[:, :R], eps) * w[pre + "dkv.norm"]
    kr = turn_neighbours(lat[:, None, R:], pos, freq, amp)                     # [T, 1, dr]
    qr = turn_neighbours(q[..., d:], pos, freq, amp)
    kn = (c @ w[pre + "uk"].T).reshape(T, H, d)
    v = (c @ w[pre + "uv"].T).reshape(T, H, dv)
    gate = torch.sigmoid(y @ w[pre + "g"].T)                                   # [T, H]
    size = (m.get("mask") or {}).get("size") or 0
    i, j = pos[:, None], pos[None, :]
    seen = (j <= i) & ((i - j < size) if size else torch.ones_like(i, dtype=torch.bool))
    outs = []
    for h in range(H):
        s = (q[:, h, :d] @ kn[:, h].T + qr[:, h] @ kr[:, 0].T) * m["scale"]
        s = s.masked_fill(~seen, float("-inf"))
        mx = torch.maximum(s.max(-1, keepdim=True).values, w[pre + "sink"][h])
        e = torch.exp(s - mx)
        p = e / (e.sum(-1, keepdim=True) + torch.exp(w[pre + "sink"][h] - mx))
        outs.append((p @ v[:, h]) * gate[:, h:h + 1])
    return torch.cat(outs, dim=1) @ w[pre + "o"].T


def gated_ff(y, w, pre):
    return (gelu_tanh(y @ w[pre + "gate"].T) * (y @ w[pre + "up"].T)) @ w[pre + "down"].T


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (and the stream after every layer run when asked)."""
    eps, groups, alpha = cfg["norm"]["eps"], cfg["norm"].get("groups", 1), cfg.get("postln_alpha", 1.0)
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)].to(F)
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        src = layer.get("weights_of")
        pre = f"l{i if src is None else src}."
        if layer["type"] == "attention":
            r = attention_mixer(x, w, pre + "mix.", layer["mixer"], eps)
        elif layer["type"] == "latent_attention":
            r = latent_attention_mixer(x, w, pre + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = group_norm(alpha * x + r, w[pre + "norm1"], groups, eps)
        if layer.get("mlp"):
            x = group_norm(alpha * x + gated_ff(x, w, pre + "mlp."), w[pre + "norm2"], groups, eps)
        layers.append(x.clone())
    logits = group_norm(x, w["final.norm"], groups, eps) @ w["head"].T
    return (logits, layers) if return_layers else logits
