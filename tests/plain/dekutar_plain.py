"""Plain, slow Dekutar: whole sequences, no cache, one function per mechanism.

It is the oracle of the Dekutar tests and shares no code with the package under
test (the container reader is the other oracle's).  Everything runs in float64
torch operations, token after token where the design is a recurrence.

The design, in this file's notation.  S copies x_1 .. x_S of the residual stream [T, width] (S = `streams`).

* embedding:     every x_s = E[token] * embedding.scale
* sublayer q of a layer (1: the mixer, 2: the feed-forward, if any), with vectors a_q, b_q [S] and a matrix M_q [S, S]:
                 u = sum_s a_q[s] x_s;  y = sublayer(N_q(u));  x_t <- sum_s M_q[s, t] x_s + b_q[t] y   (all t from the old x)
                 without `streams` in the configuration there is one x and x <- x + sublayer(N_q(x))
* norm:          N(x) = x / sqrt(mean(x^2) + eps) * (1 + w)
* 'latent_attention':  cq = rms(W_dq y) * w_dq;  q = W_uq cq, per head [dim plain | rot_dim turned];
                 [c | kr] = W_dkv y, c = rms(c) * w_dkv; k_h = [W_uk c | turn(kr)], v_h = W_uv c;
                 turned pairs are (i, i + dims/2) inside the turned part; causal softmax of scale q.k;
                 the heads side by side times sigmoid(W_g y), element by element; W_o
* 'attention':   q = W_q y (H heads), k = W_k y (G heads), v = k as projected; pairs (2i, 2i + 1) of the first rot.dims
                 features of q and k turn; then every head of q and k is divided by its root mean square;
                 query i sees key j <= i when i - j < mask.size or j < mask.keep_first; softmax of scale q.k;
                 head h times sigmoid(W_g y)[h]; W_o
* 'mlstm':       q = W_q y / sqrt(dim), k = W_k y, v = W_v y; per head i = cap tanh((W_i y + b_i) / cap),
                 f = logsigmoid(cap tanh((W_f y + b_f) / cap)); m' = max(f + m, i);
                 C <- e^(f + m - m') C + e^(i - m') k v^T, n likewise with k alone; o = C^T q / (max(|n.q|, e^(-m')) + 1e-6);
                 m, C, n start at 0; o per head divided by its root mean square, the heads side by side times w_norm
                 times sigmoid(W_g y); W_o
* feed-forward:  z = W_r y, s = softmax(z) over experts + identity entries; the `top` largest s + correction are chosen;
                 w_e = s_e / (sum of chosen s + 1e-20); expert(y) = W_down (silu(W_gate y) * (W_up y)); the last `identity`
                 entries return y itself;  ff(y) = sum_chosen w_e expert_e(y) + sigmoid(w_sg . y) shared(y)
* output:        x = sum_s x_s;  logits = head N(x) * logit_scale
"""
from __future__ import annotations

import math

import torch

from .gemma2_plain import load_folder  # noqa: F401  (the folder reader: config dict and float64 tensors)

F = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def turn_halves(x, pos, base, dims):
    """x [T, n, d]: feature i of the first `dims` turns with feature i + dims/2 by pos * base^(-2i/dims)."""
    out = x.clone()
    half = dims // 2
    for i in range(half):
        a = pos.to(F) * base ** (-2.0 * i / dims)
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def turn_neighbours(x, pos, base, dims):
    """x [T, n, d]: feature 2i of the first `dims` turns with feature 2i + 1 by pos * base^(-2i/dims)."""
    out = x.clone()
    for i in range(dims // 2):
        a = pos.to(F) * base ** (-2.0 * i / dims)
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def softmax_attend(q, k, v, scale, seen):
    """q [T, H, d], k [T, H, d], v [T, H, dv], seen(i, j) -> bool: o [T, H, dv], query after query."""
    T, H, _ = q.shape
    o = torch.zeros(T, H, v.shape[-1], dtype=F)
    for i in range(T):
        js = torch.tensor([j for j in range(i + 1) if seen(i, j)])
        s = (k[js] * q[i]).sum(-1) * scale                  # [keys, H]
        p = torch.softmax(s, 0)
        o[i] = (p[:, :, None] * v[js]).sum(0)
    return o


def latent_attention(y, t, p, m, eps):
    T = y.shape[0]
    H, d, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms(y @ t[p + ".dq"].T, eps) * t[p + ".dq.norm"]
    q = (cq @ t[p + ".uq"].T).view(T, H, d + dr)
    ckr = y @ t[p + ".dkv"].T
    c = rms(ckr[:, :R], eps) * t[p + ".dkv.norm"]
    kr = ckr[:, R:].view(T, 1, dr)
    if dr:
        q = torch.cat([q[..., :d], turn_halves(q[..., d:], pos, m["rot"]["base"], m["rot"]["dims"])], -1)
        kr = turn_halves(kr, pos, m["rot"]["base"], m["rot"]["dims"])
    k = torch.cat([(c @ t[p + ".uk"].T).view(T, H, d), kr.expand(T, H, dr)], -1)
    v = (c @ t[p + ".uv"].T).view(T, H, dv)
    o = softmax_attend(q, k, v, m["scale"], lambda i, j: True)
    o = o.reshape(T, H * dv) * torch.sigmoid(y @ t[p + ".g"].T)
    return o @ t[p + ".o"].T


def window_seen(size, keep_first):
    return lambda i, j: (size <= 0 or i - j < size) or j < keep_first


def window_attention(y, t, p, m, eps):
    T = y.shape[0]
    H, G, d = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
    pos = torch.arange(T)
    q = (y @ t[p + ".q"].T).view(T, H, d)
    k = (y @ t[p + ".k"].T).view(T, G, d)
    v = k.clone()
    rot = m.get("rot")
    if rot and rot.get("dims", 0):
        q = turn_neighbours(q, pos, rot["base"], rot["dims"])
        k = turn_neighbours(k, pos, rot["base"], rot["dims"])
    q, k = rms(q, eps), rms(k, eps)
    rep = H // G
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(rep, dim=1)
    mask = m.get("mask") or {}
    o = softmax_attend(q, kk, vv, m["scale"], window_seen(mask.get("size", 0), mask.get("keep_first", 0)))
    o = o * torch.sigmoid(y @ t[p + ".g"].T)[:, :, None]
    return o.reshape(T, H * d) @ t[p + ".o"].T


def capped(z, cap):
    return cap * torch.tanh(z / cap)


def mlstm(y, t, p, m, eps):
    T = y.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (y @ t[p + ".q"].T).view(T, H, d) / math.sqrt(d)
    k = (y @ t[p + ".k"].T).view(T, H, d)
    v = (y @ t[p + ".v"].T).view(T, H, dv)
    gi = capped(y @ t[p + ".i"].T + t[p + ".i.b"], cap)
    gf = torch.nn.functional.logsigmoid(capped(y @ t[p + ".f"].T + t[p + ".f.b"], cap))
    C = torch.zeros(H, d, dv, dtype=F)
    n = torch.zeros(H, d, dtype=F)
    mm = torch.zeros(H, dtype=F)
    o = torch.zeros(T, H, dv, dtype=F)
    for s in range(T):
        new = torch.maximum(gf[s] + mm, gi[s])
        keep = torch.exp(gf[s] + mm - new)
        take = torch.exp(gi[s] - new)
        C = keep[:, None, None] * C + take[:, None, None] * k[s][:, :, None] * v[s][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[s]
        mm = new
        num = torch.einsum("hdv,hd->hv", C, q[s])
        den = torch.maximum((n * q[s]).sum(-1).abs(), torch.exp(-mm)) + 1e-6
        o[s] = num / den[:, None]
    o = rms(o, eps).reshape(T, H * dv) * t[p + ".norm"] * torch.sigmoid(y @ t[p + ".g"].T)
    return o @ t[p + ".o"].T


def expert(y, t, p):
    return (silu(y @ t[p + ".gate"].T) * (y @ t[p + ".up"].T)) @ t[p + ".down"].T


def route(z, correction, top):
    """z [T, n]: the chosen entries [T, top] and their weights."""
    s = torch.softmax(z, -1)
    chosen = torch.topk(s + correction, top, dim=-1).indices
    w = torch.gather(s, 1, chosen)
    return chosen, w / (w.sum(-1, keepdim=True) + 1e-20)


def experts(y, t, p, f):
    r = f["router"]
    E, I, top = r["experts"], r.get("identity", 0), r["top"]
    chosen, w = route(y @ t[p + ".router"].T, t[p + ".correction"], top)
    out = torch.zeros_like(y)
    for i in range(y.shape[0]):
        for e, we in zip(chosen[i].tolist(), w[i]):
            out[i] += we * (expert(y[i:i + 1], t, f"{p}.e{e}")[0] if e < E else y[i])
    if f.get("shared"):
        out = out + torch.sigmoid(y @ t[p + ".shared.sg"].T) * expert(y, t, p + ".shared")
    return out


MIXERS = {"latent_attention": latent_attention, "attention": window_attention, "mlstm": mlstm}


def forward(cfg: dict, t: dict, tokens, layers_out: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from position 0; `layers_out` receives the sum of the streams after every layer."""
    eps = cfg["norm"]["eps"]
    S = cfg.get("streams")
    x0 = t["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    xs = [x0.clone() for _ in range(S or 1)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        subs = [(1, lambda y: MIXERS[layer["type"]](y, t, p + ".mix", layer["mixer"], eps))]
        if layer.get("mlp"):
            subs.append((2, lambda y: experts(y, t, p + ".mlp", layer["mlp"])))
        for qn, fn in subs:
            if S:
                a, b, M = t[f"{p}.hc{qn}.in"], t[f"{p}.hc{qn}.out"], t[f"{p}.hc{qn}.mix"]
                u = sum(a[s] * xs[s] for s in range(S))
                y = fn(norm(u, t[f"{p}.norm{qn}"], eps))
                xs = [sum(M[s, k] * xs[s] for s in range(S)) + b[k] * y for k in range(S)]
            else:
                xs = [xs[0] + fn(norm(xs[0], t[f"{p}.norm{qn}"], eps))]
        if layers_out is not None:
            layers_out.append(sum(xs))
    x = sum(xs)
    return norm(x, t["final.norm"], eps) @ t["head"].T * cfg.get("logit_scale", 1.0)
