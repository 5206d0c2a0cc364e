"""Plain torch statements of what each CUDA kernel computes, with the kernels' signatures.

Two uses, both in tests only: the `-m gpu` tests compare each kernel with the
function of the same name here; the CPU tests hand this module to the engine in
place of the kernels, which checks the host side (batching, cache bookkeeping,
schedules) against the plain model without a GPU.  Sums run in float64.
"""
from __future__ import annotations

import math

import numpy as np
import torch

PAGE = 64
GEMV_MAX_ROWS = 64
GEMV_FAST_ROWS = 16
EPI_NONE, EPI_GATED_GELU, EPI_SOFTCAP, EPI_GATED_SILU = 0, 1, 2, 3
GATE_GROUP = 8
ACT_GELU_TANH, ACT_SILU = 0, 1


def embed(tokens, table, scale, out):
    out.copy_((table[tokens.long()].double() * float(np.float32(scale))).to(out.dtype))
    return out


def _norm(x, w, eps):
    x = x.double()
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w.double()


def rmsnorm(x, weight, eps, out, rows=None):
    src = x if rows is None else x[rows.long()]
    out.copy_(_norm(src, weight, eps).to(out.dtype))
    return out


def add_rmsnorm(h, res, w_post, eps_post, w_next=None, eps_next=0.0, out=None, n_part=1):
    r = res.double()
    if n_part > 1:
        r = r.sum(0)
    add = _norm(r, w_post, eps_post) if w_post is not None else r
    h.copy_((h.double() + add).float())
    if w_next is not None:
        out.copy_(_norm(h, w_next, eps_next).to(out.dtype))
    return out


def _act(g, act):
    if act == ACT_GELU_TANH:
        return 0.5 * g * (1.0 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))
    return g / (1.0 + torch.exp(-g))


def gated_act(gu, out, act=ACT_GELU_TANH, group=GATE_GROUP):
    R, I2 = gu.shape
    I = I2 // 2
    v = gu.double().view(R, I // group, 2, group)
    out.copy_((_act(v[:, :, 0], act) * v[:, :, 1]).reshape(R, I).to(out.dtype))
    return out


def rope_store(qkv, tok_pos, tok_seq, seq_slot, seq_end, inv_freq, rot, nq, nkv, hd, kpool=None, vpool=None,
               page_table=None, ring_len=0, store=True, write_cache=True):
    T = qkv.shape[0]
    half = rot // 2
    n_rot = nq + nkv if store else nq
    if half:
        theta = (tok_pos[:T].float()[:, None] * inv_freq.float()[None, :]).float()      # float32 angles
        c, s = torch.cos(theta.double())[:, None, :], torch.sin(theta.double())[:, None, :]
        a, b = qkv[:, :n_rot, :half].double(), qkv[:, :n_rot, half:rot].double()
        qkv[:, :n_rot, :half] = (a * c - b * s).to(qkv.dtype)
        qkv[:, :n_rot, half:rot] = (a * s + b * c).to(qkv.dtype)
    if not store or not write_cache:
        return qkv
    return kv_store(qkv, tok_pos, tok_seq, seq_slot, seq_end, nq, nkv, hd, kpool, vpool, page_table, ring_len)


def kv_store(qkv, tok_pos, tok_seq, seq_slot, seq_end, nq, nkv, hd, kpool, vpool, page_table, ring_len=0):
    T = qkv.shape[0]
    for t in range(T):
        seq = int(tok_seq[t])
        slot = int(seq_slot[seq])
        if slot < 0:
            continue
        pos = int(tok_pos[t])
        idx = pos
        if ring_len > 0:
            if pos < int(seq_end[seq]) - ring_len:
                continue
            idx = pos % ring_len
        page = int(page_table[slot, idx // PAGE])
        kpool[page, :, idx % PAGE, :] = qkv[t, nq:nq + nkv]
        vpool[page, :, idx % PAGE, :] = qkv[t, nq + nkv:nq + 2 * nkv]
    return qkv


def gemv_rope_store(x, w, qkv, tok_pos, tok_seq, seq_slot, seq_end, inv_freq, nq, nkv, hd, kpool=None, vpool=None,
                    page_table=None, ring_len=0, store=True):
    heads = nq + 2 * nkv if store else nq
    M = x.shape[0]
    full = (x.double() @ w.double().T).to(qkv.dtype).view(M, heads, hd)
    rope_store(full, tok_pos, tok_seq, seq_slot, seq_end, inv_freq, hd, nq, nkv, hd, kpool, vpool, page_table,
               ring_len, store)
    qkv[:, :nq] = full[:, :nq]
    return qkv


def gemm_f32(x, w, out, cap=0.0):
    v = x.double() @ w.double().T
    if cap > 0:
        v = cap * torch.tanh(v / cap)
    out.copy_(v.to(out.dtype))
    return out


def gemv_bf16(x, w, out, epilogue=EPI_NONE, cap=0.0, cluster=0):
    v = x.double() @ w.double().T
    if epilogue in (EPI_GATED_GELU, EPI_GATED_SILU):
        M, N = v.shape
        g = v.view(M, N // 16, 2, 8)
        v = (_act(g[:, :, 0], ACT_GELU_TANH if epilogue == EPI_GATED_GELU else ACT_SILU) * g[:, :, 1]).reshape(M, N // 2)
    elif epilogue == EPI_SOFTCAP and cap > 0:
        v = cap * torch.tanh(v / cap)
    out.copy_(v.to(out.dtype))
    return out


def matmul_bf16_to_f32(x, w, out):
    out.copy_((x.double() @ w.double().T).float())
    return out


def softcap(x, cap):
    x.copy_((cap * torch.tanh(x.double() / cap)).float())
    return x


TC05_MAX_ROWS = 64


def gemm_tc05(x, w, out, epilogue=EPI_NONE, cap=0.0, split=0):
    return gemv_bf16(x, w, out, epilogue, cap)


def linear_bf16(x, w, out):
    return gemv_bf16(x, w, out)


def _attend(q, k, v, scale, cap):
    """q [nq, hd], k/v [n, nkv, hd] (all visible) -> [nq, hd], float64."""
    nq, nkv = q.shape[0], k.shape[1]
    rep = nq // nkv
    out = torch.empty(nq, q.shape[1], dtype=torch.float64)
    for h in range(nq):
        s = (k[:, h // rep].double() @ q[h].double()) * scale
        if cap > 0:
            s = cap * torch.tanh(s / cap)
        p = torch.softmax(s, dim=0)
        out[h] = p @ v[:, h // rep].double()
    return out


def attn_prefill_scratch_floats(n_tok, n_seq, nq, hd, dtype=torch.bfloat16):
    return 0


def attn_prefill(qkv, tok_pos, tok_seq, seq_first_row, out, nq, nkv, hd, scale, cap, window, kv_src=None,
                 kv_row_heads=None, kv_k_head0=None, seq_len=None, tensor_cores=True, scratch=None, seq_start=None,
                 seq_slot=None, kpool=None, vpool=None, page_table=None, ring_len=0, host_lens=None):
    T = qkv.shape[0]
    if kv_src is None:
        kv_src, kv_k_head0 = qkv, nq
    for t in range(T):
        pos = int(tok_pos[t])
        seq = int(tok_seq[t])
        start = int(seq_start[seq]) if seq_start is not None else 0
        first = int(seq_first_row[seq]) - start           # the row position 0 would have
        lo = max(0, pos - window + 1) if window > 0 else 0
        ks, vs = [], []
        if lo < start:                                    # keys and values that earlier steps stored
            slot = int(seq_slot[seq])
            idx = [(j % ring_len if ring_len > 0 else j) for j in range(lo, start)]
            pages = [int(page_table[slot, i // PAGE]) for i in idx]
            ks.append(torch.stack([kpool[p, :, i % PAGE] for p, i in zip(pages, idx)]).cpu())
            vs.append(torch.stack([vpool[p, :, i % PAGE] for p, i in zip(pages, idx)]).cpu())
        rows = kv_src[first + max(lo, start):first + pos + 1]
        ks.append(rows[:, kv_k_head0:kv_k_head0 + nkv].cpu())
        vs.append(rows[:, kv_k_head0 + nkv:kv_k_head0 + 2 * nkv].cpu())
        o = _attend(qkv[t, :nq].cpu(), torch.cat(ks), torch.cat(vs), scale, cap)
        out[t] = o.reshape(-1).to(out.dtype)
    return out


def attn_decode_scratch_floats(n_seq, nq, hd, max_chunks):
    return n_seq * nq * max_chunks * (hd + 2)


def attn_decode(qkv, kpool, vpool, page_table, seq_slot, seq_len, scratch, out, nq, nkv, hd, scale, cap, window,
                ring_len, chunk, max_chunks):
    n_seq = qkv.shape[0]
    for s in range(n_seq):
        slot = int(seq_slot[s])
        if slot < 0:
            out[s] = 0
            continue
        n = int(seq_len[s])
        lo = max(0, n - window) if window > 0 else 0
        first_chunk = lo // chunk
        if (n + chunk - 1) // chunk - first_chunk > max_chunks:
            out[s] = float("nan")
            continue
        idx = [(j % ring_len if ring_len > 0 else j) for j in range(lo, n)]
        pages = [int(page_table[slot, i // PAGE]) for i in idx]
        offs = [i % PAGE for i in idx]
        k = torch.stack([kpool[p, :, o] for p, o in zip(pages, offs)]).cpu()
        v = torch.stack([vpool[p, :, o] for p, o in zip(pages, offs)]).cpu()
        out[s] = _attend(qkv[s, :nq].cpu(), k, v, scale, cap).reshape(-1).to(out.dtype)
    return out


def argmax(logits, out):
    for r in range(logits.shape[0]):
        row = logits[r]
        out[r] = int((row == row.max()).nonzero()[0])
    return out


_M0, _M1 = 0xD2511F53, 0xCD9E8D57


def philox_uniform(seed, request, index):
    """Philox4x32-10 with key = seed (two words) and counter = (request, index, 0, 0); first word -> [0, 1)."""
    c = [request & 0xFFFFFFFF, index & 0xFFFFFFFF, 0, 0]
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = _M0 * c[0], _M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k0) & 0xFFFFFFFF, p1 & 0xFFFFFFFF, ((p0 >> 32) ^ c[3] ^ k1) & 0xFFFFFFFF,
             p0 & 0xFFFFFFFF]
        k0 = (k0 + 0x9E3779B9) & 0xFFFFFFFF
        k1 = (k1 + 0xBB67AE85) & 0xFFFFFFFF
    return float(np.float32(c[0] >> 8) * np.float32(1.0 / 16777216.0))


def sample_row(row, temp, top_p, u):
    """The choice for one row given its uniform number: float64 throughout."""
    l = row.double()
    w = torch.exp((l - l.max()) / temp)
    p = (w / w.sum()).tolist()
    if 0.0 < top_p < 1.0:
        order = sorted(range(len(p)), key=lambda i: (-p[i], i))
        keep, cum = [], 0.0
        for i in order:
            keep.append(i)
            cum += p[i]
            if cum >= top_p:
                break
        keep.sort()
    else:
        keep = list(range(len(p)))
    mass = sum(p[i] for i in keep)
    target, acc = u * mass, 0.0
    for i in keep:
        acc += p[i]
        if target <= acc:
            return i
    return keep[-1]


def sample(logits, out, temp, top_p, seed, request_ids, token_index, u_out=None):
    for r in range(logits.shape[0]):
        u = philox_uniform(int(seed), int(request_ids[r]), int(token_index[r]))
        if u_out is not None:
            u_out[r] = u
        out[r] = sample_row(logits[r].cpu(), temp, top_p, u)
    return out


def repeat_penalty(logits, recent, penalty):
    for r in range(logits.shape[0]):
        for tok in set(int(t) for t in recent[r].tolist() if 0 <= int(t) < logits.shape[1]):
            v = logits[r, tok]
            logits[r, tok] = v / penalty if v > 0 else v * penalty
    return logits


def mask_tokens(logits, ids):
    for tok in ids.tolist():
        if 0 <= tok < logits.shape[1]:
            logits[:, tok] = float("-inf")
    return logits


# ---------------------------------------------------------------------------
# mixers with run-time sizes
# ---------------------------------------------------------------------------

ACT_NONE, ACT_XIELU, ACT_GELU, ACT_SILU_PLAIN, ACT_RELU2 = 0, 1, 2, 3, 4


def bias_act(x, bias, act=ACT_NONE, a_pos=0.0, a_neg=0.0):
    z = x.double()
    if bias is not None:
        z = z + bias.double()
    if act == ACT_XIELU:
        z = torch.where(z > 0, a_pos * z * z + 0.5 * z, a_neg * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z)
    elif act == ACT_GELU:
        z = _act(z, ACT_GELU_TANH)
    elif act == ACT_SILU_PLAIN:
        z = _act(z, ACT_SILU)
    elif act == ACT_RELU2:
        z = torch.clamp(z, min=0.0) ** 2
    x.copy_(z.to(x.dtype))
    return x


def gemv_bf16_bias_act(x, w, out, bias, act=ACT_NONE, a_pos=0.0, a_neg=0.0):
    out.copy_((x.double() @ w.double().T).to(out.dtype))
    return bias_act(out, bias, act, a_pos, a_neg)


def _turn(x, pos, inv, sign=1.0):
    """x [..., n] rotated by sign * pos * inv over pairs (i, i + len(inv)); angles float32 as the kernels form them."""
    h = inv.numel()
    if h == 0:
        return x
    theta = (torch.as_tensor(float(pos), dtype=torch.float32) * inv.float()).double()
    c, s = torch.cos(theta), sign * torch.sin(theta)
    a, b = x[..., :h].double(), x[..., h:2 * h].double()
    return torch.cat([a * c - b * s, a * s + b * c, x[..., 2 * h:].double()], dim=-1)


def qkv_rotate_store(rows, tok_pos, tok_seq, seq_slot, inv_qk, rot, inv_v, H, G, d, dv, kpool=None, vpool=None,
                     page_table=None, store=True):
    T = rows.shape[0]
    for t in range(T):
        pos = int(tok_pos[t])
        n = H + G if store else H
        qk = rows[t, :n * d].view(n, d)
        qk.copy_(_turn(qk, pos, inv_qk).to(rows.dtype))
        if not store:
            continue
        v = rows[t, n * d:n * d + G * dv].view(G, dv)
        if inv_v is not None:
            v.copy_(_turn(v, pos, inv_v).to(rows.dtype))
        slot = int(seq_slot[int(tok_seq[t])])
        if slot < 0:
            continue
        page = int(page_table[slot, pos // PAGE])
        kpool[page, :, pos % PAGE] = qk[H:]
        vpool[page, :, pos % PAGE] = v
    return rows


def talk_attention(q_rows, tok_pos, tok_seq, seq_slot, kpool, vpool, page_table, talk, inv_v, out, H, G, d, dv, scale,
                   block=0, sink=False, one_row=False, max_keys=0, n_chunks=1, scratch=None, window=0, cap=0.0,
                   sink_values=None, mix_after=False, values_in_keys=False, stats=None, keep_first=0):
    T = q_rows.shape[0]
    rep = H // G
    for t in range(T):
        pos, slot = int(tok_pos[t]), int(seq_slot[int(tok_seq[t])])
        if slot < 0:
            out[t] = 0
            continue
        first = (pos // block) * block if block > 0 else 0
        if window > 0:
            first = max(first, pos - window + 1)
        js = list(range(min(keep_first, first) if window > 0 else 0)) + list(range(first, pos + 1))
        pages = [int(page_table[slot, j // PAGE]) for j in js]
        k = torch.stack([kpool[p, :, j % PAGE] for p, j in zip(pages, js)]).double()       # [n, G, d]
        v = k[..., :dv] if values_in_keys else torch.stack([vpool[p, :, j % PAGE] for p, j in zip(pages, js)]).double()
        q = q_rows[t, :H * d].view(H, d).double()
        raw = torch.einsum("hd,nhd->hn", q, k.repeat_interleave(rep, dim=1)) * scale
        if cap:
            raw = cap * torch.tanh(raw / cap)
        s = talk.double() @ raw if talk is not None and not mix_after else raw
        z = sink_values.double()[:, None] if sink_values is not None else torch.zeros(H, 1, dtype=torch.float64)
        m = torch.maximum(s.max(dim=1, keepdim=True).values, z)
        e = torch.exp(s - m)
        p = e / ((torch.exp(z - m) if sink else 0.0) + e.sum(dim=1, keepdim=True))
        if talk is not None and mix_after:
            p = talk.double() @ p
        o = torch.einsum("hn,nhv->hv", p, v.repeat_interleave(rep, dim=1))
        if inv_v is not None:
            o = _turn(o, pos, inv_v, sign=-1.0)
        out[t] = o.reshape(-1).to(out.dtype)
    return out


def talk_attention_scratch_floats(T, n_chunks, H, dv):
    return T * n_chunks * H * (dv + 2) if n_chunks > 1 else 0


def talk_attention_stats_floats(T, H):
    return 2 * T * H


def talk_attention_rows_floats(dtype, T, H, G, d, dv, max_keys):
    """Scratch for the kernels that take single rows: one float, so that the plain statement is the one that runs."""
    return 1


def talk_attention_rows(q_rows, tok_pos, tok_seq, seq_slot, kpool, vpool, page_table, talk, out, H, G, d, dv, scale, scratch,
                        max_keys, sink=False, window=0, cap=0.0, sink_values=None, values_in_keys=False, keep_first=0):
    """The same mathematics as `talk_attention` with the heads mixed after the softmax."""
    return talk_attention(q_rows, tok_pos, tok_seq, seq_slot, kpool, vpool, page_table, talk, None, out, H, G, d, dv, scale,
                          0, sink, window=window, cap=cap, sink_values=sink_values, mix_after=True,
                          values_in_keys=values_in_keys, keep_first=keep_first)


def gla_scan(rows, q_off, k_off, v_off, z, z_bias, seq_slot, seq_first_row, seq_start, seq_end, state, o_out, n_seq, H,
             d, dv, q_scale, tau, decay=None):
    for s in range(n_seq):
        slot, row0, n = int(seq_slot[s]), int(seq_first_row[s]), int(seq_end[s]) - int(seq_start[s])
        if n <= 0:
            continue
        S = state[slot].double().transpose(1, 2).clone() if slot >= 0 else torch.zeros(H, d, dv, dtype=torch.float64)
        for t in range(row0, row0 + n):
            row = rows[t].double()
            q = row[q_off:q_off + H * d].view(H, d) * q_scale
            k = row[k_off:k_off + H * d].view(H, d)
            v = row[v_off:v_off + H * dv].view(H, dv)
            a = torch.exp(torch.nn.functional.logsigmoid(z[t].double() + z_bias.double()) / tau).view(H, d)
            S = a[:, :, None] * S + k[:, :, None] * v[:, None, :]
            o_out[t] = torch.einsum("hdv,hd->hv", S, q).reshape(-1).float()
        if slot >= 0:
            state[slot] = S.transpose(1, 2).float()          # stored [H, dv, d]
    return o_out


def head_norm_gate(o, rows, g_off, weight, eps, out, H, dv, gate="silu"):
    T = o.shape[0]
    x = o.double().view(T, H, dv)
    w = weight.double().view(H, dv) if weight.numel() == H * dv and H > 1 else weight.double()
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w
    if rows is not None:
        g = rows[:, g_off:g_off + H * dv].double().view(T, H, dv)
        y = y * torch.sigmoid(g) * (g if gate == "silu" else 1.0)
    out.copy_(y.reshape(T, H * dv).to(out.dtype))
    return out


# ---------------------------------------------------------------------------
# Dynamic Tanh, state-space mixers, parallel branches, mixture of experts
# ---------------------------------------------------------------------------

def dyt_norm(h, res, alpha, weight, bias, out, rows=None):
    """h += res (when given; float32 in place), then out = tanh(alpha h) * weight + bias over the rows asked for."""
    if res is not None:
        h.copy_((h.double() + res.double()).float())
    src = h if rows is None else h[rows.long()]
    out.copy_((torch.tanh(float(np.float32(alpha)) * src.double()) * weight.double() + bias.double()).to(out.dtype))
    return out


def causal_conv_silu(rows, col_off, channels, weight, bias, state, tok_seq, seq_slot, seq_first_row, seq_start, seq_end,
                     n_seq, out, one_token=False, act=True):
    taps = weight.shape[1]
    w, b = weight.double(), bias.double() if bias is not None else torch.zeros(channels, dtype=torch.float64)
    for s in range(n_seq):
        slot, row0, n = int(seq_slot[s]), int(seq_first_row[s]), int(seq_end[s]) - int(seq_start[s])
        if n <= 0:
            continue
        x = rows[row0:row0 + n, col_off:col_off + channels].double()
        past = state[slot, :taps - 1].double() if slot >= 0 else torch.zeros(taps - 1, channels, dtype=torch.float64)
        full = torch.cat([past, x], dim=0)                                  # local index i lives at i + taps - 1
        acc = b.expand(n, channels).clone()
        for j in range(taps):
            acc += w[:, taps - 1 - j] * full[taps - 1 - j:taps - 1 - j + n]
        out[row0:row0 + n] = (acc * torch.sigmoid(acc) if act else acc).to(out.dtype)
        if slot >= 0 and taps > 1:
            state[slot, :taps - 1] = full[n:n + taps - 1].float()
    return out


def selective_scan(u, u_off, dt, dt_off, dt_bias, A, a_per_state, bc, b_off, c_off, D, z, z_off, seq_slot, seq_first_row,
                   seq_start, seq_end, n_seq, state, out, C, N, ch_per_head, ch_per_group, scratch=None):
    heads = C // ch_per_head
    Af = A.double() if a_per_state else A.double()[:, None].expand(heads, N)
    Ac = Af.repeat_interleave(ch_per_head, dim=0)                           # [C, N]
    Dc = D.double().repeat_interleave(ch_per_head)
    for s in range(n_seq):
        slot, row0, n = int(seq_slot[s]), int(seq_first_row[s]), int(seq_end[s]) - int(seq_start[s])
        if n <= 0:
            continue
        S = state[slot].double().clone() if slot >= 0 else torch.zeros(C, N, dtype=torch.float64)
        for t in range(row0, row0 + n):
            raw = dt[t, dt_off:dt_off + heads].double() + dt_bias.double()
            delta = torch.logaddexp(raw, torch.zeros_like(raw)).repeat_interleave(ch_per_head)       # [C]
            x = u[t, u_off:u_off + C].double()
            groups = C // ch_per_group
            B = bc[t, b_off:b_off + groups * N].double().view(groups, N).repeat_interleave(ch_per_group, dim=0)
            Cm = bc[t, c_off:c_off + groups * N].double().view(groups, N).repeat_interleave(ch_per_group, dim=0)
            S = torch.exp(delta[:, None] * Ac) * S + (delta * x)[:, None] * B
            o = (S * Cm).sum(-1) + Dc * x
            if z is not None:
                g = z[t, z_off:z_off + C].double()
                o = o * g * torch.sigmoid(g)
            out[t] = o.to(out.dtype)
        if slot >= 0:
            state[slot] = S.float()
    return out


def selective_scan_scratch_floats(n_tok, heads):
    return 2 * n_tok * heads


def gate_group_norm(o, rows, z_off, weight, eps, n_groups, out):
    T, C = o.shape
    g = rows[:, z_off:z_off + C].double()
    x = (o.double() * g * torch.sigmoid(g)).view(T, n_groups, C // n_groups)
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    out.copy_((y.reshape(T, C) * weight.double()).to(out.dtype))
    return out


def rmsnorm_accumulate(x, weight, eps, scale, acc, first=False):
    y = _norm(x, weight, eps) * scale
    acc.copy_((y if first else acc.double() + y).float())
    return acc


def sigmoid_gate(x, rows, g_off, per=1):
    g = rows[:, g_off:g_off + x.shape[1] // per].double().repeat_interleave(per, dim=1)
    x.copy_((x.double() * torch.sigmoid(g)).to(x.dtype))
    return x


# ---------------------------------------------------------------------------
# the norm in groups after a scaled residual sum; filtered, normed and compressed attention inputs; products per head
# ---------------------------------------------------------------------------

def group_norm(h, res, alpha, weight, eps, groups, out, rows=None):
    def normed(v):
        R, H = v.shape
        g = v.view(R, groups, H // groups)
        g = g / torch.sqrt((g * g).mean(-1, keepdim=True) + eps)
        return g.reshape(R, H) * weight.double()
    if res is not None:
        v = normed(float(np.float32(alpha)) * h.double() + res.double())
        h.copy_(v.float())
        if out is not None:
            out.copy_(h.to(out.dtype))
        return out
    src = h if rows is None else h[rows.long()]
    out.copy_(normed(src.double()).to(out.dtype))
    return out


def round_rows(h, out):
    out.copy_(h.to(out.dtype))
    return out


def qkv_conv_norm_store(rows, H, G, d, dv, conv_w, conv_state, wq, wk, v_unit, eps, tok_pos, tok_seq, seq_slot,
                        seq_first_row, seq_start, seq_end, n_seq, q_out, kpool, vpool, page_table, one_token=False):
    C = H * d + G * (d + dv)
    taps = conv_w.shape[1] if conv_w is not None else 0
    for s in range(n_seq):
        slot, row0, n = int(seq_slot[s]), int(seq_first_row[s]), int(seq_end[s]) - int(seq_start[s])
        if n <= 0:
            continue
        x = rows[row0:row0 + n, :C].double()
        if taps > 1:
            past = conv_state[slot].double() if slot >= 0 else torch.zeros(taps - 1, C, dtype=torch.float64)
            full = torch.cat([past, x], dim=0)
            y = torch.zeros(n, C, dtype=torch.float64)
            for j in range(taps):
                y += conv_w.double()[:, taps - 1 - j] * full[taps - 1 - j:taps - 1 - j + n]
            if slot >= 0:
                conv_state[slot] = full[n:n + taps - 1].float()
        elif taps == 1:
            y = x * conv_w.double()[:, 0]
        else:
            y = x
        q, k, v = y[:, :H * d], y[:, H * d:H * d + G * d], y[:, H * d + G * d:].reshape(n, G, dv)
        if wq is not None:
            q = q / torch.sqrt((q * q).mean(-1, keepdim=True) + eps) * wq.double()
        if wk is not None:
            k = k / torch.sqrt((k * k).mean(-1, keepdim=True) + eps) * wk.double()
        if v_unit:
            v = v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)
        q_out[row0:row0 + n] = q.to(q_out.dtype)
        if slot < 0:
            continue
        for i in range(n):
            pos = int(tok_pos[row0 + i])
            page = int(page_table[slot, pos // PAGE])
            kpool[page, :, pos % PAGE] = k[i].view(G, d).to(kpool.dtype)
            vpool[page, :, pos % PAGE] = v[i].to(vpool.dtype)
    return q_out


def latent_rotate_store(rows, lat_off, H, d, dr, R, wc, eps, inv_freq, amp, tok_pos, tok_seq, seq_slot, qfull, kpool,
                        page_table, rot=None, q_rows=None, halves=False):
    T = rows.shape[0]
    D = R + dr
    for t in range(T):
        pos, slot = int(tok_pos[t]), int(seq_slot[int(tok_seq[t])])
        ang = float(np.float32(pos)) * inv_freq.double()
        cs, sn = torch.cos(ang) * float(np.float32(amp)), torch.sin(ang) * float(np.float32(amp))
        if rot is not None:                   # pairs from rot / 2 on pass as they are
            cs[rot // 2:], sn[rot // 2:] = 1.0, 0.0

        def turn(x):
            if halves:
                w = dr if rot is None else rot
                a, b = x[..., :w // 2], x[..., w // 2:w]
                out = x.clone()
                out[..., :w // 2] = a * cs[:w // 2] - b * sn[:w // 2]
                out[..., w // 2:w] = b * cs[:w // 2] + a * sn[:w // 2]
                return out
            a, b = x[..., 0::2], x[..., 1::2]
            out = torch.empty_like(x)
            out[..., 0::2] = a * cs - b * sn
            out[..., 1::2] = b * cs + a * sn
            return out
        row = rows[t].double()
        q = (q_rows[t].double() if q_rows is not None else row)[:H * (d + dr)].view(H, d + dr)
        qfull.view(T, H, D)[t, :, R:] = turn(q[:, d:]).to(qfull.dtype)
        if slot < 0:
            continue
        lat = row[lat_off:lat_off + D]
        c = lat[:R] / torch.sqrt((lat[:R] * lat[:R]).mean() + eps) * wc.double()
        page = int(page_table[slot, pos // PAGE])
        kpool[page, 0, pos % PAGE, :R] = c.to(kpool.dtype)
        kpool[page, 0, pos % PAGE, R:] = turn(lat[R:]).to(kpool.dtype)
    return qfull


def head_linear(x, x_head, x_off, w, out, o_head, o_off):
    Hn, O, I = w.shape
    for h in range(Hn):
        xi = x[:, h * x_head + x_off:h * x_head + x_off + I].double()
        out[:, h * o_head + o_off:h * o_head + o_off + O] = (xi @ w[h].double().T).to(out.dtype)
    return out


def moe_route(z, correction, n_experts, group_count, group_keep, top, scale, shared_gate, out, n_identity=0, softmax=False):
    T = z.shape[0]
    real = n_experts
    n_experts = real + n_identity          # the entries that are scored and chosen
    s = torch.softmax(z[:, :n_experts].double(), -1) if softmax else torch.sigmoid(z[:, :n_experts].double())
    c = s + correction.double()
    per = n_experts // group_count
    out.zero_()
    for t in range(T):
        gs = [sum(sorted(c[t, g * per:(g + 1) * per].tolist(), reverse=True)[:2]) for g in range(group_count)]
        kept = sorted(range(group_count), key=lambda g: (-gs[g], g))[:group_keep]
        cand = [e for g in sorted(kept) for e in range(g * per, (g + 1) * per)]
        chosen = sorted(cand, key=lambda e: (-float(c[t, e]), e))[:top]
        total = sum(float(s[t, e]) for e in chosen) + 1e-20
        for e in chosen:
            if e < real:
                out[t, e] = float(s[t, e]) / total * scale
            else:
                out[t, -1] += float(s[t, e]) / total * scale
    if shared_gate:
        out[:, real] = torch.sigmoid(z[:, n_experts].double()).float()
    return out


def moe_identity_add(out, y, wts, col):
    out.copy_((out.double() + wts[:, col:col + 1].double() * y.double()).to(out.dtype))
    return out


def moe_expert_act(gu, wts, n_experts, ff, limit, shared_ff, shared_limit, alpha, out, up_add=1.0):
    T = gu.shape[0]
    v = gu.double()
    E = n_experts
    g = v[:, :2 * E * ff].view(T, E, 2, ff)
    gate, up = torch.clamp(g[:, :, 0], max=limit), torch.clamp(g[:, :, 1], min=-limit, max=limit)
    a = gate * torch.sigmoid(alpha * gate) * (up + up_add) * wts[:, :E].double()[:, :, None]
    out[:, :E * ff] = a.reshape(T, E * ff).to(out.dtype)
    if shared_ff:
        sg = v[:, 2 * E * ff:].view(T, 2, shared_ff)
        gate, up = torch.clamp(sg[:, 0], max=shared_limit), torch.clamp(sg[:, 1], min=-shared_limit, max=shared_limit)
        out[:, E * ff:] = (gate * torch.sigmoid(alpha * gate) * (up + up_add) * wts[:, E:E + 1].double()).to(out.dtype)
    return out


# ---------------------------------------------------------------------------
# copies of the stream behind small maps, queries and keys turned and normed, the matrix memory, a constant on logits
# ---------------------------------------------------------------------------

def scale_values(x, factor):
    x.mul_(factor)
    return x


def hc_spread(x, h, copies):
    T, W = x.shape
    h.view(T, copies, W).copy_(x[:, None, :].expand(T, copies, W))
    return h


def hc_read_norm(h, copies, a, weight, eps, out, rows=None):
    R, W = out.shape
    x = h.double().view(-1, copies, W)
    if rows is not None:
        x = x[rows.long()]
    av = a.double() if a is not None else torch.ones(copies, dtype=torch.float64)
    u = (x * av[None, :, None]).sum(1)
    out.copy_((u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps) * weight.double()).to(out.dtype))
    return out


def hc_update(h, res, copies, mix, b, a_next=None, w_next=None, eps_next=0.0, out=None):
    T, W = res.shape
    x = h.double().view(T, copies, W)
    new = torch.einsum("sk,tsw->tkw", mix.double(), x) + b.double()[None, :, None] * res.double()[:, None, :]
    h.copy_(new.reshape(T, copies * W).float())
    if w_next is None:
        return None
    return hc_read_norm(h, copies, a_next, w_next, eps_next, out)


def qk_rotate_norm_store(rows, tok_pos, tok_seq, seq_slot, inv_freq, rot, halves, unit_norm, eps, H, G, d, kpool, vpool,
                         page_table):
    T = rows.shape[0]
    for t in range(T):
        pos, slot = int(tok_pos[t]), int(seq_slot[int(tok_seq[t])])
        heads = rows[t, :(H + G) * d].double().view(H + G, d)
        raw_k = heads[H:].clone()
        y = heads.clone()
        if rot:
            ang = float(np.float32(pos)) * inv_freq.double()[:rot // 2]
            cs, sn = torch.cos(ang), torch.sin(ang)
            if halves:
                a, b = heads[:, :rot // 2], heads[:, rot // 2:rot]
                y[:, :rot // 2], y[:, rot // 2:rot] = a * cs - b * sn, b * cs + a * sn
            else:
                a, b = heads[:, 0:rot:2], heads[:, 1:rot:2]
                y[:, 0:rot:2], y[:, 1:rot:2] = a * cs - b * sn, b * cs + a * sn
        if unit_norm:
            y = y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)
        rows[t, :H * d] = y[:H].reshape(-1).to(rows.dtype)
        if slot < 0:
            continue
        page = int(page_table[slot, pos // PAGE])
        kpool[page, :, pos % PAGE] = y[H:].to(kpool.dtype)
        if vpool is not None:
            vpool[page, :, pos % PAGE] = raw_k.to(vpool.dtype)
    return rows


def mlstm_scan(rows, q_off, k_off, v_off, z, bias, cap, seq_slot, seq_first_row, seq_start, seq_end, state_c, state_n,
               state_m, o_out, n_seq, H, d, dv, q_scale, coef):
    for s in range(n_seq):
        slot, row0, n = int(seq_slot[s]), int(seq_first_row[s]), int(seq_end[s]) - int(seq_start[s])
        if n <= 0:
            continue
        if slot >= 0:
            C = state_c[slot].double().transpose(1, 2).clone()       # stored [H, dv, d]
            nn = state_n[slot, :, 0].double().clone()
            m = state_m[slot].double().clone()
        else:
            C, nn, m = torch.zeros(H, d, dv, dtype=torch.float64), torch.zeros(H, d, dtype=torch.float64), torch.zeros(H, dtype=torch.float64)
        for t in range(row0, row0 + n):
            row = rows[t].double()
            q = row[q_off:q_off + H * d].view(H, d) * q_scale
            k = row[k_off:k_off + H * d].view(H, d)
            v = row[v_off:v_off + H * dv].view(H, dv)
            zz = z[t].double() + bias.double()
            gi = cap * torch.tanh(zz[:H] / cap)
            gf = torch.nn.functional.logsigmoid(cap * torch.tanh(zz[H:] / cap))
            m_new = torch.maximum(gf + m, gi)
            keep, take = torch.exp(gf + m - m_new), torch.exp(gi - m_new)
            C = keep[:, None, None] * C + take[:, None, None] * k[:, :, None] * v[:, None, :]
            nn = keep[:, None] * nn + take[:, None] * k
            m = m_new
            den = torch.maximum((nn * q).sum(-1).abs(), torch.exp(-m)) + 1e-6
            o_out[t] = (torch.einsum("hdv,hd->hv", C, q) / den[:, None]).reshape(-1).float()
        if slot >= 0:
            state_c[slot] = C.transpose(1, 2).float()
            state_n[slot] = nn.float()[:, None, :].expand(H, state_n.shape[2], d)
            state_m[slot] = m.float()
    return o_out
