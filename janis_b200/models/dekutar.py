"""Dekutar as an arrangement of parts.

A decoder whose layers are listed in the configuration.  With `streams` the residual stream has that many copies
and every sublayer reads and writes them through hyper-connections (`HyperConnectionBlock`); without, a layer is
the plain pre-norm one (`PreNormBlock`).  The norms are RMS norms whose weight is stored around zero (1 + w).  Each
layer has one of three mixers and a mixture of experts as its feed-forward, or none:

* "latent_attention": `LatentAttention` with the queries through a compressed row of their own, the rotated part
  turned by halves, no window, no sink, and a gate per feature of the heads side by side.
* "attention": `TalkingHeadsAttention` without head mixing or sink: grouped heads whose values are the keys as
  projected, neighbouring pairs of the first `rot.dims` features turned, queries and keys divided by their root mean
  square after the turn, a sliding window that keeps the sequence's first positions, and a gate per head.
* "mlstm": `MatrixMemory`.
* feed-forward: `RoutedExperts` with softmax scores over experts and identity entries, plain silu experts and a
  gated shared expert.

Tensor names: `embed`, `l<i>.norm1|norm2`, `l<i>.hc1|hc2.in|out|mix`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.
The embedding constant multiplies in float32; the head is a table of its own whose logits are multiplied by
`logit_scale`.
"""
from __future__ import annotations

from ..config.dekutar import DekutarConfig
from ..engine.model import DecoderModel, LayerCall
from ..parts import registry as parts
from ..registry import register_architecture


def _latent(W, p, m, eps):
    position = None
    if m.rot_dim:
        position = parts.make("position", "rotary", head_dim=m.rot_dim, base=m.rot_base, rotary_dims=m.rot_dims, pairs="halves")
    names = {"dq": f"{p}.dq", "dq_norm": f"{p}.dq.norm", "uq": f"{p}.uq", "dkv": f"{p}.dkv", "dkv_norm": f"{p}.dkv.norm",
             "uk": f"{p}.uk", "uv": f"{p}.uv", "g": f"{p}.g", "o": f"{p}.o"}
    return parts.make("mixer", "latent_attention", hidden=W, n_heads=m.heads, key_dim=m.dim, rot_dim=m.rot_dim,
                      value_dim=m.vdim, rank=m.kv_rank, q_rank=m.q_rank, scale=m.scale, window=0, sink=False, norm_eps=eps,
                      position=position, gate="element", names=names)


def _window(W, p, m, eps):
    position = parts.make("position", "rotary", head_dim=m.dim, base=m.rot_base, rotary_dims=m.rot_dims, pairs="neighbours")
    return parts.make("mixer", "talking_heads_attention", hidden=W, n_heads=m.heads, n_kv_heads=m.kv_heads, key_dim=m.dim,
                      value_dim=m.vdim, scale=m.scale, window=m.window, keep_first=m.keep_first, sink=False,
                      values_from_keys=True, unit_norm_eps=eps, gate="head", position=position,
                      names={k: f"{p}.{k}" for k in ("q", "k", "g", "o")})


def _matrix_memory(W, p, m, eps):
    return parts.make("mixer", "matrix_memory", hidden=W, n_heads=m.heads, key_dim=m.dim, value_dim=m.vdim,
                      gate_cap=m.gate_cap, norm_eps=eps,
                      names={"q": f"{p}.q", "k": f"{p}.k", "v": f"{p}.v", "g": f"{p}.g", "o": f"{p}.o", "i": f"{p}.i",
                             "i_bias": f"{p}.i.b", "f": f"{p}.f", "f_bias": f"{p}.f.b", "norm": f"{p}.norm"})


_MIXERS = {"latent_attention": _latent, "attention": _window, "mlstm": _matrix_memory}


def _experts(W, p, f):
    names = {"router": f"{p}.router", "correction": f"{p}.correction", "expert": p + ".e{e}.{w}"}
    if f.shared_ff:
        names.update(shared=p + ".shared.{w}", shared_gate=f"{p}.shared.sg")
    return parts.make("feed_forward", "routed_experts", hidden=W, n_experts=f.experts, n_identity=f.identity, top=f.top,
                      expert_ff=f.expert_ff, limit=0.0, scale=1.0, shared_ff=f.shared_ff, score="softmax", act="silu",
                      names=names)


def build_dekutar(cfg: DekutarConfig) -> DecoderModel:
    W, S, eps = cfg.width, cfg.streams, cfg.norm_eps

    def norm(name, in_name=None):
        if S:
            return parts.make("norm", "hyper_read", width=W, copies=S, eps=eps, weight_name=name, in_name=in_name, offset=1.0)
        return parts.make("norm", "rms_norm", width=W, eps=eps, weight_name=name, offset=1.0)

    blocks = []
    # what a folder may carry without its model using it: the second sublayer's norm and maps of a layer that has no
    # feed-forward, and maps of copies in a model with one stream and the plain sum
    unused = [] if S else ["l*.hc1.*", "l*.hc2.*"]
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}"
        mixer = _MIXERS[layer.type](W, f"{p}.mix", layer.mixer, eps)
        ff = _experts(W, f"{p}.mlp", layer.mlp) if layer.mlp is not None else None
        if ff is None:
            unused += [f"{p}.norm2", f"{p}.hc2.*"]
        if S:
            names = {"mix1": f"{p}.hc1.mix", "out1": f"{p}.hc1.out"}
            if ff is not None:
                names.update(mix2=f"{p}.hc2.mix", out2=f"{p}.hc2.out")
            blocks.append(parts.make("block", "hyper_connections", mixer=mixer, feed_forward=ff,
                                     mixer_read=norm(f"{p}.norm1", f"{p}.hc1.in"),
                                     ff_read=norm(f"{p}.norm2", f"{p}.hc2.in") if ff is not None else None, names=names))
        else:
            blocks.append(parts.make("block", "pre_norm", mixer=mixer, feed_forward=ff, input_norm=norm(f"{p}.norm1"),
                                     pre_ff_norm=norm(f"{p}.norm2") if ff is not None else None))
    return DecoderModel(
        cfg,
        embedding=parts.make("embedding", "scaled_table", vocab=cfg.vocab, hidden=W, table_name="embed",
                             scale=cfg.embedding_scale, round_scale=False, init_std=1.0, copies=S or 1),
        blocks=blocks,
        final_norm=norm("final.norm"),          # with copies: their plain sum, then the norm
        head=parts.make("head", "capped_linear", vocab=cfg.vocab, hidden=W, table_name="head", softcap=0.0,
                        scale=cfg.logit_scale, init_std=W ** -0.5),
        schedule=[LayerCall(i, i) for i in range(len(blocks))],
        ignorable_tensors=unused,
        max_context=1 << 20)


register_architecture("Dekutar", DekutarConfig, build_dekutar, model_types=("dekutar",), replace=True)
