"""Vivazen as an arrangement of parts.

A decoder whose layers are listed in the configuration, in the arrangement that norms after the sum
(`PostNormBlock`: x <- N1(a x + Mixer(x)); x <- N2(a x + FF(x)), a = postln_alpha) with RMS norms in groups, each
layer with one of two mixers and a gated dense feed-forward (tanh form of gelu), or none:

* "attention": `FilteredAttention`: grouped-query softmax attention without positions whose projections pass a
  short causal filter, are normed over the whole projection (values per head), whose scores are capped and whose
  heads' weights are mixed after the softmax.
* "latent_attention": `LatentAttention`: a compressed key/value row per position, a rotated part shared by all
  heads (neighbouring pairs, ramp-scaled frequencies), a sliding window, a sink per head in the softmax and a gate
  per head on the output.

A layer with `weights_of: j` is layer j's block run once more, with a cache line of its own: the schedule names
block j twice.  Tensor names: `embed`, `l<i>.norm1|norm2`, `l<i>.mix.*`, `l<i>.mlp.gate|up|down`, `final.norm`,
`head`.
"""
from __future__ import annotations

from ..config.vivazen import VivazenConfig
from ..engine.model import DecoderModel, LayerCall
from ..parts import registry as parts
from ..registry import register_architecture


def _filtered(W, p, m, eps):
    names = {"q": f"{p}.q", "k": f"{p}.k", "v": f"{p}.v", "o": f"{p}.o", "q_norm": f"{p}.q.norm",
             "k_norm": f"{p}.k.norm", "talk": f"{p}.talk"}
    if m.conv:
        names.update(q_conv=f"{p}.q.conv", k_conv=f"{p}.k.conv", v_conv=f"{p}.v.conv")
    return parts.make("mixer", "filtered_attention", hidden=W, n_heads=m.heads, n_kv_heads=m.kv_heads, key_dim=m.dim,
                      value_dim=m.vdim, scale=m.scale, taps=m.conv, cap=m.softcap, norm_eps=eps, names=names)


def _latent(W, p, m, eps):
    position = None
    if m.rot_dim:
        position = parts.make("position", "rotary", head_dim=m.rot_dim, base=m.rot_base, rotary_dims=m.rot_dims,
                              ramp_scaling=m.rot_scaling.to_dict() if m.rot_scaling is not None else None,
                              pairs="neighbours")
    names = {"q": f"{p}.q", "dkv": f"{p}.dkv", "dkv_norm": f"{p}.dkv.norm", "uk": f"{p}.uk", "uv": f"{p}.uv",
             "sink": f"{p}.sink", "g": f"{p}.g", "o": f"{p}.o"}
    return parts.make("mixer", "latent_attention", hidden=W, n_heads=m.heads, key_dim=m.dim, rot_dim=m.rot_dim,
                      value_dim=m.vdim, rank=m.kv_rank, scale=m.scale, window=m.window, sink=True, norm_eps=eps,
                      position=position, names=names)


def build_vivazen(cfg: VivazenConfig) -> DecoderModel:
    W = cfg.width

    def norm(name):
        return parts.make("norm", "group_rms_norm", width=W, eps=cfg.norm_eps, groups=cfg.norm_groups, weight_name=name)

    blocks, schedule = {}, []
    for i, layer in enumerate(cfg.layers):
        src = cfg.weight_layer(i)
        if src == i:
            p = f"l{i}"
            make = _filtered if layer.type == "attention" else _latent
            mixer = make(W, f"{p}.mix", layer.mixer, cfg.norm_eps)
            ff = None
            if layer.mlp is not None:
                ff = parts.make("feed_forward", "gated_mlp", hidden=W, intermediate=layer.mlp.ff, act="gelu_tanh",
                                names={k: f"{p}.mlp.{k}" for k in ("gate", "up", "down")})
            blocks[i] = parts.make("block", "post_norm", mixer=mixer, feed_forward=ff, post_mixer_norm=norm(f"{p}.norm1"),
                                   post_ff_norm=norm(f"{p}.norm2") if ff is not None else None, alpha=cfg.postln_alpha)
    order = sorted(blocks)                       # a layer that borrows tensors may stand before their owner
    index = {i: n for n, i in enumerate(order)}
    for i in range(len(cfg.layers)):
        schedule.append(LayerCall(index[cfg.weight_layer(i)], i))
    return DecoderModel(
        cfg,
        embedding=parts.make("embedding", "scaled_table", vocab=cfg.vocab, hidden=W, table_name="embed", scale=1.0,
                             round_scale=False, init_std=1.0),
        blocks=[blocks[i] for i in order],
        final_norm=norm("final.norm"),
        head=parts.make("head", "capped_linear", vocab=cfg.vocab, hidden=W, table_name="head", softcap=0.0,
                        init_std=W ** -0.5),
        schedule=schedule,
        max_context=1 << 20)


register_architecture("Vivazen", VivazenConfig, build_vivazen, model_types=("vivazen",), replace=True)
