"""Dekutar's configuration: the keys of its config.json, typed.

config.json names the architecture under `architecture` and nests its values:

    vocab, width, streams (optional), embedding.scale, norm.eps, logit_scale,
    layers: [ {type: "latent_attention" | "attention" | "mlstm", mixer: {...}, mlp: {kind: "moe", ...} | null}, ... ]

`streams` is the number of copies of the residual stream that the layers' hyper-connections read and write;
without the key a layer is the plain pre-norm one with a single stream.

A "latent_attention" mixer gives heads, dim (the part of a query/key head that is not rotated), rot_dim (the
rotated part), vdim, kv_rank (the compressed key/value row), q_rank (the compressed query row), scale, rot.base and
rot.dims (the first features of the rotated part that turn: all of them, as a rule).  An "attention" mixer gives
heads, kv_heads, dim (queries and keys; the values are the keys as projected, so vdim equals dim), scale, rot.base,
rot.dims (the first features of a head that turn; absent or 0: none),
mask.size (the sliding window; absent or 0: every earlier key is seen) and mask.keep_first (the sequence's first
positions that stay seen behind the window).  An "mlstm" mixer gives heads, dim (queries and keys), vdim and
gate_cap.  A feed-forward gives expert.ff, router.experts (the experts that have tensors), router.identity (further
router entries that return their input), router.top, and shared.ff (or no `shared`).  Every size and constant of a
model comes from here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, ConfigReader
from .sigalorn import _sub


@dataclass(frozen=True)
class QueryLatentAttentionSpec:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_base: float
    rot_dims: int

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
                "q_rank": self.q_rank, "scale": self.scale, "rot": {"base": self.rot_base, "dims": self.rot_dims}}


@dataclass(frozen=True)
class KeptWindowAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float
    rot_dims: int                  # 0: nothing turns
    window: int                    # 0: every earlier key is seen
    keep_first: int

    def to_dict(self) -> dict:
        d: dict = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        if self.window:
            d["mask"] = {"size": self.window, "keep_first": self.keep_first}
        return d


@dataclass(frozen=True)
class MatrixMemorySpec:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "gate_cap": self.gate_cap}


@dataclass(frozen=True)
class SoftmaxMoeSpec:
    experts: int                   # experts with tensors
    identity: int                  # router entries behind them that return their input
    top: int
    expert_ff: int
    shared_ff: int                 # 0: no shared expert
    kind: str = "moe"

    def to_dict(self) -> dict:
        return {"kind": self.kind, "expert": {"ff": self.expert_ff},
                "router": {"experts": self.experts, "identity": self.identity, "top": self.top},
                "shared": {"ff": self.shared_ff} if self.shared_ff else None}


@dataclass(frozen=True)
class LayerSpec:
    type: str                      # "latent_attention" | "attention" | "mlstm"
    mixer: Any
    mlp: SoftmaxMoeSpec | None

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None}


def _rot(r: ConfigReader, limit: int, required: bool):
    rot = _sub(r, "rot", required=required)
    if rot is None:
        return 10000.0, 0
    base = rot.number("base", default=10000.0, minimum=0.0, exclusive=True)
    dims = rot.integer("dims", default=limit, minimum=0)
    if dims % 2 or dims > limit:
        raise ConfigError(f"{r.where}: rot.dims must be even and at most {limit}, found {dims}")
    return base, dims


def _latent(r: ConfigReader) -> QueryLatentAttentionSpec:
    dim = r.integer("dim", minimum=0)
    rot_dim = r.integer("rot_dim", default=0, minimum=0)
    if dim + rot_dim < 1:
        raise ConfigError(f"{r.where}: a query head needs at least one feature")
    base, dims = _rot(r, rot_dim, required=rot_dim > 0)
    return QueryLatentAttentionSpec(heads=r.integer("heads", minimum=1), dim=dim, rot_dim=rot_dim,
                                    vdim=r.integer("vdim", minimum=1), kv_rank=r.integer("kv_rank", minimum=1),
                                    q_rank=r.integer("q_rank", minimum=1),
                                    scale=r.number("scale", default=(dim + rot_dim) ** -0.5, minimum=0.0, exclusive=True),
                                    rot_base=base, rot_dims=dims)


def _window(r: ConfigReader) -> KeptWindowAttentionSpec:
    heads = r.integer("heads", minimum=1)
    kv = r.integer("kv_heads", default=heads, minimum=1)
    if heads % kv:
        raise ConfigError(f"{r.where}: heads ({heads}) not divisible by kv_heads ({kv})")
    dim = r.integer("dim", minimum=1)
    vdim = r.integer("vdim", default=dim, minimum=1)
    if vdim != dim:
        raise ConfigError(f"{r.where}: the values are the keys as projected, so vdim ({vdim}) must equal dim ({dim})")
    base, dims = _rot(r, dim, required=False)
    mask = _sub(r, "mask", required=False)
    window = mask.integer("size", default=0, minimum=0) if mask is not None else 0
    keep = mask.integer("keep_first", default=0, minimum=0) if mask is not None else 0
    return KeptWindowAttentionSpec(heads=heads, kv_heads=kv, dim=dim, vdim=vdim,
                                   scale=r.number("scale", default=dim ** -0.5, minimum=0.0, exclusive=True),
                                   rot_base=base, rot_dims=dims, window=window, keep_first=keep if window else 0)


def _matrix_memory(r: ConfigReader) -> MatrixMemorySpec:
    dim = r.integer("dim", minimum=1)
    return MatrixMemorySpec(heads=r.integer("heads", minimum=1), dim=dim, vdim=r.integer("vdim", default=dim, minimum=1),
                            gate_cap=r.number("gate_cap", minimum=0.0, exclusive=True))


def _moe(r: ConfigReader) -> SoftmaxMoeSpec:
    kind = r.string("kind", default="moe")
    if kind != "moe":
        raise ConfigError(f"{r.where}: unknown kind {kind!r} (known: moe)")
    router = _sub(r, "router")
    expert = _sub(r, "expert")
    shared = _sub(r, "shared", required=False)
    experts = router.integer("experts", minimum=0)
    identity = router.integer("identity", default=0, minimum=0)
    top = router.integer("top", minimum=1)
    if top > experts + identity:
        raise ConfigError(f"{r.where}: {top} chosen of {experts} experts and {identity} identity entries")
    return SoftmaxMoeSpec(experts=experts, identity=identity, top=top,
                          expert_ff=expert.integer("ff", minimum=1),
                          shared_ff=shared.integer("ff", minimum=1) if shared is not None else 0, kind=kind)


_MIXERS = {"latent_attention": _latent, "attention": _window, "mlstm": _matrix_memory}


@dataclass(frozen=True)
class DekutarConfig:
    vocab: int
    width: int
    streams: int                   # 0: one stream and the plain residual sum
    embedding_scale: float
    norm_eps: float
    logit_scale: float
    layers: tuple[LayerSpec, ...]
    architecture: str = "Dekutar"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str = "config.json") -> "DekutarConfig":
        r = ConfigReader(raw, where)
        norm = _sub(r, "norm", required=False)
        emb = _sub(r, "embedding", required=False)
        listed = r.raw.get("layers")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        layers: list[LayerSpec] = []
        for i, entry in enumerate(listed):
            if not isinstance(entry, Mapping):
                raise ConfigError(f"{where}: layers[{i}] must be an object")
            lr = ConfigReader(entry, f"{where}: layers[{i}]")
            kind = lr.string("type")
            if kind not in _MIXERS:
                raise ConfigError(f"{where}: layers[{i}]: unknown layer type {kind!r} (known: {', '.join(_MIXERS)})")
            mr = _sub(lr, "mixer")
            mr.where = f"{where}: layers[{i}].mixer"
            fr = _sub(lr, "mlp", required=False)
            if fr is not None:
                fr.where = f"{where}: layers[{i}].mlp"
            layers.append(LayerSpec(kind, _MIXERS[kind](mr), _moe(fr) if fr is not None else None))
        streams = r.integer("streams", default=0, minimum=0)
        if streams > 8:
            raise ConfigError(f"{where}: 'streams' must be at most 8, found {streams}")
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1), streams=streams,
                   embedding_scale=emb.number("scale", default=1.0) if emb is not None else 1.0,
                   norm_eps=norm.number("eps", default=1e-6, minimum=0.0) if norm is not None else 1e-6,
                   logit_scale=r.number("logit_scale", default=1.0),
                   layers=tuple(layers), architecture=r.string("architecture", default="Dekutar"))

    def to_dict(self) -> dict:
        """The config.json that reads back to this object."""
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
             "logit_scale": self.logit_scale, "layers": [l.to_dict() for l in self.layers]}
        if self.streams:
            d["streams"] = self.streams
        return d
