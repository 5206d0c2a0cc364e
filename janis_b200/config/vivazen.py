"""Vivazen's configuration: the keys of its config.json, typed.

config.json names the architecture under `architecture` and nests its values:

    vocab, width, postln_alpha, norm.eps, norm.groups,
    layers: [ {type: "attention" | "latent_attention", mixer: {...}, mlp: {kind: "dense", ff} | null,
               weights_of: j (optional)}, ... ]

An "attention" mixer gives heads, kv_heads, dim (queries and keys), vdim (values), scale, softcap (a cap on the
scaled scores; absent or 0: none) and conv (the taps of the short causal filter on its projections; absent or 0:
none).  A "latent_attention" mixer gives heads, dim (the part of a query/key head that is not rotated), rot_dim (the
rotated part), vdim, kv_rank (the size of the compressed key/value row), scale, rot.base, rot.dims, rot.scaling
(factor, original, fast, slow; absent: frequencies as they are) and mask.size (the sliding window; absent or 0: every
earlier key is seen).  A layer with `weights_of: j` has no tensors of its own and uses layer j's, with a cache of its
own; its entry must otherwise equal layer j's.  Every size and constant of a model comes from here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, ConfigReader
from .sigalorn import DenseSpec, _sub


@dataclass(frozen=True)
class RampScaling:
    """Frequencies stretched by `factor` below a ramp over the rotary pairs (see parts.position.ramp_scaled_frequencies)."""
    factor: float
    original: float
    fast: float
    slow: float

    def to_dict(self) -> dict:
        return {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}


@dataclass(frozen=True)
class FilteredAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float                 # 0: no cap
    conv: int                      # taps of the filter on q, k and v; 0: none

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.softcap:
            d["softcap"] = self.softcap
        if self.conv:
            d["conv"] = self.conv
        return d


@dataclass(frozen=True)
class LatentAttentionSpec:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    rot_scaling: RampScaling | None
    window: int                    # 0: every earlier key is seen

    def to_dict(self) -> dict:
        rot: dict = {"base": self.rot_base, "dims": self.rot_dims}
        if self.rot_scaling is not None:
            rot["scaling"] = self.rot_scaling.to_dict()
        d = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
             "scale": self.scale, "rot": rot}
        if self.window:
            d["mask"] = {"size": self.window}
        return d


@dataclass(frozen=True)
class LayerSpec:
    type: str                      # "attention" | "latent_attention"
    mixer: Any
    mlp: DenseSpec | None
    weights_of: int | None = None

    def to_dict(self) -> dict:
        d = {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None}
        if self.weights_of is not None:
            d["weights_of"] = self.weights_of
        return d


def _filtered(r: ConfigReader) -> FilteredAttentionSpec:
    heads = r.integer("heads", minimum=1)
    kv = r.integer("kv_heads", default=heads, minimum=1)
    if heads % kv:
        raise ConfigError(f"{r.where}: heads ({heads}) not divisible by kv_heads ({kv})")
    dim = r.integer("dim", minimum=1)
    conv = r.integer("conv", default=0, minimum=0)
    if conv > 16:
        raise ConfigError(f"{r.where}: a filter of {conv} taps (up to 16 are taken)")
    return FilteredAttentionSpec(heads=heads, kv_heads=kv, dim=dim, vdim=r.integer("vdim", default=dim, minimum=1),
                                 scale=r.number("scale", default=dim ** -0.5, minimum=0.0, exclusive=True),
                                 softcap=r.number("softcap", default=0.0, minimum=0.0), conv=conv)


def _latent(r: ConfigReader) -> LatentAttentionSpec:
    dim = r.integer("dim", minimum=0)
    rot_dim = r.integer("rot_dim", default=0, minimum=0)
    if dim + rot_dim < 1:
        raise ConfigError(f"{r.where}: a query head needs at least one feature")
    rot = _sub(r, "rot", required=rot_dim > 0)
    rot_base, rot_dims, scaling = 10000.0, 0, None
    if rot is not None:
        rot_base = rot.number("base", default=10000.0, minimum=0.0, exclusive=True)
        rot_dims = rot.integer("dims", default=rot_dim, minimum=0)
        if rot_dims % 2 or rot_dims > rot_dim:
            raise ConfigError(f"{r.where}: rot.dims must be even and at most rot_dim ({rot_dim}), found {rot_dims}")
        sc = _sub(rot, "scaling", required=False)
        if sc is not None:
            scaling = RampScaling(factor=sc.number("factor", minimum=0.0, exclusive=True),
                                  original=sc.number("original", minimum=0.0, exclusive=True),
                                  fast=sc.number("fast", default=32.0, minimum=0.0, exclusive=True),
                                  slow=sc.number("slow", default=1.0, minimum=0.0, exclusive=True))
    mask = _sub(r, "mask", required=False)
    return LatentAttentionSpec(heads=r.integer("heads", minimum=1), dim=dim, rot_dim=rot_dim,
                               vdim=r.integer("vdim", minimum=1), kv_rank=r.integer("kv_rank", minimum=1),
                               scale=r.number("scale", default=(dim + rot_dim) ** -0.5, minimum=0.0, exclusive=True),
                               rot_base=rot_base, rot_dims=rot_dims, rot_scaling=scaling,
                               window=mask.integer("size", default=0, minimum=0) if mask is not None else 0)


@dataclass(frozen=True)
class VivazenConfig:
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    postln_alpha: float
    layers: tuple[LayerSpec, ...]
    architecture: str = "Vivazen"

    def weight_layer(self, i: int) -> int:
        """The layer whose tensors layer i uses (itself, unless it names another)."""
        seen = set()
        while self.layers[i].weights_of is not None:
            if i in seen:
                raise ConfigError(f"layers[{i}]: weights_of runs in a circle")
            seen.add(i)
            i = self.layers[i].weights_of
        return i

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str = "config.json") -> "VivazenConfig":
        r = ConfigReader(raw, where)
        norm = _sub(r, "norm", required=False)
        listed = r.raw.get("layers")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        layers: list[LayerSpec] = []
        for i, entry in enumerate(listed):
            if not isinstance(entry, Mapping):
                raise ConfigError(f"{where}: layers[{i}] must be an object")
            lr = ConfigReader(entry, f"{where}: layers[{i}]")
            kind = lr.string("type")
            mr = _sub(lr, "mixer")
            mr.where = f"{where}: layers[{i}].mixer"
            if kind == "attention":
                mixer = _filtered(mr)
            elif kind == "latent_attention":
                mixer = _latent(mr)
            else:
                raise ConfigError(f"{where}: layers[{i}]: unknown layer type {kind!r} (known: attention, latent_attention)")
            fr = _sub(lr, "mlp", required=False)
            mlp = None
            if fr is not None:
                fk = fr.string("kind", default="dense")
                if fk != "dense":
                    raise ConfigError(f"{where}: layers[{i}].mlp: unknown kind {fk!r} (known: dense)")
                mlp = DenseSpec(ff=fr.integer("ff", minimum=1), kind=fk)
            src = lr.integer("weights_of", minimum=0) if lr.has("weights_of") else None
            layers.append(LayerSpec(kind, mixer, mlp, src))
        width = r.integer("width", minimum=1)
        groups = norm.integer("groups", default=1, minimum=1) if norm is not None else 1
        if width % groups:
            raise ConfigError(f"{where}: norm.groups ({groups}) does not divide width ({width})")
        cfg = cls(vocab=r.integer("vocab", minimum=1), width=width,
                  norm_eps=norm.number("eps", default=1e-6, minimum=0.0) if norm is not None else 1e-6,
                  norm_groups=groups, postln_alpha=r.number("postln_alpha", default=1.0),
                  layers=tuple(layers), architecture=r.string("architecture", default="Vivazen"))
        for i, layer in enumerate(layers):
            j = layer.weights_of
            if j is None:
                continue
            if j >= len(layers) or j == i:
                raise ConfigError(f"{where}: layers[{i}]: weights_of {j} names no other layer")
            o = layers[cfg.weight_layer(i)]
            if (o.type, o.mixer, o.mlp) != (layer.type, layer.mixer, layer.mlp):
                raise ConfigError(f"{where}: layers[{i}] uses layer {j}'s tensors but is described differently")
        return cfg

    def to_dict(self) -> dict:
        """The config.json that reads back to this object."""
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "postln_alpha": self.postln_alpha,
                "layers": [l.to_dict() for l in self.layers]}
