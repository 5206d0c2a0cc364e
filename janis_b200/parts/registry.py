"""Kinds of parts by name, so that a configuration can choose them layer by layer.

An architecture's builder looks a kind up with `make(family, kind, **params)`;
a user's code can add kinds of its own with `register(family, kind, factory)`
and use them from a builder of its own, without touching this package.
"""
from __future__ import annotations

from typing import Any, Callable

FAMILIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")

_KINDS: dict[str, dict[str, Callable[..., Any]]] = {f: {} for f in FAMILIES}


def register(family: str, kind: str, factory: Callable[..., Any], replace: bool = False) -> None:
    if family not in _KINDS:
        raise ValueError(f"unknown family of parts {family!r} (families: {', '.join(FAMILIES)})")
    if kind in _KINDS[family] and not replace:
        raise ValueError(f"{family} kind {kind!r} is already registered")
    _KINDS[family][kind] = factory


def unregister(family: str, kind: str) -> None:
    _KINDS.get(family, {}).pop(kind, None)


def kinds(family: str) -> tuple[str, ...]:
    return tuple(sorted(_KINDS[family]))


def make(family: str, kind: str, **params):
    try:
        factory = _KINDS[family][kind]
    except KeyError:
        raise ValueError(f"unknown {family} kind {kind!r} (registered: {', '.join(kinds(family)) or 'none'})") from None
    return factory(**params)


def _register_builtin() -> None:
    from .attention import SoftmaxAttention
    from .block import PostNormBlock, PreNormBlock, SandwichBlock
    from .embedding import Embedding, LMHead
    from .feedforward import DenseMLP, GatedMLP
    from .filtered_attention import FilteredAttention
    from .hyper import HyperConnectionBlock, HyperRead
    from .matrix_memory import MatrixMemory
    from .latent_attention import LatentAttention
    from .linear_attention import GatedLinearAttention
    from .talking_attention import TalkingHeadsAttention
    from .moe import RoutedExperts
    from .norm import DynamicTanh, GroupRMSNorm, RMSNorm
    from .parallel import ParallelMixers
    from .state_space import DualityMixer, SelectiveScanMixer
    from .position import NoPosition, RotaryEncoding

    register("mixer", "softmax_attention", SoftmaxAttention)
    register("mixer", "talking_heads_attention", TalkingHeadsAttention)   # heads mixed before the softmax, sink, block mask
    register("mixer", "filtered_attention", FilteredAttention)             # filtered and normed projections, capped scores, weights mixed after the softmax
    register("mixer", "latent_attention", LatentAttention)                 # one compressed row cached per position, a sink per head, a window
    register("mixer", "gated_linear_attention", GatedLinearAttention)     # a matrix of state per head, decays per key channel
    register("mixer", "matrix_memory", MatrixMemory)                      # a matrix, a normaliser and a running maximum per head, exponential gates
    register("mixer", "selective_scan", SelectiveScanMixer)               # a state per channel, step sizes through a low rank
    register("mixer", "state_space_duality", DualityMixer)                # a scalar decay per head, grouped B and C
    register("mixer", "parallel", ParallelMixers)                         # branches on one input, normed and averaged
    register("feed_forward", "gated_mlp", GatedMLP)
    register("feed_forward", "dense_mlp", DenseMLP)                       # up, activation, down, with biases
    register("feed_forward", "routed_experts", RoutedExperts)             # a router over small gated experts, a shared one
    register("norm", "rms_norm", RMSNorm)
    register("norm", "dynamic_tanh", DynamicTanh)
    register("norm", "group_rms_norm", GroupRMSNorm)       # each run of the row by its own root mean square; norms the stream in place
    register("norm", "hyper_read", HyperRead)              # a weighted sum of the stream's copies, then the RMS norm
    register("position", "rotary", RotaryEncoding)
    register("position", "none", NoPosition)
    register("block", "sandwich", SandwichBlock)
    register("block", "pre_norm", PreNormBlock)
    register("block", "post_norm", PostNormBlock)          # the norm after the sum, the stream scaled by a constant
    register("block", "hyper_connections", HyperConnectionBlock)   # copies of the stream read and written through small stored maps
    register("embedding", "scaled_table", Embedding)       # rows of a table times a constant (1 for most models)
    register("head", "capped_linear", LMHead)              # y W^T, tied to the embedding's table or not, then an optional cap


_register_builtin()
