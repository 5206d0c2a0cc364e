"""Position encodings applied to queries and keys inside a mixer.

`RotaryEncoding` is the half-split rotary encoding the reference applies to a
whole head (`gemma/gemma.go:73-74`; `cpu/cpu_attn.go:13-62`, non-traditional):
inv_i = base^(-2i/dims) computed in float64 and rounded to float32, theta =
float32(pos) * inv_i, pair (i, i + dims/2); a mixer that turns neighbouring pairs instead takes the same table.  It is handed to the kernel as a
table of inverse frequencies, so scaled frequencies (`qwen/attention.go:23-42`)
or a rotation of part of the head (`qwen/config.go:55`) are other tables, not
other kernels.  `NoPosition` rotates nothing and only stores keys and values.

Keys are cached after encoding (`gemma/gemma.go:73-75`), so the order of the
places in a ring does not matter.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .base import PositionEncoding, Runtime, StepContext


def band_scaled_frequencies(inv_freq, factor: float, low: float, high: float, original: float):
    """Inverse frequencies rescaled by wavelength, for a model that was trained on contexts of `original`
    positions and runs on longer ones: a component whose wavelength 2 pi / f is shorter than original / high is
    kept; one longer than original / low is slowed down to f / factor; in between the two are blended with
    s = (original / wavelength - low) / (high - low): (1 - s) f / factor + s f.  Computed in float64."""
    out = []
    for f in inv_freq:
        f = float(f)
        wave = 2.0 * math.pi / f
        if wave < original / high:
            out.append(f)
        elif wave > original / low:
            out.append(f / factor)
        else:
            s = (original / wave - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return out


def ramp_scaled_frequencies(inv_freq, dims: int, base: float, factor: float, original: float, fast: float,
                            slow: float):
    """Inverse frequencies stretched by `factor` along a ramp over the pair index, and the amplitude that goes with
    them.  A pair that makes t turns over `original` positions sits at index x(t) = dims ln(original / (2 pi t)) /
    (2 ln base); with lo = max(floor(x(fast)), 0) and hi = min(ceil(x(slow)), dims - 1), pair i gets
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) and the frequency f_i / factor * r_i + f_i (1 - r_i): pairs that
    turn fast keep their frequency, slow ones are stretched.  Sine and cosine are multiplied by 0.1 ln(factor) + 1.
    Computed in float64; returns (frequencies, amplitude)."""
    def index_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(fast)), 0)
    hi = min(math.ceil(index_of(slow)), dims - 1)
    out = []
    for i, f in enumerate(inv_freq):
        f = float(f)
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * r + f * (1.0 - r))
    return out, 0.1 * math.log(factor) + 1.0


class RotaryEncoding(PositionEncoding):
    """pairs="halves": element i turns with element i + dims/2 (the kernels of `encode`); pairs="neighbours": element
    2i with 2i + 1 (a mixer with a kernel of its own reads `inv_freq` and `amplitude` from here).  `amplitude`
    multiplies sine and cosine; it is 1 unless `ramp_scaling` ({"factor", "original", "fast", "slow"}) sets it."""

    def __init__(self, head_dim: int, base: float, rotary_dims: int | None = None, inv_freq=None,
                 band_scaling: dict | None = None, ramp_scaling: dict | None = None, pairs: str = "halves"):
        if pairs not in ("halves", "neighbours"):
            raise ValueError(f"unknown pairing {pairs!r} (known: halves, neighbours)")
        self.pairs = pairs
        self.amplitude = 1.0
        rot = head_dim if rotary_dims is None else int(rotary_dims)
        if rot % 2 or rot < 0 or rot > head_dim:
            raise ValueError(f"rotary width {rot} must be even and at most the head size {head_dim}")
        self.head_dim = head_dim
        self.rot = rot
        self.base = float(base)
        if inv_freq is None:
            inv_freq = [math.pow(self.base, -float(2 * i) / float(rot)) for i in range(rot // 2)]
            if band_scaling:          # {"factor", "low", "high", "original"}: see band_scaled_frequencies
                inv_freq = band_scaled_frequencies(inv_freq, **band_scaling)
            if ramp_scaling and rot:
                inv_freq, self.amplitude = ramp_scaled_frequencies(inv_freq, rot, self.base, **ramp_scaling)
        self._inv_host = np.asarray(inv_freq, dtype=np.float32)
        if self._inv_host.shape != (rot // 2,):
            raise ValueError("inv_freq must hold rotary_dims / 2 values")
        self.inv_freq = None

    def load(self, store, rt: Runtime):
        self.inv_freq = torch.from_numpy(self._inv_host.copy()).to(rt.device)

    def _halves_only(self):
        if self.pairs != "halves" or self.amplitude != 1.0:
            raise NotImplementedError("the rotary kernels of whole heads turn halves with amplitude 1; neighbouring "
                                      "pairs and amplitudes belong to a mixer that turns its own vectors")

    def encode(self, qkv, ctx: StepContext, nq: int, nkv: int, hd: int, with_keys: bool):
        self._halves_only()
        return ctx.rt.ops.rope_store(qkv, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, ctx.seq_end, self.inv_freq, self.rot,
                                     nq, nkv, hd, store=with_keys, write_cache=False)

    def encode_and_store(self, qkv, ctx: StepContext, nq: int, nkv: int, hd: int, kv_line):
        self._halves_only()
        ops = ctx.rt.ops
        if kv_line is None or not kv_line.write:
            return ops.rope_store(qkv, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, ctx.seq_end, self.inv_freq,
                                  self.rot, nq, nkv, hd, store=False)
        return ops.rope_store(qkv, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, ctx.seq_end, self.inv_freq, self.rot,
                              nq, nkv, hd, kv_line.k, kv_line.v, kv_line.table, kv_line.ring_len, store=True)


    def project_encode_store(self, x, w, qkv, ctx: StepContext, nq: int, nkv: int, hd: int, kv_line):
        """A decode step of up to 16 rows in bfloat16 that rotates the whole head: projection, encoding and cache
        write are one kernel (the product's tiles pair each element with its partner half a head on)."""
        self._halves_only()
        ops = ctx.rt.ops
        fused = (ctx.mode == "decode" and ctx.rt.dtype == torch.bfloat16 and self.rot == hd and hd % 16 == 0
                 and x.shape[0] <= getattr(ops, "GEMV_FAST_ROWS", 0) and hasattr(ops, "gemv_rope_store"))
        if not fused:
            return super().project_encode_store(x, w, qkv, ctx, nq, nkv, hd, kv_line)
        if kv_line is None or not kv_line.write:
            return ops.gemv_rope_store(x, w, qkv, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, ctx.seq_end, self.inv_freq,
                                       nq, nkv, hd, store=False)
        return ops.gemv_rope_store(x, w, qkv, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, ctx.seq_end, self.inv_freq,
                                   nq, nkv, hd, kv_line.k, kv_line.v, kv_line.table, kv_line.ring_len, store=True)


class NoPosition(RotaryEncoding):
    """No encoding: keys and values are stored as projected."""

    def __init__(self, head_dim: int):
        super().__init__(head_dim, 10000.0, rotary_dims=0)
