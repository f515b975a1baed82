"""Rotary position encoding (rotate_half convention).

params: ``head_dim``, ``theta``, optional ``rotary_dim`` (defaults to head_dim; a
smaller even value rotates only the first dims of each head).  The part owns a
float32 table [max_position, rotary_dim] of cos (first half of a row) and sin
(second half), computed in float64 from angle = p * theta^(-2j/rotary_dim), which is
how the reference forms its angles (backend/model.cu:176-178).

Interface of a position part used by the attention mixer:
``apply(q, k, v, ctx, cache, n_heads, n_kv_heads)`` rotates q in place and, when the
layer writes its cache, stores rotated k and v into the pages.  Optional:
``full_rotary_table()`` returns the cos/sin table when the whole head is rotated, for
a mixer whose kernel can do the rotation itself.
"""
from __future__ import annotations

import torch

from .. import kernels
from .spec import BuildEnv, PartSpec, register_part


def rotary_frequencies(dims: int, base: float, scaling=None):
    """(frequencies float64 [dims / 2], amplitude) of a rotation of ``dims`` values: f_i =
    base^(-2i / dims), changed by ``scaling`` (None, or a dict with ``kind``):

    ``kind`` "wavelength" (``factor``, ``low``, ``high``, ``original``): with the wavelength l = 2 pi / f,
    f stays where l < original / high, becomes f / factor where l > original / low, and in between,
    with s = (original / l - low) / (high - low), (1 - s) f / factor + s f.

    ``kind`` "ramp" (``factor``, ``original``, ``fast``, ``slow``): with where(t) = dims ln(original /
    (2 pi t)) / (2 ln base), lo = max(floor(where(fast)), 0), hi = min(ceil(where(slow)), dims - 1) and
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1): f_i / factor * ramp_i + f_i (1 - ramp_i); the
    amplitude, which multiplies cos and sin, is 0.1 ln(factor) + 1.
    """
    import math
    half = dims // 2
    freq = [float(base) ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return torch.tensor(freq, dtype=torch.float64), 1.0
    kind, factor, orig = scaling["kind"], float(scaling["factor"]), float(scaling["original"])
    if kind == "wavelength":
        low, high = float(scaling["low"]), float(scaling["high"])
        out = []
        for f in freq:
            wave = 2.0 * math.pi / f
            if wave < orig / high:
                out.append(f)
            elif wave > orig / low:
                out.append(f / factor)
            else:
                s = (orig / wave - low) / (high - low)
                out.append((1.0 - s) * f / factor + s * f)
        return torch.tensor(out, dtype=torch.float64), 1.0
    if kind == "ramp":
        def where(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))
        lo = max(math.floor(where(float(scaling["fast"]))), 0)
        hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
        out = []
        for i, f in enumerate(freq):
            ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
            out.append(f / factor * ramp + f * (1.0 - ramp))
        return torch.tensor(out, dtype=torch.float64), 0.1 * math.log(factor) + 1.0
    raise ValueError(f"rotary scaling of kind {kind!r} (wavelength, ramp)")


class RotaryEmbedding:
    def __init__(self, spec: PartSpec, env: BuildEnv):
        self.head_dim = int(spec.params["head_dim"])
        self.theta = float(spec.params["theta"])
        self.rotary_dim = int(spec.params.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or not (0 < self.rotary_dim <= self.head_dim):
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and within head_dim {self.head_dim}")
        half = self.rotary_dim // 2
        j = torch.arange(half, dtype=torch.float64)
        freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * j / self.rotary_dim)
        ang = torch.arange(env.max_position, dtype=torch.float64)[:, None] * freq[None, :]
        table = torch.cat([torch.cos(ang), torch.sin(ang)], dim=1).to(torch.float32)
        self.cos_sin = table.contiguous().to(env.device)

    def tensor_specs(self):
        return []

    def bind(self, tensors):
        pass

    def full_rotary_table(self):
        return self.cos_sin if self.rotary_dim == self.head_dim else None

    def apply(self, q, k, v, ctx, cache, n_heads, n_kv_heads):
        writes = cache.writes and cache.k is not None
        kernels.rope_append(q, k, v, self.cos_sin, ctx.positions, ctx.token_req,
                            cache.block_table if writes else None,
                            cache.k if writes else None, cache.v if writes else None,
                            n_heads, n_kv_heads, self.head_dim)


register_part("position", "rotary", RotaryEmbedding)
