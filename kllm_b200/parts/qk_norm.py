"""RMS norm of queries and keys over the WHOLE projection (all heads at once, before
they are split), with a temperature on the queries that grows with the position:
a ``qk_transform`` of the attention mixer for layers without rotation.

    q <- q / sqrt(mean(q^2 over H * dk) + eps) * g_q * (1 + coef * ln(floor((p + 1) / every) + 1))
    k <- k / sqrt(mean(k^2 over G * dk) + eps) * g_k

params: ``q_dim`` (H * dk), ``k_dim`` (G * dk), ``eps``, ``q_gain`` / ``k_gain`` (full tensor
names, plain gains, float32), ``temp_coef`` (0 or absent: no temperature), ``temp_every``,
``rotary_dim`` and ``theta`` (optional: AFTER the norm the first ``rotary_dim`` values of every query and
key head are rotated, pair (i, i + rotary_dim / 2) by position * theta^(-2i / rotary_dim), the angle formed
in double precision on the device, in the same kernel; ``scaling`` as in ``rotary.rotary_frequencies``).
It offers ``prepare`` (see ``parts/attention.py``): it takes the projection's float32
result, so sums, scales and the temperature are float32 in both dtypes, returns the queries
in the model dtype and writes keys and values (of their own head size) into the layer's
pages, all in one kernel (csrc/qknorm_append.cu).
"""
from __future__ import annotations

import torch

from .. import kernels
from .spec import BuildEnv, PartSpec, TensorSpec, register_part


class WholeProjectionNorm:
    def __init__(self, spec: PartSpec, env: BuildEnv):
        p = spec.params
        self.q_dim, self.k_dim = int(p["q_dim"]), int(p["k_dim"])
        self.eps = float(p["eps"])
        self.q_name, self.k_name = p["q_gain"], p["k_gain"]
        self.coef = float(p.get("temp_coef") or 0.0)
        self.every = int(p.get("temp_every") or 1)
        if self.coef != 0.0 and self.every < 1:
            raise ValueError(f"query temperature: period {self.every} must be positive")
        self.dtype = env.dtype
        self.q_gain = self.k_gain = None
        self.rot, self.freq = int(p.get("rotary_dim") or 0), None
        if self.rot:
            from .rotary import rotary_frequencies
            if self.rot % 2:
                raise ValueError(f"rotary_dim {self.rot} must be even")
            freq, amplitude = rotary_frequencies(self.rot, float(p["theta"]), p.get("scaling"))
            if amplitude != 1.0:
                raise ValueError("whole_rmsnorm: a rotation whose scaling changes the amplitude has no kernel here")
            self.freq = freq.to(env.device)

    def tensor_specs(self):
        return [TensorSpec(self.q_name, (self.q_dim,), store="float32", init="gain"),
                TensorSpec(self.k_name, (self.k_dim,), store="float32", init="gain")]

    def bind(self, tensors):
        self.q_gain, self.k_gain = tensors[self.q_name], tensors[self.k_name]

    def prepare(self, qkv, ctx, cache, attn):
        q = torch.empty((qkv.shape[0], self.q_dim), dtype=self.dtype, device=qkv.device)
        writes = cache.writes
        kernels.qknorm_append(q, qkv, self.q_gain, self.k_gain if writes else None, self.eps, self.coef, self.every,
                              ctx.positions, ctx.token_req, cache.block_table if writes else None,
                              cache.k if writes else None, cache.v if writes else None,
                              attn.n_heads, attn.n_kv, attn.head_dim, attn.v_head_dim, rot=self.rot, freq=self.freq)
        return q


class HeadNormRotary:
    """``head_rmsnorm_rotary``: every query and key head is divided by its root mean square over its
    ``head_dim`` values and multiplied by a gain [head_dim] that all heads share (``q_gain`` /
    ``k_gain``: full tensor names, float32; None: no norm on that side), then the first ``rotary_dim``
    values of every head are rotated (pair (i, i + rotary_dim / 2), angle position * f_i; ``theta``,
    ``scaling`` as in ``rotary.rotary_frequencies``), before which the projections' biases are added
    (the attention's ``bias``).  It offers ``prepare``: it takes the float32 result of the stacked
    projection, so biases, sums, scales and the rotation are float32 and the angle is formed in double
    precision on the device (no table, no bound on the position); it returns the queries in the model
    dtype and writes keys and values, which may have fewer heads than the keys, into the layer's pages:
    one kernel (csrc/qk_headnorm.cu)."""

    def __init__(self, spec: PartSpec, env: BuildEnv):
        from .rotary import rotary_frequencies
        p = spec.params
        self.head_dim = int(p["head_dim"])
        self.eps = float(p.get("eps") or 0.0)
        self.q_name, self.k_name = p.get("q_gain"), p.get("k_gain")
        self.rot = int(p.get("rotary_dim") or 0)
        if self.rot % 2 or self.rot > self.head_dim:
            raise ValueError(f"rotary_dim {self.rot} must be even and within head_dim {self.head_dim}")
        self.freq, self.amplitude = None, 1.0
        if self.rot:
            freq, self.amplitude = rotary_frequencies(self.rot, float(p["theta"]), p.get("scaling"))
            self.freq = freq.to(env.device)
        self.dtype = env.dtype
        self.q_gain = self.k_gain = None

    def tensor_specs(self):
        return [TensorSpec(n, (self.head_dim,), store="float32", init="gain") for n in (self.q_name, self.k_name) if n]

    def bind(self, tensors):
        self.q_gain = tensors[self.q_name] if self.q_name else None
        self.k_gain = tensors[self.k_name] if self.k_name else None

    def prepare(self, qkv, ctx, cache, attn):
        q_heads, k_heads = attn.n_heads * attn.maps, attn.n_kv * attn.maps
        q = torch.empty((qkv.shape[0], q_heads * self.head_dim), dtype=self.dtype, device=qkv.device)
        writes = cache.writes
        kernels.headnorm_rope_append(q, qkv, attn.bias, self.q_gain, self.k_gain, self.eps, self.freq, self.amplitude,
                                     self.rot, ctx.positions, ctx.token_req, cache.block_table if writes else None,
                                     cache.k if writes else None, cache.v if writes else None, q_heads, k_heads,
                                     attn.n_kv, self.head_dim, attn.v_head_dim)
        return q


register_part("qk_transform", "whole_rmsnorm", WholeProjectionNorm)
register_part("qk_transform", "head_rmsnorm_rotary", HeadNormRotary)
