"""Causal grouped-query attention over a paged cache: the mixer of a Llama layer.

params: ``hidden``, ``n_heads``, ``n_kv_heads``, ``head_dim``; optional ``window``
(None: every earlier key is visible; W: the last W keys, the query's own included),
``scale`` (default 1/sqrt(head_dim)), ``position`` (a PartSpec of the position
family, e.g. rotary; None for no position encoding), ``qk_transform`` (a PartSpec of
the qk_transform family, None for Llama: something applied to the projected queries
and keys before the position encoding, such as a norm per head or a bias; interface
``tensor_specs()``, ``bind(tensors)``, ``apply(q, k, ctx, n_heads, n_kv_heads,
head_dim)`` which changes q [n, H*hd] and k [n, G*hd] (None when the layer reads
another layer's cache) in place; with one, a decode step takes the separate rotary
and attention kernels, since the fused kernel rotates the raw projections itself),
``score_slopes`` (a list of one float per head, None for Llama: slope[h] * (key
position - query position) is added to the scaled scores, the form of position
encodings that act on the scores; such a layer runs the CUDA-core attention kernel, the
only one that takes the argument), ``v_head_dim`` (the size of a head's values and of its
output where it differs from ``head_dim``; same kernel), ``exact_weights`` (True: the softmax
weights stay float32 until they have met the values; same kernel), ``tensors`` (a dict
q/k/v/o -> full tensor names where they are not ``<prefix>.{q,k,v,o}_proj.weight``).
A ``qk_transform`` that offers ``prepare(qkv, ctx, cache, attention) -> q`` is given the
float32 result of the stacked projection instead: it returns the queries in the model dtype
and writes keys and values into the cache itself (one kernel between the product and the
attention, as the rotary kernel is for Llama); it needs ``position`` None.
``segment`` (C: positions are cut into segments of C counted from 0 of the sequence, and a query
sees only the earlier keys of its own segment), ``bias`` (True: q, k and v have biases, tensors
``<weight name>.b`` or ``tensors`` entries q_bias / k_bias / v_bias, float32, handed to a
``qk_transform`` with ``prepare``, which adds them), ``differential`` (a dict {``diff``, ``eps``,
``tensors``: lq1, lk1, lq2, lk2 -> full names of float32 vectors [head_dim]}: every head has TWO
attention maps over the same values, q [H * 2 * hd] and k [G * 2 * hd] laid out head by head as
[map 1, map 2]; with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff the head's output is
a1 - lambda a2, divided by its root mean square over the head's values (eps inside the root) and
multiplied by 1 - diff.  The two maps run as 2H query heads over 2G key heads and G value heads,
the queries' rows reordered when the weights are bound so that the heads of a key head are
neighbours; the maps' outputs stay float32 until they are combined).
``score_mix`` (the full name of a float32 tensor M [H, H]: the heads' scaled scores are mixed before mask and
softmax, s_h = sum_g M[h, g] * scale * q_g . k_kv(g); such a layer runs a kernel of its own, csrc/attention_mixed.cu,
which holds all heads of a tile of rows in one CTA, and needs a ``qk_transform`` with ``prepare``),
``sink`` ("zero": a term exp(0) = 1 joins every head's softmax denominator, a sink without key, value or tensor;
or the full name of a float32 tensor [H] of learned sink scores; taken by the mixed kernel and by the kernels
that take ``sinks``).
Tensors: ``<prefix>.{q,k,v,o}_proj.weight`` with shapes [H*hd, d], [G*hd, d],
[G*vd, d], [d, H*vd]; no bias (reference backend/model.cu:1090-1104).  At bind time
q, k and v are stacked into one [(H+2G)*hd, d] matrix so the three projections are
one product.

Interface of a mixer part:
  ``cache_need()`` -> PagedKVNeed | StateNeed | None
  ``forward(xn, ctx, cache) -> [n, hidden]`` in float32 or the model dtype, xn being
  the normed input [n, hidden]; the residual sum is the block's business.
  Optional: ``forward_residual(x, norm, ctx, cache) -> bool`` takes the float32
  residual stream itself, applies ``norm`` inside its first kernel and adds its
  result into x; it returns False when it cannot (sizes, dtype, kind of norm) and
  the block then takes the general route.  Here it serves steps of a few tokens
  (decode): both projections become weight-streaming products with the norm as
  prologue and the residual sum as epilogue (csrc/skinny_gemm.cu).
The new keys and values of a step are written to the pages before attention runs,
so a query sees the keys of its own portion through the cache, like every other
key (reference :1096-1102).
"""
from __future__ import annotations

import math

import torch

from .. import kernels
from .spec import BuildEnv, PagedKVNeed, PartSpec, TensorSpec, part_factory, register_part


class PagedAttention:
    def __init__(self, spec: PartSpec, env: BuildEnv):
        p = spec.params
        self.hidden = int(p["hidden"])
        self.n_heads = int(p["n_heads"])
        self.n_kv = int(p["n_kv_heads"])
        self.head_dim = int(p["head_dim"])
        if self.n_heads % self.n_kv:
            raise ValueError(f"{self.n_heads} heads are not a multiple of {self.n_kv} kv heads")
        self.window = p.get("window")
        self.scale = float(p.get("scale") or 1.0 / math.sqrt(self.head_dim))
        self.v_head_dim = int(p.get("v_head_dim") or self.head_dim)
        self.exact_weights = bool(p.get("exact_weights", False))
        self.segment = int(p.get("segment") or 0)
        self.has_bias = bool(p.get("bias", False))
        self.differential = p.get("differential")
        self.maps = 2 if self.differential else 1
        self.q_dim = self.n_heads * self.maps * self.head_dim
        self.kv_dim = self.n_kv * self.maps * self.head_dim
        self.v_dim = self.n_kv * self.v_head_dim
        self.o_dim = self.n_heads * self.v_head_dim
        self.prefix = spec.prefix
        self.names = dict(p.get("tensors") or {})
        self.dtype = env.dtype
        pos = p.get("position")
        self.position = part_factory("position", pos.kind)(pos, env) if pos is not None else None
        qt = p.get("qk_transform")
        self.qk_transform = part_factory("qk_transform", qt.kind)(qt, env) if qt is not None else None
        self._prepares = hasattr(self.qk_transform, "prepare")
        if self._prepares and pos is not None:
            raise ValueError("attention: a qk_transform that stores keys and values goes without a position part")
        if (self.has_bias or self.differential) and not self._prepares:
            raise ValueError("attention: biases and differential maps need a qk_transform that takes the float32 "
                             "projections (prepare)")
        self.bias = None
        self.lam = 0.0
        self.mix_name = p.get("score_mix")
        self.mix = None
        self.sink_name = p.get("sink")
        self.sinks = None
        if self.sink_name == "zero":
            self.sinks = torch.zeros(self.n_heads, dtype=torch.float32, device=env.device)
        if self.mix_name and (not self._prepares or self.differential or self.segment or p.get("score_slopes")):
            raise ValueError("attention: mixed scores need a qk_transform that stores keys and values (prepare) and go "
                             "without differential maps, segments and score slopes")
        if self.sink_name and not self._prepares:
            raise ValueError("attention: a sink needs a qk_transform that stores keys and values (prepare)")
        slopes = p.get("score_slopes")
        if slopes == "geometric":
            # the slopes 2^(-8 (h + 1) / H) of a bias that grows with the distance, head by head
            slopes = [2.0 ** (-8.0 * (h + 1) / self.n_heads) for h in range(self.n_heads)]
        if slopes is not None and len(slopes) != self.n_heads:
            raise ValueError(f"score_slopes: {len(slopes)} values for {self.n_heads} heads")
        self.score_slopes = None if slopes is None else torch.tensor([float(v) for v in slopes], dtype=torch.float32,
                                                                     device=env.device)
        self.w_qkv = None
        self.w_o = None
        # Zeroed scratch of the fused decode kernel, which leaves it zero.  A captured decode
        # graph holds the address of the buffer it was recorded with, so a buffer is never
        # freed once it has been used: a larger step gets a new one and the old ones stay.
        self._counters = None
        self._counters_kept = []
        self._after = []           # weights streamed right after this part (see set_prefetch_targets)

    def _names(self):
        n = {k: self.names.get(k) or f"{self.prefix}.{k}_proj.weight" for k in "qkvo"}
        for k in "qkv":
            n[k + "_bias"] = self.names.get(k + "_bias") or n[k] + ".b"
        return n

    def tensor_specs(self):
        n = self._names()
        out = [TensorSpec(n["q"], (self.q_dim, self.hidden)),
               TensorSpec(n["k"], (self.kv_dim, self.hidden)),
               TensorSpec(n["v"], (self.v_dim, self.hidden)),
               TensorSpec(n["o"], (self.hidden, self.o_dim))]
        if self.has_bias:
            out += [TensorSpec(n["q_bias"], (self.q_dim,), store="float32", init="normal"),
                    TensorSpec(n["k_bias"], (self.kv_dim,), store="float32", init="normal"),
                    TensorSpec(n["v_bias"], (self.v_dim,), store="float32", init="normal")]
        if self.differential:
            out += [TensorSpec(self.differential["tensors"][k], (self.head_dim,), store="float32", init="normal")
                    for k in ("lq1", "lk1", "lq2", "lk2")]
        if self.mix_name:
            out.append(TensorSpec(self.mix_name, (self.n_heads, self.n_heads), store="float32", init="eye"))
        if self.sink_name and self.sink_name != "zero":
            out.append(TensorSpec(self.sink_name, (self.n_heads,), store="float32", init="zeros"))
        return out + (self.position.tensor_specs() if self.position else []) + \
            (self.qk_transform.tensor_specs() if self.qk_transform else [])

    def _by_key_head(self, t):
        """Rows of a query tensor [H * maps * hd, ...] laid out head by head as [map 1, map 2], reordered to
        [kv head][map][head of the group]: the heads that share a key head (of one map) become neighbours."""
        if self.maps == 1:
            return t
        gs = self.n_heads // self.n_kv
        rest = tuple(t.shape[1:])
        t = t.reshape((self.n_kv, gs, self.maps, self.head_dim) + rest)
        return t.transpose(1, 2).reshape((self.q_dim,) + rest)

    def bind(self, tensors):
        n = self._names()
        self.w_qkv = torch.cat([self._by_key_head(tensors[n["q"]]), tensors[n["k"]], tensors[n["v"]]], dim=0).contiguous()
        self.w_o = tensors[n["o"]]
        if self.has_bias:
            self.bias = torch.cat([self._by_key_head(tensors[n["q_bias"]]), tensors[n["k_bias"]],
                                   tensors[n["v_bias"]]]).contiguous()
        if self.differential:
            import math
            v = {k: tensors[self.differential["tensors"][k]].double() for k in ("lq1", "lk1", "lq2", "lk2")}
            self.lam = (math.exp(float((v["lq1"] * v["lk1"]).sum())) - math.exp(float((v["lq2"] * v["lk2"]).sum()))
                        + float(self.differential["diff"]))
        if self.mix_name:
            self.mix = tensors[self.mix_name].contiguous()
        if self.sink_name and self.sink_name != "zero":
            self.sinks = tensors[self.sink_name].contiguous()
        if self.position:
            self.position.bind(tensors)
        if self.qk_transform:
            self.qk_transform.bind(tensors)

    def cache_need(self):
        return PagedKVNeed(self.n_kv * self.maps, self.head_dim, self.window,
                           None if self.v_head_dim == self.head_dim else self.v_head_dim,
                           n_v_heads=self.n_kv if self.maps > 1 else None)

    def _split(self, qkv, writes):
        q = qkv[:, :self.q_dim]
        if not writes:
            return q, q, q
        if self.v_head_dim != self.head_dim:
            raise ValueError("attention: values of another size than the keys need a qk_transform that stores them "
                             "(the rotary kernels write keys and values of one size)")
        return q, qkv[:, self.q_dim:self.q_dim + self.kv_dim], qkv[:, self.q_dim + self.kv_dim:]

    def streamed_weights(self):
        """The matrices this part streams in a small step, in kernel order."""
        return [self.w_qkv, self.w_o]

    def set_prefetch_targets(self, weights):
        """What the kernels after this part stream first (the next part's
        ``streamed_weights``): in a small step the attention kernel and the output
        projection ask for them to be brought into L2 while they run."""
        self._after = list(weights)

    def _target(self, i):
        return self._after[i] if i < len(self._after) else None

    def _attend_prepared(self, qkv, ctx, cache):
        """The route of a ``qk_transform`` with ``prepare``: it takes the float32 projections,
        returns q and has stored k and v."""
        q = self.qk_transform.prepare(qkv, ctx, cache, self)
        n = q.shape[0]
        attn = torch.empty((n, self.o_dim), dtype=self.dtype, device=q.device)
        if self.mix is not None:
            kernels.attention_mixed(attn, q, cache.k, cache.v, self.mix, ctx, cache.block_table, self.n_heads, self.n_kv,
                                    self.head_dim, self.v_head_dim, self.window or 0, self.scale, sinks=self.sinks)
            return attn
        if self.maps == 1:
            kernels.attention(attn, q, cache.k, cache.v, ctx, cache.block_table, self.n_heads, self.n_kv,
                              self.head_dim, self.window or 0, self.scale, score_slopes=self.score_slopes,
                              v_head_dim=self.v_head_dim, exact_weights=self.exact_weights, segment=self.segment,
                              sinks=self.sinks)
            return attn
        # two maps per head: 2H query heads over 2G key heads and G value heads, combined afterwards
        both = torch.empty((n, self.maps * self.o_dim), dtype=torch.float32, device=q.device)
        kernels.attention(both, q, cache.k, cache.v, ctx, cache.block_table, self.n_heads * self.maps,
                          self.n_kv * self.maps, self.head_dim, self.window or 0, self.scale,
                          score_slopes=self.score_slopes, v_head_dim=self.v_head_dim, exact_weights=True,
                          segment=self.segment)
        kernels.maps_combine(attn, both, self.n_kv, self.n_heads // self.n_kv, self.v_head_dim, self.lam,
                             float(self.differential["eps"]), 1.0 - float(self.differential["diff"]))
        return attn

    def _attend(self, q, k, v, ctx, cache, prefetch=None):
        n = q.shape[0]
        group = self.n_heads // self.n_kv
        table = getattr(self.position, "full_rotary_table", lambda: None)() if self.position is not None else None
        if self.qk_transform is not None:
            self.qk_transform.apply(q, k if cache.writes else None, ctx, self.n_heads, self.n_kv, self.head_dim)
            table = None          # the fused decode kernel takes the raw projections
        if self.score_slopes is not None or self.v_head_dim != self.head_dim or self.exact_weights or self.segment:
            table = None          # ... and has no bias on its scores, one head size, bfloat16 weights, no segments
        if (table is not None and cache.writes and ctx.all_single and self.dtype == torch.bfloat16 and group <= 16
                and self.head_dim in kernels.TC_HEAD_DIMS and self.head_dim % 32 == 0):
            # decode: rotary encoding, cache write and attention in one kernel
            if self._counters is None or self._counters.numel() < n * self.n_kv:
                if self._counters is not None:
                    self._counters_kept.append(self._counters)
                self._counters = torch.zeros(max(256, 2 * n) * self.n_kv, dtype=torch.int32, device=q.device)
            attn = torch.empty((n, self.q_dim), dtype=self.dtype, device=q.device)
            kernels.attention_decode_fused(
                attn, q, k, v, table, cache.k, cache.v, ctx.positions, None, cache.block_table,   # token t is request t
                self._counters, self.n_heads, self.n_kv, self.head_dim, self.window or 0, self.scale,
                kernels.decode_splits(n, self.n_kv, ctx.split_bound or ctx.max_ctx), prefetch=prefetch)
            return attn
        if self.position is not None:
            self.position.apply(q, k, v, ctx, cache, self.n_heads, self.n_kv)
        elif cache.writes:
            kernels.rope_append(q, k, v, None, ctx.positions, ctx.token_req, cache.block_table,
                                cache.k, cache.v, self.n_heads, self.n_kv, self.head_dim)
        attn = torch.empty((n, self.o_dim), dtype=self.dtype, device=q.device)
        kernels.attention(attn, q, cache.k, cache.v, ctx, cache.block_table, self.n_heads, self.n_kv,
                          self.head_dim, self.window or 0, self.scale, score_slopes=self.score_slopes,
                          v_head_dim=self.v_head_dim, exact_weights=self.exact_weights, segment=self.segment)
        return attn

    def forward(self, xn, ctx, cache):
        # a layer that reads another layer's cache projects its queries only
        w = self.w_qkv if cache.writes else self.w_qkv[:self.q_dim]
        if self._prepares:
            attn = self._attend_prepared(kernels.linear(xn, w, out_dtype=torch.float32, small_ok=True), ctx, cache)
            return kernels.linear(attn, self.w_o, out_dtype=torch.float32, small_ok=True)
        q, k, v = self._split(kernels.linear(xn, w), cache.writes)
        attn = self._attend(q, k, v, ctx, cache)
        # float32 out: the result goes into the residual stream unrounded
        return kernels.linear(attn, self.w_o, out_dtype=torch.float32)

    def forward_residual(self, x, norm, ctx, cache):
        n = x.shape[0]
        if self._prepares:
            return False
        w = self.w_qkv if cache.writes else self.w_qkv[:self.q_dim]
        if not (getattr(norm, "fusable_rmsnorm", False) and kernels.skinny_fits(n, self.hidden, self.dtype)
                and kernels.skinny_fits(n, self.q_dim, self.dtype, sliced=True)):
            # larger steps: the library's products, the last one adding into the residual stream
            q, k, v = self._split(kernels.linear(norm.forward(x, None), w), cache.writes)
            kernels.linear_add(x, self._attend(q, k, v, ctx, cache), self.w_o)
            return True
        qkv = kernels.skinny_gemm(w, x_f32=x, gain=norm.gain, eps=norm.eps, epilogue="store")
        q, k, v = self._split(qkv, cache.writes)
        attn = self._attend(q, k, v, ctx, cache, prefetch=self._target(0))
        kernels.skinny_gemm(self.w_o, x=attn, epilogue="add", out=x, prefetch=self._target(1))
        return True


register_part("mixer", "paged_attention", PagedAttention)
