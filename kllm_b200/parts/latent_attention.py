"""Attention through low-rank latents over a paged cache, without positions.

    c_q = rmsnorm(W_dq h) * g_q          query latent, Rq values
    c   = rmsnorm(W_dkv h) * g_kv        key/value latent, R values: the only thing cached
    q_h = W_uq,h c_q;  k_h = W_uk,h c;  v_h = W_uv,h c        per head h
    a_h = softmax_j( scale * q_h . k_h(j) )  over the keys j the query sees, with exp(sink_h)
          as one more term of the denominator (no key, no value, not scaled)
    out = W_o [a_1 v .. a_H v]

The keys and values are never formed.  Since q_h . (W_uk,h c_j) = (W_uk,h^T q_h) . c_j, the
queries are carried into the latent space (one small product per head) and the attention is
that of H heads over ONE key/value head whose keys and values are both the cached rows c_j;
its output, H rows of R values, goes through W_uv,h per head and then W_o.  The cache holds R
values per token, [pages, 1, page_size, R], and the attention kernels read it as keys and as
values (``PagedKVNeed.values_are_keys``).

A second form, chosen by ``rot_dim`` > 0, adds positions and drops the query latent:

    q_h = W_q,h h = [q_h plain (dk) | q_h rotated (dr)]            straight from the input
    W_dkv h = [b (R) | k_rot (dr)];  c = rmsnorm(b) * g_kv;  k_rot is rotated, one part for all heads
    score_h(j) = scale * (q_h plain . W_uk,h c_j + rot(q_h rotated) . rot(k_rot_j))
    out = W_o ([a_1 v .. a_H v] * sigmoid(W_g h))                   with ``gate``

The cached row is [c | rot(k_rot)], R + dr values, key of all heads; its first R values are also the
value (``PagedKVNeed(values_are_keys, v_head_dim=R)``; in bfloat16 with R + dr a head size of the
tensor-core kernels the whole row runs as the value and the last dr columns of every head's result are
not read).  The query that meets it is
[W_uk,h^T q_h plain | rot(q_h rotated)].  The rotation (``rotary``: {theta, scaling}, see
``rotary.rotary_frequencies``) acts on all dr values, pair (i, i + dr / 2); angles are formed in double
precision on the device, cos and sin carry the scaling's amplitude.  W_q, W_dkv and W_g are one stacked
product whose float32 result feeds one kernel (csrc/latent.cu: latent norm, both rotations, cache write).

params: ``hidden``, ``n_heads``, ``head_dim`` (dk), ``v_head_dim`` (dv), ``q_rank`` (Rq; None or 0 in
the second form), ``rot_dim`` (dr, 0: the first form), ``rotary``, ``gate``, ``q`` / ``g`` among ``tensors``,
``kv_rank`` (R), ``scale``, ``eps`` (of both latent norms), ``window`` (None: every earlier
key; W: the last W keys, the query's own included), ``cache_window`` (what the cache must
keep: the widest window of all layers that read this cache; None: everything), ``sinks`` (True:
a learned sink per head), ``own_latent`` (False: the layer reads the rows that another
layer cached, in the second form the latent and the rotated key part, and has no W_dkv), ``tensors`` (dq, dq_norm, uq, dkv, dkv_norm, uk, uv, sink, o ->
full names).
"""
from __future__ import annotations

import torch

from .. import kernels
from .spec import BuildEnv, PagedKVNeed, PartSpec, TensorSpec, register_part

_NAMES = ("dq", "dq_norm", "uq", "dkv", "dkv_norm", "uk", "uv", "sink", "o", "q", "g")


class LatentAttention:
    def __init__(self, spec: PartSpec, env: BuildEnv):
        p = spec.params
        self.hidden = int(p["hidden"])
        self.H, self.dk, self.dv = int(p["n_heads"]), int(p["head_dim"]), int(p["v_head_dim"])
        self.Rq, self.R = int(p.get("q_rank") or 0), int(p["kv_rank"])
        self.dr = int(p.get("rot_dim") or 0)
        self.gate = bool(p.get("gate", False))
        if (self.dr > 0) == (self.Rq > 0):
            raise ValueError("latent attention: either a query latent (q_rank) or rotated parts (rot_dim)")
        if (self.dr == 0 and self.gate) or self.dr % 2:
            raise ValueError("latent attention: the gate belongs to the rotated form; rot_dim must be even")
        self.freq, self.amplitude = None, 1.0
        if self.dr:
            from .rotary import rotary_frequencies
            rot = p["rotary"]
            freq, self.amplitude = rotary_frequencies(self.dr, float(rot["theta"]), rot.get("scaling"))
            self.freq = freq.to(env.device)
        self.scale = float(p["scale"])
        self.eps = float(p["eps"])
        self.window = p.get("window")
        self.cache_window = p.get("cache_window", self.window)
        if self.cache_window is not None and (self.window is None or self.window > self.cache_window):
            raise ValueError("latent attention: the cache keeps fewer keys than the layer's window sees")
        self.has_sinks = bool(p.get("sinks", False))
        self.own_latent = bool(p.get("own_latent", True))
        names = dict(p.get("tensors") or {})
        self.names = {k: names.get(k) or f"{spec.prefix}.{k}" for k in _NAMES}
        self.dtype = env.dtype
        # bfloat16 rows of a size the tensor-core attention is built for: the whole cached row serves as value
        self.whole_rows = bool(self.dr) and kernels.tensor_core_rows(self.R + self.dr, self.H, self.dtype)

    def tensor_specs(self):
        n, d, H = self.names, self.hidden, self.H
        if self.dr:
            out = [TensorSpec(n["q"], (H * (self.dk + self.dr), d)),
                   TensorSpec(n["uk"], (H * self.dk, self.R)),
                   TensorSpec(n["uv"], (H * self.dv, self.R)),
                   TensorSpec(n["o"], (d, H * self.dv))]
            if self.own_latent:
                out += [TensorSpec(n["dkv"], (self.R + self.dr, d)),
                        TensorSpec(n["dkv_norm"], (self.R,), store="float32", init="gain")]
            if self.gate:
                out.append(TensorSpec(n["g"], (H * self.dv, d)))
            if self.has_sinks:
                out.append(TensorSpec(n["sink"], (H,), store="float32", init="zeros"))
            return out
        out = [TensorSpec(n["dq"], (self.Rq, d)),
               TensorSpec(n["dq_norm"], (self.Rq,), store="float32", init="gain"),
               TensorSpec(n["uq"], (H * self.dk, self.Rq)),
               TensorSpec(n["uk"], (H * self.dk, self.R)),
               TensorSpec(n["uv"], (H * self.dv, self.R)),
               TensorSpec(n["o"], (d, H * self.dv))]
        if self.own_latent:
            out += [TensorSpec(n["dkv"], (self.R, d)),
                    TensorSpec(n["dkv_norm"], (self.R,), store="float32", init="gain")]
        if self.has_sinks:
            out.append(TensorSpec(n["sink"], (H,), store="float32", init="zeros"))
        return out

    def bind(self, tensors):
        n = self.names
        self.w_uk = tensors[n["uk"]].view(self.H, self.dk, self.R)      # head h: [dk, R], q_h^T times it
        self.w_uv = tensors[n["uv"]].view(self.H, self.dv, self.R)      # head h: [dv, R]
        self.w_o = tensors[n["o"]]
        self.sink = tensors[n["sink"]].contiguous() if self.has_sinks else None
        if self.dr:
            # queries, latent with the rotated key part, gate: one product
            # (a layer that reads another layer's cached rows has no latent of its own: queries and gate alone)
            rows = [tensors[n["q"]]] + ([tensors[n["dkv"]]] if self.own_latent else []) + \
                ([tensors[n["g"]]] if self.gate else [])
            self.w_in = torch.cat(rows, dim=0).contiguous()
            self.g_kv = tensors[n["dkv_norm"]] if self.own_latent else None
            return
        self.w_dq = tensors[n["dq"]]
        # both down-projections are one product
        self.w_down = torch.cat([tensors[n["dq"]], tensors[n["dkv"]]], dim=0).contiguous() if self.own_latent else self.w_dq
        self.g_q = tensors[n["dq_norm"]]
        self.g_kv = tensors[n["dkv_norm"]] if self.own_latent else None
        self.w_uq = tensors[n["uq"]]

    def cache_need(self):
        if not self.own_latent:
            return None
        if self.dr:
            return PagedKVNeed(1, self.R + self.dr, self.cache_window, self.R, values_are_keys=True)
        return PagedKVNeed(1, self.R, self.cache_window, None, values_are_keys=True)

    def _forward_rotated(self, xn, ctx, cache):
        n, H, R, dr = xn.shape[0], self.H, self.R, self.dr
        writes = cache.writes and self.own_latent
        proj = kernels.linear(xn, self.w_in, out_dtype=torch.float32, small_ok=True)
        q_plain = torch.empty((n, H * self.dk), dtype=self.dtype, device=xn.device)
        q_full = torch.empty((n, H * (R + dr)), dtype=self.dtype, device=xn.device)
        kernels.latent_rope_append(q_plain, q_full, proj, self.g_kv if writes else None, self.eps, self.freq,
                                   self.amplitude, ctx.positions, ctx.token_req, cache.block_table if writes else None,
                                   cache.k if writes else None, H, self.dk, dr, R)
        # the plain query parts into the latent space, into the head of every head's row
        kernels.linear_per_head(q_plain, self.w_uk, transposed=True, out=q_full.view(n, H, R + dr)[:, :, :R])
        if self.whole_rows:
            # the tensor-core kernels take values as wide as keys: the whole row is the value, and the
            # dr columns that the rotated key part adds to every head's result are left unread
            o_lat = torch.empty((n, H * (R + dr)), dtype=self.dtype, device=xn.device)
            kernels.attention(o_lat, q_full, cache.k, cache.k, ctx, cache.block_table, H, 1, R + dr, self.window or 0,
                              self.scale, sinks=self.sink, exact_weights=True)
            o = kernels.linear_per_head(o_lat.view(n, H, R + dr)[:, :, :R], self.w_uv)   # [n, H * dv]
        else:
            o_lat = torch.empty((n, H * R), dtype=self.dtype, device=xn.device)
            kernels.attention(o_lat, q_full, cache.k, cache.k, ctx, cache.block_table, H, 1, R + dr, self.window or 0,
                              self.scale, v_head_dim=R, sinks=self.sink, exact_weights=True)
            o = kernels.linear_per_head(o_lat, self.w_uv)                                # [n, H * dv]
        if self.gate:
            off = H * (self.dk + dr) + (R + dr if self.own_latent else 0)
            kernels.sigmoid_gate(o, o, proj[:, off:off + H * self.dv])
        return kernels.linear(o, self.w_o, out_dtype=torch.float32, small_ok=True)

    def forward(self, xn, ctx, cache):
        if self.dr:
            return self._forward_rotated(xn, ctx, cache)
        n = xn.shape[0]
        writes = cache.writes and self.own_latent
        proj = kernels.linear(xn, self.w_down if writes else self.w_dq, out_dtype=torch.float32, small_ok=True)
        cq = torch.empty((n, self.Rq), dtype=self.dtype, device=xn.device)
        kernels.latent_norm_append(cq, proj, self.g_q, self.g_kv if writes else None, self.eps, ctx.positions,
                                   ctx.token_req, cache.block_table if writes else None, cache.k if writes else None)
        q = kernels.linear(cq, self.w_uq)
        q_lat = kernels.linear_per_head(q, self.w_uk, transposed=True)                  # [n, H * R]
        o_lat = torch.empty((n, self.H * self.R), dtype=self.dtype, device=xn.device)
        kernels.attention(o_lat, q_lat, cache.k, cache.k, ctx, cache.block_table, self.H, 1, self.R,
                          self.window or 0, self.scale, sinks=self.sink, exact_weights=True)
        o = kernels.linear_per_head(o_lat, self.w_uv)                                    # [n, H * dv]
        return kernels.linear(o, self.w_o, out_dtype=torch.float32, small_ok=True)


register_part("mixer", "latent_attention", LatentAttention)
