"""Linear attention with one fixed decay per head ("lightning attention"): a recurrent mixer.

With h the mixer's input:

    q, k = silu(W_q h), silu(W_k h)     [heads * dk]        v = silu(W_v h)     [heads * dv]
    S_t  = decay_h S_(t-1) + k_t v_t^T          o_t = S_t^T q_t                  per head, S [dk, dv]
    y    = W_o (rmsnorm(concat_heads(o)) * gain * sigmoid(W_g h))

the norm being ONE RMS norm over all heads' values with a plain gain.  No other scale.

params: ``hidden``, ``heads``, ``head_dim`` (dk), ``v_head_dim`` (dv), ``decay`` (one number per head, in
(0, 1]), ``eps`` (of the norm), optional ``tensors`` (q, k, v, g, norm, o -> full names; default
``<prefix>.<name>``).

State (``StateNeed``): per request one float32 vector [heads][dk][dv], zero when the request opens.
The four projections are one stacked product whose float32 result feeds the recurrence kernel; the
activation, the decay's powers, the state, the sums, the norm and the gate are float32 in both dtypes
(csrc/lightning.cu: the recurrence in chunks of rows, and the norm with the gate).  A position's result does
not depend on how its prompt was cut beyond the order of float32 additions: the state is carried through
the slot.
"""
from __future__ import annotations

import torch

from .. import kernels
from .spec import BuildEnv, PartSpec, StateNeed, TensorSpec, register_part


class LightningAttention:
    def __init__(self, spec: PartSpec, env: BuildEnv):
        p = spec.params
        self.hidden, self.heads = int(p["hidden"]), int(p["heads"])
        self.dk, self.dv = int(p["head_dim"]), int(p["v_head_dim"])
        decay = [float(v) for v in p["decay"]]
        if len(decay) != self.heads or not all(0.0 < v <= 1.0 for v in decay):
            raise ValueError(f"lightning attention: {len(decay)} decays for {self.heads} heads, each in (0, 1]")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=env.device)
        self.eps = float(p["eps"])
        self.A, self.B = self.heads * self.dk, self.heads * self.dv
        self.dtype = env.dtype
        names = dict(p.get("tensors") or {})
        self.n = {k: names.get(k) or f"{spec.prefix}.{k}" for k in ("q", "k", "v", "g", "norm", "o")}

    def tensor_specs(self):
        n, d = self.n, self.hidden
        return [TensorSpec(n["q"], (self.A, d)), TensorSpec(n["k"], (self.A, d)), TensorSpec(n["v"], (self.B, d)),
                TensorSpec(n["g"], (self.B, d)), TensorSpec(n["norm"], (self.B,), store="float32", init="gain"),
                TensorSpec(n["o"], (d, self.B))]

    def bind(self, tensors):
        n = self.n
        self.w_in = torch.cat([tensors[n[s]] for s in ("q", "k", "v", "g")], dim=0).contiguous()
        self.gain = tensors[n["norm"]]
        self.w_o = tensors[n["o"]]

    def cache_need(self):
        return StateNeed((self.heads * self.dk * self.dv,), "float32")

    def forward(self, xn, ctx, cache):
        A, B = self.A, self.B
        proj = kernels.linear(xn, self.w_in, out_dtype=torch.float32, small_ok=True)
        o = kernels.lightning_scan(proj[:, :A], proj[:, A:2 * A], proj[:, 2 * A:2 * A + B], self.decay, cache.state, ctx,
                                   self.heads, self.dk, self.dv)
        y = kernels.lightning_gate_norm(o, proj[:, 2 * A + B:], self.gain, self.eps, self.dtype)
        return kernels.linear(y, self.w_o, out_dtype=torch.float32, small_ok=True)


register_part("mixer", "lightning_attention", LightningAttention)
