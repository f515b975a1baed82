"""Routed experts: a feed-forward in which every token runs ``top`` of ``experts`` small
gated feed-forwards, chosen by a router.

    z = W_router h (float32);  s = sigmoid(z) or softmax(z);  the ``top`` largest s are chosen
    expert_e(x) = W_down,e (silu(W_gate,e x) * (W_up,e x))
    y = sum over the chosen e of  expert_e(s_e h)        (``weight_on`` "input")
     or sum over the chosen e of  s_e expert_e(h)        (``weight_on`` "output")

params: ``hidden``, ``experts``, ``top``, ``expert_ff``, ``score`` ("sigmoid" | "softmax"),
``renormalize`` (divide the chosen scores by their sum), ``weight_on`` ("input" | "output"),
optional ``router_tensor`` and ``expert_tensors`` (a format string with ``{e}`` and ``{m}``
for the expert's number and matrix gate/up/down; default ``<prefix>.e{e}.{m}``).
The router table stays float32 in both dtypes.  At bind time the experts' matrices are
stacked into [E, 2f, d] (gate rows, then up rows) and [E, d, f].

Further options, all absent by default:
``groups`` {``count``, ``keep``}: the experts form ``count`` equal groups of neighbours, a group scores as
its best expert, and only experts of the ``keep`` best groups can be chosen (the scores stay those over
all experts).
``routing`` "table": no router; an integer table ``table_tensor`` [vocab, top] gives every token
id its experts (the entries of a row differ), each with the weight ``table_weight`` (default
1 / top), applied where ``weight_on`` says.  The ids are the step's own (``ctx.token_ids``;
an id that is still on the device from the step before is resolved there).
``activation`` "clamped" with ``limit`` L and ``alpha`` a: the expert computes
W_down (g sigmoid(a g) (u + 1)) with g = min(W_gate x, L), u = clamp(W_up x, -L, L) instead
of silu(W_gate x) * (W_up x).
``planned_rows`` (128): with a table, a step whose ids the host knows and that brings at least this
many rows per expert on average is sorted by the host: every expert's rows become a block padded to
the fullest expert's count and the experts' products two batched products of the library (the
grouped kernels find their ranges on the device and reach a sixth of the library's speed over a
prompt); not when one expert's share would make the padding more than double the work.
``shared``: a dict {``ff``, ``activation``, ``limit``, ``alpha``, ``tensors`` (gate, up, down and
optionally gate_logit -> full names)}: one more expert that every token runs, added to the
routed ones, multiplied by sigmoid(w . x) when ``gate_logit`` names a [1, d] tensor.  Its gate,
up and logit rows are one product; the sigmoid and the sum are part of the combine kernel.

A step sorts its (token, choice) pairs by expert on the device and runs two grouped
products over the sorted rows (csrc/moe.cu); shapes and launch sizes depend on the number
of tokens alone, never on the routing, so decode steps can be replayed as CUDA graphs.
The result is float32 [n, hidden].
"""
from __future__ import annotations

import torch

from .. import kernels
from .spec import BuildEnv, PartSpec, TensorSpec, register_part


class RoutedExperts:
    def __init__(self, spec: PartSpec, env: BuildEnv):
        p = spec.params
        self.hidden = int(p["hidden"])
        self.experts = int(p["experts"])
        self.top = int(p["top"])
        self.ff = int(p["expert_ff"])
        if not (1 <= self.top <= self.experts <= 1024):
            raise ValueError(f"routed experts: {self.top} of {self.experts} (at most 1024 experts)")
        self.score = p.get("score", "sigmoid")
        self.renormalize = bool(p.get("renormalize", False))
        self.weight_on = p.get("weight_on", "input")
        if self.score not in ("sigmoid", "softmax") or self.weight_on not in ("input", "output"):
            raise ValueError(f"routed experts: score {self.score!r}, weight on {self.weight_on!r}")
        self.router_name = p.get("router_tensor") or f"{spec.prefix}.router"
        self.fmt = p.get("expert_tensors") or (spec.prefix + ".e{e}.{m}")
        self.dtype = env.dtype
        self.routing = p.get("routing", "scores")
        if self.routing not in ("scores", "table"):
            raise ValueError(f"routed experts: routing {self.routing!r} (scores, table)")
        self.table_name = p.get("table_tensor") or f"{spec.prefix}.table"
        self.table_weight = float(p.get("table_weight") or 1.0 / self.top)
        self.table_vocab = int(p.get("vocab") or 0)
        if self.routing == "table" and self.table_vocab <= 0:
            raise ValueError("routed experts: a routing table needs the vocabulary's size ('vocab')")
        grp = p.get("groups") or {}
        self.groups, self.groups_keep = int(grp.get("count") or 1), int(grp.get("keep") or 1)
        if self.groups > 1 and (self.experts % self.groups or not (1 <= self.groups_keep <= self.groups)
                                or self.top > self.groups_keep * (self.experts // self.groups)):
            raise ValueError(f"routed experts: {self.top} of {self.experts} experts in {self.groups} groups of which "
                             f"{self.groups_keep} are kept")
        self.act = self._activation(p)
        # a step with at least this many rows per expert on average, a table and ids that the host knows runs
        # the library's products expert by expert (``_forward_planned``); below it the grouped kernels
        self.planned_rows = int(p.get("planned_rows") or 128)
        sh = p.get("shared")
        self.shared = None
        if sh:
            self.shared = {"ff": int(sh["ff"]), "act": self._activation(sh), "names": dict(sh["tensors"])}

    @staticmethod
    def _activation(p):
        kind = p.get("activation", "silu")
        if kind not in ("silu", "clamped"):
            raise ValueError(f"routed experts: activation {kind!r} (silu, clamped)")
        limit, alpha = float(p.get("limit") or 0.0), float(p.get("alpha") or 1.0)
        if kind == "clamped" and not limit > 0:
            raise ValueError("routed experts: the clamped activation needs a positive limit")
        return {"activation": kind, "limit": limit, "alpha": alpha}

    def _name(self, e, m):
        return self.fmt.format(e=e, m=m)

    def tensor_specs(self):
        if self.routing == "table":
            out = [TensorSpec(self.table_name, (self.table_vocab, self.top), store="int32",
                              init=f"distinct:{self.experts}")]
        else:
            out = [TensorSpec(self.router_name, (self.experts, self.hidden), store="float32")]
        if self.shared:
            f, n = self.shared["ff"], self.shared["names"]
            out += [TensorSpec(n["gate"], (f, self.hidden)), TensorSpec(n["up"], (f, self.hidden)),
                    TensorSpec(n["down"], (self.hidden, f))]
            if n.get("gate_logit"):
                out.append(TensorSpec(n["gate_logit"], (1, self.hidden)))
        for e in range(self.experts):
            out += [TensorSpec(self._name(e, "gate"), (self.ff, self.hidden)),
                    TensorSpec(self._name(e, "up"), (self.ff, self.hidden)),
                    TensorSpec(self._name(e, "down"), (self.hidden, self.ff))]
        return out

    def bind(self, tensors):
        self.router = tensors[self.router_name] if self.routing == "scores" else None
        self.table = tensors[self.table_name].contiguous() if self.routing == "table" else None
        # for steps planned on the host; 16-bit, which numpy sorts by radix
        self.table_host = self.table.cpu().numpy().astype("int16") if self.routing == "table" else None
        if self.shared:
            n = self.shared["names"]
            rows = [tensors[n["gate"]], tensors[n["up"]]] + ([tensors[n["gate_logit"]]] if n.get("gate_logit") else [])
            self.shared["w_in"] = torch.cat(rows, dim=0).contiguous()       # gate rows, up rows, the logit's row
            self.shared["w_down"] = tensors[n["down"]]
        self.w_gate_up = torch.stack([torch.cat([tensors[self._name(e, "gate")], tensors[self._name(e, "up")]], dim=0)
                                      for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([tensors[self._name(e, "down")] for e in range(self.experts)]).contiguous()

    def _shared(self, xn):
        """(rows float32 [n, d], gate logits float32 [n, 1] or None) of the expert that every token runs."""
        sh, f = self.shared, self.shared["ff"]
        gu = kernels.linear(xn, sh["w_in"], out_dtype=torch.float32, small_ok=True)
        act = torch.empty((xn.shape[0], f), dtype=self.dtype, device=xn.device)
        if sh["act"]["activation"] == "clamped":
            kernels.clamped_glu(act, gu[:, :f], gu[:, f:2 * f], sh["act"]["limit"], sh["act"]["alpha"])
        else:
            kernels.silu_mul(act, gu[:, :f], gu[:, f:2 * f])
        rows = kernels.linear(act, sh["w_down"], out_dtype=torch.float32, small_ok=True)
        return rows, (gu[:, 2 * f:] if gu.shape[1] > 2 * f else None)

    def _plan(self, ctx, n):
        """The host's sort of a step's (token, choice) pairs by expert, for a table and ids that the host knows:
        (rows per expert padded to the fullest expert's count, for every padded row the token it reads, for
        every pair its padded row), or None when one expert has so many rows that padding would more than
        double the work."""
        import numpy as np
        top, E = self.top, self.experts
        flat = self.table_host[ctx.host_token_ids].reshape(-1)
        counts = np.bincount(flat, minlength=E)
        width = int(counts.max())
        if width * E > 2 * n * top:
            return None
        order = np.argsort(flat, kind="stable")
        starts = np.concatenate([[0], np.cumsum(counts)[:-1]])
        sorted_expert = flat[order].astype(np.int64)
        padded = sorted_expert * width + (np.arange(n * top) - starts[sorted_expert])     # sorted row -> padded row
        src = np.zeros(E * width, dtype=np.int32)              # rows that pad an expert read token 0; nobody reads them back
        src[padded] = order // top
        back = np.empty(n * top, dtype=np.int32)
        back[order] = padded
        return width, src, back

    def _forward_planned(self, xn, plan):
        """A large step sorted by the host: every expert's rows are a block of equal (padded) height, so the
        experts' products are two batched products of the library over gathered rows."""
        n, top, E, f = xn.shape[0], self.top, self.experts, self.ff
        import numpy as np
        width, src, back = plan
        host = torch.from_numpy(np.concatenate([src, back]))
        if xn.is_cuda:
            host = host.pin_memory()
        idx = host.to(xn.device, non_blocking=True)
        xs = torch.empty((E * width, self.hidden), dtype=self.dtype, device=xn.device)
        kernels.gather_rows(xs, xn, idx[:E * width])
        gu = kernels.linear_batched(xs.view(E, width, self.hidden), self.w_gate_up).view(E * width, 2 * f)
        act = torch.empty((E * width, f), dtype=self.dtype, device=xn.device)
        if self.act["activation"] == "clamped":
            kernels.clamped_glu(act, gu[:, :f], gu[:, f:], self.act["limit"], self.act["alpha"])
        else:
            kernels.silu_mul(act, gu[:, :f], gu[:, f:])
        rows = kernels.linear_batched(act.view(E, width, f), self.w_down).view(E * width, self.hidden)
        parts = torch.empty((n * top, self.hidden), dtype=torch.float32, device=xn.device)
        kernels.gather_rows(parts, rows, idx[E * width:])
        shared, logit = self._shared(xn) if self.shared is not None else (None, None)
        return kernels.moe_combine(parts, top, shared=shared, gate=logit, scale=self.table_weight)

    def forward(self, xn, ctx):
        if (self.routing == "table" and self.weight_on == "output" and getattr(ctx, "host_token_ids", None) is not None
                and xn.shape[0] * self.top >= self.planned_rows * self.experts):
            plan = self._plan(ctx, xn.shape[0])
            if plan is not None:
                return self._forward_planned(xn, plan)
        if self.routing == "table":
            idx, wt = kernels.moe_table_route(ctx.token_ids, self.table, self.experts, self.table_weight, ctx.last_token)
        else:
            idx, wt = kernels.moe_route(xn, self.router, self.top, self.score, self.renormalize, self.groups,
                                        self.groups_keep)
        offsets, perm = kernels.moe_sort(idx, self.experts)
        on_input = self.weight_on == "input"
        if kernels.moe_gemm_tcgen05_pays(xn, self.w_gate_up, perm.numel(), True, on_input):
            # a large step in bfloat16: tiles of 128 rows per expert on the tcgen05 tensor cores
            act = kernels.moe_gemm_tcgen05(xn, self.w_gate_up, offsets, perm, wt, self.top, gated=True, **self.act)
            parts = kernels.moe_gemm_tcgen05(act, self.w_down, offsets, perm, wt, self.top, gated=False, scale_out=True)
        else:
            act = kernels.moe_gemm(xn, self.w_gate_up, offsets, perm, wt, self.top, gated=True, scale_in=on_input, **self.act)
            parts = kernels.moe_gemm(act, self.w_down, offsets, perm, wt, self.top, gated=False, scale_out=not on_input)
        if self.shared is None:
            return kernels.moe_combine(parts, self.top)
        rows, logit = self._shared(xn)
        return kernels.moe_combine(parts, self.top, shared=rows, gate=logit)


register_part("feed_forward", "routed_experts", RoutedExperts)
