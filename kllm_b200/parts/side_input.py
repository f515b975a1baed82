"""A per-layer input from the token itself: a second embedding table gives every token a row of
L * P values, layer i reads columns [i P, (i + 1) P), and

    e = table[token, i P : (i + 1) P]
    y = W_proj (gelu_tanh(W_gate h) * e)            h: the residual stream, [n, hidden]

which the block norms and adds to the stream (``OutputNormBlock``: ``side`` / ``side_norm``).

params: ``hidden``, ``dim`` (P), ``offset`` (i P), ``columns`` (L P), ``vocab``, ``table`` (the table's full
tensor name, shared by all layers), ``gate`` / ``proj`` (full names, [P, hidden] and [hidden, P]).
The gate's product comes out in float32 and meets the activation and the table's values unrounded
(csrc/embedding.cu, gated_slice); the result is float32 [n, hidden].

Interface of a side-input part: ``forward(h, ctx) -> [n, hidden]`` float32; it may read ``ctx.token_ids``
(an id -(s + 1) stands for ``ctx.last_token[s]``).
"""
from __future__ import annotations

import torch

from .. import kernels
from .spec import BuildEnv, PartSpec, TensorSpec, register_part


class TokenSideInput:
    def __init__(self, spec: PartSpec, env: BuildEnv):
        p = spec.params
        self.hidden, self.dim = int(p["hidden"]), int(p["dim"])
        self.offset, self.columns, self.vocab = int(p["offset"]), int(p["columns"]), int(p["vocab"])
        if not (0 <= self.offset and self.offset + self.dim <= self.columns):
            raise ValueError(f"token side input: columns [{self.offset}, {self.offset + self.dim}) of {self.columns}")
        self.table_name, self.gate_name, self.proj_name = p["table"], p["gate"], p["proj"]
        self.dtype = env.dtype

    def tensor_specs(self):
        return [TensorSpec(self.table_name, (self.vocab, self.columns)),
                TensorSpec(self.gate_name, (self.dim, self.hidden)),
                TensorSpec(self.proj_name, (self.hidden, self.dim))]

    def bind(self, tensors):
        self.table = tensors[self.table_name]
        self.w_gate, self.w_proj = tensors[self.gate_name], tensors[self.proj_name]

    def forward(self, h, ctx):
        gate = kernels.linear(h, self.w_gate, out_dtype=torch.float32, small_ok=True)
        g = kernels.gated_slice(gate, self.table, self.offset, ctx.token_ids, ctx.last_token)
        return kernels.linear(g, self.w_proj, out_dtype=torch.float32, small_ok=True)


register_part("side_input", "token_side", TokenSideInput)
