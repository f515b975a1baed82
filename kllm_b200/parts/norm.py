"""RMSNorm with the residual sum folded in, and layer norm with gain and bias (``LayerNorm``, at the end).

params: ``width``, ``eps``, optional ``tensor`` (the gain's full name where it is not
``<prefix>.weight``), optional ``offset`` (the files hold the gain minus this number, e.g. a weight
stored around zero that acts as 1 + w: the offset is added once, in float32, when the weights are bound;
random weights then start at zero).  Tensor: ``<prefix>.weight`` [width], kept in float32
(reference backend/model.cu:101-122, 144-165; the gain is used as stored, no 1 + w).
Interface of a norm part:
``forward(x, res, rows=None) -> out``: x is the float32 residual stream [n, width];
``res`` (float32 or model dtype, or None) is added into x first and x is written back; the
result is in the model dtype.  With ``rows`` only those rows are normalised and x
is left as it is.
``add_normed(x, y, then=None)``: x += rmsnorm(y) * gain for a float32 sublayer output y, the
form of a norm that sits AFTER a sublayer; with ``then`` (another norm of this kind) it also
returns that norm of the updated x, computed in the same kernel; with ``then="rows"`` it returns the
updated rows themselves in the model dtype (for a sublayer that reads the stream without a norm in front).

A part that can apply this norm inside its own kernel (see ``forward_residual`` of
the attention and feed-forward parts) recognises it by ``fusable_rmsnorm`` and
reads ``gain`` and ``eps``.
"""
from __future__ import annotations

import torch

from .. import kernels
from .spec import BuildEnv, PartSpec, TensorSpec, register_part


class RMSNorm:
    fusable_rmsnorm = True

    def __init__(self, spec: PartSpec, env: BuildEnv):
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.name = spec.params.get("tensor") or spec.prefix + ".weight"
        self.offset = float(spec.params.get("offset") or 0.0)
        self.dtype = env.dtype
        self.gain = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.width,), store="float32", init="zeros" if self.offset else "gain")]

    def bind(self, tensors):
        self.gain = tensors[self.name] + self.offset if self.offset else tensors[self.name]

    def forward(self, x, res=None, rows=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.width), dtype=self.dtype, device=x.device)
        kernels.add_rmsnorm(x, res, out, self.gain, self.eps, rows=rows)
        return out


    def add_normed(self, x, y, then=None):
        if then is None:
            kernels.rmsnorm_add(x, y, self.gain, self.eps)
            return None
        out = torch.empty(x.shape, dtype=self.dtype, device=x.device)
        if isinstance(then, str):
            if then != "rows":
                raise ValueError(f"add_normed: then={then!r} (a norm, or 'rows')")
            kernels.rmsnorm_add(x, y, self.gain, self.eps, out=out)
            return out
        kernels.rmsnorm_add(x, y, self.gain, self.eps, out=out, gain2=then.gain, eps2=then.eps)
        return out


class LayerNorm:
    """Layer norm with gain and bias: (x - mean) / sqrt(var + eps) * w + b, the variance being the
    mean of the squared deviations.  params: ``width``, ``eps``, optional ``tensor`` (the gain's
    full name where it is not ``<prefix>.weight``) and ``bias_tensor`` (default: the gain's name
    + ``.b``).  Both tensors stay float32; mean, variance and scale are float32 in both dtypes.
    Same interface as ``RMSNorm.forward``; no part folds this norm into its own kernels."""

    def __init__(self, spec: PartSpec, env: BuildEnv):
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.name = spec.params.get("tensor") or spec.prefix + ".weight"
        self.bias_name = spec.params.get("bias_tensor") or self.name + ".b"
        self.dtype = env.dtype
        self.gain = self.bias = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.width,), store="float32", init="gain"),
                TensorSpec(self.bias_name, (self.width,), store="float32", init="zeros")]

    def bind(self, tensors):
        self.gain, self.bias = tensors[self.name], tensors[self.bias_name]

    def forward(self, x, res=None, rows=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.width), dtype=self.dtype, device=x.device)
        kernels.add_layernorm(x, res, out, self.gain, self.bias, self.eps, rows=rows)
        return out


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "layernorm", LayerNorm)
