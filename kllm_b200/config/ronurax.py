"""``RonuraxConfig``: the keys of a Ronurax ``config.json`` as the engine reads them.

    architecture   "Ronurax"
    vocab, width   sizes of the embedding
    norm           {eps}: of every norm of the model
    layers         a list; each entry {type, mixer, mlp, weights_of}:
                   type "attention": mixer {heads, kv_heads, dim, vdim, scale, diff, mask {size},
                       rot {base, dims, scaling {factor, low, high, original}}}
                       two attention maps per head, combined with ``diff``; mask absent: plain causal;
                       rot absent: no rotation; scaling absent: plain frequencies
                   type "latent_attention": mixer {heads, dim, rot_dim, vdim, kv_rank, scale,
                       rot {base, dims, scaling {factor, original, fast, slow}}}
                       rot.dims equals rot_dim
                   mlp null | {kind "moe", expert {ff}, router {experts, top, groups {count, keep}}}
                       groups absent: every expert can be chosen
                   weights_of j (optional): the layer has no tensors of its own and runs layer j's, with a
                       cache of its own; the rest of its entry equals layer j's

Everything a model of this design may vary is read from here; nothing is defaulted to the
values of one particular model.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigError, ModelConfig, take_float, take_int


def _obj(d, key, where="config.json"):
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: '{key}' must be an object")
    return v


@dataclass(frozen=True)
class RotaryConfig:
    base: float
    dims: int
    scaling: Optional[Tuple[Tuple[str, float], ...]]     # the scaling's keys and numbers, None: plain frequencies

    def to_dict(self):
        d = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            d["scaling"] = {k: (int(v) if k == "original" and float(v).is_integer() else v) for k, v in self.scaling}
        return d

    def scaling_dict(self):
        return dict(self.scaling) if self.scaling is not None else None


def _rotary(m, where, keys) -> Optional[RotaryConfig]:
    r = m.get("rot")
    if r is None:
        return None
    if not isinstance(r, dict):
        raise ConfigError(f"{where}: 'rot' must be an object")
    base, dims = take_float(r, "base"), take_int(r, "dims", minimum=2)
    if dims % 2 or base <= 1.0:
        raise ConfigError(f"{where}: rot.dims {dims} must be even and rot.base {base} above 1")
    sc = r.get("scaling")
    scaling = None
    if sc is not None:
        if not isinstance(sc, dict):
            raise ConfigError(f"{where}: rot.scaling must be an object")
        scaling = tuple((k, take_float(sc, k)) for k in keys)
        vals = dict(scaling)
        if vals["factor"] <= 0 or vals["original"] <= 0:
            raise ConfigError(f"{where}: rot.scaling factor and original must be positive")
        if "low" in vals and not (vals["high"] > vals["low"] > 0):
            raise ConfigError(f"{where}: rot.scaling needs 0 < low < high")
        if "fast" in vals and not (vals["fast"] > 0 and vals["slow"] > 0):
            raise ConfigError(f"{where}: rot.scaling fast and slow must be positive")
    return RotaryConfig(base, dims, scaling)


@dataclass(frozen=True)
class DiffAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    segment: Optional[int]          # mask.size; None: plain causal
    rot: Optional[RotaryConfig]

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
             "diff": self.diff}
        if self.segment is not None:
            d["mask"] = {"size": self.segment}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class RotatedLatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: RotaryConfig

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                "kv_rank": self.kv_rank, "scale": self.scale, "rot": self.rot.to_dict()}


@dataclass(frozen=True)
class RonuraxMlpConfig:
    ff: int
    experts: int
    top: int
    groups: int = 0             # 0: no groups
    keep: int = 0

    def to_dict(self):
        r = {"experts": self.experts, "top": self.top}
        if self.groups:
            r["groups"] = {"count": self.groups, "keep": self.keep}
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": r}


@dataclass(frozen=True)
class RonuraxLayerConfig:
    type: str                   # "attention" | "latent_attention"
    mixer: object
    mlp: Optional[RonuraxMlpConfig]
    weights_of: Optional[int]   # None: tensors of its own

    def to_dict(self):
        d = {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None}
        if self.weights_of is not None:
            d["weights_of"] = self.weights_of
        return d


@dataclass(frozen=True)
class RonuraxConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[RonuraxLayerConfig, ...]

    @classmethod
    def from_dict(cls, d: dict) -> "RonuraxConfig":
        vocab = take_int(d, "vocab", minimum=1)
        width = take_int(d, "width", minimum=1)
        eps = take_float(_obj(d, "norm"), "eps")
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw):
            where = f"config.json: layers[{i}]"
            if not isinstance(L, dict):
                raise ConfigError(f"{where} must be an object")
            m = _obj(L, "mixer", where)
            kind = L.get("type")
            if kind == "attention":
                mask, segment = m.get("mask"), None
                if mask is not None:
                    if not isinstance(mask, dict):
                        raise ConfigError(f"{where}: 'mask' must be an object")
                    segment = take_int(mask, "size", minimum=1)
                mixer = DiffAttentionConfig(take_int(m, "heads", minimum=1), take_int(m, "kv_heads", minimum=1),
                                            take_int(m, "dim", minimum=1), take_int(m, "vdim", minimum=1),
                                            take_float(m, "scale"), take_float(m, "diff"), segment,
                                            _rotary(m, where, ("factor", "low", "high", "original")))
                if mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"{where}: {mixer.heads} heads are not a multiple of {mixer.kv_heads} kv heads")
                if mixer.rot is not None and mixer.rot.dims > mixer.dim:
                    raise ConfigError(f"{where}: rot.dims {mixer.rot.dims} exceeds dim {mixer.dim}")
            elif kind == "latent_attention":
                rot = _rotary(m, where, ("factor", "original", "fast", "slow"))
                mixer = RotatedLatentConfig(take_int(m, "heads", minimum=1), take_int(m, "dim", minimum=1),
                                            take_int(m, "rot_dim", minimum=2), take_int(m, "vdim", minimum=1),
                                            take_int(m, "kv_rank", minimum=1), take_float(m, "scale"), rot)
                if rot is None or rot.dims != mixer.rot_dim:
                    raise ConfigError(f"{where}: 'rot' is required and rot.dims must equal rot_dim {mixer.rot_dim}")
            else:
                raise ConfigError(f"{where}: unknown layer type {kind!r} (attention, latent_attention)")
            ml, mlp = L.get("mlp"), None
            if ml is not None:
                if not isinstance(ml, dict) or ml.get("kind") != "moe":
                    raise ConfigError(f"{where}: 'mlp' must be null or an object of kind 'moe'")
                r = _obj(ml, "router", where)
                grp = r.get("groups")
                if grp is not None and not isinstance(grp, dict):
                    raise ConfigError(f"{where}: router.groups must be an object")
                mlp = RonuraxMlpConfig(take_int(_obj(ml, "expert", where), "ff", minimum=1),
                                       take_int(r, "experts", minimum=1), take_int(r, "top", minimum=1),
                                       take_int(grp, "count", minimum=1) if grp else 0,
                                       take_int(grp, "keep", minimum=1) if grp else 0)
                if mlp.top > mlp.experts:
                    raise ConfigError(f"{where}: top {mlp.top} of {mlp.experts} experts")
                if mlp.groups and (mlp.experts % mlp.groups or mlp.keep > mlp.groups
                                   or mlp.top > mlp.keep * (mlp.experts // mlp.groups)):
                    raise ConfigError(f"{where}: {mlp.experts} experts in {mlp.groups} groups of which {mlp.keep} are "
                                      f"kept cannot give {mlp.top} choices")
            src = L.get("weights_of")
            if src is not None:
                src = take_int(L, "weights_of", minimum=0)
                if src >= i or layers[src].weights_of is not None:
                    raise ConfigError(f"{where}: weights_of {src} must name an earlier layer with tensors of its own")
                if (layers[src].type, layers[src].mixer, layers[src].mlp) != (kind, mixer, mlp):
                    raise ConfigError(f"{where}: a layer that runs layer {src}'s weights must equal it in everything else")
            layers.append(RonuraxLayerConfig(kind, mixer, mlp, src))
        return cls(architecture="Ronurax", vocab=vocab, width=width, norm_eps=eps, layers=tuple(layers))

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "layers": [L.to_dict() for L in self.layers]}
