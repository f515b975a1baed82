"""``SenulixConfig``: the keys of a Senulix ``config.json`` as the engine reads them.

    architecture   "Senulix"
    vocab, width   sizes of the embedding
    norm           {eps}: of every norm of the model
    token_side     {dim} (optional): every layer adds an input from the token's row of a second table, dim values a layer
    logit_softcap  c (optional): logits become c * tanh(logits / c)
    layers         a list; each entry {type, mixer, mlp}:
                   type "attention": mixer {heads, kv_heads, dim, vdim, scale, mask {size}, rot {base, dims}}
                       scores mixed across the heads, a window of mask.size keys (absent: plain causal), a sink of score 0
                   type "latent_attention": mixer {heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims}, kv_from}
                       rot.dims equals rot_dim; kv_from j (optional): the layer reads what layer j cached
                   type "lightning": mixer {heads, dim, vdim, decay [one number per head]}
                   mlp null | {kind "dense", ff}

Everything a model of this design may vary is read from here; nothing is defaulted to the
values of one particular model.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigError, ModelConfig, take_float, take_int
from .ronurax import RotaryConfig, _obj, _rotary


@dataclass(frozen=True)
class MixedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]           # mask.size; None: plain causal
    rot: Optional[RotaryConfig]

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class SharedLatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: RotaryConfig
    kv_from: Optional[int]          # None: a latent of its own

    def to_dict(self):
        d = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
             "scale": self.scale, "rot": self.rot.to_dict()}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class LightningConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class SenulixLayerConfig:
    type: str                       # "attention" | "latent_attention" | "lightning"
    mixer: object
    ff: Optional[int]               # None: no feed-forward

    def to_dict(self):
        return {"type": self.type, "mixer": self.mixer.to_dict(),
                "mlp": {"kind": "dense", "ff": self.ff} if self.ff is not None else None}


@dataclass(frozen=True)
class SenulixConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    side_dim: int                   # 0: no token side input
    logit_softcap: float            # 0: none
    layers: Tuple[SenulixLayerConfig, ...]

    @classmethod
    def from_dict(cls, d: dict) -> "SenulixConfig":
        vocab = take_int(d, "vocab", minimum=1)
        width = take_int(d, "width", minimum=1)
        eps = take_float(_obj(d, "norm"), "eps")
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        side = d.get("token_side")
        if side is not None and not isinstance(side, dict):
            raise ConfigError("config.json: 'token_side' must be an object")
        side_dim = take_int(side, "dim", minimum=1) if side else 0
        cap = take_float(d, "logit_softcap", 0.0) if d.get("logit_softcap") is not None else 0.0
        if cap < 0:
            raise ConfigError(f"config.json: logit_softcap must be positive, got {cap}")
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
                mask, window = m.get("mask"), None
                if mask is not None:
                    if not isinstance(mask, dict):
                        raise ConfigError(f"{where}: 'mask' must be an object")
                    window = take_int(mask, "size", minimum=1)
                mixer = MixedAttentionConfig(take_int(m, "heads", minimum=1), take_int(m, "kv_heads", minimum=1),
                                             take_int(m, "dim", minimum=1), take_int(m, "vdim", minimum=1),
                                             take_float(m, "scale"), window, _rotary(m, where, ()))
                if mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"{where}: {mixer.heads} heads are not a multiple of {mixer.kv_heads} kv heads")
                if mixer.rot is not None and (mixer.rot.dims > mixer.dim or mixer.rot.scaling is not None):
                    raise ConfigError(f"{where}: rot.dims {mixer.rot.dims} exceeds dim {mixer.dim}, or rot.scaling is given")
            elif kind == "latent_attention":
                rot = _rotary(m, where, ())
                src = m.get("kv_from")
                if src is not None:
                    src = take_int(m, "kv_from", minimum=0)
                mixer = SharedLatentConfig(take_int(m, "heads", minimum=1), take_int(m, "dim", minimum=1),
                                           take_int(m, "rot_dim", minimum=2), take_int(m, "vdim", minimum=1),
                                           take_int(m, "kv_rank", minimum=1), take_float(m, "scale"), rot, src)
                if rot is None or rot.dims != mixer.rot_dim or rot.scaling is not None:
                    raise ConfigError(f"{where}: 'rot' is required without scaling and rot.dims must equal rot_dim {mixer.rot_dim}")
                if src is not None:
                    o = layers[src] if src < i else None
                    if (o is None or o.type != "latent_attention" or o.mixer.kv_from is not None
                            or (o.mixer.kv_rank, o.mixer.rot_dim, o.mixer.rot) != (mixer.kv_rank, mixer.rot_dim, rot)):
                        raise ConfigError(f"{where}: kv_from {src} must name an earlier latent_attention layer with a latent "
                                          "of its own and the same kv_rank, rot_dim and rot")
            elif kind == "lightning":
                decay = m.get("decay")
                heads = take_int(m, "heads", minimum=1)
                if (not isinstance(decay, list) or len(decay) != heads
                        or not all(isinstance(v, (int, float)) and not isinstance(v, bool) and 0.0 < v <= 1.0 for v in decay)):
                    raise ConfigError(f"{where}: 'decay' must list one number in (0, 1] per head")
                mixer = LightningConfig(heads, take_int(m, "dim", minimum=1), take_int(m, "vdim", minimum=1),
                                        tuple(float(v) for v in decay))
            else:
                raise ConfigError(f"{where}: unknown layer type {kind!r} (attention, latent_attention, lightning)")
            ml, ff = L.get("mlp"), None
            if ml is not None:
                if not isinstance(ml, dict) or ml.get("kind") != "dense":
                    raise ConfigError(f"{where}: 'mlp' must be null or an object of kind 'dense'")
                ff = take_int(ml, "ff", minimum=1)
            layers.append(SenulixLayerConfig(kind, mixer, ff))
        return cls(architecture="Senulix", vocab=vocab, width=width, norm_eps=eps, side_dim=side_dim,
                   logit_softcap=cap, layers=tuple(layers))

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "layers": [L.to_dict() for L in self.layers]}
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        return d
