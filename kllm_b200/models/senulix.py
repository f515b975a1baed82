"""The Senulix architecture as a ``ModelSpec``: a decoder whose sublayers read the residual stream itself and
are normed on their OUTPUT (RMS norms whose weights are stored around zero and act as 1 + w), with three kinds
of mixer: grouped attention in a sliding window with RMS norms over the whole query and key projections, a
partial rotation, scores mixed across the heads before the softmax and a sink of score 0; attention through a
cached latent with one rotated key part shared by the heads, where a layer may read the rows another layer
cached; and linear attention with one fixed decay per head.  The feed-forward is a plain MLP with the
error-function gelu, or absent.  Every layer ends with an input from the token's own row of a second embedding
table, gated by a projection of the stream.  The logits are soft-capped.

This file holds no sizes and no kernels: it translates ``SenulixConfig`` into part descriptions.  What the
design fixes is written here as parameters of general parts.  Tensor names: ``embed``, ``side.embed``, ``head``,
``final.norm``, and ``l<i>.{norm1,norm2}``, ``l<i>.mix.*``, ``l<i>.mlp.{up,down}``, ``l<i>.side.{gate,proj,norm}`` for
layer i.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.senulix import SenulixConfig
from ..parts.spec import BlockSpec, LayerCall, ModelSpec, PartSpec

MAX_POSITION = 1 << 24          # angles are formed on the device from the position: the cache's size is the only bound


def build_senulix_spec(cfg: SenulixConfig) -> ModelSpec:
    d, n_layers = cfg.width, len(cfg.layers)

    def norm(name, offset=1.0):
        return PartSpec("rmsnorm", "", {"width": d, "eps": cfg.norm_eps, "tensor": name, "offset": offset})

    owners = [i for i, L in enumerate(cfg.layers) if getattr(L.mixer, "kv_from", None) is None]
    slot_of = {owner: n for n, owner in enumerate(owners)}
    blocks, schedule = [], []
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}", L.mixer
        owner = i
        if L.type == "attention":
            mixer = PartSpec("paged_attention", p + ".mix", {
                "hidden": d, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                "window": m.window, "scale": m.scale, "position": None, "score_mix": p + ".mix.talk", "sink": "zero",
                "tensors": {k: f"{p}.mix.{k}" for k in "qkvo"},
                "qk_transform": PartSpec("whole_rmsnorm", "", {
                    "q_dim": m.heads * m.dim, "k_dim": m.kv_heads * m.dim, "eps": cfg.norm_eps,
                    "q_gain": p + ".mix.q.norm", "k_gain": p + ".mix.k.norm",
                    "rotary_dim": m.rot.dims if m.rot else 0, "theta": m.rot.base if m.rot else 0.0})})
        elif L.type == "latent_attention":
            own = m.kv_from is None
            owner = i if own else m.kv_from
            mixer = PartSpec("latent_attention", p + ".mix", {
                "hidden": d, "n_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_head_dim": m.vdim,
                "kv_rank": m.kv_rank, "scale": m.scale, "eps": cfg.norm_eps, "window": None, "gate": False,
                "own_latent": own, "rotary": {"theta": m.rot.base, "scaling": None},
                "tensors": {"dkv_norm": p + ".mix.dkv.norm"}})
        else:
            mixer = PartSpec("lightning_attention", p + ".mix", {
                "hidden": d, "heads": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim, "decay": list(m.decay),
                "eps": cfg.norm_eps})
        ff = None
        if L.ff is not None:
            ff = PartSpec("plain_mlp", p + ".mlp", {"hidden": d, "intermediate": L.ff, "activation": "gelu"})
        params = {}
        if cfg.side_dim:
            params = {"side": PartSpec("token_side", p + ".side", {
                          "hidden": d, "dim": cfg.side_dim, "offset": i * cfg.side_dim, "columns": n_layers * cfg.side_dim,
                          "vocab": cfg.vocab, "table": "side.embed", "gate": p + ".side.gate", "proj": p + ".side.proj"}),
                      "side_norm": norm(p + ".side.norm", offset=0.0)}
        blocks.append(BlockSpec(kind="output_norm", prefix=p, mixer=mixer, feed_forward=ff, mixer_norm=norm(p + ".norm1"),
                                ff_norm=norm(p + ".norm2") if ff else None, params=params))
        schedule.append(LayerCall(block=i, cache=slot_of[owner], writes_cache=owner == i))
    return ModelSpec(
        hidden_size=d, vocab_size=cfg.vocab, max_position=MAX_POSITION,
        embedding=PartSpec("token_embedding", "", {"vocab": cfg.vocab, "width": d, "tensor": "embed"}),
        blocks=blocks, schedule=schedule, final_norm=norm("final.norm"),
        head=PartSpec("linear_head", "", {"vocab": cfg.vocab, "width": d, "tied_to": None, "tensor": "head",
                                          "softcap": cfg.logit_softcap}),
        eos_token_ids=())


register_architecture("Senulix", SenulixConfig, build_senulix_spec)
