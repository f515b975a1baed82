"""The Ronurax architecture as a ``ModelSpec``: a decoder of pre-norm layers with layer norms
(gain and bias) whose mixer is either a differential attention (two softmax maps per head over the
same values, grouped key/value heads, biased projections, an RMS norm per query and key head, a partial
rotation with frequencies stretched by wavelength, a mask that cuts the positions into segments) or an
attention through a cached latent with one rotated key part shared by the heads (ramp-scaled
frequencies, causal, a sigmoid gate on the heads' outputs); the feed-forward is routed experts
(softmax scores over all experts, the choice limited to the best groups of neighbouring experts, the
scores as weights on the outputs) or absent.  A layer may run another layer's weights with a cache of
its own.

This file holds no sizes and no kernels: it translates ``RonuraxConfig`` into part descriptions.
What the design fixes is written here as parameters of general parts.  Tensor names: ``embed``,
``head``, ``final.norm`` (+ ``.b``), and ``l<i>.{norm1,norm2}`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.*``
for layer i.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.ronurax import RonuraxConfig
from ..parts.spec import BlockSpec, LayerCall, ModelSpec, PartSpec

MAX_POSITION = 1 << 24          # angles are formed on the device from the position: the cache's size is the only bound


def _scaling(rot, kind):
    sc = rot.scaling_dict()
    return dict(sc, kind=kind) if sc else None


def build_ronurax_spec(cfg: RonuraxConfig) -> ModelSpec:
    d = cfg.width

    def norm(name):
        return PartSpec("layernorm", "", {"width": d, "eps": cfg.norm_eps, "tensor": name, "bias_tensor": name + ".b"})

    blocks, block_of, schedule = [], {}, []
    for i, L in enumerate(cfg.layers):
        if L.weights_of is not None:
            schedule.append(LayerCall(block=block_of[L.weights_of], cache=i))
            continue
        p, m = f"l{i}", L.mixer
        if L.type == "attention":
            mixer = PartSpec("paged_attention", p + ".mix", {
                "hidden": d, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                "window": None, "segment": m.segment, "scale": m.scale, "position": None, "bias": True,
                "tensors": {k: f"{p}.mix.{k}" for k in "qkvo"},
                "differential": {"diff": m.diff, "eps": cfg.norm_eps,
                                 "tensors": {k: f"{p}.mix.{k}" for k in ("lq1", "lk1", "lq2", "lk2")}},
                "qk_transform": PartSpec("head_rmsnorm_rotary", "", {
                    "head_dim": m.dim, "eps": cfg.norm_eps, "q_gain": p + ".mix.q.norm", "k_gain": p + ".mix.k.norm",
                    "rotary_dim": m.rot.dims if m.rot else 0, "theta": m.rot.base if m.rot else 0.0,
                    "scaling": _scaling(m.rot, "wavelength") if m.rot else None})})
        else:
            mixer = PartSpec("latent_attention", p + ".mix", {
                "hidden": d, "n_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_head_dim": m.vdim,
                "kv_rank": m.kv_rank, "scale": m.scale, "eps": cfg.norm_eps, "window": None, "gate": True,
                "rotary": {"theta": m.rot.base, "scaling": _scaling(m.rot, "ramp")},
                "tensors": {"dkv_norm": p + ".mix.dkv.norm"}})
        ff = None
        if L.mlp is not None:
            ff = PartSpec("routed_experts", p + ".mlp", {
                "hidden": d, "experts": L.mlp.experts, "top": L.mlp.top, "expert_ff": L.mlp.ff,
                "score": "softmax", "renormalize": False, "weight_on": "output",
                "groups": {"count": L.mlp.groups, "keep": L.mlp.keep} if L.mlp.groups else None})
        block_of[i] = len(blocks)
        blocks.append(BlockSpec(kind="pre_norm", prefix=p, mixer=mixer, feed_forward=ff, mixer_norm=norm(p + ".norm1"),
                                ff_norm=norm(p + ".norm2") if ff else None))
        schedule.append(LayerCall(block=block_of[i], cache=i))
    return ModelSpec(
        hidden_size=d, vocab_size=cfg.vocab, max_position=MAX_POSITION,
        embedding=PartSpec("token_embedding", "", {"vocab": cfg.vocab, "width": d, "tensor": "embed"}),
        blocks=blocks, schedule=schedule, final_norm=norm("final.norm"),
        head=PartSpec("linear_head", "", {"vocab": cfg.vocab, "width": d, "tied_to": None, "tensor": "head"}),
        eos_token_ids=())


register_architecture("Ronurax", RonuraxConfig, build_ronurax_spec)
