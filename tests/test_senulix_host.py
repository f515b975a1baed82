"""Host-side tests of the Senulix design: configuration, the model's description (tensors, schedule,
cache needs) against the plain implementation's own list, the cache manager with its window groups and
state slots, random weights, and the plain recurrence cut in pieces."""
import numpy as np
import pytest

from plain import senulix_plain as P
from test_gpu_senulix import CFG_A, CFG_B, CFGS


def test_config_round_trip_and_refusals():
    import kllm_b200.models  # noqa: F401  (registers the architectures)
    from kllm_b200.config import ConfigError, parse_config
    for cfg, _ in CFGS.values():
        c = parse_config(cfg)
        assert parse_config(c.to_dict()) == c
        assert c.to_dict() == cfg
    lat, att, lig = CFG_B["layers"][0], CFG_B["layers"][1], CFG_B["layers"][2]

    def one(layer, **kw):
        return dict(CFG_B, layers=[dict(layer, mixer=dict(layer["mixer"], **kw))])
    for bad in (one(att, heads=4), one(att, kv_heads=0), one(att, mask={"size": 0}), one(att, rot={"base": 100.0, "dims": 3}),
                one(att, rot={"base": 100.0, "dims": 12}), one(lat, rot_dim=4), one(lat, kv_rank=0), one(lat, rot=None),
                one(lat, kv_from=0),                                                   # itself
                dict(CFG_B, layers=[att, dict(lat, mixer=dict(lat["mixer"], kv_from=0))]),          # another kind of layer
                dict(CFG_B, layers=[lat, dict(lat, mixer=dict(lat["mixer"], kv_from=0, kv_rank=12))]),   # another latent size
                dict(CFG_B, layers=[lat, dict(lat, mixer=dict(lat["mixer"], kv_from=0)),
                                    dict(lat, mixer=dict(lat["mixer"], kv_from=1))]),               # a layer without a latent
                one(lig, decay=[1.2]), one(lig, decay=[0.5, 0.5]), one(lig, decay=[0.0]),
                dict(CFG_B, layers=[dict(att, type="wkv")]),
                dict(CFG_B, layers=[dict(att, mlp={"kind": "moe", "ff": 8})]),
                dict(CFG_B, token_side={"dim": 0}), dict(CFG_B, logit_softcap=-1.0),
                dict(CFG_B, norm={"eps": 0.0}), dict(CFG_B, layers=[]),
                {k: v for k, v in CFG_B.items() if k != "vocab"}):
        with pytest.raises(ConfigError):
            parse_config(bad)


@pytest.mark.parametrize("name", sorted(CFGS))
def test_model_description(name):
    import torch
    import kllm_b200.models  # noqa: F401
    from kllm_b200.config import build_model_spec, parse_config
    from kllm_b200.parts.model import DecoderModel
    from kllm_b200.parts.spec import PagedKVNeed, StateNeed
    cfg, _ = CFGS[name]
    model = DecoderModel(build_model_spec(parse_config(cfg)), torch.float32, "cpu")
    shapes = P.tensor_shapes(cfg)
    specs = {s.name: s for s in model.tensor_specs()}
    assert set(specs) == set(shapes)
    for n, shape in shapes.items():
        assert specs[n].fits(shape), (n, specs[n].shape, shape)
        assert specs[n].store == ("compute" if len(shape) == 2 and not n.endswith(".talk") else "float32"), n
    # a layer that reads another layer's rows has no cache slot of its own and does not write
    owners = [L["mixer"].get("kv_from", i) for i, L in enumerate(cfg["layers"])]
    slots = {o: k for k, o in enumerate(sorted(set(owners)))}
    assert [(c.block, c.cache, c.writes_cache) for c in model.schedule] == \
        [(i, slots[o], o == i) for i, o in enumerate(owners)]
    needs = model.cache_needs()
    assert len(needs) == len(slots)
    for i, L in enumerate(cfg["layers"]):
        m = L["mixer"]
        if owners[i] != i:
            continue
        need = needs[slots[i]]
        if L["type"] == "lightning":
            assert need == StateNeed((m["heads"] * m["dim"] * m["vdim"],), "float32")
        elif L["type"] == "attention":
            assert need == PagedKVNeed(m["kv_heads"], m["dim"], m["mask"]["size"] if "mask" in m else None,
                                       None if m["vdim"] == m["dim"] else m["vdim"])
        else:
            assert need == PagedKVNeed(1, m["kv_rank"] + m["rot_dim"], None, m["kv_rank"], values_are_keys=True)


def test_cache_manager_windows_and_state_slots():
    """Window groups give pages back behind the window, state slots are zeroed at reuse; the pool of a trace
    sized by the live tokens suffices."""
    import torch
    import kllm_b200.models  # noqa: F401
    from kllm_b200.cache.manager import CacheManager
    from kllm_b200.config import build_model_spec, parse_config
    from kllm_b200.parts.model import DecoderModel
    model = DecoderModel(build_model_spec(parse_config(CFG_A)), torch.float32, "cpu")
    cm = CacheManager(model.cache_needs(), 16, 12, max_requests=2, dtype=torch.float32, device="cpu")
    a = cm.open()
    for n in (100, 1, 1, 50, 1):
        cm.reserve(a, n)
        cm.commit(a, n)
        cm.audit()
    windows = {g.window for g in cm.groups}
    assert windows == {None, 40, 7, 300}
    for gi, g in enumerate(cm.groups):
        held = sum(1 for p in a.tables[gi] if p >= 0)
        if g.window is not None and g.window < 153:
            assert held <= (g.window - 1) // 16 + 2
        else:
            assert held == -(-153 // 16)
    slot = a.state_slot
    cm.close(a)
    b = cm.open()
    assert b.state_slot == slot and b.length == 0
    cm.close(b)
    cm.audit()


def test_random_weights_mode(tmp_path):
    import torch
    from kllm_b200.weights import write_random_model
    from kllm_b200.weights.safetensors_io import ModelFiles
    d = write_random_model(str(tmp_path / "m"), CFG_A, seed=3, dtype=torch.bfloat16)
    shapes = P.tensor_shapes(CFG_A)
    with ModelFiles(d) as f:
        assert set(f.names()) == set(shapes)
        for n in f.names():
            assert tuple(f.entry(n).shape) == tuple(shapes[n])
        # weights stored around zero (one-plus norms) start at zero, plain gains at one, the mixing at the identity
        assert float(f.read("l0.norm1").abs().max()) == 0.0
        assert float((f.read("l1.mix.q.norm") - 1).abs().max()) == 0.0
        assert torch.equal(f.read("l1.mix.talk").float(), torch.eye(4))


def test_plain_recurrence_in_pieces():
    """The plain scan carried over a cut equals the scan over the whole (its state argument is what the tests of
    the kernel compare the slots with)."""
    rng = np.random.default_rng(0)
    q, k, v = rng.standard_normal((20, 2, 5)), rng.standard_normal((20, 2, 5)), rng.standard_normal((20, 2, 3))
    whole, S = P.decayed_state_scan(q, k, v, [0.7, 1.0])
    a, Sa = P.decayed_state_scan(q[:7], k[:7], v[:7], [0.7, 1.0])
    b, Sb = P.decayed_state_scan(q[7:], k[7:], v[7:], [0.7, 1.0], Sa)
    assert np.allclose(np.concatenate([a, b]), whole) and np.allclose(Sb, S)
