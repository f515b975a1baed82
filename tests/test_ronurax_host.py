"""Host-side tests of the Ronurax design: configuration, the model's description (tensors, schedule,
cache needs) against the plain implementation's own list, the rotation's frequencies under both
scalings, the cache manager's store for key heads that share value heads, and random weights."""
import numpy as np
import pytest

from plain import ronurax_plain as P
from test_gpu_ronurax import CFG_A, CFG_B, CFGS


def test_config_round_trip_and_refusals():
    import kllm_b200.models  # noqa: F401  (registers the architectures)
    from kllm_b200.config import ConfigError, parse_config
    for cfg, _ in CFGS.values():
        c = parse_config(cfg)
        assert parse_config(c.to_dict()) == c
        assert c.to_dict() == cfg
    att, lat = CFG_B["layers"][1], CFG_B["layers"][0]

    def one(layer, **kw):
        return dict(CFG_B, layers=[dict(layer, mixer=dict(layer["mixer"], **kw))])
    moe = att["mlp"]
    for bad in (one(att, heads=4), one(att, kv_heads=0), one(att, mask={"size": 0}), one(att, rot={"base": 100.0, "dims": 3}),
                one(att, rot={"base": 100.0, "dims": 12}), one(att, rot={"base": 100.0, "dims": 4, "scaling": {"factor": 2.0}}),
                one(lat, rot_dim=4), one(lat, kv_rank=0), one(lat, rot=None),
                dict(CFG_B, layers=[dict(att, type="wkv")]),
                dict(CFG_B, layers=[dict(att, mlp={"kind": "dense", "ff": 8})]),
                dict(CFG_B, layers=[dict(att, mlp=dict(moe, router={"experts": 6, "top": 7}))]),
                dict(CFG_B, layers=[dict(att, mlp=dict(moe, router={"experts": 6, "top": 2, "groups": {"count": 4, "keep": 1}}))]),
                dict(CFG_B, layers=[dict(att, mlp=dict(moe, router={"experts": 6, "top": 3, "groups": {"count": 3, "keep": 1}}))]),
                dict(CFG_B, layers=[att, dict(lat, weights_of=0)]),          # another kind of layer
                dict(CFG_B, layers=[dict(att, weights_of=0)]),               # itself
                dict(CFG_B, layers=[att, dict(att, weights_of=0), dict(att, weights_of=1)]),   # a layer without tensors
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
    from kllm_b200.parts.spec import PagedKVNeed
    cfg, _ = CFGS[name]
    model = DecoderModel(build_model_spec(parse_config(cfg)), torch.float32, "cpu")
    shapes = P.tensor_shapes(cfg)
    specs = {s.name: s for s in model.tensor_specs()}
    assert set(specs) == set(shapes)
    for n, (shape, kind) in shapes.items():
        assert specs[n].fits(shape), (n, specs[n].shape, shape)
        assert specs[n].store == ("compute" if kind in ("matrix", "qk") else "float32"), n
    # a layer that runs another layer's weights runs that layer's block with a cache slot of its own
    owners = [L.get("weights_of", i) for i, L in enumerate(cfg["layers"])]
    blocks = {o: k for k, o in enumerate(sorted(set(owners)))}
    assert [(c.block, c.cache, c.writes_cache) for c in model.schedule] == [(blocks[o], i, True) for i, o in enumerate(owners)]
    needs = model.cache_needs()
    assert len(needs) == len(cfg["layers"])
    for L, need in zip(cfg["layers"], needs):
        m = L["mixer"]
        if L["type"] == "attention":
            assert need == PagedKVNeed(2 * m["kv_heads"], m["dim"], None, None if m["vdim"] == m["dim"] else m["vdim"],
                                       n_v_heads=m["kv_heads"])
        else:
            assert need == PagedKVNeed(1, m["kv_rank"] + m["rot_dim"], None, m["kv_rank"], values_are_keys=True)


def test_frequencies_under_both_scalings():
    from kllm_b200.parts.rotary import rotary_frequencies
    for dims, base in ((8, 100.0), (16, 10000.0), (2, 10.0), (64, 500.0)):
        plain = P.base_frequencies(dims, base)
        f, amp = rotary_frequencies(dims, base, None)
        assert np.allclose(f.numpy(), plain, rtol=1e-14) and amp == 1.0
        for sc in (dict(factor=8.0, low=1.0, high=4.0, original=64), dict(factor=3.0, low=2.0, high=8.0, original=128),
                   dict(factor=2.0, low=0.5, high=1.5, original=4096)):
            f, amp = rotary_frequencies(dims, base, dict(sc, kind="wavelength"))
            assert np.allclose(f.numpy(), P.stretched_by_wavelength(plain, sc), rtol=1e-13) and amp == 1.0
        for sc in (dict(factor=4.0, original=32, fast=4.0, slow=1.0), dict(factor=1.5, original=8, fast=2.0, slow=0.5),
                   dict(factor=40.0, original=4096, fast=32.0, slow=1.0), dict(factor=2.0, original=16, fast=1.0, slow=1.0)):
            f, amp = rotary_frequencies(dims, base, dict(sc, kind="ramp"))
            want, wamp = P.stretched_by_ramp(plain, dims, base, sc)
            assert np.allclose(f.numpy(), want, rtol=1e-13) and abs(amp - wamp) < 1e-15
    # the bands of the first scaling are all met by the first case, and the ramp takes 0, a fraction and 1
    f = P.stretched_by_wavelength(P.base_frequencies(8, 100.0), dict(factor=8.0, low=1.0, high=4.0, original=64))
    ratio = f / P.base_frequencies(8, 100.0)
    assert ratio[0] == 1.0 and ratio[-1] == 1 / 8.0 and any(1 / 8.0 < r < 1.0 for r in ratio)


def test_cache_manager_keeps_fewer_value_heads_than_key_heads():
    import torch
    from kllm_b200.cache.manager import CacheManager
    from kllm_b200.parts.spec import PagedKVNeed
    needs = [PagedKVNeed(4, 8, None, 12, n_v_heads=2), PagedKVNeed(1, 24 + 4, None, 24, values_are_keys=True),
             PagedKVNeed(4, 8, None, 12, n_v_heads=2)]
    cm = CacheManager(needs, page_size=4, num_pages=6, max_requests=2, dtype=torch.float32, device="cpu")
    assert len(cm.groups) == 2 and cm.groups[0].slots == [0, 2]
    assert cm.bytes_per_page() == (2 * 4 * (4 * 8 + 2 * 12) + 4 * 28) * 4
    caches = cm.layer_caches({0: None, 1: None})
    assert tuple(caches[0].k.shape) == (6, 4, 4, 8) and tuple(caches[0].v.shape) == (6, 2, 4, 12)
    assert caches[2].k.data_ptr() != caches[0].k.data_ptr()
    assert caches[1].k.data_ptr() == caches[1].v.data_ptr() and tuple(caches[1].k.shape) == (6, 1, 4, 28)
    with pytest.raises(ValueError):
        CacheManager([PagedKVNeed(3, 8, None, 12, n_v_heads=2)], page_size=4, num_pages=6, max_requests=2,
                     dtype=torch.float32, device="cpu")
    r = cm.open()
    cm.reserve(r, 24)
    cm.commit(r, 24)
    assert sum(p >= 0 for p in r.tables[1]) == 6 and sum(p >= 0 for p in r.tables[0]) == 6
    cm.close(r)
    cm.audit()


def test_random_weights_of_the_design(tmp_path):
    """Random-weights mode fills every tensor of the design and the loader binds what it wrote."""
    import torch
    from kllm_b200.config import build_model_spec, parse_config
    from kllm_b200.parts.model import DecoderModel
    from kllm_b200.weights import load_weights
    from kllm_b200.weights.random_init import write_random_model
    d = write_random_model(str(tmp_path / "m"), CFG_A, seed=3, dtype=torch.bfloat16)
    model = DecoderModel(build_model_spec(parse_config(CFG_A)), torch.bfloat16, "cpu")
    t = load_weights(d, model.tensor_specs(), torch.bfloat16, "cpu")
    assert set(t) == set(P.tensor_shapes(CFG_A))
    assert t["l0.norm1.b"].dtype == torch.float32 and t["l0.mix.q"].dtype == torch.bfloat16
    model.bind(t)
