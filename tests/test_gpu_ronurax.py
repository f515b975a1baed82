"""The Ronurax design in the engine against its plain implementation (tests/plain/ronurax_plain.py).

Small configurations of their own, random weights whose values are bfloat16 numbers (so both
dtypes load the same model): each mechanism's kernel alone, whole prompts, prompts against
token-by-token decoding, portions down to two tokens, unequal batches, slots and pages that
are used again, keys far away, at page borders and just inside and outside a mask segment that one
score makes stand out, the first tokens, long decoding through CUDA graphs, and greedy generation
through the scheduler.
"""
import numpy as np
import pytest

from helpers import write_model_dir
from plain import ronurax_plain as P
from test_gpu_sozarax import _ctx, _t, check_rows, engine_for, run_cut

pytestmark = pytest.mark.gpu


def _rot(base, dims, **scaling):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = scaling
    return r


def _attn(heads, kv_heads, dim, vdim, scale, diff, segment, rot):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff,
            "mask": {"size": segment}, "rot": rot}


def _latent(heads, dim, rot_dim, vdim, kv_rank, scale, rot):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot}


def _moe(ff, experts, top, groups=None):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def _layer(kind, mixer, mlp, weights_of=None):
    L = {"type": kind, "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        L["weights_of"] = weights_of
    return L


# The wavelength bands of the attention's frequencies are chosen so that the pairs fall into all three
# (kept, blended, divided); the ramp of the latent layers' so that it takes 0, a fraction and 1.
_WAVE = dict(factor=8.0, low=1.0, high=4.0, original=64)
_RAMP = dict(factor=4.0, original=32, fast=4.0, slow=1.0)

# A: sizes that suit vector widths; layers that run another layer's weights (both kinds), a layer
# without a feed-forward, several groups of which more than one is kept, values wider and narrower
# than keys, segments shorter and longer than a page, than a chunk of decoded keys and than the prompt.
_A0 = _layer("attention", _attn(4, 2, 16, 24, 0.3, 0.6, 40, _rot(100.0, 8, **_WAVE)), _moe(24, 6, 3, (3, 2)))
_A1 = _layer("latent_attention", _latent(3, 16, 8, 12, 32, 0.3, _rot(100.0, 8, **_RAMP)), _moe(16, 4, 2, (2, 1)))
CFG_A = {
    "architecture": "Ronurax", "vocab": 96, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        _A0, _A1, dict(_A0, weights_of=0),
        _layer("latent_attention", _latent(2, 8, 4, 16, 24, 0.4, _rot(50.0, 4, factor=2.0, original=16, fast=8.0, slow=2.0)), None),
        _layer("attention", _attn(6, 1, 8, 8, 0.5, 0.3, 300, _rot(10000.0, 8)), _moe(40, 5, 1)),
        dict(_A1, weights_of=1),
        _layer("attention", _attn(2, 2, 32, 16, 0.2, 0.8, 16, _rot(1000.0, 16, factor=3.0, low=2.0, high=8.0, original=128)),
               _moe(24, 8, 4, (4, 2))),
    ],
}
# B: sizes that fit no vector width or tile; a segment of one position (a token sees itself alone)
# and of two; one group that is kept (no limit on the choice); every expert chosen.
CFG_B = {
    "architecture": "Ronurax", "vocab": 61, "width": 50, "norm": {"eps": 1e-6},
    "layers": [
        _layer("latent_attention", _latent(5, 6, 2, 5, 10, 0.5, _rot(10.0, 2, **_RAMP)), _moe(7, 3, 3, (1, 1))),
        _layer("attention", _attn(3, 3, 10, 6, 0.4, 0.5, 7, _rot(100.0, 4, **_WAVE)), _moe(9, 6, 2, (2, 2))),
        _layer("attention", _attn(2, 1, 6, 9, 0.6, 0.2, 1, _rot(20.0, 6)), None),
        _layer("attention", _attn(1, 1, 12, 7, 0.3, 0.7, 2, _rot(30.0, 2)), _moe(11, 2, 1, (2, 1))),
        _layer("latent_attention", _latent(1, 12, 6, 7, 22, 0.3, _rot(100.0, 6, factor=1.5, original=8, fast=2.0, slow=0.5)),
               _moe(5, 4, 2)),
    ],
}
# C: head sizes of the tensor-core kernels (keys of 64 and 128, latent rows of 128 + 64 and 64 + 32), many
# heads on one key head, the whole head rotated, a latent layer first and repeated three times.
_C0 = _layer("latent_attention", _latent(4, 32, 64, 32, 128, 0.1, _rot(10000.0, 64, factor=2.0, original=64, fast=32.0, slow=1.0)),
             _moe(32, 8, 2, (4, 1)))
CFG_C = {
    "architecture": "Ronurax", "vocab": 80, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        _C0, dict(_C0, weights_of=0),
        _layer("attention", _attn(8, 2, 64, 64, 0.125, 0.35, 64, _rot(10000.0, 64, **_WAVE)), _moe(48, 4, 2, (2, 1))),
        dict(_C0, weights_of=0),
        _layer("attention", _attn(2, 1, 128, 64, 0.09, 0.5, 200, _rot(500.0, 32)), None),
        _layer("latent_attention", _latent(6, 16, 32, 48, 64, 0.15, _rot(100.0, 32)), _moe(16, 6, 2, (3, 1))),
    ],
}
CFGS = {"A": (CFG_A, 41), "B": (CFG_B, 42), "C": (CFG_C, 43)}


def make_model(tmp_path, name, qk_boost=3.0):
    """``qk_boost`` scales the query and key projections.  At 3 the attention of C is so sharp that bfloat16
    rounding of queries and keys alone moves its logits by a quarter of their range (two bfloat16 routes of
    the engine differ from each other by as much); the bfloat16 runs of C take 1."""
    cfg, seed = CFGS[name]
    w = P.random_weights(cfg, seed, qk_boost=qk_boost)
    d = write_model_dir(str(tmp_path / f"ronurax_{name}"), cfg, {k: np.asarray(v, dtype=np.float32) for k, v in w.items()})
    return cfg, w, d


# ---- whole models --------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompt_and_every_way_of_cutting(tmp_path, name, dtype):
    cfg, w, d = make_model(tmp_path, name, 1.0 if (name, dtype) == ("C", "bfloat16") else 3.0)
    rng = np.random.default_rng(5)
    ids = rng.integers(0, cfg["vocab"], size=150).tolist()
    taps = []
    want = P.forward(w, cfg, ids, taps)
    eng = engine_for(d, dtype)
    try:
        got_taps = []
        eng.model.tap = lambda i, x: got_taps.append(x.detach().float().cpu().numpy().copy())
        whole = run_cut(eng, ids, [len(ids)])
        eng.model.tap = None
        check_rows(whole, want, dtype, f"{name} whole")
        assert len(got_taps) == len(taps)
        for i, (g, t) in enumerate(zip(got_taps, taps)):      # the residual stream after every layer run
            assert np.abs(g - t).max() <= (1e-4 if dtype == "float32" else 1e-1) * np.abs(t).max(), (name, i)
        check_rows(run_cut(eng, ids[:3], [3]), want[:3], dtype, f"{name} first tokens")
        check_rows(run_cut(eng, ids[:1], [1]), want[:1], dtype, f"{name} one token")
        check_rows(run_cut(eng, ids, [len(ids) - 70, 1]), want, dtype, f"{name} prompt then decode")
        check_rows(run_cut(eng, ids[:70], [1]), want[:70], dtype, f"{name} decode from the start")
        for cuts in ([2], [3, 2, 37, 16, 5, 2, 64, 1], [17], [16, 16, 1, 31, 2]):
            got = run_cut(eng, ids, cuts)
            check_rows(got, want, dtype, f"{name} portions {cuts}")
            if dtype == "float32":
                # small steps take other product kernels (rows by FMAs) than large ones (SGEMM): sums in another order
                assert np.abs(got - whole).max() <= 3e-5 * np.abs(want).max(), cuts
        eng.cache.audit()
    finally:
        eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_and_reuse_of_slots_and_pages(tmp_path, dtype):
    """Up to four requests of unequal length in one batch, portions of some beside single tokens of
    others, then new requests in the slots and pages that the finished ones gave back; a pool that
    holds little more than what is live.  Every request alone is the yardstick."""
    from kllm_b200.engine.step import StepEntry
    cfg, w, d = make_model(tmp_path, "A")
    rng = np.random.default_rng(9)
    lens = [37, 90, 5, 64, 21, 50, 83]
    seqs = [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lens]
    want = [P.forward(w, cfg, s) for s in seqs]
    eng = engine_for(d, dtype, num_blocks=20, max_batch=4)      # 320 tokens of pages, four slots
    try:
        got = [np.zeros_like(x) for x in want]
        fed = [0] * len(seqs)
        caches, queue = {}, list(range(len(seqs)))
        sizes = [3, 1, 16, 2, 29, 1, 7]
        turn, slots_seen, pages_seen = 0, [], []
        while queue or caches:
            while queue and len(caches) < 4:
                i = queue.pop(0)
                caches[i] = eng.cache.open()
                slots_seen.append(caches[i].state_slot)
            entries, order = [], []
            for i in list(caches):
                if (turn + i) % 5 == 4 and len(caches) > 1:
                    continue                                     # a request that sits a step out
                left = len(seqs[i]) - fed[i]
                n = 1 if left <= 8 else min(left, sizes[(turn + i) % len(sizes)])
                entries.append(StepEntry(caches[i], seqs[i][fed[i]:fed[i] + n], list(range(n))))
                order.append((i, n))
            if entries:
                lg = eng.runner.run(entries).float().cpu().numpy()
                r = 0
                for i, n in order:
                    got[i][fed[i]:fed[i] + n] = lg[r:r + n]
                    r += n
                    fed[i] += n
                    pages_seen += [p for t in caches[i].tables for p in t if p >= 0]
                    if fed[i] == len(seqs[i]):
                        eng.cache.close(caches.pop(i))
            turn += 1
            eng.cache.audit()
        assert len(slots_seen) > len(set(slots_seen)), "no slot was used again"
        assert sum(lens) > 320, "the pool holds everything at once: no page had to be used again"
        for i in range(len(seqs)):
            check_rows(got[i], want[i], dtype, f"request {i} in mixed batches")
    finally:
        eng.close()


@pytest.mark.parametrize("name,dtype,length", [("B", "float32", 600), ("C", "bfloat16", 330), ("A", "float32", 420)])
def test_long_decoding(tmp_path, name, dtype, length):
    """A short prompt and then hundreds of single tokens: the decode route (graphs, the attention's key
    chunks and their merge, pages added one by one) over many segment, chunk and page borders."""
    cfg, w, d = make_model(tmp_path, name, 1.0 if dtype == "bfloat16" else 3.0)
    rng = np.random.default_rng(3)
    ids = rng.integers(0, cfg["vocab"], size=length).tolist()
    want = P.forward(w, cfg, ids)
    eng = engine_for(d, dtype, max_seq=640, num_blocks=40)
    try:
        check_rows(run_cut(eng, ids, [9, 1]), want, dtype, "long decoding")
    finally:
        eng.close()


def test_greedy_generation_through_the_scheduler(tmp_path):
    """``Engine.generate`` (scheduler, sampler, pipelined steps) on several prompts at once against
    greedy decoding with the plain implementation."""
    cfg, w, d = make_model(tmp_path, "A")
    rng = np.random.default_rng(21)
    prompts = [rng.integers(0, cfg["vocab"], size=n).tolist() for n in (7, 30, 2, 19, 45)]
    steps = 12
    eng = engine_for(d, "float32", max_step_tokens=48, max_batch=3)
    try:
        outs = eng.generate(prompts, max_new_tokens=steps)
        alone = eng.generate(prompts[1], max_new_tokens=steps)
    finally:
        eng.close()
    assert alone == outs[1]
    for p, out in zip(prompts, outs):
        ids = list(p)
        for k in range(steps):
            z = P.forward(w, cfg, ids)[-1]
            best = int(z.argmax())
            assert out[k] == best or z[best] - z[out[k]] < 1e-4 * np.abs(z).max(), (len(p), k)
            ids.append(out[k])


def test_replay_program(tmp_path):
    """bin/trace_run on a model of this design: whole, decode, portions and mixed batches of up to four
    live requests in a pool as small as the trace allows."""
    from test_gpu_replay import build_trace
    from trace_tools import run_trace
    cfg, w, d = make_model(tmp_path, "A")
    rng = np.random.default_rng(4)
    seqs = [rng.integers(0, cfg["vocab"], size=n).tolist() for n in (5, 33, 64, 100, 18)]
    want = [P.forward(w, cfg, s) for s in seqs]
    tb = build_trace(seqs, [7, 2, 13, 3, 1, 29], seed=8)
    for dtype in ("float32", "bfloat16"):
        rows = run_trace(d, dtype, tb, str(tmp_path / ("out_" + dtype)), cfg["vocab"])
        by_way = {}
        for (rid, pos), z in rows.items():
            by_way.setdefault((rid[0], int(rid[1:])), {})[pos] = z
        for (way, i), zs in by_way.items():
            pos = sorted(zs)
            check_rows(np.stack([zs[p] for p in pos]), want[i][pos], dtype, f"replay {way}{i}")


# ---- each mechanism's kernel alone ----------------------------------------------------------------

def _freq(f):
    import torch
    return torch.tensor(np.asarray(f, dtype=np.float64), dtype=torch.float64, device="cuda")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d", [50, 64, 1000])
def test_layer_norm_with_gain_and_bias(dtype, d):
    """The residual sum and the layer norm in one kernel, on all rows and on chosen rows."""
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(d)
    n = 11
    x = rng.standard_normal((n, d)) * 3 + 2.0          # a mean far from zero: the variance is about the mean
    res = P.round_bf16(rng.standard_normal((n, d)))
    gain, bias = rng.uniform(0.5, 1.5, d), rng.standard_normal(d)
    tdt = getattr(torch, dtype)
    tol = 2e-5 if dtype == "float32" else 2e-2
    xt, out = _t(x), torch.empty((n, d), dtype=tdt, device="cuda")
    kernels.add_layernorm(xt, _t(res, dtype), out, _t(gain), _t(bias), 1e-5)
    assert np.abs(xt.cpu().numpy() - (x + res)).max() <= 1e-6 * np.abs(x).max()
    want = P.layer_norm(x + res, gain, bias, 1e-5)
    assert np.abs(out.float().cpu().numpy() - want).max() <= tol * np.abs(want).max()
    rows = [7, 0, 3]
    out2 = torch.empty((len(rows), d), dtype=tdt, device="cuda")
    kernels.add_layernorm(xt, None, out2, _t(gain), _t(bias), 1e-5, rows=_t(rows, "int32"))
    assert np.abs(out2.float().cpu().numpy() - want[rows]).max() <= tol * np.abs(want).max()
    # an eps that matters: rows that are almost constant
    flat = np.full((2, d), 0.25) + rng.standard_normal((2, d)) * 1e-4
    out3 = torch.empty((2, d), dtype=torch.float32, device="cuda")
    kernels.add_layernorm(_t(flat), None, out3, _t(gain), _t(bias), 1e-3)
    assert np.abs(out3.cpu().numpy() - P.layer_norm(flat, gain, bias, 1e-3)).max() <= 1e-4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Hq,Hk,Hv,dk,dv,rot", [(8, 4, 2, 16, 24, 8), (3, 3, 3, 10, 6, 4), (4, 2, 1, 32, 32, 32),
                                                 (2, 2, 2, 12, 7, 0), (16, 4, 2, 64, 64, 16)])
def test_bias_head_norm_partial_rotation_and_cache_write(dtype, Hq, Hk, Hv, dk, dv, rot):
    """Biases, the RMS norm per head with a shared gain, the rotation of the first ``rot`` values of
    every head (positions up to a few thousand, scaled frequencies, an amplitude) and the write of
    keys and values into pages, for three requests of which one brings a single token."""
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(Hq * dk + rot)
    page = 4
    n_new, start = [5, 1, 2], [3, 4001, 0]
    ctx = _ctx(n_new, start)
    n = sum(n_new)
    width = (Hq + Hk) * dk + Hv * dv
    qkv, bias = rng.standard_normal((n, width + 3)) * 2, rng.standard_normal(width)
    gq, gk = rng.uniform(.5, 1.5, dk), rng.uniform(.5, 1.5, dk)
    freq = P.stretched_by_wavelength(P.base_frequencies(rot, 100.0), _WAVE) if rot else None
    amp = 1.25
    table = np.full((3, 1002), -1)
    table[0, :2], table[1, 1000], table[2, 0] = [5, 1], 2, 3
    tdt = getattr(torch, dtype)
    kc = torch.full((8, Hk, page, dk), float("nan"), dtype=tdt, device="cuda")
    vc = torch.full((8, Hv, page, dv), float("nan"), dtype=tdt, device="cuda")
    q = torch.empty((n, Hq * dk), dtype=tdt, device="cuda")
    kernels.headnorm_rope_append(q, _t(qkv), _t(bias), _t(gq), _t(gk), 1e-5, _freq(freq) if rot else None, amp, rot,
                                 ctx.positions, ctx.token_req, _t(table, "int32"), kc, vc, Hq, Hk, Hv, dk, dv)
    pos = ctx.positions.cpu().numpy()
    z = qkv[:, :width] + bias
    want_q = P.rms_norm(z[:, :Hq * dk].reshape(n, Hq, dk), gq, 1e-5)
    want_k = P.rms_norm(z[:, Hq * dk:(Hq + Hk) * dk].reshape(n, Hk, dk), gk, 1e-5)
    if rot:
        want_q, want_k = P.rotate(want_q, pos, freq, rot, amp), P.rotate(want_k, pos, freq, rot, amp)
    want_v = z[:, (Hq + Hk) * dk:].reshape(n, Hv, dv)
    tol = 2e-5 if dtype == "float32" else 2e-2
    assert np.abs(q.float().cpu().numpy() - want_q.reshape(n, -1)).max() <= tol * np.abs(want_q).max()
    req = ctx.token_req.cpu().numpy()
    for t in range(n):
        pg, sl = table[req[t], pos[t] // page], pos[t] % page
        assert np.abs(kc[pg, :, sl].float().cpu().numpy() - want_k[t]).max() <= tol * np.abs(want_k).max()
        assert np.abs(vc[pg, :, sl].float().cpu().numpy() - want_v[t]).max() <= tol * np.abs(want_v).max()
    assert int(torch.isfinite(kc.float()).sum()) == n * Hk * dk and int(torch.isfinite(vc.float()).sum()) == n * Hv * dv
    # queries alone (a layer that reads another layer's pages) are the same queries
    q2 = torch.empty_like(q)
    kernels.headnorm_rope_append(q2, _t(qkv[:, :Hq * dk]), _t(bias), _t(gq), None, 1e-5, _freq(freq) if rot else None, amp,
                                 rot, ctx.positions, ctx.token_req, None, None, None, Hq, Hk, Hv, dk, dv)
    assert torch.equal(q, q2)


def _page_order(T, page, n_pages, seed):
    return np.random.default_rng(seed).permutation(n_pages)[:-(-T // page)]


def _into_pages(rows, page, n_pages, ids):
    """rows [T, heads, size] laid into pages [n_pages, heads, page, size] in the order ``ids``; NaN elsewhere."""
    T, heads, size = rows.shape
    store = np.full((n_pages, heads, page, size), np.nan)
    for t in range(T):
        store[ids[t // page], :, t % page] = rows[t]
    return store


def _two_map_case(rng, T, H, G, dk, dv, far, boost=True):
    """Random queries, keys and values of T positions; the last query looks for key ``far`` on the
    first map of every head, with a score that beats every other key if that key is visible."""
    q = P.round_bf16(rng.standard_normal((T, H, 2, dk)))
    k = P.round_bf16(rng.standard_normal((T, G, 2, dk)))
    v = P.round_bf16(rng.standard_normal((T, G, dv)))
    if boost:
        kf = k[far, :, 0]
        kf = P.round_bf16(kf / np.linalg.norm(kf, axis=1, keepdims=True) * np.sqrt(dk))
        q[-1, :, 0] = P.round_bf16(np.repeat(kf, H // G, axis=0) * 6.0)
        k[far, :, 0] = kf * 4.0
    return q, k, v


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dk,dv", [(4, 2, 16, 24), (6, 1, 8, 4), (2, 2, 32, 64), (3, 1, 10, 6), (8, 2, 64, 64),
                                       (4, 1, 128, 128), (5, 5, 48, 16)])
def test_two_map_attention_at_segment_edges(dtype, H, G, dk, dv):
    """Two softmax maps per head over the same values, combined and normed, with a mask that cuts the
    positions into segments.  One key is made to stand out: the first key of the query's segment (seen),
    the last key of the segment before (not seen, however loud), a key far back in a long segment, at
    page and chunk borders; the query is the first or the last position of a segment or lies inside it,
    as a row of a portion that crosses segment borders and as a single decoded token.  Unused pages
    hold NaN.  2H query heads run over 2G key heads and G value heads."""
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(H * 100 + dk)
    page, scale, diff, eps = 16, 0.4, 0.35, 1e-5
    lam = P.map_lambda(rng.standard_normal(dk) * 0.2, rng.standard_normal(dk) * 0.2, rng.standard_normal(dk) * 0.2,
                       rng.standard_normal(dk) * 0.2, diff)
    gs = H // G
    # (segment, positions, the key that stands out)
    cases = [(100, 700, 600), (100, 700, 599), (64, 641, 639), (64, 641, 640), (64, 640, 576), (64, 640, 575),
             (300, 700, 600), (300, 700, 599), (1000, 700, 0), (1000, 700, 255), (1000, 700, 256), (1000, 530, 17),
             (1, 70, 68), (2, 70, 68), (2, 71, 69)]
    for C, T, far in cases:
        q, k, v = _two_map_case(rng, T, H, G, dk, dv, far)
        want = P.two_map_heads(q, k, v, P.segment_mask(T, C), scale, lam, diff, eps).reshape(T, H * dv)
        seen = far // C == (T - 1) // C
        if not seen:     # a loud key behind the edge changes nothing: the same result as without it
            k2 = k.copy()
            k2[far] = 0.0
            quiet = P.two_map_heads(q[-1:], k2, v, P.segment_mask(T, C)[-1:], scale, lam, diff, eps)
            assert np.abs(quiet.reshape(-1) - want[-1]).max() < 1e-9
        ids = _page_order(T, page, 64, far)
        kc, vc = _into_pages(k.reshape(T, G * 2, dk), page, 64, ids), _into_pages(v, page, 64, ids)
        table = np.full((1, 50), -1)
        table[0, :len(ids)] = ids
        qk = q.reshape(T, G, gs, 2, dk).transpose(0, 1, 3, 2, 4).reshape(T, -1)      # [kv head][map][head of the group]
        tol = 3e-5 if dtype == "float32" else 3e-2
        for n_new in (1, 70):
            ctx = _ctx([n_new], [T - n_new])
            both = torch.empty((n_new, 2 * H * dv), dtype=torch.float32, device="cuda")
            kernels.attention(both, _t(qk[T - n_new:], dtype), _t(kc, dtype), _t(vc, dtype), ctx, _t(table, "int32"),
                              2 * H, 2 * G, dk, 0, scale, v_head_dim=dv, exact_weights=True, segment=C)
            out = torch.empty((n_new, H * dv), dtype=getattr(torch, dtype), device="cuda")
            kernels.maps_combine(out, both, G, gs, dv, lam, eps, 1.0 - diff)
            got = out.float().cpu().numpy()
            assert np.isfinite(got).all(), (C, T, far, n_new)
            assert np.abs(got - want[T - n_new:]).max() <= tol * np.abs(want).max(), (C, T, far, n_new)


def _plain_rows(q, k, v, pos, first, scale):
    """softmax(scale q . k) v of one row over the keys first .. pos, in double precision."""
    sc = (k[first:pos + 1] @ q) * scale
    w = np.exp(sc - sc.max())
    return (w / w.sum()) @ v[first:pos + 1]


@pytest.mark.parametrize("dk,dv,Hk,Hv,gs,row", [(64, 128, 4, 2, 2, 128), (32, 64, 2, 2, 3, 64), (128, 64, 2, 1, 1, 64),
                                                (48, 16, 1, 1, 5, 48), (16, 32, 6, 3, 1, 40), (96, 96, 2, 1, 4, 96)])
@pytest.mark.parametrize("segment,window", [(0, 0), (50, 0), (0, 33), (128, 70), (7, 0)])
def test_mixed_step_with_values_of_another_size(dk, dv, Hk, Hv, gs, row, segment, window):
    """One launch of single tokens and portions of unequal requests in bfloat16, keys of one size, values of
    another in a store of fewer heads whose rows may be longer than the values, float32 results: every row
    against the plain softmax over the keys that its segment and its window leave.  Portions begin and end
    inside segments, windows and 64-key tiles; the pages are scattered and unused ones hold NaN."""
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(dk * 7 + dv + segment + window)
    page, n_pages, scale = 16, 96, 0.3
    # (tokens of this step, tokens before): two single tokens first, then portions
    reqs = [(1, 130), (1, 0), (70, 0), (3, 125), (129, 60), (1, 77), (2, 510), (64, 64)]
    H = Hk * gs
    free = list(rng.permutation(n_pages))
    kc = np.full((n_pages, Hk, page, dk), np.nan)
    vc = np.full((n_pages, Hv, page, row), np.nan)
    table = np.full((len(reqs), 48), -1)
    qs, want = [], []
    for r, (n, before) in enumerate(reqs):
        T = n + before
        q = P.round_bf16(rng.standard_normal((T, H, dk)))
        k = P.round_bf16(rng.standard_normal((T, Hk, dk)))
        v = P.round_bf16(rng.standard_normal((T, Hv, row)))
        ids = [free.pop() for _ in range(-(-T // page))]
        table[r, :len(ids)] = ids
        for t in range(T):
            kc[ids[t // page], :, t % page] = k[t]
            vc[ids[t // page], :, t % page] = v[t]
        for t in range(before, T):
            first = max(t - t % segment if segment else 0, t + 1 - window if window else 0)
            want.append([_plain_rows(q[t, h], k[:, h // gs], v[:, (h // gs) // (Hk // Hv), :dv], t, first, scale)
                         for h in range(H)])
        qs.append(q[before:].reshape(n, H * dk))
    want = np.asarray(want).reshape(-1, H * dv)
    ctx = _ctx([n for n, _ in reqs], [b for _, b in reqs])
    out = torch.full((ctx.n_tokens, H * dv), float("nan"), dtype=torch.float32, device="cuda")
    kernels.attention(out, _t(np.concatenate(qs), "bfloat16"), _t(kc, "bfloat16"), _t(vc, "bfloat16"), ctx,
                      _t(table, "int32"), H, Hk, dk, window, scale, v_head_dim=dv, exact_weights=True, segment=segment)
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    bad = np.abs(got - want).max(axis=1)
    assert bad.max() <= 1e-4 * np.abs(want).max(), (int(bad.argmax()), float(bad.max()))
    if dv % 16 == 0 and dk % 16 == 0:
        from kllm_b200.csrc.build import loaded_libraries
        name = f"attention_tc-KLLM_HD{dk}" + ("" if dv == dk else f"-KLLM_VD{dv}")
        assert name in loaded_libraries(), "the portions did not run on the tensor-core kernel"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,dk,dr,dv,R", [(3, 16, 8, 12, 32), (5, 6, 2, 5, 10), (4, 32, 64, 32, 128), (1, 12, 6, 7, 22),
                                          (16, 64, 32, 64, 96), (40, 8, 4, 8, 16)])
def test_latent_attention_with_a_rotated_key_part(dtype, H, dk, dr, dv, R):
    """From the stacked projection to the heads' outputs: the latent's norm, both rotations, the cache row
    [latent | rotated key part], the attention of H heads over that one row per key with the row's head
    as value.  The plain side forms every head's keys and values.  One key far back (at a page or chunk
    border, or the very first) carries the last query of every head through the rotated parts; the
    sequence is cut in two, the last rows as a portion and as a single token."""
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(H * 10 + dr)
    page, scale, eps, T = 16, 0.3, 1e-5, 600
    tdt = getattr(torch, dtype)
    w_uk = P.round_bf16(rng.standard_normal((H, dk, R)) / np.sqrt(R))
    w_uv = P.round_bf16(rng.standard_normal((H, dv, R)) / np.sqrt(R))
    gain = rng.uniform(0.5, 1.5, R)
    freq, amp = P.stretched_by_ramp(P.base_frequencies(dr, 50.0), dr, 50.0, _RAMP)
    for far in (0, 255, 256, 31, 32, 597):
        proj = rng.standard_normal((T, H * (dk + dr) + R + dr + 5))          # five more columns that nobody reads
        down = proj[:, H * (dk + dr):H * (dk + dr) + R + dr]                  # a view: [latent before its norm | key part]
        down[far, R:] *= 5.0
        c = P.rms_norm(down[:, :R], gain, eps)
        k_plain = np.einsum("tr,hkr->thk", c, w_uk)
        v = np.einsum("tr,hvr->thv", c, w_uv)
        # the last query's rotated part is, once both are rotated, a multiple of the key part at `far`: a
        # score of 30 on every head, which only the right angle at that distance gives
        qv = proj[:, :H * (dk + dr)].reshape(T, H, dk + dr).copy()
        kr = down[far, R:]
        turned = P.rotate(kr[None], np.array([far - (T - 1)]), freq, dr, 1.0)[0]
        qv[-1, :, dk:] = turned * (30.0 / scale / (amp * amp * (kr * kr).sum()))
        qv[-1, :, :dk] *= 0.2
        proj[:, :H * (dk + dr)] = qv.reshape(T, -1)
        pos = np.arange(T)
        q_rot = P.rotate(qv[:, :, dk:], pos, freq, dr, amp)
        k_rot = P.rotate(down[:, R:], pos, freq, dr, amp)
        want = P.latent_heads(qv[:, :, :dk], q_rot, k_plain, k_rot, v, P.causal_mask(T), scale)
        ids = _page_order(T, page, 64, far + 1)
        table = np.full((1, 50), -1)
        table[0, :len(ids)] = ids
        tol = 3e-5 if dtype == "float32" else 3e-2
        for n_new in (1, 45):
            store = torch.full((64, 1, page, R + dr), float("nan"), dtype=tdt, device="cuda")
            outs = []
            for a, b in ((0, T - n_new), (T - n_new, T)):
                ctx = _ctx([b - a], [a])
                q_plain = torch.empty((b - a, H * dk), dtype=tdt, device="cuda")
                q_full = torch.zeros((b - a, H * (R + dr)), dtype=tdt, device="cuda")
                kernels.latent_rope_append(q_plain, q_full, _t(proj[a:b]), _t(gain), eps, _freq(freq), amp, ctx.positions,
                                           ctx.token_req, _t(table, "int32"), store, H, dk, dr, R)
                if a == 0:
                    continue
                assert np.abs(q_plain.float().cpu().numpy().reshape(b - a, H, dk) - qv[a:b, :, :dk]).max() \
                    <= tol * np.abs(qv[a:b, :, :dk]).max()
                qf = q_full.view(b - a, H, R + dr)
                assert np.abs(qf[:, :, R:].float().cpu().numpy() - q_rot[a:b]).max() <= tol * np.abs(q_rot).max()
                # the plain query parts into the latent space: q_h^T W_uk,h, R values a head
                kernels.linear_per_head(q_plain, _t(w_uk, dtype), transposed=True, out=qf[:, :, :R])
                o_lat = torch.empty((b - a, H * R), dtype=tdt, device="cuda")
                kernels.attention(o_lat, q_full, store, store, ctx, _t(table, "int32"), H, 1, R + dr, 0, scale,
                                  v_head_dim=R, exact_weights=True)
                outs = kernels.linear_per_head(o_lat, _t(w_uv, dtype)).float().cpu().numpy().reshape(b - a, H, dv)
                if kernels.tensor_core_rows(R + dr, H, tdt):
                    # the form of the tensor-core kernels: the whole row as value, the result's tail unread
                    o_wide = torch.empty((b - a, H * (R + dr)), dtype=tdt, device="cuda")
                    kernels.attention(o_wide, q_full, store, store, ctx, _t(table, "int32"), H, 1, R + dr, 0, scale,
                                      exact_weights=True)
                    wide = kernels.linear_per_head(o_wide.view(b - a, H, R + dr)[:, :, :R], _t(w_uv, dtype))
                    assert np.abs(wide.float().cpu().numpy().reshape(b - a, H, dv) - want[a:b]).max() \
                        <= tol * np.abs(want).max(), (far, n_new, "whole rows")
            rows = store.float().cpu().numpy()
            for t in (0, far, T - 1):
                got = rows[ids[t // page], 0, t % page]
                assert np.abs(got[:R] - c[t]).max() <= tol * np.abs(c).max() and \
                    np.abs(got[R:] - k_rot[t]).max() <= tol * np.abs(k_rot).max(), t
            assert np.isfinite(rows).sum() == T * (R + dr)
            assert np.abs(outs - want[T - n_new:]).max() <= tol * np.abs(want).max(), (far, n_new)
        if dr >= 4:     # the far key carries the last row (one rotated pair alone cannot tell keys apart that well)
            assert np.abs(want[-1] - v[far]).max() < 0.05 * np.abs(v[far]).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,groups,keep", [(8, 3, 2, 1), (12, 2, 4, 1), (12, 4, 4, 2), (6, 3, 3, 2), (9, 9, 3, 3),
                                               (5, 2, 1, 1), (16, 1, 8, 3), (64, 6, 8, 4)])
def test_router_with_groups(dtype, E, top, groups, keep):
    """Softmax scores over all experts; a group scores as its best expert; only experts of the kept groups
    can be chosen; the weights are the scores themselves, not renormalized."""
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(E * 10 + top)
    n, d = 200, 40
    h = P.round_bf16(rng.standard_normal((n, d)))
    router = P.round_bf16(rng.standard_normal((E, d)) * 0.4)
    r = {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}}
    idx_w, wt_w = P.route(h, router, r)
    idx, wt = kernels.moe_route(_t(h, dtype), _t(router), top, score="softmax", renormalize=False, groups=groups, keep=keep)
    assert np.array_equal(idx.cpu().numpy(), idx_w)
    assert np.abs(wt.cpu().numpy() - wt_w).max() <= 1e-5
    assert (wt_w.sum(axis=1) < 1.0 + 1e-9).all()
    free, _ = P.route(h, router, {"experts": E, "top": top})
    sz = E // groups
    assert all(len({int(e) // sz for e in row}) <= keep for row in idx_w)
    if keep < groups and keep < top < E:
        # the limit matters in this test: some rows would have chosen otherwise
        assert (np.sort(free, axis=1) != np.sort(idx_w, axis=1)).any()
    elif keep >= min(groups, top):
        # the k best experts lie in the k best groups: no more experts than kept groups, no limit
        assert np.array_equal(free, idx_w)
    # without the option the kernel is the free choice
    idx0, _ = kernels.moe_route(_t(h, dtype), _t(router), top, score="softmax")
    assert np.array_equal(idx0.cpu().numpy(), free)


@pytest.mark.parametrize("n,E,top,d,f,act", [(700, 6, 3, 72, 104, "silu"), (1500, 4, 2, 128, 256, "silu"),
                                             (520, 3, 1, 200, 72, "clamped"), (600, 4, 2, 64, 64, "silu"), (900, 8, 4, 64, 520, "silu")])
def test_experts_of_a_large_step_on_the_tensor_cores(n, E, top, d, f, act):
    """The experts' two products of a large bfloat16 step in tiles of 128 rows per expert: experts with no rows,
    with a handful and with most of them, widths that end inside a k block and inside a 32-column chunk, weights
    on the outputs; against the sums in double precision, pair by pair."""
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(n + E)
    h = P.round_bf16(rng.standard_normal((n, d)))
    gate = P.round_bf16(rng.standard_normal((E, f, d)) / 6)
    up = P.round_bf16(rng.standard_normal((E, f, d)) / 6)
    down = P.round_bf16(rng.standard_normal((E, d, f)) / 5)
    # the choice: expert 1 is never taken, expert 0 by five tokens, the rest unevenly
    idx = np.zeros((n, top), dtype=np.int64)
    others = [e for e in range(E) if e != 1]
    weights_of = np.array([3.0 if e == others[-1] else 1.0 for e in others])
    for t in range(n):
        pool = others if t < 5 else others[1:]
        pw = weights_of[len(others) - len(pool):]
        idx[t] = rng.choice(pool, size=top, replace=False, p=pw / pw.sum()) if len(pool) >= top else rng.permutation(others)[:top]
    wt = rng.uniform(0.05, 1.0, (n, top))
    limit, alpha = (2.5, 1.7) if act == "clamped" else (0.0, 1.0)
    want = np.zeros((n, d))
    for e in range(E):
        for j in range(top):
            rows = np.nonzero(idx[:, j] == e)[0]
            if not len(rows):
                continue
            g, u = h[rows] @ gate[e].T, h[rows] @ up[e].T
            if act == "clamped":
                g, u = np.minimum(g, limit), np.clip(u, -limit, limit)
                a = g * P.sigmoid(alpha * g) * (u + 1.0)
            else:
                a = g * P.sigmoid(g) * u
            want[rows] += wt[rows, j:j + 1] * (P.round_bf16(a) @ down[e].T)
    gu = _t(np.concatenate([gate, up], axis=1), "bfloat16")
    offsets, perm = kernels.moe_sort(_t(idx, "int32"), E)
    wt_d = _t(wt.reshape(-1))
    x = _t(h, "bfloat16")
    assert kernels.moe_gemm_tcgen05_pays(x, gu, n * top, True, False)
    kw = dict(activation=act, limit=limit, alpha=alpha)
    a_s = kernels.moe_gemm_tcgen05(x, gu, offsets, perm, wt_d, top, gated=True, **kw)
    parts = kernels.moe_gemm_tcgen05(a_s, _t(down, "bfloat16"), offsets, perm, wt_d, top, gated=False, scale_out=True)
    kernels.check_status(x.device)
    y = kernels.moe_combine(parts, top).cpu().numpy()
    assert np.isfinite(y).all()
    assert np.abs(y - want).max() <= 1e-2 * np.abs(want).max()
    # the grouped mma.sync kernel gives the same rows but for the order of the sums
    a_m = kernels.moe_gemm(x, gu, offsets, perm, wt_d, top, gated=True, **kw)
    assert (a_m.float() - a_s.float()).abs().max().item() <= 2e-2 * a_m.float().abs().max().item()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sigmoid_gate_on_strided_rows(dtype):
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(8)
    n, f = 13, 42
    a = P.round_bf16(rng.standard_normal((n, f)))
    wide = rng.standard_normal((n, f + 30)) * 3
    gate = _t(wide)[:, 7:7 + f]
    out = torch.empty((n, f), dtype=getattr(torch, dtype), device="cuda")
    kernels.sigmoid_gate(out, _t(a, dtype), gate)
    want = a * P.sigmoid(wide[:, 7:7 + f])
    assert np.abs(out.float().cpu().numpy() - want).max() <= (1e-6 if dtype == "float32" else 1e-2) * np.abs(want).max()
