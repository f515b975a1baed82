"""The Senulix design in the engine against its plain implementation (tests/plain/senulix_plain.py).

Small configurations of their own, random weights whose values are bfloat16 numbers (so both
dtypes load the same model): each mechanism's kernel alone, whole prompts, prompts against
token-by-token decoding, portions down to two tokens, unequal batches, slots and pages that
are used again, keys far away, at page borders and just inside and outside a window that one
score makes stand out, the first tokens, long decoding through CUDA graphs, and greedy generation
through the scheduler.
"""
import numpy as np
import pytest

from helpers import write_model_dir
from plain import senulix_plain as P
from test_gpu_sozarax import _ctx, _paged, _t, check_rows, engine_for, run_cut

pytestmark = pytest.mark.gpu


def _attn(heads, kv_heads, dim, vdim, scale, window, rot):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return m


def _latent(heads, dim, rot_dim, vdim, kv_rank, scale, base, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _light(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


# A: sizes that suit vector widths.  A recurrent layer first, windows shorter and longer than a page and than
# the prompts, two layers that read the rows another layer cached (with heads and sizes of their own, one
# right behind its source, one further on), layers with and without a feed-forward, a decay of exactly 1.
CFG_A = {
    "architecture": "Senulix", "vocab": 96, "width": 64, "norm": {"eps": 1e-5}, "token_side": {"dim": 8},
    "logit_softcap": 12.0,
    "layers": [
        _layer("lightning", _light(3, 16, 24, [0.5, 0.93, 1.0]), 48),
        _layer("attention", _attn(4, 2, 16, 24, 0.3, 40, (100.0, 8)), 72),
        _layer("latent_attention", _latent(3, 16, 8, 12, 32, 0.3, 100.0), None),
        _layer("latent_attention", _latent(2, 8, 8, 16, 32, 0.4, 100.0, kv_from=2), 40),
        _layer("attention", _attn(6, 1, 8, 8, 0.5, 7, (10000.0, 8)), None),
        _layer("lightning", _light(2, 8, 8, [0.8, 0.99]), None),
        _layer("latent_attention", _latent(4, 8, 8, 8, 32, 0.35, 100.0, kv_from=2), 56),
        _layer("attention", _attn(2, 2, 32, 16, 0.2, 300, (1000.0, 16)), 64),
    ],
}
# B: sizes that fit no vector width or tile; no token side input and no cap on the logits; a window of one
# position (a token sees itself and the sink alone) and of two; no rotation at all in one layer, the whole head
# rotated in another; a layer without a window; one head, one kv head, values of another size than keys.
CFG_B = {
    "architecture": "Senulix", "vocab": 61, "width": 50, "norm": {"eps": 1e-6},
    "layers": [
        _layer("latent_attention", _latent(5, 6, 2, 5, 10, 0.5, 10.0), 22),
        _layer("attention", _attn(3, 3, 10, 6, 0.4, 1, (100.0, 4)), 18),
        _layer("lightning", _light(1, 12, 7, [0.97]), 14),
        _layer("attention", _attn(2, 1, 6, 9, 0.6, 2, None), None),
        _layer("attention", _attn(1, 1, 12, 7, 0.3, None, (30.0, 12)), 26),
        _layer("latent_attention", _latent(1, 12, 2, 7, 10, 0.3, 10.0, kv_from=0), 10),
    ],
}
# C: head sizes of the tensor-core kernels (latent rows of 128 + 64), many heads on one key head, values wider
# than a recurrent layer's slice of value channels, a token side input of an odd size.
CFG_C = {
    "architecture": "Senulix", "vocab": 80, "width": 128, "norm": {"eps": 1e-6}, "token_side": {"dim": 12},
    "logit_softcap": 50.0,
    "layers": [
        _layer("attention", _attn(8, 2, 64, 64, 0.125, 64, (10000.0, 32)), 96),
        _layer("latent_attention", _latent(4, 32, 64, 32, 128, 0.1, 10000.0), 64),
        _layer("lightning", _light(2, 64, 96, [0.9, 0.999]), None),
        _layer("latent_attention", _latent(6, 16, 64, 48, 128, 0.15, 10000.0, kv_from=1), 32),
        _layer("attention", _attn(20, 1, 16, 32, 0.2, 33, (500.0, 16)), None),
    ],
}
# D: sizes in steps of 16 as a small served model has them, other than C's: heads in blocks that straddle kv heads on
# the cluster form (12 heads on 4 kv heads), values wider than keys, a window that is no multiple of a page or a
# tile, two readers of one latent, recurrent layers of many small heads, a token side input of a vector width.
CFG_D = {
    "architecture": "Senulix", "vocab": 160, "width": 256, "norm": {"eps": 1e-6}, "token_side": {"dim": 32},
    "logit_softcap": 25.0,
    "layers": [
        _layer("latent_attention", _latent(4, 48, 32, 32, 96, 0.11, 20000.0), 320),
        _layer("attention", _attn(12, 4, 32, 48, 0.18, 77, (20000.0, 16)), 320),
        _layer("lightning", _light(8, 16, 32, [0.7, 0.8, 0.9, 0.95, 0.97, 0.98, 0.99, 0.995]), None),
        _layer("latent_attention", _latent(8, 16, 32, 16, 96, 0.14, 20000.0, kv_from=0), 192),
        _layer("attention", _attn(4, 4, 48, 16, 0.14, 130, (20000.0, 48)), 192),
        _layer("latent_attention", _latent(2, 64, 32, 64, 96, 0.1, 20000.0, kv_from=0), None),
        _layer("lightning", _light(2, 64, 64, [0.9, 0.99]), 256),
    ],
}
CFGS = {"A": (CFG_A, 51), "B": (CFG_B, 52), "C": (CFG_C, 53), "D": (CFG_D, 54)}


def make_model(tmp_path, name, qk_boost=2.0):
    cfg, seed = CFGS[name]
    w = P.random_weights(cfg, seed, qk_boost=qk_boost)
    d = write_model_dir(str(tmp_path / f"senulix_{name}"), cfg, {k: np.asarray(v, dtype=np.float32) for k, v in w.items()})
    return cfg, w, d


# ---- whole models --------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompt_and_every_way_of_cutting(tmp_path, name, dtype):
    cfg, w, d = make_model(tmp_path, name, 2.0 if dtype == "float32" else 1.0)
    rng = np.random.default_rng(5)
    ids = rng.integers(0, cfg["vocab"], size=150).tolist()
    want, layers = P.forward(w, cfg, ids, return_layers=True)
    eng = engine_for(d, dtype)
    try:
        got_taps = []
        eng.model.tap = lambda i, x: got_taps.append(x.detach().float().cpu().numpy().copy())
        whole = run_cut(eng, ids, [len(ids)])
        eng.model.tap = None
        assert len(got_taps) == len(layers)
        for i, (g, t) in enumerate(zip(got_taps, layers)):      # the residual stream after every layer
            assert np.abs(g - t).max() <= (1e-4 if dtype == "float32" else 1e-1) * np.abs(t).max(), (name, i)
        check_rows(whole, want, dtype, f"{name} whole")
        check_rows(run_cut(eng, ids[:3], [3]), want[:3], dtype, f"{name} first tokens")
        check_rows(run_cut(eng, ids[:1], [1]), want[:1], dtype, f"{name} one token")
        check_rows(run_cut(eng, ids, [len(ids) - 70, 1]), want, dtype, f"{name} prompt then decode")
        check_rows(run_cut(eng, ids[:70], [1]), want[:70], dtype, f"{name} decode from the start")
        for cuts in ([2], [3, 2, 37, 16, 5, 2, 64, 1], [17], [16, 16, 1, 31, 2]):
            got = run_cut(eng, ids, cuts)
            check_rows(got, want, dtype, f"{name} portions {cuts}")
            if dtype == "float32":
                # small steps take other product kernels than large ones, chunks other sums: another order
                assert np.abs(got - whole).max() <= 3e-5 * np.abs(want).max(), cuts
    finally:
        eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_and_reuse_of_slots_and_pages(tmp_path, dtype):
    """Four requests of unequal length in one batch, portions of some beside single tokens of
    others, then new requests in the slots and pages that the finished ones gave back; a pool
    that holds little more than what is live.  Every request also runs alone."""
    from kllm_b200.engine.step import StepEntry
    cfg, w, d = make_model(tmp_path, "A", 2.0 if dtype == "float32" else 1.0)
    rng = np.random.default_rng(9)
    lens = [37, 90, 5, 64, 21, 50]
    seqs = [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lens]
    want = [P.forward(w, cfg, s) for s in seqs]
    eng = engine_for(d, dtype, num_blocks=20, max_batch=4)      # 320 tokens of pages, four slots
    try:
        got = [np.zeros_like(x) for x in want]
        fed = [0] * len(seqs)
        caches = {}
        queue = list(range(len(seqs)))
        sizes = [3, 1, 16, 2, 29, 1, 7]
        turn = 0
        slots_seen = []
        while queue or caches:
            while queue and len(caches) < 4:
                i = queue.pop(0)
                caches[i] = eng.cache.open()
                slots_seen.append(caches[i].state_slot)
            entries, order = [], []
            for i in list(caches):
                left = len(seqs[i]) - fed[i]
                n = 1 if left <= 8 else min(left, sizes[(turn + i) % len(sizes)])
                entries.append(StepEntry(caches[i], seqs[i][fed[i]:fed[i] + n], list(range(n))))
                order.append((i, n))
            lg = eng.runner.run(entries).float().cpu().numpy()
            r = 0
            for i, n in order:
                got[i][fed[i]:fed[i] + n] = lg[r:r + n]
                r += n
                fed[i] += n
                if fed[i] == len(seqs[i]):
                    eng.cache.close(caches.pop(i))
            turn += 1
            eng.cache.audit()
        assert len(slots_seen) > len(set(slots_seen)), "no state slot was used again"
        for i in range(len(seqs)):
            check_rows(got[i], want[i], dtype, f"request {i} in mixed batches")
            alone = run_cut(eng, seqs[i], [len(seqs[i])])
            tol = 3e-5 if dtype == "float32" else 8e-2
            assert np.abs(alone - got[i]).max() <= tol * np.abs(want[i]).max(), f"request {i} alone against the batch"
    finally:
        eng.close()


def test_long_decoding(tmp_path):
    """A short prompt and then hundreds of single tokens: the decode route (graphs, pages added one by one, a
    window that passes over decoded tokens and gives its pages back, a state carried through hundreds of steps)."""
    cfg, w, d = make_model(tmp_path, "A")
    rng = np.random.default_rng(3)
    ids = rng.integers(0, cfg["vocab"], size=420).tolist()
    want = P.forward(w, cfg, ids)
    eng = engine_for(d, "float32", max_seq=448, num_blocks=30)
    try:
        check_rows(run_cut(eng, ids, [9, 1]), want, "float32", "long decoding")
    finally:
        eng.close()


def test_greedy_generation_through_the_scheduler(tmp_path):
    """``Engine.generate`` (scheduler, sampler, pipelined steps whose token ids stay on the device, which the
    token side input must read there) on several prompts at once against greedy decoding with the plain
    implementation."""
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


@pytest.mark.parametrize("name", ["A", "D"])
def test_replay_program(tmp_path, name):
    """bin/trace_run on a model of this design: whole, decode, portions and mixed batches of up
    to four live requests in a pool as small as the trace allows."""
    from test_gpu_replay import build_trace
    from trace_tools import run_trace
    cfg, w, d = make_model(tmp_path, name, 1.0)
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

@pytest.mark.parametrize("heads,dk,dv", [(2, 16, 16), (3, 24, 40), (1, 64, 96), (2, 128, 128), (1, 7, 5)])
def test_lightning_scan_carries_its_state(heads, dk, dv):
    """The recurrence over two requests of unequal length in one launch, cut in two launches at an odd place
    (chunks that end in the middle, a second launch that starts from the slot), in slots 2 and 0, against the
    plain token-by-token scan over each whole sequence; the state left in the slots too."""
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(dk)
    lens = [75, 9]
    A, B = heads * dk, heads * dv
    q, k = rng.standard_normal((sum(lens), A)), rng.standard_normal((sum(lens), A))
    v = rng.standard_normal((sum(lens), B))
    decay = np.linspace(0.6, 1.0, heads)
    state = torch.zeros((3, heads * dk * dv + 4), device="cuda")
    slots, offs = [2, 0], [0, lens[0]]
    got = np.zeros((sum(lens), B))
    for part in ([(0, 41), (0, 4)], [(41, 75), (4, 9)]):
        rows = np.concatenate([np.arange(offs[s] + a, offs[s] + b) for s, (a, b) in enumerate(part)])
        ctx = _ctx([b - a for a, b in part], [a for a, _ in part], slots)
        got[rows] = kernels.lightning_scan(_t(q[rows]), _t(k[rows]), _t(v[rows]), _t(decay), state, ctx, heads, dk,
                                           dv).cpu().numpy()
    st = state.cpu().numpy()
    for s in range(2):
        sl = slice(offs[s], offs[s] + lens[s])
        want, S = P.decayed_state_scan(P.silu(q[sl]).reshape(-1, heads, dk), P.silu(k[sl]).reshape(-1, heads, dk),
                                       P.silu(v[sl]).reshape(-1, heads, dv), decay)
        assert np.abs(got[sl] - want.reshape(-1, B)).max() <= 2e-5 * np.abs(want).max()
        assert np.abs(st[slots[s], :heads * dk * dv].reshape(heads, dk, dv) - S).max() <= 2e-5 * np.abs(S).max()
    assert np.all(st[1] == 0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_lightning_gate_norm_and_output_norm_kernels(dtype):
    """One norm over ALL heads' values with a gain and a sigmoid gate; x += norm(y) with the updated rows handed on
    in the model dtype; the activations and the soft cap."""
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(2)
    n, width = 7, 72
    o, g, gain = rng.standard_normal((n, width)) * 3, rng.standard_normal((n, width)), 1 + 0.3 * rng.standard_normal(width)
    y = kernels.lightning_gate_norm(_t(o), _t(g), _t(gain), 1e-5, getattr(torch, dtype)).float().cpu().numpy()
    want = P.norm_plain(o, gain, 1e-5) * P.sigmoid(g)
    tol = 1e-5 if dtype == "float32" else 1e-2
    assert np.abs(y - want).max() <= tol * np.abs(want).max()
    x, yy = rng.standard_normal((n, width)), rng.standard_normal((n, width)) * 5
    xt, out = _t(x), torch.empty((n, width), dtype=getattr(torch, dtype), device="cuda")
    kernels.rmsnorm_add(xt, _t(yy), _t(gain), 1e-6, out=out)
    want = x + P.norm_plain(yy, gain, 1e-6)
    assert np.abs(xt.cpu().numpy() - want).max() <= 1e-5 * np.abs(want).max()
    assert np.abs(out.float().cpu().numpy() - want).max() <= tol * np.abs(want).max()
    z = rng.standard_normal((n, width)) * 4
    for op, fn in (("gelu", P.gelu_erf), ("gelu_tanh", P.gelu_tanh), ("copy", lambda a: a)):
        assert np.abs(kernels.unary(_t(z), op, torch.float32).cpu().numpy() - fn(z)).max() <= 1e-5
    zt = _t(z * 10)
    kernels.unary(zt, "softcap", torch.float32, arg=7.0, out=zt)
    assert np.abs(zt.cpu().numpy() - 7.0 * np.tanh(z * 10 / 7.0)).max() <= 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_token_side_slice(dtype):
    """A slice of each token's row of the second table, gated; an id that is still on the device."""
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(4)
    vocab, cols, Pn, off, n = 19, 30, 6, 12, 5
    table = P.round_bf16(rng.standard_normal((vocab, cols)).astype(np.float32))
    gate = rng.standard_normal((n, Pn)) * 2
    ids = np.array([3, 18, -2, 0, 7])
    last = np.array([11, 5, 9])
    got = kernels.gated_slice(_t(gate), _t(table, dtype), off, _t(ids, "int32"), _t(last, "int32")).float().cpu().numpy()
    real = np.where(ids < 0, last[np.maximum(-ids - 1, 0)], ids)
    want = P.gelu_tanh(gate) * table[real, off:off + Pn]
    assert np.abs(got - want).max() <= (1e-5 if dtype == "float32" else 1e-2) * np.abs(want).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dk,dv,rot", [(4, 2, 16, 24, 8), (3, 3, 10, 6, 10), (2, 1, 64, 32, 0), (6, 2, 12, 12, 4)])
def test_whole_projection_norm_rotation_and_cache_write(dtype, H, G, dk, dv, rot):
    """Norm over the whole q and k projections, then the rotation of each head's first values, q out, k and v into
    shuffled pages; a layer that only reads another's cache produces q alone."""
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(H * dk)
    n_new, start = [5, 1, 9], [3, 40, 0]
    ctx = _ctx(n_new, start)
    n = sum(n_new)
    Q, K, V = H * dk, G * dk, G * dv
    qkv = rng.standard_normal((n, Q + K + V)) * 2
    qg, kg = 1 + 0.3 * rng.standard_normal(Q), 1 + 0.3 * rng.standard_normal(K)
    page, pages = 8, 12
    table = np.full((3, 6), -1, dtype=np.int32)
    perm = rng.permutation(pages)
    used = 0
    for s in range(3):
        need = -(-(start[s] + n_new[s]) // page)
        table[s, :need] = perm[used:used + need]
        used += need
    td = getattr(torch, dtype)
    kc = torch.zeros((pages, G, page, dk), dtype=td, device="cuda")
    vc = torch.zeros((pages, G, page, dv), dtype=td, device="cuda")
    q_out = torch.empty((n, Q), dtype=td, device="cuda")
    base = 100.0
    freq = _t(base ** (-2.0 * np.arange(rot // 2) / max(rot, 1)), "float64") if rot else None
    kernels.qknorm_append(q_out, _t(qkv), _t(qg), _t(kg), 1e-5, 0.0, 1, ctx.positions, ctx.token_req, _t(table, "int32"), kc,
                          vc, H, G, dk, dv, rot=rot, freq=freq)
    pos = ctx.positions.cpu().numpy()
    q, k = P.normed_rotated_qk(qkv[:, :Q], qkv[:, Q:Q + K], qg, kg, 1e-5, H, G, dk, pos, {"dims": rot, "base": base} if rot else None)
    tol = 1e-5 if dtype == "float32" else 1e-2
    assert np.abs(q_out.float().cpu().numpy() - q.reshape(n, Q)).max() <= tol * np.abs(q).max()
    req = ctx.token_req.cpu().numpy()
    kcn, vcn = kc.float().cpu().numpy(), vc.float().cpu().numpy()
    for t in range(n):
        pg, sl = table[req[t], pos[t] // page], pos[t] % page
        assert np.abs(kcn[pg, :, sl] - k[t]).max() <= tol * np.abs(k).max()
        assert np.abs(vcn[pg, :, sl] - qkv[t, Q + K:].reshape(G, dv)).max() <= tol * np.abs(qkv).max()
    q_only = torch.empty((n, Q), dtype=td, device="cuda")
    kernels.qknorm_append(q_only, _t(qkv[:, :Q]), _t(qg), None, 1e-5, 0.0, 1, ctx.positions, ctx.token_req, None, None, None,
                          H, G, dk, dv, rot=rot, freq=freq)
    assert torch.equal(q_only, q_out)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dk,dv,window", [(4, 2, 16, 24, 40), (6, 3, 8, 4, 33), (3, 1, 10, 6, 16), (8, 2, 64, 64, 64),
                                              (40, 2, 16, 16, 100), (2, 2, 32, 64, 0), (5, 5, 12, 8, 1), (32, 8, 128, 128, 48)])
def test_mixed_attention_window_edges_far_keys_and_page_borders(dtype, H, G, dk, dv, window):
    """Scores mixed across the heads with a matrix far from the identity.  For every probed query one key is made
    to stand out (a large score in one head, which the mixing spreads to the others): the key just inside the
    window, the key just outside it (whose value must NOT show), a key at a page border, the first key.  Portions
    cut at odd places beside single tokens in one launch, pages in a shuffled order."""
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(H * 100 + dk)
    T, page = 150, 16
    W = window or None
    q = rng.standard_normal((T, H, dk)) * 0.3
    k = rng.standard_normal((T, G, dk)) * 0.3
    v = rng.standard_normal((T, G, dv))
    talk = np.eye(H) + 0.4 * rng.standard_normal((H, H))
    scale = 0.5
    # probes: query position -> the key that stands out for it
    far = (window or 120)
    probes = {}
    for qp, kp in ((130, 130 - far + 1), (131, 131 - far), (149, 144), (140, 128), (100, max(0, 100 - far + 1)), (47, 0)):
        if 0 <= kp <= qp:
            probes[qp] = kp
    marks = {}                 # key position -> (head, direction): two queries that probe one key share them
    for qp, kp in probes.items():
        if kp not in marks:
            u = rng.standard_normal(dk)
            marks[kp] = (int(rng.integers(0, H)), u / np.linalg.norm(u))
            k[kp, marks[kp][0] // (H // G)] = marks[kp][1] * 6.0
            v[kp] = 5.0 + rng.standard_normal((G, dv))
        q[qp, marks[kp][0]] = marks[kp][1] * 6.0
    if dtype == "bfloat16":
        q, k, v = P.round_bf16(q), P.round_bf16(k), P.round_bf16(v)
    want = P.mixed_window_attention(q, k, v, talk, scale, W).reshape(T, H * dv)
    kc, vc, ids = _paged(k, v, page, 14, 3)
    table = np.full((1, 12), -1, dtype=np.int32)
    table[0, :len(ids)] = ids
    td = getattr(torch, dtype)
    kct, vct = _t(np.nan_to_num(kc), dtype), _t(np.nan_to_num(vc), dtype)
    qt = _t(q.reshape(T, H * dk), dtype)
    tol = 2e-5 if dtype == "float32" else 2e-2
    sinks = torch.zeros(H, device="cuda")

    def run(n_new, start, rows):
        ctx = _ctx(n_new, start)
        out = torch.empty((len(rows), H * dv), dtype=td, device="cuda")
        tab = _t(np.repeat(table, len(n_new), axis=0), "int32")
        kernels.attention_mixed(out, qt[rows], kct, vct, _t(talk), ctx, tab, H, G, dk, dv, window, scale, sinks=sinks)
        return out.float().cpu().numpy()

    got = run([T], [0], np.arange(T))                                   # the whole prompt
    assert np.abs(got - want).max() <= tol * np.abs(want).max(), "whole"
    # a portion that starts in the middle of a page beside single tokens of the same sequence at other places
    rows = np.concatenate([np.arange(93, 150), [47], [131], [130]])
    got = run([57, 1, 1, 1], [93, 47, 131, 130], rows)
    assert np.abs(got - want[rows]).max() <= tol * np.abs(want).max(), "portion beside single tokens"
    singles = np.array(sorted(probes))
    got = run([1] * len(singles), list(singles), singles)              # decoding steps
    assert np.abs(got - want[singles]).max() <= tol * np.abs(want).max(), "single tokens"
    if window and 131 in probes:
        # the key just outside the window carried values around 5: they must not show
        inside = P.mixed_window_attention(q, k, v, talk, scale, window + 1).reshape(T, H * dv)
        assert np.abs(inside[131] - want[131]).max() > 0.5, "the probe does not tell the window's edge"
    # without the sink the denominators differ
    ctx = _ctx([T], [0])
    out = torch.empty((T, H * dv), dtype=td, device="cuda")
    kernels.attention_mixed(out, qt, kct, vct, _t(talk), ctx, _t(table, "int32"), H, G, dk, dv, window, scale)
    plain = P.mixed_window_attention(q, k, v, talk, scale, W, sink=False).reshape(T, H * dv)
    assert np.abs(out.float().cpu().numpy() - plain).max() <= tol * np.abs(plain).max(), "no sink"


@pytest.mark.parametrize("H,G,dk,dv", [(8, 2, 64, 64), (32, 8, 128, 128), (6, 3, 16, 48), (20, 1, 16, 32), (12, 4, 32, 16),
                                       (40, 2, 16, 16), (7, 7, 16, 16), (13, 1, 32, 32)])
def test_mixed_attention_forms_agree(H, G, dk, dv):
    """bfloat16 portions: the two tensor-core forms (one with a cluster of CTAs that share their raw scores) against
    the CUDA-core form on the same operands (all keep scores, mixing and weights in float32, so they differ by the
    order of sums and the weights' second bfloat16 term)."""
    import torch
    from kllm_b200 import kernels
    from kllm_b200.csrc.build import load_library
    assert load_library("attention_mixed").kllm_attention_mixed_mma_fits(H, G, dk, dv)
    g = torch.Generator(device="cuda").manual_seed(H)
    T, page, window = 200, 16, 70
    pages = -(-T // page)
    q = (torch.randn(T, H * dk, device="cuda", generator=g) * 0.3).bfloat16()
    kc = (torch.randn(pages, G, page, dk, device="cuda", generator=g) * 0.3).bfloat16()
    vc = torch.randn(pages, G, page, dv, device="cuda", generator=g).bfloat16()
    mix = (torch.eye(H, device="cuda") + 0.3 * torch.randn(H, H, device="cuda", generator=g)).contiguous()
    table = torch.arange(pages, dtype=torch.int32, device="cuda").view(1, pages).repeat(3, 1).contiguous()
    ctx = _ctx([1, 150, 37], [199, 13, 0])
    rows = torch.tensor([199] + list(range(13, 163)) + list(range(37)), device="cuda")
    outs = {}
    lib = load_library("attention_mixed")
    forms = {"cuda cores": (False, False), "tensor cores": (True, False)}
    if lib.kllm_attention_mixed_cluster_fits(H, G, dk, dv):
        forms["cluster"] = (True, True)
    try:
        for name, (mma, cluster) in forms.items():
            kernels.MIXED_MMA, kernels.MIXED_CLUSTER = mma, cluster
            out = torch.empty((len(rows), H * dv), dtype=torch.bfloat16, device="cuda")
            kernels.attention_mixed(out, q[rows], kc, vc, mix, ctx, table, H, G, dk, dv, window, dk ** -0.5,
                                    sinks=torch.zeros(H, device="cuda"))
            outs[name] = out.float()
    finally:
        kernels.MIXED_MMA = kernels.MIXED_CLUSTER = True
    torch.cuda.synchronize()
    want = outs.pop("cuda cores")
    for name, got in outs.items():
        assert float((got - want).abs().max()) <= 2e-2 * float(want.abs().max()), name
        assert float((got - want).abs().mean()) <= 2e-3 * float(want.abs().max()), name


def test_shared_latent_reads_the_other_layers_rows(tmp_path):
    """A layer with ``kv_from`` must read its source's cached rows, not rows of its own: with the source's
    down-projection changed, the plain implementation and the engine change alike."""
    cfg, w, d = make_model(tmp_path, "A")
    rng = np.random.default_rng(1)
    ids = rng.integers(0, cfg["vocab"], size=60).tolist()
    w2 = dict(w)
    w2["l2.mix.dkv"] = P.round_bf16(np.asarray(w["l2.mix.dkv"]) * 1.5)
    d2 = write_model_dir(str(tmp_path / "senulix_A2"), cfg, {k: np.asarray(v_, dtype=np.float32) for k, v_ in w2.items()})
    a, b = P.forward(w, cfg, ids), P.forward(w2, cfg, ids)
    assert np.abs(a - b).max() > 1e-2 * np.abs(a).max()
    for folder, want in ((d, a), (d2, b)):
        eng = engine_for(folder, "float32")
        try:
            check_rows(run_cut(eng, ids, [23, 1, 5]), want, "float32", "shared latent")
        finally:
            eng.close()
