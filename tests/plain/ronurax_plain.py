"""Plain, slow Ronurax forward pass in numpy float64: the yardstick of its tests.

Whole sequences, no cache, no paging, no batches; one function per mechanism.
Nothing here is imported by the product package and nothing of the product
package is imported here.  Weights arrive as a dict of tensor name -> numpy
array and are widened to float64; ``cfg`` is the dict of a config.json.

Notation: T tokens, d the model width, H query heads, G key/value heads, dk the per-head
(and per-map) query/key size, dv the per-head value size, R the size of the key/value
latent, dr the rotated size, C the size of a mask segment, E experts.
"""
from __future__ import annotations

import math

import numpy as np


def f64(a):
    return np.asarray(a, dtype=np.float64)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def layer_norm(x, gain, bias, eps):
    """(x - mean) / sqrt(var + eps) * gain + bias, the variance being the mean squared deviation."""
    x = f64(x)
    mu = x.mean(axis=-1, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * f64(gain) + f64(bias)


def rms_norm(x, gain, eps):
    x = f64(x)
    y = x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    return y if gain is None else y * f64(gain)


def softmax_rows(scores, visible):
    s = np.where(visible, scores, -np.inf)
    e = np.where(visible, np.exp(s - s.max(axis=-1, keepdims=True)), 0.0)
    return e / e.sum(axis=-1, keepdims=True)


# ---- rotary positions ---------------------------------------------------------------

def base_frequencies(dims, base):
    i = np.arange(dims // 2, dtype=np.float64)
    return base ** (-2.0 * i / dims)


def stretched_by_wavelength(freq, sc):
    """Frequency scaling by wavelength bands: short waves stay, long waves are divided by
    ``factor``, those between are blended."""
    if not sc:
        return freq
    factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
    out = np.empty_like(freq)
    for n, f in enumerate(freq):
        wave = 2.0 * math.pi / f
        if wave < orig / high:
            out[n] = f
        elif wave > orig / low:
            out[n] = f / factor
        else:
            s = (orig / wave - low) / (high - low)
            out[n] = (1.0 - s) * f / factor + s * f
    return out


def stretched_by_ramp(freq, dims, base, sc):
    """YaRN: (frequencies, amplitude).  A ramp over the pair index blends f / factor into f;
    cos and sin are multiplied by the amplitude."""
    if not sc:
        return freq, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def where(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    i = np.arange(dims // 2, dtype=np.float64)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, freq, dims, amplitude=1.0):
    """Rotate the first ``dims`` values of the last axis of x [T, ..., n]; pair (i, i + dims / 2)."""
    x = f64(x).copy()
    half = dims // 2
    ang = f64(positions)[:, None] * freq[None, :]                   # [T, half]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (half,)
    c, s = (np.cos(ang) * amplitude).reshape(shape), (np.sin(ang) * amplitude).reshape(shape)
    u, v = x[..., :half].copy(), x[..., half:dims].copy()
    x[..., :half] = u * c - v * s
    x[..., half:dims] = v * c + u * s
    return x


# ---- masks ------------------------------------------------------------------------------

def causal_mask(T):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return j <= i


def segment_mask(T, size):
    """j <= i and both in the same segment of ``size`` positions counted from 0."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & ((i // size) == (j // size))


# ---- mixers -----------------------------------------------------------------------------

def two_map_heads(q, k, v, visible, scale, lam, diff, eps):
    """q [T, H, 2, dk], k [T, G, 2, dk], v [T, G, dv] -> [T, H, dv]: every head has two softmax maps over
    the same values; o = a1 - lam a2, divided by its root mean square over dv, times (1 - diff)."""
    T, H = q.shape[:2]
    G, dv = v.shape[1], v.shape[2]
    out = np.zeros((T, H, dv))
    for hh in range(H):
        g = hh // (H // G)
        a = [softmax_rows(q[:, hh, mp] @ k[:, g, mp].T * scale, visible) @ v[:, g] for mp in (0, 1)]
        out[:, hh] = rms_norm(a[0] - lam * a[1], None, eps) * (1.0 - diff)
    return out


def map_lambda(lq1, lk1, lq2, lk2, diff):
    return math.exp(float(np.sum(f64(lq1) * f64(lk1)))) - math.exp(float(np.sum(f64(lq2) * f64(lk2)))) + diff


def differential_attention(h, w, p, m, eps):
    """Two softmax maps per head over the same values, combined as a1 - lambda a2."""
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    h = f64(h)
    q = (h @ f64(w[p + "q"]).T + f64(w[p + "q.b"])).reshape(T, H, 2, dk)
    k = (h @ f64(w[p + "k"]).T + f64(w[p + "k.b"])).reshape(T, G, 2, dk)
    v = (h @ f64(w[p + "v"]).T + f64(w[p + "v.b"])).reshape(T, G, dv)
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    rot = m.get("rot")
    if rot:
        freq = stretched_by_wavelength(base_frequencies(rot["dims"], float(rot["base"])), rot.get("scaling"))
        pos = np.arange(T)
        q = rotate(q, pos, freq, rot["dims"])
        k = rotate(k, pos, freq, rot["dims"])
    vis = segment_mask(T, m["mask"]["size"]) if m.get("mask") else causal_mask(T)
    diff = float(m["diff"])
    lam = map_lambda(w[p + "lq1"], w[p + "lk1"], w[p + "lq2"], w[p + "lk2"], diff)
    out = two_map_heads(q, k, v, vis, float(m["scale"]), lam, diff, eps)
    return out.reshape(T, H * dv) @ f64(w[p + "o"]).T


def latent_heads(q_plain, q_rot, k_plain, k_rot, v, visible, scale):
    """q_plain [T, H, dk], q_rot [T, H, dr] (rotated), k_plain [T, H, dk], k_rot [T, dr] (rotated, one for
    all heads), v [T, H, dv] -> [T, H, dv]."""
    T, H = q_plain.shape[:2]
    out = np.zeros((T, H, v.shape[2]))
    for hh in range(H):
        s = (q_plain[:, hh] @ k_plain[:, hh].T + q_rot[:, hh] @ k_rot.T) * scale
        out[:, hh] = softmax_rows(s, visible) @ v[:, hh]
    return out


def latent_attention(h, w, p, m, eps):
    """Keys and values through a cached latent plus one rotated key part shared by the heads;
    a sigmoid gate on the concatenated heads."""
    H, dk, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    h = f64(h)
    q = (h @ f64(w[p + "q"]).T).reshape(T, H, dk + dr)
    down = h @ f64(w[p + "dkv"]).T
    c = rms_norm(down[:, :R], w[p + "dkv.norm"], eps)
    k_plain = (c @ f64(w[p + "uk"]).T).reshape(T, H, dk)
    v = (c @ f64(w[p + "uv"]).T).reshape(T, H, dv)
    rot = m["rot"]
    freq, amp = stretched_by_ramp(base_frequencies(dr, float(rot["base"])), dr, float(rot["base"]), rot.get("scaling"))
    pos = np.arange(T)
    q_rot = rotate(q[:, :, dk:], pos, freq, dr, amp)
    k_rot = rotate(down[:, R:], pos, freq, dr, amp)
    out = latent_heads(q[:, :, :dk], q_rot, k_plain, k_rot, v, causal_mask(T), float(m["scale"]))
    gate = sigmoid(h @ f64(w[p + "g"]).T)
    return (out.reshape(T, H * dv) * gate) @ f64(w[p + "o"]).T


# ---- feed-forward -----------------------------------------------------------------------

def route(h, w_router, r):
    """(chosen experts [T, top], their weights [T, top]): softmax scores, only experts of the
    ``keep`` groups with the largest best score may be chosen, the scores are the weights."""
    z = f64(h) @ f64(w_router).T
    s = np.exp(z - z.max(axis=-1, keepdims=True))
    s /= s.sum(axis=-1, keepdims=True)
    T, E = s.shape
    allowed = np.ones((T, E), dtype=bool)
    grp = r.get("groups")
    if grp:
        n, keep = grp["count"], grp["keep"]
        best = s.reshape(T, n, E // n).max(axis=-1)
        order = np.argsort(-best, axis=-1, kind="stable")[:, :keep]
        ok = np.zeros((T, n), dtype=bool)
        np.put_along_axis(ok, order, True, axis=-1)
        allowed = np.repeat(ok, E // n, axis=-1)
    masked = np.where(allowed, s, -1.0)
    idx = np.argsort(-masked, axis=-1, kind="stable")[:, :r["top"]]
    return idx, np.take_along_axis(s, idx, axis=-1)


def experts(h, w, p, ml):
    h = f64(h)
    idx, wt = route(h, w[p + "router"], ml["router"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(idx[t], wt[t]):
            g = f64(w[f"{p}e{e}.gate"]) @ h[t]
            u = f64(w[f"{p}e{e}.up"]) @ h[t]
            out[t] += s * (f64(w[f"{p}e{e}.down"]) @ (g * sigmoid(g) * u))
    return out


# ---- the model --------------------------------------------------------------------------

def forward(w, cfg, ids, taps=None):
    """Logits [T, vocab] of a whole sequence; ``taps`` (a list) receives the residual stream
    after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x = f64(w["embed"])[np.asarray(ids, dtype=np.int64)]
    for i, L in enumerate(cfg["layers"]):
        src = L.get("weights_of", i)
        p = f"l{src}."
        hn = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        if L["type"] == "attention":
            x = x + differential_attention(hn, w, p + "mix.", L["mixer"], eps)
        elif L["type"] == "latent_attention":
            x = x + latent_attention(hn, w, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        if L.get("mlp") is not None:
            hn = layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps)
            x = x + experts(hn, w, p + "mlp.", L["mlp"])
        if taps is not None:
            taps.append(x.copy())
    xn = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return xn @ f64(w["head"]).T


# ---- random models for the tests --------------------------------------------------------

def round_bf16(a):
    """Round float values to the nearest bfloat16 (ties to even), returned as float64."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    bits = a.view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).astype(np.float64).reshape(a.shape)


def tensor_shapes(cfg):
    """name -> (shape, kind) of every tensor of a configuration."""
    d, out = cfg["width"], {}
    out["embed"] = ((cfg["vocab"], d), "matrix")
    for i, L in enumerate(cfg["layers"]):
        if "weights_of" in L:
            continue
        p, m = f"l{i}.", L["mixer"]
        for nm in ("norm1",) + (("norm2",) if L.get("mlp") else ()):
            out[p + nm] = ((d,), "gain")
            out[p + nm + ".b"] = ((d,), "bias")
        if L["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out[p + "mix.q"] = ((H * 2 * dk, d), "qk")
            out[p + "mix.k"] = ((G * 2 * dk, d), "qk")
            out[p + "mix.v"] = ((G * dv, d), "matrix")
            out[p + "mix.q.b"], out[p + "mix.k.b"], out[p + "mix.v.b"] = ((H * 2 * dk,), "bias"), ((G * 2 * dk,), "bias"), \
                ((G * dv,), "bias")
            out[p + "mix.q.norm"], out[p + "mix.k.norm"] = ((dk,), "gain"), ((dk,), "gain")
            for nm in ("lq1", "lk1", "lq2", "lk2"):
                out[p + "mix." + nm] = ((dk,), "lambda")
            out[p + "mix.o"] = ((d, H * dv), "matrix")
        else:
            H, dk, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            out[p + "mix.q"] = ((H * (dk + dr), d), "qk")
            out[p + "mix.dkv"] = ((R + dr, d), "qk")
            out[p + "mix.dkv.norm"] = ((R,), "gain")
            out[p + "mix.uk"] = ((H * dk, R), "matrix")
            out[p + "mix.uv"] = ((H * dv, R), "matrix")
            out[p + "mix.g"] = ((H * dv, d), "matrix")
            out[p + "mix.o"] = ((d, H * dv), "matrix")
        if L.get("mlp"):
            f, E = L["mlp"]["expert"]["ff"], L["mlp"]["router"]["experts"]
            out[p + "mlp.router"] = ((E, d), "router")
            for e in range(E):
                out[f"{p}mlp.e{e}.gate"], out[f"{p}mlp.e{e}.up"] = ((f, d), "matrix"), ((f, d), "matrix")
                out[f"{p}mlp.e{e}.down"] = ((d, f), "matrix")
    out["final.norm"], out["final.norm.b"] = ((d,), "gain"), ((d,), "bias")
    out["head"] = ((cfg["vocab"], d), "matrix")
    return out


def random_weights(cfg, seed, std=0.08, qk_boost=2.0):
    """Random tensors, all exactly representable in bfloat16.  Query and key projections are
    scaled up so that attention is far from uniform; router rows are spread so that choices are
    not close calls."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        if kind == "matrix":
            a = rng.normal(0.0, std, size=shape)
        elif kind == "qk":
            a = rng.normal(0.0, std * qk_boost, size=shape)
        elif kind == "router":
            a = rng.normal(0.0, 0.5, size=shape)
        elif kind == "gain":
            a = 1.0 + rng.normal(0.0, 0.1, size=shape)
        elif kind == "bias":
            a = rng.normal(0.0, 0.1, size=shape)
        elif kind == "lambda":
            a = rng.normal(0.0, 0.15, size=shape)
        w[name] = round_bf16(a.astype(np.float32))
    return w
