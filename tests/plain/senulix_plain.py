"""Plain, slow Senulix forward pass in numpy float64: the yardstick of its tests.

Whole sequences, no cache, no paging, no batches; one function per mechanism.
Nothing here is imported by the product package and nothing of the product
package is imported here.  Weights arrive as a dict of tensor name -> numpy
array and are widened to float64; ``cfg`` is the dict of a config.json.

Notation: T tokens, d the model width, H query heads, G key/value heads, dk the per-head
query/key size, dv the per-head value size, R the size of the key/value latent, dr the
rotated size of a latent layer, W the width of a window, P the per-layer size of the token
side table.
"""
from __future__ import annotations

import math

import numpy as np


def f64(a):
    return np.asarray(a, dtype=np.float64)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


_erf = np.vectorize(math.erf, otypes=[np.float64])


def gelu_erf(z):
    return 0.5 * z * (1.0 + _erf(z / math.sqrt(2.0)))


def unit_rms(x, eps):
    x = f64(x)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def norm_plain(x, w, eps):
    """x / rms(x) * w."""
    return unit_rms(x, eps) * f64(w)


def norm_one_plus(x, w, eps):
    """x / rms(x) * (1 + w): the weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + f64(w))


# ---- rotation ---------------------------------------------------------------------------

def rotate(x, positions, dims, base):
    """x [T, heads, size]: the first ``dims`` values of every head are turned, value i paired with
    value i + dims / 2, by the angle position * base^(-2 i / dims); the rest stays."""
    x = f64(x).copy()
    half = dims // 2
    f = base ** (-2.0 * np.arange(half, dtype=np.float64) / dims)
    a = f64(positions)[:, None, None] * f[None, None, :]
    u, v = x[..., :half].copy(), x[..., half:dims].copy()
    x[..., :half] = u * np.cos(a) - v * np.sin(a)
    x[..., half:dims] = v * np.cos(a) + u * np.sin(a)
    return x


# ---- mixers -----------------------------------------------------------------------------

def decayed_state_scan(q, k, v, decay, state=None):
    """q, k [T, H, dk], v [T, H, dv], decay [H]: S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, token by token.
    Returns (o [T, H, dv], the last state [H, dk, dv])."""
    T, H, dk = q.shape
    dv = v.shape[2]
    S = np.zeros((H, dk, dv)) if state is None else f64(state).copy()
    o = np.zeros((T, H, dv))
    for t in range(T):
        for hd in range(H):
            S[hd] = float(decay[hd]) * S[hd] + np.outer(k[t, hd], v[t, hd])
            o[t, hd] = S[hd].T @ q[t, hd]
    return o, S


def lightning_mixer(h, w, p, m, eps):
    """Linear attention with one fixed decay per head, one norm over all heads' outputs, a sigmoid gate."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ f64(w[p + ".q"]).T).reshape(T, H, dk)
    k = silu(h @ f64(w[p + ".k"]).T).reshape(T, H, dk)
    v = silu(h @ f64(w[p + ".v"]).T).reshape(T, H, dv)
    o, _ = decayed_state_scan(q, k, v, m["decay"])
    y = norm_plain(o.reshape(T, H * dv), w[p + ".norm"], eps) * sigmoid(h @ f64(w[p + ".g"]).T)
    return y @ f64(w[p + ".o"]).T


def latent_kv(h, w, p, m, eps, positions):
    """(latent c [T, R], rotated shared key part [T, dr]) of a latent layer that owns its down-projection."""
    R, dr = m["kv_rank"], m["rot_dim"]
    down = h @ f64(w[p + ".dkv"]).T
    c = norm_plain(down[:, :R], w[p + ".dkv.norm"], eps)
    kr = rotate(down[:, None, R:], positions, m["rot"]["dims"], m["rot"]["base"])[:, 0]
    return c, kr


def latent_mixer(h, w, p, m, eps, positions, kv):
    """Attention through a latent: kv = (c, kr) is this layer's own or another layer's."""
    T = h.shape[0]
    H, dk, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    c, kr = kv
    q = (h @ f64(w[p + ".q"]).T).reshape(T, H, dk + dr)
    q_plain = q[..., :dk]
    q_rot = rotate(q[..., dk:], positions, m["rot"]["dims"], m["rot"]["base"])
    k_plain = (c @ f64(w[p + ".uk"]).T).reshape(T, H, dk)
    val = (c @ f64(w[p + ".uv"]).T).reshape(T, H, dv)
    out = np.zeros((T, H, dv))
    for hd in range(H):
        for i in range(T):
            s = (k_plain[:i + 1, hd] @ q_plain[i, hd] + kr[:i + 1] @ q_rot[i, hd]) * m["scale"]
            e = np.exp(s - s.max())
            out[i, hd] = (e / e.sum()) @ val[:i + 1, hd]
    return out.reshape(T, H * dv) @ f64(w[p + ".o"]).T


def mixed_window_attention(q, k, v, talk, scale, size, positions=None, sink=True):
    """q [T, H, dk] at ``positions`` (default 0 .. T-1) over keys k [S, G, dk] and values v [S, G, dv] at positions
    0 .. S-1: the heads' scaled scores are mixed by ``talk`` [H, H], a query at p sees the keys j with
    0 <= p - j < size (size None: every j <= p), and a sink of score 0 joins the softmax's denominator."""
    q, k, v = f64(q), f64(k), f64(v)
    T, H, _ = q.shape
    G, dv = k.shape[1], v.shape[2]
    per = H // G
    positions = np.arange(T) if positions is None else np.asarray(positions)
    raw = np.stack([q[:, hd] @ k[:, hd // per].T for hd in range(H)]) * scale             # [H, T, S]
    mixed = np.einsum("hg,gij->hij", f64(talk), raw)
    out = np.zeros((T, H, dv))
    for i, p in enumerate(positions):
        lo = 0 if size is None else max(0, p - size + 1)
        for hd in range(H):
            s = mixed[hd, i, lo:p + 1]
            top = max(s.max(), 0.0) if sink else s.max()
            e = np.exp(s - top)
            out[i, hd] = (e / ((np.exp(-top) if sink else 0.0) + e.sum())) @ v[lo:p + 1, hd // per]
    return out


def normed_rotated_qk(qp, kp, q_gain, k_gain, eps, H, G, dk, positions, rot):
    """RMS norm over each WHOLE projection (all heads at once, plain gains), then the rotation of every head."""
    T = qp.shape[0]
    q = norm_plain(qp, q_gain, eps).reshape(T, H, dk)
    k = norm_plain(kp, k_gain, eps).reshape(T, G, dk)
    if rot:
        q, k = rotate(q, positions, rot["dims"], rot["base"]), rotate(k, positions, rot["dims"], rot["base"])
    return q, k


def window_attention_mixer(h, w, p, m, eps, positions):
    """Grouped attention with norms over the whole q and k projections, a partial rotation, scores
    mixed across the heads, a window and a sink of score 0."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k = normed_rotated_qk(h @ f64(w[p + ".q"]).T, h @ f64(w[p + ".k"]).T, w[p + ".q.norm"], w[p + ".k.norm"], eps,
                             H, G, dk, positions, m.get("rot"))
    v = (h @ f64(w[p + ".v"]).T).reshape(T, G, dv)
    size = m["mask"]["size"] if m.get("mask") else None
    out = mixed_window_attention(q, k, v, w[p + ".talk"], m["scale"], size)
    return out.reshape(T, H * dv) @ f64(w[p + ".o"]).T


# ---- the rest of a layer ----------------------------------------------------------------

def dense_ff(h, w, p):
    return gelu_erf(h @ f64(w[p + ".up"]).T) @ f64(w[p + ".down"]).T


def token_side(x, w, layer, ids, P, eps):
    """What the layer adds from the token's own row of the side table."""
    p = f"l{layer}.side"
    e = f64(w["side.embed"])[np.asarray(ids), layer * P:(layer + 1) * P]
    y = (gelu_tanh(x @ f64(w[p + ".gate"]).T) * e) @ f64(w[p + ".proj"]).T
    return norm_plain(y, w[p + ".norm"], eps)


def forward(w, cfg, ids, return_layers=False):
    """Logits float64 [T, vocab] for the token ids of one sequence, positions 0 .. T-1."""
    ids = np.asarray(ids, dtype=np.int64)
    eps = float(cfg["norm"]["eps"])
    positions = np.arange(len(ids))
    x = f64(w["embed"])[ids]
    kept, layers = {}, []
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix", L["mixer"]
        if L["type"] == "lightning":
            y = lightning_mixer(x, w, p, m, eps)
        elif L["type"] == "latent_attention":
            if m.get("kv_from") is None:
                kept[i] = latent_kv(x, w, p, m, eps, positions)
            y = latent_mixer(x, w, p, m, eps, positions, kept[i if m.get("kv_from") is None else m["kv_from"]])
        elif L["type"] == "attention":
            y = window_attention_mixer(x, w, p, m, eps, positions)
        else:
            raise ValueError(L["type"])
        x = x + norm_one_plus(y, w[f"l{i}.norm1"], eps)
        if L.get("mlp") is not None:
            x = x + norm_one_plus(dense_ff(x, w, f"l{i}.mlp"), w[f"l{i}.norm2"], eps)
        if cfg.get("token_side"):
            x = x + token_side(x, w, i, ids, int(cfg["token_side"]["dim"]), eps)
        layers.append(x.copy())
    z = norm_one_plus(x, w["final.norm"], eps) @ f64(w["head"]).T
    cap = cfg.get("logit_softcap")
    if cap:
        z = float(cap) * np.tanh(z / float(cap))
    return (z, np.stack(layers)) if return_layers else z


# ---- random models ----------------------------------------------------------------------

def tensor_shapes(cfg):
    d, V = cfg["width"], cfg["vocab"]
    P = int(cfg["token_side"]["dim"]) if cfg.get("token_side") else 0
    out = {"embed": (V, d), "final.norm": (d,), "head": (V, d)}
    if P:
        out["side.embed"] = (V, P * len(cfg["layers"]))
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}", L["mixer"]
        out[p + ".norm1"] = (d,)
        if L["type"] == "lightning":
            A, B = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            out.update({p + ".mix.q": (A, d), p + ".mix.k": (A, d), p + ".mix.v": (B, d), p + ".mix.g": (B, d),
                        p + ".mix.norm": (B,), p + ".mix.o": (d, B)})
        elif L["type"] == "latent_attention":
            H = m["heads"]
            out.update({p + ".mix.q": (H * (m["dim"] + m["rot_dim"]), d), p + ".mix.uk": (H * m["dim"], m["kv_rank"]),
                        p + ".mix.uv": (H * m["vdim"], m["kv_rank"]), p + ".mix.o": (d, H * m["vdim"])})
            if m.get("kv_from") is None:
                out.update({p + ".mix.dkv": (m["kv_rank"] + m["rot_dim"], d), p + ".mix.dkv.norm": (m["kv_rank"],)})
        else:
            H, G = m["heads"], m["kv_heads"]
            out.update({p + ".mix.q": (H * m["dim"], d), p + ".mix.k": (G * m["dim"], d), p + ".mix.v": (G * m["vdim"], d),
                        p + ".mix.q.norm": (H * m["dim"],), p + ".mix.k.norm": (G * m["dim"],), p + ".mix.talk": (H, H),
                        p + ".mix.o": (d, H * m["vdim"])})
        if L.get("mlp") is not None:
            out.update({p + ".norm2": (d,), p + ".mlp.up": (L["mlp"]["ff"], d), p + ".mlp.down": (d, L["mlp"]["ff"])})
        if P:
            out.update({p + ".side.gate": (P, d), p + ".side.proj": (d, P), p + ".side.norm": (d,)})
    return out


def random_weights(cfg, seed, std=0.08, qk_boost=1.0):
    """Weights that make every mechanism count, all of them bfloat16 numbers (both dtypes load the same model):
    matrices N(0, std) scaled by 1 / sqrt(fan-in / 64), one-plus weights around zero, plain weights around one,
    a head-mixing matrix near the identity with sizeable off-diagonal terms; ``qk_boost`` scales the attention
    layers' query and key projections, which sharpens the attention."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith(".talk"):
            t = np.eye(shape[0]) + 0.3 * rng.standard_normal(shape)
        elif name.endswith((".norm1", ".norm2")) or name == "final.norm":
            t = 0.2 * rng.standard_normal(shape)
        elif len(shape) == 1:
            t = 1.0 + 0.2 * rng.standard_normal(shape)
        elif name in ("embed", "side.embed"):
            t = rng.standard_normal(shape)
        else:
            t = rng.standard_normal(shape) * std * math.sqrt(64.0 / shape[1]) * 1.5
            if name.endswith((".mix.q", ".mix.k", ".mix.dkv")):
                t = t * qk_boost
        w[name] = round_bf16(t.astype(np.float32))
    return w


def round_bf16(a):
    """float32 array rounded to the nearest bfloat16 (ties to even), as float32."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).reshape(np.shape(a))
