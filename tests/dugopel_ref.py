"""Plain, slow restatement of the Dugopel design, one function per mechanism, in float64 on the
CPU.  Test oracle only: it shares no code with the library (no paged cache, no absorbed
projections, no batching — a whole sequence at a time, keys and values expanded per head).

Notation: x residual stream [T, W]; h = norm(x); per head q = [q_n (dim) | q_r (rot_dim)];
latent c [T, kv_rank]; k_r [T, rot_dim] shared by the heads.
"""
from __future__ import annotations

import math

import numpy as np

F = np.float64


def layer_norm_noshift(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w with the biased variance; no additive term."""
    x = np.asarray(x, F)
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * np.asarray(w, F)


def rms_norm(x, w, eps):
    x = np.asarray(x, F)
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * np.asarray(w, F)


def rotate_half(v, pos, base, dims):
    """Rotary position code on the first `dims` entries of the last axis: entry i pairs with
    i + dims/2, angle pos * base^(-2i/dims).  v [T, ..., D], pos [T]."""
    v = np.array(v, F)
    half = dims // 2
    i = np.arange(half, dtype=F)
    f = np.asarray(base, F) ** (-2.0 * i / dims)
    a = np.asarray(pos, F)[:, None] * f[None, :]
    shape = (v.shape[0],) + (1,) * (v.ndim - 2) + (half,)
    c, s = np.cos(a).reshape(shape), np.sin(a).reshape(shape)
    u, w = v[..., :half].copy(), v[..., half:dims].copy()
    v[..., :half] = u * c - w * s
    v[..., half:dims] = w * c + u * s
    return v


def softmax(z):
    z = z - z.max(-1, keepdims=True)
    e = np.exp(z)
    return e / e.sum(-1, keepdims=True)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def latent_kv(h, m, wt, pos, eps):
    """What a layer with its own down-projection leaves for itself and its followers:
    (normed latent c [T, kv_rank], rotated shared key part [T, rot_dim])."""
    r = m["kv_rank"]
    d = np.asarray(h, F) @ np.asarray(wt["dkv"], F).T
    c = rms_norm(d[:, :r], wt["dkv.norm"], eps)
    kr = rotate_half(d[:, r:], pos, m["rot"]["base"], m["rot"]["dims"])
    return c, kr


def latent_attention(h, m, wt, pos, eps, c, kr):
    """Causal attention of one whole sequence through the latent (c, kr) of `latent_kv`."""
    H, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    h = np.asarray(h, F)
    T = h.shape[0]
    cq = rms_norm(h @ np.asarray(wt["dq"], F).T, wt["dq.norm"], eps)
    q = (cq @ np.asarray(wt["uq"], F).T).reshape(T, H, dn + dr)
    qn = q[..., :dn]
    qr = rotate_half(q[..., dn:], pos, m["rot"]["base"], m["rot"]["dims"])
    kn = (c @ np.asarray(wt["uk"], F).T).reshape(T, H, dn)
    v = (c @ np.asarray(wt["uv"], F).T).reshape(T, H, dv)
    gate = sigmoid(h @ np.asarray(wt["g"], F).T)  # [T, H]
    out = np.zeros((T, H, dv), F)
    for hd in range(H):
        s = (qn[:, hd] @ kn[:, hd].T + qr[:, hd] @ kr.T) * m["scale"]
        s = np.where(np.tril(np.ones((T, T), bool)), s, -np.inf)
        out[:, hd] = softmax(s) @ v[:, hd]
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ np.asarray(wt["o"], F).T


def clamped_glu(h, gate, up, down, limit):
    """g = min(Wg h, limit), u = clamp(Wu h, +-limit), y = g * sigmoid(1.702 g) * (u + 1)."""
    h = np.asarray(h, F)
    g = np.minimum(h @ np.asarray(gate, F).T, limit)
    u = np.clip(h @ np.asarray(up, F).T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ np.asarray(down, F).T


def route(h, router_w, rc):
    """Group-limited top-k routing.  Returns (experts [T, top], weights [T, top])."""
    E, top = rc["experts"], rc["top"]
    G, keep = rc["groups"]["count"], rc["groups"]["keep"]
    s = softmax(np.asarray(h, F) @ np.asarray(router_w, F).T)
    T = s.shape[0]
    idx = np.zeros((T, top), np.int64)
    wts = np.zeros((T, top), F)
    per = E // G
    for t in range(T):
        gs = s[t].reshape(G, per).max(-1)
        best = np.argsort(-gs, kind="stable")[:keep]
        ok = np.zeros(E, bool)
        for g in best:
            ok[g * per:(g + 1) * per] = True
        cand = np.where(ok, s[t], -np.inf)
        pick = np.argsort(-cand, kind="stable")[:top]
        idx[t] = pick
        wts[t] = s[t, pick] * rc["scale"]
    return idx, wts


def moe(h, mlp, wt):
    idx, wts = route(h, wt["router"], mlp["router"])
    h = np.asarray(h, F)
    out = np.zeros((h.shape[0], np.asarray(wt["e0.down"]).shape[0]), F)
    lim = mlp["expert"]["limit"]
    for t in range(h.shape[0]):
        for e, w in zip(idx[t], wts[t]):
            out[t] += w * clamped_glu(h[t:t + 1], wt[f"e{e}.gate"], wt[f"e{e}.up"], wt[f"e{e}.down"], lim)[0]
    return out


def feed_forward(h, mlp, wt):
    if mlp is None:
        return 0.0
    if mlp["kind"] == "dense":
        return clamped_glu(h, wt["gate"], wt["up"], wt["down"], mlp["limit"])
    return moe(h, mlp, wt)


def softcap(z, cap):
    return cap * np.tanh(z / cap)


def forward(cfg: dict, w: dict, tokens, keep_layers=False):
    """Logits [T, vocab] of one sequence (positions 0..T-1); w maps tensor names to arrays."""
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    pos = np.arange(T)
    x = np.asarray(w["embed"], F)[np.asarray(tokens)] * cfg["embedding"]["scale"]
    latents = {}
    per_layer = []
    for i, lc in enumerate(cfg["layers"]):
        sub = lambda pre: {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)}
        mix, mlp = sub(f"l{i}.mix."), sub(f"l{i}.mlp.")
        m = lc["mixer"]
        h = layer_norm_noshift(x, w[f"l{i}.norm1"], eps)
        if m.get("kv_from") is None:
            latents[i] = latent_kv(h, m, mix, pos, eps)
            c, kr = latents[i]
        else:
            c, kr = latents[m["kv_from"]]
        x = x + (latent_attention(h, m, mix, pos, eps, c, kr) + feed_forward(h, lc["mlp"], mlp))
        per_layer.append(x.copy())
    y = layer_norm_noshift(x, w["final.norm"], eps)
    logits = softcap(y @ np.asarray(w["head"], F).T, cfg["logit_softcap"])
    return (logits, per_layer) if keep_layers else logits
