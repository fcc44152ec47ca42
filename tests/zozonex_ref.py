"""Plain float64 restatement of the Zozonex design, one function per mechanism, for the tests.
Nothing here is shared with the product path: numpy only, whole sequences at once, no cache.

Notation: x [T, W] the residual stream of one sequence, tokens at positions 0 .. T-1;
a linear map with weight M [out, in] is x @ M.T."""
import numpy as np


def rms_div(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose weight is stored around zero."""
    return rms_div(x, eps) * (1.0 + w)


def silu(x):
    return x / (1.0 + np.exp(-x))


def softplus(x):
    return np.logaddexp(0.0, x)


def embed_positions(tokens, table, scale):
    """Scaled embedding plus interleaved sinusoids: entry 2i sin, entry 2i + 1 cos of p * 10000^(-2i / W)."""
    T, W = len(tokens), table.shape[1]
    x = table[np.asarray(tokens)] * scale
    p = np.arange(T, dtype=np.float64)[:, None]
    f = 10000.0 ** (-2.0 * np.arange(W // 2, dtype=np.float64) / W)[None, :]
    x = x.copy()
    x[:, 0::2] += np.sin(p * f)
    x[:, 1::2] += np.cos(p * f)
    return x


def short_conv(u, taps_w):
    """Causal convolution over time per channel; taps_w [C, taps], the last column multiplies the
    current token, zeros before the start.  Then SiLU."""
    T, C = u.shape
    taps = taps_w.shape[1]
    out = np.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1 - j)
            if src >= 0:
                out[t] += u[src] * taps_w[:, j]
    return silu(out)


def delta_rule(q, k, v, beta, g):
    """One head.  q, k [T, dim], v [T, vdim], beta, g [T].  State S [dim, vdim] from zero:
    S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, dim = q.shape
    S = np.zeros((dim, v.shape[1]))
    o = np.zeros_like(v)
    for t in range(T):
        S = g[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        o[t] = S.T @ q[t]
    return o


def delta_mixer(h, w, pre, m, eps):
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = short_conv(h @ w[pre + "q"].T, w[pre + "q.conv"]).reshape(T, G, dim)
    k = short_conv(h @ w[pre + "k"].T, w[pre + "k.conv"]).reshape(T, G, dim)
    v = short_conv(h @ w[pre + "v"].T, w[pre + "v.conv"]).reshape(T, H, vdim)
    q = q / np.sqrt(np.sum(q * q, -1, keepdims=True) + 1e-6) / np.sqrt(dim)
    k = k / np.sqrt(np.sum(k * k, -1, keepdims=True) + 1e-6)
    beta = 1.0 / (1.0 + np.exp(-(h @ w[pre + "b"].T)))
    g = np.exp(-np.exp(w[pre + "A_log"]) * softplus(h @ w[pre + "a"].T + w[pre + "dt_bias"]))
    gate = silu(h @ w[pre + "g"].T).reshape(T, H, vdim)
    o = np.zeros((T, H, vdim))
    for hh in range(H):
        kh = hh // (H // G)
        o[:, hh] = delta_rule(q[:, kh], k[:, kh], v[:, hh], beta[:, hh], g[:, hh])
    o = rms_div(o, eps) * w[pre + "norm"] * gate
    return o.reshape(T, H * vdim) @ w[pre + "o"].T


def window_attention(q, k, v, scale, window):
    """One head.  q, k [T, dim], v [T, vdim]; i sees j with 0 <= i - j < window; the softmax has a
    sink of score 0 that carries no value."""
    T = q.shape[0]
    o = np.zeros((T, v.shape[1]))
    for i in range(T):
        j0 = max(0, i - window + 1)
        s = (k[j0:i + 1] @ q[i]) * scale
        mx = max(s.max(), 0.0)
        e = np.exp(s - mx)
        o[i] = (e / (np.exp(-mx) + e.sum())) @ v[j0:i + 1]
    return o


def attention_mixer(h, w, pre, m, eps, kv_store, layer):
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rms_div((h @ w[pre + "q"].T).reshape(T, H, dim), eps)
    if m.get("kv_from") is not None:
        k, v = kv_store[m["kv_from"]]
    else:
        k = rms_div((h @ w[pre + "k"].T).reshape(T, G, dim), eps)
        v = (h @ w[pre + "v"].T).reshape(T, G, vdim)
        kv_store[layer] = (k, v)
    o = np.zeros((T, H, vdim))
    for hh in range(H):
        kh = hh // (H // G)
        o[:, hh] = window_attention(q[:, hh], k[:, kh], v[:, kh], m["scale"], m["mask"]["size"])
    return o.reshape(T, H * vdim) @ w[pre + "o"].T


def relu2_ffn(h, up, down):
    a = np.maximum(h @ up.T, 0.0)
    return (a * a) @ down.T


def forward(cfg, w, tokens, residuals=None):
    """Logits [T, vocab] of one sequence (float64).  cfg: the config.json dictionary; w: name -> array."""
    w = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = embed_positions(tokens, w["embed"], cfg["embedding"]["scale"])
    kv_store = {}
    for i, lc in enumerate(cfg["layers"]):
        pre = f"l{i}.mix."
        if lc["type"] == "delta":
            y = delta_mixer(x, w, pre, lc["mixer"], eps)
        else:
            y = attention_mixer(x, w, pre, lc["mixer"], eps, kv_store, i)
        x = x + offset_norm(y, w[f"l{i}.norm1"], eps)
        if lc["mlp"] is not None:
            x = x + offset_norm(relu2_ffn(x, w[f"l{i}.mlp.up"], w[f"l{i}.mlp.down"]), w[f"l{i}.norm2"], eps)
        if residuals is not None:
            residuals.append(x.copy())
    return offset_norm(x, w["final.norm"], eps) @ w["embed"].T


def greedy(cfg, w, prompt, steps):
    toks = list(prompt)
    out = []
    for _ in range(steps):
        t = int(np.argmax(forward(cfg, w, toks)[-1]))
        out.append(t)
        toks.append(t)
    return out
