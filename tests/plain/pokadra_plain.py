"""A plain, slow restatement of the Pokadra decoder in numpy (float64), one function per mechanism, written from the
equations and sharing nothing with the engine.  A whole sequence at a time, no cache, no batches.

Notation: T tokens, width W; a linear layer with weight M [out, in] maps x to x M^T.
"""

from __future__ import annotations

import math

import numpy as np


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def gelu_tanh(x):
    return 0.5 * x * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x**3)))


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def group_norm(x, weight, groups, eps):
    """The last axis in ``groups`` equal consecutive parts, each divided by its own root mean square; then the weight."""
    parts = x.reshape(*x.shape[:-1], groups, x.shape[-1] // groups)
    return rms_unit(parts, eps).reshape(x.shape) * weight


def embed(cfg, w, tokens):
    """Token rows times a factor, plus the hashed pair rows (a sequence's first token: the pair table's last row)."""
    tokens = np.asarray(tokens, dtype=np.int64)
    x = w["embed"][tokens] * cfg.get("embedding", {}).get("scale", 1.0)
    pair = cfg.get("embedding", {}).get("bigram")
    if pair:
        rows = np.empty(len(tokens), dtype=np.int64)
        rows[0] = pair["buckets"]
        rows[1:] = (tokens[:-1] * pair["mul_prev"] + tokens[1:] * pair["mul_cur"]) % pair["buckets"]
        x = x + w["bigram"][rows]
    return x


def rotary_frequencies(rot):
    """(frequencies [dims / 2], factor on cos and sin) with the YaRN correction when ``scaling`` is given."""
    dims, base = rot["dims"], rot["base"]
    freq = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if not sc:
        return freq, 1.0
    pair_of = lambda turns: dims * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(base))
    lo, hi = max(math.floor(pair_of(sc["fast"])), 0), min(math.ceil(pair_of(sc["slow"])), dims - 1)
    ramp = np.clip((np.arange(dims // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return freq / sc["factor"] * ramp + freq * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate_pairs(x, rot, positions):
    """x [T, ..., D]: dimensions (2i, 2i + 1), 2i < rot.dims, turned by the angle position * f_i."""
    if not rot or not rot["dims"]:
        return x
    freq, amp = rotary_frequencies(rot)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (len(freq),)
    c, s = (np.cos(ang) * amp).reshape(shape), (np.sin(ang) * amp).reshape(shape)
    out = x.copy()
    d = rot["dims"]
    even, odd = x[..., 0:d:2], x[..., 1:d:2]
    out[..., 0:d:2] = even * c - odd * s
    out[..., 1:d:2] = odd * c + even * s
    return out


def visible(T, mask):
    """[T, T] bool: query i sees key j."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    ok = j <= i
    if mask:
        ok &= (i - j < mask["size"]) | (j < mask.get("keep_first", 0))
    return ok


def diff_lambda(w, p, m):
    return math.exp(float(np.sum(w[p + "lq1"] * w[p + "lk1"]))) - math.exp(float(np.sum(w[p + "lq2"] * w[p + "lk2"]))) + m["diff"]


def attention_keys_values(w, p, m, x, eps):
    """The keys (normed, rotated) [T, G, 2, d] and values [T, G, dv] that a layer with projections of its own caches."""
    T, G, d = x.shape[0], m["kv_heads"], m["dim"]
    k = rms_unit((x @ w[p + "k"].T).reshape(T, G, 2, d), eps) * w[p + "k.norm"]
    return rotate_pairs(k, m.get("rot"), np.arange(T)), (x @ w[p + "v"].T).reshape(T, G, m["vdim"])


def diff_attention(w, p, m, x, eps, keys_values=None):
    """Differential attention of layer prefix p on x [T, W]; ``keys_values``: another layer's, for a layer without its own."""
    T, H, G, d, dv = x.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_unit((x @ w[p + "q"].T).reshape(T, H, 2, d), eps) * w[p + "q.norm"]
    q = rotate_pairs(q, m.get("rot"), np.arange(T))
    k, v = keys_values if keys_values is not None else attention_keys_values(w, p, m, x, eps)
    see = visible(T, m.get("mask"))
    lam = diff_lambda(w, p, m)
    heads = np.empty((T, H, dv))
    for a in range(H):
        g = a // (H // G)
        maps = []
        for which in range(2):
            s = np.where(see, (q[:, a, which] @ k[:, g, which].T) * m["scale"], -np.inf)
            e = np.exp(s - s.max(axis=1, keepdims=True))
            maps.append((e / e.sum(axis=1, keepdims=True)) @ v[:, g])
        heads[:, a] = rms_unit(maps[0] - lam * maps[1], eps) * (1.0 - m["diff"])
    heads *= sigmoid(x @ w[p + "g"].T)[:, :, None]
    return heads.reshape(T, H * dv) @ w[p + "o"].T


def mingru(w, p, m, x, state=None):
    """The recurrence on x [T, W]; returns (output, last state)."""
    z = sigmoid(x @ w[p + "z"].T + w[p + "z.b"])
    u = x @ w[p + "x"].T + w[p + "x.b"]
    cand = np.where(u >= 0, u + 0.5, sigmoid(u))
    s = np.zeros(m["width"]) if state is None else state
    states = np.empty((x.shape[0], m["width"]))
    for t in range(x.shape[0]):
        s = (1.0 - z[t]) * s + z[t] * cand[t]
        states[t] = s
    g = x @ w[p + "g"].T
    return (states * (g * sigmoid(g))) @ w[p + "o"].T, s


def feed_forward(w, p, m, x):
    lim = m["limit"]
    g = np.minimum(x @ w[p + "gate"].T, lim)
    u = np.clip(x @ w[p + "up"].T, -lim, lim)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def token_side(cfg, w, i, x, tokens, eps):
    """What layer i adds from the tokens themselves (before the factor m)."""
    dim = cfg["token_side"]["dim"]
    e = w["side.embed"][np.asarray(tokens, dtype=np.int64)][:, i * dim : (i + 1) * dim]
    y = (gelu_tanh(x @ w[f"l{i}.side.gate"].T) * e) @ w[f"l{i}.side.proj"].T
    return rms_unit(y, eps) * w[f"l{i}.side.norm"]


def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence.  ``layers_out``: a list that receives the stream behind every layer."""
    eps, groups, m = cfg["norm"]["eps"], cfg["norm"].get("groups", 1), cfg.get("residual_mult", 1.0)
    x = embed(cfg, w, tokens)
    results = [x]
    cached = {}
    for i, layer in enumerate(cfg["layers"]):
        p, mix = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "attention":
            if mix.get("kv_from") is None:
                cached[i] = attention_keys_values(w, p, mix, x, eps)
            a = diff_attention(w, p, mix, x, eps, cached[i if mix.get("kv_from") is None else mix["kv_from"]])
        else:
            a, _ = mingru(w, p, mix, x)
        x = x + m * group_norm(a, w[f"l{i}.norm1"], groups, eps)
        if layer.get("mlp"):
            x = x + m * group_norm(feed_forward(w, f"l{i}.mlp.", layer["mlp"], x), w[f"l{i}.norm2"], groups, eps)
        if cfg.get("token_side"):
            x = x + m * token_side(cfg, w, i, x, tokens, eps)
        results.append(x)
        x = sum(w[f"l{i}.dwa"][j] * results[j] for j in range(i + 2))
        if layers_out is not None:
            layers_out.append(x)
    return group_norm(x, w["final.norm"], groups, eps) @ w["head"].T
