"""Plain, slow implementation of the Lokolorn decoder in numpy: whole sequences, no cache, one function per
mechanism.  It shares no code with the engine: it reads config.json keys itself and walks tokens and keys with
ordinary loops where the engine has kernels.

A Lokolorn layer is pre-norm with a learned scale per feature on each sublayer's output,

    x <- x + s1 * mixer(N1(x));    x <- x + s2 * ff(N2(x)),      N(x) = x / rms(x) * (1 + w)

The mixer is one of: softmax attention and a decayed linear recurrence side by side on the same input ("parallel");
a delta rule whose state decays per key channel ("channel_delta"); attention over a cached latent with a sliding
window and a sink ("latent_attention").  ff is a routed mixture of small gated feed-forwards (or absent).  A span
of layers may run several times with the same weights; every pass is entered through a product that reads the
stream and the embedding output side by side.

All arithmetic is float64; tensors come as a dict of arrays.
"""

from __future__ import annotations

import math

import numpy as np


def rms_unit(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def offset_norm(x, w, eps):
    return rms_unit(x, eps) * (1.0 + w)


def sigmoid(z):
    return 1 / (1 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0)


def causal_conv(u, taps_w):
    """u [T, C], taps_w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = taps_w.shape[1]
    y = np.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += taps_w[:, j] * u[s]
    return y


def rotate_half_layout(x, positions, dims, base):
    """x [T, heads, d]: dimension i < dims/2 pairs with i + dims/2; angle p * base^(-2i/dims)."""
    out = x.copy()
    half = dims // 2
    for i in range(half):
        a = positions * base ** (-2.0 * i / dims)
        c, s = np.cos(a)[:, None], np.sin(a)[:, None]
        u, v = x[..., i], x[..., i + half]
        out[..., i], out[..., i + half] = u * c - v * s, v * c + u * s
    return out


def scaled_frequencies(dims, base, scaling):
    """Frequencies of the pairs and the factor on cosines and sines, with the ramp between kept and divided ones."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return f, 1.0
    factor, original = scaling["factor"], scaling["original"]

    def where(turns):
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(where(scaling["fast"])), 0)
    hi = min(math.ceil(where(scaling["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_neighbours(x, positions, dims, base, scaling):
    """x [T, ..., d]: dimension 2i pairs with 2i + 1; frequencies possibly scaled; cos and sin times the factor."""
    out = x.copy()
    freq, amp = scaled_frequencies(dims, base, scaling)
    shape = (len(positions),) + (1,) * (x.ndim - 2)
    for i, f in enumerate(freq):
        a = positions * f
        c, s = (np.cos(a) * amp).reshape(shape), (np.sin(a) * amp).reshape(shape)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i], out[..., 2 * i + 1] = u * c - v * s, v * c + u * s
    return out


def softmax_attention(h, w, px, m, eps):
    """The left half of a parallel mixer: biased projections, short convolutions, rotation, unit RMS per head, causal softmax."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T, dtype=np.float64)
    parts = {}
    for name in ("q", "k", "v"):
        u = h @ w[px + name].T + w[px + name + ".b"]
        parts[name] = causal_conv(u, w[px + name + ".conv"])
    q = parts["q"].reshape(T, H, d)
    k = parts["k"].reshape(T, G, d)
    v = parts["v"].reshape(T, G, dv)
    rot = m.get("rot")
    if rot:
        q = rotate_half_layout(q, pos, rot["dims"], rot["base"])
        k = rotate_half_layout(k, pos, rot["dims"], rot["base"])
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    out = np.zeros((T, H, dv))
    for a in range(H):
        g = a // (H // G)
        for t in range(T):
            s = (k[: t + 1, g] @ q[t, a]) * m["scale"]
            p = np.exp(s - s.max())
            out[t, a] = (p / p.sum()) @ v[: t + 1, g]
    return out.reshape(T, H * dv) @ w[px + "o"].T + w[px + "o.b"]


def decayed_recurrence(h, w, px, m, eps):
    """The right half of a parallel mixer: every projection reads its own blend of the token and the one before it;
    per head a matrix state that decays per key channel, and a bonus for the current token only."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    before = np.vstack([np.zeros((1, h.shape[1])), h[:-1]])

    def mix(s):
        return h + (before - h) * w[px + "mu." + s]

    r = (mix("r") @ w[px + "r"].T).reshape(T, H, d)
    k = (mix("k") @ w[px + "k"].T).reshape(T, H, d)
    v = (mix("v") @ w[px + "v"].T).reshape(T, H, d)
    gate = silu(mix("g") @ w[px + "g"].T)
    decay = np.exp(-np.exp(np.tanh(mix("w") @ w[px + "w1"].T) @ w[px + "w2"].T + w[px + "w0"])).reshape(T, H, d)
    bonus = w[px + "u"].reshape(H, d)
    out = np.zeros((T, H, d))
    for a in range(H):
        S = np.zeros((d, d))
        for t in range(T):
            kv = np.outer(k[t, a], v[t, a])
            out[t, a] = (S + bonus[a][:, None] * kv).T @ r[t, a]
            S = decay[t, a][:, None] * S + kv
    y = rms_unit(out, eps).reshape(T, H * d) * w[px + "norm"] * gate
    return y @ w[px + "o"].T


def parallel_mixer(h, w, px, m, eps):
    left = softmax_attention(h, w, px + "left.", m["left"], eps)
    right = decayed_recurrence(h, w, px + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def unit_vector(x):
    return x / np.sqrt((x * x).sum(-1, keepdims=True) + 1e-6)


def channel_delta(h, w, px, m, eps):
    """Delta rule with one decay per head and key channel."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[px + "q"].T, w[px + "q.conv"])).reshape(T, G, d)
    k = silu(causal_conv(h @ w[px + "k"].T, w[px + "k.conv"])).reshape(T, G, d)
    v = silu(causal_conv(h @ w[px + "v"].T, w[px + "v.conv"])).reshape(T, H, dv)
    q, k = unit_vector(q) * d ** -0.5, unit_vector(k)
    beta = sigmoid(h @ w[px + "b"].T)
    step = softplus((h @ w[px + "a1"].T) @ w[px + "a2"].T + w[px + "dt_bias"]).reshape(T, H, d)
    decay = np.exp(-np.exp(w[px + "A_log"])[None, :, None] * step)
    out = np.zeros((T, H, dv))
    for a in range(H):
        g = a // (H // G)
        S = np.zeros((d, dv))
        for t in range(T):
            S = decay[t, a][:, None] * S
            u = beta[t, a] * (v[t, a] - S.T @ k[t, g])
            S = S + np.outer(k[t, g], u)
            out[t, a] = S.T @ q[t, g]
    gate = sigmoid((h @ w[px + "g1"].T) @ w[px + "g2"].T).reshape(T, H, dv)
    y = rms_unit(out, eps) * w[px + "norm"] * gate
    return y.reshape(T, H * dv) @ w[px + "o"].T


def latent_attention(h, w, px, m, eps):
    """Keys and values made from one small vector per token, a rotated key part shared by the heads, a sliding
    window, and a sink in the softmax denominator."""
    T = h.shape[0]
    H, d, dr, dv, rank = m["heads"], m["dim"], m.get("rot_dim", 0), m["vdim"], m["kv_rank"]
    pos = np.arange(T, dtype=np.float64)
    q = (h @ w[px + "q"].T).reshape(T, H, d + dr)
    down = h @ w[px + "dkv"].T
    c = rms_unit(down[:, :rank], eps) * w[px + "dkv.norm"]
    q_plain, q_rot = q[..., :d], q[..., d:]
    k_rot = down[:, rank:]
    if dr:
        rot = m["rot"]
        q_rot = rotate_neighbours(q_rot, pos, rot["dims"], rot["base"], rot.get("scaling"))
        k_rot = rotate_neighbours(k_rot, pos, rot["dims"], rot["base"], rot.get("scaling"))
    keys = (c @ w[px + "uk"].T).reshape(T, H, d)
    values = (c @ w[px + "uv"].T).reshape(T, H, dv)
    size = (m.get("mask") or {}).get("size")
    out = np.zeros((T, H, dv))
    for a in range(H):
        for t in range(T):
            first = 0 if size is None else max(0, t - size + 1)
            s = (keys[first : t + 1, a] @ q_plain[t, a] + k_rot[first : t + 1] @ q_rot[t, a]) * m["scale"]
            sink = w[px + "sink"][a] if px + "sink" in w else -np.inf
            top = max(s.max(), sink)
            p = np.exp(s - top)
            out[t, a] = (p / (p.sum() + np.exp(sink - top))) @ values[first : t + 1, a]
    return out.reshape(T, H * dv) @ w[px + "o"].T


def route(h, w, px, r):
    """Which experts a token uses and with what weights: [T, top] indices and weights."""
    s = sigmoid(h @ w[px + "router"].T)
    choice = s + w[px + "correction"]
    T, E = s.shape
    groups = r.get("groups")
    ids = np.zeros((T, r["top"]), dtype=np.int64)
    weights = np.zeros((T, r["top"]))
    for t in range(T):
        allowed = np.ones(E, dtype=bool)
        if groups:
            per = E // groups["count"]
            score = [np.sort(choice[t, g * per : (g + 1) * per])[-2:].sum() for g in range(groups["count"])]
            best = np.argsort(-np.asarray(score), kind="stable")[: groups["keep"]]
            allowed[:] = False
            for g in best:
                allowed[g * per : (g + 1) * per] = True
        c = np.where(allowed, choice[t], -np.inf)
        ids[t] = np.argsort(-c, kind="stable")[: r["top"]]
        picked = s[t, ids[t]]
        weights[t] = picked / (picked.sum() + 1e-20) * r["scale"]
    return ids, weights


def expert(h, w, px):
    return (silu(h @ w[px + "gate"].T) * (h @ w[px + "up"].T)) @ w[px + "down"].T


def routed_feed_forward(h, w, px, mlp):
    ids, weights = route(h, w, px, mlp["router"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(ids[t], weights[t]):
            out[t] += g * expert(h[t : t + 1], w, f"{px}e{e}.")[0]
    return out


MIXERS = {"parallel": parallel_mixer, "channel_delta": channel_delta, "latent_attention": latent_attention}


def layer_runs(cfg):
    """(layer, pass entered here or None) in the order the layers run."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def layer(x, w, cfg, i, only_mixer=False):
    eps = cfg["norm"]["eps"]
    entry, p = cfg["layers"][i], f"l{i}."
    x = x + w[p + "ls1"] * MIXERS[entry["type"]](offset_norm(x, w[p + "norm1"], eps), w, p + "mix.", entry["mixer"], eps)
    if entry.get("mlp") is not None and not only_mixer:
        x = x + w[p + "ls2"] * routed_feed_forward(offset_norm(x, w[p + "norm2"], eps), w, p + "mlp.", entry["mlp"])
    return x


def forward(cfg, w, tokens, trace=None):
    """Logits [T, vocab] of one sequence; ``trace`` (a list) collects the stream after every layer run."""
    w = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    x0 = w["embed"][np.asarray(tokens)]
    x = x0
    for i, entered in layer_runs(cfg):
        if entered is not None:
            x = np.concatenate([x, x0], -1) @ w["loop.in"].T
        x = layer(x, w, cfg, i)
        if trace is not None:
            trace.append(x.copy())
    return offset_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["head"].T


def greedy(cfg, w, prompt, new_tokens):
    tokens = list(prompt)
    for _ in range(new_tokens):
        tokens.append(int(np.argmax(forward(cfg, w, tokens)[-1])))
    return tokens[len(prompt):]
