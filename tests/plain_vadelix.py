"""A plain, slow Vadelix in float64 numpy: the oracle of the Vadelix tests.

One function per mechanism, whole sequences, no cache, no batching, nothing shared
with the package.  ``cfg`` is the dictionary of a config.json, ``W`` maps tensor
names to float64 arrays.  Notation: X [T, width] the residual stream of one
sequence, t the position (from 0), m the residual multiplier, N the grouped RMS
norm, C the short causal convolution in front of every mixer.

    layer:   h = N1(X);  h <- h + C(h);  X += m mix(h);  X += m ff(N2(X))
    N(x)   = per group g of the `groups` equal consecutive parts: x_g / sqrt(mean(x_g^2) + eps), all times w
    C(h)_t = sum_j taps[:, j] * h_{t - K + 1 + j}      (K taps, zeros before the sequence)
    logits = head N(X)
"""

from __future__ import annotations

import math

import numpy as np


def unit_rms(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def grouped_norm(x, w, eps, groups):
    T, n = x.shape
    return unit_rms(x.reshape(T, groups, n // groups), eps).reshape(T, n) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    return 0.5 * z * (1.0 + np.vectorize(math.erf)(z / math.sqrt(2.0)))


def short_conv(h, taps):
    """C(h): taps [channels, K]; the last tap meets the current token."""
    T, K = h.shape[0], taps.shape[1]
    y = np.zeros_like(h)
    for j in range(K):
        lag = K - 1 - j
        if lag < T:
            y[lag:] += h[:T - lag] * taps[:, j]
    return y


def previous(h):
    """Each token's predecessor's row, zeros for the first."""
    return np.concatenate([np.zeros_like(h[:1]), h[:-1]], axis=0)


def rotary_frequencies(rot):
    """Angular step of each of the dims/2 pairs, and the factor on cos and sin (YaRN where ``scaling`` is given)."""
    dims, base = rot["dims"], float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    s, L = float(sc["factor"]), float(sc["original"])
    c = lambda r: dims * math.log(L / (2.0 * math.pi * r)) / (2.0 * math.log(base))
    lo = max(math.floor(c(float(sc["fast"]))), 0)
    hi = min(math.ceil(c(float(sc["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / s * ramp + f * (1.0 - ramp), 0.1 * math.log(s) + 1.0


def rotate(x, rot, positions):
    """x [T, heads, dim]: element i of the first rot.dims of every head is paired with element i + dims/2."""
    dims = rot["dims"]
    f, mag = rotary_frequencies(rot)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    cos, sin = np.cos(ang)[:, None, :] * mag, np.sin(ang)[:, None, :] * mag
    a, b = x[..., :dims // 2], x[..., dims // 2:dims]
    out = x.copy()
    out[..., :dims // 2] = a * cos - b * sin
    out[..., dims // 2:dims] = b * cos + a * sin
    return out


def mixed_values(v, W, p, c, shared):
    """Value mixing between the layers that ask for it: the first such layer publishes its values, every later one
    blends its own with them by its own number ``vmix``."""
    if not c.get("v_mix"):
        return v
    if "v_first" not in shared:
        shared["v_first"] = v
        return v
    lam = float(W[p + "vmix"])
    return (1.0 - lam) * v + lam * shared["v_first"]


def sink_softmax_sum(s, js, sink, values):
    """sum_j p_j values_j with p_j = exp(s_j) / (exp(sink) + sum_j exp(s_j)): the sink takes weight and gives nothing."""
    top = max(s[js].max(), sink)
    w = np.exp(s[js] - top)
    return (w / (w.sum() + math.exp(sink - top))) @ values[js]


def attention(h, W, p, c, eps, shared):
    """Mixer 'attention': RMS norm of the whole q and of the whole k projection, partial rotary positions, every value
    head to unit RMS, causal softmax with a learned sink per head."""
    T = h.shape[0]
    H, G, D, DV = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = unit_rms(h @ W[p + "q"].T, eps) * W[p + "q.norm"]
    k = unit_rms(h @ W[p + "k"].T, eps) * W[p + "k.norm"]
    pos = np.arange(T)
    q, k = rotate(q.reshape(T, H, D), c["rot"], pos), rotate(k.reshape(T, G, D), c["rot"], pos)
    v = unit_rms((h @ W[p + "v"].T).reshape(T, G, DV), eps)
    v = mixed_values(v, W, p, c, shared)
    out = np.zeros((T, H, DV))
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * float(c["scale"])
        for i in range(T):
            out[i, a] = sink_softmax_sum(s[i], list(range(i + 1)), float(W[p + "sink"][a]), v[:, g])
    return out.reshape(T, H * DV) @ W[p + "o"].T


def window_attention(h, W, p, c, shared):
    """Mixer 'attention_2': no rotation; queries grow with ln of their position's block; a bias falls linearly with the
    distance, at a slope of the head's own; a sliding window; a sink of score 0."""
    T = h.shape[0]
    H, G, D, DV = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    pos = np.arange(T)
    temp = 1.0 + float(c["q_temp"]["coef"]) * np.log(np.floor((pos + 1) / int(c["q_temp"]["every"])) + 1.0)
    q = (h @ W[p + "q"].T).reshape(T, H, D) * temp[:, None, None]
    k = (h @ W[p + "k"].T).reshape(T, G, D)
    v = mixed_values((h @ W[p + "v"].T).reshape(T, G, DV), W, p, c, shared)
    size = int(c["mask"]["size"])
    out = np.zeros((T, H, DV))
    for a in range(H):
        g = a // (H // G)
        slope = 2.0 ** (-8.0 * (a + 1) / H)
        s = (q[:, a] @ k[:, g].T) * float(c["scale"]) - slope * (pos[:, None] - pos[None, :])
        for i in range(T):
            out[i, a] = sink_softmax_sum(s[i], list(range(max(0, i - size + 1), i + 1)), 0.0, v[:, g])
    return out.reshape(T, H * DV) @ W[p + "o"].T


def wkv(h, W, p, c, eps):
    """Mixer 'wkv': r, k, v, g, w each read h + (h_prev - h) mu of their own; decay per head and key channel
    w = exp(-exp(W2 tanh(W1 x_w) + w0)); per head o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t, S_t = diag(w_t) S_{t-1} +
    k_t v_t^T; each head's o to unit RMS, times a weight, times silu of the gate, then the output projection."""
    T = h.shape[0]
    H, D = c["heads"], c["dim"]
    d = previous(h) - h
    x = {s: h + d * W[p + "mu." + s] for s in "rkvgw"}
    r = (x["r"] @ W[p + "r"].T).reshape(T, H, D)
    k = (x["k"] @ W[p + "k"].T).reshape(T, H, D)
    v = (x["v"] @ W[p + "v"].T).reshape(T, H, D)
    gate = silu(x["g"] @ W[p + "g"].T)
    w = np.exp(-np.exp(np.tanh(x["w"] @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"])).reshape(T, H, D)
    o = np.zeros((T, H, D))
    for a in range(H):
        S = np.zeros((D, D))
        for t in range(T):
            kv = np.outer(k[t, a], v[t, a])
            o[t, a] = (S + W[p + "u"][a][:, None] * kv).T @ r[t, a]
            S = w[t, a][:, None] * S + kv
    o = unit_rms(o, eps).reshape(T, H * D) * W[p + "norm"]
    return (o * gate) @ W[p + "o"].T


def dense_ff(h, W, p):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def plain_expert(h, W, p):
    return gelu_erf(h @ W[p + "up"].T) @ W[p + "down"].T


def route(z, top, count, keep):
    """For the router logits z [T, E]: (chosen experts [T, top], their weights).  Softmax over all experts; the experts
    stand in ``count`` groups of neighbours, a group is worth its best expert, only the ``keep`` best groups may be
    chosen from; the chosen experts' scores are divided by their sum."""
    T, E = z.shape
    s = np.exp(z - z.max(-1, keepdims=True))
    s /= s.sum(-1, keepdims=True)
    per = E // count
    chosen = np.zeros((T, top), dtype=np.int64)
    weights = np.zeros((T, top))
    for t in range(T):
        worth = s[t].reshape(count, per).max(-1)
        groups = np.argsort(-worth, kind="stable")[:keep]
        allowed = [e for e in range(E) if e // per in groups]
        best = sorted(allowed, key=lambda e: (-s[t, e], e))[:top]
        chosen[t] = best
        weights[t] = s[t, best] / (s[t, best].sum() + 1e-20)
    return chosen, weights


def moe_ff(h, W, p, c):
    r = c["router"]
    g = r.get("groups") or {"count": 1, "keep": 1}
    chosen, weights = route(h @ W[p + "router"].T, int(r["top"]), int(g["count"]), int(g["keep"]))
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t], weights[t]):
            out[t] += w * plain_expert(h[t:t + 1], W, f"{p}e{e}.")[0]
    if c.get("shared"):
        out += plain_expert(h, W, p + "shared.")
    return out


def layer(cfg, W, i, X, shared):
    spec = cfg["layers"][i]
    eps, groups, m = float(cfg["norm"]["eps"]), int(cfg["norm"]["groups"]), float(cfg["residual_mult"])
    p = f"l{i}."
    h = grouped_norm(X, W[p + "norm1"], eps, groups)
    h = h + short_conv(h, W[p + "canon1"])
    kind, c = spec["type"], spec["mixer"]
    if kind == "attention":
        a = attention(h, W, p + "mix.", c, eps, shared)
    elif kind == "attention_2":
        a = window_attention(h, W, p + "mix.", c, shared)
    else:
        a = wkv(h, W, p + "mix.", c, eps)
    X = X + m * a
    if spec.get("mlp"):
        h = grouped_norm(X, W[p + "norm2"], eps, groups)
        f = dense_ff(h, W, p + "mlp.") if spec["mlp"]["kind"] == "dense" else moe_ff(h, W, p + "mlp.", spec["mlp"])
        X = X + m * f
    return X


def forward(cfg, W, tokens, streams=None):
    """Logits [T, vocab] of one sequence; ``streams`` (a list) receives the stream after every layer."""
    X = W["embed"][np.asarray(tokens)]
    shared = {}
    for i in range(len(cfg["layers"])):
        X = layer(cfg, W, i, X, shared)
        if streams is not None:
            streams.append(X.copy())
    eps, groups = float(cfg["norm"]["eps"]), int(cfg["norm"]["groups"])
    return grouped_norm(X, W["final.norm"], eps, groups) @ W["head"].T


def greedy(cfg, W, prompt, new_tokens):
    """The prompt's continuation by the largest logit, token by token (each time over the whole sequence)."""
    ids = list(prompt)
    for _ in range(new_tokens):
        ids.append(int(np.argmax(forward(cfg, W, ids)[-1])))
    return ids[len(prompt):]
