"""A plain, slow restatement of the Nizedra design in float64 numpy: whole sequences, no cache, no batching,
one function per mechanism.  It shares no code with the package and is what the package is compared with.

A model is (cfg, w): ``cfg`` the dictionary of config.json, ``w`` {tensor name: float64 array} (integer tables
as they are).  Linear weights are [out, in] and act as W x.
"""

from __future__ import annotations

import math

import numpy as np


def rms_norm(x, eps, weight=None):
    """x / sqrt(mean(x^2) + eps) over the last axis, times ``weight`` if given."""
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y if weight is None else y * weight


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    ap, aq = softplus(np.float64(p)), 0.5 + softplus(np.float64(q))
    zn = np.minimum(z, 0.0)
    return np.where(z > 0.0, ap * z * z + 0.5 * z, aq * (np.expm1(zn) - zn) + 0.5 * z)


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of a distance-bias table of ``rows`` rows for the distance n >= 0: one row for each of the first rows/2
    distances, the rest spread evenly over ln(n) up to ``far``, the last row for everything beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def softmax_rows(s, visible):
    s = np.where(visible, s, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    e = np.exp(s)
    return e / e.sum(axis=-1, keepdims=True)


def mixed_heads_attention(h, w, pre, m, eps):
    """The 'attention' mixer: grouped queries, q and k to unit RMS, score scaled, times a number per head, soft-capped,
    plus a bias by bucketed distance, then mixed across heads by a matrix, then softmax over j <= i."""
    T = h.shape[0]
    H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T + w[pre + "q.b"]).reshape(T, H, D)
    k = (h @ w[pre + "k"].T + w[pre + "k.b"]).reshape(T, G, D)
    v = (h @ w[pre + "v"].T + w[pre + "v.b"]).reshape(T, G, DV)
    q, k = rms_norm(q, eps), rms_norm(k, eps)
    rel, talk, temp = w[pre + "rel"], w[pre + "talk"], w[pre + "temp"]
    rows = rel.shape[0]
    cap = m.get("softcap")        # absent: no cap
    buckets = np.array([[distance_bucket(i - j, rows, m["bias_max"]) if j <= i else 0 for j in range(T)] for i in range(T)])
    s = np.zeros((H, T, T))
    for g in range(H):
        raw = q[:, g, :] @ k[:, g // (H // G), :].T * m["scale"] * temp[g]
        s[g] = (cap * np.tanh(raw / cap) if cap else raw) + rel[buckets, g]
    s = np.einsum("hg,gij->hij", talk, s)
    visible = np.tril(np.ones((T, T), dtype=bool))
    out = np.zeros((T, H, DV))
    for hd in range(H):
        out[:, hd, :] = softmax_rows(s[hd], visible) @ v[:, hd // (H // G), :]
    return out.reshape(T, H * DV) @ w[pre + "o"].T + w[pre + "o.b"]


def lightning(h, w, pre, m, eps):
    """The 'lightning' mixer: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with q, k, v = silu of their
    projections; the heads side by side are RMS-normed together with a weight, gated by sigmoid(W_g h), projected."""
    T = h.shape[0]
    H, D, DV = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[pre + "q"].T).reshape(T, H, D)
    k = silu(h @ w[pre + "k"].T).reshape(T, H, D)
    v = silu(h @ w[pre + "v"].T).reshape(T, H, DV)
    o = np.zeros((T, H, DV))
    for hd in range(H):
        S = np.zeros((D, DV))
        for t in range(T):
            S = m["decay"][hd] * S + np.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    o = rms_norm(o.reshape(T, H * DV), eps, w[pre + "norm"]) * sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


def rotate_interleaved(x, positions, dims, base):
    """Pairs (2i, 2i+1) of the first ``dims`` elements of the last axis turn by p * base^(-2i/dims); x: [T, ..., n]."""
    out = x.copy()
    i = np.arange(dims // 2)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * base ** (-2.0 * i / dims)
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (dims // 2,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def latent_attention(h, w, pre, m, eps):
    """The 'latent_attention' mixer: queries through a normed latent; keys and values from one normed latent per token
    plus one rotated key part that all heads share; a sliding window; softmax."""
    T = h.shape[0]
    H, D, R, DV, KR = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T)
    cq = rms_norm(h @ w[pre + "dq"].T, eps, w[pre + "dq.norm"])
    q = (cq @ w[pre + "uq"].T).reshape(T, H, D + R)
    kv = h @ w[pre + "dkv"].T
    c = rms_norm(kv[:, :KR], eps, w[pre + "dkv.norm"])
    k_rot = rotate_interleaved(kv[:, KR:], pos, m["rot"]["dims"], m["rot"]["base"])
    q_rot = rotate_interleaved(q[:, :, D:], pos, m["rot"]["dims"], m["rot"]["base"])
    k_plain = (c @ w[pre + "uk"].T).reshape(T, H, D)
    v = (c @ w[pre + "uv"].T).reshape(T, H, DV)
    window = (m.get("mask") or {}).get("size", 0)
    ii, jj = np.meshgrid(np.arange(T), np.arange(T), indexing="ij")
    visible = (jj <= ii) & ((ii - jj < window) if window else True)
    out = np.zeros((T, H, DV))
    for hd in range(H):
        s = (q[:, hd, :D] @ k_plain[:, hd, :].T + q_rot[:, hd, :] @ k_rot.T) * m["scale"]
        out[:, hd, :] = softmax_rows(s, visible) @ v[:, hd, :]
    return out.reshape(T, H * DV) @ w[pre + "o"].T


def dense_ff(h, w, pre):
    p, q = w[pre + "act"]
    return xielu(h @ w[pre + "up"].T, p, q) @ w[pre + "down"].T


MIXERS = {"attention": mixed_heads_attention, "lightning": lightning, "latent_attention": latent_attention}


def layer(x, cfg, w, i):
    """x + norm1b(mixer(norm1(x))), then x + norm2b(ff(norm2(x)))."""
    eps = cfg["norm"]["eps"]
    spec = cfg["layers"][i]
    p = f"l{i}."
    a = MIXERS[spec["type"]](rms_norm(x, eps, w[p + "norm1"]), w, p + "mix.", spec["mixer"], eps)
    x = x + rms_norm(a, eps, w[p + "norm1b"])
    if spec.get("mlp") is not None:
        f = dense_ff(rms_norm(x, eps, w[p + "norm2"]), w, p + "mlp.")
        x = x + rms_norm(f, eps, w[p + "norm2b"])
    return x


def run_order(cfg):
    """[(layer, whether a pass of the loop starts with this run)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    order = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        order += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, False) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, streams=None):
    """Logits [T, vocab] of one whole sequence; ``streams``: a list that gets the stream after every layer run."""
    x0 = w["embed"][np.asarray(tokens)]
    x = x0
    for i, pass_begins in run_order(cfg):
        if pass_begins:
            x = np.concatenate([x, x0], axis=-1) @ w["loop.in"].T
        x = layer(x, cfg, w, i)
        if streams is not None:
            streams.append(x.copy())
    return rms_norm(x, cfg["norm"]["eps"], w["final.norm"]) @ w["head"].T


def greedy(cfg, w, prompt, n):
    """The n tokens that follow ``prompt`` when the most probable token is taken every time."""
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(np.argmax(forward(cfg, w, ids)[-1])))
    return ids[len(prompt):]
