"""Helpers of the Nizedra tests: small configurations, random weights made to show faults, model folders."""

from __future__ import annotations

import json
import math
import os

import numpy as np
import torch
from safetensors.torch import save_file


def attention(heads, kv_heads, dim, vdim, bias_max, rel_rows, softcap=0.0, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5,
         "bias_max": bias_max, "_rel_rows": rel_rows}
    if softcap:
        m["softcap"] = softcap
    return "attention", m


def lightning(heads, dim, vdim, decay):
    return "lightning", {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, base, dims=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5, "rot": {"base": base, "dims": dims or rot_dim}}
    if window:
        m["mask"] = {"size": window}
    return "latent_attention", m


def layer(mixer, ff):
    return {"type": mixer[0], "mixer": mixer[1], "mlp": {"kind": "dense", "ff": ff} if ff else None}


def model(vocab, width, layers, eps, loop) -> dict:
    cfg = {"architecture": "Nizedra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


def config(which: str) -> dict:
    """A: value rows of another size than key rows everywhere, 4 heads on 2 kv heads, a bias table of 12 rows that ends
       at distance 100, a latent layer that rotates half of its rotated part under a window of 20, a layer without
       feed-forward, the first two layers looped three times.
    B: what the other models leave out or make equal or 1: no loop, no soft cap, as many kv heads as heads, one
       lightning head, value rows as long as key rows, a latent layer without a window that rotates all of its rotated
       part, a bias table of 2 rows, a sharp softmax in the attention.
    C: sizes that are multiples of nothing (width 100, 3 heads of 12 with values of 20, latents of 28 and 24, a rotated
       part of 6), a window of 7 (less than a page), a bias table of 6 rows ending at distance 17, the last two layers
       looped twice.
    D: sizes of the tensor-core kernels (width 128, heads of 64, kept rows of 128), windows of 48 and 80, a bias
       table of 32 rows ending at 300, the middle layer looped twice."""
    if which == "A":
        layers = [layer(attention(4, 2, 16, 24, 100, 12, softcap=30.0), 80),
                  layer(lightning(3, 8, 16, (0.7, 0.97, 0.999)), 0),
                  layer(latent(3, 16, 8, 24, 40, 32, 20, 5000.0, dims=4), 72),
                  layer(lightning(2, 16, 8, (0.9, 0.99)), 64)]
        return model(211, 96, layers, 1e-5, (0, 2, 3))
    if which == "B":
        layers = [layer(lightning(1, 32, 32, (0.98,)), 96),
                  layer(latent(2, 16, 16, 16, 32, 32, 0, 10000.0), 96),
                  layer(attention(2, 2, 32, 32, 64, 2, scale=2.0), 96)]
        return model(300, 64, layers, 1e-6, None)
    if which == "C":
        layers = [layer(latent(3, 12, 6, 20, 28, 24, 7, 777.0), 60),
                  layer(attention(3, 3, 12, 20, 17, 6, softcap=8.0), 0),
                  layer(lightning(5, 12, 20, (0.8, 0.9, 0.95, 0.99, 0.999)), 36)]
        return model(157, 100, layers, 1e-5, (1, 3, 2))
    if which == "D":
        layers = [layer(attention(4, 2, 64, 64, 300, 32, softcap=40.0), 160),
                  layer(latent(4, 64, 64, 64, 96, 64, 48, 30000.0, dims=32), 160),
                  layer(lightning(2, 64, 64, (0.97, 0.995)), 0),
                  layer(latent(2, 32, 32, 128, 64, 96, 80, 30000.0), 128)]
        return model(320, 128, layers, 1e-6, (1, 2, 2))
    raise KeyError(which)


def random_weights(cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    """bfloat16 tensors by the design's names.  Matrices give unit-variance outputs for unit-variance inputs; norm weights
    lie around 1; the numbers per head lie between 1 and 3; the distance biases are of the scores' own size, so that a
    key in the wrong bucket shows; the matrix that mixes the heads is the identity plus a third of noise."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    bf = lambda t: t.to(torch.bfloat16)
    mat = lambda out, inp, gain=1.0: bf(torch.randn(out, inp, generator=g) * gain / math.sqrt(inp))
    around_one = lambda n: bf(1.0 + 0.2 * torch.randn(n, generator=g))
    small = lambda *n: bf(0.1 * torch.randn(*n, generator=g))
    t = {"embed": bf(torch.randn(V, W, generator=g)), "final.norm": around_one(W), "head": mat(V, W, 3.0)}
    if cfg.get("loop"):
        t["loop.in"] = mat(W, 2 * W, 1.4)
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        t[p + "norm1"], t[p + "norm1b"] = around_one(W), around_one(W)
        if lay["type"] == "attention":
            H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", H * D), ("k", G * D), ("v", G * DV)):
                t[p + "mix." + n], t[p + "mix." + n + ".b"] = mat(rows, W), small(rows)
            t[p + "mix.o"], t[p + "mix.o.b"] = mat(W, H * DV), small(W)
            t[p + "mix.temp"] = bf(1.0 + 2.0 * torch.rand(H, generator=g))
            t[p + "mix.rel"] = bf(1.5 * torch.randn(m["_rel_rows"], H, generator=g))
            t[p + "mix.talk"] = bf(torch.eye(H) + 0.3 * torch.randn(H, H, generator=g))
        elif lay["type"] == "lightning":
            H, D, DV = m["heads"], m["dim"], m["vdim"]
            t[p + "mix.q"], t[p + "mix.k"] = mat(H * D, W, 1.5), mat(H * D, W, 1.5)
            t[p + "mix.v"], t[p + "mix.g"] = mat(H * DV, W, 1.5), mat(H * DV, W, 1.5)
            t[p + "mix.norm"] = around_one(H * DV)
            t[p + "mix.o"] = mat(W, H * DV)
        else:
            H, D, R, DV, QR, KR = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            t[p + "mix.dq"], t[p + "mix.dq.norm"] = mat(QR, W), around_one(QR)
            t[p + "mix.uq"] = mat(H * (D + R), QR, 1.5)
            t[p + "mix.dkv"], t[p + "mix.dkv.norm"] = mat(KR + R, W), around_one(KR)
            t[p + "mix.uk"], t[p + "mix.uv"] = mat(H * D, KR, 1.5), mat(H * DV, KR)
            t[p + "mix.o"] = mat(W, H * DV)
        if lay.get("mlp"):
            F = lay["mlp"]["ff"]
            t[p + "norm2"], t[p + "norm2b"] = around_one(W), around_one(W)
            t[p + "mlp.up"], t[p + "mlp.down"] = mat(F, W, 1.5), mat(W, F)
            t[p + "mlp.act"] = bf(torch.randn(2, generator=g))
    return t


def clean(cfg: dict) -> dict:
    """The configuration as a file holds it (the helpers' private keys taken out)."""
    out = json.loads(json.dumps(cfg))
    for lay in out["layers"]:
        lay["mixer"] = {k: v for k, v in lay["mixer"].items() if not k.startswith("_")}
    return out


def write_model(folder: str, cfg: dict, seed: int, weights: dict | None = None) -> str:
    os.makedirs(folder, exist_ok=True)
    weights = weights if weights is not None else random_weights(cfg, seed)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(clean(cfg), fh)
    save_file({n: t.contiguous() for n, t in weights.items()}, os.path.join(folder, "model.safetensors"))
    return folder


def read_folder(folder: str):
    """(config dictionary, {name: float64 numpy array}) of a model folder."""
    from safetensors import safe_open
    with open(os.path.join(folder, "config.json"), encoding="utf-8") as fh:
        cfg = json.load(fh)
    tensors = {}
    with safe_open(os.path.join(folder, "model.safetensors"), "pt") as f:
        for k in f.keys():
            tensors[k] = f.get_tensor(k).to(torch.float64).numpy()
    return cfg, tensors


def row_errors(got, want) -> np.ndarray:
    """Per row: the root mean square of the difference, each side's mean taken off, over that of the wanted row."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    d = (got - got.mean(-1, keepdims=True)) - (want - want.mean(-1, keepdims=True))
    ref = np.maximum(np.sqrt(((want - want.mean(-1, keepdims=True)) ** 2).mean(-1)), 1e-12)
    return np.sqrt((d ** 2).mean(-1)) / ref
