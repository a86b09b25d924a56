"""Helpers of the Vadelix tests: small configurations, random weights made to show faults, model folders."""

from __future__ import annotations

import json
import math
import os

import numpy as np
import torch
from safetensors.torch import save_file


def rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def attention(heads, kv_heads, dim, vdim, rotary, v_mix=False, scale=None):
    return "attention", {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                         "scale": scale if scale is not None else dim ** -0.5, "v_mix": v_mix, "rot": rotary}


def window_attention(heads, kv_heads, dim, vdim, window, temp, v_mix=False, scale=None):
    return "attention_2", {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                           "scale": scale if scale is not None else dim ** -0.5, "v_mix": v_mix, "mask": {"size": window},
                           "q_temp": {"coef": temp[0], "every": temp[1]}}


def wkv(heads, dim, rank=8):
    return "wkv", {"heads": heads, "dim": dim, "_rank": rank}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, count, keep, ff, shared):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(mixer, mlp):
    return {"type": mixer[0], "mixer": mixer[1], "mlp": mlp}


def model(vocab, width, layers, eps, groups, mult, taps) -> dict:
    return {"architecture": "Vadelix", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups},
            "residual_mult": mult, "canon": {"taps": taps}, "layers": layers}


def config(which: str) -> dict:
    """A: every mechanism at sizes of its own: norms in 3 groups, 3 taps, a recurrence of 3 heads first, value rows longer
       than key rows, 4 heads on 2 kv heads, rotation of half a head with scaled frequencies, 6 experts in 3 groups of
       which 2 are kept, a window of 20, a layer without feed-forward; three layers blend values (source: a rotated one).
    B: what the other models leave out or make equal or 1: one norm group, one tap (the convolution keeps nothing), a
       residual factor of 1, as many kv heads as heads, value rows as long as key rows, rotation of the whole head
       without scaling, no layer blends values, a temperature that grows every position, one recurrence head, one
       group of experts, one choice, no shared expert, a sharp softmax.
    C: sizes that are multiples of nothing (width 100 in 5 groups, 3 heads of 12 with values of 20), 5 taps, a window of
       7 (less than a page), 5 experts each a group of its own; the source of the blended values is a windowed layer.
    D: sizes of the tensor-core kernels (width 128, heads of 64 and 128), windows of 48 and 80, 8 experts in 4 groups."""
    if which == "A":
        layers = [layer(wkv(3, 16), dense(80)),
                  layer(attention(4, 2, 16, 24, rot(5000.0, 8, (4.0, 64, 16.0, 2.0)), v_mix=True), moe(6, 2, 3, 2, 40, 56)),
                  layer(window_attention(4, 2, 16, 24, 20, (0.4, 16), v_mix=True), None),
                  layer(attention(2, 2, 32, 24, rot(100.0, 32), v_mix=True, scale=0.3), dense(64))]
        return model(211, 96, layers, 1e-5, 3, 0.6, 3)
    if which == "B":
        layers = [layer(attention(2, 2, 32, 32, rot(10000.0, 32), scale=1.5), moe(4, 1, 1, 1, 48, 0)),
                  layer(wkv(1, 32, rank=4), dense(96)),
                  layer(window_attention(2, 2, 16, 16, 40, (0.25, 1)), dense(96))]
        return model(300, 64, layers, 1e-6, 1, 1.0, 1)
    if which == "C":
        layers = [layer(window_attention(3, 3, 12, 20, 7, (0.3, 5), v_mix=True), moe(5, 2, 5, 2, 36, 28)),
                  layer(wkv(5, 12, rank=6), None),
                  layer(attention(3, 3, 12, 20, rot(777.0, 6, (2.0, 32, 8.0, 1.0)), v_mix=True), dense(60)),
                  layer(window_attention(6, 3, 8, 20, 33, (0.5, 11), v_mix=True), moe(5, 2, 5, 2, 36, 28))]
        return model(157, 100, layers, 1e-5, 5, 0.8, 5)
    if which == "D":
        layers = [layer(attention(4, 1, 64, 64, rot(30000.0, 32, (2.0, 128, 16.0, 1.0)), v_mix=True), dense(160)),
                  layer(wkv(2, 64), moe(8, 3, 4, 2, 64, 96)),
                  layer(window_attention(2, 1, 64, 64, 48, (0.3, 32), v_mix=True), dense(128)),
                  layer(window_attention(2, 2, 128, 128, 80, (0.2, 50)), moe(8, 2, 4, 1, 32, 0)),
                  layer(attention(2, 2, 128, 128, rot(500.0, 128)), None)]
        return model(320, 128, layers, 1e-6, 2, 0.7, 2)
    raise KeyError(which)


def random_weights(cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    """bfloat16 tensors by the design's names.  Matrices give unit-variance outputs for unit-variance inputs; norm weights
    lie around 1; sinks are of the scores' own size; the blending numbers lie between 0.2 and 0.8; the decays'
    offsets give decays between 0.2 and 0.95; the router's logits are a few units apart."""
    g = torch.Generator().manual_seed(seed)
    W, V, K = cfg["width"], cfg["vocab"], cfg["canon"]["taps"]
    bf = lambda t: t.to(torch.bfloat16)
    mat = lambda out, inp, gain=1.0: bf(torch.randn(out, inp, generator=g) * gain / math.sqrt(inp))
    around_one = lambda *n: bf(1.0 + 0.2 * torch.randn(*n, generator=g))
    t = {"embed": bf(torch.randn(V, W, generator=g)), "final.norm": around_one(W), "head": mat(V, W, 3.0)}
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        t[p + "norm1"] = around_one(W)
        t[p + "canon1"] = bf(0.4 * torch.randn(W, K, generator=g))
        if lay["type"] == "wkv":
            H, D, R = m["heads"], m["dim"], m["_rank"]
            for s in "rkvgw":
                t[p + "mix.mu." + s] = bf(torch.rand(W, generator=g))
            for n in "rkvg":
                t[p + "mix." + n] = mat(H * D, W, 1.2)
            t[p + "mix.w1"], t[p + "mix.w2"] = mat(R, W, 1.5), mat(H * D, R, 1.0)
            t[p + "mix.w0"] = bf(-1.5 + 1.0 * torch.randn(H * D, generator=g))
            t[p + "mix.u"] = bf(0.5 * torch.randn(H, D, generator=g))
            t[p + "mix.norm"] = around_one(H * D)
            t[p + "mix.o"] = mat(W, H * D)
        else:
            H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"] = mat(H * D, W, 1.5), mat(G * D, W, 1.5), mat(G * DV, W)
            t[p + "mix.o"] = mat(W, H * DV)
            if m.get("v_mix"):
                t[p + "mix.vmix"] = bf(0.2 + 0.6 * torch.rand((), generator=g))
            if lay["type"] == "attention":
                t[p + "mix.q.norm"], t[p + "mix.k.norm"] = around_one(H * D), around_one(G * D)
                t[p + "mix.sink"] = bf(torch.randn(H, generator=g))
        mlp = lay.get("mlp")
        if mlp:
            t[p + "norm2"] = around_one(W)
        if mlp and mlp["kind"] == "dense":
            F = mlp["ff"]
            t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = mat(F, W, 1.5), mat(F, W), mat(W, F)
        elif mlp:
            F, E = mlp["expert"]["ff"], mlp["router"]["experts"]
            t[p + "mlp.router"] = mat(E, W, 2.0)
            for e in range(E):
                t[f"{p}mlp.e{e}.up"], t[f"{p}mlp.e{e}.down"] = mat(F, W, 1.5), mat(W, F, 1.5)
            if mlp.get("shared"):
                S = mlp["shared"]["ff"]
                t[p + "mlp.shared.up"], t[p + "mlp.shared.down"] = mat(S, W, 1.5), mat(W, S)
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
