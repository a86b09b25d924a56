"""The Nizedra design as a plan of parts.

Every layer is a ``sandwich`` block over a float32 residual stream: an RMS norm in front of and behind each of its two
parts.  A layer's mixer is one of

  ``attention``         the framework's grouped-query ``attention`` with biases, q and k brought to unit RMS (no
                        weights), no position encoding, and the score steps (a number per head, a soft cap, a bias by
                        bucketed distance, a mix across heads before the softmax);
  ``lightning``         ``retention`` without positions or key scale, over silu(q), silu(k), silu(v), the heads normed
                        together with a weight, a sigmoid gate;
  ``latent_attention``  attention through kept latents with interleaved rotary positions on a shared key part, under a
                        sliding window.

The feed-forward is ``dense`` with the two-parameter activation, or absent.  A looped stretch of layers appears in
the schedule once for every pass, each run with a cache slot of its own, and the first layer of every pass is
preceded by the mix of the stream with the embedding output through ``loop.in``.

What the design fixes is written here as parameters of the parts; what a model of the design may choose comes from
``NizedraConfig``.
"""

from __future__ import annotations

from ..config.nizedra import MAX_POSITIONS, LatentSpec, LightningSpec, MixedHeadsSpec, NizedraConfig
from ..config.registry import register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry

LOOP_MATRIX = "loop.in"     # [width, 2 width]: a pass starts from W [stream; embedding output]


def _attention(m: MixedHeadsSpec, eps: float) -> PartSpec:
    score = {"temp": "temp", "rel": "rel", "far": m.bias_max, "talk": "talk"}
    if m.softcap:
        score["softcap"] = m.softcap
    names = {r: r for r in ("q", "k", "v", "o")}
    names.update({r + ".bias": r + ".b" for r in ("q", "k", "v", "o")})
    return PartSpec("attention", {
        "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim, "scale": m.scale,
        "position": PartSpec("none"), "qk_norm_eps": eps, "qk_norm_weights": False, "prefix": "mix.", "names": names,
        "bias": True, "score": score})


def _lightning(m: LightningSpec, eps: float) -> PartSpec:
    return PartSpec("retention", {
        "num_heads": m.heads, "dim": m.dim, "value_dim": m.vdim, "decay": m.decay, "norm_eps": eps, "position": None,
        "k_scale": 1.0, "prefix": "mix.", "input_act": "silu", "joint_norm": "norm", "gate_fn": "sigmoid"})


def _latent(m: LatentSpec, eps: float) -> PartSpec:
    position = PartSpec("rotary", {"dim": m.rot_dims, "theta": m.rot_base, "max_positions": MAX_POSITIONS, "exact": True})
    return PartSpec("latent_attention", {
        "num_heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "value_dim": m.vdim, "q_rank": m.q_rank,
        "kv_rank": m.kv_rank, "scale": m.scale, "norm_eps": eps, "position": position, "window": m.window,
        "prefix": "mix."})


_MIXERS = {"attention": _attention, "lightning": _lightning, "latent_attention": _latent}


def nizedra_plan(cfg: NizedraConfig) -> ModelPlan:
    norm = PartSpec("rmsnorm", {"eps": cfg.norm_eps, "tensor": ""})
    layers = []
    for i, layer in enumerate(cfg.layers):
        ff = PartSpec("dense", {"intermediate_size": layer.ff, "activation": "xielu", "prefix": "mlp."}) if layer.ff else None
        layers.append(LayerSpec(f"l{i}.", "sandwich", _MIXERS[layer.type](layer.mixer, cfg.norm_eps), ff, norm,
                                norm_prefixes=("norm1", "norm2"), options={"post_norms": ("norm1b", "norm2b")}))
    n = len(layers)
    if cfg.loop is None:
        order = [(i, False) for i in range(n)]
    else:
        start, stop, times = cfg.loop
        order = [(i, False) for i in range(start)]
        for _ in range(times):
            order += [(i, i == start) for i in range(start, stop)]
        order += [(i, False) for i in range(stop, n)]
    # every run of a layer keeps its own pages and states
    schedule = tuple(ScheduleEntry(i, slot, True, None, LOOP_MATRIX if begins else None)
                     for slot, (i, begins) in enumerate(order))
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        layers=tuple(layers), schedule=schedule, final_norm=norm, embedding_name="embed", final_norm_prefix="final.norm",
        head_name="head", tied_head=False, residual_dtype="float32",
        stream_matrices={LOOP_MATRIX: (cfg.width, 2 * cfg.width)} if cfg.loop is not None else {})


register_architecture("Nizedra", NizedraConfig, nizedra_plan)
