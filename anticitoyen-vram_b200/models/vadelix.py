"""The Vadelix design as a plan of parts.

Pre-norm layers (``rmsnorm`` taken in groups) over a float32 residual stream, each
with a short causal convolution on its mixer's input (block option ``input_conv``)
and the constant ``residual_mult`` on what it adds.  The mixers: ``attention`` with
a norm over the whole of q and of k, partial rotary positions with YaRN scaling,
value heads of unit RMS and a learned sink; ``attention`` with a query
temperature, distance slopes, a sliding window and a sink of score 0; ``wkv``.
Attention layers that blend values share them through the step under one key: the
first such layer is the source.  The feed-forward is ``swiglu`` with a gelu gate,
``moe`` with plain experts chosen from the best groups, or absent.

What the design fixes is written here as parameters of the parts; what a model
of the design may choose comes from ``VadelixConfig``.
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.vadelix import MAX_POSITIONS, VadelixConfig
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, default_schedule

SLOPE_RATE = 8.0            # slope_h = 2^(-8 (h + 1) / heads) of the distance bias
ZERO_SINK = 0.0             # "one added to the denominator": a sink whose score is 0
ROUTER_SUM_EPS = 1e-20      # joins the sum that the chosen experts' scores are divided by
SHARED_VALUES = "v_first"   # the step's key under which the first value-mixing layer leaves its values
ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm"}


def _attention(kind: str, m, eps: float, share_role: str | None) -> PartSpec:
    params = {"num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim, "scale": m.scale,
              "prefix": "mix.", "names": ATTENTION_NAMES, "bias": False}
    if share_role is not None:
        params["value_share"] = {"key": SHARED_VALUES, "role": share_role, "tensor": "vmix"}
    if kind == "attention":
        rot = PartSpec("none") if m.rot is None else PartSpec("rotary", {
            "dim": m.rot.dims, "theta": m.rot.base, "max_positions": MAX_POSITIONS, "scaling": m.rot.scaling, "exact": True})
        params.update(position=rot, qk_norm_eps=eps, qk_norm_scope="all", value_norm_eps=eps, sink="sink")
    else:
        params.update(position=PartSpec("none"), window=m.window, q_temp=m.q_temp, sink=ZERO_SINK, slope_rate=SLOPE_RATE)
    return PartSpec("attention", params)


def vadelix_plan(cfg: VadelixConfig) -> ModelPlan:
    norm = PartSpec("rmsnorm", {"eps": cfg.norm_eps, "tensor": "", "groups": cfg.norm_groups})
    options = {"residual_mult": cfg.residual_mult, "input_conv": {"tensor": "canon1", "taps": cfg.conv_taps}}
    layers = []
    source_seen = False
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "wkv":
            mixer = PartSpec("wkv", {"num_heads": m.heads, "dim": m.dim, "norm_eps": cfg.norm_eps, "prefix": "mix."})
        else:
            role = None
            if m.v_mix:
                role, source_seen = ("mix" if source_seen else "source"), True
            mixer = _attention(layer.type, m, cfg.norm_eps, role)
        ff = None
        if layer.mlp is not None and layer.mlp.kind == "dense":
            ff = PartSpec("swiglu", {"intermediate_size": layer.mlp.ff, "prefix": "mlp.", "bias": False, "activation": "gelu_tanh",
                                     "names": {"gate": "gate", "up": "up", "down": "down"}})
        elif layer.mlp is not None:
            f = layer.mlp
            ff = PartSpec("moe", {"experts": f.experts, "top": f.top, "expert_ff": f.ff, "expert_limit": 0.0,
                                  "shared_ff": f.shared_ff, "scoring": "softmax", "renormalize": True,
                                  "renorm_eps": ROUTER_SUM_EPS, "weight_on": "output", "prefix": "mlp.", "expert_form": "plain",
                                  "activation": "gelu", "groups": f.groups, "shared_gate": False})
        layers.append(LayerSpec(f"l{i}.", "prenorm", mixer, ff, norm, norm_prefixes=("norm1", "norm2"), options=options))
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        layers=tuple(layers), schedule=default_schedule(len(layers)), final_norm=norm, embedding_name="embed",
        final_norm_prefix="final.norm", head_name="head", tied_head=False, residual_dtype="float32")


register_architecture("Vadelix", VadelixConfig, vadelix_plan)
