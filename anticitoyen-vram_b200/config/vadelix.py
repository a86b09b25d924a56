"""Typed configuration of the Vadelix design.

A small decoder-only model over a float32 residual stream.  Every layer is
pre-norm (RMS norms taken in groups) with a short causal convolution on what its
mixer reads and a constant ``residual_mult`` on what its parts add to the stream.
A layer's mixer is one of three: ``attention`` (grouped queries, an RMS norm over
the whole of q and of k, partial rotary positions with YaRN scaling, value heads
of unit RMS, a learned softmax sink per head), ``attention_2`` (no rotation; a
query temperature that grows with the position, a distance bias with a slope per
head, a sliding window, a sink of score 0) or ``wkv`` (an RWKV-style recurrence
with decays of the token's own).  Attention layers of either kind that say
``v_mix`` blend their values with those of the first such layer.  The feed-forward
is a gated unit (``dense``), a mixture of experts without gates, chosen from the
best groups of experts, beside a shared expert (``moe``), or absent.  config.json
is nested:

    {"architecture": "Vadelix", "vocab": V, "width": W, "norm": {"eps": e, "groups": g}, "residual_mult": m,
     "canon": {"taps": K},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "v_mix",
                           "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}}},
                 "mlp": null | {"kind": "dense", "ff": F}
                             | {"kind": "moe", "expert": {"ff"}, "shared": {"ff"},
                                "router": {"experts", "top", "groups": {"count", "keep"}}}},
                {"type": "attention_2", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "v_mix", "mask": {"size"},
                                                  "q_temp": {"coef", "every"}}, "mlp": ...},
                {"type": "wkv", "mixer": {"heads", "dim"}, "mlp": ...}, ...]}

Every size and constant that may differ between models is read from there.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, take_float, take_int
from .redudra import RotarySpec, _section

MAX_POSITIONS = 1 << 17     # rows of the rotary tables; the design itself names no longest sequence


def _heads(m: Mapping[str, Any], where: str) -> tuple[int, int, int, int, float, bool]:
    heads, dim = take_int(m, "heads"), take_int(m, "dim")
    kv = take_int(m, "kv_heads", heads)
    if heads % kv:
        raise ConfigError(f"{where}heads {heads} is not a multiple of kv_heads {kv}")
    v_mix = m.get("v_mix", False)
    if not isinstance(v_mix, bool):
        raise ConfigError(f"{where}'v_mix' must be true or false")
    return heads, kv, dim, take_int(m, "vdim", dim), take_float(m, "scale", dim ** -0.5), v_mix


@dataclass(frozen=True)
class SinkAttentionSpec:
    """Mixer ``attention``."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    v_mix: bool
    rot: RotarySpec | None

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "SinkAttentionSpec":
        heads, kv, dim, vdim, scale, v_mix = _heads(m, where)
        rot = _section(m, "rot", where, optional=True)
        return cls(heads, kv, dim, vdim, scale, v_mix, RotarySpec.from_dict(rot, where, dim) if rot else None)

    def to_dict(self) -> dict:
        out: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale, "v_mix": self.v_mix}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        return out


@dataclass(frozen=True)
class WindowAttentionSpec:
    """Mixer ``attention_2``."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    v_mix: bool
    window: int                         # 0: every earlier key is seen
    q_temp: tuple[float, int] | None    # (coef, every)

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "WindowAttentionSpec":
        heads, kv, dim, vdim, scale, v_mix = _heads(m, where)
        mask = _section(m, "mask", where, optional=True)
        temp = _section(m, "q_temp", where, optional=True)
        return cls(heads, kv, dim, vdim, scale, v_mix, take_int(mask, "size", 0, minimum=0) if mask else 0,
                   (take_float(temp, "coef", positive=False), take_int(temp, "every")) if temp else None)

    def to_dict(self) -> dict:
        out: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale, "v_mix": self.v_mix}
        if self.window:
            out["mask"] = {"size": self.window}
        if self.q_temp is not None:
            out["q_temp"] = {"coef": self.q_temp[0], "every": self.q_temp[1]}
        return out


@dataclass(frozen=True)
class TimeMixSpec:
    """Mixer ``wkv``."""

    heads: int
    dim: int

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "TimeMixSpec":
        return cls(take_int(m, "heads"), take_int(m, "dim"))

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim}


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str                   # "dense" | "moe"
    ff: int                     # dense: the gated unit's inner size; moe: an expert's
    experts: int = 0
    top: int = 0
    groups: tuple[int, int] = (1, 1)    # (count, keep)
    shared_ff: int = 0          # 0: no shared expert

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "FeedForwardSpec":
        kind = m.get("kind", "dense")
        if kind == "dense":
            return cls("dense", take_int(m, "ff"))
        if kind != "moe":
            raise ConfigError(f"{where}mlp.kind = {kind!r}: the design's feed-forwards are 'dense' and 'moe'")
        router = _section(m, "router", where + "mlp: ")
        experts, top = take_int(router, "experts"), take_int(router, "top")
        groups = _section(router, "groups", where + "mlp.router: ", optional=True)
        count, keep = (take_int(groups, "count"), take_int(groups, "keep")) if groups else (1, 1)
        if experts % count or not 1 <= keep <= count or top > keep * (experts // count):
            raise ConfigError(f"{where}mlp.router: {experts} experts in {count} groups of which {keep} are kept cannot give "
                              f"{top} choices")
        shared = _section(m, "shared", where + "mlp: ", optional=True)
        return cls("moe", take_int(_section(m, "expert", where + "mlp: "), "ff"), experts, top, (count, keep),
                   take_int(shared, "ff") if shared else 0)

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        out: dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff},
                               "router": {"experts": self.experts, "top": self.top,
                                          "groups": {"count": self.groups[0], "keep": self.groups[1]}}}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class VadelixLayer:
    type: str                               # "attention" | "attention_2" | "wkv"
    mixer: SinkAttentionSpec | WindowAttentionSpec | TimeMixSpec
    mlp: FeedForwardSpec | None


@dataclass(frozen=True)
class VadelixConfig:
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    residual_mult: float
    conv_taps: int
    layers: tuple[VadelixLayer, ...]

    architecture = "Vadelix"
    MIXERS = {"attention": SinkAttentionSpec, "attention_2": WindowAttentionSpec, "wkv": TimeMixSpec}

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any]) -> "VadelixConfig":
        raw = cfg.get("layers")
        if not isinstance(raw, (list, tuple)) or not raw:
            raise ConfigError("config key 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]: "
            if not isinstance(entry, Mapping):
                raise ConfigError(f"{where}must be an object")
            kind = entry.get("type")
            spec = cls.MIXERS.get(kind)
            if spec is None:
                raise ConfigError(f"{where}'type' = {kind!r}: the mixers built for this design are: {', '.join(sorted(cls.MIXERS))}")
            mixer = spec.from_dict(_section(entry, "mixer", where), where)
            mlp = entry.get("mlp")
            if mlp is not None and not isinstance(mlp, Mapping):
                raise ConfigError(f"{where}'mlp' must be an object or null")
            layers.append(VadelixLayer(kind, mixer, FeedForwardSpec.from_dict(mlp, where) if mlp is not None else None))
        sharing = [l.mixer for l in layers if getattr(l.mixer, "v_mix", False)]
        if len({(m.kv_heads, m.vdim) for m in sharing}) > 1:
            raise ConfigError("layers with 'v_mix' blend their values with the first such layer's: their kv_heads and vdim must agree")
        width = take_int(cfg, "width")
        norm = _section(cfg, "norm", "")
        groups = take_int(norm, "groups", 1)
        if width % groups:
            raise ConfigError(f"norm.groups {groups} does not divide the width {width}")
        canon = _section(cfg, "canon", "")
        return cls(vocab=take_int(cfg, "vocab"), width=width, norm_eps=take_float(norm, "eps"), norm_groups=groups,
                   residual_mult=take_float(cfg, "residual_mult", 1.0, positive=False), conv_taps=take_int(canon, "taps"),
                   layers=tuple(layers))

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "residual_mult": self.residual_mult,
                "canon": {"taps": self.conv_taps},
                "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": l.mlp.to_dict() if l.mlp else None}
                           for l in self.layers]}
