"""Typed configuration of the Nizedra design.

A small decoder-only model over a float32 residual stream.  Every layer puts an RMS norm in front of and behind each
of its two parts, x += norm_b(part(norm(x))).  The mixer is one of

  ``attention``         grouped queries under the full causal mask; q and k brought to unit RMS; the score is scaled,
                        multiplied by a number of its head, soft-capped, gets a learned bias by bucketed distance, and is
                        then mixed across the heads by a learned matrix before the softmax; projections with biases;
  ``lightning``         linear attention with a fixed decay per head over silu(q), silu(k), silu(v), the heads normed
                        together, a sigmoid gate;
  ``latent_attention``  queries and keys/values through normed low-rank latents; a head's key is an unrotated part made
                        from the latent and a rotated part (interleaved pairs) shared by all heads; only the latent and
                        the rotated part are kept; a sliding window.

The feed-forward is W_down act(W_up h) with a two-parameter activation, or absent.  A stretch of layers may run several
times over the same weights (``loop``); every pass keeps a cache and states of its own and begins by mixing the stream
with the embedding output through ``loop.in``.  config.json is nested:

    {"architecture": "Nizedra", "vocab": V, "width": W, "norm": {"eps": e}, "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap", "bias_max"},
                 "mlp": null | {"kind": "dense", "ff": F}},
                {"type": "lightning", "mixer": {"heads", "dim", "vdim", "decay": [...]}, "mlp": ...},
                {"type": "latent_attention", "mixer": {"heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale",
                 "mask": {"size"}, "rot": {"base", "dims"}}, "mlp": ...}, ...]}

Every size and constant that may differ between models is read from there (the rows of the distance-bias table are the
tensor's own first dimension: the loader reports them).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, take_float, take_int

MAX_POSITIONS = 1 << 17     # rows of the rotary tables; the design itself names no longest sequence


def _section(cfg: Mapping[str, Any], key: str, where: str, optional: bool = False):
    value = cfg.get(key)
    if value is None and optional:
        return None
    if not isinstance(value, Mapping):
        raise ConfigError(f"{where}'{key}' must be an object")
    return value


@dataclass(frozen=True)
class MixedHeadsSpec:
    """``attention``: scores mixed across heads."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float          # 0: none
    bias_max: float         # the distance from which every key gets the bias table's last row

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "MixedHeadsSpec":
        heads, dim = take_int(m, "heads"), take_int(m, "dim")
        kv = take_int(m, "kv_heads", heads)
        if heads % kv:
            raise ConfigError(f"{where}heads {heads} is not a multiple of kv_heads {kv}")
        cap = m.get("softcap")
        return cls(heads, kv, dim, take_int(m, "vdim", dim), take_float(m, "scale", dim ** -0.5),
                   take_float(m, "softcap") if cap else 0.0, take_float(m, "bias_max"))

    def to_dict(self) -> dict:
        out: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale, "bias_max": _plain(self.bias_max)}
        if self.softcap:
            out["softcap"] = self.softcap
        return out


def _plain(v: float):
    return int(v) if float(v).is_integer() else v


@dataclass(frozen=True)
class LightningSpec:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "LightningSpec":
        heads, dim = take_int(m, "heads"), take_int(m, "dim")
        decay = m.get("decay")
        if not isinstance(decay, (list, tuple)) or len(decay) != heads or \
                any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
            raise ConfigError(f"{where}'decay' must list one number for each of the {heads} heads")
        return cls(heads, dim, take_int(m, "vdim", dim), tuple(float(d) for d in decay))

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class LatentSpec:
    heads: int
    dim: int                # unrotated elements of a head's query and key
    rot_dim: int            # rotated elements (one key part for all heads)
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: int             # 0: every earlier key is seen
    rot_base: float
    rot_dims: int           # elements of the rotated part that turn (the rest pass unchanged)

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "LatentSpec":
        heads, dim, rot_dim = take_int(m, "heads"), take_int(m, "dim"), take_int(m, "rot_dim")
        mask = _section(m, "mask", where, optional=True)
        rot = _section(m, "rot", where)
        dims = take_int(rot, "dims", rot_dim, minimum=2)
        if dims % 2 or dims > rot_dim:
            raise ConfigError(f"{where}rot.dims {dims} must be even and at most rot_dim {rot_dim}")
        return cls(heads, dim, rot_dim, take_int(m, "vdim", dim), take_int(m, "q_rank"), take_int(m, "kv_rank"),
                   take_float(m, "scale", (dim + rot_dim) ** -0.5), take_int(mask, "size", 0, minimum=0) if mask else 0,
                   take_float(rot, "base"), dims)

    def to_dict(self) -> dict:
        out: dict[str, Any] = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                               "q_rank": self.q_rank, "kv_rank": self.kv_rank, "scale": self.scale,
                               "rot": {"base": self.rot_base, "dims": self.rot_dims}}
        if self.window:
            out["mask"] = {"size": self.window}
        return out


@dataclass(frozen=True)
class NizedraLayer:
    type: str               # "attention" | "lightning" | "latent_attention"
    mixer: MixedHeadsSpec | LightningSpec | LatentSpec
    ff: int                 # 0: the layer has no feed-forward


@dataclass(frozen=True)
class NizedraConfig:
    vocab: int
    width: int
    norm_eps: float
    loop: tuple[int, int, int] | None       # (start, stop, times)
    layers: tuple[NizedraLayer, ...]

    architecture = "Nizedra"
    MIXERS = {"attention": MixedHeadsSpec, "lightning": LightningSpec, "latent_attention": LatentSpec}

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any]) -> "NizedraConfig":
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
            ff = 0
            if mlp is not None:
                if not isinstance(mlp, Mapping):
                    raise ConfigError(f"{where}'mlp' must be an object or null")
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"{where}mlp.kind = {mlp.get('kind')!r}: the design's feed-forward is 'dense'")
                ff = take_int(mlp, "ff")
            layers.append(NizedraLayer(kind, mixer, ff))
        loop = None
        raw_loop = cfg.get("loop")
        if raw_loop is not None:
            if not isinstance(raw_loop, Mapping):
                raise ConfigError("'loop' must be an object or absent")
            start, stop = take_int(raw_loop, "start", minimum=0), take_int(raw_loop, "stop", minimum=0)
            times = take_int(raw_loop, "times", 1)
            if not start < stop <= len(layers):
                raise ConfigError(f"loop: start {start} and stop {stop} must name a stretch of the {len(layers)} layers")
            loop = (start, stop, times)
        return cls(vocab=take_int(cfg, "vocab"), width=take_int(cfg, "width"),
                   norm_eps=take_float(_section(cfg, "norm", ""), "eps"), loop=loop, layers=tuple(layers))

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
            "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": {"kind": "dense", "ff": l.ff} if l.ff else None}
                       for l in self.layers]}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return out
