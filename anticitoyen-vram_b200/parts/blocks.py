"""Arrangements of a layer's parts."""

from __future__ import annotations

import torch

from ..cache.manager import StateNeed
from ..kernels import ops
from ..weights.needs import TensorNeed
from .base import CacheView, Runtime
from .norms import LayerNorm
from .plan import LayerSpec
from .registry import build, register


@register("block", "prenorm")
class PreNormBlock:
    """x += mixer(norm(x)); x += feed_forward(norm(x)) (acvram/engine/couches.py:404-425).

    The residual travels as (x, delta): the sum x + delta is made inside the next
    norm's kernel, as the reference's deferred-residual path does
    (acvram/engine/couches.py:427-443), so the stream is read and written once per
    sub-block.

    Options (``LayerSpec.options``):
      ``residual_mult`` m: x += m * mixer(...), x += m * feed_forward(...); the factor is applied inside the next norm's
        kernel, in 32-bit, as the part's output joins the stream.
      ``token_shift``: the name (behind the layer's prefix) of a vector mu of the stream's width.  What the mixer reads is
        then h'[t] = h[t] + (h[t-1] - h[t]) * mu, h the first norm's output and h[t-1] the same of the request's previous
        token (zeros before its first): the layer keeps one row of h for every request, in a state slot beside what its
        mixer keeps, and the mix is made in 32-bit before h' is rounded to the parts' element type.
      ``input_conv``: {"tensor": name behind the layer's prefix, "taps": K}: what the mixer reads is h + conv(h), h the
        first norm's output and conv a causal convolution over time on every channel by itself, conv(h)[t] =
        sum_j w[:, j] h[t - K + 1 + j] (w: [width, K], zeros before the request's first token).  The layer keeps the last
        K - 1 rows of h for every request in a state slot beside what its mixer keeps; norm output, convolution and kept
        rows are 32-bit, the sum is rounded once to the parts' element type."""

    def __init__(self, spec: LayerSpec, hidden_size: int) -> None:
        self.hidden_size = hidden_size
        self.residual_mult = float(spec.options.get("residual_mult", 1.0))
        self.token_shift = spec.options.get("token_shift")
        self.shift_mu = None
        self.input_conv = spec.options.get("input_conv")
        self.conv_taps = None
        if self.input_conv is not None and self.token_shift is not None:
            raise ValueError("the pre-norm block takes a token shift or an input convolution, not both")
        self.prefix = spec.prefix
        self.pre_mixer, self.pre_ff = spec.norm_prefixes
        self.input_norm = build("norm", spec.norm, hidden_size)
        self.mixer = build("mixer", spec.mixer, hidden_size)
        # a layer without a feed-forward is its mixer alone: x += mixer(norm(x))
        self.post_norm = build("norm", spec.norm, hidden_size) if spec.feed_forward is not None else None
        self.feed_forward = build("feed_forward", spec.feed_forward, hidden_size) if spec.feed_forward is not None else None
        self.run_dtype = None
        # Small decode steps can run the whole layer as one persistent kernel (csrc/decode_layer.cu).  Off unless asked
        # for: measured on a B200 at the layer sizes of Qwen3-8B it is slower than the seven separate launches (a step's
        # time goes to the chain of dependent phases, which one kernel does not shorten).
        self.fuse_decode = False

    def tensor_needs(self):
        needs = {}
        for name, need in self.input_norm.tensor_needs().items():
            needs[self.pre_mixer + name] = need
        needs.update(self.mixer.tensor_needs())
        if self.feed_forward is not None:
            for name, need in self.post_norm.tensor_needs().items():
                needs[self.pre_ff + name] = need
            needs.update(self.feed_forward.tensor_needs())
        if self.token_shift is not None:
            needs[self.token_shift] = TensorNeed((self.hidden_size,))
        if self.input_conv is not None:
            needs[self.input_conv["tensor"]] = TensorNeed((self.hidden_size, int(self.input_conv["taps"])))
        return needs

    def load(self, tensors, rt: Runtime) -> None:
        sub = lambda p: {n[len(p):]: t for n, t in tensors.items() if n.startswith(p)}
        self.run_dtype = rt.dtype
        self.input_norm.load(sub(self.pre_mixer), rt)
        self.mixer.load(tensors, rt)
        if self.feed_forward is not None:
            self.post_norm.load(sub(self.pre_ff), rt)
            self.feed_forward.load(tensors, rt)
        if self.token_shift is not None:
            self.shift_mu = tensors[self.token_shift].to(device=rt.device, dtype=torch.float32).contiguous()
        if self.input_conv is not None:
            self.conv_taps = tensors[self.input_conv["tensor"]].to(device=rt.device, dtype=torch.float32).contiguous()
            self.conv_taps_t = self.conv_taps.t().contiguous()

    def cache_need(self):
        need = self.mixer.cache_need()
        if self.input_conv is not None:
            # (a convolution of one tap keeps nothing; its slot of one row is never touched)
            conv = StateNeed((max(int(self.input_conv["taps"]) - 1, 1), self.hidden_size), "float32")
            return {"mixer": need, "conv": conv} if need is not None else {"conv": conv}
        if self.token_shift is None:
            return need
        shift = StateNeed((self.hidden_size,), "float32")
        return {"mixer": need, "shift": shift} if need is not None else {"shift": shift}

    def _normed_shifted(self, x, delta, ctx, shift_view: CacheView, kw: dict, scale: dict):
        """The first norm's output with the token shift applied, in the parts' element type."""
        slots = ctx.state_slots[shift_view.group]
        out_dtype = kw.get("out_dtype", x.dtype)
        if ctx.max_q_len == 1 and ctx.num_tokens == ctx.num_seqs and isinstance(self.input_norm, LayerNorm) \
                and x.dtype == torch.float32:
            # every request brings one token: sum, norm, shift and the state's replacement in one launch
            out = torch.empty((x.shape[0], x.shape[1]), device=x.device, dtype=out_dtype)
            n = self.input_norm
            return ops.add_layernorm_shift(x, delta, n.weight, n.bias, n.eps, self.shift_mu, shift_view.state, slots, out,
                                           scale.get("delta_scale", 1.0))
        normed = self.input_norm.forward(x, delta, out_dtype=torch.float32, **scale)
        out = torch.empty(normed.shape, device=x.device, dtype=out_dtype)
        return ops.token_shift(normed, self.shift_mu, shift_view.state, slots, ctx.cu_q, ctx.seq_of_token, out)

    def _normed_conv(self, x, delta, ctx, conv_view: CacheView, kw: dict, scale: dict):
        """h + conv(h), h the first norm's output, in the parts' element type."""
        slots = ctx.state_slots[conv_view.group]
        out = torch.empty((x.shape[0], x.shape[1]), device=x.device, dtype=kw.get("out_dtype", x.dtype))
        n = self.input_norm
        if ctx.max_q_len == 1 and ctx.num_tokens == ctx.num_seqs and hasattr(n, "groups") and x.dtype == torch.float32 \
                and (delta is None or delta.dtype == out.dtype):
            # every request brings one token: sum, norm, convolution and the state's shift in one launch
            return ops.add_group_rmsnorm_conv(x, delta, n.weight, n.eps, n.groups, self.conv_taps, conv_view.state, slots, out,
                                              scale.get("delta_scale", 1.0))
        normed = n.forward(x, delta, out_dtype=torch.float32, **scale)
        return ops.input_conv(normed, self.conv_taps, conv_view.state, slots, ctx.cu_q, ctx.seq_of_token, out, self.conv_taps_t)

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in (self.input_norm, self.post_norm, self.mixer, self.feed_forward) if p is not None)

    def step_weight_bytes(self, num_tokens: int) -> int:
        """Weights that a step of ``num_tokens`` tokens reads: a part that reads only some of its weights (routed
        experts) says how many (``step_weight_bytes``); every other part reads all of them."""
        parts = (self.input_norm, self.post_norm, self.mixer, self.feed_forward)
        return sum(p.step_weight_bytes(num_tokens) if hasattr(p, "step_weight_bytes") else p.weight_bytes()
                   for p in parts if p is not None)

    def flops(self, num_tokens: int) -> float:
        return self.mixer.flops(num_tokens) + (self.feed_forward.flops(num_tokens) if self.feed_forward is not None else 0.0)

    def _fused_decode(self, x, delta, ctx, cache: CacheView | None):
        """A step of up to 16 one-token requests in bfloat16 runs the whole layer as one persistent kernel, when the
        parts are of the kinds that kernel knows (each part says so itself: ``decode_layer_spec``) and the sizes fit;
        None otherwise, and the parts run one by one."""
        if x.dtype != torch.bfloat16 or cache is None or not cache.writes or ctx.max_q_len != 1 or self.feed_forward is None:
            return None
        T = x.shape[0]
        if T > ops.DECODE_LAYER_TOKENS or T != ctx.num_seqs:
            return None
        specs = [getattr(part, "decode_layer_spec", lambda: None)()
                 for part in (self.input_norm, self.post_norm, self.mixer, self.feed_forward)]
        if any(s is None for s in specs):
            return None
        n1, n2, m, f = specs
        if n1["eps"] != n2["eps"] or cache.k_pages is None:
            return None
        if not ops.decode_layer_takes(T, x.shape[1], f["intermediate_size"], m["num_heads"], m["num_kv_heads"], m["head_dim"],
                                      cache.k_pages.shape[2], m["window"]):
            return None
        work = ctx.work.get(m["metadata_key"], {})
        out = torch.empty_like(x)
        ops.decode_layer(x, delta, out, n1["weight"], n2["weight"], n1["eps"], m["w_qkv"], m["w_o"], f["w_gate_up_pairs"],
                         f["w_down"], m["q_norm"], m["k_norm"], m["qk_eps"], m["cos_sin"], m["num_heads"], m["num_kv_heads"],
                         m["head_dim"], m["scale"], ctx.positions, ctx.seq_of_token, ctx.kv_len, ctx.block_tables[cache.group],
                         ctx.table_rows, cache.k_pages, cache.v_pages, int(work.get("max_dec_kv", 0)))
        return x, out

    def forward(self, x, delta, ctx, cache: CacheView | None):
        if self.fuse_decode:
            fused = self._fused_decode(x, delta, ctx, cache)
            if fused is not None:
                return fused
        # a stream kept in float32 beside parts that run in bfloat16: the norms are told the parts' element type
        kw = {"out_dtype": self.run_dtype} if self.run_dtype is not None and x.dtype != self.run_dtype else {}
        # (the pending output of the layer before belongs to a block of the same arrangement and factor)
        scale = {"delta_scale": self.residual_mult} if self.residual_mult != 1.0 else {}
        if self.token_shift is not None:
            h = self._normed_shifted(x, delta, ctx, cache.parts["shift"], kw, scale)
            cache = cache.parts.get("mixer")
        elif self.input_conv is not None:
            h = self._normed_conv(x, delta, ctx, cache.parts["conv"], kw, scale)
            cache = cache.parts.get("mixer")
        else:
            h = self.input_norm.forward(x, delta, **kw, **scale)
        a = self.mixer.forward(h, ctx, cache)
        if self.feed_forward is None:
            return x, a
        h = self.post_norm.forward(x, a, **kw, **scale)
        return x, self.feed_forward.forward(h, ctx)


class NormedDelta:
    """A part's output that has not joined the stream yet, with the norm it passes through on its way in:
    x += tensor / sqrt(mean(tensor^2) + eps) * weight.  The sum is made by the kernel of whatever reads the stream
    next (the next block's first norm), or by ``settle``."""

    __slots__ = ("tensor", "weight", "eps")

    def __init__(self, tensor: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
        self.tensor, self.weight, self.eps = tensor, weight, eps


def settle(x: torch.Tensor, delta):
    """(x, None) with whatever was pending added to the stream x."""
    if isinstance(delta, NormedDelta):
        ops.add_normed_rmsnorm(x, delta.tensor, delta.weight, delta.eps, None, 0.0, None)
        return x, None
    if delta is not None:
        raise ValueError("settle: only an output with a norm of its own is added here; others join in the next norm")
    return x, None


@register("block", "sandwich")
class SandwichBlock:
    """x += norm_1b(mixer(norm_1(x))); x += norm_2b(feed_forward(norm_2(x))): an RMS norm in front of and behind each
    part, over a float32 residual stream.  A part's output travels as a ``NormedDelta``: its norm, the sum into the
    stream and the next part's input norm are one kernel (``ops.add_normed_rmsnorm``), so the stream is read and
    written once per part.  The four norms are ``LayerSpec.norm`` (kind ``rmsnorm``) under the names
    ``norm_prefixes`` (in front) and ``options["post_norms"]`` (behind)."""

    residual_mult = 1.0

    def __init__(self, spec: LayerSpec, hidden_size: int) -> None:
        self.hidden_size = hidden_size
        self.prefix = spec.prefix
        self.pre_mixer, self.pre_ff = spec.norm_prefixes
        self.post_mixer, self.post_ff = spec.options.get("post_norms", ("norm1b", "norm2b"))
        has_ff = spec.feed_forward is not None
        self.input_norm = build("norm", spec.norm, hidden_size)
        self.mixer_out_norm = build("norm", spec.norm, hidden_size)
        self.mixer = build("mixer", spec.mixer, hidden_size)
        self.post_norm = build("norm", spec.norm, hidden_size) if has_ff else None
        self.ff_out_norm = build("norm", spec.norm, hidden_size) if has_ff else None
        self.feed_forward = build("feed_forward", spec.feed_forward, hidden_size) if has_ff else None
        for n in (self.input_norm, self.mixer_out_norm, self.post_norm, self.ff_out_norm):
            if n is not None and not (hasattr(n, "weight") and hasattr(n, "eps") and not hasattr(n, "bias")):
                raise ValueError("the sandwich block is built for RMS norms")
        self.run_dtype = None

    def _norms(self):
        return ((self.pre_mixer, self.input_norm), (self.post_mixer, self.mixer_out_norm), (self.pre_ff, self.post_norm),
                (self.post_ff, self.ff_out_norm))

    def tensor_needs(self):
        needs = {}
        for prefix, norm in self._norms():
            if norm is not None:
                for name, need in norm.tensor_needs().items():
                    needs[prefix + name] = need
        needs.update(self.mixer.tensor_needs())
        if self.feed_forward is not None:
            needs.update(self.feed_forward.tensor_needs())
        return needs

    def load(self, tensors, rt: Runtime) -> None:
        self.run_dtype = rt.dtype
        for prefix, norm in self._norms():
            if norm is not None:
                norm.load({n[len(prefix):]: t for n, t in tensors.items() if n.startswith(prefix)
                           and n[len(prefix):] in norm.tensor_needs()}, rt)
        self.mixer.load(tensors, rt)
        if self.feed_forward is not None:
            self.feed_forward.load(tensors, rt)

    def cache_need(self):
        return self.mixer.cache_need()

    def weight_bytes(self) -> int:
        parts = [n for _, n in self._norms()] + [self.mixer, self.feed_forward]
        return sum(p.weight_bytes() for p in parts if p is not None)

    def flops(self, num_tokens: int) -> float:
        return self.mixer.flops(num_tokens) + (self.feed_forward.flops(num_tokens) if self.feed_forward is not None else 0.0)

    def _enter(self, x, delta, norm):
        """The pending output joins the stream; returns ``norm`` of the stream in the parts' element type."""
        if isinstance(delta, NormedDelta):
            out = torch.empty(x.shape, device=x.device, dtype=self.run_dtype)
            return ops.add_normed_rmsnorm(x, delta.tensor, delta.weight, delta.eps, norm.weight, norm.eps, out)
        return norm.forward(x, delta, out_dtype=self.run_dtype)

    def forward(self, x, delta, ctx, cache: CacheView | None):
        if x.dtype != torch.float32:
            raise ValueError("the sandwich block is built for a float32 residual stream (ModelPlan.residual_dtype)")
        h = self._enter(x, delta, self.input_norm)
        a = NormedDelta(self.mixer.forward(h, ctx, cache), self.mixer_out_norm.weight, self.mixer_out_norm.eps)
        if self.feed_forward is None:
            return x, a
        h = self._enter(x, a, self.post_norm)
        return x, NormedDelta(self.feed_forward.forward(h, ctx), self.ff_out_norm.weight, self.ff_out_norm.eps)
