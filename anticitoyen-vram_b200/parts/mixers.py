"""Token mixers over the paged cache: attention, differential attention, and two mixers side by side."""

from __future__ import annotations

import torch

from ..cache.manager import PagedNeed
from ..kernels import ops
from ..weights.needs import TensorNeed
from .base import CacheView, Mixer, Runtime, StepMetadata
from .linear import Linear
from .plan import PartSpec
from .position import NoPosition
from .registry import build, register


@register("mixer", "attention")
class Attention(Mixer):
    """Grouped-query attention over the paged cache, with optional per-head RMS norm
    of q and k before the position encoding (acvram/engine/attention.py:142-145,
    290-365).  q-head h reads kv-head h // (heads/kv_heads); scale defaults to
    head_dim^-1/2 (acvram/engine/attention.py:149-151); ``window`` > 0 limits a query
    to the last ``window`` keys.  Tensor names are the Hugging Face ones, kept by the
    reference (acvram/engine/loader.py:1013-1023).  ``bias``: True, the four projections have
    biases; False, none; None, those that the weight file holds (acvram/engine/loader.py:269-270).

    ``value_dim``: elements of a value vector (and of a head's output) where they differ from ``head_dim``.
    ``keep_first`` > 0 (with a window): the first ``keep_first`` tokens of a request stay visible to every later query,
    at their own positions.  ``names``: the four projections' tensor names behind ``prefix`` ({"q": name, ...}; biases
    are then read only under names given as "q.bias" ...).  ``out_scale``: a constant on the mixer's output, for a mixer
    whose output enters a weighted sum; it is applied to the values as they are written to their pages.

    ``qk_norm_weights`` False: q and k are brought to unit RMS and nothing else (no weight tensors).
    ``score``: more steps between the score's product and the softmax, each optional, all 32-bit:
        s_g = <q_g, k> * scale * temp[g]           "temp": tensor [heads]
        s_g = cap * tanh(s_g / cap)                 "softcap": cap
        s_g += rel[bucket(i - j)][g]                "rel": tensor [rows, heads] (rows: whatever the file holds), "far":
                                                    the distance from which every key reads the last row; rows/2 single
                                                    distances first, the rest spread evenly over ln(distance)
        m_h = sum_g talk[h][g] s_g                  "talk": tensor [heads, heads]; the softmax is taken over m_h
    (tensor names behind ``prefix``).  Such a layer runs ``ops.attention_mixed``.

    Steps that span more than a head, each optional, all 32-bit (``ops.qkv_prepare`` between projection and attention):
    ``qk_norm_scope`` "all": one root mean square over the whole of q (and one over the whole of k) with a weight for
    every element (names["q_norm"], names["k_norm"]) instead of a norm per head; ``value_norm_eps``: every value head is
    divided by its root mean square before it is kept; ``q_temp`` = (coef, every): the query at position p is multiplied
    by 1 + coef ln(floor((p + 1) / every) + 1); ``value_share`` = {"key", "role", "tensor"}: the layer with role "source"
    leaves its values (as it keeps them) under ``key`` for the later layers of the step, a layer with role "mix" keeps
    (1 - lambda) v + lambda v_source, lambda its own number in ``tensor``.
    ``sink``: the softmax's denominator also holds exp(sink_h), a score with no key and no value: a tensor's name (one
    learned number per query head) or a constant for all heads.  ``slope_rate`` r: slope_h (i - j) is taken off the score
    of query i and key j, slope_h = 2^(-r (h + 1) / heads)."""

    ROLES = ("q", "k", "v", "o")

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, position: PartSpec,
                 qk_norm_eps: float | None = None, scale: float | None = None, window: int = 0,
                 prefix: str = "self_attn.", bias: bool | None = None, value_dim: int | None = None, keep_first: int = 0,
                 names: dict | None = None, out_scale: float = 1.0, qk_norm_weights: bool = True,
                 score: dict | None = None, qk_norm_scope: str = "head", value_norm_eps: float | None = None,
                 q_temp: tuple | None = None, value_share: dict | None = None, sink: str | float | None = None,
                 slope_rate: float | None = None) -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} kv heads")
        if qk_norm_scope not in ("head", "all"):
            raise ValueError(f"attention: qk_norm_scope is 'head' or 'all', got {qk_norm_scope!r}")
        if value_share is not None and (value_share.get("role") not in ("source", "mix") or "key" not in value_share
                                        or (value_share["role"] == "mix" and "tensor" not in value_share)):
            raise ValueError("attention: value_share is {'key', 'role': 'source' | 'mix', 'tensor' (of a 'mix')}")
        self.qk_norm_scope = qk_norm_scope
        self.value_norm_eps = float(value_norm_eps) if value_norm_eps is not None else None
        self.q_temp = (float(q_temp[0]), int(q_temp[1])) if q_temp else None
        self.value_share = dict(value_share) if value_share else None
        self.sink = sink
        self.slope_rate = float(slope_rate) if slope_rate is not None else None
        self.sinks = self.slopes = None
        self.share_weight = 0.0
        # steps that one warp per (token, head) cannot make: they run in a kernel that holds a token's whole projection
        self.wide = qk_norm_scope == "all" and qk_norm_eps is not None or self.value_norm_eps is not None \
            or self.q_temp is not None or self.value_share is not None
        if (self.wide or sink is not None or slope_rate is not None) and (score or keep_first or out_scale != 1.0):
            raise ValueError("attention: sinks, slopes and the steps over whole projections are not built beside score steps, "
                             "kept first tokens or an output factor")
        self.hidden_size = hidden_size
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.qk_norm_weights = bool(qk_norm_weights)
        self.score = dict(score) if score else None
        if self.score is not None:
            unknown = set(self.score) - {"temp", "softcap", "rel", "far", "talk"}
            if unknown or ("rel" in self.score) != ("far" in self.score):
                raise ValueError(f"attention score steps: unknown {sorted(unknown)}, or 'rel' without 'far'")
            if keep_first:
                raise ValueError("attention: kept first tokens beside score steps are not built")
        self.temp = self.rel = self.talk = self.bucket_of = None
        self.rel_last = 0
        self.value_dim = int(value_dim) if value_dim else head_dim
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.qk_norm_eps = qk_norm_eps
        self.window = int(window)
        self.keep_first = int(keep_first) if self.window > 0 else 0
        self.out_scale = float(out_scale)
        self.prefix = prefix
        self.bias = bias
        if names is None:
            self.names = {r: f"{r}_proj.weight" for r in self.ROLES}
            self.names.update({r + ".bias": f"{r}_proj.bias" for r in self.ROLES})
        else:
            self.names = dict(names)
        self.position = build("position", position, hidden_size)
        self.q_size = num_heads * head_dim
        self.kv_size = num_kv_heads * head_dim
        self.v_size = num_kv_heads * self.value_dim
        self.in_size = self.q_size + self.kv_size + self.v_size      # columns of the stacked input projection
        self.inner_size = num_heads * self.value_dim                 # columns in front of the output projection

    def cache_need(self):
        return PagedNeed(self.num_kv_heads, self.head_dim, self.window,
                         self.value_dim if self.value_dim != self.head_dim else 0, 0, self.keep_first)

    # what the attention kernels want of a step beside the generic batch: their work lists.  One set serves every
    # attention layer of a model (the lists depend on the step's requests only), hence one key.
    metadata_key = "attention"

    def step_metadata(self, q_lens, kv_lens, cu_q) -> StepMetadata:
        return StepMetadata(*ops.attention_work(q_lens, kv_lens, cu_q))

    def decode_metadata(self, padded: int, max_kv: int) -> StepMetadata:
        return StepMetadata(*ops.attention_work_decode(padded, max_kv))

    def tensor_needs(self):
        H = self.hidden_size
        needs = {}
        for role, n_out, n_in in (("q", self.q_size, H), ("k", self.kv_size, H), ("v", self.v_size, H),
                                  ("o", H, self.inner_size)):
            needs[self.prefix + self.names[role]] = TensorNeed((n_out, n_in))
            if self.bias is not False and role + ".bias" in self.names:
                needs[self.prefix + self.names[role + ".bias"]] = TensorNeed((n_out,), "bias", optional=self.bias is None)
        if self.qk_norm_eps is not None and self.qk_norm_weights:
            whole = self.qk_norm_scope == "all"
            needs[self.prefix + self.names.get("q_norm", "q_norm.weight")] = TensorNeed((self.q_size if whole else self.head_dim,), "norm")
            needs[self.prefix + self.names.get("k_norm", "k_norm.weight")] = TensorNeed((self.kv_size if whole else self.head_dim,), "norm")
        if isinstance(self.sink, str):
            needs[self.prefix + self.sink] = TensorNeed((self.num_heads,), "norm")
        if self.value_share is not None and "tensor" in self.value_share:
            # (the source layer's number is read by nobody; a file may carry it all the same)
            needs[self.prefix + self.value_share["tensor"]] = TensorNeed((), "norm", optional=self.value_share["role"] == "source")
        if self.score is not None:
            NH = self.num_heads
            for key, shape, role in (("temp", (NH,), "norm"), ("rel", (-1, NH), "matrix"), ("talk", (NH, NH), "matrix")):
                if key in self.score:
                    needs[self.prefix + self.score[key]] = TensorNeed(shape, role)
        for name, need in self.position.tensor_needs().items():
            needs[self.prefix + name] = need
        return needs

    def load(self, tensors, rt: Runtime) -> None:
        w = lambda r: tensors[self.prefix + self.names[r]].to(device=rt.device, dtype=rt.dtype)

        def b(role):
            name = self.prefix + self.names.get(role + ".bias", "\0")
            return tensors[name].to(device=rt.device, dtype=torch.float32) if name in tensors else None

        self.qkv = Linear.stacked([w("q"), w("k"), w("v")], [b("q"), b("k"), b("v")])
        self.o = Linear(w("o"), b("o"))
        self.q_norm = self.k_norm = None
        f = lambda n: tensors[n].to(device=rt.device, dtype=torch.float32).contiguous()
        if self.qk_norm_eps is not None and self.qk_norm_weights:
            self.q_norm = f(self.prefix + self.names.get("q_norm", "q_norm.weight"))
            self.k_norm = f(self.prefix + self.names.get("k_norm", "k_norm.weight"))
        elif self.qk_norm_eps is not None and self.qk_norm_scope == "all":
            self.q_norm = torch.ones(self.q_size, device=rt.device, dtype=torch.float32)
            self.k_norm = torch.ones(self.kv_size, device=rt.device, dtype=torch.float32)
        elif self.qk_norm_eps is not None:
            self.q_norm = self.k_norm = torch.ones(self.head_dim, device=rt.device, dtype=torch.float32)
        if isinstance(self.sink, str):
            self.sinks = f(self.prefix + self.sink)
        elif self.sink is not None:
            self.sinks = torch.full((self.num_heads,), float(self.sink), device=rt.device, dtype=torch.float32)
        if self.slope_rate is not None:
            steps = torch.arange(1, self.num_heads + 1, dtype=torch.float64)
            self.slopes = torch.exp2(-self.slope_rate * steps / self.num_heads).to(device=rt.device, dtype=torch.float32)
        if self.value_share is not None and self.value_share["role"] == "mix":
            self.share_weight = float(tensors[self.prefix + self.value_share["tensor"]].to(torch.float64))
        if self.score is not None:
            sc = self.score
            self.temp = f(self.prefix + sc["temp"]) if "temp" in sc else None
            self.talk = f(self.prefix + sc["talk"]) if "talk" in sc else None
            if "rel" in sc:
                self.rel = f(self.prefix + sc["rel"])
                buckets, self.rel_last = ops.distance_buckets(self.rel.shape[0], float(sc["far"]))
                self.bucket_of = buckets.to(rt.device)
        self.position.load({n[len(self.prefix):]: t for n, t in tensors.items() if n.startswith(self.prefix)}, rt)

    def decode_layer_spec(self):
        """What the fused decode-layer kernel needs of this mixer (it knows rotary positions over the whole head,
        applied by table, and no biases)."""
        rotary = self.position.rotary_table()
        if self.qkv.bias is not None or self.o.bias is not None or rotary is None or rotary.shape[1] != self.head_dim \
                or self.value_dim != self.head_dim or self.keep_first or self.out_scale != 1.0 or self.wide \
                or self.sinks is not None or self.slopes is not None or self.score is not None:
            return None
        return {"num_heads": self.num_heads, "num_kv_heads": self.num_kv_heads, "head_dim": self.head_dim,
                "window": self.window, "scale": self.scale, "w_qkv": self.qkv.weight, "w_o": self.o.weight,
                "q_norm": self.q_norm, "k_norm": self.k_norm, "qk_eps": self.qk_norm_eps or 0.0, "cos_sin": rotary,
                "metadata_key": self.metadata_key}

    # ---- cost of a step
    def extra_weight_bytes(self) -> int:
        return sum(t.numel() * 4 for t in (self.q_norm, self.k_norm, self.temp, self.rel, self.talk, self.sinks) if t is not None)

    def _attend(self, qkv, out, ctx, cache: CacheView, table) -> None:
        """From normed, positioned queries (the first columns of ``qkv``) and the pages to the heads' outputs."""
        NH, NKV, D, DV = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        if self.score is not None:
            ops.attention_mixed(qkv, out, cache.k_pages, cache.v_pages, ctx.positions, ctx.seq_of_token, table, NH, NKV, D,
                                self.scale, self.window, table_rows=ctx.table_rows, value_dim=DV, temp=self.temp,
                                softcap=float(self.score.get("softcap", 0.0) or 0.0), rel=self.rel, bucket_of=self.bucket_of,
                                last_row=self.rel_last, talk=self.talk, ctx=ctx, work=ctx.work.get(self.metadata_key))
            return
        ops.attention(qkv, out, cache.k_pages, cache.v_pages, ctx, table, NH, NKV, D, self.scale, self.window,
                      work=ctx.work[self.metadata_key], value_dim=DV, keep_first=self.keep_first, sinks=self.sinks,
                      slopes=self.slopes)

    def _prepare(self, qkv, ctx, table, rows, kp, vp) -> None:
        """The steps over a token's whole projection, rotation and append in one launch."""
        share = self.value_share
        shared_values = None
        if share is not None:
            T = qkv.shape[0]
            if share["role"] == "source":
                shared_values = ctx.shared[share["key"]] = torch.empty((T, self.v_size), device=qkv.device, dtype=torch.float32)
            else:
                shared_values = ctx.shared.get(share["key"])
                if shared_values is None or shared_values.shape != (T, self.v_size):
                    raise ValueError(f"attention: no layer before this one left values of this size under '{share['key']}'")
        whole = self.qk_norm_scope == "all" and self.qk_norm_eps is not None
        if self.q_norm is not None and not whole:
            # a norm per head beside steps over the whole projection: the per-head kernel first (no rotation, no append)
            ops.qk_norm_rope_append(qkv, self.num_heads, self.num_kv_heads, self.head_dim, self.q_norm, self.k_norm,
                                    self.qk_norm_eps, None, ctx.positions, ctx.seq_of_token, None, None, None,
                                    value_dim=self.value_dim if self.value_dim != self.head_dim else 0)
        rotary = self.position.rotary_table()
        if rotary is None and not isinstance(self.position, NoPosition):
            raise ValueError("attention: the steps over whole projections take rotary positions by table, or none")
        ops.qkv_prepare(qkv, self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim,
                        self.q_norm if whole else None, self.k_norm if whole else None, self.qk_norm_eps or 0.0, rotary,
                        ctx.positions, ctx.seq_of_token, table if kp is not None else None, kp, vp, table_rows=rows,
                        temp=self.q_temp, value_norm_eps=self.value_norm_eps, shared_values=shared_values,
                        share=share["role"] if share else None, share_weight=self.share_weight)

    def weight_bytes(self) -> int:
        return self.qkv.weight_bytes() + self.o.weight_bytes() + self.extra_weight_bytes()

    def flops(self, num_tokens: int) -> float:
        return self.qkv.flops(num_tokens) + self.o.flops(num_tokens)

    def _seen(self, q: int, kv: int) -> float:
        """Keys that the q queries at the end of a context of kv tokens see, summed over the queries."""
        full = q * (kv - q) + q * (q + 1) / 2
        if self.window <= 0:
            return full
        # inside the window, plus the kept first keys that the window has passed
        return sum(min(self.window, p + 1) + min(self.keep_first, max(0, p + 1 - self.window)) for p in range(kv - q, kv))

    def mixing_flops(self, q_lens, kv_lens) -> float:
        return 2.0 * self.num_heads * (self.head_dim + self.value_dim) * sum(self._seen(q, kv) for q, kv in zip(q_lens, kv_lens))

    def cache_bytes_read(self, q_lens, kv_lens, itemsize: int) -> int:
        keys = sum(min(kv, self.window + q - 1 + self.keep_first) if self.window > 0 else kv for q, kv in zip(q_lens, kv_lens))
        return keys * (self.kv_size + self.v_size) * itemsize

    def mix(self, qkv, ctx, cache: CacheView, out) -> None:
        """From the stacked projection ``qkv`` ([T, in_size], dense rows at any stride; its queries are changed in
        place) to the heads' outputs ``out`` ([T, inner_size], likewise): norm, positions, append, attention."""
        NH, NKV, D, DV = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        table = ctx.block_tables[cache.group]
        rows = ctx.table_rows
        kp, vp = (cache.k_pages, cache.v_pages) if cache.writes else (None, None)
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 0.0
        rotary = self.position.rotary_table()
        extra = {"value_dim": DV, "v_scale": self.out_scale} if (DV != D or self.out_scale != 1.0) else {}
        if self.wide:
            self._prepare(qkv, ctx, table, rows, kp, vp)
        elif rotary is not None:
            ops.qk_norm_rope_append(qkv, NH, NKV, D, self.q_norm, self.k_norm, eps, rotary, ctx.positions,
                                    ctx.seq_of_token, table if kp is not None else None, kp, vp, table_rows=rows, **extra)
        elif isinstance(self.position, NoPosition):
            # nothing happens between norm and append: one launch for both
            ops.qk_norm_rope_append(qkv, NH, NKV, D, self.q_norm, self.k_norm, eps, None, ctx.positions,
                                    ctx.seq_of_token, table if kp is not None else None, kp, vp, table_rows=rows, **extra)
        else:
            if self.q_norm is not None:
                ops.qk_norm_rope_append(qkv, NH, NKV, D, self.q_norm, self.k_norm, eps, None, ctx.positions,
                                        ctx.seq_of_token, None, None, None, **extra)
            T = qkv.shape[0]
            self.position.apply(qkv[:, :self.q_size].unflatten(1, (NH, D)),
                                qkv[:, self.q_size:self.q_size + self.kv_size].unflatten(1, (NKV, D)), ctx)
            if kp is not None:
                ops.qk_norm_rope_append(qkv, NH, NKV, D, None, None, 0.0, None, ctx.positions, ctx.seq_of_token,
                                        table, kp, vp, table_rows=rows, **extra)
        self._attend(qkv, out, ctx, cache, table)

    def forward(self, h, ctx, cache: CacheView):
        NH, NKV, D = self.num_heads, self.num_kv_heads, self.head_dim
        if self.value_dim != D or self.out_scale != 1.0 or self.score is not None or isinstance(self.position, NoPosition) \
                or self.wide or self.sinks is not None or self.slopes is not None:
            qkv = self.qkv(h)
            out = torch.empty((qkv.shape[0], self.inner_size), device=h.device, dtype=h.dtype)
            self.mix(qkv, ctx, cache, out)
            return self.o(out)
        table = ctx.block_tables[cache.group]
        rows = ctx.table_rows
        kp, vp = (cache.k_pages, cache.v_pages) if cache.writes else (None, None)
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 0.0
        rotary = self.position.rotary_table()
        if rotary is not None and self.qkv.bias is None and ops.gemm_tc_qkv_takes(h, self.qkv.weight, D, rotary, kp):
            # a few tokens: norm, rotation and append ride on the projection's kernel as its tile leaves
            qkv = torch.empty((h.shape[0], self.qkv.out_features), device=h.device, dtype=h.dtype)
            ops.gemm_tc_qkv(h, self.qkv.weight, qkv, NH, NKV, D, self.q_norm, self.k_norm, eps, rotary, ctx.positions,
                            ctx.seq_of_token, table, kp, vp, static_weights=True, table_rows=rows)
        elif rotary is not None:
            qkv = self.qkv(h)
            ops.qk_norm_rope_append(qkv, NH, NKV, D, self.q_norm, self.k_norm, eps, rotary, ctx.positions,
                                    ctx.seq_of_token, table if kp is not None else None, kp, vp, table_rows=rows)
        else:
            # another position encoding: norm, then the part's own change of q and k, then the append
            qkv = self.qkv(h)
            if self.q_norm is not None:
                ops.qk_norm_rope_append(qkv, NH, NKV, D, self.q_norm, self.k_norm, eps, None, ctx.positions,
                                        ctx.seq_of_token, None, None, None)
            T = qkv.shape[0]
            self.position.apply(qkv[:, :self.q_size].view(T, NH, D),
                                qkv[:, self.q_size:self.q_size + self.kv_size].view(T, NKV, D), ctx)
            if kp is not None:
                ops.qk_norm_rope_append(qkv, NH, NKV, D, None, None, 0.0, None, ctx.positions, ctx.seq_of_token,
                                        table, kp, vp, table_rows=rows)
        out = torch.empty((qkv.shape[0], self.q_size), device=h.device, dtype=h.dtype)
        ops.attention(qkv, out, cache.k_pages, cache.v_pages, ctx, table, NH, NKV, D, self.scale, self.window,
                      work=ctx.work[self.metadata_key], **({"keep_first": self.keep_first} if self.keep_first else {}))
        return self.o(out)


@register("mixer", "diff_attention")
class DiffAttention(Mixer):
    """Differential attention over the paged cache: every head has two query vectors and, per kv-head, two key
    vectors of ``dim`` elements, [map 1 | map 2], and one value vector of ``value_dim``.  Each map is a softmax
    attention of its own over the same values; a head's output is

        o = o1 - lambda * o2,    lambda = exp(<lq1, lk1>) - exp(<lq2, lk2>) + diff      (one number for the layer)
        out = o / sqrt(mean(o^2) + eps) * (1 - diff)                                     (over the head, no weight)

    Query and key vectors are brought to unit RMS and multiplied by a weight of ``dim`` elements that all heads and
    both maps share (``norm_eps`` None: no norm).  No position encoding: order enters through the mask alone, which
    is causal, limited to the last ``window`` keys (``window`` > 0) and/or to the query's own chunk of ``chunk``
    positions counted from the request's position 0 (``chunk`` > 0).  With ``own_kv`` false the layer has no key and
    value projections and reads the cache slot that another layer writes (the plan's schedule says which).

    Scores, both softmaxes, lambda and the head norm are 32-bit in every run precision.  ``names``: the tensors'
    names behind ``prefix`` (default: q, k, v, o, q.norm, k.norm, lq1, lk1, lq2, lk2)."""

    NAMES = {n: n for n in ("q", "k", "v", "o", "q.norm", "k.norm", "lq1", "lk1", "lq2", "lk2")}
    metadata_key = "attention"      # the work lists of the attention kernels serve these layers as well

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, value_dim: int, scale: float | None,
                 diff: float, norm_eps: float | None, chunk: int = 0, window: int = 0, own_kv: bool = True,
                 prefix: str = "mix.", names: dict | None = None) -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} kv heads")
        self.hidden_size = hidden_size
        self.num_heads, self.num_kv_heads, self.dim, self.value_dim = num_heads, num_kv_heads, dim, value_dim
        self.scale = float(scale) if scale is not None else dim ** -0.5
        self.diff = float(diff)
        self.norm_eps = norm_eps
        self.chunk, self.window = int(chunk), int(window)
        self.own_kv = own_kv
        self.prefix = prefix
        self.names = {**self.NAMES, **(names or {})}
        self.q_size = num_heads * 2 * dim
        self.k_size = num_kv_heads * 2 * dim
        self.v_size = num_kv_heads * value_dim
        self.lam = self.diff

    def _n(self, role: str) -> str:
        return self.prefix + self.names[role]

    def cache_need(self):
        return PagedNeed(self.num_kv_heads, 2 * self.dim, self.window,
                         self.value_dim if self.value_dim != 2 * self.dim else 0, self.chunk)

    def step_metadata(self, q_lens, kv_lens, cu_q) -> StepMetadata:
        return StepMetadata(*ops.attention_work(q_lens, kv_lens, cu_q))

    def decode_metadata(self, padded: int, max_kv: int) -> StepMetadata:
        return StepMetadata(*ops.attention_work_decode(padded, max_kv))

    def tensor_needs(self):
        H = self.hidden_size
        needs = {self._n("q"): TensorNeed((self.q_size, H)), self._n("o"): TensorNeed((H, self.num_heads * self.value_dim))}
        if self.own_kv:
            needs[self._n("k")] = TensorNeed((self.k_size, H))
            needs[self._n("v")] = TensorNeed((self.v_size, H))
        if self.norm_eps is not None:
            needs[self._n("q.norm")] = TensorNeed((self.dim,), "norm")
            if self.own_kv:
                needs[self._n("k.norm")] = TensorNeed((self.dim,), "norm")
        for role in ("lq1", "lk1", "lq2", "lk2"):
            needs[self._n(role)] = TensorNeed((self.dim,))
        return needs

    def load(self, tensors, rt: Runtime) -> None:
        w = lambda role: tensors[self._n(role)].to(device=rt.device, dtype=rt.dtype)
        f = lambda role: tensors[self._n(role)].to(device=rt.device, dtype=torch.float32).contiguous()
        self.qkv = Linear.stacked([w("q"), w("k"), w("v")]) if self.own_kv else Linear(w("q"))
        self.o = Linear(w("o"))
        self.q_norm = f("q.norm") if self.norm_eps is not None else None
        self.k_norm = f("k.norm") if self.norm_eps is not None and self.own_kv else None
        # lambda is a constant of the layer's weights: folded once, in 32-bit, when they are loaded
        v = {role: tensors[self._n(role)].to(torch.float32) for role in ("lq1", "lk1", "lq2", "lk2")}
        self.lam = (float(torch.exp((v["lq1"] * v["lk1"]).sum())) - float(torch.exp((v["lq2"] * v["lk2"]).sum()))
                    + self.diff)

    # ---- cost of a step
    def weight_bytes(self) -> int:
        norms = sum(t.numel() * 4 for t in (self.q_norm, self.k_norm) if t is not None)
        return self.qkv.weight_bytes() + self.o.weight_bytes() + norms

    def flops(self, num_tokens: int) -> float:
        return self.qkv.flops(num_tokens) + self.o.flops(num_tokens)

    def _seen(self, q: int, kv: int) -> float:
        """Keys that the q queries at the end of a context of kv tokens see, summed over the queries."""
        total = 0
        for p in range(kv - q, kv):
            lo = p // self.chunk * self.chunk if self.chunk > 0 else 0
            if self.window > 0:
                lo = max(lo, p - self.window + 1)
            total += p - lo + 1
        return float(total)

    def mixing_flops(self, q_lens, kv_lens) -> float:
        # two score products of dim and two weighted sums of value_dim for every (query, key) pair of a head
        return 4.0 * self.num_heads * (self.dim + self.value_dim) * sum(self._seen(q, kv) for q, kv in zip(q_lens, kv_lens))

    def cache_bytes_read(self, q_lens, kv_lens, itemsize: int) -> int:
        keys = 0
        for q, kv in zip(q_lens, kv_lens):
            need = PagedNeed(1, 1, self.window, 0, self.chunk)
            keys += kv - need.first_needed(kv - q)
        return keys * (self.k_size + self.v_size) * itemsize

    def forward(self, h, ctx, cache: CacheView):
        NH, NKV, D, DV = self.num_heads, self.num_kv_heads, self.dim, self.value_dim
        if cache.writes != self.own_kv:
            raise ValueError("a diff_attention layer writes its cache slot exactly when it has key and value projections")
        table = ctx.block_tables[cache.group]
        rows = ctx.table_rows
        qkv = self.qkv(h)
        T = qkv.shape[0]
        eps = self.norm_eps if self.norm_eps is not None else 0.0
        pages = (table, cache.k_pages, cache.v_pages) if self.own_kv else (None, None, None)
        out = torch.empty((T, NH * DV), device=h.device, dtype=h.dtype)
        work = ctx.work.get(self.metadata_key)
        if work is not None and ops.diff_attention_as_heads_takes(h.dtype, NH, NKV, D, DV):
            # key and value rows of one size that the tensor-core attention kernels take: each map runs as a head of its
            # own (its query vector padded with zeros to a key row) on the prompt and decode kernels of plain attention,
            # under the same mask; a small kernel then combines the two maps of every head
            wide = torch.empty((T, 2 * NH * 2 * D), device=h.device, dtype=h.dtype)
            ops.heads_norm_append(qkv, 2 * NH, 2 * NKV, NKV, D, DV, self.q_norm, self.k_norm, eps, ctx.positions,
                                  ctx.seq_of_token, *pages, table_rows=rows, q_out=wide)
            # the maps leave the attention kernels as float: the difference of two nearly equal maps keeps its digits
            maps = torch.empty((T, 2 * NH * DV), device=h.device, dtype=torch.float32)
            ops.attention(wide, maps, cache.k_pages, cache.v_pages, ctx, table, 2 * NH, NKV, 2 * D, self.scale, self.window,
                          work=work, chunk=self.chunk)
            ops.diff_combine(maps, out, NH, DV, self.lam, eps, 1.0 - self.diff)
            return self.o(out)
        ops.heads_norm_append(qkv, 2 * NH, 2 * NKV, NKV, D, DV, self.q_norm, self.k_norm, eps, ctx.positions,
                              ctx.seq_of_token, *pages, table_rows=rows)
        ops.diff_attention(qkv, out, cache.k_pages, cache.v_pages, ctx, table, NH, NKV, D, DV, self.scale, self.lam, eps,
                           1.0 - self.diff, self.window, self.chunk, work=work)
        return self.o(out)


@register("mixer", "parallel")
class ParallelMixers(Mixer):
    """Two mixers side by side over the same input; the result is the sum of their outputs (each mixer applies its own
    constant, ``out_scale`` of its parameters, so that the sum is weighted).  Each keeps what it keeps: the cache view
    has the parts "left" and "right".

    Both sides must be mixers that can be driven from outside their projections: ``in_size``, ``inner_size``, ``qkv``
    and ``o`` (their stacked input projection and their output projection) and ``mix(projected, ctx, cache, out)``.
    The two input projections then run as one product over the shared input, and the two output projections as one
    product over the heads' outputs laid side by side, [left | right] @ [W_left | W_right]^T, which is the sum."""

    def __init__(self, hidden_size: int, left: PartSpec, right: PartSpec) -> None:
        self.hidden_size = hidden_size
        self.left = build("mixer", left, hidden_size)
        self.right = build("mixer", right, hidden_size)
        for side in (self.left, self.right):
            if not all(hasattr(side, a) for a in ("in_size", "inner_size", "mix")):
                raise ValueError(f"a '{side.kind}' mixer cannot stand beside another one (it offers no mix())")

    def metadata_providers(self) -> dict:
        return {**self.right.metadata_providers(), **self.left.metadata_providers()}

    def cache_need(self):
        needs = {"left": self.left.cache_need(), "right": self.right.cache_need()}
        return {k: v for k, v in needs.items() if v is not None} or None

    def tensor_needs(self):
        return {**self.left.tensor_needs(), **self.right.tensor_needs()}

    def load(self, tensors, rt: Runtime) -> None:
        self.left.load(tensors, rt)
        self.right.load(tensors, rt)
        l, r = self.left, self.right
        self.inp = Linear.stacked([l.qkv.weight, r.qkv.weight], [l.qkv.bias, r.qkv.bias])
        if (l.o.bias is None) != (r.o.bias is None):
            bias = (l.o.bias if l.o.bias is not None else r.o.bias)
        else:
            bias = l.o.bias + r.o.bias if l.o.bias is not None else None
        self.o = Linear(torch.cat([l.o.weight, r.o.weight], dim=1), bias)
        # the sides' own copies of the stacked weights are not read again
        l.qkv = l.o = r.qkv = r.o = None

    def weight_bytes(self) -> int:
        # the sides' projections are the two stacked products here; what else a side reads (norm weights) it reports itself
        extra = sum(getattr(side, "extra_weight_bytes", lambda: 0)() for side in (self.left, self.right))
        return self.inp.weight_bytes() + self.o.weight_bytes() + extra

    def flops(self, num_tokens: int) -> float:
        return self.inp.flops(num_tokens) + self.o.flops(num_tokens)

    def mixing_flops(self, q_lens, kv_lens) -> float:
        return self.left.mixing_flops(q_lens, kv_lens) + self.right.mixing_flops(q_lens, kv_lens)

    def cache_bytes_read(self, q_lens, kv_lens, itemsize: int) -> int:
        return self.left.cache_bytes_read(q_lens, kv_lens, itemsize) + self.right.cache_bytes_read(q_lens, kv_lens, itemsize)

    def forward(self, h, ctx, cache: CacheView):
        l, r = self.left, self.right
        proj = self.inp(h)
        inner = torch.empty((h.shape[0], l.inner_size + r.inner_size), device=h.device, dtype=h.dtype)
        l.mix(proj[:, :l.in_size], ctx, cache.parts.get("left"), inner[:, :l.inner_size])
        r.mix(proj[:, l.in_size:], ctx, cache.parts.get("right"), inner[:, l.inner_size:])
        return self.o(inner)


@register("mixer", "latent_attention")
class LatentAttention(Mixer):
    """Attention whose queries, keys and values pass through normed low-rank latents:

        c_q = norm(W_dq h) w_dq,   q_h = W_uq,h c_q = [q_plain (dim) | q_rot (rot_dim)]
        [c' | r'] = W_dkv h,        c = norm(c') w_dkv  (rank elements),   r = rot(r')  (rot_dim elements, one for all heads)
        key_h = [W_uk,h c | r],     value_h = W_uv,h c,   score = scale <q_h, key_h> with q_rot rotated as r is

    under a causal mask, with ``window`` > 0 limited to the last ``window`` keys; softmax; W_o over the heads.  rot
    turns interleaved pairs (2i, 2i+1) of the first ``position.dim`` elements by position * theta^(-2i/dim).

    Per token the layer keeps [c | r] and nothing else: one key/value head of rank + rot_dim elements whose values are
    the first ``rank`` elements of the same rows.  The products with W_uk and W_uv are made on the query's side
    (csrc/latent_attention.cu): the query that meets the kept rows is [W_uk,h^T q_plain | q_rot], and the weighted sum
    of latents is projected by W_uv,h afterwards; both are one batched product over the heads.

    Tensors behind ``prefix``: dq, dq.norm, uq, dkv, dkv.norm, uk, uv, o (``names`` renames them); no biases."""

    NAMES = {n: n for n in ("dq", "dq.norm", "uq", "dkv", "dkv.norm", "uk", "uv", "o")}
    metadata_key = "attention"      # the work lists of the attention kernels serve this layer as well

    def step_metadata(self, q_lens, kv_lens, cu_q) -> StepMetadata:
        return StepMetadata(*ops.attention_work(q_lens, kv_lens, cu_q))

    def decode_metadata(self, padded: int, max_kv: int) -> StepMetadata:
        return StepMetadata(*ops.attention_work_decode(padded, max_kv))

    def __init__(self, hidden_size: int, num_heads: int, dim: int, rot_dim: int, value_dim: int, q_rank: int, kv_rank: int,
                 scale: float | None, norm_eps: float, position: PartSpec, window: int = 0, prefix: str = "mix.",
                 names: dict | None = None) -> None:
        self.hidden_size = hidden_size
        self.num_heads, self.dim, self.rot_dim, self.value_dim = num_heads, dim, rot_dim, value_dim
        self.q_rank, self.kv_rank = q_rank, kv_rank
        self.scale = float(scale) if scale is not None else (dim + rot_dim) ** -0.5
        self.norm_eps = float(norm_eps)
        self.window = int(window)
        self.prefix = prefix
        self.names = {**self.NAMES, **(names or {})}
        self.position = build("position", position, hidden_size)
        self.row = kv_rank + rot_dim            # elements of a kept row, and of a query that meets it

    def _n(self, role: str) -> str:
        return self.prefix + self.names[role]

    def cache_need(self):
        return PagedNeed(1, self.row, self.window, self.kv_rank, 0, 0, True)

    def tensor_needs(self):
        W, H, D, R, DV = self.hidden_size, self.num_heads, self.dim, self.rot_dim, self.value_dim
        return {self._n("dq"): TensorNeed((self.q_rank, W)), self._n("dq.norm"): TensorNeed((self.q_rank,), "norm"),
                self._n("uq"): TensorNeed((H * (D + R), self.q_rank)), self._n("dkv"): TensorNeed((self.row, W)),
                self._n("dkv.norm"): TensorNeed((self.kv_rank,), "norm"), self._n("uk"): TensorNeed((H * D, self.kv_rank)),
                self._n("uv"): TensorNeed((H * DV, self.kv_rank)), self._n("o"): TensorNeed((W, H * DV))}

    def load(self, tensors, rt: Runtime) -> None:
        w = lambda role: tensors[self._n(role)].to(device=rt.device, dtype=rt.dtype)
        f = lambda role: tensors[self._n(role)].to(device=rt.device, dtype=torch.float32).contiguous()
        H, D, DV, KR = self.num_heads, self.dim, self.value_dim, self.kv_rank
        # both down projections read the same input: one stacked product, [c_q' | c' | r']
        self.down = Linear.stacked([w("dq"), w("dkv")])
        self.uq = Linear(w("uq"))
        self.o = Linear(w("o"))
        self.q_norm, self.kv_norm = f("dq.norm"), f("dkv.norm")
        # per head: W_uk,h^T as the weight [rank, dim] of q_plain -> latent space; W_uv,h [value_dim, rank] as it is
        self.uk_t = w("uk").view(H, D, KR).transpose(1, 2).contiguous()
        self.uv = w("uv").view(H, DV, KR).contiguous()
        self.position.load({}, rt)
        if self.position.rotary_table() is None:
            raise ValueError("latent_attention takes a position encoding that offers a rotary table")
        if self.position.rotary_table().shape[1] > self.rot_dim:
            raise ValueError("latent_attention: more rotated elements than the rotated part has")

    # ---- cost of a step
    def weight_bytes(self) -> int:
        own = sum(t.numel() * t.element_size() for t in (self.uk_t, self.uv, self.q_norm, self.kv_norm))
        return self.down.weight_bytes() + self.uq.weight_bytes() + self.o.weight_bytes() + own

    def flops(self, num_tokens: int) -> float:
        per_head = 2.0 * num_tokens * self.num_heads * self.kv_rank * (self.dim + self.value_dim)
        return self.down.flops(num_tokens) + self.uq.flops(num_tokens) + self.o.flops(num_tokens) + per_head

    def _seen(self, q: int, kv: int) -> float:
        if self.window <= 0:
            return q * (kv - q) + q * (q + 1) / 2
        return float(sum(min(self.window, p + 1) for p in range(kv - q, kv)))

    def mixing_flops(self, q_lens, kv_lens) -> float:
        # scores over the kept rows, weighted sums over their latents
        return 2.0 * self.num_heads * (self.row + self.kv_rank) * sum(self._seen(q, kv) for q, kv in zip(q_lens, kv_lens))

    def cache_bytes_read(self, q_lens, kv_lens, itemsize: int) -> int:
        keys = sum(min(kv, self.window + q - 1) if self.window > 0 else kv for q, kv in zip(q_lens, kv_lens))
        return keys * self.row * itemsize

    def forward(self, h, ctx, cache: CacheView):
        H, D, R, DV, KR = self.num_heads, self.dim, self.rot_dim, self.value_dim, self.kv_rank
        T = h.shape[0]
        table = ctx.block_tables[cache.group]
        down = self.down(h)                                     # [T, q_rank + rank + rot_dim]
        cq = torch.empty((T, self.q_rank), device=h.device, dtype=h.dtype)
        ops.rmsnorm_rows(down[:, :self.q_rank], self.q_norm, self.norm_eps, cq)
        q = self.uq(cq)                                         # [T, H, dim + rot_dim]
        met = torch.empty((T, H * self.row), device=h.device, dtype=h.dtype)      # the queries that meet the kept rows
        ops.latent_prepare(q, met, down[:, self.q_rank:], self.kv_norm, self.norm_eps, self.position.rotary_table(),
                           ctx.positions, ctx.seq_of_token, table if cache.writes else None,
                           cache.k_pages if cache.writes else None, H, D, R, KR, table_rows=ctx.table_rows)
        ops.gemm_batched(q.view(T, H, D + R)[:, :, :D], self.uk_t, met.view(T, H, self.row)[:, :, :KR])
        lat = torch.empty((T, H * KR), device=h.device, dtype=h.dtype)            # weighted sums of latents
        ops.attention_latent(met, lat, cache.k_pages, ctx, table, H, self.row, KR, self.scale, self.window,
                             work=ctx.work.get(self.metadata_key))
        out = torch.empty((T, H * DV), device=h.device, dtype=h.dtype)
        ops.gemm_batched(lat.view(T, H, KR), self.uv, out.view(T, H, DV))
        return self.o(out)
