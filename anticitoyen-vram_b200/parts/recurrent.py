"""Token mixers that keep a state of fixed size for each request instead of pages: retention and a gated
linear recurrence.  Their states are 32-bit in every run precision and live in the cache manager's state slots
(zeroed when a request begins); a step may bring any mix of portions of prompts and single tokens."""

from __future__ import annotations

import math

import torch

from ..cache.manager import StateNeed
from ..kernels import ops
from ..weights.needs import TensorNeed
from .base import CacheView, Mixer, Runtime, StepMetadata
from .linear import Linear
from .plan import PartSpec
from .registry import build, register


class SegmentedRecurrence(Mixer):
    """What the mixers with a linear recurrence ask of every step: the list of (request, segment) items that their
    kernels run side by side (``ops.segment_work``).  One list serves every such layer of a model."""

    metadata_key = "segments"

    def step_metadata(self, q_lens, kv_lens, cu_q) -> StepMetadata:
        return StepMetadata(*ops.segment_work(q_lens))

    def decode_metadata(self, padded: int, max_kv: int) -> StepMetadata:
        return StepMetadata(*ops.segment_work_decode(padded))


@register("mixer", "retention")
class Retention(SegmentedRecurrence):
    """Linear attention with a fixed decay per head, without softmax or denominator:

        S_t = decay_h S_{t-1} + k_t v_t^T,   o_t = S_t^T q_t            S: [dim, value_dim] per head, float32

    q and k get the position encoding (``position``; None: none), k is then multiplied by ``k_scale`` (default
    dim^-1/2).  Each head's o is brought to unit RMS (``norm_eps``, no weight), the heads side by side are multiplied
    by silu(W_g h) and by ``out_scale``, and projected by W_o.  Tensors behind ``prefix``: q, k, v, g, o (``names``
    renames them); no biases.

    Variants: ``input_act`` "silu": q, k and v are silu of their projections (in float, before anything else);
    ``joint_norm``: the name of a weight over all heads' values: the heads side by side are then normed together,
    o / sqrt(mean over all heads of o^2 + eps) * weight, instead of each head to unit RMS; ``gate_fn`` "sigmoid"
    instead of "silu"."""

    NAMES = {n: n for n in ("q", "k", "v", "g", "o")}

    def __init__(self, hidden_size: int, num_heads: int, dim: int, value_dim: int, decay, norm_eps: float,
                 position: PartSpec | None = None, k_scale: float | None = None, prefix: str = "mix.",
                 names: dict | None = None, out_scale: float = 1.0, input_act: str | None = None,
                 joint_norm: str | None = None, gate_fn: str = "silu") -> None:
        if input_act not in (None, "silu") or gate_fn not in ("silu", "sigmoid"):
            raise ValueError(f"retention: input_act {input_act!r} / gate_fn {gate_fn!r} are not built")
        self.input_act, self.joint_norm, self.gate_fn = input_act, joint_norm, gate_fn
        self.norm_weight = None
        decay = [float(d) for d in decay]
        if len(decay) != num_heads:
            raise ValueError(f"{len(decay)} decays for {num_heads} heads")
        self.hidden_size = hidden_size
        self.num_heads, self.dim, self.value_dim = num_heads, dim, value_dim
        self.decay_values = decay
        self.norm_eps = float(norm_eps)
        self.k_scale = float(k_scale) if k_scale is not None else dim ** -0.5
        self.out_scale = float(out_scale)
        self.prefix = prefix
        self.names = {**self.NAMES, **(names or {})}
        self.position = build("position", position, hidden_size) if position is not None else None
        self.qk_size = num_heads * dim
        self.inner_size = num_heads * value_dim
        self.in_size = 2 * self.qk_size + 2 * self.inner_size        # [q | k | v | g]

    def _n(self, role: str) -> str:
        return self.prefix + self.names[role]

    def cache_need(self):
        return StateNeed((self.num_heads, self.dim, self.value_dim), "float32")

    def tensor_needs(self):
        H = self.hidden_size
        needs = {self._n("q"): TensorNeed((self.qk_size, H)), self._n("k"): TensorNeed((self.qk_size, H)),
                 self._n("v"): TensorNeed((self.inner_size, H)), self._n("g"): TensorNeed((self.inner_size, H)),
                 self._n("o"): TensorNeed((H, self.inner_size))}
        if self.joint_norm is not None:
            needs[self.prefix + self.joint_norm] = TensorNeed((self.inner_size,), "norm")
        return needs

    def load(self, tensors, rt: Runtime) -> None:
        w = lambda role: tensors[self._n(role)].to(device=rt.device, dtype=rt.dtype)
        self.qkv = Linear.stacked([w("q"), w("k"), w("v"), w("g")])
        self.o = Linear(w("o"))
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=rt.device)
        if self.joint_norm is not None:
            self.norm_weight = tensors[self.prefix + self.joint_norm].to(device=rt.device, dtype=torch.float32).contiguous()
        if self.position is not None:
            self.position.load({}, rt)
            if self.position.rotary_table() is None:
                raise ValueError("retention takes a position encoding that offers a rotary table")

    def extra_weight_bytes(self) -> int:
        return self.norm_weight.numel() * 4 if self.norm_weight is not None else 0

    def weight_bytes(self) -> int:
        return self.qkv.weight_bytes() + self.o.weight_bytes() + self.extra_weight_bytes()

    def flops(self, num_tokens: int) -> float:
        return self.qkv.flops(num_tokens) + self.o.flops(num_tokens)

    def mixing_flops(self, q_lens, kv_lens) -> float:
        # per token and head: the state's update and its product with q
        return 4.0 * self.num_heads * self.dim * self.value_dim * sum(q_lens)

    def cache_bytes_read(self, q_lens, kv_lens, itemsize: int) -> int:
        return len(q_lens) * self.num_heads * self.dim * self.value_dim * 4

    def mix(self, proj, ctx, cache: CacheView, out) -> None:
        H, D, DV = self.num_heads, self.dim, self.value_dim
        a, b = self.qk_size, 2 * self.qk_size
        o = torch.empty((proj.shape[0], self.inner_size), device=proj.device, dtype=torch.float32)
        table = self.position.rotary_table() if self.position is not None else None
        ops.retention(proj[:, :a], proj[:, a:b], proj[:, b:b + self.inner_size], table, ctx.positions, self.decay,
                      self.k_scale, cache.state, ctx.state_slots[cache.group], ctx.cu_q, ctx.num_seqs, o, H, D, DV,
                      work=ctx.work.get(self.metadata_key), silu_inputs=self.input_act == "silu")
        ops.retention_gate(o, proj[:, b + self.inner_size:], out, H, DV, self.norm_eps, self.out_scale,
                           weight=self.norm_weight, joint=self.joint_norm is not None, gate_fn=self.gate_fn)

    def forward(self, h, ctx, cache: CacheView):
        proj = self.qkv(h)
        out = torch.empty((h.shape[0], self.inner_size), device=h.device, dtype=h.dtype)
        self.mix(proj, ctx, cache, out)
        return self.o(out)


@register("mixer", "rglru")
class GatedLinearRecurrence(SegmentedRecurrence):
    """The recurrent block of Griffin (De et al., "Griffin: Mixing Gated Linear Recurrences with Local Attention for
    Efficient Language Models"): two branches of ``width`` channels,

        y = gelu_tanh(W_y h + b_y)
        u = conv(W_x h + b_x)               a causal convolution of ``conv`` taps per channel, the last tap the current token's
        r = sigmoid(A_b u_b + a_b),  g = sigmoid(B_b u_b + b_b)        per block b of ``blocks`` equal parts of the channels
        a = exp(-rate * r * softplus(lam)),   S_t = a S_{t-1} + sqrt(1 - a^2) * g * u          (S_{-1} = 0)
        out = W_o (S * y)

    What a request keeps: the last ``conv`` - 1 inputs of the convolution and S, both float32.  Gates, decays and the
    recurrence are 32-bit in every run precision; the two input projections leave their product as float32, and in
    bfloat16 runs the gates' projections take u rounded to bfloat16 (with float accumulation).
    Tensors behind ``prefix``: y, y.b, x, x.b, conv, conv.b, ra, ra.b, ri, ri.b, lam, o."""

    NAMES = {n: n for n in ("y", "y.b", "x", "x.b", "conv", "conv.b", "ra", "ra.b", "ri", "ri.b", "lam", "o")}

    def __init__(self, hidden_size: int, width: int, blocks: int, conv: int, rate: float = 8.0, prefix: str = "mix.",
                 names: dict | None = None) -> None:
        if width % blocks:
            raise ValueError(f"{width} channels do not split into {blocks} equal blocks")
        if conv < 1:
            raise ValueError("the convolution has at least one tap")
        self.hidden_size, self.width, self.blocks, self.taps, self.rate = hidden_size, width, blocks, conv, float(rate)
        self.prefix = prefix
        self.names = {**self.NAMES, **(names or {})}

    def _n(self, role: str) -> str:
        return self.prefix + self.names[role]

    def cache_need(self):
        needs = {"state": StateNeed((self.width,), "float32")}
        if self.taps > 1:
            needs["conv"] = StateNeed((self.taps - 1, self.width), "float32")
        return needs

    def tensor_needs(self):
        H, C, B = self.hidden_size, self.width, self.blocks
        bw = C // B
        return {self._n("y"): TensorNeed((C, H)), self._n("y.b"): TensorNeed((C,), "bias"),
                self._n("x"): TensorNeed((C, H)), self._n("x.b"): TensorNeed((C,), "bias"),
                self._n("conv"): TensorNeed((C, self.taps)), self._n("conv.b"): TensorNeed((C,), "bias"),
                self._n("ra"): TensorNeed((B, bw, bw)), self._n("ra.b"): TensorNeed((B, bw), "bias"),
                self._n("ri"): TensorNeed((B, bw, bw)), self._n("ri.b"): TensorNeed((B, bw), "bias"),
                self._n("lam"): TensorNeed((C,)), self._n("o"): TensorNeed((H, C))}

    def load(self, tensors, rt: Runtime) -> None:
        w = lambda role: tensors[self._n(role)].to(device=rt.device, dtype=rt.dtype)
        f = lambda role: tensors[self._n(role)].to(device=rt.device, dtype=torch.float32).contiguous()
        self.xy = Linear.stacked([w("x"), w("y")])           # biases join in the kernels that read the product
        self.o = Linear(w("o"))
        self.x_bias, self.y_bias = f("x.b"), f("y.b")
        self.conv_w, self.conv_b = f("conv"), f("conv.b")
        self.conv_w_t = self.conv_w.t().contiguous()         # [taps, channels]: four channels' taps of a lag are one vector
        # [blocks, out, in] -> [blocks, in, out]: the threads of a warp then read neighbouring outputs
        self.wa_t, self.wb_t = f("ra").transpose(1, 2).contiguous(), f("ri").transpose(1, 2).contiguous()
        self.ba, self.bb = f("ra.b").reshape(-1).contiguous(), f("ri.b").reshape(-1).contiguous()
        # a bfloat16 run makes the two gate projections on the tensor cores, from the weights as the file has them
        self.gate_weights = (w("ra").contiguous(), w("ri").contiguous()) if rt.dtype == torch.bfloat16 else None
        # softplus of the decay parameter is a constant of the weights: folded once, in float64
        lam = tensors[self._n("lam")].to(torch.float64)
        self.softplus_lam = torch.nn.functional.softplus(lam).to(device=rt.device, dtype=torch.float32).contiguous()

    def weight_bytes(self) -> int:
        small = (self.x_bias, self.y_bias, self.conv_w, self.conv_b, self.wa_t, self.wb_t, self.ba, self.bb, self.softplus_lam)
        return self.xy.weight_bytes() + self.o.weight_bytes() + sum(t.numel() * 4 for t in small)

    def flops(self, num_tokens: int) -> float:
        gates = 4.0 * num_tokens * self.width * (self.width // self.blocks)
        return self.xy.flops(num_tokens) + self.o.flops(num_tokens) + gates

    def cache_bytes_read(self, q_lens, kv_lens, itemsize: int) -> int:
        return len(q_lens) * self.taps * self.width * 4

    def forward(self, h, ctx, cache: CacheView):
        C = self.width
        T = h.shape[0]
        xy = self.xy(h, out_dtype=torch.float32)
        u = torch.empty((T, C), device=h.device, dtype=torch.float32)
        if self.taps > 1:
            conv = cache.parts["conv"]
            conv_state, conv_slots = conv.state, ctx.state_slots[conv.group]
        else:
            conv_state, conv_slots = u, ctx.state_slots[cache.parts["state"].group]      # never read: no tap reaches back
        ops.causal_conv(xy[:, :C], self.x_bias, self.conv_w, self.conv_b, conv_state, conv_slots, ctx.cu_q,
                        ctx.seq_of_token, u, taps_t=self.conv_w_t)
        a, b = torch.empty_like(u), torch.empty_like(u)
        ops.block_gates(u, self.wa_t, self.ba, self.wb_t, self.bb, self.softplus_lam, -self.rate, a, b,
                        bf16_weights=self.gate_weights)
        st = cache.parts["state"]
        mixed = torch.empty((T, C), device=h.device, dtype=h.dtype)
        ops.gated_scan(a, b, xy[:, C:], self.y_bias, st.state, ctx.state_slots[st.group], ctx.cu_q, ctx.num_seqs, mixed,
                       work=ctx.work.get(self.metadata_key))
        return self.o(mixed)


@register("mixer", "wkv")
class TimeMix(SegmentedRecurrence):
    """Time mixing in the manner of RWKV: a linear recurrence per head whose decay depends on the token and on the key
    channel, with a bonus for the current token.  With h' the previous token's input (zeros before a request's first
    token) each of r, k, v, g, w reads a mix of its own, x_s = h + (h' - h) * mu_s:

        r, k, v = W_r x_r, W_k x_k, W_v x_v  (heads x dim),     gate = silu(W_g x_g)
        w = exp(-exp(W_2 tanh(W_1 x_w) + w_0))                    per head and key channel
        o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t;   S_t = diag(w_t) S_{t-1} + k_t v_t^T        S: [dim, dim] per head

    Each head's o is brought to unit RMS (``norm_eps``), the heads side by side are multiplied by a weight and by the gate,
    and projected by W_o.  The mixer keeps two things for every request: the state S (float32) and the previous token's
    input.  32-bit in every run precision: the mixes (rounded once as they enter the projections), tanh, the second
    product, both exponentials, the decays, the recurrence with its state, the head norm and the gate's silu.
    Tensors behind ``prefix`` (``names`` renames them): mu.r, mu.k, mu.v, mu.g, mu.w, r, k, v, g, w1, w2, w0, u, norm, o."""

    NAMES = {n: n for n in ("mu.r", "mu.k", "mu.v", "mu.g", "mu.w", "r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o")}
    MIXES = ("r", "k", "v", "g", "w")

    def __init__(self, hidden_size: int, num_heads: int, dim: int, norm_eps: float, prefix: str = "mix.",
                 names: dict | None = None) -> None:
        self.hidden_size, self.num_heads, self.dim = hidden_size, int(num_heads), int(dim)
        self.norm_eps = float(norm_eps)
        self.prefix = prefix
        self.names = {**self.NAMES, **(names or {})}
        self.inner_size = self.num_heads * self.dim
        self.rank = None        # rows of W_1: whatever the file holds

    def _n(self, role: str) -> str:
        return self.prefix + self.names[role]

    def cache_need(self):
        return {"state": StateNeed((self.num_heads, self.dim, self.dim), "float32"),
                "previous": StateNeed((self.hidden_size,), "float32")}

    def tensor_needs(self):
        H, I = self.hidden_size, self.inner_size
        needs = {self._n("mu." + s): TensorNeed((H,), "norm") for s in self.MIXES}
        for role in ("r", "k", "v", "g"):
            needs[self._n(role)] = TensorNeed((I, H))
        needs[self._n("w1")] = TensorNeed((-1, H))          # the decay's inner size is the file's to choose
        needs[self._n("w2")] = TensorNeed((I, -1))
        needs[self._n("w0")] = TensorNeed((I,), "norm")
        needs[self._n("u")] = TensorNeed((self.num_heads, self.dim), "norm")
        needs[self._n("norm")] = TensorNeed((I,), "norm")
        needs[self._n("o")] = TensorNeed((H, I))
        return needs

    def load(self, tensors, rt: Runtime) -> None:
        w = lambda role: tensors[self._n(role)].to(device=rt.device, dtype=rt.dtype)
        f = lambda role: tensors[self._n(role)].to(device=rt.device, dtype=torch.float32).contiguous()
        self.mu = torch.stack([f("mu." + s) for s in self.MIXES]).contiguous()      # [5, H], the order of MIXES
        self.proj = {role: Linear(w(role)) for role in ("r", "k", "v", "g")}
        self.w1 = Linear(w("w1"))
        self.rank = self.w1.out_features
        if tuple(tensors[self._n("w2")].shape) != (self.inner_size, self.rank):
            raise ValueError(f"wkv: w2 is {tuple(tensors[self._n('w2')].shape)}, w1 has {self.rank} rows")
        self.w2_t = f("w2").t().contiguous()        # [rank, I]: the threads of a warp read neighbouring channels
        self.w0, self.u, self.norm_weight = f("w0"), f("u").reshape(-1).contiguous(), f("norm")
        self.o = Linear(w("o"))

    def weight_bytes(self) -> int:
        return sum(l.weight_bytes() for l in (*self.proj.values(), self.w1, self.o)) + \
            sum(t.numel() * 4 for t in (self.mu, self.w2_t, self.w0, self.u, self.norm_weight))

    def flops(self, num_tokens: int) -> float:
        return sum(l.flops(num_tokens) for l in (*self.proj.values(), self.w1, self.o)) + 2.0 * num_tokens * self.rank * self.inner_size

    def mixing_flops(self, q_lens, kv_lens) -> float:
        # per token, head and state element: the bonus, the product with r, the decay and the update
        return 7.0 * self.num_heads * self.dim * self.dim * sum(q_lens)

    def cache_bytes_read(self, q_lens, kv_lens, itemsize: int) -> int:
        return len(q_lens) * (self.num_heads * self.dim * self.dim + self.hidden_size) * 4

    def forward(self, h, ctx, cache: CacheView):
        T = h.shape[0]
        H, D, I = self.num_heads, self.dim, self.inner_size
        state, previous = cache.parts["state"], cache.parts["previous"]
        x = torch.empty((len(self.MIXES), T, self.hidden_size), device=h.device, dtype=h.dtype)
        ops.token_shift_multi(h, self.mu, previous.state, ctx.state_slots[previous.group], ctx.cu_q, ctx.seq_of_token, x)
        # what enters the recurrence leaves its product unrounded
        r, k, v = (self.proj[role](x[i], out_dtype=torch.float32) for i, role in enumerate(("r", "k", "v")))
        gate = self.proj["g"](x[3])
        decay = torch.empty((T, I), device=h.device, dtype=torch.float32)
        # many tokens against a few dozen rows of W1: one column of tiles, so the reduction is split eight ways to put
        # more than a ninth of the SMs to work
        plan = (0, 128, 8, 4, 0) if h.dtype == torch.bfloat16 and T >= 512 and self.hidden_size >= 2048 \
            and self.rank <= 128 and self.rank % 8 == 0 else None
        ops.wkv_decay(self.w1(x[4], out_dtype=torch.float32, plan=plan), self.w2_t, self.w0, decay)
        o = torch.empty((T, I), device=h.device, dtype=torch.float32)
        ops.wkv(r, k, v, decay, self.u, state.state, ctx.state_slots[state.group], ctx.cu_q, ctx.num_seqs, o, H, D, D,
                work=ctx.work.get(self.metadata_key))
        out = torch.empty((T, I), device=h.device, dtype=h.dtype)
        ops.retention_gate(o, gate, out, H, D, self.norm_eps, weight=self.norm_weight)
        return self.o(out)
