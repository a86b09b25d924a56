"""Feed-forward parts."""

from __future__ import annotations

import math

import torch

from ..kernels import ops
from ..weights.needs import TensorNeed
from .base import FeedForward, Runtime
from .linear import Linear
from .registry import register


@register("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """y = (silu(x Wg^T) * (x Wu^T)) Wd^T, gate and up as one stacked product
    (acvram/engine/attention.py:705-783)."""

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str = "mlp.", bias: bool | None = None,
                 names: dict | None = None, activation: str = "silu") -> None:
        """``bias``: True, the three projections have biases; False, none; None, those that the file holds.
        ``names``: the tensors' names behind ``prefix``, {"gate": w, "gate.bias": b, "up": ..., "down": ...}.
        ``activation``: what the gate passes through, "silu" or "gelu_tanh" (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))),
        computed in float."""
        if activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"gated feed-forward: no activation '{activation}' (silu and gelu_tanh are built)")
        self.activation = activation
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.prefix = prefix
        self.bias = bias
        if names is None:
            names = {}
            for role in ("gate", "up", "down"):
                names[role], names[role + ".bias"] = f"{role}_proj.weight", f"{role}_proj.bias"
        self.names = dict(names)

    def tensor_needs(self):
        H, I = self.hidden_size, self.intermediate_size
        needs = {}
        for role, n_out, n_in in (("gate", I, H), ("up", I, H), ("down", H, I)):
            needs[self.prefix + self.names[role]] = TensorNeed((n_out, n_in))
            if self.bias is not False and role + ".bias" in self.names:
                needs[self.prefix + self.names[role + ".bias"]] = TensorNeed((n_out,), "bias", optional=self.bias is None)
        return needs

    def weight_bytes(self) -> int:
        return self.gate_up.weight_bytes() + self.down.weight_bytes()

    def flops(self, num_tokens: int) -> float:
        return self.gate_up.flops(num_tokens) + self.down.flops(num_tokens)

    def load(self, tensors, rt: Runtime) -> None:
        w = lambda role: tensors[self.prefix + self.names[role]].to(device=rt.device, dtype=rt.dtype)

        def b(role):
            name = self.prefix + self.names.get(role + ".bias", "\0")
            return tensors[name].to(device=rt.device, dtype=torch.float32) if name in tensors else None

        gate, up = w("gate"), w("up")
        gate_b, up_b, down_b = b("gate"), b("up"), b("down")
        # bfloat16 with 16-byte aligned rows: gate and up rows are interleaved (g0, u0, g1, u1 ...) so that the
        # tensor-core product's epilogue holds each pair together and applies SiLU(gate) * up itself; the
        # stacked product's output [T, 2I] is then never written.  Otherwise: stacked product, then the kernel.
        # (biases of gate and up are interleaved the same way and join the accumulators in that epilogue)
        self.fused = rt.dtype == torch.bfloat16 and self.hidden_size % 8 == 0
        self.fused_act = ops.GATED_EPILOGUE_ACTS.get(self.activation)
        if self.fused:
            pair_bias = None
            if gate_b is not None or up_b is not None:
                zeros = torch.zeros(self.intermediate_size, device=rt.device, dtype=torch.float32)
                pair_bias = torch.stack([gate_b if gate_b is not None else zeros, up_b if up_b is not None else zeros],
                                        dim=1).reshape(-1)
            self.gate_up = Linear(torch.stack([gate, up], dim=1).reshape(2 * self.intermediate_size, self.hidden_size), pair_bias)
        else:
            self.gate_up = Linear.stacked([gate, up], [gate_b, up_b])
        self.down = Linear(w("down"), down_b)

    def decode_layer_spec(self):
        """What the fused decode-layer kernel needs of this feed-forward: gate and up rows interleaved, no biases."""
        if not self.fused or self.down.bias is not None or self.gate_up.bias is not None or self.activation != "silu":
            return None
        return {"intermediate_size": self.intermediate_size, "w_gate_up_pairs": self.gate_up.weight, "w_down": self.down.weight}

    def forward(self, h, ctx):
        if self.fused and self.fused_act is not None and h.shape[0] and ops.gemm_tc_takes(h, self.gate_up.weight):
            act = torch.empty((h.shape[0], self.intermediate_size), device=h.device, dtype=h.dtype)
            ops.linear_bf16_swiglu(h, self.gate_up.weight, act, static_weights=True, bias=self.gate_up.bias,
                                   **({"act": self.fused_act} if self.activation != "silu" else {}))
            return self.down(act)
        act = torch.empty((h.shape[0], self.intermediate_size), device=h.device, dtype=h.dtype)
        if self.activation != "silu":
            # the gate's activation in float on the stacked product's output, rounded once
            return self.down(ops.glu(self.gate_up(h), act, ops.ACTIVATIONS[self.activation], 0.0, 0.0, pairs=self.fused))
        if self.fused:      # an input the tensor-core kernel does not take: undo the interleaving for this call
            gu = self.gate_up(h).view(h.shape[0], self.intermediate_size, 2).transpose(1, 2).reshape(h.shape[0], -1)
        else:
            gu = self.gate_up(h)
        ops.swiglu(gu, act)
        return self.down(act)


@register("feed_forward", "moe")
class RoutedExperts(FeedForward):
    """Mixture of experts with an optional shared expert.

    Router: z = W_r h in 32-bit; scores sigmoid(z) (``scoring`` "sigmoid") or softmax(z) ("softmax"); the ``top``
    largest choose the experts (ties: the lower index); their scores are the weights, divided by their sum with
    ``renormalize``.  An expert is a gated unit with clamps,

        g = min(W_gate x, limit),  u = clamp(W_up x, -limit, limit),  y = g * sigmoid(alpha g) * (u + 1),  W_down y,

    and the weight w multiplies its input (``weight_on`` "input": x = w h, which the kernels apply to the
    accumulators of the first product, W (w h) = w (W h), in 32-bit) or its output ("output").  The shared expert
    (``shared_ff`` > 0: the same unit with sizes and a limit of its own) runs for every token and is added times
    sigmoid(<w_sg, h>), one number per token, computed in 32-bit with the router.

    Variants: ``expert_form`` "plain": an expert (and the shared one) has no gate, W_down act(W_up x) with ``activation`` a
    name of ``ops.ACTIVATIONS`` ("gelu": the exact one, with erf), no clamps; ``groups`` = (count, keep): the experts stand in
    ``count`` equal groups of neighbours, a group is worth its best score, and only experts of the ``keep`` best groups can
    be chosen; ``renorm_eps`` joins the sum that the chosen scores are divided by; ``shared_gate`` False: the shared
    expert's output is added as it is (no tensor shared.sg).

    The step is the same launches whatever the routing is (rows grouped by expert on the device, tiles that belong
    to no expert return at once), so it runs inside a captured graph.  Tensors behind ``prefix``: router, e<i>.gate,
    e<i>.up, e<i>.down, shared.gate, shared.up, shared.down, shared.sg."""

    def __init__(self, hidden_size: int, experts: int, top: int, expert_ff: int, expert_limit: float, shared_ff: int = 0,
                 shared_limit: float = 0.0, alpha: float = 1.702, scoring: str = "sigmoid", renormalize: bool = False,
                 weight_on: str = "input", prefix: str = "mlp.", expert_form: str = "glu", activation: str | None = None,
                 groups: tuple | None = None, renorm_eps: float = 0.0, shared_gate: bool = True) -> None:
        if scoring not in ("sigmoid", "softmax"):
            raise ValueError(f"router scoring '{scoring}' is not built (sigmoid and softmax are)")
        if weight_on not in ("input", "output"):
            raise ValueError(f"weight_on must be 'input' or 'output', got '{weight_on}'")
        if not 1 <= top <= experts:
            raise ValueError(f"top {top} must lie in 1..{experts}")
        if expert_form not in ("glu", "plain"):
            raise ValueError(f"expert_form is 'glu' or 'plain', got '{expert_form}'")
        self.plain = expert_form == "plain"
        if self.plain and (activation not in ops.ACTIVATIONS or ops.ACTIVATIONS[activation] == 0):
            raise ValueError(f"plain experts: no activation '{activation}'")
        if self.plain and weight_on != "output":
            raise ValueError("plain experts are not linear in their input: the weight goes on the output")
        self.activation = activation
        self.groups = (int(groups[0]), int(groups[1])) if groups else None
        if self.groups is not None:
            count, keep = self.groups
            if count < 1 or experts % count or not 1 <= keep <= count or top > keep * (experts // count):
                raise ValueError(f"{experts} experts in {count} groups of which {keep} are kept cannot give {top} choices")
        self.renorm_eps = float(renorm_eps)
        self.shared_gated = bool(shared_gate)
        self.hidden_size, self.experts, self.top = hidden_size, experts, top
        self.expert_ff, self.expert_limit = expert_ff, float(expert_limit)
        self.shared_ff, self.shared_limit = shared_ff, float(shared_limit)
        self.alpha, self.scoring, self.renormalize, self.weight_on = float(alpha), scoring, bool(renormalize), weight_on
        self.prefix = prefix

    def tensor_needs(self):
        H, F, p = self.hidden_size, self.expert_ff, self.prefix
        needs = {p + "router": TensorNeed((self.experts, H))}
        for e in range(self.experts):
            if not self.plain:
                needs[f"{p}e{e}.gate"] = TensorNeed((F, H))
            needs[f"{p}e{e}.up"] = TensorNeed((F, H))
            needs[f"{p}e{e}.down"] = TensorNeed((H, F))
        if self.shared_ff:
            S = self.shared_ff
            needs.update({p + "shared.up": TensorNeed((S, H)), p + "shared.down": TensorNeed((H, S))})
            if not self.plain:
                needs[p + "shared.gate"] = TensorNeed((S, H))
            if self.shared_gated:
                needs[p + "shared.sg"] = TensorNeed((1, H))
        return needs

    def load(self, tensors, rt: Runtime) -> None:
        p = self.prefix
        w = lambda n: tensors[p + n].to(device=rt.device, dtype=rt.dtype)
        self.router = tensors[p + "router"].to(device=rt.device, dtype=torch.float32).contiguous()
        self.run_dtype = rt.dtype
        # [E, 2F, H]: an expert's gate and up rows; [E, H, F].  bfloat16 with rows of 16-byte alignment: (gate, up) row by
        # row, the layout that the tcgen05 product's epilogue wants (the other kernels read either); else all gate
        # rows, then all up rows
        self.pairs = rt.dtype == torch.bfloat16 and self.hidden_size % 8 == 0 and self.expert_ff % 8 == 0 and not self.plain
        self.gate_up = torch.stack([w(f"e{e}.up") for e in range(self.experts)]).contiguous() if self.plain else torch.stack([
            torch.stack([w(f"e{e}.gate"), w(f"e{e}.up")], dim=1).reshape(2 * self.expert_ff, self.hidden_size) if self.pairs
            else torch.cat([w(f"e{e}.gate"), w(f"e{e}.up")], dim=0) for e in range(self.experts)]).contiguous()
        self.down = torch.stack([w(f"e{e}.down") for e in range(self.experts)]).contiguous()
        # plain experts on the grouped tcgen05 product: bfloat16 with rows of 16-byte alignment
        self.tc_plain = self.plain and rt.dtype == torch.bfloat16 and self.hidden_size % 8 == 0 and self.expert_ff % 8 == 0
        self.shared_gate_up = self.shared_down = self.shared_gate = None
        if self.shared_ff and self.plain:
            self.shared_pairs = False
            self.shared_gate_up, self.shared_down = Linear(w("shared.up")), Linear(w("shared.down"))
        elif self.shared_ff:
            # with rows of 16-byte alignment in bfloat16: (gate, up) row by row, so that a step of many tokens applies the
            # activation in the product's epilogue
            self.shared_pairs = rt.dtype == torch.bfloat16 and self.hidden_size % 8 == 0 and self.shared_ff % 8 == 0
            self.shared_gate_up = (Linear(torch.stack([w("shared.gate"), w("shared.up")], dim=1).reshape(2 * self.shared_ff, self.hidden_size))
                                   if self.shared_pairs else Linear.stacked([w("shared.gate"), w("shared.up")]))
            self.shared_down = Linear(w("shared.down"))
        if self.shared_ff and self.shared_gated:
            self.shared_gate = tensors[p + "shared.sg"].to(device=rt.device, dtype=torch.float32).reshape(-1).contiguous()
        # The router's logits (and the shared gate's) as one matrix product with 32-bit accumulation: in a float32 run
        # the CUDA-core product; in a bfloat16 run the tensor-core product with float output, which is the same 32-bit
        # arithmetic when the weights are bfloat16 values anyway (products of two bfloat16 numbers are exact in float).
        # Weights that bfloat16 cannot hold keep the router kernel that reads them as float.
        rows = [self.router] + ([self.shared_gate[None, :]] if self.shared_gate is not None else [])
        stacked = torch.cat(rows + [torch.zeros((-len(torch.cat(rows)) % 8, self.hidden_size), device=rt.device)])
        self.router_linear = None
        if rt.dtype == torch.float32 or bool((stacked.to(torch.bfloat16).float() == stacked).all()):
            self.router_linear = Linear(stacked.to(rt.dtype))

    # ---- cost of a step
    def weight_bytes(self) -> int:
        """All experts' weights: what a step reads once its tokens' choices cover them (a lower bound for few tokens
        is ``active_weight_bytes``)."""
        n = self.router.numel() * 4 + (self.gate_up.numel() + self.down.numel()) * self.gate_up.element_size()
        if self.shared_ff:
            n += self.shared_gate_up.weight_bytes() + self.shared_down.weight_bytes() + \
                (self.shared_gate.numel() * 4 if self.shared_gate is not None else 0)
        return n

    def step_weight_bytes(self, num_tokens: int) -> int:
        """Weights that a step of ``num_tokens`` tokens is expected to read: the experts that at least one token
        chooses when choices fall evenly, E (1 - (1 - top/E)^tokens), and everything that runs for every token."""
        active = self.experts * (1.0 - (1.0 - self.top / self.experts) ** num_tokens)
        per = (self.gate_up.numel() + self.down.numel()) // self.experts * self.gate_up.element_size()
        n = self.router.numel() * 4 + int(active * per)
        if self.shared_ff:
            n += self.shared_gate_up.weight_bytes() + self.shared_down.weight_bytes() + \
                (self.shared_gate.numel() * 4 if self.shared_gate is not None else 0)
        return n

    def flops(self, num_tokens: int) -> float:
        H = self.hidden_size
        per = 4.0 if self.plain else 6.0        # an expert is two products, or three with a gate
        n = 2.0 * num_tokens * self.experts * H + per * num_tokens * self.top * self.expert_ff * H
        return n + (per * num_tokens * self.shared_ff * H if self.shared_ff else 0.0)

    def forward(self, h, ctx):
        T, H = h.shape
        E, top, F = self.experts, self.top, self.expert_ff
        dev = h.device
        rows = T * top
        tiles = ops.moe_max_tiles(rows, E)
        ids = torch.empty(rows, device=dev, dtype=torch.int32)
        weights = torch.empty(rows, device=dev, dtype=torch.float32)
        gate = torch.empty(T, device=dev, dtype=torch.float32) if self.shared_gate is not None else None
        route = {"groups": self.groups, "renorm_eps": self.renorm_eps}
        if self.router_linear is not None:
            # many tokens against a few dozen router rows: one column of tiles, so the reduction is split eight ways
            # to put more than a ninth of the SMs to work
            plan = (0, 128, 8, 4, 0) if h.dtype == torch.bfloat16 and T >= 512 and H >= 2048 and self.router_linear.out_features <= 128 else None
            logits = self.router_linear(h, out_dtype=torch.float32, plan=plan)
            ops.moe_route(h, None, None, top, self.scoring == "softmax", self.renormalize, ids, weights, gate, logits=logits,
                          experts=E, **route)
        else:
            ops.moe_route(h, self.router, self.shared_gate, top, self.scoring == "softmax", self.renormalize, ids, weights, gate,
                          **route)
        place = torch.empty(rows, device=dev, dtype=torch.int32)
        w_in = weights if self.weight_on == "input" else None
        w_out = weights if self.weight_on == "output" else None
        if self.tc_plain and rows >= ops.MOE_TC_ROWS and rows >= ops.MOE_TC_ROWS_PER_EXPERT * E:
            # plain experts, many rows: the same grouping; the activation is the first product's epilogue, the row's weight
            # the second's (on the float accumulators)
            tile = ops.MOE_TC_TILE
            tiles = ops.moe_max_tiles(rows, E, tile)
            grouped = torch.empty(tiles * tile, device=dev, dtype=torch.int32)
            tile_expert = torch.empty(tiles, device=dev, dtype=torch.int32)
            used = torch.empty(1, device=dev, dtype=torch.int32)
            ops.moe_group(ids, E, grouped, place, tile_expert, tile, used)
            hg = torch.empty((tiles * tile, H), device=dev, dtype=h.dtype)
            scale = torch.empty(tiles * tile, device=dev, dtype=torch.float32)
            ops.moe_gather(h, grouped, weights, top, hg, scale, used, tile)
            act = torch.empty((tiles * tile, F), device=dev, dtype=h.dtype)
            ops.gemm_tc_grouped(hg, self.gate_up, act, tile_expert, used, unary=self.activation)
            parts = torch.empty((tiles * tile, H), device=dev, dtype=h.dtype)
            ops.gemm_tc_grouped(act, self.down, parts, tile_expert, used, row_scale=scale)
        elif self.pairs and rows >= ops.MOE_TC_ROWS and rows >= ops.MOE_TC_ROWS_PER_EXPERT * E and w_out is None:
            # many rows: tiles of 128 rows on the tcgen05 product, the tokens' rows copied into grouped order first
            tile = ops.MOE_TC_TILE
            tiles = ops.moe_max_tiles(rows, E, tile)
            grouped = torch.empty(tiles * tile, device=dev, dtype=torch.int32)
            tile_expert = torch.empty(tiles, device=dev, dtype=torch.int32)
            used = torch.empty(1, device=dev, dtype=torch.int32)
            ops.moe_group(ids, E, grouped, place, tile_expert, tile, used)
            hg = torch.empty((tiles * tile, H), device=dev, dtype=h.dtype)
            scale = torch.empty(tiles * tile, device=dev, dtype=torch.float32)
            ops.moe_gather(h, grouped, w_in, top, hg, scale, used, tile)
            act = torch.empty((tiles * tile, F), device=dev, dtype=h.dtype)
            ops.gemm_tc_grouped(hg, self.gate_up, act, tile_expert, used, True, scale, self.expert_limit, self.alpha)
            # the experts' outputs leave the product as bfloat16 (as every projection's do); their sum is 32-bit
            parts = torch.empty((tiles * tile, H), device=dev, dtype=h.dtype)
            ops.gemm_tc_grouped(act, self.down, parts, tile_expert, used)
        else:
            grouped = torch.empty(tiles * ops.MOE_TILE, device=dev, dtype=torch.int32)
            tile_expert = torch.empty(tiles, device=dev, dtype=torch.int32)
            ops.moe_group(ids, E, grouped, place, tile_expert)
            act = torch.empty((tiles * ops.MOE_TILE, F), device=dev, dtype=h.dtype)
            ops.moe_experts_up(h, self.gate_up, act, grouped, tile_expert, w_in, top, self.expert_limit, self.alpha, self.pairs,
                               plain_act=self.activation if self.plain else None)
            parts = torch.empty((tiles * ops.MOE_TILE, H), device=dev, dtype=torch.float32)
            ops.moe_experts_down(act, self.down, parts, grouped, tile_expert, w_out, top)
        shared = None
        if self.shared_ff and self.plain:
            shared = self.shared_down(self.shared_gate_up(h, unary=self.activation))
        elif self.shared_ff:
            sact = torch.empty((T, self.shared_ff), device=dev, dtype=h.dtype)
            if self.shared_pairs and ops.linear_bf16_glu_takes(h, self.shared_gate_up.weight):
                ops.linear_bf16_glu(h, self.shared_gate_up.weight, sact, self.shared_limit, self.alpha)
            else:
                gu = self.shared_gate_up(h)
                ops.glu(gu, sact, ops.GLU_SWISH_CLAMPED, self.shared_limit, self.alpha, self.shared_pairs)
            shared = self.shared_down(sact)
        out = torch.empty((T, H), device=dev, dtype=h.dtype)
        return ops.moe_combine(parts, place, top, shared, gate, out)


@register("feed_forward", "dense")
class DenseFF(FeedForward):
    """y = W_down act(W_up x): two products and an activation between them, no gate.  ``activation``:

        "xielu"      z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2, with the layer's two
                     learned numbers (p, q) in the tensor ``names["act"]``, folded once at load in double precision
        "gelu_tanh"  0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
        "silu"

    computed in float on the product's output and rounded once."""

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "xielu", prefix: str = "mlp.",
                 names: dict | None = None) -> None:
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"dense feed-forward: no activation '{activation}'; known: {', '.join(ops.ACTIVATIONS)}")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.activation = activation
        self.prefix = prefix
        self.names = {"up": "up", "down": "down", "act": "act", **(names or {})}
        self.p0 = self.p1 = 0.0

    def tensor_needs(self):
        H, I = self.hidden_size, self.intermediate_size
        needs = {self.prefix + self.names["up"]: TensorNeed((I, H)), self.prefix + self.names["down"]: TensorNeed((H, I))}
        if self.activation == "xielu":
            needs[self.prefix + self.names["act"]] = TensorNeed((2,))
        return needs

    def load(self, tensors, rt: Runtime) -> None:
        w = lambda role: tensors[self.prefix + self.names[role]].to(device=rt.device, dtype=rt.dtype)
        self.up, self.down = Linear(w("up")), Linear(w("down"))
        if self.activation == "xielu":
            p, q = (float(v) for v in tensors[self.prefix + self.names["act"]].to(torch.float64).cpu())
            softplus = lambda z: math.log1p(math.exp(-abs(z))) + max(z, 0.0)
            self.p0, self.p1 = softplus(p), 0.5 + softplus(q)

    def weight_bytes(self) -> int:
        return self.up.weight_bytes() + self.down.weight_bytes()

    def flops(self, num_tokens: int) -> float:
        return self.up.flops(num_tokens) + self.down.flops(num_tokens)

    def forward(self, h, ctx):
        z = self.up(h)
        ops.activation(z, z, self.activation, self.p0, self.p1)
        return self.down(z)
