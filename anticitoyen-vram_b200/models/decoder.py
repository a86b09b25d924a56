"""A decoder put together from a ModelPlan: embedding, scheduled blocks, final norm, head."""

from __future__ import annotations

import torch

from ..cache.manager import CachePlan
from ..kernels import ops
from ..parts import BLOCKS, CacheView, ModelPlan, Runtime, build
from ..parts.blocks import NormedDelta, settle
from ..parts.linear import Linear
from ..weights.needs import TensorNeed


class DecoderModel:
    """embed -> blocks in ``plan.schedule`` order -> final norm of the wanted rows -> logits in float32
    (acvram/engine/model.py:143-307).  Knows the plan, not the architecture."""

    def __init__(self, plan: ModelPlan) -> None:
        self.plan = plan
        self.blocks = []
        for spec in plan.layers:
            cls = BLOCKS.get(spec.block)
            if cls is None:
                raise KeyError(f"no block arrangement named '{spec.block}'; known: {', '.join(sorted(BLOCKS))}")
            self.blocks.append(cls(spec, plan.hidden_size))
        self.final_norm = build("norm", plan.final_norm, plan.hidden_size)
        self.rt: Runtime | None = None
        for e in plan.schedule:
            if not 0 <= e.layer < len(self.blocks):
                raise ValueError(f"schedule names layer {e.layer}, the plan has {len(self.blocks)}")

    # ------------------------------------------------------------------ weights
    def tensor_needs(self) -> dict[str, TensorNeed]:
        plan = self.plan
        needs = {plan.embedding_name: TensorNeed((plan.vocab_size, plan.hidden_size), "embedding")}
        for block in self.blocks:
            for name, need in block.tensor_needs().items():
                needs[block.prefix + name] = need
        for name, need in self.final_norm.tensor_needs().items():
            needs[plan.final_norm_prefix + name] = need
        for name, shape in plan.stream_vectors.items():
            needs[name] = TensorNeed(tuple(shape))
        for name, shape in plan.stream_matrices.items():
            needs[name] = TensorNeed(tuple(shape))
        # a tied head reads the embedding; a file that still carries the head's tensor is accepted
        needs[plan.head_name] = TensorNeed((plan.vocab_size, plan.hidden_size), "matrix", optional=plan.tied_head)
        return needs

    def load(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        plan = self.plan
        self.rt = rt
        self.embedding = tensors[plan.embedding_name].to(device=rt.device, dtype=rt.dtype).contiguous()
        for block in self.blocks:
            p = block.prefix
            block.load({n[len(p):]: t for n, t in tensors.items() if n.startswith(p)}, rt)
        p = plan.final_norm_prefix
        self.final_norm.load({n[len(p):]: t for n, t in tensors.items() if n.startswith(p)}, rt)
        self.stream_vectors = {name: tensors[name].to(device=rt.device, dtype=torch.float32).contiguous()
                               for name in plan.stream_vectors}
        self.stream_matrices = {name: Linear(tensors[name].to(device=rt.device, dtype=rt.dtype))
                                for name in plan.stream_matrices}
        if plan.tied_head:
            self.head = Linear(self.embedding)  # the same storage, no copy
        else:
            self.head = Linear(tensors[plan.head_name].to(device=rt.device, dtype=rt.dtype))

    def weight_bytes(self) -> int:
        seen, total = set(), 0

        def visit(obj):
            nonlocal total
            if isinstance(obj, torch.Tensor):
                key = obj.untyped_storage().data_ptr()
                if key not in seen:
                    seen.add(key)
                    total += obj.numel() * obj.element_size()
            elif isinstance(obj, Linear):
                visit(obj.weight)
            elif hasattr(obj, "__dict__") and not isinstance(obj, (type, Runtime, ModelPlan)):
                for v in vars(obj).values():
                    visit(v)
            elif isinstance(obj, (list, tuple)):
                for v in obj:
                    visit(v)

        visit(self)
        return total

    # ------------------------------------------------------------------ cache
    @staticmethod
    def _leaves(need, path=()):
        """(path, need) of every single need inside ``need``, which may be a dict of needs by name, nested."""
        if isinstance(need, dict):
            for name, sub in need.items():
                yield from DecoderModel._leaves(sub, path + (name,))
        elif need is not None:
            yield path, need

    def cache_plan(self) -> CachePlan:
        """One need for each thing that a scheduled run keeps.  A layer that keeps several things (pages beside a
        state, say) names them; each becomes a slot of the cache manager, and ``self.slot_leaves`` remembers which
        manager slots make up which of the plan's cache slots."""
        composite = [None] * self.plan.num_cache_slots
        for e in self.plan.schedule:
            if e.cache >= 0 and isinstance(self.blocks[e.layer].cache_need(), dict):
                if not e.writes or composite[e.cache] not in (None, e.layer):
                    raise ValueError(f"cache slot {e.cache}: a layer that keeps several things shares its slot with no other run")
                composite[e.cache] = e.layer
        if any(c is not None for c in composite):
            flat, self.slot_leaves = [], {}
            for slot, layer in enumerate(composite):
                if layer is None:
                    need = next((self.blocks[e.layer].cache_need() for e in self.plan.schedule
                                 if e.cache == slot and e.writes), None)
                    self.slot_leaves[slot] = [((), len(flat))]
                    flat.append(need)
                    continue
                self.slot_leaves[slot] = []
                for path, need in self._leaves(self.blocks[layer].cache_need()):
                    self.slot_leaves[slot].append((path, len(flat)))
                    flat.append(need)
            return CachePlan(flat)
        self.slot_leaves = None
        needs = [None] * self.plan.num_cache_slots
        for e in self.plan.schedule:
            if e.cache < 0:
                continue
            need = self.blocks[e.layer].cache_need()
            if e.writes:
                if needs[e.cache] is not None and needs[e.cache] != need:
                    raise ValueError(f"cache slot {e.cache} is written by layers with different needs")
                needs[e.cache] = need
        for e in self.plan.schedule:
            if e.cache >= 0 and not e.writes:
                need = self.blocks[e.layer].cache_need()
                have = needs[e.cache]
                if have is not None and have != need and hasattr(have, "widened") and hasattr(need, "widened"):
                    # a reader that forgets by another rule than the writer (another window, another chunk size):
                    # rows of the same sizes, and the slot keeps what either of them may read again
                    try:
                        needs[e.cache] = have = need = have.widened(need)
                    except ValueError:
                        pass
                if have is None or have != need:
                    raise ValueError(f"layer {e.layer} reads cache slot {e.cache}, which no layer of equal need writes")
        return CachePlan(needs)

    def step_cost(self, q_lens, kv_lens, logit_rows: int, cache_itemsize: int | None = None) -> dict:
        """What one step has to read and compute, summed over the scheduled layers as the parts report it:
        ``weight_bytes`` (each weight once; a layer that runs twice reads its weights twice), ``cache_bytes`` of the
        requests (``q_lens`` new tokens each, ``kv_lens`` held after the step), and ``flops`` of the products, the
        mixing and the head at ``logit_rows`` rows."""
        T = sum(q_lens)
        itemsize = cache_itemsize or self.rt.dtype.itemsize
        weight_bytes = self.head.weight_bytes() + self.final_norm.weight_bytes()
        cache_bytes, flops = 0, self.head.flops(logit_rows)
        for e in self.plan.schedule:
            block = self.blocks[e.layer]
            weight_bytes += block.step_weight_bytes(T) if hasattr(block, "step_weight_bytes") else block.weight_bytes()
            flops += block.flops(T)
            mixer = getattr(block, "mixer", None)
            if mixer is not None and e.cache >= 0:
                flops += mixer.mixing_flops(q_lens, kv_lens)
                cache_bytes += mixer.cache_bytes_read(q_lens, kv_lens, itemsize)
        return {"weight_bytes": weight_bytes, "cache_bytes": cache_bytes, "flops": flops}

    def uncapturable_parts(self) -> list[str]:
        """Kinds of the parts whose ``capturable`` is false (their forward cannot run inside a CUDA graph)."""
        out = []
        for block in self.blocks:
            for part in (block, *vars(block).values()):
                if getattr(part, "capturable", True) is False and getattr(part, "kind", "?") not in out:
                    out.append(getattr(part, "kind", "?"))
        return out

    def metadata_providers(self) -> dict:
        """{key: a mixer that makes the per-step data its kind needs}: one for each distinct ``metadata_key``."""
        out = {}
        for block in self.blocks:
            mixer = getattr(block, "mixer", None)
            if hasattr(mixer, "metadata_providers"):
                for key, provider in mixer.metadata_providers().items():
                    out.setdefault(key, provider)
            elif getattr(mixer, "metadata_key", None) is not None:
                out.setdefault(mixer.metadata_key, mixer)
        return out

    def _view(self, storage, slot: int, writes: bool) -> CacheView | None:
        """The cache view of one manager slot."""
        cplan = storage.manager.plan
        g = cplan.group_of_slot[slot]
        if g < 0:
            return None
        if cplan.groups[g].kind == "paged":
            k, v = storage.pages(slot)
            return CacheView(g, writes, k_pages=k, v_pages=v)
        return CacheView(g, writes, state=storage.state(slot))

    def _cache_view(self, storage, e) -> CacheView | None:
        if e.cache < 0:
            return None
        if self.slot_leaves is None:
            return self._view(storage, e.cache, e.writes)
        leaves = self.slot_leaves[e.cache]
        if len(leaves) == 1 and leaves[0][0] == ():
            return self._view(storage, leaves[0][1], e.writes)
        root = CacheView(-1, e.writes)
        for path, slot in leaves:
            node = root
            for name in path[:-1]:
                node = node.parts.setdefault(name, CacheView(-1, e.writes))
            node.parts[path[-1]] = self._view(storage, slot, e.writes)
        return root

    # ------------------------------------------------------------------ the step
    def forward(self, ctx, storage) -> torch.Tensor:
        """Run the step's tokens through every scheduled layer; logits float32 [R, V] at ctx.logit_rows."""
        rt = self.rt
        plan = self.plan
        if plan.residual_dtype == "float32" or plan.embedding_scale != 1.0:
            # the stream in float32 whatever the run's precision (a scaled embedding row is not rounded either)
            if plan.residual_dtype != "float32" and rt.dtype != torch.float32:
                raise ValueError("a scaled embedding is built for a float32 residual stream")
            x = torch.empty((ctx.num_tokens, plan.hidden_size), device=rt.device, dtype=torch.float32)
            ops.embed_scaled(self.embedding, ctx.tokens, x, plan.embedding_scale)
        else:
            x = torch.empty((ctx.num_tokens, plan.hidden_size), device=rt.device, dtype=rt.dtype)
            ops.embed(self.embedding, ctx.tokens, x)
        delta = None
        if not hasattr(self, "slot_leaves"):
            self.cache_plan()
        mult = 1.0
        both = None
        if any(e.stream_mix is not None for e in plan.schedule):
            # [stream | embedding output] in the parts' element type: the right half is written once
            H = plan.hidden_size
            both = torch.empty((ctx.num_tokens, 2 * H), device=rt.device, dtype=rt.dtype)
            ops.cast_rows_f32(x, both[:, H:])
        for e in plan.schedule:
            if e.stream_mix is not None:
                x, delta = settle(x, delta)
                ops.cast_rows_f32(x, both[:, :plan.hidden_size])
                x = self.stream_matrices[e.stream_mix](both, out_dtype=torch.float32)
            if e.stream_add is not None:
                # a vector of the model joins the stream (the pending output of the layer before joins it later, in
                # the next norm's kernel: the two sums commute)
                name, row = e.stream_add
                ops.add_row_f32(x, self.stream_vectors[name][row])
            block = self.blocks[e.layer]
            x, delta = block.forward(x, delta, ctx, self._cache_view(storage, e))
            mult = getattr(block, "residual_mult", 1.0)
        if ctx.num_logit_rows == 0:
            return torch.empty((0, plan.vocab_size), device=rt.device, dtype=torch.float32)
        if isinstance(delta, NormedDelta):
            x, delta = settle(x, delta)
        kw = {"out_dtype": rt.dtype} if x.dtype != rt.dtype else {}
        if mult != 1.0:
            kw["delta_scale"] = mult        # the last layer's output joins the stream with its block's factor
        h = self.final_norm.forward(x, delta, rows=ctx.logit_rows, **kw)
        logits = self.head(h, out_dtype=torch.float32)
        if plan.logit_scale != 1.0:
            ops.scale_f32(logits, plan.logit_scale)
        if plan.logit_softcap > 0.0:
            ops.softcap_f32(logits, plan.logit_softcap)
        return logits
