"""Norms with the residual sum fused in."""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.needs import TensorNeed
from .base import Norm, Runtime
from .registry import register


@register("norm", "rmsnorm")
class RMSNorm(Norm):
    """out = cast(x32 * rsqrt(mean(x32^2) + eps)) * w, the weight being plain ``w``
    (acvram/engine/layers.py:607-630); with ``delta`` the sum x + delta is made first,
    in 32-bit, and written back (acvram/engine/layers.py:633-651)."""

    def __init__(self, hidden_size: int, eps: float, size: int | None = None, tensor: str = "weight", groups: int = 1) -> None:
        """``tensor``: the weight's name behind the norm's prefix ("" where the prefix is the whole name).
        ``groups`` > 1: the row is split into that many equal consecutive parts and each is divided by its own root mean
        square (the weight still spans the whole row); such a norm wants a float32 residual stream."""
        self.size = size or hidden_size
        self.groups = int(groups)
        if self.groups < 1 or self.size % self.groups:
            raise ValueError(f"a norm over {self.size} elements does not split into {groups} equal groups")
        self.eps = float(eps)
        self.tensor = tensor
        self.weight: torch.Tensor | None = None

    def tensor_needs(self):
        return {self.tensor: TensorNeed((self.size,), "norm")}

    def load(self, tensors, rt: Runtime) -> None:
        self.weight = tensors[self.tensor].to(device=rt.device, dtype=torch.float32).contiguous()

    def decode_layer_spec(self):
        """What the fused decode-layer kernel needs of this norm."""
        return {"weight": self.weight, "eps": self.eps} if self.groups == 1 else None

    def weight_bytes(self) -> int:
        return 0 if self.weight is None else self.weight.numel() * 4

    def forward(self, x, delta, rows=None, out_dtype=None, delta_scale: float = 1.0):
        """A float32 stream beside parts that run in ``out_dtype`` (bfloat16): sum and norm stay 32-bit, the norm's output
        is rounded once.  ``delta_scale``: x += delta_scale * delta (float32 stream only)."""
        n = rows.shape[0] if rows is not None else x.shape[0]
        out_dtype = out_dtype or (delta.dtype if delta is not None else x.dtype)
        out = torch.empty((n, x.shape[1]), device=x.device, dtype=out_dtype)
        if self.groups > 1 or delta_scale != 1.0 or (x.dtype == torch.float32 and delta is not None and delta.dtype != out_dtype):
            if x.dtype != torch.float32:
                raise ValueError("a grouped norm or a factor on the residual wants a float32 residual stream (ModelPlan.residual_dtype)")
            return ops.add_group_rmsnorm(x, delta, self.weight, self.eps, self.groups, out, rows, delta_scale)
        if x.dtype == torch.float32 and out_dtype != torch.float32:
            return ops.add_rmsnorm_f32(x, delta, self.weight, self.eps, out, rows)
        return ops.add_rmsnorm(x, delta, self.weight, self.eps, out, rows)


@register("norm", "layernorm")
class LayerNorm(Norm):
    """out = (x - mean) / sqrt(var + eps) * w + b over a float32 residual stream, var the mean of the squared
    deviations; the sum x += delta_scale * delta is made first, in 32-bit, and written back.  Mean, variance and the
    affine step are 32-bit in every run precision; the result is rounded once to the parts' element type.
    ``tensor`` and ``bias_tensor``: the names of w and b behind the norm's prefix (``bias_tensor`` None: no b)."""

    def __init__(self, hidden_size: int, eps: float, size: int | None = None, tensor: str = "weight",
                 bias_tensor: str | None = "bias") -> None:
        self.size = size or hidden_size
        self.eps = float(eps)
        self.tensor, self.bias_tensor = tensor, bias_tensor
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    def tensor_needs(self):
        needs = {self.tensor: TensorNeed((self.size,), "norm")}
        if self.bias_tensor is not None:
            needs[self.bias_tensor] = TensorNeed((self.size,), "bias")
        return needs

    def load(self, tensors, rt: Runtime) -> None:
        f = lambda n: tensors[n].to(device=rt.device, dtype=torch.float32).contiguous()
        self.weight = f(self.tensor)
        self.bias = f(self.bias_tensor) if self.bias_tensor is not None else None

    def weight_bytes(self) -> int:
        return sum(t.numel() * 4 for t in (self.weight, self.bias) if t is not None)

    def forward(self, x, delta, rows=None, out_dtype=None, delta_scale: float = 1.0):
        if x.dtype != torch.float32:
            raise ValueError("the layer norm is built for a float32 residual stream (ModelPlan.residual_dtype)")
        n = rows.shape[0] if rows is not None else x.shape[0]
        out_dtype = out_dtype or (delta.dtype if delta is not None else x.dtype)
        out = torch.empty((n, x.shape[1]), device=x.device, dtype=out_dtype)
        return ops.add_layernorm(x, delta, self.weight, self.bias, self.eps, out, rows, delta_scale)
