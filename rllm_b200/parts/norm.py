"""RMSNorm as a part. Formula and rounding: src/gpu/cuda/shaders/rms_norm.cu:78-115 of the
reference (sum of squares and scaling in float, weight used as stored). `offset`: the checkpoint stores
the weight minus this number (weights "around zero": offset 1); the sum is formed once, in float."""
from __future__ import annotations

from .base import Param, Part, Source, register_part


class RMSNorm(Part):
    graph_safe = True

    def __init__(self, size: int, eps: float, weight_name: str = "weight", offset: float = 0.0):
        self.size, self.eps, self.weight_name, self.offset = size, float(eps), weight_name, float(offset)
        self.weight = self.stored = None

    def params(self):
        if self.offset:
            # what the checkpoint holds is bound to `stored`; `weight` is made from it when the weights are bound
            return [Param("stored", (Source(self.weight_name, (self.size,), init="normal"),), role="vector")]
        return [Param("weight", (Source(self.weight_name, (self.size,), init="norm"),), role="vector")]

    def forward(self, h, ctx):
        """h: float32 residual stream [T, size] -> normalised activations in the run dtype."""
        return ctx.backend.rmsnorm(h, self.weight, self.eps)

    def deferred(self, h, ctx, rows=None):
        """The same norm (of rows `rows` of h when given) for a consumer that may run it inside its
        own first product: a tensor, or the backend's deferred form that its products accept."""
        return ctx.backend.normed(h, self.weight, self.eps, rows)

    def weight_f32(self):
        """The weight as float32 (kernels that norm in float throughout take it so); made once."""
        if getattr(self, "_w32", None) is None:
            self._w32 = self.weight.float().contiguous()
        return self._w32

    def finalize(self, device, dtype):
        self._w32 = None            # weights were (re)bound
        if self.offset:
            self.weight = (self.stored.float() + self.offset).contiguous()

    def forward_f32(self, h, ctx):
        import torch
        return ctx.backend.rmsnorm(h, self.weight, self.eps, out_dtype=torch.float32)


register_part("norm", "rmsnorm", RMSNorm)
