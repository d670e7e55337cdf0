"""RMSNorm."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..registry import register_norm
from ..weights.loader import TensorSpec
from .base import Norm


@register_norm("rms_norm")
class RMSNorm(Norm):
    """y = x / sqrt(mean(x^2) + eps) * (offset + w), statistics in float32
    (crates/metal-backend/src/shaders/elementwise.metal:31-46; no +1 offset for Llama).
    `offset` 1 is for checkpoints that keep a norm's weight as its difference from 1; the sum is made once, in float32, when the
    weights are bound."""

    graph_safe = True
    folds_pending = True

    def __init__(self, size: int, eps: float, offset: float = 0.0):
        self.size = size
        self.eps = float(eps)
        self.offset = float(offset)
        self.weight: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.size,))}

    def bind(self, weights, runtime) -> None:
        weight = weights["weight"]
        if self.offset != 0.0:
            weight = weight.to(torch.float32) + self.offset
        self.weight = weight.contiguous()

    def forward(self, hidden, ctx, rows=None):
        # partial sums a product left for the residual stream are added in the same pass
        pending = ctx.take_pending()
        return ops.rms_norm(hidden, self.weight, self.eps, ctx.runtime.dtype, rows=rows, partials=pending)

    def add_into(self, hidden, y, ctx, mult=1.0, then=None):
        # one pass: the sublayer's output is normalized, scaled and added to the stream, and the
        # updated row goes through the next sublayer's norm while it is still in registers
        fused = isinstance(then, RMSNorm) and then.weight.dtype == self.weight.dtype
        out = ops.rms_norm_add_(hidden, y, self.weight, self.eps, mult,
                                then.weight if fused else None, then.eps if fused else None,
                                ctx.runtime.dtype if fused else None)
        if then is not None and not fused:
            out = then.forward(hidden, ctx)
        return out
