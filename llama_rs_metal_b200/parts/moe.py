"""Mixture of experts: a router picks a few small gated feed-forwards per token."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import InvalidError, UnsupportedError
from ..kernels import ops
from ..registry import register_feed_forward
from ..weights.loader import TensorSpec
from .base import FeedForward
from .linear import LinearWeight


@register_feed_forward("moe")
class MixtureOfExperts(FeedForward):
    """z = W_r x (+ b_r) in float32; the `top` experts with the largest z are chosen and weighted
    by the softmax over the chosen z only; the output is the weighted sum of their outputs,
    added to the residual stream.

    An expert (activation "clamped_gate"): g = min(W_gate x, limit), u = clamp(W_up x, -limit,
    limit), y = g sigmoid(alpha g) (u + 1), output W_down y; no biases.

    The router's matrix is kept in float32 whatever the runtime, so its product runs on the
    float32 kernel. The experts' matrices are stacked, gate_up [E, 2 ff, h] and down [h, E, ff],
    and serve two ways of computing (csrc/moe.cu). Token by token (decoding, float32, many
    experts per choice): one launch reads, for every token, only the experts it chose; their
    outputs come back as float32 planes that are added to the stream in a fixed order (by the
    next norm where it folds them). All experts at once (bfloat16 steps of DENSE_ROWS tokens and
    more when at most DENSE_RATIO experts exist per chosen one): two tensor-core products over
    every expert, with the weights of the experts a token did not choose set to zero between
    them."""

    graph_safe = True
    ROUTER_ROWS = 256  # up to this many tokens the router always runs as one launch, a CTA per token
    DENSE_ROWS = 64   # from this many tokens on a step is a prompt: the tensor-core products pay
    DENSE_RATIO = 4   # experts per chosen expert up to which computing all of them is the faster way

    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top: int,
                 activation: str = "clamped_gate", limit: float = 7.0, alpha: float = 1.702,
                 router_bias: bool = True):
        if activation != "clamped_gate":
            raise UnsupportedError(f"expert activation {activation!r}")
        if num_experts <= 0 or not 0 < top <= num_experts:
            raise InvalidError("the router chooses between 1 and all of the experts")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.num_experts, self.top = num_experts, top
        self.limit, self.alpha, self.router_bias = float(limit), float(alpha), bool(router_bias)
        self.router: Optional[LinearWeight] = None
        self.bias: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        h, f = self.hidden_size, self.intermediate_size
        out = {"router.weight": TensorSpec((self.num_experts, h))}
        if self.router_bias:
            out["router.bias"] = TensorSpec((self.num_experts,))
        for e in range(self.num_experts):
            out[f"experts.{e}.gate_proj.weight"] = TensorSpec((f, h))
            out[f"experts.{e}.up_proj.weight"] = TensorSpec((f, h))
            out[f"experts.{e}.down_proj.weight"] = TensorSpec((h, f))
        return out

    def bind(self, weights, runtime) -> None:
        self.router = LinearWeight(weights["router.weight"].to(torch.float32))
        self.bias = weights["router.bias"].to(torch.float32).contiguous() if self.router_bias else None
        E, f, h = self.num_experts, self.intermediate_size, self.hidden_size
        self.gate_up = torch.stack([torch.cat([weights[f"experts.{e}.gate_proj.weight"],
                                               weights[f"experts.{e}.up_proj.weight"]]) for e in range(E)]).contiguous()
        self.down = torch.stack([weights[f"experts.{e}.down_proj.weight"] for e in range(E)], dim=1).contiguous()
        # the same storage seen as two plain matrices, for the products over every expert
        self.gate_up_all = LinearWeight(self.gate_up.view(E * 2 * f, h))
        self.down_all = LinearWeight(self.down.view(h, E * f))

    def route(self, x):
        """(expert ids int32 [T, top], weights float32 [T, top]). One launch per step; steps of
        many tokens make the logits with the float32 matrix kernel first when there are many
        experts to a token's CTA."""
        routed = ops.moe_router(x, self.router.weight, self.bias, self.top) \
            if x.shape[0] <= self.ROUTER_ROWS or self.num_experts <= 16 else None
        if routed is None:
            routed = ops.moe_route(self.router(x, out_dtype=torch.float32), self.bias, self.top)
        return routed

    def forward(self, x, ctx, residual):
        ids, weights = self.route(x)
        if (x.dtype == torch.bfloat16 and self.gate_up.dtype == torch.bfloat16 and x.shape[0] >= self.DENSE_ROWS
                and self.num_experts <= self.DENSE_RATIO * self.top):
            # gate and up stay float32 up to the activation, as they do token by token
            both = self.gate_up_all(x, out_dtype=torch.float32)
            y = ops.moe_dense_gate(both, ids, weights, self.num_experts, self.limit, self.alpha, out_dtype=x.dtype)
            return self.down_all(y, epilogue=ops.ADD, out=residual, ctx=ctx)
        planes = ops.moe_experts_rows(x, self.gate_up, self.down, ids, weights, self.limit, self.alpha)
        if ctx.may_defer:
            ctx.settle(residual)  # at most one set of partial sums is pending at a time
            ctx.pending = planes
            return residual
        return ops.add_planes_(residual, planes)
