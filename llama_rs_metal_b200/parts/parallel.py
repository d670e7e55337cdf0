"""Two mixers side by side on the same input."""
from __future__ import annotations

from typing import Dict

from ..registry import MIXERS, build_part, register_mixer
from ..weights.loader import TensorSpec
from .base import CompositeRequest, Mixer, PartSpec


@register_mixer("parallel")
class ParallelMixer(Mixer):
    """left_scale * left(x) + right_scale * right(x), both added to the residual stream.

    `left` and `right` are PartSpecs of registered mixers that take `output_scale`; each gets its
    scale there (it multiplies the mixer's heads before its output projection, so the weighted
    sum costs no pass of its own) and the part of the layer's cache it asked for. Their tensors
    are this part's, under "left." and "right."."""

    def __init__(self, left: PartSpec, right: PartSpec, left_scale: float = 1.0, right_scale: float = 1.0):
        self.left = build_part(MIXERS, PartSpec(left.kind, {**left.params, "output_scale": float(left_scale)}),
                               "mixer")
        self.right = build_part(MIXERS, PartSpec(right.kind, {**right.params, "output_scale": float(right_scale)}),
                                "mixer")

    @property
    def graph_safe(self) -> bool:
        return self.left.graph_safe and self.right.graph_safe

    def tensors(self) -> Dict[str, TensorSpec]:
        out = {"left." + n: s for n, s in self.left.tensors().items()}
        out.update({"right." + n: s for n, s in self.right.tensors().items()})
        return out

    def bind(self, weights, runtime) -> None:
        self.left.bind({n[len("left."):]: t for n, t in weights.items() if n.startswith("left.")}, runtime)
        self.right.bind({n[len("right."):]: t for n, t in weights.items() if n.startswith("right.")}, runtime)

    def cache_request(self):
        return CompositeRequest((self.left.cache_request(), self.right.cache_request()))

    def forward(self, x, ctx, cache, residual):
        left_cache, right_cache = cache if cache is not None else (None, None)
        residual = self.left.forward(x, ctx, left_cache, residual)
        return self.right.forward(x, ctx, right_cache, residual)
