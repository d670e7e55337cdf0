"""Configuration of the Kikalix decoder, read from its own config.json keys.

    {"architecture": "Kikalix", "vocab": V, "width": W, "norm": {"eps": e},
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "retention" | "parallel", "mixer": {...}, "mlp": {...} | null}, ...]}

A retention mixer: heads, dim, vdim, decay (one per head), rot {dims, base}. A parallel mixer:
left {heads, kv_heads, dim, vdim, scale, mask {size}}, right {heads, kv_heads, dim, vdim, conv},
left_scale, right_scale. A feed-forward: kind "moe", expert {ff, limit}, router {experts, top}.
Every size and every constant that can differ between models comes from here; the inner ranks
of the right mixer's two low-rank products are no configuration keys and are read off the
checkpoint's tensors (the optional keys right.decay_rank and right.gate_rank give them to the
random-weights mode, which has no checkpoint to ask).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import InvalidError, UnsupportedError
from .base import read_int, read_real


def _table(parent: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = parent.get(key)
    if not isinstance(value, Mapping):
        raise InvalidError(f"missing config.{where}{key}")
    return value


def _positive(table: Mapping[str, Any], key: str, where: str) -> int:
    value = read_int(table, key, None)
    if value is None or value <= 0:
        raise InvalidError(f"config.{where}{key} must be a positive integer")
    return value


def _real(table: Mapping[str, Any], key: str, where: str) -> float:
    value = table.get(key)
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise InvalidError(f"missing config.{where}{key}")
    return read_real(table, key, 0.0)


@dataclass(frozen=True)
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot_dims: int
    rot_base: float

    @classmethod
    def read(cls, m: Mapping[str, Any], where: str) -> "RetentionConfig":
        heads, dim, vdim = (_positive(m, k, where) for k in ("heads", "dim", "vdim"))
        decay = m.get("decay")
        if not isinstance(decay, list) or len(decay) != heads or \
                any(isinstance(a, bool) or not isinstance(a, (int, float)) for a in decay):
            raise InvalidError(f"config.{where}decay must list one number per head")
        rot = m.get("rot")
        dims, base = 0, 10000.0
        if isinstance(rot, Mapping):
            dims = read_int(rot, "dims", 0)
            base = _real(rot, "base", where + "rot.") if dims else 10000.0
        if dims % 2 or dims > dim or (dims and base <= 0):
            raise InvalidError(f"config.{where}rot: dims must be even and at most dim, base positive")
        return cls(heads, dim, vdim, tuple(float(a) for a in decay), dims, base)

    def to_dict(self) -> dict:
        out = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}
        if self.rot_dims:
            out["rot"] = {"dims": self.rot_dims, "base": self.rot_base}
        return out


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int

    @classmethod
    def read(cls, m: Mapping[str, Any], where: str) -> "WindowAttentionConfig":
        heads, kv_heads, dim, vdim = (_positive(m, k, where) for k in ("heads", "kv_heads", "dim", "vdim"))
        if heads % kv_heads:
            raise InvalidError(f"config.{where}heads must be a multiple of kv_heads")
        window = _positive(_table(m, "mask", where), "size", where + "mask.")
        return cls(heads, kv_heads, dim, vdim, _real(m, "scale", where), window)

    def to_dict(self) -> dict:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                "scale": self.scale, "mask": {"size": self.window}}


@dataclass(frozen=True)
class DeltaRuleConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: Optional[int] = None
    gate_rank: Optional[int] = None

    @classmethod
    def read(cls, m: Mapping[str, Any], where: str) -> "DeltaRuleConfig":
        heads, kv_heads, dim, vdim, conv = (_positive(m, k, where) for k in ("heads", "kv_heads", "dim", "vdim", "conv"))
        if heads % kv_heads:
            raise InvalidError(f"config.{where}heads must be a multiple of kv_heads")
        return cls(heads, kv_heads, dim, vdim, conv, read_int(m, "decay_rank", None), read_int(m, "gate_rank", None))

    def to_dict(self) -> dict:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}
        if self.decay_rank is not None:
            out["decay_rank"] = self.decay_rank
        if self.gate_rank is not None:
            out["gate_rank"] = self.gate_rank
        return out


@dataclass(frozen=True)
class ParallelConfig:
    left: WindowAttentionConfig
    right: DeltaRuleConfig
    left_scale: float
    right_scale: float

    @classmethod
    def read(cls, m: Mapping[str, Any], where: str) -> "ParallelConfig":
        return cls(WindowAttentionConfig.read(_table(m, "left", where), where + "left."),
                   DeltaRuleConfig.read(_table(m, "right", where), where + "right."),
                   _real(m, "left_scale", where), _real(m, "right_scale", where))

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class ExpertsConfig:
    ff: int
    limit: float
    experts: int
    top: int

    @classmethod
    def read(cls, m: Mapping[str, Any], where: str) -> "ExpertsConfig":
        kind = m.get("kind")
        if kind != "moe":
            raise UnsupportedError(f"config.{where}kind {kind!r}: only \"moe\" is built")
        expert, router = _table(m, "expert", where), _table(m, "router", where)
        ff = _positive(expert, "ff", where + "expert.")
        experts, top = _positive(router, "experts", where + "router."), _positive(router, "top", where + "router.")
        if top > experts:
            raise InvalidError(f"config.{where}router.top exceeds the number of experts")
        return cls(ff, _real(expert, "limit", where + "expert."), experts, top)

    def to_dict(self) -> dict:
        return {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit},
                "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class KikalixLayer:
    kind: str  # "retention" | "parallel"
    mixer: Any  # RetentionConfig | ParallelConfig
    mlp: Optional[ExpertsConfig]

    def to_dict(self) -> dict:
        return {"type": self.kind, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None}


@dataclass(frozen=True)
class KikalixConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[KikalixLayer, ...]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    architecture: str = "Kikalix"

    @classmethod
    def from_dict(cls, root: Mapping[str, Any]) -> "KikalixConfig":
        vocab, width = _positive(root, "vocab", ""), _positive(root, "width", "")
        eps = _real(_table(root, "norm", ""), "eps", "norm.")
        if eps <= 0:
            raise InvalidError("config.norm.eps must be positive")
        listed = root.get("layers")
        if not isinstance(listed, list) or not listed or len(listed) > 1024:
            raise InvalidError("config.layers must list 1 to 1024 layers")
        layers = []
        for i, item in enumerate(listed):
            where = f"layers[{i}]."
            if not isinstance(item, Mapping):
                raise InvalidError(f"config.layers[{i}] must be an object")
            kind, mixer = item.get("type"), _table(item, "mixer", where)
            if kind == "retention":
                mixer = RetentionConfig.read(mixer, where + "mixer.")
            elif kind == "parallel":
                mixer = ParallelConfig.read(mixer, where + "mixer.")
            else:
                raise UnsupportedError(f"config.{where}type {kind!r}: \"retention\" and \"parallel\" are built")
            mlp = item.get("mlp")
            if mlp is not None and not isinstance(mlp, Mapping):
                raise InvalidError(f"config.{where}mlp must be an object or null")
            layers.append(KikalixLayer(kind, mixer, ExpertsConfig.read(mlp, where + "mlp.") if mlp is not None else None))
        start, stop, times = 0, 0, 1
        loop = root.get("loop")
        if isinstance(loop, Mapping):
            start, stop = read_int(loop, "start"), read_int(loop, "stop")
            times = _positive(loop, "times", "loop.")
            if not 0 <= start <= stop <= len(layers) or times > 1024:
                raise InvalidError("config.loop: 0 <= start <= stop <= number of layers, times at most 1024")
        return cls(vocab, width, eps, tuple(layers), start, stop, times)

    @property
    def loops(self) -> bool:
        return self.loop_stop > self.loop_start

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "layers": [layer.to_dict() for layer in self.layers]}
        if self.loops:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return out
