"""Configuration of the Pibuvik decoder, read from its own config.json keys.

    {"architecture": "Pibuvik", "vocab": V, "width": W, "norm": {"eps": e}, "residual_mult": m,
     "embedding": {"scale": s}, "logit_scale": z,
     "layers": [{"type": "rglru" | "attention" | "latent_attention", "mixer": {...}, "mlp": {...} | null}, ...]}

An rglru mixer: width (channels), blocks, conv (taps). An attention mixer: heads, kv_heads, dim,
vdim (the values are the keys, so vdim equals dim), scale, q_temp {coef, every} (optional). A
latent_attention mixer: heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot {dims, base},
mask {size} (optional: without it every earlier position is seen), kv_from (optional: the layer
whose cached latent this layer reads). A feed-forward: kind "dense", ff, limit. Every size and every
constant that can differ between models comes from here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import InvalidError, UnsupportedError
from .base import read_int
from .kikalix import _positive, _real, _table


@dataclass(frozen=True)
class RecurrenceConfig:
    width: int
    blocks: int
    conv: int

    @classmethod
    def read(cls, m: Mapping[str, Any], where: str) -> "RecurrenceConfig":
        width, blocks, conv = (_positive(m, k, where) for k in ("width", "blocks", "conv"))
        if width % blocks:
            raise InvalidError(f"config.{where}width must be a multiple of blocks")
        return cls(width, blocks, conv)

    def to_dict(self) -> dict:
        return {"width": self.width, "blocks": self.blocks, "conv": self.conv}


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    temp_coef: Optional[float] = None
    temp_every: Optional[int] = None

    @classmethod
    def read(cls, m: Mapping[str, Any], where: str) -> "SinkAttentionConfig":
        heads, kv_heads, dim = (_positive(m, k, where) for k in ("heads", "kv_heads", "dim"))
        vdim = read_int(m, "vdim", dim)
        if heads % kv_heads:
            raise InvalidError(f"config.{where}heads must be a multiple of kv_heads")
        if vdim != dim:
            raise InvalidError(f"config.{where}vdim must equal dim: the values are the keys")
        coef, every = None, None
        temp = m.get("q_temp")
        if isinstance(temp, Mapping):
            coef, every = _real(temp, "coef", where + "q_temp."), _positive(temp, "every", where + "q_temp.")
        return cls(heads, kv_heads, dim, vdim, _real(m, "scale", where), coef, every)

    def to_dict(self) -> dict:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.temp_every is not None:
            out["q_temp"] = {"coef": self.temp_coef, "every": self.temp_every}
        return out


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_base: float
    window: Optional[int] = None
    kv_from: Optional[int] = None

    @classmethod
    def read(cls, m: Mapping[str, Any], where: str) -> "LatentAttentionConfig":
        heads, dim, rot_dim, vdim, kv_rank, q_rank = (
            _positive(m, k, where) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"))
        rot = _table(m, "rot", where)
        if read_int(rot, "dims", rot_dim) != rot_dim or rot_dim % 2:
            raise InvalidError(f"config.{where}rot.dims must equal rot_dim, an even number")
        base = _real(rot, "base", where + "rot.")
        if base <= 0:
            raise InvalidError(f"config.{where}rot.base must be positive")
        window = None
        if isinstance(m.get("mask"), Mapping):
            window = _positive(m["mask"], "size", where + "mask.")
        return cls(heads, dim, rot_dim, vdim, kv_rank, q_rank, _real(m, "scale", where), base, window,
                   read_int(m, "kv_from", None))

    def to_dict(self) -> dict:
        out = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
               "kv_rank": self.kv_rank, "q_rank": self.q_rank, "scale": self.scale,
               "rot": {"dims": self.rot_dim, "base": self.rot_base}}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class DenseConfig:
    ff: int
    limit: float

    @classmethod
    def read(cls, m: Mapping[str, Any], where: str) -> "DenseConfig":
        kind = m.get("kind")
        if kind != "dense":
            raise UnsupportedError(f"config.{where}kind {kind!r}: only \"dense\" is built")
        return cls(_positive(m, "ff", where), _real(m, "limit", where))

    def to_dict(self) -> dict:
        return {"kind": "dense", "ff": self.ff, "limit": self.limit}


MIXERS = {"rglru": RecurrenceConfig, "attention": SinkAttentionConfig, "latent_attention": LatentAttentionConfig}


@dataclass(frozen=True)
class PibuvikLayer:
    kind: str  # a key of MIXERS
    mixer: Any
    mlp: Optional[DenseConfig]

    def to_dict(self) -> dict:
        return {"type": self.kind, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None}


@dataclass(frozen=True)
class PibuvikConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    embedding_scale: float
    logit_scale: float
    layers: Tuple[PibuvikLayer, ...]
    architecture: str = "Pibuvik"

    @classmethod
    def from_dict(cls, root: Mapping[str, Any]) -> "PibuvikConfig":
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
            kind = item.get("type")
            if kind not in MIXERS:
                raise UnsupportedError(f"config.{where}type {kind!r}: built are {', '.join(sorted(MIXERS))}")
            mixer = MIXERS[kind].read(_table(item, "mixer", where), where + "mixer.")
            mlp = item.get("mlp")
            if mlp is not None and not isinstance(mlp, Mapping):
                raise InvalidError(f"config.{where}mlp must be an object or null")
            layers.append(PibuvikLayer(kind, mixer, DenseConfig.read(mlp, where + "mlp.") if mlp is not None else None))
        for i, layer in enumerate(layers):
            source = getattr(layer.mixer, "kv_from", None)
            if source is None:
                continue
            where = f"layers[{i}].mixer."
            if not 0 <= source < i or layers[source].kind != "latent_attention" or layers[source].mixer.kv_from is not None:
                raise InvalidError(f"config.{where}kv_from must name an earlier latent_attention layer with a latent of its own")
            theirs, mine = layers[source].mixer, layer.mixer
            if (theirs.kv_rank, theirs.rot_dim, theirs.rot_base) != (mine.kv_rank, mine.rot_dim, mine.rot_base):
                raise InvalidError(f"config.{where}kv_from: kv_rank, rot_dim and rot must equal the named layer's")
        embedding = root.get("embedding")
        return cls(vocab, width, eps, _real(root, "residual_mult", "") if "residual_mult" in root else 1.0,
                   _real(embedding, "scale", "embedding.") if isinstance(embedding, Mapping) and "scale" in embedding else 1.0,
                   _real(root, "logit_scale", "") if "logit_scale" in root else 1.0, tuple(layers))

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "residual_mult": self.residual_mult, "embedding": {"scale": self.embedding_scale},
                "logit_scale": self.logit_scale, "layers": [layer.to_dict() for layer in self.layers]}
