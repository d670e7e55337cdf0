"""The Pibuvik decoder as a plan of parts.

Every layer has a norm in front of and behind each sublayer, and what a sublayer adds to the
residual stream is multiplied by one factor: x <- x + m * norm_b(sublayer(norm_a(x))), first for
a mixer, then for a clamped-gate feed-forward (or nothing). Three kinds of mixer: `rglru`, a
gated linear recurrence per channel behind a short convolution; `attention`, causal grouped-query
attention without rotation whose values are its keys, with a per-head sink in the softmax and a
query temperature that grows with the position; `latent_attention`, windowed attention whose
keys and values are unfolded from a small cached latent, with rotary positions on a key part all
heads share and a sigmoid gate per head, and which may read the latent another layer cached.
The embedding is scaled, the head is the embedding table, and the logits are scaled.

Checkpoint names: `embed`, `final.norm`, and per layer i `l<i>.norm1`, `l<i>.norm1b`, `l<i>.norm2`,
`l<i>.norm2b`, `l<i>.mix.*`, `l<i>.mlp.*`; a projection's bias is the matrix's name + `.b`, a
latent's norm weight the down-projection's name + `.norm`.
"""
from __future__ import annotations

from ..config.pibuvik import PibuvikConfig
from ..parts.base import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
from ..registry import register_architecture

MAX_POSITIONS = 1 << 20  # the design names no limit
DECAY_FACTOR = 8.0       # a = exp(-DECAY_FACTOR * r * softplus(lam)) in the recurrent mixer
GATE_ALPHA = 1.702       # g * sigmoid(GATE_ALPHA * g) in the feed-forward


def _recurrence(config: PibuvikConfig, m, p: str) -> PartSpec:
    names = {"x_proj.weight": p + "x", "x_proj.bias": p + "x.b", "y_proj.weight": p + "y", "y_proj.bias": p + "y.b",
             "conv.weight": p + "conv", "conv.bias": p + "conv.b", "decay_gate.weight": p + "ra",
             "decay_gate.bias": p + "ra.b", "input_gate.weight": p + "ri", "input_gate.bias": p + "ri.b",
             "lam": p + "lam", "o_proj.weight": p + "o"}
    return PartSpec("gated_linear_recurrence", dict(hidden_size=config.width, channels=m.width, blocks=m.blocks,
                                                    conv_taps=m.conv, decay_factor=DECAY_FACTOR), names=names)


def _sink_attention(config: PibuvikConfig, m, p: str) -> PartSpec:
    names = {"q_proj.weight": p + "q", "k_proj.weight": p + "k", "o_proj.weight": p + "o", "sinks": p + "sink"}
    temperature = (m.temp_coef, m.temp_every) if m.temp_every is not None else None
    return PartSpec("attention", dict(
        hidden_size=config.width, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, position=None,
        window=None, scale=m.scale, values_are_keys=True, sinks=True, query_temperature=temperature), names=names)


def _latent_attention(config: PibuvikConfig, m, p: str, cache_window) -> PartSpec:
    names = {"q_down.weight": p + "dq", "q_down.norm": p + "dq.norm", "q_up.weight": p + "uq",
             "kv_down.weight": p + "dkv", "kv_down.norm": p + "dkv.norm", "k_up.weight": p + "uk",
             "v_up.weight": p + "uv", "gate.weight": p + "g", "o_proj.weight": p + "o"}
    position = PartSpec("rope", dict(head_dim=m.rot_dim, rotary_dim=m.rot_dim, theta=m.rot_base))
    return PartSpec("latent_attention", dict(
        hidden_size=config.width, num_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim,
        kv_rank=m.kv_rank, q_rank=m.q_rank, eps=config.eps, scale=m.scale, position=position, window=m.window,
        owns_latent=m.kv_from is None, cache_window=cache_window), names=names)


def _dense(config: PibuvikConfig, f, p: str) -> PartSpec:
    names = {"gate_proj.weight": p + "gate", "up_proj.weight": p + "up", "down_proj.weight": p + "down"}
    return PartSpec("gated_mlp", dict(hidden_size=config.width, intermediate_size=f.ff, activation="clamped_gate",
                                      limit=f.limit, alpha=GATE_ALPHA), names=names)


def pibuvik_plan(config: PibuvikConfig) -> ModelPlan:
    norm = dict(size=config.width, eps=config.eps)
    # a cached latent is kept for as long as its widest reader looks back (forever, if one has no window)
    readers = {}
    for i, layer in enumerate(config.layers):
        if layer.kind == "latent_attention":
            readers.setdefault(i if layer.mixer.kv_from is None else layer.mixer.kv_from, []).append(layer.mixer.window)
    layers, schedule, cache_of = [], [], {}
    for i, layer in enumerate(config.layers):
        p = f"l{i}."
        m = layer.mixer
        if layer.kind == "rglru":
            mixer = _recurrence(config, m, p + "mix.")
        elif layer.kind == "attention":
            mixer = _sink_attention(config, m, p + "mix.")
        else:
            windows = readers[i if m.kv_from is None else m.kv_from]
            mixer = _latent_attention(config, m, p + "mix.", None if None in windows else max(windows))
        parts = dict(mixer=mixer, mixer_norm=PartSpec("rms_norm", norm, names={"weight": p + "norm1"}),
                     mixer_post_norm=PartSpec("rms_norm", norm, names={"weight": p + "norm1b"}))
        if layer.mlp is not None:
            parts.update(feed_forward=_dense(config, layer.mlp, p + "mlp."),
                         feed_forward_norm=PartSpec("rms_norm", norm, names={"weight": p + "norm2"}),
                         feed_forward_post_norm=PartSpec("rms_norm", norm, names={"weight": p + "norm2b"}))
        layers.append(LayerSpec("sandwich_norm" if layer.mlp is not None else "sandwich_norm_mixer", parts=parts,
                                options=dict(residual_mult=config.residual_mult)))
        source = getattr(m, "kv_from", None)
        if source is None:
            cache_of[i] = len(cache_of)  # a cache entry of its own
            schedule.append(ScheduleEntry(layer=i, cache=cache_of[i]))
        else:
            schedule.append(ScheduleEntry(layer=i, cache=cache_of[source], writes_cache=False))
    return ModelPlan(
        hidden_size=config.width, vocab_size=config.vocab, max_positions=MAX_POSITIONS,
        embedding_name="embed", layers=tuple(layers), schedule=tuple(schedule),
        final_norm=PartSpec("rms_norm", norm, names={"weight": "final.norm"}), head_name=None,
        embedding_scale=config.embedding_scale if config.embedding_scale != 1.0 else None,
        logit_scale=config.logit_scale if config.logit_scale != 1.0 else None)


register_architecture("Pibuvik", PibuvikConfig, pibuvik_plan, model_types=("pibuvik",))
