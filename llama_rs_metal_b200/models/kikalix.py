"""The Kikalix decoder as a plan of parts.

Layers are pre-norm (a norm multiplies by 1 + its stored weight): a mixer, then a mixture of experts or
nothing. Two kinds of mixer: `retention` (a decayed outer-product state with rotary positions),
and `parallel`, a weighted sum of windowed grouped-query attention with a linear distance
penalty (biases on q, k, v, no rotation) and a gated delta rule. A run of layers may loop: it
runs several times in a row with the same weights, every pass with cache entries of its own,
and before each pass a vector of the table `loop.step` is added to the residual stream.

Checkpoint names: `embed`, `head`, `final.norm`, `loop.step`, and per layer i `l<i>.norm1`,
`l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.*`; a projection's bias is the matrix's name + `.b`, a
convolution's taps the matrix's name + `.conv`.
"""
from __future__ import annotations

from ..config.kikalix import KikalixConfig
from ..parts.base import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
from ..registry import register_architecture

MAX_POSITIONS = 1 << 20  # the design names no limit; the state mixers have none and the window is short


def _retention(config: KikalixConfig, m, p: str) -> PartSpec:
    position = None
    if m.rot_dims:
        position = PartSpec("rope", dict(head_dim=m.dim, rotary_dim=m.rot_dims, theta=m.rot_base))
    names = {f"{own}_proj.weight": p + own for own in ("q", "k", "v", "g", "o")}
    return PartSpec("retention", dict(hidden_size=config.width, num_heads=m.heads, head_dim=m.dim, value_dim=m.vdim,
                                      decay=m.decay, eps=config.eps, position=position), names=names)


def _window_attention(config: KikalixConfig, m) -> PartSpec:
    return PartSpec("attention", dict(
        hidden_size=config.width, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim,
        position=PartSpec("distance_penalty", dict(num_heads=m.heads)), window=m.window, scale=m.scale, bias=True))


def _attention_names(p: str) -> dict:
    names = {f"{own}_proj.weight": p + own for own in ("q", "k", "v", "o")}
    names.update({f"{own}_proj.bias": p + own + ".b" for own in ("q", "k", "v")})
    return names


def _delta_rule(config: KikalixConfig, m) -> PartSpec:
    return PartSpec("gated_delta_rule", dict(
        hidden_size=config.width, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim,
        conv_taps=m.conv, eps=config.eps, decay_rank=m.decay_rank, gate_rank=m.gate_rank))


def _delta_rule_names(p: str) -> dict:
    names = {f"{own}_proj.weight": p + own for own in ("q", "k", "v", "b", "o")}
    names.update({f"{own}_conv.weight": p + own + ".conv" for own in ("q", "k", "v")})
    names.update({"A_log": p + "A_log", "dt_bias": p + "dt_bias", "norm.weight": p + "norm",
                  "a_down.weight": p + "a1", "a_up.weight": p + "a2",
                  "g_down.weight": p + "g1", "g_up.weight": p + "g2"})
    return names


def _parallel(config: KikalixConfig, m, p: str) -> PartSpec:
    names = {"left." + own: full for own, full in _attention_names(p + "left.").items()}
    names.update({"right." + own: full for own, full in _delta_rule_names(p + "right.").items()})
    return PartSpec("parallel", dict(left=_window_attention(config, m.left), right=_delta_rule(config, m.right),
                                     left_scale=m.left_scale, right_scale=m.right_scale), names=names)


def _experts(config: KikalixConfig, f, p: str) -> PartSpec:
    names = {"router.weight": p + "router", "router.bias": p + "router.b"}
    for e in range(f.experts):
        for own in ("gate", "up", "down"):
            names[f"experts.{e}.{own}_proj.weight"] = f"{p}e{e}.{own}"
    return PartSpec("moe", dict(hidden_size=config.width, intermediate_size=f.ff, num_experts=f.experts, top=f.top,
                                activation="clamped_gate", limit=f.limit, alpha=1.702, router_bias=True), names=names)


def kikalix_plan(config: KikalixConfig) -> ModelPlan:
    norm = dict(size=config.width, eps=config.eps, offset=1.0)
    layers = []
    for i, layer in enumerate(config.layers):
        p = f"l{i}."
        mixer = _retention(config, layer.mixer, p + "mix.") if layer.kind == "retention" \
            else _parallel(config, layer.mixer, p + "mix.")
        parts = dict(mixer=mixer, mixer_norm=PartSpec("rms_norm", norm, names={"weight": p + "norm1"}))
        if layer.mlp is not None:
            parts.update(feed_forward=_experts(config, layer.mlp, p + "mlp."),
                         feed_forward_norm=PartSpec("rms_norm", norm, names={"weight": p + "norm2"}))
        layers.append(LayerSpec("pre_norm" if layer.mlp is not None else "pre_norm_mixer", **parts))
    # the order of layer runs: the looped run repeats, each pass on cache entries of its own
    runs = [(i, None) for i in range(config.loop_start)] if config.loops else []
    if config.loops:
        for t in range(config.loop_times):
            runs += [(i, t if i == config.loop_start else None) for i in range(config.loop_start, config.loop_stop)]
        runs += [(i, None) for i in range(config.loop_stop, len(layers))]
    else:
        runs = [(i, None) for i in range(len(layers))]
    schedule = tuple(ScheduleEntry(layer=i, cache=n, add_offset=t) for n, (i, t) in enumerate(runs))
    return ModelPlan(
        hidden_size=config.width, vocab_size=config.vocab, max_positions=MAX_POSITIONS,
        embedding_name="embed", layers=tuple(layers), schedule=schedule,
        final_norm=PartSpec("rms_norm", norm, names={"weight": "final.norm"}), head_name="head",
        stream_offsets=("loop.step", config.loop_times) if config.loops else None)


register_architecture("Kikalix", KikalixConfig, kikalix_plan, model_types=("kikalix",))
