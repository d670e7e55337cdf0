"""The Kikalix decoder without a GPU: configuration, plan, cache cells, and the plain implementation
against closed forms."""
import copy
import math

import pytest
import torch

import helpers
import plain_kikalix as P
from llama_rs_metal_b200.cache import Cache
from llama_rs_metal_b200.config.kikalix import KikalixConfig
from llama_rs_metal_b200.engine.model import DecoderModel
from llama_rs_metal_b200.errors import InvalidError, UnsupportedError
from llama_rs_metal_b200.parts.base import CompositeRequest, KeyValueRequest, StateRequest
from llama_rs_metal_b200.registry import find_architecture
from llama_rs_metal_b200.runtime import Runtime


def build(name):
    root = helpers.KIKALIX[name]["config"]
    arch = find_architecture(root)
    config = arch.config_class.from_dict(root)
    return config, arch.plan(config)


# --------------------------------------------------------------------------- configuration
@pytest.mark.parametrize("name", sorted(helpers.KIKALIX))
def test_configuration_reads_every_size_and_writes_it_back(name):
    config, _ = build(name)
    root = helpers.KIKALIX[name]["config"]
    assert config.vocab == root["vocab"] and config.width == root["width"] and config.eps == root["norm"]["eps"]
    assert [layer.kind for layer in config.layers] == [layer["type"] for layer in root["layers"]]
    assert KikalixConfig.from_dict(config.to_dict()) == config
    assert find_architecture({"architecture": "Kikalix"}).name == "Kikalix"


def test_configuration_names_what_is_missing_or_not_built():
    root = copy.deepcopy(helpers.KIKALIX["K1"]["config"])
    del root["layers"][0]["mixer"]["left"]["mask"]
    with pytest.raises(InvalidError, match=r"layers\[0\]\.mixer\.left\.mask"):
        KikalixConfig.from_dict(root)
    root = copy.deepcopy(helpers.KIKALIX["K1"]["config"])
    root["layers"][1]["mixer"]["decay"] = [0.9]
    with pytest.raises(InvalidError, match="decay"):
        KikalixConfig.from_dict(root)
    root = copy.deepcopy(helpers.KIKALIX["K1"]["config"])
    root["layers"][2]["type"] = "convolution"
    with pytest.raises(UnsupportedError, match="convolution"):
        KikalixConfig.from_dict(root)
    root = copy.deepcopy(helpers.KIKALIX["K1"]["config"])
    root["loop"] = dict(start=2, stop=1, times=2)
    with pytest.raises(InvalidError, match="loop"):
        KikalixConfig.from_dict(root)
    root = copy.deepcopy(helpers.KIKALIX["K1"]["config"])
    root["layers"][0]["mlp"]["router"]["top"] = 9
    with pytest.raises(InvalidError, match="top"):
        KikalixConfig.from_dict(root)


# --------------------------------------------------------------------------- plan
def test_looped_layers_run_in_order_with_a_cache_entry_per_run_and_an_offset_per_pass():
    _, plan = build("K1")                                  # three layers, layers 1 and 2 three times
    assert [e.layer for e in plan.schedule] == [0, 1, 2, 1, 2, 1, 2]
    assert [e.cache for e in plan.schedule] == list(range(7))
    assert [e.add_offset for e in plan.schedule] == [None, 0, None, 1, None, 2, None]
    assert plan.stream_offsets == ("loop.step", 3)
    assert [(i, t) for i, t in P.layer_runs(helpers.KIKALIX["K1"]["config"])] == \
        [(e.layer, e.add_offset) for e in plan.schedule]
    _, plan = build("K3")                                  # no loop: every layer once, no table
    assert [e.layer for e in plan.schedule] == [0, 1] and plan.stream_offsets is None
    assert [layer.block for layer in plan.layers] == ["pre_norm_mixer", "pre_norm_mixer"]


def test_tensor_names_and_shapes_follow_the_configuration():
    _, plan = build("K1")
    specs = DecoderModel(plan, Runtime(torch.device("cpu"), torch.float32)).tensor_specs()
    assert specs["embed"].shape == (211, 72) and specs["head"].shape == (211, 72)
    assert specs["loop.step"].shape == (3, 72) and specs["final.norm"].shape == (72,)
    assert specs["l0.mix.left.q"].shape == (4 * 16, 72) and specs["l0.mix.left.q.b"].shape == (64,)
    assert specs["l0.mix.left.v"].shape == (2 * 24, 72) and specs["l0.mix.left.o"].shape == (72, 4 * 24)
    assert specs["l0.mix.right.k.conv"].shape == (2 * 24, 3) and specs["l0.mix.right.v"].shape == (4 * 8, 72)
    assert specs["l0.mix.right.a1"].shape == (5, 72) and specs["l0.mix.right.a2"].shape == (4 * 24, 5)
    assert specs["l0.mix.right.g2"].shape == (4 * 8, 7) and specs["l0.mix.right.norm"].shape == (8,)
    assert specs["l0.mix.right.A_log"].shape == (4,) and specs["l0.mix.right.dt_bias"].shape == (96,)
    assert specs["l0.mlp.e4.down"].shape == (72, 40) and specs["l0.mlp.router.b"].shape == (5,)
    assert specs["l1.mix.g"].shape == (3 * 12, 72) and "l1.norm2" not in specs and "l1.mlp.router" not in specs
    # without the optional rank keys the ranks are the checkpoint's: any number fits
    root = copy.deepcopy(helpers.KIKALIX["K1"]["config"])
    for key in ("decay_rank", "gate_rank"):
        del root["layers"][0]["mixer"]["right"][key]
    arch = find_architecture(root)
    specs = DecoderModel(arch.plan(arch.config_class.from_dict(root)),
                         Runtime(torch.device("cpu"), torch.float32)).tensor_specs()
    assert specs["l0.mix.right.a1"].shape == (None, 72)
    assert specs["l0.mix.right.a1"].fits((24, 72)) and not specs["l0.mix.right.a1"].fits((24, 71))


def test_random_folder_is_read_back_by_the_plain_implementation(tmp_path):
    folder = helpers.make_kikalix_dir(str(tmp_path), "K3")
    config, tensors = P.read_model(folder)
    assert config["architecture"] == "Kikalix" and tensors["l0.mix.right.q.conv"].shape == (8, 1)
    logits = P.forward(config, tensors, [1, 2, 3])
    assert logits.shape == (3, 300) and bool(torch.isfinite(logits).all())


# --------------------------------------------------------------------------- cache cells
def test_a_mixer_that_keeps_several_things_gets_a_view_of_each():
    window = KeyValueRequest(2, 16, 7, 24)
    state, tail = StateRequest((4, 24, 8)), StateRequest((2, 80))
    both = CompositeRequest((window, CompositeRequest((state, tail))))
    cache = Cache([StateRequest((3, 20, 12)), both, both, None], torch.float32, torch.device("cpu"), 256, 3, 256)
    assert len(cache.kv_groups) == 1 and len(cache.state_groups) == 3
    kv, (s, t) = cache.view(1)
    assert kv.k.shape[1:] == (2, 64, 16) and kv.v.shape[1:] == (2, 64, 24) and kv.window == 7
    assert s.state.shape == (3, 4, 24, 8) and t.state.shape == (3, 2, 80)
    assert cache.view(2)[0].k.data_ptr() != kv.k.data_ptr()               # storage of its own per entry
    assert cache.view(2)[0].page_table.data_ptr() == kv.page_table.data_ptr()
    assert cache.view(0).state.shape == (3, 3, 20, 12) and cache.view(3) is None
    slot = cache.open_slot()
    s.state[slot] += 1.0
    t.state[slot] += 2.0
    cache.close_slot(slot)
    assert cache.open_slot() == slot                                       # the same slot again: from zero
    assert float(s.state[slot].abs().max()) == 0.0 and float(t.state[slot].abs().max()) == 0.0
    assert torch.equal(cache.snapshot(slot, (1, 1, 0)), torch.zeros(4, 24, 8))


# --------------------------------------------------------------------------- the plain implementation itself
def test_plain_retention_equals_its_closed_form():
    """o_t = sum_(s <= t) a^(t-s) (q_t . k_s) v_s before the read-out norm."""
    torch.manual_seed(0)
    T, H, d, dv, width = 9, 2, 4, 6, 10
    m = dict(heads=H, dim=d, vdim=dv, decay=[0.9, 0.5], rot=dict(dims=4, base=10.0))
    w = {n: torch.randn(s, dtype=torch.float64) for n, s in
         (("q", (H * d, width)), ("k", (H * d, width)), ("v", (H * dv, width)), ("g", (H * dv, width)),
          ("o", (width, H * dv)))}
    h = torch.randn(T, width, dtype=torch.float64)
    pos = torch.arange(T)
    q = P.rotate_half((h @ w["q"].T).reshape(T, H, d), pos, 4, 10.0)
    k = P.rotate_half((h @ w["k"].T).reshape(T, H, d), pos, 4, 10.0) * d ** -0.5
    v = (h @ w["v"].T).reshape(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=torch.float64)
    for t in range(T):
        for s in range(t + 1):
            for head in range(H):
                o[t, head] += m["decay"][head] ** (t - s) * (q[t, head] @ k[s, head]) * v[s, head]
    want = (P.unit_rms(o, 1e-6).reshape(T, -1) * P.silu(h @ w["g"].T)) @ w["o"].T
    assert torch.allclose(P.retention(h, w, "", m, 1e-6), want, atol=1e-10)
    # the rotation turns pairs (i, i + dims/2) and keeps lengths
    x = torch.randn(3, 1, 6, dtype=torch.float64)
    y = P.rotate_half(x, torch.tensor([0, 1, 5]), 4, 10.0)
    assert torch.equal(y[0], x[0]) and torch.equal(y[..., 4:], x[..., 4:])
    assert torch.allclose((y[..., :4] ** 2).sum(-1), (x[..., :4] ** 2).sum(-1))
    angle = 5 * 10.0 ** (-2.0 / 4)
    assert math.isclose(float(y[2, 0, 1]), float(x[2, 0, 1] * math.cos(angle) - x[2, 0, 3] * math.sin(angle)))


def test_plain_window_and_penalty_by_hand():
    """Zero queries: every visible key scores -slope (i - j), so the weights are known."""
    H, width, window = 2, 4, 3
    m = dict(heads=H, kv_heads=1, dim=2, vdim=1, scale=1.0, mask=dict(size=window))
    w = {"q": torch.zeros(H * 2, width, dtype=torch.float64), "q.b": torch.zeros(H * 2, dtype=torch.float64),
         "k": torch.zeros(2, width, dtype=torch.float64), "k.b": torch.zeros(2, dtype=torch.float64),
         "v": torch.zeros(1, width, dtype=torch.float64), "v.b": torch.zeros(1, dtype=torch.float64),
         "o": torch.eye(width, H, dtype=torch.float64)}
    w["v"][0, 0] = 1.0
    h = torch.zeros(6, width, dtype=torch.float64)
    h[:, 0] = torch.arange(6, dtype=torch.float64)          # v_j = j
    out = P.biased_window_attention(h, w, "", m)
    slopes = P.distance_slopes(H)
    assert slopes == [2.0 ** -4, 2.0 ** -8]
    for head in range(H):
        e = [math.exp(-slopes[head] * n) for n in range(window)]
        assert math.isclose(float(out[5, head]), (5 * e[0] + 4 * e[1] + 3 * e[2]) / sum(e))   # sees 3, 4, 5 only
        assert math.isclose(float(out[1, head]), (1 * e[0] + 0 * e[1]) / (e[0] + e[1]))         # the first tokens
        assert float(out[0, head]) == 0.0


def test_plain_delta_rule_stores_and_replaces_values():
    """With unit step size and no decay, writing v under a unit key and reading with the same key
    returns v; writing another value under the same key replaces it."""
    d, dv = 3, 2
    S = torch.zeros(d, dv, dtype=torch.float64)
    k = torch.tensor([0.0, 1.0, 0.0], dtype=torch.float64)
    for v in (torch.tensor([1.0, 2.0]), torch.tensor([-3.0, 5.0])):
        v = v.double()
        u = 1.0 * (v - S.T @ k)
        S = S + torch.outer(k, u)
        assert torch.allclose(S.T @ k, v)
    # the same through the mixer's function: one head, identity-like projections, conv of one tap
    width = d + dv
    w = {"q": torch.zeros(d, width), "k": torch.zeros(d, width), "v": torch.zeros(dv, width),
         "q.conv": torch.ones(d, 1), "k.conv": torch.ones(d, 1), "v.conv": torch.ones(dv, 1),
         "b": torch.zeros(1, width), "A_log": torch.zeros(1), "dt_bias": torch.full((d,), -50.0),
         "a1": torch.zeros(1, width), "a2": torch.zeros(d, 1), "g1": torch.zeros(1, width),
         "g2": torch.zeros(dv, 1), "norm": torch.ones(dv), "o": torch.eye(width, dv)}
    w = {n: t.double() for n, t in w.items()}
    w["q"][:, :d] = torch.eye(d, dtype=torch.float64)
    w["k"][:, :d] = torch.eye(d, dtype=torch.float64)
    w["v"][:, d:] = torch.eye(dv, dtype=torch.float64)
    h = torch.tensor([[0.0, 9.0, 0.0, 1.0, 2.0], [0.0, 9.0, 0.0, 1.0, 2.0]], dtype=torch.float64)
    m = dict(heads=1, kv_heads=1, dim=d, vdim=dv, conv=1)
    out = P.gated_delta_rule(h, w, "", m, 1e-6)
    # decay exp(-softplus(-50)) = 1, step size sigmoid(0) = 1/2: the second write adds half of what is missing
    assert torch.allclose(out[1, :dv] / out[0, :dv], torch.ones(dv, dtype=torch.float64))   # same direction after the norm
    assert bool(torch.isfinite(out).all())


def test_plain_experts_choose_the_largest_logits_and_weigh_by_their_softmax():
    width, ff, E = 3, 2, 4
    w = {"router": torch.zeros(E, width, dtype=torch.float64), "router.b": torch.tensor([0.0, 2.0, 1.0, -1.0]).double()}
    for e in range(E):
        w[f"e{e}.gate"] = torch.full((ff, width), 1.0 + e, dtype=torch.float64)
        w[f"e{e}.up"] = torch.zeros(ff, width, dtype=torch.float64)
        w[f"e{e}.down"] = torch.ones(width, ff, dtype=torch.float64)
    f = dict(router=dict(experts=E, top=2), expert=dict(limit=1.5))
    x = torch.tensor([[0.1, 0.0, 0.0]], dtype=torch.float64)
    out = P.mixture_of_experts(x, w, "", f)
    a = math.exp(2.0) / (math.exp(2.0) + math.exp(1.0))       # experts 1 and 2 win
    act = lambda g: min(g, 1.5) / (1 + math.exp(-1.702 * min(g, 1.5)))  # noqa: E731  (u = 0: y = g sigmoid(1.702 g))
    want = ff * (a * act(0.2) + (1 - a) * act(0.3))
    assert math.isclose(float(out[0, 0]), want, rel_tol=1e-12)
    big = P.clamped_expert(torch.tensor([100.0, 0.0, 0.0]).double(), w, "e0.", 1.5)          # the gate is capped
    assert math.isclose(float(big[0]), ff * 1.5 / (1 + math.exp(-1.702 * 1.5)))
