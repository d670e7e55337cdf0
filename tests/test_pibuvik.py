"""The Pibuvik decoder without a GPU: configuration, plan, tensor names, cache requests, and the
plain implementation's mechanisms against values worked out by hand."""
import math

import pytest
import torch

import helpers
import plain_pibuvik as P
from llama_rs_metal_b200.config.pibuvik import PibuvikConfig
from llama_rs_metal_b200.engine.model import DecoderModel
from llama_rs_metal_b200.errors import InvalidError, UnsupportedError
from llama_rs_metal_b200.parts.base import CompositeRequest, KeyValueRequest, StateRequest
from llama_rs_metal_b200.registry import find_architecture
from llama_rs_metal_b200.runtime import Runtime

F64 = torch.float64


def build(name):
    root = helpers.PIBUVIK[name]["config"]
    arch = find_architecture(root)
    config = arch.config_class.from_dict(root)
    return config, arch.plan(config)


@pytest.mark.parametrize("name", sorted(helpers.PIBUVIK))
def test_configuration_reads_every_size_and_writes_it_back(name):
    config, _ = build(name)
    again = PibuvikConfig.from_dict(config.to_dict())
    assert again == config
    assert len(config.layers) == len(helpers.PIBUVIK[name]["config"]["layers"])


def test_absent_scales_are_one_and_absent_options_are_off():
    config, plan = build("P3")
    assert (config.residual_mult, config.embedding_scale, config.logit_scale) == (1.0, 1.0, 1.0)
    assert plan.embedding_scale is None and plan.logit_scale is None
    assert config.layers[1].mixer.temp_every is None and config.layers[2].mixer.window is None
    assert plan.layers[1].mixer.params["query_temperature"] is None


def test_configuration_names_what_is_missing_or_not_built():
    root = helpers.PIBUVIK["P1"]["config"]

    def changed(path, value):
        import copy
        out = copy.deepcopy(root)
        at = out
        for key in path[:-1]:
            at = at[key]
        if value is None:
            del at[path[-1]]
        else:
            at[path[-1]] = value
        return out
    with pytest.raises(InvalidError, match="width"):
        PibuvikConfig.from_dict(changed(["width"], None))
    with pytest.raises(InvalidError, match="kv_rank"):
        PibuvikConfig.from_dict(changed(["layers", 0, "mixer", "kv_rank"], None))
    with pytest.raises(UnsupportedError, match="type"):
        PibuvikConfig.from_dict(changed(["layers", 1, "type"], "convolution"))
    with pytest.raises(UnsupportedError, match="dense"):
        PibuvikConfig.from_dict(changed(["layers", 0, "mlp", "kind"], "moe"))
    with pytest.raises(InvalidError, match="blocks"):
        PibuvikConfig.from_dict(changed(["layers", 2, "mixer", "blocks"], 5))
    with pytest.raises(InvalidError, match="kv_from"):
        PibuvikConfig.from_dict(changed(["layers", 3, "mixer", "kv_from"], 1))      # not a latent layer
    with pytest.raises(InvalidError, match="kv_from"):
        PibuvikConfig.from_dict(changed(["layers", 3, "mixer", "kv_rank"], 24))     # another latent width
    with pytest.raises(InvalidError, match="vdim"):
        PibuvikConfig.from_dict(changed(["layers", 1, "mixer", "vdim"], 16))        # values are the keys


def test_a_layer_that_reads_another_layers_latent_shares_its_cache_entry():
    config, plan = build("P1")
    model = DecoderModel(plan, Runtime(torch.device("cpu"), torch.float32))
    entries = [(e.layer, e.cache, e.writes_cache) for e in plan.schedule]
    assert entries == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 0, False), (4, 3, True)]
    requests = model.cache_requests()
    # the latent is kept for its widest reader (70), one key head of kv_rank + rot_dim, values inside
    assert requests[0] == KeyValueRequest(1, 26, 70, 20, values_in_keys=True)
    assert requests[1] == KeyValueRequest(2, 12, None, None, values_in_keys=True)
    assert requests[2] == CompositeRequest((StateRequest((48,), torch.float32), StateRequest((2, 48), torch.float32)))
    assert requests[3] == CompositeRequest((StateRequest((40,), torch.float32), StateRequest((0, 40), torch.float32)))
    # without a mask on one reader the latent is kept for good
    _, plan3 = build("P3")
    assert DecoderModel(plan3, Runtime(torch.device("cpu"), torch.float32)).cache_requests()[2].window is None


def test_tensor_names_and_shapes_follow_the_configuration():
    _, plan = build("P1")
    specs = DecoderModel(plan, Runtime(torch.device("cpu"), torch.float32)).tensor_specs()
    shapes = {n: tuple(s.shape) for n, s in specs.items()}
    assert shapes["embed"] == (211, 72) and shapes["final.norm"] == (72,) and "head" not in shapes
    assert shapes["l0.mix.dkv"] == (26, 72) and shapes["l0.mix.dkv.norm"] == (20,)
    assert shapes["l0.mix.uq"] == (3 * 18, 28) and shapes["l0.mix.uk"] == (36, 20) and shapes["l0.mix.uv"] == (30, 20)
    assert shapes["l0.mix.g"] == (3, 72) and shapes["l0.mix.o"] == (72, 30)
    assert "l3.mix.dkv" not in shapes and "l3.mix.dkv.norm" not in shapes and shapes["l3.mix.uk"] == (16, 20)
    assert shapes["l1.mix.q"] == (48, 72) and shapes["l1.mix.k"] == (24, 72) and shapes["l1.mix.sink"] == (4,)
    assert "l1.mix.v" not in shapes and "l1.mlp.gate" not in shapes and "l1.norm2" not in shapes
    assert shapes["l2.mix.ra"] == (3, 16, 16) and shapes["l2.mix.ri.b"] == (3, 16) and shapes["l2.mix.conv"] == (48, 3)
    assert shapes["l2.mix.lam"] == (48,) and shapes["l2.mlp.down"] == (72, 56)
    for i in range(5):
        assert shapes[f"l{i}.norm1"] == (72,) and shapes[f"l{i}.norm1b"] == (72,)
    assert shapes["l0.norm2b"] == (72,)


def test_random_folder_is_read_back_by_the_plain_implementation(tmp_path):
    folder = helpers.make_pibuvik_dir(str(tmp_path / "p1"), "P1")
    config, tensors = P.read_model(folder)
    assert config["layers"][3]["mixer"]["kv_from"] == 0
    logits = P.forward(config, tensors, [1, 2, 3, 4, 5])
    assert logits.shape == (5, 211) and torch.isfinite(logits).all()


# --------------------------------------------------------------------------- the plain mechanisms by hand
def test_plain_recurrence_equals_its_closed_form():
    """One channel, constant gates: S_t = sum_j a^(t-j) sqrt(1 - a^2) i u_j."""
    width = 1
    w = {"y": torch.zeros(1, 2, dtype=F64), "y.b": torch.tensor([1.3], dtype=F64),
         "x": torch.tensor([[1.0, 0.0]], dtype=F64), "x.b": torch.zeros(1, dtype=F64),
         "conv": torch.tensor([[0.0, 1.0]], dtype=F64), "conv.b": torch.zeros(1, dtype=F64),
         "ra": torch.zeros(1, 1, 1, dtype=F64), "ra.b": torch.tensor([[0.4]], dtype=F64),
         "ri": torch.zeros(1, 1, 1, dtype=F64), "ri.b": torch.tensor([[-0.2]], dtype=F64),
         "lam": torch.tensor([0.7], dtype=F64), "o": torch.ones(1, 1, dtype=F64)}
    u = torch.tensor([0.5, -1.0, 2.0, 0.25], dtype=F64)
    h = torch.stack([u, torch.zeros(4, dtype=F64)], dim=1)
    out = P.gated_linear_recurrence(h, w, "", dict(width=width, blocks=1, conv=2))
    r, i = 1 / (1 + math.exp(-0.4)), 1 / (1 + math.exp(0.2))
    a = math.exp(-8.0 * r * math.log1p(math.exp(0.7)))
    y = 0.5 * 1.3 * (1 + math.tanh(math.sqrt(2 / math.pi) * (1.3 + 0.044715 * 1.3 ** 3)))
    for t in range(4):
        want = sum(a ** (t - j) * math.sqrt(1 - a * a) * i * float(u[j]) for j in range(t + 1)) * y
        assert abs(float(out[t, 0]) - want) < 1e-12


def test_plain_convolution_starts_from_zeros_and_ends_on_the_current_token():
    x = torch.tensor([[1.0], [10.0], [100.0]], dtype=F64)
    taps = torch.tensor([[0.5, 2.0, 3.0]], dtype=F64)
    out = P.causal_conv(x, taps, torch.tensor([0.25], dtype=F64))
    assert out[:, 0].tolist() == [3.25, 32.25, 320.75]


def test_plain_sink_takes_its_share_and_the_temperature_grows_in_steps():
    """One head whose key is its value; a query that is zero makes every score 0, so the weights are
    1 / (t + 1 + e^sink) each; then a sharp query picks one key as the temperature rises."""
    d = 2
    w = {"q": torch.zeros(d, d, dtype=F64), "k": torch.eye(d, dtype=F64), "sink": torch.tensor([math.log(3.0)], dtype=F64),
         "o": torch.eye(d, dtype=F64)}
    h = torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]], dtype=F64)
    m = dict(heads=1, kv_heads=1, dim=d, vdim=d, scale=1.0)
    out = P.sink_attention(h, w, "", m)
    assert torch.allclose(out[0], h[0] / 4.0) and torch.allclose(out[2], h.sum(0) / 6.0)
    # temperature: factor 1 + coef ln(floor((t + 1) / every) + 1) is 1 for t + 1 < every
    w["q"] = torch.eye(d, dtype=F64)
    w["sink"] = torch.tensor([-50.0], dtype=F64)
    cold = P.sink_attention(h, w, "", m)
    hot = P.sink_attention(h, w, "", dict(m, q_temp=dict(coef=2.0, every=3)))
    assert torch.allclose(cold[:2], hot[:2])                      # positions 0 and 1: floor(./3) = 0
    factor = 1 + 2.0 * math.log(2.0)
    scores = (h @ h[2]) * factor
    assert torch.allclose(hot[2], torch.softmax(scores, 0) @ h)


def test_plain_latent_window_and_shared_rotated_key_by_hand():
    """kv_rank 1, one head, identity-like matrices: the score is q_plain * c + q_rot . k_rot, the
    window keeps `size` positions counting the query's own."""
    torch.manual_seed(0)
    T, width = 6, 4
    m = dict(heads=1, dim=1, rot_dim=2, vdim=1, kv_rank=1, q_rank=2, scale=1.0, rot=dict(dims=2, base=10.0),
             mask=dict(size=3))
    w = {k: torch.randn(*shape, dtype=F64) for k, shape in dict(
        dq=(2, width), uq=(3, 2), dkv=(3, width), uk=(1, 1), uv=(1, 1), g=(1, width), o=(width, 1)).items()}
    w["dq.norm"], w["dkv.norm"] = torch.ones(2, dtype=F64), torch.ones(1, dtype=F64)
    h = torch.randn(T, width, dtype=F64)
    kept = P.latent_keys(h, w, "", m, 1e-6)
    out = P.latent_attention(h, w, "", m, 1e-6, kept)
    c, shared = kept
    assert torch.allclose(c.abs(), torch.ones_like(c), atol=1e-5)   # a latent of one number is its sign
    t = 5
    cq = P.rms_norm(h[t] @ w["dq"].T, w["dq.norm"], 1e-6)
    q = cq @ w["uq"].T
    angle = float(t)                                               # pair 0 of 1: frequency base^0 = 1
    q_rot = torch.stack([q[1] * math.cos(angle) - q[2] * math.sin(angle), q[2] * math.cos(angle) + q[1] * math.sin(angle)])
    scores = torch.stack([q[0] * w["uk"][0, 0] * c[j, 0] + q_rot @ shared[j] for j in (3, 4, 5)])
    value = torch.softmax(scores, 0) @ (c[3:6, 0] * w["uv"][0, 0])
    want = value * torch.sigmoid(h[t] @ w["g"][0]) * w["o"][:, 0]
    assert torch.allclose(out[t], want, atol=1e-12)


def test_plain_feed_forward_clamps_the_gate_from_above_and_the_other_branch_on_both_sides():
    w = {"gate": torch.tensor([[1.0]], dtype=F64), "up": torch.tensor([[-3.0]], dtype=F64),
         "down": torch.tensor([[2.0]], dtype=F64)}
    out = P.clamped_gate_mlp(torch.tensor([[5.0], [-5.0]], dtype=F64), w, "", dict(limit=1.5))
    g0, g1 = 1.5, -5.0
    want0 = g0 / (1 + math.exp(-1.702 * g0)) * (-1.5 + 1.0) * 2.0
    want1 = g1 / (1 + math.exp(-1.702 * g1)) * (1.5 + 1.0) * 2.0
    assert abs(float(out[0, 0]) - want0) < 1e-12 and abs(float(out[1, 0]) - want1) < 1e-12
