"""The Pibuvik decoder through the engine, compared with the plain implementation (plain_pibuvik.py).

Model level, on three tiny configurations (helpers.PIBUVIK): whole prompts, the residual stream
layer by layer, prefill against token-by-token decoding, portions down to two tokens, batches of
unequal requests, slots that are freed and used again, long decoding through captured steps,
greedy generation through Session.generate, a replay through bin/trace_run, configurations drawn
at random. Mechanism level, with inputs made so that a fault shows: the recurrence and its
carried state, the convolution's tail, attention with sinks and the query temperature (a far key
that must win, a sink that must take its share), latent attention's window (keys just inside
and just outside it, at a page's border, in prompts, portions and decoding), the block products,
the norm behind a sublayer, the clamped gate.
"""
import math

import numpy as np
import pytest
import torch

import helpers
import plain_pibuvik as P

pytestmark = pytest.mark.gpu
DEV = "cuda"
NAMES = ["P1", "P2", "P3"]
F64 = torch.float64


@pytest.fixture(scope="module")
def engine():
    from llama_rs_metal_b200 import Engine
    return Engine()


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: helpers.make_pibuvik_dir(str(tmp_path_factory.mktemp(f"pibuvik_{n}")), n) for n in NAMES}


@pytest.fixture(scope="module")
def plain(folders):
    return {name: P.read_model(path) for name, path in folders.items()}


_REFS = {}


def reference(plain, name, tokens):
    key = (name, tuple(tokens))
    if key not in _REFS:
        config, tensors = plain[name]
        _REFS[key] = P.forward(config, tensors, tokens).numpy()
    return _REFS[key]


# Allowed error of a row of logits as a fraction of the largest reference logit. float32: sums in
# another order than the plain implementation's float64, and a recurrence that feeds back what it
# adds up. bfloat16: activations are rounded between kernels; a fault of any mechanism is far above.
TOLERANCE = {"float32": 5e-5, "bfloat16": 5e-2}


def close(got, ref, dtype, what, factor=1.0):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape and np.all(np.isfinite(got)), what
    err = np.abs(got - ref).max(axis=-1) / max(float(np.abs(ref).max()), 1e-30)
    worst = int(err.argmax())
    assert err[worst] <= factor * TOLERANCE[dtype], (
        f"{what}: row {worst} off by {err[worst]:.3e} of the largest logit (allowed {factor * TOLERANCE[dtype]:.0e}); "
        f"first such row {int(np.argmax(err > factor * TOLERANCE[dtype]))}; median {np.median(err):.3e}")


def vocab_of(name):
    return helpers.PIBUVIK[name]["config"]["vocab"]


def open_runner(engine, folder, dtype, max_tokens=2048, max_slots=8, use_graphs=True):
    from llama_rs_metal_b200.cache import Cache
    from llama_rs_metal_b200.engine.session import build_model
    from llama_rs_metal_b200.engine.step import StepRunner
    from llama_rs_metal_b200.runtime import Runtime, parse_dtype
    rt = Runtime(engine.device, parse_dtype(dtype))
    _, _, model, _ = build_model(folder, rt)
    cache = Cache(model.cache_requests(), rt.dtype, rt.device, max_tokens, max_slots, max_tokens)
    return StepRunner(model, cache, rt, use_graphs=use_graphs), cache, model


def entry(slot, tokens, want=None):
    from llama_rs_metal_b200.engine.batch import StepEntry
    return StepEntry(slot, tokens, range(len(tokens)) if want is None else want)


# --------------------------------------------------------------------------- whole prompts
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_match_the_plain_implementation(engine, folders, plain, name, dtype):
    runner, cache, _ = open_runner(engine, folders[name], dtype)
    for i, n in enumerate([150, 37, 1, 2]):       # the first tokens of a sequence are rows 0, 1, ...
        tokens = helpers.random_tokens(300 + i, n, vocab_of(name))
        slot = cache.open_slot()
        got = runner.step([entry(slot, tokens)]).cpu().numpy()
        cache.close_slot(slot)                     # the next prompt takes the same slot and state
        close(got, reference(plain, name, tokens), dtype, f"{name} prompt of {n}")
    runner.check_device_status()


@pytest.mark.parametrize("name", ["P1", "P2"])
def test_every_layer_matches_the_plain_residual_stream(engine, folders, plain, name):
    runner, cache, model = open_runner(engine, folders[name], "float32", use_graphs=False)
    seen = []
    for block in model.blocks:
        def wrapped(hidden, ctx, view, inner=block.forward):
            out = inner(hidden, ctx, view)
            seen.append(out.detach().clone().cpu().to(F64))
            return out
        block.forward = wrapped
    tokens = helpers.random_tokens(8, 90, vocab_of(name))
    slot = cache.open_slot()
    runner.step([entry(slot, tokens, [])])
    config, tensors = plain[name]
    streams = []
    P.forward(config, tensors, tokens, streams)
    assert len(seen) == len(streams)
    for i, (got, want) in enumerate(zip(seen, streams)):
        err = float((got[:len(tokens)] - want).abs().max() / want.abs().max())
        assert err < 2e-5, f"{name}: the stream after layer {i} is off by {err:.2e}"


# --------------------------------------------------------------------------- prefill against decoding
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_prefill_then_decoding_in_an_unequal_batch(engine, folders, plain, name, dtype):
    """Prompts of unequal lengths in one step, then one token each per step, past the windows and
    past a page's border; the shorter requests end earlier and the batch shrinks."""
    runner, cache, _ = open_runner(engine, folders[name], dtype)
    V = vocab_of(name)
    totals, prompts = [140, 75, 9, 58], [100, 60, 1, 2]
    seqs = [helpers.random_tokens(40 + i, n, V) for i, n in enumerate(totals)]
    refs = [reference(plain, name, s) for s in seqs]
    slots = [cache.open_slot() for _ in seqs]
    out = runner.step([entry(sl, s[:n]) for sl, s, n in zip(slots, seqs, prompts)]).cpu().numpy()
    row = 0
    for b, n in enumerate(prompts):
        close(out[row:row + n], refs[b][:n], dtype, f"{name} prompt {b} in the batch")
        row += n
    at = list(prompts)
    while any(a < t for a, t in zip(at, totals)):
        live = [b for b in range(len(seqs)) if at[b] < totals[b]]
        out = runner.step([entry(slots[b], [seqs[b][at[b]]]) for b in live]).cpu().numpy()
        for i, b in enumerate(live):
            close(out[i:i + 1], refs[b][at[b]][None], dtype, f"{name} sequence {b}, position {at[b]}")
            at[b] += 1
            if at[b] == totals[b]:
                cache.close_slot(slots[b])
    runner.check_device_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P1", "P2"])
def test_a_prompt_geometry_that_comes_again_is_captured_and_replayed(engine, folders, plain, name, dtype):
    """Short prompt batches are filled up to whole rows, and a geometry seen before runs as a
    captured graph: the same shape of batch four times with other tokens, in slots that were used
    before (state and tails must start from zero each time, also under replay)."""
    runner, cache, _ = open_runner(engine, folders[name], dtype)
    V = vocab_of(name)
    for round_ in range(4):
        seqs = [helpers.random_tokens(500 + 10 * round_ + i, n, V) for i, n in enumerate([70, 3, 41])]
        slots = [cache.open_slot() for _ in seqs]
        out = runner.step([entry(sl, s) for sl, s in zip(slots, seqs)]).cpu().numpy()
        row = 0
        for s in seqs:
            close(out[row:row + len(s)], reference(plain, name, s), dtype, f"{name} round {round_}")
            row += len(s)
        nxt = [int(t) for t in helpers.random_tokens(900 + round_, len(seqs), V)]
        out = runner.step([entry(sl, [t]) for sl, t in zip(slots, nxt)]).cpu().numpy()
        for i, (s, t) in enumerate(zip(seqs, nxt)):
            close(out[i:i + 1], reference(plain, name, s + [t])[-1:], dtype, f"{name} round {round_}, next token")
        for sl in slots:
            cache.close_slot(sl)
    runner.check_device_status()


@pytest.mark.parametrize("sizes", [[2], [3, 64, 5], [1, 70, 2], [64], [17]])
@pytest.mark.parametrize("name", ["P1", "P2"])
def test_portions_of_any_size_give_the_whole_prompt(engine, folders, plain, name, sizes):
    for dtype in ("float32", "bfloat16"):
        runner, cache, _ = open_runner(engine, folders[name], dtype)
        tokens = helpers.random_tokens(77, 150 if sizes != [2] else 40, vocab_of(name))
        ref = reference(plain, name, tokens)
        slot, at, i, rows = cache.open_slot(), 0, 0, []
        while at < len(tokens):
            n = min(sizes[min(i, len(sizes) - 1)], len(tokens) - at)
            rows.append(runner.step([entry(slot, tokens[at:at + n])]).cpu().numpy())
            at, i = at + n, i + 1
        close(np.concatenate(rows), ref, dtype, f"{name} in portions of {sizes}")
        cache.close_slot(slot)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_company_in_the_batch_changes_nothing_beyond_rounding(engine, folders, plain, dtype):
    name = "P2"
    runner, cache, _ = open_runner(engine, folders[name], dtype)
    V = vocab_of(name)
    mine = helpers.random_tokens(5, 130, V)
    others = [helpers.random_tokens(6 + i, n, V) for i, n in enumerate([200, 3, 64])]
    slot = cache.open_slot()
    alone = runner.step([entry(slot, mine)]).cpu().numpy()
    cache.close_slot(slot)
    slots = [cache.open_slot() for _ in range(4)]
    together = runner.step([entry(slots[0], others[0], []), entry(slots[1], mine), entry(slots[2], others[1], []),
                            entry(slots[3], others[2], [])]).cpu().numpy()
    limit = 0.0 if dtype == "float32" else 2e-2
    assert np.abs(alone - together).max() <= limit * np.abs(alone).max() + (1e-5 if dtype == "float32" else 0)
    close(together, reference(plain, name, mine), dtype, "in company")


def test_a_freed_slot_and_its_pages_start_from_nothing(engine, folders, plain):
    """The state and the convolution's tail of a slot are cleared when it is taken again, and
    the pages a sequence gave back hold another sequence's keys when they are used again."""
    name = "P1"
    for dtype in ("float32", "bfloat16"):
        runner, cache, _ = open_runner(engine, folders[name], dtype, max_tokens=512, max_slots=2)
        V = vocab_of(name)
        first = helpers.random_tokens(1, 200, V)
        slot = cache.open_slot()
        runner.step([entry(slot, first, [])])
        for t in helpers.random_tokens(2, 5, V):
            runner.step([entry(slot, [t], [])])
        cache.close_slot(slot)
        second = helpers.random_tokens(3, 90, V)
        again = cache.open_slot()
        assert again == slot
        got = [runner.step([entry(again, second[:50])]).cpu().numpy()]
        for t in second[50:]:
            got.append(runner.step([entry(again, [t])]).cpu().numpy())
        close(np.concatenate(got), reference(plain, name, second), dtype, "the slot's second sequence")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_captured_steps(engine, folders, plain, dtype):
    """300 tokens one by one from the very first: every window and several pages pass by, the
    recurrence's state is carried through hundreds of captured steps."""
    name = "P1"
    runner, cache, _ = open_runner(engine, folders[name], dtype)
    tokens = helpers.random_tokens(9, 300, vocab_of(name))
    ref = reference(plain, name, tokens)
    slot = cache.open_slot()
    rows = [runner.step([entry(slot, [t])]).cpu().numpy() for t in tokens]
    close(np.concatenate(rows), ref, dtype, "token by token from the start", factor=2.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_session(engine, folders, plain, dtype):
    from llama_rs_metal_b200 import GenerationOptions, Sampling
    name = "P2"
    model = engine.load(folders[name], dtype=dtype)
    session = model.session(context=256, max_batch=4)
    V = vocab_of(name)
    prompts = [helpers.random_tokens(60 + i, n, V) for i, n in enumerate([70, 5, 33])]
    results = session.generate(prompts, GenerationOptions(max_tokens=12, sampling=Sampling(temperature=0.0)))
    config, tensors = plain[name]
    for prompt, result in zip(prompts, results):
        tokens = list(prompt)
        assert len(result.tokens) == 12
        for chosen in result.tokens:
            logits = P.forward(config, tensors, tokens)[-1].numpy()
            best = int(logits.argmax())
            if chosen != best:   # a near tie may fall the other way under rounding
                gap = (logits[best] - logits[chosen]) / np.abs(logits).max()
                assert gap < (1e-4 if dtype == "float32" else 5e-2), f"chose {chosen}, the plain model {best} by {gap:.2e}"
            tokens.append(chosen)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_through_the_trace_runner(folders, plain, dtype, tmp_path):
    name = "P1"
    V = vocab_of(name)
    requests = {f"r{i}": helpers.random_tokens(90 + i, n, V) for i, n in enumerate([120, 40, 77])}
    trace = helpers.Trace()
    trace.whole("whole:r0", requests["r0"])
    trace.tail_one_by_one("tail:r1", requests["r1"], tail=20)
    trace.batch({f"batch:{n}": t for n, t in requests.items()}, {"batch:r0": 90, "batch:r1": 10, "batch:r2": 70})
    outputs = helpers.run_trace(folders[name], dtype, trace, 1024, str(tmp_path / "out"))
    refs = {n: reference(plain, name, t) for n, t in requests.items()}
    for step in sorted(trace.rows):
        rows = trace.rows[step]
        ref = np.stack([refs[rid.split(":")[-1]][pos] for rid, pos in rows])
        close(outputs[step], ref, dtype, f"step {step}")


# --------------------------------------------------------------------------- configurations drawn at random
def drawn_configuration(seed):
    rng = np.random.default_rng(seed)

    def pick(*values):
        return values[int(rng.integers(len(values)))]
    width = int(pick(40, 64, 88, 136))
    layers, latents = [], []
    for i in range(int(rng.integers(2, 6))):
        kind = pick("rglru", "attention", "latent_attention")
        if kind == "rglru":
            blocks = int(pick(1, 2, 4))
            mixer = dict(width=blocks * int(pick(8, 12, 20)), blocks=blocks, conv=int(pick(1, 2, 4, 5)))
        elif kind == "attention":
            kv = int(pick(1, 2, 3))
            mixer = dict(heads=kv * int(pick(1, 2, 4)), kv_heads=kv, dim=int(pick(8, 20, 32, 64)), scale=float(pick(0.1, 0.3)))
            mixer["vdim"] = mixer["dim"]
            if rng.integers(2):
                mixer["q_temp"] = dict(coef=float(pick(0.1, 0.7)), every=int(pick(1, 7, 64)))
        else:
            source = latents[int(rng.integers(len(latents)))] if latents and rng.integers(2) else None
            if source is None:
                kv_rank, rot_dim, base = int(pick(8, 24, 40)), int(pick(2, 8, 16)), float(pick(30.0, 10000.0))
                latents.append((i, kv_rank, rot_dim, base))
            else:
                _, kv_rank, rot_dim, base = source
            mixer = helpers._latent(int(pick(1, 2, 5)), int(pick(4, 16, 24)), rot_dim, int(pick(8, 12, 32)), kv_rank,
                                    int(pick(8, 24)), float(pick(0.1, 0.4)), base, window=int(pick(1, 2, 33, 64, 65, 200)),
                                    kv_from=source[0] if source is not None else None)
        mlp = helpers._dense(int(pick(24, 64, 100)), float(pick(0.5, 3.0))) if rng.integers(3) else None
        layers.append(dict(type=kind, mixer=mixer, mlp=mlp))
    config = dict(architecture="Pibuvik", vocab=int(pick(97, 256, 333)), width=width, norm=dict(eps=float(pick(1e-6, 1e-4))),
                  residual_mult=float(pick(0.3, 1.0, 1.4)), embedding=dict(scale=float(pick(0.5, 1.0, 3.0))),
                  logit_scale=float(pick(0.2, 1.0)), layers=layers)
    return dict(config=config, seed=1000 + seed, std=float(pick(0.08, 0.15)))


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(engine, tmp_path, seed):
    """Other sizes, orders of layers and constants than the fixed configurations: a prompt whole,
    then tokens one by one, a second sequence beside it in portions."""
    spec = drawn_configuration(seed)
    folder = helpers.make_pibuvik_dir(str(tmp_path / "drawn"), spec)
    config, tensors = P.read_model(folder)
    V = config["vocab"]
    a, b = helpers.random_tokens(seed, 150, V), helpers.random_tokens(seed + 50, 100, V)
    ref_a, ref_b = P.forward(config, tensors, a).numpy(), P.forward(config, tensors, b).numpy()
    for dtype in ("float32", "bfloat16"):
        runner, cache, _ = open_runner(engine, folder, dtype)
        sa, sb = cache.open_slot(), cache.open_slot()
        out = runner.step([entry(sa, a[:120]), entry(sb, b[:3])]).cpu().numpy()
        close(out[:120], ref_a[:120], dtype, f"seed {seed}: prompt a", factor=2.0)
        close(out[120:], ref_b[:3], dtype, f"seed {seed}: prompt b", factor=2.0)
        out = runner.step([entry(sa, a[120:121]), entry(sb, b[3:70])]).cpu().numpy()     # one token and a portion
        close(out[:1], ref_a[120:121], dtype, f"seed {seed}: a's next token", factor=2.0)
        close(out[1:], ref_b[3:70], dtype, f"seed {seed}: b's portion", factor=2.0)
        for t in range(121, 150):
            entries = [entry(sa, [a[t]])] + ([entry(sb, [b[t - 51]])] if t - 51 < 100 else [])
            out = runner.step(entries).cpu().numpy()
            close(out[:1], ref_a[t:t + 1], dtype, f"seed {seed}: a at {t}", factor=2.0)
            if len(entries) > 1:
                close(out[1:], ref_b[t - 51:t - 50], dtype, f"seed {seed}: b at {t - 51}", factor=2.0)
        runner.check_device_status()


# --------------------------------------------------------------------------- mechanisms
def _ints(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def step_arrays(lengths):
    """cu_seqlens, seq_of_token, positions-from-zero for packed sequences of these lengths."""
    cu = np.concatenate([[0], np.cumsum(lengths)])
    seq = np.concatenate([np.full(n, b) for b, n in enumerate(lengths)])
    return _ints(cu), _ints(seq)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("C,blocks,lengths", [(48, 3, [5, 1, 130]), (256, 4, [300]), (20, 1, [64, 65])])
def test_recurrence_matches_its_definition_and_carries_its_state(dtype, C, blocks, lengths):
    """Whole sequences (the serial and the chunked kernel), then the same sequences cut in two
    steps through the carried state, in slots that are not in order."""
    from llama_rs_metal_b200.kernels import ops
    gen = torch.Generator().manual_seed(C)
    T = sum(lengths)
    u = (torch.randn(T, C, generator=gen)).to(dtype)
    gates = torch.randn(T, 2 * C, generator=gen) * 2
    y = torch.randn(T, C + 3, generator=gen)
    y_bias, lam = torch.randn(C, generator=gen), torch.randn(C, generator=gen) * 2 - 3
    rate = 8.0 * torch.nn.functional.softplus(lam)
    size = C // blocks
    g = gates.view(T, blocks, 2, size).to(F64)
    r, i = torch.sigmoid(g[:, :, 0]).reshape(T, C), torch.sigmoid(g[:, :, 1]).reshape(T, C)
    a = torch.exp(-rate.to(F64) * r)
    want = torch.zeros(T, C, dtype=F64)
    at = 0
    for n in lengths:
        s = torch.zeros(C, dtype=F64)
        for t in range(at, at + n):
            s = a[t] * s + torch.sqrt(1 - a[t] ** 2) * (i[t] * u[t].to(F64))
            want[t] = s * P.gelu_tanh(y[t, 3:].to(F64) + y_bias.to(F64))
        at += n
    slots = [3, 0, 5][:len(lengths)]
    dev = lambda t: t.to(DEV).contiguous()
    tol = 1e-5 if dtype == torch.float32 else 1e-2

    def run(state, cuts):
        cu, _ = step_arrays(cuts)
        return ops.gated_linear_scan(dev(u_part), dev(g_part), dev(y_part), 3, dev(y_bias), dev(rate), state, cu,
                                     _ints(slots), max(cuts), blocks).float().cpu()
    state = torch.zeros(8, C, device=DEV)
    u_part, g_part, y_part = u, gates, y
    got = run(state, lengths)
    assert (got.to(F64) - want).abs().max() <= tol * want.abs().max(), "whole sequences"
    # the same in two steps: the first half of every sequence, then the rest
    state2 = torch.zeros(8, C, device=DEV)
    firsts = [max(1, n // 2) for n in lengths]
    starts = np.concatenate([[0], np.cumsum(lengths)])[:-1]
    rows1 = np.concatenate([np.arange(s, s + f) for s, f in zip(starts, firsts)])
    rows2 = np.concatenate([np.arange(s + f, s + n) for s, f, n in zip(starts, firsts, lengths)])
    u_part, g_part, y_part = u[rows1], gates[rows1], y[rows1]
    got1 = run(state2, firsts)
    rest = [n - f for n, f in zip(lengths, firsts)]
    keep = [b for b, n in enumerate(rest) if n > 0]
    u_part, g_part, y_part = u[rows2], gates[rows2], y[rows2]
    slots_all, slots = slots, [slots[b] for b in keep]
    got2 = run(state2, [rest[b] for b in keep])
    slots = slots_all
    assert (got1.to(F64) - want[rows1]).abs().max() <= tol * want.abs().max()
    assert (got2.to(F64) - want[rows2]).abs().max() <= tol * want.abs().max(), "the second step starts from the carried state"
    assert (state2[slots_all] - state[slots_all]).abs().max() <= 1e-5 * max(1.0, float(state.abs().max()))
    untouched = [s for s in range(8) if s not in slots_all]
    assert float(state[untouched].abs().max()) == 0.0


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_convolution_tail_makes_portions_equal_to_the_whole(taps):
    from llama_rs_metal_b200.kernels import ops
    gen = torch.Generator().manual_seed(taps)
    C, lengths = 24, [9, 1, 30]
    T = sum(lengths)
    src = torch.randn(T, C + 5, generator=gen)
    in_bias, conv_bias, w = torch.randn(C, generator=gen), torch.randn(C, generator=gen), torch.randn(C, taps, generator=gen)
    want = torch.zeros(T, C, dtype=F64)
    at = 0
    for n in lengths:
        x = src[at:at + n, 5:].to(F64) + in_bias.to(F64)
        want[at:at + n] = P.causal_conv(x, w.to(F64), conv_bias.to(F64))
        at += n
    slots = _ints([2, 0, 1])
    dev = lambda t: t.to(DEV).contiguous()

    def run(rows, cuts, tails):
        cu, seq = step_arrays(cuts)
        return ops.short_conv(dev(src[rows]), 5, C, dev(in_bias), dev(w), dev(conv_bias), tails, cu, seq, slots,
                              torch.float32).cpu()
    tails = torch.zeros(3, taps - 1, C, device=DEV)
    got = run(np.arange(T), lengths, tails)
    assert (got.to(F64) - want).abs().max() < 1e-5
    starts = np.concatenate([[0], np.cumsum(lengths)])[:-1]
    tails = torch.zeros(3, taps - 1, C, device=DEV)
    done = [0, 0, 0]
    out = torch.zeros(T, C)
    for cut in ([2, 1, 1], [1, 0, 2], [3, 0, 20], [3, 0, 7]):      # portions shorter and longer than the tail
        live = [b for b in range(3) if cut[b] > 0]
        rows = np.concatenate([np.arange(starts[b] + done[b], starts[b] + done[b] + cut[b]) for b in live])
        cu, seq = step_arrays([cut[b] for b in live])
        got = ops.short_conv(dev(src[rows]), 5, C, dev(in_bias), dev(w), dev(conv_bias), tails, cu, seq,
                             _ints([[2, 0, 1][b] for b in live]), torch.float32).cpu()
        out[rows] = got
        for b in live:
            done[b] += cut[b]
    assert done == lengths
    assert (out.to(F64) - want).abs().max() < 1e-5, "portions through the tail"


def plain_attention(q, k, v, scale, window, sinks, temperature, first_query=0):
    """q [n, H, d] are the queries of positions first_query .. over keys k [T, G, d], values v [T, G, dv]."""
    n, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(n, H, v.shape[2], dtype=F64)
    for i in range(n):
        pos = first_query + i
        lo = max(0, pos - window + 1) if window else 0
        factor = 1.0
        if temperature is not None:
            factor = 1.0 + temperature[0] * math.log((pos + 1) // temperature[1] + 1)
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:pos + 1, g] @ q[i, h]) * scale * factor
            top = s.max() if sinks is None else torch.maximum(s.max(), sinks[h])
            e = torch.exp(s - top)
            denom = e.sum() + (torch.exp(sinks[h] - top) if sinks is not None else 0.0)
            out[i, h] = (e[:, None] * v[lo:pos + 1, g]).sum(0) / denom
    return out


class PagedKeys:
    """A cache view over pages handed out in a scrambled order, filled by hand."""

    def __init__(self, rows, kv_heads, value_dim, window, dtype, seed=0, values_in_keys=True):
        from llama_rs_metal_b200.cache.cache import KeyValueView
        T, width = rows.shape[0], rows.shape[-1]
        pages = -(-T // 64) + 3
        order = np.random.default_rng(seed).permutation(pages)
        self.k = torch.zeros(pages, kv_heads, 64, width // kv_heads if rows.dim() == 2 else width, dtype=dtype, device=DEV)
        table = torch.full((2, pages), -1, dtype=torch.int32)
        data = rows.reshape(T, kv_heads, -1).to(dtype)
        for p in range(-(-T // 64)):
            table[1, p] = int(order[p])
            chunk = data[64 * p:64 * p + 64]
            self.k[int(order[p]), :, :chunk.shape[0]] = chunk.transpose(0, 1).to(DEV)
        self.view = KeyValueView(self.k, self.k, table.to(DEV), 64, kv_heads, self.k.shape[3], window, 0, value_dim,
                                 values_in_keys)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d", [(4, 2, 12), (8, 2, 64), (3, 3, 32), (2, 1, 128)])
def test_sinks_temperature_and_a_far_key(dtype, H, G, d):
    """Values are the keys. Prompts, portions and decoding against the definition. One key, hundreds
    of positions back and not at a page's start, points along every query and is longer than the
    rest: it must hold most of the weight however far the query is. The sinks differ per head and
    one of them is large enough to take most of a head's weight."""
    from llama_rs_metal_b200.kernels import ops
    from llama_rs_metal_b200.kernels.attention_dispatch import Extras
    gen = torch.Generator().manual_seed(H * d)
    T, far = 700, 67
    q = torch.randn(T, H, d, generator=gen)
    k = torch.randn(T, G, d, generator=gen) * 0.3
    direction = torch.randn(d, generator=gen)
    direction /= direction.norm()
    q[600:] = q[600:] * 0.3 + 6.0 * direction             # late queries look for the far key
    k[far] = 4.0 * direction
    q, k = q.to(dtype), k.to(dtype)
    sinks = torch.linspace(-2.0, 1.0, H)
    sinks[0] = 25.0                                        # about the far key's score: it takes half of head 0
    temperature, scale = (0.4, 50), 0.5
    want = plain_attention(q.to(F64), k.to(F64), k.to(F64), scale, None, sinks.to(F64), temperature)
    plain_weight = plain_attention(q[650:651].to(F64), k.to(F64), torch.eye(T, dtype=F64)[:, None, :].expand(T, G, T),
                                   scale, None, sinks.to(F64), temperature, first_query=650)
    assert float(plain_weight[0, 1, far]) > 0.5 and float(plain_weight[0, 0].sum()) < 0.9   # the test shows what it claims
    extras = Extras(sinks.to(DEV), temperature)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    cu, seq = step_arrays([T])
    got = ops.attention_prefill(q.to(DEV), k.to(DEV), None, cu, seq, T, scale, None, extras=extras).float().cpu()
    assert (got.view(T, H, d).to(F64) - want).abs().max() <= tol * want.abs().max(), "prompt"
    paged = PagedKeys(k.reshape(T, G * d), G, d, None, dtype, seed=d)
    for pos in (far, 599, 650, T - 1):                                            # decoding at these positions
        got = ops.attention_decode(q[pos:pos + 1].to(DEV), paged.view, _ints([1]), _ints([pos + 1]), pos + 1, scale,
                                   None, extras=extras).float().cpu()
        assert (got.view(H, d).to(F64) - want[pos]).abs().max() <= tol * want.abs().max(), f"decoding at {pos}"
    lo, hi = 590, 690                                                            # a portion onto a started sequence
    cu, seq = step_arrays([hi - lo])
    got = ops.attention_extend(q[lo:hi].to(DEV), paged.view, cu, seq, _ints(list(range(lo, hi))), _ints([1]),
                               _ints([hi]), hi - lo, scale, None, extras=extras).float().cpu()
    assert (got.view(hi - lo, H, d).to(F64) - want[lo:hi]).abs().max() <= tol * want.abs().max(), "portion"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,width,dv,window", [(3, 26, 20, 7), (4, 128, 96, 64), (2, 40, 24, 65), (1, 24, 16, 1),
                                               (6, 96, 64, 65), (16, 288, 256, 100), (20, 64, 48, 33), (2, 544, 512, 130)])
def test_window_edges_over_keys_that_hold_their_values(dtype, H, width, dv, window):
    """One key head whose rows' first dv columns are the values (latent attention's cache). For
    chosen queries the key just inside the window and the key just outside it are both made to
    stand out; only the first may be seen. In prompts, portions and decoding, with windows that
    end inside a page, at its border, and one key wide."""
    from llama_rs_metal_b200.kernels import ops
    gen = torch.Generator().manual_seed(width + window)
    T = 200
    q = torch.randn(T, H, width, generator=gen) * 0.5
    rows = torch.randn(T, width, generator=gen) * 0.5
    direction = torch.randn(width, generator=gen)
    direction /= direction.norm()
    probes = [window - 1, window, 63, 64, 127, 128, 150, T - 1]
    probes = [p for p in probes if p - window >= 0]
    for p in probes:
        q[p] = 5.0 * direction
    scale = 1.0
    for p in probes:                                 # just inside: p - window + 1; just outside: p - window
        rows[p - window] = 6.0 * direction
        if window > 1:
            rows[p - window + 1] = 3.0 * direction
    q, rows = q.to(dtype), rows.to(dtype)
    keys = rows.to(F64).view(T, 1, width)
    want = plain_attention(q.to(F64), keys, keys[:, :, :dv], scale, window, None, None)
    unmasked = plain_attention(q[probes[-1]:probes[-1] + 1].to(F64), keys, keys[:, :, :dv], scale, window + 1, None, None,
                               first_query=probes[-1])
    assert (unmasked[0] - want[probes[-1]]).abs().max() > 0.1 * want.abs().max()      # one key more would show
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    cu, seq = step_arrays([T])
    got = ops.attention_prefill(q.to(DEV), rows.view(T, 1, width).to(DEV), None, cu, seq, T, scale, window,
                                value_dim=dv).float().cpu()
    assert (got.view(T, H, dv).to(F64) - want).abs().max() <= tol * want.abs().max(), "prompt"
    paged = PagedKeys(rows, 1, dv, window, dtype, seed=window)
    from llama_rs_metal_b200.kernels import attention_dispatch
    for splits in (None, 1, 3, 7):      # the keys of a decode step whole, and cut into more splits than tiles
        attention_dispatch.force_shared_key_splits = splits
        try:
            for pos in probes:
                got = ops.attention_decode(q[pos:pos + 1].to(DEV), paged.view, _ints([1]), _ints([pos + 1]), pos + 1,
                                           scale, window).float().cpu()
                assert (got.view(H, dv).to(F64) - want[pos]).abs().max() <= tol * want.abs().max(), \
                    f"decoding at {pos} in {splits} splits"
        finally:
            attention_dispatch.force_shared_key_splits = None
    lo = 60
    cu, seq = step_arrays([T - lo])
    got = ops.attention_extend(q[lo:].to(DEV), paged.view, cu, seq, _ints(list(range(lo, T))), _ints([1]), _ints([T]),
                               T - lo, scale, window).float().cpu()
    assert (got.view(T - lo, H, dv).to(F64) - want[lo:]).abs().max() <= tol * want.abs().max(), "portion"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,B,n,m,lead,gap", [(70, 3, 37, 21, 5, 4), (150, 5, 100, 48, 8, 8), (9, 2, 64, 160, 0, 0)])
def test_block_products_with_strides_bias_and_row_scale(dtype, T, B, n, m, lead, gap):
    """Blocks inside wider rows on both sides; the second and third shapes start every block on a
    16-byte boundary, which in bfloat16 is the tensor-core kernel's case."""
    from llama_rs_metal_b200.kernels import ops
    gen = torch.Generator().manual_seed(4 + m)
    x = torch.randn(T, lead + B * (m + gap), generator=gen).to(dtype)
    w = torch.randn(B, n, m, generator=gen).to(dtype)
    bias, scale = torch.randn(B, n, generator=gen), torch.rand(T, B, generator=gen)
    blocks = torch.stack([x[:, lead + b * (m + gap):lead + b * (m + gap) + m] for b in range(B)], dim=1).to(F64)
    want = (torch.einsum("tbi,boi->tbo", blocks, w.to(F64)) + bias.to(F64)) * scale.to(F64)[:, :, None]
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for out_dtype in (torch.float32, dtype):
        out = torch.full((T, 2 + B * (n + 1)), 7.0, dtype=out_dtype, device=DEV)
        ops.blockwise_linear(x.to(DEV), w.to(DEV), bias=bias.to(DEV), row_scale=scale.to(DEV), x_column=lead,
                             x_block=m + gap, out=out, out_column=2, out_block=n + 1)
        got = torch.stack([out[:, 2 + b * (n + 1):2 + b * (n + 1) + n] for b in range(B)], dim=1).cpu().to(F64)
        assert (got - want).abs().max() <= tol * want.abs().max()
        assert float(out[:, :2].min()) == 7.0 and float(out[:, 2 + n].min()) == 7.0          # nothing beside the blocks
    first = x[:, lead:lead + m].contiguous()
    plain = ops.blockwise_linear(first.to(DEV), w[:1].contiguous().to(DEV)).float().cpu()
    assert (plain.to(F64) - blocks[:, 0] @ w[0].to(F64).T).abs().max() <= (1e-5 if dtype == torch.float32 else 2e-2) * want.abs().max()


def test_latent_rows_norms_rotation_and_gates():
    from llama_rs_metal_b200.kernels import ops
    gen = torch.Generator().manual_seed(11)
    T, q_rank, kv_rank, rot, H = 9, 28, 20, 6, 3
    proj = torch.randn(T, q_rank + kv_rank + rot + H, generator=gen)
    wq, wc = torch.rand(q_rank, generator=gen) + 0.5, torch.rand(kv_rank, generator=gen) + 0.5
    positions = [0, 1, 2, 70, 71, 500, 3, 4, 5]
    inv_freq = torch.tensor([100.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=F64).float()
    cq, rows, gate = ops.latent_prepare(proj.to(DEV), 0, wq.to(DEV), q_rank, wc.to(DEV), rot, _ints(positions),
                                        inv_freq.to(DEV), 1e-6, q_rank + kv_rank + rot, H, torch.float32)
    p64 = proj.to(F64)
    assert (cq.cpu().to(F64) - P.rms_norm(p64[:, :q_rank], wq.to(F64), 1e-6)).abs().max() < 1e-5
    assert (rows[:, :kv_rank].cpu().to(F64) - P.rms_norm(p64[:, q_rank:q_rank + kv_rank], wc.to(F64), 1e-6)).abs().max() < 1e-5
    rotated = P.rotate_half(p64[:, q_rank + kv_rank:q_rank + kv_rank + rot], torch.tensor(positions), rot, 100.0)
    assert (rows[:, kv_rank:].cpu().to(F64) - rotated).abs().max() < 2e-4
    assert (gate.cpu().to(F64) - torch.sigmoid(p64[:, -H:])).abs().max() < 1e-6
    # the same rotation for every head of a query
    src = torch.randn(T, 2 * (4 + rot), generator=gen)
    dst = torch.zeros(T, 2 * (kv_rank + rot), device=DEV)
    ops.rope_heads(src.to(DEV), 4, 4 + rot, dst, kv_rank, kv_rank + rot, _ints(positions), inv_freq.to(DEV), 2)
    for h in range(2):
        want = P.rotate_half(src[:, h * (4 + rot) + 4:(h + 1) * (4 + rot)].to(F64), torch.tensor(positions), rot, 100.0)
        got = dst[:, h * (kv_rank + rot) + kv_rank:(h + 1) * (kv_rank + rot)].cpu().to(F64)
        assert (got - want).abs().max() < 2e-4


@pytest.mark.parametrize("width", [72, 320, 2304])
def test_norm_behind_a_sublayer_and_the_norm_after_it(width):
    from llama_rs_metal_b200.kernels import ops
    gen = torch.Generator().manual_seed(width)
    T = 5
    stream, y = torch.randn(T, width, generator=gen), torch.randn(T, width, generator=gen) * 3
    w, w2 = torch.rand(width, generator=gen) + 0.5, torch.rand(width, generator=gen) + 0.5
    want = stream.to(F64) + 0.7 * P.rms_norm(y.to(F64), w.to(F64), 1e-5)
    s1 = stream.to(DEV).clone()
    assert ops.rms_norm_add_(s1, y.to(DEV), w.to(DEV), 1e-5, 0.7) is None
    assert (s1.cpu().to(F64) - want).abs().max() < 1e-5
    s2 = stream.to(DEV).clone()
    out = ops.rms_norm_add_(s2, y.to(DEV), w.to(DEV), 1e-5, 0.7, w2.to(DEV), 1e-4, torch.float32)
    assert torch.equal(s1, s2)
    assert (out.cpu().to(F64) - P.rms_norm(want, w2.to(F64), 1e-4)).abs().max() < 1e-5


def test_clamped_gate_from_float32_sums():
    from llama_rs_metal_b200.kernels import ops
    gen = torch.Generator().manual_seed(2)
    T, inter, block = 6, 24, 8
    both = torch.randn(T, 2 * inter, generator=gen) * 3
    pairs = both.view(T, inter // block, 2, block).to(F64)
    g = torch.clamp(pairs[:, :, 0], max=1.5).reshape(T, inter)
    u = torch.clamp(pairs[:, :, 1], min=-1.5, max=1.5).reshape(T, inter)
    want = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    got = ops.clamped_gate_mul(both.to(DEV), block, 1.5, 1.702).cpu().to(F64)
    assert (got - want).abs().max() < 1e-5
    rounded = ops.clamped_gate_mul(both.to(DEV), block, 1.5, 1.702, out_dtype=torch.bfloat16).float().cpu().to(F64)
    assert (rounded - want).abs().max() < 2e-2
