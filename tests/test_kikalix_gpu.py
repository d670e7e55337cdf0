"""The Kikalix decoder through the engine, compared with the plain implementation (plain_kikalix.py).

Model level, on three tiny configurations (helpers.KIKALIX): whole prompts, prefill against
token-by-token decoding, portions down to two tokens, batches of unequal requests, slots that
are freed and used again, long decoding through captured steps, greedy generation through
Session.generate, and a replay through bin/trace_run. Mechanism level: the state scan, the
convolution's tail, windowed attention with the distance penalty (keys just inside and just
outside the window, at a page's border, prompts and decoding), the router and the experts.
"""
import math

import numpy as np
import pytest
import torch

import helpers
import plain_kikalix as P

pytestmark = pytest.mark.gpu
DEV = "cuda"
NAMES = ["K1", "K2", "K3"]


@pytest.fixture(scope="module")
def engine():
    from llama_rs_metal_b200 import Engine
    return Engine()


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """(name, dtype) -> model folder: float32 runs compare on free routing, bfloat16 runs on the
    variant whose choice of experts does not hang on a rounding (helpers.make_kikalix_dir)."""
    out = {}
    for n in NAMES:
        out[n, "float32"] = helpers.make_kikalix_dir(str(tmp_path_factory.mktemp(f"kikalix_{n}")), n)
        out[n, "bfloat16"] = helpers.make_kikalix_dir(str(tmp_path_factory.mktemp(f"kikalix_{n}_steady")), n,
                                                      steady_routing=True)
    return out


@pytest.fixture(scope="module")
def plain(folders):
    return {key: P.read_model(path) for key, path in folders.items()}


_REFS = {}


def reference(plain, name, tokens, dtype="float32"):
    key = (name, dtype, tuple(tokens))
    if key not in _REFS:
        config, tensors = plain[name, dtype]
        _REFS[key] = P.forward(config, tensors, tokens).numpy()
    return _REFS[key]


# Allowed error of a row of logits as a fraction of the largest reference logit.
# float32: the state mixers add up hundreds of tokens in float32 where the plain implementation
# has float64, and what they add up is fed back, so the allowance is five times the one of the
# attention-only models; a fault of any mechanism is orders of magnitude above it, and every row
# is held to it.
# bfloat16: a layer rounds its activations about twice as often as a layer of attention and one
# feed-forward does. And the design has places where a rounding is amplified without bound: a
# head's read-out is divided by its own root mean square, so at a sequence's first tokens, where
# the state is one outer product, the result hangs on the sign of a single small dot product.
# So in bfloat16 one row in twenty may be beyond the allowance (none by more than half the largest
# logit) and the median row must be well within it; the bfloat16 kernels themselves are held to
# their tolerance row by row in the mechanism tests below.
TOLERANCE = {"float32": 1e-4, "bfloat16": 6e-2}


def close(got, ref, dtype, what, drawn=False):
    """`drawn`: a configuration drawn at random may have heads of four values or a window of one
    key, where bfloat16 rounding weighs more than in the fixed configurations; there bfloat16 is
    only held to being finite, near in the median and nowhere far off (float32 stays strict)."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape and np.all(np.isfinite(got)), what
    err = np.abs(got - ref).max(axis=-1) / max(float(np.abs(ref).max()), 1e-30)
    worst, beyond = int(err.argmax()), int(np.count_nonzero(err > TOLERANCE[dtype]))
    allowed = 0 if dtype == "float32" else len(err) if drawn else max(1, len(err) // 20)
    ok = beyond <= allowed and (dtype == "float32" or (
        err[worst] <= 0.5 and (len(err) < 8 or np.median(err) <= TOLERANCE[dtype] / (1 if drawn else 3))))
    assert ok, (f"{what}: {beyond} of {len(err)} rows beyond {TOLERANCE[dtype]:.0e} of the largest logit, row {worst} "
                f"by {err[worst]:.3e}; first such row {int(np.argmax(err > TOLERANCE[dtype]))}; median {np.median(err):.3e}")


def vocab_of(name):
    return helpers.KIKALIX[name]["config"]["vocab"]


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
    runner, cache, _ = open_runner(engine, folders[name, dtype], dtype)
    for i, n in enumerate([150, 37, 1, 2]):       # the first tokens of a sequence are rows 0, 1, ...
        tokens = helpers.random_tokens(300 + i, n, vocab_of(name))
        slot = cache.open_slot()
        got = runner.step([entry(slot, tokens)]).cpu().numpy()
        cache.close_slot(slot)                     # the next prompt takes the same slot and state
        close(got, reference(plain, name, tokens, dtype), dtype, f"{name} prompt of {n}")
    runner.check_device_status()


def test_every_layer_run_matches_the_plain_residual_stream(engine, folders, plain):
    """float32, layer run by layer run (a looped layer counts each time)."""
    name = "K1"
    runner, cache, model = open_runner(engine, folders[name, "float32"], "float32", use_graphs=False)
    runner.pads_prompts = False
    streams = []
    for block in model.blocks:
        def wrapped(hidden, ctx, view, inner=block.forward):
            out = inner(hidden, ctx, view)
            ctx.settle(out)                         # partial sums a part left for the next norm
            streams.append(out.clone())
            return out
        block.forward = wrapped
    tokens = helpers.random_tokens(7, 29, vocab_of(name))
    runner.step([entry(cache.open_slot(), tokens)])
    config, tensors = plain[name, "float32"]
    expected = []
    P.forward(config, tensors, tokens, expected)
    assert len(streams) == len(expected) == 1 + 3 * 2
    for i, (got, ref) in enumerate(zip(streams, expected)):
        scale = float(ref.abs().max())
        assert float((got.cpu().double() - ref).abs().max()) <= 2e-5 * scale, f"layer run {i}"


# --------------------------------------------------------------------------- cutting and batching
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_prefill_then_decoding_in_an_unequal_batch(engine, folders, plain, name, dtype):
    """Prompts of 3 tokens in one step, then token by token; shorter sequences end earlier.
    Decoding crosses the windows (7 and 70 tokens) and a page's border."""
    lengths = [140, 9, 33, 71]
    seqs = [helpers.random_tokens(40 + i, n, vocab_of(name)) for i, n in enumerate(lengths)]
    runner, cache, _ = open_runner(engine, folders[name, dtype], dtype)
    slots = [cache.open_slot() for _ in seqs]
    got = [[] for _ in seqs]
    out = runner.step([entry(sl, s[:3]) for sl, s in zip(slots, seqs)])
    for b in range(len(seqs)):
        got[b].append(out[3 * b:3 * b + 3])
    for p in range(3, max(lengths)):
        live = [b for b in range(len(seqs)) if p < len(seqs[b])]
        out = runner.step([entry(slots[b], [seqs[b][p]]) for b in live])
        for row, b in enumerate(live):
            got[b].append(out[row:row + 1].clone())
    for b, s in enumerate(seqs):
        close(torch.cat(got[b]).cpu().numpy(), reference(plain, name, s, dtype), dtype,
              f"{name} sequence {b} decoded in a batch")
    runner.check_device_status()


@pytest.mark.parametrize("sizes", [[2], [17], [1, 2, 63, 64], [5, 3], [64, 1]])
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_any_size_give_the_whole_prompt(engine, folders, plain, name, sizes):
    seqs = [helpers.random_tokens(60 + i, n, vocab_of(name)) for i, n in enumerate([133, 20, 66])]
    if sizes == [2]:
        seqs = seqs[1:]
    runner, cache, _ = open_runner(engine, folders[name, "float32"], "float32")
    slots = [cache.open_slot() for _ in seqs]
    got, at, i = [[] for _ in seqs], [0] * len(seqs), 0
    while any(at[b] < len(seqs[b]) for b in range(len(seqs))):
        n = sizes[min(i, len(sizes) - 1)]
        live = [b for b in range(len(seqs)) if at[b] < len(seqs[b])]
        out = runner.step([entry(slots[b], seqs[b][at[b]:at[b] + n]) for b in live])
        row = 0
        for b in live:
            m = min(n, len(seqs[b]) - at[b])
            got[b].append(out[row:row + m].clone())
            row, at[b] = row + m, at[b] + m
        i += 1
    for b, s in enumerate(seqs):
        close(torch.cat(got[b]).cpu().numpy(), reference(plain, name, s), "float32",
              f"{name} sequence {b} in portions {sizes}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_company_in_the_batch_changes_nothing_beyond_rounding(engine, folders, plain, dtype):
    name = "K2"
    runner, cache, _ = open_runner(engine, folders[name, dtype], dtype)
    a, b, c = (helpers.random_tokens(80 + i, n, vocab_of(name)) for i, n in enumerate([20, 130, 64]))
    s1, s2, s3 = cache.open_slot(), cache.open_slot(), cache.open_slot()
    both = runner.step([entry(s2, b), entry(s1, a), entry(s3, c)]).cpu().numpy()
    close(both[:130], reference(plain, name, b, dtype), dtype, "long request in a batch")
    close(both[130:150], reference(plain, name, a, dtype), dtype, "short request in a batch")
    close(both[150:], reference(plain, name, c, dtype), dtype, "one-page request in a batch")


def test_a_freed_slot_starts_from_nothing(engine, folders, plain):
    """State, convolution tails and pages of a finished sequence must not reach the next one that
    takes its slot, whether it starts with a prompt or with a single token."""
    name = "K1"
    runner, cache, _ = open_runner(engine, folders[name, "float32"], "float32", max_slots=2)
    first = helpers.random_tokens(1, 90, vocab_of(name))
    for tokens in (helpers.random_tokens(2, 50, vocab_of(name)), helpers.random_tokens(3, 1, vocab_of(name))):
        slot = cache.open_slot()
        runner.step([entry(slot, first[:80])])
        for t in first[80:]:
            runner.step([entry(slot, [t])])
        cache.close_slot(slot)
        again = cache.open_slot()
        assert again == slot
        got = runner.step([entry(again, tokens)]).cpu().numpy()
        close(got, reference(plain, name, tokens), "float32", "a request in a used slot")
        cache.close_slot(again)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_captured_steps(engine, folders, plain, dtype):
    name = "K2"
    tokens = helpers.random_tokens(5, 260, vocab_of(name))
    runner, cache, _ = open_runner(engine, folders[name, dtype], dtype)
    assert runner.use_graphs
    slot = cache.open_slot()
    rows = [runner.step([entry(slot, tokens[:20])])]
    for t in tokens[20:]:
        rows.append(runner.step([entry(slot, [t])]).clone())
    close(torch.cat(rows).cpu().numpy(), reference(plain, name, tokens, dtype), dtype, "260 tokens, 240 of them decoded")


# --------------------------------------------------------------------------- generation and replay
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_session(engine, folders, plain, dtype):
    from llama_rs_metal_b200 import GenerationOptions, Sampling
    name = "K1"
    config, tensors = plain[name, dtype]
    model = engine.load(folders[name, dtype], dtype=dtype)
    session = model.session(context=128, max_batch=4)
    prompts = [helpers.random_tokens(8 + i, n, vocab_of(name)) for i, n in enumerate([1, 9, 33, 12, 5])]
    results = session.generate(prompts, GenerationOptions(max_tokens=8, sampling=Sampling(temperature=0.0)),
                               stop_token_ids=())
    for prompt, result in zip(prompts, results):
        assert len(result.tokens) == 8 and result.finish_reason == "length"
        seq = list(prompt)
        for token in result.tokens:
            logits = P.forward(config, tensors, seq)[-1].numpy()
            best = int(np.argmax(logits))
            slack = TOLERANCE[dtype] * 2 * np.abs(logits).max()
            assert token == best or logits[best] - logits[token] <= slack
            seq.append(token)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_through_the_trace_runner(folders, plain, dtype, tmp_path):
    name = "K1"
    requests = {f"r{i}": helpers.random_tokens(100 + i, n, vocab_of(name)) for i, n in enumerate([5, 70, 40, 1, 130])}
    refs = {rid: reference(plain, name, tokens, dtype) for rid, tokens in requests.items()}
    trace = helpers.Trace()
    for rid, tokens in requests.items():
        trace.whole("whole:" + rid, tokens)
        trace.tail_one_by_one("tail:" + rid, tokens)
    trace.chunks("chunks:r4", requests["r4"], [17])
    trace.batch({f"batch:{n}": requests[n] for n in requests},
                {f"batch:{n}": max(1, len(requests[n]) - 4 - 3 * i) for i, n in enumerate(requests)})
    need = sum(-(-len(t) // 64) * 64 for t in requests.values())
    outputs = helpers.run_trace(folders[name, dtype], dtype, trace, need, str(tmp_path))
    for step in sorted(trace.rows):
        rows = trace.rows[step]
        ref = np.stack([refs[rid.split(":")[-1]][pos] for rid, pos in rows])
        close(outputs[step], ref, dtype, f"step {step} ({rows[0][0]} pos {rows[0][1]} ..)")


# --------------------------------------------------------------------------- mechanisms: the state scan
def plain_scan(q, k, v, state, decay=None, g=None, beta=None):
    """One sequence, float64: q, k [T, KH, d], v [T, H, dv], state [H, d, dv] (updated in place)."""
    T, KH, d = q.shape
    H, dv = v.shape[1], v.shape[2]
    out = torch.zeros(T, H, dv, dtype=torch.float64)
    for t in range(T):
        for h in range(H):
            kh = h // (H // KH)
            if g is None:
                state[h] = decay[h] * state[h] + torch.outer(k[t, kh], v[t, h])
            else:
                state[h] = g[t, h][:, None] * state[h]
                u = beta[t, h] * (v[t, h] - state[h].T @ k[t, kh])
                state[h] = state[h] + torch.outer(k[t, kh], u)
            out[t, h] = state[h].T @ q[t, kh]
    return out


@pytest.mark.parametrize("delta", [False, True])
@pytest.mark.parametrize("H,KH,d,dv", [(3, 1, 24, 40), (2, 2, 80, 8), (4, 2, 64, 32), (1, 1, 5, 3), (2, 1, 130, 16)])
def test_state_scan_matches_the_recurrence_and_carries_its_state(H, KH, d, dv, delta):
    """Several sequences of unequal lengths and one of padding (slot -1); then a second step onto
    the same slots in portions of 1, 2 and 17 tokens. Decays close to 1: the first tokens still
    count at the end."""
    from llama_rs_metal_b200.kernels import ops
    gen = torch.Generator().manual_seed(H * 1000 + d)
    lengths, slots = [37, 1, 16, 5], [2, 0, -1, 3]
    state = torch.zeros(4, H, d, dv, dtype=torch.float32, device=DEV)
    plain_state = torch.zeros(4, H, d, dv, dtype=torch.float64)
    decay = torch.tensor([0.999 - 0.01 * h for h in range(H)], dtype=torch.float64)
    for step_lengths in (lengths, [1, 2, 17, 1]):
        T = sum(step_lengths)
        q, k = (torch.randn(T, KH, d, generator=gen, dtype=torch.float64) / math.sqrt(d) for _ in range(2))
        v = torch.randn(T, H, dv, generator=gen, dtype=torch.float64)
        g = 1.0 - 0.02 * torch.rand(T, H, d, generator=gen, dtype=torch.float64)
        beta = torch.rand(T, H, generator=gen, dtype=torch.float64)
        cu = torch.tensor([0] + list(np.cumsum(step_lengths)), dtype=torch.int32, device=DEV)
        f = lambda t: t.to(torch.float32).to(DEV).contiguous()  # noqa: E731
        if delta:
            got = ops.linear_state_scan(f(q), f(k), f(v), state, cu, torch.tensor(slots, dtype=torch.int32, device=DEV),
                                        g=f(g), beta=f(beta))
        else:
            got = ops.linear_state_scan(f(q), f(k), f(v), state, cu, torch.tensor(slots, dtype=torch.int32, device=DEV),
                                        head_decay=f(decay))
        at = 0
        for n, slot in zip(step_lengths, slots):
            s = plain_state[slot] if slot >= 0 else torch.zeros(H, d, dv, dtype=torch.float64)
            f32 = lambda t: t.to(torch.float32).double()  # noqa: E731  (the kernel sees the float32 rounding)
            ref = plain_scan(f32(q[at:at + n]), f32(k[at:at + n]), f32(v[at:at + n]), s,
                             f32(decay), f32(g[at:at + n]) if delta else None, f32(beta[at:at + n]) if delta else None)
            scale = float(ref.abs().max())
            assert float((got[at:at + n].cpu().double() - ref).abs().max()) <= 2e-5 * scale, f"slot {slot}"
            at += n
        for slot in (0, 2, 3):
            assert float((state[slot].cpu().double() - plain_state[slot]).abs().max()) <= \
                2e-5 * float(plain_state[slot].abs().max())
        assert float(state[1].abs().max()) == 0.0       # no sequence held slot 1; padding stored nothing


@pytest.mark.parametrize("taps", [1, 2, 5])
def test_convolution_tail_makes_portions_equal_to_the_whole(taps):
    from llama_rs_metal_b200.kernels import ops
    H, G, d, dv = 2, 1, 8, 4
    C = 2 * G * d + H * dv
    gen = torch.Generator().manual_seed(taps)
    T = 23
    proj = torch.randn(T, C + H, generator=gen).to(DEV)
    a = torch.randn(T, H * d, generator=gen).to(DEV)
    dt_bias, rate = torch.randn(H * d, generator=gen).to(DEV), torch.rand(H, generator=gen).to(DEV)
    w = torch.randn(C, taps, generator=gen).to(DEV)

    def run(cuts):
        tails = torch.zeros(2, taps - 1, C, device=DEV)
        parts = []
        for lo, hi in zip(cuts[:-1], cuts[1:]):
            n = hi - lo
            cu = torch.tensor([0, n], dtype=torch.int32, device=DEV)
            parts.append(ops.delta_prepare(proj[lo:hi].contiguous(), 0, C, a[lo:hi].contiguous(), dt_bias, rate, w,
                                           tails, cu, torch.zeros(n, dtype=torch.int32, device=DEV),
                                           torch.tensor([1], dtype=torch.int32, device=DEV), H, G, d, dv, 1e-6, 0.5))
        return [torch.cat([p[i] for p in parts]) for i in range(5)], tails
    whole, tails = run([0, T])
    for cuts in ([0, 1, 2, 3, 4, 5, 6, 23], [0, 2, 4, 9, 23], [0, 22, 23]):
        cut, cut_tails = run(cuts)
        for x, y in zip(whole, cut):
            assert torch.equal(x, y)
        assert torch.equal(tails, cut_tails)
    # against the definition: y_t = silu(sum_j w[:, n-1-j] x_(t-j)), q and k unit vectors per head
    x = proj[:, :C].cpu().double()
    y = torch.zeros(T, C, dtype=torch.float64)
    for t in range(T):
        for j in range(taps):
            if t - j >= 0:
                y[t] += w[:, taps - 1 - j].cpu().double() * x[t - j]
    y = y * torch.sigmoid(y)
    qh = y[:, :G * d].reshape(T, G, d)
    qh = qh / torch.sqrt((qh * qh).sum(-1, keepdim=True) + 1e-6) * 0.5
    assert float((whole[0].cpu().double() - qh).abs().max()) < 1e-5
    assert float((whole[2].cpu().double().reshape(T, -1) - y[:, 2 * G * d:]).abs().max()) < 1e-5
    z = a.cpu().double() + dt_bias.cpu().double()
    g = torch.exp(-rate.cpu().double().repeat_interleave(d) * torch.nn.functional.softplus(z))
    assert float((whole[3].cpu().double().reshape(T, -1) - g).abs().max()) < 1e-5
    assert float((whole[4].cpu().double() - torch.sigmoid(proj[:, C:].cpu().double())).abs().max()) < 1e-5


# --------------------------------------------------------------------------- mechanisms: windowed attention
def plain_attention(q, k, v, scale, window, slopes, first_query=0):
    """float64; q [n, H, d] are the queries at positions first_query .., k, v [L, G, d|dv]."""
    n, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(n, H, v.shape[2], dtype=torch.float64)
    for i in range(n):
        pos = first_query + i
        lo = max(0, pos - window + 1)
        for h in range(H):
            kh = h // (H // G)
            s = (k[lo:pos + 1, kh] @ q[i, h]) * scale - slopes[h] * (pos - torch.arange(lo, pos + 1, dtype=torch.float64))
            out[i, h] = torch.softmax(s, 0) @ v[lo:pos + 1, kh]
    return out


@pytest.mark.parametrize("dtype,d,dv,window", [(torch.float32, 24, 40, 7), (torch.float32, 16, 16, 70),
                                               (torch.bfloat16, 64, 64, 70), (torch.bfloat16, 32, 32, 64),
                                               (torch.bfloat16, 128, 128, 100), (torch.bfloat16, 48, 16, 65)])
def test_window_edge_and_distance_penalty_in_prompts_decoding_and_portions(dtype, d, dv, window):
    """One key stands out: its score is far above all others for every query that sees it, so a
    query's output is that key's value while the key is inside the window (also at distance
    window - 1) and something else from distance `window` on. A window that is one token off, or
    a penalty that is left out, shows in whole rows. The spike sits so that the window's edge
    falls on and next to a page's border."""
    from llama_rs_metal_b200.cache import Cache
    from llama_rs_metal_b200.kernels import ops
    from llama_rs_metal_b200.parts.base import KeyValueRequest
    H, G, L = 4, 2, 210
    gen = torch.Generator().manual_seed(d + window)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=torch.float64)
    for spike in (64 - window + 64, 5, 127):
        if spike < 0 or spike + window + 6 >= L:
            continue
        q = torch.randn(L, H, d, generator=gen, dtype=torch.float64) * 0.1
        k = torch.randn(L, G, d, generator=gen, dtype=torch.float64) * 0.1
        v = torch.randn(L, G, dv, generator=gen, dtype=torch.float64)
        q[:, :, 0] = 6.0
        k[spike, :, 0] = 6.0                      # score 36 * scale above the rest
        v[spike] = 9.0
        scale = 1.0
        r = lambda t: t.to(dtype).to(DEV).contiguous()  # noqa: E731
        rq, rk, rv = r(q), r(k), r(v)
        ref = plain_attention(rq.cpu().double(), rk.cpu().double(), rv.cpu().double(), scale, window, slopes)
        inside, outside = ref[spike + window - 1], ref[spike + window]
        assert float((inside - 9.0).abs().max()) < 0.5 and float((outside - 9.0).abs().min()) > 3.0
        tol = 2e-5 if dtype == torch.float32 else 3e-2
        dev_slopes = slopes.to(torch.float32).to(DEV)
        cu = torch.tensor([0, L], dtype=torch.int32, device=DEV)
        seq_of = torch.zeros(L, dtype=torch.int32, device=DEV)
        got = ops.attention_prefill(rq, rk, rv, cu, seq_of, L, scale, window, dev_slopes, 1.0)
        assert float((got.cpu().double().reshape(L, H, dv) - ref).abs().max()) <= tol * 9.0, "prompt"
        # the same over the paged cache: keys stored by the split kernel, then queries one by one
        # (decoding) and in portions of 3 (several queries per sequence)
        request = KeyValueRequest(G, d, window, None if dv == d else dv)
        cache = Cache([request], dtype, torch.device(DEV), 512, 2, 512)
        cache.open_slot()
        slot = cache.open_slot()
        for portion in (1, 3):
            cache.reset_slot(slot)
            rows = []
            first = spike + window - 4
            cache.grow([(slot, first)])
            cache.sync()
            dest = torch.tensor(cache.destination_rows([slot], [0], [first])[0], device=DEV)
            packed = torch.cat([rq[:first].reshape(first, -1), rk[:first].reshape(first, -1),
                                rv[:first].reshape(first, -1)], dim=1).contiguous()
            ops.qkv_bias_store(packed, None, H, G, d, dv, kv=cache.view(0), dest_rows=dest, keep_packed=False)
            cache.commit([(slot, first)])
            for at in range(first, first + 9, portion):
                n = portion
                cache.grow([(slot, at + n, at)])
                cache.sync()
                dest = torch.tensor(cache.destination_rows([slot], [at], [n])[0], device=DEV)
                packed = torch.cat([rq[at:at + n].reshape(n, -1), rk[at:at + n].reshape(n, -1),
                                    rv[at:at + n].reshape(n, -1)], dim=1).contiguous()
                qn, _, _ = ops.qkv_bias_store(packed, None, H, G, d, dv, kv=cache.view(0), dest_rows=dest,
                                              keep_packed=False)
                cache.commit([(slot, at + n)])
                slots_t = torch.tensor([slot], dtype=torch.int32, device=DEV)
                lens = torch.tensor([at + n], dtype=torch.int32, device=DEV)
                if portion == 1:
                    out = ops.attention_decode(qn, cache.view(0), slots_t, lens, 256, scale, window, dev_slopes, 1.0)
                else:
                    out = ops.attention_extend(qn, cache.view(0), torch.tensor([0, n], dtype=torch.int32, device=DEV),
                                               torch.zeros(n, dtype=torch.int32, device=DEV),
                                               torch.arange(at, at + n, dtype=torch.int32, device=DEV), slots_t, lens,
                                               n, scale, window, dev_slopes, 1.0)
                rows.append(out.reshape(n, H, dv))
            got = torch.cat(rows).cpu().double()
            assert float((got - ref[first:first + 9]).abs().max()) <= tol * 9.0, f"portions of {portion}"


def test_split_adds_biases_and_scales_nothing_else():
    from llama_rs_metal_b200.kernels import ops
    H, G, d, dv, T = 3, 1, 8, 5, 6
    x = torch.randn(T, H * d + G * d + G * dv, device=DEV)
    bias = torch.randn(x.shape[1], device=DEV)
    q, k, v = ops.qkv_bias_store(x, bias, H, G, d, dv)
    y = x + bias
    assert torch.equal(q.reshape(T, -1), y[:, :H * d]) and torch.equal(k.reshape(T, -1), y[:, H * d:H * d + G * d])
    assert torch.equal(v.reshape(T, -1), y[:, H * d + G * d:])


# --------------------------------------------------------------------------- mechanisms: router and experts
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,width,ff,E,top", [(5, 72, 40, 5, 3), (1, 64, 200, 3, 3), (70, 128, 96, 8, 1), (300, 64, 64, 4, 2)])
def test_router_and_experts_match_the_definition(dtype, T, width, ff, E, top):
    from llama_rs_metal_b200.kernels import ops
    gen = torch.Generator().manual_seed(T + width)
    limit, alpha = 0.8, 1.702
    w = {"router": torch.randn(E, width, generator=gen), "router.b": torch.randn(E, generator=gen)}
    for e in range(E):
        w[f"e{e}.gate"] = torch.randn(ff, width, generator=gen) / math.sqrt(width) * 2
        w[f"e{e}.up"] = torch.randn(ff, width, generator=gen) / math.sqrt(width) * 2
        w[f"e{e}.down"] = torch.randn(width, ff, generator=gen) / math.sqrt(ff)
    w = {n: t.to(dtype) for n, t in w.items()}
    x = torch.randn(T, width, generator=gen).to(dtype)
    f = dict(router=dict(experts=E, top=top), expert=dict(limit=limit))
    ref = P.mixture_of_experts(x.double(), {n: t.double() for n, t in w.items()}, "", f)
    logits = ops.linear(x.float().to(DEV), w["router"].float().to(DEV))
    ids, weights = ops.moe_route(logits, w["router.b"].float().to(DEV), top)
    ref_logits = x.double() @ w["router"].double().T + w["router.b"].double()
    assert torch.equal(ids.cpu().long().sort(1).values, torch.topk(ref_logits, top).indices.sort(1).values)
    assert float((weights.sum(1) - 1).abs().max()) < 1e-5
    gate_up = torch.stack([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(E)]).to(DEV).contiguous()
    down = torch.stack([w[f"e{e}.down"] for e in range(E)], dim=1).to(DEV).contiguous()
    planes = ops.moe_experts_rows(x.to(DEV), gate_up, down, ids, weights, limit, alpha)
    got = ops.add_planes_(torch.zeros(T, width, device=DEV), planes).cpu().double()
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert float((got - ref).abs().max()) <= tol * float(ref.abs().max())
    # the same through the products over every expert, the unchosen ones' weights set to zero
    all_gu = ops.linear(x.to(DEV), gate_up.view(E * 2 * ff, width))
    y = ops.moe_dense_gate(all_gu, ids, weights, E, limit, alpha)
    chosen = torch.zeros(T, E, dtype=torch.bool)
    chosen.scatter_(1, ids.cpu().long(), True)
    assert bool(((y.view(T, E, ff).float().abs().sum(-1) != 0).cpu() <= chosen).all())
    got = ops.linear(y, down.view(width, E * ff), out_dtype=torch.float32).cpu().double()
    assert float((got - ref).abs().max()) <= (2e-5 if dtype == torch.float32 else 3e-2) * float(ref.abs().max())


# --------------------------------------------------------------------------- small pieces
def test_norm_with_an_offset_and_row_added_to_the_stream():
    from llama_rs_metal_b200.kernels import ops
    from llama_rs_metal_b200.parts.norm import RMSNorm
    from llama_rs_metal_b200.runtime import Runtime
    x = torch.randn(7, 72, device=DEV)
    w = (torch.randn(72) * 0.2).to(torch.bfloat16)
    norm = RMSNorm(72, 1e-6, offset=1.0)
    norm.bind({"weight": w.to(DEV)}, Runtime(torch.device(DEV), torch.float32))
    got = ops.rms_norm(x, norm.weight, norm.eps, torch.float32)
    ref = P.offset_norm(x.cpu().double(), w.double(), 1e-6)
    assert float((got.cpu().double() - ref).abs().max()) < 1e-5
    row = torch.randn(72, device=DEV)
    y = x.clone()
    ops.add_row_(y, row)
    assert torch.equal(y, x + row)


# --------------------------------------------------------------------------- configurations drawn at random
def drawn_configuration(seed):
    """Sizes, head counts, layer order, windows, constants and the loop, all drawn: nothing in the
    library may rest on the values of one model."""
    rng = np.random.default_rng(seed)
    pick = lambda *values: values[int(rng.integers(len(values)))]  # noqa: E731
    width = int(pick(40, 64, 100, 136))
    layers = []
    for _ in range(int(rng.integers(2, 5))):
        experts = int(pick(2, 3, 6, 9))
        mlp = None if rng.random() < 0.25 else helpers._moe(int(pick(8, 20, 32, 56)), float(pick(0.5, 1.5, 7.0)), experts,
                                                            int(rng.integers(1, experts + 1)))
        if rng.random() < 0.4:
            heads, dim = int(pick(1, 2, 5)), int(pick(6, 16, 32))
            dims = int(pick(2, dim // 2 * 2, dim // 2 // 2 * 2 or 2))
            layers.append(dict(type="retention", mlp=mlp, mixer=dict(
                heads=heads, dim=dim, vdim=int(pick(4, 16, 40)), decay=[float(a) for a in 1 - rng.random(heads) * 0.2],
                rot=dict(dims=dims, base=float(pick(10.0, 1e4, 1e6))))))
        else:
            kv, group = int(pick(1, 2, 3)), int(pick(1, 2, 4))
            rkv, rgroup = int(pick(1, 2)), int(pick(1, 3))
            dim = int(pick(8, 24, 32, 64))
            layers.append(dict(type="parallel", mlp=mlp, mixer=dict(
                left=dict(heads=kv * group, kv_heads=kv, dim=dim, vdim=int(pick(dim, 8, 48)),
                          scale=float(pick(0.1, 0.35, dim ** -0.5)), mask=dict(size=int(pick(1, 2, 5, 33, 64, 65, 200)))),
                left_scale=float(pick(1.0, 0.3, 1.7)),
                right=dict(heads=rkv * rgroup, kv_heads=rkv, dim=int(pick(4, 12, 32)), vdim=int(pick(4, 20, 32)),
                           conv=int(pick(1, 2, 4, 7)), decay_rank=int(pick(1, 4, 9)), gate_rank=int(pick(2, 8))),
                right_scale=float(pick(1.0, 0.5, 2.0)))))
    start = int(rng.integers(0, len(layers)))
    stop = int(rng.integers(start + 1, len(layers) + 1))
    return dict(architecture="Kikalix", vocab=int(pick(50, 257, 601)), width=width,
                norm=dict(eps=float(pick(1e-5, 1e-6, 1e-3))), layers=layers,
                loop=dict(start=start, stop=stop, times=int(pick(1, 2, 3))))


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(engine, tmp_path, seed):
    spec = dict(config=drawn_configuration(seed), seed=100 + seed, std=0.15)
    folder = helpers.make_kikalix_dir(str(tmp_path / "free"), spec)
    steady = helpers.make_kikalix_dir(str(tmp_path / "steady"), spec, steady_routing=True)
    vocab = drawn_configuration(seed)["vocab"]
    seqs = [helpers.random_tokens(seed * 10 + i, n, vocab) for i, n in enumerate([90, 7, 1])]
    for path, dtype in ((folder, "float32"), (steady, "bfloat16")):
        config, tensors = P.read_model(path)
        refs = [P.forward(config, tensors, s).numpy() for s in seqs]
        runner, cache, _ = open_runner(engine, path, dtype)
        slots = [cache.open_slot() for _ in seqs]
        heads = [max(1, len(s) - 12) for s in seqs]                      # prompts, then decoding together
        out = runner.step([entry(sl, s[:n]) for sl, s, n in zip(slots, seqs, heads)])
        got, row = [[] for _ in seqs], 0
        for b, n in enumerate(heads):
            got[b].append(out[row:row + n].clone())
            row += n
        for p in range(12):
            live = [b for b in range(len(seqs)) if heads[b] + p < len(seqs[b])]
            if not live:
                break
            out = runner.step([entry(slots[b], [seqs[b][heads[b] + p]]) for b in live])
            for r, b in enumerate(live):
                got[b].append(out[r:r + 1].clone())
        for b in range(len(seqs)):
            close(torch.cat(got[b]).cpu().numpy(), refs[b], dtype, f"drawn configuration {seed}, sequence {b}",
                  drawn=True)
        runner.check_device_status()
