"""The Ramosun design in the engine against the plain float64 model of ``plain_ramosun.py``: whole prompts,
decoding token by token, portions down to two tokens, batches of unequal requests, pages and slots used
again, windows' edges and far tokens with weights that make them show, and greedy generation through
``Engine``. float32 path to 2e-4 of the logits' spread, bfloat16 path to a few percent."""
from __future__ import annotations

import numpy as np
import pytest

import plain_ramosun as plain
import ramosun_models as rm

pytestmark = pytest.mark.gpu

# bfloat16: these small models repeat layers and amplify rounding (one and the same token differs by a tenth of the
# logits' spread between two bfloat16 kernels for the same product), so the path is held to a fifth at worst and to
# a few percent in the middle; the float32 path is the sharp test, and the bfloat16 kernels are tested alone, tightly.
LIMIT = {"float32": 2e-4, "bfloat16": 2e-1}
TYPICAL = {"float32": 1e-4, "bfloat16": 5e-2}


def spread_error(got: np.ndarray, want: np.ndarray) -> np.ndarray:
    """Per row: rms of the difference (mean taken off) over the rms of the wanted row (mean taken off)."""
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / np.sqrt((w ** 2).mean(-1))


def check(got, want, dtype, what):
    err = spread_error(np.asarray(got, dtype=np.float64), want)
    worst = int(np.argmax(err))
    assert err[worst] <= LIMIT[dtype], f"{what}: row {worst} differs by {err[worst]:.3e} of the row's spread"
    assert np.median(err) <= TYPICAL[dtype], f"{what}: half of the rows differ by {np.median(err):.3e} and more"


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    base = tmp_path_factory.mktemp("ramosun")
    out = {}
    for name, (raw, seed) in rm.CONFIGS.items():
        folder = str(base / name)
        raw, tensors = rm.write_model(folder, raw, seed)
        out[name] = (folder, raw, plain.as_float64(tensors))
    return out


def load(folder, dtype, **kw):
    from celeg_b200.engine.loading import load_model
    args = dict(dtype=dtype, max_requests=4, cache_tokens=1024, max_batched_tokens=512, max_context=512)
    args.update(kw)
    return load_model(folder, **args)


def run_steps(loaded, steps):
    """steps: lists of (request, tokens); every place is wanted. Returns {request: [its logits rows in order]}."""
    from celeg_b200.engine.step import StepEntry
    rows = {}
    for step in steps:
        step = [(name, tokens) for name, tokens in step if len(tokens) > 0]
        entries = [StepEntry(name, list(tokens), list(range(len(tokens)))) for name, tokens in step]
        logits = loaded.step.run(entries, auto_begin=True).cpu().numpy()
        loaded.step.raise_on_device_error()
        at = 0
        for name, tokens in step:
            rows.setdefault(name, []).append(logits[at:at + len(tokens)].copy())
            at += len(tokens)
    return {name: np.concatenate(parts) for name, parts in rows.items()}


def cut(tokens, sizes):
    """tokens in portions of the given sizes, cycled."""
    out, at, i = [], 0, 0
    while at < len(tokens):
        n = sizes[i % len(sizes)]
        out.append(tokens[at:at + n])
        at += n
        i += 1
    return out


def tokens_of(vocab, length, seed):
    return np.random.default_rng(seed).integers(0, vocab, size=length).tolist()


# ------------------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(rm.CONFIGS))
def test_whole_prompt_then_token_by_token(models, name, dtype):
    folder, raw, tensors = models[name]
    tokens = tokens_of(raw["vocab"], 90, 1)
    want = plain.forward(raw, tensors, tokens)
    loaded = load(folder, dtype)
    whole = run_steps(loaded, [[("w", tokens)]])["w"]
    check(whole, want, dtype, f"{name} whole")
    loaded.step.end("w")
    steps = [[("d", tokens[:37])]] + [[("d", [t])] for t in tokens[37:]]
    decoded = run_steps(loaded, steps)["d"]
    check(decoded, want, dtype, f"{name} prompt of 37 then token by token")
    if dtype == "float32":       # how the prompt is cut changes nothing beyond rounding
        assert np.abs(decoded - whole).max() <= 1e-3 * np.abs(whole).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(rm.CONFIGS))
def test_portions_of_several_sizes_down_to_two_tokens(models, name, dtype):
    folder, raw, tensors = models[name]
    tokens = tokens_of(raw["vocab"], 131, 2)
    want = plain.forward(raw, tensors, tokens)
    loaded = load(folder, dtype)
    for tag, sizes in (("a", [2, 3, 17, 2, 33]), ("b", [16, 16, 1, 15, 48]), ("c", [5, 2, 2, 64])):
        got = run_steps(loaded, [[(tag, part)] for part in cut(tokens, sizes)])[tag]
        check(got, want, dtype, f"{name} in portions of {sizes}")
        loaded.step.end(tag)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "mixed", "loop_from_start", "straight"])
def test_batches_of_unequal_requests_equal_each_alone(models, name, dtype):
    folder, raw, tensors = models[name]
    requests = {"p": tokens_of(raw["vocab"], 70, 3), "q": tokens_of(raw["vocab"], 23, 4),
                "r": tokens_of(raw["vocab"], 120, 5), "s": tokens_of(raw["vocab"], 9, 6)}
    want = {key: plain.forward(raw, tensors, value) for key, value in requests.items()}
    # portions of some beside single tokens of others; q joins late, s is left out of steps and goes on later
    plan = {"p": [40] + [1] * 30, "q": [0, 0, 2, 19, 1, 1], "r": [3, 50, 1, 1, 1, 62, 1, 1], "s": [1, 0, 0, 1, 0, 5, 2]}
    at = {key: 0 for key in requests}
    steps = []
    for n in range(40):
        step = []
        for key in ("s", "p", "q", "r"):
            sizes = plan[key]
            count = sizes[n] if n < len(sizes) else 1
            count = min(count, len(requests[key]) - at[key])
            if count > 0:
                step.append((key, requests[key][at[key]:at[key] + count]))
                at[key] += count
        if step:
            steps.append(step)
    assert all(at[key] == len(requests[key]) for key in requests)
    got = run_steps(load(folder, dtype), steps)
    for key in requests:
        check(got[key], want[key], dtype, f"{name} request {key} in a batch")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pages_and_slots_are_used_again(models, dtype):
    """Two slots and a pool of 160 positions for six requests one after the other, two live at a time: every
    later request sits in a slot and in pages that an earlier one has left full of its own state."""
    folder, raw, tensors = models["mixed"]
    loaded = load(folder, dtype, max_requests=2, cache_tokens=160)
    lengths = [75, 60, 31, 80, 17, 66]
    for round_ in range(3):
        pair = {f"x{2 * round_}": tokens_of(raw["vocab"], lengths[2 * round_], 20 + round_),
                f"y{2 * round_}": tokens_of(raw["vocab"], lengths[2 * round_ + 1], 30 + round_)}
        (a, ta), (b, tb) = pair.items()
        steps = [[(a, ta[:20]), (b, tb[:3])], [(a, ta[20:21]), (b, tb[3:])], [(a, ta[21:])]]
        got = run_steps(loaded, steps)
        for key, tokens in pair.items():
            check(got[key], plain.forward(raw, tensors, tokens), dtype, f"round {round_} request {key}")
            loaded.step.end(key)
        loaded.manager.check_invariants()
    assert loaded.manager.free_slots == 2


def test_long_decoding_from_the_first_token(models):
    folder, raw, tensors = models["loop_from_start"]
    tokens = tokens_of(raw["vocab"], 200, 7)
    got = run_steps(load(folder, "float32"), [[("l", [t])] for t in tokens])["l"]
    check(got, plain.forward(raw, tensors, tokens), "float32", "200 tokens one by one")


# ------------------------------------------------------------------------- one mechanism, made to show
def one_layer_model(tmp_path, layer, seed, **weights):
    raw = rm.single_layer(layer)
    folder = str(tmp_path / "one")
    raw, tensors = rm.write_model(folder, raw, seed, **weights)
    return folder, raw, plain.as_float64(tensors)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,rot", [(16, 8), (21, 16), (5, None)])
def test_window_edges_in_prompts_and_in_decoding(tmp_path, window, rot, dtype):
    """One attention layer with a sharpened softmax, and the token that draws most of the probed position's
    attention when it sits just inside the window (found by trying all). Just inside, it moves the probe's
    logits by a fifth and more; just outside, not at all; the engine follows the plain model in both, with the
    probe inside a prompt, as the first token of a portion, and decoded alone. Windows of one page, of a page and
    some, and of less than a page."""
    folder, raw, tensors = one_layer_model(tmp_path, rm.attention(2, 1, 16, window, rot_dims=rot), 40, sharpen=2.5)
    base = tokens_of(raw["vocab"], 64, 8)
    probe = 47
    inside, outside = probe - window + 1, probe - window
    loaded = load(folder, dtype)
    reference = plain.forward(raw, tensors, base)

    def moved_by(place, token):
        changed = list(base)
        changed[place] = token
        return spread_error(plain.forward(raw, tensors, changed)[probe:probe + 1], reference[probe:probe + 1])[0]

    # the token that, put just inside the window, draws most of the probe's attention
    loud = max(range(raw["vocab"]), key=lambda token: moved_by(inside, token))
    assert moved_by(inside, loud) > 0.2 and moved_by(outside, loud) < 1e-9, "the plain model itself"
    for place in (inside, outside):
        changed = list(base)
        changed[place] = loud
        want = plain.forward(raw, tensors, changed)
        for tag, steps in (("prompt", [changed]), ("portion", [changed[:probe], changed[probe:]]),
                           ("decoded", [changed[:30]] + [[t] for t in changed[30:]])):
            name = f"{tag}{place}"
            got = run_steps(loaded, [[(name, part)] for part in steps])[name]
            check(got, want, dtype, f"window {window}, changed place {place}, probe {tag}")
            loaded.step.end(name)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sink_takes_its_share(tmp_path, dtype):
    """With large sinks most of the softmax's weight goes nowhere; with very negative ones the sink vanishes.
    Both must match, and they must differ from each other (a left-out sink would pass neither)."""
    raw = rm.single_layer(rm.attention(4, 2, 8, 12, rot_dims=8))
    tensors = rm.make_tensors(raw, 41)
    tokens = tokens_of(raw["vocab"], 40, 9)
    outputs = []
    for tag, value in (("big", 4.0), ("none", -30.0)):
        import torch
        tensors["l0.mix.sink"] = torch.full((4,), value).to(torch.bfloat16)
        folder = str(tmp_path / tag)
        rm.write_model(folder, raw, 0, tensors=tensors)
        want = plain.forward(raw, plain.as_float64(tensors), tokens)
        loaded = load(folder, dtype)
        check(run_steps(loaded, [[("a", tokens)]])["a"], want, dtype, f"sinks of {value}")
        check(run_steps(loaded, [[("b", [t])] for t in tokens])["b"], want, dtype, f"sinks of {value}, decoded")
        outputs.append(want)
    assert spread_error(outputs[0], outputs[1]).min() > 0.05


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["mlstm", "delta"])
def test_a_far_token_shows_through_the_state(tmp_path, kind, dtype):
    """One recurrent layer whose gates remember, a sequence of tokens that write little, and at place 3 a token
    that writes much. Which token that is moves the logits 250 tokens later; the engine follows the plain model
    whether the tokens between came as one prompt, in portions, or one by one."""
    import torch
    layer = rm.mlstm(2, 16, 24) if kind == "mlstm" else rm.delta(1, 1, 16, 24, conv=4)
    raw = rm.single_layer(layer)
    bf16 = rm.make_tensors(raw, 42, remember=True)
    gate = "l0.mix.i" if kind == "mlstm" else "l0.mix.b"            # what decides how much a token writes
    bf16[gate] = (bf16[gate].float() * 8.0).to(torch.bfloat16)
    folder = str(tmp_path / "one")
    rm.write_model(folder, raw, 0, tensors=bf16)
    tensors = plain.as_float64(bf16)
    # in a model of one layer a token's gate depends on the token alone: quiet tokens fill the sequence, the two
    # loudest take turns at place 3
    pre = plain.norm_of(tensors, "l0.norm1", tensors["embed"]) @ tensors[gate].T
    quiet = np.argsort(pre.max(axis=1))[:raw["vocab"] // 4]
    loud = np.argsort(pre.min(axis=1))[-2:]
    base = np.random.default_rng(10).choice(quiet, size=256).tolist()
    base[3] = int(loud[0])
    changed = list(base)
    changed[3] = int(loud[1])
    want_base, want = plain.forward(raw, tensors, base), plain.forward(raw, tensors, changed)
    assert spread_error(want[250:], want_base[250:]).min() > 0.02, "the plain model itself forgot the far token"
    loaded = load(folder, dtype)
    for tag, steps in (("whole", [changed]), ("portions", cut(changed, [2, 70, 33, 16, 7])),
                       ("decoded", [changed[:6]] + [[t] for t in changed[6:]])):
        got = run_steps(loaded, [[(tag, part)] for part in steps])[tag]
        check(got, want, dtype, f"{kind}, {tag}")
        loaded.step.end(tag)


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_short_convolution_across_portion_borders(tmp_path, taps):
    """The delta rule's carried inputs: portions shorter than the kernel, equal to it, and longer."""
    folder, raw, tensors = one_layer_model(tmp_path, rm.delta(2, 2, 8, 8, conv=taps), 43)
    tokens = tokens_of(raw["vocab"], 40, 11)
    want = plain.forward(raw, tensors, tokens)
    loaded = load(folder, "float32")
    for tag, sizes in (("a", [1, 1, 2, 1, 3]), ("b", [taps, max(1, taps - 1), taps + 1]), ("c", [2, 9])):
        got = run_steps(loaded, [[(tag, part)] for part in cut(tokens, sizes)])[tag]
        check(got, want, "float32", f"{taps} taps, portions {sizes}")
        loaded.step.end(tag)


@pytest.mark.parametrize("dim,vdim", [(8, 5), (32, 32), (40, 70), (72, 16), (136, 24), (200, 8)])
@pytest.mark.parametrize("kind", ["mlstm", "delta"])
def test_key_and_value_sizes_of_the_recurrent_mixers(tmp_path, kind, dim, vdim):
    """One, two, four and eight lanes a column, value sizes that fill no warp evenly."""
    layer = rm.mlstm(2, dim, vdim) if kind == "mlstm" else rm.delta(2, 1, dim, vdim, conv=3)
    folder, raw, tensors = one_layer_model(tmp_path, layer, 44)
    tokens = tokens_of(raw["vocab"], 45, 12)
    want = plain.forward(raw, tensors, tokens)
    got = run_steps(load(folder, "float32"), [[("a", tokens[:20])], [("a", tokens[20:21])], [("a", tokens[21:])]])["a"]
    check(got, want, "float32", f"{kind} with keys of {dim} and values of {vdim}")


# ---------------------------------------------------------------------------- the engine's own entry point
@pytest.mark.parametrize("name", ["mixed", "straight"])
def test_greedy_generation_through_the_engine(models, name):
    """Prompts of unequal length through ``Engine.generate`` (scheduler, portions, sampler) in float32 against
    greedy decoding with the plain model."""
    from celeg_b200 import Engine, EngineOptions
    folder, raw, tensors = models[name]
    prompts = [tokens_of(raw["vocab"], n, 50 + n) for n in (5, 41, 18)]
    new = 12
    engine = Engine(folder, max_context=128, dtype="float32",
                    options=EngineOptions(max_active_requests=4, max_batched_tokens=32, page_tokens=16))
    got = engine.generate(prompts, max_new_tokens=new, temperature=0.0, repetition_penalty=1.0)
    compared = 0
    for prompt, generated in zip(prompts, got):
        assert len(generated) == new
        sequence = list(prompt)
        for token in generated:
            logits = plain.forward(raw, tensors, sequence)[-1]
            top = np.sort(logits)[-2:]
            if top[1] - top[0] > 1e-2 * (logits.max() - logits.min()):      # (no near tie in the plain model)
                assert int(token) == int(np.argmax(logits))
                compared += 1
            sequence.append(int(token))
    assert compared >= 2 * new


def test_greedy_generation_in_bfloat16_with_graphs(models):
    """The serving path (bfloat16, CUDA graphs, run-ahead): the tokens it generates are the plain model's wherever
    the plain model's best two logits are not close."""
    from celeg_b200 import Engine, EngineOptions
    folder, raw, tensors = models["mixed"]
    prompts = [tokens_of(raw["vocab"], n, 70 + n) for n in (9, 30)]
    engine = Engine(folder, max_context=128, dtype="bfloat16",
                    options=EngineOptions(max_active_requests=4, max_batched_tokens=64, page_tokens=16))
    got = engine.generate(prompts, max_new_tokens=10, temperature=0.0, repetition_penalty=1.0)
    for prompt, generated in zip(prompts, got):
        sequence = list(prompt)
        for token in generated:
            logits = plain.forward(raw, tensors, sequence)[-1]
            top = np.sort(logits)[-2:]
            if top[1] - top[0] > 0.05 * (logits.max() - logits.min()):
                assert int(token) == int(np.argmax(logits))
            sequence.append(int(token))


# ------------------------------------------------------------------------------- configurations drawn at random
def random_config(rng):
    """A configuration with every open size drawn anew: widths that are multiples of 4 only, head sizes from 4 to
    256, groupings up to 20 query heads a key head, windows from 1 token to longer than any sequence, 1 to 6 taps,
    the repeated run anywhere (or nowhere), layers with and without a feed-forward."""
    width = int(rng.choice([20, 36, 64, 100, 128, 192]))
    vocab = int(rng.integers(17, 300))
    layers = []
    for _ in range(int(rng.integers(1, 6))):
        kind = rng.choice(["attention", "mlstm", "delta"])
        if kind == "attention":
            dim = int(rng.choice([4, 8, 12, 16, 24, 32, 64, 96, 128, 256]))
            kv_heads = int(rng.integers(1, 4))
            heads = kv_heads * int(rng.choice([1, 1, 2, 3, 4, 20]))
            if heads * dim > 2048:
                heads = kv_heads
            window = None if rng.random() < 0.2 else int(rng.choice([1, 2, 7, 16, 17, 31, 64, 200]))
            rot = None if rng.random() < 0.2 else int(rng.choice([d for d in (2, 4, dim // 2, dim) if d % 2 == 0 and 0 < d <= dim]))
            scaling = None if rng.random() < 0.5 else {"factor": float(rng.choice([2.0, 8.0])), "low": 1.0,
                                                       "high": float(rng.choice([2.0, 4.0])), "original": int(rng.choice([16, 64, 512]))}
            layer = rm.attention(heads, kv_heads, dim, window, rot_dims=rot, base=float(rng.choice([50.0, 10000.0])),
                                 scaling=scaling, scale=float(rng.choice([dim ** -0.5, 0.2, 1.0])))
        elif kind == "mlstm":
            layer = rm.mlstm(int(rng.integers(1, 4)), int(rng.choice([4, 8, 20, 32, 64, 130])), int(rng.choice([4, 9, 32, 80])),
                             gate_cap=float(rng.choice([3.0, 15.0, 30.0])))
        else:
            kv_heads = int(rng.integers(1, 3))
            layer = rm.delta(kv_heads * int(rng.choice([1, 2, 3])), kv_heads, int(rng.choice([4, 8, 20, 32, 64, 130])),
                             int(rng.choice([4, 9, 32, 80])), conv=int(rng.integers(1, 7)))
        layers.append(rm.with_mlp(layer, None if rng.random() < 0.3 else int(rng.choice([8, 44, 128]))))
    loop = None
    if rng.random() < 0.7:
        start = int(rng.integers(0, len(layers)))
        loop = (start, int(rng.integers(start + 1, len(layers) + 1)), int(rng.integers(1, 4)))
    return rm.config(vocab, width, layers, loop=loop, eps=float(rng.choice([1e-5, 1e-6, 1e-3])),
                     softcap=None if rng.random() < 0.3 else float(rng.choice([5.0, 30.0])))


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Whole prompt, portions beside single tokens of a second request, and decoding, in both precisions."""
    rng = np.random.default_rng(1000 + seed)
    raw = random_config(rng)
    folder = str(tmp_path / "drawn")
    raw, bf16 = rm.write_model(folder, raw, 500 + seed)
    tensors = plain.as_float64(bf16)
    first, second = tokens_of(raw["vocab"], 75, seed), tokens_of(raw["vocab"], 33, 100 + seed)
    want = {"a": plain.forward(raw, tensors, first), "b": plain.forward(raw, tensors, second)}
    steps = [[("a", first[:19])], [("a", first[19:21]), ("b", second[:1])], [("b", second[1:2]), ("a", first[21:60])],
             [("a", first[60:61]), ("b", second[2:30])]]
    steps += [[("a", first[61 + i:62 + i])] + ([("b", second[30 + i:31 + i])] if 30 + i < len(second) else []) for i in range(14)]
    for dtype in ("float32", "bfloat16"):
        loaded = load(folder, dtype, page_tokens=int(rng.choice([8, 16, 32])))
        whole = run_steps(loaded, [[("w", first)]])["w"]
        loaded.step.end("w")
        got = run_steps(loaded, steps)
        if dtype == "float32":
            check(whole, want["a"], dtype, f"{raw['layers']} whole")
            for key in ("a", "b"):
                check(got[key], want[key], dtype, f"{raw['layers']} request {key}")
        else:
            # (random sizes amplify bfloat16 rounding at will: the path must follow the plain model in the middle)
            for rows, target in ((whole, want["a"]), (got["a"], want["a"]), (got["b"], want["b"])):
                assert np.median(spread_error(np.asarray(rows, dtype=np.float64), target)) < 0.15


# ------------------------------------------------------------------------------ command line, scheduler under load
def plain_greedy(raw, tensors, prompt, new):
    sequence = list(prompt)
    for _ in range(new):
        sequence.append(int(np.argmax(plain.forward(raw, tensors, sequence)[-1])))
    return sequence[len(prompt):]


def test_command_line_generates_and_dumps_logits(models, tmp_path, capsys):
    from celeg_b200.cli import main
    folder, raw, tensors = models["straight"]
    prompt = tokens_of(raw["vocab"], 12, 90)
    dump = str(tmp_path / "last.f32")
    code = main(["--model", folder, "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "6", "--dtype", "fp32",
                 "--temperature", "0", "--repetition-penalty", "1.0", "--runtime-tokens", "--dump-logits", dump,
                 "--context", "128"])
    assert code == 0
    captured = capsys.readouterr()
    want = plain_greedy(raw, tensors, prompt, 6)
    assert f"CELEG_GENERATED_TOKEN_IDS=[{','.join(map(str, want))}]" in captured.out
    logits = np.fromfile(dump, dtype="<f4").astype(np.float64)
    assert spread_error(logits[None, :], plain.forward(raw, tensors, prompt)[-1:])[0] < 2e-4
    assert main(["--model", folder, "--print-config"]) == 0
    assert '"architecture": "Ramosun"' in capsys.readouterr().out


def test_many_requests_through_a_small_pool_with_preemption(models):
    """Sixteen requests through three slots and a pool of pages that holds about two of them, growing while they
    decode (MAX_UTILIZATION): requests wait, are left out of steps, are preempted and run again from their prompt,
    in slots and pages others have used. Every request still gets the tokens it gets alone, wherever the plain
    model's choice is not a near tie (float32, greedy)."""
    from celeg_b200 import Engine, EngineOptions, RequestOptions, SamplingParams, SchedulerPolicy
    folder, raw, tensors = models["mixed"]
    rng = np.random.default_rng(60)
    lengths = rng.integers(1, 50, size=16).tolist()
    prompts = [tokens_of(raw["vocab"], n, 200 + i) for i, n in enumerate(lengths)]
    new_tokens = rng.integers(1, 16, size=16).tolist()
    options = EngineOptions(max_active_requests=3, max_batched_tokens=32, prefill_chunk_tokens=13, page_tokens=16,
                            logical_kv_pages=7, scheduler_policy=SchedulerPolicy.MAX_UTILIZATION)
    engine = Engine(folder, max_context=128, dtype="float32", options=options)
    greedy = SamplingParams(temperature=0.0, top_k=1, repetition_penalty=1.0)
    ids = [engine.submit(p, RequestOptions(max_new_tokens=n, eos_tokens=(), generation=greedy))
           for p, n in zip(prompts, new_tokens)]
    outputs = {i: [] for i in ids}
    pending = set(ids)
    steps = 0
    while pending:
        assert engine.step() or not engine.scheduler.has_work()
        engine.loaded.manager.check_invariants()
        for i in list(pending):
            result = engine.poll(i)
            outputs[i].extend(result.tokens)
            if result.finished:
                assert result.status.value == "finished", result.error
                pending.discard(i)
        steps += 1
        assert steps < 3000
    compared = 0
    for i, prompt, count in zip(ids, prompts, new_tokens):
        assert len(outputs[i]) == count
        sequence = list(prompt)
        for token in outputs[i]:
            logits = plain.forward(raw, tensors, sequence)[-1]
            top = np.sort(logits)[-2:]
            if top[1] - top[0] > 1e-2 * (logits.max() - logits.min()):
                assert int(token) == int(np.argmax(logits)), f"request {i} after {len(sequence)} tokens"
                compared += 1
            sequence.append(int(token))
    assert compared > sum(new_tokens) // 2
    assert engine.loaded.manager.free_slots == 3
