"""The Kedesun design in the engine against the plain float64 model of ``plain_kedesun.py``: whole prompts,
decoding token by token, portions down to two tokens, batches of unequal requests, pages and slots used again,
far keys and page borders with weights that make one key show, a far token through the retention's state, the
router's choices, and greedy generation through ``Engine`` and the command line. float32 path to 2e-4 of the
logits' spread, bfloat16 path to a few percent."""
from __future__ import annotations

import numpy as np
import pytest

import kedesun_models as km
import plain_kedesun as plain

pytestmark = pytest.mark.gpu

LIMIT = {"float32": 2e-4, "bfloat16": 1.5e-1}
TYPICAL = {"float32": 1e-4, "bfloat16": 5e-2}


def spread_error(got: np.ndarray, want: np.ndarray) -> np.ndarray:
    """Per row: rms of the difference (mean taken off) over the rms of the wanted row (mean taken off)."""
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / np.sqrt((w ** 2).mean(-1))


def check(got, want, dtype, what, routed=False):
    """``routed``: the model chooses experts. In bfloat16 a token whose best choices lie close together may take
    another expert than in the plain model, and its row (and, fading, the rows after it) then differs by more than
    rounding; one row in twelve may, by at most the row's whole spread. float32 is held to the limit everywhere."""
    err = spread_error(np.asarray(got, dtype=np.float64), want)
    worst = int(np.argmax(err))
    if routed and dtype == "bfloat16":
        assert err[worst] <= 1.0, f"{what}: row {worst} differs by {err[worst]:.3e} of the row's spread"
        assert (err > LIMIT[dtype]).sum() <= max(1, len(err) // 12), f"{what}: {(err > LIMIT[dtype]).sum()} rows over the limit"
    else:
        assert err[worst] <= LIMIT[dtype], f"{what}: row {worst} differs by {err[worst]:.3e} of the row's spread"
    assert np.median(err) <= TYPICAL[dtype], f"{what}: half of the rows differ by {np.median(err):.3e} and more"


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    base = tmp_path_factory.mktemp("kedesun")
    out = {}
    for name, (raw, seed) in km.CONFIGS.items():
        folder = str(base / name)
        raw, tensors = km.write_model(folder, raw, seed)
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
@pytest.mark.parametrize("name", list(km.CONFIGS))
def test_whole_prompt_then_token_by_token(models, name, dtype):
    folder, raw, tensors = models[name]
    tokens = tokens_of(raw["vocab"], 90, 1)
    want = plain.logits(raw, tensors, tokens)
    loaded = load(folder, dtype)
    whole = run_steps(loaded, [[("w", tokens)]])["w"]
    check(whole, want, dtype, f"{name} whole", routed=True)
    loaded.step.end("w")
    steps = [[("d", tokens[:37])]] + [[("d", [t])] for t in tokens[37:]]
    decoded = run_steps(loaded, steps)["d"]
    check(decoded, want, dtype, f"{name} prompt of 37 then token by token", routed=True)
    if dtype == "float32":       # how the prompt is cut changes nothing beyond rounding
        assert np.abs(decoded - whole).max() <= 1e-3 * np.abs(whole).max()


def test_the_stream_after_every_block(models):
    """The depth average's history holds every block's result; weighted, it is the plain model's stream."""
    folder, raw, tensors = models["mixed"]
    tokens = tokens_of(raw["vocab"], 40, 21)
    want = plain.streams(raw, tensors, tokens)
    loaded = load(folder, "float32")
    run_steps(loaded, [[("a", tokens)]])
    for index, layer in enumerate(loaded.model.layers):
        part = layer.parts["after"]
        history = part.history[:index + 2, :len(tokens)].cpu().numpy().astype(np.float64)
        stream = (history * part.weights.cpu().numpy().astype(np.float64)[:, None, None]).sum(0)
        assert np.abs(stream - want[index]).max() <= 2e-5 * np.abs(want[index]).max(), f"after block {index}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(km.CONFIGS))
def test_portions_of_several_sizes_down_to_two_tokens(models, name, dtype):
    folder, raw, tensors = models[name]
    tokens = tokens_of(raw["vocab"], 131, 2)
    want = plain.logits(raw, tensors, tokens)
    loaded = load(folder, dtype)
    for tag, sizes in (("a", [2, 3, 17, 2, 33]), ("b", [16, 16, 1, 15, 48]), ("c", [5, 2, 2, 64])):
        got = run_steps(loaded, [[(tag, part)] for part in cut(tokens, sizes)])[tag]
        check(got, want, dtype, f"{name} in portions of {sizes}", routed=True)
        loaded.step.end(tag)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(km.CONFIGS))
def test_batches_of_unequal_requests_equal_each_alone(models, name, dtype):
    folder, raw, tensors = models[name]
    requests = {"p": tokens_of(raw["vocab"], 70, 3), "q": tokens_of(raw["vocab"], 23, 4),
                "r": tokens_of(raw["vocab"], 120, 5), "s": tokens_of(raw["vocab"], 9, 6)}
    want = {key: plain.logits(raw, tensors, value) for key, value in requests.items()}
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
        check(got[key], want[key], dtype, f"{name} request {key} in a batch", routed=True)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pages_and_slots_are_used_again(models, dtype):
    """Two slots and a pool of 160 positions for six requests one after the other, two live at a time: every
    later request sits in a slot and in pages that an earlier one has left full of its own state."""
    folder, raw, tensors = models["mixed"]
    loaded = load(folder, dtype, max_requests=2, cache_tokens=160)
    lengths = [75, 60, 31, 80, 17, 66]
    for turn in range(3):
        pair = {f"x{2 * turn}": tokens_of(raw["vocab"], lengths[2 * turn], 20 + turn),
                f"y{2 * turn}": tokens_of(raw["vocab"], lengths[2 * turn + 1], 30 + turn)}
        (a, ta), (b, tb) = pair.items()
        steps = [[(a, ta[:20]), (b, tb[:3])], [(a, ta[20:21]), (b, tb[3:])], [(a, ta[21:])]]
        got = run_steps(loaded, steps)
        for key, tokens in pair.items():
            check(got[key], plain.logits(raw, tensors, tokens), dtype, f"turn {turn} request {key}", routed=True)
            loaded.step.end(key)
        loaded.manager.check_invariants()
    assert loaded.manager.free_slots == 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_long_portions_beside_short_ones(models, name, dtype):
    """Portions of hundreds of tokens (the retention scans them in segments, the experts' pairs are grouped) beside
    single tokens and short portions of other requests, from states and caches that earlier portions left."""
    folder, raw, tensors = models[name]
    long_one, short_one, other = tokens_of(raw["vocab"], 1100, 31), tokens_of(raw["vocab"], 140, 32), tokens_of(raw["vocab"], 400, 33)
    want = {"a": plain.logits(raw, tensors, long_one), "b": plain.logits(raw, tensors, short_one), "c": plain.logits(raw, tensors, other)}
    loaded = load(folder, dtype, cache_tokens=2048, max_batched_tokens=1024, max_context=2048)
    steps = [[("b", short_one[:1]), ("a", long_one[:449])], [("b", short_one[1:2]), ("a", long_one[449:450]), ("c", other[:385])],
             [("b", short_one[2:131]), ("a", long_one[450:1027]), ("c", other[385:])], [("b", short_one[131:]), ("a", long_one[1027:])]]
    got = run_steps(loaded, steps)
    for key in want:
        check(got[key], want[key], dtype, f"{name} request {key} in long portions", routed=True)


def test_long_decoding_from_the_first_token(models):
    folder, raw, tensors = models["mixed"]
    tokens = tokens_of(raw["vocab"], 200, 7)
    got = run_steps(load(folder, "float32"), [[("l", [t])] for t in tokens])["l"]
    check(got, plain.logits(raw, tensors, tokens), "float32", "200 tokens one by one")


# ------------------------------------------------------------------------- one mechanism, made to show
def one_layer_model(tmp_path, layer, seed, mlp=None, **weights):
    raw = km.single_layer(layer, mlp)
    folder = str(tmp_path / "one")
    raw, tensors = km.write_model(folder, raw, seed, **weights)
    return folder, raw, plain.as_float64(tensors)


def single_out(bf16, token, column, value=4.0):
    """Column ``column`` of the embedding table becomes zero for every token but ``token``: in a model of one layer
    that input dimension then speaks for this token alone."""
    import torch
    table = bf16["embed"].float().numpy().copy()
    table[:, column] = 0.0
    table[token, column] = value
    bf16["embed"] = torch.from_numpy(table).to(torch.bfloat16)


def set_column(bf16, name, rows, column, values):
    import torch
    matrix = bf16[name].float().numpy().copy()
    matrix[rows, column] = values
    bf16[name] = torch.from_numpy(matrix).to(torch.bfloat16)


def louder(bf16, name, factor):
    import torch
    bf16[name] = (bf16[name].float() * factor).to(torch.bfloat16)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes,far", [((2, 16, 8, 16, 24), 0), ((4, 8, 16, 8, 48), 15), ((3, 12, 4, 20, 12), 16),
                                       ((2, 16, 8, 16, 24), 17), ((20, 8, 8, 24, 24), 63), ((4, 32, 32, 16, 96), 271)])
def test_a_far_key_among_hundreds(tmp_path, sizes, far, dtype):
    """One latent-attention layer in which every head's query of ONE token (the probe's, through an input dimension
    that only this token has) points at the key that ONE other token makes, so that this score stands out among
    hundreds. That token sits at place ``far`` (the first position, the last of a page, the first of the next, the
    one after, deep inside, near the probe); whether it sits there moves the probe's logits, and the engine follows
    the plain model with the probe inside a prompt, as the first token of a portion, and decoded alone."""
    heads, dim, rot, vdim, rank = sizes
    raw = km.single_layer(km.latent(heads, dim, rot, vdim, rank, yarn=km.YARN))
    bf16 = km.make_tensors(raw, 40)
    vocab = raw["vocab"]
    key_token, probe_token, other_token = vocab - 1, vocab - 2, vocab - 3
    single_out(bf16, probe_token, 1)
    tensors = plain.as_float64(bf16)
    mixer = raw["layers"][0]["mixer"]
    h = plain.rms_norm(tensors["embed"], tensors["l0.norm1"], 1e-5)
    latent_of_key = plain.rms_norm((h[key_token] @ tensors["l0.mix.dkv"].T)[:rank], tensors["l0.mix.dkv.norm"], 1e-5)
    for head in range(heads):
        key = tensors["l0.mix.uk"][head * dim:(head + 1) * dim] @ latent_of_key
        size = np.linalg.norm(key)
        set_column(bf16, "l0.mix.q", slice(head * (dim + rot), head * (dim + rot) + dim), 1,
                   14.0 / (size * mixer["scale"] * h[probe_token][1]) * key / size)
    louder(bf16, "l0.mix.o", 8.0)
    folder = str(tmp_path / "one")
    km.write_model(folder, raw, 0, tensors=bf16)
    tensors = plain.as_float64(bf16)
    probe = 317
    changed = np.random.default_rng(8).integers(0, vocab - 3, size=330).tolist()
    changed[probe] = probe_token
    without = list(changed)
    changed[far], without[far] = key_token, other_token
    want, reference = plain.logits(raw, tensors, changed), plain.logits(raw, tensors, without)
    assert spread_error(want[probe:probe + 1], reference[probe:probe + 1])[0] > 0.2, "the plain model itself does not see the far key"
    loaded = load(folder, dtype)
    for tag, steps in (("prompt", [changed]), ("portion", [changed[:probe], changed[probe:]]),
                       ("decoded", [changed[:300]] + [[t] for t in changed[300:]])):
        got = run_steps(loaded, [[(tag, part)] for part in steps])[tag]
        check(got, want, dtype, f"far key at {far}, probe {tag}")
        assert spread_error(got[probe:probe + 1].astype(np.float64), reference[probe:probe + 1])[0] > 0.15
        loaded.step.end(tag)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_token_shows_through_the_retention_state(tmp_path, dtype):
    """One retention layer whose decays forget slowly, ONE token that writes a large value under its key, and ONE
    probe token whose query points at that key (each through an input dimension of its own): whether the writing
    token stood at place 3 moves the logits 250 tokens later; the engine follows the plain model whether the tokens
    between came as one prompt, in portions, or one by one."""
    raw = km.single_layer(km.retention(2, 16, 24, [0.9990234375, 1.0]))
    bf16 = km.make_tensors(raw, 42)
    vocab = raw["vocab"]
    key_token, probe_token, other_token = vocab - 1, vocab - 2, vocab - 3
    single_out(bf16, key_token, 0)
    single_out(bf16, probe_token, 1)
    tensors = plain.as_float64(bf16)
    h = plain.rms_norm(tensors["embed"], tensors["l0.norm1"], 1e-5)
    for head in range(2):
        key = (tensors["l0.mix.k"] @ h[key_token])[16 * head:16 * (head + 1)]
        set_column(bf16, "l0.mix.q", slice(16 * head, 16 * (head + 1)), 1, 10.0 * key / np.linalg.norm(key))
        value = (tensors["l0.mix.v"] @ h[key_token])[24 * head:24 * (head + 1)]
        set_column(bf16, "l0.mix.v", slice(24 * head, 24 * (head + 1)), 0, 30.0 * value / np.linalg.norm(value))
    louder(bf16, "l0.mix.o", 8.0)
    folder = str(tmp_path / "one")
    km.write_model(folder, raw, 0, tensors=bf16)
    tensors = plain.as_float64(bf16)
    changed = np.random.default_rng(10).integers(0, vocab - 3, size=256).tolist()
    changed[250] = changed[255] = probe_token
    without = list(changed)
    changed[3], without[3] = key_token, other_token
    want, reference = plain.logits(raw, tensors, changed), plain.logits(raw, tensors, without)
    assert spread_error(want[[250, 255]], reference[[250, 255]]).min() > 0.2, "the plain model itself forgot the far token"
    loaded = load(folder, dtype)
    for tag, steps in (("whole", [changed]), ("portions", cut(changed, [2, 70, 33, 16, 7])),
                       ("decoded", [changed[:6]] + [[t] for t in changed[6:]])):
        got = run_steps(loaded, [[(tag, part)] for part in steps])[tag]
        check(got, want, dtype, f"retention, {tag}")
        assert spread_error(got[[250, 255]].astype(np.float64), reference[[250, 255]]).min() > 0.15
        loaded.step.end(tag)


@pytest.mark.parametrize("dim,vdim", [(8, 5), (32, 32), (40, 70), (72, 16), (136, 24), (200, 8)])
def test_key_and_value_sizes_of_the_retention(tmp_path, dim, vdim):
    """One, two, four and eight lanes a column, value sizes that fill no warp evenly; a decay of exactly one."""
    folder, raw, tensors = one_layer_model(tmp_path, km.retention(2, dim, vdim, [0.75, 1.0]), 44)
    tokens = tokens_of(raw["vocab"], 45, 12)
    want = plain.logits(raw, tensors, tokens)
    got = run_steps(load(folder, "float32"), [[("a", tokens[:20])], [("a", tokens[20:21])], [("a", tokens[21:])]])["a"]
    check(got, want, "float32", f"retention with keys of {dim} and values of {vdim}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts,top,shared", [(4, 1, None), (8, 8, 16), (40, 3, 24), (64, 6, None), (3, 2, 8)])
def test_experts_choices_and_the_shared_expert(tmp_path, experts, top, shared, dtype):
    """One block whose feed-forward is a mixture: one choice, all experts chosen, more experts than a warp has
    lanes, with and without the gated shared expert; in steps of few tokens (the experts' rows stream) and of many
    (pairs grouped by expert), which must agree."""
    folder, raw, tensors = one_layer_model(tmp_path, km.retention(1, 8, 8), 45, mlp=km.moe(experts, top, 24, shared=shared))
    tokens = tokens_of(raw["vocab"], 150, 13)
    want = plain.logits(raw, tensors, tokens)
    loaded = load(folder, dtype)
    whole = run_steps(loaded, [[("w", tokens)]])["w"]
    check(whole, want, dtype, f"{experts} experts, {top} chosen, whole", routed=True)
    pieces = run_steps(loaded, [[("p", part)] for part in cut(tokens, [3, 16, 17, 1, 40])])["p"]
    check(pieces, want, dtype, f"{experts} experts, {top} chosen, portions", routed=True)


def test_the_correction_moves_the_choice_and_not_the_weights(tmp_path):
    """A correction that lifts two experts over all others: the engine chooses them, and weighs them by their
    uncorrected scores. Without it the output differs."""
    import torch
    raw = km.single_layer(km.retention(1, 8, 8), km.moe(6, 2, 16))
    bf16 = km.make_tensors(raw, 46)
    tokens = tokens_of(raw["vocab"], 30, 14)
    outputs = []
    for tag, correction in (("plain", [0.0] * 6), ("lifted", [0.0, 2.0, 0.0, 0.0, 3.0, 0.0])):
        bf16["l0.mlp.correction"] = torch.tensor(correction).to(torch.bfloat16)
        folder = str(tmp_path / tag)
        km.write_model(folder, raw, 0, tensors=bf16)
        tensors = plain.as_float64(bf16)
        want = plain.logits(raw, tensors, tokens)
        check(run_steps(load(folder, "float32"), [[("a", tokens)]])["a"], want, "float32", f"correction {tag}")
        outputs.append(want)
    h = plain.rms_norm(plain.as_float64(bf16)["embed"][tokens], plain.as_float64(bf16)["l0.norm1"], 1e-5)
    chosen, _ = plain.route(plain.as_float64(bf16), "l0.mlp.", raw["layers"][0]["mlp"], h)
    assert set(np.unique(chosen)) == {1, 4}
    assert np.median(spread_error(outputs[0], outputs[1])) > 0.01


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rotation_of_part_of_the_rotated_part_with_and_without_yarn(tmp_path, dtype):
    for tag, layer in (("part", km.latent(2, 8, 16, 8, 16, dims=6, base=30.0)),
                       ("yarn", km.latent(2, 8, 16, 8, 16, base=100.0, yarn={"factor": 16.0, "original": 32, "fast": 8.0, "slow": 0.5})),
                       ("all_slow", km.latent(2, 8, 4, 8, 16, base=10000.0, yarn={"factor": 4.0, "original": 8, "fast": 64.0, "slow": 32.0}))):
        raw = km.single_layer(layer, km.dense(32))
        folder = str(tmp_path / tag)
        raw, bf16 = km.write_model(folder, raw, 47, sharpen=1.5)
        tokens = tokens_of(raw["vocab"], 100, 15)
        want = plain.logits(raw, plain.as_float64(bf16), tokens)
        got = run_steps(load(folder, dtype), [[("a", tokens[:61])]] + [[("a", [t])] for t in tokens[61:]])["a"]
        check(got, want, dtype, f"rotation {tag}")


# ---------------------------------------------------------------------------- the engine's own entry point
@pytest.mark.parametrize("name", ["mixed", "wide"])
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
            logits = plain.logits(raw, tensors, sequence)[-1]
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
            logits = plain.logits(raw, tensors, sequence)[-1]
            top = np.sort(logits)[-2:]
            if top[1] - top[0] > 0.05 * (logits.max() - logits.min()):
                assert int(token) == int(np.argmax(logits))
            sequence.append(int(token))


def test_command_line_generates_and_dumps_logits(models, tmp_path, capsys):
    from celeg_b200.cli import main
    folder, raw, tensors = models["odd"]
    prompt = tokens_of(raw["vocab"], 12, 90)
    dump = str(tmp_path / "last.f32")
    code = main(["--model", folder, "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "6", "--dtype", "fp32",
                 "--temperature", "0", "--repetition-penalty", "1.0", "--runtime-tokens", "--dump-logits", dump,
                 "--context", "128"])
    assert code == 0
    captured = capsys.readouterr()
    sequence = list(prompt)
    for _ in range(6):
        sequence.append(int(np.argmax(plain.logits(raw, tensors, sequence)[-1])))
    assert f"CELEG_GENERATED_TOKEN_IDS=[{','.join(map(str, sequence[len(prompt):]))}]" in captured.out
    logits = np.fromfile(dump, dtype="<f4").astype(np.float64)
    assert spread_error(logits[None, :], plain.logits(raw, tensors, prompt)[-1:])[0] < 2e-4
    assert main(["--model", folder, "--print-config"]) == 0
    assert '"architecture": "Kedesun"' in capsys.readouterr().out


# ------------------------------------------------------------------------------- configurations drawn at random
def random_config(rng):
    width = int(rng.choice([20, 36, 64, 100, 128]))
    vocab = int(rng.integers(17, 300))
    layers = []
    for _ in range(int(rng.integers(1, 6))):
        if rng.random() < 0.5:
            rot = int(rng.choice([2, 4, 8, 16, 32]))
            dims = int(rng.choice([d for d in (2, rot // 2, rot) if d % 2 == 0 and 0 < d <= rot]))
            yarn = None if rng.random() < 0.4 else {"factor": float(rng.choice([2.0, 8.0, 40.0])), "original": int(rng.choice([16, 64, 4096])),
                                                     "fast": float(rng.choice([8.0, 32.0])), "slow": float(rng.choice([0.5, 1.0, 2.0]))}
            dim = int(rng.choice([4, 8, 12, 32, 64]))
            layer = km.latent(int(rng.choice([1, 2, 3, 4, 8, 16, 20])), dim, rot, int(rng.choice([4, 9, 16, 80])),
                              int(rng.choice([5, 8, 16, 24, 32, 56, 96, 224])), base=float(rng.choice([50.0, 10000.0, 1e6])),
                              dims=dims, yarn=yarn, scale=float(rng.choice([(dim + rot) ** -0.5, 0.125, 0.5])))
        else:
            heads = int(rng.integers(1, 5))
            layer = km.retention(heads, int(rng.choice([4, 8, 20, 32, 64, 130])), int(rng.choice([4, 9, 32, 80])),
                                 [float(rng.choice([0.5, 0.9, 0.96875, 0.999, 1.0])) for _ in range(heads)])
        pick = rng.random()
        if pick < 0.2:
            mlp = None
        elif pick < 0.55:
            mlp = km.dense(int(rng.choice([8, 44, 128])))
        else:
            experts = int(rng.choice([2, 3, 8, 16, 33, 70]))
            mlp = km.moe(experts, int(rng.integers(1, min(experts, 8) + 1)), int(rng.choice([8, 20, 64])),
                         shared=None if rng.random() < 0.4 else int(rng.choice([8, 36])))
        layers.append(km.with_mlp(layer, mlp))
    return km.config(vocab, width, layers, eps=float(rng.choice([1e-5, 1e-6, 1e-3])))


@pytest.mark.parametrize("seed", range(10))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Whole prompt, portions beside single tokens of a second request, and decoding, in both precisions."""
    rng = np.random.default_rng(2000 + seed)
    raw = random_config(rng)
    folder = str(tmp_path / "drawn")
    raw, bf16 = km.write_model(folder, raw, 600 + seed)
    tensors = plain.as_float64(bf16)
    first, second = tokens_of(raw["vocab"], 75, seed), tokens_of(raw["vocab"], 33, 100 + seed)
    want = {"a": plain.logits(raw, tensors, first), "b": plain.logits(raw, tensors, second)}
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
            for rows, target in ((whole, want["a"]), (got["a"], want["a"]), (got["b"], want["b"])):
                assert np.median(spread_error(np.asarray(rows, dtype=np.float64), target)) < 0.1
