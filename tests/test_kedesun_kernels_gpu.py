"""The kernels behind the Kedesun parts, each alone against a float64 restatement: the depth-weighted average with
and without the norm after it, the latent attention's token-parallel step and its per-head products, the attention
kernels with values read out of the keys, the retention scan and its decoding kernel, the router, the grouping of
pairs by expert, both forms of the experts' products, and the weighted sum."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_kedesun as plain
from test_kernels_gpu import close, dev, rounded

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,rows,blocks", [(36, 5, 3), (256, 7, 4), (1028, 3, 2), (2048, 4, 6), (5000, 2, 2)])
def test_depth_average_with_and_without_the_norm_after_it(dtype, width, rows, blocks):
    from celeg_b200 import kernels
    rng = np.random.default_rng(1)
    capacity = rows + 3
    history = torch.full((blocks + 1, capacity, width), 7.0, dtype=torch.float32, device="cuda")
    stream0 = rng.normal(size=(rows, width)).astype(np.float32)
    stream = dev(np.concatenate([stream0, np.zeros((3, width), np.float32)]))
    results = [stream0.astype(np.float64)]
    x = results[0]
    norm_w = rng.normal(1.0, 0.2, size=width).astype(np.float32)
    for index in range(blocks):
        da = rounded(rng.normal(size=(capacity, width)), dtype)
        db = rounded(rng.normal(size=(capacity, width)), dtype) if index % 2 == 0 else None
        weights = rng.normal(0.4, 0.5, size=index + 2).astype(np.float32)
        results.append(x + da[:rows] + (db[:rows] if db is not None else 0.0))
        x = plain.depth_average(results, weights.astype(np.float64))
        out = torch.zeros((capacity, width), dtype=dtype, device="cuda")
        with_norm = index % 3 != 1
        kernels.depth_average(stream, dev(da, dtype), None if db is None else dev(db, dtype), history, dev(weights), index,
                              rows, norm_weight=dev(norm_w) if with_norm else None, out=out if with_norm else None, eps=1e-5)
        close(stream[:rows], x, torch.float32, scale=np.abs(x).max())
        close(history[index + 1, :rows], results[-1], torch.float32, scale=4.0)
        if with_norm:
            close(out[:rows], plain.rms_norm(x, norm_w.astype(np.float64), 1e-5), dtype, scale=3.0)
        assert torch.all(stream[rows:] == 0) and torch.all(history[:, rows:] == 7.0)      # rows beyond the step stay
        x = stream[:rows].double().cpu().numpy()         # (go on from what the kernel left, rounding and all)
        results[-1] = history[index + 1, :rows].double().cpu().numpy()
    close(history[0, :rows], stream0.astype(np.float64), torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,rot,turned,rank,page", [(3, 8, 6, 4, 13, 8), (4, 32, 32, 32, 64, 16), (17, 4, 2, 2, 5, 32)])
def test_latent_prepare_writes_the_cache_and_the_rotated_queries(dtype, heads, dim, rot, turned, rank, page):
    from celeg_b200 import kernels
    rng = np.random.default_rng(2)
    rot_config = {"base": 100.0, "dims": turned, "scaling": {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}}
    freq, magnitude = plain.yarn_frequencies(rot_config)
    lengths, starts = [5, 1, 11], [3, 20, 0]                    # three requests: their portion and where it begins
    tokens = sum(lengths)
    positions = np.concatenate([np.arange(s, s + n) for s, n in zip(starts, lengths)]).astype(np.int32)
    token_span = np.concatenate([np.full(n, r) for r, n in enumerate(lengths)]).astype(np.int32)
    pages = 12
    table = np.full((3, 4), -1, dtype=np.int32)
    table[0, :1], table[1, :1 + 20 // page], table[2, :2] = [7], list(range(1, 2 + 20 // page)), [9, 4] if page <= 8 else [9, 10]
    q = rounded(rng.normal(size=(tokens, heads * (dim + rot))), dtype)
    down = rounded(rng.normal(size=(tokens, rank + rot)), dtype)
    norm_w = rng.normal(1.0, 0.3, size=rank).astype(np.float32)
    cache = torch.zeros((pages, 1, page, rank + rot), dtype=dtype, device="cuda")
    query = torch.zeros((tokens, heads * (rank + rot)), dtype=dtype, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    kernels.latent_prepare(dev(q, dtype), dev(down, dtype), dev(norm_w), dev(freq.astype(np.float32)), magnitude, 1e-6,
                           dev(positions), dev(token_span), dev(table), cache, page, query, tokens, heads, dim, rot, turned,
                           rank, flag)
    assert int(flag.item()) == 0
    want_latent = plain.rms_norm(down[:, :rank], norm_w.astype(np.float64), 1e-6)
    want_key = plain.rotate_interleaved(down[:, rank:], positions, rot_config)
    want_q = plain.rotate_interleaved(q.reshape(tokens, heads, dim + rot)[:, :, dim:], positions, rot_config)
    for t in range(tokens):
        place = cache[table[token_span[t], positions[t] // page], 0, positions[t] % page]
        close(place[:rank], want_latent[t], dtype, scale=2.0)
        close(place[rank:], want_key[t], dtype, scale=2.0)
    got_q = query.view(tokens, heads, rank + rot)
    close(got_q[:, :, rank:], want_q, dtype, scale=2.0)
    assert torch.all(got_q[:, :, :rank] == 0)                    # (the absorbed part is another kernel's)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,heads,n,k", [(1, 2, 5, 7), (70, 3, 64, 16), (130, 5, 100, 33), (9, 17, 24, 192)])
def test_head_project_in_both_orientations_with_the_gate(dtype, tokens, heads, n, k):
    from celeg_b200 import kernels
    rng = np.random.default_rng(3)
    pad = 3
    x = rounded(rng.normal(size=(tokens, heads * (k + pad))), dtype)
    gate = rounded(rng.normal(size=(tokens, heads)), dtype)
    xd = x.reshape(tokens, heads, k + pad)[:, :, :k]
    # the sum runs over the head's rows of the stored matrix
    stored = rounded(rng.normal(size=(heads * k, n)) / np.sqrt(k), dtype)
    out = torch.zeros((tokens, heads * (n + 2)), dtype=dtype, device="cuda")
    kernels.head_project(dev(x, dtype), k + pad, dev(stored, dtype), True, out, n + 2, tokens, heads, n, k)
    want = np.einsum("thk,hkn->thn", xd, stored.reshape(heads, k, n))
    close(out.view(tokens, heads, n + 2)[:, :, :n], want, dtype, scale=2.0)
    # the sum runs over its columns, and the head's gate multiplies
    stored = rounded(rng.normal(size=(heads * n, k)) / np.sqrt(k), dtype)
    out = torch.zeros((tokens, heads * n), dtype=dtype, device="cuda")
    kernels.head_project(dev(x, dtype), k + pad, dev(stored, dtype), False, out, n, tokens, heads, n, k, gate=dev(gate, dtype))
    want = np.einsum("thk,hnk->thn", xd, stored.reshape(heads, n, k)) * plain.sigmoid(gate)[:, :, None]
    close(out.view(tokens, heads, n), want, dtype, scale=2.0)


def latent_attention_reference(query, cache_rows, rank, scale):
    """query [heads, rank + rot] at the last position of cache_rows [keys, rank + rot]: softmax(q . k) over all keys,
    weighted sum of the keys' first ``rank`` elements."""
    scores = query @ cache_rows.T * scale
    p = np.exp(scores - scores.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    return p @ cache_rows[:, :rank]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,rank,rot,page", [(4, 24, 8, 16), (16, 192, 64, 16), (2, 48, 16, 16), (20, 13, 6, 8), (8, 56, 8, 32)])
def test_attention_kernels_with_values_read_out_of_the_keys(dtype, heads, rank, rot, page):
    """What the latent-attention mixer asks of the paged attention: one key head of rank + rot for all query heads,
    the value cache being the key cache. Portions, single tokens, and single tokens before portions."""
    from celeg_b200.parts.mixers import PagedAttentionKernels, PagedBinding
    from celeg_b200.parts import Runtime, StepContext
    rng = np.random.default_rng(4)
    width = rank + rot
    contexts, news = [300, 17, 64, 129], [1, 1, 40, 129]       # keys each request holds after the step; its new tokens
    requests, tokens = len(contexts), sum(news)
    pages = sum(-(-c // page) for c in contexts) + 2
    order = rng.permutation(pages)
    cache = torch.zeros((pages, 1, page, width), dtype=dtype, device="cuda")
    table = np.full((requests, max(-(-c // page) for c in contexts)), -1, dtype=np.int32)
    rows, used = [], 0
    for r, c in enumerate(contexts):
        keys = rounded(rng.normal(size=(c, width)), dtype)
        rows.append(keys)
        for p in range(-(-c // page)):
            table[r, p] = order[used]
            lo, hi = p * page, min(c, (p + 1) * page)
            cache[order[used], 0, :hi - lo] = dev(keys[lo:hi], dtype)
            used += 1
    queries = rounded(rng.normal(size=(tokens, heads * width)), dtype)
    positions = np.concatenate([np.arange(c - n, c) for c, n in zip(contexts, news)]).astype(np.int32)
    span_begin = np.concatenate([[0], np.cumsum(news)]).astype(np.int32)
    token_span = np.concatenate([np.full(n, r) for r, n in enumerate(news)]).astype(np.int32)

    class Probe(PagedAttentionKernels):
        pass

    rt = Runtime(torch.device("cuda:0"), dtype, 512, max_requests=8, max_context=512)
    probe = Probe()
    probe.rt, probe.heads, probe.kv_heads, probe.head_dim = rt, heads, 1, width
    probe.window, probe.scale, probe.sinks, probe._resident_blocks = None, 0.3, None, None
    probe.binding = PagedBinding(group=0, k=cache, v=cache[..., :0], page_tokens=page)
    probe._value_cache = lambda: cache
    probe.qkv, probe.qkv_width = dev(queries, dtype), heads * width
    probe.attended = torch.zeros((tokens, heads * width), dtype=dtype, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    step = StepContext(tokens=tokens, spans=requests, token_ids=dev(np.zeros(tokens, np.int32)), positions=dev(positions),
                       token_span=dev(token_span), span_begin=dev(span_begin), span_slot=dev(np.arange(requests, dtype=np.int32)),
                       block_tables=[dev(table)], error_flag=flag, max_span=max(news), max_context=max(contexts),
                       context_bucket=512, host_span_lengths=list(news), leading_single_tokens=2)
    probe.attend(step, step.block_tables[0])
    assert int(flag.item()) == 0
    got = probe.attended.view(tokens, heads, width)[:, :, :rank]
    t = 0
    for r, (c, n) in enumerate(zip(contexts, news)):
        for i in range(n):
            seen = rows[r][:c - n + i + 1]
            want = latent_attention_reference(queries[t].reshape(heads, width), seen, rank, 0.3)
            close(got[t], want, dtype, scale=1.0)
            t += 1


@pytest.mark.parametrize("dim,vdim,heads", [(8, 5, 3), (16, 24, 2), (64, 32, 2), (40, 70, 1), (136, 24, 2)])
def test_retention_scan_and_decoding_kernel(dim, vdim, heads):
    """Spans of unequal length from states that earlier tokens left, then one token each through the decoding kernel;
    a slot stride wider than the state; a decay of one."""
    from celeg_b200 import kernels
    rng = np.random.default_rng(5)
    lengths, slots = [9, 1, 40], [2, 0, 3]
    tokens, spans = sum(lengths), len(lengths)
    decay = np.array(([1.0, 0.9, 0.96875] * 2)[:heads], dtype=np.float32)
    elements = heads * dim * vdim
    stride = (elements + 7) // 4 * 4 + 8
    state0 = rng.normal(size=(5, stride)).astype(np.float32)
    state = dev(state0)
    width = heads * (2 * dim + 2 * vdim)
    proj = rng.normal(size=(tokens, width)).astype(np.float32)
    q_off, k_off, v_off, g_off = 0, heads * dim, 2 * heads * dim, 2 * heads * dim + heads * vdim
    rows = dev(proj)
    span_begin = dev(np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32))
    span_slot = dev(np.array(slots, dtype=np.int32))
    read = torch.zeros((tokens, heads * vdim), dtype=torch.float32, device="cuda")
    kernels.recurrent_scan(kernels.SCAN_RETENTION, rows[:, q_off:k_off], rows[:, k_off:v_off], rows[:, v_off:g_off], dev(decay),
                           read, state, stride, span_begin, span_slot, spans, heads, heads, dim, vdim, dim ** -0.5)
    gated = torch.zeros((tokens, heads * vdim), dtype=torch.float32, device="cuda")
    kernels.gated_head_norm(read, rows[:, g_off:], None, False, gated, tokens, heads, vdim, 1e-5, kernels.GATE_SILU)
    states = {slot: state0[slot, :elements].astype(np.float64).reshape(heads, dim, vdim).copy() for slot in slots}
    t = 0
    p64 = proj.astype(np.float64)

    def one_token(slot, row):
        out = np.zeros((heads, vdim))
        for h in range(heads):
            q, k = row[q_off + h * dim:q_off + (h + 1) * dim], row[k_off + h * dim:k_off + (h + 1) * dim] * dim ** -0.5
            v = row[v_off + h * vdim:v_off + (h + 1) * vdim]
            states[slot][h] = float(decay[h]) * states[slot][h] + np.outer(k, v)
            out[h] = states[slot][h].T @ q
        return out

    for slot, n in zip(slots, lengths):
        for _ in range(n):
            out = one_token(slot, p64[t])
            close(read[t], out.reshape(-1), torch.float32, scale=np.abs(out).max())
            want = plain.rms_scaled(out, 1e-5).reshape(-1) * plain.silu(p64[t, g_off:])
            close(gated[t], want, torch.float32, scale=3.0)
            t += 1
    for slot in slots:
        close(state[slot, :elements], states[slot].reshape(-1), torch.float32, scale=np.abs(states[slot]).max())
    assert torch.equal(state[:, elements:], dev(state0)[:, elements:]) and torch.equal(state[1], dev(state0)[1])
    # one token a request through the decoding kernel
    for dtype in DTYPES:
        before = {slot: states[slot].copy() for slot in slots}
        held = state.clone()
        step_rows = rng.normal(size=(spans, width)).astype(np.float32)
        out = torch.zeros((spans, heads * vdim), dtype=dtype, device="cuda")
        kernels.recurrent_decode(kernels.SCAN_RETENTION, dev(step_rows), (q_off, k_off, v_off, g_off, 0, 0), None, None, 0, 0,
                                 dev(decay), dev(decay), 0.0, None, False, 1e-5, 0.0, held, stride,
                                 dev(np.arange(spans + 1, dtype=np.int32)), span_slot, spans, heads, heads, dim, vdim,
                                 dim ** -0.5, out)
        for i, slot in enumerate(slots):
            read_out = one_token(slot, step_rows[i].astype(np.float64))
            want = plain.rms_scaled(read_out, 1e-5).reshape(-1) * plain.silu(step_rows[i, g_off:].astype(np.float64))
            close(out[i], want, dtype, scale=3.0)
            close(held[slot, :elements], states[slot].reshape(-1), torch.float32, scale=np.abs(states[slot]).max())
        states.update(before)


@pytest.mark.parametrize("dim,vdim,heads,segment", [(16, 24, 2, 64), (64, 128, 3, 128), (40, 7, 1, 128), (136, 70, 2, 192)])
def test_retention_in_segments_equals_the_token_by_token_scan(dim, vdim, heads, segment):
    """Spans of unequal length (shorter than a segment, exactly one, one token more, several) from states that earlier
    tokens left: read-outs and final states as the plain scan's, and the slots' other floats untouched."""
    from celeg_b200 import kernels
    rng = np.random.default_rng(8)
    lengths = [segment * 3 + 17, 1, segment, segment + 1, 5, 2 * segment]
    slots = [4, 0, 2, 5, 1, 3]
    tokens, spans = sum(lengths), len(lengths)
    decay = dev(np.array(([1.0, 0.9, 0.99951171875] * 2)[:heads], dtype=np.float32))
    elements = heads * dim * vdim
    stride = (elements + 3) // 4 * 4 + 12
    state0 = dev(rng.normal(size=(7, stride)).astype(np.float32))
    proj = dev(rng.normal(size=(tokens, heads * (2 * dim + vdim))).astype(np.float32))
    q, k, v = proj[:, :heads * dim], proj[:, heads * dim:2 * heads * dim], proj[:, 2 * heads * dim:]
    span_begin = dev(np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32))
    span_slot = dev(np.array(slots, dtype=np.int32))
    want_state, want = state0.clone(), torch.zeros((tokens, heads * vdim), dtype=torch.float32, device="cuda")
    kernels.recurrent_scan(kernels.SCAN_RETENTION, q, k, v, decay, want, want_state, stride, span_begin, span_slot, spans,
                           heads, heads, dim, vdim, dim ** -0.5)
    segments = tokens // segment + spans
    got_state, got = state0.clone(), torch.full((tokens, heads * vdim), 9.0, dtype=torch.float32, device="cuda")
    floats = torch.full((2 * segments * elements,), 5.0, dtype=torch.float32, device="cuda")
    ints = torch.zeros(segments + spans + 2, dtype=torch.int32, device="cuda")
    kernels.retention_segmented(q, k, v, decay, got, got_state, stride, span_begin, span_slot, spans, tokens, heads, dim, vdim,
                                dim ** -0.5, segment, segments, floats, ints, torch.arange(segments, dtype=torch.int32, device="cuda"))
    scale = float(want.abs().max())
    assert float((got - want).abs().max()) <= 2e-5 * scale
    assert float((got_state - want_state).abs().max()) <= 2e-5 * float(want_state.abs().max())
    assert torch.equal(got_state[:, elements:], state0[:, elements:]) and torch.equal(got_state[6], state0[6])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,top,width,tokens", [(4, 1, 36, 9), (16, 3, 256, 70), (40, 8, 100, 33), (70, 70, 64, 5)])
def test_router_chooses_by_corrected_scores(dtype, experts, top, width, tokens):
    from celeg_b200 import kernels
    from celeg_b200.parts import Runtime
    rng = np.random.default_rng(6)
    h = rounded(rng.normal(size=(tokens, width)), dtype)
    router = rounded(rng.normal(size=(experts, width)) * 3.0 / np.sqrt(width), torch.bfloat16)
    correction = rounded(rng.normal(size=experts) / experts, torch.bfloat16)
    gate_w = rounded(rng.normal(size=width) / np.sqrt(width), torch.bfloat16)
    chosen = torch.zeros((tokens, top), dtype=torch.int32, device="cuda")
    weights = torch.zeros((tokens, top), dtype=torch.float32, device="cuda")
    shared = torch.zeros(tokens, dtype=torch.float32, device="cuda")
    # the logits as the engine makes them: one product with float32 sums, the gate's row after the experts'
    rt = Runtime(torch.device("cuda:0"), dtype, 128, max_requests=4, max_context=128)
    logits = torch.zeros((128, experts + 1), dtype=torch.float32, device="cuda")
    rt.linear(dev(np.concatenate([h, np.zeros((128 - tokens, width))]), dtype), dev(np.concatenate([router, gate_w[None, :]]), dtype),
              logits, tokens)
    kernels.moe_route(logits, experts, dev(correction, torch.float32), experts, chosen, weights, shared, tokens, top)
    tensors = {"m.router": router, "m.correction": correction}
    want_chosen, want_weights = plain.route(tensors, "m.", {"router": {"top": top}}, h)
    logits = h @ router.T
    scores = np.exp(logits - logits.max(-1, keepdims=True))
    scores /= scores.sum(-1, keepdims=True)
    choice = np.sort(scores + correction, axis=-1)[:, ::-1]
    clear = np.ones(tokens, dtype=bool) if top == experts else (choice[:, top - 1] - choice[:, top]) > 1e-5
    assert clear.sum() >= tokens - 2
    got_chosen, got_weights = chosen.cpu().numpy(), weights.double().cpu().numpy()
    for t in np.nonzero(clear)[0]:
        assert set(got_chosen[t]) == set(want_chosen[t]), f"token {t}"
        by_expert = dict(zip(want_chosen[t], want_weights[t]))
        assert np.allclose([by_expert[e] for e in got_chosen[t]], got_weights[t], rtol=2e-4, atol=1e-7)
        assert abs(got_weights[t].sum() - 1.0) < 1e-5
    close(shared, plain.sigmoid(h @ gate_w), torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,top,width,inner,tokens", [(4, 2, 40, 24, 7), (16, 3, 256, 64, 200), (5, 5, 36, 20, 70),
                                                             (40, 1, 64, 72, 130), (3, 2, 100, 33, 90), (8, 2, 512, 384, 700),
                                                             (32, 4, 512, 768, 2048)])
def test_experts_products_grouped_and_row_by_row(dtype, experts, top, width, inner, tokens):
    """The forms of the experts' two products (tile by tile over the pairs grouped by expert, on tcgen05 where the
    shapes allow, and row by row) against the plain mixture, and against each other."""
    from celeg_b200 import kernels
    rng = np.random.default_rng(7)
    h = rounded(rng.normal(size=(tokens, width)), dtype)
    up = rounded(rng.normal(size=(experts, inner, width)) / np.sqrt(width), dtype)
    down = rounded(rng.normal(size=(experts, width, inner)) / np.sqrt(inner), dtype)
    chosen_np = np.stack([rng.permutation(experts)[:top] for _ in range(tokens)]).astype(np.int32)
    if experts > 8:
        chosen_np[:, 0] = np.where(rng.random(tokens) < 0.7, 3, chosen_np[:, 0])      # one expert far busier than the rest
        for t in range(tokens):                                                       # (a token names an expert once)
            if top > 1 and chosen_np[t, 0] in chosen_np[t, 1:]:
                chosen_np[t, 0] = next(e for e in range(experts) if e not in chosen_np[t, 1:])
    weights_np = rng.random(size=(tokens, top)).astype(np.float32)
    shared_np = rounded(rng.normal(size=(tokens, width)), dtype)
    gate_np = rng.random(size=tokens).astype(np.float32)
    want = np.zeros((tokens, width))
    for t in range(tokens):
        for e, w in zip(chosen_np[t], weights_np[t]):
            want[t] += float(w) * (plain.squared_relu(h[t] @ up[e].T) @ down[e].T)
        want[t] += float(gate_np[t]) * shared_np[t]
    pairs = tokens * top
    chosen, weights = dev(chosen_np.reshape(-1)), dev(weights_np.reshape(-1))
    x, w_up, w_down = dev(h, dtype), dev(up, dtype), dev(down, dtype)
    results = []
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    for form in ("grouped", "tcgen05", "rows"):
        if form == "rows" and pairs > 1000:
            continue
        # (spare rows after the step's pairs, full of what an earlier step left: no tile may take them for its own)
        raised = torch.full((pairs + 200, inner), 3.0, dtype=dtype, device="cuda")
        lowered = torch.full((pairs + 200, width), 3.0, dtype=dtype, device="cuda")
        y = torch.zeros((tokens, width), dtype=dtype, device="cuda")
        if form == "tcgen05":
            gathered = torch.full((pairs + 200, width), 3.0, dtype=dtype, device="cuda")
            if not (kernels.expert_product_tcgen05_supported(gathered, w_up) and kernels.expert_product_tcgen05_supported(raised, w_down)):
                continue
        if form != "rows":
            tile_rows = 128 if form == "tcgen05" else kernels.MOE_TILE
            place = torch.zeros(pairs, dtype=torch.int32, device="cuda")
            source = torch.zeros(pairs, dtype=torch.int32, device="cuda")
            tiles = kernels.moe_max_tiles(pairs, experts, tile_rows)
            table = torch.zeros(4 + 3 * tiles, dtype=torch.int32, device="cuda")
            kernels.moe_group(chosen, tokens, experts, top, place, source, table, tile_rows=tile_rows)
            places = place.cpu().numpy()
            assert sorted(places.tolist()) == list(range(pairs))
            assert np.array_equal(source.cpu().numpy()[places], np.arange(pairs) // top)
            assert np.all(np.diff(chosen_np.reshape(-1)[np.argsort(places)]) >= 0)         # places are ordered by expert
            listed = table.cpu().numpy()
            assert listed[0] <= tiles and listed[4 + 2:4 + 3 * listed[0]:3].sum() == pairs
            if form == "tcgen05":
                kernels.moe_gather_rows(x, source, gathered, pairs)
                assert torch.equal(gathered[:pairs], x[source.long()])
                kernels.expert_product_tcgen05(gathered, w_up, raised, table, tiles, kernels.ACT_RELU_SQUARED, flag)
                kernels.expert_product_tcgen05(raised, w_down, lowered, table, tiles, -1, flag)
                assert int(flag.item()) == 0
            else:
                kernels.expert_product(x, source, w_up, raised, table, tiles, kernels.ACT_RELU_SQUARED)
                kernels.expert_product(raised, None, w_down, lowered, table, tiles, -1)
            assert torch.all(raised[pairs:] == 3.0) and torch.all(lowered[pairs:] == 3.0)
            kernels.moe_combine(lowered, place, weights, dev(shared_np, dtype), dev(gate_np), y, tokens, top)
        else:
            kernels.expert_rows(x, top, chosen, w_up, raised, pairs, kernels.ACT_RELU_SQUARED)
            kernels.expert_rows(raised, 1, chosen, w_down, lowered, pairs, -1)
            kernels.moe_combine(lowered, None, weights, dev(shared_np, dtype), dev(gate_np), y, tokens, top)
        close(y, want, dtype, scale=np.abs(want).max())
        results.append(y)
    if len(results) >= 2 and dtype == torch.float32:
        assert (results[0] - results[-1]).abs().max() <= 1e-5 * results[0].abs().max()
