"""The kernels behind the Ramosun parts, each alone against a float64 restatement: Dynamic Tanh with one and
two outputs and two deltas, activations, capped logits, the stream joined with embedding rows, sinks in the three
attention kernels, the norm over the whole q/k projection with values that are the keys, the mLSTM and
delta-rule scans with their token-parallel parts, and the gated per-head norm."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_ramosun as plain
from test_kernels_gpu import close, dev, paged_setup, rounded

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,rows", [(40, 5), (257, 3), (1024, 9)])
def test_dynamic_tanh_adds_two_deltas_and_writes_two_norms(dtype, width, rows):
    from celeg_b200 import kernels
    rng = np.random.default_rng(1)
    residual = rng.normal(size=(rows, width)).astype(np.float32)
    da, db = rounded(rng.normal(size=(rows, width)), dtype), rounded(rng.normal(size=(rows, width)), dtype)
    w1, b1, w2, b2 = (rng.normal(size=width).astype(np.float32) for _ in range(4))
    res = dev(residual)
    out1 = torch.zeros((rows, width), dtype=dtype, device="cuda")
    out2 = torch.zeros_like(out1)
    kernels.add_dyt(res, dev(da, dtype), dev(db, dtype), rows, (dev(w1), dev(b1), 0.7, out1), (dev(w2), dev(b2), 1.3, out2))
    x = residual.astype(np.float64) + da + db
    close(res, x, torch.float32)
    close(out1, plain.dynamic_tanh(x, w1, b1, 0.7), dtype)
    close(out2, plain.dynamic_tanh(x, w2, b2, 1.3), dtype)
    # gathered rows: the residual stays, one output, one delta
    picked = np.array([rows - 1, 0], dtype=np.int32)
    before = res.clone()
    out = torch.zeros((2, width), dtype=dtype, device="cuda")
    kernels.add_dyt(res, dev(da, dtype), None, 2, (dev(w1), dev(b1), 0.5, out), rows=dev(picked))
    assert torch.equal(res, before)
    close(out, plain.dynamic_tanh((x + da)[picked], w1, b1, 0.5), dtype)
    kernels.add_to_residual(res, None, dev(db, dtype), rows)
    close(res, x + db, torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
def test_activations_and_capped_logits(dtype):
    from celeg_b200 import kernels
    x = rounded(np.linspace(-9.0, 9.0, 7 * 130).reshape(7, 130), dtype)
    for kind, fn in ((kernels.ACT_GELU_ERF, plain.gelu_erf), (kernels.ACT_SILU, plain.silu),
                     (kernels.ACT_GELU_TANH, lambda z: 0.5 * z * (1 + np.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3))))):
        out = torch.zeros((7, 130), dtype=dtype, device="cuda")
        kernels.activation(dev(x, dtype), out, 7, kind)
        close(out, fn(x), dtype)
    logits = dev(np.linspace(-80.0, 80.0, 3 * 50).reshape(3, 50).astype(np.float32))
    want = 15.0 * np.tanh(logits.cpu().numpy().astype(np.float64) / 15.0)
    kernels.softcap(logits, 2, 15.0)
    close(logits[:2], want[:2], torch.float32)
    assert float(logits[2].abs().max()) > 15.0          # the row past the count is left alone


@pytest.mark.parametrize("dtype", DTYPES)
def test_stream_joined_with_embedding_rows(dtype):
    from celeg_b200 import kernels
    rng = np.random.default_rng(2)
    width, vocab, rows = 72, 31, 6
    residual = rng.normal(size=(rows, width)).astype(np.float32)
    da, db = rounded(rng.normal(size=(rows, width)), dtype), rounded(rng.normal(size=(rows, width)), dtype)
    table = rounded(rng.normal(size=(vocab, width)), dtype)
    tokens = rng.integers(0, vocab, size=rows).astype(np.int32)
    joined = torch.zeros((rows, 2 * width), dtype=dtype, device="cuda")
    kernels.join_stream_embedding(dev(residual), dev(da, dtype), dev(db, dtype), dev(table, dtype), dev(tokens), joined, rows)
    close(joined, np.concatenate([residual + da + db, table[tokens]], axis=1), dtype)


def sink_reference(q, k, v, pos, scale, window, sinks):
    heads, kv_heads = q.shape[0], k.shape[1]
    out = np.zeros_like(q)
    first = max(0, pos - window + 1) if window else 0
    for h in range(heads):
        kh = h // (heads // kv_heads)
        s = (k[first:pos + 1, kh] @ q[h]) * scale
        top = max(s.max(), sinks[h])
        w = np.exp(s - top)
        out[h] = (w @ v[first:pos + 1, kh]) / (w.sum() + math.exp(sinks[h] - top))
    return out


@pytest.mark.parametrize("heads,kv_heads,head_dim,page_tokens,window", [
    (4, 2, 16, 16, None), (6, 2, 96, 16, 70), (6, 3, 80, 16, 37), (3, 1, 64, 8, 9), (4, 1, 40, 16, 130), (8, 2, 64, 16, 200), (4, 4, 64, 32, None)])
def test_sinks_in_the_attention_kernels(heads, kv_heads, head_dim, page_tokens, window):
    """The general kernel (both types), the tensor-core kernels for portions (mma.sync; tcgen05 at head size 64) and
    the split-key kernel for single tokens (several splits) with a sink per head: large, small, and in between."""
    from celeg_b200 import kernels
    rng = np.random.default_rng(3)
    sinks = np.linspace(-6.0, 5.0, heads).astype(np.float32)
    lengths = [150, 301, 40, 1, 333]
    span_len = [70, 1, 2, 1, 150]
    scale = head_dim ** -0.5
    for dtype in DTYPES:
        pages = sum((n + page_tokens - 1) // page_tokens for n in lengths) + 5
        k_cache, v_cache, table, ks, vs = paged_setup(rng, dtype, lengths, kv_heads, head_dim, page_tokens, pages)
        tokens = sum(span_len)
        q = rounded(rng.normal(size=(tokens, heads, head_dim)) * 2.0, dtype)
        positions, token_span, begins = [], [], [0]
        for r, (n, m) in enumerate(zip(lengths, span_len)):
            positions += list(range(n - m, n))
            token_span += [r] * m
            begins.append(begins[-1] + m)
        want = np.stack([sink_reference(q[t], ks[token_span[t]], vs[token_span[t]], positions[t], scale, window, sinks)
                         for t in range(tokens)]).reshape(tokens, -1)
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        args = (dev(np.array(positions, dtype=np.int32)),)
        out = torch.zeros((tokens, heads * head_dim), dtype=dtype, device="cuda")
        kernels.attention_generic(dev(q.reshape(tokens, -1), dtype), heads * head_dim, out, k_cache, v_cache, args[0],
                                  dev(np.array(token_span, dtype=np.int32)), dev(table), tokens, heads, kv_heads,
                                  head_dim, page_tokens, window, scale, flag, sinks=dev(sinks))
        close(out, want, dtype)
        if dtype == torch.bfloat16:
            out = torch.zeros_like(out)
            kernels.attention_prefill(dev(q.reshape(tokens, -1), dtype), heads * head_dim, out, k_cache, v_cache, args[0],
                                      dev(np.array(begins, dtype=np.int32)), dev(table), tokens, len(lengths), heads,
                                      kv_heads, head_dim, page_tokens, window, scale, flag, sinks=dev(sinks))
            close(out, want, dtype, scale=1.5)
            if kernels.attention_prefill_tcgen05_supported(heads, kv_heads, head_dim, page_tokens, dtype):
                out = torch.zeros_like(out)
                tiles = sum((m + 127) // 128 for m in span_len)
                kernels.attention_prefill_tcgen05(dev(q.reshape(tokens, -1), dtype), heads * head_dim, out, k_cache, v_cache,
                                                  args[0], dev(np.array(begins, dtype=np.int32)), dev(table), tokens,
                                                  len(lengths), tiles, heads, kv_heads, head_dim, page_tokens, window,
                                                  scale, flag, sinks=dev(sinks))
                close(out, want, dtype, scale=1.5)
            # single tokens: the last token of every request, keys in chunks of 64 (up to six splits)
            last = [b - 1 for b in begins[1:]]
            single_q = dev(q[last].reshape(len(last), -1), dtype)
            max_splits = 8
            partial_o = torch.empty(len(last) * heads * max_splits * head_dim, dtype=torch.float32, device="cuda")
            partial_ml = torch.empty(len(last) * heads * max_splits * 2, dtype=torch.float32, device="cuda")
            counters = torch.zeros(len(last) * kv_heads, dtype=torch.int32, device="cuda")
            out = torch.zeros((len(last), heads * head_dim), dtype=dtype, device="cuda")
            kernels.attention_decode(single_q, heads * head_dim, out, k_cache, v_cache,
                                     dev(np.array([positions[t] for t in last], dtype=np.int32)),
                                     dev(np.arange(len(last), dtype=np.int32)), dev(table), len(last), heads, kv_heads,
                                     head_dim, page_tokens, window, scale, 64, max_splits, partial_o, partial_ml,
                                     counters, flag, sinks=dev(sinks))
            close(out, want[last], dtype, scale=1.5)
        assert int(flag.item()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim,rotary,page_tokens", [(4, 2, 16, 16, 16), (5, 5, 96, 48, 16),
                                                                       (3, 1, 40, 12, 8), (2, 2, 24, 0, 16)])
def test_norm_over_the_whole_projection_and_values_that_are_keys(dtype, heads, kv_heads, head_dim, rotary, page_tokens):
    from celeg_b200 import kernels
    rng = np.random.default_rng(4)
    tokens, eps = 37, 1e-5
    q_width, k_width = heads * head_dim, kv_heads * head_dim
    rows = rounded(rng.normal(size=(tokens, q_width + k_width)) * 3.0, dtype)
    wq, wk = rng.normal(1.0, 0.2, size=q_width).astype(np.float32), rng.normal(1.0, 0.2, size=k_width).astype(np.float32)
    rot = {"base": 100.0, "dims": rotary} if rotary else None
    freq = plain.rotary_frequencies(rot).astype(np.float32) if rot else None
    start = 11                                            # the span begins in the middle of a page
    positions = np.arange(start, start + tokens, dtype=np.int32)
    pages = (start + tokens + page_tokens - 1) // page_tokens
    table = np.arange(pages, dtype=np.int32)[::-1].copy()[None, :]
    k_cache = torch.zeros((pages, kv_heads, page_tokens, head_dim), dtype=dtype, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    qk = dev(rows, dtype)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    scales = torch.zeros(2 * tokens, dtype=torch.float32, device="cuda")
    kernels.qk_whole_norm_rope_store(qk, dev(wq), dev(wk), dev(freq) if rot else None, dev(positions),
                                     dev(np.zeros(tokens, dtype=np.int32)), dev(table), k_cache, v_cache, tokens, heads,
                                     kv_heads, head_dim, rotary, page_tokens, eps, True, scales, flag)
    assert int(flag.item()) == 0
    q = plain.root_mean_square_scaled(rows[:, :q_width], eps) * wq
    k = plain.root_mean_square_scaled(rows[:, q_width:], eps) * wk
    q, k = q.reshape(tokens, heads, head_dim), k.reshape(tokens, kv_heads, head_dim)
    if rot:
        q = plain.rotate_half_layout(q, positions, freq.astype(np.float64), rotary)
        k = plain.rotate_half_layout(k, positions, freq.astype(np.float64), rotary)
    close(qk[:, :q_width], q.reshape(tokens, -1), dtype, scale=3.0)
    got_k = torch.stack([k_cache[int(table[0, p // page_tokens]), :, p % page_tokens] for p in positions])
    got_v = torch.stack([v_cache[int(table[0, p // page_tokens]), :, p % page_tokens] for p in positions])
    close(got_k, k, dtype, scale=3.0)
    close(got_v, rows[:, q_width:].reshape(tokens, kv_heads, head_dim), dtype)      # the key as projected


def scan_inputs(rng, tokens, heads, kv_heads, dim, vdim):
    q = rng.normal(size=(tokens, kv_heads, dim)).astype(np.float32)
    k = rng.normal(size=(tokens, kv_heads, dim)).astype(np.float32)
    v = rng.normal(size=(tokens, heads, vdim)).astype(np.float32)
    return q, k, v


@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(2, 1, 16, 24), (3, 3, 40, 5), (2, 2, 96, 33), (1, 1, 200, 9)])
def test_delta_rule_scan_over_spans_with_carried_state(heads, kv_heads, dim, vdim):
    """Three spans (one of a single token, one longer than the staging tile) in slots 2, 0, 1 that hold state;
    a fourth slot must stay as it was."""
    from celeg_b200 import kernels
    rng = np.random.default_rng(5)
    lengths, slots = [37, 1, 18], [2, 0, 1]
    tokens = sum(lengths)
    q, k, v = scan_inputs(rng, tokens, heads, kv_heads, dim, vdim)
    k /= np.linalg.norm(k, axis=-1, keepdims=True)
    q /= np.linalg.norm(q, axis=-1, keepdims=True)
    gates = np.concatenate([rng.uniform(0.1, 0.9, size=(tokens, heads)), rng.uniform(0.7, 1.0, size=(tokens, heads))],
                           axis=1).astype(np.float32)
    elements = heads * dim * vdim
    stride = elements + 12
    state = rng.normal(size=(4, stride)).astype(np.float32)
    state_dev = dev(state)
    out = torch.zeros((tokens, heads * vdim), dtype=torch.float32, device="cuda")
    begins = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    kernels.recurrent_scan(kernels.SCAN_DELTA, dev(q.reshape(tokens, -1)), dev(k.reshape(tokens, -1)),
                           dev(v.reshape(tokens, -1)), dev(gates), out, state_dev, stride, dev(begins),
                           dev(np.array(slots, dtype=np.int32)), 3, heads, kv_heads, dim, vdim, dim ** -0.5)
    want = np.zeros((tokens, heads, vdim))
    want_state = state.astype(np.float64).copy()
    for span, (length, slot) in enumerate(zip(lengths, slots)):
        for h in range(heads):
            kv = h // (heads // kv_heads)
            s = want_state[slot, :elements].reshape(heads, dim, vdim)[h]
            for t in range(begins[span], begins[span] + length):
                s *= gates[t, heads + h]
                u = gates[t, h] * (v[t, h] - s.T @ k[t, kv])
                s += np.outer(k[t, kv], u)
                want[t, h] = s.T @ (q[t, kv] * dim ** -0.5)
    close(out, want.reshape(tokens, -1), torch.float32, scale=5.0)
    close(state_dev, want_state, torch.float32, scale=5.0)


@pytest.mark.parametrize("heads,dim,vdim", [(2, 16, 24), (3, 40, 5), (1, 130, 20)])
def test_mlstm_scan_with_gates_and_running_maximum(heads, dim, vdim):
    from celeg_b200 import kernels
    rng = np.random.default_rng(6)
    lengths, slots = [29, 1, 40], [1, 2, 0]
    tokens = sum(lengths)
    q, k, v = scan_inputs(rng, tokens, heads, heads, dim, vdim)
    pre = (rng.normal(size=(tokens, 2 * heads)) * 6.0).astype(np.float32)
    bias_i, bias_f = rng.normal(size=heads).astype(np.float32), rng.normal(2.0, 1.0, size=heads).astype(np.float32)
    cap = 5.0
    pre_dev = dev(pre)
    gates = torch.zeros((tokens, 2 * heads), dtype=torch.float32, device="cuda")
    kernels.mlstm_gates(pre_dev[:, :heads], pre_dev[:, heads:], dev(bias_i), dev(bias_f), cap, gates, tokens, heads)
    log_i = cap * np.tanh((pre[:, :heads].astype(np.float64) + bias_i) / cap)
    log_f = plain.log_sigmoid(cap * np.tanh((pre[:, heads:].astype(np.float64) + bias_f) / cap))
    close(gates, np.concatenate([log_i, log_f], axis=1), torch.float32)
    elements = heads * dim * vdim + heads * dim + heads
    state = np.zeros((3, elements + 4), dtype=np.float32)
    # slot 2 continues a sequence: some memory, a normaliser and a running maximum above zero
    state[2, :heads * dim * vdim + heads * dim] = rng.normal(size=heads * dim * vdim + heads * dim)
    state[2, heads * dim * vdim + heads * dim:elements] = 1.5
    state_dev = dev(state)
    out = torch.zeros((tokens, heads * vdim), dtype=torch.float32, device="cuda")
    begins = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    kernels.recurrent_scan(kernels.SCAN_MLSTM, dev(q.reshape(tokens, -1)), dev(k.reshape(tokens, -1)),
                           dev(v.reshape(tokens, -1)), gates, out, state_dev, elements + 4, dev(begins),
                           dev(np.array(slots, dtype=np.int32)), 3, heads, heads, dim, vdim, dim ** -0.5)
    want = np.zeros((tokens, heads, vdim))
    final = state.astype(np.float64).copy()
    for span, (length, slot) in enumerate(zip(lengths, slots)):
        row = final[slot]
        for h in range(heads):
            memory = row[:heads * dim * vdim].reshape(heads, dim, vdim)[h]
            normaliser = row[heads * dim * vdim:heads * dim * vdim + heads * dim].reshape(heads, dim)[h]
            running = row[heads * dim * vdim + heads * dim + h]
            for t in range(begins[span], begins[span] + length):
                new = max(log_f[t, h] + running, log_i[t, h])
                keep, write = math.exp(log_f[t, h] + running - new), math.exp(log_i[t, h] - new)
                memory *= keep
                memory += write * np.outer(k[t, h], v[t, h])
                normaliser *= keep
                normaliser += write * k[t, h]
                running = new
                query = q[t, h] * dim ** -0.5
                want[t, h] = (memory.T @ query) / (max(abs(normaliser @ query), math.exp(-running)) + 1e-6)
            row[heads * dim * vdim + heads * dim + h] = running
    close(out, want.reshape(tokens, -1), torch.float32, scale=5.0)
    close(state_dev, final, torch.float32, scale=5.0)


@pytest.mark.parametrize("taps", [1, 2, 4])
def test_delta_prepare_convolves_normalises_and_moves_the_carried_inputs_on(taps):
    from celeg_b200 import kernels
    rng = np.random.default_rng(7)
    heads, kv_heads, dim, vdim = 4, 2, 12, 10
    lengths, slots = [9, 1, 2], [1, 2, 0]
    tokens = sum(lengths)
    qk, vw = kv_heads * dim, heads * vdim
    channels = 2 * qk + vw
    proj = rng.normal(size=(tokens, channels + vw + 2 * heads)).astype(np.float32)
    kernel = rng.normal(size=(channels, taps)).astype(np.float32)
    a_log, dt_bias = rng.normal(size=heads).astype(np.float32), rng.normal(size=heads).astype(np.float32)
    carried = rng.normal(size=(3, (taps - 1) * channels + 8)).astype(np.float32)
    carried_dev = dev(carried)
    proj_dev = dev(proj)
    conv = torch.zeros((tokens, channels), dtype=torch.float32, device="cuda")
    gates = torch.zeros((tokens, 2 * heads), dtype=torch.float32, device="cuda")
    begins = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    token_span = np.repeat(np.arange(3), lengths).astype(np.int32)
    kernels.delta_prepare(proj_dev, dev(kernel), carried_dev, carried.shape[1], dev(token_span), dev(begins),
                          dev(np.array(slots, dtype=np.int32)), conv, proj_dev[:, channels + vw:],
                          proj_dev[:, channels + vw + heads:], dev(a_log), dev(dt_bias), gates, tokens, 3, channels, taps,
                          kv_heads, dim, heads, 1e-6)
    want = np.zeros((tokens, channels))
    want_carried = carried.astype(np.float64).copy()
    for span, (length, slot) in enumerate(zip(lengths, slots)):
        history = carried[slot, :(taps - 1) * channels].reshape(taps - 1, channels).astype(np.float64)
        rows = np.concatenate([history, proj[begins[span]:begins[span] + length, :channels]], axis=0)
        for t in range(length):
            want[begins[span] + t] = plain.silu(np.sum(rows[t:t + taps] * kernel.T, axis=0))
        want_carried[slot, :(taps - 1) * channels] = rows[len(rows) - (taps - 1):].reshape(-1) if taps > 1 else []
    unit = want[:, :2 * qk].reshape(tokens, 2 * kv_heads, dim)
    unit /= np.sqrt(np.sum(unit * unit, axis=-1, keepdims=True) + 1e-6)
    want[:, :2 * qk] = unit.reshape(tokens, -1)
    close(conv, want, torch.float32)
    beta = plain.sigmoid(proj[:, channels + vw:channels + vw + heads].astype(np.float64))
    decay = np.exp(-np.exp(a_log.astype(np.float64)) * plain.softplus(proj[:, channels + vw + heads:].astype(np.float64) + dt_bias))
    close(gates, np.concatenate([beta, decay], axis=1), torch.float32)
    close(carried_dev, want_carried, torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("per_head,gate_kind", [(True, 0), (False, 1)])
def test_gated_head_norm(dtype, per_head, gate_kind):
    from celeg_b200 import kernels
    rng = np.random.default_rng(8)
    tokens, heads, vdim, eps = 11, 3, 41, 1e-5
    o = rng.normal(size=(tokens, heads, vdim)).astype(np.float32) * 4.0
    gate_rows = rng.normal(size=(tokens, heads * vdim + 7)).astype(np.float32)
    weight = rng.normal(1.0, 0.2, size=(heads * vdim if per_head else vdim)).astype(np.float32)
    out = torch.zeros((tokens, heads * vdim), dtype=dtype, device="cuda")
    gate_dev = dev(gate_rows)
    kernels.gated_head_norm(dev(o.reshape(tokens, -1)), gate_dev[:, 3:3 + heads * vdim], dev(weight), per_head, out,
                            tokens, heads, vdim, eps, gate_kind)
    gate = gate_rows[:, 3:3 + heads * vdim].astype(np.float64)
    normed = plain.root_mean_square_scaled(o.astype(np.float64), eps)
    normed = normed * (weight.reshape(heads, vdim) if per_head else weight)
    want = normed.reshape(tokens, -1) * (plain.sigmoid(gate) if gate_kind == 0 else plain.silu(gate))
    close(out, want, dtype, scale=2.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,taps", [(3, 3, 24, 7, 3), (4, 2, 16, 24, 1), (2, 1, 64, 64, 4),
                                                            (1, 1, 200, 300, 2), (2, 2, 40, 70, 5)])
def test_decoding_kernel_of_the_delta_rule_equals_prepare_scan_and_norm(dtype, heads, kv_heads, dim, vdim, taps):
    """One token per request: the single launch against the three steps that serve prompts (each of which is
    tested against float64 above), on requests whose slots hold state and carried inputs."""
    from celeg_b200 import kernels
    torch.manual_seed(1)
    tokens = 5
    qk, vw = kv_heads * dim, heads * vdim
    channels = 2 * qk + vw
    proj = torch.randn(tokens, channels + vw + 2 * heads, device="cuda")
    kernel = torch.randn(channels, taps, device="cuda") * 0.5
    a_log, dt_bias = torch.randn(heads, device="cuda") - 1.0, torch.randn(heads, device="cuda")
    norm = torch.rand(vdim, device="cuda") + 0.5
    elements = heads * dim * vdim
    stride = elements + (taps - 1) * channels + 4
    state = torch.randn(tokens, stride, device="cuda") * 0.3
    fused_state = state.clone()
    begins = torch.arange(tokens + 1, dtype=torch.int32, device="cuda")
    slots = torch.arange(tokens, dtype=torch.int32, device="cuda").flip(0).contiguous()
    spans = torch.arange(tokens, dtype=torch.int32, device="cuda")
    gates = torch.zeros(tokens, 2 * heads, device="cuda")
    conv = torch.zeros(tokens, channels, device="cuda")
    read = torch.zeros(tokens, vw, device="cuda")
    want = torch.zeros(tokens, vw, dtype=dtype, device="cuda")
    got = torch.zeros_like(want)
    kernels.delta_prepare(proj, kernel, state[:, elements:], stride, spans, begins, slots, conv,
                          proj[:, channels + vw:channels + vw + heads], proj[:, channels + vw + heads:], a_log, dt_bias,
                          gates, tokens, tokens, channels, taps, kv_heads, dim, heads, 1e-6)
    kernels.recurrent_scan(kernels.SCAN_DELTA, conv[:, :qk], conv[:, qk:2 * qk], conv[:, 2 * qk:], gates, read, state,
                           stride, begins, slots, tokens, heads, kv_heads, dim, vdim, dim ** -0.5)
    kernels.gated_head_norm(read, proj[:, channels:channels + vw], norm, False, want, tokens, heads, vdim, 1e-5,
                            kernels.GATE_SILU)
    kernels.recurrent_decode(kernels.SCAN_DELTA, proj, (0, qk, 2 * qk, channels, channels + vw, channels + vw + heads),
                             kernel, fused_state[:, elements:], taps, channels, a_log, dt_bias, 0.0, norm, False, 1e-5,
                             1e-6, fused_state, stride, begins, slots, tokens, heads, kv_heads, dim, vdim, dim ** -0.5, got)
    close(got, want.to(torch.float64).cpu().numpy(), dtype)
    close(fused_state, state.to(torch.float64).cpu().numpy(), torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,vdim", [(3, 12, 20), (2, 64, 128), (1, 200, 8), (2, 40, 70), (1, 8, 300)])
def test_decoding_kernel_of_the_mlstm_equals_gates_scan_and_norm(dtype, heads, dim, vdim):
    from celeg_b200 import kernels
    torch.manual_seed(2)
    tokens = 5
    qk, vw = heads * dim, heads * vdim
    proj = torch.randn(tokens, 2 * qk + 2 * vw + 2 * heads, device="cuda")
    bias_i, bias_f = torch.randn(heads, device="cuda"), torch.randn(heads, device="cuda") + 2.0
    norm = torch.rand(vw, device="cuda") + 0.5
    elements = heads * dim * vdim + heads * dim + heads
    state = torch.randn(tokens, elements + 4, device="cuda") * 0.3
    state[:, elements - heads:elements] = 0.7                     # running maxima
    fused_state = state.clone()
    begins = torch.arange(tokens + 1, dtype=torch.int32, device="cuda")
    slots = torch.arange(tokens, dtype=torch.int32, device="cuda").flip(0).contiguous()
    gates = torch.zeros(tokens, 2 * heads, device="cuda")
    read = torch.zeros(tokens, vw, device="cuda")
    want = torch.zeros(tokens, vw, dtype=dtype, device="cuda")
    got = torch.zeros_like(want)
    at = 2 * qk + 2 * vw
    kernels.mlstm_gates(proj[:, at:at + heads], proj[:, at + heads:], bias_i, bias_f, 7.0, gates, tokens, heads)
    kernels.recurrent_scan(kernels.SCAN_MLSTM, proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + vw], gates, read,
                           state, elements + 4, begins, slots, tokens, heads, heads, dim, vdim, dim ** -0.5)
    kernels.gated_head_norm(read, proj[:, 2 * qk + vw:at], norm, True, want, tokens, heads, vdim, 1e-5, kernels.GATE_SIGMOID)
    kernels.recurrent_decode(kernels.SCAN_MLSTM, proj, (0, qk, 2 * qk, 2 * qk + vw, at, at + heads), None, None, 0, 0,
                             bias_i, bias_f, 7.0, norm, True, 1e-5, 0.0, fused_state, elements + 4, begins, slots, tokens,
                             heads, heads, dim, vdim, dim ** -0.5, got)
    close(got, want.to(torch.float64).cpu().numpy(), dtype)
    close(fused_state, state.to(torch.float64).cpu().numpy(), torch.float32)


@pytest.mark.parametrize("kind", [0, 1, 2])
@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (8, 1000, 256), (16, 48, 520), (5, 70, 136)])
def test_small_batch_product_with_an_activation_in_its_epilogue(m, n, k, kind):
    from celeg_b200 import kernels
    rng = np.random.default_rng(9)
    x, w = rounded(rng.normal(size=(m, k)), torch.bfloat16), rounded(rng.normal(size=(n, k)) * 0.2, torch.bfloat16)
    y = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    kernels.gemv_bf16(dev(x, torch.bfloat16), dev(w, torch.bfloat16), y, m, kernels.GEMV_ACTIVATION, taps=kind)
    product = rounded(x @ w.T, torch.bfloat16)
    want = [plain.gelu_erf, lambda z: 0.5 * z * (1 + np.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3))), plain.silu][kind](product)
    close(y, want, torch.bfloat16, scale=2.0)


@pytest.mark.parametrize("variant", [1, 3, -1])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (200, 264, 520), (2048, 384, 1024)])
def test_tcgen05_product_with_an_activation_in_its_epilogue(m, n, k, variant):
    from celeg_b200 import kernels
    rng = np.random.default_rng(10)
    x, w = rounded(rng.normal(size=(m, k)), torch.bfloat16), rounded(rng.normal(size=(n, k)) * 0.1, torch.bfloat16)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    kernels.gemm_tcgen05(dev(x, torch.bfloat16), dev(w, torch.bfloat16), y, m, kernels.TC_ACTIVATION + kernels.ACT_GELU_ERF,
                         flag, variant)
    assert int(flag.item()) == 0
    close(y, plain.gelu_erf(rounded(x @ w.T, torch.bfloat16)), torch.bfloat16, scale=2.0)
