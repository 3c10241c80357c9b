"""A plain, slow Ramosun model: whole sequences, no cache, float64, one function a mechanism.

Ramosun is a decoder-only model whose blocks add a mixer and a feed-forward side by side to the
residual stream, each behind a Dynamic-Tanh norm of its own; the mixers are a sliding-window
attention with a sink (values are the unrotated keys), an mLSTM matrix memory and a gated delta
rule; a run of layers may be repeated with the same weights, every pass entered through a
projection of [stream; embedding]. This file shares no code with the ``celeg_b200`` package: it
takes the configuration as the dict that config.json holds and the weights as a dict of arrays.
"""
from __future__ import annotations

import math
from typing import Dict, List, Sequence

import numpy as np


def as_float64(tensors) -> Dict[str, np.ndarray]:
    """{name: torch tensor} -> {name: float64 array}."""
    import torch
    return {name: value.to(torch.float64).numpy() for name, value in tensors.items()}


# ------------------------------------------------------------------------- small functions
def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x * sigmoid(x)


def softplus(x):
    return np.logaddexp(0.0, x)


def log_sigmoid(x):
    return -np.logaddexp(0.0, -x)


def gelu_erf(x):
    erf = np.vectorize(math.erf)
    return 0.5 * x * (1.0 + erf(x / math.sqrt(2.0)))


def root_mean_square_scaled(x: np.ndarray, eps: float) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def dynamic_tanh(x: np.ndarray, weight: np.ndarray, bias: np.ndarray, alpha: float) -> np.ndarray:
    """tanh(alpha x) w + b: no mean, no variance."""
    return np.tanh(float(alpha) * x) * weight + bias


def norm_of(tensors, name: str, x: np.ndarray) -> np.ndarray:
    return dynamic_tanh(x, tensors[name], tensors[name + ".b"], float(tensors[name + ".alpha"]))


# ------------------------------------------------------------------------------- rotation
def rotary_frequencies(rot: dict) -> np.ndarray:
    """f_i = base^(-2i/dims), then the wavelength-dependent scaling: short waves are kept, long ones
    divided by ``factor``, those between blended linearly in original/wavelength."""
    dims = int(rot["dims"])
    freq = np.array([float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)
    scaling = rot.get("scaling")
    if not scaling:
        return freq
    factor, low, high = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"])
    original = float(scaling["original"])
    out = np.empty_like(freq)
    for i, f in enumerate(freq):
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            out[i] = f
        elif wavelength > original / low:
            out[i] = f / factor
        else:
            s = (original / wavelength - low) / (high - low)
            out[i] = (1.0 - s) * f / factor + s * f
    return out


def rotate_half_layout(x: np.ndarray, positions: np.ndarray, freq: np.ndarray, dims: int) -> np.ndarray:
    """x: [T, heads, d]. Dimension i < dims/2 is paired with i + dims/2; dimensions from ``dims`` on pass."""
    half = dims // 2
    angle = positions[:, None].astype(np.float64) * freq[None, :]          # [T, half]
    cos, sin = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
    out = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


# --------------------------------------------------------------------------------- mixers
def attention_mixer(h: np.ndarray, tensors, prefix: str, mixer: dict, eps: float) -> np.ndarray:
    """Windowed attention with a sink; the values are the keys as projected (before norm and rotation)."""
    tokens = h.shape[0]
    heads, kv_heads, dim = int(mixer["heads"]), int(mixer["kv_heads"]), int(mixer["dim"])
    window = int(mixer["mask"]["size"]) if mixer.get("mask") else tokens        # no mask: every earlier token
    scale = float(mixer["scale"])
    q = h @ tensors[prefix + "q"].T
    k = h @ tensors[prefix + "k"].T
    values = k.reshape(tokens, kv_heads, dim)
    q = root_mean_square_scaled(q, eps) * tensors[prefix + "q.norm"]      # over the whole projection
    k = root_mean_square_scaled(k, eps) * tensors[prefix + "k.norm"]
    q = q.reshape(tokens, heads, dim)
    k = k.reshape(tokens, kv_heads, dim)
    rot = mixer.get("rot")
    if rot:
        positions = np.arange(tokens)
        freq = rotary_frequencies(rot)
        q = rotate_half_layout(q, positions, freq, int(rot["dims"]))
        k = rotate_half_layout(k, positions, freq, int(rot["dims"]))
    sink = tensors[prefix + "sink"]
    group = heads // kv_heads
    out = np.zeros((tokens, heads, dim))
    for head in range(heads):
        kv = head // group
        for i in range(tokens):
            first = max(0, i - window + 1)
            scores = (k[first:i + 1, kv] @ q[i, head]) * scale
            top = max(scores.max(), sink[head])
            weights = np.exp(scores - top)
            denominator = weights.sum() + math.exp(sink[head] - top)
            out[i, head] = (weights @ values[first:i + 1, kv]) / denominator
    return out.reshape(tokens, heads * dim) @ tensors[prefix + "o"].T


def mlstm_mixer(h: np.ndarray, tensors, prefix: str, mixer: dict, eps: float) -> np.ndarray:
    """Matrix memory with exponential gating, stabilised by a running maximum that starts at 0."""
    tokens = h.shape[0]
    heads, dim, vdim = int(mixer["heads"]), int(mixer["dim"]), int(mixer["vdim"])
    cap = float(mixer["gate_cap"])
    q = (h @ tensors[prefix + "q"].T).reshape(tokens, heads, dim) * dim ** -0.5
    k = (h @ tensors[prefix + "k"].T).reshape(tokens, heads, dim)
    v = (h @ tensors[prefix + "v"].T).reshape(tokens, heads, vdim)
    log_in = cap * np.tanh((h @ tensors[prefix + "i"].T + tensors[prefix + "i.b"]) / cap)
    log_forget = log_sigmoid(cap * np.tanh((h @ tensors[prefix + "f"].T + tensors[prefix + "f.b"]) / cap))
    out = np.zeros((tokens, heads, vdim))
    for head in range(heads):
        memory = np.zeros((dim, vdim))
        normaliser = np.zeros(dim)
        running = 0.0
        for t in range(tokens):
            new_running = max(log_forget[t, head] + running, log_in[t, head])
            keep = math.exp(log_forget[t, head] + running - new_running)
            write = math.exp(log_in[t, head] - new_running)
            memory = keep * memory + write * np.outer(k[t, head], v[t, head])
            normaliser = keep * normaliser + write * k[t, head]
            running = new_running
            denominator = max(abs(normaliser @ q[t, head]), math.exp(-running)) + 1e-6
            out[t, head] = (memory.T @ q[t, head]) / denominator
    out = root_mean_square_scaled(out, eps).reshape(tokens, heads * vdim) * tensors[prefix + "norm"]
    out = out * sigmoid(h @ tensors[prefix + "g"].T)
    return out @ tensors[prefix + "o"].T


def causal_short_convolution(x: np.ndarray, kernel: np.ndarray) -> np.ndarray:
    """x: [T, channels]; kernel: [channels, taps], the last column multiplies the current token; zeros before
    the start."""
    taps = kernel.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, x.shape[1])), x], axis=0)
    out = np.zeros_like(x)
    for tap in range(taps):
        out += padded[tap:tap + x.shape[0]] * kernel[:, tap]
    return out


def delta_mixer(h: np.ndarray, tensors, prefix: str, mixer: dict, eps: float) -> np.ndarray:
    """Gated delta rule: decay, then replace what the key reads by a step towards the value, then read."""
    tokens = h.shape[0]
    heads, kv_heads = int(mixer["heads"]), int(mixer["kv_heads"])
    dim, vdim = int(mixer["dim"]), int(mixer["vdim"])
    q = silu(causal_short_convolution(h @ tensors[prefix + "q"].T, tensors[prefix + "q.conv"]))
    k = silu(causal_short_convolution(h @ tensors[prefix + "k"].T, tensors[prefix + "k.conv"]))
    v = silu(causal_short_convolution(h @ tensors[prefix + "v"].T, tensors[prefix + "v.conv"]))
    q = q.reshape(tokens, kv_heads, dim)
    k = k.reshape(tokens, kv_heads, dim)
    v = v.reshape(tokens, heads, vdim)
    q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) * dim ** -0.5
    k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ tensors[prefix + "b"].T)
    decay = np.exp(-np.exp(tensors[prefix + "A_log"]) * softplus(h @ tensors[prefix + "a"].T + tensors[prefix + "dt_bias"]))
    group = heads // kv_heads
    out = np.zeros((tokens, heads, vdim))
    for head in range(heads):
        kv = head // group
        state = np.zeros((dim, vdim))
        for t in range(tokens):
            state = decay[t, head] * state
            update = beta[t, head] * (v[t, head] - state.T @ k[t, kv])
            state = state + np.outer(k[t, kv], update)
            out[t, head] = state.T @ q[t, kv]
    out = root_mean_square_scaled(out, eps) * tensors[prefix + "norm"]
    out = out.reshape(tokens, heads * vdim) * silu(h @ tensors[prefix + "g"].T)
    return out @ tensors[prefix + "o"].T


MIXERS = {"attention": attention_mixer, "mlstm": mlstm_mixer, "delta": delta_mixer}


# ---------------------------------------------------------------------------- feed-forward
def dense_feed_forward(h: np.ndarray, tensors, prefix: str) -> np.ndarray:
    return gelu_erf(h @ tensors[prefix + "up"].T) @ tensors[prefix + "down"].T


# ----------------------------------------------------------------------------------- model
def run_order(config: dict) -> List[tuple]:
    """[(layer index, whether a pass begins here)]: layers start..stop-1 run ``times`` times in a row."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, False) for i in range(count)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(start)]
    for _ in range(times):
        order += [(i, i == start) for i in range(start, stop)]
    order += [(i, False) for i in range(stop, count)]
    return order


def forward(config: dict, tensors, token_ids: Sequence[int], return_layers: bool = False):
    """Logits [T, vocab] of one sequence from position 0 (and the stream after every layer run)."""
    eps = float(config["norm"]["eps"])
    embedded = tensors["embed"][np.asarray(token_ids, dtype=np.int64)]
    x = embedded.copy()
    after_layers = []
    for index, begins_pass in run_order(config):
        layer = config["layers"][index]
        if begins_pass:
            x = np.concatenate([x, embedded], axis=-1) @ tensors["loop.in"].T
        name = f"l{index}."
        mixed = MIXERS[layer["type"]](norm_of(tensors, name + "norm1", x), tensors, name + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"unknown feed-forward kind {layer['mlp']['kind']}")
            mixed = mixed + dense_feed_forward(norm_of(tensors, name + "norm2", x), tensors, name + "mlp.")
        x = x + mixed
        after_layers.append(x.copy())
    logits = norm_of(tensors, "final.norm", x) @ tensors["embed"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = float(cap) * np.tanh(logits / float(cap))
    if return_layers:
        return logits, np.stack(after_layers)
    return logits
