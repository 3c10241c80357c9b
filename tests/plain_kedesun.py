"""A plain, slow Kedesun model: whole sequences, no cache, float64, one function a mechanism.

Kedesun is a decoder-only model whose blocks read ONE RMS norm of the stream and add a mixer and a
feed-forward of that same input side by side; after every block the stream becomes a learned weighted
sum of the embedding output and all blocks' results so far (a depth-weighted average). The mixers are a
latent attention (keys and values are up-projections of one low-rank vector per position, plus one rotated
key part shared by the heads; interleaved rotary pairs with YaRN-scaled frequencies; a sigmoid gate per
head) and a retention (linear attention with a fixed decay per head). The feed-forward is a SwiGLU or a
mixture of experts with squared-ReLU experts, a softmax router whose choice (not its weights) is shifted
by a stored correction, and a gated shared expert. This file shares no code with the ``celeg_b200``
package: it takes the configuration as the dict that config.json holds and the weights as a dict of arrays.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

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


def squared_relu(x):
    return np.square(np.maximum(x, 0.0))


def rms_scaled(x: np.ndarray, eps: float) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    return rms_scaled(x, eps) * weight


# ------------------------------------------------------------------------------- rotation
def yarn_frequencies(rot: dict):
    """(frequencies [dims / 2], factor of cos and sin). f_i = base^(-2i/dims); with ``scaling`` the index at
    which a wave makes t turns over the original length is d(t) = dims ln(original / (2 pi t)) / (2 ln base),
    a ramp rises from 0 at lo = floor(d(fast)) to 1 at hi = ceil(d(slow)), and the frequency becomes
    f_i / factor where the ramp is 1, f_i where it is 0, the blend between; cos and sin are then multiplied by
    0.1 ln(factor) + 1."""
    dims = int(rot["dims"])
    base = float(rot["base"])
    freq = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)
    scaling = rot.get("scaling")
    if not scaling:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def index_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index_of(float(scaling["slow"]))), dims - 1)
    out = np.empty_like(freq)
    for i, f in enumerate(freq):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out[i] = f / factor * ramp + f * (1.0 - ramp)
    return out, 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x: np.ndarray, positions: np.ndarray, rot: dict) -> np.ndarray:
    """x [tokens, ..., dims or more]: dimensions (2i, 2i + 1) of the first ``dims`` form a pair that is turned by
    position x frequency_i; the rest pass unchanged."""
    dims = int(rot["dims"])
    freq, magnitude = yarn_frequencies(rot)
    angles = positions[:, None].astype(np.float64) * freq[None, :]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (dims // 2,)
    cos, sin = np.cos(angles).reshape(shape) * magnitude, np.sin(angles).reshape(shape) * magnitude
    out = x.copy()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


# --------------------------------------------------------------------------------- mixers
def latent_attention(tensors, base: str, mixer: dict, h: np.ndarray, eps: float) -> np.ndarray:
    """Every head's key and value are made again from the latent vector of each position (nothing absorbed,
    nothing cached): the slow form."""
    heads, dim, rot_dim = int(mixer["heads"]), int(mixer["dim"]), int(mixer["rot_dim"])
    vdim, rank = int(mixer["vdim"]), int(mixer["kv_rank"])
    tokens = h.shape[0]
    positions = np.arange(tokens)
    rot = dict(mixer["rot"])
    q = (h @ tensors[base + "q"].T).reshape(tokens, heads, dim + rot_dim)
    down = h @ tensors[base + "dkv"].T
    latent = rms_norm(down[:, :rank], tensors[base + "dkv.norm"], eps)
    key_rotated = rotate_interleaved(down[:, rank:], positions, rot)                      # [tokens, rot_dim]
    q_rotated = rotate_interleaved(q[:, :, dim:], positions, rot)                          # [tokens, heads, rot_dim]
    keys = (latent @ tensors[base + "uk"].T).reshape(tokens, heads, dim)
    values = (latent @ tensors[base + "uv"].T).reshape(tokens, heads, vdim)
    gate = sigmoid(h @ tensors[base + "g"].T)                                              # [tokens, heads]
    scale = float(mixer["scale"])
    out = np.zeros((tokens, heads, vdim))
    for head in range(heads):
        scores = (q[:, head, :dim] @ keys[:, head].T + q_rotated[:, head] @ key_rotated.T) * scale
        scores = np.where(np.tril(np.ones((tokens, tokens), dtype=bool)), scores, -np.inf)
        scores -= scores.max(axis=-1, keepdims=True)
        weights = np.exp(scores)
        weights /= weights.sum(axis=-1, keepdims=True)
        out[:, head] = (weights @ values[:, head]) * gate[:, head:head + 1]
    return out.reshape(tokens, heads * vdim) @ tensors[base + "o"].T


def retention(tensors, base: str, mixer: dict, h: np.ndarray, eps: float) -> np.ndarray:
    """S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, token by token."""
    heads, dim, vdim = int(mixer["heads"]), int(mixer["dim"]), int(mixer["vdim"])
    decay = [float(d) for d in mixer["decay"]]
    tokens = h.shape[0]
    q = (h @ tensors[base + "q"].T).reshape(tokens, heads, dim)
    k = (h @ tensors[base + "k"].T).reshape(tokens, heads, dim) * dim ** -0.5
    v = (h @ tensors[base + "v"].T).reshape(tokens, heads, vdim)
    read = np.zeros((tokens, heads, vdim))
    for head in range(heads):
        state = np.zeros((dim, vdim))
        for t in range(tokens):
            state = decay[head] * state + np.outer(k[t, head], v[t, head])
            read[t, head] = state.T @ q[t, head]
    read = rms_scaled(read, eps).reshape(tokens, heads * vdim)
    return (read * silu(h @ tensors[base + "g"].T)) @ tensors[base + "o"].T


# --------------------------------------------------------------------------- feed-forward
def swiglu(tensors, base: str, h: np.ndarray) -> np.ndarray:
    return (silu(h @ tensors[base + "gate"].T) * (h @ tensors[base + "up"].T)) @ tensors[base + "down"].T


def expert(tensors, base: str, h: np.ndarray) -> np.ndarray:
    return squared_relu(h @ tensors[base + "up"].T) @ tensors[base + "down"].T


def route(tensors, base: str, mlp: dict, h: np.ndarray):
    """(chosen experts [tokens, top], their weights [tokens, top])."""
    top = int(mlp["router"]["top"])
    logits = h @ tensors[base + "router"].T
    logits -= logits.max(axis=-1, keepdims=True)
    scores = np.exp(logits)
    scores /= scores.sum(axis=-1, keepdims=True)
    choice = scores + tensors[base + "correction"]
    chosen = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    picked = np.take_along_axis(scores, chosen, axis=-1)
    return chosen, picked / (picked.sum(axis=-1, keepdims=True) + 1e-20)


def mixture_of_experts(tensors, base: str, mlp: dict, h: np.ndarray) -> np.ndarray:
    chosen, weights = route(tensors, base, mlp, h)
    out = np.zeros((h.shape[0], tensors[base + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t], weights[t]):
            out[t] += w * expert(tensors, f"{base}e{int(e)}.", h[t:t + 1])[0]
    if mlp.get("shared") is not None:
        out += expert(tensors, base + "shared.", h) * sigmoid(h @ tensors[base + "shared.sg"].T)
    return out


def feed_forward(tensors, base: str, mlp: Optional[dict], h: np.ndarray):
    if mlp is None:
        return 0.0
    if mlp["kind"] == "dense":
        return swiglu(tensors, base, h)
    if mlp["kind"] == "moe":
        return mixture_of_experts(tensors, base, mlp, h)
    raise ValueError(mlp["kind"])


# ---------------------------------------------------------------------------------- model
def mixer_of(tensors, base: str, layer: dict, h: np.ndarray, eps: float) -> np.ndarray:
    if layer["type"] == "latent_attention":
        return latent_attention(tensors, base, layer["mixer"], h, eps)
    if layer["type"] == "retention":
        return retention(tensors, base, layer["mixer"], h, eps)
    raise ValueError(layer["type"])


def depth_average(results: Sequence[np.ndarray], weights: np.ndarray) -> np.ndarray:
    """sum_j weights[j] results[j] over the embedding output and every block's result so far."""
    return sum(float(w) * r for w, r in zip(weights, results))


def streams(config: dict, tensors: Dict[str, np.ndarray], tokens: Sequence[int]) -> List[np.ndarray]:
    """The stream after every block (after the depth average) for one whole sequence."""
    eps = float(config["norm"]["eps"])
    x = tensors["embed"][np.asarray(tokens, dtype=np.int64)]
    results = [x]
    after = []
    for index, layer in enumerate(config["layers"]):
        base = f"l{index}."
        h = rms_norm(x, tensors[base + "norm1"], eps)
        result = x + (mixer_of(tensors, base + "mix.", layer, h, eps) + feed_forward(tensors, base + "mlp.", layer.get("mlp"), h))
        results.append(result)
        x = depth_average(results, tensors[base + "dwa"])
        after.append(x)
    return after


def logits(config: dict, tensors: Dict[str, np.ndarray], tokens: Sequence[int]) -> np.ndarray:
    """[tokens, vocab] for one whole sequence."""
    x = streams(config, tensors, tokens)[-1] if config["layers"] else tensors["embed"][np.asarray(tokens)]
    return rms_norm(x, tensors["final.norm"], float(config["norm"]["eps"])) @ tensors["embed"].T
