"""Small Ramosun configurations with weights of the tests' own making, written as model folders.

The sizes differ from one configuration to the next in every respect that the design leaves open (widths,
head counts and groupings, key and value sizes, windows, rotated dimensions, taps, where the repeated run
lies and how often it runs, layers without a feed-forward, with and without capped logits). Weights come
from a numpy generator and are rounded to bfloat16, so the float64 plain model and the engine read the same
numbers. ``sharpen`` scales the attention's q/k norm weights (softmax close to one-hot, so a single key
shows) and pushes the recurrent mixers' gates towards remembering (so a far token shows).
"""
from __future__ import annotations

import copy
import json
import math
import os
from typing import Dict, Optional

import numpy as np
import torch


def attention(heads, kv_heads, dim, window, rot_dims=None, base=10000.0, scaling=None, scale=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
             "scale": dim ** -0.5 if scale is None else scale}
    if window is not None:
        mixer["mask"] = {"size": window}
    if rot_dims:
        mixer["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            mixer["rot"]["scaling"] = scaling
    return {"type": "attention", "mixer": mixer}


def mlstm(heads, dim, vdim, gate_cap=15.0):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap}}


def delta(heads, kv_heads, dim, vdim, conv=4):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def with_mlp(layer, ff):
    layer = copy.deepcopy(layer)
    layer["mlp"] = None if ff is None else {"kind": "dense", "ff": ff}
    return layer


def config(vocab, width, layers, loop=None, eps=1e-5, softcap=None):
    raw = {"architecture": "Ramosun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop is not None:
        raw["loop"] = dict(zip(("start", "stop", "times"), loop))
    if softcap is not None:
        raw["logit_softcap"] = softcap
    return raw


LLAMA_SCALING = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}

# every mixer once, grouped heads, part of each head rotated with scaled frequencies, the run 1..3 twice
MIXED = config(160, 64, [
    with_mlp(attention(4, 2, 16, 24, rot_dims=8, scaling=LLAMA_SCALING, scale=0.3), 96),
    with_mlp(mlstm(2, 16, 24, gate_cap=8.0), 96),
    with_mlp(delta(4, 2, 16, 24, conv=3), None),
    with_mlp(attention(2, 2, 32, 40, rot_dims=32, base=500.0), 80),
], loop=(1, 3, 2), softcap=12.0)

# the run starts at the first layer and runs three times; one q/k head for all; two taps; no cap on the logits;
# a window smaller than a page; no rotation at all in one attention, no window in the other
LOOP_FROM_START = config(96, 48, [
    with_mlp(delta(3, 1, 8, 8, conv=2), 64),
    with_mlp(attention(3, 1, 16, 5, rot_dims=None), None),
    with_mlp(mlstm(1, 8, 40, gate_cap=20.0), 64),
    with_mlp(attention(6, 3, 8, None, rot_dims=4, base=100.0), 32),
], loop=(0, 2, 3), eps=1e-6)

# no repeated run; head sizes of 64 and 40 (the latter no multiple of 16), key size 40 in a recurrent mixer (two
# lanes a column, the second half empty), a window of exactly one page, five taps
STRAIGHT = config(200, 80, [
    with_mlp(mlstm(2, 40, 16, gate_cap=10.0), 120),
    with_mlp(attention(2, 1, 64, 16, rot_dims=64, scaling={"factor": 8.0, "low": 1.0, "high": 2.0, "original": 32}), 120),
    with_mlp(delta(2, 2, 40, 32, conv=5), 120),
    with_mlp(attention(5, 5, 40, 33, rot_dims=20), None),
], softcap=30.0)

# the whole model is the repeated run, once
LOOP_ONCE = config(64, 32, [
    with_mlp(attention(2, 2, 8, 7, rot_dims=8), 48),
    with_mlp(delta(2, 1, 16, 8, conv=4), 48),
], loop=(0, 2, 1), softcap=5.0)

# sizes that fit no vector width: a model width of 36, head sizes of 12 and 20, seventeen query heads on one key
# head (more than the split-key kernel groups), key size 24 with values of 7
ODD = config(50, 36, [
    with_mlp(attention(3, 1, 12, 9, rot_dims=6, base=50.0), 44),
    with_mlp(delta(3, 3, 24, 7, conv=3), 20),
    with_mlp(attention(17, 1, 20, 30, rot_dims=20, scaling={"factor": 2.0, "low": 1.0, "high": 3.0, "original": 16}), None),
    with_mlp(mlstm(3, 12, 20, gate_cap=6.0), 28),
], loop=(2, 4, 2), softcap=20.0)

CONFIGS = {"odd": (ODD, 15), "mixed": (MIXED, 11), "loop_from_start": (LOOP_FROM_START, 12), "straight": (STRAIGHT, 13),
           "loop_once": (LOOP_ONCE, 14)}


def single_layer(layer, vocab=96, width=48, softcap=None, ff=None):
    """A model of one layer (no feed-forward unless ``ff``), to look at one mixer alone."""
    return config(vocab, width, [with_mlp(layer, ff)], softcap=softcap)


def _round(values: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.asarray(values, dtype=np.float32)).to(torch.bfloat16)


def make_tensors(raw: dict, seed: int, sharpen: float = 1.0, remember: bool = False) -> Dict[str, torch.Tensor]:
    rng = np.random.default_rng(seed)
    width, vocab = raw["width"], raw["vocab"]
    out: Dict[str, torch.Tensor] = {}

    def matrix(name, rows, cols, gain=1.0):
        out[name] = _round(rng.normal(0.0, gain / math.sqrt(cols), size=(rows, cols)))

    def vector(name, size, mean=0.0, std=0.3):
        out[name] = _round(rng.normal(mean, std, size=(size,)))

    def norm(name):
        vector(name, width, 1.0, 0.1)
        vector(name + ".b", width, 0.0, 0.1)
        out[name + ".alpha"] = _round(np.array(rng.uniform(0.5, 1.0)))

    out["embed"] = _round(rng.normal(0.0, 1.0, size=(vocab, width)))
    if raw.get("loop"):
        matrix("loop.in", width, 2 * width, gain=1.2)
    for index, layer in enumerate(raw["layers"]):
        base = f"l{index}."
        mix, m = base + "mix.", layer["mixer"]
        norm(base + "norm1")
        if layer["type"] == "attention":
            q_width, kv_width = m["heads"] * m["dim"], m["kv_heads"] * m["dim"]
            matrix(mix + "q", q_width, width)
            matrix(mix + "k", kv_width, width)
            vector(mix + "q.norm", q_width, sharpen, 0.1)
            vector(mix + "k.norm", kv_width, sharpen, 0.1)
            vector(mix + "sink", m["heads"], 0.0, 1.0)
            matrix(mix + "o", width, q_width)
        elif layer["type"] == "mlstm":
            qk, vw = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            matrix(mix + "q", qk, width)
            matrix(mix + "k", qk, width)
            matrix(mix + "v", vw, width)
            matrix(mix + "g", vw, width)
            matrix(mix + "o", width, vw)
            vector(mix + "norm", vw, 1.0, 0.1)
            matrix(mix + "i", m["heads"], width)
            vector(mix + "i.b", m["heads"], 0.0, 0.5)
            matrix(mix + "f", m["heads"], width)
            vector(mix + "f.b", m["heads"], 6.0 if remember else 2.0, 0.5)
        else:
            qk, vw = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"]
            for name, rows in (("q", qk), ("k", qk), ("v", vw)):
                matrix(mix + name, rows, width, gain=2.0)
                out[mix + name + ".conv"] = _round(rng.normal(0.0, 0.5, size=(rows, m["conv"])))
            matrix(mix + "b", m["heads"], width)
            matrix(mix + "a", m["heads"], width)
            vector(mix + "A_log", m["heads"], -5.0 if remember else -1.0, 0.3)
            vector(mix + "dt_bias", m["heads"], 0.0, 0.3)
            vector(mix + "norm", m["vdim"], 1.0, 0.1)
            matrix(mix + "g", vw, width)
            matrix(mix + "o", width, vw)
        if layer.get("mlp") is not None:
            norm(base + "norm2")
            matrix(base + "mlp.up", layer["mlp"]["ff"], width)
            matrix(base + "mlp.down", width, layer["mlp"]["ff"])
    norm("final.norm")
    return out


def write_model(folder: str, raw: dict, seed: int, sharpen: float = 1.0, remember: bool = False,
                tensors: Optional[Dict[str, torch.Tensor]] = None):
    """Writes ``folder`` and returns (config, {name: bfloat16 tensor})."""
    from safetensors.torch import save_file
    tensors = tensors if tensors is not None else make_tensors(raw, seed, sharpen, remember)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(raw, handle, indent=1)
    save_file({name: value.contiguous() for name, value in tensors.items()}, os.path.join(folder, "model.safetensors"))
    return raw, tensors
