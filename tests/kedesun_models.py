"""Small Kedesun configurations with weights of the tests' own making, written as model folders.

The sizes differ from one configuration to the next in every respect that the design leaves open (widths, head
counts, key, rotated, value and latent sizes, how much of the rotated part turns, with and without YaRN, decays,
numbers of experts and choices, with and without a shared expert, layers without a feed-forward, which mixer comes
first). Weights come from a numpy generator and are rounded to bfloat16, so the float64 plain model and the engine
read the same numbers. ``sharpen`` scales the attention's query and down projections (softmax close to one-hot, so
a single key shows); router matrices are drawn large so that no choice of experts is a close call.
"""
from __future__ import annotations

import copy
import json
import math
import os
from typing import Dict, Optional

import numpy as np
import torch


def latent(heads, dim, rot_dim, vdim, kv_rank, scale=None, base=10000.0, dims=None, yarn=None):
    rot = {"base": base, "dims": rot_dim if dims is None else dims}
    if yarn:
        rot["scaling"] = yarn
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                      "scale": (dim + rot_dim) ** -0.5 if scale is None else scale, "rot": rot}}


def retention(heads, dim, vdim, decay=None):
    decay = decay if decay is not None else [1.0 - 2.0 ** -(3 + 2 * h) for h in range(heads)]
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def with_mlp(layer, mlp):
    layer = copy.deepcopy(layer)
    layer["mlp"] = mlp
    return layer


def config(vocab, width, layers, eps=1e-5):
    return {"architecture": "Kedesun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


YARN = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}

# both mixers twice, both feed-forwards, a latent size + rotated size of 32 and one of 64, experts with and without
# a shared one, one choice and two
MIXED = config(160, 64, [
    with_mlp(retention(2, 16, 24, [0.9, 0.99]), moe(8, 2, 32, shared=48)),
    with_mlp(latent(4, 16, 8, 24, 24, yarn=YARN), dense(96)),
    with_mlp(retention(4, 8, 8), dense(80)),
    with_mlp(latent(2, 8, 16, 8, 48, scale=0.3, base=500.0), moe(6, 1, 40)),
])

# sizes that fit no vector width: a width of 36, seventeen heads on the one cached vector (more than the split-key
# kernel groups), a cached vector of 19, part of the rotated part unturned, values of 7, five experts all chosen,
# forty experts (more than a warp), a layer without a feed-forward
ODD = config(50, 36, [
    with_mlp(latent(17, 12, 6, 7, 13, dims=4, base=50.0, yarn={"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}), moe(5, 5, 20, shared=12)),
    with_mlp(retention(3, 24, 7, [0.5, 0.875, 1.0]), None),
    with_mlp(latent(1, 20, 2, 30, 10), moe(40, 3, 8)),
    with_mlp(retention(1, 12, 20, [0.96875]), dense(44)),
], eps=1e-6)

# a cached vector of 256 (the largest the tensor-core attention kernels take) under sixteen heads, a key size of 136
# in the retention (several lanes a column), a deep stack for the depth average
WIDE = config(200, 128, [
    with_mlp(latent(16, 24, 64, 16, 192, yarn={"factor": 4.0, "original": 128, "fast": 32.0, "slow": 1.0}), dense(160)),
    with_mlp(retention(2, 136, 24), moe(12, 4, 48, shared=64)),
    with_mlp(retention(2, 32, 64), None),
    with_mlp(latent(8, 32, 32, 40, 96), moe(4, 2, 72, shared=24)),
    with_mlp(retention(1, 64, 128, [0.999]), dense(96)),
    with_mlp(latent(4, 40, 8, 48, 56), None),
])

CONFIGS = {"mixed": (MIXED, 11), "odd": (ODD, 15), "wide": (WIDE, 13)}


def single_layer(layer, mlp=None, vocab=96, width=48):
    """A model of one layer, to look at one mechanism alone."""
    return config(vocab, width, [with_mlp(layer, mlp)])


def _round(values: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.asarray(values, dtype=np.float32)).to(torch.bfloat16)


def make_tensors(raw: dict, seed: int, sharpen: float = 1.0) -> Dict[str, torch.Tensor]:
    rng = np.random.default_rng(seed)
    width, vocab = raw["width"], raw["vocab"]
    out: Dict[str, torch.Tensor] = {}

    def matrix(name, rows, cols, gain=1.0):
        out[name] = _round(rng.normal(0.0, gain / math.sqrt(cols), size=(rows, cols)))

    def vector(name, size, mean=0.0, std=0.3):
        out[name] = _round(rng.normal(mean, std, size=(size,)))

    out["embed"] = _round(rng.normal(0.0, 1.0, size=(vocab, width)))
    for index, layer in enumerate(raw["layers"]):
        base = f"l{index}."
        mix, m = base + "mix.", layer["mixer"]
        vector(base + "norm1", width, 1.0, 0.1)
        # weights of the depth average: of either sign, of the order of one over their number
        out[base + "dwa"] = _round(rng.normal(1.0 / (index + 2), 0.4, size=(index + 2,)))
        if layer["type"] == "latent_attention":
            heads, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            matrix(mix + "q", heads * (dim + rot), width, gain=sharpen)
            matrix(mix + "dkv", rank + rot, width, gain=sharpen)
            vector(mix + "dkv.norm", rank, 1.0, 0.2)
            matrix(mix + "uk", heads * dim, rank)
            matrix(mix + "uv", heads * vdim, rank)
            matrix(mix + "g", heads, width, gain=2.0)
            matrix(mix + "o", width, heads * vdim)
        else:
            heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
            matrix(mix + "q", heads * dim, width)
            matrix(mix + "k", heads * dim, width)
            matrix(mix + "v", heads * vdim, width)
            matrix(mix + "g", heads * vdim, width)
            matrix(mix + "o", width, heads * vdim)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        name = base + "mlp."
        if mlp["kind"] == "dense":
            matrix(name + "gate", mlp["ff"], width)
            matrix(name + "up", mlp["ff"], width)
            matrix(name + "down", width, mlp["ff"])
            continue
        experts = mlp["router"]["experts"]
        matrix(name + "router", experts, width, gain=3.0)
        vector(name + "correction", experts, 0.0, 1.0 / experts)
        for e in range(experts):
            matrix(f"{name}e{e}.up", mlp["expert"]["ff"], width)
            matrix(f"{name}e{e}.down", width, mlp["expert"]["ff"])
        if mlp.get("shared") is not None:
            matrix(name + "shared.up", mlp["shared"]["ff"], width)
            matrix(name + "shared.down", width, mlp["shared"]["ff"])
            matrix(name + "shared.sg", 1, width, gain=2.0)
    vector("final.norm", width, 1.0, 0.1)
    return out


def write_model(folder: str, raw: dict, seed: int, sharpen: float = 1.0,
                tensors: Optional[Dict[str, torch.Tensor]] = None):
    """Writes ``folder`` and returns (config, {name: bfloat16 tensor})."""
    from safetensors.torch import save_file
    tensors = tensors if tensors is not None else make_tensors(raw, seed, sharpen)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(raw, handle, indent=1)
    save_file({name: value.contiguous() for name, value in tensors.items()}, os.path.join(folder, "model.safetensors"))
    return raw, tensors
