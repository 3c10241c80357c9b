"""The Kedesun design as an arrangement of parts.

A block reads one RMSNorm of the stream and adds its mixer and its feed-forward, both of that same input, side by
side (``parallel_residual`` without a second norm); after it the stream part ``depth_average`` replaces the stream by
the block's own weighted sum of the embedding output and every block's result so far. Mixers: ``latent_attention``
(one cached low-rank vector and one rotated key part per position; interleaved rotary pairs with YaRN frequencies;
a sigmoid gate per head) and ``retention`` (a matrix state per head with a fixed decay). Feed-forward: ``swiglu`` or
``moe`` (squared-ReLU experts, softmax router with a stored correction of the choice, gated shared expert). Output:
RMSNorm, the embedding table as head.

Tensor names: ``embed``, ``final.norm``; layer i: ``l<i>.norm1``, ``l<i>.dwa``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

from typing import Any, Mapping

from .kedesun import DENSE, LATENT_ATTENTION, RETENTION, KedesunConfig, KedesunFeedForward, KedesunLayer
from .registry import Architecture, register_architecture
from .spec import ExecutionEntry, LayerSpec, ModelSpec, PartSpec, TensorRef

AFTER_BLOCK = "after"       # the name under which a block's arrangement finds the stream part that runs after it


def _rmsnorm(name: str, width: int, eps: float) -> PartSpec:
    return PartSpec(kind="rmsnorm", params={"width": width, "eps": eps}, tensors={"weight": TensorRef(name, (width,))})


def _mixer(layer: KedesunLayer, base: str, width: int, eps: float) -> PartSpec:
    mix = base + ".mix."
    if layer.type == LATENT_ATTENTION:
        q_width = layer.heads * (layer.dim + layer.rot_dim)
        scaling = layer.rotary.scaling
        position = PartSpec(kind="rope_interleaved", params={
            "theta": layer.rotary.base, "rotary_dim": layer.rotary.dims, "head_dim": layer.rot_dim,
            "yarn": None if scaling is None else dict(zip(("factor", "original", "fast", "slow"), scaling))})
        return PartSpec(
            kind="latent_attention",
            params={"hidden_size": width, "heads": layer.heads, "dim": layer.dim, "rot_dim": layer.rot_dim,
                    "vdim": layer.vdim, "kv_rank": layer.kv_rank, "scale": layer.scale, "eps": eps},
            tensors={"q": TensorRef(mix + "q", (q_width, width)),
                     "down": TensorRef(mix + "dkv", (layer.kv_rank + layer.rot_dim, width)),
                     "down_norm": TensorRef(mix + "dkv.norm", (layer.kv_rank,)),
                     "up_keys": TensorRef(mix + "uk", (layer.heads * layer.dim, layer.kv_rank)),
                     "up_values": TensorRef(mix + "uv", (layer.heads * layer.vdim, layer.kv_rank)),
                     "gate": TensorRef(mix + "g", (layer.heads, width)),
                     "out": TensorRef(mix + "o", (width, layer.heads * layer.vdim))},
            parts={"position": position})
    if layer.type == RETENTION:
        qk_width, v_width = layer.heads * layer.dim, layer.heads * layer.vdim
        return PartSpec(
            kind="retention",
            params={"hidden_size": width, "heads": layer.heads, "dim": layer.dim, "vdim": layer.vdim,
                    "decay": tuple(layer.decay), "eps": eps},
            tensors={"q": TensorRef(mix + "q", (qk_width, width)), "k": TensorRef(mix + "k", (qk_width, width)),
                     "v": TensorRef(mix + "v", (v_width, width)), "gate": TensorRef(mix + "g", (v_width, width)),
                     "out": TensorRef(mix + "o", (width, v_width))})
    raise AssertionError(layer.type)


def _feed_forward(mlp: KedesunFeedForward, base: str, width: int) -> PartSpec:
    name = base + ".mlp."
    if mlp.kind == DENSE:
        return PartSpec(kind="swiglu", params={"hidden_size": width, "intermediate_size": mlp.ff},
                        tensors={"gate": TensorRef(name + "gate", (mlp.ff, width)), "up": TensorRef(name + "up", (mlp.ff, width)),
                                 "down": TensorRef(name + "down", (width, mlp.ff))})
    tensors = {"router": TensorRef(name + "router", (mlp.experts, width)),
               "correction": TensorRef(name + "correction", (mlp.experts,))}
    for expert in range(mlp.experts):
        tensors[f"e{expert}.up"] = TensorRef(f"{name}e{expert}.up", (mlp.ff, width))
        tensors[f"e{expert}.down"] = TensorRef(f"{name}e{expert}.down", (width, mlp.ff))
    parts = {}
    if mlp.shared_ff is not None:
        tensors["shared_gate"] = TensorRef(name + "shared.sg", (1, width))
        parts["shared"] = PartSpec(kind="dense", category="feed_forward",
                                   params={"hidden_size": width, "intermediate_size": mlp.shared_ff, "activation": "relu2"},
                                   tensors={"up": TensorRef(name + "shared.up", (mlp.shared_ff, width)),
                                            "down": TensorRef(name + "shared.down", (width, mlp.shared_ff))})
    return PartSpec(kind="moe", params={"hidden_size": width, "intermediate_size": mlp.ff, "experts": mlp.experts,
                                        "top": mlp.top, "activation": "relu2"}, tensors=tensors, parts=parts)


def build_kedesun_spec(config: KedesunConfig) -> ModelSpec:
    width, eps = config.width, config.norm_eps
    entries = len(config.layers) + 1
    layers = []
    for index, layer in enumerate(config.layers):
        base = f"l{index}"
        average = PartSpec(kind="depth_average", category="stream",
                           params={"index": index, "entries": entries, "width": width},
                           tensors={"weights": TensorRef(base + ".dwa", (index + 2,))})
        layers.append(LayerSpec(name=base, arrangement="parallel_residual",
                                mixer_norm=_rmsnorm(base + ".norm1", width, eps),
                                mixer=_mixer(layer, base, width, eps), feed_forward_norm=None,
                                feed_forward=None if layer.mlp is None else _feed_forward(layer.mlp, base, width),
                                extra_parts={AFTER_BLOCK: average}))
    spec = ModelSpec(
        architecture=config.model_type, vocab_size=config.vocab, hidden_size=width, max_context=config.max_context,
        embedding=TensorRef("embed", (config.vocab, width)), layers=tuple(layers),
        order=tuple(ExecutionEntry(layer=index) for index in range(len(layers))),
        final_norm=_rmsnorm("final.norm", width, eps), lm_head=None,
        eos_token_ids=tuple(config.eos_token_ids), bos_token_id=config.bos_token_id)
    spec.validate()
    return spec


def kedesun_random_init(config: KedesunConfig, name: str, shape: tuple) -> str:
    """Distribution of a tensor in random-weights mode: matrices N(0, 1/fan-in), norm scales around 1, the depth
    average's weights around 0.4, the router's correction small against 1 / experts."""
    leaf = name.rsplit(".", 1)[-1]
    if leaf == "dwa":
        return "depth"
    if leaf == "correction":
        return "tiny"
    if len(shape) == 1:
        return "norm"
    return "fan_in"


def _parse(raw: Mapping[str, Any]) -> KedesunConfig:
    return KedesunConfig.from_dict(raw)


def _resolve(config: KedesunConfig, tensor_shapes: Mapping[str, Any]) -> KedesunConfig:
    return config


KEDESUN = Architecture(name="Kedesun", parse_config=_parse, resolve_config=_resolve,
                       build_spec=build_kedesun_spec, random_init=kedesun_random_init)
register_architecture(KEDESUN, replace=True)
