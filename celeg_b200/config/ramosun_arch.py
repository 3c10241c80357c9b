"""The Ramosun design as an arrangement of parts.

A block adds its mixer and its feed-forward side by side, each behind a Dynamic-Tanh norm of the same stream
(``parallel_residual``). Mixers: ``attention`` (window, sink per head, q/k norm over the whole projection, rotation
with wavelength scaling on the first dims of a head, values = keys as projected), ``mlstm`` and ``gated_delta``.
Feed-forward: ``dense`` with the exact GELU. A run of layers may repeat with the same weights: the run order names
them again (a cache of their own each time) and every pass is entered through the stream part
``embedding_reentry``. Output: Dynamic Tanh, the embedding table as head, capped logits.

Tensor names: ``embed``, ``loop.in``, ``final.norm{,.b,.alpha}``; layer i: ``l<i>.norm1|norm2{,.b,.alpha}``,
``l<i>.mix.*``, ``l<i>.mlp.up|down``.
"""
from __future__ import annotations

from typing import Any, Mapping

from .ramosun import ATTENTION, DELTA, MLSTM, RamosunConfig, RamosunLayer
from .registry import Architecture, register_architecture
from .spec import ExecutionEntry, LayerSpec, ModelSpec, PartSpec, TensorRef

REENTRY = "reentry"


def _dynamic_tanh(name: str, width: int) -> PartSpec:
    return PartSpec(kind="dynamic_tanh", params={"width": width},
                    tensors={"weight": TensorRef(name, (width,)), "bias": TensorRef(name + ".b", (width,)),
                             "alpha": TensorRef(name + ".alpha", ())})


def _mixer(layer: RamosunLayer, base: str, width: int, eps: float) -> PartSpec:
    mix = base + ".mix."
    if layer.type == ATTENTION:
        q_width, kv_width = layer.heads * layer.dim, layer.kv_heads * layer.dim
        if layer.rotary is not None:
            scaling = layer.rotary.scaling
            position = PartSpec(kind="rope_split_half", params={
                "theta": layer.rotary.base, "rotary_dim": layer.rotary.dims, "head_dim": layer.dim,
                "wavelength_scaling": None if scaling is None else dict(zip(("factor", "low", "high", "original"), scaling))})
        else:
            position = PartSpec(kind="none")
        return PartSpec(
            kind="attention",
            params={"hidden_size": width, "num_heads": layer.heads, "num_kv_heads": layer.kv_heads,
                    "head_dim": layer.dim, "qk_norm_eps": eps, "window": layer.window, "softmax_scale": layer.scale,
                    "whole_qk_norm": True, "values_are_keys": True},
            tensors={"q_proj": TensorRef(mix + "q", (q_width, width)), "k_proj": TensorRef(mix + "k", (kv_width, width)),
                     "out_proj": TensorRef(mix + "o", (width, q_width)),
                     "q_norm": TensorRef(mix + "q.norm", (q_width,)), "k_norm": TensorRef(mix + "k.norm", (kv_width,)),
                     "sinks": TensorRef(mix + "sink", (layer.heads,))},
            parts={"position": position})
    if layer.type == MLSTM:
        qk_width, v_width = layer.heads * layer.dim, layer.heads * layer.vdim
        return PartSpec(
            kind="mlstm",
            params={"hidden_size": width, "heads": layer.heads, "dim": layer.dim, "vdim": layer.vdim,
                    "gate_cap": layer.gate_cap, "eps": eps},
            tensors={"q": TensorRef(mix + "q", (qk_width, width)), "k": TensorRef(mix + "k", (qk_width, width)),
                     "v": TensorRef(mix + "v", (v_width, width)), "gate": TensorRef(mix + "g", (v_width, width)),
                     "out": TensorRef(mix + "o", (width, v_width)), "norm": TensorRef(mix + "norm", (v_width,)),
                     "input_gate": TensorRef(mix + "i", (layer.heads, width)),
                     "input_gate_bias": TensorRef(mix + "i.b", (layer.heads,)),
                     "forget_gate": TensorRef(mix + "f", (layer.heads, width)),
                     "forget_gate_bias": TensorRef(mix + "f.b", (layer.heads,))})
    if layer.type == DELTA:
        qk_width, v_width = layer.kv_heads * layer.dim, layer.heads * layer.vdim
        return PartSpec(
            kind="gated_delta",
            params={"hidden_size": width, "heads": layer.heads, "kv_heads": layer.kv_heads, "dim": layer.dim,
                    "vdim": layer.vdim, "taps": layer.taps, "eps": eps},
            tensors={"q": TensorRef(mix + "q", (qk_width, width)), "q_conv": TensorRef(mix + "q.conv", (qk_width, layer.taps)),
                     "k": TensorRef(mix + "k", (qk_width, width)), "k_conv": TensorRef(mix + "k.conv", (qk_width, layer.taps)),
                     "v": TensorRef(mix + "v", (v_width, width)), "v_conv": TensorRef(mix + "v.conv", (v_width, layer.taps)),
                     "beta": TensorRef(mix + "b", (layer.heads, width)), "decay": TensorRef(mix + "a", (layer.heads, width)),
                     "a_log": TensorRef(mix + "A_log", (layer.heads,)), "dt_bias": TensorRef(mix + "dt_bias", (layer.heads,)),
                     "norm": TensorRef(mix + "norm", (layer.vdim,)), "gate": TensorRef(mix + "g", (v_width, width)),
                     "out": TensorRef(mix + "o", (width, v_width))})
    raise AssertionError(layer.type)


def build_ramosun_spec(config: RamosunConfig) -> ModelSpec:
    width = config.width
    layers = []
    for index, layer in enumerate(config.layers):
        base = f"l{index}"
        feed_forward = feed_forward_norm = None
        if layer.ff is not None:
            feed_forward_norm = _dynamic_tanh(base + ".norm2", width)
            feed_forward = PartSpec(kind="dense",
                                    params={"hidden_size": width, "intermediate_size": layer.ff, "activation": "gelu"},
                                    tensors={"up": TensorRef(base + ".mlp.up", (layer.ff, width)),
                                             "down": TensorRef(base + ".mlp.down", (width, layer.ff))})
        layers.append(LayerSpec(name=base, arrangement="parallel_residual",
                                mixer_norm=_dynamic_tanh(base + ".norm1", width),
                                mixer=_mixer(layer, base, width, config.norm_eps),
                                feed_forward_norm=feed_forward_norm, feed_forward=feed_forward))
    embedding = TensorRef("embed", (config.vocab, width))
    stream_parts = {}
    if config.loop is not None:
        stream_parts[REENTRY] = PartSpec(kind="embedding_reentry", category="stream",
                                         tensors={"table": embedding, "weight": TensorRef("loop.in", (width, 2 * width))})
    order = tuple(ExecutionEntry(layer=index, before=(REENTRY,) if begins_pass else ())
                  for index, begins_pass in config.run_order())
    spec = ModelSpec(
        architecture=config.model_type, vocab_size=config.vocab, hidden_size=width, max_context=config.max_context,
        embedding=embedding, layers=tuple(layers), order=order,
        final_norm=_dynamic_tanh("final.norm", width), lm_head=None,
        eos_token_ids=tuple(config.eos_token_ids), bos_token_id=config.bos_token_id,
        stream_parts=stream_parts, logit_softcap=config.logit_softcap)
    spec.validate()
    return spec


def ramosun_random_init(config: RamosunConfig, name: str, shape: tuple) -> str:
    """Distribution of a tensor in random-weights mode: matrices N(0, 1/fan-in), norm scales around 1, biases,
    sinks, decay and step parameters small, alpha around 0.7."""
    leaf = name.rsplit(".", 1)[-1]
    if leaf == "alpha":
        return "alpha"
    if leaf in ("sink", "A_log", "dt_bias") or name.endswith((".i.b", ".f.b")):
        return "small"
    if leaf == "b" and len(shape) == 1:
        return "small"
    if leaf == "conv":
        return "taps"
    if len(shape) == 1:
        return "norm"
    return "fan_in"


def _parse(raw: Mapping[str, Any]) -> RamosunConfig:
    return RamosunConfig.from_dict(raw)


def _resolve(config: RamosunConfig, tensor_shapes: Mapping[str, Any]) -> RamosunConfig:
    return config


RAMOSUN = Architecture(name="Ramosun", parse_config=_parse, resolve_config=_resolve,
                       build_spec=build_ramosun_spec, random_init=ramosun_random_init)
register_architecture(RAMOSUN, replace=True)
