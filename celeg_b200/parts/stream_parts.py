"""Parts that rewrite the residual stream between two blocks (category "stream"). Interface:

    StreamPart(params, weights, parts, rt)
    run(stream, step)        stream: the step's ResidualStream; what is owed to it is the part's to settle

A position of the run order names the stream parts that run before its block.
"""
from __future__ import annotations

from typing import Mapping

import torch

from .. import kernels
from .registry import register_part
from .runtime import ResidualStream, Runtime, StepContext


@register_part("stream", "embedding_reentry")
class EmbeddingReentry:
    """x <- W [x; x0] with x0 the embedding rows of the step's tokens (W is [width, 2 width], x first): what a
    run of layers that is repeated with the same weights is entered through, every time. The result replaces
    the stream, in float32."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.table = rt.matrix(weights["table"])
        self.weight = rt.matrix(weights["weight"])
        self.multiplier = float(params.get("multiplier", 1.0))
        width = int(self.table.shape[1])
        if tuple(self.weight.shape) != (width, 2 * width):
            raise ValueError(f"embedding_reentry weight has shape {tuple(self.weight.shape)}, expected "
                             f"({width}, {2 * width})")
        self.joined = rt.scratch("reentry.joined", 2 * width)

    def run(self, stream: ResidualStream, step: StepContext) -> None:
        if stream.prepared is not None:
            raise RuntimeError("a norm was prepared for another reader than the stream part that runs")
        t = step.tokens
        kernels.join_stream_embedding(stream.residual, stream.pending, stream.pending_b, self.table,
                                      step.token_ids[:t], self.joined, t, self.multiplier)
        stream.pending = stream.pending_b = None
        self.rt.linear(self.joined, self.weight, stream.residual, t)


@register_part("stream", "depth_average")
class DepthAverage:
    """After block ``index``: the block's result X_(index+1) = stream + what the block's parts owe it is kept, and the
    stream becomes sum_j weights[j] X_j over j = 0 .. index + 1, X_0 the embedding output (a weighted average over
    depth; Pagliardini et al., "DenseFormer: Enhancing Information Flow in Transformers via Depth Weighted
    Averaging", 2024). All blocks of a model share one history [entries, rows, width] in float32, rewritten every
    step. When the stream says which norm reads it next (``stream.upcoming``), that norm's output is written in the
    same pass and left for the reader (``stream.ready``)."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.index = int(params["index"])
        self.entries = int(params["entries"])
        self.width = int(params["width"])
        if not 0 <= self.index < self.entries - 1:
            raise ValueError(f"depth_average: block {self.index} of a history of {self.entries} entries")
        self.weights = rt.vector(weights["weights"].reshape(-1))
        if self.weights.numel() != self.index + 2:
            raise ValueError(f"depth_average: block {self.index} needs {self.index + 2} weights, got {self.weights.numel()}")
        self.history = rt.flat_scratch("depth_average.history", self.entries * rt.max_tokens * self.width,
                                       torch.float32).view(self.entries, rt.max_tokens, self.width)

    def run(self, stream: ResidualStream, step: StepContext) -> None:
        if stream.prepared is not None:
            raise RuntimeError("a norm was prepared for another reader than the stream part that runs")
        t = step.tokens
        upcoming = stream.upcoming
        halves = upcoming[0].as_prologue() if upcoming is not None and hasattr(upcoming[0], "as_prologue") else None
        if halves is not None and upcoming[0].width == self.width:
            norm, out = upcoming
            weight, eps = halves
            kernels.depth_average(stream.residual, stream.pending, stream.pending_b, self.history, self.weights,
                                  self.index, t, norm_weight=weight, out=out, eps=eps)
            stream.ready = (norm, out)
        else:
            kernels.depth_average(stream.residual, stream.pending, stream.pending_b, self.history, self.weights,
                                  self.index, t)
        stream.pending = stream.pending_b = None
