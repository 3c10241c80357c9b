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
