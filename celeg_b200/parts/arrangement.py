"""Block arrangements: how a layer's norms, mixer and feed-forward sit around the residual
stream. Interface:

    Arrangement(layer_parts, rt)     layer_parts: dict with mixer_norm, mixer, feed_forward_norm,
                                     feed_forward (the last two may be None)
    run(stream, step)                stream: the step's ResidualStream, updated in place;
                                     stream.after_layer is the norm that will read the stream after this
                                     layer if its reader takes a split norm (see ResidualStream), else None
    first_norm(step)                 optional: the norm that reads the stream first, under the same condition

A part's ``forward(x, out, step)`` gets the normed activations and a buffer for its output; the
arrangement hands that buffer to the residual stream, which adds it inside the next norm kernel.
"""
from __future__ import annotations

from typing import Mapping

import torch

from .registry import register_part
from .runtime import ResidualStream, Runtime, StepContext


@register_part("arrangement", "prenorm_residual")
class PreNormResidual:
    """h = x + Mixer(Norm(x)); y = h + FeedForward(Norm(h))
    (celeg src/backend/cpu/model_forward_token.cpp:89-176; src/backend/cuda/packed/layer_executor.cu:101-216)."""

    def __init__(self, layer_parts: Mapping, rt: Runtime):
        self.rt = rt
        self.mixer_norm = layer_parts["mixer_norm"]
        self.mixer = layer_parts["mixer"]
        self.ffn_norm = layer_parts.get("feed_forward_norm")
        self.ffn = layer_parts.get("feed_forward")
        hidden = self.mixer_norm.width
        self.normed = rt.scratch("block.normed", hidden)
        self.delta_a = rt.scratch("block.delta_a", hidden)
        self.delta_b = rt.scratch("block.delta_b", hidden)

    def _sublayer(self, norm, part, delta, upcoming, stream: ResidualStream, step: StepContext) -> None:
        x = stream.normed(norm, self.normed, step.tokens)
        stream.expect(delta, upcoming if getattr(part, "ends_with_product", False) else None, step.tokens)
        part.forward(x, delta, step)
        stream.add_later(delta)

    def first_norm(self, step: StepContext):
        """The norm that reads the stream first, if its reader takes a split norm (else None)."""
        takes = getattr(self.mixer, "takes_split_norm", None)
        return self.mixer_norm if takes is not None and takes(step) else None

    def run(self, stream: ResidualStream, step: StepContext) -> None:
        after = stream.after_layer
        if self.ffn is None:
            self._sublayer(self.mixer_norm, self.mixer, self.delta_a, after, stream, step)
            return
        takes = getattr(self.ffn, "takes_split_norm", None)
        between = self.ffn_norm if takes is not None and takes(step) else None
        self._sublayer(self.mixer_norm, self.mixer, self.delta_a, between, stream, step)
        self._sublayer(self.ffn_norm, self.ffn, self.delta_b, after, stream, step)


@register_part("arrangement", "parallel_residual")
class ParallelResidual:
    """y = x + Mixer(Norm_1(x)) + FeedForward(Norm_2(x)): both read the same x, each through its own norm, and
    both outputs are owed to the stream together (added inside the next block's norm pass). Without a
    feed-forward: y = x + Mixer(Norm_1(x)). A block that names a feed-forward but no second norm has ONE norm whose
    output both read: y = x + Mixer(h) + FeedForward(h), h = Norm_1(x). A stream part under the name ``after``
    among the layer's parts runs when both outputs are owed (it settles them itself)."""

    def __init__(self, layer_parts: Mapping, rt: Runtime):
        self.rt = rt
        self.mixer_norm = layer_parts["mixer_norm"]
        self.mixer = layer_parts["mixer"]
        self.ffn_norm = layer_parts.get("feed_forward_norm")
        self.ffn = layer_parts.get("feed_forward")
        self.after = layer_parts.get("after")
        hidden = self.mixer_norm.width
        self.normed_a = rt.scratch("block.normed", hidden)
        self.normed_b = rt.scratch("block.normed_b", hidden) if self.ffn_norm is not None else None
        self.delta_a = rt.scratch("block.delta_a", hidden)
        self.delta_b = rt.scratch("block.delta_b", hidden)

    def entry_norm(self):
        """(norm, buffer) of the first thing run() asks of the stream: that norm of every row, into that buffer."""
        return self.mixer_norm, self.normed_a

    def run(self, stream: ResidualStream, step: StepContext) -> None:
        stream.expect(self.delta_a, None, step.tokens)
        if self.ffn is None:
            x = stream.normed(self.mixer_norm, self.normed_a, step.tokens)
            self.mixer.forward(x, self.delta_a, step)
            stream.add_later(self.delta_a)
            if self.after is not None:
                self.after.run(stream, step)
            return
        if self.ffn_norm is None:
            x_mixer = x_ffn = stream.normed(self.mixer_norm, self.normed_a, step.tokens)
        else:
            x_mixer, x_ffn = stream.normed_pair(self.mixer_norm, self.normed_a, self.ffn_norm, self.normed_b, step.tokens)
        rt = self.rt
        if rt.side_by_side_branches and rt.small_batch(step.tokens):
            # few rows: both chains are short kernels that leave most of the GPU idle, and they share nothing but
            # their input's source. The feed-forward goes to a second stream (two branches of the step's graph
            # when it is captured) and is joined before anything reads the stream again.
            main, side = torch.cuda.current_stream(rt.device), rt.side_stream()
            fork = torch.cuda.Event()
            fork.record(main)
            side.wait_event(fork)
            with torch.cuda.stream(side):
                self.ffn.forward(x_ffn, self.delta_b, step)
                join = torch.cuda.Event()
                join.record(side)
            self.mixer.forward(x_mixer, self.delta_a, step)
            main.wait_event(join)
        else:
            self.mixer.forward(x_mixer, self.delta_a, step)
            self.ffn.forward(x_ffn, self.delta_b, step)
        stream.add_later(self.delta_a)
        stream.add_later_beside(self.delta_b)
        if self.after is not None:
            self.after.run(stream, step)
