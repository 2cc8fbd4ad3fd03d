"""How a layer's parts are arranged in a block."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..cache import CacheView
from .base import DeltaSum, FeedForward, Mixer, Norm, NormedLazy, PostNormed, ResidualGate, StepContext, StreamSink, register_arrangement


@register_arrangement("pre_norm")
class PreNormBlock:
    """x += mixer(norm1(x)); x += feed_forward(norm2(x))
    (ExiledOfCode/KuiperLLama kuiper/source/model/llama3.cpp:155-164, tools/model.py:200-203).

    The residual stream is float32.  A block receives the stream and a *pending* delta that
    the block before it has not added yet; every norm adds the pending delta while it reads
    the row, so no add runs as a kernel of its own.  The block returns the stream and its
    own feed-forward output as the next pending delta (the mixer's, in a layer without a
    feed-forward)."""

    def __init__(self, mixer_norm: Norm, mixer: Mixer, feed_forward_norm: Optional[Norm], feed_forward: Optional[FeedForward]):
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.feed_forward_norm, self.feed_forward = feed_forward_norm, feed_forward

    def forward(self, residual: torch.Tensor, pending, step: StepContext, cache: CacheView):
        # Where the step allows it (decode), a part that can add into the stream itself is given
        # the stream, and a part that can normalise the stream's rows itself is given them lazily.
        fuse = step.allow_stream_fusion
        after = step.next_norm                       # the norm that receives this block's pending result

        def sink_for(part, norm):
            ok = fuse and part.may_accumulate and norm is not None and getattr(norm, "accepts_accumulated", False)
            return StreamSink(residual, norm) if ok else None

        n = self.mixer_norm.forward(residual, pending, step.n_tokens)
        if isinstance(n, NormedLazy) and not self.mixer.accepts_lazy_norm:
            n = n.dense()
        if self.feed_forward is None:
            step.residual_sink = sink_for(self.mixer, after)
            mixed = self.mixer.forward(n, step, cache)
            step.residual_sink = None
            return residual, mixed
        step.residual_sink = sink_for(self.mixer, self.feed_forward_norm)
        mixed = self.mixer.forward(n, step, cache)
        n = self.feed_forward_norm.forward(residual, mixed, step.n_tokens)
        if isinstance(n, NormedLazy) and not self.feed_forward.accepts_lazy_norm:
            n = n.dense()
        step.residual_sink = sink_for(self.feed_forward, after)
        out = self.feed_forward.forward(n, step)
        step.residual_sink = None
        return residual, out


@register_arrangement("sandwich")
class SandwichBlock:
    """A norm before and a norm after every sublayer, and optionally a gate on its result:

        h = norm1(x);  x += norm1b(gate1(h) * mixer(h))
        h = norm2(x);  x += norm2b(gate2(h) * feed_forward(h))        (left out without a feed-forward)

    with gate(h) = sigmoid(R h + r).  As in the pre-norm block the stream is float32 and no add
    runs as a kernel of its own: a sublayer's result travels as ``PostNormed`` to the norm that
    reads the stream next, whose kernel gates it, norms it, adds it and norms the sum.
    KuiperLLama has the pre-norm block alone (kuiper/source/model/llama3.cpp:155-164)."""

    def __init__(self, mixer_norm: Norm, mixer: Mixer, feed_forward_norm: Optional[Norm], feed_forward: Optional[FeedForward],
                 mixer_post_norm: Optional[Norm] = None, feed_forward_post_norm: Optional[Norm] = None,
                 mixer_gate: Optional[ResidualGate] = None, feed_forward_gate: Optional[ResidualGate] = None):
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.feed_forward_norm, self.feed_forward = feed_forward_norm, feed_forward
        self.mixer_post_norm, self.feed_forward_post_norm = mixer_post_norm, feed_forward_post_norm
        self.mixer_gate, self.feed_forward_gate = mixer_gate, feed_forward_gate
        if mixer_gate is not None:
            mixer_gate.attach(mixer)
        if feed_forward_gate is not None and feed_forward is not None:
            feed_forward_gate.attach(feed_forward)

    @staticmethod
    def _result(y, h, gate: Optional[ResidualGate], norm: Optional[Norm]) -> PostNormed:
        if gate is None:                                 # y may be float32 pieces of a product: the norm kernel adds them
            return PostNormed(y, norm=norm)
        return PostNormed(y, gate=gate.pre_activation(h), gate_bias=gate.bias, norm=norm)

    def forward(self, residual: torch.Tensor, pending, step: StepContext, cache: CacheView):
        step.residual_sink = None
        h = self.mixer_norm.forward(residual, pending, step.n_tokens)
        if isinstance(h, NormedLazy):
            h = h.dense()
        pending = self._result(self.mixer.forward(h, step, cache), h, self.mixer_gate, self.mixer_post_norm)
        if self.feed_forward is None:
            return residual, pending
        h = self.feed_forward_norm.forward(residual, pending, step.n_tokens)
        if isinstance(h, NormedLazy):
            h = h.dense()
        return residual, self._result(self.feed_forward.forward(h, step), h, self.feed_forward_gate, self.feed_forward_post_norm)


@register_arrangement("parallel")
class ParallelBlock:
    """Both sublayers read the same stream and their results are added together:

        x += (mixer(norm1(x)) + feed_forward(norm2(x)))          (x += mixer(norm1(x)) without a feed-forward)

    The two RMS norms share their root mean square, so one kernel adds what the block before left
    pending (32-bit), writes the stream and makes both normalised rows; the block's own two results
    travel on as ``DeltaSum`` to the norm that reads the stream next.  Norms of other kinds run one
    after the other.  KuiperLLama has the sequential pre-norm block alone
    (kuiper/source/model/llama3.cpp:155-164)."""

    def __init__(self, mixer_norm: Norm, mixer: Mixer, feed_forward_norm: Optional[Norm], feed_forward: Optional[FeedForward]):
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.feed_forward_norm, self.feed_forward = feed_forward_norm, feed_forward

    def forward(self, residual: torch.Tensor, pending, step: StepContext, cache: CacheView):
        step.residual_sink = None
        a, b = self.mixer_norm, self.feed_forward_norm if self.feed_forward is not None else None
        if b is not None and hasattr(a, "forward_pair") and type(a) is type(b) and a.eps == b.eps:
            h1, h2 = a.forward_pair(residual, pending, b)
        else:
            h1 = a.forward(residual, pending, step.n_tokens)
            if isinstance(h1, NormedLazy):
                h1 = h1.dense()
            h2 = b.forward(residual, None, step.n_tokens) if b is not None else None
        mixed = self.mixer.forward(h1, step, cache)
        if self.feed_forward is None:
            return residual, mixed
        return residual, DeltaSum(mixed, self.feed_forward.forward(h2, step))
