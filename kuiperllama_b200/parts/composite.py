"""Mixers made of other mixers: a short convolution in front of one, and several side by side."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache import CacheView, KVRequest, StateRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorDecl
from .base import Mixer, NormedLazy, PositionEncoding, Runtime, StepContext, part_class, register_mixer
from .linear import Linear, StackedInput


def _state_size(req: Optional[StateRequest]) -> int:
    if req is None:
        return 0
    if req.dtype != torch.float32:
        raise ValueError("mixers inside a composite mixer keep float32 state")
    n = 1
    for s in req.shape:
        n *= int(s)
    return n


def _view(cache: CacheView, state: Optional[torch.Tensor], with_kv: bool) -> CacheView:
    """What one inner mixer sees: its columns of the slot's state and, if it is the one that asked for them, the pages."""
    return CacheView(k=cache.k if with_kv else None, v=cache.v if with_kv else None,
                     block_table=cache.block_table if with_kv else None, state=state, writable=cache.writable)


class BranchMixer(Mixer):
    """A mixer that can also run as one branch of ``ParallelMixer``: its input projections may ride on a product it
    shares with other branches, and its result before the output projection may go into a column slice of a shared
    buffer, times a factor.  A subclass gives ``core_width`` (the output projection's input size), ``o_weight``
    [hidden, core_width], ``add_inputs(stacked, tag)`` and ``core(stacked, tag, step, cache, out, out_scale)``; this base
    makes an ordinary mixer of it."""

    core_width: int
    o_weight: torch.Tensor

    def add_inputs(self, stacked: StackedInput, tag: str) -> None:
        raise NotImplementedError

    def core(self, stacked: StackedInput, tag: str, step: StepContext, cache: CacheView, out: torch.Tensor, out_scale: float) -> None:
        raise NotImplementedError

    def _alone(self):
        if getattr(self, "_inputs", None) is None:
            self._inputs = StackedInput(self.runtime)
            self.add_inputs(self._inputs, "")
            self._o = Linear(self.o_weight, self.runtime)
        return self._inputs, self._o

    def forward(self, x, step: StepContext, cache: CacheView) -> torch.Tensor:
        if isinstance(x, NormedLazy):
            x = x.dense()
        inputs, o = self._alone()
        inputs.forward(x)
        # rows that belong to no sequence (a small step's padding) are not written by the kernels: keep them defined
        make = torch.empty if step.n_tokens == step.n_seqs else torch.zeros
        act = make((step.n_tokens, self.core_width), dtype=self.runtime.dtype, device=x.device)
        self.core(inputs, "", step, cache, act, 1.0)
        return o.forward(act, allow_partials=True)


@register_mixer("input_conv")
class InputConvMixer(Mixer):
    """A short causal convolution in front of another mixer, added to its input: the inner mixer reads

        h'_t = h_t + sum_j w[:, j] * h_(t - taps + 1 + j)           (one filter of ``taps`` per channel, no bias)

    with nothing before a sequence's first token.  The last taps - 1 inputs are state of the sequence: the slot's state is
    the inner mixer's, then [taps - 1, hidden] float32.  The sum runs in 32 bits.  Spec: ``hidden_size``, ``taps``, the
    filter's ``name`` and ``inner``, the ``PartSpec`` of the mixer behind it.  KuiperLLama has no convolution
    (kuiper/source/model/llama3.cpp:146-166)."""

    @classmethod
    def manifest(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorDecl]:
        inner = spec["inner"]
        m = dict(part_class("mixer", inner.kind).manifest(inner, prefix))
        m[prefix + spec["name"]] = TensorDecl((spec["hidden_size"], spec["taps"]), role="vector")
        return m

    def __init__(self, spec, prefix, tensors, runtime: Runtime, position: Optional[PositionEncoding] = None):
        super().__init__(spec, prefix, tensors, runtime, position)
        self.hidden, self.taps = int(spec["hidden_size"]), int(spec["taps"])
        if not 1 <= self.taps <= ops.SHORT_CONV_MAX_TAPS:
            raise ValueError(f"the convolution kernel takes 1 to {ops.SHORT_CONV_MAX_TAPS} taps, got {self.taps}")
        inner = spec["inner"]
        self.inner = part_class("mixer", inner.kind)(inner, prefix, tensors, runtime, position)
        self.weight = tensors[prefix + spec["name"]].to(device=runtime.device, dtype=torch.float32).contiguous()
        self.inner_state = _state_size(self.inner.state_request())
        self.own_state = (self.taps - 1) * self.hidden
        self._no_state = None

    def kv_request(self) -> Optional[KVRequest]:
        return self.inner.kv_request()

    def state_request(self) -> Optional[StateRequest]:
        total = self.inner_state + self.own_state
        return StateRequest((total,), torch.float32) if total else None

    def forward(self, x, step: StepContext, cache: CacheView) -> torch.Tensor:
        if isinstance(x, NormedLazy):
            x = x.dense()
        make = torch.empty if step.n_tokens == step.n_seqs else torch.zeros
        h = make((step.n_tokens, self.hidden), dtype=self.runtime.dtype, device=x.device)
        if self.own_state:
            own = cache.state[:, self.inner_state:]
        else:                                   # one tap: nothing is carried; the kernel still wants an address
            if self._no_state is None:
                self._no_state = torch.zeros((1, 1), dtype=torch.float32, device=x.device)
            own = self._no_state.expand(cache.state.shape[0] if cache.state is not None else 1, 1)
        ops.short_conv(x, self.weight, None, own, step, h, add_input=True, update_state=cache.writable)
        inner_state = cache.state[:, :self.inner_state] if self.inner_state else None
        return self.inner.forward(h, step, _view(cache, inner_state, True))


@register_mixer("parallel")
class ParallelMixer(Mixer):
    """Several mixers side by side that read the same rows; the result is sum_b scale_b * branch_b(h).

    Branches are ``BranchMixer``s: all their input projections are one product, every branch writes what goes into its
    output projection (times its scale, in 32 bits before the rounding) into its columns of one buffer, and the output
    projections, laid side by side, are one product too.  At most one branch may ask for pages of keys and values; the
    slot's state is the branches' states one after the other.  Spec: ``branches``: a list of {"mixer": PartSpec,
    "scale": number}.  KuiperLLama's layers have one mixer (kuiper/source/model/llama3.cpp:651-675)."""

    @classmethod
    def manifest(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorDecl]:
        m: Dict[str, TensorDecl] = {}
        for b in spec["branches"]:
            m.update(part_class("mixer", b["mixer"].kind).manifest(b["mixer"], prefix))
        return m

    def __init__(self, spec, prefix, tensors, runtime: Runtime, position: Optional[PositionEncoding] = None):
        super().__init__(spec, prefix, tensors, runtime, position)
        self.branches: List[BranchMixer] = []
        self.scales: List[float] = []
        for b in spec["branches"]:
            part = part_class("mixer", b["mixer"].kind)(b["mixer"], prefix, tensors, runtime, position)
            if not isinstance(part, BranchMixer):
                raise ValueError(f"a {b['mixer'].kind!r} mixer cannot run as a branch of a parallel mixer")
            self.branches.append(part)
            self.scales.append(float(b.get("scale", 1.0)))
        if not self.branches:
            raise ValueError("a parallel mixer needs at least one branch")
        if sum(1 for p in self.branches if p.kv_request() is not None) > 1:
            raise ValueError("at most one branch of a parallel mixer may keep keys and values")
        self.inputs = StackedInput(runtime)
        self.offsets, self.state_offsets = [], []
        width = state = 0
        for i, p in enumerate(self.branches):
            p.add_inputs(self.inputs, f"b{i}.")
            self.offsets.append(width)
            width += -(-p.core_width // StackedInput.ALIGN) * StackedInput.ALIGN       # every branch's columns start on a 16-byte boundary
            self.state_offsets.append(state)
            state += _state_size(p.state_request())
        self.width, self.state_total = width, state
        dev, dt = runtime.device, runtime.dtype
        o = torch.zeros((self.branches[0].o_weight.shape[0], width), dtype=dt, device=dev)
        for p, at in zip(self.branches, self.offsets):
            o[:, at:at + p.core_width] = p.o_weight.to(device=dev, dtype=dt)
        self.o = Linear(o, runtime)

    def kv_request(self) -> Optional[KVRequest]:
        return next((r for r in (p.kv_request() for p in self.branches) if r is not None), None)

    def state_request(self) -> Optional[StateRequest]:
        return StateRequest((self.state_total,), torch.float32) if self.state_total else None

    def forward(self, x, step: StepContext, cache: CacheView) -> torch.Tensor:
        if isinstance(x, NormedLazy):
            x = x.dense()
        self.inputs.forward(x)
        # padding columns between the branches meet zero weights, but must hold numbers: zeros
        act = torch.zeros((step.n_tokens, self.width), dtype=self.runtime.dtype, device=x.device)
        for i, p in enumerate(self.branches):
            size = _state_size(p.state_request())
            at = self.state_offsets[i]
            state = cache.state[:, at:at + size] if size else None
            p.core(self.inputs, f"b{i}.", step, _view(cache, state, p.kv_request() is not None),
                   act[:, self.offsets[i]:self.offsets[i] + p.core_width], self.scales[i])
        return self.o.forward(act, allow_partials=True)
