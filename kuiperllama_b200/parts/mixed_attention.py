"""Softmax attention without rotation whose heads exchange their weights after the softmax."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache import CacheView, KVRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorDecl
from .base import PositionEncoding, Runtime, StepContext, register_mixer
from .composite import BranchMixer
from .linear import StackedInput


@register_mixer("mixed_head_attention")
class MixedHeadAttentionMixer(BranchMixer):
    """q = Wq n (heads x dim), k = Wk n (kv_heads x dim), v = Wv n (kv_heads x vdim), no biases, no rotation; head h reads
    key/value head h // (heads / kv_heads).  For a query at position i and a key at j:

        s = scale * (q . k);   s <- softcap * tanh(s / softcap)   (where a soft cap is given);
        s <- s - r1_h * ln(1 + r2_h * (i - j))                    (where the distance bias is given: two numbers per head)
        visible: j <= i and (i - j < window or j < keep_first)    (no window: every earlier key)

    an ordinary softmax over the visible keys; then the heads' weights are mixed, w_h(i, j) = sum_g talk[h, g] p_g(i, j)
    (where ``talk`` is given), head h applies its mixed weights to the values of its own key/value head, its result is
    multiplied by sigmoid of one number per head (Wg n, where a gate is given), and the output projection follows.
    Kept first keys keep their true distances.  Scores, weights and sums are 32-bit.  The cache holds keys and values in
    pages of their own sizes; pages that neither the window nor the kept first keys reach go back to the pool.

    Spec: ``hidden_size``, ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``softcap`` (None: none), ``window`` (None: none),
    ``keep_first`` and ``names``: q, k, v, o and optionally r1, r2, talk, g.  KuiperLLama's attention is
    mha_kernel.cu:61,74-106 (rotated, every earlier key, scale fixed at head_dim ** -0.5)."""

    @classmethod
    def manifest(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorDecl]:
        hid, H, G, d, dv, n = (spec[k] for k in ("hidden_size", "heads", "kv_heads", "dim", "vdim", "names"))
        m = {prefix + n["q"]: TensorDecl((H * d, hid)), prefix + n["k"]: TensorDecl((G * d, hid)),
             prefix + n["v"]: TensorDecl((G * dv, hid)), prefix + n["o"]: TensorDecl((hid, H * dv))}
        for key in ("r1", "r2"):
            if n.get(key):
                m[prefix + n[key]] = TensorDecl((H,), role="vector", init="one_plus_normal")
        if n.get("talk"):
            m[prefix + n["talk"]] = TensorDecl((H, H), role="vector")
        if n.get("g"):
            m[prefix + n["g"]] = TensorDecl((H, hid))
        return m

    def __init__(self, spec, prefix, tensors, runtime: Runtime, position: Optional[PositionEncoding] = None):
        super().__init__(spec, prefix, tensors, runtime, position)
        self.hidden = int(spec["hidden_size"])
        self.H, self.G, self.d, self.dv = (int(spec[k]) for k in ("heads", "kv_heads", "dim", "vdim"))
        if self.H % self.G:
            raise ValueError(f"{self.H} heads are not a multiple of {self.G} key/value heads")
        self.scale = float(spec["scale"])
        self.softcap = float(spec.get("softcap") or 0.0)
        self.window = int(spec.get("window") or 0)
        self.keep_first = int(spec.get("keep_first") or 0) if self.window else 0
        n = spec["names"]
        if bool(n.get("r1")) != bool(n.get("r2")):
            raise ValueError("the distance bias needs both of its numbers per head (r1 and r2)")
        self._w = {k: tensors[prefix + n[k]] for k in ("q", "k", "v") + (("g",) if n.get("g") else ())}
        self.gated = bool(n.get("g"))
        self.o_weight = tensors[prefix + n["o"]]
        self.core_width = self.H * self.dv
        f32 = lambda name: tensors[prefix + name].to(device=runtime.device, dtype=torch.float32).contiguous()
        self.r1 = f32(n["r1"]) if n.get("r1") else None
        self.r2 = f32(n["r2"]) if n.get("r2") else None
        self.talk = f32(n["talk"]) if n.get("talk") else None

    def kv_request(self) -> Optional[KVRequest]:
        return KVRequest(kv_heads=self.G, head_dim=self.d, kind="full", window=self.window or None,
                         value_dim=self.dv if self.dv != self.d else None, keep_first=self.keep_first)

    def add_inputs(self, stacked: StackedInput, tag: str) -> None:
        for k in ("q", "k", "v") + (("g",) if self.gated else ()):
            stacked.add(tag + k, self._w[k])
        self._w = None

    def core(self, stacked: StackedInput, tag: str, step: StepContext, cache: CacheView, out: torch.Tensor, out_scale: float) -> None:
        proj = stacked.last
        if cache.writable:
            ops.kv_append(proj, stacked.column(tag + "k"), stacked.column(tag + "v"), cache.k, cache.v, cache.block_table, step,
                          self.G, self.d, self.dv)
        ops.attention_mixed(stacked.view(tag + "q"), stacked.view(tag + "g") if self.gated else None, out, cache.k, cache.v,
                            cache.block_table, step, self.H, self.G, self.d, self.dv, self.scale, self.softcap, self.r1, self.r2, self.talk,
                            self.window, self.keep_first, out_scale)
