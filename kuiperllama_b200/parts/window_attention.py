"""Grouped-query attention over a window of recent keys, with the options that softmax attention in the plain
Llama form does not have: biased projections, a norm on q and k heads, interleaved rotary pairs, values of
another size, a sink, sigmoid weights, and pooled blocks before the window."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache import CacheView, KVRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorDecl
from .base import Mixer, PositionEncoding, Runtime, StepContext, register_mixer
from .linear import Linear, StackedInput


@register_mixer("window_attention")
class WindowAttentionMixer(Mixer):
    """q = Wq n (+ bq), k = Wk n (+ bk), v = Wv n (+ bv) or, with ``values`` = "keys", v = k as projected; the first
    ``rotary_dim`` elements of every q and k head turn by the position (either pairing; no rotation without a
    position part); with ``head_norm`` every q and k head is then divided by its root mean square (eps inside the
    root) and multiplied by a weight per element shared by the heads where ``names`` gives ``q_norm`` / ``k_norm``;
    score = (q . k) * ``scale``; token i sees key j when 0 <= i - j < ``window`` (None: every earlier key) and, with
    ``pool`` = P, one mean key and mean value (of the keys and values as the cache holds them) for every block of P
    positions that lies wholly before the window; ``weights`` "softmax" over what is seen (with ``names['sink']`` a
    learned number per head joins the denominator as exp(sink)) or "sigmoid": sigmoid(score + b_h) with
    ``names['head_bias']``, not normalised; head h reads kv head h // (H / KV); out = Wo on the heads side by side.

    One product makes q | k | v; ``ops.qk_prepare`` does bias, rotation, norm and the cache write in one kernel;
    ``ops.pool_blocks`` writes the means of the blocks that the step completes.  Softmax without pooled blocks
    runs on the attention kernels of ``AttentionMixer`` where they take the sizes; a sink, sigmoid weights and pooled blocks
    are options of the windowed tensor-core kernel (bfloat16, equal key and value sizes of 64 or 128, groups of up to 16
    heads); everything else runs on the plain kernels.

    Spec: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``value_dim``, ``scale``, ``window``, ``values``
    ("own" | "keys"), ``weights`` ("softmax" | "sigmoid"), ``pool`` (None), ``head_norm`` (None | {"eps"}), ``names``
    (q, k, o and optionally v, q_bias, k_bias, v_bias, q_norm, k_norm, sink, head_bias).  KuiperLLama's attention is
    the unbiased causal softmax over every earlier key (kuiper/source/model/llama3.cpp:610-639, mha_kernel.cu:61,74-106)."""

    KERNEL = "mma"                # "simt": the plain kernels also for bfloat16 (for comparisons)

    @classmethod
    def manifest(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorDecl]:
        hid, H, KV, hd = spec["hidden_size"], spec["num_heads"], spec["num_kv_heads"], spec["head_dim"]
        vd = spec.get("value_dim") or hd
        n = spec["names"]
        m = {prefix + n["q"]: TensorDecl((H * hd, hid)), prefix + n["k"]: TensorDecl((KV * hd, hid)),
             prefix + n["o"]: TensorDecl((hid, H * vd))}
        if spec.get("values", "own") != "keys":
            m[prefix + n["v"]] = TensorDecl((KV * vd, hid))
        for key, size in (("q_bias", H * hd), ("k_bias", KV * hd), ("v_bias", KV * vd), ("sink", H), ("head_bias", H)):
            if n.get(key):
                m[prefix + n[key]] = TensorDecl((size,), role="vector")
        for key in ("q_norm", "k_norm"):
            if n.get(key):
                m[prefix + n[key]] = TensorDecl((hd,), role="vector", init="one_plus_normal")
        return m

    def __init__(self, spec, prefix, tensors, runtime: Runtime, position: Optional[PositionEncoding] = None):
        super().__init__(spec, prefix, tensors, runtime, position)
        self.hidden = int(spec["hidden_size"])
        self.H, self.KV, self.hd = int(spec["num_heads"]), int(spec["num_kv_heads"]), int(spec["head_dim"])
        self.vd = int(spec.get("value_dim") or self.hd)
        if self.H % self.KV:
            raise ValueError(f"{self.H} heads are not a multiple of {self.KV} kv heads")
        self.values_are_keys = spec.get("values", "own") == "keys"
        if self.values_are_keys and self.vd != self.hd:
            raise ValueError(f"values that are the keys have the keys' size {self.hd}, not {self.vd}")
        self.window = spec.get("window")
        self.pool = int(spec.get("pool") or 0)
        if self.pool and not self.window:
            raise ValueError("pooled blocks lie before a window: a window is needed")
        self.weights = str(spec.get("weights", "softmax"))
        if self.weights not in ops.ATTENTION_WEIGHTS:
            raise ValueError(f"unknown attention weights {self.weights!r} (softmax, sigmoid)")
        self.scale = float(spec["scale"])
        norm = spec.get("head_norm")
        self.head_norm, self.eps = norm is not None, float(norm["eps"]) if norm is not None else 0.0
        n = spec["names"]
        dev = runtime.device
        f32 = lambda key: tensors[prefix + n[key]].to(device=dev, dtype=torch.float32).contiguous() if n.get(key) else None
        self.q_bias, self.k_bias, self.v_bias = f32("q_bias"), f32("k_bias"), f32("v_bias")
        self.q_norm, self.k_norm = f32("q_norm"), f32("k_norm")
        self.sink, self.head_bias = f32("sink"), f32("head_bias")
        if self.sink is not None and self.weights != "softmax":
            raise ValueError("a sink joins a softmax's denominator; sigmoid weights have none")
        self.inputs = StackedInput(runtime)                 # q | k | v from one product
        self.inputs.add("q", tensors[prefix + n["q"]])
        self.inputs.add("k", tensors[prefix + n["k"]])
        if not self.values_are_keys:
            self.inputs.add("v", tensors[prefix + n["v"]])
        self.o = Linear(tensors[prefix + n["o"]], runtime)
        rot = position.rotary() if position is not None else None
        self.inv_freq, self.rotary_dim = rot if rot is not None else (None, 0)
        if position is not None and getattr(position, "magnitude", 1.0) != 1.0:
            raise ValueError("this mixer's kernel rotates with unit magnitude")
        self.interleaved = getattr(position, "pairing", "half") == "interleaved"

    def kv_request(self) -> Optional[KVRequest]:
        value_dim = None if self.vd == self.hd else self.vd
        if self.pool:
            return KVRequest(kv_heads=self.KV, head_dim=self.hd, kind="pooled", window=self.window, value_dim=value_dim, pool=self.pool)
        return KVRequest(kv_heads=self.KV, head_dim=self.hd, kind="full", window=self.window, value_dim=value_dim)

    def forward(self, x, step: StepContext, cache: CacheView) -> torch.Tensor:
        if hasattr(x, "dense"):
            x = x.dense()
        n, dt = step.n_tokens, self.runtime.dtype
        proj = self.inputs.forward(x)
        q_col = self.inputs.column("q")
        write = cache.writable
        ops.qk_prepare(proj, q_col, self.inputs.column("k"), None if self.values_are_keys else self.inputs.column("v"),
                       step.positions, step.token_slot, cache.block_table, cache.k if write else None, cache.v if write else None,
                       n, self.H, self.KV, self.hd, self.vd, q_bias=self.q_bias, k_bias=self.k_bias, v_bias=self.v_bias,
                       inv_freq=self.inv_freq, rotary_dim=self.rotary_dim, interleaved=self.interleaved, head_norm=self.head_norm,
                       eps=self.eps, q_norm_weight=self.q_norm, k_norm_weight=self.k_norm)
        if self.pool and write:
            ops.pool_blocks(cache.k, cache.v, cache.block_table, cache.pooled, step, self.KV, self.hd, self.vd)
        # rows that belong to no sequence (a small step's padding) are not written by the kernels: keep them defined
        make = torch.zeros if n > sum(step.host_new) else torch.empty
        attn = make((n, self.H * self.vd), dtype=dt, device=proj.device)
        q = proj[:, q_col:q_col + self.H * self.hd]
        window = int(self.window or 0)
        if self.weights == "softmax" and not self.pool and self.sink is None and self.vd == self.hd:
            ops.attention(q, proj.stride(0), attn, cache.k, cache.v, cache.block_table, step, self.H, self.KV, self.hd, self.scale, window)
        elif (dt == torch.bfloat16 and self.KERNEL == "mma" and self.vd == self.hd and self.hd in ops.MMA_HEAD_DIMS and self.H // self.KV <= 16
              and proj.stride(0) % 2 == 0 and q.data_ptr() % 4 == 0):
            # the tensor cores: sink, sigmoid weights and pooled rows are options of the windowed kernel
            splits = 1
            if step.is_decode:
                splits = ops.decode_attention_splits(step.n_seqs, self.KV, self.hd, getattr(step, "context_class", 0))
            ops.attention_mma(q, proj.stride(0), attn, cache.k, cache.v, cache.block_table, step.cu_tokens, step.seq_slots, step.seq_starts,
                              step.seq_new, step.n_seqs, step.max_new, n, self.H, self.KV, self.hd, self.scale, window, splits,
                              few_rows=step.is_decode, sink=self.sink, weights=self.weights, head_bias=self.head_bias,
                              pooled=cache.pooled if self.pool else None)
        elif self.weights == "softmax" and not self.pool:
            ops.attention_simt(q, proj.stride(0), attn, cache.k, cache.v, cache.block_table, step.positions, step.token_slot, n,
                               self.H, self.KV, self.hd, self.scale, window, value_dim=self.vd, sink=self.sink)
        else:
            ops.attention_pooled(q, attn, cache.k, cache.v, cache.block_table, step.positions, step.token_slot, n, self.H, self.KV,
                                 self.hd, self.vd, self.scale, window, weights=self.weights, sink=self.sink, head_bias=self.head_bias,
                                 pooled=cache.pooled if self.pool else None)
        return self.o.forward(attn, allow_partials=True)
