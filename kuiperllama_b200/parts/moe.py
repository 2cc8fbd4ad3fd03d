"""A mixture of experts as a feed-forward: a router, a grouped product per projection, a weighted sum."""
from __future__ import annotations

import os
from typing import Dict

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorDecl
from .base import FeedForward, NormedLazy, Runtime, StepContext, register_feed_forward
from .linear import Linear


@register_feed_forward("moe")
class MoEFeedForward(FeedForward):
    """``experts`` small gated feed-forwards of which every token uses ``top``:

        z = W_router n (32-bit);  s = softmax(z) over all experts;  the ``top`` largest s are chosen
        expert e:  g = min(W_gate[e] n, limit), u = clamp(W_up[e] n, -limit, limit),
                   f_e = W_down[e] (g * sigmoid(alpha * g) * (u + shift))          (no clamp when limit is None)
        out = sum over the chosen e of s_e * f_e     (the weights are divided by their sum + ``renorm_eps`` if ``renormalise``)

    With ``gated`` False an expert has no gate: f_e = W_down[e] act(W_up[e] n) with ``activation`` one of the element-wise
    activations (``ops.ACTIVATIONS``).  ``names['router_bias']``: a bias per expert joins the router's logits (32 bits).  With
    ``renormalise`` and no ``renorm_eps`` the weights are the softmax over the chosen logits alone.  ``shared_size``: one more
    expert of that size and of the ungated form (``names['shared_up']``, ``names['shared_down']``) runs for every token and is
    added, as a second float32 piece.

    With ``groups`` > 1 the experts form that many equal groups of neighbours; a group's score is the largest score in
    it, and only experts of the ``keep_groups`` best groups can be chosen.

    Routing stays on the device (``ops.moe_route`` / ``moe_plan``): the (token, choice) pairs are sorted by
    expert into a list padded to whole tiles, one grouped product makes gate, up and the activation for
    the whole list, one more the down projection, and ``moe_combine`` adds each token's results in the
    order of its choices in 32 bits.  The result is handed on as one float32 piece.  The grouped products run on the
    tensor cores where the sizes allow (bfloat16, expert size % 64, hidden size % 8): tokens as tile rows from
    ``TENSOR_CORE_ROWS_PER_EXPERT`` rows per expert on, weights as tile rows below (a decode step); on FMA kernels
    otherwise (float32, odd sizes).

    Spec: ``hidden_size``, ``experts``, ``top``, ``expert_size``, ``limit``, ``alpha``, ``shift``, ``renormalise``,
    ``renorm_eps``, ``groups``, ``keep_groups``, ``gated``, ``activation``, ``shared_size``, ``names``: router and, with ``{e}`` for the
    expert's number, gate, up, down.  KuiperLLama's only feed-forward is
    the dense SwiGLU (kuiper/source/model/llama3.cpp:692-718)."""

    # Mean rows per expert from which the list is cut into tiles of 128 for the tensor cores.  Measured at width 2,048 with 16
    # experts of 2,048 (ms per decode step of 16 layers): 64 sequences (16 rows per expert) 3.15 on the tensor cores against 9.5 on
    # the warp-per-rows form; 8 sequences (2 rows per expert) 2.08 with weights as tile rows, 2.76 on the warp-per-rows form.
    TENSOR_CORE_ROWS_PER_EXPERT = 8
    SKINNY = os.environ.get("KL_MOE_SKINNY", "tcgen05")     # "gemv": the warp-per-rows form (for comparisons)

    @classmethod
    def manifest(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorDecl]:
        hid, E, ff, n = spec["hidden_size"], spec["experts"], spec["expert_size"], spec["names"]
        m = {prefix + n["router"]: TensorDecl((E, hid))}
        if n.get("router_bias"):
            m[prefix + n["router_bias"]] = TensorDecl((E,), role="vector")
        for e in range(E):
            if spec.get("gated", True):
                m[prefix + n["gate"].format(e=e)] = TensorDecl((ff, hid))
            m[prefix + n["up"].format(e=e)] = TensorDecl((ff, hid))
            m[prefix + n["down"].format(e=e)] = TensorDecl((hid, ff))
        if spec.get("shared_size"):
            m[prefix + n["shared_up"]] = TensorDecl((spec["shared_size"], hid))
            m[prefix + n["shared_down"]] = TensorDecl((hid, spec["shared_size"]))
        return m

    def __init__(self, spec, prefix, tensors, runtime: Runtime):
        super().__init__(spec, prefix, tensors, runtime)
        self.hidden, self.E, self.top, self.ff = (int(spec[k]) for k in ("hidden_size", "experts", "top", "expert_size"))
        if not 0 < self.top <= self.E <= ops.MOE_MAX_EXPERTS:
            raise ValueError(f"{self.top} of {self.E} experts: the routing kernels take up to {ops.MOE_MAX_EXPERTS} experts")
        limit = spec.get("limit")
        self.activation = (float(limit) if limit is not None else 0.0, float(spec.get("alpha", 1.0)), float(spec.get("shift", 0.0)))
        self.renormalise = bool(spec.get("renormalise", False))
        self.renorm_eps = float(spec.get("renorm_eps", 0.0))
        self.groups, self.keep_groups = int(spec.get("groups", 1)), int(spec.get("keep_groups", 1))
        if self.E % self.groups or not 1 <= self.keep_groups <= self.groups or self.top > self.keep_groups * (self.E // self.groups):
            raise ValueError(f"{self.E} experts in {self.groups} groups of which {self.keep_groups} are kept do not hold {self.top} choices")
        n = spec["names"]
        dev, dt = runtime.device, runtime.dtype
        get = lambda key, e: tensors[prefix + n[key].format(e=e)].to(device=dev, dtype=dt)
        self.router = Linear(tensors[prefix + n["router"]], runtime)
        self.router_bias = None
        if n.get("router_bias"):
            self.router_bias = tensors[prefix + n["router_bias"]].to(device=dev, dtype=torch.float32).contiguous()
        self.gated = bool(spec.get("gated", True))
        self.act_kind = str(spec.get("activation", "relu2"))
        if not self.gated and self.act_kind not in ops.ACTIVATIONS:
            raise ValueError(f"unknown activation {self.act_kind!r} (known: {', '.join(sorted(ops.ACTIVATIONS))})")
        if self.gated:
            # [experts, 2 ff, hidden]: an expert's gate rows, then its up rows (or, where the tensor-core product can run,
            # blocks of 64 gate rows and the 64 up rows of the same outputs); [experts, hidden, ff]
            self.tensor_cores = dt == torch.bfloat16 and self.ff % 64 == 0 and self.hidden % 8 == 0
            stack = ops.interleave_gate_up if self.tensor_cores else (lambda g, u: torch.cat([g, u], dim=0))
            self.gate_up = torch.stack([stack(get("gate", e), get("up", e)) for e in range(self.E)]).contiguous()
        else:
            # [experts, ff, hidden]: the up rows alone
            self.tensor_cores = dt == torch.bfloat16 and self.ff % 8 == 0 and self.hidden % 8 == 0
            self.gate_up = torch.stack([get("up", e) for e in range(self.E)]).contiguous()
            self.activation = None
        # the up product's epilogue applies the ungated activation itself where it can; a kernel of its own follows otherwise
        self.fused_act = self.act_kind if not self.gated and self.act_kind in ops.EPILOGUE_ACTIVATIONS else None
        self.down = torch.stack([get("down", e) for e in range(self.E)]).contiguous()
        self.shared_size = int(spec.get("shared_size") or 0)
        if self.shared_size:
            self.shared_up = Linear(tensors[prefix + n["shared_up"]], runtime)
            self.shared_down = Linear(tensors[prefix + n["shared_down"]], runtime)

    def _activate(self, act: torch.Tensor) -> None:
        if not self.gated and self.fused_act is None:
            ops.activation(act, act, self.act_kind)

    def forward(self, x, step: StepContext):
        if isinstance(x, NormedLazy):
            x = x.dense()
        n, dev, dt = step.n_tokens, x.device, self.runtime.dtype
        logits = self.router.forward(x, out_dtype=torch.float32)
        choice, weight = ops.moe_route(logits, self.top, self.renormalise, self.groups, self.keep_groups, self.renorm_eps,
                                       bias=self.router_bias)
        if self.tensor_cores and n * self.top >= self.TENSOR_CORE_ROWS_PER_EXPERT * self.E and x.stride(0) % 8 == 0:
            # enough rows per expert to fill tiles of 128: both products on the tensor cores, the activation in the first one's epilogue
            pair_pos, list_rows, tile_group = ops.moe_plan(choice, self.E, 128, step.token_slot)
            cap = list_rows.numel()
            rows = ops.moe_gather(x, list_rows)
            act = torch.empty((cap, self.ff), dtype=dt, device=dev)
            ops.gemm_tcgen05_grouped(rows, self.gate_up, act, tile_group, gated=self.activation, activation=self.fused_act)
            self._activate(act)
            res = torch.empty((cap, self.hidden), dtype=dt, device=dev)
            ops.gemm_tcgen05_grouped(act, self.down, res, tile_group)
        else:
            tile = 16 if n * self.top <= 16 * self.E else 64
            pair_pos, list_rows, tile_group = ops.moe_plan(choice, self.E, tile, step.token_slot)
            cap = list_rows.numel()
            act = torch.empty((cap, self.ff), dtype=dt, device=dev)
            res = torch.empty((cap, self.hidden), dtype=dt, device=dev)
            if tile == 16 and self.tensor_cores and self.SKINNY == "tcgen05" and x.stride(0) % 8 == 0:
                # a few rows per expert: the chosen experts' weights stream once through the tensor-core kernel's TMA ring
                rows = ops.moe_gather(x, list_rows)
                ops.gemm_tcgen05_grouped_skinny(rows, self.gate_up, act, tile_group, gated=self.activation, activation=self.fused_act)
                self._activate(act)
                ops.gemm_tcgen05_grouped_skinny(act, self.down, res, tile_group)
            elif tile == 16 and dt == torch.bfloat16 and self.hidden % 8 == 0 and self.ff % 8 == 0 and x.stride(0) % 8 == 0:
                # a few rows per expert: bound by reading the chosen experts' weights once
                ops.grouped_gemv(x, self.gate_up, act, list_rows, tile_group, tile, gated=self.activation,
                                 interleaved=self.tensor_cores and self.gated, activation=self.fused_act)
                self._activate(act)
                ops.grouped_gemv(act, self.down, res, None, tile_group, tile, live_rows=list_rows)
            else:
                ops.grouped_gemm(x, self.gate_up, act, a_rows=list_rows, tile_group=tile_group, tile_rows=tile, gated=self.activation,
                                 interleaved=self.tensor_cores and self.gated, activation=self.fused_act)
                self._activate(act)
                ops.grouped_gemm(act, self.down, res, a_rows=None, tile_group=tile_group, tile_rows=tile)
        out = torch.empty((2 if self.shared_size else 1, n, self.hidden), dtype=torch.float32, device=dev)
        ops.moe_combine(res, pair_pos, weight, out[0])
        if self.shared_size:
            # the expert every token takes: its down product writes the second float32 piece
            up = self.shared_up.forward(x)
            ops.activation(up, up, self.act_kind)
            self.shared_down.forward(up, out=out[1][:x.shape[0]])
        return out
