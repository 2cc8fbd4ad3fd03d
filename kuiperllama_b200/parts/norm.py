"""Norms fused with the residual add: RMSNorm and the layer norm with weight and bias."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorDecl
from .base import Accumulated, DeltaSum, Norm, NormedLazy, PostNormed, Runtime, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """out = w * x * rsqrt(mean(x^2) + eps) on x = residual + delta, statistics in 32 bits
    (ExiledOfCode/KuiperLLama rmsnorm_kernel.cu:70-106; the add is its add_kernel.cu:4-12,
    fused here).  ``size``, ``eps`` and the tensor's ``name`` come from the spec; with ``weight_offset`` c the
    stored tensor is w - c (a weight kept around zero: the norm multiplies by c + stored); with ``scalar`` the
    stored tensor is ONE number (shape ()), the weight of every coordinate."""

    @classmethod
    def manifest(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorDecl]:
        init = "normal" if spec.get("weight_offset") else "one_plus_normal"
        return {prefix + spec["name"]: TensorDecl(() if spec.get("scalar") else (spec["size"],), role="vector", init=init)}

    def __init__(self, spec, prefix, tensors, runtime: Runtime):
        super().__init__(spec, prefix, tensors, runtime)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight = tensors[prefix + spec["name"]].to(device=runtime.device, dtype=torch.float32).contiguous()
        if spec.get("scalar"):
            self.weight = self.weight.reshape(1).expand(self.size).contiguous()          # the kernels read a weight per coordinate
        if spec.get("weight_offset"):
            self.weight = (self.weight + float(spec["weight_offset"])).contiguous()      # exact for a bfloat16 checkpoint: 32-bit sum

    accepts_accumulated = True

    def forward(self, residual: torch.Tensor, delta, n_rows: int, rows: Optional[torch.Tensor] = None):
        if isinstance(delta, PostNormed):
            return chain_forward(self, residual, delta, rows)
        if isinstance(delta, DeltaSum):
            return self.forward_pair(residual, delta, None, rows)[0]
        if isinstance(delta, Accumulated):
            # the stream holds the sum already; if the rows times this norm's weight came with it,
            # the product that follows only has to apply 1 / rms
            if rows is None and delta.norm is self and delta.scaled is not None:
                return NormedLazy(residual, self.weight, self.eps, delta.ss, delta.scaled, self.runtime.dtype)
            delta = None
        n_out = rows.numel() if rows is not None else residual.shape[0]
        out = torch.empty((n_out, self.size), dtype=self.runtime.dtype, device=residual.device)
        ops.add_rmsnorm(residual, delta, self.weight, out, self.eps, rows)
        return out


def _forward_pair(self, residual: torch.Tensor, delta, other: Optional["RMSNorm"], rows: Optional[torch.Tensor] = None):
    """This norm and ``other`` (a second RMS norm with the same eps, or None) of the same stream after ``delta`` (None, a
    tensor, pieces or ``DeltaSum``) has been added: one kernel, one root mean square, two weights."""
    parts = (delta.first, delta.second) if isinstance(delta, DeltaSum) else (delta,)
    n_out = rows.numel() if rows is not None else residual.shape[0]
    dt, dev = self.runtime.dtype, residual.device
    out1 = torch.empty((n_out, self.size), dtype=dt, device=dev)
    out2 = torch.empty((n_out, self.size), dtype=dt, device=dev) if other is not None else None
    ops.pair_rmsnorm(residual, parts, self.weight, other.weight if other is not None else None, out1, out2, self.eps, rows, dtype=dt)
    return out1, out2


RMSNorm.forward_pair = _forward_pair


def chain_forward(norm: Norm, residual: torch.Tensor, delta, rows: Optional[torch.Tensor]) -> torch.Tensor:
    """``norm`` of the stream after ``delta`` (None, rows in the compute dtype, or ``PostNormed``: a
    result that is gated and normed on its way into the stream) has been added, in one kernel."""
    n_out = rows.numel() if rows is not None else residual.shape[0]
    out = torch.empty((n_out, residual.shape[1]), dtype=norm.runtime.dtype, device=residual.device)
    value = gate = gate_bias = post = None
    if isinstance(delta, PostNormed):
        value, gate, gate_bias = delta.value, delta.gate, delta.gate_bias
        if delta.norm is not None:
            post = (delta.norm.weight, delta.norm.bias, delta.norm.eps, delta.norm.kind)
    elif delta is not None:
        value = delta                                              # rows, or float32 pieces of a product
    ops.norm_chain(residual, value, out, norm.weight, norm.bias, norm.eps, norm.kind, gate=gate, gate_bias=gate_bias,
                   post=post, rows=rows)
    return out


def add_to_stream(residual: torch.Tensor, delta) -> None:
    """Add a pending delta to the stream without a norm after it (what a caller that wants the
    stream itself does after the last block)."""
    if delta is None:
        return
    if isinstance(delta, DeltaSum):
        ops.pair_rmsnorm(residual, (delta.first, delta.second), None, None, None, None, 0.0,
                         dtype=next((d.dtype for d in (delta.first, delta.second) if d is not None and d.dim() == 2), torch.float32))
        return
    if isinstance(delta, PostNormed):
        post = None
        if delta.norm is not None:
            post = (delta.norm.weight, delta.norm.bias, delta.norm.eps, delta.norm.kind)
        ops.norm_chain(residual, delta.value, None, None, None, 0.0, "layernorm", gate=delta.gate, gate_bias=delta.gate_bias, post=post)
    else:
        ops.norm_chain(residual, delta, None, None, None, 0.0, "layernorm")


@register_norm("none")
class NoNorm(Norm):
    """No norm before a sublayer: the sublayer reads the stream itself (in the compute dtype).  It still is the
    place where what is pending gets added, so a block whose sublayers are normed only AFTER they ran
    (x += norm(sublayer(x))) is the sandwich block with this part in front.  No tensors; spec: ``size``."""

    kind = "none"
    weight = None
    eps = 0.0

    def __init__(self, spec, prefix, tensors, runtime: Runtime):
        super().__init__(spec, prefix, tensors, runtime)
        self.size = int(spec["size"])

    def forward(self, residual: torch.Tensor, delta, n_rows: int, rows: Optional[torch.Tensor] = None):
        return chain_forward(self, residual, delta, rows)


@register_norm("layernorm")
class LayerNorm(Norm):
    """out = (x - mean) / sqrt(mean((x - mean)^2) + eps) * w + b on x = residual + delta, statistics
    and sum in 32 bits.  Spec: ``size``, ``eps``, the weight's ``name`` and the bias's ``bias``
    (None: no bias).  KuiperLLama has the RMS norm alone (rmsnorm_kernel.cu:70-106)."""

    kind = "layernorm"

    @classmethod
    def manifest(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorDecl]:
        m = {prefix + spec["name"]: TensorDecl((spec["size"],), role="vector", init="one_plus_normal")}
        if spec.get("bias"):
            m[prefix + spec["bias"]] = TensorDecl((spec["size"],), role="vector")
        return m

    def __init__(self, spec, prefix, tensors, runtime: Runtime):
        super().__init__(spec, prefix, tensors, runtime)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight = tensors[prefix + spec["name"]].to(device=runtime.device, dtype=torch.float32).contiguous()
        self.bias = None
        if spec.get("bias"):
            self.bias = tensors[prefix + spec["bias"]].to(device=runtime.device, dtype=torch.float32).contiguous()

    def forward(self, residual: torch.Tensor, delta, n_rows: int, rows: Optional[torch.Tensor] = None):
        return chain_forward(self, residual, delta, rows)
