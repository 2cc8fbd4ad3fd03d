"""Recurrent mixers whose state is a matrix per head, fed by outer products: a state-space layer and gated linear attention."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache import CacheView, StateRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorDecl
from .base import Mixer, NormedLazy, PositionEncoding, Runtime, StepContext, register_mixer
from .composite import BranchMixer
from .linear import Linear, StackedInput


@register_mixer("mamba2")
class Mamba2Mixer(Mixer):
    """The state-space mixer of Dao and Gu, "Transformers are SSMs: Generalized Models and Efficient Algorithms Through
    Structured State Space Duality" (2024), in its recurrent form.  With inner = heads * vdim, N = state, G = groups, one
    product makes [z: inner | x: inner | B: G N | C: G N | dt: heads]; x, B and C pass a causal convolution per channel
    over ``conv`` inputs with bias and SiLU; dt = softplus(dt + dt_bias) (no clamp).  Per head h, which reads group
    h // (heads / G), with S [N, vdim] starting at zero:

        S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T;     y_t = S_t^T C_t + D_h x_t

    then y * silu(z), an RMS norm over each of ``norm_groups`` equal parts of the inner channels (the gate comes before
    the norm), times the norm's weight, and the output projection.  The convolution's sums, dt, the decay, S and y are
    32-bit; the slot's state is S as [heads, N, vdim], then the convolution's last conv - 1 inputs, float32.  Spec:
    ``hidden_size``, ``heads``, ``vdim``, ``state``, ``groups``, ``conv``, ``norm_groups``, ``norm_eps`` and ``names`` (in,
    conv, conv_bias, dt_bias, A_log, D, norm, o).  KuiperLLama has no recurrent mixer (its mixer is
    mha_kernel.cu:61,74-106)."""

    @classmethod
    def manifest(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorDecl]:
        hid, H, P, N, G, K, n = (spec[k] for k in ("hidden_size", "heads", "vdim", "state", "groups", "conv", "names"))
        inner, C = H * P, H * P + 2 * G * N
        vec = lambda shape, init="normal": TensorDecl(shape, role="vector", init=init)
        return {prefix + n["in"]: TensorDecl((inner + C + H, hid)), prefix + n["o"]: TensorDecl((hid, inner)),
                prefix + n["conv"]: vec((C, K)), prefix + n["conv_bias"]: vec((C,)), prefix + n["dt_bias"]: vec((H,)),
                prefix + n["A_log"]: vec((H,)), prefix + n["D"]: vec((H,), "one_plus_normal"),
                prefix + n["norm"]: vec((inner,), "one_plus_normal")}

    def __init__(self, spec, prefix, tensors, runtime: Runtime, position: Optional[PositionEncoding] = None):
        super().__init__(spec, prefix, tensors, runtime, position)
        self.hidden = int(spec["hidden_size"])
        self.H, self.P, self.N, self.G, self.taps = (int(spec[k]) for k in ("heads", "vdim", "state", "groups", "conv"))
        self.norm_groups, self.norm_eps = int(spec["norm_groups"]), float(spec["norm_eps"])
        self.inner = self.H * self.P
        self.channels = self.inner + 2 * self.G * self.N
        if self.H % self.G:
            raise ValueError(f"{self.H} heads are not a multiple of {self.G} groups")
        if self.inner % self.norm_groups:
            raise ValueError(f"{self.inner} inner channels do not split into {self.norm_groups} equal parts for the norm")
        if not 1 <= self.taps <= ops.SHORT_CONV_MAX_TAPS:
            raise ValueError(f"the convolution kernel takes 1 to {ops.SHORT_CONV_MAX_TAPS} taps, got {self.taps}")
        if self.N > 1024:
            raise ValueError(f"a state of {self.N} rows per head is above the recurrence kernel's 1,024")
        n = spec["names"]
        self.input = Linear(tensors[prefix + n["in"]], runtime)
        self.o = Linear(tensors[prefix + n["o"]], runtime)
        f32 = lambda name: tensors[prefix + name].to(device=runtime.device, dtype=torch.float32).contiguous()
        self.conv_weight, self.conv_bias = f32(n["conv"]), f32(n["conv_bias"])
        self.dt_bias, self.A_log, self.D, self.norm_weight = f32(n["dt_bias"]), f32(n["A_log"]), f32(n["D"]), f32(n["norm"])
        self.conv_off = self.H * self.N * self.P

    def state_request(self) -> Optional[StateRequest]:
        return StateRequest((self.conv_off + (self.taps - 1) * self.channels,), torch.float32)

    def forward(self, x, step: StepContext, cache: CacheView) -> torch.Tensor:
        if isinstance(x, NormedLazy):
            x = x.dense()
        n, dev = step.n_tokens, x.device
        inner, C, GN = self.inner, self.channels, self.G * self.N
        proj = self.input.forward(x)
        # rows that belong to no sequence (a small step's padding) are not written by the kernels: keep them defined
        make = torch.empty if n == step.n_seqs else torch.zeros
        xbc = make((n, C), dtype=torch.float32, device=dev)
        conv_state = cache.state[:, self.conv_off:] if self.taps > 1 else cache.state
        ops.short_conv(proj[:, inner:inner + C], self.conv_weight, self.conv_bias, conv_state, step, xbc, silu=True,
                       update_state=cache.writable)
        dt = torch.empty((n, self.H), dtype=torch.float32, device=dev)
        decay = torch.empty((n, self.H), dtype=torch.float32, device=dev)
        ops.decay_softplus(proj[:, inner + C:], self.dt_bias, self.A_log, n, dt, decay)
        y = make((n, inner), dtype=torch.float32, device=dev)
        ops.outer_recurrence(xbc[:, inner + GN:], xbc[:, inner:inner + GN], xbc[:, :inner], decay, cache.state, y, step,
                             self.H, self.G, self.N, self.P, c=dt, skip=self.D)
        gated = torch.empty((n, inner), dtype=self.runtime.dtype, device=dev)
        ops.head_rmsnorm_gate(y, proj[:, :inner], self.norm_weight, gated, self.norm_groups, inner // self.norm_groups,
                              self.norm_eps, gate_first=True)
        return self.o.forward(gated, allow_partials=True)


@register_mixer("gated_linear_attention")
class GatedLinearAttentionMixer(BranchMixer):
    """Linear attention with a decay per key channel (Yang et al., "Gated Linear Attention Transformers with
    Hardware-Efficient Training", 2024), in its recurrent form.  q = Wq n * q_scale and k = Wk n (heads x dim), v = Wv n
    (heads x vdim); alpha = sigmoid(z)^(1 / tau) with z = Wa2 (Wa1 n) + b (heads x dim, through a low rank).  Per head,
    with S [dim, vdim] starting at zero:

        S_t = diag(alpha_t) S_(t-1) + k_t v_t^T;     o_t = S_t^T q_t

    then each head's o over its root mean square (over vdim) times a weight the heads share, times silu(Wg n), and the
    output projection.  alpha, S, o and the norm are 32-bit; the slot's state is S as [heads, dim, vdim] float32.  Spec:
    ``hidden_size``, ``heads``, ``dim``, ``vdim``, ``rank``, ``tau``, ``q_scale``, ``norm_eps`` and ``names`` (q, k, v, g, o, norm, a1,
    a2, a2_bias).  KuiperLLama has no recurrent mixer (its mixer is mha_kernel.cu:61,74-106)."""

    @classmethod
    def manifest(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorDecl]:
        hid, H, d, dv, r, n = (spec[k] for k in ("hidden_size", "heads", "dim", "vdim", "rank", "names"))
        return {prefix + n["q"]: TensorDecl((H * d, hid)), prefix + n["k"]: TensorDecl((H * d, hid)),
                prefix + n["v"]: TensorDecl((H * dv, hid)), prefix + n["g"]: TensorDecl((H * dv, hid)),
                prefix + n["o"]: TensorDecl((hid, H * dv)), prefix + n["norm"]: TensorDecl((dv,), role="vector", init="one_plus_normal"),
                prefix + n["a1"]: TensorDecl((r, hid)), prefix + n["a2"]: TensorDecl((H * d, r), role="vector"),
                prefix + n["a2_bias"]: TensorDecl((H * d,), role="vector")}

    def __init__(self, spec, prefix, tensors, runtime: Runtime, position: Optional[PositionEncoding] = None):
        super().__init__(spec, prefix, tensors, runtime, position)
        self.hidden = int(spec["hidden_size"])
        self.H, self.d, self.dv, self.rank = (int(spec[k]) for k in ("heads", "dim", "vdim", "rank"))
        self.tau, self.q_scale, self.norm_eps = float(spec["tau"]), float(spec["q_scale"]), float(spec["norm_eps"])
        if not self.tau > 0:
            raise ValueError(f"tau must be positive, got {self.tau}")
        if self.d > 1024:
            raise ValueError(f"a key size of {self.d} is above the recurrence kernel's 1,024")
        n = spec["names"]
        self._w = {k: tensors[prefix + n[k]] for k in ("q", "k", "v", "g", "a1")}
        self.o_weight = tensors[prefix + n["o"]]
        self.core_width = self.H * self.dv
        f32 = lambda name: tensors[prefix + name].to(device=runtime.device, dtype=torch.float32).contiguous()
        self.a2, self.a2_bias, self.norm_weight = f32(n["a2"]), f32(n["a2_bias"]), f32(n["norm"])

    def state_request(self) -> Optional[StateRequest]:
        return StateRequest((self.H * self.d * self.dv,), torch.float32)

    def add_inputs(self, stacked: StackedInput, tag: str) -> None:
        for k in ("q", "k", "v", "g", "a1"):
            stacked.add(tag + k, self._w[k])
        self._w = None

    def core(self, stacked: StackedInput, tag: str, step: StepContext, cache: CacheView, out: torch.Tensor, out_scale: float) -> None:
        n, dev = step.n_tokens, out.device
        alpha = torch.empty((n, self.H * self.d), dtype=torch.float32, device=dev)
        ops.decay_lowrank(stacked.view(tag + "a1"), self.a2, self.a2_bias, self.tau, n, alpha)
        make = torch.empty if n == step.n_seqs else torch.zeros
        o = make((n, self.H * self.dv), dtype=torch.float32, device=dev)
        ops.outer_recurrence(stacked.view(tag + "q"), stacked.view(tag + "k"), stacked.view(tag + "v"), alpha, cache.state, o, step,
                             self.H, self.H, self.d, self.dv, q_scale=self.q_scale)
        ops.head_rmsnorm_gate(o, stacked.view(tag + "g"), self.norm_weight, out, self.H, self.dv, self.norm_eps, out_scale=out_scale)
