"""Attention over a latent that all heads share: the cache holds one short row per token."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache import CacheView, KVRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorDecl
from .base import Mixer, NormedLazy, PositionEncoding, Runtime, StepContext, register_mixer
from .linear import Linear, StackedInput


@register_mixer("latent_attention")
class LatentAttentionMixer(Mixer):
    """Per token the mixer keeps c = rmsnorm(the first ``kv_rank`` rows of W_dkv n) and one rotated key part
    k_r (the last ``rot_dim`` rows of W_dkv n, turned by the position).  Head h has an unrotated key
    W_uk[h] c and a value W_uv[h] c; its query is [q_n | q_r] (``dim`` unrotated, ``rot_dim`` rotated
    columns) and its score (q_n . W_uk[h] c + q_r . k_r) * scale.  Softmax over the keys up to the token's
    own position (of the last ``window`` positions only, where one is given), optionally with a sink per head in
    the denominator; optionally each head's result times sigmoid of one number per head (W_g n), or with ``gate`` =
    "element" the heads side by side times sigmoid(W_g n) element by element; out = W_o on the heads side by side.
    With ``q_rank`` the queries come through a latent of their own: q = W_q rmsnorm(W_dq n) with a plain weight.

    The scores are computed as (W_uk[h]^T q_n) . c + q_r . k_r and the values as W_uv[h] (sum_j p_j c_j),
    so the kernels see attention of H query heads over ONE key head whose rows [c | k_r] are read from
    the cache as they lie there, values being the rows' first ``kv_rank`` columns; nothing per head is
    ever built for a cached token.  W_uk^T and W_uv are applied by one grouped product each.  A layer
    with ``own_latent`` False has no W_dkv and reads the rows that the execution named by the
    schedule's ``cache_from`` wrote.

    Spec: ``hidden_size``, ``num_heads``, ``dim``, ``rot_dim``, ``vdim``, ``kv_rank``, ``scale``, ``norm_eps``,
    ``own_latent``, ``q_rank`` (None), ``window`` (None), ``gate`` ("head" | "element"), ``names`` (q, dkv, dkv_norm, uk, uv, o
    and optionally sink, g, dq, dq_norm).  KuiperLLama's
    attention keeps whole keys and values per kv head (kuiper/source/model/llama3.cpp:610-639,
    mha_kernel.cu:61,74-106)."""

    @classmethod
    def manifest(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorDecl]:
        hid, H, d, rd, dv, r = (spec[k] for k in ("hidden_size", "num_heads", "dim", "rot_dim", "vdim", "kv_rank"))
        n = spec["names"]
        qr = spec.get("q_rank")
        m = {prefix + n["q"]: TensorDecl((H * (d + rd), qr or hid)), prefix + n["uk"]: TensorDecl((H * d, r)),
             prefix + n["uv"]: TensorDecl((H * dv, r)), prefix + n["o"]: TensorDecl((hid, H * dv))}
        if spec.get("own_latent", True):
            m[prefix + n["dkv"]] = TensorDecl((r + rd, hid))
            m[prefix + n["dkv_norm"]] = TensorDecl((r,), role="vector", init="one_plus_normal")
        if n.get("sink"):
            m[prefix + n["sink"]] = TensorDecl((H,), role="vector")
        if n.get("g"):
            m[prefix + n["g"]] = TensorDecl((H * dv if spec.get("gate", "head") == "element" else H, hid))
        if qr:
            m[prefix + n["dq"]] = TensorDecl((qr, hid))
            m[prefix + n["dq_norm"]] = TensorDecl((qr,), role="vector", init="one_plus_normal")
        return m

    def __init__(self, spec, prefix, tensors, runtime: Runtime, position: Optional[PositionEncoding] = None):
        super().__init__(spec, prefix, tensors, runtime, position)
        self.hidden, self.H = int(spec["hidden_size"]), int(spec["num_heads"])
        self.d, self.rd, self.dv, self.r = int(spec["dim"]), int(spec["rot_dim"]), int(spec["vdim"]), int(spec["kv_rank"])
        self.Dk = self.r + self.rd
        if self.r > 512:
            raise ValueError(f"kv_rank {self.r} is not supported by the attention kernels (up to 512)")
        self.scale, self.eps = float(spec["scale"]), float(spec["norm_eps"])
        self.own = bool(spec.get("own_latent", True))
        n = spec["names"]
        dev, dt = runtime.device, runtime.dtype
        f32 = lambda name: tensors[prefix + name].to(device=dev, dtype=torch.float32).contiguous()
        self.window = spec.get("window")
        self.q_rank = int(spec.get("q_rank") or 0)
        self.gate_kind = str(spec.get("gate", "head"))
        if self.gate_kind not in ("head", "element"):
            raise ValueError(f"unknown gate {self.gate_kind!r} (head, element)")
        self.inputs = StackedInput(runtime)               # q (or its latent) | dkv | g from one product
        if self.q_rank:
            self.inputs.add("dq", tensors[prefix + n["dq"]])
            self.dq_norm = f32(n["dq_norm"])
            self.uq = Linear(tensors[prefix + n["q"]], runtime)
        else:
            self.inputs.add("q", tensors[prefix + n["q"]])
        if self.own:
            self.inputs.add("dkv", tensors[prefix + n["dkv"]])
            self.norm_weight = f32(n["dkv_norm"])
        else:
            self.norm_weight = None
        self.gated = bool(n.get("g"))
        if self.gated:
            self.inputs.add("g", tensors[prefix + n["g"]])
        self.sink = f32(n["sink"]) if n.get("sink") else None
        # W_uk^T per head, [H, kv_rank, dim]: the product that takes a query's unrotated part to the latent's side
        uk = tensors[prefix + n["uk"]].to(device=dev, dtype=dt).reshape(self.H, self.d, self.r)
        self.uk_t = uk.transpose(1, 2).contiguous()
        self.uv = tensors[prefix + n["uv"]].to(device=dev, dtype=dt).reshape(self.H, self.dv, self.r).contiguous()
        self.o = Linear(tensors[prefix + n["o"]], runtime)
        rot = position.rotary() if position is not None else None
        self.inv_freq, self.rot_dims = rot if rot is not None else (None, 0)
        if self.rot_dims > self.rd:
            raise ValueError(f"{self.rot_dims} rotated dimensions do not fit the rotated part of {self.rd}")
        self.magnitude = float(getattr(position, "magnitude", 1.0)) if position is not None else 1.0
        self.interleaved = getattr(position, "pairing", "half") == "interleaved"

    def kv_request(self) -> Optional[KVRequest]:
        return KVRequest(kv_heads=1, head_dim=self.Dk, kind="keys", window=self.window)

    def forward(self, x, step: StepContext, cache: CacheView) -> torch.Tensor:
        if isinstance(x, NormedLazy):
            x = x.dense()
        if cache.writable != self.own:
            raise RuntimeError("a latent-attention layer writes the cache exactly when it has a down-projection of its own")
        n, dt, dev = step.n_tokens, self.runtime.dtype, x.device
        proj = self.inputs.forward(x)
        if self.q_rank:
            # the queries' latent: its norm (32-bit statistics) and the product that makes every head's query from it
            cq = torch.empty((proj.shape[0], self.q_rank), dtype=dt, device=dev)
            ops.rows_rmsnorm(self.inputs.view("dq"), self.dq_norm, cq, self.eps)
            qsrc, q_col = self.uq.forward(cq), 0
        else:
            qsrc, q_col = proj, self.inputs.column("q")
        # rows that belong to no sequence (a small step's padding) are not written by the kernels: keep them defined
        make = torch.zeros if n > sum(step.host_new) else torch.empty
        qfull = make((n, self.H * self.Dk), dtype=dt, device=dev)
        ops.latent_prepare(proj, q_col, self.inputs.column("dkv") if self.own else None, self.norm_weight, self.eps, self.inv_freq,
                           self.rot_dims, self.magnitude, self.interleaved, step.positions, step.token_slot, cache.block_table,
                           cache.k, qfull, n, self.H, self.d, self.rd, self.r, q=qsrc)
        ops.grouped_gemm(qsrc[:, q_col:q_col + self.H * (self.d + self.rd)], self.uk_t, qfull, a_group_stride=self.d + self.rd,
                         out_group_stride=self.Dk, rows=n, tile_rows=16 if n <= 16 else 64)
        lat = make((n, self.H * self.r), dtype=dt, device=dev)
        ops.latent_attention(qfull, lat, cache.k, cache.block_table, step, self.H, self.Dk, self.r, self.scale, self.sink,
                             window=int(self.window or 0))
        attn = torch.empty((n, self.H * self.dv), dtype=dt, device=dev)
        # W_uv per head, and each head's result times sigmoid of its gate number (or of every element's own) in the same kernel
        ops.grouped_gemm(lat, self.uv, attn, a_group_stride=self.r, out_group_stride=self.dv, rows=n, tile_rows=16 if n <= 16 else 64,
                         row_gate=self.inputs.view("g") if self.gated else None, gate_elements=self.gate_kind == "element")
        return self.o.forward(attn, allow_partials=True)
