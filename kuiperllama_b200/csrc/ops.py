"""Python side of the CUDA kernels: loads each module's shared library (building it at first
use), checks shapes, types and devices, and calls the C entry points on torch's current
stream.  Nothing here computes on the CPU and nothing falls back to a library kernel: a
missing extension or a refused size raises.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Dict, Optional

import torch

from . import build
from .build import ExtensionError

PAGE = 64                      # tokens per cache page; equals kl::PAGE in common.cuh

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

_ERRORS = {-1: "unsupported dtype", -2: "unsupported size", -3: "misaligned pointer or stride",
           -4: "the kernel reported an error through its status word", -5: "set-up failed"}


class KernelError(RuntimeError):
    pass


_libs: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def lib(name: str) -> ctypes.CDLL:
    """The loaded shared library of one kernel module."""
    got = _libs.get(name)
    if got is not None:
        return got
    with _lock:
        if name not in _libs:
            path = build.ensure_built(name)
            try:
                _libs[name] = ctypes.CDLL(path)
            except OSError as e:
                raise ExtensionError(f"cannot load {path}: {e}") from None
        return _libs[name]


def loaded_libraries() -> Dict[str, str]:
    return {n: l._name for n, l in _libs.items()}


launch_count = 0       # kernels of this package launched so far (counted per entry-point call)


def _check(code: int, what: str, launches: int = 1) -> None:
    global launch_count
    if code == 0:
        launch_count += launches
        return
    if code in _ERRORS:
        raise KernelError(f"{what}: {_ERRORS[code]}")
    raise KernelError(f"{what}: CUDA error {code}")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not supported by the kernels (float32, bfloat16)") from None


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


# The current stream's handle, once per launch: torch.cuda.current_stream() builds a Stream object and
# looks the device up three times (7 us); the raw call behind it takes a fraction of a microsecond.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> ctypes.c_void_p:
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel arguments must live on a CUDA device; there is no CPU path")


def _i32(t: Optional[torch.Tensor], name: str) -> None:
    if t is not None:
        _need(t.dtype == torch.int32 and t.is_contiguous(), f"{name} must be a contiguous int32 tensor")


# --------------------------------------------------------------------------- row-wise

def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, error_flag: torch.Tensor,
              scale: float = 1.0) -> None:
    """out[t] = scale * float32(table[ids[t]]); ids outside the table set error_flag[0] = 1."""
    _cuda(ids, table, out, error_flag)
    _i32(ids, "ids"); _i32(error_flag, "error_flag")
    n, (vocab, hidden) = ids.numel(), table.shape
    _need(table.is_contiguous() and out.is_contiguous() and out.dtype == torch.float32, "embedding: bad layout")
    _need(out.shape[0] >= n and out.shape[1] == hidden, "embedding: output shape")
    _check(lib("rowwise").kl_embedding(_ptr(ids), n, _ptr(table), dtype_code(table.dtype), vocab, hidden,
                                       ctypes.c_float(scale), _ptr(out), _ptr(error_flag), _stream()), "embedding")


def logit_transform(logits: torch.Tensor, scale: float = 1.0, softcap: float = 0.0) -> None:
    """In place on float32 logits [rows, vocab]: x = scale * x, then with ``softcap`` c > 0
    x = c * tanh(x / c)."""
    _cuda(logits)
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1, "logit_transform: float32 rows")
    _need(softcap >= 0.0, "logit_transform: the soft cap must not be negative")
    rows, vocab = logits.shape
    _check(lib("rowwise").kl_logit_transform(_ptr(logits), ctypes.c_longlong(logits.stride(0)), rows, vocab,
                                             ctypes.c_float(scale), ctypes.c_float(softcap), _stream()), "logit_transform")


def _partials(delta: Optional[torch.Tensor]) -> bool:
    """A delta given as float32 partial sums [S, rows, width] (the pieces of a product whose K
    range was cut), to be added in ascending order by the kernel that consumes it."""
    return delta is not None and delta.dim() == 3


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor,
                eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """x = residual (+ delta); out = weight * x * rsqrt(mean(x^2) + eps).

    ``delta`` is [rows, hidden] in the output's dtype, or float32 partial sums
    [S, rows, hidden].  Without ``rows`` every row is processed and, when ``delta`` is given,
    the sum is written back to ``residual``.  With ``rows`` (int32 indices) only those rows
    are read, into out[0..len(rows)), and ``residual`` is left as it is."""
    _cuda(residual, delta, weight, out, rows)
    _i32(rows, "rows")
    hidden = residual.shape[-1]
    n = rows.numel() if rows is not None else residual.shape[0]
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "add_rmsnorm: the residual stream is float32")
    _need(weight.dtype == torch.float32 and weight.numel() == hidden, "add_rmsnorm: weight must be float32 [hidden]")
    _need(out.is_contiguous() and out.shape[-1] == hidden and out.shape[0] >= n, "add_rmsnorm: output shape")
    plain, parts, n_parts, stride = delta, None, 0, 0
    if _partials(delta):
        _need(delta.dtype == torch.float32 and delta.is_contiguous() and tuple(delta.shape[1:]) == tuple(residual.shape),
              "add_rmsnorm: partial sums must be float32 [S, rows, hidden]")
        plain, parts, n_parts, stride = None, delta, delta.shape[0], delta.shape[1] * delta.shape[2]
    elif delta is not None:
        _need(delta.dtype == out.dtype and delta.is_contiguous() and delta.shape == residual.shape,
              "add_rmsnorm: delta must match the residual's shape and the output's dtype")
    _check(lib("rowwise").kl_add_rmsnorm(_ptr(residual), _ptr(plain), _ptr(parts), n_parts, ctypes.c_longlong(stride),
                                         _ptr(weight), _ptr(out), _ptr(rows), n, hidden, ctypes.c_float(eps),
                                         dtype_code(out.dtype), _stream()), "add_rmsnorm")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _cuda(gate_up, out)
    tokens, two_i = gate_up.shape
    _need(two_i % 2 == 0 and out.shape == (tokens, two_i // 2), "swiglu: shapes")
    _need(gate_up.is_contiguous() and out.is_contiguous() and gate_up.dtype == out.dtype, "swiglu: layout")
    _check(lib("rowwise").kl_swiglu(_ptr(gate_up), _ptr(out), tokens, two_i // 2, dtype_code(out.dtype), _stream()),
           "swiglu")


# --------------------------------------------------------------------------- norm chains, activations, gates

NORM_KINDS = {"layernorm": 0, "rmsnorm": 1, "none": 2}      # "none": the rows themselves in the compute dtype
ACTIVATIONS = {"xielu": 0, "gelu_tanh": 1, "silu": 2, "relu2": 3}      # relu2: max(z, 0)^2


def _columns(t: Optional[torch.Tensor], n: int, width: int, name: str) -> None:
    """``t`` is [>= n, width] with unit column stride (rows may be a stacked product's column slice)."""
    if t is not None:
        _need(t.dim() == 2 and t.shape[0] >= n and t.shape[1] == width and t.stride(1) == 1, f"{name}: expected [{n}, {width}] rows")


def norm_chain(residual: torch.Tensor, delta: Optional[torch.Tensor], out: Optional[torch.Tensor], weight: Optional[torch.Tensor],
               bias: Optional[torch.Tensor], eps: float, kind: str, gate: Optional[torch.Tensor] = None,
               gate_bias: Optional[torch.Tensor] = None, post: Optional[tuple] = None, rows: Optional[torch.Tensor] = None,
               dtype: Optional[torch.dtype] = None) -> None:
    """d = delta * sigmoid(gate + gate_bias); d = post-norm(d); x = residual + d (written back unless
    ``rows``); out = norm(x).  Every step but the last is optional: ``delta`` None adds nothing,
    ``post`` = (weight, bias or None, eps, kind) or None, ``out`` None only updates the stream.
    ``delta`` and ``gate`` are [n, hidden] in the compute dtype with any row stride; ``delta`` may also be
    float32 pieces [S, n, hidden] of a product whose K range was cut (their sum is the delta)."""
    _cuda(residual, delta, out, weight, bias, gate, gate_bias, rows)
    _i32(rows, "rows")
    hidden = residual.shape[-1]
    n = rows.numel() if rows is not None else residual.shape[0]
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "norm_chain: the residual stream is float32")
    parts, n_parts, stride = None, 0, 0
    if _partials(delta):
        _need(delta.dtype == torch.float32 and delta.is_contiguous() and tuple(delta.shape[1:]) == tuple(residual.shape),
              "norm_chain: pieces must be float32 [S, rows, hidden]")
        parts, n_parts, stride, delta = delta, delta.shape[0], delta.shape[1] * delta.shape[2], None
    if dtype is None:
        dtype = next((t.dtype for t in (out, delta, gate) if t is not None), torch.float32)
    for t, nm in ((delta, "delta"), (gate, "gate")):
        if t is not None:
            _need(t.dtype == dtype and t.dim() == 2 and t.shape[1] == hidden and t.stride(1) == 1 and t.shape[0] >= residual.shape[0],
                  f"norm_chain: {nm} must be [rows, hidden] in the compute dtype")
    _need(gate is None or delta is not None or parts is not None, "norm_chain: a gate needs something to gate")
    for t in (weight, bias, gate_bias) + (tuple(post[:2]) if post is not None else ()):
        _need(t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == hidden), "norm_chain: float32 [hidden] vectors")
    if out is not None:
        _need(out.is_contiguous() and out.dtype == dtype and out.shape[-1] == hidden and out.shape[0] >= n
              and (weight is not None or kind == "none"), "norm_chain: output shape")
    pw, pb, peps, pkind = post if post is not None else (None, None, 0.0, kind)
    _check(lib("norms").kl_norm_chain(
        _ptr(residual), _ptr(delta), ctypes.c_longlong(delta.stride(0) if delta is not None else 0), _ptr(parts), n_parts,
        ctypes.c_longlong(stride), _ptr(gate),
        ctypes.c_longlong(gate.stride(0) if gate is not None else 0), _ptr(gate_bias), _ptr(pw), _ptr(pb), ctypes.c_float(peps),
        NORM_KINDS[pkind], _ptr(weight), _ptr(bias), ctypes.c_float(eps), NORM_KINDS[kind], _ptr(out), _ptr(rows), n, hidden,
        dtype_code(dtype), _stream()), "norm_chain")


def head_rmsnorm_gate(x: torch.Tensor, gate: Optional[torch.Tensor], weight: Optional[torch.Tensor], out: torch.Tensor,
                      heads: int, dim: int, eps: float, gate_first: bool = False, out_scale: float = 1.0) -> None:
    """out[t, h, :] = x[t, h, :] / sqrt(mean(x[t, h, :]^2) + eps) * weight * silu(gate[t, h, :]); x float32
    [tokens, heads * dim], gate (compute dtype, any row stride) and weight (float32 [dim], or [heads * dim]: a weight
    per channel) optional.  ``gate_first``: the gate comes before the norm, out = norm(x * silu(gate)) * weight.  ``out`` may
    be a column slice of a wider matrix; the result is multiplied by ``out_scale`` (in 32 bits, before it is rounded)."""
    _cuda(x, gate, weight, out)
    n = x.shape[0]
    _need(x.dtype == torch.float32 and x.is_contiguous() and x.shape[1] == heads * dim, "head_rmsnorm_gate: x")
    _columns(out, n, heads * dim, "head_rmsnorm_gate: out")
    _columns(gate, n, heads * dim, "head_rmsnorm_gate: gate")
    _need(gate is None or gate.dtype == out.dtype, "head_rmsnorm_gate: gate dtype")
    _need(weight is None or (weight.dtype == torch.float32 and weight.numel() in (dim, heads * dim) and weight.is_contiguous()),
          "head_rmsnorm_gate: weight")
    wide = weight is not None and weight.numel() == heads * dim and heads > 1
    _check(lib("norms").kl_head_rmsnorm_gate(_ptr(x), _ptr(gate), ctypes.c_longlong(gate.stride(0) if gate is not None else 0),
                                             _ptr(weight), _ptr(out), ctypes.c_longlong(out.stride(0)), ctypes.c_float(out_scale), n, heads, dim,
                                             ctypes.c_float(eps), int(bool(gate_first)), int(wide),
                                             dtype_code(out.dtype), _stream()), "head_rmsnorm_gate")


def rows_rmsnorm(x: torch.Tensor, weight: Optional[torch.Tensor], out: torch.Tensor, eps: float) -> None:
    """out[t] = x[t] / sqrt(mean(x[t]^2) + eps) * weight for rows in the compute dtype (any row stride) that are no part of the
    residual stream; statistics in 32 bits, ``weight`` float32 [width] or None."""
    _cuda(x, weight, out)
    n, width = x.shape
    _columns(x, n, width, "rows_rmsnorm: x"); _columns(out, n, width, "rows_rmsnorm: out")
    _need(x.dtype == out.dtype, "rows_rmsnorm: dtypes differ")
    _need(weight is None or (weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == width), "rows_rmsnorm: weight")
    _check(lib("norms").kl_rows_rmsnorm(_ptr(x), ctypes.c_longlong(x.stride(0)), _ptr(weight), _ptr(out), ctypes.c_longlong(out.stride(0)),
                                        n, width, ctypes.c_float(eps), dtype_code(x.dtype), _stream()), "rows_rmsnorm")


def pair_rmsnorm(residual: torch.Tensor, deltas, w1: Optional[torch.Tensor], w2: Optional[torch.Tensor], out1: Optional[torch.Tensor],
                 out2: Optional[torch.Tensor], eps: float, rows: Optional[torch.Tensor] = None, dtype: Optional[torch.dtype] = None) -> None:
    """x = residual + (d1 + d2), written back unless ``rows``; out1 = x / rms(x) * w1, out2 = x / rms(x) * w2 (one root mean
    square for both).  ``deltas``: up to two tensors, each [n, hidden] in the compute dtype (any row stride) or float32
    pieces [S, n, hidden]; outputs may be None."""
    deltas = [d for d in (deltas or ()) if d is not None]
    _need(len(deltas) <= 2, "pair_rmsnorm: at most two deltas")
    _cuda(residual, w1, w2, out1, out2, rows, *deltas)
    _i32(rows, "rows")
    hidden = residual.shape[-1]
    n = rows.numel() if rows is not None else residual.shape[0]
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "pair_rmsnorm: the residual stream is float32")
    if dtype is None:
        dtype = next((t.dtype for t in (out1, out2) if t is not None), None) or next((d.dtype for d in deltas if d.dim() == 2), torch.float32)
    args = []
    for d in deltas + [None] * (2 - len(deltas)):
        if d is None:
            args += [ctypes.c_void_p(0), ctypes.c_longlong(0), ctypes.c_void_p(0), 0, ctypes.c_longlong(0)]
        elif d.dim() == 3:
            _need(d.dtype == torch.float32 and d.is_contiguous() and tuple(d.shape[1:]) == tuple(residual.shape),
                  "pair_rmsnorm: pieces must be float32 [S, rows, hidden]")
            args += [ctypes.c_void_p(0), ctypes.c_longlong(0), _ptr(d), d.shape[0], ctypes.c_longlong(d.shape[1] * d.shape[2])]
        else:
            _need(d.dtype == dtype and d.dim() == 2 and d.shape[1] == hidden and d.stride(1) == 1 and d.shape[0] >= residual.shape[0],
                  "pair_rmsnorm: a delta must be [rows, hidden] in the compute dtype")
            args += [_ptr(d), ctypes.c_longlong(d.stride(0)), ctypes.c_void_p(0), 0, ctypes.c_longlong(0)]
    for w, o in ((w1, out1), (w2, out2)):
        _need(w is None or (w.dtype == torch.float32 and w.is_contiguous() and w.numel() == hidden), "pair_rmsnorm: float32 [hidden] weights")
        _need(o is None or (w is not None and o.is_contiguous() and o.dtype == dtype and o.shape[-1] == hidden and o.shape[0] >= n),
              "pair_rmsnorm: output shape")
    _check(lib("norms").kl_pair_rmsnorm(_ptr(residual), *args, _ptr(w1), _ptr(w2), ctypes.c_float(eps), _ptr(out1), _ptr(out2), _ptr(rows),
                                        n, hidden, dtype_code(dtype), _stream()), "pair_rmsnorm")


def activation(x: torch.Tensor, out: torch.Tensor, kind: str, params: Optional[torch.Tensor] = None) -> None:
    """out = act(x) element by element; ``kind`` in ACTIVATIONS.  "xielu" takes ``params`` = float32
    [softplus(p), 1/2 + softplus(q)]: a z^2 + z / 2 above zero, b (exp(z) - 1 - z) + z / 2 below."""
    _cuda(x, out, params)
    n, width = x.shape
    _columns(x, n, width, "activation: x"); _columns(out, n, width, "activation: out")
    _need(x.dtype == out.dtype, "activation: dtypes differ")
    _need(params is None or (params.dtype == torch.float32 and params.numel() >= 2 and params.is_contiguous()), "activation: params")
    _check(lib("elementwise").kl_activation(_ptr(x), ctypes.c_longlong(x.stride(0)), _ptr(out), ctypes.c_longlong(out.stride(0)), n, width,
                                            ACTIVATIONS[kind], _ptr(params), dtype_code(x.dtype), _stream()), "activation")


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor, group: int = 1) -> None:
    """x[t, i] *= sigmoid(gate[t, i // group]) in place; x [tokens, width] and gate [tokens, width / group] in the
    compute dtype, any row stride.  ``group`` = a head's width gates every head by one number."""
    _cuda(x, gate)
    n, width = x.shape
    _need(group >= 1 and width % group == 0, "sigmoid_gate: the width must be a multiple of the group")
    _columns(x, n, width, "sigmoid_gate: x"); _columns(gate, n, width // group, "sigmoid_gate: gate")
    _need(x.dtype == gate.dtype, "sigmoid_gate: dtypes differ")
    _check(lib("elementwise").kl_sigmoid_gate(_ptr(x), ctypes.c_longlong(x.stride(0)), _ptr(gate), ctypes.c_longlong(gate.stride(0)),
                                              n, width, group, dtype_code(x.dtype), _stream()), "sigmoid_gate")


# --------------------------------------------------------------------------- recurrent mixers

MINGRU_CHUNK = 32              # equals MG_CHUNK in recurrent.cu
MINGRU_CHUNKED_FROM = 256      # tokens of the longest sequence from which a step takes the chunked scan


def mingru_scan(proj: torch.Tensor, z_col: int, x_col: int, g_col: int, bias_z: Optional[torch.Tensor], bias_x: Optional[torch.Tensor],
                state: torch.Tensor, out: torch.Tensor, step, width: int) -> None:
    """The minGRU recurrence over a ragged step.  ``proj`` [rows, >= 3 width] holds the z, x and gate
    projections at the given columns; ``state`` float32 [slots, width] is read and left updated."""
    _cuda(proj, bias_z, bias_x, state, out)
    _need(proj.dim() == 2 and proj.stride(1) == 1 and max(z_col, x_col, g_col) + width <= proj.shape[1], "mingru_scan: projections")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.shape[1] == width and state.stride(1) == 1, "mingru_scan: state")
    _need(out.is_contiguous() and out.dtype == proj.dtype and out.shape[1] == width and out.shape[0] >= step.n_tokens, "mingru_scan: out")
    for b in (bias_z, bias_x):
        _need(b is None or (b.dtype == torch.float32 and b.numel() == width and b.is_contiguous()), "mingru_scan: bias")
    # Steps with long sequences run in chunks of 32 tokens (three passes, every chunk at once); a thread that
    # walks its channel alone is faster while a sequence brings few chunks.
    scratch, launches = None, 1
    if step.max_new >= MINGRU_CHUNKED_FROM:
        chunks = -(-step.max_new // MINGRU_CHUNK)
        scratch = torch.empty(step.n_seqs * chunks * 3 * width, dtype=torch.float32, device=proj.device)
        launches = 3
    _check(lib("recurrent").kl_mingru_scan(_ptr(proj), ctypes.c_longlong(proj.stride(0)), z_col, x_col, g_col, _ptr(bias_z), _ptr(bias_x),
                                           _ptr(state), ctypes.c_longlong(state.stride(0)), _ptr(out), _ptr(step.cu_tokens),
                                           _ptr(step.seq_slots), step.n_seqs, step.max_new, _ptr(scratch), width,
                                           dtype_code(proj.dtype), _stream()), "mingru_scan", launches)


def gated_delta_rule(proj: torch.Tensor, conv_col: int, b_col: int, a_col: int, conv_weight: torch.Tensor, A_log: torch.Tensor,
                     dt_bias: torch.Tensor, state: torch.Tensor, conv_off: int, out: torch.Tensor, step, heads: int, kv_heads: int,
                     dim: int, vdim: int, q_scale: float, unit_eps: float) -> None:
    """The gated delta rule over a ragged step (see recurrent.cu).  ``proj`` holds q | k | v at
    ``conv_col`` and the projections of beta and of the decay at ``b_col`` and ``a_col``;
    ``conv_weight`` float32 [2 G d + H dv, taps]; ``state`` float32 [slots, S | convolution state];
    ``out`` float32 [rows, H * dv]."""
    _cuda(proj, conv_weight, A_log, dt_bias, state, out)
    C = 2 * kv_heads * dim + heads * vdim
    taps = conv_weight.shape[1]
    n = step.n_tokens
    _need(proj.dim() == 2 and proj.stride(1) == 1 and conv_col + C <= proj.shape[1] and max(b_col, a_col) + heads <= proj.shape[1],
          "gated_delta_rule: projections")
    _need(conv_weight.dtype == torch.float32 and conv_weight.is_contiguous() and conv_weight.shape[0] == C, "gated_delta_rule: taps")
    _need(all(t.dtype == torch.float32 and t.numel() == heads and t.is_contiguous() for t in (A_log, dt_bias)), "gated_delta_rule: per-head vectors")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1
          and state.shape[1] >= conv_off + (taps - 1) * C and conv_off >= heads * vdim * dim, "gated_delta_rule: state")
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.shape[0] >= n and out.shape[1] == heads * vdim, "gated_delta_rule: out")
    _need(dim <= 256, f"gated_delta_rule: key size {dim} is above 256")
    prep = torch.empty((n, C), dtype=torch.float32, device=proj.device)
    bg = torch.empty((n, 2 * heads + kv_heads), dtype=torch.float32, device=proj.device)
    _check(lib("recurrent").kl_gated_delta_rule(
        _ptr(proj), ctypes.c_longlong(proj.stride(0)), conv_col, b_col, a_col, _ptr(conv_weight), taps, _ptr(A_log), _ptr(dt_bias),
        _ptr(state), ctypes.c_longlong(state.stride(0)), ctypes.c_longlong(conv_off), _ptr(prep), _ptr(bg), _ptr(out),
        _ptr(step.cu_tokens), _ptr(step.seq_slots), step.n_seqs, step.max_new, heads, kv_heads, dim, vdim, ctypes.c_float(q_scale),
        ctypes.c_float(unit_eps), dtype_code(proj.dtype), _stream()), "gated_delta_rule", 2)


# --------------------------------------------------------------------------- position encoding + cache write

def rope_kv_write(qkv: torch.Tensor, inv_freq: Optional[torch.Tensor], rotary_dim: int, positions: torch.Tensor,
                  token_slot: torch.Tensor, block_table: torch.Tensor, k_cache: Optional[torch.Tensor],
                  v_cache: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int,
                  partials: Optional[torch.Tensor] = None, values_are_keys: bool = False) -> None:
    """Rotate the query heads of ``qkv`` [tokens, (H + 2 KV) * hd] in place; rotate the key
    heads and store them, and the value heads, into the paged cache
    [pages, KV, PAGE, hd] (skipped when both caches are None).  With ``partials`` (float32
    [S, tokens, width]) the projections are the sum of those pieces and ``qkv`` only receives
    the rotated queries.  ``qkv`` may be wider than that (the leading columns of a stacked product
    count).  With ``values_are_keys`` it holds no value heads: the key heads as they are, before
    rotation, are stored as values."""
    _cuda(qkv, inv_freq, positions, token_slot, block_table, k_cache, v_cache, partials)
    n_parts, stride = 0, 0
    if partials is not None:
        _need(partials.dtype == torch.float32 and partials.is_contiguous() and tuple(partials.shape[1:]) == tuple(qkv.shape),
              "rope_kv_write: partial sums must be float32 [S, tokens, width]")
        n_parts, stride = partials.shape[0], partials.shape[1] * partials.shape[2]
    _i32(positions, "positions"); _i32(token_slot, "token_slot"); _i32(block_table, "block_table")
    n = qkv.shape[0]
    cols = (num_heads + (1 if values_are_keys else 2) * num_kv_heads) * head_dim
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= cols, "rope_kv_write: qkv shape")
    _need(partials is None or (qkv.is_contiguous() and qkv.shape[1] == cols and not values_are_keys), "rope_kv_write: pieces need plain rows")
    _need(positions.numel() >= n and token_slot.numel() >= n, "rope_kv_write: one position and slot per token")
    write = k_cache is not None
    if write:
        _need(v_cache is not None and k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype, "rope_kv_write: cache dtype")
        _need(k_cache.is_contiguous() and v_cache.is_contiguous()
              and tuple(k_cache.shape[1:]) == (num_kv_heads, PAGE, head_dim) and k_cache.shape == v_cache.shape,
              "rope_kv_write: cache layout must be [pages, kv_heads, 64, head_dim]")
    if rotary_dim:
        _need(inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2,
              "rope_kv_write: inv_freq must be float32 [rotary_dim / 2]")
    _check(lib("rope_kv").kl_rope_kv_write(_ptr(qkv), _ptr(partials), n_parts, ctypes.c_longlong(stride),
                                           _ptr(inv_freq), rotary_dim, _ptr(positions), _ptr(token_slot),
                                           _ptr(block_table), block_table.shape[1], _ptr(k_cache), _ptr(v_cache), n,
                                           num_heads, num_kv_heads, head_dim, int(write), ctypes.c_longlong(qkv.stride(0)),
                                           int(values_are_keys), dtype_code(qkv.dtype), _stream()), "rope_kv_write")


# --------------------------------------------------------------------------- attention

def attention_simt(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                   block_table: torch.Tensor, positions: torch.Tensor, token_slot: torch.Tensor, n_tokens: int,
                   num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: int = 0,
                   value_dim: Optional[int] = None, sink: Optional[torch.Tensor] = None) -> None:
    """out[t, h] = softmax(scale * q[t, h] . K[slot_t, lo..pos_t]) V over the paged cache.  ``value_dim``: the
    values are the first so many columns of ``v_cache``'s rows (which may be the key cache itself);
    ``sink``: float32 [heads], exp(sink[h]) joins head h's denominator."""
    _cuda(q, out, k_cache, v_cache, block_table, positions, token_slot, sink)
    _i32(positions, "positions"); _i32(token_slot, "token_slot"); _i32(block_table, "block_table")
    vd = head_dim if value_dim is None else int(value_dim)
    _need(out.is_contiguous() and out.shape[0] >= n_tokens and out.shape[1] == num_heads * vd, "attention: out shape")
    _need(q.dtype == out.dtype == k_cache.dtype == v_cache.dtype, "attention: dtypes differ")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous()
          and tuple(k_cache.shape[1:]) == (num_kv_heads, PAGE, head_dim), "attention: cache layout")
    _need(tuple(v_cache.shape[1:3]) == (num_kv_heads, PAGE) and v_cache.shape[3] >= vd, "attention: value cache layout")
    _need(0 < vd <= 512, f"attention: value size {vd} must be at most 512")
    _need(num_heads % num_kv_heads == 0, "attention: heads must be a multiple of kv heads")
    _need(sink is None or (sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == num_heads), "attention: sink")
    _check(lib("attention_simt").kl_attention_simt(_ptr(q), q_stride, _ptr(out), _ptr(k_cache), _ptr(v_cache),
                                                   _ptr(block_table), block_table.shape[1], _ptr(positions),
                                                   _ptr(token_slot), n_tokens, num_heads, num_kv_heads, head_dim,
                                                   ctypes.c_float(scale), int(window or 0), vd, int(v_cache.shape[3]), _ptr(sink),
                                                   dtype_code(q.dtype), _stream()), "attention_simt")


def qk_prepare(proj: torch.Tensor, q_col: int, k_col: int, v_col: Optional[int], positions: torch.Tensor, token_slot: torch.Tensor,
               block_table: Optional[torch.Tensor], k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], n_tokens: int,
               num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, *, q_bias: Optional[torch.Tensor] = None,
               k_bias: Optional[torch.Tensor] = None, v_bias: Optional[torch.Tensor] = None, inv_freq: Optional[torch.Tensor] = None,
               rotary_dim: int = 0, interleaved: bool = False, head_norm: bool = False, eps: float = 0.0,
               q_norm_weight: Optional[torch.Tensor] = None, k_norm_weight: Optional[torch.Tensor] = None) -> None:
    """For every token of ``proj`` [tokens, ...] (q heads from column ``q_col``, k heads from ``k_col``, v heads from ``v_col``):
    add the biases (float32), turn the first ``rotary_dim`` elements of every q and k head by the position (pairs (2i, 2i + 1)
    if ``interleaved``, else (i, i + rotary_dim / 2)), with ``head_norm`` divide every q and k head by its root mean square
    (``eps`` inside the root) and multiply by ``q_norm_weight`` / ``k_norm_weight`` (float32 [head_dim]) where given; q goes back
    in place, k into ``k_cache`` [pages, KV, PAGE, head_dim], v into ``v_cache`` [pages, KV, PAGE, value_dim].  ``v_col`` None:
    the key heads as projected (with bias, before rotation and norm) are the values.  Both caches None: only q is made."""
    _cuda(proj, positions, token_slot, block_table, k_cache, v_cache, q_bias, k_bias, v_bias, inv_freq, q_norm_weight, k_norm_weight)
    _i32(positions, "positions"); _i32(token_slot, "token_slot"); _i32(block_table, "block_table")
    H, KV, hd, vd = num_heads, num_kv_heads, head_dim, value_dim
    _need(proj.dim() == 2 and proj.stride(1) == 1 and proj.shape[0] >= n_tokens, "qk_prepare: projections")
    _need(q_col + H * hd <= proj.shape[1] and k_col + KV * hd <= proj.shape[1] and (v_col is None or v_col + KV * vd <= proj.shape[1]),
          "qk_prepare: columns")
    _need(positions.numel() >= n_tokens and token_slot.numel() >= n_tokens, "qk_prepare: one position and slot per token")
    for b, size, name in ((q_bias, H * hd, "q_bias"), (k_bias, KV * hd, "k_bias"), (v_bias, KV * vd, "v_bias"),
                          (q_norm_weight, hd, "q_norm_weight"), (k_norm_weight, hd, "k_norm_weight")):
        _need(b is None or (b.dtype == torch.float32 and b.is_contiguous() and b.numel() == size), f"qk_prepare: {name} must be float32 [{size}]")
    _need(rotary_dim == 0 or (inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2),
          "qk_prepare: inv_freq must be float32 [rotary_dim / 2]")
    _need((k_cache is None) == (v_cache is None), "qk_prepare: both caches or none")
    if k_cache is not None:
        _need(block_table is not None and k_cache.dtype == proj.dtype == v_cache.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
              and tuple(k_cache.shape[1:]) == (KV, PAGE, hd) and tuple(v_cache.shape[1:]) == (KV, PAGE, vd), "qk_prepare: cache layout")
    _need(v_col is not None or vd == hd, "qk_prepare: values that are keys have the keys' size")
    _check(lib("qk_prepare").kl_qk_prepare(
        _ptr(proj), ctypes.c_longlong(proj.stride(0)), q_col, k_col, -1 if v_col is None else v_col, _ptr(q_bias), _ptr(k_bias), _ptr(v_bias),
        _ptr(inv_freq), int(rotary_dim), int(bool(interleaved)), int(bool(head_norm)), ctypes.c_float(eps), _ptr(q_norm_weight),
        _ptr(k_norm_weight), _ptr(positions), _ptr(token_slot), _ptr(block_table), 0 if block_table is None else block_table.shape[1],
        _ptr(k_cache), _ptr(v_cache), n_tokens, H, KV, hd, vd, dtype_code(proj.dtype), _stream()), "qk_prepare")


ATTENTION_WEIGHTS = {"softmax": 0, "sigmoid": 1}


def attention_pooled(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                     positions: torch.Tensor, token_slot: torch.Tensor, n_tokens: int, num_heads: int, num_kv_heads: int, head_dim: int,
                     value_dim: int, scale: float, window: int, *, weights: str = "softmax", sink: Optional[torch.Tensor] = None,
                     head_bias: Optional[torch.Tensor] = None, pooled=None) -> None:
    """out[t, h] = sum over what token t sees of weight * value: the keys of the last ``window`` positions (0: all) and, with
    ``pooled`` (k, v [pages, KV, PAGE, dim] in the cache's dtype, block_table, pool), the mean key and value of every block of ``pool``
    positions that lies wholly before the window.  ``weights`` "softmax" (``sink``: float32 [heads] in the denominator) or
    "sigmoid" (sigmoid(score + head_bias[h]), not normalised).  ``q`` [tokens, >= heads * head_dim] with any row stride."""
    pk = pv = pt = None
    pool = 0
    if pooled is not None:
        pk, pv, pt, pool = pooled.k, pooled.v, pooled.block_table, int(pooled.pool)
    _cuda(q, out, k_cache, v_cache, block_table, positions, token_slot, sink, head_bias, pk, pv, pt)
    _i32(positions, "positions"); _i32(token_slot, "token_slot"); _i32(block_table, "block_table"); _i32(pt, "pooled block_table")
    H, KV, hd, vd = num_heads, num_kv_heads, head_dim, value_dim
    _need(q.dim() == 2 and q.stride(1) == 1 and q.shape[1] >= H * hd and q.shape[0] >= n_tokens, "attention_pooled: q")
    _need(out.is_contiguous() and out.shape[0] >= n_tokens and out.shape[1] == H * vd, "attention_pooled: out shape")
    _need(q.dtype == out.dtype == k_cache.dtype == v_cache.dtype, "attention_pooled: dtypes differ")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous() and tuple(k_cache.shape[1:]) == (KV, PAGE, hd)
          and tuple(v_cache.shape[1:]) == (KV, PAGE, vd), "attention_pooled: cache layout")
    _need(H % KV == 0 and 0 < vd <= 512, "attention_pooled: heads must be a multiple of kv heads, values at most 512 wide")
    for b, name in ((sink, "sink"), (head_bias, "head_bias")):
        _need(b is None or (b.dtype == torch.float32 and b.is_contiguous() and b.numel() == H), f"attention_pooled: {name} must be float32 [heads]")
    _need(weights in ATTENTION_WEIGHTS, f"attention_pooled: weights {weights!r} (softmax, sigmoid)")
    if pool:
        _need(window > 0 and pk.dtype == pv.dtype == k_cache.dtype and pk.is_contiguous() and pv.is_contiguous()
              and tuple(pk.shape[1:]) == (KV, PAGE, hd) and tuple(pv.shape[1:]) == (KV, PAGE, vd), "attention_pooled: pooled rows")
    _check(lib("attention_pooled").kl_attention_pooled(
        _ptr(q), ctypes.c_longlong(q.stride(0)), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
        _ptr(pk), _ptr(pv), _ptr(pt), 0 if pt is None else pt.shape[1], pool, _ptr(positions), _ptr(token_slot), n_tokens, H, KV, hd,
        ctypes.c_float(scale), int(window or 0), vd, _ptr(sink), _ptr(head_bias), ATTENTION_WEIGHTS[weights], dtype_code(q.dtype),
        _stream()), "attention_pooled")


def pool_blocks(k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor, pooled, step, num_kv_heads: int, head_dim: int,
                value_dim: int) -> None:
    """Writes the mean key and mean value (32-bit sums, stored in the cache's dtype) of every block of ``pooled.pool`` positions
    whose last position is one of the step's tokens, from the rows the cache holds."""
    _cuda(k_cache, v_cache, block_table, pooled.k, pooled.v, pooled.block_table)
    _i32(block_table, "block_table"); _i32(pooled.block_table, "pooled block_table")
    KV, hd, vd = num_kv_heads, head_dim, value_dim
    _need(k_cache.dtype == v_cache.dtype and k_cache.is_contiguous() and v_cache.is_contiguous() and tuple(k_cache.shape[1:]) == (KV, PAGE, hd)
          and tuple(v_cache.shape[1:]) == (KV, PAGE, vd), "pool_blocks: cache layout")
    _need(pooled.k.dtype == pooled.v.dtype == k_cache.dtype and pooled.k.is_contiguous() and pooled.v.is_contiguous()
          and tuple(pooled.k.shape[1:]) == (KV, PAGE, hd) and tuple(pooled.v.shape[1:]) == (KV, PAGE, vd), "pool_blocks: pooled rows")
    _check(lib("attention_pooled").kl_pool_blocks(
        _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(pooled.k), _ptr(pooled.v), _ptr(pooled.block_table),
        pooled.block_table.shape[1], int(pooled.pool), _ptr(step.seq_slots), _ptr(step.seq_starts), _ptr(step.seq_new), step.n_seqs,
        step.max_new, KV, hd, vd, dtype_code(k_cache.dtype), _stream()), "pool_blocks")


# --------------------------------------------------------------------------- grouped products

GROUPED_MMA_FROM_ROWS = 32       # rows from which a batched bfloat16 product takes the tensor-core kernel
EPILOGUE_ACTIVATIONS = {"relu2": 1}     # what the grouped products' plain epilogues can apply themselves: max(y, 0)^2


def _epilogue_activation(activation: Optional[str], gated) -> int:
    if activation is None:
        return 0
    _need(gated is None and activation in EPILOGUE_ACTIVATIONS,
          f"an ungated grouped product's epilogue applies one of {sorted(EPILOGUE_ACTIVATIONS)}, not {activation!r}")
    return EPILOGUE_ACTIVATIONS[activation]



def grouped_gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, a_group_stride: int = 0, out_group_stride: int = 0,
                 rows: Optional[int] = None, a_rows: Optional[torch.Tensor] = None, tile_group: Optional[torch.Tensor] = None,
                 tile_rows: int = 64, gated: Optional[tuple] = None, interleaved: bool = False,
                 row_gate: Optional[torch.Tensor] = None, activation: Optional[str] = None, gate_elements: bool = False) -> None:
    """out_g = a_g @ w[g]^T for every group g, with ``w`` [groups, N (2 N if gated), K].

    Batched (``tile_group`` None): all ``rows`` rows for every group; group g reads the columns of ``a`` from
    g * a_group_stride and writes the columns of ``out`` from g * out_group_stride.  Routed: ``tile_group``
    [tiles] names the group of every tile of ``tile_rows`` list places (-1: none) and ``a_rows`` [tiles *
    tile_rows] the row of ``a`` each place reads (-1: padding; None: the place itself); ``out`` is indexed by
    place.  ``gated`` = (limit, alpha, shift): the weights hold N gate rows then N up rows and the result
    is min(g, limit) * sigmoid(alpha * min(g, limit)) * (clamp(u, -limit, limit) + shift); limit <= 0 clamps nothing.
    ``interleaved``: the gated weights alternate 64 gate rows and the 64 up rows of the same outputs instead.
    ``row_gate`` [rows, groups] (batched, plain): group g's result of row t is multiplied by sigmoid(row_gate[t, g]); with
    ``gate_elements`` it is [rows, groups * N] and every output has a number of its own, sigmoid(row_gate[t, g * N + n]).
    ``activation`` (plain): an activation of the result in the same kernel (``EPILOGUE_ACTIVATIONS``)."""
    _cuda(a, w, out, a_rows, tile_group)
    act = _epilogue_activation(activation, gated)
    _i32(a_rows, "a_rows"); _i32(tile_group, "tile_group")
    _need(w.dim() == 3 and w.is_contiguous() and a.dtype == w.dtype, "grouped_gemm: weights must be contiguous [groups, N, K] in a's dtype")
    G, NW, K = w.shape
    N = NW // 2 if gated is not None else NW
    _need(gated is None or NW % 2 == 0, "grouped_gemm: gated weights hold gate rows and up rows")
    _need(a.dim() == 2 and a.stride(1) == 1 and out.dim() == 2 and out.stride(1) == 1, "grouped_gemm: rows must be contiguous")
    _need(tile_rows in (16, 64), "grouped_gemm: tiles of 16 or 64 rows")
    _need(not interleaved or (gated is not None and N % 64 == 0), "grouped_gemm: interleaved rows come in blocks of 64 gate and 64 up rows")
    if tile_group is None:
        M = a.shape[0] if rows is None else int(rows)
        _need(a_rows is None and M <= a.shape[0] and M <= out.shape[0], "grouped_gemm: rows")
        _need((G - 1) * a_group_stride + K <= a.shape[1] and (G - 1) * out_group_stride + N <= out.shape[1], "grouped_gemm: columns")
        tiles = 0
    else:
        tiles = tile_group.numel()
        M = tiles * tile_rows
        _need(out.shape[0] >= M and out.shape[1] >= N and a.shape[1] >= K, "grouped_gemm: shapes")
        _need(a_rows is None or a_rows.numel() >= M, "grouped_gemm: one source row per list place")
        _need(a_rows is not None or a.shape[0] >= M, "grouped_gemm: a holds fewer rows than the list")
        a_group_stride = out_group_stride = 0
    lim, alpha, shift = gated if gated is not None else (0.0, 1.0, 0.0)
    if row_gate is not None:
        _cuda(row_gate)
        _need(tile_group is None and gated is None and row_gate.dtype == a.dtype and row_gate.dim() == 2 and row_gate.stride(1) == 1
              and row_gate.shape[0] >= M and row_gate.shape[1] == (G * N if gate_elements else G),
              "grouped_gemm: row_gate is [rows, groups] (or [rows, groups * N]) of a batched plain product")
    if (tile_group is None and gated is None and not act and a.dtype == out.dtype == torch.bfloat16 and M >= GROUPED_MMA_FROM_ROWS and K % 8 == 0
            and a.stride(0) % 8 == 0 and a_group_stride % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
        # a prompt's per-head projections: the tensor cores
        _check(lib("grouped_gemm").kl_grouped_gemm_mma(
            _ptr(a), ctypes.c_longlong(a.stride(0)), ctypes.c_longlong(a_group_stride), _ptr(w), ctypes.c_longlong(NW * K), _ptr(out),
            ctypes.c_longlong(out.stride(0)), ctypes.c_longlong(out_group_stride), G, M, N, K, _ptr(row_gate),
            ctypes.c_longlong(0 if row_gate is None else row_gate.stride(0)), int(bool(gate_elements)), _stream()), "grouped_gemm_mma")
        return
    _check(lib("grouped_gemm").kl_grouped_gemm(
        _ptr(a), ctypes.c_longlong(a.stride(0)), ctypes.c_longlong(a_group_stride), _ptr(a_rows), _ptr(w), ctypes.c_longlong(NW * K),
        _ptr(out), ctypes.c_longlong(out.stride(0)), ctypes.c_longlong(out_group_stride), _ptr(tile_group), tiles, tile_rows, G, M, N, K,
        int(gated is not None), ctypes.c_float(lim), ctypes.c_float(alpha), ctypes.c_float(shift), int(bool(interleaved)), _ptr(row_gate),
        ctypes.c_longlong(0 if row_gate is None else row_gate.stride(0)), dtype_code(a.dtype),
        dtype_code(out.dtype), act, int(bool(gate_elements)), _stream()), "grouped_gemm")


def grouped_gemv(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, a_rows: Optional[torch.Tensor], tile_group: torch.Tensor,
                 tile_rows: int, gated: Optional[tuple] = None, interleaved: bool = False, live_rows: Optional[torch.Tensor] = None,
                 activation: Optional[str] = None) -> None:
    """The routed product of ``grouped_gemm`` for few rows per group (a decode step): every group's weights are read once,
    a warp per four weight rows.  bfloat16 operands whose rows start on 16-byte boundaries.  ``a_rows`` None: a place reads
    its own row of ``a``, and ``live_rows`` (the list's rows, -1 at padding) says which places there are."""
    _cuda(a, w, out, a_rows, tile_group, live_rows)
    _i32(a_rows, "a_rows"); _i32(tile_group, "tile_group"); _i32(live_rows, "live_rows")
    G, NW, K = w.shape
    N = NW // 2 if gated is not None else NW
    tiles = tile_group.numel()
    _need(w.is_contiguous() and a.dtype == w.dtype == torch.bfloat16 and a.stride(1) == 1 and out.stride(1) == 1 and a.shape[1] == K
          and out.shape[0] >= tiles * tile_rows and out.shape[1] >= N, "grouped_gemv: shapes")
    _need(K % 8 == 0 and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0, "grouped_gemv: rows on 16-byte boundaries")
    _need(a_rows is None or a_rows.numel() >= tiles * tile_rows, "grouped_gemv: one source row per list place")
    lim, alpha, shift = gated if gated is not None else (0.0, 1.0, 0.0)
    _need(live_rows is None or live_rows.numel() >= tiles * tile_rows, "grouped_gemv: live_rows")
    _check(lib("grouped_gemm").kl_grouped_gemv(
        _ptr(a), ctypes.c_longlong(a.stride(0)), _ptr(a_rows), _ptr(live_rows), _ptr(w), ctypes.c_longlong(NW * K), _ptr(out),
        ctypes.c_longlong(out.stride(0)), _ptr(tile_group), tiles, tile_rows, N, K, int(gated is not None), ctypes.c_float(lim),
        ctypes.c_float(alpha), ctypes.c_float(shift), int(bool(interleaved)), dtype_code(out.dtype), _epilogue_activation(activation, gated),
        _stream()), "grouped_gemv")


# --------------------------------------------------------------------------- mixture of experts

MOE_MAX_EXPERTS = 256          # equals MOE_MAX_EXPERTS in moe.cu


def moe_route(logits: torch.Tensor, top: int, renormalise: bool = False, groups: int = 1, keep_groups: int = 1,
              renorm_eps: float = 0.0, bias: Optional[torch.Tensor] = None):
    """(choice int32 [tokens, top], weight float32 [tokens, top]) from float32 router logits [tokens, experts]:
    softmax over all experts, the ``top`` largest, their scores (divided by their sum + ``renorm_eps`` if ``renormalise``).
    With ``groups`` > 1 the experts form that many equal groups of neighbours, a group's score is its largest score, and
    only experts of the ``keep_groups`` best groups can be chosen.  ``bias``: float32 [experts], added to the logits first."""
    _cuda(logits, bias)
    n, E = logits.shape
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == E), "moe_route: float32 bias per expert")
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "moe_route: float32 logits")
    _need(0 < top <= E <= MOE_MAX_EXPERTS, f"moe_route: {top} of {E} experts (at most {MOE_MAX_EXPERTS})")
    choice = torch.empty((n, top), dtype=torch.int32, device=logits.device)
    weight = torch.empty((n, top), dtype=torch.float32, device=logits.device)
    _need(groups >= 1 and E % groups == 0 and 1 <= keep_groups <= groups and top <= keep_groups * (E // groups),
          f"moe_route: {groups} groups of which {keep_groups} are kept do not hold {top} of {E} experts")
    _check(lib("moe").kl_moe_route(_ptr(logits), ctypes.c_longlong(logits.stride(0)), _ptr(bias), n, E, top, int(bool(renormalise)), int(groups),
                                   int(keep_groups), ctypes.c_float(renorm_eps), _ptr(choice), _ptr(weight), _stream()), "moe_route")
    return choice, weight


def moe_plan(choice: torch.Tensor, experts: int, tile_rows: int, token_slot: Optional[torch.Tensor] = None):
    """The list of (token, choice) pairs sorted by expert, every expert's run padded to whole tiles:
    (pair_pos int32 [tokens * top]: each pair's place, -1 for rows that belong to no sequence; list_rows int32
    [cap]: the token row of every place, -1 for padding; tile_group int32 [cap / tile_rows]: the expert of every tile)."""
    _cuda(choice, token_slot)
    _i32(choice, "choice"); _i32(token_slot, "token_slot")
    n, top = choice.shape
    cap = -(-(n * top + experts * (tile_rows - 1)) // tile_rows) * tile_rows
    tiles = cap // tile_rows
    dev = choice.device
    scratch = torch.empty(2 * n * top + cap + tiles, dtype=torch.int32, device=dev)
    rank, pair_pos, list_rows, tile_group = torch.split(scratch, [n * top, n * top, cap, tiles])
    _need(token_slot is None or token_slot.numel() >= n, "moe_plan: one slot per row")
    _check(lib("moe").kl_moe_plan(_ptr(choice), _ptr(token_slot), n, top, experts, tile_rows, cap, tiles, _ptr(rank), _ptr(pair_pos),
                                  _ptr(list_rows), _ptr(tile_group), _stream()), "moe_plan")
    return pair_pos, list_rows, tile_group


def moe_gather(x: torch.Tensor, list_rows: torch.Tensor) -> torch.Tensor:
    """bfloat16 [places, width]: x[list_rows[p]] at every place of the list, zeros at its padding places."""
    _cuda(x, list_rows)
    _i32(list_rows, "list_rows")
    _need(x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1, "moe_gather: bfloat16 rows")
    rows = torch.empty((list_rows.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    _check(lib("moe").kl_moe_gather(_ptr(x), ctypes.c_longlong(x.stride(0)), _ptr(list_rows), list_rows.numel(), x.shape[1], _ptr(rows),
                                    _stream()), "moe_gather")
    return rows


def gemm_tcgen05_grouped(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tile_group: torch.Tensor,
                         gated: Optional[tuple] = None, activation: Optional[str] = None) -> None:
    """out[p] = a[p] @ w[g]^T on the tensor cores for a list of places sorted by group, every tile of 128 places
    in one group (``tile_group`` [places / 128], -1: skipped).  ``w`` [groups, rows, K] bfloat16; ``gated`` =
    (limit, alpha, shift): a group's rows alternate 64 gate rows and 64 up rows, out has rows / 2 columns."""
    _cuda(a, w, out, tile_group)
    _i32(tile_group, "tile_group")
    G, R, K = w.shape
    M = tile_group.numel() * 128
    _need(w.is_contiguous() and a.shape[1] == K and a.shape[0] >= M and out.shape[0] >= M and out.dtype == torch.bfloat16
          and out.shape[1] == (R // 2 if gated is not None else R), "gemm_tcgen05_grouped: shapes")
    _need(_tc_ok(a, w[0], out) and (gated is None or R % 128 == 0), "gemm_tcgen05_grouped: bfloat16 operands with 16-byte aligned rows")
    lim, alpha, shift = gated if gated is not None else (0.0, 1.0, 0.0)
    _check(lib("gemm_tcgen05").kl_gemm_tcgen05_grouped(
        _ptr(a), ctypes.c_longlong(a.stride(0)), _ptr(w), ctypes.c_longlong(K), _ptr(out), ctypes.c_longlong(out.stride(0)), M, R, K, G,
        _ptr(tile_group), int(gated is not None), ctypes.c_float(lim), ctypes.c_float(alpha), ctypes.c_float(shift),
        _epilogue_activation(activation, gated), _status_ptr(a.device), _stream()), "gemm_tcgen05_grouped")


def gemm_tcgen05_grouped_skinny(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tile_group: torch.Tensor,
                                gated: Optional[tuple] = None, activation: Optional[str] = None) -> None:
    """The grouped product for few rows per group on the tensor cores, weights as tile rows: ``a`` holds the list's rows (tiles of
    16 places, ``tile_group`` [places / 16], -1: skipped); every chosen group's weights stream once through the TMA ring.
    Operands as for ``gemm_tcgen05_grouped``."""
    _cuda(a, w, out, tile_group)
    _i32(tile_group, "tile_group")
    G, R, K = w.shape
    M = tile_group.numel() * 16
    _need(w.is_contiguous() and a.shape[1] == K and a.shape[0] >= M and out.shape[0] >= M and out.dtype == torch.bfloat16
          and out.shape[1] == (R // 2 if gated is not None else R), "gemm_tcgen05_grouped_skinny: shapes")
    _need(_tc_ok(a, w[0], out) and (gated is None or R % 128 == 0), "gemm_tcgen05_grouped_skinny: bfloat16 operands with 16-byte aligned rows")
    lim, alpha, shift = gated if gated is not None else (0.0, 1.0, 0.0)
    _check(lib("gemm_tcgen05").kl_gemm_tcgen05_grouped_skinny(
        _ptr(a), ctypes.c_longlong(a.stride(0)), _ptr(w), ctypes.c_longlong(K), _ptr(out), ctypes.c_longlong(out.stride(0)), M, R, K, G,
        _ptr(tile_group), int(gated is not None), ctypes.c_float(lim), ctypes.c_float(alpha), ctypes.c_float(shift),
        _epilogue_activation(activation, gated), _status_ptr(a.device), _stream()), "gemm_tcgen05_grouped_skinny")


def moe_combine(results: torch.Tensor, pair_pos: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = sum_k weight[t, k] * results[pair_pos[t * top + k]] (float32 [tokens, hidden]), in the order of k."""
    _cuda(results, pair_pos, weight, out)
    n, top = weight.shape
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.shape[0] >= n and results.stride(1) == 1
          and results.shape[1] == out.shape[1], "moe_combine: shapes")
    _check(lib("moe").kl_moe_combine(_ptr(results), ctypes.c_longlong(results.stride(0)), _ptr(pair_pos), _ptr(weight), n, top,
                                     out.shape[1], _ptr(out), dtype_code(results.dtype), _stream()), "moe_combine")


# --------------------------------------------------------------------------- attention over a shared latent

def latent_prepare(proj: torch.Tensor, q_col: int, kv_col: Optional[int], norm_weight: Optional[torch.Tensor], eps: float,
                   inv_freq: Optional[torch.Tensor], rot_dims: int, mscale: float, interleaved: bool, positions: torch.Tensor,
                   token_slot: torch.Tensor, block_table: Optional[torch.Tensor], cache: Optional[torch.Tensor], qfull: torch.Tensor,
                   n_tokens: int, heads: int, dim: int, rot_dim: int, kv_rank: int, q: Optional[torch.Tensor] = None) -> None:
    """Per token: the normed latent and the rotated shared key part into the cache row (unless ``kv_col`` is
    None: the layer reads another layer's cache), and every head's rotated query part into the last
    ``rot_dim`` columns of its [kv_rank + rot_dim] slice of ``qfull`` (see latent.cu).  ``q``: the matrix that holds the
    queries from column ``q_col`` on, where that is not ``proj`` (queries that came through a latent of their own)."""
    _cuda(proj, norm_weight, inv_freq, positions, token_slot, block_table, cache, qfull, q)
    qsrc = proj if q is None else q
    _need(qsrc.dim() == 2 and qsrc.stride(1) == 1 and qsrc.dtype == proj.dtype and qsrc.shape[0] >= n_tokens, "latent_prepare: queries")
    _i32(positions, "positions"); _i32(token_slot, "token_slot"); _i32(block_table, "block_table")
    Dk = kv_rank + rot_dim
    _need(proj.dim() == 2 and proj.stride(1) == 1 and q_col + heads * (dim + rot_dim) <= qsrc.shape[1], "latent_prepare: projections")
    _need(qfull.is_contiguous() and qfull.dtype == proj.dtype and qfull.shape[0] >= n_tokens and qfull.shape[1] == heads * Dk,
          "latent_prepare: query buffer")
    if kv_col is not None:
        _need(kv_col + Dk <= proj.shape[1], "latent_prepare: the down-projection's columns")
        _need(cache is not None and cache.is_contiguous() and cache.dtype == proj.dtype and tuple(cache.shape[1:]) == (1, PAGE, Dk),
              "latent_prepare: cache layout")
        _need(norm_weight is not None and norm_weight.dtype == torch.float32 and norm_weight.numel() == kv_rank, "latent_prepare: norm weight")
    _need(rot_dims == 0 or (inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dims // 2),
          "latent_prepare: one frequency per pair")
    _check(lib("latent").kl_latent_prepare(
        _ptr(proj), ctypes.c_longlong(proj.stride(0)), _ptr(qsrc), ctypes.c_longlong(qsrc.stride(0)), q_col, -1 if kv_col is None else kv_col,
        _ptr(norm_weight), ctypes.c_float(eps),
        _ptr(inv_freq), rot_dims, ctypes.c_float(mscale), int(bool(interleaved)), _ptr(positions), _ptr(token_slot),
        _ptr(block_table), 0 if block_table is None else block_table.shape[1], _ptr(cache if kv_col is not None else None), _ptr(qfull),
        n_tokens, heads, dim, rot_dim, kv_rank, dtype_code(proj.dtype), _stream()), "latent_prepare")


def latent_decode_splits(n_seqs: int, heads: int, context_class: int) -> int:
    """Into how many runs a decode step cuts every sequence's pages: by the step's class of context length (never by the
    length itself: a captured step is replayed while the context grows inside its class), at least two pages a run, and
    no more CTAs than two for every multiprocessor."""
    head_blocks = -(-heads // 64)
    pages = 16 << max(0, int(context_class))                   # the most pages of the class
    room = max(1, (2 * sm_count()) // max(1, n_seqs * head_blocks))
    return max(1, min(pages // 2, room, 32))


LATENT_KERNEL = "mma"           # "simt": the plain kernel also for bfloat16 (for comparisons)


def latent_attention(qfull: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, step, heads: int,
                     key_dim: int, value_dim: int, scale: float, sink: Optional[torch.Tensor] = None, window: int = 0) -> None:
    """Causal attention of ``heads`` query heads [key_dim] over the one key head of the cache's rows, the values being
    each row's first ``value_dim`` columns; out [tokens, heads * value_dim].  bfloat16 with key and value sizes that are
    multiples of 16 and values up to 256 wide: the tensor-core kernel (attention_latent.cu); everything else: the plain one.
    ``window``: a token reads the keys of the last so many positions only (0: all)."""
    if (qfull.dtype == torch.bfloat16 and LATENT_KERNEL == "mma" and key_dim % 16 == 0 and value_dim % 16 == 0
            and value_dim <= 256 and 3 * 64 * (key_dim + 8) * 2 <= 220 * 1024):
        _cuda(qfull, out, cache, block_table, sink)
        _i32(block_table, "block_table")
        n = step.n_tokens
        _need(qfull.is_contiguous() and out.is_contiguous() and cache.is_contiguous() and out.dtype == cache.dtype == torch.bfloat16
              and qfull.shape[0] >= n and qfull.shape[1] == heads * key_dim and out.shape[0] >= n and out.shape[1] == heads * value_dim
              and tuple(cache.shape[1:]) == (1, PAGE, key_dim), "latent_attention: layouts")
        _need(sink is None or (sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == heads), "latent_attention: sink")
        splits, part = 1, None
        if step.is_decode and n == step.n_seqs:
            splits = latent_decode_splits(step.n_seqs, heads, getattr(step, "context_class", 0))
            if splits > 1:
                part = torch.empty(n * heads * splits * (value_dim + 2), dtype=torch.float32, device=qfull.device)
        _check(lib("attention_latent").kl_latent_attention_mma(
            _ptr(qfull), _ptr(out), _ptr(cache), _ptr(block_table), block_table.shape[1], _ptr(step.cu_tokens), _ptr(step.seq_slots),
            _ptr(step.seq_starts), _ptr(step.seq_new), step.n_seqs, step.max_new, _ptr(sink), heads, key_dim, value_dim,
            ctypes.c_float(scale), splits, _ptr(part), n, int(window or 0), _stream()), "latent_attention_mma", 2 if splits > 1 else 1)
        return
    attention_simt(qfull, heads * key_dim, out, cache, cache, block_table, step.positions, step.token_slot, step.n_tokens,
                   heads, 1, key_dim, scale, int(window or 0), value_dim=value_dim, sink=sink)


# --------------------------------------------------------------------------- gated linear recurrence

LINEAR_SCAN_CHUNK = 64           # tokens per chunk of the chunked scan
LINEAR_SCAN_CHUNKED_FROM = 256   # tokens of the longest sequence from which a step takes it


def causal_conv(proj: torch.Tensor, x_col: int, x_bias: Optional[torch.Tensor], weight: torch.Tensor, bias: Optional[torch.Tensor],
                state: torch.Tensor, step, width: int, out: torch.Tensor) -> None:
    """out[t, c] (float32) = bias[c] + sum_k weight[c, k] * x[t - (taps - 1 - k), c], x = proj[:, x_col + c] + x_bias[c];
    inputs before the step come from ``state`` [slots, width * taps] (S, then the last taps - 1 inputs)."""
    _cuda(proj, x_bias, weight, bias, state, out)
    taps = weight.shape[1]
    _need(weight.dtype == torch.float32 and weight.is_contiguous() and weight.shape[0] == width, "causal_conv: weight [width, taps]")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1 and state.shape[1] >= width * taps, "causal_conv: state")
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.shape[1] == width and out.shape[0] >= step.n_tokens, "causal_conv: out")
    _need(proj.dim() == 2 and proj.stride(1) == 1 and x_col + width <= proj.shape[1], "causal_conv: projections")
    for b in (x_bias, bias):
        _need(b is None or (b.dtype == torch.float32 and b.numel() == width and b.is_contiguous()), "causal_conv: bias")
    _check(lib("linear_recurrence").kl_causal_conv(
        _ptr(proj), ctypes.c_longlong(proj.stride(0)), x_col, _ptr(x_bias), _ptr(weight), _ptr(bias), taps, _ptr(state),
        ctypes.c_longlong(state.stride(0)), _ptr(step.cu_tokens), _ptr(step.seq_slots), _ptr(step.seq_new), step.n_seqs, step.max_new,
        width, _ptr(out), dtype_code(proj.dtype), _stream()), "causal_conv")


def rglru_gate(gates: torch.Tensor, u: torch.Tensor, r_bias: torch.Tensor, i_bias: torch.Tensor, softplus_lambda: torch.Tensor,
               decay_scale: float, n_tokens: int, width: int, block: int) -> None:
    """In place on ``gates`` float32 [tokens, blocks, 2 block] (recurrence gate then input gate pre-activations of
    every block): a = exp(-decay_scale * sigmoid(r) * softplus_lambda) over r, sqrt(1 - a^2) * sigmoid(i) * u over i."""
    _cuda(gates, u, r_bias, i_bias, softplus_lambda)
    for t in (gates, u, r_bias, i_bias, softplus_lambda):
        _need(t.dtype == torch.float32 and t.is_contiguous(), "rglru_gate: float32 tensors")
    _need(gates.shape[0] >= n_tokens and gates.shape[1] == 2 * width and u.shape[1] == width and width % block == 0, "rglru_gate: shapes")
    _check(lib("linear_recurrence").kl_rglru_gate(_ptr(gates), _ptr(u), _ptr(r_bias), _ptr(i_bias), _ptr(softplus_lambda),
                                                  ctypes.c_float(decay_scale), n_tokens, width, block, _stream()), "rglru_gate")


def linear_scan(gates: torch.Tensor, block: int, proj: torch.Tensor, y_col: int, x_col: int, y_bias: Optional[torch.Tensor],
                x_bias: Optional[torch.Tensor], taps: int, state: torch.Tensor, step, width: int, out: torch.Tensor) -> None:
    """S_t = a_t S_(t-1) + b_t per channel from the slot's state, a and b as ``rglru_gate`` left them;
    out[t, c] = S_t * gelu_tanh(proj[t, y_col + c] + y_bias[c]); the state (S and the convolution's last inputs) moves on."""
    _cuda(gates, proj, y_bias, x_bias, state, out)
    _need(gates.dtype == torch.float32 and gates.is_contiguous() and gates.shape[1] == 2 * width, "linear_scan: gates")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1 and state.shape[1] >= width * taps, "linear_scan: state")
    _need(out.is_contiguous() and out.dtype == proj.dtype and out.shape[1] == width and out.shape[0] >= step.n_tokens, "linear_scan: out")
    _need(proj.stride(1) == 1 and max(y_col, x_col) + width <= proj.shape[1], "linear_scan: projections")
    # A step with long sequences runs in chunks side by side (a chunk's decay product and result from zero; the states at the
    # chunks' starts; the chunks again with their outputs); a thread that walks its channel alone is faster for few tokens.
    scratch, launches = None, 1
    if step.max_new >= LINEAR_SCAN_CHUNKED_FROM:
        chunks = -(-step.max_new // LINEAR_SCAN_CHUNK)
        scratch = torch.empty(step.n_seqs * chunks * 2 * width, dtype=torch.float32, device=proj.device)
        launches = 3
    _check(lib("linear_recurrence").kl_linear_scan(
        _ptr(gates), block, _ptr(proj), ctypes.c_longlong(proj.stride(0)), y_col, x_col, _ptr(y_bias), _ptr(x_bias), taps, _ptr(state),
        ctypes.c_longlong(state.stride(0)), _ptr(step.cu_tokens), _ptr(step.seq_slots), _ptr(step.seq_new), step.n_seqs, step.max_new,
        width, _ptr(out), _ptr(scratch), LINEAR_SCAN_CHUNK, dtype_code(proj.dtype), _stream()), "linear_scan", launches)


# --------------------------------------------------------------------------- short convolutions, matrix-state recurrences

SHORT_CONV_MAX_TAPS = 16         # equals SC_MAX_TAPS in short_conv.cu


def short_conv(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor, step, out: torch.Tensor,
               add_input: bool = False, silu: bool = False, update_state: bool = True) -> None:
    """out[t, c] = act((x[t, c] if add_input) + bias[c] + sum_j weight[c, j] * x[t - (taps - 1) + j, c]) over a ragged step;
    inputs before the step come from ``state`` float32 [slots, >= (taps - 1) * channels] (the last taps - 1 inputs, oldest
    first; zeros in a fresh slot), which moves on unless ``update_state`` is False.  ``x`` [rows, channels] in the compute
    dtype (any row stride); ``out`` in the compute dtype or float32; act = SiLU if ``silu``."""
    _cuda(x, weight, bias, state, out)
    C, taps = weight.shape
    _need(weight.dtype == torch.float32 and weight.is_contiguous() and 1 <= taps <= SHORT_CONV_MAX_TAPS, "short_conv: weight [channels, taps]")
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == C), "short_conv: bias")
    _columns(x, step.n_tokens, C, "short_conv: x"); _columns(out, step.n_tokens, C, "short_conv: out")
    _need(out.dtype in (x.dtype, torch.float32), "short_conv: the output is float32 or in the input's dtype")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1 and state.shape[1] >= (taps - 1) * C, "short_conv: state")
    _check(lib("short_conv").kl_short_conv(
        _ptr(x), ctypes.c_longlong(x.stride(0)), _ptr(weight), _ptr(bias), taps, _ptr(state), ctypes.c_longlong(state.stride(0)),
        _ptr(step.cu_tokens), _ptr(step.seq_slots), step.n_seqs, step.max_new, C, int(bool(add_input)), int(bool(silu)), _ptr(out),
        ctypes.c_longlong(out.stride(0)), int(out.dtype == torch.float32), int(bool(update_state)), dtype_code(x.dtype), _stream()),
        "short_conv", 2 if update_state and taps > 1 else 1)


def decay_softplus(raw: torch.Tensor, bias: torch.Tensor, A_log: torch.Tensor, n_rows: int, dt: torch.Tensor, a: torch.Tensor) -> None:
    """dt = softplus(raw + bias) and a = exp(-exp(A_log) * dt) per (row, head), float32 [rows, heads]; ``raw`` [rows, heads] in the
    compute dtype (any row stride)."""
    _cuda(raw, bias, A_log, dt, a)
    heads = bias.numel()
    _columns(raw, n_rows, heads, "decay_softplus: raw")
    for t in (bias, A_log):
        _need(t.dtype == torch.float32 and t.is_contiguous() and t.numel() == heads, "decay_softplus: per-head vectors")
    for t in (dt, a):
        _need(t.dtype == torch.float32 and t.is_contiguous() and t.shape[0] >= n_rows and t.shape[1] == heads, "decay_softplus: outputs")
    _check(lib("outer_recurrence").kl_decay_softplus(_ptr(raw), ctypes.c_longlong(raw.stride(0)), 0, dtype_code(raw.dtype), _ptr(bias),
                                                     _ptr(A_log), n_rows, heads, _ptr(dt), _ptr(a), _stream()), "decay_softplus")


def decay_lowrank(r1: torch.Tensor, W2: torch.Tensor, b: Optional[torch.Tensor], tau: float, n_rows: int, a: torch.Tensor) -> None:
    """a = sigmoid(z)^(1 / tau), z = W2 r1 + b, float32 [rows, channels]; ``r1`` [rows, rank] in the compute dtype (any row
    stride), ``W2`` float32 [channels, rank]."""
    _cuda(r1, W2, b, a)
    C, rank = W2.shape
    _columns(r1, n_rows, rank, "decay_lowrank: r1")
    _need(W2.dtype == torch.float32 and W2.is_contiguous(), "decay_lowrank: W2")
    _need(b is None or (b.dtype == torch.float32 and b.is_contiguous() and b.numel() == C), "decay_lowrank: bias")
    _need(a.dtype == torch.float32 and a.is_contiguous() and a.shape[0] >= n_rows and a.shape[1] == C, "decay_lowrank: out")
    _check(lib("outer_recurrence").kl_decay_lowrank(_ptr(r1), ctypes.c_longlong(r1.stride(0)), 0, rank, _ptr(W2), _ptr(b),
                                                    ctypes.c_float(tau), n_rows, C, _ptr(a), dtype_code(r1.dtype), _stream()), "decay_lowrank")


def outer_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor, state: torch.Tensor, y: torch.Tensor, step,
                     heads: int, groups: int, N: int, P: int, c: Optional[torch.Tensor] = None, skip: Optional[torch.Tensor] = None,
                     q_scale: float = 1.0) -> None:
    """S_t = diag(a_t) S_(t-1) + (c_t k_t) v_t^T and y_t = S_t^T (q_scale q_t) + skip v_t per head over a ragged step, from and
    into ``state`` float32 [slots, >= heads * N * P] (S as [heads, N, P]).  ``q``, ``k`` [rows, groups * N] and ``v``
    [rows, heads * P] share one dtype (float32 or the compute dtype) and may be column slices; ``a`` float32 [rows, heads]
    (one decay per head) or [rows, heads * N] (one per row of S); ``c`` float32 [rows, heads] or None; ``skip`` float32
    [heads] or None; ``y`` float32 [rows, heads * P]."""
    _cuda(q, k, v, a, state, y, c, skip)
    n = step.n_tokens
    _columns(q, n, groups * N, "outer_recurrence: q"); _columns(k, n, groups * N, "outer_recurrence: k")
    _columns(v, n, heads * P, "outer_recurrence: v")
    _need(q.dtype == k.dtype == v.dtype, "outer_recurrence: q, k and v share a dtype")
    _need(a.dtype == torch.float32 and a.dim() == 2 and a.stride(1) == 1 and a.shape[0] >= n and a.shape[1] in (heads, heads * N),
          "outer_recurrence: a is float32 [rows, heads] or [rows, heads * N]")
    per_row = a.shape[1] == heads * N and N > 1
    _need(c is None or (c.dtype == torch.float32 and c.dim() == 2 and c.stride(1) == 1 and c.shape[0] >= n and c.shape[1] == heads),
          "outer_recurrence: c")
    _need(skip is None or (skip.dtype == torch.float32 and skip.is_contiguous() and skip.numel() == heads), "outer_recurrence: skip")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1 and state.shape[1] >= heads * N * P, "outer_recurrence: state")
    _need(y.dtype == torch.float32 and y.dim() == 2 and y.stride(1) == 1 and y.shape[0] >= n and y.shape[1] == heads * P, "outer_recurrence: y")
    _need(heads % groups == 0 and N <= 1024, "outer_recurrence: heads in equal groups, at most 1,024 rows of state")
    _check(lib("outer_recurrence").kl_outer_recurrence(
        _ptr(q), ctypes.c_longlong(q.stride(0)), 0, _ptr(k), ctypes.c_longlong(k.stride(0)), 0, _ptr(v), ctypes.c_longlong(v.stride(0)), 0,
        _ptr(a), ctypes.c_longlong(a.stride(0)), int(per_row), _ptr(c), ctypes.c_longlong(c.stride(0) if c is not None else 0), _ptr(skip),
        _ptr(state), ctypes.c_longlong(state.stride(0)), _ptr(y), ctypes.c_longlong(y.stride(0)), _ptr(step.cu_tokens),
        _ptr(step.seq_slots), step.n_seqs, int(step.max_new), heads, groups, N, P, ctypes.c_float(q_scale), dtype_code(q.dtype), _stream()), "outer_recurrence")


# --------------------------------------------------------------------------- attention with mixed heads

def kv_append(src: torch.Tensor, k_col: int, v_col: int, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
              step, kv_heads: int, dim: int, vdim: int) -> None:
    """Keys (``src[:, k_col:]``, kv_heads * dim wide) and values (``src[:, v_col:]``, kv_heads * vdim wide) of the step's tokens
    into the paged cache, as they are (no rotation)."""
    _cuda(src, k_cache, v_cache, block_table)
    _i32(block_table, "block_table")
    n = step.n_tokens
    _need(src.dim() == 2 and src.stride(1) == 1 and src.shape[0] >= n and k_col + kv_heads * dim <= src.shape[1]
          and v_col + kv_heads * vdim <= src.shape[1], "kv_append: projections")
    _need(k_cache.dtype == v_cache.dtype == src.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
          and tuple(k_cache.shape[1:]) == (kv_heads, PAGE, dim) and tuple(v_cache.shape[1:]) == (kv_heads, PAGE, vdim), "kv_append: cache layout")
    _check(lib("attention_mixed").kl_kv_append(_ptr(src), ctypes.c_longlong(src.stride(0)), k_col, v_col, _ptr(k_cache), _ptr(v_cache),
                                               _ptr(block_table), block_table.shape[1], _ptr(step.positions), _ptr(step.token_slot), n,
                                               kv_heads, dim, vdim, dtype_code(src.dtype), _stream()), "kv_append")


def mixed_attention_splits(n_seqs: int, context_class: int, window: int, keep_first: int) -> int:
    """Into how many pieces a decode step cuts each sequence's visible keys for the mixed-head attention: chunks of 32
    keys dealt to the pieces in turn, about one CTA per SM over all sequences, at most one piece per chunk and 32.  Planned
    from the engine's class of the longest sequence (16 pages, then one class per doubling), so a captured step stays valid."""
    chunks = (16 << max(0, int(context_class))) * (PAGE // 32)
    if window:
        chunks = min(chunks, (int(window) + 31) // 32 + 1 + (int(keep_first or 0) + 31) // 32)
    want = -(-sm_count() // max(1, int(n_seqs)))
    return max(1, min(chunks, want, 32))


def attention_mixed(q: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    block_table: torch.Tensor, step, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, softcap: float = 0.0,
                    r1: Optional[torch.Tensor] = None, r2: Optional[torch.Tensor] = None, talk: Optional[torch.Tensor] = None,
                    window: int = 0, keep_first: int = 0, out_scale: float = 1.0, tiled: Optional[bool] = None,
                    splits: Optional[int] = None) -> None:
    """Attention of every token of ``step`` over its sequence's cache with soft-capped scores, a distance bias
    r1_h ln(1 + r2_h (i - j)) taken off, a sliding window that also keeps the first ``keep_first`` keys, the heads' softmax
    weights mixed by ``talk`` [heads, heads], and head h's result times out_scale * sigmoid(gate[t, h]) (see
    attention_mixed.cu).  ``q`` [rows, heads * dim], ``gate`` [rows, heads], ``out`` [rows, heads * vdim]: the compute dtype,
    any row stride.  The tiled kernel (attention_mixed_tiled.cu) runs where its shared memory holds the sizes, else the
    plain one; ``tiled=False`` asks for the plain one, and ``splits`` (1 to 32) sets into how many pieces a step of single
    tokens cuts each sequence's keys instead of ``mixed_attention_splits``."""
    _cuda(q, gate, out, k_cache, v_cache, block_table, r1, r2, talk)
    _i32(block_table, "block_table")
    n = step.n_tokens
    _columns(q, n, heads * dim, "attention_mixed: q"); _columns(out, n, heads * vdim, "attention_mixed: out")
    _columns(gate, n, heads, "attention_mixed: gate")
    _need(q.dtype == out.dtype == k_cache.dtype == v_cache.dtype and (gate is None or gate.dtype == q.dtype), "attention_mixed: dtypes differ")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous() and tuple(k_cache.shape[1:]) == (kv_heads, PAGE, dim)
          and tuple(v_cache.shape[1:]) == (kv_heads, PAGE, vdim), "attention_mixed: cache layout")
    for t, count in ((r1, heads), (r2, heads), (talk, heads * heads)):
        _need(t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == count), "attention_mixed: float32 per-head tensors")
    _need((r1 is None) == (r2 is None), "attention_mixed: the distance bias needs both of its numbers")
    _need(heads % kv_heads == 0, "attention_mixed: heads must be a multiple of kv heads")
    L = lib("attention_mixed_tiled")
    max_new = int(step.max_new)
    fits = L.kl_attention_mixed_tiled_fits(heads, kv_heads, dim, vdim, dtype_code(q.dtype), int(talk is not None), max_new)
    _need(not (tiled and not fits), "attention_mixed: the tiled kernel cannot hold these sizes")
    if fits and tiled is not False:
        if splits is None:
            splits = mixed_attention_splits(step.n_seqs, getattr(step, "context_class", 0), window, keep_first) if max_new == 1 else 1
        _need(1 <= splits <= 32, "attention_mixed: 1 to 32 splits")
        ml = torch.empty((n, heads, splits, 2), dtype=torch.float32, device=q.device)
        part = torch.empty((n, splits, heads * vdim), dtype=torch.float32, device=q.device) if splits > 1 else None
        _check(L.kl_attention_mixed_tiled(
            _ptr(q), ctypes.c_longlong(q.stride(0)), _ptr(gate), ctypes.c_longlong(gate.stride(0) if gate is not None else 0), _ptr(out),
            ctypes.c_longlong(out.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(step.cu_tokens),
            _ptr(step.seq_slots), _ptr(step.seq_starts), _ptr(step.token_slot), n, step.n_seqs, max_new, heads, kv_heads, dim, vdim,
            ctypes.c_float(scale), ctypes.c_float(softcap or 0.0), _ptr(r1), _ptr(r2), _ptr(talk), int(window or 0), int(keep_first or 0),
            ctypes.c_float(out_scale), splits, _ptr(ml), _ptr(part), dtype_code(q.dtype), _stream()), "attention_mixed_tiled",
            3 if splits > 1 else 2)
        return
    _check(lib("attention_mixed").kl_attention_mixed(
        _ptr(q), ctypes.c_longlong(q.stride(0)), _ptr(gate), ctypes.c_longlong(gate.stride(0) if gate is not None else 0), _ptr(out),
        ctypes.c_longlong(out.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(step.positions),
        _ptr(step.token_slot), n, heads, kv_heads, dim, vdim, ctypes.c_float(scale), ctypes.c_float(softcap or 0.0), _ptr(r1), _ptr(r2),
        _ptr(talk), int(window or 0), int(keep_first or 0), ctypes.c_float(out_scale), dtype_code(q.dtype), _stream()), "attention_mixed")


# --------------------------------------------------------------------------- matrix products

def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T in plain 32-bit FMA arithmetic; any size."""
    _cuda(a, w, out)
    (M, K), (N, K2) = a.shape, w.shape
    _need(K == K2 and out.shape[0] >= M and out.shape[1] == N, f"gemm: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    _need(a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "gemm: rows must be contiguous")
    _need(a.dtype == w.dtype, "gemm: operand dtypes differ")
    _check(lib("gemm_simt").kl_gemm_simt(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), M, N, K,
                                         dtype_code(a.dtype), dtype_code(out.dtype), _stream()), "gemm_simt")


# --------------------------------------------------------------------------- sampling

def argmax_rows(logits: torch.Tensor, out: torch.Tensor) -> None:
    _cuda(logits, out)
    _i32(out, "out")
    rows, vocab = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1 and out.numel() >= rows, "argmax: layout")
    L = lib("sampling")
    sv = si = None
    launches = 1
    if vocab >= 16384:                                              # wide rows: many CTAs per row, then one pick
        chunks = L.kl_argmax_chunks(vocab)
        sv = torch.empty((rows, chunks), dtype=torch.float32, device=logits.device)
        si = torch.empty((rows, chunks), dtype=torch.int32, device=logits.device)
        launches = 2
    _check(L.kl_argmax_rows(_ptr(logits), ctypes.c_longlong(logits.stride(0)), rows, vocab, _ptr(out), _ptr(sv), _ptr(si),
                            _stream()), "argmax_rows", launches)


def sample_rows(logits: torch.Tensor, temperature: float, top_k: int, seed: int, request_ids: torch.Tensor,
                steps: torch.Tensor, out: torch.Tensor) -> None:
    _cuda(logits, request_ids, steps, out)
    _i32(out, "out"); _i32(request_ids, "request_ids"); _i32(steps, "steps")
    rows, vocab = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "sample: layout")
    _need(request_ids.numel() >= rows and steps.numel() >= rows and out.numel() >= rows, "sample: one id and step per row")
    _need(temperature > 0, "sample: temperature must be positive (0 means argmax)")
    _check(lib("sampling").kl_sample_rows(_ptr(logits), ctypes.c_longlong(logits.stride(0)), rows, vocab,
                                          ctypes.c_float(temperature), int(top_k or 0),
                                          ctypes.c_ulonglong(seed & (2**64 - 1)), _ptr(request_ids), _ptr(steps),
                                          _ptr(out), _stream()), "sample_rows")


def token_logprob(logits: torch.Tensor, tokens: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 [rows]: log softmax(logits[row])[tokens[row]]."""
    _cuda(logits, tokens, out)
    _i32(tokens, "tokens")
    rows, vocab = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1 and tokens.numel() >= rows, "token_logprob: layout")
    if out is None:
        out = torch.empty(rows, dtype=torch.float32, device=logits.device)
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.numel() >= rows, "token_logprob: out")
    _check(lib("sampling").kl_token_logprob(_ptr(logits), ctypes.c_longlong(logits.stride(0)), rows, vocab, _ptr(tokens),
                                            _ptr(out), _stream()), "token_logprob")
    return out


# --------------------------------------------------------------------------- dispatch by dtype and shape

_device_words: Dict[int, torch.Tensor] = {}


def device_words(device: torch.device) -> torch.Tensor:
    """Two int32 words per device through which kernels report what the host must not miss:
    word 0 is the status word (kernels with bounded waits write a non-zero code into it when a
    wait runs out), word 1 the flag that the embedding kernel sets when it meets a token id
    outside the vocabulary.  ``check_device_words`` reads both with one copy."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _device_words:
        with torch.inference_mode(False):   # an ordinary tensor also when first asked for under inference mode: it is cleared in place later
            _device_words[idx] = torch.zeros(2, dtype=torch.int32, device=device)
    return _device_words[idx]


def status_word(device: torch.device) -> torch.Tensor:
    return device_words(device)[0:1]


def _status_ptr(device: torch.device) -> ctypes.c_void_p:
    """The status word's address (word 0 of ``device_words``) for a launch, without a tensor view."""
    return ctypes.c_void_p(device_words(device).data_ptr())


def error_word(device: torch.device) -> torch.Tensor:
    return device_words(device)[1:2]


class TokenIdError(ValueError):
    """A token id outside the vocabulary reached the embedding kernel."""


def check_device_words(device: torch.device) -> None:
    """Read both words (that synchronises), clear what was set, and raise for it: ``KernelError``
    for a wait that ran out (whatever the kernels wrote after it is not to be trusted),
    ``TokenIdError`` for a bad token id."""
    words = device_words(device)
    status, bad_id = words.tolist()
    if status or bad_id:
        words.zero_()
    if status:
        raise KernelError(f"a tensor-core kernel gave up waiting (code {status}: 1 = loader, 2 = MMA issuer, 3 = epilogue); "
                          "the results of this run are not valid")
    if bad_id:
        raise TokenIdError("a token id outside the vocabulary reached the embedding kernel")


def check_status(device: torch.device) -> None:
    """The status word alone (the token-id flag is left as it is)."""
    word = status_word(device)
    code = int(word.item())
    if code:
        word.zero_()
        raise KernelError(f"a tensor-core kernel gave up waiting (code {code}: 1 = loader, 2 = MMA issuer, 3 = epilogue)")


def _tc_ok(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor]) -> bool:
    """Whether the TMA-fed tensor-core kernels take these operands: bfloat16, rows that start
    on 16-byte boundaries (K and the row strides multiples of 8 elements).  ``out`` None: the
    kernel's own float32 pieces."""
    K = a.shape[1]
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and (out is None or (out.dtype in (torch.bfloat16, torch.float32) and out.stride(1) == 1))
            and K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and a.stride(1) == 1 and w.stride(1) == 1)


_sm_counts: Dict[int, int] = {}


def sm_count(device: Optional[torch.device] = None) -> int:
    """Streaming multiprocessors of ``device`` (default: the current one), asked of the driver once."""
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    if idx not in _sm_counts:
        _sm_counts[idx] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
    return _sm_counts[idx]


def skinny_splits(N: int, K: int, M: int = 1) -> int:
    """Into how many pieces the K range is cut for a product with few tokens, so that about two
    CTAs per SM stream weights: 128 output features per CTA, at least 4 k-blocks of 64 each.
    Every piece is written as float32 [M, N] and read again by the kernel that adds the pieces, so
    with many tokens and a short k range fewer pieces are better: their bytes stay under a quarter
    of the weights' (pieces * M * 4 <= K * 2 / 4)."""
    tiles = ((N + 127) // 128) * max(1, (M + 127) // 128)    # CTAs per cut: weight tiles x token tiles (of 128 beyond 64 tokens)
    k_blocks = (K + 63) // 64
    # never more CTAs than the two per SM that are resident at once: one CTA too many is a second round
    want = max(1, min((2 * sm_count()) // tiles, k_blocks // 4, 32, max(1, K // (8 * max(M, 1)))))
    per = (k_blocks + want - 1) // want
    return (k_blocks + per - 1) // per


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False) -> None:
    """out[M, N] = a @ w^T on the tensor cores, tokens as tile rows (any M; pairs of CTAs on tiles of
    256 tokens where the token count suits, single CTAs on tiles of 128 otherwise).  With ``swiglu``
    the rows of ``w`` alternate 64 gate rows and 64 up rows and out[M, N / 2] receives
    silu(gate) * up."""
    _cuda(a, w, out)
    (M, K), (N, K2) = a.shape, w.shape
    _need(K == K2 and out.shape[0] >= M and out.shape[1] == (N // 2 if swiglu else N), "gemm_tcgen05: shapes")
    _need(not swiglu or (N % 128 == 0 and out.dtype == torch.bfloat16), "gemm_tcgen05: swiglu needs N % 128 == 0 and bf16 out")
    _need(_tc_ok(a, w, out), "gemm_tcgen05: operands must be bfloat16 with 16-byte aligned rows")
    _check(lib("gemm_tcgen05").kl_gemm_tcgen05(_ptr(a), ctypes.c_longlong(a.stride(0)), _ptr(w),
                                               ctypes.c_longlong(w.stride(0)), _ptr(out), ctypes.c_longlong(out.stride(0)),
                                               M, N, K, int(out.dtype == torch.float32), int(swiglu),
                                               _status_ptr(a.device), _stream()), "gemm_tcgen05")


# arguments of kl_gemm_tcgen05_skinny that switch the residual-stream forms off
_NO_STREAM_FUSION = (ctypes.c_void_p(0), 0, ctypes.c_float(0.0), ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_void_p(0),
                     ctypes.c_void_p(0), ctypes.c_void_p(0))

STREAM_FUSION_MAX_ROWS = 64
STREAM_SINK_MAX_ROWS = 4        # measured on the 8B shape: faster than a norm kernel of its own up to 4 rows, slower from 8


def stream_fusable(rows: int, w: torch.Tensor) -> bool:
    """Whether a product of ``rows`` tokens with ``w`` can add its result into the float32 residual
    stream, or apply a norm's 1 / rms to its rows, inside the kernel (decode steps, bfloat16)."""
    return (rows <= STREAM_FUSION_MAX_ROWS and w.dtype == torch.bfloat16 and w.is_cuda and w.shape[1] % 8 == 0
            and w.stride(1) == 1 and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny_stream(w: torch.Tensor, a: torch.Tensor, row_scale=None, sink=None, swiglu: bool = False,
                       splits: Optional[int] = None):
    """A decode step's product with the residual stream folded in (see gemm_tcgen05.cu).

    ``a``: bfloat16 [M, K].  ``row_scale`` = (ss float32 [pieces, 64], eps): row m of the result is
    multiplied by rsqrt(sum_p ss[p, m] / K + eps); with a = bf16(x * norm_weight) that is the
    product of the normalised rows of x.
    Result: with ``sink`` = (stream float32 [M, N], next norm's weight float32 [N] or None) the
    product is added into the stream and (ss float32 [N / 128 tiles, 64], bf16(stream * weight)
    [M, N] or None) comes back; with ``swiglu`` a bfloat16 [M, N / 2] tensor; else float32 pieces
    [S, M, N]."""
    N, K = w.shape
    M = a.shape[0]
    _cuda(a, w)
    _need(a.dtype == torch.bfloat16 and a.shape[1] == K and a.stride(1) == 1 and a.stride(0) % 8 == 0
          and a.data_ptr() % 16 == 0, "gemm_skinny_stream: activations")
    _need(stream_fusable(M, w), "gemm_skinny_stream: shape or layout not supported")
    if row_scale is not None:
        ss, eps = row_scale
        _cuda(ss)
        _need(ss.dtype == torch.float32 and ss.is_contiguous() and ss.dim() == 2 and ss.shape[1] == 64,
              "gemm_skinny_stream: sums of squares")
        scale_args = (_ptr(ss), ss.shape[0], ctypes.c_float(eps))
    else:
        scale_args = (ctypes.c_void_p(0), 0, ctypes.c_float(0.0))
    dev = w.device
    L = lib("gemm_tcgen05")
    st = _status_ptr(dev)
    null = ctypes.c_void_p(0)
    if swiglu:
        _need(sink is None and N % 128 == 0, "gemm_skinny_stream: swiglu")
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=dev)
        _check(L.kl_gemm_tcgen05_skinny(_ptr(a), ctypes.c_longlong(a.stride(0)), _ptr(w), ctypes.c_longlong(w.stride(0)), _ptr(out),
                                        ctypes.c_longlong(out.stride(0)), M, N, K, 1, 0, 1, *scale_args, null, null, null, null,
                                        null, st, _stream()), "gemm_skinny_stream")
        return out
    splits = skinny_splits(N, K, M) if splits is None else splits
    partial = torch.empty((splits, M, N), dtype=torch.float32, device=dev)
    result = partial
    sink_args = (null, null, null, null, null)
    if sink is not None:
        stream, next_w = sink
        _cuda(stream)
        _need(stream.dtype == torch.float32 and stream.is_contiguous() and tuple(stream.shape) == (M, N), "gemm_skinny_stream: sink")
        tiles = (N + 127) // 128
        ss_out = torch.empty((tiles, 64), dtype=torch.float32, device=dev)
        scaled = None
        if next_w is not None:
            _cuda(next_w)
            _need(next_w.dtype == torch.float32 and next_w.is_contiguous() and next_w.numel() == N, "gemm_skinny_stream: norm weight")
            scaled = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        sink_args = (_ptr(stream), _ptr(ss_out), _ptr(_zero_counters(dev, tiles, "gemm")),
                     _ptr(next_w) if next_w is not None else null, _ptr(scaled) if scaled is not None else null)
        result = (ss_out, scaled)
    _check(L.kl_gemm_tcgen05_skinny(_ptr(a), ctypes.c_longlong(a.stride(0)), _ptr(w), ctypes.c_longlong(w.stride(0)), _ptr(partial),
                                    ctypes.c_longlong(N), M, N, K, splits, 1, 0, *scale_args, *sink_args, st, _stream()),
           "gemm_skinny_stream")
    return result


# Which way round a product of M tokens and N features runs.  Weights as tile rows (tiles of 128
# features x 16 to 128 tokens, the K range cut so that all SMs stream): every weight crosses from HBM
# once and 16 KB of it per CTA and k block.  Tokens as tile rows (128 x 256 or 256 x 256): both operands
# are reused, but a product of 128 tokens and 4,096 features has 16 tiles for 148 SMs (8B shape, 96
# sequences: 7.6 ms per decode step that way, 5.5 ms with weights as rows).  Measured per product on
# the 8B shape, us with tokens / weights as rows:
#   128 tokens: q/k/v (24 tiles) 29.2 / 18.2, output (16) 26.7 / 13.9, gate/up (112) 43.1 / 53.6, down (16) 82.9 / 28.9
#   384 tokens: q/k/v (72) 29.6 / 23.2, output (48) 26.8 / 21.7, gate/up (336) 85.0 / -, down (48) 82.6 / 46.1
#   512 tokens: q/k/v (96) 27.6 / 34.1, output (64) 24.2 / 21.9, down (64) 70.2 / 58.5
# and on the 1B shape at 128 tokens: gate/up (64 tiles) 18.0 / 25.9.  So beyond 64 tokens: weights as rows
# while the other way has fewer tiles than 0.6 of the SMs; the gate/up product, whose K range cannot be
# cut (its epilogue needs whole sums), while it has fewer than a third of them, and already from 33 tokens on
# (8B shape, ms per decode step with the gate/up product's weights / tokens as rows: 48 sequences 4.06 / 4.02,
# 64 sequences 4.44 / 4.36; 24 and 32 sequences, were they included: 3.42 / 3.49 and 3.52 / 3.62).
SKINNY_MAX_ROWS = 512


SWIGLU_WEIGHT_ROWS_MAX = 32     # tokens up to which the gate/up product takes the weights as tile rows


def weights_as_rows(M: int, N: int, swiglu: bool = False) -> bool:
    if M <= (SWIGLU_WEIGHT_ROWS_MAX if swiglu else 64):
        return True
    if M > SKINNY_MAX_ROWS:
        return False
    tiles = ((M + 127) // 128) * ((N + 255) // 256)
    return tiles * 3 < sm_count() if swiglu else tiles * 5 < sm_count() * 3


def gemm_skinny_partials(a: torch.Tensor, w: torch.Tensor, splits: Optional[int] = None) -> Optional[torch.Tensor]:
    """The pieces of a @ w^T for few tokens (``weights_as_rows``) as float32 [S, M, N], for a consumer that adds
    them itself (the norm after a projection, the rotary kernel after q/k/v); None when the
    product is not cut (S == 1) or the operands do not fit the tensor-core kernel."""
    (M, K), (N, K2) = a.shape, w.shape
    if not weights_as_rows(M, N) or a.dtype != torch.bfloat16 or K != K2:
        return None
    if not _tc_ok(a, w, None):
        return None
    splits = skinny_splits(N, K, M) if splits is None else splits
    if splits <= 1:
        return None
    partial = torch.empty((splits, M, N), dtype=torch.float32, device=a.device)
    _check(lib("gemm_tcgen05").kl_gemm_tcgen05_skinny(
        _ptr(a), ctypes.c_longlong(a.stride(0)), _ptr(w), ctypes.c_longlong(w.stride(0)), _ptr(partial),
        ctypes.c_longlong(N), M, N, K, splits, 1, 0, *_NO_STREAM_FUSION, _status_ptr(a.device), _stream()),
        "gemm_skinny")
    return partial


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, splits: Optional[int] = None,
                swiglu: bool = False) -> None:
    """out[M, N] = a @ w^T for M <= SKINNY_MAX_ROWS tokens: weights as tile rows, each weight read once, the
    K range cut into ``splits`` pieces whose float32 partial sums are added in a fixed order.
    With ``swiglu`` (rows of ``w`` alternate 64 gate and 64 up rows; no cut) out[M, N / 2]
    receives silu(gate) * up."""
    _cuda(a, w, out)
    (M, K), (N, K2) = a.shape, w.shape
    _need(K == K2 and out.shape[0] >= M and out.shape[1] == (N // 2 if swiglu else N) and M <= SKINNY_MAX_ROWS, "gemm_skinny: shapes")
    _need(_tc_ok(a, w, out), "gemm_skinny: operands must be bfloat16 with 16-byte aligned rows")
    _need(not swiglu or (N % 128 == 0 and out.dtype == torch.bfloat16), "gemm_skinny: swiglu needs N % 128 == 0 and bf16 out")
    splits = 1 if swiglu else (skinny_splits(N, K, M) if splits is None else splits)
    L = lib("gemm_tcgen05")
    st = _status_ptr(a.device)
    if splits == 1:
        _check(L.kl_gemm_tcgen05_skinny(_ptr(a), ctypes.c_longlong(a.stride(0)), _ptr(w), ctypes.c_longlong(w.stride(0)),
                                        _ptr(out), ctypes.c_longlong(out.stride(0)), M, N, K, 1,
                                        int(out.dtype == torch.float32), int(swiglu), *_NO_STREAM_FUSION, st, _stream()),
               "gemm_skinny")
        return
    partial = torch.empty((splits, M, N), dtype=torch.float32, device=a.device)
    _check(L.kl_gemm_tcgen05_skinny(_ptr(a), ctypes.c_longlong(a.stride(0)), _ptr(w), ctypes.c_longlong(w.stride(0)),
                                    _ptr(partial), ctypes.c_longlong(N), M, N, K, splits, 1, 0, *_NO_STREAM_FUSION, st,
                                    _stream()), "gemm_skinny")
    _check(L.kl_splitk_reduce(_ptr(partial), splits, M, N, _ptr(out), ctypes.c_longlong(out.stride(0)),
                              int(out.dtype == torch.float32), _stream()), "splitk_reduce")


def matmul(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out = a @ w^T with the kernel that fits the dtype and the shape.  float32 operands
    always take the plain 32-bit kernel; bfloat16 operands take the tensor-core kernels when
    their rows are 16-byte aligned (few tokens: weights as tile rows), else the plain kernel."""
    if a.dtype == torch.bfloat16 and _tc_ok(a, w, out):
        if weights_as_rows(a.shape[0], w.shape[0]):
            gemm_skinny(a, w, out)
        else:
            gemm_tcgen05(a, w, out)
    else:
        gemm_simt(a, w, out)


DECODE_HEAD_DIMS = (16, 32, 64, 128, 256)


def decode_splits(rows: int, num_heads: int, num_kv_heads: int) -> int:
    """Into how many pieces each sequence's keys are cut in decode attention: enough CTAs for
    about two per SM, from the batch size alone (never from the lengths, so that a captured
    graph stays valid while the sequences grow)."""
    group = num_heads // num_kv_heads
    tiles = (group + 3) // 4 if group >= 3 else 1
    ctas = max(1, rows * num_kv_heads * tiles)
    return max(1, min(32, (2 * sm_count() + ctas - 1) // ctas))


def attention_decode(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     block_table: torch.Tensor, positions: torch.Tensor, token_slot: torch.Tensor, rows: int,
                     num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: int = 0,
                     splits: Optional[int] = None) -> None:
    """One query token per row against its sequence's cache, keys cut over ``splits`` CTAs."""
    _cuda(q, out, k_cache, v_cache, block_table, positions, token_slot)
    _i32(positions, "positions"); _i32(token_slot, "token_slot"); _i32(block_table, "block_table")
    _need(q.dtype == out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16, "attention_decode: bfloat16 only")
    _need(head_dim in DECODE_HEAD_DIMS, f"attention_decode: head_dim {head_dim} not in {DECODE_HEAD_DIMS}")
    _need(out.is_contiguous() and out.shape[0] >= rows and out.shape[1] == num_heads * head_dim, "attention_decode: out shape")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous()
          and tuple(k_cache.shape[1:]) == (num_kv_heads, PAGE, head_dim), "attention_decode: cache layout")
    _need(num_heads % num_kv_heads == 0, "attention_decode: heads must be a multiple of kv heads")
    splits = decode_splits(rows, num_heads, num_kv_heads) if splits is None else splits
    po = pml = None
    if splits > 1:
        po = torch.empty((rows, num_heads, splits, head_dim), dtype=torch.float32, device=q.device)
        pml = torch.empty((rows, num_heads, splits, 2), dtype=torch.float32, device=q.device)
    _check(lib("attention_decode").kl_attention_decode(
        _ptr(q), q_stride, _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
        _ptr(positions), _ptr(token_slot), _ptr(po), _ptr(pml), rows, num_heads, num_kv_heads, head_dim,
        ctypes.c_float(scale), int(window or 0), splits, _stream()), "attention_decode", 2 if splits > 1 else 1)


MMA_HEAD_DIMS = (64, 128)


def attention_mma(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  block_table: torch.Tensor, cu_tokens: torch.Tensor, seq_slots: torch.Tensor, seq_starts: torch.Tensor,
                  seq_new: torch.Tensor, n_seqs: int, max_new: int, n_rows: int, num_heads: int, num_kv_heads: int,
                  head_dim: int, scale: float, window: int = 0, splits: int = 1, few_rows: bool = False, *,
                  sink: Optional[torch.Tensor] = None, weights: str = "softmax", head_bias: Optional[torch.Tensor] = None,
                  pooled=None) -> None:
    """Tensor-core attention of a ragged batch over the paged cache (bfloat16, head sizes 64
    and 128).  ``few_rows``: the layout for one token per sequence; ``splits``: pieces each
    sequence's pages are cut into.  Options: ``sink`` (float32 [heads], joins the softmax's denominator), ``weights``
    "sigmoid" (sigmoid(score + head_bias[h]), not normalised), ``pooled`` (block means in pages of their own, seen once the
    whole block lies before the window)."""
    extra = sink is not None or weights != "softmax" or head_bias is not None or pooled is not None
    pk = pv = pt = None
    if pooled is not None:
        pk, pv, pt = pooled.k, pooled.v, pooled.block_table
    _cuda(q, out, k_cache, v_cache, block_table, cu_tokens, seq_slots, seq_starts, seq_new, sink, head_bias, pk, pv, pt)
    for t, nm in ((block_table, "block_table"), (cu_tokens, "cu_tokens"), (seq_slots, "seq_slots"),
                  (seq_starts, "seq_starts"), (seq_new, "seq_new")):
        _i32(t, nm)
    _need(q.dtype == out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16, "attention_mma: bfloat16 only")
    _need(head_dim in MMA_HEAD_DIMS, f"attention_mma: head_dim {head_dim} not in {MMA_HEAD_DIMS}")
    _need(out.is_contiguous() and out.shape[0] >= n_rows and out.shape[1] == num_heads * head_dim, "attention_mma: out shape")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous()
          and tuple(k_cache.shape[1:]) == (num_kv_heads, PAGE, head_dim), "attention_mma: cache layout")
    _need(num_heads % num_kv_heads == 0 and num_heads // num_kv_heads <= 16, "attention_mma: group size up to 16")
    po = pml = None
    if splits > 1:
        po = torch.empty((n_rows, num_heads, splits, head_dim), dtype=torch.float32, device=q.device)
        pml = torch.empty((n_rows, num_heads, splits, 2), dtype=torch.float32, device=q.device)
    if extra:
        _i32(pt, "pooled block_table")
        _need(weights in ATTENTION_WEIGHTS and (weights == "softmax" or sink is None), "attention_mma: softmax (with a sink) or sigmoid weights")
        for b, name in ((sink, "sink"), (head_bias, "head_bias")):
            _need(b is None or (b.dtype == torch.float32 and b.is_contiguous() and b.numel() == num_heads), f"attention_mma: {name} must be float32 [heads]")
        if pooled is not None:
            _need(window and pk.dtype == pv.dtype == torch.bfloat16 and pk.is_contiguous() and pv.is_contiguous()
                  and tuple(pk.shape[1:]) == tuple(pv.shape[1:]) == (num_kv_heads, PAGE, head_dim), "attention_mma: pooled rows")
        _check(lib("attention_mma").kl_attention_mma_extra(
            _ptr(q), q_stride, _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
            _ptr(cu_tokens), _ptr(seq_slots), _ptr(seq_starts), _ptr(seq_new), _ptr(po), _ptr(pml), n_seqs, max_new, n_rows,
            num_heads, num_kv_heads, head_dim, ctypes.c_float(scale), int(window or 0), splits, int(few_rows), _ptr(sink),
            _ptr(head_bias), ATTENTION_WEIGHTS[weights], _ptr(pk), _ptr(pv), _ptr(pt), 0 if pt is None else pt.shape[1],
            0 if pooled is None else int(pooled.pool), _stream()), "attention_mma", 2 if splits > 1 else 1)
        return
    _check(lib("attention_mma").kl_attention_mma(
        _ptr(q), q_stride, _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
        _ptr(cu_tokens), _ptr(seq_slots), _ptr(seq_starts), _ptr(seq_new), _ptr(po), _ptr(pml), n_seqs, max_new, n_rows,
        num_heads, num_kv_heads, head_dim, ctypes.c_float(scale), int(window or 0), splits, int(few_rows), _stream()),
        "attention_mma", 2 if splits > 1 else 1)


def swiglu_fusable(hidden: int, inter: int, dtype: torch.dtype) -> bool:
    """Whether gate and up can be one product whose epilogue applies silu(gate) * up: bfloat16,
    rows on 16-byte boundaries, and an intermediate size that is a multiple of 64 (the weights
    are then stored as alternating blocks of 64 gate rows and 64 up rows)."""
    return dtype == torch.bfloat16 and inter % 64 == 0 and hidden % 8 == 0


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[I, K] and [I, K] -> [2 I, K]: 64 gate rows, the 64 up rows of the same features, and so on."""
    inter, k = gate.shape
    return torch.stack([gate.view(inter // 64, 64, k), up.view(inter // 64, 64, k)], dim=1).reshape(2 * inter, k).contiguous()


def matmul_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, I] = silu(a @ gate^T) * (a @ up^T) in one kernel; ``w_gate_up`` from ``interleave_gate_up``."""
    if weights_as_rows(a.shape[0], w_gate_up.shape[0], swiglu=True):
        gemm_skinny(a, w_gate_up, out, swiglu=True)
    else:
        gemm_tcgen05(a, w_gate_up, out, swiglu=True)


def attention_tcgen05(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      block_table: torch.Tensor, cu_tokens: torch.Tensor, seq_slots: torch.Tensor, seq_starts: torch.Tensor,
                      seq_new: torch.Tensor, n_seqs: int, max_new: int, n_rows: int, num_heads: int, num_kv_heads: int,
                      head_dim: int, scale: float) -> None:
    """Prefill attention with both products on tcgen05 (bfloat16, head size 64 or 128, no window)."""
    _cuda(q, out, k_cache, v_cache, block_table, cu_tokens, seq_slots, seq_starts, seq_new)
    for t, nm in ((block_table, "block_table"), (cu_tokens, "cu_tokens"), (seq_slots, "seq_slots"),
                  (seq_starts, "seq_starts"), (seq_new, "seq_new")):
        _i32(t, nm)
    _need(q.dtype == out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16, "attention_tcgen05: bfloat16 only")
    _need(head_dim in (64, 128) and q_stride % 8 == 0 and q.data_ptr() % 16 == 0, "attention_tcgen05: head_dim 64 or 128, aligned rows")
    _need(out.is_contiguous() and out.shape[0] >= n_rows and out.shape[1] == num_heads * head_dim, "attention_tcgen05: out shape")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous()
          and tuple(k_cache.shape[1:]) == (num_kv_heads, PAGE, head_dim), "attention_tcgen05: cache layout")
    _need(q.shape[0] >= n_rows, "attention_tcgen05: q rows")
    cache_rows = k_cache.shape[0] * num_kv_heads * PAGE
    _check(lib("attention_tcgen05").kl_attention_tcgen05(
        _ptr(q), q_stride, _ptr(out), _ptr(k_cache), _ptr(v_cache), ctypes.c_longlong(cache_rows), _ptr(block_table),
        block_table.shape[1], _ptr(cu_tokens), _ptr(seq_slots), _ptr(seq_starts), _ptr(seq_new), n_seqs, max_new,
        q.shape[0], num_heads, num_kv_heads, head_dim, ctypes.c_float(scale), _status_ptr(q.device), _stream()),
        "attention_tcgen05")


# Which kernel prefill steps of the bfloat16 path use for head sizes 64 and 128: "tcgen05", or "mma"
# (the kernel that serves windows and other group sizes).  Kept as a switch so that tests can run
# whole models through the second kernel too (tests/test_gpu_schedules.py).
PREFILL_KERNEL = "tcgen05"

_counters: Dict[tuple, torch.Tensor] = {}


COUNTERS = 1 << 18     # int32 counters per device and use (1 MiB): one per (sequence, kv head) or per tile


def _zero_counters(device: torch.device, n: int, use: str = "attention") -> torch.Tensor:
    """int32 counters that kernels leave at zero (the last CTA of a group resets its own); one
    buffer per device and per use, so that kernels of different kinds never share a counter.
    The buffer is made once and never replaced: captured graphs and kernels in flight hold its
    address."""
    idx = (device.index if device.index is not None else torch.cuda.current_device(), use)
    have = _counters.get(idx)
    if have is None:
        have = _counters[idx] = torch.zeros(COUNTERS, dtype=torch.int32, device=device)
    _need(n <= COUNTERS, f"{use}: {n} counters wanted, {COUNTERS} exist")
    return have


def decode_attention_splits(n_seqs: int, num_kv_heads: int, head_dim: int = 128, context_class: int = 0) -> int:
    """Pieces a sequence's keys are cut into for the tensor-core decode kernel.

    Up to 1,024 tokens (``context_class`` 0; the engine's class of the longest sequence: 16 pages,
    then one class per doubling): as many as keep all CTAs in one round (three CTAs fit an SM, four
    with a head size of 64), at most 16.  A CTA's time is its chain of pages, so a second round
    costs more than longer chains (32 sequences of 8 kv heads, 512 tokens: 27 us with one piece,
    35 us with two).  For longer sequences, measured on the 8B shape inside the decode step:

    * where one round has room for two pieces or more per (sequence, kv head) pair: still one
      round, but up to a piece per four pages (1 sequence of 32,768 tokens: 55 pieces 166 us per
      layer, 16 pieces 200 us; 2 sequences: 27 pieces 169 us, 16 pieces 197 us);
    * where it has not, but two pieces per pair fit the light CTAs' round of four per SM: two
      pieces beyond 4,096 tokens (32 sequences of 8,300 tokens: 307 against 334 us per layer; of
      2,100 tokens: 192 against 191 us; more pieces in more rounds were never faster)."""
    pairs = max(1, n_seqs * num_kv_heads)
    places = (4 if head_dim == 64 else 3) * sm_count()
    one_round = max(1, places // pairs)
    if context_class <= 0:
        return min(16, one_round)
    pages = 16 << context_class                          # the class's longest sequence
    if one_round >= 2:
        return max(1, min(one_round, max(16, pages // 4)))
    if context_class >= 3 and head_dim == 128 and pairs * 2 <= 4 * sm_count():
        return 2
    return 1


def decode_fusable(dtype: torch.dtype, head_dim: int, rotary_dim: int, num_heads: int, num_kv_heads: int) -> bool:
    """Whether a decode step's rotation, cache write, attention and split merge run as one kernel."""
    return (dtype == torch.bfloat16 and head_dim in MMA_HEAD_DIMS and rotary_dim == head_dim
            and num_heads % num_kv_heads == 0 and num_heads // num_kv_heads <= 16)


def attention_decode_fused(qkv: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor,
                           v_cache: torch.Tensor, block_table: torch.Tensor, step, num_heads: int, num_kv_heads: int,
                           head_dim: int, scale: float, window: int = 0, splits: Optional[int] = None) -> None:
    """One token per sequence (a decode step, rows in sequence order, no padding rows).  ``qkv``
    is the q/k/v projection, bfloat16 [rows, (H + 2 KV) * hd] or float32 pieces [S, rows, width].
    Rotates q and k, appends k and v to the cache, attends, merges the splits: one kernel."""
    _cuda(qkv, inv_freq, out, k_cache, v_cache, block_table)
    n = step.n_seqs
    _need(step.is_decode and step.n_tokens == n, "attention_decode_fused: one token per sequence and no padding rows")
    _need(decode_fusable(out.dtype, head_dim, 2 * inv_freq.numel(), num_heads, num_kv_heads), "attention_decode_fused: not fusable")
    width = (num_heads + 2 * num_kv_heads) * head_dim
    parts, plain, n_parts, stride = None, None, 0, 0
    if qkv.dim() == 3:
        _need(qkv.dtype == torch.float32 and qkv.is_contiguous() and tuple(qkv.shape[1:]) == (n, width), "attention_decode_fused: pieces")
        parts, n_parts, stride = qkv, qkv.shape[0], n * width
    else:
        _need(qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and tuple(qkv.shape) == (n, width), "attention_decode_fused: qkv")
        plain = qkv
    _need(out.is_contiguous() and out.shape[0] >= n and out.shape[1] == num_heads * head_dim, "attention_decode_fused: out shape")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.dtype == torch.bfloat16
          and tuple(k_cache.shape[1:]) == (num_kv_heads, PAGE, head_dim), "attention_decode_fused: cache layout")
    _need(inv_freq.dtype == torch.float32 and inv_freq.numel() == head_dim // 2, "attention_decode_fused: inv_freq")
    _need(all(t.data_ptr() % 16 == 0 for t in (qkv, inv_freq, out, k_cache, v_cache)), "attention_decode_fused: 16-byte aligned operands")
    if splits is None:
        splits = decode_attention_splits(n, num_kv_heads, head_dim, getattr(step, "context_class", 0))
    po = pml = None
    if splits > 1:
        po = torch.empty((n, num_heads, splits, head_dim), dtype=torch.float32, device=out.device)
        pml = torch.empty((n, num_heads, splits, 2), dtype=torch.float32, device=out.device)
    counters = _zero_counters(out.device, n * num_kv_heads)
    _check(lib("attention_mma").kl_attention_decode_fused(
        _ptr(plain), _ptr(parts), n_parts, ctypes.c_longlong(stride), _ptr(inv_freq), _ptr(out), _ptr(k_cache), _ptr(v_cache),
        _ptr(block_table), block_table.shape[1], _ptr(step.cu_tokens), _ptr(step.seq_slots), _ptr(step.seq_starts),
        _ptr(step.seq_new), _ptr(po), _ptr(pml), _ptr(counters), n, num_heads, num_kv_heads, head_dim, ctypes.c_float(scale),
        int(window or 0), splits, _stream()), "attention_decode_fused")


# Which kernel decode steps of the bfloat16 path use when both fit: "mma" (tensor cores) or
# "simt" (attention_decode.cu, which otherwise serves head sizes 16, 32 and 256); a switch for tests.
DECODE_KERNEL = "mma"


def attention(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
              block_table: torch.Tensor, step, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
              window: int = 0) -> None:
    """Attention of every token of ``step`` over its sequence's cache.  The bfloat16 path
    takes the tensor-core kernel (head sizes 64 and 128) or, for decode steps with other head
    sizes, the split-KV kernel; float32 and everything else takes the plain kernel."""
    bf = q.dtype == torch.bfloat16
    group = num_heads // num_kv_heads
    if (bf and not step.is_decode and PREFILL_KERNEL == "tcgen05" and head_dim in (64, 128) and not window and group <= 128
            and q_stride % 8 == 0 and q.data_ptr() % 16 == 0 and step.max_new >= 8):
        attention_tcgen05(q, q_stride, out, k_cache, v_cache, block_table, step.cu_tokens, step.seq_slots, step.seq_starts,
                          step.seq_new, step.n_seqs, step.max_new, step.n_tokens, num_heads, num_kv_heads, head_dim, scale)
    elif (bf and head_dim in MMA_HEAD_DIMS and group <= 16 and (not step.is_decode or DECODE_KERNEL == "mma")
          and q_stride % 2 == 0 and q.data_ptr() % 4 == 0):
        splits = 1
        if step.is_decode:
            splits = decode_attention_splits(step.n_seqs, num_kv_heads, head_dim, getattr(step, "context_class", 0))
        attention_mma(q, q_stride, out, k_cache, v_cache, block_table, step.cu_tokens, step.seq_slots, step.seq_starts,
                      step.seq_new, step.n_seqs, step.max_new, step.n_tokens, num_heads, num_kv_heads, head_dim, scale,
                      window, splits, few_rows=step.is_decode)
    elif bf and step.is_decode and head_dim in DECODE_HEAD_DIMS and q_stride % 8 == 0 and q.data_ptr() % 16 == 0:
        attention_decode(q, q_stride, out, k_cache, v_cache, block_table, step.positions, step.token_slot, step.n_tokens,
                         num_heads, num_kv_heads, head_dim, scale, window)
    else:
        attention_simt(q, q_stride, out, k_cache, v_cache, block_table, step.positions, step.token_slot, step.n_tokens,
                       num_heads, num_kv_heads, head_dim, scale, window)
