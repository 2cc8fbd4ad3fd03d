"""Small Bededra configurations and random weights for the tests, written as model folders (config.json,
model.safetensors in bfloat16).  The sizes differ from layer to layer and avoid equalities that would hide a
mix-up (key size = value size, one group, one part of the norm, as many heads left as right, top = 1, scales of 1)."""
from __future__ import annotations

import functools
import json
import os
from typing import Dict, Optional, Sequence

import torch

import plain_bededra as P
from terolix_helpers import tokens, write_folder  # noqa: F401  (shared by the tests)


def _ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}}


def _par(left, right, left_scale, right_scale):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def _left(heads, kv_heads, dim, vdim, scale, softcap, size=None, keep_first=0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap}
    if size is not None:
        m["mask"] = {"size": size, "keep_first": keep_first}
    return m


def _right(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, count=None, keep=None):
    r = {"experts": experts, "top": top}
    if count is not None:
        r["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "router": r, "expert": {"ff": ff}}


def _model(vocab, width, taps, layers, eps=1e-5):
    return {"architecture": "Bededra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps}, "layers": layers}


CONFIGS: Dict[str, dict] = {
    # every mechanism in another order than the usual one, a layer without feed-forward, two groups of B and C, a norm in three
    # parts, windows of 40 and 70 with 5 and 0 kept tokens, one layer without a window, 2 of 3 groups of experts kept
    "mixed": _model(97, 64, 4, [
        dict(_par(_left(4, 2, 12, 20, 0.4, 15.0, 40, 5), _right(3, 8, 16, 6.0, 5), 0.8, 1.3), mlp=_moe(6, 3, 24, 3, 2)),
        dict(_ssm(6, 8, 12, 2, 3, 3), mlp=_dense(80)),
        dict(_par(_left(6, 6, 8, 8, 0.5, 30.0, 70, 0), _right(2, 16, 8, 3.0, 7), 1.1, 0.6), mlp=None),
        dict(_ssm(3, 16, 20, 3, 1, 1), mlp=_moe(5, 1, 40)),
        dict(_par(_left(3, 1, 16, 12, 0.3, None), _right(4, 12, 12, 9.0, 3), -0.7, 0.9), mlp=_dense(40))]),
    # sizes that are multiples of nothing: rows on no 16-byte boundary, five taps, seven experts in one group, one tap in front
    "odd": _model(131, 100, 1, [
        dict(_ssm(5, 6, 9, 1, 5, 5), mlp=_moe(7, 4, 18)),
        dict(_par(_left(6, 3, 10, 14, 0.35, 9.0, 33, 3), _right(5, 6, 10, 2.5, 4), 1.0, 1.0), mlp=_dense(52)),
        dict(_ssm(10, 3, 33, 5, 2, 2), mlp=None)], eps=3e-6),
    # sizes on which the bfloat16 tensor-core products run (16-byte rows everywhere), more heads, longer states
    "wide": _model(320, 256, 3, [
        dict(_ssm(8, 64, 64, 2, 4, 2), mlp=_moe(16, 2, 128, 4, 2)),
        dict(_par(_left(8, 2, 64, 32, 0.125, 50.0, 96, 16), _right(4, 64, 48, 16.0, 16), 1.2, 1.1), mlp=_dense(512)),
        dict(_par(_left(16, 4, 32, 48, 0.18, 20.0, 130, 64), _right(8, 32, 32, 8.0, 8), 0.9, 1.4), mlp=_moe(8, 4, 64, 2, 1))], eps=1e-6),
}
# one mechanism alone (a layer needs a mixer: the feed-forwards ride on a tiny state-space one)
CONFIGS["only_ssm"] = _model(61, 64, 2, [dict(CONFIGS["mixed"]["layers"][1], mlp=None)])
CONFIGS["only_parallel"] = _model(61, 64, 3, [dict(CONFIGS["mixed"]["layers"][0], mlp=None)])
CONFIGS["only_moe"] = _model(61, 64, 2, [dict(_ssm(1, 8, 4, 1, 2, 1), mlp=_moe(9, 2, 24, 3, 1))])
CONFIGS["only_dense"] = _model(61, 64, 2, [dict(_ssm(1, 8, 4, 1, 2, 1), mlp=_dense(136))])
# a window of three pages' width that decoding passes over, tokens kept up to the middle of the first page
CONFIGS["window"] = _model(53, 48, 2, [
    dict(_par(_left(3, 3, 12, 8, 0.6, 25.0, 150, 20), _right(1, 8, 8, 4.0, 2), 1.5, 0.4), mlp=None),
    dict(_par(_left(2, 1, 16, 20, 0.5, 40.0, 64, 64), _right(2, 4, 4, 4.0, 2), 1.0, 0.5), mlp=_dense(32))])


def tensor_shapes(c: dict) -> Dict[str, tuple]:
    W = c["width"]
    s = {"embed": (c["vocab"], W), "final.norm": (W,), "head": (c["vocab"], W)}
    for i, layer in enumerate(c["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        s[p + "norm1"] = (W,)
        s[p + "canon1"] = (W, c["canon"]["taps"])
        if layer["type"] == "mamba2":
            H, P_, N, G, K = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, C = H * P_, H * P_ + 2 * G * N
            s.update({p + "mix.in": (inner + C + H, W), p + "mix.conv": (C, K), p + "mix.conv.b": (C,), p + "mix.dt_bias": (H,),
                      p + "mix.A_log": (H,), p + "mix.D": (H,), p + "mix.norm": (inner,), p + "mix.o": (W, inner)})
        else:
            l, r = m["left"], m["right"]
            H, G, d, dv = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            s.update({p + "mix.left.q": (H * d, W), p + "mix.left.k": (G * d, W), p + "mix.left.v": (G * dv, W), p + "mix.left.r1": (H,),
                      p + "mix.left.r2": (H,), p + "mix.left.talk": (H, H), p + "mix.left.g": (H, W), p + "mix.left.o": (W, H * dv)})
            H, d, dv, rank = r["heads"], r["dim"], r["vdim"], r["rank"]
            s.update({p + "mix.right.q": (H * d, W), p + "mix.right.k": (H * d, W), p + "mix.right.v": (H * dv, W), p + "mix.right.g": (H * dv, W),
                      p + "mix.right.o": (W, H * dv), p + "mix.right.norm": (dv,), p + "mix.right.a1": (rank, W),
                      p + "mix.right.a2": (H * d, rank), p + "mix.right.a2.b": (H * d,)})
        mlp = layer["mlp"]
        if mlp is None:
            continue
        s[p + "norm2"] = (W,)
        if mlp["kind"] == "dense":
            s.update({p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
        else:
            f = mlp["expert"]["ff"]
            s[p + "mlp.router"] = (mlp["router"]["experts"], W)
            for e in range(mlp["router"]["experts"]):
                s.update({f"{p}mlp.e{e}.gate": (f, W), f"{p}mlp.e{e}.up": (f, W), f"{p}mlp.e{e}.down": (W, f)})
    return s


def random_weights(c: dict, seed: int, gain: float = 1.0) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors.  Matrices N(0, gain / sqrt(fan-in)); norm weights around 1; taps, biases and skips of order 1/2; positive
    distance-bias numbers; a head-mixing matrix near the identity with sizeable off-diagonal entries; decay biases that leave
    the linear attention's memory long; routers wide enough that the choices differ from token to token."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(c).items():
        r = torch.randn(shape, generator=g)
        if name == "embed":
            t = r
        elif name.endswith(("norm1", "norm2", "final.norm", "mix.norm", "right.norm")):
            t = 1.0 + 0.2 * r
        elif name.endswith((".conv", "canon1")):
            t = 0.5 * r
        elif name.endswith(".r1"):
            t = 0.3 + 0.3 * r.abs()
        elif name.endswith(".r2"):
            t = 0.05 + 0.5 * r.abs()
        elif name.endswith(".talk"):
            t = torch.eye(shape[0]) + 0.35 * r
        elif name.endswith(".A_log"):
            t = -0.5 + 0.7 * r
        elif name.endswith(".D"):
            t = 1.0 + 0.3 * r
        elif name.endswith("a2.b"):
            t = 2.0 + r
        elif name.endswith(".router"):
            t = 4.0 * r / shape[1] ** 0.5
        elif len(shape) == 2:
            t = r * gain / shape[1] ** 0.5
        else:
            t = 0.5 * r
        out[name] = t.to(torch.bfloat16)
    return out


def read_folder(folder: str):
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        c = json.load(f)
    return c, {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


@functools.lru_cache(maxsize=128)
def _oracle(folder: str, toks: tuple) -> torch.Tensor:
    c, W = read_folder(folder)
    return P.forward(W, c, list(toks)).float()


def oracle_logits(folder: str, toks: Sequence[int]) -> torch.Tensor:
    """float32 logits [T, vocab] of the whole sequence from the plain implementation (computed in float64)."""
    return _oracle(folder, tuple(int(t) for t in toks))


OBSERVED: Dict[tuple, float] = {}      # (dtype, what) -> the largest row error seen, for the report at the end of a run


def row_errors(got: torch.Tensor, ref: torch.Tensor) -> torch.Tensor:
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    d = got - ref
    d = d - d.mean(dim=-1, keepdim=True)
    return d.pow(2).mean(dim=-1).sqrt() / (ref - ref.mean(dim=-1, keepdim=True)).pow(2).mean(dim=-1).sqrt().clamp_min(1e-9)


def assert_logits(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str) -> None:
    """Per row, the difference with its mean taken off, root mean square over the vocabulary, relative to the reference row's
    spread.  float32 (the sharp test: only the order of sums differs): 1e-4 for every row.  bfloat16 is judged by shares (half
    of the rows within 5 %, nine in ten within 30 %), because a router whose scores around the cut are close picks another
    expert than float64 does, which moves that row by much of its spread, under every cut and batch alike."""
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    err = row_errors(got, ref)
    worst = int(err.argmax())
    key = (dtype, what.split(":")[0])
    OBSERVED[key] = max(OBSERVED.get(key, 0.0), float(err.max()))
    if dtype == "float32":
        assert float(err.max()) <= 1e-4, f"{what}: row {worst} is off by {float(err.max()):.3e} of its spread (limit 1e-04)"
        return
    half, most = float(err.quantile(0.5)), float(err.quantile(0.9))
    assert half <= 5e-2, f"{what}: half of the rows are off by more than {half:.3e} of their spread (limit 5e-02)"
    if err.numel() >= 20:
        assert most <= 3e-1, f"{what}: a tenth of the rows is off by more than {most:.3e} of their spread (limit 3e-01)"
