"""Small Dofevik configurations and random weights for the tests, written as model folders (config.json,
model.safetensors in bfloat16).  The sizes differ from layer to layer and avoid equalities that would hide a
mix-up (key size = value size, heads = kv heads, a window that is a multiple of the block, top = 1, a full rotation)."""
from __future__ import annotations

import functools
import json
import os
from typing import Dict, Optional, Sequence

import torch

import plain_dofevik as P
from terolix_helpers import tokens, write_folder  # noqa: F401  (shared by the tests)


def _att(heads, kv_heads, dim, vdim, scale, size, base, dims, factor=None):
    rot = {"base": base, "dims": dims}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                           "mask": {"size": size}, "rot": rot}}


def _att2(heads, kv_heads, dim, scale, size, pool):
    return {"type": "attention_2", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale,
                                             "mask": {"size": size, "pool": pool}}}


def _lat(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, size, base):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                                                  "q_rank": q_rank, "scale": scale, "mask": {"size": size},
                                                  "rot": {"base": base, "dims": rot_dim}}}


def _moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def _model(vocab, width, layers, eps=1e-5):
    return {"architecture": "Dofevik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


CONFIGS: Dict[str, dict] = {
    # every mixer twice with other sizes, in another order than the usual one; a layer without feed-forward; a window shorter
    # than a block of pooled positions; a window longer than the prompts; experts with and without a shared one; top 1
    "mixed": _model(97, 64, [
        dict(_att2(4, 2, 12, 0.4, 37, 5), mlp=_moe(6, 3, 24, 40)),
        dict(_lat(3, 8, 4, 12, 20, 24, 0.3, 50, 5000.0), mlp=_moe(5, 1, 16)),
        dict(_att(6, 3, 16, 20, 0.25, 70, 10000.0, 8, 3.0), mlp=None),
        dict(_lat(2, 16, 8, 8, 12, 16, 0.2, 33, 300.0), mlp=_moe(4, 2, 32, 8)),
        dict(_att2(3, 1, 16, 0.3, 8, 20), mlp=_moe(7, 4, 8)),
        dict(_att(2, 2, 8, 8, 0.5, 200, 50.0, 8), mlp=_moe(3, 3, 24, 24))]),
    # sizes that are multiples of nothing: rows on no 16-byte boundary, blocks of 3 and 7, windows of 1 and 2
    "odd": _model(131, 100, [
        dict(_att(5, 5, 10, 6, 0.35, 31, 777.0, 6, 1.7), mlp=_moe(7, 4, 18, 13)),
        dict(_att2(6, 3, 18, 0.2, 2, 3), mlp=_moe(5, 2, 9)),
        dict(_lat(5, 6, 2, 10, 9, 11, 0.4, 65, 10000.0), mlp=None),
        dict(_att2(2, 2, 6, 0.5, 1, 7), mlp=_moe(2, 1, 50, 3))], eps=3e-6),
    # sizes on which the bfloat16 tensor-core kernels run (16-byte rows everywhere, head sizes of 64 and 128)
    "wide": _model(320, 256, [
        dict(_lat(8, 32, 32, 64, 128, 96, 0.1, 130, 20000.0), mlp=_moe(12, 4, 64, 128)),
        dict(_att(8, 2, 64, 64, 0.125, 96, 1000000.0, 32, 8.0), mlp=_moe(8, 2, 128, 64)),
        dict(_att2(8, 4, 64, 0.11, 72, 16), mlp=_moe(16, 2, 64)),
        dict(_att(4, 1, 128, 128, 0.09, 150, 10000.0, 128), mlp=_moe(4, 1, 256, 256))], eps=1e-6),
}
# one mechanism alone (a layer needs a mixer: the experts ride on a tiny attention)
CONFIGS["only_attention"] = _model(61, 64, [dict(CONFIGS["mixed"]["layers"][2], mlp=None)])
CONFIGS["only_attention_2"] = _model(61, 64, [dict(CONFIGS["mixed"]["layers"][0], mlp=None)])
CONFIGS["only_latent"] = _model(61, 64, [dict(CONFIGS["mixed"]["layers"][1], mlp=None)])
CONFIGS["only_moe"] = _model(61, 64, [dict(_att(1, 1, 4, 4, 0.5, 3, 100.0, 2), mlp=_moe(9, 2, 24, 16))])
# windows that decoding passes over, in every mixer; blocks of 24 and of 64 positions (a page's worth)
CONFIGS["window"] = _model(53, 48, [
    dict(_att2(3, 3, 12, 0.4, 100, 24), mlp=None),
    dict(_att(4, 2, 12, 8, 0.3, 150, 10000.0, 4), mlp=None),
    dict(_lat(2, 8, 4, 8, 12, 8, 0.3, 64, 1000.0), mlp=_moe(4, 2, 16, 8)),
    dict(_att2(2, 1, 8, 0.5, 65, 64), mlp=None)])


def tensor_shapes(c: dict) -> Dict[str, tuple]:
    W = c["width"]
    s = {"embed": (c["vocab"], W), "final.norm": (), "head": (c["vocab"], W)}
    for i, layer in enumerate(c["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        s[p + "norm1"] = ()
        if layer["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            s.update({p + "mix.q": (H * d, W), p + "mix.q.b": (H * d,), p + "mix.k": (G * d, W), p + "mix.k.b": (G * d,),
                      p + "mix.v": (G * dv, W), p + "mix.v.b": (G * dv,), p + "mix.sink": (H,), p + "mix.o": (W, H * dv)})
        elif layer["type"] == "attention_2":
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            s.update({p + "mix.q": (H * d, W), p + "mix.k": (G * d, W), p + "mix.q.norm": (d,), p + "mix.k.norm": (d,),
                      p + "mix.pb": (H,), p + "mix.o": (W, H * d)})
        else:
            H, d, rd, dv, r, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            s.update({p + "mix.dq": (qr, W), p + "mix.dq.norm": (qr,), p + "mix.uq": (H * (d + rd), qr), p + "mix.dkv": (r + rd, W),
                      p + "mix.dkv.norm": (r,), p + "mix.uk": (H * d, r), p + "mix.uv": (H * dv, r), p + "mix.g": (H * dv, W),
                      p + "mix.o": (W, H * dv)})
        mlp = layer["mlp"]
        if mlp is None:
            continue
        s[p + "norm2"] = ()
        f, E = mlp["expert"]["ff"], mlp["router"]["experts"]
        s[p + "mlp.router"], s[p + "mlp.router.b"] = (E, W), (E,)
        for e in range(E):
            s.update({f"{p}mlp.e{e}.up": (f, W), f"{p}mlp.e{e}.down": (W, f)})
        if mlp.get("shared") is not None:
            s.update({p + "mlp.shared.up": (mlp["shared"]["ff"], W), p + "mlp.shared.down": (W, mlp["shared"]["ff"])})
    return s


def random_weights(c: dict, seed: int, gain: float = 1.0) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors.  Matrices N(0, gain / sqrt(fan-in)); norm weights around 1 (the layers' norms are single numbers);
    biases and sinks of order 1/2; the sigmoid's per-head numbers around -1; routers wide enough that the choices differ from
    token to token."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(c).items():
        r = torch.randn(shape, generator=g)
        if name == "embed":
            t = r
        elif name.endswith(("norm1", "norm2", "final.norm", ".norm")):
            t = 1.0 + 0.2 * r
        elif name.endswith(".pb"):
            t = -1.0 + 0.7 * r
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


CLOSE_CALL = 0.1      # a router's choice counts as close where the cut lies within a tenth of the logits' spread


@functools.lru_cache(maxsize=128)
def _oracle(folder: str, toks: tuple):
    c, W = read_folder(folder)
    margins = []
    logits = P.forward(c, W, list(toks), margins)[0].float()
    logits.close_from = len(toks)                    # the first row at which some router's choice is a close call
    if margins:
        close = (torch.stack(margins).min(dim=0).values < CLOSE_CALL).nonzero()
        if close.numel():
            logits.close_from = int(close[0])
    return logits


def oracle_logits(folder: str, toks: Sequence[int]) -> torch.Tensor:
    """float32 logits [T, vocab] of the whole sequence from the plain implementation (computed in float64).  Its attribute
    ``close_from`` is the first row at which a router's choice is a close call (the number of rows if there is none)."""
    return _oracle(folder, tuple(int(t) for t in toks))


OBSERVED: Dict[tuple, float] = {}      # (dtype, what) -> the largest row error seen, for the report at the end of a run


def row_errors(got: torch.Tensor, ref: torch.Tensor) -> torch.Tensor:
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    d = got - ref
    d = d - d.mean(dim=-1, keepdim=True)
    return d.pow(2).mean(dim=-1).sqrt() / (ref - ref.mean(dim=-1, keepdim=True)).pow(2).mean(dim=-1).sqrt().clamp_min(1e-9)


def assert_logits(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str, rows: Optional[Sequence[int]] = None) -> None:
    """Per row, the difference with its mean taken off, root mean square over the vocabulary, relative to the reference row's
    spread.  float32 (the sharp test: only the order of sums differs): 1e-4 for every row.  bfloat16 is judged by shares (half
    of the rows within 5 %, nine in ten within 30 %), because a router whose logits around the cut are close picks another
    expert than float64 does, which moves that row by much of its spread, under every cut and batch alike; where the shares fail
    and ``ref`` comes from ``oracle_logits`` of a whole sequence, the rows before the plain implementation's first close call
    are judged instead (each within a tenth).  ``rows``: rows
    that must hold the float32 limit, or a tenth of their spread in bfloat16, each (the rows a test is about)."""
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    err = row_errors(got, ref)
    worst = int(err.argmax())
    key = (dtype, what.split(":")[0])
    OBSERVED[key] = max(OBSERVED.get(key, 0.0), float(err.max()))
    if rows is not None:
        limit = 1e-4 if dtype == "float32" else 1e-1
        for r in rows:
            assert float(err[r]) <= limit, f"{what}: row {r} is off by {float(err[r]):.3e} of its spread (limit {limit:.0e})"
    if dtype == "float32":
        assert float(err.max()) <= 1e-4, f"{what}: row {worst} is off by {float(err.max()):.3e} of its spread (limit 1e-04)"
        return
    half, most = float(err.quantile(0.5)), float(err.quantile(0.9))
    sure = getattr(ref, "close_from", None)
    if (half > 5e-2 or most > 3e-1) and sure is not None and sure < err.numel() and (sure == 0 or float(err[:sure].max()) <= 1e-1):
        # A router with a close call picked another expert than float64 does and moved that row and, through the cache, the
        # rows after it; the rows before the first close call all lie within a tenth of their spread.
        return
    assert half <= 5e-2, f"{what}: half of the rows are off by more than {half:.3e} of their spread (limit 5e-02)"
    if err.numel() >= 20:
        assert most <= 3e-1, f"{what}: a tenth of the rows is off by more than {most:.3e} of their spread (limit 3e-01)"
