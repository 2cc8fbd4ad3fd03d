"""A plain, slow implementation of the Dofevik decoder in float64 on the CPU: whole sequences, no cache,
one function per mechanism, written from the design's equations.  It shares no code with the package.

A model is an embedding table, a list of pre-norm layers, a final norm and a classifier:

    x = embed[token];   x += mixer(N1(x));   x += ff(N2(x));   logits = head N(x)
    N(y) = y / sqrt(mean(y^2) + eps) * g          (g: ONE number per norm)

Mixers (positions count from 0; "window W": query i sees key j when 0 <= i - j < W):

* ``attention``: biased q, k, v projections, H query heads on G key/value heads; the first ``dims`` elements of
  every q and k head turn in interleaved pairs (2i, 2i + 1) by the angle p * base^(-2i / dims) / factor; then
  each head of q and k is divided by its root mean square; softmax over the window whose denominator also
  holds exp(sink_h).
* ``attention_2``: q, k without biases, the values are the keys as projected; q and k heads RMS-normed with a
  weight of their own; no rotation; the window, and before it one pooled key and value (means over P
  neighbours, of the normed keys and of the values) for every block of P positions that has wholly left
  the window; the weight of whatever is seen is sigmoid(score + b_h), not normalised.
* ``latent_attention``: queries through a normed latent; one normed latent c and one rotated key part
  (pairs (i, i + dims / 2)) per token; per head key [W_uk c | rotated part], value W_uv c; softmax over the
  window; the heads side by side times sigmoid(W_g h); W_o.

Feed-forward: a router with bias picks the ``top`` largest logits, weights = softmax over the picked logits;
expert = W_down relu(W_up h)^2; a shared expert of the same form is added for every token.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F = torch.float64


def scalar_rms_norm(x: torch.Tensor, g, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * g


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def angles(n: int, rot: dict) -> torch.Tensor:
    """[n, dims / 2]: position times frequency."""
    dims = rot["dims"]
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    f = torch.tensor([float(rot["base"]) ** (-2.0 * i / dims) / factor for i in range(dims // 2)], dtype=F)
    return torch.arange(n, dtype=F)[:, None] * f[None, :]


def rotate(x: torch.Tensor, rot: dict, layout: str) -> torch.Tensor:
    """x [n, heads, d]: the first rot['dims'] elements of every head turn, the rest pass."""
    n, dims = x.shape[0], rot["dims"]
    a = angles(n, rot)
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    out = x.clone()
    if layout == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2] = u * c - v * s
        out[..., dims // 2:dims] = v * c + u * s
    return out


def window_mask(n: int, size: int) -> torch.Tensor:
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return (i - j >= 0) & (i - j < size)


def softmax_with_sink(scores: torch.Tensor, mask: torch.Tensor, sink: Optional[torch.Tensor]) -> torch.Tensor:
    """scores [H, n, n]; sink [H] or None.  Rows of weights over the keys (they sum to less than 1 with a sink)."""
    s = scores.masked_fill(~mask[None], -math.inf)
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink[:, None, None] - m)
    return e / den


def attention_sink(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], eps: float) -> torch.Tensor:
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T + w["q.b"]).view(n, H, d)
    k = (h @ w["k"].T + w["k.b"]).view(n, G, d)
    v = (h @ w["v"].T + w["v.b"]).view(n, G, dv)
    q, k = rotate(q, m["rot"], "interleaved"), rotate(k, m["rot"], "interleaved")
    q, k = rms_norm(q, None, eps), rms_norm(k, None, eps)
    rep = H // G
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    p = softmax_with_sink(scores, window_mask(n, m["mask"]["size"]), w["sink"])
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(n, H * dv)
    return o @ w["o"].T


def pooled_blocks(x: torch.Tensor, P: int) -> torch.Tensor:
    """x [n, G, d] -> [n // P, G, d]: the mean over every complete block of P positions."""
    nb = x.shape[0] // P
    return x[:nb * P].view(nb, P, *x.shape[1:]).mean(1)


def attention_pooled_sigmoid(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], eps: float) -> torch.Tensor:
    n = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    W, P = m["mask"]["size"], m["mask"]["pool"]
    q = (h @ w["q"].T).view(n, H, d)
    k = (h @ w["k"].T).view(n, G, d)
    v = k                                              # the keys as projected
    q, k = rms_norm(q, w["q.norm"], eps), rms_norm(k, w["k.norm"], eps)
    rep = H // G
    kb, vb = pooled_blocks(k, P), pooled_blocks(v, P)                       # the means of the normed keys, and of the values
    k, v, kb, vb = (t.repeat_interleave(rep, dim=1) for t in (k, v, kb, vb))
    bias = w["pb"][:, None, None]
    seen = window_mask(n, W)
    weight = torch.sigmoid(torch.einsum("ihd,jhd->hij", q, k) * m["scale"] + bias) * seen[None]
    out = torch.einsum("hij,jhd->ihd", weight, v)
    if kb.shape[0]:
        last = torch.arange(kb.shape[0])[None, :] * P + P - 1               # a block's last position
        whole = last <= torch.arange(n)[:, None] - W                        # the block lies wholly before the window
        weight = torch.sigmoid(torch.einsum("ihd,bhd->hib", q, kb) * m["scale"] + bias) * whole[None]
        out = out + torch.einsum("hib,bhd->ihd", weight, vb)
    return out.reshape(n, H * d) @ w["o"].T


def latent_attention(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], eps: float) -> torch.Tensor:
    n = h.shape[0]
    H, d, rd, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).view(n, H, d + rd)
    qn, qr = q[..., :d], rotate(q[..., d:], m["rot"], "half")
    ckv = h @ w["dkv"].T
    c = rms_norm(ckv[:, :r], w["dkv.norm"], eps)
    kr = rotate(ckv[:, None, r:], m["rot"], "half")[:, 0]             # one part for all heads
    kn = (c @ w["uk"].T).view(n, H, d)
    v = (c @ w["uv"].T).view(n, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
    p = softmax_with_sink(scores, window_mask(n, m["mask"]["size"]), None)
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(n, H * dv)
    o = o * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def relu2_expert(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return torch.relu(h @ up.T) ** 2 @ down.T


def route(h: torch.Tensor, router: torch.Tensor, bias: torch.Tensor, top: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(choice [n, top], weight [n, top]): the largest logits (lowest index among equals), softmax over them alone."""
    z = h @ router.T + bias
    val, idx = torch.sort(z, dim=-1, descending=True, stable=True)
    val, idx = val[:, :top], idx[:, :top]
    return idx, torch.softmax(val, dim=-1)


def route_margin(h: torch.Tensor, router: torch.Tensor, bias: torch.Tensor, top: int) -> torch.Tensor:
    """[n]: how far the last chosen logit lies above the first one left out, in units of the row's spread (inf: all chosen)."""
    z = h @ router.T + bias
    if z.shape[-1] <= top:
        return torch.full((h.shape[0],), math.inf, dtype=F)
    val = torch.sort(z, dim=-1, descending=True).values
    return (val[:, top - 1] - val[:, top]) / z.std(dim=-1).clamp_min(1e-30)


def moe(h: torch.Tensor, mlp: dict, w: Dict[str, torch.Tensor], margins: Optional[list] = None) -> torch.Tensor:
    choice, weight = route(h, w["router"], w["router.b"], mlp["router"]["top"])
    if margins is not None:
        margins.append(route_margin(h, w["router"], w["router.b"], mlp["router"]["top"]))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c, p in zip(choice[t].tolist(), weight[t]):
            out[t] += p * relu2_expert(h[t:t + 1], w[f"e{c}.up"], w[f"e{c}.down"])[0]
    if mlp.get("shared") is not None:
        out = out + relu2_expert(h, w["shared.up"], w["shared.down"])
    return out


MIXERS = {"attention": attention_sink, "attention_2": attention_pooled_sigmoid, "latent_attention": latent_attention}


def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(F) for k, v in weights.items() if k.startswith(prefix)}


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: List[int], margins: Optional[list] = None) -> Tuple[torch.Tensor, List[torch.Tensor]]:
    """(logits [n, vocab], the stream after every layer) of one whole sequence.  ``margins`` collects every router's ``route_margin``."""
    eps = float(config["norm"]["eps"])
    x = weights["embed"].to(F)[torch.tensor(tokens, dtype=torch.long)]
    streams = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = scalar_rms_norm(x, weights[p + "norm1"].to(F), eps)
        x = x + MIXERS[layer["type"]](h, layer["mixer"], sub(weights, p + "mix."), eps)
        if layer.get("mlp") is not None:
            h = scalar_rms_norm(x, weights[p + "norm2"].to(F), eps)
            x = x + moe(h, layer["mlp"], sub(weights, p + "mlp."), margins)
        streams.append(x)
    x = scalar_rms_norm(x, weights["final.norm"].to(F), eps)
    return x @ weights["head"].to(F).T, streams
