"""A plain, slow implementation of the Bededra decoder: whole sequences, no cache, float64 on the
CPU, one function per mechanism.  It shares no code with the package and is what the tests of
the package's Bededra parts compare against.

A model is an embedding table, layers, a final RMS norm and a classifier of its own.  A layer reads
the stream twice and adds both results at once:

    x <- x + (mixer(h + conv(h)) + ff(norm2(x))),   h = norm1(x)

where conv is a short causal convolution per channel.  Mixers: a state-space layer (``mamba2``) and
a pair of mixers side by side (``parallel``): windowed softmax attention whose weights are mixed
between the heads, and gated linear attention.  Feed-forwards: up, squared relu, down; or a mixture
of SiLU-gated experts chosen among the best groups of experts.  ``weights`` maps tensor names to
arrays; ``cfg`` is the config.json dictionary.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def t64(a) -> torch.Tensor:
    return torch.as_tensor(a, dtype=F)


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """h [T, C], w [C, taps]: out_t = sum_j w[:, j] * h_(t - taps + 1 + j); nothing before the first token."""
    T, taps = h.shape[0], w.shape[1]
    out = torch.zeros_like(h)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            out[back:] += w[:, j] * h[:T - back]
    return out


def mamba2_mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """The state-space mixer.  W: in, conv, conv.b, dt_bias, A_log, D, norm, o."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = h @ W["in"].T
    z, xBC, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xBC = silu(causal_conv(xBC, W["conv"]) + W["conv.b"])
    x = xBC[:, :inner].reshape(T, H, P)
    B = xBC[:, inner:inner + G * N].reshape(T, G, N)
    C = xBC[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + W["dt_bias"])                             # [T, H]
    decay = torch.exp(-torch.exp(W["A_log"]) * dt)               # [T, H]
    y = torch.zeros(T, H, P, dtype=F)
    S = torch.zeros(H, N, P, dtype=F)
    per = H // G
    for t in range(T):
        for hh in range(H):
            g = hh // per
            S[hh] = decay[t, hh] * S[hh] + dt[t, hh] * torch.outer(B[t, g], x[t, hh])
            y[t, hh] = S[hh].T @ C[t, g] + W["D"][hh] * x[t, hh]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_norm(y.reshape(T, parts, inner // parts), None, eps).reshape(T, inner) * W["norm"]
    return y @ W["o"].T


def visible(i: int, j: int, size: int, keep_first: int) -> bool:
    return j <= i and (i - j < size or j < keep_first)


def mixed_attention_weights(q: torch.Tensor, k: torch.Tensor, m: dict, r1, r2, talk):
    """q [T, H, d], k [T, G, d] -> (softmax weights [H, T, T], the weights after the heads were mixed [H, T, T])."""
    T, H = q.shape[0], q.shape[1]
    per = H // k.shape[1]
    mask_cfg = m.get("mask")
    size, keep = (mask_cfg["size"], mask_cfg.get("keep_first", 0)) if mask_cfg else (T + 1, 0)
    cap, scale = m.get("softcap"), float(m["scale"])
    idx = torch.arange(T)
    dist = (idx[:, None] - idx[None, :]).clamp(min=0).to(F)                  # i - j
    mask = torch.tensor([[visible(i, j, size, keep) for j in range(T)] for i in range(T)])
    weights = torch.zeros(H, T, T, dtype=F)
    for hh in range(H):
        s = (q[:, hh] @ k[:, hh // per].T) * scale
        if cap is not None:
            s = float(cap) * torch.tanh(s / float(cap))
        if r1 is not None:
            s = s - r1[hh] * torch.log1p(r2[hh] * dist)
        s = s.masked_fill(~mask, -math.inf)
        weights[hh] = torch.softmax(s, dim=-1)
    mixed = weights if talk is None else torch.einsum("hg,gij->hij", talk, weights)
    return weights, mixed


def mixed_head_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], m: dict) -> torch.Tensor:
    """Softmax attention without rotation: soft-capped scores less a distance bias, a sliding window that also keeps the
    first tokens, the heads' weights mixed after the softmax, a gate per head.  W: q, k, v, r1, r2, talk, g, o."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W["q"].T).reshape(T, H, d)
    k = (h @ W["k"].T).reshape(T, G, d)
    v = (h @ W["v"].T).reshape(T, G, dv)
    _, mixed = mixed_attention_weights(q, k, m, W.get("r1"), W.get("r2"), W.get("talk"))
    gate = torch.sigmoid(h @ W["g"].T)                                       # [T, H]
    out = torch.zeros(T, H, dv, dtype=F)
    for hh in range(H):
        out[:, hh] = (mixed[hh] @ v[:, hh // (H // G)]) * gate[:, hh:hh + 1]
    return out.reshape(T, H * dv) @ W["o"].T


def gated_linear_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head.  W: q, k, v, g, o, norm, a1, a2, a2.b."""
    T = h.shape[0]
    H, d, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (h @ W["q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ W["k"].T).reshape(T, H, d)
    v = (h @ W["v"].T).reshape(T, H, dv)
    zed = (h @ W["a1"].T) @ W["a2"].T + W["a2.b"]
    alpha = torch.sigmoid(zed).pow(1.0 / tau).reshape(T, H, d)
    o = torch.zeros(T, H, dv, dtype=F)
    S = torch.zeros(H, d, dv, dtype=F)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(o, W["norm"], eps).reshape(T, H * dv)
    return (o * silu(h @ W["g"].T)) @ W["o"].T


def parallel_mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    left = mixed_head_attention(h, {k[5:]: v for k, v in W.items() if k.startswith("left.")}, m["left"])
    right = gated_linear_attention(h, {k[6:]: v for k, v in W.items() if k.startswith("right.")}, m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def dense_ff(h: torch.Tensor, W: Dict[str, torch.Tensor]) -> torch.Tensor:
    return torch.relu(h @ W["up"].T) ** 2 @ W["down"].T


def route(scores: torch.Tensor, top: int, groups: int, keep: int) -> List[int]:
    """The chosen experts of one token from its softmax scores: the ``top`` largest among the experts of the ``keep``
    groups (of neighbouring experts) whose largest score is largest.  The lower index wins among equals."""
    E = scores.numel()
    per = E // groups
    best = [max(float(scores[g * per + i]) for i in range(per)) for g in range(groups)]
    kept = sorted(range(groups), key=lambda g: (-best[g], g))[:keep]
    allowed = [e for e in range(E) if e // per in kept]
    return sorted(allowed, key=lambda e: (-float(scores[e]), e))[:top]


def moe_ff(h: torch.Tensor, W: Dict[str, torch.Tensor], mlp: dict) -> torch.Tensor:
    r = mlp["router"]
    E, top = r["experts"], r["top"]
    grp = r.get("groups") or {"count": 1, "keep": 1}
    s = torch.softmax(h @ W["router"].T, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = route(s[t], top, grp["count"], grp["keep"])
        total = sum(float(s[t, e]) for e in chosen) + 1e-20
        for e in chosen:
            f = (silu(h[t] @ W[f"e{e}.gate"].T) * (h[t] @ W[f"e{e}.up"].T)) @ W[f"e{e}.down"].T
            out[t] += float(s[t, e]) / total * f
    return out


def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: t64(v) for k, v in weights.items() if k.startswith(prefix)}


def layer_forward(x: torch.Tensor, weights, i: int, layer: dict, cfg: dict) -> torch.Tensor:
    eps = float(cfg["norm"]["eps"])
    p = f"l{i}."
    h = rms_norm(x, t64(weights[p + "norm1"]), eps)
    h = h + causal_conv(h, t64(weights[p + "canon1"]))
    W = sub(weights, p + "mix.")
    if layer["type"] == "mamba2":
        mixed = mamba2_mixer(h, W, layer["mixer"], eps)
    elif layer["type"] == "parallel":
        mixed = parallel_mixer(h, W, layer["mixer"], eps)
    else:
        raise ValueError(layer["type"])
    mlp = layer.get("mlp")
    if mlp is None:
        return x + mixed
    h2 = rms_norm(x, t64(weights[p + "norm2"]), eps)
    Wf = sub(weights, p + "mlp.")
    ff = dense_ff(h2, Wf) if mlp["kind"] == "dense" else moe_ff(h2, Wf, mlp)
    return x + (mixed + ff)


def forward(weights, cfg: dict, tokens, return_layers: bool = False):
    """float64 logits [T, vocab] of one sequence (and the stream after every layer)."""
    x = t64(weights["embed"])[torch.as_tensor(tokens, dtype=torch.long)]
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        x = layer_forward(x, weights, i, layer, cfg)
        streams.append(x.clone())
    logits = rms_norm(x, t64(weights["final.norm"]), float(cfg["norm"]["eps"])) @ t64(weights["head"]).T
    return (logits, streams) if return_layers else logits


def greedy(weights, cfg: dict, prompt, n_new: int) -> List[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(torch.argmax(forward(weights, cfg, toks)[-1])))
    return toks[len(prompt):]
