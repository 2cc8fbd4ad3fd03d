"""Typed configuration of the Bededra decoder, read from its config.json.

Bededra is a small decoder-only design whose layers read the stream twice and add both results at once,
x += (mixer(h + conv(h)) + ff(norm2(x))) with h = norm1(x), RMS norms, and a short causal convolution per channel in
front of every mixer.  The mixer is a state-space layer (``mamba2``) or two mixers side by side (``parallel``): softmax
attention without rotation (soft-capped scores, a logarithmic distance bias, a sliding window that keeps the first
tokens, weights mixed between the heads, a gate per head) and gated linear attention.  The feed-forward is up, squared
relu, down, or a mixture of SiLU-gated experts chosen among the best groups of experts.  config.json lists the layers::

    {"architecture": "Bededra", "vocab": V, "width": W, "norm": {"eps": e}, "canon": {"taps": k},
     "layers": [{"type": "mamba2", "mixer": {"heads", "vdim", "state", "groups", "conv", "norm_groups"},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap", "mask": {"size", "keep_first"}},
                           "right": {"heads", "dim", "vdim", "tau"}, "left_scale": a, "right_scale": b},
                 "mlp": {"kind": "moe", "router": {"experts", "top", "groups": {"count", "keep"}}, "expert": {"ff"}} or null}]}

Tensor names: ``embed``, ``head``, ``final.norm``, and under ``l<i>.``: ``norm1``, ``norm2``, ``canon1``, ``mix.*`` (``mix.left.*``
and ``mix.right.*`` in a parallel layer) and ``mlp.*`` (experts: ``mlp.e<k>.gate|up|down``, ``mlp.router``).  The rank of the
gated linear attention's decay projection is not in config.json; ``from_folder_shapes`` reads it from the tensor's shape.
ExiledOfCode/KuiperLLama has no such model; its model classes are picked in ``main`` (demo/main.cpp:58).
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .registry import ConfigError, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MIXER_TYPES = ("mamba2", "parallel")
# Constants the design fixes (parameters of the parts, so another design may choose others).
ROUTER_RENORM_EPS = 1e-20        # the chosen experts' scores are divided by their sum + 1e-20
DEFAULT_DECAY_RANK = 16          # the decay's low rank where config.json and the tensors do not say (random weights)
DEFAULT_MAX_POSITIONS = 1 << 17  # the design names no longest sequence; "max_positions" may raise it


def _is_int(v: Any) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _is_num(v: Any) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


@register_architecture("Bededra")
@dataclass(frozen=True)
class BededraConfig:
    vocab: int
    width: int
    norm_eps: float
    canon_taps: int
    layers: Tuple[dict, ...]              # as in config.json, checked
    max_positions: int = DEFAULT_MAX_POSITIONS

    architecture = "Bededra"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "BededraConfig":
        problems: List[str] = []

        def positive_int(where: str, obj: Any, key: str) -> int:
            v = obj.get(key) if isinstance(obj, dict) else None
            if not _is_int(v) or v <= 0:
                problems.append(f'{where}"{key}" must be a positive integer, got {v!r}')
                return 1
            return v

        def number(where: str, obj: Any, key: str, positive: bool = False) -> float:
            v = obj.get(key) if isinstance(obj, dict) else None
            if not _is_num(v) or (positive and v <= 0):
                problems.append(f'{where}"{key}" must be a {"positive " if positive else ""}number, got {v!r}')
                return 1.0
            return float(v)

        vocab = positive_int("", d, "vocab")
        width = positive_int("", d, "width")
        eps = number('"norm": ', d.get("norm"), "eps", positive=True)
        taps = positive_int('"canon": ', d.get("canon"), "taps")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            problems.append('"layers" must be a list with at least one layer')
            layers = []
        for i, layer in enumerate(layers):
            at = f"layers[{i}]: "
            if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
                problems.append(f'{at}"type" must be one of {list(MIXER_TYPES)}, got {layer.get("type") if isinstance(layer, dict) else layer!r}')
                continue
            m = layer.get("mixer")
            if not isinstance(m, dict):
                problems.append(f'{at}"mixer" must be an object')
                continue
            if layer["type"] == "mamba2":
                H, G = positive_int(at, m, "heads"), positive_int(at, m, "groups")
                P = positive_int(at, m, "vdim")
                positive_int(at, m, "state"); positive_int(at, m, "conv")
                parts = positive_int(at, m, "norm_groups")
                if H % G:
                    problems.append(f'{at}"heads" {H} is not a multiple of "groups" {G}')
                if (H * P) % parts:
                    problems.append(f'{at}"norm_groups" {parts} does not divide the {H * P} inner channels')
            else:
                left, right = m.get("left"), m.get("right")
                at_l, at_r = at + '"left": ', at + '"right": '
                H, G = positive_int(at_l, left, "heads"), positive_int(at_l, left, "kv_heads")
                positive_int(at_l, left, "dim"); positive_int(at_l, left, "vdim")
                number(at_l, left, "scale")
                if isinstance(left, dict) and left.get("softcap") is not None:
                    number(at_l, left, "softcap", positive=True)
                if H % G:
                    problems.append(f'{at_l}"heads" {H} is not a multiple of "kv_heads" {G}')
                mask = left.get("mask") if isinstance(left, dict) else None
                if mask is not None:
                    positive_int(at_l + '"mask": ', mask, "size")
                    kf = mask.get("keep_first", 0) if isinstance(mask, dict) else 0
                    if not _is_int(kf) or kf < 0:
                        problems.append(f'{at_l}"mask": "keep_first" must be a non-negative integer, got {kf!r}')
                for k in ("heads", "dim", "vdim"):
                    positive_int(at_r, right, k)
                number(at_r, right, "tau", positive=True)
                if isinstance(right, dict) and right.get("rank") is not None:
                    positive_int(at_r, right, "rank")
                number(at, m, "left_scale"); number(at, m, "right_scale")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                problems.append(f'{at}"mlp" must be null or have "kind": "dense" or "moe", got {mlp!r}')
            elif mlp["kind"] == "dense":
                positive_int(at + '"mlp": ', mlp, "ff")
            else:
                r = mlp.get("router")
                E = positive_int(at + '"mlp": "router": ', r, "experts")
                top = positive_int(at + '"mlp": "router": ', r, "top")
                positive_int(at + '"mlp": "expert": ', mlp.get("expert"), "ff")
                count = keep = 1
                grp = r.get("groups") if isinstance(r, dict) else None
                if grp is not None:
                    count = positive_int(at + '"mlp": "router": "groups": ', grp, "count")
                    keep = positive_int(at + '"mlp": "router": "groups": ', grp, "keep")
                if E % count or keep > count:
                    problems.append(f'{at}"mlp": {E} experts do not form {count} equal groups of which {keep} are kept')
                elif top > keep * (E // count):
                    problems.append(f'{at}"mlp": "top" {top} exceeds the {keep * (E // count)} experts of the kept groups')
        max_positions = d.get("max_positions", DEFAULT_MAX_POSITIONS)
        if not _is_int(max_positions) or max_positions <= 0:
            problems.append(f'"max_positions" must be a positive integer, got {max_positions!r}')
        if problems:
            raise ConfigError("config.json (Bededra): " + "; ".join(problems))
        return cls(vocab=vocab, width=width, norm_eps=eps, canon_taps=taps, layers=tuple(json.loads(json.dumps(l)) for l in layers),
                   max_positions=max_positions)

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "canon": {"taps": self.canon_taps}, "layers": json.loads(json.dumps(list(self.layers))),
             "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        return d

    # ------------------------------------------------------------------ sizes that only the tensors give
    def with_tensor_shapes(self, shapes: Dict[str, Tuple[int, ...]]) -> "BededraConfig":
        """The same configuration with every size that config.json leaves to the tensors filled in from ``shapes`` (tensor
        name -> shape): the rank of a parallel layer's decay projection, ``right.rank``, from ``l<i>.mix.right.a1``."""
        layers = json.loads(json.dumps(list(self.layers)))
        for i, layer in enumerate(layers):
            if layer["type"] == "parallel" and layer["mixer"]["right"].get("rank") is None:
                shape = shapes.get(f"l{i}.mix.right.a1")
                if shape is not None and len(shape) == 2:
                    layer["mixer"]["right"]["rank"] = int(shape[0])
        return BededraConfig(self.vocab, self.width, self.norm_eps, self.canon_taps, tuple(layers), self.max_positions)

    # ------------------------------------------------------------------ the model it describes
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "name": name})

    def _mixer(self, kind: str, m: dict) -> PartSpec:
        if kind == "mamba2":
            inner = PartSpec("mamba2", {
                "hidden_size": self.width, "heads": m["heads"], "vdim": m["vdim"], "state": m["state"], "groups": m["groups"],
                "conv": m["conv"], "norm_groups": m["norm_groups"], "norm_eps": self.norm_eps,
                "names": {"in": "mix.in", "conv": "mix.conv", "conv_bias": "mix.conv.b", "dt_bias": "mix.dt_bias", "A_log": "mix.A_log",
                          "D": "mix.D", "norm": "mix.norm", "o": "mix.o"}})
        else:
            left, right = m["left"], m["right"]
            mask = left.get("mask")
            attention = PartSpec("mixed_head_attention", {
                "hidden_size": self.width, "heads": left["heads"], "kv_heads": left["kv_heads"], "dim": left["dim"], "vdim": left["vdim"],
                "scale": float(left["scale"]), "softcap": None if left.get("softcap") is None else float(left["softcap"]),
                "window": None if mask is None else mask["size"], "keep_first": 0 if mask is None else mask.get("keep_first", 0),
                "names": {"q": "mix.left.q", "k": "mix.left.k", "v": "mix.left.v", "o": "mix.left.o", "r1": "mix.left.r1",
                          "r2": "mix.left.r2", "talk": "mix.left.talk", "g": "mix.left.g"}})
            linear = PartSpec("gated_linear_attention", {
                "hidden_size": self.width, "heads": right["heads"], "dim": right["dim"], "vdim": right["vdim"],
                "rank": right.get("rank") or DEFAULT_DECAY_RANK, "tau": float(right["tau"]), "q_scale": float(right["dim"]) ** -0.5,
                "norm_eps": self.norm_eps,
                "names": {"q": "mix.right.q", "k": "mix.right.k", "v": "mix.right.v", "g": "mix.right.g", "o": "mix.right.o",
                          "norm": "mix.right.norm", "a1": "mix.right.a1", "a2": "mix.right.a2", "a2_bias": "mix.right.a2.b"}})
            inner = PartSpec("parallel", {"branches": [{"mixer": attention, "scale": float(m["left_scale"])},
                                                       {"mixer": linear, "scale": float(m["right_scale"])}]})
        return PartSpec("input_conv", {"hidden_size": self.width, "taps": self.canon_taps, "name": "canon1", "inner": inner})

    def _feed_forward(self, mlp: Optional[dict]) -> Optional[PartSpec]:
        if mlp is None:
            return None
        if mlp["kind"] == "dense":
            return PartSpec("dense", {"hidden_size": self.width, "intermediate_size": mlp["ff"], "activation": "relu2",
                                      "names": {"up": "mlp.up", "down": "mlp.down"}})
        r = mlp["router"]
        grp = r.get("groups") or {"count": 1, "keep": 1}
        return PartSpec("moe", {
            "hidden_size": self.width, "experts": r["experts"], "top": r["top"], "expert_size": mlp["expert"]["ff"],
            "limit": None, "alpha": 1.0, "shift": 0.0, "renormalise": True, "renorm_eps": ROUTER_RENORM_EPS,
            "groups": grp["count"], "keep_groups": grp["keep"],
            "names": {"router": "mlp.router", "gate": "mlp.e{e}.gate", "up": "mlp.e{e}.up", "down": "mlp.e{e}.down"}})

    def to_model_spec(self) -> ModelSpec:
        layers, schedule = [], []
        for i, layer in enumerate(self.layers):
            ff = self._feed_forward(layer.get("mlp"))
            layers.append(LayerSpec(
                prefix=f"l{i}.", arrangement="parallel", mixer=self._mixer(layer["type"], layer["mixer"]), feed_forward=ff,
                mixer_norm=self._norm("norm1"), feed_forward_norm=self._norm("norm2") if ff else None, position=None))
            schedule.append(ScheduleEntry(layer=i))
        unread = tuple(f"l{i}.norm2" for i, layer in enumerate(self.layers) if layer.get("mlp") is None)
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab, max_positions=self.max_positions,
            layers=tuple(layers), schedule=tuple(schedule), embedding_name="embed", final_norm=self._norm("norm"),
            final_norm_prefix="final.", lm_head_name="head", ignorable_suffixes=unread)
        spec.validate()
        return spec
