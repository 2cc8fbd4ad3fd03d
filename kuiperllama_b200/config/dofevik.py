"""Typed configuration of the Dofevik decoder, read from its config.json.

Dofevik is a small decoder-only design: an embedding table, pre-norm layers (x += mixer(norm1(x));
x += ff(norm2(x))), a final norm and a classifier of its own.  Every norm is an RMS norm with ONE learned
number as its weight.  A layer's mixer is one of three kinds of attention, each over a window of the most
recent keys: ``attention`` (biased grouped-query projections, interleaved rotary pairs on part of a head with
linearly scaled positions, q and k divided by their root mean square after the rotation, a sink in the
softmax), ``attention_2`` (values are the keys as projected, a weighted RMS norm on q and k, no rotation,
sigmoid weights with a number per head, and a pooled key and value for every block of positions that has
left the window) and ``latent_attention`` (queries and keys through normed latents, one rotated key part for
all heads, an output gate).  The feed-forward is a mixture of squared-relu experts whose router has a bias
and weighs the chosen experts by a softmax over their logits alone, plus a shared expert.  config.json::

    {"architecture": "Dofevik", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"},
                           "rot": {"base", "dims", "scaling": {"factor"} (optional)}},
                 "mlp": {"kind": "moe", "router": {"experts", "top"}, "expert": {"ff"}, "shared": {"ff"} (optional)} or null},
                {"type": "attention_2", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size", "pool"}}, ...},
                {"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "mask": {"size"},
                           "rot": {"base", "dims"}}, ...}]}

Tensor names: ``embed``, ``head``, ``final.norm`` and under ``l<i>.``: ``norm1``, ``norm2``, ``mix.*``, ``mlp.router``,
``mlp.router.b``, ``mlp.e<k>.up|down``, ``mlp.shared.up|down``.  ExiledOfCode/KuiperLLama has no such model; its
model classes are picked in ``main`` (demo/main.cpp:58).
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .registry import ConfigError, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MIXER_TYPES = ("attention", "attention_2", "latent_attention")
EXPERT_ACTIVATION = "relu2"      # an expert is W_down relu(W_up h)^2
DEFAULT_MAX_POSITIONS = 1 << 17  # the design names no longest sequence; "max_positions" may raise it


def _is_int(v: Any) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _is_num(v: Any) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


@register_architecture("Dofevik")
@dataclass(frozen=True)
class DofevikConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[dict, ...]              # as in config.json, checked
    max_positions: int = DEFAULT_MAX_POSITIONS

    architecture = "Dofevik"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "DofevikConfig":
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

        def rotation(at: str, m: dict, limit_key: str) -> None:
            rot = m.get("rot")
            if not isinstance(rot, dict) or not _is_num(rot.get("base")) or rot.get("base", 0) <= 1:
                problems.append(f'{at}"rot" needs a "base" above 1')
                return
            dims = positive_int(at + '"rot": ', rot, "dims")
            if dims % 2 or (_is_int(m.get(limit_key)) and dims > m[limit_key]):
                problems.append(f'{at}"rot": "dims" {dims} must be even and at most "{limit_key}" {m.get(limit_key)!r}')
            sc = rot.get("scaling")
            if sc is not None and not (isinstance(sc, dict) and _is_num(sc.get("factor")) and sc["factor"] > 0):
                problems.append(f'{at}"rot": "scaling" needs a positive "factor"')

        vocab = positive_int("", d, "vocab")
        width = positive_int("", d, "width")
        eps = number('"norm": ', d.get("norm"), "eps", positive=True)
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
            kind = layer["type"]
            number(at, m, "scale")
            positive_int(at + '"mask": ', m.get("mask"), "size")
            if kind == "latent_attention":
                for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"):
                    positive_int(at, m, k)
                rotation(at, m, "rot_dim")
            else:
                H, G = positive_int(at, m, "heads"), positive_int(at, m, "kv_heads")
                dim = positive_int(at, m, "dim")
                # the values of "attention_2" are its keys: "vdim" may be left out there
                vdim = dim if kind == "attention_2" and "vdim" not in m else positive_int(at, m, "vdim")
                if H % G:
                    problems.append(f'{at}"heads" {H} is not a multiple of "kv_heads" {G}')
                if kind == "attention":
                    rotation(at, m, "dim")
                else:
                    positive_int(at + '"mask": ', m.get("mask"), "pool")
                    if vdim != dim:
                        problems.append(f'{at}the values are the keys, so "vdim" {vdim} must equal "dim" {dim}')
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                problems.append(f'{at}"mlp" must be null or have "kind": "moe", got {mlp!r}')
                continue
            E = positive_int(at + '"mlp": "router": ', mlp.get("router"), "experts")
            top = positive_int(at + '"mlp": "router": ', mlp.get("router"), "top")
            if top > E:
                problems.append(f'{at}"mlp": "top" {top} exceeds "experts" {E}')
            positive_int(at + '"mlp": "expert": ', mlp.get("expert"), "ff")
            if mlp.get("shared") is not None:
                positive_int(at + '"mlp": "shared": ', mlp.get("shared"), "ff")
        max_positions = d.get("max_positions", DEFAULT_MAX_POSITIONS)
        if not _is_int(max_positions) or max_positions <= 0:
            problems.append(f'"max_positions" must be a positive integer, got {max_positions!r}')
        if problems:
            raise ConfigError("config.json (Dofevik): " + "; ".join(problems))
        return cls(vocab=vocab, width=width, norm_eps=eps, layers=tuple(json.loads(json.dumps(l)) for l in layers),
                   max_positions=max_positions)

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "layers": json.loads(json.dumps(list(self.layers))),
             "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        return d

    # ------------------------------------------------------------------ the model it describes
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "name": name, "scalar": True})

    @staticmethod
    def _rope(rot: dict, head_dim: int, pairing: str) -> PartSpec:
        sc = rot.get("scaling")
        return PartSpec("rope", {"head_dim": head_dim, "rotary_dim": rot["dims"], "theta": float(rot["base"]), "pairing": pairing,
                                 "scaling": None if sc is None else {"rope_type": "linear", "factor": float(sc["factor"])}})

    def _mixer(self, kind: str, m: dict) -> Tuple[PartSpec, Optional[PartSpec]]:
        window = int(m["mask"]["size"])
        if kind == "latent_attention":
            return PartSpec("latent_attention", {
                "hidden_size": self.width, "num_heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
                "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "scale": float(m["scale"]), "norm_eps": self.norm_eps, "own_latent": True,
                "window": window, "gate": "element",
                "names": {"dq": "mix.dq", "dq_norm": "mix.dq.norm", "q": "mix.uq", "dkv": "mix.dkv", "dkv_norm": "mix.dkv.norm",
                          "uk": "mix.uk", "uv": "mix.uv", "g": "mix.g", "o": "mix.o"}}), self._rope(m["rot"], m["rot_dim"], "half")
        common = {"hidden_size": self.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                  "value_dim": m.get("vdim", m["dim"]), "scale": float(m["scale"]), "window": window}
        if kind == "attention":
            return PartSpec("window_attention", {
                **common, "values": "own", "weights": "softmax", "head_norm": {"eps": self.norm_eps},
                "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o", "q_bias": "mix.q.b", "k_bias": "mix.k.b",
                          "v_bias": "mix.v.b", "sink": "mix.sink"}}), self._rope(m["rot"], m["dim"], "interleaved")
        return PartSpec("window_attention", {
            **common, "values": "keys", "weights": "sigmoid", "pool": int(m["mask"]["pool"]), "head_norm": {"eps": self.norm_eps},
            "names": {"q": "mix.q", "k": "mix.k", "o": "mix.o", "q_norm": "mix.q.norm", "k_norm": "mix.k.norm",
                      "head_bias": "mix.pb"}}), None

    def _feed_forward(self, mlp: Optional[dict]) -> Optional[PartSpec]:
        if mlp is None:
            return None
        shared = mlp.get("shared")
        names = {"router": "mlp.router", "router_bias": "mlp.router.b", "up": "mlp.e{e}.up", "down": "mlp.e{e}.down"}
        if shared is not None:
            names.update({"shared_up": "mlp.shared.up", "shared_down": "mlp.shared.down"})
        return PartSpec("moe", {
            "hidden_size": self.width, "experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
            "expert_size": mlp["expert"]["ff"], "gated": False, "activation": EXPERT_ACTIVATION, "renormalise": True,
            "shared_size": None if shared is None else shared["ff"], "names": names})

    def to_model_spec(self) -> ModelSpec:
        layers, schedule = [], []
        for i, layer in enumerate(self.layers):
            mixer, position = self._mixer(layer["type"], layer["mixer"])
            ff = self._feed_forward(layer.get("mlp"))
            layers.append(LayerSpec(
                prefix=f"l{i}.", arrangement="pre_norm", mixer=mixer, feed_forward=ff, position=position,
                mixer_norm=self._norm("norm1"), feed_forward_norm=self._norm("norm2") if ff else None))
            schedule.append(ScheduleEntry(layer=i))
        unread = tuple(f"l{i}.norm2" for i, layer in enumerate(self.layers) if layer.get("mlp") is None)
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab, max_positions=self.max_positions,
            layers=tuple(layers), schedule=tuple(schedule), embedding_name="embed", final_norm=self._norm("norm"),
            final_norm_prefix="final.", lm_head_name="head", ignorable_suffixes=unread)
        spec.validate()
        return spec
