"""The Bededra configuration on the CPU: reading config.json, its faults, the model it describes, the tensors that
model reads, what it asks of the cache, and the plain implementation's own mechanisms against values worked out by hand."""
from __future__ import annotations

import json
import math
import random

import pytest
import torch

import plain_bededra as P
from bededra_helpers import CONFIGS, tensor_shapes


def _cfg(name):
    from kuiperllama_b200.config import config_from_dict
    return config_from_dict(json.loads(json.dumps(CONFIGS[name])))


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_manifest_names_and_shapes(name):
    from kuiperllama_b200.engine.model import model_manifest
    cfg = _cfg(name)
    assert type(cfg).__name__ == "BededraConfig"
    got = {k: tuple(v.shape) for k, v in model_manifest(cfg.to_model_spec()).items()}
    assert got == tensor_shapes(CONFIGS[name])


def test_round_trip_and_spec():
    from kuiperllama_b200.config import config_from_dict
    cfg = _cfg("mixed")
    again = config_from_dict(cfg.to_dict())
    assert again.to_dict() == cfg.to_dict() and again.to_dict()["layers"] == CONFIGS["mixed"]["layers"]
    spec = cfg.to_model_spec()
    assert spec.lm_head_name == "head" and spec.embedding_name == "embed" and spec.hidden_size == 64 and spec.vocab_size == 97
    assert (spec.embedding_multiplier, spec.logit_scale, spec.logit_softcap) == (None, None, None)
    assert all(l.arrangement == "parallel" and l.mixer.kind == "input_conv" and l.mixer["taps"] == 4 and l.position is None for l in spec.layers)
    assert [l.mixer["inner"].kind for l in spec.layers] == ["parallel", "mamba2", "parallel", "mamba2", "parallel"]
    assert [l.feed_forward.kind if l.feed_forward else None for l in spec.layers] == ["moe", "dense", None, "moe", "dense"]
    assert spec.layers[2].feed_forward_norm is None and "l2.norm2" in spec.ignorable_suffixes
    left, right = (b["mixer"] for b in spec.layers[0].mixer["inner"]["branches"])
    assert [b["scale"] for b in spec.layers[0].mixer["inner"]["branches"]] == [0.8, 1.3]
    assert (left.kind, left["heads"], left["kv_heads"], left["dim"], left["vdim"], left["scale"], left["softcap"], left["window"], left["keep_first"]) \
        == ("mixed_head_attention", 4, 2, 12, 20, 0.4, 15.0, 40, 5)
    assert (right.kind, right["heads"], right["dim"], right["vdim"], right["rank"], right["tau"]) == ("gated_linear_attention", 3, 8, 16, 5, 6.0)
    assert right["q_scale"] == 8 ** -0.5
    no_window = spec.layers[4].mixer["inner"]["branches"][0]["mixer"]
    assert no_window["window"] is None and no_window["softcap"] is None and spec.layers[4].mixer["inner"]["branches"][0]["scale"] == -0.7
    moe = spec.layers[0].feed_forward
    assert (moe["experts"], moe["top"], moe["expert_size"], moe["limit"], moe["alpha"], moe["shift"], moe["renormalise"], moe["renorm_eps"],
            moe["groups"], moe["keep_groups"]) == (6, 3, 24, None, 1.0, 0.0, True, 1e-20, 3, 2)
    assert (spec.layers[3].feed_forward["groups"], spec.layers[3].feed_forward["keep_groups"]) == (1, 1)
    assert spec.layers[1].feed_forward["activation"] == "relu2"
    ssm = spec.layers[1].mixer["inner"]
    assert (ssm["heads"], ssm["vdim"], ssm["state"], ssm["groups"], ssm["conv"], ssm["norm_groups"]) == (6, 8, 12, 2, 3, 3)


def test_the_decay_rank_comes_from_the_tensor_where_the_configuration_is_silent():
    from kuiperllama_b200.config import config_from_dict
    c = json.loads(json.dumps(CONFIGS["mixed"]))
    for layer in c["layers"]:
        if layer["type"] == "parallel":
            del layer["mixer"]["right"]["rank"]
    cfg = config_from_dict(c).with_tensor_shapes(tensor_shapes(CONFIGS["mixed"]))
    ranks = [l["mixer"]["right"]["rank"] for l in cfg.layers if l["type"] == "parallel"]
    assert ranks == [5, 7, 3]


def test_faults_are_listed_together():
    from kuiperllama_b200.config import ConfigError, config_from_dict
    c = json.loads(json.dumps(CONFIGS["mixed"]))
    c["vocab"] = 0
    c["canon"] = {}
    c["layers"][0]["mixer"]["left"]["kv_heads"] = 3                 # 4 heads
    c["layers"][0]["mlp"]["router"]["groups"] = {"count": 4, "keep": 1}     # 6 experts
    c["layers"][1]["mixer"]["norm_groups"] = 5                      # 48 inner channels
    c["layers"][3]["mlp"]["router"]["top"] = 9                      # 5 experts
    c["layers"][4]["type"] = "attention"
    del c["layers"][2]["mixer"]["right"]["tau"]
    with pytest.raises(ConfigError) as e:
        config_from_dict(c)
    msg = str(e.value)
    for part in ('"vocab"', '"taps"', "layers[0]", '"kv_heads" 3', "4 equal groups", "layers[1]", '"norm_groups" 5', "layers[3]", "layers[4]",
                 '"tau"'):
        assert part in msg, (part, msg)
    c = json.loads(json.dumps(CONFIGS["mixed"]))
    c["layers"][0]["mlp"]["router"]["top"] = 5                      # two kept groups of two experts
    with pytest.raises(ConfigError, match="kept groups"):
        config_from_dict(c)


def test_cache_requests_of_the_parts():
    """What a model asks of the cache: pages with a window, kept first keys and a value size of their own; state for the
    recurrences and for every layer's convolution in front."""
    from kuiperllama_b200.cache import KVRequest
    from kuiperllama_b200.parts import part_class
    from kuiperllama_b200.parts.base import Runtime
    from kuiperllama_b200.weights.random_init import RandomTensors
    from kuiperllama_b200.engine.model import model_manifest
    spec = _cfg("mixed").to_model_spec()
    tensors = RandomTensors(model_manifest(spec), 0, "cpu", torch.float32)
    rt = Runtime(device=torch.device("cpu"), dtype=torch.float32)
    mixers = [part_class("mixer", l.mixer.kind)(l.mixer, l.prefix, tensors, rt, None) for l in spec.layers]
    assert mixers[0].kv_request() == KVRequest(2, 12, "full", window=40, value_dim=20, keep_first=5)
    assert mixers[2].kv_request() == KVRequest(6, 8, "full", window=70, value_dim=None, keep_first=0)
    assert mixers[4].kv_request() == KVRequest(1, 16, "full", window=None, value_dim=12, keep_first=0)
    assert mixers[1].kv_request() is None
    taps = 3 * 64
    assert mixers[0].state_request().shape == (3 * 8 * 16 + taps,)
    assert mixers[1].state_request().shape == (6 * 12 * 8 + 2 * (48 + 2 * 2 * 12) + taps,)
    assert mixers[3].state_request().shape == (3 * 20 * 16 + 0 + taps,)


def test_a_window_that_keeps_first_keys_keeps_their_pages():
    from kuiperllama_b200.cache import PAGE, KVRequest, SequenceCache
    from kuiperllama_b200.cache.allocators import pages_for
    W, KEEP = 100, 70                                    # the kept keys reach into the second page
    kv = [KVRequest(2, 16, value_dim=24), KVRequest(2, 16, window=W, keep_first=KEEP)]
    c = SequenceCache(kv, [None] * 2, [None] * 2, max_tokens=PAGE * 32, max_seq_len=PAGE * 16, dtype=torch.float32, device="cpu")
    full, win = c.groups
    assert tuple(full.k.shape[-2:]) == (PAGE, 16) and tuple(full.v.shape[-2:]) == (PAGE, 24) and tuple(win.v.shape[-2:]) == (PAGE, 16)
    a, b = c.alloc_slot(), c.alloc_slot()
    lengths = {a: 0, b: 0}
    rng = random.Random(7)
    for slot, n in [(a, 400), (b, 30)] + [(rng.choice([a, b]), rng.choice([1, 1, 1, 50])) for _ in range(200)]:
        before = lengths[slot]
        if before + n > c.max_seq_len:
            continue
        c.reserve(slot, before + n)
        lengths[slot] = c.lengths[slot] = before + n
        for s, length in lengths.items():
            pages = win.slot_pages[s]
            first_needed = max(0, (length - n if s == slot else length) - W + 1) // PAGE if length else 0
            assert all(p >= 0 for p in pages[first_needed:]) and all(p >= 0 for p in pages[:pages_for(KEEP, PAGE)])
        held = [p for s in lengths for p in win.pages_of(s)]
        assert len(held) == len(set(held)) == win.pages.held()
    assert any(p < 0 for p in win.slot_pages[a]) and win.pages.held() < full.pages.held()
    assert all(len(win.pages_of(s)) <= pages_for(W, PAGE) + 2 + pages_for(KEEP, PAGE) for s in lengths)
    c.free_slot(a); c.free_slot(b)
    assert c.pages_held() == [0, 0]


# ----------------------------------------------------------------------------- the plain implementation against hand values

def test_plain_convolution_and_visibility():
    h = torch.tensor([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0], [4.0, 40.0]], dtype=torch.float64)
    w = torch.tensor([[0.5, -1.0, 2.0], [1.0, 0.0, 0.1]], dtype=torch.float64)       # last column: the current token
    out = P.causal_conv(h, w)
    assert out[0].tolist() == [2.0, 1.0] and out[1].tolist() == [-1.0 + 4.0, 2.0]
    assert out[3].tolist() == [0.5 * 2 - 3 + 8, 20.0 + 4.0]
    # a window of 3 that keeps the first 2: position 6 sees 4, 5, 6 and 0, 1
    assert [j for j in range(8) if P.visible(6, j, 3, 2)] == [0, 1, 4, 5, 6]
    assert [j for j in range(8) if P.visible(1, j, 3, 2)] == [0, 1]


def test_plain_router_groups():
    s = torch.tensor([0.05, 0.30, 0.10, 0.02, 0.25, 0.28], dtype=torch.float64)     # groups of two: best scores 0.30, 0.10, 0.28
    assert P.route(s, 2, 1, 1) == [1, 5]
    assert P.route(s, 2, 3, 1) == [1, 0]                  # only the best group
    assert P.route(s, 3, 3, 2) == [1, 5, 4]               # groups 0 and 2
    assert P.route(torch.full((6,), 1 / 6, dtype=torch.float64), 3, 3, 2) == [0, 1, 2]     # equal scores: the lower index


def test_plain_recurrences_on_two_tokens():
    """One head, state of two rows, one value column, by hand."""
    W = {"in": torch.zeros(1 + 1 + 2 + 2 + 1, 1, dtype=torch.float64), "conv": torch.tensor([[1.0]] * 5, dtype=torch.float64),
         "conv.b": torch.zeros(5, dtype=torch.float64), "dt_bias": torch.tensor([0.0], dtype=torch.float64),
         "A_log": torch.tensor([0.0], dtype=torch.float64), "D": torch.tensor([0.5], dtype=torch.float64),
         "norm": torch.tensor([1.0], dtype=torch.float64), "o": torch.tensor([[1.0]], dtype=torch.float64)}
    W["in"][:, 0] = torch.tensor([1.0, 1.0, 1.0, 2.0, 1.0, -1.0, 0.0])       # z, x, B (2), C (2), dt for an input of 1
    m = {"heads": 1, "vdim": 1, "state": 2, "groups": 1, "conv": 1, "norm_groups": 1}
    h = torch.tensor([[1.0], [2.0]], dtype=torch.float64)
    got = P.mamba2_mixer(h, W, m, 0.0)
    silu = lambda v: v / (1 + math.exp(-v))
    dt = math.log(2.0)                                   # softplus(0)
    x1, B1, C1 = silu(1.0), [silu(1.0), silu(2.0)], [silu(1.0), silu(-1.0)]
    S1 = [dt * b * x1 for b in B1]
    y1 = S1[0] * C1[0] + S1[1] * C1[1] + 0.5 * x1
    x2, B2, C2 = silu(2.0), [silu(2.0), silu(4.0)], [silu(2.0), silu(-2.0)]
    S2 = [math.exp(-dt) * s + dt * b * x2 for s, b in zip(S1, B2)]
    y2 = S2[0] * C2[0] + S2[1] * C2[1] + 0.5 * x2
    # one channel, eps 0: the norm leaves the sign of y * silu(z)
    assert got[:, 0].tolist() == pytest.approx([math.copysign(1.0, y1 * silu(1.0)), math.copysign(1.0, y2 * silu(2.0))])
    # gated linear attention with one key channel: S_2 = alpha_2 k_1 v_1 + k_2 v_2
    Wg = {"q": torch.tensor([[1.0]]), "k": torch.tensor([[2.0]]), "v": torch.tensor([[1.0], [3.0]]), "g": torch.tensor([[1.0], [1.0]]),
          "o": torch.eye(2), "norm": torch.ones(2), "a1": torch.tensor([[1.0]]), "a2": torch.tensor([[1.0]]), "a2.b": torch.tensor([0.5])}
    Wg = {k: v.double() for k, v in Wg.items()}
    mg = {"heads": 1, "dim": 1, "vdim": 2, "tau": 2.0}
    out = P.gated_linear_attention(h, Wg, mg, 0.0)
    alpha2 = (1 / (1 + math.exp(-2.5))) ** 0.5
    o2 = [(alpha2 * 2 * 1 + 4 * 2) * 2 * c for c in (1.0, 3.0)]       # S (k v summed with decay) times q = 2
    rms = math.sqrt((o2[0] ** 2 + o2[1] ** 2) / 2)
    assert out[1].tolist() == pytest.approx([o2[0] / rms * silu(2.0), o2[1] / rms * silu(2.0)])


def test_plain_attention_mixes_normalised_weights():
    """Two heads, two tokens: with talk = [[1, 0], [1, 1]] the second head's weights are the sum of both heads' (each summing to
    one), so with values of ones its result is 2 and the first head's is 1; the gate halves both (a zero gate matrix)."""
    W = {"q": torch.randn(2 * 3, 4), "k": torch.randn(3, 4), "v": torch.zeros(2, 4), "r1": torch.tensor([0.3, 0.0]), "r2": torch.tensor([1.0, 2.0]),
         "talk": torch.tensor([[1.0, 0.0], [1.0, 1.0]]), "g": torch.zeros(2, 4), "o": torch.eye(4)}
    W = {k: v.double() for k, v in W.items()}
    h = torch.randn(2, 4, dtype=torch.float64)
    h[:, 0] = 1.0
    W["v"][:, 0] = 1.0                                    # every value is (1, 1) whatever the token
    m = {"heads": 2, "kv_heads": 1, "dim": 3, "vdim": 2, "scale": 0.7, "softcap": 5.0, "mask": {"size": 1, "keep_first": 1}}
    out = P.mixed_head_attention(h, W, m)
    assert out[1].tolist() == pytest.approx([0.5, 0.5, 1.0, 1.0])
