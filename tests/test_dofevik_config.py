"""The Dofevik configuration on the CPU: reading config.json, its faults, the model it describes, the tensors that
model reads, what it asks of the cache (the pooled kind's pages among them), and the plain implementation's own
mechanisms against values worked out by hand."""
from __future__ import annotations

import json
import math

import pytest
import torch

import plain_dofevik as P
from dofevik_helpers import CONFIGS, tensor_shapes


def _cfg(name):
    from kuiperllama_b200.config import config_from_dict
    return config_from_dict(json.loads(json.dumps(CONFIGS[name])))


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_manifest_names_and_shapes(name):
    from kuiperllama_b200.engine.model import model_manifest
    cfg = _cfg(name)
    assert type(cfg).__name__ == "DofevikConfig"
    got = {k: tuple(v.shape) for k, v in model_manifest(cfg.to_model_spec()).items()}
    assert got == tensor_shapes(CONFIGS[name])


def test_round_trip_and_spec():
    from kuiperllama_b200.config import config_from_dict
    cfg = _cfg("mixed")
    again = config_from_dict(cfg.to_dict())
    assert again.to_dict() == cfg.to_dict() and again.to_dict()["layers"] == CONFIGS["mixed"]["layers"]
    spec = cfg.to_model_spec()
    assert spec.lm_head_name == "head" and spec.embedding_name == "embed" and spec.hidden_size == 64 and spec.vocab_size == 97
    assert all(l.arrangement == "pre_norm" and l.mixer_norm["scalar"] and l.mixer_norm["eps"] == 1e-5 for l in spec.layers)
    assert spec.final_norm["scalar"] and spec.final_norm["name"] == "norm"
    assert [l.mixer.kind for l in spec.layers] == ["window_attention", "latent_attention", "window_attention", "latent_attention",
                                                   "window_attention", "window_attention"]
    assert spec.layers[2].feed_forward is None and spec.layers[2].feed_forward_norm is None and "l2.norm2" in spec.ignorable_suffixes
    a2, lat, att = spec.layers[0].mixer, spec.layers[1].mixer, spec.layers[2].mixer
    assert (a2["num_heads"], a2["num_kv_heads"], a2["head_dim"], a2["value_dim"], a2["scale"], a2["window"], a2["pool"], a2["values"],
            a2["weights"]) == (4, 2, 12, 12, 0.4, 37, 5, "keys", "sigmoid")
    assert a2["head_norm"] == {"eps": 1e-5} and a2["names"]["q_norm"] == "mix.q.norm" and a2["names"]["head_bias"] == "mix.pb"
    assert spec.layers[0].position is None
    assert (att["num_heads"], att["num_kv_heads"], att["head_dim"], att["value_dim"], att["scale"], att["window"], att.get("pool"),
            att["values"], att["weights"]) == (6, 3, 16, 20, 0.25, 70, None, "own", "softmax")
    assert att["names"]["sink"] == "mix.sink" and att["names"]["v_bias"] == "mix.v.b" and "q_norm" not in att["names"]
    pos = spec.layers[2].position
    assert (pos["head_dim"], pos["rotary_dim"], pos["theta"], pos["pairing"], pos["scaling"]) == (16, 8, 10000.0, "interleaved",
                                                                                                  {"rope_type": "linear", "factor": 3.0})
    assert spec.layers[5].position["scaling"] is None
    assert (lat["num_heads"], lat["dim"], lat["rot_dim"], lat["vdim"], lat["kv_rank"], lat["q_rank"], lat["scale"], lat["window"],
            lat["gate"], lat["own_latent"]) == (3, 8, 4, 12, 20, 24, 0.3, 50, "element", True)
    assert "sink" not in lat["names"] and spec.layers[1].position["pairing"] == "half" and spec.layers[1].position["rotary_dim"] == 4
    moe = spec.layers[0].feed_forward
    assert (moe["experts"], moe["top"], moe["expert_size"], moe["gated"], moe["activation"], moe["renormalise"], moe["shared_size"]) \
        == (6, 3, 24, False, "relu2", True, 40)
    assert spec.layers[1].feed_forward["shared_size"] is None and "shared_up" not in spec.layers[1].feed_forward["names"]


def test_values_that_are_keys_need_no_size_of_their_own():
    from kuiperllama_b200.config import config_from_dict
    c = json.loads(json.dumps(CONFIGS["only_attention_2"]))
    del c["layers"][0]["mixer"]["vdim"]
    spec = config_from_dict(c).to_model_spec()
    assert spec.layers[0].mixer["value_dim"] == spec.layers[0].mixer["head_dim"] == 12


def test_linear_scaling_divides_every_frequency():
    from kuiperllama_b200.parts.position import rotary_inverse_frequencies
    plain = rotary_inverse_frequencies(8, 10000.0, None)
    scaled = rotary_inverse_frequencies(8, 10000.0, {"rope_type": "linear", "factor": 3.0})
    assert plain == [10000.0 ** (-2.0 * i / 8) for i in range(4)]
    assert all(abs(s - p / 3.0) < 1e-15 for s, p in zip(scaled, plain))
    a = P.angles(5, {"base": 10000.0, "dims": 8, "scaling": {"factor": 3.0}})
    assert torch.allclose(a[4], torch.tensor([4 * f for f in scaled], dtype=torch.float64))


def test_faults_are_listed_together():
    from kuiperllama_b200.config import ConfigError, config_from_dict
    c = json.loads(json.dumps(CONFIGS["mixed"]))
    c["vocab"] = 0
    c["norm"] = {}
    c["layers"][0]["mixer"]["kv_heads"] = 3                        # 4 heads
    c["layers"][0]["mixer"]["vdim"] = 16                           # the values are the keys of size 12
    del c["layers"][0]["mixer"]["mask"]["pool"]
    c["layers"][1]["mixer"]["rot"]["dims"] = 6                     # a rotated part of 4
    del c["layers"][1]["mixer"]["q_rank"]
    c["layers"][2]["mixer"]["rot"]["scaling"] = {"factor": 0}
    c["layers"][3]["mlp"]["router"]["top"] = 9                     # 4 experts
    c["layers"][4]["type"] = "mamba"
    c["layers"][5]["mlp"]["kind"] = "dense"
    with pytest.raises(ConfigError) as e:
        config_from_dict(c)
    msg = str(e.value)
    for part in ('"vocab"', '"eps"', "layers[0]", '"kv_heads" 3', '"vdim" 16', '"pool"', "layers[1]", '"dims" 6', '"q_rank"', "layers[2]",
                 '"factor"', "layers[3]", '"top" 9', "layers[4]", '"type"', "layers[5]", '"kind"'):
        assert part in msg, (part, msg)


def test_cache_requests():
    """An attention with pooled blocks asks for the pooled kind, the others for a window of paged keys (the latent: one row per
    token without values), and layers with equal requests share a group."""
    from kuiperllama_b200.cache import KVRequest
    from kuiperllama_b200.parts import part_class
    from kuiperllama_b200.parts.base import Runtime
    spec = _cfg("mixed").to_model_spec()
    got = []
    for layer in spec.layers:
        cls = part_class("mixer", layer.mixer.kind)
        m = cls.__new__(cls)
        p = layer.mixer
        if layer.mixer.kind == "latent_attention":
            m.Dk, m.window = p["kv_rank"] + p["rot_dim"], p["window"]
        else:
            m.KV, m.hd, m.vd, m.window, m.pool = p["num_kv_heads"], p["head_dim"], p["value_dim"], p["window"], int(p.get("pool") or 0)
        got.append(m.kv_request())
    assert got == [KVRequest(2, 12, "pooled", 37, None, 0, 5), KVRequest(1, 24, "keys", 50), KVRequest(3, 16, "full", 70, 20),
                   KVRequest(1, 20, "keys", 33), KVRequest(1, 16, "pooled", 8, None, 0, 20), KVRequest(2, 8, "full", 200)]


def test_pooled_cache_pages():
    """The pooled kind on the host: a block's positions stay in their pages until the block is complete, also where the window is
    shorter than a block; one row of means per complete block, in pages of a second pool; everything goes back at the end."""
    from kuiperllama_b200.cache import KVRequest, SequenceCache
    req = KVRequest(kv_heads=2, head_dim=4, kind="pooled", window=10, pool=100)
    cache = SequenceCache([req], [None], [None], max_tokens=64 * 40, max_seq_len=64 * 40, dtype=torch.float32, device="cpu", max_slots=2)
    g = cache.groups[0]
    k, v, table, pooled = g.view(0)
    assert pooled.pool == 100 and pooled.k.dtype == torch.float32 and tuple(pooled.k.shape[1:]) == (2, 64, 4) and pooled.v.shape == pooled.k.shape
    s = cache.alloc_slot()
    length = 0
    for new in (30, 60, 9, 1, 1, 150, 1):                               # 99 tokens, then the block's last, then more
        cache.reserve(s, length + new)
        cache.lengths[s] = length = length + new
        first_held = next(b for b, p in enumerate(g.slot_pages[s]) if p >= 0)
        # at the start of the next step every position of the incomplete block and of the window is still there
        needed = min(max(0, length - 10 + 1), length // 100 * 100)
        assert first_held * 64 <= needed, (length, first_held)
    assert len(g.pool_slot_pages[s]) == 1 and g.first_needed(251) == 200 and g.first_needed(299) == 200 and g.first_needed(305) == 296
    cache.reserve(s, 2500)
    assert len(g.pool_slot_pages[s]) == 1                               # 25 rows: one page of 64
    t = cache.alloc_slot()
    cache.reserve(t, 130)
    assert g.pool_slot_pages[t] != g.pool_slot_pages[s] and g.pool_pages.held() == 2
    cache.free_slot(s)
    cache.free_slot(t)
    assert g.held() == 0 and g.pool_pages.held() == 0 and cache.slots.held() == 0
    # token by token, asking for room only where the cache says a token needs new storage: a page of keys, or a page of means
    for pool in (1, 3, 64, 100):
        cache = SequenceCache([KVRequest(1, 4, "pooled", 5, None, 0, pool)], [None], [None], 64 * 80, 64 * 80, torch.float32, "cpu", max_slots=1)
        g, s = cache.groups[0], cache.alloc_slot()
        for length in range(64 * 70):
            if cache.grows_at(s):
                cache.reserve(s, length + 1)
            cache.lengths[s] = length + 1
            assert len(g.slot_pages[s]) * 64 >= length + 1 and len(g.pool_slot_pages[s]) * 64 >= (length + 1) // pool, (pool, length)
    with pytest.raises(Exception):
        SequenceCache([KVRequest(1, 4, "pooled", None, None, 0, 4)], [None], [None], 640, 640, torch.float32, "cpu")


# ----------------------------------------------------------------------------- the plain implementation against hand values

def test_plain_norm_and_rotations():
    x = torch.tensor([[3.0, 4.0, 0.0, 0.0]], dtype=torch.float64)
    assert torch.allclose(P.scalar_rms_norm(x, 2.0, 0.0), x / 2.5 * 2.0)
    assert torch.allclose(P.scalar_rms_norm(x, 1.0, 6.25), x / math.sqrt(12.5))
    rot = {"base": 100.0, "dims": 4}
    v = torch.tensor([[[1.0, 0.0, 0.0, 1.0, 5.0, 6.0]], [[1.0, 0.0, 0.0, 1.0, 5.0, 6.0]]], dtype=torch.float64)     # positions 0 and 1
    inter, half = P.rotate(v, rot, "interleaved"), P.rotate(v, rot, "half")
    assert torch.equal(inter[0], v[0]) and torch.equal(half[0], v[0])
    c0, s0, c1, s1 = math.cos(1.0), math.sin(1.0), math.cos(0.1), math.sin(0.1)
    assert torch.allclose(inter[1, 0], torch.tensor([c0, s0, -s1, c1, 5.0, 6.0], dtype=torch.float64))      # pairs (0, 1) and (2, 3)
    assert torch.allclose(half[1, 0], torch.tensor([c0, -s1, s0, c1, 5.0, 6.0], dtype=torch.float64))       # pairs (0, 2) and (1, 3)


def test_plain_window_sink_and_pooled_blocks():
    m = P.window_mask(6, 3)
    assert m[5].tolist() == [False, False, False, True, True, True] and m[1].tolist() == [True, True, False, False, False, False]
    # equal scores over a window of 3 with a sink of the same size: four equal shares, one of them without a value
    p = P.softmax_with_sink(torch.zeros(1, 6, 6, dtype=torch.float64), m, torch.zeros(1, dtype=torch.float64))
    assert torch.allclose(p[0, 5, 3:], torch.full((3,), 0.25, dtype=torch.float64)) and float(p[0, 5, :3].sum()) == 0.0
    assert torch.allclose(p[0, 0, 0], torch.tensor(0.5, dtype=torch.float64))
    x = torch.arange(14, dtype=torch.float64).reshape(7, 1, 2)
    b = P.pooled_blocks(x, 3)
    assert b.shape == (2, 1, 2) and torch.allclose(b[:, 0, 0], torch.tensor([2.0, 8.0], dtype=torch.float64))
    # keys and values of one head that make every score 0: each seen token and block weighs sigmoid(b) = 1/2
    n, W, Pp = 12, 4, 3
    w = {"q": torch.zeros(2, 2, dtype=torch.float64), "k": torch.eye(2, dtype=torch.float64), "q.norm": torch.ones(2, dtype=torch.float64),
         "k.norm": torch.ones(2, dtype=torch.float64), "pb": torch.zeros(1, dtype=torch.float64), "o": torch.eye(2, dtype=torch.float64)}
    h = torch.zeros(n, 2, dtype=torch.float64)
    h[:, 0] = 1.0                                                          # every value is (1, 0)
    out = P.attention_pooled_sigmoid(h, {"heads": 1, "kv_heads": 1, "dim": 2, "scale": 1.0, "mask": {"size": W, "pool": Pp}}, w, 1e-6)
    # position i sees min(i + 1, 4) tokens and the blocks b with 3 b + 2 <= i - 4
    seen = [min(i + 1, W) + sum(1 for b in range(n // Pp) if b * Pp + Pp - 1 <= i - W) for i in range(n)]
    assert seen == [1, 2, 3, 4, 4, 4, 5, 5, 5, 6, 6, 6]
    assert torch.allclose(out[:, 0], torch.tensor(seen, dtype=torch.float64) * 0.5)


def test_plain_router_and_experts():
    h = torch.tensor([[1.0, 0.0], [0.0, 1.0]], dtype=torch.float64)
    router = torch.tensor([[1.0, 0.0], [2.0, 0.0], [0.0, 3.0], [2.0, 3.0]], dtype=torch.float64)
    bias = torch.tensor([0.0, 0.0, 0.0, -5.0], dtype=torch.float64)
    choice, weight = P.route(h, router, bias, 2)
    assert choice.tolist() == [[1, 0], [2, 0]]                           # logits [1, 2, 0, -3] and [0, 0, 3, -2]: the lower index among equals
    assert torch.allclose(weight[0], torch.softmax(torch.tensor([2.0, 1.0], dtype=torch.float64), 0))
    assert torch.allclose(weight[1], torch.softmax(torch.tensor([3.0, 0.0], dtype=torch.float64), 0))
    up = torch.tensor([[1.0, 0.0], [-1.0, 0.0]], dtype=torch.float64)
    down = torch.tensor([[1.0, 1.0], [0.0, 2.0]], dtype=torch.float64)
    assert torch.allclose(P.relu2_expert(torch.tensor([[3.0, 7.0]], dtype=torch.float64), up, down), torch.tensor([[9.0, 0.0]], dtype=torch.float64))
