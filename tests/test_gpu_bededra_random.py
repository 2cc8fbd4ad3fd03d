"""Seeded random Bededra configurations (width, head counts, key and value sizes, states, groups, windows, kept tokens, taps,
experts and their groups, scales, layer order: every size and constant config.json carries) through the framework against
the plain implementation: a whole prompt, a prompt followed by single tokens, and two unequal requests in one batch decoded
together, in float32 and bfloat16.  The prompts are longer than most of the drawn windows, so windows and kept tokens act in
the prompt and in decoding."""
from __future__ import annotations

import random

import pytest
import torch

from bededra_helpers import assert_logits, oracle_logits, random_weights, tokens, write_folder

pytestmark = pytest.mark.gpu
N_CONFIGS = 12


def random_config(seed: int) -> dict:
    r = random.Random(seed)
    width = r.choice([40, 64, 96, 100, 160, 256])
    layers = []
    for _ in range(r.randint(2, 5)):
        kind = r.choice([None, "dense", "moe", "moe"])
        if kind == "dense":
            mlp = {"kind": "dense", "ff": r.choice([24, 72, 128, 320])}
        elif kind == "moe":
            count = r.choice([1, 1, 2, 3, 4])
            per = r.randint(1, 5)
            keep = r.randint(1, count)
            router = {"experts": count * per, "top": r.randint(1, min(keep * per, 5))}
            if count > 1 or r.random() < 0.5:
                router["groups"] = {"count": count, "keep": keep}
            mlp = {"kind": "moe", "router": router, "expert": {"ff": r.choice([8, 24, 32, 64, 96])}}
        else:
            mlp = None
        if r.random() < 0.4:
            groups = r.choice([1, 2, 3])
            heads = groups * r.randint(1, 4)
            vdim = r.choice([4, 8, 12, 16, 32, 64])
            parts = r.choice([d for d in (1, 2, 3, 4, heads) if (heads * vdim) % d == 0])
            layers.append({"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": r.choice([4, 9, 16, 24, 64, 128]),
                                                     "groups": groups, "conv": r.randint(1, 5), "norm_groups": parts}, "mlp": mlp})
            continue
        kv = r.choice([1, 2, 3, 4])
        dim = r.choice([8, 12, 16, 24, 32, 64])
        left = {"heads": kv * r.randint(1, 4), "kv_heads": kv, "dim": dim, "vdim": r.choice([8, 12, 16, 24, 32, 64]),
                "scale": round(r.uniform(0.5, 2.0) / dim ** 0.5, 4), "softcap": r.choice([None, 5.0, 20.0, 50.0])}
        if r.random() < 0.8:
            left["mask"] = {"size": r.choice([1, 2, 7, 31, 32, 33, 64, 65, 80]), "keep_first": r.choice([0, 0, 1, 3, 16, 63, 64, 70])}
        right = {"heads": r.randint(1, 6), "dim": r.choice([4, 8, 12, 16, 32, 64]), "vdim": r.choice([4, 8, 12, 16, 32, 64]),
                 "tau": r.choice([1.0, 2.5, 8.0, 16.0]), "rank": r.choice([1, 3, 8, 16])}
        layers.append({"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": round(r.uniform(-1.5, 1.5), 2),
                                                     "right_scale": round(r.uniform(0.3, 1.5), 2)}, "mlp": mlp})
    return {"architecture": "Bededra", "vocab": r.randint(50, 700), "width": width, "norm": {"eps": r.choice([1e-6, 1e-5, 1e-4])},
            "canon": {"taps": r.randint(1, 5)}, "layers": layers}


@pytest.mark.parametrize("seed", range(N_CONFIGS))
def test_random_configuration(seed, tmp_path_factory):
    from kuiperllama_b200.engine import Engine, SequenceInput, load_model
    c = random_config(2000 + seed)
    folder = write_folder(str(tmp_path_factory.mktemp(f"bededra-random-{seed}")), c, random_weights(c, seed))
    V = c["vocab"]
    a, b = tokens(90, V, seed=seed), tokens(37, V, seed=seed + 500)
    ref_a, ref_b = oracle_logits(folder, a), oracle_logits(folder, b)
    what = f"random {seed}"
    for dtype in ("float32", "bfloat16"):
        with torch.inference_mode():
            model = load_model(folder, dtype=dtype, device="cuda:0")
            eng = Engine(model, model.new_cache(max_tokens=64 * 8))
            inp = lambda slot, toks: SequenceInput(slot, list(toks), list(range(len(toks))))
            s = eng.alloc_slot()
            assert_logits(eng.step([inp(s, a)]), ref_a, dtype, f"{what}: whole")
            eng.free_slot(s)
            s = eng.alloc_slot()
            rows = [eng.step([inp(s, a[:61])]).clone()] + [eng.step([inp(s, [t])]).clone() for t in a[61:]]
            assert_logits(torch.cat(rows), ref_a, dtype, f"{what}: prompt, then tokens")
            eng.free_slot(s)
            s, t = eng.alloc_slot(), eng.alloc_slot()
            first = eng.step([inp(s, a[:70]), inp(t, b[:3])])
            ra, rb = [first[:70].clone()], [first[70:].clone()]
            for k in range(20):
                out = eng.step([inp(s, [a[70 + k]]), inp(t, [b[3 + k]])])
                ra.append(out[:1].clone())
                rb.append(out[1:].clone())
            eng.free_slot(s)
            for k in range(23, 37):                                       # the longer-lived request goes on alone
                rb.append(eng.step([inp(t, [b[k]])]).clone())
            eng.free_slot(t)
            assert_logits(torch.cat(ra), ref_a, dtype, f"{what}: in a batch, first request")
            assert_logits(torch.cat(rb), ref_b, dtype, f"{what}: in a batch, second request")
        eng.check_device_errors()
