"""Seeded random Dofevik configurations (width, head counts, key and value sizes, ranks, windows, blocks, rotated dimensions and
their scaling, experts, shared experts, scales, layer order: every size and constant config.json carries) through the framework
against the plain implementation: a whole prompt, a prompt followed by single tokens, and two unequal requests in one batch
decoded together, in float32 and bfloat16.  The prompts are longer than most of the drawn windows, so windows and pooled blocks
act in the prompt and in decoding."""
from __future__ import annotations

import random

import pytest
import torch

from dofevik_helpers import assert_logits, oracle_logits, random_weights, tokens, write_folder

pytestmark = pytest.mark.gpu
N_CONFIGS = 14


def random_config(seed: int) -> dict:
    r = random.Random(seed)
    width = r.choice([40, 64, 96, 100, 160, 256])
    layers = []
    for _ in range(r.randint(2, 6)):
        if r.random() < 0.75:
            experts = r.randint(1, 12)
            mlp = {"kind": "moe", "router": {"experts": experts, "top": r.randint(1, min(experts, 5))},
                   "expert": {"ff": r.choice([8, 24, 32, 64, 96])}}
            if r.random() < 0.6:
                mlp["shared"] = {"ff": r.choice([8, 20, 64, 128])}
        else:
            mlp = None
        size = r.choice([1, 2, 7, 31, 32, 33, 64, 65, 80, 200])
        kind = r.choice(["attention", "attention_2", "latent_attention"])
        if kind == "latent_attention":
            dim, rot_dim = r.choice([4, 8, 16, 24, 32, 64]), r.choice([2, 4, 8, 16, 32])
            m = {"heads": r.randint(1, 6), "dim": dim, "rot_dim": rot_dim, "vdim": r.choice([4, 8, 12, 16, 32, 64]),
                 "kv_rank": r.choice([5, 8, 16, 24, 48, 96]), "q_rank": r.choice([6, 8, 16, 40, 64]),
                 "scale": round(r.uniform(0.5, 2.0) / (dim + rot_dim) ** 0.5, 4), "mask": {"size": size},
                 "rot": {"base": r.choice([100.0, 10000.0, 500000.0]), "dims": rot_dim}}
        else:
            kv = r.choice([1, 2, 3, 4])
            dim = r.choice([2, 8, 12, 16, 24, 32, 64, 128])
            m = {"heads": kv * r.randint(1, 4), "kv_heads": kv, "dim": dim, "scale": round(r.uniform(0.5, 2.0) / dim ** 0.5, 4)}
            if kind == "attention":
                m["vdim"] = r.choice([dim, 4, 8, 20, 32, 64])
                m["mask"] = {"size": size}
                m["rot"] = {"base": r.choice([50.0, 10000.0, 1000000.0]), "dims": r.choice([d for d in (2, 4, 8, 16, dim) if d <= dim and d % 2 == 0])}
                if r.random() < 0.6:
                    m["rot"]["scaling"] = {"factor": r.choice([1.5, 2.0, 3.0, 4.0, 8.0])}
            else:
                m["vdim"] = dim
                m["mask"] = {"size": size, "pool": r.choice([1, 2, 3, 5, 8, 16, 32, 64, 100])}
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    return {"architecture": "Dofevik", "vocab": r.randint(50, 700), "width": width, "norm": {"eps": r.choice([1e-6, 1e-5, 1e-4])}, "layers": layers}


@pytest.mark.parametrize("seed", range(N_CONFIGS))
def test_random_configuration(seed, tmp_path_factory):
    from kuiperllama_b200.engine import Engine, SequenceInput, load_model
    c = random_config(3000 + seed)
    folder = write_folder(str(tmp_path_factory.mktemp(f"dofevik-random-{seed}")), c, random_weights(c, seed))
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
