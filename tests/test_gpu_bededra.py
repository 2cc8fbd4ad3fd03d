"""The Bededra decoder through the framework's own loader, cache, step function and generation loop,
against the plain implementation (tests/plain_bededra.py), in float32 and bfloat16.

The float32 runs are the sharp ones: they differ from the plain implementation only by the order of sums,
so a key that is missed, a window that is one token off, a state that is lost or a tap that reads the wrong
token shows at once.  The configurations are in bededra_helpers.py.
"""
from __future__ import annotations

import json
import math

import pytest
import torch

import plain_bededra as P
from bededra_helpers import CONFIGS, assert_logits, oracle_logits, random_weights, read_folder, tokens, write_folder

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
FULL = ["mixed", "odd", "wide"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name: str, seed: int = 0, gain: float = 1.0) -> str:
        key = (name, seed, gain)
        if key not in made:
            c = CONFIGS[name]
            made[key] = write_folder(str(tmp_path_factory.mktemp(f"bededra-{name}")), c, random_weights(c, seed, gain))
        return made[key]

    return get


@pytest.fixture(scope="module")
def models(folders):
    from kuiperllama_b200.engine import load_model
    made = {}

    def get(name: str, dtype: str, **kw):
        key = (name, dtype, tuple(sorted(kw.items())))
        if key not in made:
            folder = folders(name, **kw)
            with torch.inference_mode():
                made[key] = (load_model(folder, dtype=dtype, device="cuda:0"), folder)
        return made[key]

    return get


def _engine(model, max_tokens=64 * 16, use_graphs=False):
    from kuiperllama_b200.engine import Engine
    return Engine(model, model.new_cache(max_tokens=max_tokens), use_graphs=use_graphs)


def _inputs(slot, toks, want=None):
    from kuiperllama_b200.engine import SequenceInput
    return SequenceInput(slot, list(toks), list(range(len(toks))) if want is None else want)


def _run_in_steps(engine, toks, cuts):
    """One sequence fed in steps of the given sizes; logits of every token."""
    rows, at = [], 0
    with torch.inference_mode():
        slot = engine.alloc_slot()
        for n in cuts:
            rows.append(engine.step([_inputs(slot, toks[at:at + n])]).clone())
            at += n
        engine.free_slot(slot)
    assert at == len(toks)
    engine.check_device_errors()
    return torch.cat(rows)


def _step(starts, news, dev="cuda:0"):
    """A ragged step of len(starts) sequences in slots 0, 1, ...: sequence s brings news[s] tokens from position starts[s]."""
    from kuiperllama_b200.parts.base import StepContext
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    cu = [0]
    for k in news:
        cu.append(cu[-1] + k)
    pos = i32([st + i for st, k in zip(starts, news) for i in range(k)])
    tslot = i32([sl for sl, k in enumerate(news) for _ in range(k)])
    slots = list(range(len(starts)))
    return StepContext(n_tokens=cu[-1], n_seqs=len(starts), token_ids=pos, positions=pos, token_slot=tslot, seq_slots=i32(slots),
                       seq_starts=i32(starts), seq_new=i32(news), cu_tokens=i32(cu), is_decode=max(news) == 1, max_new=max(news),
                       max_context=max(a + b for a, b in zip(starts, news)), host_slots=slots, host_starts=list(starts), host_new=list(news))


# ----------------------------------------------------------------------------- each mechanism alone

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["only_ssm", "only_parallel", "only_moe", "only_dense"])
def test_one_mechanism_alone(models, name, dtype):
    model, folder = models(name, dtype, seed=3)
    toks = tokens(70, CONFIGS[name]["vocab"], seed=11)
    ref = oracle_logits(folder, toks)
    assert_logits(_run_in_steps(_engine(model), toks, [70]), ref, dtype, f"{name}: whole")
    assert_logits(_run_in_steps(_engine(model), toks, [1] * 70), ref, dtype, f"{name}: token by token")


def test_the_stream_after_every_layer(models):
    """float32: the residual stream after each layer against the plain implementation's, so that a fault is named by its layer."""
    from kuiperllama_b200.csrc import ops
    from kuiperllama_b200.parts.norm import add_to_stream
    for name in ("mixed", "wide"):
        model, folder = models(name, "float32", seed=1)
        c, W = read_folder(folder)
        toks = tokens(90, c["vocab"], seed=12)
        _, streams = P.forward(W, c, toks, return_layers=True)
        eng = _engine(model)
        with torch.inference_mode():
            slot = eng.alloc_slot()
            ctx, _, _ = eng._pack([_inputs(slot, toks)], 0)
            residual = torch.empty((ctx.n_tokens, c["width"]), dtype=torch.float32, device="cuda:0")
            ops.embedding(ctx.token_ids[:ctx.n_tokens], model.embedding, residual, model.error_flag)
            pending = None
            for i, e in enumerate(model.spec.schedule):
                ctx.next_norm = None
                residual, pending = model.blocks[e.layer].forward(residual, pending, ctx, eng.cache.view(i))
                x = residual.clone()
                add_to_stream(x, pending)
                a, b = x[:90].double().cpu(), streams[i]
                assert float((a - b).abs().max()) <= 1e-4 * float(b.abs().max()), f"{name}: the stream after layer {i} differs"
            eng.free_slot(slot)


def test_router_groups_top_and_weights():
    """Scores over all experts; a group's score is its largest; only the kept groups' experts can be chosen; the largest first,
    the lower index among equals; weights divided by their sum + 1e-20."""
    from kuiperllama_b200.csrc import ops
    g = torch.Generator().manual_seed(4)
    for E, top, groups, keep in ((12, 2, 2, 1), (12, 4, 3, 2), (16, 4, 4, 4), (7, 3, 1, 1), (40, 5, 8, 3), (6, 6, 2, 2), (9, 1, 9, 1), (9, 3, 3, 1)):
        z = torch.randn(41, E, generator=g) * 2
        z[3, :] = 0.25                                                     # all equal: the first groups, the first experts
        z[5, E - 1] = 30.0                                                 # one expert far ahead: its group is kept whatever else it holds
        choice, weight = ops.moe_route(z.cuda(), top, True, groups, keep, 1e-20)
        s = torch.softmax(z.double(), dim=-1)
        for t in range(41):
            want = P.route(s[t], top, groups, keep)
            assert choice[t].tolist() == want, (E, top, groups, keep, t)
            w = s[t][want] / (s[t][want].sum() + 1e-20)
            assert torch.allclose(weight[t].cpu().double(), w, atol=1e-6, rtol=1e-5)
        assert (E - 1) in choice[5].tolist()


@pytest.mark.parametrize("dtype", DTYPES)
def test_short_convolution_over_ragged_steps(dtype):
    """The convolution alone: a step of three sequences (one continues from state, one is shorter than the taps, one is new), with
    and without the input added, bias and SiLU; then the state it leaves, read by a second step."""
    from kuiperllama_b200.csrc import ops
    dt, dev = getattr(torch, dtype), "cuda:0"
    g = torch.Generator().manual_seed(6)
    for C, taps in ((40, 4), (7, 1), (130, 5), (64, 2)):
        w, b = torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
        seqs = [torch.randn(n, C, generator=g).to(dt) for n in (23, 2, 9)]
        state = torch.zeros(3, (taps - 1) * C + 3, device=dev)                      # wider rows than needed: the stride is the row's
        outs = [[], [], []]
        for add, silu, bias in ((True, False, None), (False, True, b)):
            state.zero_()
            got = [[], [], []]
            for cut in ((10, 1, 4), (13, 1, 5)):
                first = cut == (10, 1, 4)
                at = [0, 0, 0] if first else [10, 1, 4]
                x = torch.cat([s[a:a + n] for s, a, n in zip(seqs, at, cut)]).to(dev)
                out = torch.empty(x.shape[0], C, dtype=torch.float32, device=dev)
                ops.short_conv(x, w.to(dev), None if bias is None else bias.to(dev), state, _step(at, list(cut)), out, add_input=add, silu=silu)
                o = 0
                for i, n in enumerate(cut):
                    got[i].append(out[o:o + n].cpu().double())
                    o += n
            for i, s in enumerate(seqs):
                want = P.causal_conv(s.double(), w.double())
                want = want + (s.double() if add else 0) + (bias.double() if bias is not None else 0)
                want = P.silu(want) if silu else want
                assert torch.allclose(torch.cat(got[i]), want, atol=1e-5, rtol=1e-5), (C, taps, add, i)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, G, N, Pd, per_row", [(6, 2, 12, 8, False), (3, 3, 20, 16, False), (4, 4, 8, 16, True), (5, 5, 33, 10, True),
                                                   (8, 2, 64, 64, False), (2, 2, 128, 48, True), (1, 1, 1, 1, True), (2, 1, 300, 4, False),
                                                   (2, 2, 40, 7, True)])
def test_matrix_state_recurrence_over_ragged_steps(dtype, H, G, N, Pd, per_row):
    """S_t = diag(a_t) S_(t-1) + (c_t k_t) v_t^T, y_t = S_t^T q_t + D v_t alone: one decay per head or one per row of the state,
    keys and queries shared by groups of heads, three sequences cut differently into two steps, then one token each."""
    from kuiperllama_b200.csrc import ops
    dt, dev = getattr(torch, dtype), "cuda:0"
    g = torch.Generator().manual_seed(H * 100 + N)
    lens = (70, 3, 29)
    q = [torch.randn(n, G, N, generator=g).to(dt) for n in lens]
    k = [torch.randn(n, G, N, generator=g).to(dt) for n in lens]
    v = [torch.randn(n, H, Pd, generator=g).to(dt) for n in lens]
    a = [torch.rand(n, H, N if per_row else 1, generator=g) * 0.5 + 0.5 for n in lens]
    c = None if per_row else [torch.rand(n, H, generator=g) + 0.1 for n in lens]
    skip = None if per_row else torch.randn(H, generator=g)
    state = torch.zeros(3, H * N * Pd + 5, device=dev)
    got = [[], [], []]
    at = [0, 0, 0]
    for cut in ((40, 1, 2), (29, 1, 26), (1, 1, 1)):
        cat = lambda parts: torch.cat([p[s:s + n].reshape(n, -1) for p, s, n in zip(parts, at, cut)]).to(dev).contiguous()
        y = torch.empty(sum(cut), H * Pd, dtype=torch.float32, device=dev)
        ops.outer_recurrence(cat(q), cat(k), cat(v), cat(a), state, y, _step(at, list(cut)), H, G, N, Pd,
                             c=None if c is None else cat(c), skip=None if skip is None else skip.to(dev), q_scale=0.5)
        o = 0
        for i, n in enumerate(cut):
            got[i].append(y[o:o + n].cpu().double())
            o += n
        at = [s + n for s, n in zip(at, cut)]
    assert at == list(lens)
    per = H // G
    for i, n in enumerate(lens):
        S = torch.zeros(H, N, Pd, dtype=torch.float64)
        want = torch.zeros(n, H, Pd, dtype=torch.float64)
        for t in range(n):
            for h in range(H):
                kk = k[i][t, h // per].double() * (1.0 if c is None else float(c[i][t, h]))
                S[h] = a[i][t, h].double()[:, None] * S[h] + torch.outer(kk, v[i][t, h].double())
                want[t, h] = S[h].T @ (q[i][t, h // per].double() * 0.5) + (0.0 if skip is None else float(skip[h])) * v[i][t, h].double()
        assert torch.allclose(torch.cat(got[i]).reshape(n, H, Pd), want, atol=2e-4, rtol=2e-4), (i, n)
        assert torch.allclose(state[i, :H * N * Pd].cpu().double().reshape(H, N, Pd), S, atol=2e-4, rtol=2e-4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, G, d, dv, window, keep", [(4, 2, 12, 20, 40, 5), (6, 6, 8, 8, 70, 0), (3, 1, 16, 12, 0, 0), (8, 2, 64, 32, 96, 16),
                                                        (16, 4, 32, 48, 130, 64), (2, 1, 16, 16, 64, 64), (5, 5, 10, 6, 1, 3)])
@pytest.mark.parametrize("tiled, splits", [(None, None), (None, 1), (None, 3), (False, None)])
def test_mixed_head_attention_on_scattered_pages(dtype, H, G, d, dv, window, keep, tiled, splits):
    """The attention kernels alone (the tiled one with its own choice of pieces for single tokens, with one piece and with
    three, and the plain one) against the plain weights: prompts of unequal lengths on scattered pages, portions that start
    inside a page and inside the window, single tokens; soft cap, distance bias, mixing matrix and gate on and off."""
    from kuiperllama_b200.csrc import ops
    dt, dev = getattr(torch, dtype), "cuda:0"
    g = torch.Generator().manual_seed(H * 10 + d)
    T = 256
    table = torch.tensor([[5, 2, 9, 0], [1, 7, 3, 11], [4, 6, 8, 10]], dtype=torch.int32, device=dev)
    ks = [torch.randn(T, G, d, generator=g).to(dt) for _ in range(3)]
    vs = [torch.randn(T, G, dv, generator=g).to(dt) for _ in range(3)]
    qs = [(torch.randn(T, H, d, generator=g) * 1.5).to(dt) for _ in range(3)]
    gates = [torch.randn(T, H, generator=g).to(dt) for _ in range(3)]
    kc = torch.zeros(12, G, 64, d, dtype=dt, device=dev)
    vc = torch.zeros(12, G, 64, dv, dtype=dt, device=dev)
    for s in range(3):
        for p in range(T):
            kc[int(table[s, p // 64]), :, p % 64] = ks[s][p].to(dev)
            vc[int(table[s, p // 64]), :, p % 64] = vs[s][p].to(dev)
    r1, r2 = torch.rand(H, generator=g) * 0.5 + 0.1, torch.rand(H, generator=g) + 0.05
    talk = torch.eye(H) + 0.4 * torch.randn(H, H, generator=g)
    m = {"scale": 0.3, "softcap": 7.0}
    if window:
        m["mask"] = {"size": window, "keep_first": keep}
    tol = 2e-5 if dtype == "float32" else 3e-2
    for full in (True, False):
        mm = dict(m) if full else dict(m, softcap=None)
        rr1, rr2, tk = (r1, r2, talk) if full else (None, None, None)
        want = []
        for s in range(3):
            _, w = P.mixed_attention_weights(qs[s].double(), ks[s].double(), mm, rr1, rr2, None if tk is None else tk.double())
            o = torch.einsum("hij,jhd->ihd", w, vs[s].double().repeat_interleave(H // G, dim=1))
            want.append(o * (torch.sigmoid(gates[s].double())[..., None] if full else 1.0) * 1.25)
        for starts, news in (([0, 0, 0], [256, 1, 67]), ([100, 63, 200], [30, 2, 56]), ([150, 64, 255], [1, 1, 1]), ([0, 39, 129], [3, 110, 127])):
            step = _step(starts, news)
            rows = lambda parts: torch.cat([p[a:a + n].reshape(n, -1) for p, a, n in zip(parts, starts, news)]).to(dev).contiguous()
            out = torch.full((step.n_tokens, H * dv), 9.0, dtype=dt, device=dev)
            ops.attention_mixed(rows(qs), rows(gates) if full else None, out, kc, vc, table, step, H, G, d, dv, 0.3, 7.0 if full else 0.0,
                                None if rr1 is None else rr1.to(dev), None if rr2 is None else rr2.to(dev), None if tk is None else tk.to(dev),
                                window, keep, 1.25, tiled=tiled, splits=splits)
            ref = rows(want).to("cpu")
            assert torch.allclose(out.cpu().double(), ref, atol=tol, rtol=tol), (full, starts, news, float((out.cpu().double() - ref).abs().max()))


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_over_parts_with_the_gate_before_or_after(dtype):
    from kuiperllama_b200.csrc import ops
    dt, dev = getattr(torch, dtype), "cuda:0"
    g = torch.Generator().manual_seed(9)
    for heads, dim, wide in ((3, 16, True), (1, 48, True), (5, 10, False), (4, 64, False), (2, 96, True)):
        x, gate = torch.randn(37, heads * dim, generator=g) * 3, torch.randn(37, heads * dim, generator=g).to(dt)
        w = 1 + 0.2 * torch.randn(heads * dim if wide else dim, generator=g)
        for first in (True, False):
            out = torch.empty(37, heads * dim, dtype=dt, device=dev)
            ops.head_rmsnorm_gate(x.to(dev), gate.to(dev), w.to(dev), out, heads, dim, 1e-5, gate_first=first, out_scale=0.7)
            xs, gs = x.double().reshape(37, heads, dim), P.silu(gate.double()).reshape(37, heads, dim)
            ww = w.double().reshape(heads, dim) if wide else w.double()
            want = (P.rms_norm(xs * gs, None, 1e-5) * ww if first else P.rms_norm(xs, None, 1e-5) * ww * gs) * 0.7
            tol = 1e-5 if dtype == "float32" else 2e-2
            assert torch.allclose(out.cpu().double().reshape(37, heads, dim), want, atol=tol, rtol=tol), (heads, dim, wide, first)


# ----------------------------------------------------------------------------- cuts, batches, reuse

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", FULL)
def test_whole_prompt_portions_and_single_tokens(models, name, dtype):
    model, folder = models(name, dtype, seed=1)
    toks = tokens(150, CONFIGS[name]["vocab"], seed=21)
    ref = oracle_logits(folder, toks)
    for cuts in ([150], [118] + [1] * 32, [2] * 75, [63, 1, 2, 62, 3, 1, 1, 17], [1, 64, 64, 21], [5, 59, 2, 84]):
        assert sum(cuts) == 150
        assert_logits(_run_in_steps(_engine(model), toks, cuts), ref, dtype, f"{name}: steps of {cuts[:6]}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_long_prompts(models, name, dtype):
    """Prompts of several hundred tokens (the forms of the kernels that long steps take), a long portion after a short one and
    before one, and a long prompt beside a short one in one step."""
    model, folder = models(name, dtype, seed=1)
    V = CONFIGS[name]["vocab"]
    toks = tokens(330, V, seed=41)
    ref = oracle_logits(folder, toks)
    for cuts in ([330], [300, 30], [31, 299], [129, 130, 71]):
        assert_logits(_run_in_steps(_engine(model), toks, cuts), ref, dtype, f"{name}: long steps of {cuts}")
    short = tokens(70, V, seed=42)
    eng = _engine(model)
    with torch.inference_mode():
        a, b = eng.alloc_slot(), eng.alloc_slot()
        out = eng.step([_inputs(a, short), _inputs(b, toks)])
    eng.check_device_errors()
    assert_logits(out[:70], oracle_logits(folder, short), dtype, f"{name}: a short prompt beside a long one")
    assert_logits(out[70:], ref, dtype, f"{name}: a long prompt beside a short one")


@pytest.mark.parametrize("use_graphs", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", FULL)
def test_unequal_batches_against_each_alone(models, name, dtype, use_graphs):
    """Requests of 1 to 130 tokens in one step, then decoded together, the shorter ones leaving first."""
    model, folder = models(name, dtype, seed=1)
    V = CONFIGS[name]["vocab"]
    lens, more = [1, 3, 70, 130, 64], [2, 9, 5, 9, 7]
    seqs = [tokens(n + m, V, seed=30 + i) for i, (n, m) in enumerate(zip(lens, more))]
    refs = [oracle_logits(folder, s) for s in seqs]
    eng = _engine(model, max_tokens=64 * 12, use_graphs=use_graphs)
    with torch.inference_mode():
        slots = [eng.alloc_slot() for _ in seqs]
        got = [[] for _ in seqs]
        out = eng.step([_inputs(sl, s[:n]) for sl, s, n in zip(slots, seqs, lens)])
        at = 0
        for i, n in enumerate(lens):
            got[i].append(out[at:at + n].clone())
            at += n
        for k in range(max(more)):
            live = [i for i in range(len(seqs)) if k < more[i]]
            if use_graphs:
                out = eng.decode_step([slots[i] for i in live], [seqs[i][lens[i] + k] for i in live]).clone()
            else:
                out = eng.step([_inputs(slots[i], [seqs[i][lens[i] + k]]) for i in live])
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1].clone())
            for i in live:
                if k + 1 == more[i]:
                    eng.free_slot(slots[i])
    eng.check_device_errors()
    for i in range(len(seqs)):
        assert_logits(torch.cat(got[i]), refs[i], dtype, f"{name}: request {i} of the batch")
    assert eng.cache.slots.held() == 0 and all(h == 0 for h in eng.cache.pages_held())


@pytest.mark.parametrize("dtype", DTYPES)
def test_slots_and_pages_are_reused(models, dtype):
    """A cache with room for little: four rounds of requests on the same slots and pages, whose old contents (keys and values,
    both recurrent states, both convolutions' inputs) must not leak into the next request."""
    model, folder = models("mixed", dtype, seed=1)
    V = CONFIGS["mixed"]["vocab"]
    eng = _engine(model, max_tokens=64 * 5)
    for rnd in range(4):
        lens = [[100, 70], [3, 129], [64, 65], [1, 2]][rnd]
        seqs = [tokens(n + 3, V, seed=50 + 10 * rnd + i) for i, n in enumerate(lens)]
        with torch.inference_mode():
            slots = [eng.alloc_slot() for _ in seqs]
            first = eng.step([_inputs(sl, s[:n]) for sl, s, n in zip(slots, seqs, lens)])
            rest = [eng.step([_inputs(sl, [s[n + k]]) for sl, s, n in zip(slots, seqs, lens)]).clone() for k in range(3)]
            for sl in slots:
                eng.free_slot(sl)
        at = 0
        for i, (s, n) in enumerate(zip(seqs, lens)):
            got = torch.cat([first[at:at + n]] + [r[i:i + 1] for r in rest])
            at += n
            assert_logits(got, oracle_logits(folder, s), dtype, f"round {rnd}, request {i}")
    eng.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_the_first_tokens_of_a_sequence(models, name, dtype):
    """Prompts shorter than the convolutions' taps, a prompt of one token, and what follows token by token: the states start at
    zero, the first token takes no other path, and taps before the start read zeros."""
    model, folder = models(name, dtype, seed=1)
    V = CONFIGS[name]["vocab"]
    for n in (1, 2, 3, 4, 5):
        toks = tokens(n + 8, V, seed=60 + n)
        assert_logits(_run_in_steps(_engine(model), toks, [n] + [1] * 8), oracle_logits(folder, toks), dtype, f"{name}: prompt of {n}")
        assert_logits(_run_in_steps(_engine(model), toks, [n, 2, 2, 4]), oracle_logits(folder, toks), dtype, f"{name}: prompt of {n}, portions")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_window_passes_over_decoded_tokens(models, dtype):
    """Windows of 150 and of 64 tokens with 20 and 64 kept first tokens: a prompt shorter than the window followed by 330 single
    tokens from captured decode steps, so that the window's edge crosses the kept tokens, page borders and the prompt's end, and
    pages that no key of the window lies in go back to the pool while the kept ones stay."""
    model, folder = models("window", dtype, seed=1)
    toks = tokens(400, CONFIGS["window"]["vocab"], seed=70)
    ref = oracle_logits(folder, toks)
    eng = _engine(model, max_tokens=64 * 8, use_graphs=True)
    with torch.inference_mode():
        slot = eng.alloc_slot()
        rows = [eng.step([_inputs(slot, toks[:70])]).clone()]
        for t in toks[70:]:
            rows.append(eng.decode_step([slot], [t]).clone())
        held = eng.cache.pages_held()
        eng.free_slot(slot)
    eng.check_device_errors()
    assert_logits(torch.cat(rows), ref, dtype, "window: long decoding")
    assert max(held) < 7, f"pages out of every window were kept: {held}"
    for cuts in ([400], [149, 1, 1, 1, 148, 100], [151, 63, 186], [20, 1, 129, 250]):
        assert_logits(_run_in_steps(_engine(model), toks, cuts), ref, dtype, f"window: steps of {cuts}")


# ----------------------------------------------------------------------------- what random weights would hide

def _needle_folder(tmp_path_factory, mask, pairs, T, seed=9):
    """One parallel layer whose attention is made so that chosen queries read single keys: keys read the first ``dim`` coordinates
    of the normed row alone, ordinary tokens have zeros there (their keys are zero, their scores are the distance bias alone),
    a needle token B has a large entry there, and the query token A's embedding is a rotation R^T of B's while every head's
    query map is beta * (its key map) * R; so A's query scores highest on B's key, wherever it lies, if the mask lets it.  The
    input convolution is zeroed (it would mix A with its neighbours); ``pairs`` lists (query position, needle position)."""
    c = json.loads(json.dumps(CONFIGS["window"]))
    c["layers"] = [dict(c["layers"][0])]
    left = c["layers"][0]["mixer"]["left"]
    left.pop("mask", None)
    if mask is not None:
        left["mask"] = dict(mask)
    left["softcap"], left["scale"] = 40.0, 1.0
    W = {k: v.float() for k, v in random_weights(c, seed).items()}
    H, G, d, width, V = left["heads"], left["kv_heads"], left["dim"], c["width"], c["vocab"]
    g = torch.Generator().manual_seed(12)
    R = torch.linalg.qr(torch.randn(width, width, generator=g, dtype=torch.float64)).Q
    W["l0.norm1"] = torch.ones(width)
    W["l0.canon1"] = torch.zeros(width, c["canon"]["taps"])
    W["embed"][:, :d] = 0.0
    K = torch.zeros(G * d, width, dtype=torch.float64)
    for kv in range(G):
        K[kv * d:(kv + 1) * d, :d] = torch.eye(d, dtype=torch.float64)
    W["l0.mix.left.k"] = K.float()
    W["l0.mix.left.q"] = torch.cat([3.0 * K[(h // (H // G)) * d:(h // (H // G) + 1) * d] @ R for h in range(H)]).float()
    W["l0.mix.left.r1"] = torch.full((H,), 0.25)
    W["l0.mix.left.r2"] = torch.full((H,), 0.5)
    toks = tokens(T, V - 2 * len(pairs), seed=80)                        # the last ids of the vocabulary are kept for the pairs
    for i, (query_at, needle_at) in enumerate(pairs):
        a, b = V - 1 - 2 * i, V - 2 - 2 * i
        e = torch.randn(width, generator=g, dtype=torch.float64)
        e[:d] = 2.5 * torch.sign(torch.randn(d, generator=g, dtype=torch.float64))
        W["embed"][b] = e.float()
        W["embed"][a] = (R.T @ e).float()
        toks[needle_at], toks[query_at] = b, a
    W = {k: v.to(torch.bfloat16) for k, v in W.items()}
    return write_folder(str(tmp_path_factory.mktemp("bededra-needle")), c, W), toks


def _needle_weights(folder, toks):
    c, W = read_folder(folder)
    left = c["layers"][0]["mixer"]["left"]
    h = P.rms_norm(W["embed"][torch.tensor(toks)], W["l0.norm1"], c["norm"]["eps"])
    T = len(toks)
    q = (h @ W["l0.mix.left.q"].T).reshape(T, left["heads"], left["dim"])
    k = (h @ W["l0.mix.left.k"].T).reshape(T, left["kv_heads"], left["dim"])
    w, _ = P.mixed_attention_weights(q, k, left, W["l0.mix.left.r1"], W["l0.mix.left.r2"], None)
    return w


@pytest.mark.parametrize("dtype", DTYPES)
def test_keys_at_the_edges_of_the_window_and_of_the_kept_tokens_show(tmp_path_factory, dtype):
    """A window of 150 with 20 kept first tokens.  Queries whose one key lies at the window's last place (seen), one further
    (not seen), at the last kept place (seen from far away) and one after it (not seen), at a page's last and first place
    inside the window, and right before the query.  The plain implementation first proves which are read; then prompts,
    portions that end at the edges, and decoding over them."""
    from kuiperllama_b200.engine import load_model
    T = 420
    seen = [(200, 51), (230, 19), (260, 0), (300, 191), (301, 192), (330, 329), (340, 338), (405, 256), (410, 18), (419, 270)]
    unseen = [(210, 60), (240, 20), (275, 21), (320, 170), (400, 249)]
    folder, toks = _needle_folder(tmp_path_factory, {"size": 150, "keep_first": 20}, seen + unseen, T)
    w = _needle_weights(folder, toks)
    for qa, na in seen:
        assert float(w[:, qa, na].min()) > 0.5, f"the query at {qa} does not read the key at {na}"
    for qa, na in unseen:
        assert float(w[:, qa, na].max()) == 0.0, f"the query at {qa} reads the key at {na}"
    ref = oracle_logits(folder, toks)
    with torch.inference_mode():
        model = load_model(folder, dtype=dtype, device="cuda:0")
    assert_logits(_run_in_steps(_engine(model), toks, [T]), ref, dtype, "edges: whole")
    assert_logits(_run_in_steps(_engine(model), toks, [200, 10, 20, 10, 30, 30, 1, 19, 80, 20]), ref, dtype, "edges: portions that end at the queries")
    assert_logits(_run_in_steps(_engine(model), toks, [64, 128, 8, 1, 199, 20]), ref, dtype, "edges: portions at page borders")
    assert_logits(_run_in_steps(_engine(model), toks, [195] + [1] * 225), ref, dtype, "edges: prompt, then the queries one by one")
    assert_logits(_run_in_steps(_engine(model), toks, [2] * 210), ref, dtype, "edges: portions of two")


@pytest.mark.parametrize("dtype", DTYPES)
def test_far_keys_without_a_window_show(tmp_path_factory, dtype):
    """No window: queries that read one key each four and five pages back, at every page's last and first place between, in a
    prompt, in portions and in decoding."""
    from kuiperllama_b200.engine import load_model
    T = 360
    pairs = [(359, 0), (357, 63), (355, 64), (353, 127), (351, 128), (349, 191), (347, 192), (345, 255), (343, 256), (341, 30)]
    folder, toks = _needle_folder(tmp_path_factory, None, pairs, T, seed=10)
    w = _needle_weights(folder, toks)
    for qa, na in pairs:
        assert float(w[:, qa, na].min()) > 0.5, f"the query at {qa} does not read the key at {na}"
    ref = oracle_logits(folder, toks)
    with torch.inference_mode():
        model = load_model(folder, dtype=dtype, device="cuda:0")
    assert_logits(_run_in_steps(_engine(model), toks, [T]), ref, dtype, "far: whole")
    assert_logits(_run_in_steps(_engine(model), toks, [64, 63, 1, 65, 62, 85, 20]), ref, dtype, "far: portions at page borders")
    assert_logits(_run_in_steps(_engine(model), toks, [335] + [1] * 25), ref, dtype, "far: prompt, then the queries one by one")


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_linear_attention_remembers_a_far_token(tmp_path_factory, dtype):
    """The right branch alone carries a token over 300 positions: decay biases of +9 (alpha near 1), the attention switched off
    (left_scale 0).  Changing the first token must change the last logits in the plain implementation, and the framework must
    agree with it, in a prompt, in portions and token by token."""
    from kuiperllama_b200.engine import load_model
    c = json.loads(json.dumps(CONFIGS["only_parallel"]))
    c["layers"][0]["mixer"]["left_scale"] = 0.0
    W = random_weights(c, 5)
    W["l0.mix.right.a2.b"] = torch.full_like(W["l0.mix.right.a2.b"], 9.0)
    W["l0.mix.right.a2"] = W["l0.mix.right.a2"] * 0.1
    folder = write_folder(str(tmp_path_factory.mktemp("bededra-memory")), c, W)
    toks = tokens(320, c["vocab"], seed=81)
    other = [(toks[0] + 1) % c["vocab"]] + toks[1:]
    ref, ref_other = oracle_logits(folder, toks), oracle_logits(folder, other)
    assert float((ref[-1] - ref_other[-1]).abs().max()) > 1e-2 * float(ref[-1].std()), "the first token is forgotten: the test shows nothing"
    with torch.inference_mode():
        model = load_model(folder, dtype=dtype, device="cuda:0")
    for cuts in ([320], [1, 319], [100, 3, 217], [300] + [1] * 20):
        assert_logits(_run_in_steps(_engine(model), toks, cuts), ref, dtype, f"memory: steps of {cuts[:4]}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_from_graphs(models, dtype):
    """400 tokens one by one through captured decode steps after a prompt of five: both recurrent states, the convolutions'
    inputs and the keys over six pages."""
    model, folder = models("mixed", dtype, seed=1)
    toks = tokens(405, CONFIGS["mixed"]["vocab"], seed=70)
    eng = _engine(model, max_tokens=64 * 8, use_graphs=True)
    with torch.inference_mode():
        slot = eng.alloc_slot()
        rows = [eng.step([_inputs(slot, toks[:5])]).clone()]
        for t in toks[5:]:
            rows.append(eng.decode_step([slot], [t]).clone())
        eng.free_slot(slot)
    eng.check_device_errors()
    assert_logits(torch.cat(rows), oracle_logits(folder, toks), dtype, "long decoding")


# ----------------------------------------------------------------------------- the entry points

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    """``load(...).generate``: scheduler, batches that reuse slots, captured decode steps, sampler.  float32 gives the plain
    greedy tokens (where the plain logits' two best are apart); in bfloat16 a token may differ where they are close, and the
    run is compared up to there."""
    import kuiperllama_b200 as kl
    folder = folders(name, seed=1)
    c, W = read_folder(folder)
    prompts = [tokens(n, c["vocab"], seed=90 + n) for n in (7, 1, 66, 20, 3)]
    m = kl.load(folder, dtype=dtype, device="cuda:0", max_tokens=64 * 8, max_batch=2)
    got = m.generate(prompts, max_new_tokens=10, stop_ids=[])
    for p, out in zip(prompts, got):
        assert len(out) == 10
        seq = list(p)
        for tok in out:
            logits = P.forward(W, c, seq)[-1]
            top = torch.topk(logits, 2).values
            if int(logits.argmax()) != tok:
                close = float(top[0] - top[1]) < (1e-3 if dtype == "float32" else 0.15) * float(logits.std())
                assert close and float(logits[tok]) >= float(top[1]) - 1e-9, f"{name} {dtype}: token {tok} is not the plain greedy token"
                break
            seq.append(tok)


def test_cli_runs_a_bededra_folder(folders, capsys):
    from kuiperllama_b200.cli import main
    folder = folders("mixed", seed=1)
    assert main([folder, "--prompt-ids", "1,2,3", "--max-new-tokens", "4", "--dtype", "float32", "--stop-ids", ""]) == 0
    out = capsys.readouterr().out
    c, W = read_folder(folder)
    assert " ".join(str(t) for t in P.greedy(W, c, [1, 2, 3], 4)) in out


def test_trace_run_replays_a_bededra_folder(folders, tmp_path):
    """bin/trace_run as a user runs it, in float32: five requests in one step, then two steps of a token each with the
    shortest leaving first."""
    import os
    import subprocess
    import sys

    import numpy as np
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder = folders("mixed", seed=1)
    V = CONFIGS["mixed"]["vocab"]
    lens = [1, 3, 65, 2, 66]
    seqs = [tokens(n + 2, V, seed=110 + i) for i, n in enumerate(lens)]
    steps = [{"step": 0, "entries": [{"id": f"r{i}", "tokens": s[:n], "want": [n - 1]} for i, (s, n) in enumerate(zip(seqs, lens))], "end": []},
             {"step": 1, "entries": [{"id": f"r{i}", "tokens": [s[n]], "want": [0]} for i, (s, n) in enumerate(zip(seqs, lens))], "end": ["r0"]},
             {"step": 2, "entries": [{"id": f"r{i}", "tokens": [s[n + 1]], "want": [0]} for i, (s, n) in enumerate(zip(seqs, lens)) if i],
              "end": [f"r{i}" for i in range(1, 5)]}]
    out = str(tmp_path / "out")
    cmd = [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", out,
           "--max-tokens", str(sum(lens) + 2 * len(lens))]
    p = subprocess.run(cmd, input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    refs = [oracle_logits(folder, s) for s in seqs]
    read = lambda k: torch.from_numpy(np.fromfile(os.path.join(out, f"{k}.f32"), dtype="<f4").reshape(-1, V).copy())
    assert_logits(read(0), torch.stack([r[n - 1] for r, n in zip(refs, lens)]), "float32", "replay: prompts")
    assert_logits(read(1), torch.stack([r[n] for r, n in zip(refs, lens)]), "float32", "replay: first tokens")
    assert_logits(read(2), torch.stack([r[n + 1] for r, n in list(zip(refs, lens))[1:]]), "float32", "replay: second tokens")
