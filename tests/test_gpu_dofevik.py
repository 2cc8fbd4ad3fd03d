"""The Dofevik decoder through the framework's own loader, cache, step function and generation loop,
against the plain implementation (tests/plain_dofevik.py), in float32 and bfloat16.

The float32 runs are the sharp ones: they differ from the plain implementation only by the order of sums,
so a key that is missed, a window that is one token off, a pooled block that is seen too early or a sink that
is left out shows at once.  The configurations are in dofevik_helpers.py.
"""
from __future__ import annotations

import json
import math

import pytest
import torch

import plain_dofevik as P
from dofevik_helpers import CONFIGS, assert_logits, oracle_logits, random_weights, read_folder, tokens, write_folder

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
            made[key] = write_folder(str(tmp_path_factory.mktemp(f"dofevik-{name}")), c, random_weights(c, seed, gain))
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


# ----------------------------------------------------------------------------- the new kernels alone

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("aligned", [False, True])
@pytest.mark.parametrize("H, G, d, dv, rot, interleaved, norm, weighted, own_v, biased",
                         [(6, 3, 16, 20, 8, True, True, False, True, True), (4, 2, 12, 12, 0, False, True, True, False, False),
                          (5, 5, 10, 6, 6, True, True, False, True, True), (8, 2, 64, 64, 32, False, False, False, True, False),
                          (2, 1, 128, 128, 128, True, True, True, False, True), (3, 1, 18, 7, 4, False, False, False, True, True),
                          (4, 2, 32, 64, 16, False, True, True, True, True), (3, 1, 256, 8, 64, True, True, False, True, True),
                          (40, 8, 64, 64, 64, False, True, True, False, False), (7, 7, 8, 16, 6, True, True, True, True, True),
                          (5, 1, 64, 64, 0, False, True, False, True, True)])
def test_bias_rotation_head_norm_and_cache_write(dtype, aligned, H, G, d, dv, rot, interleaved, norm, weighted, own_v, biased):
    """``ops.qk_prepare`` alone on a ragged step over scattered pages: every option on and off, q and k columns that start
    anywhere in a wider matrix (or on 16-byte boundaries, where bfloat16 rows of head sizes 8, 16, ... 256 take the form with
    eight elements a lane), values of another size than the keys and values that are the keys as projected."""
    from kuiperllama_b200.csrc import ops
    dt, dev = getattr(torch, dtype), "cuda:0"
    g = torch.Generator().manual_seed(H * 7 + d)
    starts, news = [5, 100, 0], [70, 1, 9]
    step = _step(starts, news)
    n = step.n_tokens
    gap = (lambda n: -n % 8) if aligned else (lambda n: 0)
    q_col = 8
    k_col = q_col + H * d + (gap(H * d) if aligned else 3)
    v_col = k_col + G * d + (gap(G * d) if aligned else 5)
    width = v_col + G * dv + 2
    width += gap(width)
    proj = torch.randn(n, width, generator=g).to(dt)
    f32 = lambda size, on=True: (0.5 * torch.randn(size, generator=g)).to(dev) if on else None
    qb, kb, vb = f32(H * d, biased), f32(G * d, biased), f32(G * dv, biased and own_v)
    qw, kw = f32(d, weighted), f32(d, weighted)
    rope = {"base": 300.0, "dims": rot, "scaling": {"factor": 1.7}}
    inv = None
    if rot:
        inv = torch.tensor([300.0 ** (-2.0 * i / rot) / 1.7 for i in range(rot // 2)], dtype=torch.float64).float().to(dev)
    table = torch.tensor([[5, 2, 9, 0], [1, 7, 3, 11], [4, 6, 8, 10]], dtype=torch.int32, device=dev)
    kc = torch.zeros(12, G, 64, d, dtype=dt, device=dev)
    vc = torch.zeros(12, G, 64, dv if own_v else d, dtype=dt, device=dev)
    vd = dv if own_v else d
    x = proj.to(dev).clone()
    ops.qk_prepare(x, q_col, k_col, v_col if own_v else None, step.positions, step.token_slot, table, kc, vc, n, H, G, d, vd,
                   q_bias=qb, k_bias=kb, v_bias=vb, inv_freq=inv, rotary_dim=rot, interleaved=interleaved, head_norm=norm, eps=1e-5,
                   q_norm_weight=qw, k_norm_weight=kw)
    tol = 2e-5 if dtype == "float32" else 2e-2
    row = 0
    for s, (st, k_new) in enumerate(zip(starts, news)):
        rows = proj[row:row + k_new].double()
        q = rows[:, q_col:q_col + H * d].reshape(k_new, H, d) + (qb.cpu().double().reshape(H, d) if biased else 0)
        k = rows[:, k_col:k_col + G * d].reshape(k_new, G, d) + (kb.cpu().double().reshape(G, d) if biased else 0)
        v = (rows[:, v_col:v_col + G * dv].reshape(k_new, G, dv) + (vb.cpu().double().reshape(G, dv) if vb is not None else 0)) if own_v else k
        if rot:
            full = lambda t: torch.cat([torch.zeros(st, *t.shape[1:], dtype=torch.float64), t])       # so that row i is position i
            q = P.rotate(full(q), rope, "interleaved" if interleaved else "half")[st:]
            k = P.rotate(full(k), rope, "interleaved" if interleaved else "half")[st:]
        if norm:
            q = P.rms_norm(q, qw.cpu().double() if weighted else None, 1e-5)
            k = P.rms_norm(k, kw.cpu().double() if weighted else None, 1e-5)
        got_q = x[row:row + k_new, q_col:q_col + H * d].cpu().double().reshape(k_new, H, d)
        assert torch.allclose(got_q, q, atol=tol, rtol=tol), ("q", s)
        for i in range(k_new):
            p = st + i
            page = int(table[s, p // 64])
            assert torch.allclose(kc[page, :, p % 64].cpu().double(), k[i], atol=tol, rtol=tol), ("k", s, i)
            assert torch.allclose(vc[page, :, p % 64].cpu().double(), v[i], atol=tol, rtol=tol), ("v", s, i)
        row += k_new
    # what lies between and beside the q columns is untouched
    assert torch.equal(x[:, :q_col].cpu(), proj[:, :q_col]) and torch.equal(x[:, q_col + H * d:].cpu(), proj[:, q_col + H * d:])


@pytest.mark.parametrize("dtype, kernel", [("float32", "plain"), ("bfloat16", "plain"), ("bfloat16", "mma"), ("bfloat16", "mma3")])
@pytest.mark.parametrize("weights", ["sigmoid", "softmax"])
@pytest.mark.parametrize("H, G, d, dv, window, pool", [(4, 2, 12, 12, 37, 5), (3, 1, 16, 16, 8, 20), (6, 3, 18, 10, 2, 3), (2, 2, 6, 6, 1, 7),
                                                        (8, 4, 64, 64, 72, 16), (2, 1, 8, 8, 65, 64), (3, 3, 12, 20, 100, 1), (2, 1, 16, 8, 40, 0),
                                                        (2, 2, 8, 8, 0, 0), (8, 1, 128, 128, 100, 3), (6, 2, 64, 64, 1, 1), (4, 4, 128, 128, 70, 0),
                                                        (5, 1, 64, 64, 0, 0), (16, 1, 64, 64, 33, 64)])
def test_window_and_pooled_blocks_on_scattered_pages(dtype, kernel, weights, H, G, d, dv, window, pool):
    """``ops.pool_blocks`` and ``ops.attention_pooled`` alone, and the tensor-core kernel with the same options (head sizes 64 and
    128; single tokens with the keys in one piece and cut into three): three sequences on scattered pages (the rows of means too)
    grow in ragged steps whose portions start and end inside blocks, pages and windows; after every step every new token's result
    is compared with plain arithmetic over what it may see: the window's keys and the blocks that lie wholly before it."""
    from kuiperllama_b200.cache import PooledView
    from kuiperllama_b200.csrc import ops
    if kernel != "plain" and not (d in (64, 128) and dv == d):
        pytest.skip("the tensor-core kernel takes equal key and value sizes of 64 and 128")
    dt, dev = getattr(torch, dtype), "cuda:0"
    g = torch.Generator().manual_seed(H * 10 + d + window)
    T = 256
    table = torch.tensor([[5, 2, 9, 0], [1, 7, 3, 11], [4, 6, 8, 10]], dtype=torch.int32, device=dev)
    ptable = torch.tensor([[3, 1, 6, 8], [0, 5, 2, 9], [7, 4, 10, 11]], dtype=torch.int32, device=dev)
    ks = [torch.randn(T, G, d, generator=g).to(dt) for _ in range(3)]
    vs = [torch.randn(T, G, dv, generator=g).to(dt) for _ in range(3)]
    qs = [(torch.randn(T, H, d, generator=g) * 1.5).to(dt) for _ in range(3)]
    sink = (0.5 * torch.randn(H, generator=g)).to(dev) if weights == "softmax" else None
    bias = (-1.0 + 0.5 * torch.randn(H, generator=g)).to(dev) if weights == "sigmoid" else None
    kc = torch.zeros(12, G, 64, d, dtype=dt, device=dev)
    vc = torch.zeros(12, G, 64, dv, dtype=dt, device=dev)
    pooled = None
    if pool:
        pooled = PooledView(torch.full((12, G, 64, d), 7.0, dtype=dt, device=dev), torch.full((12, G, 64, dv), 7.0, dtype=dt, device=dev), ptable, pool)
    scale, rep = 0.3, H // G
    want = []
    for s in range(3):
        k, v, q = ks[s].double().repeat_interleave(rep, 1), vs[s].double().repeat_interleave(rep, 1), qs[s].double()
        sc = torch.einsum("ihd,jhd->hij", q, k) * scale
        i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
        seen = (j <= i) & ((i - j < window) if window else (j <= i))
        vals = v
        if pool:
            kb, vb = P.pooled_blocks(k, pool), P.pooled_blocks(v, pool)
            whole = (torch.arange(kb.shape[0])[None, :] * pool + pool - 1) <= (torch.arange(T)[:, None] - window)
            sc = torch.cat([sc, torch.einsum("ihd,bhd->hib", q, kb) * scale], dim=2)
            seen = torch.cat([seen, whole], dim=1)
            vals = torch.cat([v, vb], dim=0)
        if weights == "sigmoid":
            w = torch.sigmoid(sc + bias.cpu().double()[:, None, None]) * seen[None]
        else:
            w = P.softmax_with_sink(sc, seen, sink.cpu().double())
        want.append(torch.einsum("hij,jhd->ihd", w, vals))
    tol = 3e-5 if dtype == "float32" else 3e-2
    at = [0, 0, 0]
    for news in ([100, 1, 67], [30, 2, 56], [1, 1, 1], [3, 110, 60], [122, 142, 72]):
        step = _step(at, news)
        for s in range(3):
            for p in range(at[s], at[s] + news[s]):
                kc[int(table[s, p // 64]), :, p % 64] = ks[s][p].to(dev)
                vc[int(table[s, p // 64]), :, p % 64] = vs[s][p].to(dev)
        if pool:
            ops.pool_blocks(kc, vc, table, pooled, step, G, d, dv)
        rows = lambda parts: torch.cat([p[a:a + n].reshape(n, -1) for p, a, n in zip(parts, at, news)])
        out = torch.full((step.n_tokens, H * dv), 9.0, dtype=dt, device=dev)
        if kernel == "plain":
            ops.attention_pooled(rows(qs).to(dev).contiguous(), out, kc, vc, table, step.positions, step.token_slot, step.n_tokens, H, G, d, dv,
                                 scale, window, weights=weights, sink=sink, head_bias=bias, pooled=pooled)
        else:
            ops.attention_mma(rows(qs).to(dev).contiguous(), H * d, out, kc, vc, table, step.cu_tokens, step.seq_slots, step.seq_starts, step.seq_new,
                              step.n_seqs, step.max_new, step.n_tokens, H, G, d, scale, window, 3 if kernel == "mma3" and step.is_decode else 1,
                              few_rows=step.is_decode, sink=sink, weights=weights, head_bias=bias, pooled=pooled)
        ref = rows(want)
        # the tensor cores take the weights as bfloat16: a sum of hundreds of unnormalised weights times values is off by a part of
        # its largest terms, not of itself
        atol = tol if kernel == "plain" else max(tol, 0.01 * float(ref.abs().max()))
        assert torch.allclose(out.cpu().double(), ref, atol=atol, rtol=tol), (at, news, float((out.cpu().double() - ref).abs().max()))
        at = [a + n for a, n in zip(at, news)]
    assert at == [T] * 3
    if pool:
        for s in range(3):                                                    # every complete block's means, and nothing beyond them
            kb = P.pooled_blocks(ks[s].double(), pool)
            for b in range(kb.shape[0]):
                got = pooled.k[int(ptable[s, b // 64]), :, b % 64].cpu().double()
                assert torch.allclose(got, kb[b], atol=1e-5 if dtype == "float32" else 1e-2, rtol=1e-5 if dtype == "float32" else 1e-2), (s, b)


@pytest.mark.parametrize("H, Dk, Dv, window", [(6, 96, 64, 70), (32, 288, 256, 129), (3, 160, 144, 1), (4, 48, 16, 64), (2, 80, 32, 200)])
def test_latent_attention_with_a_window_on_the_tensor_cores(H, Dk, Dv, window):
    """The tensor-core kernel for many heads over one key head with a window against the plain kernel (bfloat16): prompts of
    unequal lengths on scattered pages, portions that start inside a page and inside the window, single tokens whose pages are
    cut into one and into several pieces; with and without sinks."""
    from kuiperllama_b200.csrc import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(H)
    cache = (torch.randn(12, 1, 64, Dk, generator=g)).bfloat16().to(dev)
    table = torch.tensor([[5, 2, 9, 0], [1, 7, 3, 11], [4, 6, 8, 10]], dtype=torch.int32, device=dev)
    sink = torch.randn(H, generator=g).to(dev) * 2
    for starts, news in (([0, 0, 0], [230, 1, 67]), ([100, 63, 200], [30, 2, 56]), ([150, 64, 255], [1, 1, 1]), ([69, 0, 128], [150, 256, 2])):
        step = _step(starts, news)
        n = step.n_tokens
        q = (torch.randn(n, H * Dk, generator=g) / 4).bfloat16().to(dev)
        for cls in (0, 1):
            step.context_class = cls                                          # a decode step: another number of pieces
            for sk in (None, sink):
                want = torch.empty(n, H * Dv, dtype=torch.bfloat16, device=dev)
                got = torch.full_like(want, 9.0)
                ops.attention_simt(q, H * Dk, want, cache, cache, table, step.positions, step.token_slot, n, H, 1, Dk, 0.3, window, value_dim=Dv, sink=sk)
                ops.latent_attention(q, got, cache, table, step, H, Dk, Dv, 0.3, sk, window=window)
                assert torch.allclose(got.float(), want.float(), atol=3e-2, rtol=3e-2), (starts, news, cls, sk is not None)


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_of_rows_between_two_products(dtype):
    from kuiperllama_b200.csrc import ops
    dt, dev = getattr(torch, dtype), "cuda:0"
    g = torch.Generator().manual_seed(3)
    for width in (11, 24, 128, 1536):
        wide = (torch.randn(37, width + 13, generator=g) * 3).to(dt)
        w = 1 + 0.2 * torch.randn(width, generator=g)
        out = torch.empty(37, width, dtype=dt, device=dev)
        ops.rows_rmsnorm(wide.to(dev)[:, 5:5 + width], w.to(dev), out, 1e-5)
        want = P.rms_norm(wide[:, 5:5 + width].double(), w.double(), 1e-5)
        tol = 1e-5 if dtype == "float32" else 2e-2
        assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol), width


def test_router_bias_and_weights_over_the_chosen():
    """The largest logits after the bias, the lower index among equals; weights = softmax over the chosen logits alone."""
    from kuiperllama_b200.csrc import ops
    g = torch.Generator().manual_seed(4)
    for E, top in ((12, 2), (16, 4), (7, 3), (40, 5), (6, 6), (9, 1), (2, 1)):
        z = torch.randn(41, E, generator=g) * 2
        b = torch.randn(E, generator=g)
        z[3, :], b[0] = 0.25, 0.0                                          # (set below) equal logits: the lower index wins
        z[5, E - 1] = 30.0                                                 # one expert far ahead
        b = (b * 4).round() / 4                                            # quarters: row 3's sums are exact and equal in pairs
        z[3, :] = 0.25 - b
        choice, weight = ops.moe_route(z.cuda(), top, True, bias=b.cuda())
        zz = (z + b).double()                                              # the 32-bit sum, as the kernel makes it
        assert float(zz[3].max()) == float(zz[3].min()) == 0.25
        for t in range(41):
            order = sorted(range(E), key=lambda e: (-float(zz[t, e]), e))[:top]
            assert choice[t].tolist() == order, (E, top, t)
            want = torch.softmax(zz[t][choice[t].cpu().long()], dim=0)
            assert torch.allclose(weight[t].cpu().double(), want, atol=1e-6, rtol=1e-5)
        assert (E - 1) in choice[5].tolist()


@pytest.mark.parametrize("E, K, ff, n, top", [(7, 200, 128, 9, 3), (5, 64, 24, 40, 2), (16, 256, 64, 700, 4), (3, 100, 18, 30, 1)])
def test_the_experts_activation_inside_the_grouped_products(E, K, ff, n, top):
    """Ungated experts: relu(W_up x)^2 from the epilogue of every form of the routed product (32-bit FMA tiles in both dtypes, a
    warp per four weight rows, the tensor cores with tokens and with weights as tile rows) against the product and the
    activation made apart."""
    from kuiperllama_b200.csrc import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(E * 10 + ff)
    x = torch.randn(n, K, generator=g)
    choice = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(n)]).int().to(dev)
    up = torch.randn(E, ff, K, generator=g) / 8
    relu2 = lambda t: torch.relu(t.double()) ** 2
    for dt in (torch.float32, torch.bfloat16):
        xd, w = x.to(dt).to(dev), up.to(dt).to(dev)
        tol = 1e-5 if dt == torch.float32 else 3e-2
        for tile in (16, 64):
            pair_pos, list_rows, tile_group = ops.moe_plan(choice, E, tile)
            live = (list_rows >= 0).cpu()
            cap = list_rows.numel()
            plain, fused = (torch.zeros(cap, ff, dtype=dt, device=dev) for _ in range(2))
            ops.grouped_gemm(xd, w, plain, a_rows=list_rows, tile_group=tile_group, tile_rows=tile)
            ops.grouped_gemm(xd, w, fused, a_rows=list_rows, tile_group=tile_group, tile_rows=tile, activation="relu2")
            want = relu2(plain.cpu())[live]
            assert float(want.abs().max()) > 0.05
            assert torch.allclose(fused.cpu().double()[live], want, atol=tol, rtol=tol), (dt, tile)
            if dt == torch.bfloat16 and K % 8 == 0 and tile == 16:
                got = torch.zeros_like(fused)
                ops.grouped_gemv(xd, w, got, list_rows, tile_group, 16, activation="relu2")
                assert torch.allclose(got.cpu().double()[live], want, atol=tol, rtol=tol), "a warp per four weight rows"
                rows = ops.moe_gather(xd, list_rows)
                got = torch.zeros_like(fused)
                ops.gemm_tcgen05_grouped_skinny(rows, w, got, tile_group, activation="relu2")
                ops.check_status(torch.device(dev))
                assert torch.allclose(got.cpu().double()[live], want, atol=tol, rtol=tol), "weights as tile rows"
        if dt == torch.bfloat16 and K % 8 == 0:
            pair_pos, list_rows, tile_group = ops.moe_plan(choice, E, 128)
            live = (list_rows >= 0).cpu()
            rows = ops.moe_gather(xd, list_rows)
            plain, got = (torch.zeros(list_rows.numel(), ff, dtype=dt, device=dev) for _ in range(2))
            ops.gemm_tcgen05_grouped(rows, w, plain, tile_group)
            ops.gemm_tcgen05_grouped(rows, w, got, tile_group, activation="relu2")
            ops.check_status(torch.device(dev))
            assert torch.allclose(got.cpu().double()[live], relu2(plain.cpu())[live], atol=tol, rtol=tol), "tokens as tile rows"


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_gate_number_per_output_inside_the_per_head_product(dtype):
    """The batched product per head whose epilogue multiplies every output by sigmoid of a number of its own (the gate's row holds
    them head by head): the 32-bit FMA tiles of 16 and 64 rows, and with many rows in bfloat16 the tensor-core form."""
    from kuiperllama_b200.csrc import ops
    dt, dev = getattr(torch, dtype), "cuda:0"
    g = torch.Generator().manual_seed(2)
    rnd = lambda *s: torch.randn(*s, generator=g)
    tol = 1e-5 if dtype == "float32" else 2e-2
    for rows, G, K, N, a_gs, o_gs, tile in ((37, 5, 12, 7, 20, 9, 16), (37, 5, 12, 7, 20, 9, 64), (150, 3, 40, 70, 48, 72, 64), (9, 4, 16, 24, 16, 24, 16)):
        a, w = rnd(rows, G * a_gs).to(dt), (rnd(G, N, K) / 3).to(dt)
        wide = rnd(rows, G * N + 11).to(dt).to(dev)                       # the gate's numbers are columns 3 .. of a wider matrix
        gate = wide[:, 3:3 + G * N]
        out = torch.zeros(rows, G * o_gs, dtype=dt, device=dev)
        ops.grouped_gemm(a.to(dev), w.to(dev), out, a_group_stride=a_gs, out_group_stride=o_gs, rows=rows, tile_rows=tile, row_gate=gate,
                         gate_elements=True)
        want = torch.einsum("tgk,gnk->tgn", a.double().reshape(rows, G, a_gs)[..., :K], w.double())
        want = want * torch.sigmoid(gate.cpu().double().reshape(rows, G, N))
        got = out.cpu().double().reshape(rows, G, o_gs)
        assert torch.allclose(got[..., :N], want, atol=2 * tol, rtol=tol), (rows, G, tile)
        assert o_gs == N or float(got[..., N:].abs().max()) == 0.0


# ----------------------------------------------------------------------------- each mechanism alone, layer by layer

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["only_attention", "only_attention_2", "only_latent", "only_moe"])
def test_one_mechanism_alone(models, name, dtype):
    model, folder = models(name, dtype, seed=3)
    toks = tokens(90, CONFIGS[name]["vocab"], seed=11)
    ref = oracle_logits(folder, toks)
    assert_logits(_run_in_steps(_engine(model), toks, [90]), ref, dtype, f"{name}: whole")
    assert_logits(_run_in_steps(_engine(model), toks, [1] * 90), ref, dtype, f"{name}: token by token")


def test_the_stream_after_every_layer(models):
    """float32: the residual stream after each layer against the plain implementation's, so that a fault is named by its layer."""
    from kuiperllama_b200.csrc import ops
    from kuiperllama_b200.parts.norm import add_to_stream
    for name in ("mixed", "wide", "odd"):
        model, folder = models(name, "float32", seed=1)
        c, W = read_folder(folder)
        toks = tokens(90, c["vocab"], seed=12)
        _, streams = P.forward(c, W, toks)
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
    """Prompts of several hundred tokens (every window and many blocks left behind), a long portion after a short one and before
    one, and a long prompt beside a short one in one step."""
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
    """A cache with room for little: four rounds of requests on the same slots and pages (the pages of block means too), whose
    old contents must not leak into the next request."""
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
    for grp in eng.cache.groups:
        assert grp.held() == 0 and (not hasattr(grp, "pool_pages") or grp.pool_pages.held() == 0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_the_first_tokens_of_a_sequence(models, name, dtype):
    """Prompts of one to five tokens and what follows token by token and in small portions: windows of one and two keys, blocks
    that are not complete yet, the first token alone with the sink."""
    model, folder = models(name, dtype, seed=1)
    V = CONFIGS[name]["vocab"]
    for n in (1, 2, 3, 4, 5):
        toks = tokens(n + 8, V, seed=60 + n)
        assert_logits(_run_in_steps(_engine(model), toks, [n] + [1] * 8), oracle_logits(folder, toks), dtype, f"{name}: prompt of {n}")
        assert_logits(_run_in_steps(_engine(model), toks, [n, 2, 2, 4]), oracle_logits(folder, toks), dtype, f"{name}: prompt of {n}, portions")


@pytest.mark.parametrize("dtype", DTYPES)
def test_windows_pass_over_decoded_tokens(models, dtype):
    """Windows of 64 to 150 keys and blocks of 24 and 64 positions: a prompt shorter than every window followed by 340 single tokens
    from captured decode steps, so that every window's edge crosses page borders and the prompt's end, blocks become complete and
    seen while decoding, and pages that no window reaches go back to the pool."""
    model, folder = models("window", dtype, seed=1)
    toks = tokens(400, CONFIGS["window"]["vocab"], seed=70)
    ref = oracle_logits(folder, toks)
    eng = _engine(model, max_tokens=64 * 8, use_graphs=True)
    with torch.inference_mode():
        slot = eng.alloc_slot()
        rows = [eng.step([_inputs(slot, toks[:60])]).clone()]
        for t in toks[60:]:
            rows.append(eng.decode_step([slot], [t]).clone())
        held = eng.cache.pages_held()
        eng.free_slot(slot)
    eng.check_device_errors()
    assert_logits(torch.cat(rows), ref, dtype, "window: long decoding")
    assert max(held) <= 4, f"pages out of every window were kept: {held}"
    for cuts in ([400], [149, 1, 1, 1, 148, 100], [151, 63, 186], [20, 1, 129, 250], [99, 1, 23, 1, 276]):
        assert_logits(_run_in_steps(_engine(model), toks, cuts), ref, dtype, f"window: steps of {cuts}")


# ----------------------------------------------------------------------------- what random weights would hide

def _needle_folder(tmp_path_factory, kind, size, pool, pairs, T, seed=9):
    """One layer of the given mixer whose weights are made so that chosen queries read single keys.  Keys read the first d
    coordinates of the normed row alone; ordinary tokens have zeros there (their keys are zero and score 0 with every query),
    a needle token B has entries of +-2.5 there, and the query token A's embedding is a rotation R^T of B's while every head's
    query map is (its key map) R: A's query points along B's key and scores scale * d on it, wherever B lies, if the mask lets
    it.  ``pairs`` lists (query position, needle positions); every pair has token ids of its own."""
    d, width, V = 16, 48, 40 + 2 * len(pairs)
    if kind == "attention":
        layer = {"type": kind, "mixer": {"heads": 4, "kv_heads": 2, "dim": d, "vdim": 12, "scale": 1.0, "mask": {"size": size},
                                         "rot": {"base": 10000.0, "dims": 4, "scaling": {"factor": 2.0}}}, "mlp": None}
    elif kind == "attention_2":
        layer = {"type": kind, "mixer": {"heads": 3, "kv_heads": 3, "dim": d, "vdim": d, "scale": 1.0, "mask": {"size": size, "pool": pool}},
                 "mlp": None}
    else:
        layer = {"type": kind, "mixer": {"heads": 2, "dim": d, "rot_dim": 4, "vdim": 12, "kv_rank": d, "q_rank": 20, "scale": 1.0,
                                         "mask": {"size": size}, "rot": {"base": 1000.0, "dims": 4}}, "mlp": None}
    c = {"architecture": "Dofevik", "vocab": V, "width": width, "norm": {"eps": 1e-6}, "layers": [layer]}
    W = {k: v.float() for k, v in random_weights(c, seed).items()}
    g = torch.Generator().manual_seed(12)
    R = torch.linalg.qr(torch.randn(width, width, generator=g, dtype=torch.float64)).Q
    W["l0.norm1"] = torch.tensor(1.0)
    W["embed"][:, :d] = 0.0
    eye = torch.zeros(d, width, dtype=torch.float64)
    eye[:, :d] = torch.eye(d, dtype=torch.float64)
    m = layer["mixer"]
    if kind == "latent_attention":
        W["l0.mix.dkv"] = torch.cat([eye, torch.zeros(m["rot_dim"], width, dtype=torch.float64)]).float()      # c = the row's first d coordinates, no rotated part
        W["l0.mix.dkv.norm"] = torch.ones(d)
        W["l0.mix.dq"] = R[:m["q_rank"]].float()
        W["l0.mix.dq.norm"] = torch.ones(m["q_rank"])
        head = torch.zeros(d + m["rot_dim"], m["q_rank"], dtype=torch.float64)
        head[:d, :d] = torch.eye(d, dtype=torch.float64)
        W["l0.mix.uq"] = torch.cat([head] * m["heads"]).float()
        W["l0.mix.uk"] = torch.cat([torch.eye(d, dtype=torch.float64)] * m["heads"]).float()
    else:
        G, H = m["kv_heads"], m["heads"]
        W["l0.mix.k"] = torch.cat([eye] * G).float()
        W["l0.mix.q"] = torch.cat([eye @ R] * H).float()
        if kind == "attention":
            W["l0.mix.q.b"], W["l0.mix.k.b"] = torch.zeros(H * d), torch.zeros(G * d)
        else:
            W["l0.mix.q.norm"], W["l0.mix.k.norm"] = torch.ones(d), torch.ones(d)
            W["l0.mix.pb"] = torch.full((H,), -6.0)
    toks = tokens(T, V - 2 * len(pairs), seed=80)                        # the last ids of the vocabulary are kept for the pairs
    for i, (query_at, needles_at) in enumerate(pairs):
        a, b = V - 1 - 2 * i, V - 2 - 2 * i
        e = torch.randn(width, generator=g, dtype=torch.float64)
        e[:d] = 2.5 * torch.sign(torch.randn(d, generator=g, dtype=torch.float64))
        W["embed"][b] = e.float()
        W["embed"][a] = (R.T @ e).float()
        toks[query_at] = a
        for p in needles_at:
            toks[p] = b
    W = {k: v.to(torch.bfloat16) for k, v in W.items()}
    return write_folder(str(tmp_path_factory.mktemp(f"dofevik-needle-{kind}")), c, W), toks, V


def _check_needles(folder, toks, V, seen, unseen):
    """The plain implementation proves which needles are read: taking a pair's needle tokens away changes the query's logits by
    much where they are seen, and by nothing at all where they are not."""
    ref = oracle_logits(folder, toks)
    for i, (qa, needles) in enumerate(seen + unseen):
        b = V - 2 - 2 * i
        without = [0 if (t == b) else t for t in toks]
        other = oracle_logits(folder, without)
        diff = float((ref[qa] - other[qa]).abs().max()) / float(ref[qa].std())
        if i < len(seen):
            assert diff > 0.2, f"the query at {qa} does not read its needle at {needles}: {diff:.3e}"
        else:
            assert diff == 0.0, f"the query at {qa} reads its needle at {needles}: {diff:.3e}"
    return ref


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["attention", "latent_attention"])
def test_keys_at_the_edges_of_the_window_show(tmp_path_factory, kind, dtype):
    """A window of 150.  Queries whose one key lies at the window's last place (seen), one further (not seen), at a page's last
    and first place inside the window, right before the query, and far outside.  Then prompts, portions that end at the edges,
    and decoding over them."""
    from kuiperllama_b200.engine import load_model
    T = 420
    seen = [(200, [51]), (300, [191]), (301, [192]), (330, [329]), (405, [256]), (419, [270]), (149, [0])]
    unseen = [(210, [60]), (320, [170]), (400, [249]), (415, [3]), (151, [1])]
    folder, toks, V = _needle_folder(tmp_path_factory, kind, 150, None, seen + unseen, T)
    ref = _check_needles(folder, toks, V, seen, unseen)
    rows = [q for q, _ in seen + unseen]
    with torch.inference_mode():
        model = load_model(folder, dtype=dtype, device="cuda:0")
    assert_logits(_run_in_steps(_engine(model), toks, [T]), ref, dtype, "edges: whole", rows)
    assert_logits(_run_in_steps(_engine(model), toks, [200, 10, 20, 70, 1, 19, 80, 20]), ref, dtype, "edges: portions that end at the queries", rows)
    assert_logits(_run_in_steps(_engine(model), toks, [64, 128, 8, 1, 199, 20]), ref, dtype, "edges: portions at page borders", rows)
    assert_logits(_run_in_steps(_engine(model), toks, [140] + [1] * 280), ref, dtype, "edges: prompt, then the queries one by one", rows)
    assert_logits(_run_in_steps(_engine(model), toks, [2] * 210), ref, dtype, "edges: portions of two", rows)


@pytest.mark.parametrize("dtype", DTYPES)
def test_pooled_blocks_just_seen_and_not_yet_seen_show(tmp_path_factory, dtype):
    """A window of 70 and blocks of 4, whose first three positions hold the needle: queries at the first position from which a
    block is seen and one before it (the needles have left the window, the block is not complete for the window yet), blocks at
    the borders of the pages of means (rows 63, 64), the first block from the last position, and keys at the window's edge."""
    from kuiperllama_b200.engine import load_model
    T, W, Pp = 420, 70, 4
    block = lambda b: [4 * b, 4 * b + 1, 4 * b + 2]
    seen = [(4 * 25 + 3 + W, block(25)), (419, block(0)), (4 * 63 + 3 + W, block(63)), (4 * 64 + 3 + W, block(64)), (400, block(31)),
            (300, [231]), (402, [401])]
    unseen = [(4 * 40 + 3 + W - 1, block(40)), (4 * 50 + 3 + W - 1, block(50)), (310, [240]), (4 * 70 + 3 + W - 1, block(70))]
    folder, toks, V = _needle_folder(tmp_path_factory, "attention_2", W, Pp, seen + unseen, T)
    ref = _check_needles(folder, toks, V, seen, unseen)
    rows = [q for q, _ in seen + unseen]
    with torch.inference_mode():
        model = load_model(folder, dtype=dtype, device="cuda:0")
    assert_logits(_run_in_steps(_engine(model), toks, [T]), ref, dtype, "blocks: whole", rows)
    assert_logits(_run_in_steps(_engine(model), toks, [101, 1, 1, 69, 1, 59, 100, 88]), ref, dtype, "blocks: portions that end inside blocks", rows)
    assert_logits(_run_in_steps(_engine(model), toks, [64, 128, 8, 1, 199, 20]), ref, dtype, "blocks: portions at page borders", rows)
    assert_logits(_run_in_steps(_engine(model), toks, [100] + [1] * 320), ref, dtype, "blocks: prompt, then token by token", rows)
    assert_logits(_run_in_steps(_engine(model), toks, [2] * 210), ref, dtype, "blocks: portions of two", rows)
    assert_logits(_run_in_steps(_engine(model), toks, [3] * 140), ref, dtype, "blocks: portions of three", rows)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_sink_takes_its_share(tmp_path_factory, dtype):
    """Sinks of +6 and -6 on the heads of one attention layer with zero keys: with the large sink the layer adds next to nothing,
    with the small one it adds the mean of the values; the plain implementation proves the difference before the comparison."""
    from kuiperllama_b200.engine import load_model
    c = json.loads(json.dumps(CONFIGS["only_attention"]))
    refs = []
    for sink in (6.0, -6.0):
        W = random_weights(c, 5)
        W["l0.mix.k"] = torch.zeros_like(W["l0.mix.k"])
        W["l0.mix.k.b"] = torch.zeros_like(W["l0.mix.k.b"])
        W["l0.mix.sink"] = torch.full_like(W["l0.mix.sink"], sink)
        folder = write_folder(str(tmp_path_factory.mktemp("dofevik-sink")), c, W)
        toks = tokens(40, c["vocab"], seed=81)
        ref = oracle_logits(folder, toks)
        refs.append(ref)
        with torch.inference_mode():
            model = load_model(folder, dtype=dtype, device="cuda:0")
        for cuts in ([40], [1] * 40, [7, 33]):
            assert_logits(_run_in_steps(_engine(model), toks, cuts), ref, dtype, f"sink {sink}: steps of {cuts[:3]}", rows=range(40))
    assert float((refs[0] - refs[1]).abs().max()) > 0.1 * float(refs[1].std()), "the sink changes nothing: the test shows nothing"


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_from_graphs(models, dtype):
    """400 tokens one by one through captured decode steps after a prompt of five: windows, blocks and pages of every layer."""
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

def _greedy(c, W, prompt, n):
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(P.forward(c, W, seq)[0][-1].argmax()))
    return seq[len(prompt):]


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
            logits = P.forward(c, W, seq)[0][-1]
            top = torch.topk(logits, 2).values
            if int(logits.argmax()) != tok:
                close = float(top[0] - top[1]) < (1e-3 if dtype == "float32" else 0.15) * float(logits.std())
                assert close and float(logits[tok]) >= float(top[1]) - 1e-9, f"{name} {dtype}: token {tok} is not the plain greedy token"
                break
            seq.append(tok)


def test_cli_runs_a_dofevik_folder(folders, capsys):
    from kuiperllama_b200.cli import main
    folder = folders("mixed", seed=1)
    assert main([folder, "--prompt-ids", "1,2,3", "--max-new-tokens", "4", "--dtype", "float32", "--stop-ids", ""]) == 0
    out = capsys.readouterr().out
    c, W = read_folder(folder)
    assert " ".join(str(t) for t in _greedy(c, W, [1, 2, 3], 4)) in out


def test_trace_run_replays_a_dofevik_folder(folders, tmp_path):
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
