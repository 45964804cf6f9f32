"""The Mosurax design on the GPU against the plain implementation (tests/plain_mosurax.py):
each mechanism alone at the kernel's or part's own interface, then the engine - whole prompts,
prompts against token-by-token decoding, portions down to two tokens, unequal batches against
each request alone, slots and pages used again, windows' edges in prompts and in decoding, long
decoding - and greedy generation through ``Runner.generate``."""
import functools
import math

import pytest
import torch

import mosurax_configs as C
import plain_mosurax as P
from gpu_helpers import BF16_REL_MAX, BF16_REL_MEAN, F32_REL, random_tokens

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
NAMES = list(C.CONFIGS)
DEV = "cuda:0"


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("mosurax")
    return {n: C.write_model(n, str(root / n)) for n in NAMES}


@functools.lru_cache(maxsize=None)
def _plain(d):
    return P.load_model_dir(d)


_LOGITS = {}


def plain_logits(d, tokens):
    key = (d, tuple(tokens))
    if key not in _LOGITS:
        cfg, w = _plain(d)
        _LOGITS[key] = P.forward(cfg, w, list(tokens))
    return _LOGITS[key]


@functools.lru_cache(maxsize=None)
def runner(d, dtype, max_cache_tokens=64 * 40, max_batch=8):
    from rustyllm_b200 import Runner
    return Runner.from_path(d, dtype=dtype, max_cache_tokens=max_cache_tokens, max_batch=max_batch)[0]


def layer_runs(cfg):
    n, loop = len(cfg["layers"]), cfg.get("loop")
    return n + ((loop["stop"] - loop["start"]) * (loop["times"] - 1) if loop else 0)


def close(got, ref, dtype, cfg, what):
    """32-bit: 3e-5 of a logit row's rms (two orders above float32 accumulation, two below a wrong
    key).  bfloat16: the bound derived for three layer runs (gpu_helpers), grown with the square
    root of the layer runs (rounding noise adds up like a random walk) and doubled, because these
    weights make attention and routing sharp where the Llama test weights leave them flat."""
    got, ref = got.detach().to("cpu", torch.float64), ref.detach().to("cpu", torch.float64)
    assert got.shape == ref.shape, f"{what}: {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    err = (got - ref).abs() / ref.pow(2).mean(dim=-1, keepdim=True).sqrt().clamp_min(1e-30)
    if dtype == "float32":
        assert err.max().item() <= F32_REL, f"{what}: {err.max().item():.3e} (row {err.max(dim=-1).values.argmax().item()})"
    else:
        # A router's close call may fall the other way once its input is rounded to bfloat16; that token
        # (and, diluted, the tokens that attend to it) then differs by far more than rounding.  With
        # experts, up to a tenth of the rows may therefore exceed the bound; every row stays within
        # the scale of a logit row, and the mean over all rows within the mean bound.
        grow = 2.0 * math.sqrt(max(1.0, layer_runs(cfg) / 3.0))
        rows = err.max(dim=-1).values
        over = (rows > BF16_REL_MAX * grow).double().mean().item()
        has_experts = any((l.get("mlp") or {}).get("kind") == "moe" for l in cfg["layers"])
        allowed = max(0.1, 1.0 / rows.numel()) if has_experts else 0.0
        assert over <= allowed, f"{what}: {over:.2%} of the rows above {BF16_REL_MAX * grow:.3f} (worst {rows.max().item():.3e}, row {rows.argmax().item()})"
        assert rows.max().item() <= 1.5, f"{what}: max {rows.max().item():.3e} (row {rows.argmax().item()})"
        assert err.mean().item() <= BF16_REL_MEAN * grow, f"{what}: mean {err.mean().item():.3e}"


# =========================================================================== mechanisms alone
def _attention_through_cache(dtype, H, G, hd, vd, window, scale, q, k, v, portions, sink=True, gate=None, mma_prefill=False):
    """q [n, H*hd], k [n, G*hd], v [n, G*vd] (float64, one sequence) fed in ``portions`` through the cache
    write and the attention dispatcher, as a mixer does it; returns [n, H*vd] float64."""
    from rustyllm_b200 import kernels as K
    from rustyllm_b200.cache.sequence_cache import KVNeed, SequenceCache
    from rustyllm_b200.engine.step import StepState
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    n = q.shape[0]
    cache = SequenceCache([KVNeed(G, hd, window, vd)], [None], 64 * (n // 64 + 3), tdt, DEV, max_slots=3)
    cache.alloc_slot()                 # the sequence lives in slot 1, behind a slot that stays empty
    slot = cache.alloc_slot()
    group, layer = cache.kv_entry(0)
    inv_freq = torch.zeros(1, dtype=torch.float32, device=DEV)
    outs, at = [], 0
    for cnt in portions:
        cache.prepare([slot], [cnt])
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
        st = StepState(cnt, 1, i32([0] * cnt), i32(list(range(at, at + cnt))), i32([slot] * cnt), i32([0, cnt]), i32([slot]),
                       i32([at + cnt]), i32([]), [cnt], [at + cnt], cnt, at + cnt, cnt == 1)
        parts = [q[at:at + cnt], k[at:at + cnt], v[at:at + cnt]] + ([gate[at:at + cnt]] if gate is not None else [])
        qkv = torch.cat(parts, dim=1).to(tdt).to(DEV).contiguous()
        K.rope_kv_write(qkv, st.positions, st.slot_of_token, group.page_table, inv_freq, H, G, hd, 0, False,
                        group.k_pool(layer), group.v_pool(layer), value_dim=vd)
        out = torch.empty((cnt, H * vd), dtype=tdt, device=DEV)
        if mma_prefill and cnt > 1:        # the mma.sync prompt kernel, which the dispatcher takes where TMA cannot address q
            K.attention_prefill(qkv, group.k_pool(layer), group.v_pool(layer), group.page_table, st.cu_seqlens, st.seq_slots,
                                st.kv_lens, st.q_lens, out, H, G, hd, scale, window or 0, sink=sink,
                                gate=qkv[:, (H + G) * hd + G * vd:] if gate is not None else None)
        else:
            K.attention(qkv, group.k_pool(layer), group.v_pool(layer), group.page_table, st, out, H, G, hd, scale,
                        window or 0, value_dim=vd, sink=sink, gate=qkv[:, (H + G) * hd + G * vd:] if gate is not None else None)
        cache.commit([slot], [cnt])
        outs.append(out.double().cpu())
        at += cnt
    K.check_device_errors()
    return torch.cat(outs)


SHAPES = [(4, 2, 16, 24), (2, 1, 64, 64), (2, 2, 128, 128), (3, 3, 32, 8)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,hd,vd", SHAPES)
@pytest.mark.parametrize("window", [None, 1, 9, 70, 130])
def test_attention_with_sink_window_and_gate_alone(dtype, H, G, hd, vd, window):
    """Random rows rounded to bfloat16, a prompt portion, a second portion, then single tokens."""
    g = torch.Generator().manual_seed(hd * 1000 + (window or 0))
    n = 150
    rnd = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).double()
    q, k, v, gate = rnd(n, H * hd), rnd(n, G * hd), rnd(n, G * vd), rnd(n, H * vd)
    scale = 1.3 / math.sqrt(hd)
    ref = P.windowed_sink_attention(q.view(n, H, hd), k.view(n, G, hd), v.view(n, G, vd), scale, window).reshape(n, H * vd)
    ref = ref / (1.0 + torch.exp(-gate))
    got = _attention_through_cache(dtype, H, G, hd, vd, window, scale, q, k, v, [67, 61] + [1] * 22, gate=gate)
    tol = 2e-5 if dtype == "float32" else 2e-2
    assert (got - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())
    if dtype == "bfloat16" and hd == vd and hd in (64, 128):
        got = _attention_through_cache(dtype, H, G, hd, vd, window, scale, q, k, v, [67, 61, 22], gate=gate, mma_prefill=True)
        assert (got - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,hd,vd", SHAPES)
def test_the_sink_takes_its_share(dtype, H, G, hd, vd):
    """All scores far below 0: with the sink nearly nothing of the values comes through (a plain softmax
    would return their mean); all scores 0 over c keys: exactly c / (c + 1) of their mean."""
    n = 40
    k = torch.zeros(n, G * hd, dtype=torch.float64)
    k[:, ::hd] = 1.0                                       # every key head: (1, 0, 0, ...)
    v = torch.ones(n, G * vd, dtype=torch.float64)
    for first, want in ((-12.0, lambda c: c * math.exp(-12.0) / (1 + c * math.exp(-12.0))), (0.0, lambda c: c / (c + 1.0))):
        q = torch.zeros(n, H * hd, dtype=torch.float64)
        q[:, ::hd] = first
        got = _attention_through_cache(dtype, H, G, hd, vd, None, 1.0, q, k, v, [33] + [1] * 7)
        for i in (0, 1, 32, 33, 39):
            assert abs(got[i].mean().item() - want(i + 1)) <= (1e-6 if dtype == "float32" else 4e-3), (first, i)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,hd,vd", SHAPES)
@pytest.mark.parametrize("window,n", [(None, 700), (9, 150), (64, 200), (70, 200), (130, 330)])
def test_one_key_that_stands_out_is_seen_exactly_inside_the_window(dtype, H, G, hd, vd, window, n):
    """Key j* answers every query with a score of +14 and carries the only non-zero value; all other
    scores are 0.  A query at i then returns nearly that value where 0 <= i - j* < window and exactly 0
    elsewhere - in a prompt portion, at a portion's start and in single tokens; without a window the key
    is hundreds of positions back."""
    jstar = 3
    k = torch.zeros(n, G * hd, dtype=torch.float64)
    v = torch.zeros(n, G * vd, dtype=torch.float64)
    for g_ in range(G):
        k[jstar, g_ * hd + 1] = 1.0
        v[jstar, g_ * vd:(g_ + 1) * vd] = 1.0
    q = torch.zeros(n, H * hd, dtype=torch.float64)
    q[:, 1::hd] = 14.0
    edge = jstar + (window if window is not None else n)       # the first position that no longer sees j*
    cut = min(max(edge - 2, jstar + 2), n - 8)                 # the prompt portion ends two before the edge ...
    portions = [cut] + ([5] if cut + 5 <= n else []) + [1] * (n - cut - (5 if cut + 5 <= n else 0))   # ... a portion straddles it
    got = _attention_through_cache(dtype, H, G, hd, vd, window, 1.0, q, k, v, portions).view(n, H, vd)
    for i in range(n):
        seen = i >= jstar and (window is None or i - jstar < window)
        c = min(i + 1, window or n)                           # keys in sight
        want = math.exp(14.0) / (1.0 + math.exp(14.0) + (c - 1)) if seen else 0.0
        assert (got[i] - want).abs().max().item() <= (1e-5 if dtype == "float32" else 8e-3), (i, seen, portions[:3])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,top,d,F", [(5, 2, 64, 24), (3, 3, 48, 16), (4, 1, 128, 40), (1, 1, 32, 8), (12, 4, 96, 72)])
def test_router_and_experts_alone(dtype, E, top, d, F):
    from rustyllm_b200 import kernels as K
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(E * 100 + top)
    rnd = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).double()
    M = 37
    x, wr, b = rnd(M, d), rnd(E, d) / math.sqrt(d) * 2, rnd(E)
    wg, wu, wd = rnd(E, F, d) / math.sqrt(d), rnd(E, F, d) / math.sqrt(d), rnd(E, d, F) / math.sqrt(F)
    wg, wu, wd = (t.to(torch.bfloat16).double() for t in (wg, wu, wd))
    wr = wr.to(torch.bfloat16).double()
    ids = torch.empty((M, top), dtype=torch.int32, device=DEV)
    wts = torch.empty((M, top), dtype=torch.float32, device=DEV)
    K.moe_route(x.to(tdt).to(DEV), wr.to(tdt).to(DEV), b.float().to(DEV), top, ids, wts)
    # the selection alone, from logits made elsewhere (as steps of many tokens make them: one matrix product)
    ids2, wts2 = torch.empty_like(ids), torch.empty_like(wts)
    K.moe_select((x @ wr.T + b).float().to(DEV), top, ids2, wts2)
    res0 = rnd(M, d)
    res = res0.float().to(DEV)
    if dtype == "float32":
        K.moe_experts(x.to(tdt).to(DEV), torch.stack([wg, wu], dim=1).to(tdt).to(DEV).contiguous(), wd.to(tdt).to(DEV), ids, wts, res)
    else:       # a bfloat16 run keeps a gate row and its up row in turn
        K.moe_experts(x.to(tdt).to(DEV), torch.stack([wg, wu], dim=2).to(tdt).to(DEV).contiguous(), wd.to(tdt).to(DEV), ids, wts, res,
                      interleaved=True)
    for m in range(M):
        chosen, weights = P.route(wr @ x[m] + b, top)
        assert ids[m].tolist() == chosen and ids2[m].tolist() == chosen, m
        assert max(abs(a - c) for a, c in zip(wts[m].tolist(), weights)) <= 2e-6
        assert max(abs(a - c) for a, c in zip(wts2[m].tolist(), weights)) <= 2e-6
        y = sum(w_ * P.gated_ff(x[m:m + 1], wg[e], wu[e], wd[e])[0] for e, w_ in zip(chosen, weights))
        tol = 2e-5 if dtype == "float32" else 2e-2
        assert (res[m].double().cpu() - res0[m] - y).abs().max().item() <= tol * max(1.0, y.abs().max().item()), m


@pytest.mark.parametrize("E,top,d,F,M", [(5, 2, 64, 24, 300), (3, 3, 48, 16, 77), (4, 1, 128, 40, 513), (12, 4, 96, 72, 1000),
                                          (6, 2, 256, 136, 2100), (5, 2, 64, 24, 1), (16, 3, 128, 64, 8), (4, 2, 128, 256, 4500)])
def test_experts_as_grouped_tensor_core_products(E, top, d, F, M):
    """The pairs ordered by expert, two grouped products, from one token to thousands (token tiles of 16 to
    256 rows; from 128 on the persistent kernel).  Routing is skewed (one expert takes most tokens, one may
    take none), so tiles of every fill occur."""
    from rustyllm_b200 import kernels as K
    g = torch.Generator().manual_seed(E * 7 + M)
    rnd = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).double()
    x = rnd(M, d)
    wg, wu, wd = (t.to(torch.bfloat16).double() for t in (rnd(E, F, d) / math.sqrt(d), rnd(E, F, d) / math.sqrt(d), rnd(E, d, F) / math.sqrt(F)))
    bias = torch.zeros(E, dtype=torch.float64)
    bias[0], bias[-1] = 3.0, -30.0 if E > top else 0.0
    wr = (rnd(E, d) / math.sqrt(d)).to(torch.bfloat16).double()
    ids = torch.empty((M, top), dtype=torch.int32, device=DEV)
    wts = torch.empty((M, top), dtype=torch.float32, device=DEV)
    xb = x.to(torch.bfloat16).to(DEV)
    K.moe_route(xb, wr.to(torch.bfloat16).to(DEV), bias.float().to(DEV), top, ids, wts)
    res = torch.zeros((M, d), dtype=torch.float32, device=DEV)
    gu = torch.stack([wg, wu], dim=2).to(torch.bfloat16).to(DEV).contiguous()          # [E, F, 2, d]
    assert K.moe_experts_grouped_supported(xb, gu, wd.to(torch.bfloat16).to(DEV))
    K.moe_experts_grouped(xb, gu, wd.to(torch.bfloat16).to(DEV), ids, wts, res)
    K.check_device_errors()
    same = torch.zeros((M, d), dtype=torch.float32, device=DEV)
    K.moe_experts(xb, gu, wd.to(torch.bfloat16).to(DEV), ids, wts, same, interleaved=True)
    ids_h, wts_h = ids.cpu(), wts.double().cpu()
    counts = torch.bincount(ids_h.flatten().long(), minlength=E)
    assert E == top or counts.max().item() > 2 * counts.min().item()
    ref = torch.zeros(M, d, dtype=torch.float64)
    for e in range(E):
        for c in range(top):
            rows = (ids_h[:, c] == e).nonzero().flatten()
            if rows.numel():
                ref[rows] += wts_h[rows, c:c + 1] * P.gated_ff(x[rows], wg[e], wu[e], wd[e])
    scale = ref.abs().max().item()
    assert (res.double().cpu() - ref).abs().max().item() <= 2e-2 * scale
    assert (same.double().cpu() - ref).abs().max().item() <= 2e-2 * scale


def test_embedding_with_positions_pass_entry_soft_cap_and_gate_alone():
    from rustyllm_b200 import kernels as K
    g = torch.Generator().manual_seed(5)
    V, Pn, d, M = 31, 50, 40, 9
    for tdt in (torch.float32, torch.bfloat16):
        table, pos = torch.randn(V, d, generator=g).to(tdt), torch.randn(Pn, d, generator=g).to(tdt)
        ids = torch.randint(0, V, (M,), generator=g).int()
        where = torch.randint(0, Pn, (M,), generator=g).int()
        out = torch.empty((M, d), dtype=torch.float32, device=DEV)
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        K.embedding_pos(table.to(DEV), pos.to(DEV), ids.to(DEV), where.to(DEV), out, err)
        ref = torch.stack([table[int(t)].double() + pos[int(p)].double() for t, p in zip(ids, where)])
        assert (out.double().cpu() - ref).abs().max().item() <= 1e-6 and int(err.item()) == 0
        K.embedding_pos(table.to(DEV), pos.to(DEV), ids.to(DEV), (where + Pn).to(DEV), out, err)
        assert int(err.item()) == 2                      # a position beyond the table is refused, not read
    x = torch.randn(M, d, generator=g)
    again, vec = torch.randn(M, d, generator=g), torch.randn(d, generator=g)
    for a, v_ in ((again, vec), (None, vec), (again, None)):
        y = x.clone().to(DEV)
        K.residual_inject(y, None if a is None else a.to(DEV), None if v_ is None else v_.to(DEV))
        ref = x.double() + (0 if a is None else a.double()) + (0 if v_ is None else v_.double())
        assert (y.double().cpu() - ref).abs().max().item() <= 1e-6
    z = (torch.randn(M, d, generator=g) * 20).to(DEV)
    ref = P.soft_cap(z.double().cpu(), 7.5)
    K.softcap(z, 7.5)
    assert (z.double().cpu() - ref).abs().max().item() <= 2e-6
    y, gt = torch.randn(M, d, generator=g), torch.randn(M, 2 * d, generator=g)
    yy = y.clone().to(DEV)
    K.sigmoid_gate(yy, gt.to(DEV)[:, d:])
    assert (yy.double().cpu() - y.double() / (1 + torch.exp(-gt[:, d:].double()))).abs().max().item() <= 1e-6


@pytest.mark.parametrize("name", NAMES)
def test_the_residual_after_every_layer_run_in_32_bit(dirs, name):
    """Layer by layer: the decoder's stream after each run of a block against the plain implementation's."""
    d = dirs[name]
    cfg, w = _plain(d)
    r = runner(d, "float32")
    toks = random_tokens(cfg["vocab"], 75, 11)
    want = []
    P.forward(cfg, w, toks, want)
    got = []
    blocks = r.model.blocks
    originals = [b.forward for b in blocks]
    try:
        for b, f in zip(blocks, originals):
            def wrapped(x, step, cache, *a, _f=f, **kw):
                out = _f(x, step, cache, *a, **kw)
                got.append(x.double().cpu())
                return out
            b.forward = wrapped
        s = r.engine.alloc_slot()
        r.engine.step([s], [toks], None)
        r.engine.free_slot(s)
    finally:
        for b, f in zip(blocks, originals):
            b.forward = f
    assert len(got) == len(want) == layer_runs(cfg)
    for i, (a, b_) in enumerate(zip(got, want)):
        assert (a - b_).abs().max().item() <= 3e-5 * b_.abs().max().item(), f"{name}: after layer run {i}"


# =========================================================================== the engine
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_and_first_tokens(dirs, name, dtype):
    d = dirs[name]
    cfg, _ = _plain(d)
    r = runner(d, dtype)
    for seed, n in enumerate([1, 2, 3, 17, 64, 65, 129, 150]):
        toks = random_tokens(cfg["vocab"], n, 100 + seed)
        s = r.engine.alloc_slot()
        got = r.engine.step([s], [toks], "all")
        r.engine.free_slot(s)
        close(got, plain_logits(d, toks), dtype, cfg, f"{name} whole n={n}")
    r.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_token_by_token_with_windows_passing_over_decoded_tokens(dirs, name, dtype):
    d = dirs[name]
    cfg, _ = _plain(d)
    r = runner(d, dtype)
    for n, tail in ((40, 39), (150, 90), (200, 32)):
        toks = random_tokens(cfg["vocab"], n, 200 + n)
        s = r.engine.alloc_slot()
        rows = [r.engine.step([s], [toks[:n - tail]], "all")]
        for t in toks[n - tail:]:
            rows.append(r.engine.step([s], [[t]], "last"))
        r.engine.free_slot(s)
        close(torch.cat(rows), plain_logits(d, toks), dtype, cfg, f"{name} n={n} last {tail} one by one")
    r.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("portion", [2, 3, 7, 64, 100])
def test_a_prompt_in_portions(dirs, name, dtype, portion):
    d = dirs[name]
    cfg, _ = _plain(d)
    r = runner(d, dtype)
    n = 131 if portion < 7 else 197
    toks = random_tokens(cfg["vocab"], n, 300 + portion)
    s = r.engine.alloc_slot()
    rows = [r.engine.step([s], [toks[i:i + portion]], "all") for i in range(0, n, portion)]
    r.engine.free_slot(s)
    close(torch.cat(rows), plain_logits(d, toks), dtype, cfg, f"{name} portions of {portion}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_equal_each_request_alone_and_reuse_slots_and_pages(dirs, name, dtype):
    """Two batches through a cache that only just holds one: prompts of unequal lengths in one step, decoded
    together, the shorter requests ending earlier; the second batch gets the first one's slots and pages
    with what they held."""
    d = dirs[name]
    cfg, _ = _plain(d)
    from rustyllm_b200 import Runner
    r, _ = Runner.from_path(d, dtype=dtype, max_cache_tokens=64 * 7, max_batch=4)
    eng = r.engine
    for batch_no, (lens, total) in enumerate([([5, 70, 17, 1], [13, 140, 17, 30]), ([64, 3, 130], [66, 90, 141])]):
        seqs = [random_tokens(cfg["vocab"], t, 400 + 10 * batch_no + i) for i, t in enumerate(total)]
        slots = [eng.alloc_slot() for _ in seqs]
        assert sorted(slots) == list(range(len(seqs))), "freed slots are handed out again, lowest first"
        got = [[] for _ in seqs]
        out = eng.step(slots, [s[:n] for s, n in zip(seqs, lens)], "all")
        o = 0
        for i, n in enumerate(lens):
            got[i].append(out[o:o + n])
            o += n
        at = list(lens)
        live = [i for i in range(len(seqs)) if at[i] < total[i]]
        for i in range(len(seqs)):
            if i not in live:
                eng.free_slot(slots[i])
        while live:
            out = eng.step([slots[i] for i in live], [[seqs[i][at[i]]] for i in live], "last")
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
                at[i] += 1
            for i in [i for i in live if at[i] == total[i]]:
                eng.free_slot(slots[i])
            live = [i for i in live if at[i] < total[i]]
        for i, s in enumerate(seqs):
            close(torch.cat(got[i]), plain_logits(d, s), dtype, cfg, f"{name} batch {batch_no} request {i}")
        r.cache.check()
    assert r.cache.free_pages == r.cache.num_pages


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_long_decoding_from_the_first_token(dirs, name, dtype):
    """One token, then 260 more one by one: across four page borders and, in windowed layers, with pages given
    back on the way; the captured single-token step takes over after the first eager one."""
    d = dirs[name]
    cfg, _ = _plain(d)
    n = min(261, cfg["max_positions"])
    r = runner(d, dtype)
    toks = random_tokens(cfg["vocab"], n, 77)
    s = r.engine.alloc_slot()
    rows = [r.engine.step([s], [[t]], "last") for t in toks]
    r.engine.free_slot(s)
    close(torch.cat(rows), plain_logits(d, toks), dtype, cfg, f"{name} {n} single tokens")
    r.cache.check()


@pytest.mark.parametrize("name", NAMES)
def test_logits_do_not_depend_on_the_batch_or_the_cut_in_32_bit(dirs, name):
    """The same request alone and whole, beside others, and in portions: equal to a few float32 roundings."""
    d = dirs[name]
    cfg, _ = _plain(d)
    r = runner(d, "float32")
    a, b, c = (random_tokens(cfg["vocab"], n, 500 + n) for n in (90, 33, 141))
    s = r.engine.alloc_slot()
    alone = r.engine.step([s], [a], "all")
    r.engine.free_slot(s)
    slots = [r.engine.alloc_slot() for _ in range(3)]
    first = r.engine.step(slots, [b, a[:50], c], [[], list(range(50)), []])
    second = r.engine.step(slots[1:], [a[50:], [1, 2]], [list(range(40)), []])
    for s in slots:
        r.engine.free_slot(s)
    both = torch.cat([first, second])
    assert (both - alone).abs().max().item() <= 1e-5 * alone.abs().max().item()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_runner(dirs, name, dtype):
    """Prompts of unequal lengths through ``Runner.generate`` (its batches, prompt step, captured decode steps,
    sampler at temperature 0) against the plain greedy loop.  In bfloat16 a step whose two best logits lie
    within rounding of one another may pick the other token; from there on the texts differ, so the
    comparison ends there (and must not end at once)."""
    from rustyllm_b200 import GenerationOptions, SamplerConfig
    d = dirs[name]
    cfg, w = _plain(d)
    r = runner(d, dtype, 64 * 12, 3)
    prompts = [random_tokens(cfg["vocab"], n, 600 + n) for n in (1, 40, 9, 75, 12)]
    new = 12
    results = r.generate(prompts, GenerationOptions(max_tokens=new, sampler=SamplerConfig.greedy(), seed=1, ignore_eos=True))
    for p, res in zip(prompts, results):
        got = list(res.token_ids)
        assert len(got) == new
        if dtype == "float32":
            assert got == P.greedy(cfg, w, p, new)
        else:
            toks = list(p)
            for i, t in enumerate(got):
                row = P.forward(cfg, w, toks)[-1]
                best = int(row.argmax())
                if t != best:
                    assert float(row[best] - row[t]) <= 0.05 * float(row.std()), (name, i)
                    break
                toks.append(t)
    r.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_of_short_requests_with_the_cache_sized_by_their_tokens(dirs, tmp_path, dtype):
    """``bin/trace_run`` as a subprocess: nine requests of 3 to 40 tokens in one batch, decoded together, the
    shorter ones ending earlier; ``--max-tokens`` is the number of tokens the live requests hold at most - not
    rounded to pages, of which every request needs a last, partly empty one."""
    from test_trace_gpu import read_step, run_trace
    d = dirs["S"]
    cfg, _ = _plain(d)
    V = cfg["vocab"]
    lens = [3, 40, 7, 12, 5, 33, 9, 21, 4]
    extra = [0, 6, 2, 9, 1, 4, 9, 3, 5]
    reqs = [random_tokens(V, n + e, 900 + i) for i, (n, e) in enumerate(zip(lens, extra))]
    steps = [{"step": 0, "entries": [{"id": f"q{i}", "tokens": r[:n], "want": [0, n - 1]} for i, (r, n) in enumerate(zip(reqs, lens))],
              "end": [f"q{i}" for i, e in enumerate(extra) if e == 0]}]
    expect = {0: [(i, [0, n - 1]) for i, n in enumerate(lens)]}
    for k in range(max(extra)):
        live = [i for i, e in enumerate(extra) if e > k]
        steps.append({"step": k + 1, "entries": [{"id": f"q{i}", "tokens": [reqs[i][lens[i] + k]], "want": [0]} for i in live],
                      "end": [f"q{i}" for i in live if extra[i] == k + 1]})
        expect[k + 1] = [(i, [lens[i] + k]) for i in live]
    out_dir = str(tmp_path / dtype)
    run_trace(d, dtype, steps, out_dir, max_tokens=sum(len(r) for r in reqs))
    for step, exp in expect.items():
        got = read_step(out_dir, step, V)
        ref = torch.cat([plain_logits(d, reqs[i])[pos] for i, pos in exp])
        close(got, ref, dtype, cfg, f"step {step}")


def test_command_line_generates_benchmarks_and_times_kernels(dirs, capsys, tmp_path):
    """``bin/rustyllm``'s entry point on a Mosurax folder: greedy ids equal the plain loop's, the benchmark and the
    kernel benchmark run (the latter on a layer of experts and on a dense one, from random weights)."""
    import json
    from rustyllm_b200 import cli
    d = dirs["P"]
    cfg, w = _plain(d)
    prompt = random_tokens(cfg["vocab"], 9, 81)
    assert cli.main([d, "--dtype", "float32", "-p", " ".join(map(str, prompt)), "-n", "5", "-t", "0", "--ignore-eos"]) == 0
    assert [int(t) for t in capsys.readouterr().out.split()] == P.greedy(cfg, w, prompt, 5)
    assert cli.main([d, "--bench-json", "--bench-runs", "2", "--batch", "3", "--prompt-len", "20", "-n", "4", "--seed", "5", "--ignore-eos"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["architecture"] == "Mosurax" and rep["results"][0]["prompt_tokens"] == 60 and rep["results"][0]["generated_tokens"] == 12
    for layer, names in ((0, ("attn_qkv.fused", "ffn_gate_up.fused", "ffn_down", "attn_scan.ctx128")),
                         (1, ("ffn_router", "ffn_experts.chosen", "ffn_shared_gate_up.fused", "output"))):
        assert cli.main([d, "--random", "--kernel-bench-json", "--kernel-bench-runs", "3", "--kernel-bench-layer", str(layer)]) == 0
        rows = {r["name"]: r for r in json.loads(capsys.readouterr().out)["rows"]}
        for name in names:
            assert rows[name]["avg_us"] > 0, name
