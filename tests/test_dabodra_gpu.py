"""Dabodra on the GPU against the plain implementation: each kernel and each mechanism alone, whole prompts against
token-by-token decoding, prompts fed in portions, unequal batches, pages and slots used again, keys just inside and
just outside a window in prompts and in decoding, the sink, the first tokens, long decoding across windows and pages,
state carried by the delta rule, generation through the entry point."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from dabodra_helpers import (assert_rows_close as assert_close, attention, clear_tokens, config, delta, layer, make,
                             plain_logits)
from helpers import TOL
from plain import dabodra_plain as D

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def _engine(path, dtype, max_tokens=1024):
    from stratum_b200.engine import Engine, load_model
    model, _ = load_model(path, torch.float32 if dtype == "float32" else torch.bfloat16, "cuda")
    return Engine(model, max_tokens=max_tokens)


@pytest.fixture(scope="module", params=[(n, d) for n in ("A", "B", "TC") for d in DTYPES], ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, tmp_path_factory):
    name, dtype = request.param
    path, cfg, w = make(str(tmp_path_factory.mktemp(f"dab{name}_{dtype}")), name, dtype, seed=len(name) + 1)
    return name, dtype, cfg, w, _engine(path, dtype), path


def _dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype).cuda()


# ------------------------------------------------------------------------------------------ kernels alone
def test_norm_into_residual_kernel():
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(0)
    for rows, width in ((1, 72), (5, 70), (300, 512), (3, 4100)):
        y, x, w = rng.standard_normal((rows, width)) * 3, rng.standard_normal((rows, width)), rng.uniform(-0.4, 0.4, width)
        want = x + D.one_plus_norm(y, w, 1e-5)
        xd, copy = _dev(x), torch.empty(rows, width, dtype=torch.bfloat16, device="cuda")
        K.norm_into_residual(_dev(y), _dev(1.0 + w), 1e-5, xd, True, copy)
        assert np.max(np.abs(xd.cpu().numpy() - want)) <= 2e-6 * np.max(np.abs(want))
        assert torch.equal(copy, xd.to(torch.bfloat16))
        yd = _dev(y)
        K.norm_into_residual(yd, _dev(1.0 + w), 1e-5, yd, False, None)           # in place, nothing added
        assert np.max(np.abs(yd.cpu().numpy() - D.one_plus_norm(y, w, 1e-5))) <= 2e-6 * np.max(np.abs(want))


@pytest.mark.parametrize("heads,kv,dim,rot", [(6, 2, 24, 16), (3, 3, 20, 6), (4, 1, 64, 64), (2, 2, 16, 0)])
def test_qk_norm_rope_kernel(heads, kv, dim, rot):
    """Queries and keys normalised over their whole rows, rotated in neighbouring pairs, keys appended to pages that
    lie anywhere, the values the keys as projected."""
    from stratum_b200 import kernels as K
    from stratum_b200.parts.rope import inverse_frequencies
    rng = np.random.default_rng(dim)
    T, pages = 9, 5
    pos = np.array([0, 1, 2, 63, 64, 65, 130, 131, 191])
    proj = rng.standard_normal((T, (heads + kv) * dim + 3))
    qg, kg = rng.uniform(0.5, 1.5, heads * dim), rng.uniform(0.5, 1.5, kv * dim)
    table = np.array([[4, 0, 2]], dtype=np.int32)
    q_out = torch.zeros(T, heads * dim + 8, device="cuda")
    kc, vc = torch.zeros(pages, kv, 64, dim, device="cuda"), torch.zeros(pages, kv, 64, dim, device="cuda")
    inv = torch.from_numpy(inverse_frequencies(rot, 777.0, None)[0]).cuda() if rot else None
    K.qk_norm_rope(_dev(proj), _dev(pos, torch.int32), torch.zeros(T, dtype=torch.int32, device="cuda"),
                   _dev(table, torch.int32), _dev(qg), _dev(kg), inv, 1e-5, q_out, kc, vc, heads, kv, dim, 64, True)
    q_raw, k_raw = proj[:, :heads * dim], proj[:, heads * dim:(heads + kv) * dim]
    q = D.rms_norm(q_raw, qg, 1e-5).reshape(T, heads, dim)
    k = D.rms_norm(k_raw, kg, 1e-5).reshape(T, kv, dim)
    if rot:
        q, k = D.rotate_pairs(q, pos, 777.0, rot), D.rotate_pairs(k, pos, 777.0, rot)
    tol = 3e-5                                           # float32 angles of positions near 200
    assert np.max(np.abs(q_out[:, :heads * dim].cpu().numpy() - q.reshape(T, -1))) <= tol * np.max(np.abs(q))
    for t in range(T):
        page, row = table[0, pos[t] // 64], pos[t] % 64
        assert np.max(np.abs(kc[page, :, row].cpu().numpy() - k[t])) <= tol * np.max(np.abs(k))
        assert np.max(np.abs(vc[page, :, row].cpu().numpy() - k_raw[t].reshape(kv, dim))) <= 1e-6
    assert float(kc[1].abs().max()) == 0.0 and float(kc[3].abs().max()) == 0.0            # pages of nobody stay clean


@pytest.mark.parametrize("experts,top,groups,keep", [(6, 2, 3, 2), (8, 3, 1, 1), (12, 4, 4, 2), (4, 1, 4, 2), (5, 5, 1, 1)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_router_kernel(experts, top, groups, keep, dtype):
    """The chosen experts and their weights; corrections push every choice score below zero for half of the tokens,
    where a closed group that counted as 0 instead of minus infinity would win."""
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(experts * 10 + top)
    T, W = 40, 72
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    h = _dev(rng.standard_normal((T, W)), td)
    hp = h.float().cpu().numpy().astype(np.float64)
    wr = _dev(rng.standard_normal((experts, W)) * 0.3)
    r = {"experts": experts, "top": top, "scale": 1.7, "groups": {"count": groups, "keep": keep}}
    for shift in (0.0, -3.0):
        corr = _dev(rng.uniform(-0.5, 0.5, experts) + shift)
        dense = torch.full((T, experts + 2), 7.0, device="cuda")
        chosen = torch.zeros(T, top, dtype=torch.int32, device="cuda")
        weights = torch.zeros(T, top, device="cuda")
        K.moe_route(h, wr, corr, dense, chosen, weights, top, groups, keep, 1.7)
        margins = []
        want_c, want_w = D.route(hp, wr.cpu().numpy(), corr.cpu().numpy(), r, margins)
        chosen, weights, dense = chosen.cpu().numpy(), weights.cpu().numpy(), dense.cpu().numpy()
        per_token = max(1, len(margins) // T)
        for t in range(T):
            if min(margins[t * per_token:(t + 1) * per_token], default=1.0) < 1e-4:
                continue                                 # a tie within rounding: either choice is right
            assert list(chosen[t]) == list(want_c[t]), (t, chosen[t], want_c[t])
            np.testing.assert_allclose(weights[t], want_w[t], rtol=2e-5)
            row = np.zeros(experts)
            row[want_c[t]] = want_w[t]
            np.testing.assert_allclose(dense[t, :experts], row, rtol=2e-5)
            assert (dense[t, experts:] == 7.0).all()


@pytest.mark.parametrize("heads,kv,dim,vdim,taps", [(4, 2, 24, 40, 3), (3, 3, 40, 16, 5), (2, 1, 64, 32, 4), (1, 1, 8, 8, 1),
                                                    (2, 2, 130, 70, 2), (4, 2, 128, 36, 4), (1, 1, 260, 12, 2),
                                                    (2, 1, 100, 24, 3)])
@pytest.mark.parametrize("long", [77, 520])
def test_delta_rule_kernels(heads, kv, dim, vdim, taps, long):
    """The three kernels of the delta rule on projections made here: two sequences of unequal lengths whose tokens
    come in three steps (many, three and two, one), states in slots that lie apart, against the plain loop over whole
    sequences."""
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(dim + vdim)
    C = 2 * kv * dim + heads * vdim
    width = C + 2 * heads + heads * vdim
    lens = (long, 9)               # 520: dozens of staged token groups in the recurrence
    proj = [rng.standard_normal((n, width)) for n in lens]
    conv = rng.uniform(-0.8, 0.8, (C, taps))
    a_log, dt_bias, gain = rng.uniform(-2, 0.5, heads), rng.uniform(-1, 1, heads), rng.uniform(0.5, 1.5, vdim)
    # the plain loop, fed the projections directly: identity matrices in place of the weights
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": taps}
    eye = np.eye(width)
    w = {"q": eye[:kv * dim], "k": eye[kv * dim:2 * kv * dim], "v": eye[2 * kv * dim:C], "b": eye[C:C + heads],
         "a": eye[C + heads:C + 2 * heads], "g": eye[C + 2 * heads:], "q.conv": conv[:kv * dim],
         "k.conv": conv[kv * dim:2 * kv * dim], "v.conv": conv[2 * kv * dim:], "A_log": a_log, "dt_bias": dt_bias,
         "norm": gain, "o": np.eye(heads * vdim)}
    want = [D.gated_delta(p, w, m, 1e-5) for p in proj]
    n_state = heads * dim * vdim + (taps - 1) * C
    state = torch.zeros(6, n_state, device="cuda")
    slots = (4, 1)
    done = [0, 0]
    got = [[], []]
    for cut in ((long - 4, 6), (3, 2), (1, 1)):
        rows_ = np.concatenate([proj[i][done[i]:done[i] + cut[i]] for i in range(2)])
        T = rows_.shape[0]
        pos = np.concatenate([np.arange(done[i], done[i] + cut[i]) for i in range(2)])
        seq = np.concatenate([np.full(cut[i], i) for i in range(2)])
        start = np.array([0, cut[0], T])
        act = torch.empty(T, C + 2 * heads + kv, device="cuda")
        o_raw = torch.empty(T, heads * vdim, device="cuda")
        out = torch.empty(T, heads * vdim, device="cuda")
        K.delta_rule(_dev(rows_), _dev(conv), _dev(a_log), _dev(dt_bias), _dev(gain), act, o_raw, out, state,
                     _dev(pos, torch.int32), _dev(seq, torch.int32), _dev(start, torch.int32),
                     _dev(np.array(slots), torch.int32), heads, kv, dim, vdim, 1e-5, True)
        o = out.cpu().numpy()
        got[0].append(o[:cut[0]]); got[1].append(o[cut[0]:])
        done = [done[i] + cut[i] for i in range(2)]
    for i in range(2):
        g = np.concatenate(got[i])
        assert np.max(np.abs(g - want[i])) <= 3e-5 * np.max(np.abs(want[i])), (i, np.max(np.abs(g - want[i])))
    assert float(state[0].abs().max()) == 0.0 and float(state[5].abs().max()) == 0.0


def test_general_attention_with_sink_and_window_both_kernels():
    """The CUDA-core and the tensor-core general attention with a window and a sink against a plain softmax, for
    prompt rows and single rows at positions around the window's edge and the pages' borders."""
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(5)
    heads, kv, dim, window, n = 4, 2, 32, 70, 200
    keys, vals = rng.standard_normal((n, kv, dim)), rng.standard_normal((n, kv, dim))
    sink = rng.uniform(-1, 2, heads)
    table = np.array([[3, 1, 0, 2]], dtype=np.int32)
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 2e-2)):
        kc, vc = torch.zeros(4, kv, 64, dim, dtype=dtype, device="cuda"), torch.zeros(4, kv, 64, dim, dtype=dtype, device="cuda")
        for t in range(n):
            kc[table[0, t // 64], :, t % 64] = _dev(keys[t], dtype)
            vc[table[0, t // 64], :, t % 64] = _dev(vals[t], dtype)
        kq, vq = kc.float().cpu().numpy().astype(np.float64), vc.float().cpu().numpy().astype(np.float64)
        shape = K.AttentionShape(heads, heads // kv, 1, dim, dim, False, 0.3, window=window, sink=_dev(sink))
        for rows in (list(range(120, 200)), [199], [69], [70], [0]):
            q = _dev(rng.standard_normal((len(rows), heads * dim)), dtype)
            qp = q.float().cpu().numpy().astype(np.float64).reshape(len(rows), heads, dim)
            pos, seq = _dev(np.array(rows), torch.int32), torch.zeros(len(rows), dtype=torch.int32, device="cuda")
            want = np.zeros((len(rows), heads, dim))
            for i, p in enumerate(rows):
                for h in range(heads):
                    js = np.arange(max(0, p - window + 1), p + 1)
                    kk = np.stack([kq[table[0, j // 64], h // 2, j % 64] for j in js])
                    vv = np.stack([vq[table[0, j // 64], h // 2, j % 64] for j in js])
                    s = np.append(kk @ qp[i, h] * 0.3, sink[h])
                    a = np.exp(s - s.max()); a /= a.sum()
                    want[i, h] = a[:-1] @ vv
            out = torch.zeros(len(rows), heads * dim, dtype=dtype, device="cuda")
            K.attention_general(shape, q, kc, vc, pos, seq, _dev(table, torch.int32), out, 64)
            assert np.max(np.abs(out.float().cpu().numpy().reshape(want.shape) - want)) <= tol * np.max(np.abs(want))
            if dtype == torch.bfloat16:
                out2 = torch.zeros_like(out)
                if len(rows) == 1:
                    n_splits, chunk = 4, 64
                    part_o = torch.empty(heads * n_splits * dim, device="cuda")
                    part_ml = torch.empty(heads * n_splits * 2, device="cuda")
                    K.attention_general_mma(shape, q, kc, vc, pos, seq, _dev(table, torch.int32), out2, 64, None, 8,
                                            n_splits, chunk, part_o, part_ml)
                else:
                    qb = (torch.zeros(10, dtype=torch.int32, device="cuda"),
                          torch.arange(0, 80, 8, dtype=torch.int32, device="cuda"),
                          torch.full((10,), 8, dtype=torch.int32, device="cuda"))
                    K.attention_general_mma(shape, q, kc, vc, pos, seq, _dev(table, torch.int32), out2, 64, qb, 8, 1, 256,
                                            None, None)
                assert np.max(np.abs(out2.float().cpu().numpy().reshape(want.shape) - want)) <= tol * np.max(np.abs(want))


# ------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["att", "delta", "moe"])
def test_one_mechanism_alone(name, dtype, tmp_path):
    from stratum_b200.engine import StepEntry
    path, cfg, w = make(str(tmp_path / name), name, dtype, seed=7)
    engine = _engine(path, dtype)
    toks = clear_tokens(np.random.default_rng(1), 90, cfg, w, dtype)
    slot = engine.acquire()
    got = engine.step([StepEntry(slot, toks, list(range(90)))]).cpu().numpy()
    engine.release(slot)
    assert_close(got, plain_logits(cfg, w, toks), dtype, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["moe", "A", "TC"])
def test_experts_both_ways(name, dtype, tmp_path, monkeypatch):
    """The experts run on stretches of gathered rows (the way of long prompts, here forced on short ones) and as two
    stacked products (the way of decode steps): both against the plain implementation, and against one another."""
    from stratum_b200.engine import StepEntry
    from stratum_b200.parts import moe as M
    path, cfg, w = make(str(tmp_path / name), name, dtype, seed=5)
    engine = _engine(path, dtype)
    n = 150
    toks = clear_tokens(np.random.default_rng(6), n, cfg, w, dtype)
    ref = plain_logits(cfg, w, toks)
    got = {}
    for way, rows in (("stacked", 1 << 30), ("grouped", 0)):
        monkeypatch.setattr(M, "GROUPED_MIN_ROWS", rows)
        slot = engine.acquire()
        a = engine.step([StepEntry(slot, toks[:97], list(range(97)))]).cpu().numpy()
        b = engine.step([StepEntry(slot, toks[97:], list(range(n - 97)))]).cpu().numpy()
        engine.release(slot)
        got[way] = np.concatenate([a, b])
        assert_close(got[way], ref, dtype, f"{name} experts {way}")
    if dtype == "float32":
        assert np.max(np.abs(got["stacked"] - got["grouped"])) <= 2e-5 * np.max(np.abs(ref))


def test_grouping_kernels():
    """Pairs in the order of their experts, tokens in order within an expert; rows gathered; outputs combined."""
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(2)
    T, top, E, W = 700, 3, 7, 40
    chosen = np.stack([rng.permutation(E)[:top] for _ in range(T)]).astype(np.int32)
    counts, order, where = K.moe_group(_dev(chosen, torch.int32), E)
    counts, order, where = counts.cpu().numpy(), order.cpu().numpy(), where.cpu().numpy()
    flat = chosen.reshape(-1)
    assert list(counts) == [int(np.sum(flat == e)) for e in range(E)]
    want = np.argsort(flat, kind="stable")
    assert list(order) == list(want) and list(where[order]) == list(range(T * top))
    x = rng.standard_normal((T, W))
    rows = torch.empty(T * top, W, device="cuda")
    K.gather_rows(_dev(x), _dev(order, torch.int32), top, rows)
    assert np.array_equal(rows.cpu().numpy(), x.astype(np.float32)[order // top])
    outs, wts = rng.standard_normal((T * top, W)), rng.uniform(0, 1, (T, top))
    y = _dev(rng.standard_normal((T, W)))
    base = y.cpu().numpy().astype(np.float64)
    K.moe_combine(_dev(outs), _dev(where, torch.int32), _dev(wts), y, True)
    ref = base + np.einsum("tk,tkw->tw", wts, outs.astype(np.float32).astype(np.float64)[where.reshape(T, top)])
    assert np.max(np.abs(y.cpu().numpy() - ref)) <= 1e-5 * np.max(np.abs(ref))


# ------------------------------------------------------------------------------------------ whole models
def test_whole_prompt_all_positions(setup):
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine, _ = setup
    rng = np.random.default_rng(1)
    for n in (1, 2, 5, 6, 37, 38, 63, 64, 65, 200):
        toks = clear_tokens(rng, n, cfg, w, dtype)
        slot = engine.acquire()
        got = engine.step([StepEntry(slot, toks, list(range(n)))]).cpu().numpy()
        engine.release(slot)
        assert_close(got, plain_logits(cfg, w, toks), dtype, f"{name} whole n={n}")
    engine.cache.check()


def test_prefill_against_token_by_token(setup):
    """The same tokens whole, and one by one from the first: the same logits (float32: to rounding)."""
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine, _ = setup
    n = 150
    toks = clear_tokens(np.random.default_rng(2), n, cfg, w, dtype)
    a, b = engine.acquire(), engine.acquire()
    whole = engine.step([StepEntry(a, toks, list(range(n)))]).cpu().numpy()
    single = np.concatenate([engine.step([StepEntry(b, [t], [0])]).cpu().numpy() for t in toks])
    engine.release(a); engine.release(b)
    ref = plain_logits(cfg, w, toks)
    assert_close(whole, ref, dtype, f"{name} whole")
    assert_close(single, ref, dtype, f"{name} one by one")
    if dtype == "float32":
        assert np.max(np.abs(whole - single)) <= 2e-5 * np.max(np.abs(ref))


def test_the_same_bits_every_run(setup):
    """A batch of prompts and some decoded tokens, three times over in slots, pages and state rows that were just given
    back: every run's logits are the same bits (the small kernels begin while the kernel before them still runs; a
    value read too early, or a sum whose order depends on timing, would show here)."""
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine, _ = setup
    rng = np.random.default_rng(17)
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab"], n)] for n in (90, 7, 64, 33)]
    more = [[int(t) for t in rng.integers(0, cfg["vocab"], 6)] for _ in prompts]
    runs = []
    for _ in range(3):
        slots = [engine.acquire() for _ in prompts]
        got = [engine.step([StepEntry(s, p, list(range(len(p)))) for s, p in zip(slots, prompts)]).cpu().numpy()]
        for i in range(6):
            got.append(engine.step([StepEntry(s, [m[i]], [0]) for s, m in zip(slots, more)]).cpu().numpy())
        for s in slots:
            engine.release(s)
        runs.append(np.concatenate(got))
    assert np.isfinite(runs[0]).all()
    assert np.array_equal(runs[0], runs[1]) and np.array_equal(runs[0], runs[2]), f"{name} {dtype}: runs differ"


@pytest.mark.parametrize("portion", [2, 3, 31, 64, 100])
def test_prompt_in_portions(setup, portion):
    """A prompt cut into portions of a few sizes, down to two tokens (fewer than the convolutions' taps); portions
    start inside pages and windows and on their borders."""
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine, _ = setup
    n = 150 if portion > 3 else 80
    toks = clear_tokens(np.random.default_rng(portion), n, cfg, w, dtype)
    ref = plain_logits(cfg, w, toks)
    slot = engine.acquire()
    got = [engine.step([StepEntry(slot, toks[i:i + portion], list(range(len(toks[i:i + portion]))))]).cpu().numpy()
           for i in range(0, n, portion)]
    engine.release(slot)
    assert_close(np.concatenate(got), ref, dtype, f"{name} portions of {portion}")


def test_unequal_batches_against_each_alone_slots_reused(setup):
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine, _ = setup
    rng = np.random.default_rng(3)
    for batch_no, lens in enumerate([(5, 9, 12), (1, 67), (70, 3, 33, 64)]):
        extra_n = [3 + 2 * i for i in range(len(lens))]
        full = [clear_tokens(rng, n + k, cfg, w, dtype) for n, k in zip(lens, extra_n)]
        prompts = [f[:n] for f, n in zip(full, lens)]
        extra = [f[n:] for f, n in zip(full, lens)]
        refs = [plain_logits(cfg, w, f) for f in full]
        slots = [engine.acquire() for _ in lens]
        out = engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)]).cpu().numpy()
        alone = []
        for p in prompts:                                   # each alone, in a slot and pages of its own
            s = engine.acquire()
            alone.append(engine.step([StepEntry(s, p, [len(p) - 1])]).cpu().numpy()[0])
            engine.release(s)
        for i, p in enumerate(prompts):
            assert_close(out[i], refs[i][len(p) - 1], dtype, f"{name} batch {batch_no} prompt {i}")
            if dtype == "float32":
                assert np.max(np.abs(out[i] - alone[i])) <= 2e-5 * np.max(np.abs(refs[i]))
        live, step = list(range(len(lens))), 0
        while live:
            out = engine.step([StepEntry(slots[i], [extra[i][step]], [0]) for i in live]).cpu().numpy()
            for row, i in enumerate(live):
                assert_close(out[row], refs[i][len(prompts[i]) + step], dtype, f"{name} batch {batch_no} seq {i} +{step}")
            step += 1
            for i in list(live):
                if step >= len(extra[i]):
                    engine.release(slots[i])
                    live.remove(i)
        engine.cache.check()
    assert engine.cache.tokens_held() == 0


def test_pages_and_slots_used_again(setup):
    """A cache of four pages and few slots: every request takes pages and a state row another one has just given
    back (a state row that was not cleared would show at once)."""
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, _, path = setup
    engine = _engine(path, dtype, max_tokens=256)
    rng = np.random.default_rng(4)
    held = []
    for n in (130, 60, 190, 64, 129):
        while held and engine.cache.tokens_held() + ((n + 63) // 64) * 64 > 256:
            engine.release(held.pop(0))
        toks = clear_tokens(rng, n, cfg, w, dtype)
        slot = engine.acquire()
        got = engine.step([StepEntry(slot, toks[:-1], [n - 2])]).cpu().numpy()
        got = np.concatenate([got, engine.step([StepEntry(slot, toks[-1:], [0])]).cpu().numpy()])
        assert_close(got, plain_logits(cfg, w, toks)[-2:], dtype, f"{name} reuse n={n}")
        held.append(slot)
        engine.cache.check()


def test_first_tokens_and_long_decoding(setup):
    """Positions 0, 1, 2 one by one, then on across several pages and many times the windows' lengths; windowed layers
    hand their pages back on the way."""
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine, _ = setup
    n = 270
    toks = clear_tokens(np.random.default_rng(5), n, cfg, w, dtype)
    ref = plain_logits(cfg, w, toks)
    slot = engine.acquire()
    check = {0, 1, 2, 3, 4, 5, 6} | set(range(7, n, 29)) | {36, 37, 38, 63, 64, 65, 69, 70, 71, 127, 128, 129, 130, 131,
                                                             191, 192, 193, n - 1}
    got = []
    for i in range(n):
        out = engine.step([StepEntry(slot, [toks[i]], [0] if i in check else [])])
        if i in check:
            got.append(out.cpu().numpy())
    engine.release(slot)
    assert_close(np.concatenate(got), ref[sorted(check)], dtype, f"{name} long decode")
    engine.cache.check()


# ------------------------------------------------------------------------------------------ a window's edge decides
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,last", [(70, 259), (70, 133), (64, 200), (65, 128), (5, 70), (130, 199)])
def test_a_key_at_the_windows_edge_decides(window, last, dtype, tmp_path_factory):
    """One attention layer under weights that give one marked token a value that towers over all others (the values
    are the keys as projected, so a key matrix that reads one dimension strongly, which only the marked token has, does
    it; the scale is small, so every key in sight gets a fair share).  With the marked token on the window's last place
    the logits are its; one place further out it is invisible and the logits are another matter.  Both must agree
    with the plain implementation, as a whole prompt and with the asking token decoded alone: a window off by one
    fails one of the two."""
    from stratum_b200.engine import StepEntry
    cfg_raw = config([layer("attention", attention(heads=4, kv_heads=2, dim=32, window=window, rot=8, scale=0.05))],
                     vocab=120, width=64)

    def edit(t):
        e = t["embed"].float()
        e[:, 0] = 0.0
        e[7, 0] = 3.0                     # only the marked token (id 7) has anything in the first dimension ...
        t["embed"] = e.to(t["embed"].dtype)
        for name in list(t):
            if name.endswith(".mix.k"):   # ... which its key, and so its value, reads fifty times as strongly
                m = t[name].float()
                m[:, 0] = torch.sign(m[:, 0]) * 6.0
                t[name] = m.to(t[name].dtype)
            if name.endswith(".mix.q"):   # the queries do not read it: nobody's score depends on being marked
                m = t[name].float()
                m[:, 0] = 0.0
                t[name] = m.to(t[name].dtype)
    key = f"edge{window}_{last}_{dtype}"
    path, cfg, w = make(str(tmp_path_factory.mktemp(key)), None, dtype, seed=9, edit=edit, cfg=cfg_raw)
    engine = _engine(path, dtype)
    rng = np.random.default_rng(window + last)
    n = last + 1
    outcomes = []
    for back in (window - 1, window):                       # the last place inside, the first place outside
        toks = [int(t) for t in rng.integers(9, cfg["vocab"], n)]
        toks[last - back] = 7
        ref = plain_logits(cfg, w, toks)[-1]
        outcomes.append(ref)
        slot = engine.acquire()
        whole = engine.step([StepEntry(slot, toks, [n - 1])]).cpu().numpy()[0]
        engine.release(slot)
        slot = engine.acquire()
        engine.step([StepEntry(slot, toks[:n - 1], [])])
        decoded = engine.step([StepEntry(slot, toks[n - 1:], [0])]).cpu().numpy()[0]
        engine.release(slot)
        assert_close(whole, ref, dtype, f"marked token {back} back, whole")
        assert_close(decoded, ref, dtype, f"marked token {back} back, decoded")
        moved = list(toks)
        moved[last - back] = 9
        changed = np.max(np.abs(plain_logits(cfg, w, moved)[-1] - ref)) / np.max(np.abs(ref))
        assert (changed > 0.05) == (back == window - 1), f"the marked token {back} back changes the logits by {changed}"
    assert np.max(np.abs(outcomes[0] - outcomes[1])) > 0.05 * np.max(np.abs(outcomes[0]))


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_sink_takes_its_share(dtype, tmp_path):
    """With a few keys in sight and large sinks most of the softmax's mass goes to the sink: leaving it out, scaling it
    or counting it per key would change the logits wholesale (shown on the plain implementation first)."""
    from stratum_b200.engine import StepEntry
    cfg_raw = config([layer("attention", attention(heads=4, kv_heads=1, dim=16, window=4, rot=4, scale=0.2))], vocab=90, width=48)

    def edit(t):
        for name in list(t):
            if name.endswith(".sink"):
                t[name] = torch.tensor([3.0, -2.0, 1.5, 4.0]).to(t[name].dtype)
    path, cfg, w = make(str(tmp_path / "sink"), None, dtype, seed=2, edit=edit, cfg=cfg_raw)
    toks = [int(t) for t in np.random.default_rng(0).integers(0, 90, 40)]
    ref = plain_logits(cfg, w, toks)
    w2 = dict(w)
    w2["l0.mix.sink"] = np.full(4, -30.0)
    assert np.max(np.abs(plain_logits(cfg, w2, toks) - ref)) > 0.05 * np.max(np.abs(ref))
    engine = _engine(path, dtype)
    slot = engine.acquire()
    got = engine.step([StepEntry(slot, toks[:33], list(range(33)))]).cpu().numpy()
    got = np.concatenate([got] + [engine.step([StepEntry(slot, [t], [0])]).cpu().numpy() for t in toks[33:]])
    assert_close(got, ref, dtype, "sink")


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_delta_state_carries_a_token_from_far_back(dtype, tmp_path):
    """One delta layer with decays close to one: what the first token wrote still shapes the output hundreds of tokens
    later (shown on the plain implementation), through a prompt cut in two and decoded tokens."""
    from stratum_b200.engine import StepEntry
    cfg_raw = config([layer("delta", delta(heads=2, kv_heads=2, dim=16, vdim=24, conv=3))], vocab=90, width=48)

    def edit(t):
        for name in list(t):
            if name.endswith(".A_log"):
                t[name] = torch.full_like(t[name], -7.0)
    path, cfg, w = make(str(tmp_path / "far"), None, dtype, seed=4, edit=edit, cfg=cfg_raw)
    toks = [int(t) for t in np.random.default_rng(1).integers(1, 90, 300)]
    ref = plain_logits(cfg, w, toks)
    other = [0] + toks[1:]
    assert np.max(np.abs(plain_logits(cfg, w, other)[-1] - ref[-1])) > 1e-3 * np.max(np.abs(ref[-1]))
    engine = _engine(path, dtype)
    slot = engine.acquire()
    engine.step([StepEntry(slot, toks[:131], [])])
    got = engine.step([StepEntry(slot, toks[131:290], [158])]).cpu().numpy()
    got = np.concatenate([got] + [engine.step([StepEntry(slot, [t], [0])]).cpu().numpy() for t in toks[290:]])
    assert_close(got, ref[289:], dtype, "delta state from far back")


# ------------------------------------------------------------------------------------------ generation
@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(dtype, tmp_path):
    """Stratum.generate: the scheduler's batches, replayed decode graphs, slots given back; every picked token is the
    plain implementation's best (or within rounding of it)."""
    from stratum_b200 import Stratum
    path, cfg, w = make(str(tmp_path / "gen"), "A", dtype, seed=11)
    rng = np.random.default_rng(0)
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab"], n)] for n in (5, 70, 12, 1)]
    llm = Stratum(path, dtype=dtype, max_tokens=1024)
    res = llm.generate(prompts, max_new_tokens=10, stop_ids=())
    for p, r in zip(prompts, res):
        assert len(r.tokens) == 10
        seq = list(p)
        for tok in r.tokens:
            margins = []
            ref = D.forward(cfg, w, seq, margins=margins)[-1]
            if min(margins) < (1e-4 if dtype == "float32" else 0.04):
                break                                    # a router near a tie: what follows is no test
            assert ref[tok] >= ref.max() - 2 * TOL[dtype] * float(np.max(np.abs(ref))), (p, r.tokens, tok)
            seq.append(tok)
    serial = llm.generate(prompts, max_new_tokens=10, stop_ids=(), max_batch=2)
    if dtype == "float32":
        assert [r.tokens for r in serial] == [r.tokens for r in res]
    llm.engine.cache.check()
    assert llm.engine.cache.tokens_held() == 0


def test_trace_replay_program(tmp_path):
    """`bin/trace_run` fed steps on standard input: a batch of two requests, then single tokens, one request ending
    earlier, then a request that takes the pages and the state row given back."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path, cfg, w = make(str(tmp_path / "lively"), "A", "float32", seed=21)
    rng = np.random.default_rng(8)
    V = cfg["vocab"]
    a, b, c = (clear_tokens(rng, n, cfg, w, "float32") for n in (70, 9, 33))
    ra, rb, rc = (plain_logits(cfg, w, t) for t in (a, b, c))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:60], "want": [0, 59]},
                                     {"id": "b", "tokens": b[:5], "want": []}], "end": []}]
    for i in range(10):
        ents = [{"id": "a", "tokens": [a[60 + i]], "want": [0]}]
        end = ["a"] if i == 9 else []
        if i < 4:
            ents.append({"id": "b", "tokens": [b[5 + i]], "want": [0]})
            if i == 3:
                end.append("b")
        steps.append({"step": 1 + i, "entries": ents, "end": end})
    steps.append({"step": 11, "entries": [{"id": "c", "tokens": c, "want": list(range(33))}], "end": ["c"]})
    out = str(tmp_path / "out")
    p = subprocess.Popen([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", path, "--dtype", "float32",
                          "--out", out, "--max-tokens", "192"], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    for s in steps:
        p.stdin.write(json.dumps(s) + "\n")
        p.stdin.flush()
        assert p.stdout.readline().strip() == f"done {s['step']}"
    p.stdin.close()
    assert p.wait(timeout=600) == 0
    read = lambda n: np.fromfile(os.path.join(out, f"{n}.f32"), dtype="<f4").reshape(-1, V)   # noqa: E731
    assert_close(read(0), ra[[0, 59]], "float32", "trace step 0")
    for i in range(10):
        got = read(1 + i)
        assert_close(got[0], ra[60 + i], "float32", f"trace a {i}")
        if i < 4:
            assert_close(got[1], rb[5 + i], "float32", f"trace b {i}")
    assert_close(read(11), rc, "float32", "trace c")
