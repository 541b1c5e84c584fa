"""Nibelorn on the GPU against the plain implementation: each mechanism alone, whole prompts against token-by-token
decoding, prompts fed in portions, unequal batches, pages and slots used again, keys far back and at page borders,
the first tokens, long decoding, generation through the entry point."""
import numpy as np
import pytest
import torch

from helpers import TOL, assert_close, rand_tokens
from nibelorn_helpers import CONFIGS, make, plain_logits
from plain import nibelorn_plain as N

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def _engine(path, dtype, max_tokens=1024):
    from stratum_b200.engine import Engine, load_model
    model, _ = load_model(path, torch.float32 if dtype == "float32" else torch.bfloat16, "cuda")
    return Engine(model, max_tokens=max_tokens)


@pytest.fixture(scope="module", params=[(n, d) for n in ("A", "B", "TC") for d in DTYPES], ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, tmp_path_factory):
    name, dtype = request.param
    path, cfg, w = make(str(tmp_path_factory.mktemp(f"nib{name}_{dtype}")), name, dtype, seed=len(name) + 1)
    return name, dtype, cfg, w, _engine(path, dtype), path


# ------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_dynamic_tanh_kernel(dtype):
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(0)
    x = rng.normal(size=(37, 200)) * 3
    w, b, alpha = rng.uniform(0.5, 1.5, 200), rng.normal(size=200) * 0.2, 0.7
    dev = lambda a: torch.tensor(a, dtype=torch.float32, device="cuda")                     # noqa: E731
    out = torch.empty((37, 200), dtype=torch.float32 if dtype == "float32" else torch.bfloat16, device="cuda")
    K.dynamic_tanh(dev(x), dev([alpha]), dev(w), dev(b), out)
    ref = N.dynamic_tanh(np.float32(x), np.float32(w), np.float32(b), np.float32(alpha))
    assert np.max(np.abs(out.float().cpu().numpy() - ref)) <= (2e-6 if dtype == "float32" else 1e-2)
    rows = torch.tensor([5, 0, 36], dtype=torch.int32, device="cuda")
    part = torch.empty((3, 200), dtype=out.dtype, device="cuda")
    K.dynamic_tanh(dev(x), dev([alpha]), dev(w), dev(b), part, rows)
    assert torch.equal(part, out[[5, 0, 36]])


def test_gelu_kernel_both_forms():
    from stratum_b200 import kernels as K
    z = np.linspace(-6, 6, 1001).astype(np.float32).reshape(7, 143)
    for kind, ref in ((K.GELU_ERF, N.gelu_erf(z)),
                      (K.GELU_TANH, 0.5 * z * (1 + np.tanh(np.sqrt(2 / np.pi) * (z + 0.044715 * z.astype(np.float64) ** 3))))):
        x = torch.tensor(z, device="cuda")
        K.gelu(x, kind)
        assert np.max(np.abs(x.cpu().numpy() - ref)) <= 2e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["latent", "diff", "ff"])
def test_one_mechanism_alone(name, dtype, tmp_path):
    """A model that is one mixer (or one small mixer and a feed-forward) and nothing else."""
    from stratum_b200.engine import StepEntry
    path, cfg, w = make(str(tmp_path / name), name, dtype, seed=5)
    engine = _engine(path, dtype)
    rng = np.random.default_rng(1)
    toks = rand_tokens(rng, 90, cfg["vocab"])
    slot = engine.acquire()
    got = engine.step([StepEntry(slot, toks, list(range(90)))]).cpu().numpy()
    assert_close(got, plain_logits(cfg, w, toks), dtype, name)


def test_general_attention_kernel_window_and_cap():
    """The kernel's parameters beyond what the architecture uses today: a window of keys, no cap, no factor."""
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(2)
    T, H, G, D, Dv, win = 150, 4, 2, 12, 20, 37
    q, k, v = rng.normal(size=(T, H, D)), rng.normal(size=(T, G, D)), rng.normal(size=(T, G, Dv))
    pages = 3
    kc = torch.zeros((pages, G, 64, D), dtype=torch.float32, device="cuda")
    vc = torch.zeros((pages, G, 64, Dv), dtype=torch.float32, device="cuda")
    table = [2, 0, 1]
    for t in range(T):
        kc[table[t // 64], :, t % 64] = torch.tensor(k[t], dtype=torch.float32)
        vc[table[t // 64], :, t % 64] = torch.tensor(v[t], dtype=torch.float32)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")                       # noqa: E731
    out = torch.empty((T, H * Dv), dtype=torch.float32, device="cuda")
    shape = K.AttentionShape(H, H // G, 1, D, Dv, False, 0.4, window=win)
    K.attention_general(shape, torch.tensor(q.reshape(T, -1), dtype=torch.float32, device="cuda"), kc, vc,
                        i32(np.arange(T)), i32(np.zeros(T)), i32([table]), out, 64)
    pos = np.arange(T)
    ref = np.zeros((T, H, Dv))
    for j in range(H):
        s = q[:, j] @ k[:, j // (H // G)].T * 0.4
        s = np.where(pos[None, :] > pos[:, None] - win, s, -np.inf)         # the last `win` keys, the token's own among them
        ref[:, j] = N.causal_softmax(s, pos, pos) @ v[:, j // (H // G)]
    assert np.max(np.abs(out.cpu().numpy().reshape(T, H, Dv) - ref)) <= 1e-4


# ------------------------------------------------------------------------------------------ whole models
def test_whole_prompt_all_positions(setup):
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine, _ = setup
    rng = np.random.default_rng(1)
    for n in (1, 2, 63, 64, 65, 200):
        toks = rand_tokens(rng, n, cfg["vocab"])
        slot = engine.acquire()
        got = engine.step([StepEntry(slot, toks, list(range(n)))]).cpu().numpy()
        engine.release(slot)
        assert_close(got, plain_logits(cfg, w, toks), dtype, f"{name} whole n={n}")
    engine.cache.check()


def test_prefill_against_token_by_token(setup):
    """The same tokens whole, and one by one from the first: the same logits (float32: to rounding)."""
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine, _ = setup
    rng = np.random.default_rng(2)
    n = 140
    toks = rand_tokens(rng, n, cfg["vocab"])
    a, b = engine.acquire(), engine.acquire()
    whole = engine.step([StepEntry(a, toks, list(range(n)))]).cpu().numpy()
    single = np.concatenate([engine.step([StepEntry(b, [t], [0])]).cpu().numpy() for t in toks])
    engine.release(a); engine.release(b)
    ref = plain_logits(cfg, w, toks)
    assert_close(whole, ref, dtype, f"{name} whole")
    assert_close(single, ref, dtype, f"{name} one by one")
    if dtype == "float32":
        assert np.max(np.abs(whole - single)) <= 2e-5 * np.max(np.abs(ref))


@pytest.mark.parametrize("portion", [2, 3, 31, 64, 100])
def test_prompt_in_portions(setup, portion):
    """A prompt cut into portions of a few sizes, down to two tokens; portions start inside pages and on their
    borders."""
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine, _ = setup
    rng = np.random.default_rng(portion)
    n = 150 if portion > 3 else 70
    toks = rand_tokens(rng, n, cfg["vocab"])
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
    V = cfg["vocab"]
    for batch_no, lens in enumerate([(5, 9, 12), (1, 67), (70, 3, 33, 64)]):
        prompts = [rand_tokens(rng, n, V) for n in lens]
        extra = [rand_tokens(rng, k, V) for k in (3 + 2 * i for i in range(len(lens)))]
        refs = [plain_logits(cfg, w, p + e) for p, e in zip(prompts, extra)]
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
    """A cache of four pages: every request takes pages another one has just given back, in another order."""
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, _, path = setup
    engine = _engine(path, dtype, max_tokens=256)
    rng = np.random.default_rng(4)
    V = cfg["vocab"]
    held = []
    for n in (130, 60, 190, 64, 129):
        while held and engine.cache.tokens_held() + ((n + 63) // 64) * 64 > 256:
            engine.release(held.pop(0))
        toks = rand_tokens(rng, n, V)
        slot = engine.acquire()
        got = engine.step([StepEntry(slot, toks[:-1], [n - 2])]).cpu().numpy()
        got = np.concatenate([got, engine.step([StepEntry(slot, toks[-1:], [0])]).cpu().numpy()])
        assert_close(got, plain_logits(cfg, w, toks)[-2:], dtype, f"{name} reuse n={n}")
        held.append(slot)
        engine.cache.check()


def test_first_tokens_and_long_decoding(setup):
    """Positions 0, 1, 2 one by one, then on across several pages and many steps of the query factor."""
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine, _ = setup
    rng = np.random.default_rng(5)
    n = 270
    toks = rand_tokens(rng, n, cfg["vocab"])
    ref = plain_logits(cfg, w, toks)
    slot = engine.acquire()
    check = {0, 1, 2, 3} | set(range(4, n, 29)) | {63, 64, 65, 127, 128, 129, 191, 192, 193, n - 1}
    got = []
    for i in range(n):
        out = engine.step([StepEntry(slot, [toks[i]], [0] if i in check else [])])
        if i in check:
            got.append(out.cpu().numpy())
    engine.release(slot)
    assert_close(np.concatenate(got), ref[sorted(check)], dtype, f"{name} long decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("where", [0, 1, 63, 64, 65, 128, 200])
def test_one_far_key_decides(where, dtype, tmp_path_factory):
    """Weights under which the last token's output is whatever one marked key, far back, carries: a lost key, a key
    read from the wrong page or a row off by one changes the logits wholesale.  The marked token's key and the last
    token's query are made large and parallel in both mixers (their embeddings are one large vector that the query
    and key weights pass through); all other tokens have small embeddings."""
    from stratum_b200.engine import StepEntry

    def edit(t):
        e = t["embed"].float()
        e[:] = e * 0.02
        e[7] = 0.0
        e[7, :8] = 6.0                                   # the marked token and the asking token (id 8) share a direction
        e[8] = 0.0
        e[8, :8] = 6.0
        e[8, 8:16] = 3.0                                 # ... and differ elsewhere, so that their values differ
        t["embed"] = e.to(t["embed"].dtype)
        for name in list(t):
            if name.endswith((".q", ".k", ".dkv")):      # queries and keys both read the shared direction strongly
                m = t[name].float()
                m[:, :8] = m[:, :8].abs() * 20
                t[name] = m.to(t[name].dtype)
    key = f"far{where}{dtype}"
    path, cfg, w = make(str(tmp_path_factory.mktemp(key)), "TC", dtype, seed=9, edit=edit)
    engine = _engine(path, dtype)
    rng = np.random.default_rng(where)
    n = 260
    toks = [int(t) for t in rng.integers(9, cfg["vocab"], n)]
    toks[where], toks[-1] = 7, 8
    ref = plain_logits(cfg, w, toks)
    moved = list(toks)
    moved[where] = toks[where + 1] if where + 1 < n - 1 else 9
    assert np.max(np.abs(plain_logits(cfg, w, moved)[-1] - ref[-1])) > 0.05 * np.max(np.abs(ref[-1])), "the key does not matter"
    slot = engine.acquire()
    whole = engine.step([StepEntry(slot, toks, [n - 1])]).cpu().numpy()[0]
    engine.release(slot)
    slot = engine.acquire()
    engine.step([StepEntry(slot, toks[:n - 1], [])])
    decoded = engine.step([StepEntry(slot, toks[n - 1:], [0])]).cpu().numpy()[0]
    engine.release(slot)
    assert_close(whole, ref[-1], dtype, f"far key at {where}, whole")
    assert_close(decoded, ref[-1], dtype, f"far key at {where}, decoded")


# ------------------------------------------------------------------------------------------ generation
@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(dtype, tmp_path):
    """Stratum.generate: the scheduler's batches, replayed decode graphs, slots given back; every picked token is the
    plain implementation's best (or within rounding of it)."""
    from stratum_b200 import Stratum
    path, cfg, w = make(str(tmp_path / "gen"), "A", dtype, seed=11)
    rng = np.random.default_rng(0)
    prompts = [rand_tokens(rng, n, cfg["vocab"]) for n in (5, 70, 12, 1)]
    llm = Stratum(path, dtype=dtype, max_tokens=1024)
    res = llm.generate(prompts, max_new_tokens=10, stop_ids=())
    for p, r in zip(prompts, res):
        assert len(r.tokens) == 10
        seq = list(p)
        for tok in r.tokens:
            ref = plain_logits(cfg, w, seq)[-1]
            assert ref[tok] >= ref.max() - 2 * TOL[dtype] * float(np.max(np.abs(ref))), (p, r.tokens, tok)
            seq.append(tok)
    serial = llm.generate(prompts, max_new_tokens=10, stop_ids=(), max_batch=2)
    if dtype == "float32":
        assert [r.tokens for r in serial] == [r.tokens for r in res]
    llm.engine.cache.check()
    assert llm.engine.cache.tokens_held() == 0


# ------------------------------------------------------------------------------------------ tensor-core attention
def _fill_cache(rng, seq_lens, n_k, D, n_v, Dv, v_in_k):
    """A paged cache with shuffled pages holding random keys (and values) for sequences of the given lengths."""
    pages_of = [(n + 63) // 64 for n in seq_lens]
    order = rng.permutation(sum(pages_of) + 3)
    tables, at = [], 0
    for n in pages_of:
        tables.append([int(x) for x in order[at:at + n]])
        at += n
    width = max(pages_of)
    kc = torch.zeros((len(order), n_k, 64, D), dtype=torch.bfloat16, device="cuda")
    vc = None if v_in_k else torch.zeros((len(order), n_v, 64, Dv), dtype=torch.bfloat16, device="cuda")
    for tb, n in zip(tables, seq_lens):
        for j, page in enumerate(tb):
            m = min(64, n - 64 * j)
            kc[page, :, :m] = torch.tensor(rng.normal(size=(n_k, m, D)), dtype=torch.bfloat16)
            if vc is not None:
                vc[page, :, :m] = torch.tensor(rng.normal(size=(n_v, m, Dv)), dtype=torch.bfloat16)
    table = torch.tensor([tb + [-1] * (width - len(tb)) for tb in tables], dtype=torch.int32, device="cuda")
    return kc, vc, table


@pytest.mark.parametrize("case", [
    # heads, group, maps, D, Dv, v_in_k, new tokens per sequence, cached before
    dict(H=5, group=5, maps=1, D=136, Dv=120, v_in_k=True, new=(1, 1, 1), before=(0, 63, 700)),
    dict(H=16, group=16, maps=1, D=576, Dv=512, v_in_k=True, new=(1, 1), before=(300, 1100)),
    dict(H=20, group=20, maps=1, D=72, Dv=64, v_in_k=True, new=(5, 70), before=(0, 130)),
    dict(H=6, group=3, maps=2, D=56, Dv=88, v_in_k=False, new=(1, 1, 1, 1), before=(5, 64, 127, 900)),
    dict(H=6, group=2, maps=2, D=16, Dv=24, v_in_k=False, new=(33, 1, 130), before=(0, 77, 64)),
    dict(H=8, group=8, maps=1, D=40, Dv=40, v_in_k=True, new=(150,), before=(0,), window=37),
    dict(H=16, group=16, maps=1, D=320, Dv=288, v_in_k=True, new=(9, 140), before=(100, 3)),
    dict(H=3, group=1, maps=2, D=24, Dv=136, v_in_k=False, new=(77, 2, 64), before=(0, 200, 1)),
])
def test_tensor_core_attention_against_cuda_cores(case):
    """The same bfloat16 queries and cache through both kernels: decode steps with the keys cut into ranges,
    prompts in query blocks, sizes up to those of a large model's latent, two maps combined, a window."""
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(7)
    H, group, maps, D, Dv, v_in_k = (case[k] for k in ("H", "group", "maps", "D", "Dv", "v_in_k"))
    new, before = case["new"], case["before"]
    lens = [a + b for a, b in zip(new, before)]
    n_k, n_v = (H // group) * maps, H // group
    kc, vc, table = _fill_cache(rng, lens, n_k, D, n_v, Dv, v_in_k)
    T = sum(new)
    pos = np.concatenate([np.arange(b, b + n) for n, b in zip(new, before)])
    seq = np.concatenate([np.full(n, i) for i, n in enumerate(new)])
    gate = maps == 2
    width = H * maps * D + (H if gate else 0)
    ld = (width + 7) // 8 * 8
    q = torch.zeros((T, ld), dtype=torch.bfloat16, device="cuda")
    q[:, :width] = torch.tensor(rng.normal(size=(T, width)) * 0.5, dtype=torch.bfloat16)
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device="cuda")          # noqa: E731
    shape = K.AttentionShape(H, group, maps, D, Dv, v_in_k, 0.3, softcap=5.0 if gate else 0.0,
                             window=case.get("window", 0), temp_coef=0.4 if gate else 0.0, temp_every=50,
                             lam=0.45, out_scale=0.7, eps=1e-5, gate_col=H * maps * D if gate else -1)
    ref = torch.zeros((T, (H * Dv + 7) // 8 * 8), dtype=torch.bfloat16, device="cuda")
    K.attention_general(shape, q, kc, vc, i32(pos), i32(seq), table, ref, 64)
    per_block = 16 // min(group, 16)
    single = all(n == 1 for n in new)
    assert K.attention_general_mma_row_groups(Dv) in (1, 2)
    # decode steps: one group of 16 rows, the keys in one, three or sixteen ranges; prompts: one and two groups
    for n_splits, chunk, groups in ([(1, 2048, 1), (3, 384, 1), (16, 128, 1)] if single else [(1, 2048, 1), (1, 2048, 2)]):
        qblocks = None
        if not single:
            qs, qt, qn, r = [], [], [], 0
            for i, n in enumerate(new):
                for b in range(0, n, per_block * groups):
                    qs.append(i); qt.append(r + b); qn.append(min(per_block * groups, n - b))
                r += n
            qblocks = (i32(qs), i32(qt), i32(qn))
        n_part = T * H * maps * n_splits
        part_o = torch.full((n_part * Dv,), float("nan"), dtype=torch.float32, device="cuda")
        part_ml = torch.full((n_part * 2,), float("nan"), dtype=torch.float32, device="cuda")
        out = torch.zeros_like(ref)
        K.attention_general_mma(shape, q, kc, vc, i32(pos), i32(seq), table, out, 64, qblocks, per_block, n_splits,
                                chunk, part_o, part_ml, groups)
        torch.cuda.synchronize()
        a, b = out.float().cpu().numpy()[:, :H * Dv], ref.float().cpu().numpy()[:, :H * Dv]
        assert np.isfinite(a).all()
        # both round their result to bfloat16 once: one unit in the last place of the larger values
        assert np.max(np.abs(a - b)) <= 2 ** -7 * max(1.0, np.max(np.abs(b))), (n_splits, np.max(np.abs(a - b)))


@pytest.mark.parametrize("rows,inner,dtype", [(4, 64, "bfloat16"), (200, 64, "bfloat16"), (700, 512, "bfloat16"),
                                              (9, 70, "bfloat16"), (33, 70, "float32")])
def test_activation_on_the_product_epilogue(rows, inner, dtype):
    """gelu(x W^T) by every matrix-product kernel that can carry the activation: the weight-streaming one (few rows),
    the tcgen05 one, and the CUDA-core one (sizes no vector load divides; float32)."""
    from stratum_b200 import kernels as K
    from stratum_b200.parts.base import Runtime
    from stratum_b200.parts.linear import STORE, Linear
    rng = np.random.default_rng(rows)
    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    x = torch.tensor(rng.normal(size=(rows, inner)), dtype=dt, device="cuda")
    w = torch.tensor(rng.normal(size=(150, inner)) * 0.3, dtype=dt, device="cuda")
    lin = Linear(Runtime(dt, "cuda"), w)
    pre = lin(x, mode=STORE).float().cpu().numpy()
    for act, ref in ((K.ACT_GELU_ERF, N.gelu_erf),
                     (K.ACT_GELU_TANH, lambda z: 0.5 * z * (1 + np.tanh(np.sqrt(2 / np.pi) * (z + 0.044715 * z ** 3))))):
        got = lin(x, mode=STORE, act=act).float().cpu().numpy()
        exact = ref(x.float().cpu().numpy().astype(np.float64) @ w.float().cpu().numpy().astype(np.float64).T)
        tol = 1e-5 if dtype == "float32" else 2 ** -8
        assert np.max(np.abs(got - exact)) <= tol * max(1.0, np.max(np.abs(exact))), (act, np.max(np.abs(got - exact)))
        assert np.max(np.abs(got - pre)) > 0.1              # and it is not the plain product


@pytest.mark.parametrize("rows", [1, 8, 20, 33, 300])
@pytest.mark.parametrize("heads,n,k,x_step,o_step", [(4, 128, 32, 48, 144), (16, 64, 256, 256, 64), (3, 40, 24, 32, 40),
                                                      (2, 17, 13, 19, 17)])
def test_per_head_products(rows, heads, n, k, x_step, o_step):
    """HeadLinear: all heads in one launch, on tensor cores where the sizes allow and on the CUDA cores elsewhere
    (the last shape), against the definition."""
    from stratum_b200.parts.base import Runtime
    from stratum_b200.parts.linear import HeadLinear
    rng = np.random.default_rng(rows + n)
    ldx, ldo = (heads * x_step + 7) // 8 * 8, (heads * o_step + 7) // 8 * 8
    x = torch.tensor(rng.normal(size=(rows, ldx)), dtype=torch.bfloat16, device="cuda")
    w = torch.tensor(rng.normal(size=(heads, n, k)) * 0.2, dtype=torch.bfloat16, device="cuda")
    out = torch.full((rows, ldo), 7.0, dtype=torch.bfloat16, device="cuda")
    HeadLinear(Runtime(torch.bfloat16, "cuda"), w)(x, x_step, out, o_step)
    xf, wf = x.float().cpu().numpy().astype(np.float64), w.float().cpu().numpy().astype(np.float64)
    got = out.float().cpu().numpy()
    for j in range(heads):
        ref = xf[:, j * x_step: j * x_step + k] @ wf[j].T
        assert np.max(np.abs(got[:, j * o_step: j * o_step + n] - ref)) <= 2 ** -8 * max(1.0, np.max(np.abs(ref)))
    if o_step > n:                                         # columns between the heads' results are left alone
        assert np.all(got[:, n:o_step] == 7.0)


# ------------------------------------------------------------------------------------------ the programs
def test_command_line_and_trace_replay_program(tmp_path):
    """`./stratum` on a Nibelorn folder (random weights written by the command line itself from a config file), and
    `bin/trace_run` fed steps on standard input: a batch of two requests, then single tokens, one request ending
    earlier, then a request that takes the pages given back."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(CONFIGS["A"]))
    folder = str(tmp_path / "written")
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    r = subprocess.run([sys.executable, os.path.join(root, "stratum"), folder, "4", *map(str, prompt), "--fp32",
                        "--random-weights", "3", "--config", str(cfg_file)], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr
    assert "architecture: Nibelorn" in r.stderr
    from helpers import load_plain
    cfg, w = load_plain(folder)
    seq = list(prompt)
    for _ in range(5):
        seq.append(int(np.argmax(plain_logits(cfg, w, seq)[-1])))
    assert r.stdout.split() == [str(t) for t in seq[len(prompt):]]

    path, cfg, w = make(str(tmp_path / "lively"), "A", "float32", seed=21)
    rng = np.random.default_rng(8)
    V = cfg["vocab"]
    a, b, c = (rand_tokens(rng, n, V) for n in (70, 9, 33))
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


def test_long_prompts_take_the_per_head_form(setup, monkeypatch):
    """bfloat16 prompts that begin at position 0 and bring 256 tokens or more form their heads' keys and values
    (latent attention) instead of attending in the latent space: the same logits, to bfloat16 rounding, as the plain
    implementation and as the absorbed form; the cache they leave serves the decoded tokens that follow; a portion that
    continues a sequence takes the absorbed form again."""
    from stratum_b200 import kernels as K
    from stratum_b200.engine import StepEntry
    name, dtype, cfg, w, engine, _ = setup
    if dtype != "bfloat16" or name == "B":
        pytest.skip("the per-head form is a bfloat16 form for sizes in multiples of 8")
    dense_calls = []
    real = K.attention_general_mma

    def spy(*args, **kw):
        dense_calls.append(kw.get("seq_start") is not None)
        return real(*args, **kw)
    monkeypatch.setattr(K, "attention_general_mma", spy)
    rng = np.random.default_rng(12)
    V = cfg["vocab"]
    prompts = [rand_tokens(rng, n, V) for n in (300, 70, 257)]
    tails = [rand_tokens(rng, 3, V) for _ in prompts]
    refs = [plain_logits(cfg, w, p + t) for p, t in zip(prompts, tails)]
    slots = [engine.acquire() for _ in prompts]
    out = engine.step([StepEntry(s, p, [0, len(p) // 2, len(p) - 1]) for s, p in zip(slots, prompts)]).cpu().numpy()
    assert any(dense_calls), "no layer took the per-head form"
    for i, p in enumerate(prompts):
        assert_close(out[3 * i: 3 * i + 3], refs[i][[0, len(p) // 2, len(p) - 1]], dtype, f"{name} per-head prompt {i}")
    for k in range(3):                                  # decoded tokens read the cache the prompt step wrote
        out = engine.step([StepEntry(s, [t[k]], [0]) for s, t in zip(slots, tails)]).cpu().numpy()
        for i, p in enumerate(prompts):
            assert_close(out[i], refs[i][len(p) + k], dtype, f"{name} after per-head prompt {i} +{k}")
    for s in slots:
        engine.release(s)
    # the same prompt with the form switched off, and in two portions (the second continues: absorbed form)
    monkeypatch.setenv("STRATUM_LATENT_PER_HEAD", "0")
    del dense_calls[:]
    s = engine.acquire()
    absorbed = engine.step([StepEntry(s, prompts[0], [299])]).cpu().numpy()
    engine.release(s)
    assert not any(dense_calls)
    assert_close(absorbed, refs[0][[299]], dtype, f"{name} absorbed form")
    monkeypatch.delenv("STRATUM_LATENT_PER_HEAD")
    s = engine.acquire()
    engine.step([StepEntry(s, prompts[0][:10], [])])
    del dense_calls[:]
    second = engine.step([StepEntry(s, prompts[0][10:], [289])]).cpu().numpy()
    engine.release(s)
    assert not any(dense_calls)
    assert_close(second, refs[0][[299]], dtype, f"{name} continued portion")
