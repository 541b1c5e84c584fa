"""Small Dabodra configurations and model folders for the tests.  None of them is anyone's model: sizes are chosen so
that no two of a layer's sizes are equal by accident, that counts are not 1 where the formulas divide by them, and
that the layers of one model differ from one another (windows, rotated dimensions, taps, experts, groups)."""
import numpy as np
import torch

from helpers import load_plain, make_model_dir
from plain import dabodra_plain as D


def attention(heads=6, kv_heads=2, dim=24, window=37, rot=16, base=10000.0, scale=0.21):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "mask": {"size": window},
            "rot": {"base": base, "dims": rot}}


def delta(heads=4, kv_heads=2, dim=24, vdim=40, conv=3):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def moe(experts=6, top=2, groups=3, keep=2, scale=2.5, ff=40, shared=56):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale,
                                      "groups": {"count": groups, "keep": keep}},
            "expert": {"ff": ff}, "shared": {"ff": shared}}


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(layers, vocab=211, width=72, eps=1e-5):
    return {"architecture": "Dabodra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# attention first, a delta layer without feed-forward, a delta layer whose key size needs two lanes a column and whose
# heads each have q and k of their own, a second attention with a window of five and another base
DAB_A = config([layer("attention", attention(), moe()),
                layer("delta", delta()),
                layer("delta", delta(heads=3, kv_heads=3, dim=40, vdim=16, conv=5), moe(experts=8, top=3, groups=1, keep=1, scale=1.0, ff=24, shared=16)),
                layer("attention", attention(heads=2, kv_heads=1, dim=16, window=5, rot=8, base=500.0, scale=0.3),
                      moe(experts=4, top=1, groups=4, keep=2, scale=0.7, ff=32, shared=8))])
# sizes that no vector load divides (width 70, heads of 20 and 18): every fallback kernel
DAB_B = config([layer("delta", delta(heads=2, kv_heads=1, dim=20, vdim=18, conv=2), moe(experts=5, top=2, groups=1, keep=1, ff=30, shared=22)),
                layer("attention", attention(heads=3, kv_heads=3, dim=20, window=70, rot=6, scale=0.3), None)],
               vocab=97, width=70, eps=1e-6)
# one mechanism each, alone
DAB_ATT = config([layer("attention", attention(heads=4, kv_heads=2, dim=16, window=9, rot=16))], width=64)
DAB_DELTA = config([layer("delta", delta(heads=4, kv_heads=1, dim=8, vdim=32, conv=4))], width=64)
DAB_MOE = config([layer("delta", delta(heads=1, kv_heads=1, dim=8, vdim=8, conv=2), moe(experts=12, top=4, groups=4, keep=2))], width=64)
# sizes of the tensor-core kernels: multiples of 16 everywhere, a window beyond one page
DAB_TC = config([layer("delta", delta(heads=4, kv_heads=2, dim=64, vdim=32, conv=4), moe(experts=4, top=2, groups=2, keep=1, ff=32, shared=48)),
                 layer("attention", attention(heads=4, kv_heads=2, dim=32, window=70, rot=32), moe(experts=4, top=2, groups=1, keep=1, ff=32, shared=48)),
                 layer("attention", attention(heads=8, kv_heads=1, dim=64, window=130, rot=16, scale=0.11), None)],
                vocab=331, width=128)

CONFIGS = {"A": DAB_A, "B": DAB_B, "att": DAB_ATT, "delta": DAB_DELTA, "moe": DAB_MOE, "TC": DAB_TC}


def lively(tensors, seed=0, decisive=False):
    """Random weights as the writer makes them are tame: norms of gain one, sinks of zero, no correction, decays that
    are all alike.  Give every constant a value of its own and make scores spread.  decisive: the routers' corrections
    lie far apart (each more than twice the next, so that no two groups' sums come close either) and the routers'
    own scores vary little: the choice of experts then survives the rounding of the bfloat16 path."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda t, lo, hi: (torch.rand(t.shape, generator=g) * (hi - lo) + lo).to(t.dtype)      # noqa: E731
    for name, t in tensors.items():
        if name.endswith(("norm1", "norm2", "final.norm", "embed.norm")):
            tensors[name] = rnd(t, -0.4, 0.4)
        elif name.endswith((".q.norm", ".k.norm", ".mix.norm")):
            tensors[name] = rnd(t, 0.5, 1.5)
        elif name.endswith(".sink"):
            tensors[name] = rnd(t, -1.0, 2.0)
        elif name.endswith(".correction"):
            if decisive:
                n = t.numel()
                tensors[name] = (0.3 * 2.1 ** torch.randperm(n, generator=g).float()).to(t.dtype)
            else:
                tensors[name] = rnd(t, -0.6, 0.3)
        elif name.endswith(".A_log"):
            tensors[name] = rnd(t, -2.0, 0.5)
        elif name.endswith(".dt_bias"):
            tensors[name] = rnd(t, -1.0, 1.0)
        elif name.endswith(".conv"):
            tensors[name] = rnd(t, -0.8, 0.8)
        elif name.endswith(".router"):
            tensors[name] = (t.float() * (0.3 if decisive else 6.0)).to(t.dtype)
        elif name == "embed":
            tensors[name] = (t.float() * 30).to(t.dtype)
        elif name.endswith((".q", ".k", ".v", ".b", ".a", ".g", ".o", ".gate", ".up", ".down")) or name == "head":
            tensors[name] = (t.float() * 2.5).to(t.dtype)


def make(path, name, dtype, seed=0, edit=None, cfg=None):
    decisive = dtype == "bfloat16"

    def both(tensors):
        lively(tensors, seed, decisive)
        if edit is not None:
            edit(tensors)
    path = make_model_dir(path, cfg or CONFIGS[name], seed=seed, dtype=dtype, std=0.05, edit=both)
    cfg, w = load_plain(path)
    return path, cfg, w


def plain_logits(cfg, w, tokens):
    return D.forward(cfg, w, tokens)


def clear_tokens(rng, n, cfg, w, dtype, fixed=None):
    """n random tokens (fixed: position -> token) on which no router is near a tie: a choice that rounding could turn
    is no test of anything.  float32 keeps 1e-4 away, bfloat16 (with decisive corrections) 0.04."""
    need = 1e-4 if dtype == "float32" else 0.04
    for _ in range(200):
        toks = [int(t) for t in rng.integers(0, cfg["vocab"], n)]
        for p, t in (fixed or {}).items():
            toks[p] = t
        margins = []
        D.forward(cfg, w, toks, margins=margins)
        if not margins or min(margins) > need:
            return toks
    raise AssertionError("no token sequence keeps the routers away from ties")


def assert_rows_close(got, ref, dtype, what=""):
    """float32: every logit within the float32 tolerance.  bfloat16: a position here and there sits where rounding
    is amplified (a near-empty vector made a unit vector, a norm behind an output that nearly cancels), so the
    tolerance holds for 19 of 20 positions and three times the tolerance for all of them."""
    from helpers import TOL, assert_close
    if dtype == "float32":
        return assert_close(got, ref, dtype, what)
    got, ref = np.atleast_2d(np.asarray(got, np.float64)), np.atleast_2d(np.asarray(ref, np.float64))
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    err = np.max(np.abs(got - ref), axis=-1) / np.max(np.abs(ref))
    assert err.max() <= 3 * TOL[dtype], f"{what}: worst position off by {err.max():.3e} of the largest logit"
    over = int(np.sum(err > TOL[dtype]))
    assert over <= max(1, len(err) // 20), f"{what}: {over} of {len(err)} positions beyond {TOL[dtype]:.0e}"
