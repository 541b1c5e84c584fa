"""Small Nibelorn configurations and model folders for the tests.  None of them is anyone's model: sizes are
chosen so that no two of a layer's sizes are equal by accident, that counts are not 1 where the formulas divide
by them, and that the layers of one model differ from one another."""
import numpy as np
import torch

from helpers import load_plain, make_model_dir
from plain import nibelorn_plain as N


def latent(heads=3, dim=24, rot=8, vdim=40, rank=56, base=10000.0, scale=0.19):
    return {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "scale": scale,
            "rot": {"base": base, "dims": rot}}


def differential(heads=6, kv_heads=2, dim=16, vdim=24, scale=0.23, softcap=7.0, diff=0.35, coef=0.4, every=5):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap,
            "diff": diff, "q_temp": {"coef": coef, "every": every}}


def layer(kind, mixer, ff=None, weights_of=None):
    d = {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


def config(layers, vocab=211, width=72, eps=1e-5):
    return {"architecture": "Nibelorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# a differential layer first, three kv heads... ; a latent layer without feed-forward; layers that reuse tensors
NIB_A = config([layer("attention", differential(), ff=96),
                layer("latent_attention", latent(), ff=None),
                layer("latent_attention", latent(heads=2, dim=16, rot=16, vdim=24, rank=40, base=500.0), ff=120),
                layer("attention", differential(), ff=96, weights_of=0),
                layer("latent_attention", latent(), ff=None, weights_of=1)])
# sizes that no vector load divides (width 70, heads of 20 + 6): every fallback kernel
NIB_B = config([layer("latent_attention", latent(heads=2, dim=20, rot=6, vdim=18, rank=34, scale=0.3), ff=50),
                layer("attention", differential(heads=2, kv_heads=2, dim=10, vdim=14, every=3, softcap=3.0), ff=None)],
               vocab=97, width=70, eps=1e-6)
# one layer each, alone: the mechanisms one by one
NIB_LATENT = config([layer("latent_attention", latent(heads=4, dim=16, rot=8, vdim=16, rank=32), ff=None)], width=64)
NIB_DIFF = config([layer("attention", differential(heads=4, kv_heads=1, dim=8, vdim=32, every=7), ff=None)], width=64)
NIB_FF = config([layer("latent_attention", latent(heads=1, dim=8, rot=4, vdim=8, rank=16), ff=136)], width=64)
# sizes of the tensor-core kernels: multiples of 16 everywhere
NIB_TC = config([layer("latent_attention", latent(heads=4, dim=32, rot=32, vdim=48, rank=96), ff=160),
                 layer("attention", differential(heads=4, kv_heads=2, dim=32, vdim=64, every=9), ff=160),
                 layer("latent_attention", latent(heads=4, dim=32, rot=32, vdim=48, rank=96), ff=160, weights_of=0)],
                vocab=331, width=128)

CONFIGS = {"A": NIB_A, "B": NIB_B, "latent": NIB_LATENT, "diff": NIB_DIFF, "ff": NIB_FF, "TC": NIB_TC}


def lively(tensors, seed=0):
    """Random weights as the writer makes them are tame: norms with gain 1 and no bias, a lambda that equals `diff`,
    attention that is almost uniform.  Give every constant a value of its own and make scores spread."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda t, lo, hi: (torch.rand(t.shape, generator=g) * (hi - lo) + lo).to(t.dtype)      # noqa: E731
    for name, t in tensors.items():
        if name.endswith(".alpha"):
            tensors[name] = rnd(t, 0.4, 1.3)
        elif name.endswith(".b"):
            tensors[name] = rnd(t, -0.3, 0.3)
        elif name.endswith(("norm1", "norm2", "final.norm", "dkv.norm")):
            tensors[name] = rnd(t, 0.5, 1.5)
        elif name.endswith((".lq1", ".lk1", ".lq2", ".lk2")):
            tensors[name] = rnd(t, -0.35, 0.35)
        elif name == "embed":
            tensors[name] = (t.float() * 40).to(t.dtype)
        elif name.endswith((".q", ".k", ".dkv", ".uk")):
            tensors[name] = (t.float() * 2).to(t.dtype)
        elif name.endswith((".v", ".uv", ".o", ".up", ".down", ".g")) or name == "head":
            tensors[name] = (t.float() * 2).to(t.dtype)


def make(path, name, dtype, seed=0, edit=None):
    def both(tensors):
        lively(tensors, seed)
        if edit is not None:
            edit(tensors)
    path = make_model_dir(path, CONFIGS[name], seed=seed, dtype=dtype, std=0.05, edit=both)
    cfg, w = load_plain(path)
    return path, cfg, w


def plain_logits(cfg, w, tokens):
    return N.forward(cfg, w, tokens)
