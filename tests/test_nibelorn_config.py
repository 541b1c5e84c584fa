"""Nibelorn on the CPU: the configuration reader, the tensor list, the schedule of shared layers, what each layer
keeps in the cache, and the plain implementation's own properties."""
import copy

import numpy as np
import pytest

from nibelorn_helpers import CONFIGS, NIB_A, NIB_B
from plain import nibelorn_plain as N


def _cfg(raw):
    from stratum_b200.config import find_architecture
    return find_architecture(raw).config_class.from_dict(raw)


def test_configuration_round_trip_and_registry():
    from stratum_b200.config import NibelornConfig, find_architecture
    assert find_architecture({"architecture": "Nibelorn"}).config_class is NibelornConfig
    for raw in CONFIGS.values():
        cfg = _cfg(raw)
        assert NibelornConfig.from_dict(cfg.to_dict()) == cfg
        assert len(cfg.layers) == len(raw["layers"])


def test_configuration_problems_are_listed_together():
    from stratum_b200.config import ConfigError
    raw = copy.deepcopy(NIB_A)
    del raw["width"]
    raw["layers"][0]["mixer"]["heads"] = 5                 # 5 heads on 2 kv heads
    raw["layers"][1]["mixer"]["rot"]["dims"] = 7
    raw["layers"][2]["type"] = "recurrent"
    raw["layers"][4]["weights_of"] = 3                     # layer 3 uses layer 0's, which is another kind of layer
    with pytest.raises(ConfigError) as e:
        _cfg(raw)
    text = str(e.value)
    for piece in ("width", "kv_heads", "rot.dims", "recurrent", "differs from layers[0]"):
        assert piece in text, (piece, text)


def test_borrowed_tensors_through_another_borrower():
    raw = copy.deepcopy(NIB_A)
    raw["layers"].append(dict(raw["layers"][3], weights_of=3))          # 5 -> 3 -> 0
    cfg = _cfg(raw)
    assert cfg.layers[5].weights_of == 0
    raw["layers"][0]["weights_of"] = 5                                  # a ring: nobody has tensors
    from stratum_b200.config import ConfigError
    with pytest.raises(ConfigError, match="no layer with tensors"):
        _cfg(raw)


def test_tensor_names_and_shapes():
    from stratum_b200.engine.model import expected_tensors
    t = expected_tensors(_cfg(NIB_A))
    names = set(t)
    assert {"embed", "head", "final.norm", "final.norm.b", "final.norm.alpha"} <= names
    assert not any(n.startswith(("l3.", "l4.")) for n in names)            # layers 3 and 4 use 0's and 1's
    assert not any(n.startswith("l1.norm2") or n.startswith("l1.mlp") for n in names)      # no feed-forward there
    d, m = NIB_A["layers"][0]["mixer"], NIB_A["layers"][1]["mixer"]
    W = NIB_A["width"]
    assert t["l0.mix.q"].shape == (d["heads"] * 2 * d["dim"], W)
    assert t["l0.mix.k"].shape == (d["kv_heads"] * 2 * d["dim"], W)
    assert t["l0.mix.v"].shape == (d["kv_heads"] * d["vdim"], W)
    assert t["l0.mix.g"].shape == (d["heads"], W) and t["l0.mix.lq1"].shape == (d["dim"],)
    assert t["l0.mix.o"].shape == (W, d["heads"] * d["vdim"])
    assert t["l1.mix.q"].shape == (m["heads"] * (m["dim"] + m["rot_dim"]), W)
    assert t["l1.mix.dkv"].shape == (m["kv_rank"] + m["rot_dim"], W) and t["l1.mix.dkv.norm"].shape == (m["kv_rank"],)
    assert t["l1.mix.uk"].shape == (m["heads"] * m["dim"], m["kv_rank"])
    assert t["l1.mix.uv"].shape == (m["heads"] * m["vdim"], m["kv_rank"])
    assert t["l0.norm1.alpha"].shape == () and t["l0.mlp.up"].shape == (96, W)


def test_shared_layers_are_stops_with_their_own_cache():
    from stratum_b200.cache import SequenceCache
    from stratum_b200.cache.store import KVSpec
    from stratum_b200.config import find_architecture
    from stratum_b200.engine.model import Model
    import torch
    model = Model(find_architecture(NIB_A).describe_model(_cfg(NIB_A)), None)
    assert [e.layer for e in model.schedule] == [0, 1, 2, 0, 1] and len(model.layers) == 3
    specs = model.cache_specs()
    assert all(isinstance(s, KVSpec) for s in specs) and specs[0] == specs[3] and specs[1] == specs[4] != specs[2]
    lat = NIB_A["layers"][1]["mixer"]
    assert specs[1].n_kv_heads == 1 and specs[1].head_dim == lat["kv_rank"] + lat["rot_dim"] and specs[1].v_heads == 0
    dif = NIB_A["layers"][0]["mixer"]
    assert specs[0].n_kv_heads == 2 * dif["kv_heads"] and specs[0].v_heads == dif["kv_heads"]
    assert specs[0].v_dim == dif["vdim"] and specs[0].head_dim == dif["dim"]
    cache = SequenceCache(specs, 256, 4, torch.float32, "cpu")
    assert len(cache.groups) == 3 and sorted(len(g.layers) for g in cache.groups) == [1, 2, 2]
    for g in cache.groups:
        if g.spec.v_heads == 0:
            assert g.v is None and g.k.shape[-1] == g.spec.head_dim
        else:
            assert g.v.shape[2:] == (g.spec.v_heads, 64, g.spec.v_dim)


def _random_weights(raw, seed):
    import torch
    from nibelorn_helpers import lively
    from stratum_b200.engine.model import expected_tensors
    from stratum_b200.weights.random_init import random_tensors
    t = random_tensors(expected_tensors(_cfg(raw)), seed, 0.05, torch.float32)
    lively(t, seed)
    return {k: v.numpy().astype(np.float64) for k, v in t.items()}


def test_plain_implementation_is_causal_and_uses_every_constant():
    raw = NIB_B
    w = _random_weights(raw, 3)
    rng = np.random.default_rng(0)
    toks = rng.integers(0, raw["vocab"], 40).tolist()
    full = N.forward(raw, w, toks)
    assert np.allclose(N.forward(raw, w, toks[:17]), full[:17], rtol=0, atol=1e-9)         # later tokens change nothing
    for path, value in ((("layers", 1, "mixer", "softcap"), 1.0), (("layers", 1, "mixer", "diff"), 0.1),
                        (("layers", 1, "mixer", "q_temp", "every"), 4), (("layers", 1, "mixer", "q_temp", "coef"), 0.0),
                        (("layers", 0, "mixer", "rot", "base"), 77.0), (("layers", 0, "mixer", "scale"), 0.1),
                        (("norm", "eps"), 1e-2)):
        other = copy.deepcopy(raw)
        node = other
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        assert np.max(np.abs(N.forward(other, w, toks) - full)) > 1e-6, path


def test_plain_latent_attention_equals_its_absorbed_form():
    """The identity the product relies on: scoring in the latent space and expanding afterwards gives what per-head
    keys and values give."""
    m = NIB_A["layers"][1]["mixer"]
    rng = np.random.default_rng(1)
    T, W = 9, 24
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    w = {"q": rng.normal(size=(H * (d + r), W)), "dkv": rng.normal(size=(rank + r, W)),
         "dkv.norm": rng.uniform(0.5, 1.5, rank), "uk": rng.normal(size=(H * d, rank)) * 0.2,
         "uv": rng.normal(size=(H * dv, rank)) * 0.2, "o": rng.normal(size=(W, H * dv))}
    h = rng.normal(size=(T, W))
    ref = N.latent_attention(h, w, m, 1e-5)
    pos = np.arange(T)
    q = N.linear(h, w["q"]).reshape(T, H, d + r)
    dkv = N.linear(h, w["dkv"])
    c = N.unit_rms(dkv[:, :rank], 1e-5) * w["dkv.norm"]
    kr = N.rotate_half(dkv[:, rank:], pos, m["rot"]["base"], m["rot"]["dims"])
    out = np.zeros((T, H, dv))
    for j in range(H):
        ql = q[:, j, :d] @ w["uk"][j * d:(j + 1) * d]                                      # [T, rank]
        s = (ql @ c.T + N.rotate_half(q[:, j, d:], pos, m["rot"]["base"], m["rot"]["dims"]) @ kr.T) * m["scale"]
        out[:, j] = (N.causal_softmax(s, pos, pos) @ c) @ w["uv"][j * dv:(j + 1) * dv].T
    assert np.allclose(N.linear(out.reshape(T, -1), w["o"]), ref, rtol=1e-10, atol=1e-10)
