"""The Nibelorn decoder as data: NibelornConfig -> ModelSpec.

Every layer is pre-norm around the residual stream: x += mixer(norm1(x)); x += ff(norm2(x)) (a layer may have no
feed-forward), with Dynamic Tanh norms.  The mixer is latent attention or differential attention, layer by layer
as the configuration lists them; the feed-forward is dense with the exact GELU.  A layer that names another
layer's tensors runs as one more stop of that layer in the schedule: shared weights, a cache of its own.  Tensor
names: embed, l<i>.norm1[.b|.alpha], l<i>.norm2[...], l<i>.mix.*, l<i>.mlp.up / .down, final.norm[...], head.
"""
from __future__ import annotations

from ..config.nibelorn import NibelornConfig
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _mixer(cfg: NibelornConfig, layer) -> PartSpec:
    m = layer.mixer
    if layer.kind == "latent_attention":
        rope = PartSpec("rope", {"rope_dim": m.rot_dims, "theta": m.rot_base, "interleaved": False, "scaling": None})
        return PartSpec("latent_attention", {
            "hidden": cfg.width, "n_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_dim": m.vdim,
            "kv_rank": m.kv_rank, "scale": m.scale, "eps": cfg.eps, "position": rope, "window": 0, "prefix": "mix."})
    return PartSpec("differential_attention", {
        "hidden": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_dim": m.vdim,
        "scale": m.scale, "softcap": m.softcap, "diff": m.diff, "eps": cfg.eps, "temp_coef": m.temp_coef,
        "temp_every": m.temp_every, "gate": True, "window": 0, "prefix": "mix."})


def describe_nibelorn(cfg: NibelornConfig) -> ModelSpec:
    norm = lambda name: PartSpec("dynamic_tanh", {"size": cfg.width, "name": name})      # noqa: E731
    layers, index_of, schedule = [], {}, []
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is None:
            parts = {"mixer_norm": norm("norm1"), "mixer": _mixer(cfg, layer)}
            if layer.ff is not None:
                parts["feed_forward_norm"] = norm("norm2")
                parts["feed_forward"] = PartSpec("dense_gelu", {"hidden": cfg.width, "intermediate": layer.ff,
                                                                "activation": "gelu_erf", "prefix": "mlp."})
            index_of[i] = len(layers)
            layers.append(LayerSpec("prenorm_residual", parts, f"l{i}."))
    for i, layer in enumerate(cfg.layers):
        schedule.append(ScheduleEntry(index_of[i if layer.weights_of is None else layer.weights_of]))
    return ModelSpec(
        hidden=cfg.width, vocab=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab, "hidden": cfg.width, "tensor": "embed"}),
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "hidden": cfg.width, "tied": False, "tensor": "head"}))


NIBELORN = register_architecture(Architecture(
    names=("Nibelorn",),
    description="Nibelorn decoder: latent and differential attention layers, Dynamic Tanh norms, dense GELU",
    config_class=NibelornConfig,
    describe_model=describe_nibelorn,
    # a layer without a feed-forward has no use for a second norm; a file that carries one all the same is accepted
    ignored_tensor_suffixes=(".norm2", ".norm2.b", ".norm2.alpha")), replace=True)
