"""The Dabodra decoder as data: DabodraConfig -> ModelSpec.

The embedded tokens pass a norm; every layer then adds the *normalised output* of its sublayers to the residual
stream, x += norm1(mixer(x)); x += norm2(ff(x)), the sublayers reading x itself (a layer may have no feed-forward);
the norms are RMS norms whose stored weight w acts as 1 + w.  The mixer is attention over a sliding window with a
sink in the softmax's denominator, or a gated delta rule with state of a fixed size, layer by layer as the
configuration lists them; the feed-forward is a mixture of routed experts and a shared one.  Tensor names: embed,
embed.norm, l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.*, final.norm, head.
"""
from __future__ import annotations

from ..config.dabodra import DabodraConfig
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _mixer(cfg: DabodraConfig, layer) -> PartSpec:
    m = layer.mixer
    if layer.kind == "attention":
        rope = None
        if m.rot_dims:
            rope = PartSpec("rope", {"rope_dim": m.rot_dims, "theta": m.rot_base, "interleaved": True, "scaling": None})
        return PartSpec("sink_attention", {
            "hidden": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "scale": m.scale,
            "window": m.window, "eps": cfg.eps, "position": rope, "prefix": "mix."})
    return PartSpec("gated_delta_rule", {
        "hidden": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_dim": m.vdim,
        "taps": m.conv, "eps": cfg.eps, "prefix": "mix."})


def describe_dabodra(cfg: DabodraConfig) -> ModelSpec:
    norm = lambda name: PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.eps, "tensor": name,      # noqa: E731
                                             "one_plus": True})
    layers = []
    for i, layer in enumerate(cfg.layers):
        parts = {"mixer": _mixer(cfg, layer), "mixer_norm": norm("norm1")}
        if layer.mlp is not None:
            f = layer.mlp
            parts["feed_forward"] = PartSpec("routed_experts", {
                "hidden": cfg.width, "n_experts": f.experts, "top": f.top, "scale": f.scale, "n_groups": f.groups,
                "keep": f.keep, "intermediate": f.ff, "shared_intermediate": f.shared_ff, "prefix": "mlp."})
            parts["feed_forward_norm"] = norm("norm2")
        layers.append(LayerSpec("output_norm_residual", parts, f"l{i}."))
    return ModelSpec(
        hidden=cfg.width, vocab=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab, "hidden": cfg.width, "tensor": "embed",
                                               "norm": norm("embed.norm")}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "hidden": cfg.width, "tied": False, "tensor": "head"}))


DABODRA = register_architecture(Architecture(
    names=("Dabodra",),
    description="Dabodra decoder: windowed attention with a sink and gated delta rule layers, routed experts, "
                "norms behind the sublayers",
    config_class=DabodraConfig,
    describe_model=describe_dabodra,
    # a layer without a feed-forward has no use for a second norm; a file that carries one all the same is accepted
    ignored_tensor_suffixes=(".norm2",)), replace=True)
