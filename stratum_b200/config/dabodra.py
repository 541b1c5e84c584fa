"""DabodraConfig: the sizes and constants of a Dabodra decoder, read from config.json.

A Dabodra config.json names its architecture under "architecture", gives "vocab", "width" and "norm": {"eps"}, and
lists its layers one by one: each entry gives the mixer's kind ("type": "attention" or "delta"), the mixer's sizes
and constants ("mixer") and its feed-forward ("mlp": a mixture of experts, or null for a layer that is a mixer
alone).  Nothing about a layer is assumed from another layer: sizes, windows and constants may differ from one entry
to the next, and the two kinds may come in any order.

  attention mixer   heads, kv_heads, dim, vdim (= dim: the values are the keys as projected), scale,
                    mask: {size} (the sliding window), rot: {base, dims}
  delta mixer       heads, kv_heads, dim, vdim, conv (taps of the short convolution)
  mlp               kind "moe"; router: {experts, top, scale, groups: {count, keep}}; expert: {ff}; shared: {ff}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import KeyReader, ModelConfig

MIXER_KINDS = ("attention", "delta")
MLP_KINDS = ("moe",)


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int              # mask.size: a token sees itself and the window - 1 before it; 0: every token before it
    rot_base: float
    rot_dims: int            # how many of a head's first dimensions are rotated (0: none)

    @classmethod
    def from_reader(cls, r: KeyReader) -> "SinkAttentionConfig":
        heads = r.integer("heads", hi=1 << 14)
        dim = r.integer("dim", hi=1 << 14)
        mask, rot = r.child("mask"), r.child("rot")
        out = cls(heads=heads, kv_heads=r.integer("kv_heads", default=heads, hi=1 << 14), dim=dim,
                  vdim=r.integer("vdim", default=dim, hi=1 << 14), scale=r.number("scale", lo=0.0),
                  window=mask.integer("size", hi=1 << 30) if mask else 0,
                  rot_base=rot.number("base", lo=1.0) if rot else 10000.0,
                  rot_dims=rot.integer("dims", lo=0, hi=1 << 14) if rot else 0)
        for sub in (mask, rot):
            if sub is not None:
                r.adopt(sub)
        if out.heads and out.kv_heads:
            r.require(out.heads % out.kv_heads == 0, f"heads={out.heads} is not a multiple of kv_heads={out.kv_heads}")
        if out.dim and out.vdim:
            r.require(out.vdim == out.dim, f"vdim={out.vdim} must equal dim={out.dim}: the values are the keys as projected")
        if out.dim and out.rot_dims is not None:
            r.require(out.rot_dims % 2 == 0 and out.rot_dims <= out.dim,
                      f"rot.dims={out.rot_dims} must be even and at most dim={out.dim}")
        return out

    def to_dict(self) -> Dict[str, Any]:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
             "rot": {"base": self.rot_base, "dims": self.rot_dims}}
        if self.window:
            d["mask"] = {"size": self.window}
        return d


@dataclass(frozen=True)
class DeltaMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int                # taps of the short convolution, the current token's included

    @classmethod
    def from_reader(cls, r: KeyReader) -> "DeltaMixerConfig":
        heads = r.integer("heads", hi=1 << 14)
        out = cls(heads=heads, kv_heads=r.integer("kv_heads", default=heads, hi=1 << 14),
                  dim=r.integer("dim", hi=512), vdim=r.integer("vdim", hi=1 << 14), conv=r.integer("conv", hi=64))
        if out.heads and out.kv_heads:
            r.require(out.heads % out.kv_heads == 0, f"heads={out.heads} is not a multiple of kv_heads={out.kv_heads}")
        return out

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}


_MIXER_CONFIGS = {"attention": SinkAttentionConfig, "delta": DeltaMixerConfig}


@dataclass(frozen=True)
class RoutedExpertsConfig:
    experts: int
    top: int
    scale: float
    groups: int
    keep: int
    ff: int
    shared_ff: Optional[int]     # None: no shared expert

    @classmethod
    def from_reader(cls, r: KeyReader) -> "RoutedExpertsConfig":
        r.string("kind", choices=MLP_KINDS)
        router, expert = r.child("router"), r.child("expert")
        for key, sub in (("router", router), ("expert", expert)):
            if sub is None:
                r.problems.append(f"missing required key '{key}'")
        groups = router.child("groups") if router else None
        shared = r.child("shared")
        out = cls(experts=router.integer("experts", hi=4096) if router else None,
                  top=router.integer("top", hi=4096) if router else None,
                  scale=router.number("scale", default=1.0) if router else None,
                  groups=groups.integer("count", hi=4096) if groups else 1,
                  keep=groups.integer("keep", hi=4096) if groups else 1,
                  ff=expert.integer("ff", hi=1 << 24) if expert else None,
                  shared_ff=shared.integer("ff", hi=1 << 24) if shared else None)
        if groups is not None:
            router.adopt(groups)
        for sub in (router, expert, shared):
            if sub is not None:
                r.adopt(sub)
        if out.experts and out.groups and out.keep and out.top:
            r.require(out.experts % out.groups == 0, f"experts={out.experts} do not form {out.groups} equal groups")
            r.require(out.keep <= out.groups, f"groups.keep={out.keep} exceeds groups.count={out.groups}")
            if out.experts % out.groups == 0:
                r.require(out.top <= (out.experts // out.groups) * out.keep,
                          f"top={out.top} exceeds the experts of {out.keep} groups")
        return out

    def to_dict(self) -> Dict[str, Any]:
        d = {"kind": "moe", "router": {"experts": self.experts, "top": self.top, "scale": self.scale,
                                       "groups": {"count": self.groups, "keep": self.keep}},
             "expert": {"ff": self.ff}}
        if self.shared_ff is not None:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class DabodraLayer:
    kind: str                                  # one of MIXER_KINDS
    mixer: Any                                 # SinkAttentionConfig | DeltaMixerConfig
    mlp: Optional[RoutedExpertsConfig]         # None: no feed-forward

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.kind, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class DabodraConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    layers: Tuple[DabodraLayer, ...]
    torch_dtype: str = "bfloat16"

    architecture = "Dabodra"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "DabodraConfig":
        r = KeyReader(raw)
        vocab = r.integer("vocab", hi=1 << 26)
        width = r.integer("width", hi=1 << 20)
        norm = r.child("norm")
        eps = norm.number("eps", lo=0.0, hi=1.0) if norm is not None else None
        if norm is None:
            r.problems.append("missing required key 'norm'")
        else:
            r.adopt(norm)
        entries = raw.get("layers")
        layers = []
        if not isinstance(entries, list) or not entries:
            r.problems.append("'layers' must be a non-empty list")
            entries = []
        for i, e in enumerate(entries):
            lr = KeyReader(e if isinstance(e, dict) else {}, f"config.json:layers[{i}]")
            if not isinstance(e, dict):
                lr.problems.append("must be an object")
            kind = lr.string("type", choices=MIXER_KINDS)
            mr = lr.child("mixer")
            mixer = None
            if mr is None:
                lr.problems.append("missing required key 'mixer'")
            elif kind is not None:
                mixer = _MIXER_CONFIGS[kind].from_reader(mr)
                lr.adopt(mr)
            mlp = None
            if isinstance(e, dict) and e.get("mlp") is not None:
                fr = lr.child("mlp")
                if fr is not None:
                    mlp = RoutedExpertsConfig.from_reader(fr)
                    lr.adopt(fr)
            layers.append(DabodraLayer(kind, mixer, mlp))
            r.adopt(lr)
        r.finish()
        return cls(vocab=vocab, width=width, eps=eps, layers=tuple(layers),
                   torch_dtype=raw.get("torch_dtype", "bfloat16"))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.eps}, "layers": [layer.to_dict() for layer in self.layers],
                "torch_dtype": self.torch_dtype}
