"""NibelornConfig: the sizes and constants of a Nibelorn decoder, read from config.json.

A Nibelorn config.json names its architecture under "architecture" and lists its layers one by one: each entry
gives the mixer's kind ("type"), the mixer's sizes and constants ("mixer"), its feed-forward ("mlp": {"kind",
"ff"}, or null for a layer that is a mixer alone) and, optionally, "weights_of": the index of the layer whose
tensors it uses (it keeps a cache of its own).  The norm is Dynamic Tanh throughout; "norm": {"eps"} is the eps of
the root mean squares inside the mixers.  Nothing about a layer is assumed from another layer: sizes may differ
from one entry to the next.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, KeyReader, ModelConfig

MIXER_KINDS = ("latent_attention", "attention")
MLP_KINDS = ("dense",)


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int                 # unrotated query/key dimensions per head
    rot_dim: int             # rotated query/key dimensions per head (the key's are shared by the heads)
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int            # how many of the rot_dim dimensions are rotated

    @classmethod
    def from_reader(cls, r: KeyReader) -> "LatentMixerConfig":
        rot = r.child("rot")
        if rot is None:
            r.problems.append("missing required key 'rot'")
        out = cls(heads=r.integer("heads", hi=1 << 14), dim=r.integer("dim", hi=1 << 14),
                  rot_dim=r.integer("rot_dim", hi=1 << 14), vdim=r.integer("vdim", hi=1 << 14),
                  kv_rank=r.integer("kv_rank", hi=1 << 16), scale=r.number("scale", lo=0.0),
                  rot_base=rot.number("base", lo=1.0) if rot else None,
                  rot_dims=rot.integer("dims", hi=1 << 14) if rot else None)
        if rot is not None:
            r.adopt(rot)
        if out.rot_dims and out.rot_dim:
            r.require(out.rot_dims % 2 == 0 and out.rot_dims <= out.rot_dim,
                      f"rot.dims={out.rot_dims} must be even and at most rot_dim={out.rot_dim}")
        return out

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                "kv_rank": self.kv_rank, "scale": self.scale, "rot": {"base": self.rot_base, "dims": self.rot_dims}}


@dataclass(frozen=True)
class DifferentialMixerConfig:
    heads: int
    kv_heads: int
    dim: int                 # query/key dimensions per head and map
    vdim: int
    scale: float
    softcap: float
    diff: float
    temp_coef: float
    temp_every: int

    @classmethod
    def from_reader(cls, r: KeyReader) -> "DifferentialMixerConfig":
        temp = r.child("q_temp")
        if temp is None:
            r.problems.append("missing required key 'q_temp'")
        heads = r.integer("heads", hi=1 << 14)
        out = cls(heads=heads, kv_heads=r.integer("kv_heads", default=heads, hi=1 << 14),
                  dim=r.integer("dim", hi=1 << 14), vdim=r.integer("vdim", hi=1 << 14),
                  scale=r.number("scale", lo=0.0), softcap=r.number("softcap", lo=0.0), diff=r.number("diff"),
                  temp_coef=temp.number("coef") if temp else None,
                  temp_every=temp.integer("every", hi=1 << 30) if temp else None)
        if temp is not None:
            r.adopt(temp)
        if out.heads and out.kv_heads:
            r.require(out.heads % out.kv_heads == 0, f"heads={out.heads} is not a multiple of kv_heads={out.kv_heads}")
        return out

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                "scale": self.scale, "softcap": self.softcap, "diff": self.diff,
                "q_temp": {"coef": self.temp_coef, "every": self.temp_every}}


_MIXER_CONFIGS = {"latent_attention": LatentMixerConfig, "attention": DifferentialMixerConfig}


@dataclass(frozen=True)
class NibelornLayer:
    kind: str                                  # one of MIXER_KINDS
    mixer: Any                                 # LatentMixerConfig | DifferentialMixerConfig
    ff: Optional[int]                          # inner size of the dense feed-forward; None: no feed-forward
    weights_of: Optional[int] = None           # the layer whose tensors this one uses

    def to_dict(self) -> Dict[str, Any]:
        d = {"type": self.kind, "mixer": self.mixer.to_dict(),
             "mlp": None if self.ff is None else {"kind": "dense", "ff": self.ff}}
        if self.weights_of is not None:
            d["weights_of"] = self.weights_of
        return d


@dataclass(frozen=True)
class NibelornConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    layers: Tuple[NibelornLayer, ...]
    torch_dtype: str = "bfloat16"

    architecture = "Nibelorn"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "NibelornConfig":
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
            ff = None
            if e.get("mlp") is not None if isinstance(e, dict) else False:
                fr = lr.child("mlp")
                if fr is not None:
                    fr.string("kind", choices=MLP_KINDS)
                    ff = fr.integer("ff", hi=1 << 24)
                    lr.adopt(fr)
            of = lr.integer("weights_of", default=None, lo=0, hi=len(entries) - 1)
            if of is not None:
                lr.require(of != i, "weights_of names the layer itself")
            layers.append(NibelornLayer(kind, mixer, ff, of))
            r.adopt(lr)
        # a layer that borrows tensors borrows them, directly or through other borrowers, from a layer that has its
        # own, of the same shape
        for i, layer in enumerate(layers):
            if layer.weights_of is None or layer.weights_of >= len(layers):
                continue
            j, seen = layer.weights_of, {i}
            while j not in seen and j < len(layers) and layers[j].weights_of is not None:
                seen.add(j)
                j = layers[j].weights_of
            if j in seen or j >= len(layers):
                r.problems.append(f"layers[{i}].weights_of={layer.weights_of} leads to no layer with tensors of its own")
                continue
            src = layers[j]
            if j != layer.weights_of:
                layers[i] = NibelornLayer(layer.kind, layer.mixer, layer.ff, j)
            r.require((src.kind, src.mixer, src.ff) == (layer.kind, layer.mixer, layer.ff),
                      f"layers[{i}] differs from layers[{j}], whose tensors it uses")
        r.finish()
        return cls(vocab=vocab, width=width, eps=eps, layers=tuple(layers),
                   torch_dtype=raw.get("torch_dtype", "bfloat16"))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.eps}, "layers": [layer.to_dict() for layer in self.layers],
                "torch_dtype": self.torch_dtype}
