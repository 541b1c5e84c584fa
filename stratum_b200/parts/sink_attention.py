"""Grouped-query attention over a sliding window, with normalised queries and keys, values that are the keys as
projected, and a sink in the softmax.

Per token, with h the mixer's input and p its position:  q = Wq h ([heads][d]), k = Wk h ([kv heads][d]), v = k as
projected (there is no value matrix).  q and k are each divided by the root mean square of their whole row (all heads
together, eps inside the root) and multiplied by a gain per column; then the first dimensions of every head are
rotated by the position encoding, pairs (2i, 2i + 1).  Head j (kv head j / (heads / kv heads)):

    s_t = (q_j . k_t) * scale         for the keys t with 0 <= p - t < window (window 0: every t <= p)
    a_t = exp(s_t) / (sum_t exp(s_t) + exp(sink_j))            (the sink has no key and no value and is not scaled)
    o_j = sum_t a_t v_t;      result = Wo concat_j(o_j)

The two projections run as one product whose float32 sums go to one kernel that normalises, rotates, rounds once and
appends to the cache (keys and values have caches of the same shape: csrc/qk_norm_rope.cu); the attention itself is
the general kernel (kernels.AttentionShape) with its window and sink parameters.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import kernels as K
from ..cache.pages import PAGE_TOKENS
from ..cache.store import KVSpec, LayerCache
from .base import Mixer
from .latent_attention import padded
from .linear import ADD_TO_F32, STORE_F32, Linear
from .registry import find_part, register_part
from .spec import PartSpec, TensorSpec


@register_part("mixer", "sink_attention")
class SinkAttention(Mixer):
    """params: hidden, n_heads, n_kv_heads, head_dim, scale, window (0 = all keys), eps (of the two norms), position
    (PartSpec of a rotating position encoding with neighbouring pairs, or None), sink (whether heads have one;
    default yes), prefix, and the tensor names q, k, o, q_norm, k_norm, sink (defaults: q, k, o, q.norm, k.norm,
    sink)."""
    stores_output = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden, self.n_heads, self.n_kv = int(spec["hidden"]), int(spec["n_heads"]), int(spec["n_kv_heads"])
        self.d = int(spec["head_dim"])
        if self.n_heads % self.n_kv:
            raise ValueError(f"attention: {self.n_heads} heads are not a multiple of {self.n_kv} kv heads")
        self.scale, self.eps = float(spec["scale"]), float(spec["eps"])
        self.window = int(spec.get("window", 0) or 0)
        self.has_sink = bool(spec.get("sink", True))
        pos: Optional[PartSpec] = spec.get("position")
        self.position = find_part("position", pos.kind)(pos, runtime) if pos is not None else None
        if self.position is not None:
            layout = self.position.pair_layout()
            if layout is None or not layout[1] or 2 * layout[0] > self.d:
                raise ValueError("sink_attention rotates neighbouring pairs of a head's first dimensions")
        defaults = {"q": "q", "k": "k", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "sink": "sink"}
        self.names = {k: self.prefix + str(spec.get(k + "_tensor", v)) for k, v in defaults.items()}
        self.q_cols, self.k_cols = self.n_heads * self.d, self.n_kv * self.d
        self.w_in: Optional[Linear] = None
        self.w_o: Optional[Linear] = None
        self.shape: Optional[K.AttentionShape] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        n = self.names
        t = {n["q"]: TensorSpec((self.q_cols, self.hidden)), n["k"]: TensorSpec((self.k_cols, self.hidden)),
             n["o"]: TensorSpec((self.hidden, self.q_cols)),
             n["q_norm"]: TensorSpec((self.q_cols,), role="vector", init="ones"),
             n["k_norm"]: TensorSpec((self.k_cols,), role="vector", init="ones")}
        if self.has_sink:
            t[n["sink"]] = TensorSpec((self.n_heads,), role="vector", init="zeros")
        return t

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        self.w_in = Linear(self.runtime, torch.cat([weights[n["q"]], weights[n["k"]]], dim=0).contiguous())
        self.w_o = Linear(self.runtime, weights[n["o"]])
        self.q_gain, self.k_gain = weights[n["q_norm"]].contiguous(), weights[n["k_norm"]].contiguous()
        self.sink = weights[n["sink"]].contiguous() if self.has_sink else None
        self.shape = K.AttentionShape(self.n_heads, self.n_heads // self.n_kv, 1, self.d, self.d, False, self.scale,
                                      window=self.window, sink=self.sink)

    def cache_spec(self) -> KVSpec:
        return KVSpec(self.n_kv, self.d, self.window, "normed_rotated_values_raw")

    def forward(self, xin, residual: torch.Tensor, step, cache: LayerCache, store: bool = False) -> None:
        T = xin.shape[0]
        width = self.q_cols + self.k_cols
        proj = self.runtime.empty(T, padded(width), dtype=torch.float32)
        self.w_in(xin, out=proj[:, :width], mode=STORE_F32)
        q = self.runtime.empty(T, padded(self.q_cols))
        rot = self.position.rotary() if self.position is not None else None
        K.qk_norm_rope(proj, step.token_pos, step.token_seq, cache.block_table, self.q_gain, self.k_gain,
                       None if rot is None else rot.inv_freq, self.eps, q, cache.k, cache.v, self.n_heads, self.n_kv,
                       self.d, PAGE_TOKENS, cache.writes)
        out = self.runtime.empty(T, padded(self.q_cols))
        from . import attention_dispatch
        attention_dispatch.run_general(self, self.shape, q, cache, step, out)
        self.w_o(out[:, :self.q_cols], out=residual, mode=STORE_F32 if store else ADD_TO_F32)
