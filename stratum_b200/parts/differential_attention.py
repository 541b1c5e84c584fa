"""Differential attention: every head computes two attention maps over the same values and keeps their
difference.

Per token, with h the mixer's input and p its position:  q = Wq h ([heads][2][d]), k = Wk h ([kv heads][2][d]),
v = Wv h ([kv heads][dv]); no rotation.  Map m of head j (kv head j / (heads / kv heads)):

    s_t = (q_jm . k_tm) * scale * (1 + coef ln(floor((p + 1) / every) + 1)),   s_t <- cap tanh(s_t / cap),
    a_m = sum_t softmax_t(s) v_t                                   (causal, optionally the last `window` keys)

    o = a_0 - lambda a_1,   lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff       (one number per layer)
    o <- o / sqrt(mean(o^2) + eps) * (1 - diff) * sigmoid((Wg h)_j);   residual += Wo concat_j(o)

The query factor multiplies the float32 score (it is the same number for every key of a row), so q is not rounded
a second time.  q, k, v and the gate's pre-activations come from one matrix product over the stacked weights; the
cache keeps keys as 2 x kv heads of d and values as kv heads of dv.
"""
from __future__ import annotations

import math
from typing import Dict, Mapping, Optional

import torch

from .. import kernels as K
from ..cache.pages import PAGE_TOKENS
from ..cache.store import KVSpec, LayerCache
from .base import Mixer
from .latent_attention import padded
from .linear import ADD_TO_F32, STORE, Linear
from .registry import register_part
from .spec import TensorSpec


@register_part("mixer", "differential_attention")
class DifferentialAttention(Mixer):
    """params: hidden, n_heads, n_kv_heads, head_dim, v_dim, scale, softcap (0 = none), diff, eps, temp_coef and
    temp_every (the query factor; coef 0 = none), gate (whether heads have an output gate), window (0 = all
    keys), prefix, and the tensor names q, k, v, g, o, lq1, lk1, lq2, lk2 (defaults: those words)."""
    replays_prompts = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden, self.n_heads, self.n_kv = int(spec["hidden"]), int(spec["n_heads"]), int(spec["n_kv_heads"])
        self.d, self.dv = int(spec["head_dim"]), int(spec["v_dim"])
        if self.n_heads % self.n_kv:
            raise ValueError(f"attention: {self.n_heads} heads are not a multiple of {self.n_kv} kv heads")
        self.scale, self.softcap = float(spec["scale"]), float(spec.get("softcap", 0.0) or 0.0)
        self.diff, self.eps = float(spec["diff"]), float(spec["eps"])
        self.temp_coef, self.temp_every = float(spec.get("temp_coef", 0.0) or 0.0), int(spec.get("temp_every", 1) or 1)
        self.gate = bool(spec.get("gate", True))
        self.window = int(spec.get("window", 0) or 0)
        self.names = {k: self.prefix + str(spec.get(k, k)) for k in ("q", "k", "v", "g", "o", "lq1", "lk1", "lq2", "lk2")}
        self.q_cols = self.n_heads * 2 * self.d
        self.k_cols, self.v_cols = self.n_kv * 2 * self.d, self.n_kv * self.dv
        self.shape: Optional[K.AttentionShape] = None
        self.w_in: Optional[Linear] = None
        self.w_o: Optional[Linear] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        n = self.names
        t = {n["q"]: TensorSpec((self.q_cols, self.hidden)), n["k"]: TensorSpec((self.k_cols, self.hidden)),
             n["v"]: TensorSpec((self.v_cols, self.hidden)), n["o"]: TensorSpec((self.hidden, self.n_heads * self.dv))}
        for key in ("lq1", "lk1", "lq2", "lk2"):
            t[n[key]] = TensorSpec((self.d,), role="vector")
        if self.gate:
            t[n["g"]] = TensorSpec((self.n_heads, self.hidden))
        return t

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        stack = [weights[n["q"]], weights[n["k"]], weights[n["v"]]] + ([weights[n["g"]]] if self.gate else [])
        self.w_in = Linear(self.runtime, torch.cat(stack, dim=0).contiguous())
        self.w_o = Linear(self.runtime, weights[n["o"]])
        # lambda: a constant of the layer, evaluated once in float32 from the four vectors
        f = lambda key: weights[n[key]].to(torch.float32)                        # noqa: E731
        lam = torch.exp(torch.sum(f("lq1") * f("lk1"))) - torch.exp(torch.sum(f("lq2") * f("lk2")))
        self.lam = float(lam.item()) + self.diff
        self.shape = K.AttentionShape(self.n_heads, self.n_heads // self.n_kv, 2, self.d, self.dv, False, self.scale,
                                      softcap=self.softcap, window=self.window, temp_coef=self.temp_coef,
                                      temp_every=self.temp_every, lam=self.lam, out_scale=1.0 - self.diff,
                                      eps=self.eps,
                                      gate_col=self.q_cols + self.k_cols + self.v_cols if self.gate else -1)

    def cache_spec(self) -> KVSpec:
        return KVSpec(2 * self.n_kv, self.d, self.window, "two_maps_per_head", value_heads=self.n_kv,
                      value_dim=self.dv)

    def forward(self, xn, residual: torch.Tensor, step, cache: LayerCache, emit=None) -> None:
        T = xn.shape[0]
        width = self.q_cols + self.k_cols + self.v_cols + (self.n_heads if self.gate else 0)
        proj = self.runtime.empty(T, padded(width))
        self.w_in(xn, out=proj[:, :width], mode=STORE)
        K.mixer_prep(proj, step.token_pos, step.token_seq, cache.block_table, cache.k, cache.v, PAGE_TOKENS,
                     cache.writes, keys=(2 * self.n_kv, self.d, self.q_cols),
                     values=(self.n_kv, self.dv, self.q_cols + self.k_cols))
        out = self.runtime.empty(T, padded(self.n_heads * self.dv))
        from . import attention_dispatch
        attention_dispatch.run_general(self, self.shape, proj, cache, step, out)
        self.w_o(out[:, :self.n_heads * self.dv], out=residual, mode=ADD_TO_F32)
