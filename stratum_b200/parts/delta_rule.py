"""The gated delta rule: a recurrent mixer that keeps, per sequence and head, one matrix S [d][dv] in float32.

Per token, with h the mixer's input:  q = Wq h, k = Wk h ([kv heads][d]), v = Wv h ([heads][dv]); each passes a short
causal convolution over time per channel (taps per channel, the last one the current token's, zeros before the
sequence's start) and silu; q and k become unit vectors per head (x / sqrt(sum x^2 + 1e-6)) and q is divided by
sqrt(d).  beta = sigmoid(Wb h) and decay = exp(-exp(A_log) softplus(Wa h + dt_bias)), one each per head.  Head j (its
q and k are those of head j / (heads / kv heads)), in this order:

    S <- decay S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q           (o sees the token's own write)

    o <- o / sqrt(mean(o^2) + eps) * gain * silu(Wg h)_j;      result = Wo concat_j(o)

What a sequence keeps between steps is S and the last taps - 1 inputs of the convolution: a block of fixed size per
sequence (cache.StateSpec), whatever its length.  All six projections run as one product with float32 sums;
everything between them and the output product is float32 (csrc/delta_rule.cu).
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import kernels as K
from ..cache.store import LayerCache, StateSpec
from .base import Mixer
from .latent_attention import padded
from .linear import ADD_TO_F32, STORE_F32, Linear
from .registry import register_part
from .spec import TensorSpec


@register_part("mixer", "gated_delta_rule")
class GatedDeltaRule(Mixer):
    """params: hidden, n_heads, n_kv_heads, head_dim, v_dim, taps, eps (of the output norm), prefix, and the tensor
    names q, k, v, b, a, g, o, norm, A_log, dt_bias (defaults: those words; the taps of q, k, v are name + ".conv")."""
    stores_output = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden, self.n_heads, self.n_kv = int(spec["hidden"]), int(spec["n_heads"]), int(spec["n_kv_heads"])
        self.d, self.dv, self.taps = int(spec["head_dim"]), int(spec["v_dim"]), int(spec["taps"])
        if self.n_heads % self.n_kv:
            raise ValueError(f"delta rule: {self.n_heads} heads are not a multiple of {self.n_kv} q/k heads")
        self.eps = float(spec["eps"])
        keys = ("q", "k", "v", "b", "a", "g", "o", "norm", "A_log", "dt_bias")
        self.names = {k: self.prefix + str(spec.get(k + "_tensor", k)) for k in keys}
        self.qk_cols, self.v_cols = self.n_kv * self.d, self.n_heads * self.dv
        self.channels = 2 * self.qk_cols + self.v_cols
        self.width = self.channels + 2 * self.n_heads + self.v_cols          # columns of the fused projection
        self.w_in: Optional[Linear] = None
        self.w_o: Optional[Linear] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        n, H = self.names, self.hidden
        t = {n["q"]: TensorSpec((self.qk_cols, H)), n["k"]: TensorSpec((self.qk_cols, H)),
             n["v"]: TensorSpec((self.v_cols, H)), n["b"]: TensorSpec((self.n_heads, H)),
             n["a"]: TensorSpec((self.n_heads, H)), n["g"]: TensorSpec((self.v_cols, H)),
             n["o"]: TensorSpec((H, self.v_cols)),
             n["norm"]: TensorSpec((self.dv,), role="vector", init="ones"),
             n["A_log"]: TensorSpec((self.n_heads,), role="vector", init="zeros"),
             n["dt_bias"]: TensorSpec((self.n_heads,), role="vector", init="zeros")}
        for key, cols in (("q", self.qk_cols), ("k", self.qk_cols), ("v", self.v_cols)):
            t[n[key] + ".conv"] = TensorSpec((cols, self.taps), role="vector")
        return t

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        stack = [weights[n[k]] for k in ("q", "k", "v", "b", "a", "g")]
        self.w_in = Linear(self.runtime, torch.cat(stack, dim=0).contiguous())
        self.w_o = Linear(self.runtime, weights[n["o"]])
        self.conv_w = torch.cat([weights[n[k] + ".conv"] for k in ("q", "k", "v")], dim=0).contiguous()
        self.a_log, self.dt_bias = weights[n["A_log"]].contiguous(), weights[n["dt_bias"]].contiguous()
        self.gain = weights[n["norm"]].contiguous()

    def cache_spec(self) -> StateSpec:
        return StateSpec((self.n_heads * self.d * self.dv + (self.taps - 1) * self.channels,), "float32")

    def forward(self, xin, residual: torch.Tensor, step, cache: LayerCache, store: bool = False) -> None:
        T = xin.shape[0]
        f32 = torch.float32
        proj = self.runtime.empty(T, padded(self.width), dtype=f32)
        self.w_in(xin, out=proj[:, :self.width], mode=STORE_F32)
        act = self.runtime.empty(T, padded(self.channels + 2 * self.n_heads + self.n_kv), dtype=f32)
        o_raw = self.runtime.empty(T, self.v_cols, dtype=f32)
        out = self.runtime.empty(T, padded(self.v_cols))
        K.delta_rule(proj, self.conv_w, self.a_log, self.dt_bias, self.gain, act, o_raw, out, cache.state,
                     step.token_pos, step.token_seq, step.seq_start, step.seq_slot, self.n_heads, self.n_kv, self.d,
                     self.dv, self.eps, cache.writes)
        self.w_o(out[:, :self.v_cols], out=residual, mode=STORE_F32 if store else ADD_TO_F32)
