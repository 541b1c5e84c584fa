"""Latent attention: keys and values of all heads are expansions of one small vector per token, and only that
vector (with one rotated key part shared by the heads) is kept in the cache.

Per token, with h the mixer's input:  q = Wq h, per head [d plain | r rotated];  Wdkv h = [c' | kr];
c = c' / sqrt(mean(c'^2) + eps) * g;  kr and the rotated part of every query head are rotated by the position.
Head j's key is Wuk_j c and its value Wuv_j c, so its score against token t is

    (q_plain_j . Wuk_j c_t + q_rot_j . kr_t) * scale  =  ((Wuk_j^T q_plain_j) . c_t + q_rot_j . kr_t) * scale

and its output Wuv_j (sum_t a_t c_t).  The right-hand forms are what runs: the query is carried into the latent
space once per token ([Wuk_j^T q_plain_j | q_rot_j], rank + r numbers), every head attends over the same cached
rows [c_t | kr_t], whose first `rank` numbers are also the values, and the head's mixed latent is expanded by
Wuv_j afterwards.  Neither keys nor values of the heads are ever formed for cached tokens, which is the point of
the design: a step reads rank + r numbers per cached token, whatever the number of heads.

A prompt that begins at position 0 has no cached tokens to spare: all its keys are this step's own.  There the
left-hand form costs a quarter of the arithmetic (heads of d + r and dv numbers against rank + r and rank), and on
the bfloat16 path, where attention over a long prompt is bound by the tensor cores, it is what runs: the heads' keys
[Wuk_j c | kr] come from one product of the step's rows [c | kr] with the matrix that stacks [Wuk_j 0; 0 I] per
head, the values from Wuv c, and the general attention reads them as plain matrices.  The cache is written all
the same, for the steps that follow.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import os

import torch

from .. import kernels as K
from ..cache.pages import PAGE_TOKENS
from ..cache.store import KVSpec, LayerCache
from .base import Mixer
from .linear import ADD_TO_F32, STORE, HeadLinear, Linear
from .registry import find_part, register_part
from .spec import PartSpec, TensorSpec


# prompts from this many tokens on take the per-head form on the bfloat16 path (below it the absorbed form's
# arithmetic is not what a step waits for; STRATUM_LATENT_PER_HEAD=0 turns the form off: measurements)
PER_HEAD_MIN_TOKENS = int(os.environ.get("STRATUM_LATENT_PER_HEAD_MIN", 256))


def padded(n: int, to: int = 8) -> int:
    return (n + to - 1) // to * to


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    """params: hidden, n_heads, head_dim (the unrotated query/key size), rot_dim, v_dim, kv_rank, scale, eps (of
    the latent's norm), position (PartSpec of a rotating position encoding over at most rot_dim dimensions),
    window (0 = all keys), prefix, and the tensor names q, dkv, dkv_norm, uk, uv, o (defaults: those words, with
    "dkv.norm")."""

    @property
    def replays_prompts(self) -> bool:
        return bool(getattr(self.position, "replays_prompts", False))

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden, self.n_heads = int(spec["hidden"]), int(spec["n_heads"])
        self.d, self.r, self.dv, self.rank = (int(spec["head_dim"]), int(spec["rot_dim"]), int(spec["v_dim"]),
                                              int(spec["kv_rank"]))
        self.scale, self.eps = float(spec["scale"]), float(spec["eps"])
        self.window = int(spec.get("window", 0) or 0)
        pos: PartSpec = spec["position"]
        self.position = find_part("position", pos.kind)(pos, runtime)
        layout = self.position.pair_layout()
        if layout is None or layout[1] or 2 * layout[0] > self.r:
            raise ValueError("latent attention rotates pairs (i, i + n/2) of at most rot_dim dimensions")
        self.names = {k: self.prefix + str(spec.get(k, k if k != "dkv_norm" else "dkv.norm"))
                      for k in ("q", "dkv", "dkv_norm", "uk", "uv", "o")}
        self.shape = K.AttentionShape(self.n_heads, self.n_heads, 1, self.rank + self.r, self.rank, True, self.scale,
                                      window=self.window)
        self.w_in: Optional[Linear] = None
        self.w_o: Optional[Linear] = None
        self.uk: Optional[HeadLinear] = None
        self.uv: Optional[HeadLinear] = None
        self.gain: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        n, H = self.names, self.n_heads
        return {n["q"]: TensorSpec((H * (self.d + self.r), self.hidden)),
                n["dkv"]: TensorSpec((self.rank + self.r, self.hidden)),
                n["dkv_norm"]: TensorSpec((self.rank,), role="vector", init="ones"),
                n["uk"]: TensorSpec((H * self.d, self.rank)),
                n["uv"]: TensorSpec((H * self.dv, self.rank)),
                n["o"]: TensorSpec((self.hidden, H * self.dv))}

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        n, H = self.names, self.n_heads
        self.w_in = Linear(self.runtime, torch.cat([weights[n["q"]], weights[n["dkv"]]], dim=0).contiguous())
        self.gain = weights[n["dkv_norm"]]
        # head j carries its plain query into the latent space with Wuk_j^T: a matrix [rank, d] per head
        self.uk = HeadLinear(self.runtime, weights[n["uk"]].view(H, self.d, self.rank).transpose(1, 2).contiguous())
        self.uv = HeadLinear(self.runtime, weights[n["uv"]].view(H, self.dv, self.rank))
        self.w_o = Linear(self.runtime, weights[n["o"]])
        # the per-head form of whole prompts (bfloat16): keys of all heads from the rows [c | kr] in one product
        self.w_keys = self.w_values = None
        if self.runtime.dtype == torch.bfloat16 and (self.d + self.r) % 8 == 0 and self.dv % 8 == 0:
            d, r, rank = self.d, self.r, self.rank
            stack = torch.zeros((H, d + r, rank + r), dtype=torch.bfloat16, device=weights[n["uk"]].device)
            stack[:, :d, :rank] = weights[n["uk"]].view(H, d, rank)
            stack[:, d:, rank:] = torch.eye(r, dtype=torch.bfloat16, device=stack.device)
            self.w_keys = Linear(self.runtime, stack.view(H * (d + r), rank + r))
            self.w_values = Linear(self.runtime, weights[n["uv"]])
            self.head_shape = K.AttentionShape(H, 1, 1, d + r, self.dv, False, self.scale, window=self.window)

    def cache_spec(self) -> KVSpec:
        return KVSpec(1, self.rank + self.r, self.window, f"latent_{self.rank}_then_rotated", value_heads=0)

    def _per_head_form(self, step, cache: LayerCache) -> bool:
        """Whether this step forms the heads' keys and values instead of carrying queries into the latent space:
        bfloat16, a prompt step launched launch by launch (a replayed step's shape says nothing about where its
        sequences begin) in which every sequence begins at position 0 and the longest brings PER_HEAD_MIN_TOKENS."""
        if self.w_keys is None or step.all_single or step.fixed_qblocks is not None or step.sizes_seen is not None:
            return False
        if not cache.writes or self.window or os.environ.get("STRATUM_LATENT_PER_HEAD", "1") == "0":
            return False
        before = (step.host or {}).get("before")
        return bool(before) and all(b == 0 for b in before) and step.max_new >= PER_HEAD_MIN_TOKENS

    def _forward_per_head(self, proj, step, cache: LayerCache, residual: torch.Tensor) -> None:
        H, d, r, rank, dv = self.n_heads, self.d, self.r, self.rank, self.dv
        T = proj.shape[0]
        q_cols = H * (d + r)
        rows = self.runtime.empty(T, padded(rank + r))            # [c | kr] of the step's tokens
        K.mixer_prep(proj, step.token_pos, step.token_seq, cache.block_table, cache.k, None, PAGE_TOKENS, True,
                     queries=(H, d + r, 0), q_rot_off=d, keys=(1, rank + r, q_cols), k_rot_off=rank,
                     inv_freq=self.position.rotary().inv_freq, k_norm_gain=self.gain, eps=self.eps, k_out=rows)
        # 64 rows beyond the step's: the last tile of the last sequence reads (and ignores) them
        keys = self.runtime.empty(T + PAGE_TOKENS, padded(H * (d + r)))
        values = self.runtime.empty(T + PAGE_TOKENS, padded(H * dv))
        keys[T:].zero_()
        values[T:].zero_()
        self.w_keys(rows[:, :rank + r], out=keys[:T, :H * (d + r)], mode=STORE)
        self.w_values(rows[:, :rank], out=values[:T, :H * dv], mode=STORE)
        heads = self.runtime.empty(T, padded(H * dv))
        from . import attention_dispatch
        attention_dispatch.run_general_dense(self, self.head_shape, proj, keys, values, step, heads)
        self.w_o(heads[:, :H * dv], out=residual, mode=ADD_TO_F32)

    def forward(self, xn, residual: torch.Tensor, step, cache: LayerCache, emit=None) -> None:
        H, d, r, rank, dv = self.n_heads, self.d, self.r, self.rank, self.dv
        T = xn.shape[0]
        q_cols, width = H * (d + r), H * (d + r) + rank + r
        proj = self.runtime.empty(T, padded(width))
        self.w_in(xn, out=proj[:, :width], mode=STORE)
        if self._per_head_form(step, cache) and K.attention_general_mma_ok(self.head_shape, proj, proj, PAGE_TOKENS):
            self._forward_per_head(proj, step, cache, residual)
            return
        q_lat = self.runtime.empty(T, padded(H * (rank + r)))
        K.mixer_prep(proj, step.token_pos, step.token_seq, cache.block_table, cache.k, None, PAGE_TOKENS, cache.writes,
                     queries=(H, d + r, 0), q_rot_off=d, keys=(1, rank + r, q_cols), k_rot_off=rank,
                     inv_freq=self.position.rotary().inv_freq, k_norm_gain=self.gain, eps=self.eps,
                     q_out=q_lat, q_out_step=rank + r, q_out_off=rank)
        self.uk(proj, d + r, q_lat, rank + r)
        mixed = self.runtime.empty(T, padded(H * rank))
        from . import attention_dispatch
        attention_dispatch.run_general(self, self.shape, q_lat, cache, step, mixed)
        heads = self.runtime.empty(T, padded(H * dv))
        self.uv(mixed, rank, heads, dv)
        self.w_o(heads[:, :H * dv], out=residual, mode=ADD_TO_F32)
