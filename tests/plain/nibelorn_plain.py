"""Plain, slow restatement of the Nibelorn decoder, used only as a test oracle.

Whole sequences, no cache, one function per mechanism, float64 throughout, no code shared with
the product package.  Notation: h is a mixer's input [T, width]; p the positions 0..T-1; a
weight matrix is [out, in] and acts as h @ W.T.

  dynamic tanh        y = tanh(alpha x) * w + b                     (elementwise; no row statistic)
  rotation            pairs (i, i + n/2), i < n/2, angle p * base^(-2i/n):
                      (u, v) -> (u cos - v sin, v cos + u sin)
  latent attention    q = Wq h split per head into [d plain | r rotated];  Wdkv h = [c' | kr];
                      c = c' / rms(c') * g;  kr rotated once for all heads;  per head
                      k = Wuk c, v = Wuv c;  s = (q_plain . k + rot(q_rot) . rot(kr)) * scale;
                      causal softmax;  o = Wo concat_h(sum_j a_j v_j)
  differential attn   q, k hold two maps per head; both maps attend over the same v;
                      q *= 1 + coef ln(floor((p + 1) / every) + 1);
                      s = cap tanh(q . k scale / cap);  lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff;
                      o = a1 - lambda a2;  o /= rms(o);  o *= 1 - diff;  o *= sigmoid(Wg h)_head;  Wo
  feed-forward        Wdown gelu_erf(Wup h)
"""
from __future__ import annotations

import math
from typing import Dict, List, Sequence

import numpy as np

F64 = np.float64


def linear(x, w):
    return np.asarray(x, F64) @ np.asarray(w, F64).T


def dynamic_tanh(x, w, b, alpha):
    return np.tanh(F64(alpha) * np.asarray(x, F64)) * np.asarray(w, F64) + np.asarray(b, F64)


def unit_rms(x, eps):
    x = np.asarray(x, F64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + F64(eps))


def rotate_half(x, pos, base, n):
    """x [..., T, m] with m >= n: the first n dimensions rotated, pair (i, i + n/2); the rest unchanged."""
    x = np.array(x, F64)
    half = n // 2
    f = F64(base) ** (-2.0 * np.arange(half, dtype=F64) / F64(n))
    a = np.asarray(pos, F64)[:, None] * f[None, :]
    c, s = np.cos(a), np.sin(a)
    u, v = x[..., :half].copy(), x[..., half:n].copy()
    x[..., :half] = u * c - v * s
    x[..., half:n] = v * c + u * s
    return x


def causal_softmax(scores, pos_q, pos_k):
    """scores [Tq, Tk]; key j is visible to query i when pos_k[j] <= pos_q[i]."""
    vis = np.asarray(pos_k)[None, :] <= np.asarray(pos_q)[:, None]
    s = np.where(vis, scores, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    e = np.exp(s)
    return e / e.sum(axis=-1, keepdims=True)


def gelu_erf(z):
    z = np.asarray(z, F64)
    return 0.5 * z * (1.0 + np.vectorize(math.erf)(z / math.sqrt(2.0)))


def latent_attention(h, w: Dict[str, np.ndarray], m: dict, eps: float, pos=None):
    """w: the mixer's tensors by their short names (q, dkv, dkv.norm, uk, uv, o); m: the mixer's sizes."""
    T = h.shape[0]
    pos = np.arange(T) if pos is None else np.asarray(pos)
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base, n_rot = m["rot"]["base"], m["rot"]["dims"]
    q = linear(h, w["q"]).reshape(T, H, d + r)
    dkv = linear(h, w["dkv"])
    c = unit_rms(dkv[:, :rank], eps) * np.asarray(w["dkv.norm"], F64)
    kr = rotate_half(dkv[:, rank:], pos, base, n_rot)                      # [T, r], one for all heads
    k = linear(c, w["uk"]).reshape(T, H, d)
    v = linear(c, w["uv"]).reshape(T, H, dv)
    out = np.zeros((T, H, dv), F64)
    for j in range(H):
        qr = rotate_half(q[:, j, d:], pos, base, n_rot)
        s = (q[:, j, :d] @ k[:, j].T + qr @ kr.T) * F64(m["scale"])
        out[:, j] = causal_softmax(s, pos, pos) @ v[:, j]
    return linear(out.reshape(T, H * dv), w["o"])


def differential_attention(h, w: Dict[str, np.ndarray], m: dict, eps: float, pos=None):
    """w: q, k, v, lq1, lk1, lq2, lk2, g, o."""
    T = h.shape[0]
    pos = np.arange(T) if pos is None else np.asarray(pos)
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = linear(h, w["q"]).reshape(T, H, 2, d)
    k = linear(h, w["k"]).reshape(T, G, 2, d)
    v = linear(h, w["v"]).reshape(T, G, dv)
    temp = 1.0 + F64(m["q_temp"]["coef"]) * np.log(np.floor((pos + 1) / m["q_temp"]["every"]) + 1.0)
    q = q * temp[:, None, None, None]
    lam = (math.exp(float(np.sum(np.asarray(w["lq1"], F64) * np.asarray(w["lk1"], F64))))
           - math.exp(float(np.sum(np.asarray(w["lq2"], F64) * np.asarray(w["lk2"], F64)))) + m["diff"])
    gate = 1.0 / (1.0 + np.exp(-linear(h, w["g"])))                        # [T, H]
    cap = F64(m["softcap"])
    out = np.zeros((T, H, dv), F64)
    for j in range(H):
        g = j // (H // G)
        maps = []
        for n in range(2):
            s = q[:, j, n] @ k[:, g, n].T * F64(m["scale"])
            s = cap * np.tanh(s / cap)
            maps.append(causal_softmax(s, pos, pos) @ v[:, g])
        o = maps[0] - lam * maps[1]
        out[:, j] = unit_rms(o, eps) * (1.0 - m["diff"]) * gate[:, j:j + 1]
    return linear(out.reshape(T, H * dv), w["o"])


def dense_feed_forward(h, w: Dict[str, np.ndarray]):
    return linear(gelu_erf(linear(h, w["up"])), w["down"])


MIXERS = {"latent_attention": latent_attention, "attention": differential_attention}


def _sub(w, prefix):
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def _norm(x, w, name):
    return dynamic_tanh(x, w[name], w[name + ".b"], float(np.asarray(w[name + ".alpha"]).reshape(())))


def forward(cfg: dict, w: Dict[str, np.ndarray], tokens: Sequence[int], layers_out: List[np.ndarray] = None):
    """Logits [T, vocab] of one whole sequence; layers_out, if given, receives the residual stream after every
    layer run."""
    eps = cfg["norm"]["eps"]
    x = np.asarray(w["embed"], F64)[np.asarray(tokens, np.int64)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', i)}."
        x = x + MIXERS[layer["type"]](_norm(x, w, p + "norm1"), _sub(w, p + "mix."), layer["mixer"], eps)
        if layer.get("mlp") is not None:
            x = x + dense_feed_forward(_norm(x, w, p + "norm2"), _sub(w, p + "mlp."))
        if layers_out is not None:
            layers_out.append(x.copy())
    return linear(_norm(x, w, "final.norm"), w["head"])
