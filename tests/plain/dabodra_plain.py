"""Plain, slow restatement of the Dabodra decoder, used only as a test oracle.

Whole sequences, no cache, one function per mechanism, float64 throughout, no code shared with the product
package.  Notation: h is a sublayer's input [T, width]; p the positions 0..T-1; a weight matrix is [out, in] and
acts as h @ W.T.

  layer               x += N1(mixer(x));  x += N2(ff(x)):  the sublayers read x, the norm stands behind them
  N (one-plus norm)   y / sqrt(mean(y^2) + eps) * (1 + w)
  windowed attention  q = Wq h, k = Wk h, v = k (as projected);  q, k: RMS over the whole row with gains, then the
                      first n dimensions of every head rotated, pairs (2i, 2i + 1), angle p * base^(-2i/n);
                      s_ij = q_i . k_j * scale for 0 <= i - j < window;  a_ij = exp(s_ij) / (sum_j exp(s_ij) + exp(sink));
                      o_i = sum_j a_ij v_j;  Wo on the heads side by side
  gated delta rule    q, k, v = silu(causal_conv(W h));  q, k unit vectors per head (q also / sqrt(dim));
                      beta = sigmoid(Wb h);  g = exp(-exp(A_log) softplus(Wa h + dt_bias));  per head and token:
                      S = g S;  u = beta (v - S^T k);  S = S + k u^T;  o = S^T q;
                      o / rms(o) * w * silu(Wg h);  Wo
  routed experts      z = Wr h;  s = sigmoid(z);  c = s + correction;  groups of neighbouring experts scored by their two
                      largest c, the best `keep` groups stay;  the `top` largest c among them are chosen;  weights
                      s / (sum of the chosen s + 1e-20) * scale;  sum of weighted expert outputs + the shared expert;
                      expert: Wdown (silu(Wgate h) * Wup h)
"""
from __future__ import annotations

from typing import Dict, List

import numpy as np

F64 = np.float64


def linear(x, w):
    return np.asarray(x, F64) @ np.asarray(w, F64).T


def silu(z):
    z = np.asarray(z, F64)
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.asarray(z, F64)))


def softplus(z):
    z = np.asarray(z, F64)
    return np.where(z > 30, z, np.log1p(np.exp(np.minimum(z, 30))))


def rms_norm(x, gain, eps):
    x = np.asarray(x, F64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + F64(eps)) * np.asarray(gain, F64)


def one_plus_norm(x, w, eps):
    return rms_norm(x, 1.0 + np.asarray(w, F64), eps)


def rotate_pairs(x, pos, base, n):
    """x [T, heads, m], m >= n: in every head the pairs (2i, 2i + 1), i < n/2, turned by the angle p * base^(-2i/n)."""
    x = np.array(x, F64)
    i = np.arange(n // 2, dtype=F64)
    f = F64(base) ** (-2.0 * i / F64(n))
    a = np.asarray(pos, F64)[:, None] * f[None, :]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    u, v = x[..., 0:n:2].copy(), x[..., 1:n:2].copy()
    x[..., 0:n:2] = u * c - v * s
    x[..., 1:n:2] = v * c + u * s
    return x


def windowed_sink_attention(h, w: Dict[str, np.ndarray], m: dict, eps: float):
    """m: heads, kv_heads, dim, vdim, mask.size, rot.base, rot.dims, scale.  w: q, k, q.norm, k.norm, sink, o."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    pos = np.arange(T)
    q_raw, k_raw = linear(h, w["q"]), linear(h, w["k"])
    v = k_raw.reshape(T, G, D)
    q = rms_norm(q_raw, w["q.norm"], eps).reshape(T, H, D)
    k = rms_norm(k_raw, w["k.norm"], eps).reshape(T, G, D)
    if m.get("rot") and m["rot"]["dims"]:
        q = rotate_pairs(q, pos, m["rot"]["base"], m["rot"]["dims"])
        k = rotate_pairs(k, pos, m["rot"]["base"], m["rot"]["dims"])
    window = m["mask"]["size"] if m.get("mask") else T
    out = np.zeros((T, H, D), F64)
    for head in range(H):
        kv = head // (H // G)
        s = (q[:, head] @ k[:, kv].T) * F64(m["scale"])
        i, j = pos[:, None], pos[None, :]
        vis = (i - j >= 0) & (i - j < window)
        s = np.where(vis, s, -np.inf)
        sink = F64(w["sink"][head])
        mx = np.maximum(s.max(axis=-1, keepdims=True), sink)
        e = np.exp(s - mx)
        a = e / (e.sum(axis=-1, keepdims=True) + np.exp(sink - mx))
        out[:, head] = a @ v[:, kv]
    return linear(out.reshape(T, H * D), w["o"])


def causal_conv(x, taps):
    """x [T, C], taps [C, n]: y_t = sum_i taps[:, n - 1 - i] x_{t - i}, zeros before the start."""
    x, taps = np.asarray(x, F64), np.asarray(taps, F64)
    n = taps.shape[1]
    y = np.zeros_like(x)
    for i in range(min(n, x.shape[0])):
        y[i:] += x[:x.shape[0] - i] * taps[:, n - 1 - i][None, :]
    return y


def unit(x):
    return x / np.sqrt(np.sum(x * x, axis=-1, keepdims=True) + F64(1e-6))


def gated_delta(h, w: Dict[str, np.ndarray], m: dict, eps: float):
    """m: heads, kv_heads, dim, vdim, conv.  w: q, k, v, q.conv, k.conv, v.conv, b, a, A_log, dt_bias, g, norm, o."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(linear(h, w["q"]), w["q.conv"])).reshape(T, G, D)
    k = silu(causal_conv(linear(h, w["k"]), w["k.conv"])).reshape(T, G, D)
    v = silu(causal_conv(linear(h, w["v"]), w["v.conv"])).reshape(T, H, V)
    q = unit(q) * F64(D) ** -0.5
    k = unit(k)
    beta = sigmoid(linear(h, w["b"]))                                             # [T, H]
    decay = np.exp(-np.exp(np.asarray(w["A_log"], F64))[None, :] *
                   softplus(linear(h, w["a"]) + np.asarray(w["dt_bias"], F64)[None, :]))
    gate = silu(linear(h, w["g"])).reshape(T, H, V)
    out = np.zeros((T, H, V), F64)
    for head in range(H):
        kv = head // (H // G)
        S = np.zeros((D, V), F64)
        for t in range(T):
            S = decay[t, head] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, kv])
            S = S + np.outer(k[t, kv], u)
            out[t, head] = S.T @ q[t, kv]
    out = rms_norm(out, np.asarray(w["norm"], F64)[None, None, :], eps) * gate
    return linear(out.reshape(T, H * V), w["o"])


def expert(h, w: Dict[str, np.ndarray], prefix: str):
    return linear(silu(linear(h, w[prefix + "gate"])) * linear(h, w[prefix + "up"]), w[prefix + "down"])


def route(h, w_router, correction, r: dict, margins: List[float] = None):
    """(chosen experts [T, top], their weights [T, top]); r: experts, top, scale, groups.count, groups.keep.
    margins (a list) receives, per token, by how much the last choice made (of a group, of an expert) led the best
    one not made: a test keeps away from inputs on which rounding could make another choice."""
    E, top = r["experts"], r["top"]
    n_groups, keep = r["groups"]["count"], r["groups"]["keep"]
    s = sigmoid(linear(h, w_router))
    c = s + np.asarray(correction, F64)[None, :]
    per = E // n_groups
    T = h.shape[0]
    chosen = np.zeros((T, top), np.int64)
    weights = np.zeros((T, top), F64)
    for t in range(T):
        grouped = c[t].reshape(n_groups, per)
        score = np.sort(grouped, axis=-1)[:, ::-1][:, :2].sum(axis=-1)
        best = np.argsort(-score, kind="stable")[:keep]
        allowed = np.full(E, -np.inf)
        for gi in best:
            allowed[gi * per:(gi + 1) * per] = c[t, gi * per:(gi + 1) * per]
        order = np.argsort(-allowed, kind="stable")
        idx = order[:top]
        if margins is not None:
            ranked = np.sort(score)[::-1]
            if keep < n_groups:
                margins.append(float(ranked[keep - 1] - ranked[keep]))
            if top < len(order) and np.isfinite(allowed[order[top]]):
                margins.append(float(allowed[order[top - 1]] - allowed[order[top]]))
        chosen[t] = idx
        weights[t] = s[t, idx] / (s[t, idx].sum() + 1e-20) * F64(r["scale"])
    return chosen, weights


def routed_experts(h, w: Dict[str, np.ndarray], mlp: dict, margins: List[float] = None):
    """w: router, correction, e<i>.gate/up/down, shared.gate/up/down."""
    chosen, weights = route(h, w["router"], w["correction"], mlp["router"], margins)
    out = expert(h, w, "shared.") if mlp.get("shared") else np.zeros_like(np.asarray(h, F64))
    per_expert = [expert(h, w, f"e{e}.") for e in range(mlp["router"]["experts"])]
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t], weights[t]):
            out[t] += wt * per_expert[e][t]
    return out


def sub(tensors: Dict[str, np.ndarray], prefix: str) -> Dict[str, np.ndarray]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: Dict[str, np.ndarray], tokens, after_layers: List[np.ndarray] = None,
            margins: List[float] = None):
    """Logits [T, vocab] of one whole sequence; after_layers (a list) receives the residual stream after every layer,
    margins (a list) the routers' margins (see route)."""
    eps = config["norm"]["eps"]
    x = one_plus_norm(np.asarray(tensors["embed"], F64)[np.asarray(tokens)], tensors["embed.norm"], eps)
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        mix = sub(tensors, p + "mix.")
        if layer["type"] == "attention":
            y = windowed_sink_attention(x, mix, layer["mixer"], eps)
        elif layer["type"] == "delta":
            y = gated_delta(x, mix, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + one_plus_norm(y, tensors[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            y = routed_experts(x, sub(tensors, p + "mlp."), layer["mlp"], margins)
            x = x + one_plus_norm(y, tensors[p + "norm2"], eps)
        if after_layers is not None:
            after_layers.append(x.copy())
    return linear(one_plus_norm(x, tensors["final.norm"], eps), tensors["head"])
