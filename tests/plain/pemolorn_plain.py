"""A plain, slow statement of the Pemolorn decoder in float64 NumPy: one function per mechanism,
whole sequences from position 0, the recurrence token by token, attention query by query.  It
shares nothing with the package: it reads the raw ``config.json`` dictionary and a dictionary of
arrays by tensor name.

Notation: ``h`` [T, width] is a sublayer's input, ``W`` [out, in] is applied as ``h @ W.T``.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import numpy as np

F = np.float64


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rms_unit(x, eps):
    """x over its root mean square along the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose gain is one number for all coordinates."""
    return rms_unit(x, eps) * float(np.asarray(g).reshape(()))


def short_conv(u, w):
    """Causal convolution over time per channel: u [T, C], w [C, taps];
    y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C), F), u])
    y = np.zeros((T, C), F)
    for j in range(taps):
        y += padded[j:j + T] * w[:, j]
    return y


def rotate_adjacent(x, pos, dims: int, base: float):
    """Turn the pairs (2i, 2i+1), i < dims/2, of the last axis of x [T, heads, dim] by
    pos * base^(-2i/dims); the other channels pass."""
    out = x.copy()
    i = np.arange(dims // 2)
    ang = pos[:, None].astype(F) * base ** (-2.0 * i / dims)
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def sink_softmax_sum(scores, values, sink: Optional[float]):
    """Softmax over ``scores`` [n] whose denominator also holds exp(sink); the weighted sum of
    ``values`` [n, d]."""
    top = scores.max() if sink is None else max(scores.max(), sink)
    e = np.exp(scores - top)
    den = e.sum() + (0.0 if sink is None else np.exp(sink - top))
    return (e / den) @ values


def attend(q, k, v, scale, sinks, visible: Callable[[int], np.ndarray], pooled=None,
           round_cache: Callable = lambda a: a):
    """q [T, H, d], k [T, G, d], v [T, G, dv].  ``visible(i)`` gives the indices of the token
    keys position i sees.  ``pooled = (P, size)``: beside them one key and value per block of P
    positions that ends at or before i - size, the means of the block's keys and values as the
    cache holds them (``round_cache``)."""
    T, H, _ = q.shape
    G = k.shape[1]
    k, v = round_cache(k), round_cache(v)
    out = np.zeros((T, H, v.shape[2]), F)
    if pooled is not None:
        P, size = pooled
        nb = T // P
        kp = round_cache(k[:nb * P].reshape(nb, P, G, -1).mean(axis=1)) if nb else None
        vp = round_cache(v[:nb * P].reshape(nb, P, G, -1).mean(axis=1)) if nb else None
    for i in range(T):
        js = visible(i)
        for hq in range(H):
            g = hq // (H // G)
            keys, vals = k[js, g], v[js, g]
            if pooled is not None:
                seen = max(0, (i - size + 1) // P)        # blocks with b P + P - 1 <= i - size
                if seen:
                    keys = np.concatenate([kp[:seen, g], keys])
                    vals = np.concatenate([vp[:seen, g], vals])
            out[i, hq] = sink_softmax_sum((keys @ q[i, hq]) * scale, vals,
                                          None if sinks is None else float(sinks[hq]))
    return out


def window_visible(size: int):
    return lambda i: np.arange(max(0, i - size + 1), i + 1)


def window_kept_visible(size: int, keep: int):
    def f(i):
        j = np.arange(i + 1)
        return j[(i - j < size) | (j < keep)]
    return f


def pooled_window_attention(h, t, p, m, eps, round_cache=lambda a: a):
    """The left half of a parallel mixer: projections, a short convolution on each, RMS norm of
    the whole query and key rows, rotation of adjacent pairs, a sliding window beside pooled
    blocks, a sink in the softmax."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = (h @ t[p + r].T for r in "qkv")
    if m.get("conv"):
        q, k, v = (short_conv(x, t[p + r + ".conv"]) for x, r in ((q, "q"), (k, "k"), (v, "v")))
    q = rms_unit(q, eps) * t[p + "q.norm"]
    k = rms_unit(k, eps) * t[p + "k.norm"]
    q, k, v = q.reshape(T, H, d), k.reshape(T, G, d), v.reshape(T, G, dv)
    pos = np.arange(T)
    rot = m.get("rot")
    if rot is not None:
        q = rotate_adjacent(q, pos, int(rot["dims"]), float(rot["base"]))
        k = rotate_adjacent(k, pos, int(rot["dims"]), float(rot["base"]))
    size, P = int(m["mask"]["size"]), int(m["mask"]["pool"])
    o = attend(q, k, v, float(m["scale"]), t.get(p + "sink"), window_visible(size), (P, size),
               round_cache)
    return o.reshape(T, H * dv) @ t[p + "o"].T


def min_gru(h, t, p, m):
    """The right half: S_t = (1 - z_t) S_(t-1) + z_t c_t with z = sigmoid(W_z h + b_z) and the
    candidate c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0), u = W_x h + b_x; out = W_o (S silu(W_g h))."""
    T = h.shape[0]
    z = sigmoid(h @ t[p + "z"].T + t[p + "z.b"])
    u = h @ t[p + "x"].T + t[p + "x.b"]
    cand = np.where(u >= 0, u + 0.5, sigmoid(u))
    S = np.zeros(z.shape[1], F)
    out = np.zeros_like(z)
    for i in range(T):
        S = (1.0 - z[i]) * S + z[i] * cand[i]
        out[i] = S
    return (out * silu(h @ t[p + "g"].T)) @ t[p + "o"].T


def parallel_mixer(h, t, p, m, eps, round_cache=lambda a: a):
    left = pooled_window_attention(h, t, p + "left.", m["left"], eps, round_cache)
    right = min_gru(h, t, p + "right.", m["right"])
    return 0.5 * (rms_unit(left, eps) * t[p + "left.out"] + rms_unit(right, eps) * t[p + "right.out"])


def kept_window_attention(h, t, p, m, eps, shared_kv=None, round_cache=lambda a: a):
    """Attention with a norm per head of queries and keys, no rotation, a sliding window beside
    the first ``keep_first`` tokens, a sink.  Returns (output, (k, v)) so that a later layer can
    use this one's keys and values (``shared_kv``)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_unit((h @ t[p + "q"].T).reshape(T, H, d), eps) * t[p + "q.norm"]
    if shared_kv is None:
        k = rms_unit((h @ t[p + "k"].T).reshape(T, G, d), eps) * t[p + "k.norm"]
        v = (h @ t[p + "v"].T).reshape(T, G, dv)
    else:
        k, v = shared_kv
    mask = m.get("mask") or {}
    size, keep = int(mask.get("size") or T + 1), int(mask.get("keep_first") or 0)
    o = attend(q, k, v, float(m["scale"]), t.get(p + "sink"), window_kept_visible(size, keep),
               None, round_cache)
    return o.reshape(T, H * dv) @ t[p + "o"].T, (k, v)


def dense_ff(h, t, p):
    return np.maximum(h @ t[p + "up"].T, 0.0) ** 2 @ t[p + "down"].T


def route(h, t, p, mlp, margins: Optional[list] = None):
    """(chosen [T, top], weights [T, top]): softmax over all router outputs, the choice by the
    score plus a correction, the weight the score itself.  ``margins`` collects, per token, how
    far the last chosen choice score lies above the best one not chosen, in units of the larger
    of the two softmax scores (a move of a logit by x moves its score by about x times itself)."""
    z = h @ t[p + "router"].T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z) / np.exp(z).sum(axis=-1, keepdims=True)
    choice = s + t[p + "correction"]
    top = int(mlp["router"]["top"])
    order = np.argsort(-choice, axis=-1, kind="stable")
    chosen = order[:, :top]
    if margins is not None and top < s.shape[1]:
        a, b = order[:, top - 1:top], order[:, top:top + 1]
        gap = np.take_along_axis(choice, a, -1) - np.take_along_axis(choice, b, -1)
        unit = np.maximum(np.take_along_axis(s, a, -1), np.take_along_axis(s, b, -1))
        margins.append((gap / unit)[:, 0])
    return chosen, np.take_along_axis(s, chosen, axis=-1)


def expert(h, t, p, limit):
    g = np.minimum(h @ t[p + "gate"].T, limit)
    u = np.clip(h @ t[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ t[p + "down"].T


def moe_ff(h, t, p, mlp, margins: Optional[list] = None):
    E = int(mlp["router"]["experts"])
    limit = float(mlp["expert"]["limit"])
    chosen, w = route(h, t, p, mlp, margins)
    out = np.zeros_like(h)
    for i in range(h.shape[0]):
        for e, we in zip(chosen[i], w[i]):
            y = h[i:i + 1] if e >= E else expert(h[i:i + 1], t, f"{p}e{e}.", limit)
            out[i] += we * y[0]
    return out


# --------------------------------------------------------------------------------------------
def forward(cfg: dict, tensors: Dict[str, np.ndarray], tokens, layers_out: Optional[List] = None,
            round_cache: Callable = lambda a: a, margins: Optional[list] = None):
    """Logits [T, vocab] of one sequence from position 0.  ``layers_out`` collects the residual
    stream behind every layer, ``margins`` the routers' margins per token (see :func:`route`)."""
    t = {n: np.asarray(a, F) for n, a in tensors.items()}
    eps = float(cfg["norm"]["eps"])
    x = t["embed"][np.asarray(tokens)]
    kv_of = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = scalar_norm(x, t[p + "norm1"], eps)
        if layer["type"] == "parallel":
            y = parallel_mixer(h, t, p + "mix.", m, eps, round_cache)
        else:
            src = m.get("kv_from")
            y, kv_of[i] = kept_window_attention(h, t, p + "mix.", m, eps,
                                                None if src is None else kv_of[src], round_cache)
        x = x + scalar_norm(y, t[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = scalar_norm(x, t[p + "norm2"], eps)
            y = dense_ff(h, t, p + "mlp.") if mlp.get("kind", "dense") == "dense" \
                else moe_ff(h, t, p + "mlp.", mlp, margins)
            x = x + scalar_norm(y, t[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return scalar_norm(x, t["final.norm"], eps) @ t["head"].T
