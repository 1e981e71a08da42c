"""A plain, slow statement of the Pavatar decoder in float64 NumPy: one function per mechanism,
whole sequences from position 0, the recurrence token by token, attention query by query.  It
shares nothing with the package: it reads the raw ``config.json`` dictionary and a dictionary of
arrays by tensor name.

Notation: ``h`` [T, width] is a sublayer's input, ``W`` [out, in] is applied as ``h @ W.T``;
a layer is ``x <- x + mixer(n(x)) + experts(n(x))`` with one RMS norm ``n`` for both sublayers.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

import numpy as np

F = np.float64
UNIT_FLOOR = 1e-6        # inside the root of the unit vectors of the delta rule
WEIGHT_FLOOR = 1e-20     # beside the sum of the chosen experts' scores


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.maximum(z, 0.0) + np.log1p(np.exp(-np.abs(z)))


def rms_unit(x, eps):
    """x over its root mean square along the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def short_conv(u, w):
    """Causal convolution over time per channel: u [T, C], w [C, taps]; the last column of w
    meets the current token, zeros stand before the start."""
    T, C = u.shape
    taps = w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C), F), u])
    y = np.zeros((T, C), F)
    for j in range(taps):
        y += padded[j:j + T] * w[:, j]
    return y


def rotate_halves(x, pos, dims: int, base: float):
    """Turn the pairs (i, i + dims/2), i < dims/2, of the last axis of x [T, heads, dim] by
    pos * base^(-2i/dims); channels from ``dims`` on pass."""
    out = x.copy()
    half = dims // 2
    i = np.arange(half)
    ang = pos[:, None].astype(F) * base ** (-2.0 * i / dims)
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def query_temperature(pos, coef: float, every: int):
    """The factor on the queries of position p: 1 + coef ln(floor((p + 1) / every) + 1)."""
    return 1.0 + coef * np.log(np.floor((pos.astype(F) + 1.0) / every) + 1.0)


def causal_attend(q, k, v, scale):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head a reads key head a // (H / G); row i
    sees the keys j <= i through a softmax of scale * (q . k)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]), F)
    for a in range(H):
        g = a // (H // G)
        for i in range(T):
            s = (k[:i + 1, g] @ q[i, a]) * scale
            e = np.exp(s - s.max())
            out[i, a] = (e / e.sum()) @ v[:i + 1, g]
    return out


def biased_attention(h, t: Callable[[str], np.ndarray], m: dict, pos, first_values,
                     round_cache: Callable = lambda a: a):
    """The mixer ``attention``: projections with biases, no rotation, queries scaled by their
    position's temperature, values optionally blended with ``first_values`` (those of the first
    blending layer, same tokens) before they are kept, one sigmoid gate per head.  Returns the
    output and the values as kept."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ t("q").T + t("q.b")).reshape(T, H, d)
    k = (h @ t("k").T + t("k.b")).reshape(T, G, d)
    v = (h @ t("v").T + t("v.b")).reshape(T, G, dv)
    qt = m.get("q_temp")
    if qt:
        q = q * query_temperature(pos, float(qt["coef"]), int(qt["every"]))[:, None, None]
    if m.get("v_mix") and first_values is not None:
        lam = float(np.asarray(t("vmix")).reshape(()))
        v = (1.0 - lam) * v + lam * first_values
    o = causal_attend(q, round_cache(k), round_cache(v), float(m["scale"]))
    o = o * sigmoid(h @ t("g").T)[:, :, None]
    return o.reshape(T, H * dv) @ t("o").T, v


def rotary_attention(h, t: Callable[[str], np.ndarray], m: dict, pos, eps,
                     round_cache: Callable = lambda a: a):
    """The attention half of the mixer ``parallel``: a norm per head on queries and keys (one
    gain vector for all heads), a rotation of half-split pairs, a sigmoid gate per channel."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm((h @ t("q").T).reshape(T, H, d), t("q.norm"), eps)
    k = rms_norm((h @ t("k").T).reshape(T, G, d), t("k.norm"), eps)
    v = (h @ t("v").T).reshape(T, G, dv)
    rot = m.get("rot")
    if rot:
        q = rotate_halves(q, pos, int(rot["dims"]), float(rot["base"]))
        k = rotate_halves(k, pos, int(rot["dims"]), float(rot["base"]))
    o = causal_attend(q, round_cache(k), round_cache(v), float(m["scale"]))
    o = o.reshape(T, H * dv) * sigmoid(h @ t("g").T)
    return o @ t("o").T


def delta_rule(q, k, v, beta, decay):
    """Per head and token, with S [dim, vdim] starting at zero:
    ``S <- diag(decay) S``; ``u = beta (v - S^T k)``; ``S <- S + k u^T``; ``o = S^T q``.
    q, k [T, H, d] (already per value head), v [T, H, dv], beta [T, H], decay [T, H, d]."""
    T, H, d = q.shape
    dv = v.shape[2]
    out = np.zeros((T, H, dv), F)
    for a in range(H):
        S = np.zeros((d, dv), F)
        for i in range(T):
            S = decay[i, a][:, None] * S
            u = beta[i, a] * (v[i, a] - S.T @ k[i, a])
            S = S + np.outer(k[i, a], u)
            out[i, a] = S.T @ q[i, a]
    return out


def unit_heads(x):
    return x / np.sqrt(np.sum(x * x, axis=-1, keepdims=True) + UNIT_FLOOR)


def delta_mixer(h, t: Callable[[str], np.ndarray], m: dict, eps, low_rank: bool):
    """The gated delta rule as a mixer.  ``low_rank`` False (mixer ``delta``): one decay per
    head from ``a``, output gate ``silu(W_g h)``.  True (the right half of ``parallel``): a
    decay per head and key channel from ``a2 a1``, output gate ``sigmoid(W_g2 W_g1 h)``."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ t("q").T, t("q.conv"))).reshape(T, G, d)
    k = silu(short_conv(h @ t("k").T, t("k.conv"))).reshape(T, G, d)
    v = silu(short_conv(h @ t("v").T, t("v.conv"))).reshape(T, H, dv)
    q = unit_heads(q) * d ** -0.5
    k = unit_heads(k)
    share = H // G
    q, k = np.repeat(q, share, axis=1), np.repeat(k, share, axis=1)
    beta = sigmoid(h @ t("b").T)
    rate = np.exp(t("A_log"))
    if low_rank:
        z = ((h @ t("a1").T) @ t("a2").T + t("dt_bias")).reshape(T, H, d)
        decay = np.exp(-rate[None, :, None] * softplus(z))
        gate = sigmoid((h @ t("g1").T) @ t("g2").T)
    else:
        z = h @ t("a").T + t("dt_bias")
        decay = np.repeat(np.exp(-rate[None, :] * softplus(z))[:, :, None], d, axis=2)
        gate = silu(h @ t("g").T)
    o = delta_rule(q, k, v, beta, decay)
    o = rms_unit(o, eps) * t("norm")
    return (o.reshape(T, H * dv) * gate) @ t("o").T


def parallel_mixer(h, t: Callable[[str], np.ndarray], m: dict, pos, eps,
                   round_cache: Callable = lambda a: a):
    """Half the sum of both halves' outputs, each RMS-normed over the width first."""
    left = rotary_attention(h, lambda n: t("left." + n), m["left"], pos, eps, round_cache)
    right = delta_mixer(h, lambda n: t("right." + n), m["right"], eps, low_rank=True)
    return 0.5 * (rms_norm(left, t("left.out"), eps) + rms_norm(right, t("right.out"), eps))


def route(z, correction, top: int, scale: float) -> Tuple[np.ndarray, np.ndarray]:
    """z [T, E] router outputs.  Scores are the softmax over all E; the ``top`` largest of
    score + correction are chosen (lowest index among equals); a chosen expert's weight is its
    score over the sum of the chosen scores, times ``scale``."""
    s = np.exp(z - z.max(axis=-1, keepdims=True))
    s /= s.sum(axis=-1, keepdims=True)
    ids = np.argsort(-(s + correction), axis=-1, kind="stable")[:, :top]
    w = np.take_along_axis(s, ids, axis=-1)
    return ids, w / (w.sum(axis=-1, keepdims=True) + WEIGHT_FLOOR) * scale


def routed_experts(h, t: Callable[[str], np.ndarray], f: dict):
    """Experts ``W_down relu(W_up h)^2`` summed with the router's weights."""
    r = f["router"]
    ids, w = route(h @ t("router").T, t("correction"), int(r["top"]), float(r["scale"]))
    y = np.zeros((h.shape[0], t("e0.down").shape[0]), F)
    for i in range(h.shape[0]):
        for e, we in zip(ids[i], w[i]):
            a = np.maximum(t(f"e{e}.up") @ h[i], 0.0) ** 2
            y[i] += we * (t(f"e{e}.down") @ a)
    return y


def close_calls(h, t, f: dict, margin: float) -> np.ndarray:
    """Rows whose router would choose otherwise after a move of the router outputs by about
    ``margin``: the last chosen expert and the best one not chosen lie closer in their choice
    scores than ``margin`` times the larger of their scores (a move dz of an output moves its
    score by about score * dz)."""
    r = f["router"]
    z = h @ t("router").T
    s = np.exp(z - z.max(axis=-1, keepdims=True))
    s /= s.sum(axis=-1, keepdims=True)
    top = int(r["top"])
    if top >= s.shape[1]:
        return np.zeros(h.shape[0], bool)
    c = s + t("correction")
    order = np.argsort(-c, axis=-1, kind="stable")
    a, b = order[:, top - 1:top], order[:, top:top + 1]
    gap = np.take_along_axis(c, a, -1) - np.take_along_axis(c, b, -1)
    size = np.maximum(np.take_along_axis(s, a, -1), np.take_along_axis(s, b, -1))
    return (gap < margin * size)[:, 0]


def forward(cfg: dict, tensors: Dict[str, np.ndarray], tokens, round_cache=lambda a: a,
            round_act=lambda a: a, want_layers: bool = False, close_margin: float = 0.0):
    """Logits [T, vocab] of a whole sequence.  ``round_act`` is applied to the normed input of
    a layer's sublayers (what a 16-bit engine hands to its products), ``round_cache`` to keys
    and values as attention reads them.  ``want_layers``: also the residual stream behind every
    layer [layers, T, width].  ``close_margin`` > 0: also the rows at which some router makes a
    close call."""
    W = {n: np.asarray(a, F) for n, a in tensors.items()}
    tokens = np.asarray(tokens)
    T = len(tokens)
    pos = np.arange(T)
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][tokens] * float(cfg["embedding"]["scale"])
    first_values = None
    seen: List[np.ndarray] = []
    close = np.zeros(T, bool)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = round_act(rms_norm(x, W[p + "norm1"], eps))
        t = lambda n, p=p: W[p + "mix." + n]
        m = layer["mixer"]
        if layer["type"] == "attention":
            y, kept = biased_attention(h, t, m, pos, first_values, round_cache)
            if m.get("v_mix") and first_values is None:
                first_values = kept
        elif layer["type"] == "parallel":
            y = parallel_mixer(h, t, m, pos, eps, round_cache)
        elif layer["type"] == "delta":
            y = delta_mixer(h, t, m, eps, low_rank=False)
        else:
            raise ValueError(layer["type"])
        f = layer.get("mlp")
        if f is not None:
            tf = lambda n, p=p: W[p + "mlp." + n]
            y = y + routed_experts(h, tf, f)
            if close_margin:
                close |= close_calls(h, tf, f, close_margin)
        x = x + y
        seen.append(x.copy())
    z = rms_norm(x, W["final.norm"], eps) @ W["embed"].T
    cap = float(cfg.get("logit_softcap") or 0.0)
    if cap:
        z = cap * np.tanh(z / cap)
    out = (z,)
    if want_layers:
        out += (np.stack(seen),)
    if close_margin:
        out += (close,)
    return out[0] if len(out) == 1 else out
