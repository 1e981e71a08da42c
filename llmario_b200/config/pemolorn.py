"""Typed configuration of the Pemolorn decoder, read from the keys of its ``config.json``.

A Pemolorn model is a list of layers.  Every sublayer has a norm in front of it and one behind
it (``x += norm_b(sublayer(norm_a(x)))``); these norms have one number as their gain.  A layer's
mixer is one of

* ``parallel``: an attention (``left``) and a minGRU recurrence (``right``) on the same input,
  joined as half the sum of their RMS-normed outputs.  The attention has a short convolution on
  its projections, a norm over its whole query and key rows, a rotation of adjacent pairs on
  the first ``rot.dims`` channels of a head, a sliding window beside pooled blocks of
  ``mask.pool`` tokens, and a sink;
* ``attention``: a norm per head of queries and keys, no rotation, a sliding window beside the
  first ``mask.keep_first`` tokens, a sink; with ``kv_from: j`` the layer has no key and value
  projections and reads the cache of layer j.

The feed-forward is ``dense`` (``W_down relu(W_up h)^2``), ``moe`` (routed experts with a
clamped gated activation, scores over all router outputs, a correction of the choice, and
identity experts) or absent.  Every size and constant that can differ between two models of the
design is read here and nowhere else; tensor names follow ``l<i>.<part>``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .runidra import _deep
from .spec import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec
from .vunasun import _get

MIXERS = ("parallel", "attention")


@dataclass(frozen=True)
class PemolornLayer:
    type: str
    mixer: Tuple[Tuple[str, Any], ...]
    mlp: Optional[Tuple[Tuple[str, Any], ...]]

    def m(self) -> Dict[str, Any]:
        return _deep(dict(self.mixer))

    def f(self) -> Optional[Dict[str, Any]]:
        return None if self.mlp is None else _deep(dict(self.mlp))


def _freeze_deep(v):
    if isinstance(v, dict):
        return tuple(sorted((k, _freeze_deep(x)) for k, x in v.items()))
    return v


@dataclass(frozen=True)
class PemolornConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[PemolornLayer, ...]
    max_positions: int = 1 << 17      # the design has no limit of its own: the engine's default

    architecture = "Pemolorn"
    model_type = "pemolorn"

    # ---------------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "PemolornConfig":
        vocab = _get(raw, "vocab", int, "model")
        width = _get(raw, "width", int, "model")
        eps = _get(raw.get("norm"), "eps", float, "norm")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]"
            kind = e.get("type") if isinstance(e, dict) else None
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}: unsupported type {kind!r} "
                                  f"(known: {', '.join(MIXERS)})")
            m = e.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}: missing 'mixer'")
            if kind == "parallel":
                cls._check_attention(m.get("left"), where + ".mixer.left", pooled=True)
                _get(m.get("right"), "width", int, where + ".mixer.right")
            else:
                cls._check_attention(m, where + ".mixer", pooled=False)
                src = m.get("kv_from")
                if src is not None:
                    if not isinstance(src, int) or isinstance(src, bool) or not 0 <= src < i:
                        raise ConfigError(f"config.json: {where}: kv_from {src!r} must name an "
                                          "earlier layer")
                    other = entries[src]
                    if other.get("type") != "attention" or \
                            other["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"config.json: {where}: kv_from names layer {src}, "
                                          "which is no attention layer with keys and values of "
                                          "its own")
                    for key in ("kv_heads", "dim", "vdim"):
                        if other["mixer"].get(key) != m.get(key):
                            raise ConfigError(f"config.json: {where}: '{key}' differs from "
                                              f"layer {src}, whose keys and values it reads")
            mlp = e.get("mlp")
            if mlp is not None:
                cls._check_mlp(mlp, where + ".mlp")
            layers.append(PemolornLayer(kind, _freeze_deep(m),
                                        None if mlp is None else _freeze_deep(mlp)))
        max_pos = int(raw.get("max_positions") or cls.max_positions)
        return cls(vocab, width, eps, tuple(layers), max_pos)

    @staticmethod
    def _check_attention(m: Any, where: str, pooled: bool) -> None:
        heads = _get(m, "heads", int, where)
        kv = _get(m, "kv_heads", int, where)
        for key in ("dim", "vdim"):
            _get(m, key, int, where)
        _get(m, "scale", float, where)
        if heads % kv:
            raise ConfigError(f"config.json: {where}: {heads} heads on {kv} key heads")
        mask = m.get("mask")
        if pooled:
            _get(mask, "size", int, where + ".mask")
            _get(mask, "pool", int, where + ".mask")
            if m.get("conv") is not None:
                _get(m, "conv", int, where)
            rot = m.get("rot")
            if rot is not None:
                dims = _get(rot, "dims", int, where + ".rot")
                _get(rot, "base", float, where + ".rot")
                if dims % 2 or dims > m["dim"]:
                    raise ConfigError(f"config.json: {where}.rot: dims {dims} must be even and "
                                      f"at most dim {m['dim']}")
        elif mask is not None:
            _get(mask, "size", int, where + ".mask")
            keep = mask.get("keep_first") or 0
            if not isinstance(keep, int) or keep < 0:
                raise ConfigError(f"config.json: {where}.mask: keep_first {keep!r}")

    @staticmethod
    def _check_mlp(mlp: Dict[str, Any], where: str) -> None:
        kind = mlp.get("kind", "dense")
        if kind == "dense":
            _get(mlp, "ff", int, where)
        elif kind == "moe":
            _get(mlp.get("expert"), "ff", int, where + ".expert")
            if _get(mlp.get("expert"), "limit", float, where + ".expert") <= 0:
                raise ConfigError(f"config.json: {where}.expert: limit must be positive")
            r = mlp.get("router")
            n = _get(r, "experts", int, where + ".router")
            top = _get(r, "top", int, where + ".router")
            ident = r.get("identity") or 0
            if not isinstance(ident, int) or ident < 0:
                raise ConfigError(f"config.json: {where}.router: identity {ident!r}")
            if top > n + ident:
                raise ConfigError(f"config.json: {where}: top {top} of {n + ident} experts")
        else:
            raise ConfigError(f"config.json: {where}: unsupported mlp kind {kind!r} "
                              "(known: dense, moe)")

    def to_dict(self) -> Dict[str, Any]:
        """The ``config.json`` that reads back as this configuration."""
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab,
                               "width": self.width, "norm": {"eps": self.eps}, "layers": []}
        for layer in self.layers:
            out["layers"].append({"type": layer.type, "mixer": layer.m(), "mlp": layer.f()})
        if self.max_positions != type(self).max_positions:
            out["max_positions"] = self.max_positions
        return out

    # ---------------------------------------------------------------------------------------
    def to_spec(self) -> ModelSpec:
        c = self
        W = c.width

        def norm(name: str) -> PartSpec:
            return PartSpec("rms_norm_scalar", {"width": W, "eps": c.eps,
                                                "tensors": {"weight": (name, ())}})

        # what the layers that read another layer's keys and values need that layer to keep
        keep_for: Dict[int, Tuple[Optional[int], int]] = {}
        for i, layer in enumerate(c.layers):
            m = layer.m()
            if layer.type != "attention":
                continue
            mask = m.get("mask") or {}
            mine = (mask.get("size"), int(mask.get("keep_first") or 0))
            owner = m.get("kv_from", i) if m.get("kv_from") is not None else i
            size, keep = keep_for.get(owner, (0, 0))
            size = None if size is None or mine[0] is None else max(size, mine[0])
            keep_for[owner] = (size, max(keep, mine[1]))

        layers = []
        for i, layer in enumerate(c.layers):
            p = f"l{i}."
            x = p + "mix."
            m = layer.m()
            if layer.type == "parallel":
                left, right = m["left"], m["right"]
                H, G, d, dv = left["heads"], left["kv_heads"], left["dim"], left["vdim"]
                taps = int(left.get("conv") or 0)
                rot = left.get("rot")
                lx = x + "left."
                t = {"q": (lx + "q", (H * d, W)), "k": (lx + "k", (G * d, W)),
                     "v": (lx + "v", (G * dv, W)), "o": (lx + "o", (W, H * dv)),
                     "q_norm": (lx + "q.norm", (H * d,)), "k_norm": (lx + "k.norm", (G * d,)),
                     "sink": (lx + "sink", (H,))}
                if taps >= 1:      # (one tap: a weight per channel)
                    t.update(q_conv=(lx + "q.conv", (H * d, taps)),
                             k_conv=(lx + "k.conv", (G * d, taps)),
                             v_conv=(lx + "v.conv", (G * dv, taps)))
                attn = PartSpec("pooled_window_attention", {
                    "hidden_size": W, "num_heads": H, "num_kv_heads": G, "head_dim": d,
                    "value_dim": dv, "scale": float(left["scale"]), "eps": c.eps,
                    "window": int(left["mask"]["size"]), "pool": int(left["mask"]["pool"]),
                    "conv_taps": taps,
                    "position": None if rot is None else PartSpec("rope_normal", {
                        "rot_dim": int(rot["dims"]), "theta": float(rot["base"]),
                        "freq_scale": 1.0, "attn_factor": 1.0}),
                    "tensors": t})
                R = int(right["width"])
                rx = x + "right."
                gru = PartSpec("min_gru", {
                    "hidden_size": W, "width": R,
                    "tensors": {"z": (rx + "z", (R, W)), "z_bias": (rx + "z.b", (R,)),
                                "x": (rx + "x", (R, W)), "x_bias": (rx + "x.b", (R,)),
                                "g": (rx + "g", (R, W)), "o": (rx + "o", (W, R))}})
                mixer = PartSpec("parallel", {
                    "hidden_size": W, "eps": c.eps, "left": attn, "right": gru,
                    "tensors": {"left_out": (lx + "out", (W,)), "right_out": (rx + "out", (W,))}})
            else:
                H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
                mask = m.get("mask") or {}
                shared = m.get("kv_from") is not None
                t = {"q": (x + "q", (H * d, W)), "o": (x + "o", (W, H * dv)),
                     "sink": (x + "sink", (H,))}
                if not shared:
                    t.update(k=(x + "k", (G * d, W)), v=(x + "v", (G * dv, W)))

                def head_norm(name):
                    return PartSpec("rms_norm", {"width": d, "eps": c.eps,
                                                 "tensors": {"weight": (name, (d,))}})

                params: Dict[str, Any] = {
                    "hidden_size": W, "num_heads": H, "num_kv_heads": G, "head_dim": d,
                    "value_dim": dv, "scale": float(m["scale"]),
                    "window": mask.get("size"), "keep_first": int(mask.get("keep_first") or 0),
                    "shared_kv": shared, "position": None,
                    "q_norm": head_norm(x + "q.norm"),
                    "k_norm": None if shared else head_norm(x + "k.norm"), "tensors": t}
                if not shared:
                    size, keep = keep_for[i]
                    params["cache_window"], params["cache_keep_first"] = size, keep
                mixer = PartSpec("attention", params)
            f = p + "mlp."
            mlp = layer.f()
            if mlp is None:
                ffn = PartSpec("none", {})
            elif mlp.get("kind", "dense") == "dense":
                ff = int(mlp["ff"])
                ffn = PartSpec("dense", {
                    "hidden_size": W, "intermediate_size": ff, "activation": "relu_squared",
                    "tensors": {"up": (f + "up", (ff, W)), "down": (f + "down", (W, ff))}})
            else:
                r = mlp["router"]
                E, top, ident = int(r["experts"]), int(r["top"]), int(r.get("identity") or 0)
                ff = int(mlp["expert"]["ff"])
                t = {"router": (f + "router", (E + ident, W)),
                     "correction": (f + "correction", (E + ident,))}
                for e in range(E):
                    t[f"gate{e}"] = (f"{f}e{e}.gate", (ff, W))
                    t[f"up{e}"] = (f"{f}e{e}.up", (ff, W))
                    t[f"down{e}"] = (f"{f}e{e}.down", (W, ff))
                ffn = PartSpec("moe", {
                    "hidden_size": W, "intermediate_size": ff, "experts": E, "top": top,
                    "identity": ident, "scores": "softmax_all", "activation": "clamped_swish",
                    "limit": float(mlp["expert"]["limit"]), "tensors": t})
            block = PartSpec("output_norm_residual", {
                "mixer_input_norm": norm(p + "norm1"), "mixer_norm": norm(p + "norm1b"),
                "feed_forward_input_norm": norm(p + "norm2") if mlp is not None else None,
                "feed_forward_norm": norm(p + "norm2b") if mlp is not None else None})
            layers.append(LayerSpec(block, mixer, ffn, p))

        order = []
        for i, layer in enumerate(c.layers):
            src = layer.m().get("kv_from") if layer.type == "attention" else None
            order.append(LayerCall(i, src))      # (every layer runs once: entry i is layer i)
        spec = ModelSpec(
            architecture=c.architecture, vocab_size=c.vocab, hidden_size=W,
            max_positions=c.max_positions,
            embedding=PartSpec("token_embedding", {
                "vocab_size": c.vocab, "hidden_size": W,
                "tensors": {"table": ("embed", (c.vocab, W))}}),
            layers=tuple(layers), run_order=tuple(order), final_norm=norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": c.vocab, "hidden_size": W, "tied": False,
                                          "tensors": {"weight": ("head", (c.vocab, W))}}))
        spec.validate()
        return spec


def sized_like(width: int, ff: int, heads: int, kv_heads: int, head_dim: int, layers: int,
               vocab: int, window: int = 1024, pool: int = 64, keep_first: int = 4,
               experts: int = 8, top: int = 2) -> PemolornConfig:
    """A configuration for models with random weights at the sizes of a transformer: layers
    repeating (parallel + dense, attention + routed experts, attention + routed experts,
    attention on the keys and values of the layer before + dense).  The recurrence is as wide as
    the model; the routed experts are ``experts`` of width ff / top with ``top`` chosen beside
    two identity experts."""
    heads = min(heads, 16 * kv_heads)
    left = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "conv": 4,
            "scale": head_dim ** -0.5, "mask": {"size": window, "pool": pool},
            "rot": {"dims": head_dim // 2, "base": 1e6}}
    att = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim,
           "scale": head_dim ** -0.5, "mask": {"size": window, "keep_first": keep_first}}
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": ff // top, "limit": 7.0},
           "router": {"experts": experts, "top": top, "identity": 2}}
    out = []
    for i in range(layers):
        k = i % 4
        if k == 0:
            out.append({"type": "parallel", "mixer": {"left": left, "right": {"width": width}},
                        "mlp": dense})
        elif k in (1, 2):
            out.append({"type": "attention", "mixer": dict(att), "mlp": moe})
        else:
            out.append({"type": "attention", "mixer": dict(att, kv_from=i - 1), "mlp": dense})
    return PemolornConfig.from_dict({
        "architecture": "Pemolorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
        "layers": copy.deepcopy(out)})
