"""Typed configuration of the Pavatar decoder, read from the keys of its ``config.json``.

A Pavatar model is a list of layers.  A layer has one RMS norm whose output both of its
sublayers read: ``h = norm1(x); x += mixer(h) + experts(h)``.  The embedding is multiplied by
``embedding.scale``; the logits come from the embedding table itself (without that scale) and
are soft-capped.  A layer's mixer is one of

* ``attention``: grouped-query attention with biases on q, k and v, no rotation, the queries
  scaled by ``1 + coef ln(floor((p + 1) / every) + 1)`` at position p (``q_temp``), a sigmoid gate
  per head, and (``v_mix``) values that every such layer but the first blends with the first
  one's values of the same tokens before it stores them;
* ``delta``: the gated delta rule with one decay per head, a short convolution and silu on q, k
  and v, unit q and k, an output norm per head and a ``silu`` gate;
* ``parallel``: an attention (``left``: a norm per head of q and k, a rotation of half-split
  pairs on the first ``rot.dims`` channels, a sigmoid gate per channel) beside a gated delta rule
  (``right``: a decay per head and key channel and a sigmoid gate, both through low-rank
  factors whose rank only the stored tensors give), joined as half the sum of their RMS-normed
  outputs.

The feed-forward is a mixture of experts ``W_down relu(W_up h)^2`` (scores over all router
outputs, the choice by score plus a stored correction, the chosen scores renormalised and
multiplied by ``router.scale``) or absent.  Every size and constant that can differ between two
models of the design is read here and nowhere else; tensor names follow ``l<i>.<part>``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .pemolorn import _freeze_deep
from .runidra import _deep
from .spec import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec
from .vunasun import _get

MIXERS = ("attention", "parallel", "delta")
VALUE_GROUP = "v_mix"      # the one group of layers whose values are blended


@dataclass(frozen=True)
class PavatarLayer:
    type: str
    mixer: Tuple[Tuple[str, Any], ...]
    mlp: Optional[Tuple[Tuple[str, Any], ...]]

    def m(self) -> Dict[str, Any]:
        return _deep(dict(self.mixer))

    def f(self) -> Optional[Dict[str, Any]]:
        return None if self.mlp is None else _deep(dict(self.mlp))


@dataclass(frozen=True)
class PavatarConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    logit_softcap: float           # 0: the logits are not capped
    layers: Tuple[PavatarLayer, ...]
    max_positions: int = 1 << 17      # the design has no limit of its own: the engine's default

    architecture = "Pavatar"
    model_type = "pavatar"

    # ---------------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "PavatarConfig":
        vocab = _get(raw, "vocab", int, "model")
        width = _get(raw, "width", int, "model")
        eps = _get(raw.get("norm"), "eps", float, "norm")
        scale = 1.0 if raw.get("embedding") is None else \
            _get(raw["embedding"], "scale", float, "embedding")
        cap = float(raw.get("logit_softcap") or 0.0)
        if cap < 0:
            raise ConfigError(f"config.json: logit_softcap {cap} must not be negative")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        blended = None       # (kv_heads, vdim) of the layers whose values are blended
        for i, e in enumerate(entries):
            where = f"layers[{i}]"
            kind = e.get("type") if isinstance(e, dict) else None
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}: unsupported type {kind!r} "
                                  f"(known: {', '.join(MIXERS)})")
            m = e.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}: missing 'mixer'")
            if kind == "attention":
                cls._check_attention(m, where + ".mixer")
                qt = m.get("q_temp")
                if qt is not None:
                    _get(qt, "coef", float, where + ".mixer.q_temp")
                    _get(qt, "every", int, where + ".mixer.q_temp")
                if m.get("v_mix"):
                    mine = (m["kv_heads"], m["vdim"])
                    if blended is not None and blended != mine:
                        raise ConfigError(f"config.json: {where}: v_mix blends values of "
                                          f"{blended[0]} heads of {blended[1]} channels with "
                                          f"values of {mine[0]} heads of {mine[1]}")
                    blended = mine
            elif kind == "delta":
                cls._check_delta(m, where + ".mixer")
            else:
                cls._check_attention(m.get("left"), where + ".mixer.left")
                rot = m["left"].get("rot")
                if rot is not None:
                    dims = _get(rot, "dims", int, where + ".mixer.left.rot")
                    _get(rot, "base", float, where + ".mixer.left.rot")
                    if dims % 2 or dims > m["left"]["dim"]:
                        raise ConfigError(f"config.json: {where}.mixer.left.rot: dims {dims} "
                                          f"must be even and at most dim {m['left']['dim']}")
                cls._check_delta(m.get("right"), where + ".mixer.right")
            mlp = e.get("mlp")
            if mlp is not None:
                cls._check_mlp(mlp, where + ".mlp")
            layers.append(PavatarLayer(kind, _freeze_deep(m),
                                       None if mlp is None else _freeze_deep(mlp)))
        max_pos = int(raw.get("max_positions") or cls.max_positions)
        return cls(vocab, width, eps, scale, cap, tuple(layers), max_pos)

    @staticmethod
    def _check_attention(m: Any, where: str) -> None:
        heads = _get(m, "heads", int, where)
        kv = _get(m, "kv_heads", int, where)
        for key in ("dim", "vdim"):
            _get(m, key, int, where)
        _get(m, "scale", float, where)
        if heads % kv:
            raise ConfigError(f"config.json: {where}: {heads} heads on {kv} key heads")

    @staticmethod
    def _check_delta(m: Any, where: str) -> None:
        heads = _get(m, "heads", int, where)
        kv = _get(m, "kv_heads", int, where)
        for key in ("dim", "vdim", "conv"):
            _get(m, key, int, where)
        if heads % kv:
            raise ConfigError(f"config.json: {where}: {heads} heads on {kv} key heads")
        if m.get("rank") is not None:
            _get(m, "rank", int, where)

    @staticmethod
    def _check_mlp(mlp: Dict[str, Any], where: str) -> None:
        kind = mlp.get("kind", "moe")
        if kind != "moe":
            raise ConfigError(f"config.json: {where}: unsupported mlp kind {kind!r} (known: moe)")
        _get(mlp.get("expert"), "ff", int, where + ".expert")
        r = mlp.get("router")
        n = _get(r, "experts", int, where + ".router")
        top = _get(r, "top", int, where + ".router")
        if r.get("scale") is not None:
            _get(r, "scale", float, where + ".router")
        if top > n:
            raise ConfigError(f"config.json: {where}: top {top} of {n} experts")

    def to_dict(self) -> Dict[str, Any]:
        """The ``config.json`` that reads back as this configuration."""
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab,
                               "width": self.width, "norm": {"eps": self.eps},
                               "embedding": {"scale": self.embedding_scale},
                               "logit_softcap": self.logit_softcap, "layers": []}
        for layer in self.layers:
            out["layers"].append({"type": layer.type, "mixer": layer.m(), "mlp": layer.f()})
        if self.max_positions != type(self).max_positions:
            out["max_positions"] = self.max_positions
        return out

    # ---------------------------------------------------------------------------------------
    def _delta_spec(self, m: Dict[str, Any], x: str, low_rank: bool) -> PartSpec:
        """The gated delta rule of the tensors under ``x``.  ``low_rank``: the decay per key
        channel and the sigmoid gate of the parallel mixer's half, both through two factors
        whose rank the stored tensors give (``rank`` in the configuration fixes it for models
        with random weights)."""
        W = self.width
        H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], int(m["conv"])
        t = {"q": (x + "q", (G * d, W)), "k": (x + "k", (G * d, W)), "v": (x + "v", (H * dv, W)),
             "q_conv": (x + "q.conv", (G * d, taps)), "k_conv": (x + "k.conv", (G * d, taps)),
             "v_conv": (x + "v.conv", (H * dv, taps)), "b": (x + "b", (H, W)),
             "A_log": (x + "A_log", (H,)), "norm": (x + "norm", (dv,)),
             "o": (x + "o", (W, H * dv))}
        if low_rank:
            r = m.get("rank")
            t.update(a1=(x + "a1", (r, W)), a2=(x + "a2", (H * d, r)),
                     dt_bias=(x + "dt_bias", (H * d,)),
                     g1=(x + "g1", (r, W)), g2=(x + "g2", (H * dv, r)))
        else:
            t.update(a=(x + "a", (H, W)), dt_bias=(x + "dt_bias", (H,)),
                     g=(x + "g", (H * dv, W)))
        return PartSpec("gated_delta", {
            "hidden_size": W, "num_heads": H, "num_kv_heads": G, "key_dim": d, "value_dim": dv,
            "conv_taps": taps, "eps": self.eps,
            "gate_activation": "sigmoid" if low_rank else "silu", "tensors": t})

    def to_spec(self) -> ModelSpec:
        c = self
        W = c.width

        def norm(name: str, width: int = W) -> PartSpec:
            return PartSpec("rms_norm", {"width": width, "eps": c.eps,
                                         "tensors": {"weight": (name, (width,))}})

        first_blended = next((i for i, layer in enumerate(c.layers)
                              if layer.type == "attention" and layer.m().get("v_mix")), None)
        layers = []
        for i, layer in enumerate(c.layers):
            p = f"l{i}."
            x = p + "mix."
            m = layer.m()
            if layer.type == "attention":
                H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
                t = {"q": (x + "q", (H * d, W)), "k": (x + "k", (G * d, W)),
                     "v": (x + "v", (G * dv, W)), "q_bias": (x + "q.b", (H * d,)),
                     "k_bias": (x + "k.b", (G * d,)), "v_bias": (x + "v.b", (G * dv,)),
                     "gate": (x + "g", (H, W)), "o": (x + "o", (W, H * dv))}
                params: Dict[str, Any] = {
                    "hidden_size": W, "num_heads": H, "num_kv_heads": G, "head_dim": d,
                    "value_dim": dv, "scale": float(m["scale"]), "position": None, "tensors": t}
                if m.get("q_temp") is not None:
                    params["q_temp"] = {"coef": float(m["q_temp"]["coef"]),
                                        "every": int(m["q_temp"]["every"])}
                if m.get("v_mix"):
                    t["blend"] = (x + "vmix", ())
                    params["value_blend"] = {"group": VALUE_GROUP, "source": i == first_blended}
                mixer = PartSpec("attention", params)
            elif layer.type == "delta":
                mixer = c._delta_spec(m, x, low_rank=False)
            else:
                left, right = m["left"], m["right"]
                H, G, d, dv = left["heads"], left["kv_heads"], left["dim"], left["vdim"]
                lx, rx = x + "left.", x + "right."
                rot = left.get("rot")
                attn = PartSpec("attention", {
                    "hidden_size": W, "num_heads": H, "num_kv_heads": G, "head_dim": d,
                    "value_dim": dv, "scale": float(left["scale"]),
                    "q_norm": norm(lx + "q.norm", d), "k_norm": norm(lx + "k.norm", d),
                    "position": None if rot is None else PartSpec("rope_neox", {
                        "rot_dim": int(rot["dims"]), "theta": float(rot["base"]),
                        "freq_scale": 1.0, "attn_factor": 1.0}),
                    "tensors": {"q": (lx + "q", (H * d, W)), "k": (lx + "k", (G * d, W)),
                                "v": (lx + "v", (G * dv, W)), "gate": (lx + "g", (H * dv, W)),
                                "o": (lx + "o", (W, H * dv))}})
                mixer = PartSpec("parallel", {
                    "hidden_size": W, "eps": c.eps, "left": attn,
                    "right": c._delta_spec(right, rx, low_rank=True),
                    "tensors": {"left_out": (lx + "out", (W,)), "right_out": (rx + "out", (W,))}})
            f = p + "mlp."
            mlp = layer.f()
            if mlp is None:
                ffn = PartSpec("none", {})
            else:
                r = mlp["router"]
                E, top, ff = int(r["experts"]), int(r["top"]), int(mlp["expert"]["ff"])
                t = {"router": (f + "router", (E, W)), "correction": (f + "correction", (E,))}
                for e in range(E):
                    t[f"up{e}"] = (f"{f}e{e}.up", (ff, W))
                    t[f"down{e}"] = (f"{f}e{e}.down", (W, ff))
                ffn = PartSpec("moe", {
                    "hidden_size": W, "intermediate_size": ff, "experts": E, "top": top,
                    "scores": "softmax_all_renormed",
                    "weight_scale": float(r.get("scale") if r.get("scale") is not None else 1.0),
                    "activation": "relu_squared", "tensors": t})
            block = PartSpec("shared_norm_residual", {"norm": norm(p + "norm1")})
            layers.append(LayerSpec(block, mixer, ffn, p))

        table = ("embed", (c.vocab, W))
        spec = ModelSpec(
            architecture=c.architecture, vocab_size=c.vocab, hidden_size=W,
            max_positions=c.max_positions,
            embedding=PartSpec("token_embedding", {
                "vocab_size": c.vocab, "hidden_size": W, "scale": c.embedding_scale,
                "tensors": {"table": table}}),
            layers=tuple(layers), run_order=tuple(LayerCall(i) for i in range(len(layers))),
            final_norm=norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": c.vocab, "hidden_size": W, "tied": True,
                                          "soft_cap": c.logit_softcap,
                                          "tensors": {"weight": table}}))
        spec.validate()
        return spec


def sized_like(width: int, ff: int, heads: int, kv_heads: int, head_dim: int, layers: int,
               vocab: int, experts: int = 8, top: int = 2, rank: int = 64) -> PavatarConfig:
    """A configuration for models with random weights at the sizes of a transformer: layers
    repeating (delta, attention, parallel, attention), each with ``experts`` experts of width
    ff / top of which a token uses ``top``.  The recurrences have one value head per attention
    head and one q/k head per key head, all of ``head_dim`` channels."""
    heads = min(heads, 16 * kv_heads)
    moe = {"kind": "moe", "expert": {"ff": ff // top},
           "router": {"experts": experts, "top": top, "scale": 1.0}}
    att = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim,
           "scale": head_dim ** -0.5, "q_temp": {"coef": 0.1, "every": 1024}, "v_mix": True}
    left = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim,
            "scale": head_dim ** -0.5, "rot": {"dims": head_dim, "base": 1e6}}
    delta = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "conv": 4}
    out = []
    for i in range(layers):
        k = i % 4
        if k == 0:
            out.append({"type": "delta", "mixer": dict(delta), "mlp": moe})
        elif k == 2:
            out.append({"type": "parallel",
                        "mixer": {"left": dict(left), "right": dict(delta, rank=rank)},
                        "mlp": moe})
        else:
            out.append({"type": "attention", "mixer": dict(att), "mlp": moe})
    return PavatarConfig.from_dict({
        "architecture": "Pavatar", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
        "embedding": {"scale": 1.0}, "logit_softcap": 30.0, "layers": copy.deepcopy(out)})
