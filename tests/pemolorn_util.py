"""Small Pemolorn configurations with seeded weights for the tests, the plain implementation's
logits for them, and the error bounds.  Every configuration here is the tests' own: windows that
are no multiples of their pools, pools larger than windows, key and value sizes that differ,
groups of one and of three query heads, one to four taps, routers with and without identity
experts, layers that read another layer's keys with a wider mask than its own."""
from __future__ import annotations

import functools
import json
import os
import tempfile
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from plain import pemolorn_plain as PP


def left(heads=4, kv_heads=2, dim=32, vdim=32, conv=3, size=20, pool=8, rot=8, base=10000.0,
         scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
         "mask": {"size": size, "pool": pool},
         "scale": scale if scale is not None else dim ** -0.5}
    if rot:
        m["rot"] = {"dims": rot, "base": base}
    return m


def parallel(width=40, mlp=None, **kw):
    return {"type": "parallel", "mixer": {"left": left(**kw), "right": {"width": width}},
            "mlp": mlp}


def attention(heads=6, kv_heads=2, dim=32, vdim=32, size=17, keep=3, scale=None, kv_from=None,
              mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "mask": {"size": size, "keep_first": keep},
         "scale": scale if scale is not None else dim ** -0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, top=2, identity=2, ff=24, limit=1.0):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "top": top, "identity": identity}}


def config(layers, width=64, vocab=96, eps=1e-5):
    return {"architecture": "Pemolorn", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": layers}


CONFIGS: Dict[str, dict] = {
    # one mechanism each
    "par": config([parallel(mlp=dense(96))]),
    # values shorter than keys, whole heads rotated, a group of one, a pool of five
    "par_vd": config([parallel(width=24, heads=3, kv_heads=3, dim=48, vdim=24, conv=2, size=12,
                               pool=5, rot=48, base=500.0)], width=48),
    # values longer than keys, a pool larger than the window, one tap (no convolution)
    "par_big_pool": config([parallel(width=72, heads=2, kv_heads=1, dim=16, vdim=40, conv=1,
                                     size=6, pool=16, rot=4)]),
    # a pool of one token, four taps
    "par_pool1": config([parallel(width=8, heads=2, kv_heads=2, dim=64, vdim=64, conv=4, size=9,
                                  pool=1, rot=32, mlp=dense(40))]),
    "attn": config([attention(mlp=dense(128))]),
    "attn_vd": config([attention(heads=4, kv_heads=4, dim=24, vdim=40, size=9, keep=0)]),
    "attn_keep": config([attention(heads=8, kv_heads=1, dim=64, vdim=64, size=5, keep=11,
                                   scale=0.2)], width=96),
    # two layers read the keys of the first, one with a wider window and more kept tokens
    "shared": config([attention(size=10, keep=2, mlp=dense(64)),
                      attention(heads=2, size=23, keep=5, kv_from=0),
                      attention(heads=4, size=4, keep=0, kv_from=0, mlp=dense(48))]),
    "moe": config([attention(mlp=moe())]),
    "moe_top1": config([parallel(mlp=moe(experts=3, top=1, identity=1, ff=40, limit=0.5))]),
    "moe_no_identity": config([attention(mlp=moe(experts=7, top=3, identity=0, ff=16,
                                                 limit=4.0))]),
    "moe_all": config([attention(mlp=moe(experts=2, top=3, identity=1, ff=32))]),
    # sizes that are multiples of nothing
    "odd": config([parallel(width=13, heads=3, kv_heads=1, dim=10, vdim=6, conv=3, size=7, pool=3,
                            rot=6, mlp=moe(experts=3, top=2, identity=1, ff=9)),
                   attention(heads=2, kv_heads=2, dim=10, vdim=14, size=5, keep=2,
                             mlp=dense(34))], width=50, vocab=33),
    # heads of 128 channels, sixteen and four query heads on a key head: the sizes at which the
    # keys outside the window have a kernel for a whole group of heads
    "wide_heads": config([parallel(width=32, heads=16, kv_heads=1, dim=128, vdim=128, conv=2, size=19,
                                   pool=4, rot=64),
                          attention(heads=8, kv_heads=2, dim=128, vdim=128, size=13, keep=6,
                                    mlp=dense(48))], width=64, vocab=80),
    # keys shorter than values whose size the tensor-core kernels have: the cache's rows are the
    # values', the queries and keys are padded
    "keys_shorter": config([parallel(width=20, heads=4, kv_heads=2, dim=48, vdim=64, conv=3, size=11,
                                     pool=3, rot=12),
                            attention(heads=2, kv_heads=2, dim=32, vdim=64, size=9, keep=5,
                                      mlp=dense(56))], width=72, vocab=70),
    # all of them, in an order of their own
    "mix": config([attention(size=21, keep=4, mlp=moe()),
                   parallel(mlp=moe(experts=4, top=2, identity=1)),
                   attention(heads=2, size=30, keep=1, kv_from=0, mlp=dense(64)),
                   parallel(width=56, heads=2, kv_heads=2, dim=64, vdim=64, conv=4, size=33,
                            pool=16, rot=16, base=5e5),
                   attention(heads=4, kv_heads=1, dim=64, vdim=64, size=40, keep=8,
                             mlp=dense(80))], width=64, vocab=128),
}


def random_config(seed: int) -> str:
    """A configuration drawn from a seed: three to six layers of any kind in any order, sizes of
    the kind a small model has.  Registered under the returned name."""
    name = f"random{seed}"
    if name in CONFIGS:
        return name
    rng = np.random.default_rng(7000 + seed)
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]

    def mlp():
        r = rng.random()
        if r < 0.2:
            return None
        if r < 0.55:
            return dense(pick(96, 160, 320))
        experts = pick(3, 6, 8, 12)
        ident = pick(0, 1, 2, 4)
        return moe(experts=experts, top=min(pick(1, 2, 3, 4), experts + ident), identity=ident, ff=pick(32, 48, 64),
                   limit=pick(1.0, 2.0, 7.0))

    layers: List[dict] = []
    owners: List[int] = []
    for i in range(int(rng.integers(3, 7))):
        if rng.random() < 0.4:
            heads, dim = pick(2, 4, 8), pick(32, 64, 128)
            layers.append(parallel(
                width=pick(64, 96, 224), heads=heads,
                kv_heads=pick(*[g for g in (1, 2, 4, 8) if heads % g == 0]), dim=dim,
                vdim=pick(dim, 32, 64), conv=pick(2, 3, 4), size=pick(24, 40, 72, 100),
                pool=pick(4, 8, 16, 32), rot=pick(dim // 4, dim // 2, dim),
                base=pick(1e4, 5e5), scale=pick(dim ** -0.5, 0.125), mlp=mlp()))
            continue
        size, keep = pick(16, 33, 64, 136), pick(0, 1, 4, 6)
        if owners and rng.random() < 0.4:
            src = owners[int(rng.integers(len(owners)))]
            m = layers[src]["mixer"]
            layers.append(attention(heads=m["kv_heads"] * pick(1, 2, 3), kv_heads=m["kv_heads"],
                                    dim=m["dim"], vdim=m["vdim"], size=size, keep=keep,
                                    scale=m["scale"], kv_from=src, mlp=mlp()))
            continue
        kv, dim = pick(1, 2, 4), pick(32, 64, 128)
        owners.append(i)
        layers.append(attention(heads=kv * pick(1, 2, 3, 4), kv_heads=kv, dim=dim,
                                vdim=pick(dim, 32, 64), size=size, keep=keep,
                                scale=pick(dim ** -0.5, 0.125), mlp=mlp()))
    CONFIGS[name] = config(layers, width=pick(96, 128, 160, 224, 256),
                           vocab=int(rng.integers(200, 700)))
    return name


from runidra_util import BOUND, _bf16_values, assert_close  # noqa: E402,F401  (shared helpers)


def _weights(cfg: dict, seed: int) -> Dict[str, np.ndarray]:
    """Seeded weights, already rounded to bfloat16 values so that both precisions and the
    plain implementation compute with the same numbers."""
    rng = np.random.default_rng(seed)
    W = cfg["width"]
    t: Dict[str, np.ndarray] = {}

    def mat(name, out, inn, gain=1.0):
        t[name] = rng.standard_normal((out, inn)) * gain / np.sqrt(inn)

    def vec(name, n, mean=0.0, std=1.0):
        t[name] = mean + std * rng.standard_normal(n)

    def one(name, mean=1.0, std=0.1):
        t[name] = np.asarray(mean + std * rng.standard_normal())

    t["embed"] = rng.standard_normal((cfg["vocab"], W))
    for i, layer in enumerate(cfg["layers"]):
        p, x, m = f"l{i}.", f"l{i}.mix.", layer["mixer"]
        one(p + "norm1"), one(p + "norm1b", 0.8)
        if layer["type"] == "parallel":
            l, r = m["left"], m["right"]
            H, G, d, dv, taps = l["heads"], l["kv_heads"], l["dim"], l["vdim"], l.get("conv") or 0
            lx, rx = x + "left.", x + "right."
            mat(lx + "q", H * d, W, 2.0), mat(lx + "k", G * d, W, 2.0), mat(lx + "v", G * dv, W)
            vec(lx + "q.norm", H * d, 1.0, 0.2), vec(lx + "k.norm", G * d, 1.0, 0.2)
            if taps >= 1:
                for r_, n in (("q", H * d), ("k", G * d), ("v", G * dv)):
                    t[lx + r_ + ".conv"] = rng.standard_normal((n, taps)) * 0.6
            vec(lx + "sink", H, 0.5, 1.0), mat(lx + "o", W, H * dv)
            R = r["width"]
            mat(rx + "z", R, W, 2.0), vec(rx + "z.b", R, 0.0, 1.0)
            mat(rx + "x", R, W, 2.0), vec(rx + "x.b", R, 0.0, 0.5)
            mat(rx + "g", R, W, 2.0), mat(rx + "o", W, R)
            vec(lx + "out", W, 1.0, 0.2), vec(rx + "out", W, 1.0, 0.2)
        else:
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            mat(x + "q", H * d, W, 2.0), vec(x + "q.norm", d, 1.0, 0.2)
            if m.get("kv_from") is None:
                mat(x + "k", G * d, W, 2.0), mat(x + "v", G * dv, W), vec(x + "k.norm", d, 1.0, 0.2)
            vec(x + "sink", H, 0.5, 1.0), mat(x + "o", W, H * dv)
        mlp = layer["mlp"]
        if mlp is not None:
            one(p + "norm2"), one(p + "norm2b", 0.8)
            f = p + "mlp."
            if mlp["kind"] == "dense":
                mat(f + "up", mlp["ff"], W, 1.5), mat(f + "down", W, mlp["ff"])
            else:
                E, ident = mlp["router"]["experts"], mlp["router"].get("identity") or 0
                ff = mlp["expert"]["ff"]
                for e in range(E):
                    mat(f"{f}e{e}.gate", ff, W, 2.0), mat(f"{f}e{e}.up", ff, W, 2.0)
                    mat(f"{f}e{e}.down", W, ff)
                # logits far enough apart that rounding seldom changes who is chosen; a
                # correction large enough to change the order of the scores now and then
                mat(f + "router", E + ident, W, 4.0)
                vec(f + "correction", E + ident, 0.0, 0.05)
    one("final.norm")
    mat("head", cfg["vocab"], W)
    return _bf16_values(t)


CUSTOM: Dict[str, Dict[str, np.ndarray]] = {}     # configurations whose weights a test has made


@functools.lru_cache(maxsize=None)
def weights(name: str, seed: int = 0) -> Dict[str, np.ndarray]:
    return CUSTOM[name] if name in CUSTOM else _weights(CONFIGS[name], seed)


_dirs: Dict[tuple, str] = {}


def model_dir(name: str, seed: int = 0) -> str:
    """A folder with config.json and model.safetensors (bfloat16) of the configuration."""
    from llmario_b200.weights.safetensors_io import write_safetensors

    key = (name, seed)
    if key not in _dirs:
        d = tempfile.mkdtemp(prefix=f"pemolorn_{name}_")
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(CONFIGS[name], f)
        write_safetensors(os.path.join(d, "model.safetensors"),
                          {n: torch.from_numpy(np.asarray(a)).to(torch.bfloat16)
                           for n, a in weights(name, seed).items()})
        _dirs[key] = d
    return _dirs[key]


@functools.lru_cache(maxsize=None)
def _plain(name: str, seed: int, tokens: tuple):
    margins: List[np.ndarray] = []
    logits = PP.forward(CONFIGS[name], weights(name, seed), list(tokens), margins=margins)
    closest = np.min(np.stack(margins), axis=0) if margins else np.full(len(tokens), np.inf)
    return logits, closest


def plain_logits(name: str, tokens: Sequence[int], seed: int = 0) -> np.ndarray:
    return _plain(name, seed, tuple(int(t) for t in tokens))[0]


# A router's choice between two experts whose choice scores lie closer than this (in units of
# the larger score, which is what a move of a logit is multiplied by) can fall either way once
# the router's input is rounded to 16 bits; the 16-bit tests do not compare such positions.
CLOSE_CALL = 0.08


def router_margins(name: str, tokens: Sequence[int], seed: int = 0) -> np.ndarray:
    """Per position, the smallest margin over all routed layers between the last chosen expert
    and the best one not chosen (infinite for a model without routed layers)."""
    return _plain(name, seed, tuple(int(t) for t in tokens))[1]


@functools.lru_cache(maxsize=None)
def _sensitivity(name: str, seed: int, tokens: tuple) -> np.ndarray:
    """Per position, how far the logits move when the inputs move by about one bfloat16
    rounding or two: the plain implementation run again with the embedding rows scaled by
    1 + 2^-7 N(0, 1) (the largest of four such moves)."""
    w = dict(weights(name, seed))
    rng = np.random.default_rng(99)
    embed, ref = w["embed"], _plain(name, seed, tokens)[0]
    worst = np.zeros(len(tokens))
    for _ in range(4):
        w["embed"] = embed * (1 + 2.0 ** -7 * rng.standard_normal(embed.shape))
        moved = PP.forward(CONFIGS[name], w, list(tokens))
        worst = np.maximum(worst, np.abs(moved - ref).max(axis=1))
    return worst


def sensitivity(name: str, tokens: Sequence[int], seed: int = 0) -> np.ndarray:
    return _sensitivity(name, seed, tuple(int(t) for t in tokens))


def tokens_for(name: str, n: int, seed: int) -> List[int]:
    rng = np.random.default_rng(1000 + seed)
    return [int(t) for t in rng.integers(0, CONFIGS[name]["vocab"], n)]


def slack_for(name: str, tokens: Sequence[int], dtype: str, seed: int = 0) -> Optional[np.ndarray]:
    """What a position is allowed on top of the bound.  float32: nothing.  bfloat16: three times
    what a move of the inputs by a rounding or two does to it in the plain implementation, and
    everything at a position where a router makes a close call (another expert may run)."""
    if dtype != "bfloat16":
        return None
    slack = 3.0 * sensitivity(name, tokens, seed)
    slack[router_margins(name, tokens, seed) < CLOSE_CALL] = np.inf
    return slack


def runner_for(name: str, dtype: str, page_size: int = 16, cache_tokens: int = 1024,
               max_requests: int = 4, seed: int = 0, use_graphs: bool = True,
               max_context: int = 0):
    from llmario_b200.engine.model import Model
    from llmario_b200.engine.step import ModelRunner

    model = Model.from_folder(model_dir(name, seed), dtype, "cuda:0")
    return ModelRunner(model, page_size=page_size, n_pages=-(-cache_tokens // page_size),
                       max_requests=max_requests, max_context=max_context or cache_tokens,
                       token_budget=cache_tokens, use_graphs=use_graphs)
