"""Small Pavatar configurations with seeded weights for the tests, the plain implementation's
logits for them, the error bounds, and the helpers that drive the step function.  Every
configuration here is the tests' own: key and value sizes that differ, groups of one, three and
four heads, one to four taps, rotations of a part of a head and of none, temperatures that step
every few tokens, routers that choose one expert and all of them, layers without experts."""
from __future__ import annotations

import functools
import json
import os
import tempfile
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from plain import pavatar_plain as PP
from runidra_util import BOUND, _bf16_values, assert_close  # noqa: F401  (shared helpers)


def attention(heads=6, kv_heads=2, dim=32, vdim=16, scale=None, every=7, coef=0.4, v_mix=True,
              mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": scale if scale is not None else dim ** -0.5}
    if every:
        m["q_temp"] = {"coef": coef, "every": every}
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention", "mixer": m, "mlp": mlp}


def delta_sizes(heads=4, kv_heads=2, dim=24, vdim=16, conv=3, rank=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}
    if rank:
        m["rank"] = rank
    return m


def delta(mlp=None, **kw):
    return {"type": "delta", "mixer": delta_sizes(**kw), "mlp": mlp}


def parallel(heads=4, kv_heads=2, dim=32, vdim=32, scale=None, rot=16, base=10000.0, mlp=None,
             right=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
            "scale": scale if scale is not None else dim ** -0.5}
    if rot:
        left["rot"] = {"dims": rot, "base": base}
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": left, "right": right or delta_sizes(heads=2, kv_heads=1, rank=5)}}


def moe(experts=5, top=2, ff=24, scale=1.5):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "scale": scale}}


def config(layers, width=64, vocab=96, eps=1e-5, embed_scale=3.0, cap=12.0):
    return {"architecture": "Pavatar", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": embed_scale}, "logit_softcap": cap, "layers": layers}


CONFIGS: Dict[str, dict] = {
    # one mechanism each
    "delta": config([delta(mlp=moe())]),
    # one q/k head for three value heads, values longer than keys, two taps
    "delta_shared": config([delta(heads=3, kv_heads=1, dim=16, vdim=40, conv=2)], width=48),
    # one tap (a weight per channel, no inputs kept), a head per q/k head, four taps beside it
    "delta_taps": config([delta(heads=2, kv_heads=2, dim=64, vdim=8, conv=1),
                          delta(heads=1, kv_heads=1, dim=8, vdim=64, conv=4, mlp=moe(3, 1, 16))]),
    # keys of more channels than a warp holds four at a time, and of 320
    "delta_wide": config([delta(heads=2, kv_heads=1, dim=136, vdim=24, conv=3),
                          delta(heads=1, kv_heads=1, dim=320, vdim=12, conv=2)], width=56),
    "attn": config([attention(mlp=moe(4, 4, 16, 2.0))]),
    # keys and values of one size, no temperature, no blending: the store of the standard layers
    "attn_plain": config([attention(heads=4, kv_heads=4, dim=32, vdim=32, every=0, v_mix=False),
                          attention(heads=2, kv_heads=1, dim=64, vdim=64, every=0, v_mix=False,
                                    mlp=moe()),
                          attention(heads=3, kv_heads=3, dim=16, vdim=24, every=0, v_mix=False)]),
    # three layers blend values (the first one's), one between them does not; values longer
    # than keys; a temperature that steps at every token and one that never does
    "attn_blend": config([attention(heads=2, kv_heads=2, dim=16, vdim=24, every=1, coef=0.05),
                          attention(heads=4, kv_heads=1, dim=32, vdim=32, v_mix=False, every=500),
                          attention(heads=6, kv_heads=2, dim=32, vdim=24, every=13),
                          attention(heads=2, kv_heads=2, dim=8, vdim=24, every=0, mlp=moe())]),
    "par": config([parallel(mlp=moe())]),
    # values shorter than keys, whole heads rotated, a group of one; the recurrence beside it
    # with as many q/k heads as value heads
    "par_vd": config([parallel(heads=3, kv_heads=3, dim=48, vdim=24, rot=48, base=500.0, scale=0.3,
                               right=delta_sizes(heads=3, kv_heads=3, dim=16, vdim=16, conv=4,
                                                 rank=8))], width=48),
    # no rotation at all, values longer than keys, eight query heads on one key head
    "par_norot": config([parallel(heads=8, kv_heads=1, dim=16, vdim=40, rot=0,
                                  right=delta_sizes(heads=4, kv_heads=2, dim=8, vdim=32, conv=1,
                                                    rank=3))]),
    "moe_top1": config([delta(mlp=moe(experts=3, top=1, ff=40, scale=0.7))]),
    "moe_many": config([attention(mlp=moe(experts=17, top=6, ff=8, scale=3.0))]),
    # sizes that are multiples of nothing
    "odd": config([delta(heads=3, kv_heads=1, dim=10, vdim=6, conv=3, mlp=moe(3, 2, 9)),
                   attention(heads=3, kv_heads=1, dim=10, vdim=6, every=3),
                   parallel(heads=2, kv_heads=2, dim=10, vdim=14, rot=6,
                            right=delta_sizes(heads=1, kv_heads=1, dim=6, vdim=10, conv=2, rank=7),
                            mlp=moe(2, 2, 11)),
                   attention(heads=3, kv_heads=1, dim=10, vdim=6, every=5)],
                  width=50, vocab=33, embed_scale=1.0, cap=0.0),
    # heads of 64 and 128 channels with groups that the tensor-core kernels take
    "wide_heads": config([parallel(heads=8, kv_heads=2, dim=128, vdim=128, rot=64,
                                   right=delta_sizes(heads=2, kv_heads=2, dim=128, vdim=128,
                                                     conv=4, rank=16)),
                          attention(heads=4, kv_heads=1, dim=64, vdim=64, every=9, mlp=moe(4, 2, 32)),
                          attention(heads=16, kv_heads=1, dim=64, vdim=64, every=4)],
                         width=128, vocab=80),
    # keys shorter than values whose size the tensor-core kernels have: the cache's rows are the
    # values', the queries and keys are padded
    "keys_shorter": config([attention(heads=4, kv_heads=2, dim=32, vdim=64, every=6),
                            parallel(heads=2, kv_heads=2, dim=48, vdim=64, rot=12,
                                     right=delta_sizes(heads=2, kv_heads=1, dim=64, vdim=64, conv=3,
                                                       rank=8), mlp=moe(3, 2, 48)),
                            attention(heads=8, kv_heads=2, dim=32, vdim=64, every=0)],
                           width=72, vocab=70),
    # all of them, in an order of their own
    "mix": config([attention(every=11, mlp=moe()),
                   delta(mlp=moe(4, 2, 32)),
                   parallel(mlp=moe(6, 3, 16, 2.5)),
                   delta(heads=2, kv_heads=2, dim=32, vdim=32, conv=4),
                   attention(heads=2, every=5, coef=0.2, mlp=moe()),
                   parallel(heads=2, kv_heads=1, dim=64, vdim=64, rot=32, base=5e5,
                            right=delta_sizes(heads=4, kv_heads=4, dim=16, vdim=16, conv=2,
                                              rank=4))], width=64, vocab=128),
}


def random_config(seed: int) -> str:
    """A configuration drawn from a seed: three to six layers of any kind in any order, sizes of
    the kind a small model has.  Registered under the returned name."""
    name = f"random{seed}"
    if name in CONFIGS:
        return name
    rng = np.random.default_rng(9000 + seed)
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]

    def mlp():
        if rng.random() < 0.25:
            return None
        experts = pick(3, 6, 8, 12)
        return moe(experts=experts, top=min(pick(1, 2, 3, 4), experts), ff=pick(32, 48, 64, 96),
                   scale=pick(1.0, 2.0, 2.5))

    def recur(rank=None):
        heads = pick(2, 4, 6)
        return dict(heads=heads, kv_heads=pick(*[g for g in (1, 2, 3, 6) if heads % g == 0]),
                    dim=pick(16, 32, 64), vdim=pick(16, 32, 64), conv=pick(2, 3, 4), rank=rank)

    blended = (pick(1, 2, 4), pick(16, 32, 64))
    layers: List[dict] = []
    for _ in range(int(rng.integers(3, 7))):
        r = rng.random()
        if r < 0.3:
            layers.append(delta(mlp=mlp(), **recur()))
        elif r < 0.6:
            heads, dim = pick(2, 4, 8), pick(32, 64, 128)
            layers.append(parallel(
                heads=heads, kv_heads=pick(*[g for g in (1, 2, 4, 8) if heads % g == 0]), dim=dim,
                vdim=pick(dim, 32, 64), rot=pick(dim // 4, dim // 2, dim), base=pick(1e4, 5e5),
                scale=pick(dim ** -0.5, 0.1875), right=delta_sizes(**recur(pick(4, 8, 24))),
                mlp=mlp()))
        else:
            mixes = rng.random() < 0.7
            kv, vdim = blended if mixes else (pick(1, 2, 4), pick(32, 64))
            dim = pick(32, 64, 128)
            layers.append(attention(heads=kv * pick(1, 2, 3, 4), kv_heads=kv, dim=dim, vdim=vdim,
                                    scale=pick(dim ** -0.5, 0.125), every=pick(0, 16, 50, 128),
                                    coef=pick(0.1, 0.3), v_mix=mixes, mlp=mlp()))
    CONFIGS[name] = config(layers, width=pick(96, 128, 160, 224, 256),
                           vocab=int(rng.integers(200, 700)), embed_scale=pick(1.0, 4.0, 16.0),
                           cap=pick(0.0, 15.0, 30.0))
    return name


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

    def recurrence(x, m, low_rank):
        H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
        for r, n in (("q", G * d), ("k", G * d), ("v", H * dv)):
            mat(x + r, n, W, 2.0)
            t[x + r + ".conv"] = rng.standard_normal((n, taps)) * 0.6
        mat(x + "b", H, W, 2.0)
        # rates from a percent to a few tenths a token: some heads remember hundreds of tokens
        vec(x + "A_log", H, -3.0, 1.2), vec(x + "norm", dv, 1.0, 0.2), mat(x + "o", W, H * dv)
        if low_rank:
            r = m.get("rank") or 5
            mat(x + "a1", r, W, 2.0), mat(x + "a2", H * d, r, 2.0), vec(x + "dt_bias", H * d)
            mat(x + "g1", r, W, 2.0), mat(x + "g2", H * dv, r, 2.0)
        else:
            mat(x + "a", H, W, 2.0), vec(x + "dt_bias", H), mat(x + "g", H * dv, W, 2.0)

    t["embed"] = rng.standard_normal((cfg["vocab"], W)) / cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        p, x, m = f"l{i}.", f"l{i}.mix.", layer["mixer"]
        vec(p + "norm1", W, 1.0, 0.1)
        if layer["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            mat(x + "q", H * d, W, 2.0), mat(x + "k", G * d, W, 2.0), mat(x + "v", G * dv, W)
            vec(x + "q.b", H * d, 0.0, 0.3), vec(x + "k.b", G * d, 0.0, 0.3)
            vec(x + "v.b", G * dv, 0.0, 0.3)
            if m.get("v_mix"):
                t[x + "vmix"] = np.asarray(rng.uniform(0.25, 0.75))
            mat(x + "g", H, W, 2.0), mat(x + "o", W, H * dv)
        elif layer["type"] == "delta":
            recurrence(x, m, False)
        else:
            l = m["left"]
            H, G, d, dv = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            lx, rx = x + "left.", x + "right."
            mat(lx + "q", H * d, W, 2.0), mat(lx + "k", G * d, W, 2.0), mat(lx + "v", G * dv, W)
            vec(lx + "q.norm", d, 1.0, 0.2), vec(lx + "k.norm", d, 1.0, 0.2)
            mat(lx + "g", H * dv, W, 2.0), mat(lx + "o", W, H * dv)
            recurrence(rx, m["right"], True)
            vec(lx + "out", W, 1.0, 0.2), vec(rx + "out", W, 1.0, 0.2)
        mlp = layer["mlp"]
        if mlp is not None:
            f = p + "mlp."
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            for e in range(E):
                mat(f"{f}e{e}.up", ff, W, 1.2), mat(f"{f}e{e}.down", W, ff)
            # logits far enough apart that rounding seldom changes who is chosen; a correction
            # large enough to change the order of the scores now and then
            mat(f + "router", E, W, 4.0)
            vec(f + "correction", E, 0.0, 0.05)
    vec("final.norm", W, 1.0, 0.1)
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
        d = tempfile.mkdtemp(prefix=f"pavatar_{name}_")
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(CONFIGS[name], f)
        write_safetensors(os.path.join(d, "model.safetensors"),
                          {n: torch.from_numpy(np.asarray(a)).to(torch.bfloat16)
                           for n, a in weights(name, seed).items()})
        _dirs[key] = d
    return _dirs[key]


# A router's choice between two experts whose choice scores lie closer than this (in units of
# the larger of the two scores) can fall either way once the router's input is rounded to 16
# bits; the 16-bit tests do not compare such positions.
CLOSE_CALL = 0.08


@functools.lru_cache(maxsize=None)
def _plain(name: str, seed: int, tokens: tuple):
    return PP.forward(CONFIGS[name], weights(name, seed), list(tokens), close_margin=CLOSE_CALL)


def plain_logits(name: str, tokens: Sequence[int], seed: int = 0) -> np.ndarray:
    return _plain(name, seed, tuple(int(t) for t in tokens))[0]


def close_calls(name: str, tokens: Sequence[int], seed: int = 0) -> np.ndarray:
    """Per position, whether some router of the model makes a close call there."""
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


def tokens_for(name: str, n: int, seed: int) -> List[int]:
    rng = np.random.default_rng(1000 + seed)
    return [int(t) for t in rng.integers(0, CONFIGS[name]["vocab"], n)]


def slack_for(name: str, tokens: Sequence[int], dtype: str, seed: int = 0) -> Optional[np.ndarray]:
    """What a position is allowed on top of the bound.  float32: nothing.  bfloat16: three times
    what a move of the inputs by a rounding or two does to it in the plain implementation, and
    everything at a position where a router makes a close call (another expert may run)."""
    if dtype != "bfloat16":
        return None
    toks = tuple(int(t) for t in tokens)
    slack = 3.0 * _sensitivity(name, seed, toks)
    slack[close_calls(name, toks, seed)] = np.inf
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


def run_steps(runner, steps):
    """``steps``: lists of (request, tokens, wanted places).  Returns request -> {position: logits}."""
    from llmario_b200.engine.step import StepEntry

    got = {}
    for step in steps:
        entries = [StepEntry(r, list(t), list(w)) for r, t, w in step]
        starts = {r: (runner.length(r) if runner.cache.has(r) else 0) for r, _, _ in step}
        logits = runner.step(entries).cpu().numpy()
        i = 0
        for r, _, want in step:
            for wpos in want:
                got.setdefault(r, {})[starts[r] + wpos] = logits[i].copy()
                i += 1
    return got


def check_request(got, name, tokens, dtype, what, seed=0):
    ref = plain_logits(name, tokens, seed)
    pos = sorted(got)
    slack = slack_for(name, tokens, dtype, seed)
    assert_close(np.stack([got[p] for p in pos]), ref[pos], dtype, what,
                 slack=None if slack is None else slack[pos])
