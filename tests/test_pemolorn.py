"""The Pemolorn decoder against the plain float64 implementation (tests/plain/pemolorn_plain.py):
every mechanism alone and together, in whole prompts, portions, single decoded tokens, mixed
batches, reused slots and pages, and through the engine's own entry point."""
from __future__ import annotations

import json

import numpy as np
import pytest
import torch

from plain import pemolorn_plain as PP
from pemolorn_util import (CLOSE_CALL, CONFIGS, CUSTOM, _bf16_values, _weights, assert_close,
                           attention, config, dense, model_dir, moe, parallel, plain_logits,
                           random_config, router_margins, runner_for, slack_for, tokens_for,
                           weights)

DTYPES = ("float32", "bfloat16")


# --------------------------------------------------------------------------------------------
# no GPU: configuration, and the plain implementation against itself
# --------------------------------------------------------------------------------------------
def test_configuration_round_trip_and_tensor_names():
    from llmario_b200.config import ConfigError, PemolornConfig, resolve_architecture
    from llmario_b200.weights.loader import check_tensors, expected_tensors

    for name, raw in CONFIGS.items():
        assert resolve_architecture(raw) == "Pemolorn"
        cfg = PemolornConfig.from_dict(raw)
        assert PemolornConfig.from_dict(cfg.to_dict()) == cfg
        assert cfg.to_dict() == raw, name
        spec = cfg.to_spec()
        want = expected_tensors(spec)
        have = {n: a.shape for n, a in weights(name).items()}
        assert set(want) == set(have), name
        check_tensors(spec, have)
        for i, (call, entry) in enumerate(zip(spec.run_order, raw["layers"])):
            assert call.layer == i
            assert call.reads_cache_of == entry["mixer"].get("kv_from")
        for layer, entry in zip(spec.layers, raw["layers"]):
            assert layer.mixer.kind == entry["type"]
            assert (layer.feed_forward.kind == "none") == (entry["mlp"] is None)

    def broken(name, change):
        bad = json.loads(json.dumps(CONFIGS[name]))
        change(bad)
        return bad

    with pytest.raises(ConfigError, match="unsupported type"):
        PemolornConfig.from_dict(broken("mix", lambda c: c["layers"][0].update(type="conv")))
    with pytest.raises(ConfigError, match="mlp kind"):
        PemolornConfig.from_dict(broken("mix", lambda c: c["layers"][0]["mlp"].update(kind="x")))
    with pytest.raises(ConfigError, match="top"):
        PemolornConfig.from_dict(
            broken("moe", lambda c: c["layers"][0]["mlp"]["router"].update(top=9)))
    with pytest.raises(ConfigError, match="kv_from"):
        PemolornConfig.from_dict(broken("shared", lambda c: c["layers"][1]["mixer"].update(kv_from=1)))
    with pytest.raises(ConfigError, match="kv_from"):
        PemolornConfig.from_dict(broken("shared", lambda c: c["layers"][2]["mixer"].update(kv_from=1)))
    with pytest.raises(ConfigError, match="differs"):
        PemolornConfig.from_dict(broken("shared", lambda c: c["layers"][1]["mixer"].update(dim=16)))
    with pytest.raises(ConfigError, match="eps"):
        PemolornConfig.from_dict(broken("par", lambda c: c.pop("norm")))
    with pytest.raises(ConfigError, match="dims"):
        PemolornConfig.from_dict(
            broken("par", lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7)))


def test_a_layer_that_is_read_keeps_what_its_readers_see():
    """The layer whose keys others read keeps the widest window and the most first tokens that
    any of them asks for."""
    from llmario_b200.config import PemolornConfig

    spec = PemolornConfig.from_dict(CONFIGS["shared"]).to_spec()
    owner = spec.layers[0].mixer
    assert (owner["cache_window"], owner["cache_keep_first"]) == (23, 5)
    assert (owner["window"], owner["keep_first"]) == (10, 2)
    assert spec.layers[1].mixer["shared_kv"] and "k" not in spec.layers[1].mixer["tensors"]


def test_plain_mechanisms_against_their_definitions():
    rng = np.random.default_rng(0)
    # the short convolution is a correlation with the taps, newest input under the last tap
    u, w = rng.standard_normal((9, 3)), rng.standard_normal((3, 4))
    y = PP.short_conv(u, w)
    for c in range(3):
        full = np.convolve(u[:, c], w[c, ::-1])[:9]
        np.testing.assert_allclose(y[:, c], full, atol=1e-12)
    assert np.allclose(PP.short_conv(u, w[:, 3:]), u * w[:, 3])
    # the rotation keeps lengths, leaves the channels behind `dims` alone, and makes a score a
    # function of the distance
    x = rng.standard_normal((1, 1, 12))
    a = PP.rotate_adjacent(np.repeat(x, 6, 0), np.arange(6), 8, 100.0)
    assert np.allclose(np.linalg.norm(a, axis=-1), np.linalg.norm(x)) and np.allclose(a[:, :, 8:], x[:, :, 8:])
    b = PP.rotate_adjacent(np.repeat(x, 6, 0), np.arange(6) + 11, 8, 100.0)
    assert np.allclose(a[1, 0, :8] @ a[4, 0, :8], b[1, 0, :8] @ b[4, 0, :8])
    assert np.allclose(a[0], x[0]) and not np.allclose(a[1, 0, :2], x[0, 0, :2])
    # the sink takes weight and gives nothing
    s, v = np.array([0.3, -1.0]), np.array([[1.0], [3.0]])
    e = np.exp(s)
    assert np.isclose(PP.sink_softmax_sum(s, v, 0.7)[0], (e @ v)[0] / (e.sum() + np.exp(0.7)))
    assert np.isclose(PP.sink_softmax_sum(s, v, None)[0], (e @ v)[0] / e.sum())
    # windows
    assert PP.window_visible(4)(9).tolist() == [6, 7, 8, 9]
    assert PP.window_kept_visible(3, 2)(9).tolist() == [0, 1, 7, 8, 9]
    assert PP.window_kept_visible(3, 2)(1).tolist() == [0, 1]
    # pooled blocks: with values that name their position, the mean over what position i sees
    T, P, size = 23, 4, 6
    q = np.zeros((T, 1, 2))
    k = np.zeros((T, 1, 2))
    v = np.arange(T, dtype=np.float64).reshape(T, 1, 1)
    o = PP.attend(q, k, v, 1.0, None, PP.window_visible(size), (P, size))[:, 0, 0]
    for i in range(T):
        seen = [j for j in range(i + 1) if i - j < size]
        blocks = [b for b in range(T // P) if b * P + P - 1 <= i - size]
        vals = [float(j) for j in seen] + [b * P + (P - 1) / 2 for b in blocks]
        assert np.isclose(o[i], np.mean(vals)), i
    # the recurrence in closed form for constant gates
    t = {"z": np.zeros((2, 3)), "z.b": np.array([0.0, 2.0]), "x": np.zeros((2, 3)),
         "x.b": np.array([1.5, -1.0]), "g": np.zeros((2, 3)), "o": np.eye(2)}
    t["g"][:, 0] = 1.0
    h = np.ones((5, 3))
    out = PP.min_gru(h, {"p." + n: a for n, a in t.items()}, "p.", {"width": 2})
    z = PP.sigmoid(np.array([0.0, 2.0]))
    cand = np.array([2.0, PP.sigmoid(-1.0)])
    for i in range(5):
        S = cand * (1 - (1 - z) ** (i + 1))
        np.testing.assert_allclose(out[i], S * PP.silu(1.0), atol=1e-12)
    # the router: choice by corrected score, weight the score itself, identity experts pass h
    mlp = moe(experts=2, top=2, identity=1, ff=4, limit=1.0)["router"]
    t = {"r.router": np.array([[1.0, 0], [0, 1.0], [0, 0]]), "r.correction": np.array([0.0, 0.0, 10.0])}
    chosen, wts = PP.route(np.array([[2.0, 1.0]]), t, "r.", {"router": mlp})
    s = np.exp([2.0, 1.0, 0.0]) / np.exp([2.0, 1.0, 0.0]).sum()
    assert chosen.tolist() == [[2, 0]] and np.allclose(wts, [[s[2], s[0]]])


def test_plain_edges_matter():
    """The plain statement itself: a window's edge, the kept first tokens, the pooled blocks and
    the sinks all move the logits of the needle models used below."""
    for name, key, path in (("needle_attn", "size", None), ("needle_par", "size", "left")):
        name = needle_model(name, 12)
        cfg, w = CONFIGS[name], weights(name)
        toks, probes = needle_tokens(12, 110)
        ref = PP.forward(cfg, w, toks)
        off = json.loads(json.dumps(cfg))
        m = off["layers"][0]["mixer"]
        (m[path] if path else m)["mask"]["size"] = 13
        d = np.abs(PP.forward(off, w, toks) - ref).max(axis=1)
        assert d[probes["just_outside"]].min() > 0.1 * np.abs(ref).max(), name
        w2 = {k: (v - 30.0 if k.endswith("sink") else v) for k, v in w.items()}
        assert np.abs(PP.forward(cfg, w2, toks) - ref).max() > 0.05 * np.abs(ref).max()


# --------------------------------------------------------------------------------------------
# kernels of the mechanisms, each against a few lines of NumPy
# --------------------------------------------------------------------------------------------
def _segments(rows_per_slot, n_slots):
    from llmario_b200 import kernels

    row_slot = torch.tensor([s for s, n in rows_per_slot for _ in range(n)], dtype=torch.int32,
                            device="cuda")
    seg = torch.empty(n_slots, 3, dtype=torch.int32, device="cuda")
    kernels.segment_table(row_slot, seg)
    return row_slot, seg


@pytest.mark.gpu
@pytest.mark.parametrize("width", (1, 13, 224, 1000))
def test_min_gru_kernel(width):
    """Two steps of three requests of unequal lengths, then a step of single tokens: the state
    is carried in its slot, rows of other requests do not enter."""
    from llmario_b200 import kernels

    rng = np.random.default_rng(width)
    n_slots = 5
    state = torch.zeros(n_slots, width + 3, dtype=torch.float32, device="cuda")
    ref_state = np.zeros((n_slots, width))
    zb, ub = rng.standard_normal(width), rng.standard_normal(width)
    dev = lambda a: torch.tensor(a, dtype=torch.float32, device="cuda")
    for rows_per_slot, single in (([(3, 40), (0, 1), (2, 7)], False), ([(2, 2), (3, 5)], False),
                                  ([(0, 1), (3, 1), (2, 1)], True)):
        rows = sum(n for _, n in rows_per_slot)
        zug = rng.standard_normal((rows, 3 * width + 1)) * 2
        want = np.zeros((rows, width))
        at = 0
        for s, n in rows_per_slot:
            for r in range(at, at + n):
                z = PP.sigmoid(zug[r, :width] + zb)
                u = zug[r, width:2 * width] + ub
                cand = np.where(u >= 0, u + 0.5, PP.sigmoid(u))
                ref_state[s] = (1 - z) * ref_state[s] + z * cand
                want[r] = ref_state[s] * PP.silu(zug[r, 2 * width:3 * width])
            at += n
        row_slot, seg = _segments(rows_per_slot, n_slots)
        m = dev(zug)
        for out_dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 2e-2)):
            st = state.clone()
            out = torch.empty(rows, width, dtype=out_dtype, device="cuda")
            mm = m.clone()
            kernels.min_gru(mm[:, :width], mm[:, width:2 * width], mm[:, 2 * width:3 * width],
                            dev(zb), dev(ub), st, out, row_slot, None if single else seg)
            np.testing.assert_allclose(out.float().cpu().numpy(), want, rtol=tol, atol=tol)
        state = st
        np.testing.assert_allclose(state[:, :width].cpu().numpy(), ref_state, rtol=1e-5, atol=1e-6)
    assert float(state[:, width:].abs().max()) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("taps", (1, 2, 4))
def test_short_convolution_without_activation(taps):
    """The convolution as the pooled attention uses it: no bias, no activation, the last inputs
    of a request in its slot between steps."""
    from llmario_b200 import kernels

    rng = np.random.default_rng(taps)
    C, n_slots = 37, 4
    w = rng.standard_normal((C, taps))
    lengths = {0: 11, 2: 5, 3: 23}
    u = {s: rng.standard_normal((n, C)) for s, n in lengths.items()}
    ref = {s: PP.short_conv(a, w) for s, a in u.items()}
    hist = torch.zeros(n_slots, max(C * (taps - 1), 1), dtype=torch.float32, device="cuda")
    at = {s: 0 for s in lengths}
    dev = lambda a: torch.tensor(a, dtype=torch.float32, device="cuda")
    for step in ([(3, 9), (0, 1)], [(0, 2), (2, 5), (3, 1)], [(3, 13), (0, 8)]):
        row_slot, seg = _segments(step, n_slots)
        src = np.concatenate([u[s][at[s]:at[s] + n] for s, n in step])
        want = np.concatenate([ref[s][at[s]:at[s] + n] for s, n in step])
        out = torch.empty(src.shape, dtype=torch.float32, device="cuda")
        kernels.causal_conv_silu(dev(src), dev(w), None, hist, out, row_slot, seg, activation=False)
        np.testing.assert_allclose(out.cpu().numpy(), want, rtol=1e-5, atol=1e-5)
        for s, n in step:
            at[s] += n


@pytest.mark.gpu
def test_norms_activations_and_router_kernels():
    from llmario_b200 import kernels

    rng = np.random.default_rng(5)
    dev = lambda a: torch.tensor(a, dtype=torch.float32, device="cuda")
    # half the sum of two normed rows
    for rows, width in ((3, 50), (70, 256), (2, 4100)):
        a, b = rng.standard_normal((rows, width)) * 3, rng.standard_normal((rows, width)) * 0.01
        wa, wb = rng.standard_normal(width), rng.standard_normal(width)
        ref = 0.5 * (PP.rms_unit(a, 1e-5) * wa + PP.rms_unit(b, 1e-5) * wb)
        y = torch.ones(rows, width, dtype=torch.float32, device="cuda")
        kernels.dual_norm_mean(dev(a), dev(b), dev(wa), dev(wb), y, 1e-5, accumulate=True)
        np.testing.assert_allclose(y.cpu().numpy() - 1.0, ref, rtol=1e-4, atol=1e-5)
        kernels.dual_norm_mean(dev(a), dev(b), dev(wa), dev(wb), y, 1e-5)
        np.testing.assert_allclose(y.cpu().numpy(), ref, rtol=1e-4, atol=1e-5)
    # the square of relu; the clamped gated activation
    x = rng.standard_normal((9, 34)) * 3
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-2)):
        out = torch.empty(9, 34, dtype=dtype, device="cuda")
        kernels.act_rows(dev(x), out, "relu_squared")
        np.testing.assert_allclose(out.float().cpu().numpy(), np.maximum(x, 0) ** 2, rtol=tol, atol=tol)
        gu = rng.standard_normal((9, 2 * 17)) * 3
        for limit in (0.5, 2.0, 7.0):
            g, u = np.minimum(gu[:, :17], limit), np.clip(gu[:, 17:], -limit, limit)
            out = torch.empty(9, 17, dtype=dtype, device="cuda")
            kernels.gated_act(dev(gu), None, out, "clamped_swish", limit=limit)
            np.testing.assert_allclose(out.float().cpu().numpy(), g * PP.sigmoid(1.702 * g) * (u + 1),
                                       rtol=max(tol, 1e-5), atol=max(tol, 1e-5) * 8)
    # scores over all router outputs, choice by corrected score, weights not renormalised
    for E, top in ((3, 1), (7, 3), (20, 3), (5, 5), (64, 8)):
        z = rng.standard_normal((50, E + 2)) * 2
        corr = rng.standard_normal(E) * 0.2
        t = {"r.router": np.eye(E), "r.correction": corr}
        chosen, wts = PP.route(z[:, :E], t, "r.", {"router": {"top": top}})
        ids = torch.empty(50, top, dtype=torch.int32, device="cuda")
        w_d = torch.empty(50, top, dtype=torch.float32, device="cuda")
        kernels.moe_route(dev(z)[:, :E], E, top, ids, w_d, scores="softmax_all", correction=dev(corr))
        assert np.array_equal(np.sort(ids.cpu().numpy(), 1), np.sort(chosen, 1))
        order = np.argsort(ids.cpu().numpy(), 1)
        got = np.take_along_axis(w_d.cpu().numpy(), order, 1)
        np.testing.assert_allclose(got, np.take_along_axis(wts, np.argsort(chosen, 1), 1), rtol=1e-5)


# --------------------------------------------------------------------------------------------
# whole models through the step function
# --------------------------------------------------------------------------------------------
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
    # 16-bit operands move the inputs of every layer by a rounding: see slack_for
    slack = slack_for(name, tokens, dtype, seed)
    assert_close(np.stack([got[p] for p in pos]), ref[pos], dtype, what,
                 slack=None if slack is None else slack[pos])


NAMES = sorted(CONFIGS)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompt(name, dtype):
    """Every position of a prompt that spans several pages, windows and pooled blocks, the first
    tokens included.  The configurations with one layer are one mechanism each."""
    toks = tokens_for(name, 110, 1)
    runner = runner_for(name, dtype)
    got = run_steps(runner, [[("a", toks, range(len(toks)))]])
    check_request(got["a"], name, toks, dtype, "whole prompt")
    runner.cache.check_invariants()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_single_tokens(name, dtype):
    """A prompt, then tokens one by one through recorded steps: across the borders of pages,
    windows and blocks, so that pooled entries are written by decoded tokens too."""
    toks = tokens_for(name, 90, 2)
    n = 21
    runner = runner_for(name, dtype)
    steps = [[("a", toks[:n], [0, n - 1])]] + [[("a", [t], [0])] for t in toks[n:]]
    got = run_steps(runner, steps)
    check_request(got["a"], name, toks, dtype, "prompt, then single tokens")
    assert runner.counters["graph_replays"] > 40


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_many_sizes(name, dtype):
    """Portions cut in the middle of pages, windows and blocks, down to two tokens; then single
    tokens."""
    toks = tokens_for(name, 120, 3)
    cuts = [2, 3, 2, 17, 2, 31, 5, 2, 29, 1, 2, 1, 1, 16, 2, 4]
    assert sum(cuts) == len(toks)
    steps, at = [], 0
    for c in cuts:
        steps.append([("a", toks[at:at + c], range(c))])
        at += c
    runner = runner_for(name, dtype)
    got = run_steps(runner, steps)
    check_request(got["a"], name, toks, dtype, "portions")
    # and the cut does not matter beyond rounding: the same prompt whole
    whole = run_steps(runner_for(name, dtype), [[("a", toks, range(len(toks)))]])
    a = np.stack([got["a"][p] for p in range(len(toks))])
    b = np.stack([whole["a"][p] for p in range(len(toks))])
    assert_close(a, b.astype(np.float64), dtype, "portions against whole",
                 1e-5 if dtype == "float32" else 2e-2, slack=slack_for(name, toks, dtype))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ("mix", "shared", "odd", "par_big_pool", "par_pool1", "attn_keep",
                                  "wide_heads"))
def test_mixed_batches_and_reused_slots(name, dtype):
    """Four request slots, six requests of unequal lengths: portions of some beside single tokens
    of others, requests that pause, requests that end and whose slot and pages the next one
    takes (the recurrent state, the convolution's inputs and the pooled entries with them).
    Every request must get what it gets alone (the plain implementation's logits)."""
    lengths = {"a": 70, "b": 9, "c": 41, "d": 33, "e": 52, "f": 2}
    toks = {r: tokens_for(name, n, 10 + i) for i, (r, n) in enumerate(lengths.items())}
    runner = runner_for(name, dtype, page_size=8, cache_tokens=208, max_requests=4)
    at = {r: 0 for r in toks}

    def take(r, n):
        n = min(n, lengths[r] - at[r])
        part = toks[r][at[r]:at[r] + n]
        at[r] += n
        return (r, part, range(n))

    plan = [[("a", 30), ("b", 2)], [("a", 1), ("b", 1), ("c", 17)], [("b", 6), ("c", 1), ("d", 2)],
            [("a", 1), ("c", 23), ("d", 1)], [("a", 38)], [("d", 30), ("e", 3)],
            [("e", 1), ("f", 2)], [("e", 48)]]
    got = {}
    for step in plan:
        entries = [take(r, n) for r, n in step]
        for r, res in run_steps(runner, [entries]).items():
            got.setdefault(r, {}).update(res)
        for r, _ in step:
            if at[r] == lengths[r]:
                runner.close(r)
        runner.cache.check_invariants()
    assert all(at[r] == lengths[r] for r in toks)
    for r in toks:
        assert sorted(got[r]) == list(range(lengths[r]))
        check_request(got[r], name, toks[r], dtype, f"request {r}", seed=0)
    assert runner.cache.free_slots() == 4


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ("mix", "shared", "par"))
def test_a_long_prompt_over_many_windows_and_the_engine_page(name, dtype):
    """A prompt of several hundred tokens with the engine's default page of 64 (pages behind the
    windows go back while the kept first keys and the pooled entries stay), then a second portion
    that starts inside a window and a page, then single tokens."""
    toks = tokens_for(name, 420, 6)
    runner = runner_for(name, dtype, page_size=64, cache_tokens=1024)
    steps = [[("a", toks[:333], range(333))], [("a", toks[333:410], range(77))]] \
        + [[("a", [t], [0])] for t in toks[410:]]
    got = run_steps(runner, steps)
    check_request(got["a"], name, toks, dtype, "long prompt")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_from_a_seed(seed, dtype):
    """Layers of any kind in any order with sizes drawn from a seed, the engine's page of 64:
    a prompt in portions, then single tokens, against the plain implementation."""
    name = random_config(seed)
    toks = tokens_for(name, 230, 7)
    runner = runner_for(name, dtype, page_size=64, cache_tokens=512)
    steps = [[("a", toks[:150], range(150))], [("a", toks[150:153], range(3))],
             [("a", toks[153:200], range(47))]] + [[("a", [t], [0])] for t in toks[200:]]
    got = run_steps(runner, steps)
    check_request(got["a"], name, toks, dtype, f"{name} {CONFIGS[name]['layers']}")


@pytest.mark.gpu
@pytest.mark.parametrize("name", ("mix", "par_vd", "shared"))
def test_long_decoding(name):
    """Hundreds of single tokens behind a one-token prompt: the state carries what no cache
    holds, windows and blocks pass over decoded tokens many times."""
    toks = tokens_for(name, 260, 4)
    runner = runner_for(name, "float32", page_size=32, cache_tokens=512)
    got = run_steps(runner, [[("a", [t], [0])] for t in toks])
    check_request(got["a"], name, toks, "float32", "long decoding")


# --------------------------------------------------------------------------------------------
# a key that stands out: the edges of windows, the kept first tokens, the pooled blocks, sinks
# --------------------------------------------------------------------------------------------
NEEDLE_CHANNEL = 20      # of head 0; behind the rotated channels
NEEDLE_KEEP, NEEDLE_POOL = 3, 4


def needle_model(kind: str, window: int, dim: int = 32) -> str:
    """One layer whose weights make one score stand out.  Token 0 is the needle: its embedding is
    large in coordinate 0, which only one key channel reads; token 1 is the probe, large in
    coordinate 1, which only the same query channel reads; the norms' weights of that channel
    are large.  No other token has either, so a probe's output is decided by whether it sees a
    needle (as a token, as a kept first token, or inside a pooled block), and an edge that is
    off by one shows as a large error.  The sinks are large enough to take visible weight.
    ``kind``: "needle_attn" (kept-window attention) or "needle_par" (pooled window attention
    beside a recurrence).  ``dim``: the head size (64 is one that the tensor-core kernels have, so
    in bfloat16 the keys outside the window are summed by a kernel of their own)."""
    name = f"{kind}{window}_{dim}"
    if name in CONFIGS:
        return name
    if kind == "needle_attn":
        CONFIGS[name] = config([attention(heads=2, kv_heads=1, dim=dim, vdim=dim, size=window,
                                          keep=NEEDLE_KEEP)], width=64, vocab=64)
        x = "l0.mix."
    else:
        CONFIGS[name] = config([parallel(width=16, heads=2, kv_heads=1, dim=dim, vdim=dim, conv=3,
                                         size=window, pool=NEEDLE_POOL, rot=8)], width=64, vocab=64)
        x = "l0.mix.left."
    w = {n: a.copy() for n, a in _weights(CONFIGS[name], 7).items()}
    w["embed"][:, :2] = 0.0
    w["embed"][0, 0] = 8.0
    w["embed"][1, 1] = 8.0
    c = NEEDLE_CHANNEL
    for m, col in (("q", 1), ("k", 0)):
        w[x + m] *= 0.5
        w[x + m][:, :2] = 0.0
        w[x + m][c, :] = 0.0
        w[x + m][c, col] = 2.0
        w[x + m + ".norm"][c] = 2.5
        if kind == "needle_par":
            w[x + m + ".conv"][c, :] = [0.0, 0.0, 1.0]     # the channel is not smeared over time
    w[x + "v"][:, 0] = np.linspace(-1.0, 1.0, w[x + "v"].shape[0])
    w[x + "sink"][:] = [2.0, 0.5]
    CUSTOM[name] = _bf16_values(w)
    return name


def needle_tokens(window: int, n: int, seed: int = 3, start: int = 9):
    """Tokens 2.. at random with needles (0) and probes (1) placed so that probes sit exactly
    ``window - 1`` (the last key inside) and ``window`` (the first outside) behind a needle.
    Needles stand on the first position of a block of NEEDLE_POOL, behind the kept tokens, so
    that the probe just outside sees neither the needle nor, yet, its block."""
    rng = np.random.default_rng(seed)
    toks = [int(t) for t in rng.integers(2, 64, n)]
    probes = {"just_inside": [], "just_outside": []}
    at = start
    while at + 2 * window + 2 * NEEDLE_POOL + 6 < n:
        at += -at % NEEDLE_POOL
        toks[at] = 0
        toks[at + window - 1] = 1
        probes["just_inside"].append(at + window - 1)
        at += window + 3
        at += -at % NEEDLE_POOL
        toks[at] = 0
        toks[at + window] = 1
        probes["just_outside"].append(at + window)
        at += window + 5
    return toks, probes


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ("needle_attn", "needle_par"))
@pytest.mark.parametrize("window,page,dim", [(12, 16, 32), (40, 16, 64), (64, 64, 32), (24, 32, 64),
                                             (33, 8, 64), (64, 64, 64)])
def test_a_key_that_stands_out_at_the_edges_of_windows(dtype, kind, window, page, dim):
    """Needles just inside and just outside the window of a probe, in a whole prompt, in
    portions whose cuts fall between needle and probe, and with the probes decoded one by one,
    over pages smaller than, equal to and larger than the window."""
    from llmario_b200 import driver
    name = needle_model(kind, window, dim)
    n = 6 * window + 70
    toks, probes = needle_tokens(window, n)
    assert len(probes["just_inside"]) >= 2 and len(probes["just_outside"]) >= 2
    before = driver.kernel_counts()["outside_window"]
    runner = runner_for(name, dtype, page_size=page, cache_tokens=1024)
    got = run_steps(runner, [[("a", toks, range(n))]])
    check_request(got["a"], name, toks, dtype, "needles, whole prompt")
    cuts, at = [], 0
    for c in [window - 1, 2, window + 1, 3, 2 * window - 1]:
        cuts.append((at, at + c))
        at += c
    steps = [[("b", toks[a:b], range(b - a))] for a, b in cuts] + [[("b", [t], [0])] for t in toks[at:]]
    got = run_steps(runner, steps)
    check_request(got["b"], name, toks, dtype, "needles, portions and single tokens")
    if dtype == "bfloat16":     # which kernels summed what lies outside the window
        assert (driver.kernel_counts()["outside_window"] > before) == (dim == 64)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("page,dim", ((8, 32), (64, 32), (8, 64), (32, 64)))
def test_kept_first_tokens_far_away(dtype, page, dim):
    """A needle on the last kept position is seen by probes hundreds of tokens later, one on
    the next position is not: in a prompt, in portions and decoded, while the pages between go
    back to the pool."""
    window = 16
    name = needle_model("needle_attn", window, dim)
    n = 300
    rng = np.random.default_rng(11)
    for needle_at in (NEEDLE_KEEP - 1, NEEDLE_KEEP, 0):
        toks = [int(t) for t in rng.integers(2, 64, n)]
        toks[needle_at] = 0
        where = [needle_at + window - 1, needle_at + window, 70, 128, 129, 250, 299]
        for p in where:
            toks[p] = 1
        ref = plain_logits(name, toks)
        # the plain statement says what the test is about: with one more kept token the probes
        # behind a needle on position `keep` see it
        more = json.loads(json.dumps(CONFIGS[name]))
        more["layers"][0]["mixer"]["mask"]["keep_first"] = NEEDLE_KEEP + 1
        moved = np.abs(PP.forward(more, weights(name), toks) - ref).max(axis=1)[where[2:]]
        if needle_at == NEEDLE_KEEP:
            assert moved.min() > 0.1 * np.abs(ref).max()
        else:
            assert moved.max() < 0.02 * np.abs(ref).max()
        runner = runner_for(name, dtype, page_size=page, cache_tokens=384, max_context=512)
        got = run_steps(runner, [[("a", toks[:200], range(200))], [("a", toks[200:240], range(40))]]
                        + [[("a", [t], [0])] for t in toks[240:]])
        check_request(got["a"], name, toks, dtype, f"needle at {needle_at}")
        runner.close("a")
        got = run_steps(runner, [[("b", toks[:2], range(2))]] + [[("b", [t], [0])] for t in toks[2:140]])
        check_request(got["b"], name, toks[:140], dtype, f"needle at {needle_at}, decoded")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("page,dim", ((8, 32), (64, 32), (16, 64), (64, 64)))
def test_pooled_blocks_just_seen_and_not_yet(dtype, page, dim):
    """A needle inside a block: the probe on the first position that sees the block finds it
    (weakened by the mean), the probe one position earlier sees neither token nor block; probes
    hundreds of tokens later still find the block."""
    window = 20
    P = NEEDLE_POOL
    name = needle_model("needle_par", window, dim)
    n = 330
    rng = np.random.default_rng(12)
    toks = [int(t) for t in rng.integers(2, 64, n)]
    needle_at = 5 * P + 1                      # inside block 5
    first_seen = 5 * P + P - 1 + window        # the first position that sees block 5
    toks[needle_at] = 0
    where = [first_seen - 1, first_seen, first_seen + 1, 150, 256, 329]
    for p in where:
        toks[p] = 1
    ref = plain_logits(name, toks)
    for delta, probe in ((1, first_seen), (-1, first_seen - 1)):
        off = json.loads(json.dumps(CONFIGS[name]))
        off["layers"][0]["mixer"]["left"]["mask"]["size"] = window + delta
        moved = np.abs(PP.forward(off, weights(name), toks) - ref).max(axis=1)
        assert moved[probe] > 0.05 * np.abs(ref).max(), (delta, moved[probe])
    runner = runner_for(name, dtype, page_size=page, cache_tokens=384, max_context=512)
    got = run_steps(runner, [[("a", toks, range(n))]])
    check_request(got["a"], name, toks, dtype, "pooled needle, whole prompt")
    runner.close("a")
    # cuts inside the needle's block, one token before the block is first seen, and on it
    cuts = [needle_at + 1, 2, first_seen - 1 - needle_at - 3, 1, 2, 100]
    steps, at = [], 0
    for c in cuts:
        steps.append([("b", toks[at:at + c], range(c))])
        at += c
    got = run_steps(runner, steps + [[("b", [t], [0])] for t in toks[at:]])
    check_request(got["b"], name, toks, dtype, "pooled needle, portions and single tokens")
    runner.close("b")
    # decoded from the second token on: the block's entry is written by a decoded token
    got = run_steps(runner, [[("c", toks[:1], [0])]] + [[("c", [t], [0])] for t in toks[1:160]])
    check_request(got["c"], name, toks[:160], dtype, "pooled needle, decoded")


# --------------------------------------------------------------------------------------------
# the engine's own entry point, the command line, the trace runner
# --------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_engine(dtype):
    """The engine's own entry point and scheduler: prompts of unequal lengths, more requests than
    slots, greedy tokens.  The plain implementation, reading the engine's sequence, must choose
    the same token wherever its two best logits are clearly apart."""
    from llmario_b200.engine.engine import Engine
    from llmario_b200.sampling import SamplingParams

    for name in ("mix", "shared"):
        eng = Engine(model_dir(name), dtype=dtype, page_size=16, cache_tokens=1024, max_requests=2,
                     token_budget=48, context=256)
        prompts = [tokens_for(name, n, 20 + i) for i, n in enumerate((5, 70, 33, 1, 18))]
        outs = eng.generate(prompts, SamplingParams.greedy_params(max_tokens=24, ignore_eos=True))
        margin = 1e-3 if dtype == "float32" else 8e-2
        clear = 0
        for p, o in zip(prompts, outs):
            assert len(o) == 24
            ref = plain_logits(name, list(p) + list(o))
            # (the engine chose these tokens: behind a router's close call in the sequence the
            # two computations may have gone different ways)
            close = np.nonzero(router_margins(name, list(p) + list(o)) < CLOSE_CALL)[0]
            until = int(close[0]) if len(close) and dtype == "bfloat16" else len(ref)
            for j, tok in enumerate(o):
                if len(p) - 1 + j >= until:
                    break
                l = ref[len(p) - 1 + j]
                top = np.sort(l)[-2:]
                if top[1] - top[0] > margin * np.abs(l).max():
                    clear += 1
                    assert tok == int(np.argmax(l)), f"{name}: token {j} of a request"
        assert clear > (60 if dtype == "float32" else 5)
        assert eng.stats()["graph_replays"] > 0
        eng.runner.cache.check_invariants()


@pytest.mark.gpu
def test_command_line_and_trace_runner(tmp_path):
    """The two programs a user starts: ``llmario-b200 run`` on a Pemolorn model folder (greedy ids
    against the plain implementation) and ``bin/trace_run`` (given tokens in steps, logits in
    files), which choose the model class by ``config.json``."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    name = "mix"
    prompt = tokens_for(name, 19, 40)
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "llmario-b200"), "run",
                        model_dir(name), "--tokens", ",".join(map(str, prompt)), "--max-tokens", "6",
                        "--dtype", "float32", "--page-size", "16", "--context", "128"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    out = [int(t) for t in p.stdout.strip().splitlines()[-1].split(",")]
    assert len(out) == 6
    ref = plain_logits(name, prompt + out)
    for j, tok in enumerate(out):
        l = ref[len(prompt) - 1 + j]
        top = np.sort(l)[-2:]
        if top[1] - top[0] > 1e-3 * np.abs(l).max():
            assert tok == int(np.argmax(l))
    # a preset name gives a model with random weights
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "llmario-b200"), "run", "pemolorn-tiny",
                        "--prompt-len", "5", "--n", "6", "--dtype", "bfloat16", "--page-size", "16",
                        "--context", "64"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert len(p.stdout.strip().splitlines()[-1].split(",")) == 6
    # the trace runner: three requests, portions beside single tokens, a slot given back and taken
    a, b, c = (tokens_for(name, n, 50 + i) for i, n in enumerate((40, 7, 12)))
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:25], "want": [0, 24]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[25:26], "want": [0]},
                                {"id": "b", "tokens": b, "want": [6]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": a[26:], "want": [13]},
                                {"id": "c", "tokens": c[:2], "want": []}], "end": ["a"]},
        {"step": 3, "entries": [{"id": "c", "tokens": c[2:], "want": [0, 9]}], "end": ["c"]},
    ]
    ra, rb, rc = plain_logits(name, a), plain_logits(name, b), plain_logits(name, c)
    want = {0: np.stack([ra[0], ra[24]]), 1: np.stack([ra[25], rb[6]]), 2: ra[39:40],
            3: np.stack([rc[2], rc[11]])}
    for dtype in DTYPES:
        out_dir = tmp_path / dtype
        p = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", model_dir(name),
                            "--dtype", dtype, "--out", str(out_dir), "--max-tokens", "192"],
                           input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True,
                           text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
        for i, ref in want.items():
            got = np.fromfile(out_dir / f"{i}.f32", dtype="<f4").reshape(ref.shape)
            if dtype == "float32":
                assert_close(got, ref, dtype, f"trace step {i}")
            else:
                assert np.abs(got - ref).max() < 0.15 * np.abs(ref).max()
