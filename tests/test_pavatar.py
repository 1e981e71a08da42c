"""The Pavatar decoder against the plain float64 implementation (tests/plain/pavatar_plain.py):
every mechanism alone and together, in whole prompts, portions, single decoded tokens, mixed
batches, reused slots and pages, and through the engine's own entry point."""
from __future__ import annotations

import json

import numpy as np
import pytest
import torch

from plain import pavatar_plain as PP
from pavatar_util import (CLOSE_CALL, CONFIGS, CUSTOM, _bf16_values, _weights, assert_close,
                          attention, check_request, close_calls, config, delta, delta_sizes,
                          model_dir, moe, parallel, plain_logits, random_config, run_steps,
                          runner_for, slack_for, tokens_for, weights)

DTYPES = ("float32", "bfloat16")


# --------------------------------------------------------------------------------------------
# no GPU: configuration, and the plain implementation against itself
# --------------------------------------------------------------------------------------------
def test_configuration_round_trip_and_tensor_names():
    from llmario_b200.config import ConfigError, PavatarConfig, resolve_architecture
    from llmario_b200.weights.loader import check_tensors, expected_tensors

    for name, raw in CONFIGS.items():
        assert resolve_architecture(raw) == "Pavatar"
        cfg = PavatarConfig.from_dict(raw)
        assert PavatarConfig.from_dict(cfg.to_dict()) == cfg
        assert cfg.to_dict() == raw, name
        spec = cfg.to_spec()
        want = expected_tensors(spec)
        have = {n: a.shape for n, a in weights(name).items()}
        assert set(want) == set(have), name
        check_tensors(spec, have)
        kinds = {"attention": "attention", "delta": "gated_delta", "parallel": "parallel"}
        for layer, entry in zip(spec.layers, raw["layers"]):
            assert layer.mixer.kind == kinds[entry["type"]]
            assert layer.block.kind == "shared_norm_residual"
            assert (layer.feed_forward.kind == "none") == (entry["mlp"] is None)
        assert spec.head["tied"] and spec.head["tensors"]["weight"][0] == "embed"
    # the first layer that blends values is their source, the others read it
    spec = PavatarConfig.from_dict(CONFIGS["attn_blend"]).to_spec()
    blends = [l.mixer.get("value_blend") for l in spec.layers]
    assert blends[1] is None and [b["source"] for b in blends if b] == [True, False, False]
    # the rank of the low-rank factors is the stored tensors' when the configuration is silent
    raw = json.loads(json.dumps(CONFIGS["par"]))
    del raw["layers"][0]["mixer"]["right"]["rank"]
    t = PavatarConfig.from_dict(raw).to_spec().layers[0].mixer["right"]["tensors"]
    assert t["a1"][1][0] is None and t["g2"][1][1] is None

    def broken(name, change):
        bad = json.loads(json.dumps(CONFIGS[name]))
        change(bad)
        return bad

    with pytest.raises(ConfigError, match="unsupported type"):
        PavatarConfig.from_dict(broken("mix", lambda c: c["layers"][0].update(type="conv")))
    with pytest.raises(ConfigError, match="mlp kind"):
        PavatarConfig.from_dict(broken("mix", lambda c: c["layers"][0]["mlp"].update(kind="x")))
    with pytest.raises(ConfigError, match="top"):
        PavatarConfig.from_dict(
            broken("delta", lambda c: c["layers"][0]["mlp"]["router"].update(top=9)))
    with pytest.raises(ConfigError, match="eps"):
        PavatarConfig.from_dict(broken("par", lambda c: c.pop("norm")))
    with pytest.raises(ConfigError, match="dims"):
        PavatarConfig.from_dict(
            broken("par", lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7)))
    with pytest.raises(ConfigError, match="v_mix"):
        PavatarConfig.from_dict(
            broken("attn_blend", lambda c: c["layers"][2]["mixer"].update(vdim=8)))
    with pytest.raises(ConfigError, match="key heads"):
        PavatarConfig.from_dict(broken("delta", lambda c: c["layers"][0]["mixer"].update(heads=5)))


def test_plain_mechanisms_against_their_definitions():
    rng = np.random.default_rng(0)
    # the short convolution is a correlation with the taps, newest input under the last tap
    u, w = rng.standard_normal((9, 3)), rng.standard_normal((3, 4))
    y = PP.short_conv(u, w)
    for c in range(3):
        np.testing.assert_allclose(y[:, c], np.convolve(u[:, c], w[c, ::-1])[:9], atol=1e-12)
    assert np.allclose(PP.short_conv(u, w[:, 3:]), u * w[:, 3])
    # the rotation keeps lengths, leaves the channels behind `dims` alone, pairs i with
    # i + dims/2, and makes a score a function of the distance
    x = rng.standard_normal((1, 1, 12))
    a = PP.rotate_halves(np.repeat(x, 6, 0), np.arange(6), 8, 100.0)
    assert np.allclose(np.linalg.norm(a, axis=-1), np.linalg.norm(x)) and np.allclose(a[:, :, 8:], x[:, :, 8:])
    b = PP.rotate_halves(np.repeat(x, 6, 0), np.arange(6) + 11, 8, 100.0)
    assert np.allclose(a[1, 0, :8] @ a[4, 0, :8], b[1, 0, :8] @ b[4, 0, :8])
    assert np.allclose(a[0], x[0])
    one = np.zeros((1, 1, 8))
    one[0, 0, 1] = 1.0
    turned = PP.rotate_halves(one, np.array([1]), 8, 100.0)[0, 0]
    assert np.isclose(turned[1], np.cos(100.0 ** -0.25)) and np.isclose(turned[5], np.sin(100.0 ** -0.25))
    assert np.count_nonzero(turned) == 2
    # the temperature steps where (p + 1) / every reaches the next whole number
    f = PP.query_temperature(np.arange(30), 0.5, 8)
    assert np.allclose(f[:7], 1.0) and np.allclose(f[7:15], 1 + 0.5 * np.log(2)) and np.isclose(f[23], 1 + 0.5 * np.log(4))
    # the delta rule is a memory: with unit orthogonal keys, full strength and no decay a key
    # answers with the value last written to it, however many writes lie between
    d, dv = 6, 3
    k = np.eye(d)[[0, 1, 2, 0, 3]][:, None, :]
    v = rng.standard_normal((5, 1, dv))
    o = PP.delta_rule(k, k, v, np.ones((5, 1)), np.ones((5, 1, d)))
    np.testing.assert_allclose(o, v, atol=1e-12)
    q = np.eye(d)[[0, 0, 0, 1, 0]][:, None, :]
    o = PP.delta_rule(q, k, v, np.ones((5, 1)), np.ones((5, 1, d)))
    np.testing.assert_allclose(o[:, 0], [v[0, 0], v[0, 0], v[0, 0], v[1, 0], v[3, 0]], atol=1e-12)
    # half strength moves the stored value half of the way; a decay fades it per channel
    o = PP.delta_rule(q, k, v, np.full((5, 1), 0.5), np.ones((5, 1, d)))
    np.testing.assert_allclose(o[4, 0], 0.5 * (0.5 * v[0, 0]) + 0.5 * v[3, 0], atol=1e-12)
    fade = np.ones((5, 1, d))
    fade[:, :, 0] = 0.5
    o = PP.delta_rule(q, k, v, np.ones((5, 1)), fade)
    np.testing.assert_allclose(o[2, 0], 0.25 * v[0, 0], atol=1e-12)
    # the router: choice by corrected score, weights the plain scores of the chosen, renormed
    z = np.array([[2.0, 1.0, 0.0, 1.0]])
    s = np.exp(z[0]) / np.exp(z[0]).sum()
    ids, w = PP.route(z, np.array([0.0, 0.0, 10.0, 0.0]), 2, 3.0)
    assert ids.tolist() == [[2, 0]] and np.allclose(w, 3.0 * s[[2, 0]] / s[[2, 0]].sum())
    ids, w = PP.route(z, np.zeros(4), 2, 1.0)
    assert ids.tolist() == [[0, 1]] and np.isclose(w.sum(), 1.0)      # the lower index of equals


def test_plain_edges_matter():
    """The plain statement itself: the blended values, the temperature's steps, the state of the
    recurrence and the first tokens all move the logits of the models used below."""
    toks = tokens_for("attn_blend", 40, 1)
    ref = plain_logits("attn_blend", toks)
    size = np.abs(ref).max()
    raw = json.loads(json.dumps(CONFIGS["attn_blend"]))
    raw["layers"][2]["mixer"].pop("v_mix")
    assert np.abs(PP.forward(raw, weights("attn_blend"), toks) - ref).max() > 0.05 * size
    raw = json.loads(json.dumps(CONFIGS["attn_blend"]))
    raw["layers"][2]["mixer"]["q_temp"]["every"] = 14      # the first step one token later
    moved = np.abs(PP.forward(raw, weights("attn_blend"), toks) - ref).max(axis=1)
    assert moved[:12].max() == 0 and moved[12] > 0.002 * size and moved[13] > 0
    # a token far back is remembered by the recurrence alone
    toks = tokens_for("delta_shared", 200, 2)
    ref = plain_logits("delta_shared", toks)
    other = list(toks)
    other[3] = (other[3] + 1) % CONFIGS["delta_shared"]["vocab"]
    diff = np.abs(plain_logits("delta_shared", other) - ref).max(axis=1)
    assert diff[150:].max() > 0.002 * np.abs(ref).max()


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
@pytest.mark.parametrize("per_channel", (False, True))
@pytest.mark.parametrize("grouped", (False, True))
@pytest.mark.parametrize("H,G,K,V", [(2, 1, 8, 5), (3, 3, 24, 16), (4, 2, 64, 32), (2, 2, 100, 33),
                                     (6, 2, 128, 64), (1, 1, 136, 24), (2, 1, 256, 20),
                                     (3, 1, 68, 17), (1, 1, 320, 130)])
def test_delta_rule_kernel(H, G, K, V, per_channel, grouped):
    """Steps of unequal requests with the state carried in the slots, then single tokens; unit
    vectors and the scale of q made by the kernel; both ways to make the decay; token by token
    and (``grouped``, where the kernels have that form) four tokens at a time."""
    from llmario_b200 import kernels

    rng = np.random.default_rng(K + V)
    n_slots = 5
    state = torch.zeros(n_slots, H * V * K + 7, device="cuda")
    plans = [[(2, 5), (0, 1), (3, 19)], [(3, 2), (2, 40)], None, [(0, 3), (4, 1), (2, 2)], None]
    hist = {s: [] for s in range(n_slots)}      # per slot: (q, k, v, d, beta) of its tokens so far
    rate_log = rng.standard_normal(H) - 2.0
    bias = rng.standard_normal(H * K if per_channel else H)
    for plan in plans:
        single = plan is None
        if single:
            plan = [(1, 1), (3, 1), (0, 1)]
        rows = sum(n for _, n in plan)
        q, k = rng.standard_normal((rows, G * K)), rng.standard_normal((rows, G * K))
        v = rng.standard_normal((rows, H * V))
        z = rng.standard_normal((rows, H * K if per_channel else H))
        beta = rng.standard_normal((rows, H)) * 2
        dev = lambda a: torch.tensor(a, dtype=torch.float32, device="cuda")
        row_slot, seg = _segments(plan, n_slots)
        out = torch.empty(rows, H * V, device="cuda")
        work = None
        if grouped and kernels.delta_work_floats(rows, H, K):
            work = torch.full((kernels.delta_work_floats(rows, H, K),), float("nan"), device="cuda")
        if per_channel:
            d = dev(z)
            kernels.rate_decay(d, dev(rate_log), dev(bias), K)
            kernels.delta_recurrence(dev(q), dev(k), dev(v), d, dev(beta), state, out, row_slot,
                                     None if single else seg, H, G, K, V, kernels.DECAY_VECTOR,
                                     q_scale=K ** -0.5, unit_floor=1e-6, n_requests=len(plan), work=work)
        else:
            kernels.delta_recurrence(dev(q), dev(k), dev(v), dev(z), dev(beta), state, out, row_slot,
                                     None if single else seg, H, G, K, V, kernels.DECAY_RATE_STEP,
                                     q_scale=K ** -0.5, unit_floor=1e-6, rate_log=dev(rate_log),
                                     step_bias=dev(bias), n_requests=len(plan), work=work)
        got = out.cpu().numpy().astype(np.float64)
        r0 = 0
        for s, n in plan:
            hist[s].append(tuple(a[r0:r0 + n] for a in (q, k, v, z, beta)))
            qs, ks, vs, zs, bs = (np.concatenate([h[i] for h in hist[s]]) for i in range(5))
            T = len(qs)
            f32 = lambda a: a.astype(np.float32).astype(np.float64)
            qh = np.repeat(PP.unit_heads(f32(qs).reshape(T, G, K)) * K ** -0.5, H // G, axis=1)
            kh = np.repeat(PP.unit_heads(f32(ks).reshape(T, G, K)), H // G, axis=1)
            rate = np.exp(f32(rate_log))
            if per_channel:
                decay = np.exp(-rate[None, :, None] * PP.softplus((f32(zs) + f32(bias)).reshape(T, H, K)))
            else:
                decay = np.repeat(np.exp(-rate * PP.softplus(f32(zs) + f32(bias)))[:, :, None], K, axis=2)
            ref = PP.delta_rule(qh, kh, f32(vs).reshape(T, H, V), PP.sigmoid(f32(bs)), decay)
            np.testing.assert_allclose(got[r0:r0 + n], ref[T - n:].reshape(n, H * V), atol=3e-5,
                                       err_msg=f"slot {s}")
            r0 += n
    assert float(state[:, H * V * K:].abs().max()) == 0.0      # nothing written behind the matrices


@pytest.mark.gpu
def test_delta_rule_kernel_without_unit_vectors():
    from llmario_b200 import kernels

    rng = np.random.default_rng(5)
    H, K, V, T = 2, 16, 8, 11
    q, k = rng.standard_normal((T, H * K)) * 0.3, rng.standard_normal((T, H * K)) * 0.3
    v, d = rng.standard_normal((T, H * V)), rng.uniform(0.5, 1.0, (T, H * K))
    beta = rng.standard_normal((T, H))
    dev = lambda a: torch.tensor(a, dtype=torch.float32, device="cuda")
    state = torch.zeros(1, H * V * K, device="cuda")
    row_slot, seg = _segments([(0, T)], 1)
    out = torch.empty(T, H * V, device="cuda")
    kernels.delta_recurrence(dev(q), dev(k), dev(v), dev(d), dev(beta), state, out, row_slot, seg,
                             H, H, K, V, kernels.DECAY_VECTOR, q_scale=2.0, n_requests=1)
    ref = PP.delta_rule(2.0 * q.reshape(T, H, K), k.reshape(T, H, K), v.reshape(T, H, V),
                        PP.sigmoid(beta), d.reshape(T, H, K))
    np.testing.assert_allclose(out.cpu().numpy(), ref.reshape(T, H * V), atol=2e-5)


@pytest.mark.gpu
def test_gates_store_and_router_kernels():
    from llmario_b200 import kernels

    rng = np.random.default_rng(1)
    dev = lambda a, dt=torch.float32: torch.tensor(a, device="cuda").to(dt)
    # a sigmoid gate per channel, on a column slice of a wider matrix
    for rows, cols in ((3, 7), (40, 96), (5, 1000)):
        o, wide = rng.standard_normal((rows, cols)), rng.standard_normal((rows, cols + 9))
        for dt, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-2)):
            out = dev(o, dt)
            kernels.channel_gate(out, dev(wide)[:, 4:4 + cols])
            ref = out.new_tensor(o).to(dt).double().cpu().numpy() * PP.sigmoid(
                dev(wide).double().cpu().numpy()[:, 4:4 + cols])
            np.testing.assert_allclose(out.double().cpu().numpy(), ref, atol=tol, rtol=tol)
    # the group norm behind a recurrence with a sigmoid in the place of silu
    rows, heads, V = 6, 3, 20
    o, g, w = rng.standard_normal((rows, heads * V)), rng.standard_normal((rows, heads * V)), rng.standard_normal(V)
    for act, fn in (("sigmoid", PP.sigmoid), ("silu", PP.silu)):
        out = torch.empty(rows, heads * V, device="cuda")
        kernels.gated_group_norm(dev(o), dev(g), dev(w), out, group=V, eps=1e-5, gate_first=False,
                                 gate_activation=act)
        ref = (PP.rms_unit(o.reshape(rows, heads, V), 1e-5) * w).reshape(rows, -1) * fn(g)
        np.testing.assert_allclose(out.cpu().numpy(), ref, atol=1e-5)
    # the embedding's scale
    table, toks = rng.standard_normal((9, 12)), torch.tensor([3, 0, 8], dtype=torch.int32, device="cuda")
    x, err = torch.empty(3, 12, device="cuda"), torch.zeros(1, dtype=torch.int32, device="cuda")
    kernels.embed(toks, dev(table), x, err, 16.0)
    np.testing.assert_allclose(x.cpu().numpy(), 16.0 * table[[3, 0, 8]].astype(np.float32), rtol=1e-6)
    # the router: scores over all, choice by corrected score, renormed weights times a scale;
    # equal scores go to the lower index
    for E, top, width in ((4, 2, 16), (17, 6, 40), (3, 3, 8), (12, 4, 256), (70, 1, 64)):
        h = rng.standard_normal((33, width))
        wr, corr = rng.standard_normal((E, width)), rng.standard_normal(E) * 0.1
        h[5] = 0.0                                        # all scores equal
        z = torch.empty(33, E, device="cuda")
        ids = torch.empty(33, top, dtype=torch.int32, device="cuda")
        wts = torch.empty(33, top, device="cuda")
        kernels.moe_router(dev(h), dev(wr), None, E, top, z, ids, wts, "softmax_all_renormed",
                           dev(corr), 2.5)
        f32 = lambda a: a.astype(np.float32).astype(np.float64)
        rid, rw = PP.route(f32(h) @ f32(wr).T, f32(corr), top, 2.5)
        safe = np.ones(33, bool)        # rows whose choice does not hang on the last bits
        sc = np.sort(PP.route(f32(h) @ f32(wr).T, f32(corr), E, 1.0)[1] / 1.0, axis=-1)
        got_ids = ids.cpu().numpy()
        for r in range(33):
            if sorted(got_ids[r]) != sorted(rid[r]):
                safe[r] = False
        assert safe.mean() > 0.9 and safe[5]
        order = np.argsort(got_ids, axis=1)
        ref_order = np.argsort(rid, axis=1)
        got_w = np.take_along_axis(wts.cpu().numpy(), order, 1)
        ref_w = np.take_along_axis(rw, ref_order, 1)
        np.testing.assert_allclose(got_w[safe], ref_w[safe], rtol=2e-4, atol=1e-6)
        assert np.allclose(wts.cpu().numpy()[safe].sum(axis=1), 2.5, rtol=1e-5)
        z2 = z.clone()
        kernels.moe_route(z2, E, top, ids, wts, "softmax_all_renormed", dev(corr), 2.5)
        assert sorted(ids.cpu().numpy()[5].tolist()) == sorted(rid[5].tolist())
    # experts without a gate, row by row
    E, ff, width, top = 3, 10, 24, 2
    h, up = rng.standard_normal((4, width)), rng.standard_normal((E, ff, width))
    ids = torch.tensor([[0, 2], [1, 0], [2, 1], [0, 1]], dtype=torch.int32, device="cuda")
    act = torch.empty(4, top, ff, device="cuda")
    kernels.moe_gate_up_rows(dev(h), dev(up), ids, act, "relu_squared")
    ref = np.stack([[np.maximum(up[e] @ h[r], 0) ** 2 for e in row] for r, row in enumerate(ids.cpu().numpy())])
    np.testing.assert_allclose(act.cpu().numpy(), ref, rtol=1e-4, atol=1e-5)


# --------------------------------------------------------------------------------------------
# whole models through the step function
# --------------------------------------------------------------------------------------------
NAMES = sorted(CONFIGS)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompt(name, dtype):
    """Every position of a prompt that spans several pages and steps of the temperature, the
    first tokens included.  The configurations with one layer are one mechanism each."""
    toks = tokens_for(name, 110, 1)
    runner = runner_for(name, dtype)
    got = run_steps(runner, [[("a", toks, range(len(toks)))]])
    check_request(got["a"], name, toks, dtype, "whole prompt")
    runner.cache.check_invariants()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_single_tokens(name, dtype):
    """A prompt, then tokens one by one through recorded steps: across the borders of pages and
    the temperature's steps, the state and the convolution's inputs carried from step to step."""
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
    """Portions cut in the middle of pages and of the convolution's reach, down to two tokens;
    then single tokens."""
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
@pytest.mark.parametrize("name", ("mix", "odd", "delta_taps", "delta_wide", "attn_blend", "par_vd",
                                  "wide_heads"))
def test_mixed_batches_and_reused_slots(name, dtype):
    """Four request slots, six requests of unequal lengths: portions of some beside single tokens
    of others, requests that pause, requests that end and whose slot and pages the next one
    takes (the recurrent state and the convolution's inputs with them).  Every request must get
    what it gets alone (the plain implementation's logits)."""
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
@pytest.mark.parametrize("name", ("mix", "attn_blend", "par"))
def test_a_long_prompt_and_the_engine_page(name, dtype):
    """A prompt of several hundred tokens with the engine's default page of 64, then a second
    portion that starts inside a page, then single tokens."""
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
@pytest.mark.parametrize("name", ("mix", "delta_shared", "par_norot"))
def test_long_decoding(name):
    """Hundreds of single tokens behind a one-token prompt: the state carries what no cache
    holds."""
    toks = tokens_for(name, 260, 4)
    runner = runner_for(name, "float32", page_size=32, cache_tokens=512)
    got = run_steps(runner, [[("a", [t], [0])] for t in toks])
    check_request(got["a"], name, toks, "float32", "long decoding")


# --------------------------------------------------------------------------------------------
# a key that stands out among hundreds, and a write that the recurrence must keep
# --------------------------------------------------------------------------------------------
NEEDLE, ASKER = 5, 9


def needle_model(kind: str, dim: int) -> str:
    """One layer whose head 0 is made so that the asking token's query meets the needle token's
    key with a score far above every other (the layer reads the embedding through its norm, so
    both are functions of the token alone), and the needle's value is large.  ``kind``:
    ``attention`` (no rotation; temperature steps every 50 tokens) or ``parallel`` (the marked
    channel lies behind the rotated ones)."""
    name = f"needle_{kind}_{dim}"
    if name in CONFIGS:
        return name
    if kind == "attention":
        layer = attention(heads=4, kv_heads=2, dim=dim, vdim=dim, every=50, coef=0.3, scale=1.0)
        x = "l0.mix."
    else:
        layer = parallel(heads=4, kv_heads=2, dim=dim, vdim=dim, rot=dim // 2, scale=1.0,
                         right=delta_sizes(heads=2, kv_heads=1, dim=16, vdim=16, conv=2, rank=4))
        x = "l0.mix.left."
    CONFIGS[name] = cfg = config([layer], width=64, vocab=40, embed_scale=2.0)
    w = dict(_weights(cfg, 11))
    eps = cfg["norm"]["eps"]
    h = PP.rms_norm(w["embed"] * 2.0, w["l0.norm1"], eps)
    mark = dim - 3
    for r, tok, gain in (("q", ASKER, 9.0), ("k", NEEDLE, 9.0)):
        m = w[x + r].copy()
        m[:dim] *= 0.05                              # head 0 hears little else
        m[mark] = gain * h[tok] / (h[tok] @ h[tok])
        w[x + r] = m
        if kind == "attention":
            w[x + r + ".b"] = w[x + r + ".b"] * 0.05
        else:
            w[x + r + ".norm"] = np.ones(dim)
    w[x + "v"][:dim] += 4.0 * np.outer(np.ones(dim), h[NEEDLE] / (h[NEEDLE] @ h[NEEDLE]))
    CUSTOM[name] = _bf16_values(w)
    return name


def needle_tokens(n: int, needle_at: int, askers: list, seed: int = 3):
    rng = np.random.default_rng(seed)
    toks = [int(t) for t in rng.integers(10, 40, n)]        # neither the needle nor the asker
    toks[needle_at] = NEEDLE
    for p in askers:
        toks[p] = ASKER
    return toks


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ("attention", "parallel"))
@pytest.mark.parametrize("page,dim,needle_at", [(8, 32, 7), (8, 32, 8), (64, 32, 63), (64, 64, 64),
                                                (16, 64, 0), (32, 64, 31), (64, 128, 1), (16, 128, 47)])
def test_a_key_far_back_among_hundreds(dtype, kind, page, dim, needle_at):
    """The needle stands on the last or the first place of a page (or at the very start); the
    asking token comes hundreds of tokens later, in the prompt, in a later portion, and
    decoded.  Leaving the needle out moves the asker's logits by a large part of their size."""
    name = needle_model(kind, dim)
    n = 330
    askers = [needle_at + 1, 200, 297, 310, 325]
    toks = needle_tokens(n, needle_at, askers)
    ref = plain_logits(name, toks)
    without = list(toks)
    without[needle_at] = 11
    gone = plain_logits(name, without)
    for p in askers:      # (one of four heads, beside a recurrence and behind a norm, in `parallel`)
        assert np.abs(gone[p] - ref[p]).max() > (0.2 if kind == "attention" else 0.04) * np.abs(ref[p]).max(), p
    runner = runner_for(name, dtype, page_size=page, cache_tokens=512)
    steps = [[("a", toks[:290], range(290))], [("a", toks[290:305], range(15))]] \
        + [[("a", [t], [0])] for t in toks[305:]]
    got = run_steps(runner, steps)
    check_request(got["a"], name, toks, dtype, "needle")
    # the kernels that ran: the tensor-core ones where the head size has them
    from llmario_b200 import driver

    view = runner.cache.view(0)
    assert driver.tensor_core_attention(runner.model.dtype, view, 4, 2, dim) == \
        (dtype == "bfloat16" and dim in (64, 128))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_the_recurrence_keeps_a_write_for_hundreds_of_tokens(dtype):
    """Rates of a thousandth a token: what the first tokens wrote is read 400 tokens later, in a
    prompt's portion and decoded, and a request that takes over a used slot starts from zero."""
    name = "delta_slow"
    if name not in CONFIGS:
        CONFIGS[name] = cfg = config([delta(heads=2, kv_heads=1, dim=32, vdim=16, conv=2),
                                      parallel(heads=2, kv_heads=1, dim=32, vdim=32, rot=8,
                                               right=delta_sizes(heads=2, kv_heads=2, dim=16, vdim=24,
                                                                 conv=3, rank=4))], vocab=50)
        w = dict(_weights(cfg, 5))
        w["l0.mix.A_log"] = np.full(2, -7.0)
        w["l1.mix.right.A_log"] = np.full(2, -6.5)
        CUSTOM[name] = _bf16_values(w)
    toks = tokens_for(name, 440, 8)
    ref = plain_logits(name, toks)
    other = list(toks)
    other[2] = (other[2] + 7) % 50
    moved = np.abs(plain_logits(name, other) - ref).max(axis=1)
    assert moved[400:].min() > (2e-3 if dtype == "float32" else 0.0) * np.abs(ref).max()
    runner = runner_for(name, dtype, page_size=64, cache_tokens=1024, max_requests=1)
    steps = [[("a", toks[:300], [0, 1, 2, 299])], [("a", toks[300:420], range(120))]] \
        + [[("a", [t], [0])] for t in toks[420:]]
    got = run_steps(runner, steps)
    check_request(got["a"], name, toks, dtype, "slow rates")
    runner.close("a")
    short = tokens_for(name, 30, 9)
    got = run_steps(runner, [[("b", short[:7], range(7))]] + [[("b", [t], [0])] for t in short[7:]])
    check_request(got["b"], name, short, dtype, "the slot's next request")


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

    for name in ("mix", "attn_blend"):
        eng = Engine(model_dir(name), dtype=dtype, page_size=16, cache_tokens=1024, max_requests=2,
                     token_budget=48, context=256)
        prompts = [tokens_for(name, n, 20 + i) for i, n in enumerate((5, 70, 33, 1, 18))]
        outs = eng.generate(prompts, SamplingParams.greedy_params(max_tokens=24, ignore_eos=True))
        margin = 1e-3 if dtype == "float32" else 8e-2
        clear = 0
        for p, o in zip(prompts, outs):
            assert len(o) == 24
            ref = plain_logits(name, list(p) + list(o))
            # (where a router makes a close call the two computations may have run different
            # experts)
            close = close_calls(name, list(p) + list(o))
            for j, tok in enumerate(o):
                if dtype == "bfloat16" and close[len(p) - 1 + j]:
                    continue
                l = ref[len(p) - 1 + j]
                top = np.sort(l)[-2:]
                if top[1] - top[0] > margin * np.abs(l).max():
                    clear += 1
                    assert tok == int(np.argmax(l)), f"{name}: token {j} of a request"
        assert clear > (60 if dtype == "float32" else 20)
        assert eng.stats()["graph_replays"] > 0
        eng.runner.cache.check_invariants()


@pytest.mark.gpu
def test_command_line_and_trace_runner(tmp_path):
    """The two programs a user starts: ``llmario-b200 run`` on a Pavatar model folder (greedy ids
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
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "llmario-b200"), "run", "pavatar-tiny",
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
