"""Pavatar beside Pemolorn (the closest of the other designs: an attention beside a recurrence,
routed experts chosen by corrected scores) and Qwen3 at equal sizes: prompt and decode rates of
whole models with random weights, and the design's own kernels one by one against the memory
roofline, each beside the like kernel of another design.

    python -m llmario_b200.benchmarks.pavatar [--sizes 0.6b,8b] [--layers 8] [--kernels]

A Pavatar model of a size has the width, attention heads and number of layers of the Qwen3
preset of that name; its layers repeat (gated delta rule, attention with blended values,
attention beside a gated delta rule, attention), each with eight experts of half the
feed-forward width of which a token uses two (``config.pavatar.sized_like``), so a prompt does
the feed-forward work of the dense layer and a decode step of few rows streams up to all
experts.  ``bench.py --workload pavatar`` prints the same record as its JSON line.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Any, Dict, List

from .pemolorn import _View, pemolorn_config
from .vunasun import SIZES, _rates, _time


def pavatar_config(preset: Dict[str, Any], layers: int, vocab: int = 32768):
    """The Pavatar configuration with the sizes of a Qwen3 preset."""
    from ..config.pavatar import sized_like

    return sized_like(preset["hidden_size"], preset["intermediate_size"],
                      preset["num_attention_heads"], preset["num_key_value_heads"],
                      preset["head_dim"], layers, vocab)


def compare(sizes: List[str], layers: int, batch: int = 8, prompt_len: int = 1024,
            prefill_tokens: int = 2048, steps: int = 64, warmup: int = 24,
            page_size: int = 64) -> Dict[str, Any]:
    import torch

    from ..cli import PRESETS
    from ..engine.model import Model
    from .roofline import peaks

    pk = peaks()
    out: Dict[str, Any] = {}
    for size in sizes:
        preset = dict(PRESETS[SIZES[size]], vocab_size=32768)
        rec: Dict[str, Any] = {}
        for which in ("qwen3", "pemolorn", "pavatar"):
            if which == "qwen3":
                from ..config import Qwen3Config

                cfg = Qwen3Config.from_dict(dict(preset, num_hidden_layers=layers,
                                                 tie_word_embeddings=False,
                                                 architectures=["Qwen3ForCausalLM"]))
            elif which == "pemolorn":
                cfg = pemolorn_config(preset, layers)
            else:
                cfg = pavatar_config(preset, layers)
            model = Model.random(cfg, seed=0, dtype="bfloat16", device="cuda:0")
            r = _rates(model, page_size, batch, prompt_len, prefill_tokens, steps, warmup)
            # a decode step streams the weights once (all experts counted) and every live
            # request's recurrent state twice
            moved = r["weight_bytes"] + 2 * batch * r["state_bytes_per_request"]
            r["decode_frac_of_copy_peak"] = round(moved / (r["decode_ms"] / 1e3) / (pk["hbm_gbs"] * 1e9), 3)
            rec[which] = r
            del model
            torch.cuda.empty_cache()
        out[size] = rec
    return {"layers": layers, "batch": batch, "prompt_len": prompt_len,
            "prefill_tokens": prefill_tokens, "page_size": page_size, "peaks": pk["source"],
            "sizes": out}


def kernel_table(width: int = 4096, tokens: int = 2048, batch: int = 64, heads: int = 32,
                 kv_heads: int = 8, hd: int = 128, rank: int = 64, context: int = 4096
                 ) -> List[Dict[str, Any]]:
    """The design's own kernels, each alone at the sizes of ``pavatar_config`` for ``width``,
    with the bytes they must move and the fraction of the measured copy rate; beside each the
    like kernel of another design at the same sizes.  The prompt case is a portion of
    ``tokens`` rows of one request that ends at position ``context``; the decode case is
    ``batch`` requests at position ``context`` - 1."""
    import torch

    from .. import kernels
    from .roofline import peaks

    dev = "cuda:0"
    pk = peaks()
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=dev)
    rows_out: List[Dict[str, Any]] = []

    # 32-bit operations a second of the CUDA cores: 148 SMs x 128 lanes x 2 at 1,965 MHz (nominal)
    fp32_peak = 148 * 128 * 2 * 1.965e9

    def rec(name, us, nbytes, note="", flops=0):
        r = {"kernel": name, "us": round(us, 2), "bytes": int(nbytes),
             "gb_s": round(nbytes / us / 1e3, 1),
             "frac_of_copy_peak": round(nbytes / (us * 1e-6) / (pk["hbm_gbs"] * 1e9), 3),
             "note": note}
        if flops:
            r["fp32_tflops"] = round(flops / us / 1e6, 2)
            r["frac_of_fp32_peak"] = round(flops / (us * 1e-6) / fp32_peak, 3)
        rows_out.append(r)

    f32 = lambda *s: torch.randn(*s, dtype=torch.float32, device=dev)
    b16 = lambda *s: torch.randn(*s, dtype=torch.bfloat16, device=dev)
    H, G, K, V, page = heads, kv_heads, hd, hd, 64
    pages_per = -(-context // page)
    for label, rows, single in ((f"portion of {tokens} up to position {context}", tokens, False),
                                (f"decode, batch {batch} at position {context - 1}", batch, True)):
        live = rows if single else 1
        row_slot = (torch.arange(rows, dtype=torch.int32, device=dev) if single
                    else torch.zeros(rows, dtype=torch.int32, device=dev))
        row_pos = (torch.full((rows,), context - 1, dtype=torch.int32, device=dev) if single
                   else torch.arange(context - rows, context, dtype=torch.int32, device=dev))
        seg = None
        if not single:
            seg = torch.empty(batch, 3, dtype=torch.int32, device=dev)
            kernels.segment_table(row_slot, seg)
        # ---- the recurrence: the delta rule beside the plain write, both ways to decay
        q, k, v = f32(rows, G * K), f32(rows, G * K), f32(rows, H * V)
        state = torch.zeros(batch, H * V * K, dtype=torch.float32, device=dev)
        o = torch.empty(rows, H * V, dtype=torch.float32, device=dev)
        beta, step, rate, bias = f32(rows, H), f32(rows, H), f32(H) - 3.0, f32(H)
        decay = torch.rand(rows, H * K, dtype=torch.float32, device=dev) * 0.1 + 0.9
        io = rows * (2 * G * K + 2 * H * V) * 4 + 2 * live * H * V * K * 4
        # (a portion goes four tokens at a time: preparation, groups and the rows left over)
        work = None if single else torch.empty(kernels.delta_work_floats(rows, H, K),
                                               dtype=torch.float32, device=dev)
        us = _time(lambda: kernels.delta_recurrence(
            q, k, v, step, beta, state, o, row_slot, seg, H, G, K, V, kernels.DECAY_RATE_STEP,
            q_scale=K ** -0.5, unit_floor=1e-6, rate_log=rate, step_bias=bias, n_requests=live,
            work=work), flush=flush)
        # per state element and token: the delta rule a multiply and three multiply-adds, the
        # plain write two multiply-adds
        cells = rows * H * K * V
        rec(f"delta rule, a decay per head, {H} heads of {K} x {V} ({label})", us, io + rows * H * 8,
            flops=7.0 * cells)
        state.zero_()
        us = _time(lambda: kernels.delta_recurrence(
            q, k, v, decay, beta, state, o, row_slot, seg, H, G, K, V, kernels.DECAY_VECTOR,
            q_scale=K ** -0.5, unit_floor=1e-6, n_requests=live, work=work), flush=flush)
        rec(f"delta rule, a decay per key channel ({label})", us, io + rows * H * (K + 1) * 4,
            flops=7.0 * cells)
        if not single:
            state.zero_()
            us = _time(lambda: kernels.delta_recurrence(
                q, k, v, decay, beta, state, o, row_slot, seg, H, G, K, V, kernels.DECAY_VECTOR,
                q_scale=K ** -0.5, unit_floor=1e-6, n_requests=live), flush=flush)
            rec(f"delta rule, a decay per key channel, token by token ({label})", us,
                io + rows * H * (K + 1) * 4, flops=7.0 * cells)
        del work
        state.zero_()
        us = _time(lambda: kernels.linear_recurrence(
            q, k, v, step, state, o, row_slot, seg, H, G, K, V, kernels.DECAY_RATE_STEP,
            rate_log=rate, step_bias=bias, n_requests=live), flush=flush)
        rec(f"linear recurrence, a decay per head, the state-space mixer's ({label})", us,
            io + rows * H * 4, flops=4.0 * cells)
        state.zero_()
        us = _time(lambda: kernels.linear_recurrence(
            q, k, v, decay, state, o, row_slot, seg, H, G, K, V, kernels.DECAY_VECTOR,
            q_scale=K ** -0.5, n_requests=live), flush=flush)
        rec(f"linear recurrence, a decay per key channel, gated linear attention's ({label})", us,
            io + rows * H * K * 4, flops=4.0 * cells)
        # ---- the decay per key channel from the projected step
        z, kb = f32(rows, H * K), f32(H * K)
        us = _time(lambda: kernels.rate_decay(z, rate, kb, K), flush=flush)
        rec(f"rate_decay ({label})", us, rows * H * K * 8)
        z = f32(rows, H * K)
        us = _time(lambda: kernels.bias_sigmoid_pow(z, kb, 0.0625), flush=flush)
        rec(f"bias_sigmoid_pow, gated linear attention's ({label})", us, rows * H * K * 8)
        # ---- gate and norm behind the recurrence
        gate, nw = f32(rows, H * V), f32(V)
        gated = torch.empty(rows, H * V, dtype=torch.bfloat16, device=dev)
        for act in ("sigmoid", "silu"):
            us = _time(lambda: kernels.gated_group_norm(o, gate, nw, gated, group=V, eps=1e-6,
                                                        gate_first=False, gate_activation=act),
                       flush=flush)
            rec(f"gate + norm per head, {act}{'' if act == 'sigmoid' else ' (the form of gated linear attention)'} ({label})",
                us, rows * H * V * 10)
        # ---- store: temperature and blended values, beside the plain store
        storage = b16(live * pages_per, 1, 2, G, page, hd) * 0.5
        table = torch.randperm(live * pages_per, device=dev).to(torch.int32).view(live, pages_per)
        view = _View(storage, table.contiguous(), page)
        C = (H + 2 * G) * hd
        src, v0 = f32(rows, C), f32(rows, G * hd)
        qo = torch.empty(rows, H * hd, dtype=torch.bfloat16, device=dev)
        a, b = H * hd, (H + G) * hd
        for name, kw, extra in (("temperature and blended values", dict(q_temp=(0.1, 1024), blend=(v0, 0.4)),
                                 rows * G * hd * 4), ("neither (the store of Pemolorn's attention)", {}, 0)):
            us = _time(lambda: kernels.qkv_store(src[:, :a], src[:, a:b], src[:, b:], qo, view, row_slot,
                                                 row_pos, H, G, hd, hd, hd, kernels.NORM_NONE, None, None,
                                                 0.0, **kw), flush=flush)
            rec(f"qkv_store: {name} ({label})", us, rows * (C * 4 + C * 2) + extra)
        # ---- gates on the attention's output
        out16, gch = b16(rows, H * hd), f32(rows, H * hd + H)
        us = _time(lambda: kernels.channel_gate(out16, gch[:, :H * hd]), flush=flush)
        rec(f"channel_gate: a sigmoid per channel ({label})", us, rows * H * hd * 8)
        us = _time(lambda: kernels.head_gate(out16, gch[:, H * hd:], H, hd), flush=flush)
        rec(f"head_gate: a sigmoid per head (Vunasun's) ({label})", us, rows * H * (hd * 4 + 4))
        # ---- the router
        E, top = 8, 2
        h16, wr, corr = b16(rows, width), f32(E, width), f32(E) * 0.1
        zz = torch.empty(rows, E, dtype=torch.float32, device=dev)
        ids = torch.empty(rows, top, dtype=torch.int32, device=dev)
        wts = torch.empty(rows, top, dtype=torch.float32, device=dev)
        for name, mode in (("renormed weights", "softmax_all_renormed"), ("Pemolorn's", "softmax_all")):
            us = _time(lambda: kernels.moe_router(h16, wr, None, E, top, zz, ids, wts, mode, corr,
                                                  2.0 if mode.endswith("renormed") else 1.0), flush=flush)
            rec(f"moe_router, {name} ({label})", us, rows * (width * 2 + E * 4 + top * 8) + E * width * 4)
        del storage
    return rows_out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--sizes", default="0.6b,8b")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--kernels", action="store_true", help="only the table of kernels")
    ap.add_argument("--tokens", type=int, default=2048, help="tokens of the table's prompt portion")
    a = ap.parse_args(argv)
    rec: Dict[str, Any] = {}
    if not a.kernels:
        rec = compare([s for s in a.sizes.split(",") if s], a.layers, batch=a.batch)
    rec["kernels"] = kernel_table(tokens=a.tokens, context=max(4096, a.tokens))
    json.dump(rec, sys.stdout, indent=1)
    print()
    return 0


if __name__ == "__main__":
    sys.exit(main())
