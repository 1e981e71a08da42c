"""Pemolorn beside Qwen3 at equal sizes: prompt and decode rates of whole models with random
weights, and the design's own kernels one by one against the memory roofline.

    python -m llmario_b200.benchmarks.pemolorn [--sizes 0.6b,8b] [--layers 8] [--kernels]

A Pemolorn model of a size has the width, feed-forward width, attention heads and number of
layers of the Qwen3 preset of that name; its layers repeat (pooled window attention beside a
minGRU + dense, kept-window attention + routed experts, the same, kept-window attention on the
keys and values of the layer before + dense) (``config.pemolorn.sized_like``).  A token uses two
of eight experts of half the feed-forward width, so a prompt does the feed-forward work of the
dense layer and a decode step of few rows streams up to all experts.  ``bench.py --workload
pemolorn`` prints the same record as its JSON line.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Any, Dict, List

from .vunasun import SIZES, _rates, _time


def pemolorn_config(preset: Dict[str, Any], layers: int, vocab: int = 32768, window: int = 1024,
                    pool: int = 64, keep_first: int = 4):
    """The Pemolorn configuration with the sizes of a Qwen3 preset."""
    from ..config.pemolorn import sized_like

    return sized_like(preset["hidden_size"], preset["intermediate_size"],
                      preset["num_attention_heads"], preset["num_key_value_heads"],
                      preset["head_dim"], layers, vocab, window=window, pool=pool,
                      keep_first=keep_first)


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
        for which in ("qwen3", "pemolorn"):
            if which == "qwen3":
                from ..config import Qwen3Config

                cfg = Qwen3Config.from_dict(dict(preset, num_hidden_layers=layers,
                                                 tie_word_embeddings=False,
                                                 architectures=["Qwen3ForCausalLM"]))
            else:
                cfg = pemolorn_config(preset, layers)
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


class _View:
    """A paged cache of one layer call as the kernels take it."""

    def __init__(self, storage, table, page):
        self.k, self.v = storage[0, 0, 0], storage[0, 0, 1]
        self.page_stride, self.block_table, self.page_size = storage.stride(0), table, page


def kernel_table(width: int = 4096, tokens: int = 2048, batch: int = 64, heads: int = 32,
                 kv_heads: int = 8, hd: int = 128, ff: int = 12288, window: int = 1024,
                 pool: int = 64, keep: int = 4, context: int = 4096) -> List[Dict[str, Any]]:
    """The design's own kernels, each alone at the sizes of ``pemolorn_config`` for ``width``,
    with the bytes they must move (or the operations they must do) and the fraction of the
    measured copy rate (or tensor rate); beside each the like kernel of the Qwen3 path.  The
    prompt case is a portion of ``tokens`` rows that ends at position ``context``, so that every
    row has pooled blocks and kept keys behind its window; the decode case is ``batch`` requests
    at position ``context`` - 1."""
    import torch

    from .. import kernels
    from .roofline import peaks

    dev = "cuda:0"
    pk = peaks()
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=dev)
    rows_out: List[Dict[str, Any]] = []

    def rec(name, us, nbytes, flops=0, note=""):
        r = {"kernel": name, "us": round(us, 2), "bytes": int(nbytes),
             "gb_s": round(nbytes / us / 1e3, 1),
             "frac_of_copy_peak": round(nbytes / (us * 1e-6) / (pk["hbm_gbs"] * 1e9), 3), "note": note}
        if flops:
            r["tflops"] = round(flops / us / 1e6, 1)
            r["frac_of_tensor_peak"] = round(flops / (us * 1e-6) / (pk["bf16_tflops"] * 1e12), 3)
        rows_out.append(r)

    f32 = lambda *s: torch.randn(*s, dtype=torch.float32, device=dev)
    b16 = lambda *s: torch.randn(*s, dtype=torch.bfloat16, device=dev)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    H, G, page = heads, kv_heads, 64
    group = H // G
    C = (H + 2 * G) * hd
    scale = hd ** -0.5
    pages_per = -(-context // page)
    ppages_per = -(-(context // pool) // page)
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
        storage = b16(live * pages_per, 1, 2, G, page, hd) * 0.5
        table = torch.randperm(live * pages_per, device=dev).to(torch.int32).view(live, pages_per)
        view = _View(storage, table.contiguous(), page)
        pstorage = b16(live * ppages_per, 1, 2, G, page, hd) * 0.5
        ptable = torch.arange(live * ppages_per, dtype=torch.int32, device=dev).view(live, ppages_per)
        pooled = _View(pstorage, ptable, page)
        # ---- short convolution behind the projections (no activation), the mixer's q | k | v
        src, conv = f32(rows, C), torch.empty(rows, C, dtype=torch.float32, device=dev)
        taps = 4
        cw, hist = f32(C, taps), torch.zeros(batch, C * (taps - 1), dtype=torch.float32, device=dev)
        us = _time(lambda: kernels.causal_conv_silu(src, cw, None, hist, conv, row_slot, seg,
                                                    activation=False), flush=flush)
        rec(f"causal_conv without activation, {C} channels ({label})", us,
            rows * C * 8 + 2 * live * C * (taps - 1) * 4)
        # ---- norm over the whole rows, rotation of adjacent pairs, cache write
        rot = hd // 2
        cos_sin = f32(rows, rot // 2, 2)
        qn, kn = f32(H * hd), f32(G * hd)
        q = torch.empty(rows, H * hd, dtype=torch.bfloat16, device=dev)
        a, b = H * hd, (H + G) * hd
        us = _time(lambda: kernels.qkv_store(conv[:, :a], conv[:, a:b], conv[:, b:], q, view, row_slot,
                                             row_pos, H, G, hd, hd, hd, kernels.NORM_WHOLE_ROW, qn, kn,
                                             1e-6, rot, cos_sin), flush=flush)
        moved = rows * (C * 4 + C * 2 + rot * 4)
        rec(f"qkv_store: whole-row norms, rotation, cache write ({label})", us, moved)
        inv_freq = f32(hd // 2).abs()
        hq, hk = f32(hd), f32(hd)
        us = _time(lambda: kernels.qk_norm_rope_store(src, q, view.k, view.v, view.page_stride, table, row_slot,
                                                      row_pos, hq, hk, inv_freq, 1.0, H, G, hd, hd, page,
                                                      1e-6), flush=flush)
        rec(f"qk_norm_rope_store, the Qwen3 path's ({label})", us, rows * (C * 4 + C * 2))
        # ---- the pooled entries of the blocks that the step completes
        us = _time(lambda: kernels.pool_blocks(view, pooled, row_slot, row_pos, rows, G, hd, pool), flush=flush)
        blocks = rows if single else rows // pool
        rec(f"pool_blocks: {blocks} blocks of {pool} ({label})", us, blocks * (pool + 1) * 2 * G * hd * 2,
            note="a warp per (block, key head, key or value)")
        # ---- what lies outside the window, and the window's keys with and without that part
        sink = f32(H)
        part_o = torch.empty(rows, H, hd, dtype=torch.float32, device=dev)
        part_ml = torch.empty(rows, H, 2, dtype=torch.float32, device=dev)
        qq = b16(rows, H * hd)
        out = torch.empty_like(qq)
        n_out = [max(0, (p - window + 1) // pool) + min(keep, max(0, p - window + 1))
                 for p in (row_pos.tolist())]
        us = _time(lambda: kernels.attention_outside(qq, part_o, part_ml, view, row_slot, row_pos, H, G, hd,
                                                     scale, window, sink, keep, pool, pooled), flush=flush)
        entries = live * (max(n_out) if n_out else 0)
        rec(f"attention_outside: pooled blocks, kept keys, sink ({label})", us,
            entries * 2 * G * hd * 2 + rows * H * (hd * 2 + (hd + 2) * 4),
            flops=4.0 * sum(n_out) * H * hd,
            note="a warp per (row, head): every row reads its request's entries again (L2)")
        if single:
            splits = kernels.decode_splits(rows, G, window, kernels.DECODE_TMA_CTAS_PER_SM * kernels.sm_count(),
                                           kernels.DECODE_TMA_TILE)
            splits = max(2, splits)
            po = torch.empty(rows * H * splits * hd, dtype=torch.float32, device=dev)
            pml = torch.empty(rows * H * splits * 2, dtype=torch.float32, device=dev)
            for name, extra in (("with the outside part", (part_o, part_ml)), ("the Qwen3 path's", None)):
                def fn():
                    kernels.attention_decode_tma(qq, out, storage, 0, table, None, rows, H, G, hd, page, scale,
                                                 window, splits, po, pml, row_slot, row_pos)
                    kernels.attention_merge(po, pml, out, None, rows, H, hd, splits,
                                            sink=sink if extra is None else None, outside=extra)
                us = _time(fn, flush=flush)
                rec(f"decode attention over the window + merge, {name} ({label})", us,
                    live * window * 2 * G * hd * 2 + rows * H * hd * 4)
        else:
            cap = max(1, 128 // group)
            first = context - rows
            items = i32([[s, min(cap, rows - s), 0, first + s] for s in range(0, rows, cap)]).reshape(-1)
            keys = sum(min(window, p + 1) for p in row_pos.tolist())
            for name, extra in (("with the outside part", (part_o, part_ml)), ("the Qwen3 path's", None)):
                us = _time(lambda: kernels.attention_tcgen05(
                    qq, out, view.k, view.v, view.page_stride, table, items, items.numel() // 4, H, G, hd,
                    page, scale, window, storage.shape[0], sink=sink if extra is None else None,
                    outside=extra), flush=flush)
                kernels.check_tc_status(torch.device(dev))
                rec(f"tcgen05 attention over the window, {name} ({label})", us,
                    (window + rows) * 2 * G * hd * 2 + rows * H * hd * 4, flops=4.0 * keys * H * hd)
        # ---- the recurrence beside the attention, and the mean of the two normed outputs
        W = width
        proj = f32(rows, 3 * W)
        state = torch.zeros(batch, W, dtype=torch.float32, device=dev)
        gated = torch.empty(rows, W, dtype=torch.bfloat16, device=dev)
        bz, bx = f32(W), f32(W)
        us = _time(lambda: kernels.min_gru(proj[:, :W], proj[:, W:2 * W], proj[:, 2 * W:], bz, bx, state, gated,
                                           row_slot, seg), flush=flush)
        rec(f"min_gru ({label})", us, rows * W * (12 + 2) + 2 * live * W * 4,
            note="" if single else "a prompt is one request: a thread per channel walks its tokens in order")
        ya, yb, y = f32(rows, W), f32(rows, W), f32(rows, W)
        wa, wb = f32(W), f32(W)
        us = _time(lambda: kernels.dual_norm_mean(ya, yb, wa, wb, y, 1e-6, accumulate=True), flush=flush)
        rec(f"dual_norm_mean into the residual ({label})", us, rows * W * 16)
        h16 = torch.empty(rows, W, dtype=torch.bfloat16, device=dev)
        us = _time(lambda: kernels.rms_norm(ya, wa, h16, 1e-6), flush=flush)
        rec(f"rms_norm, the Qwen3 path's ({label})", us, rows * W * 6)
        # ---- feed-forward: the squared relu, and the router over experts and identity experts
        up = f32(rows, ff)
        act = torch.empty(rows, ff, dtype=torch.bfloat16, device=dev)
        us = _time(lambda: kernels.act_rows(up, act, "relu_squared"), flush=flush)
        rec(f"act_rows: squared relu ({label})", us, rows * ff * 6)
        gu = f32(rows, 2 * ff)
        us = _time(lambda: kernels.silu_mul(gu, act), flush=flush)
        rec(f"silu_mul, the Qwen3 path's ({label})", us, rows * ff * 10)
        E, top = 10, 2
        z = f32(rows, E)
        ids = torch.empty(rows, top, dtype=torch.int32, device=dev)
        wts = torch.empty(rows, top, dtype=torch.float32, device=dev)
        corr = f32(E) * 0.1
        us = _time(lambda: kernels.moe_route(z, E, top, ids, wts, "softmax_all", corr), flush=flush)
        rec(f"moe_route: softmax over all, choice by corrected score ({label})", us, rows * (E * 4 + top * 8))
        del storage, pstorage
    return rows_out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--sizes", default="0.6b,8b")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--kernels", action="store_true", help="only the table of kernels")
    a = ap.parse_args(argv)
    rec: Dict[str, Any] = {}
    if not a.kernels:
        rec = compare([s for s in a.sizes.split(",") if s], a.layers, batch=a.batch)
    rec["kernels"] = kernel_table()
    json.dump(rec, sys.stdout, indent=1)
    print()
    return 0


if __name__ == "__main__":
    sys.exit(main())
