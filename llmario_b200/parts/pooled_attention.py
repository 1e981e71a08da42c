"""Two mixers for layers that run an attention and a recurrence side by side on one input.

``pooled_window_attention``: grouped-query attention whose queries, keys and values pass a short
causal convolution per channel directly behind their projections; queries and keys are then
RMS-normed over their whole rows (all heads at once, a weight per channel) and turned by
position in adjacent pairs.  A query at position i sees the keys j with ``0 <= i - j < window``
and, beside them, one pooled key and value for every block of ``pool`` positions that lies
wholly behind the window (``b * pool + pool - 1 <= i - window``): the means of the block's keys
and values as the cache holds them.  Tokens behind the window whose block is not complete yet
are not seen.  ``exp(sink_h)`` joins the softmax's denominator of head h.

What it keeps per request: the keys and values of the last ``max(window, pool)`` tokens in
pages, the pooled entries in pages of a cache of their own (one entry per ``pool`` tokens, none
ever given back), and the last ``taps - 1`` projected values of every convolved channel in a
state slot.  A block's entry is written by the step that brings its last token, from the cache.

``parallel``: two mixers read the same input; the result is half the sum of their outputs,
each first RMS-normed over the model width with a weight of its own.  The projections of both
that read the input are one product.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import driver, kernels
from ..cache import FixedState, PagedKV
from ..config.spec import ConfigError, PartSpec
from .base import (BoundCall, StepContext, build_part, cache_needs_of, graph_safe,
                   optional_tensor_of, register_part, streamed_weights_of, tensor_of)
from .linear import Linear
from .recurrent import _f32, _padded_rows, step_segments


class PooledWindowAttention:
    graph_safe = True

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype, device):
        self.hidden = int(spec["hidden_size"])
        self.heads = H = int(spec["num_heads"])
        self.kv_heads = G = int(spec["num_kv_heads"])
        self.dim = d = int(spec["head_dim"])
        self.value_dim = dv = int(spec.get("value_dim") or d)
        self.cache_dim = max(d, dv)
        self.scale = float(spec["scale"])
        self.window = int(spec["window"])
        self.pool = int(spec.get("pool") or 0)
        self.taps = int(spec.get("conv_taps") or 0)
        self.eps = float(spec["eps"])
        if self.window < 1 or self.pool < 0 or self.taps < 0 or H % G:
            raise ConfigError(f"pooled attention: window {self.window}, pool {self.pool}, "
                              f"{self.taps} taps, {H} heads on {G} key heads")
        refusal = kernels.attention_refusal(H, G, self.cache_dim)
        if refusal is not None:
            raise ConfigError(f"pooled attention: {refusal}")
        self.position = (build_part("position", spec["position"], weights, dtype, device)
                         if spec.get("position") is not None else None)
        if self.position is not None and not hasattr(self.position, "head_permutation"):
            raise ConfigError("pooled attention: the rotation is that of adjacent pairs "
                              "(rope_normal)")
        self.q_cols, self.k_cols, self.v_cols = H * d, G * d, G * dv
        self.channels = self.q_cols + self.k_cols + self.v_cols
        self.in_proj = _padded_rows([tensor_of(spec, r, weights) for r in ("q", "k", "v")],
                                    self.hidden)
        qn, kn = (optional_tensor_of(spec, r, weights) for r in ("q_norm", "k_norm"))
        if (qn is None) != (kn is None):
            raise ConfigError("pooled attention: q_norm and k_norm come together")
        self.q_norm = None if qn is None else _f32(qn, device).reshape(-1)
        self.k_norm = None if kn is None else _f32(kn, device).reshape(-1)
        if qn is not None and (self.q_norm.numel() != self.q_cols
                               or self.k_norm.numel() != self.k_cols):
            raise ConfigError("pooled attention: the norms have a weight per channel of the "
                              "whole query and key rows")
        self.conv_weight = None
        if self.taps >= 1:
            conv = [tensor_of(spec, r + "_conv", weights) for r in ("q", "k", "v")]
            for c, n in zip(conv, (self.q_cols, self.k_cols, self.v_cols)):
                if tuple(c.shape) != (n, self.taps):
                    raise ConfigError(f"pooled attention: a convolution of {list(c.shape)} for "
                                      f"{n} channels and {self.taps} taps")
            self.conv_weight = torch.cat([_f32(c, device) for c in conv]).contiguous()
        sink = optional_tensor_of(spec, "sink", weights)
        self.sink = None if sink is None else _f32(sink, device)
        if self.sink is not None and self.sink.numel() != H:
            raise ConfigError(f"pooled attention: a sink of {self.sink.numel()} numbers for {H} heads")
        self.o_proj = Linear(tensor_of(spec, "o", weights))

    def cache_needs(self):
        """The token cache (a block's keys must still be there when its last token comes, so it
        keeps at least ``pool`` tokens), the pooled cache, and the convolution's last inputs."""
        needs = [PagedKV(self.kv_heads, self.cache_dim, max(self.window, self.pool))]
        if self.pool:
            needs.append(PagedKV(self.kv_heads, self.cache_dim, None, 0, self.pool))
        if self.taps > 1:
            needs.append(FixedState((self.channels * (self.taps - 1),), torch.float32))
        return needs

    def streamed_weights(self):
        return [self.in_proj.weight, self.o_proj.weight]

    def run(self, ctx: StepContext, call: BoundCall, proj: torch.Tensor, x: torch.Tensor,
            accumulate: bool) -> None:
        """From the projections ``proj`` = [q | k | v] (float32) to the output."""
        rows, H, G, d, dv, hd = ctx.rows, self.heads, self.kv_heads, self.dim, self.value_dim, \
            self.cache_dim
        if not call.writes_cache:
            raise RuntimeError("pooled attention keeps a cache of its own")
        view = ctx.cache.view(call.for_need(0).cache_entry)
        pooled = ctx.cache.view(call.for_need(1).cache_entry) if self.pool else None
        src = proj[:, :self.channels]
        if self.taps >= 1:
            # (one tap keeps no inputs: a weight per channel, and the kernel reads no history)
            state = ctx.cache.state_of(call.for_need(2 if self.pool else 1).cache_entry) \
                if self.taps > 1 else ctx.buffer("pattn.nohist", (1, 1), torch.float32)
            conv = ctx.buffer("pattn.conv", (rows, self.channels), torch.float32)
            kernels.causal_conv_silu(src, self.conv_weight, None, state, conv, ctx.row_slot,
                                     step_segments(ctx), activation=False)
            src = conv
        cos_sin, rot = None, 0
        if self.position is not None:
            _, rot, _ = self.position.rotary_tables()
            cos_sin = self.position.step_angles(ctx)
        q = ctx.buffer("attn.q", (rows, H * hd))
        a, b = self.q_cols, self.q_cols + self.k_cols
        kernels.qkv_store(src[:, :a], src[:, a:b], src[:, b:b + self.v_cols], q, view,
                          ctx.row_slot, ctx.row_pos, H, G, d, dv, hd,
                          kernels.NORM_WHOLE_ROW if self.q_norm is not None else kernels.NORM_NONE,
                          self.q_norm, self.k_norm, self.eps, rot, cos_sin)
        if self.pool:
            kernels.pool_blocks(view, pooled, ctx.row_slot, ctx.row_pos, rows, G, hd, self.pool)
        out = ctx.buffer("attn.out", (rows, H * dv))
        driver.attention(ctx, q, out, view, H, G, hd, self.scale, self.window, sink=self.sink,
                         value_dim=dv if dv != hd else None, pool=self.pool, pooled_view=pooled)
        self.o_proj(out, x, accumulate=accumulate)

    def forward(self, ctx: StepContext, call: BoundCall, h: torch.Tensor, x: torch.Tensor,
                accumulate: bool = True) -> None:
        proj = ctx.buffer("pattn.proj", (ctx.rows, self.in_proj.out_features), torch.float32)
        self.in_proj(h, proj)
        self.run(ctx, call, proj, x, accumulate)


class ParallelMixers:
    """``left`` and ``right`` (nested specs) read the same input; tensor roles ``left_out`` and
    ``right_out`` ([hidden]) are the weights of the norms on their outputs."""

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype, device):
        self.hidden = int(spec["hidden_size"])
        self.eps = float(spec["eps"])
        self.left = build_part("mixer", spec["left"], weights, dtype, device)
        self.right = build_part("mixer", spec["right"], weights, dtype, device)
        self.left_weight = _f32(tensor_of(spec, "left_out", weights), device)
        self.right_weight = _f32(tensor_of(spec, "right_out", weights), device)
        if self.left_weight.numel() != self.hidden or self.right_weight.numel() != self.hidden:
            raise ConfigError("parallel mixers: the output norms have a weight per channel of "
                              "the model width")
        self.n_left = len(cache_needs_of(self.left))
        # one product for every projection of the input, when both halves can take their
        # columns of it (each says so by offering `in_proj` and `run(ctx, call, proj, x,
        # accumulate)`)
        self.in_proj = None
        if all(hasattr(m, "in_proj") and hasattr(m, "run") for m in (self.left, self.right)):
            self.in_proj = Linear.stacked([self.left.in_proj.weight, self.right.in_proj.weight])
            self.split = self.left.in_proj.out_features
            # (the halves keep no copy of their own)
            self.left.in_proj = Linear(self.in_proj.weight[:self.split])
            self.right.in_proj = Linear(self.in_proj.weight[self.split:])

    @property
    def graph_safe(self) -> bool:
        return graph_safe(self.left) and graph_safe(self.right)

    def cache_needs(self):
        return cache_needs_of(self.left) + cache_needs_of(self.right)

    def streamed_weights(self):
        # (with one product for both, the halves' own are its rows: views of one tensor)
        return streamed_weights_of(self.left) + streamed_weights_of(self.right)

    @staticmethod
    def _sub(call: BoundCall, first: int, n: int) -> BoundCall:
        """The call as a half sees it: its own needs, numbered from 0."""
        entries = call.cache_entries[first:first + n]
        return BoundCall(call.index, call.layer, call.writes_cache,
                         entries[0] if entries else None, entries)

    def forward(self, ctx: StepContext, call: BoundCall, h: torch.Tensor, x: torch.Tensor,
                accumulate: bool = True) -> None:
        shape = (ctx.rows, self.hidden)
        a = ctx.buffer("parallel.left", shape, torch.float32)
        b = ctx.buffer("parallel.right", shape, torch.float32)
        lcall = self._sub(call, 0, self.n_left)
        rcall = self._sub(call, self.n_left, len(call.cache_entries) - self.n_left)
        if self.in_proj is not None:
            proj = ctx.buffer("parallel.proj", (ctx.rows, self.in_proj.out_features),
                              torch.float32)
            self.in_proj(h, proj)
            self.left.run(ctx, lcall, proj[:, :self.split], a, False)
            self.right.run(ctx, rcall, proj[:, self.split:], b, False)
        else:
            self.left.forward(ctx, lcall, h, a, accumulate=False)
            self.right.forward(ctx, rcall, h, b, accumulate=False)
        kernels.dual_norm_mean(a, b, self.left_weight, self.right_weight, x, self.eps,
                               accumulate=accumulate)


register_part("mixer", "pooled_window_attention", PooledWindowAttention, replace=True)
register_part("mixer", "parallel", ParallelMixers, replace=True)
