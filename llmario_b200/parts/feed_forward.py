"""Gated feed-forward: ``y = W_down (silu(W_gate h) * (W_up h))`` with
``silu(z) = z / (1 + exp(-z))``, no biases (crates/engine/model/src/forward.rs:500-530;
crates/engine/cpu/src/ops.rs:83-99).  Gate and up are one product over stacked rows.

Beside it: the same form with a choice of activation and optional biases (kind ``gated``), and
routed experts (kind ``moe``): a router's logits (32-bit) choose ``top`` of ``experts`` small
silu-gated feed-forwards per token, whose outputs are summed with the softmax over the chosen
logits as weights; an optional shared feed-forward is applied to all tokens and added with a
per-token scalar weight, the sigmoid of one more projection of the input.  Options of the routed
experts: ``scores: "softmax_all"`` (the scores are the softmax over all router outputs, the choice
goes by score plus the tensor ``correction``, and a chosen expert's weight is its score, not
renormalised); ``identity`` (the last so many router outputs are experts without matrices whose
output is the input itself); ``activation: "clamped_swish"`` with ``limit``;
``scores: "softmax_all_renormed"`` (as ``softmax_all``, but the weights are the chosen scores over
their sum, times ``weight_scale``); ``activation: "relu_squared"`` (experts without a gate,
``W_down max(W_up h, 0)^2``: there are no ``gate<e>`` tensors).

And a feed-forward without a gate (kind ``dense``): ``y = W_down act(W_up h)``."""
from __future__ import annotations

from typing import Dict

import torch

from .. import kernels
from ..config.spec import ConfigError, PartSpec
from .base import StepContext, build_part, optional_tensor_of, register_part, tensor_of
from .linear import Linear


class SwiGLU:
    graph_safe = True

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype, device):
        self.hidden = int(spec["hidden_size"])
        self.ff = int(spec["intermediate_size"])
        gate, up = tensor_of(spec, "gate", weights), tensor_of(spec, "up", weights)
        # For the tensor-core product gate and up rows are stored interleaved in blocks of 16
        # (16 gate rows, their 16 up rows, ...): one 128-row weight tile then holds 64 features
        # with gate and up of a feature in the same quarter of the accumulator.
        self.interleaved = kernels.gated_interleave_ok(gate, up)
        if self.interleaved:
            ff, k = gate.shape
            both = torch.stack([gate.view(ff // 16, 16, k), up.view(ff // 16, 16, k)], dim=1)
            self.gate_up = Linear(both.reshape(2 * ff, k))
        else:
            self.gate_up = Linear.stacked([gate, up])
        self.down = Linear(tensor_of(spec, "down", weights))

    def streamed_weights(self):
        return [self.gate_up.weight, self.down.weight]

    def forward(self, ctx: StepContext, h: torch.Tensor, x: torch.Tensor,
                accumulate: bool = True) -> None:
        """Adds the result into ``x``; with ``accumulate=False`` ``x`` (float32) receives it."""
        rows = ctx.rows
        act = ctx.buffer("ffn.act", (rows, self.ff))
        kernels.gate_up_silu(ctx, h, self.gate_up.weight, act, self.interleaved)
        self.down(act, x, accumulate=accumulate)


class NoFeedForward:
    """A layer without a feed-forward: no tensors, no work."""

    graph_safe = True

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype, device):
        pass

    def streamed_weights(self):
        return []

    def forward(self, ctx: StepContext, h: torch.Tensor, x: torch.Tensor,
                accumulate: bool = True) -> None:
        if not accumulate:
            raise RuntimeError("a layer without a feed-forward has no result to hand over")


class GatedFeedForward:
    """``y = W_down (act(W_gate h + b_gate) * (W_up h + b_up)) + b_down`` with ``activation``
    ``silu`` or ``gelu_tanh`` (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))); the biases
    (tensor roles ``gate_bias``, ``up_bias``, ``down_bias``) are optional.  Without biases and
    with silu it is the standard part and runs on its fused product."""

    graph_safe = True

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype, device):
        self.hidden = int(spec["hidden_size"])
        self.ff = int(spec["intermediate_size"])
        self.activation = spec.get("activation", "silu")
        if self.activation not in kernels.ACTIVATIONS:
            raise ConfigError(f"gated feed-forward: activation '{self.activation}' (known: "
                              f"{', '.join(kernels.ACTIVATIONS)})")
        b = {r: optional_tensor_of(spec, r + "_bias", weights) for r in ("gate", "up", "down")}
        if (b["gate"] is None) != (b["up"] is None):
            raise ConfigError("gated feed-forward: the gate's and the up projection's biases "
                              "come together")
        self.plain = None
        if self.activation == "silu" and all(v is None for v in b.values()):
            self.plain = SwiGLU(spec, weights, dtype, device)
            return
        self.gate_up = Linear.stacked([tensor_of(spec, "gate", weights),
                                       tensor_of(spec, "up", weights)])
        self.gate_up_bias = None if b["gate"] is None else torch.cat(
            [b["gate"].to(torch.float32), b["up"].to(torch.float32)]).contiguous()
        self.down = Linear(tensor_of(spec, "down", weights), b["down"])

    def streamed_weights(self):
        if self.plain is not None:
            return self.plain.streamed_weights()
        return [self.gate_up.weight, self.down.weight]

    def forward(self, ctx: StepContext, h: torch.Tensor, x: torch.Tensor,
                accumulate: bool = True) -> None:
        if self.plain is not None:
            self.plain.forward(ctx, h, x, accumulate=accumulate)
            return
        rows = ctx.rows
        # (few rows: the product adds partial sums into a buffer kept at zero, which the
        # activation kernel clears again)
        kept_zero = rows <= kernels.SPLIT_K_MAX_ROWS
        gu = ctx.buffer("ffn.gate_up.z" if kept_zero else "ffn.gate_up", (rows, 2 * self.ff),
                        torch.float32, zero=kept_zero)
        self.gate_up(h, gu, out_is_zero=kept_zero)
        act = ctx.buffer("ffn.act", (rows, self.ff))
        kernels.gated_act(gu, self.gate_up_bias, act, self.activation, clear=kept_zero)
        self.down(act, x, accumulate=accumulate)


class DenseFeedForward:
    """``y = W_down act(W_up h)`` with ``activation`` ``relu_squared`` (max(z, 0)^2)."""

    graph_safe = True

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype, device):
        self.hidden = int(spec["hidden_size"])
        self.ff = int(spec["intermediate_size"])
        self.activation = spec.get("activation", "relu_squared")
        if self.activation not in kernels.PLAIN_ACTIVATIONS:
            raise ConfigError(f"dense feed-forward: activation '{self.activation}' (known: "
                              f"{', '.join(kernels.PLAIN_ACTIVATIONS)})")
        self.up = Linear(tensor_of(spec, "up", weights))
        self.down = Linear(tensor_of(spec, "down", weights))

    def streamed_weights(self):
        return [self.up.weight, self.down.weight]

    def forward(self, ctx: StepContext, h: torch.Tensor, x: torch.Tensor,
                accumulate: bool = True) -> None:
        rows = ctx.rows
        kept_zero = rows <= kernels.SPLIT_K_MAX_ROWS
        u = ctx.buffer("ffn.up.z" if kept_zero else "ffn.up", (rows, self.ff), torch.float32,
                       zero=kept_zero)
        self.up(h, u, out_is_zero=kept_zero)
        act = ctx.buffer("ffn.act", (rows, self.ff))
        kernels.act_rows(u, act, self.activation, clear=kept_zero)
        self.down(act, x, accumulate=accumulate)


class RoutedExperts:
    graph_safe = True      # which experts a row uses is read on the device
    grouped = True         # (False: always the row-wise kernels; for comparisons)

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype, device):
        self.hidden = W = int(spec["hidden_size"])
        self.ff = ff = int(spec["intermediate_size"])
        self.experts = E = int(spec["experts"])
        self.top = int(spec["top"])
        self.identity = int(spec.get("identity") or 0)       # experts without matrices
        self.routed = E + self.identity                      # router outputs that can be chosen
        self.scores = spec.get("scores", "softmax_chosen")
        self.activation = spec.get("activation", "silu")
        self.limit = float(spec.get("limit") or 0.0)
        self.weight_scale = float(spec.get("weight_scale") or 1.0)
        self.gated = self.activation != "relu_squared"
        if self.scores not in kernels.ROUTE_MODES:
            raise ConfigError(f"routed experts: scores '{self.scores}'")
        if self.activation not in ("silu", "clamped_swish", "relu_squared"):
            raise ConfigError(f"routed experts: activation '{self.activation}'")
        if self.weight_scale != 1.0 and self.scores != "softmax_all_renormed":
            raise ConfigError("routed experts: a scale of the weights needs scores "
                              "'softmax_all_renormed'")
        if not 1 <= self.top <= min(self.routed, 16):
            raise ConfigError(f"routed experts: top {self.top} of {self.routed} (at most 16)")
        router = tensor_of(spec, "router", weights).to(torch.float32)
        if router.shape[0] != self.routed:
            raise ConfigError(f"routed experts: a router of {router.shape[0]} outputs for "
                              f"{E} experts and {self.identity} identity experts")
        corr = optional_tensor_of(spec, "correction", weights)
        self.correction = None if corr is None else \
            corr.to(device=router.device, dtype=torch.float32).contiguous()
        if self.correction is not None and self.scores == "softmax_chosen":
            raise ConfigError("routed experts: a correction of the choice needs scores over "
                              "all router outputs")
        bias = optional_tensor_of(spec, "router_bias", weights)
        bias = torch.zeros(self.routed, device=router.device) if bias is None \
            else bias.to(torch.float32)
        sg = optional_tensor_of(spec, "shared_gate", weights)
        self.shared = None
        if spec.get("shared") is not None:
            if sg is None or tuple(sg.shape) != (1, W):
                raise ConfigError("routed experts: a shared expert needs its gate [1, hidden]")
            self.shared = build_part("feed_forward", spec["shared"], weights, dtype, device)
            router = torch.cat([router, sg.to(torch.float32)])
            bias = torch.cat([bias, torch.zeros(1, device=bias.device)])
        # the router (and the shared expert's gate as its last row) stays 32-bit
        self.router = Linear(router.contiguous(), bias)
        if self.gated:
            self.gate_up = torch.stack([torch.cat([tensor_of(spec, f"gate{e}", weights),
                                                   tensor_of(spec, f"up{e}", weights)])
                                        for e in range(E)]).contiguous()           # [E, 2 ff, W]
        else:       # (the name stays: without a gate it holds the up matrices alone, [E, ff, W])
            self.gate_up = torch.stack([tensor_of(spec, f"up{e}", weights)
                                        for e in range(E)]).contiguous()
        self.down = torch.stack([tensor_of(spec, f"down{e}", weights)
                                 for e in range(E)]).contiguous()              # [E, W, ff]
        if tuple(self.gate_up.shape) != (E, (2 if self.gated else 1) * ff, W) or \
                tuple(self.down.shape) != (E, W, ff):
            raise ConfigError("routed experts: the experts' matrices do not have the spec's sizes")

    def streamed_weights(self):
        """(What a step reads of the experts depends on its tokens: all of them are counted.)"""
        shared = self.shared.streamed_weights() if self.shared is not None else []
        return [self.router.weight, self.gate_up, self.down] + shared

    def forward(self, ctx: StepContext, h: torch.Tensor, x: torch.Tensor,
                accumulate: bool = True) -> None:
        rows, E, top = ctx.rows, self.experts, self.top
        R = self.routed
        z = ctx.buffer("moe.logits", (rows, self.router.out_features), torch.float32)
        ids = ctx.buffer("moe.ids", (rows, top), torch.int32)
        wts = ctx.buffer("moe.weights", (rows, top), torch.float32)
        if (self.hidden + self.router.out_features) * 4 <= 200 * 1024:
            kernels.moe_router(h, self.router.weight, self.router.bias, R, top, z, ids, wts,
                               self.scores, self.correction, self.weight_scale)
        else:           # a row too wide to stage: the product, then the choice
            self.router(h, z)
            kernels.moe_route(z, R, top, ids, wts, self.scores, self.correction,
                              self.weight_scale)
        ident = h if self.identity else None
        shared = gate = None
        kept_zero = rows <= kernels.SPLIT_K_MAX_ROWS
        if self.shared is not None:
            # (few rows: the shared expert adds into a buffer kept at zero, cleared by the kernel
            # that sums the experts)
            shared = ctx.buffer("moe.shared.z" if kept_zero else "moe.shared", (rows, self.hidden),
                                torch.float32, zero=kept_zero)
            self.shared.forward(ctx, h, shared, accumulate=kept_zero)
            gate = z[:, R]
        if kernels.moe_grouped_ok(h.dtype, self.hidden, self.ff) and self.grouped:
            # sorted by expert into tiles of rows, two grouped tensor-core products, one sum
            pairs = rows * top
            bn = kernels.moe_tile(pairs, E)
            tiles = -(-pairs // bn) + E
            pos = ctx.buffer("moe.pos", (pairs,), torch.int32)
            tile_group = ctx.buffer("moe.tiles", (tiles,), torch.int32)
            kernels.moe_align(ids, E, bn, pos, tile_group)
            xp = ctx.buffer("moe.x", (tiles * bn, self.hidden))
            kernels.moe_gather(h, pos, xp, top, ids if self.identity else None, E)
            act = ctx.buffer("moe.act", (tiles * bn, self.ff))
            if self.activation == "silu":
                kernels.gemm_grouped(xp, self.gate_up, act, tile_group, bn, gated=True)
            elif not self.gated:
                u = ctx.buffer("moe.up", (tiles * bn, self.ff), torch.float32)
                kernels.gemm_grouped(xp, self.gate_up, u, tile_group, bn, gated=False)
                kernels.act_rows(u, act, self.activation)
            else:       # the product as it is, then the activation over the padded buffer
                gu = ctx.buffer("moe.gate_up", (tiles * bn, 2 * self.ff), torch.float32)
                kernels.gemm_grouped(xp, self.gate_up, gu, tile_group, bn, gated=False)
                kernels.gated_act(gu, None, act, self.activation, limit=self.limit)
            d = ctx.buffer("moe.down", (tiles * bn, self.hidden), torch.float32)
            kernels.gemm_grouped(act, self.down, d, tile_group, bn, gated=False)
            kernels.moe_combine(d, pos, wts, x, accumulate, shared, gate, clear_shared=kept_zero,
                                ids=ids if self.identity else None, experts=E,
                                identity_input=ident)
            return
        act = ctx.buffer("moe.act", (rows, top, self.ff))
        kernels.moe_gate_up_rows(h, self.gate_up, ids, act, self.activation, self.limit)
        kernels.moe_down_rows(act, self.down, ids, wts, x, accumulate, shared, gate,
                              clear_shared=kept_zero, identity_input=ident)


register_part("feed_forward", "swiglu", SwiGLU, replace=True)
register_part("feed_forward", "gated", GatedFeedForward, replace=True)
register_part("feed_forward", "moe", RoutedExperts, replace=True)
register_part("feed_forward", "dense", DenseFeedForward, replace=True)
register_part("feed_forward", "none", NoFeedForward, replace=True)
