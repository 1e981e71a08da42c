"""Pre-norm residual arrangement: ``x += mixer(norm(x)); x += feed_forward(norm(x))``
(crates/engine/model/src/forward.rs:356-362), the arrangement with the norm on the
sublayer's output, the one over several residual streams, and the one whose two sublayers read
the same normed input (``x += mixer(norm(x)) + feed_forward(norm(x))``).  The residual stream ``x`` is 32-bit in every mode; the parts add into it."""
from __future__ import annotations

from typing import Dict

import torch

from .. import kernels
from ..config.spec import ConfigError, LayerSpec, PartSpec
from .base import (BoundCall, StepContext, build_part, cache_needs_of, graph_safe,
                   optional_tensor_of, register_part, streamed_weights_of)
from .norm import RmsNorm


class PreNormResidualBlock:
    def __init__(self, spec: PartSpec, layer: LayerSpec, weights: Dict[str, torch.Tensor],
                 dtype, device):
        self.mixer_norm = build_part("norm", spec["mixer_norm"], weights, dtype, device)
        # (a layer whose feed-forward is of kind ``none`` has only the first sublayer)
        self.ffn_norm = None if spec.get("feed_forward_norm") is None else \
            build_part("norm", spec["feed_forward_norm"], weights, dtype, device)
        self.mixer = build_part("mixer", layer.mixer, weights, dtype, device)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, weights, dtype,
                                       device)
        if self.ffn_norm is None and layer.feed_forward.kind != "none":
            raise ConfigError("a pre-norm block with a feed-forward needs its norm")

    def cache_needs(self):
        """What this block keeps between steps: one need per stateful part, in a fixed order
        (here the mixer's alone).  Each need gets a cache entry; ``call.for_need(k)`` is the
        call as the owner of the k-th need sees it."""
        return cache_needs_of(self.mixer)

    def streamed_weights(self):
        return streamed_weights_of(self.mixer) + streamed_weights_of(self.feed_forward)

    @property
    def graph_safe(self) -> bool:
        return all(graph_safe(p) for p in (self.mixer_norm, self.ffn_norm, self.mixer,
                                           self.feed_forward) if p is not None)

    def forward(self, ctx: StepContext, call: BoundCall, x: torch.Tensor) -> None:
        h = ctx.buffer("block.h", x.shape)
        self.mixer_norm.apply(ctx, x, h)
        self.mixer.forward(ctx, call.for_need(0) if call.cache_entries else call, h, x)
        if self.ffn_norm is not None:
            self.ffn_norm.apply(ctx, x, h)
            self.feed_forward.forward(ctx, h, x)


class OutputNormResidualBlock:
    """Norm on the sublayer's output only, with a scale per channel:
    ``x += s1 * norm1(mixer(x)); x += s2 * norm2(feed_forward(x))``.  The sublayers read the
    residual stream itself (rounded to the activation type); norm, scale and sum are 32-bit and
    one kernel.  A layer whose feed-forward is of kind ``none`` has only the first sublayer; the
    scales (tensor roles ``mixer_scale`` / ``feed_forward_scale``) are optional.

    With ``mixer_input_norm`` / ``feed_forward_input_norm`` a sublayer has a norm on both sides:
    ``x += norm_out(sublayer(norm_in(x)))``."""

    def __init__(self, spec: PartSpec, layer: LayerSpec, weights: Dict[str, torch.Tensor],
                 dtype, device):
        def scale(role):
            t = optional_tensor_of(spec, role, weights) if spec.get("tensors") else None
            return None if t is None else t.to(device=device, dtype=torch.float32).contiguous()

        def input_norm(key):
            return None if spec.get(key) is None else build_part("norm", spec[key], weights,
                                                                   dtype, device)

        self.mixer_norm = build_part("norm", spec["mixer_norm"], weights, dtype, device)
        self.mixer_in = input_norm("mixer_input_norm")
        self.ffn_in = input_norm("feed_forward_input_norm")
        self.mixer_scale = scale("mixer_scale")
        self.mixer = build_part("mixer", layer.mixer, weights, dtype, device)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, weights, dtype,
                                       device)
        self.has_feed_forward = layer.feed_forward.kind != "none"
        self.ffn_norm = self.ffn_scale = None
        if self.has_feed_forward:
            self.ffn_norm = build_part("norm", spec["feed_forward_norm"], weights, dtype, device)
            self.ffn_scale = scale("feed_forward_scale")
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None and not isinstance(norm, RmsNorm):
                raise ConfigError("the output-norm block fuses an RMS norm with the residual "
                                  f"sum; it has no form for {type(norm).__name__}")

    def cache_needs(self):
        return cache_needs_of(self.mixer)

    def streamed_weights(self):
        return streamed_weights_of(self.mixer) + streamed_weights_of(self.feed_forward)

    @property
    def graph_safe(self) -> bool:
        return graph_safe(self.mixer) and graph_safe(self.feed_forward)

    @staticmethod
    def _input(ctx: StepContext, x: torch.Tensor, have: bool, norm=None) -> torch.Tensor:
        """The residual stream as a sublayer reads it: rounded to the activation type, or
        through the sublayer's input norm when it has one.
        ``have``: the kernel that last added into the stream has left the rounded copy behind
        (see ``_add``); else (the first sublayer behind the embedding, or behind a block of
        another kind) it is rounded here."""
        if norm is not None:
            h = ctx.buffer("block.h", x.shape)
            norm.apply(ctx, x, h)
            return h
        if ctx.dtype == torch.float32:
            return x                   # the sublayer only reads it; x changes after it is done
        h = ctx.buffer("block.h", x.shape)
        if not have:
            kernels.cast_rows(x, h)
        return h

    @staticmethod
    def _add(ctx: StepContext, y, norm, scale, x, clear: bool, rounded: bool = True) -> None:
        """x += scale * norm(y), and (``rounded``) the next sublayer's input beside it."""
        h = ctx.buffer("block.h", x.shape) if ctx.dtype != torch.float32 and rounded else None
        kernels.norm_scale_add(y, norm.weight, scale, x, norm.eps, rounded=h, clear=clear)

    def forward(self, ctx: StepContext, call: BoundCall, x: torch.Tensor) -> None:
        # With few rows the sublayers' last products are cut along K and add partial sums.  Their
        # destination is then a buffer that is created as zeros and that the residual kernel
        # clears again once it has read it: the sublayers add into it and no clearing pass runs.
        kept_zero = ctx.rows <= kernels.SPLIT_K_MAX_ROWS
        y = ctx.buffer("block.y.z" if kept_zero else "block.y", x.shape, torch.float32,
                       zero=kept_zero)
        # the run-order entry just before this one was a block of this kind on the same stream
        have = ctx.shared.get("block.h behind") == (x.data_ptr(), call.index - 1)
        self.mixer.forward(ctx, call.for_need(0) if call.cache_entries else call,
                           self._input(ctx, x, have, self.mixer_in), y, accumulate=kept_zero)
        # (the rounded stream is left behind only for a sublayer that reads it as it is)
        last = not self.has_feed_forward
        self._add(ctx, y, self.mixer_norm, self.mixer_scale, x, kept_zero,
                  rounded=self.ffn_in is None if not last else True)
        if self.has_feed_forward:
            self.feed_forward.forward(ctx, self._input(ctx, x, True, self.ffn_in), y,
                                      accumulate=kept_zero)
            self._add(ctx, y, self.ffn_norm, self.ffn_scale, x, kept_zero)
        ctx.shared["block.h behind"] = (x.data_ptr(), call.index)


class HyperConnectionBlock:
    """Pre-norm sublayers over S residual streams ``xs`` [S, rows, hidden] (32-bit).  Sublayer q
    reads ``u = sum_s in_q[s] xs[s]``, computes ``y = sublayer(norm_q(u))`` and writes, for all
    streams at once from the old ones, ``xs[t] <- sum_s mix_q[s, t] xs[s] + out_q[t] y``.  One
    kernel does a sublayer's write together with the next sublayer's read and norm; the write of
    a layer's last sublayer is left to the block that runs next (or to the end of the step),
    which finds it under ``ctx.shared["streams.pending"]``.  Tensor roles: ``mixer_in`` [S],
    ``mixer_out`` [S], ``mixer_mix`` [S, S] (indexed [from, to]) and the same for
    ``feed_forward_*``; a feed-forward of kind ``none`` leaves a layer with one sublayer."""

    def __init__(self, spec: PartSpec, layer: LayerSpec, weights: Dict[str, torch.Tensor],
                 dtype, device):
        self.streams = int(spec["streams"])

        def coef(role, shape):
            t = optional_tensor_of(spec, role, weights)
            if t is None or tuple(t.shape) != shape:
                raise ConfigError(f"hyper-connection block: tensor '{role}' of shape {shape}")
            return t.to(device=device, dtype=torch.float32).contiguous()

        S = self.streams
        self.mixer_norm = build_part("norm", spec["mixer_norm"], weights, dtype, device)
        self.mixer = build_part("mixer", layer.mixer, weights, dtype, device)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, weights, dtype,
                                       device)
        self.has_feed_forward = layer.feed_forward.kind != "none"
        self.mixer_coef = (coef("mixer_in", (S,)), coef("mixer_out", (S,)),
                           coef("mixer_mix", (S, S)))
        self.ffn_norm = self.ffn_coef = None
        if self.has_feed_forward:
            self.ffn_norm = build_part("norm", spec["feed_forward_norm"], weights, dtype, device)
            self.ffn_coef = (coef("feed_forward_in", (S,)), coef("feed_forward_out", (S,)),
                             coef("feed_forward_mix", (S, S)))
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None and type(norm) is not RmsNorm:
                raise ConfigError("the hyper-connection block fuses an RMS norm with the mixing "
                                  f"of the streams; it has no form for {type(norm).__name__}")

    def cache_needs(self):
        return cache_needs_of(self.mixer)

    def streamed_weights(self):
        return streamed_weights_of(self.mixer) + streamed_weights_of(self.feed_forward)

    @property
    def graph_safe(self) -> bool:
        return graph_safe(self.mixer) and graph_safe(self.feed_forward)

    def forward(self, ctx: StepContext, call: BoundCall, xs: torch.Tensor) -> None:
        if xs.dim() != 3 or xs.shape[0] != self.streams:
            raise RuntimeError(f"a hyper-connection block of {self.streams} streams was given a "
                               f"residual of shape {tuple(xs.shape)}")
        shape = tuple(xs.shape[1:])
        # the sublayers' last products add partial sums when a step has few rows: their
        # destination is then kept at zero (the stream kernel clears what it has read)
        kept_zero = ctx.rows <= kernels.SPLIT_K_MAX_ROWS
        y = ctx.buffer("block.y.z" if kept_zero else "block.y", shape, torch.float32,
                       zero=kept_zero)
        h = ctx.buffer("block.h", shape)
        write = ctx.shared.pop("streams.pending", None) or {}
        cin, cout, mix = self.mixer_coef
        kernels.stream_step(xs, in_coef=cin, weight=self.mixer_norm.weight,
                            eps=self.mixer_norm.eps, out=h, **write)
        self.mixer.forward(ctx, call.for_need(0) if call.cache_entries else call, h, y,
                           accumulate=kept_zero)
        write = dict(y=y, mix=mix, out_coef=cout, clear_y=kept_zero)
        if self.has_feed_forward:
            cin, cout, mix = self.ffn_coef
            kernels.stream_step(xs, in_coef=cin, weight=self.ffn_norm.weight,
                                eps=self.ffn_norm.eps, out=h, **write)
            self.feed_forward.forward(ctx, h, y, accumulate=kept_zero)
            write = dict(y=y, mix=mix, out_coef=cout, clear_y=kept_zero)
        ctx.shared["streams.pending"] = write


class SharedNormResidualBlock:
    """One norm, both sublayers read its output: ``h = norm(x); x += mixer(h) + feed_forward(h)``.
    The sublayers add into the 32-bit stream one after the other; a feed-forward of kind ``none``
    leaves the mixer alone."""

    def __init__(self, spec: PartSpec, layer: LayerSpec, weights: Dict[str, torch.Tensor],
                 dtype, device):
        self.norm = build_part("norm", spec["norm"], weights, dtype, device)
        self.mixer = build_part("mixer", layer.mixer, weights, dtype, device)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, weights, dtype,
                                       device)

    def cache_needs(self):
        return cache_needs_of(self.mixer)

    def streamed_weights(self):
        return streamed_weights_of(self.mixer) + streamed_weights_of(self.feed_forward)

    @property
    def graph_safe(self) -> bool:
        return all(graph_safe(p) for p in (self.norm, self.mixer, self.feed_forward))

    def forward(self, ctx: StepContext, call: BoundCall, x: torch.Tensor) -> None:
        h = ctx.buffer("block.h", x.shape)
        self.norm.apply(ctx, x, h)
        self.mixer.forward(ctx, call.for_need(0) if call.cache_entries else call, h, x)
        self.feed_forward.forward(ctx, h, x)


register_part("block", "pre_norm_residual", PreNormResidualBlock, replace=True)
register_part("block", "shared_norm_residual", SharedNormResidualBlock, replace=True)
register_part("block", "hyper_connection", HyperConnectionBlock, replace=True)
register_part("block", "output_norm_residual", OutputNormResidualBlock, replace=True)
