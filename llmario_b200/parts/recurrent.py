"""Mixers that carry a matrix state per head from token to token instead of keys and values:

* ``gla``: gated linear attention with a decay per key channel,
  ``S_t = diag(alpha_t) S_{t-1} + k_t v_t^T``, ``o_t = S_t^T q_t`` with
  ``alpha = sigmoid(W_a2 W_a1 h + b)^(1/tau)`` and ``q`` scaled by ``key_dim^(-1/2)``; each
  head's output is RMS-normed (one weight over the value channels, shared by the heads),
  multiplied by ``silu(W_g h)`` and projected.
* ``mamba2``: a state-space mixer with one decay per head,
  ``S_t = exp(-exp(A_log) dt_t) S_{t-1} + dt_t B_t x_t^T``, ``y_t = S_t^T C_t + D x_t`` with
  ``dt = softplus(dt + dt_bias)``; x, B and C pass a short causal convolution per channel and
  silu first, B and C are shared by the heads of a group; ``y silu(z)`` is RMS-normed in equal
  groups of channels and projected.

* ``mlstm``: a matrix memory with exponential input and forget gates per head, kept in range by
  a running maximum ``m_t = max(f_t + m_(t-1), i_t)`` (m starts at 0):
  ``S_t = e^(f_t + m_(t-1) - m_t) S_(t-1) + e^(i_t - m_t) k_t v_t^T``, a normaliser ``z_t`` that is
  the same sum with ``k_t`` alone, ``o_t = S_t^T q_t / (max(|z_t . q_t|, e^(-m_t)) + floor)``
  with ``q`` scaled by ``key_dim^(-1/2)``, ``i = cap tanh((W_i h + b_i) / cap)`` and
  ``f = log sigmoid(cap tanh((W_f h + b_f) / cap))``; each head's output is divided by its root
  mean square, multiplied by a gain per channel and by ``sigmoid(W_g h)``, and projected.

* ``min_gru``: a vector state per channel whose gates read only the current token:
  ``S_t = (1 - z_t) S_(t-1) + z_t c_t`` with ``z = sigmoid(W_z h + b_z)`` and the candidate
  ``c = u + 1/2`` where ``u = W_x h + b_x >= 0`` and ``sigmoid(u)`` elsewhere; the output is
  ``W_o (S_t silu(W_g h))``.  It has a kernel of its own (a multiply-add per token and channel).

* ``gated_delta``: the gated delta rule, whose write is the error of the state's own answer,
  ``S <- diag(a_t) S``, ``u = b_t (v_t - S^T k_t)``, ``S <- S + k_t u^T``, ``o_t = S^T q_t`` with
  ``b = sigmoid(W_b h)``; q, k and v pass a short causal convolution per channel and silu, q and
  k are then unit vectors per head (``x / sqrt(sum x^2 + 1e-6)``) and q is scaled by
  ``key_dim^(-1/2)``; q and k heads may be shared by groups of value heads.  The decay is
  ``exp(-exp(A_log_h) softplus(z + dt_bias))`` with z one number per head (``W_a h``) or one per
  head and key channel (``W_a2 W_a1 h``); each head's output is divided by its root mean square,
  multiplied by a gain per value channel (shared by the heads) and by a gate, ``silu`` or
  ``sigmoid`` of ``W_g h`` or of ``W_g2 W_g1 h``, and projected.

The first three and the last are the same recurrence (``csrc/recurrent.cu``), told by data how the decay is made (the
matrix memory's normaliser is one more state column that is fed ones) and whether the write is the delta rule's.  The
state (and the convolution's last inputs) is 32-bit and lives in the request's fixed-size state
slot of the cache manager, which clears a slot when a request is opened in it.  Everything
behind the projections is computed in 32-bit.  Which rows belong to which request is read on
the device, so steps of single tokens can be recorded and replayed.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..cache import FixedState
from ..config.spec import ConfigError, PartSpec
from .base import BoundCall, StepContext, optional_tensor_of, register_part, tensor_of
from .linear import Linear


def step_segments(ctx: StepContext) -> Optional[torch.Tensor]:
    """The table (first row, end row) per request slot of this step, made once per step on the
    device; None when every row is a request of its own (the kernels then go by ``row_slot``)."""
    if ctx.rows == len(ctx.segments):
        return None
    seg = ctx.shared.get("segments")
    if seg is None:
        seg = ctx.buffer("segments", (ctx.cache.max_requests, 3), torch.int32)
        kernels.segment_table(ctx.row_slot, seg)
        ctx.shared["segments"] = seg
    return seg


def _f32(t: torch.Tensor, device) -> torch.Tensor:
    return t.to(device=device, dtype=torch.float32).contiguous()


def _padded_rows(mats, hidden: int):
    """The matrices stacked into one product, rows padded to a multiple of 16 (the 32-bit output
    keeps rows of whole 16-byte units)."""
    n = sum(m.shape[0] for m in mats)
    if n % 16:
        mats = list(mats) + [torch.zeros(16 - n % 16, hidden, dtype=mats[0].dtype,
                                         device=mats[0].device)]
    return Linear.stacked(mats)


class GatedLinearAttention:
    graph_safe = True

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype, device):
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["num_heads"])
        self.key_dim = int(spec["key_dim"])
        self.value_dim = int(spec["value_dim"])
        self.tau = float(spec["tau"])
        self.eps = float(spec["eps"])
        if self.tau <= 0:
            raise ConfigError(f"gla: tau {self.tau} must be positive")
        if self.key_dim > 512:
            raise ConfigError(f"gla: key_dim {self.key_dim}: the recurrence keeps at most 512 key "
                              "channels of a state column in registers")
        t = {r: tensor_of(spec, r, weights) for r in ("q", "k", "v", "g", "a1", "a2", "o")}
        self.rank = t["a1"].shape[0]          # the decay's low rank: the tensors' own size
        if t["a2"].shape[1] != self.rank:
            raise ConfigError(f"gla: the decay's two factors disagree on their rank "
                              f"({self.rank} and {t['a2'].shape[1]})")
        hk, hv = self.heads * self.key_dim, self.heads * self.value_dim
        self.col_k, self.col_v, self.col_g, self.col_a = hk, 2 * hk, 2 * hk + hv, 2 * hk + 2 * hv
        self.in_proj = _padded_rows([t["q"], t["k"], t["v"], t["g"], t["a1"]], self.hidden)
        self.decay_proj = Linear(t["a2"])
        bias = optional_tensor_of(spec, "a2_bias", weights)
        self.decay_bias = None if bias is None else _f32(bias, device)
        self.o_proj = Linear(t["o"])
        self.norm_weight = _f32(tensor_of(spec, "norm", weights), device)
        if self.norm_weight.numel() != self.value_dim:
            raise ConfigError("gla: the output norm has one weight per value channel of a head")

    def cache_need(self):
        return FixedState((self.heads * self.value_dim * self.key_dim,), torch.float32)

    def streamed_weights(self):
        return [self.in_proj.weight, self.decay_proj.weight, self.o_proj.weight]

    def forward(self, ctx: StepContext, call: BoundCall, h: torch.Tensor, x: torch.Tensor,
                accumulate: bool = True) -> None:
        rows, H, K, V = ctx.rows, self.heads, self.key_dim, self.value_dim
        state = ctx.cache.state_of(call.cache_entry)
        if state is None:
            raise RuntimeError(f"run-order entry {call.index}: the recurrence needs a state slot")
        proj = ctx.buffer("gla.proj", (rows, self.in_proj.out_features), torch.float32)
        self.in_proj(h, proj)
        low = proj[:, self.col_a:self.col_a + self.rank]
        if ctx.dtype != torch.float32:           # the operand of the second, low-rank product
            low16 = ctx.buffer("gla.low", (rows, self.rank))
            kernels.cast_rows(low, low16)
            low = low16
        z = ctx.buffer("gla.z", (rows, H * K), torch.float32)
        self.decay_proj(low, z)
        # the decay of every (token, key channel), once: bias, sigmoid and the root in one pass
        kernels.bias_sigmoid_pow(z, self.decay_bias, 1.0 / self.tau)
        o = ctx.buffer("gla.o", (rows, H * V), torch.float32)
        kernels.linear_recurrence(
            proj[:, :self.col_k], proj[:, self.col_k:self.col_v], proj[:, self.col_v:self.col_g],
            z, state, o, ctx.row_slot, step_segments(ctx), H, H, K, V, kernels.DECAY_VECTOR,
            q_scale=K ** -0.5, n_requests=len(ctx.segments))
        gated = ctx.buffer("gla.gated", (rows, H * V))
        kernels.gated_group_norm(o, proj[:, self.col_g:self.col_a], self.norm_weight, gated,
                                 group=V, eps=self.eps, gate_first=False)
        self.o_proj(gated, x, accumulate=accumulate)


class StateSpaceMixer:
    graph_safe = True

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype, device):
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["num_heads"])
        self.head_dim = int(spec["head_dim"])
        self.state_dim = int(spec["state_dim"])
        self.groups = int(spec["groups"])
        self.taps = int(spec["conv_taps"])
        self.norm_groups = int(spec["norm_groups"])
        self.eps = float(spec["eps"])
        self.inner = self.heads * self.head_dim
        if self.heads % self.groups:
            raise ConfigError(f"mamba2: {self.heads} heads cannot share {self.groups} groups")
        if self.inner % self.norm_groups:
            raise ConfigError(f"mamba2: {self.inner} channels in {self.norm_groups} norm groups")
        if self.state_dim > 512:
            raise ConfigError(f"mamba2: state {self.state_dim}: the recurrence keeps at most 512 "
                              "state rows of a column in registers")
        if self.taps < 1:
            raise ConfigError("mamba2: the convolution has at least one tap")
        gn = self.groups * self.state_dim
        self.conv_channels = self.inner + 2 * gn
        self.col_x, self.col_dt = self.inner, 2 * self.inner + 2 * gn
        self.in_proj = _padded_rows([tensor_of(spec, "in", weights)], self.hidden)
        self.o_proj = Linear(tensor_of(spec, "o", weights))
        self.conv_weight = _f32(tensor_of(spec, "conv", weights), device)
        bias = optional_tensor_of(spec, "conv_bias", weights)
        self.conv_bias = None if bias is None else _f32(bias, device)
        self.step_bias = _f32(tensor_of(spec, "dt_bias", weights), device)
        self.rate_log = _f32(tensor_of(spec, "A_log", weights), device)
        self.skip = _f32(tensor_of(spec, "D", weights), device)
        self.norm_weight = _f32(tensor_of(spec, "norm", weights), device)
        self.state_floats = self.heads * self.head_dim * self.state_dim

    def cache_need(self):
        """The matrix state of every head, then every convolved channel's last taps - 1 inputs."""
        return FixedState((self.state_floats + self.conv_channels * (self.taps - 1),),
                          torch.float32)

    def streamed_weights(self):
        return [self.in_proj.weight, self.o_proj.weight]

    def forward(self, ctx: StepContext, call: BoundCall, h: torch.Tensor, x: torch.Tensor,
                accumulate: bool = True) -> None:
        rows, H, P, N, G = ctx.rows, self.heads, self.head_dim, self.state_dim, self.groups
        state = ctx.cache.state_of(call.cache_entry)
        if state is None:
            raise RuntimeError(f"run-order entry {call.index}: the recurrence needs a state slot")
        seg = step_segments(ctx)
        proj = ctx.buffer("ssm.proj", (rows, self.in_proj.out_features), torch.float32)
        self.in_proj(h, proj)                    # [z | x | B | C | dt]
        xbc = ctx.buffer("ssm.conv", (rows, self.conv_channels), torch.float32)
        kernels.causal_conv_silu(proj[:, self.col_x:self.col_dt], self.conv_weight, self.conv_bias,
                                 state[:, self.state_floats:], xbc, ctx.row_slot, seg)
        o = ctx.buffer("ssm.o", (rows, self.inner), torch.float32)
        kernels.linear_recurrence(
            xbc[:, self.inner + G * N:], xbc[:, self.inner:self.inner + G * N], xbc[:, :self.inner],
            proj[:, self.col_dt:self.col_dt + H], state, o, ctx.row_slot, seg, H, G, N, P,
            kernels.DECAY_RATE_STEP, rate_log=self.rate_log, step_bias=self.step_bias,
            n_requests=len(ctx.segments))
        gated = ctx.buffer("ssm.gated", (rows, self.inner))
        kernels.gated_group_norm(o, proj[:, :self.inner], self.norm_weight, gated,
                                 group=self.inner // self.norm_groups, eps=self.eps,
                                 gate_first=True, skip=self.skip, skip_input=xbc[:, :self.inner],
                                 head=P)
        self.o_proj(gated, x, accumulate=accumulate)


class MatrixMemory:
    graph_safe = True

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype, device):
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["num_heads"])
        self.key_dim = int(spec["key_dim"])
        self.value_dim = int(spec["value_dim"])
        self.gate_cap = float(spec.get("gate_cap") or 0.0)      # 0: the gates are not capped
        self.eps = float(spec["eps"])
        self.floor = float(spec.get("floor", 1e-6))
        if self.key_dim > 512:
            raise ConfigError(f"mlstm: key_dim {self.key_dim}: the recurrence keeps at most 512 "
                              "key channels of a state column in registers")
        H, K, V = self.heads, self.key_dim, self.value_dim
        t = {r: tensor_of(spec, r, weights) for r in ("q", "k", "v", "g", "i", "f", "o")}
        self.col_k, self.col_v, self.col_g = H * K, 2 * H * K, 2 * H * K + H * V
        self.col_i, self.col_f = 2 * H * K + 2 * H * V, 2 * H * K + 2 * H * V + H
        self.in_proj = _padded_rows([t[r] for r in ("q", "k", "v", "g", "i", "f")], self.hidden)
        self.o_proj = Linear(t["o"])
        bi, bf = (optional_tensor_of(spec, r, weights) for r in ("i_bias", "f_bias"))
        self.bias_i = None if bi is None else _f32(bi, device)
        self.bias_f = None if bf is None else _f32(bf, device)
        self.norm_weight = _f32(tensor_of(spec, "norm", weights), device)
        if self.norm_weight.numel() != H * V:
            raise ConfigError("mlstm: the output norm has one weight per value channel of every head")
        self.state_floats = H * (V + 1) * K       # per head V value columns and the normaliser's

    def cache_need(self):
        """Every head's matrix with the normaliser as one more column, then every head's running
        maximum of the gates."""
        return FixedState((self.state_floats + self.heads,), torch.float32)

    def streamed_weights(self):
        return [self.in_proj.weight, self.o_proj.weight]

    def forward(self, ctx: StepContext, call: BoundCall, h: torch.Tensor, x: torch.Tensor,
                accumulate: bool = True) -> None:
        rows, H, K, V = ctx.rows, self.heads, self.key_dim, self.value_dim
        state = ctx.cache.state_of(call.cache_entry)
        if state is None:
            raise RuntimeError(f"run-order entry {call.index}: the recurrence needs a state slot")
        seg = step_segments(ctx)
        proj = ctx.buffer("mlstm.proj", (rows, self.in_proj.out_features), torch.float32)
        self.in_proj(h, proj)                    # [q | k | v | g | i | f]
        gates = ctx.buffer("mlstm.gates", (rows, 3 * H), torch.float32)    # [keep | take | m]
        kernels.log_gate_scan(proj[:, self.col_i:self.col_i + H], proj[:, self.col_f:self.col_f + H],
                              self.bias_i, self.bias_f, self.gate_cap,
                              state[:, self.state_floats:], gates, ctx.row_slot, seg, H,
                              n_requests=len(ctx.segments))
        o = ctx.buffer("mlstm.o", (rows, H * (V + 1)), torch.float32)
        kernels.linear_recurrence(
            proj[:, :self.col_k], proj[:, self.col_k:self.col_v], proj[:, self.col_v:self.col_g],
            gates[:, :H], state, o, ctx.row_slot, seg, H, H, K, V + 1,
            kernels.DECAY_SCALAR_INPUT, q_scale=K ** -0.5, n_requests=len(ctx.segments),
            input_weight=gates[:, H:2 * H], ones=True)
        gated = ctx.buffer("mlstm.gated", (rows, H * V))
        kernels.memory_out_norm(o, gates[:, 2 * H:], proj[:, self.col_g:self.col_i],
                                self.norm_weight, gated, H, V, self.eps, self.floor)
        self.o_proj(gated, x, accumulate=accumulate)


class GatedDeltaRule:
    """Kind ``gated_delta``.  Tensor roles: ``q``, ``k`` [groups * key_dim, hidden], ``v``
    [heads * value_dim, hidden], their convolutions ``q_conv``, ``k_conv``, ``v_conv``
    [channels, taps], ``b`` [heads, hidden], ``A_log`` [heads], ``norm`` [value_dim], ``o``;
    the decay from ``a`` [heads, hidden] with ``dt_bias`` [heads], or from ``a1`` [r, hidden] and
    ``a2`` [heads * key_dim, r] with ``dt_bias`` [heads * key_dim]; the gate from ``g``
    [heads * value_dim, hidden] or from ``g1`` [r, hidden] and ``g2`` [heads * value_dim, r]
    (the ranks are the tensors' own sizes).  ``gate_activation``: ``silu`` or ``sigmoid``."""

    graph_safe = True
    UNIT_FLOOR = 1e-6        # inside the root of the unit vectors

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype, device):
        self.hidden = W = int(spec["hidden_size"])
        self.heads = H = int(spec["num_heads"])
        self.groups = G = int(spec.get("num_kv_heads") or H)
        self.key_dim = K = int(spec["key_dim"])
        self.value_dim = V = int(spec["value_dim"])
        self.taps = int(spec["conv_taps"])
        self.eps = float(spec["eps"])
        self.gate_activation = spec.get("gate_activation", "silu")
        if self.gate_activation not in ("silu", "sigmoid"):
            raise ConfigError(f"gated_delta: gate_activation '{self.gate_activation}'")
        if H % G or self.taps < 1:
            raise ConfigError(f"gated_delta: {H} heads on {G} key heads, {self.taps} taps")
        if K > 512:
            raise ConfigError(f"gated_delta: key_dim {K}: the recurrence keeps at most 512 key "
                              "channels of a state column in registers")
        names = spec["tensors"]
        t = {r: tensor_of(spec, r, weights) for r in names}
        self.decay_per_channel = "a1" in names
        self.gate_low_rank = "g1" in names
        for a, b in (("a1", "a2"), ("g1", "g2")):
            if (a in names) != (b in names) or (a in names and t[a].shape[0] != t[b].shape[1]):
                raise ConfigError(f"gated_delta: the factors '{a}' and '{b}' come together and "
                                  "agree on their rank")
        # one product for everything that reads the mixer's input; every part starts a column
        # range of whole 16-byte units
        parts = [("q", t["q"]), ("k", t["k"]), ("v", t["v"]), ("b", t["b"]),
                 ("a", t["a1"] if self.decay_per_channel else t["a"]),
                 ("g", t["g1"] if self.gate_low_rank else t["g"])]
        mats, self.col, at = [], {}, 0
        for name, m in parts:
            if name in ("b", "a", "g") and at % 4:
                pad = 4 - at % 4
                mats.append(torch.zeros(pad, W, dtype=m.dtype, device=m.device))
                at += pad
            self.col[name] = at
            mats.append(m)
            at += m.shape[0]
        self.width_of = {name: m.shape[0] for name, m in parts}
        self.in_proj = _padded_rows(mats, W)
        self.conv_channels = 2 * G * K + H * V
        if self.col["v"] != 2 * G * K or self.col["b"] < self.conv_channels:
            raise ConfigError("gated_delta: q, k and v do not have the spec's sizes")
        conv = [t[r + "_conv"] for r in ("q", "k", "v")]
        for c, n in zip(conv, (G * K, G * K, H * V)):
            if tuple(c.shape) != (n, self.taps):
                raise ConfigError(f"gated_delta: a convolution of {list(c.shape)} for {n} "
                                  f"channels and {self.taps} taps")
        self.conv_weight = torch.cat([_f32(c, device) for c in conv]).contiguous()
        self.decay_proj = Linear(t["a2"]) if self.decay_per_channel else None
        self.gate_proj = Linear(t["g2"]) if self.gate_low_rank else None
        self.rate_log = _f32(t["A_log"], device)
        self.step_bias = _f32(t["dt_bias"], device)
        if self.rate_log.numel() != H or \
                self.step_bias.numel() != (H * K if self.decay_per_channel else H):
            raise ConfigError("gated_delta: A_log has a number per head, dt_bias one per decay")
        self.norm_weight = _f32(t["norm"], device)
        if self.norm_weight.numel() != V:
            raise ConfigError("gated_delta: the output norm has one weight per value channel of "
                              "a head")
        self.o_proj = Linear(t["o"])
        self.state_floats = H * V * K

    def cache_need(self):
        """The matrix state of every head, then every convolved channel's last taps - 1 inputs."""
        return FixedState((self.state_floats + self.conv_channels * (self.taps - 1),),
                          torch.float32)

    def streamed_weights(self):
        extra = [p.weight for p in (self.decay_proj, self.gate_proj) if p is not None]
        return [self.in_proj.weight, self.o_proj.weight] + extra

    def _second(self, ctx: StepContext, proj: torch.Tensor, name: str, second: Linear,
                out: torch.Tensor) -> None:
        """out = second(the low-rank part ``name`` of proj), its operand rounded for 16-bit."""
        low = proj[:, self.col[name]:self.col[name] + self.width_of[name]]
        if ctx.dtype != torch.float32:
            low16 = ctx.buffer("delta.low." + name, (ctx.rows, self.width_of[name]))
            kernels.cast_rows(low, low16)
            low = low16
        second(low, out)

    def run(self, ctx: StepContext, call: BoundCall, proj: torch.Tensor, x: torch.Tensor,
            accumulate: bool) -> None:
        """From the projections ``proj`` = [q | k | v | b | a | g] (float32) to the output.

        With low-rank factors a step that holds portions of prompts launches this mixer's
        kernels in plain stream order.  As programmatic dependents of one another (operand
        rounded, second product of many rows, decay or gate + norm, with the walk of the
        recurrence between them) such steps stopped making progress now and then on models of
        a width of 1,024 (four of six runs of a model of eight such layers; none of seven in
        plain stream order; no bounded wait reported).  Steps of single tokens, whose products
        are the kernels for few rows, keep the dependent launches."""
        if (self.decay_per_channel or self.gate_low_rank) and ctx.rows != len(ctx.segments):
            with kernels.plain_stream_order():
                self._run(ctx, call, proj, x, accumulate)
        else:
            self._run(ctx, call, proj, x, accumulate)

    def _run(self, ctx: StepContext, call: BoundCall, proj: torch.Tensor, x: torch.Tensor,
             accumulate: bool) -> None:
        rows, H, G, K, V = ctx.rows, self.heads, self.groups, self.key_dim, self.value_dim
        state = ctx.cache.state_of(call.cache_entry)
        if state is None:
            raise RuntimeError(f"run-order entry {call.index}: the recurrence needs a state slot")
        seg = step_segments(ctx)
        C = self.conv_channels
        conv = ctx.buffer("delta.conv", (rows, C), torch.float32)
        # (one tap keeps no inputs: a weight per channel, and the kernel reads no history)
        history = state[:, self.state_floats:] if self.taps > 1 else state
        kernels.causal_conv_silu(proj[:, :C], self.conv_weight, None, history, conv,
                                 ctx.row_slot, seg)
        beta = proj[:, self.col["b"]:self.col["b"] + H]
        if self.decay_per_channel:
            d = ctx.buffer("delta.decay", (rows, H * K), torch.float32)
            self._second(ctx, proj, "a", self.decay_proj, d)
            kernels.rate_decay(d, self.rate_log, self.step_bias, K)
            kind, rate, bias = kernels.DECAY_VECTOR, None, None
        else:
            d = proj[:, self.col["a"]:self.col["a"] + H]
            kind, rate, bias = kernels.DECAY_RATE_STEP, self.rate_log, self.step_bias
        o = ctx.buffer("delta.o", (rows, H * V), torch.float32)
        # (portions of prompts go four tokens at a time where the kernels have that form)
        work = None
        if seg is not None and kernels.delta_work_floats(rows, H, K):
            work = ctx.buffer("delta.work", (kernels.delta_work_floats(rows, H, K),), torch.float32)
        kernels.delta_recurrence(
            conv[:, :G * K], conv[:, G * K:2 * G * K], conv[:, 2 * G * K:], d, beta, state, o,
            ctx.row_slot, seg, H, G, K, V, kind, q_scale=K ** -0.5, unit_floor=self.UNIT_FLOOR,
            rate_log=rate, step_bias=bias, n_requests=len(ctx.segments), work=work)
        if self.gate_low_rank:
            gate = ctx.buffer("delta.gate", (rows, H * V), torch.float32)
            self._second(ctx, proj, "g", self.gate_proj, gate)
        else:
            gate = proj[:, self.col["g"]:self.col["g"] + H * V]
        gated = ctx.buffer("delta.gated", (rows, H * V))
        kernels.gated_group_norm(o, gate, self.norm_weight, gated, group=V, eps=self.eps,
                                 gate_first=False, gate_activation=self.gate_activation)
        self.o_proj(gated, x, accumulate=accumulate)

    def forward(self, ctx: StepContext, call: BoundCall, h: torch.Tensor, x: torch.Tensor,
                accumulate: bool = True) -> None:
        proj = ctx.buffer("delta.proj", (ctx.rows, self.in_proj.out_features), torch.float32)
        self.in_proj(h, proj)
        self.run(ctx, call, proj, x, accumulate)


class MinGru:
    graph_safe = True

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype, device):
        self.hidden = int(spec["hidden_size"])
        self.width = int(spec["width"])
        t = {r: tensor_of(spec, r, weights) for r in ("z", "x", "g", "o")}
        for r in ("z", "x", "g"):
            if tuple(t[r].shape) != (self.width, self.hidden):
                raise ConfigError(f"min_gru: tensor '{r}' of {list(t[r].shape)} for a state of "
                                  f"{self.width} channels on a width of {self.hidden}")
        # the three projections of the mixer's input are one product; each keeps a column range
        # of whole 16-byte units
        self.stride = -(-self.width // 4) * 4
        pad = self.stride - self.width

        def padded(m):
            return m if not pad else torch.cat(
                [m, torch.zeros(pad, self.hidden, dtype=m.dtype, device=m.device)])

        self.in_proj = _padded_rows([padded(t["z"]), padded(t["x"]), padded(t["g"])], self.hidden)
        bz, bx = (optional_tensor_of(spec, r, weights) for r in ("z_bias", "x_bias"))
        self.bias_z = None if bz is None else _f32(bz, device)
        self.bias_x = None if bx is None else _f32(bx, device)
        self.o_proj = Linear(t["o"])

    def cache_need(self):
        return FixedState((self.width,), torch.float32)

    def streamed_weights(self):
        return [self.in_proj.weight, self.o_proj.weight]

    def run(self, ctx: StepContext, call: BoundCall, proj: torch.Tensor, x: torch.Tensor,
            accumulate: bool) -> None:
        """From the projections ``proj`` = [z | x | g] (float32, column ranges of ``stride``
        channels each, overwritten) to the output, added into or written to ``x``."""
        state = ctx.cache.state_of(call.cache_entry)
        if state is None:
            raise RuntimeError(f"run-order entry {call.index}: the recurrence needs a state slot")
        n, W = self.stride, self.width
        gated = ctx.buffer("mingru.gated", (ctx.rows, W))
        kernels.min_gru(proj[:, :W], proj[:, n:n + W], proj[:, 2 * n:2 * n + W], self.bias_z,
                        self.bias_x, state, gated, ctx.row_slot, step_segments(ctx))
        self.o_proj(gated, x, accumulate=accumulate)

    def forward(self, ctx: StepContext, call: BoundCall, h: torch.Tensor, x: torch.Tensor,
                accumulate: bool = True) -> None:
        proj = ctx.buffer("mingru.proj", (ctx.rows, self.in_proj.out_features), torch.float32)
        self.in_proj(h, proj)
        self.run(ctx, call, proj, x, accumulate)


register_part("mixer", "min_gru", MinGru, replace=True)
register_part("mixer", "gated_delta", GatedDeltaRule, replace=True)
register_part("mixer", "gla", GatedLinearAttention, replace=True)
register_part("mixer", "mlstm", MatrixMemory, replace=True)
register_part("mixer", "mamba2", StateSpaceMixer, replace=True)
