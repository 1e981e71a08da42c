"""Grouped-query attention over the paged cache, with optional per-head norm of queries and
keys and a rotary position encoding.

Order of operations as in crates/engine/model/src/forward.rs:399-485: project q, k, v; norm each
head of q and k; rotate q and k by position; store k and v in the cache; attend from the cache
(causal, optionally only the last ``window`` keys); project the result and add it to the
residual stream.  A call that reads another call's cache projects only q.

Options that are data of the part's spec (each absent by default):

* ``chunk``: a query sees only the earlier keys of its own chunk of ``chunk`` positions, chunks
  counted from position 0 of the sequence (excludes ``window``);
* ``values: "keys"``: there is no value projection; a key head's value is the key as projected
  (with its bias), before the per-head norm and the rotation;
* tensor role ``gate`` ([heads, hidden]): head h's output is multiplied by the sigmoid of the
  h-th gate, a projection of the mixer's own input, before the output projection.
* ``keep_first`` (with ``window``): the first so many keys of a sequence are seen from every later
  position, at their true positions;
* tensor role ``sink`` ([heads]): ``exp(sink_h)`` joins the denominator of head h's softmax; it has
  no key and no value;
* ``value_dim``: the size of a value head when it is not ``head_dim`` (the cache's row is the
  larger of the two, the rest of a shorter row is zeros);
* ``shared_kv``: the layer has no key and value projections (nor their norm): every call of it
  reads the cache of an earlier call, with its own queries and mask.  The layer whose cache is
  read says with ``cache_window`` / ``cache_keep_first`` what its readers need it to keep.

* ``q_temp = {"coef": c, "every": n}``: the queries of position p are multiplied by
  ``1 + c ln(floor((p + 1) / n) + 1)``;
* ``value_blend = {"group": name, "source": bool}`` with the tensor role ``blend`` (one number
  lambda) on the layers that are no source: such a layer stores and attends to
  ``(1 - lambda) v + lambda v0`` where v0 are the values that the group's source layer projected
  for the same tokens (the source stores its own values unchanged; its ``blend`` is not read);
* tensor role ``gate`` of shape [heads * value_dim, hidden]: a sigmoid gate per output channel
  in the place of one per head.

These run through the store kernel of ``csrc/qkv_store.cu`` (which also turns adjacent
pairs itself; the pairs (i, i + rot_dim/2) of ``rope_neox`` are brought side by side by
ordering the rows of the q and k projections accordingly) and the attention call with the
matching arguments; a layer without them runs as before.  There the biases (roles ``q_bias``,
``k_bias``, ``v_bias``, ``o_bias``) and the gate per head are taken as well.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import driver, kernels
from ..cache import PagedKV
from ..config.spec import ConfigError, PartSpec
from .base import (BoundCall, StepContext, build_part, optional_tensor_of, register_part,
                   tensor_of)
from .linear import Linear


class Attention:
    graph_safe = True      # a step of single tokens reads positions and slots on the device only

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype, device):
        self.hidden = int(spec["hidden_size"])
        self.num_heads = int(spec["num_heads"])
        self.num_kv_heads = int(spec["num_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        self.scale = float(spec["scale"])
        self.window = spec.get("window")
        self.chunk = spec.get("chunk")
        self.mask = kernels.mask_code(self.window, self.chunk)   # what the kernels are told
        if spec.get("values", "projected") not in ("projected", "keys"):
            raise ConfigError(f"attention: values '{spec.get('values')}' (projected or keys)")
        self.values_are_keys = spec.get("values") == "keys"
        self.keep_first = int(spec.get("keep_first") or 0)
        self.value_dim = int(spec.get("value_dim") or self.head_dim)
        self.shared_kv = bool(spec.get("shared_kv"))
        self.cache_window = spec.get("cache_window", self.window)
        self.cache_keep_first = int(spec.get("cache_keep_first", self.keep_first) or 0)
        sink = optional_tensor_of(spec, "sink", weights)
        self.sink = None if sink is None else \
            sink.to(device=device, dtype=torch.float32).contiguous()
        if self.sink is not None and self.sink.numel() != self.num_heads:
            raise ConfigError(f"attention: a sink of {self.sink.numel()} numbers for "
                              f"{self.num_heads} heads")
        if self.keep_first and not self.window:
            raise ConfigError("attention: keep_first needs a window")
        self.fusable = False      # (see in_proj)
        self.q_temp = None
        if spec.get("q_temp") is not None:
            self.q_temp = (float(spec["q_temp"]["coef"]), int(spec["q_temp"]["every"]))
            if self.q_temp[1] < 1:
                raise ConfigError(f"attention: q_temp every {self.q_temp[1]} must be positive")
        self.blend_group = self.blend_source = self.blend = None
        if spec.get("value_blend") is not None:
            self.blend_group = str(spec["value_blend"]["group"])
            self.blend_source = bool(spec["value_blend"].get("source"))
            if not self.blend_source:
                self.blend = float(tensor_of(spec, "blend", weights).to(torch.float32).reshape(()))
        gate_entry = spec["tensors"].get("gate")
        self.gate_per_channel = gate_entry is not None and \
            int(gate_entry[1][0]) == self.num_heads * self.value_dim != self.num_heads
        # what the store kernel of several forms serves (see the module's text)
        self.general = bool(self.keep_first or self.sink is not None or self.shared_kv
                            or self.value_dim != self.head_dim or self.q_temp is not None
                            or self.blend_group is not None or self.gate_per_channel)
        if self.general:
            self._init_general(spec, weights, dtype, device)
            return
        refusal = kernels.attention_refusal(self.num_heads, self.num_kv_heads, self.head_dim)
        if refusal is not None:      # now, when the model is built, not at its first step
            raise ConfigError(f"attention: {refusal}")
        self.q_width = self.num_heads * self.head_dim
        self.kv_width = self.num_kv_heads * self.head_dim
        self.position = (build_part("position", spec["position"], weights, dtype, device)
                         if spec.get("position") is not None else None)
        qn, kn = spec.get("q_norm"), spec.get("k_norm")
        self.q_norm = build_part("norm", qn, weights, dtype, device) if qn is not None else None
        self.k_norm = build_part("norm", kn, weights, dtype, device) if kn is not None else None
        if (self.q_norm is None) != (self.k_norm is None):
            raise ValueError("q_norm and k_norm come together")
        if self.q_norm is not None and self.q_norm.eps != self.k_norm.eps:
            raise ValueError("q_norm and k_norm must share eps")
        w = {r: tensor_of(spec, r, weights) for r in ("q", "k")}
        if not self.values_are_keys:
            w["v"] = tensor_of(spec, "v", weights)
        gate = optional_tensor_of(spec, "gate", weights)
        if gate is not None and tuple(gate.shape) != (self.num_heads, self.hidden):
            raise ConfigError(f"attention: a gate of {list(gate.shape)} for {self.num_heads} "
                              f"heads of a width of {self.hidden}")
        # biases exist for the families that store them (forward.rs:399-425); tensor roles
        # "q_bias", "k_bias", "v_bias", "o_bias", each optional
        b = {r: optional_tensor_of(spec, r + "_bias", weights) for r in ("q", "k", "v", "o")}
        perm = self.position.head_permutation(self.head_dim) \
            if hasattr(self.position, "head_permutation") else None
        if perm is not None:
            # The position encoding rotates other pairs of a head than the kernels do.  A head's
            # scores do not change when queries and keys are permuted alike, so the rows of the
            # q and k projections (and what follows them per head: bias, norm gain) are permuted
            # once here and the kernels rotate their own pairs.
            perm = perm.to(device)
            for r, heads in (("q", self.num_heads), ("k", self.num_kv_heads)):
                w[r] = w[r].view(heads, self.head_dim, -1)[:, perm].reshape(w[r].shape)
                if b[r] is not None:
                    b[r] = b[r].view(heads, self.head_dim)[:, perm].reshape(-1)
            for norm in (self.q_norm, self.k_norm):
                if norm is not None:
                    norm.weight = norm.weight[perm].contiguous()
        # one product for everything that reads the mixer's input: q, k, v (unless the values
        # are the keys), the gates; its rows padded to a multiple of 16 so that the 32-bit
        # output keeps rows of whole 16-byte units
        mats = [w["q"], w["k"]] + ([] if self.values_are_keys else [w["v"]])
        biases = [b["q"], b["k"]] + ([] if self.values_are_keys else [b["v"]])
        self.kv_cols = self.kv_width * (1 if self.values_are_keys else 2)
        self.gate_col = None
        if gate is not None:
            self.gate_col = self.q_width + self.kv_cols
            mats.append(gate)
            biases.append(None)
        n_rows = sum(m.shape[0] for m in mats)
        if n_rows % 16:
            mats.append(torch.zeros(16 - n_rows % 16, self.hidden, dtype=mats[0].dtype,
                                    device=mats[0].device))
            biases.append(None)
        self.qkv_proj = Linear.stacked(mats, biases)
        self.q_proj = Linear(self.qkv_proj.weight[:self.q_width],      # the first rows, no copy
                             None if self.qkv_proj.bias is None else self.qkv_proj.bias[:self.q_width])
        self.o_proj = Linear(tensor_of(spec, "o", weights), b["o"])

    def _init_general(self, spec: PartSpec, weights, dtype, device) -> None:
        if self.chunk is not None or self.values_are_keys:
            raise ConfigError("attention: kept first keys, a sink, shared keys and values, a "
                              "value size of its own, a query temperature or blended values do "
                              "not combine with a chunked mask or values that are keys")
        if self.blend_group is not None and self.shared_kv:
            raise ConfigError("attention: a layer without values of its own blends none")
        d, dv = self.head_dim, self.value_dim
        self.cache_dim = max(d, dv)
        refusal = kernels.attention_refusal(self.num_heads, self.num_kv_heads, self.cache_dim)
        if refusal is not None:
            raise ConfigError(f"attention: {refusal}")
        self.position = (build_part("position", spec["position"], weights, dtype, device)
                         if spec.get("position") is not None else None)
        qn, kn = spec.get("q_norm"), spec.get("k_norm")
        self.q_norm = build_part("norm", qn, weights, dtype, device) if qn is not None else None
        self.k_norm = build_part("norm", kn, weights, dtype, device) if kn is not None else None
        if self.q_norm is not None and self.k_norm is not None and \
                self.q_norm.eps != self.k_norm.eps:
            raise ValueError("q_norm and k_norm must share eps")
        if (self.q_norm is None) != (self.k_norm is None) and not self.shared_kv:
            raise ValueError("q_norm and k_norm come together")
        self.q_width = self.num_heads * d
        self.k_cols, self.v_cols = self.num_kv_heads * d, self.num_kv_heads * dv
        roles = ["q"] + ([] if self.shared_kv else ["k", "v"])
        w = {r: tensor_of(spec, r, weights) for r in roles}
        b = {r: optional_tensor_of(spec, r + "_bias", weights) for r in roles + ["o"]}
        if self.position is not None and not hasattr(self.position, "head_permutation"):
            # The store kernel turns the pairs (2i, 2i + 1); this encoding turns (i, i + rot/2).
            # A head's scores do not change when queries and keys are reordered alike, so the
            # rows of the q and k projections (with bias and norm gain) are ordered once here
            # such that the members of every pair stand side by side.
            _, rot, _ = self.position.rotary_tables()
            order = [j for i in range(rot // 2) for j in (i, i + rot // 2)] + list(range(rot, d))
            perm = torch.tensor(order, dtype=torch.long, device=w["q"].device)
            for r, heads in (("q", self.num_heads), ("k", self.num_kv_heads)):
                if r not in w:
                    continue
                w[r] = w[r].view(heads, d, -1)[:, perm].reshape(w[r].shape)
                if b[r] is not None:
                    b[r] = b[r].view(heads, d)[:, perm].reshape(-1)
            for norm in (self.q_norm, self.k_norm):
                if norm is not None:
                    norm.weight = norm.weight[perm.to(norm.weight.device)].contiguous()
        mats, biases = [w[r] for r in roles], [b[r] for r in roles]
        self.gate_col = None
        gate = optional_tensor_of(spec, "gate", weights)
        if gate is not None:
            self.gate_cols = self.num_heads * (dv if self.gate_per_channel else 1)
            if tuple(gate.shape) != (self.gate_cols, self.hidden):
                raise ConfigError(f"attention: a gate of {list(gate.shape)} for "
                                  f"{self.num_heads} heads of {dv} value channels")
            # (the gates start a column range of whole 16-byte units)
            n_rows = sum(m.shape[0] for m in mats)
            if n_rows % 4:
                mats.append(torch.zeros(4 - n_rows % 4, self.hidden, dtype=mats[0].dtype,
                                        device=mats[0].device))
                biases.append(None)
            self.gate_col = sum(m.shape[0] for m in mats)
            mats.append(gate)
            biases.append(None)
        n_rows = sum(m.shape[0] for m in mats)
        if n_rows % 16:
            mats.append(torch.zeros(16 - n_rows % 16, self.hidden, dtype=mats[0].dtype,
                                    device=mats[0].device))
            biases.append(None)
        self.qkv_proj = Linear.stacked(mats, biases)
        # (attention writes value_dim channels per head, so the projection is as stored)
        self.o_proj = Linear(tensor_of(spec, "o", weights), b["o"])
        self.fusable = self.qkv_proj.bias is None and self.blend_group is None

    @property
    def in_proj(self) -> Linear:
        """The one product of the mixer's input, offered to a part that runs this mixer beside
        another one on the same input and wants a single product for both (it then calls
        :meth:`run` with this mixer's columns of the result).  Only a layer whose projections
        need nothing else (no bias, no buffer that outlives the layer) offers it."""
        if not self.fusable:
            raise AttributeError("in_proj")
        return self.qkv_proj

    @in_proj.setter
    def in_proj(self, proj: Linear) -> None:
        self.qkv_proj = proj

    def run(self, ctx: StepContext, call: BoundCall, proj: torch.Tensor, x: torch.Tensor,
            accumulate: bool) -> None:
        """From the projections ``proj`` (float32, the columns of :attr:`in_proj`) to the output."""
        self._run_general(ctx, call, proj, x, accumulate)

    def cache_need(self):
        # (no query ever looks back further than a chunk is long: pages behind that go back)
        if self.general:
            return PagedKV(self.num_kv_heads, self.cache_dim, self.cache_window,
                           self.cache_keep_first if self.cache_window else 0)
        return PagedKV(self.num_kv_heads, self.head_dim, self.window or self.chunk)

    def streamed_weights(self):
        """The matrices a step reads once: q, k, v (stacked) and the output projection."""
        return [self.qkv_proj.weight, self.o_proj.weight]

    def _forward_general(self, ctx: StepContext, call: BoundCall, h: torch.Tensor,
                         x: torch.Tensor, accumulate: bool) -> None:
        # (the values that other layers of a group blend in stay where their layer projected
        # them until the step ends)
        name = "attn.gproj" if not self.blend_source else "attn.gproj." + self.blend_group
        proj = ctx.buffer(name, (ctx.rows, self.qkv_proj.out_features), torch.float32)
        self.qkv_proj(h, proj)
        self._run_general(ctx, call, proj, x, accumulate)

    def _run_general(self, ctx: StepContext, call: BoundCall, proj: torch.Tensor,
                     x: torch.Tensor, accumulate: bool) -> None:
        rows, d, dv, hd = ctx.rows, self.head_dim, self.value_dim, self.cache_dim
        view = ctx.cache.view(call.cache_entry)
        if view is None:
            raise RuntimeError(f"run-order entry {call.index}: attention needs a cache")
        if self.shared_kv and call.writes_cache:
            raise RuntimeError(f"run-order entry {call.index}: a layer without key and value "
                               "projections must read another call's cache")
        writes = call.writes_cache
        a, c = self.q_width + self.k_cols, self.q_width + self.k_cols + self.v_cols
        blend = None
        if self.blend_group is not None and writes:
            key = ("attention.values", self.blend_group)
            if self.blend_source:
                ctx.shared[key] = proj[:, a:c]
            else:
                first = ctx.shared.get(key)
                if first is None or first.shape != (rows, self.v_cols):
                    raise RuntimeError(f"run-order entry {call.index}: the values of group "
                                       f"'{self.blend_group}' were not made in this step by a "
                                       "layer of the same value size")
                blend = (first, self.blend)
        cos_sin, rot = None, 0
        if self.position is not None:
            _, rot, _ = self.position.rotary_tables()
            cos_sin = self.position.step_angles(ctx)
        q = ctx.buffer("attn.q", (rows, self.num_heads * hd))
        norm = kernels.NORM_PER_HEAD if self.q_norm is not None else kernels.NORM_NONE
        kernels.qkv_store(
            proj[:, :self.q_width],
            proj[:, self.q_width:self.q_width + self.k_cols] if writes else None,
            proj[:, self.q_width + self.k_cols:self.q_width + self.k_cols + self.v_cols]
            if writes else None,
            q, view, ctx.row_slot, ctx.row_pos, self.num_heads, self.num_kv_heads, d, dv, hd,
            norm, self.q_norm.weight if self.q_norm is not None else None,
            self.k_norm.weight if self.k_norm is not None and writes else None,
            self.q_norm.eps if self.q_norm is not None else 0.0, rot, cos_sin,
            q_temp=self.q_temp, blend=blend)
        out = ctx.buffer("attn.out", (rows, self.num_heads * dv))
        driver.attention(ctx, q, out, view, self.num_heads, self.num_kv_heads, hd, self.scale,
                         self.mask, sink=self.sink, value_dim=dv if dv != hd else None,
                         keep_first=self.keep_first)
        if self.gate_col is not None:
            gate = proj[:, self.gate_col:self.gate_col + self.gate_cols]
            if self.gate_per_channel:
                kernels.channel_gate(out, gate)
            else:
                kernels.head_gate(out, gate, self.num_heads, dv)
        self.o_proj(out, x, accumulate=accumulate)

    def forward(self, ctx: StepContext, call: BoundCall, h: torch.Tensor, x: torch.Tensor,
                accumulate: bool = True) -> None:
        """Adds the result into ``x``; with ``accumulate=False`` ``x`` (float32) receives it."""
        if self.general:
            self._forward_general(ctx, call, h, x, accumulate)
            return
        rows = ctx.rows
        view = ctx.cache.view(call.cache_entry)
        if view is None:
            raise RuntimeError(f"run-order entry {call.index}: attention needs a cache")
        # With few rows the product is cut along K and its partial sums are added into the
        # buffer.  That buffer is created as zeros and the kernel that consumes it clears what it
        # read, which saves a clearing pass per layer.
        whole = call.writes_cache or self.gate_col is not None
        width = self.qkv_proj.out_features if whole else self.q_width
        kept_zero = rows <= kernels.SPLIT_K_MAX_ROWS
        proj = ctx.buffer("attn.proj.%s%d" % ("z" if kept_zero else "", width), (rows, width),
                          torch.float32, zero=kept_zero)
        (self.qkv_proj if whole else self.q_proj)(h, proj, out_is_zero=kept_zero)
        if whole and not call.writes_cache and kept_zero:
            proj[:, self.q_width:self.q_width + self.kv_cols].zero_()    # keys nobody consumes
        tables = self.position.rotary_tables() if self.position is not None else None
        if self.position is not None and tables is None:
            raise NotImplementedError("a position encoding that is not a rotation needs its own "
                                      "mixer")
        inv_freq, rot_dim, attn_factor = tables if tables else (None, 0, 1.0)
        angles = self.position.step_angles(ctx) if tables and hasattr(self.position, "step_angles") \
            else None
        out = ctx.buffer("attn.out", (rows, self.q_width))
        q = ctx.buffer("attn.q", (rows, self.q_width))
        plain = not self.values_are_keys and self.gate_col is None and self.chunk is None
        if plain and kernels.decode_fusion_ok(ctx, view, self.num_heads, self.num_kv_heads,
                                              self.head_dim, rot_dim, angles, self.window):
            # a step of single new tokens: norm, rotation, cache write and attention in one kernel
            kernels.attention_decode_fused(
                ctx, proj, out, view, call.writes_cache,
                self.q_norm.weight if self.q_norm is not None else None,
                self.k_norm.weight if self.k_norm is not None else None, angles,
                self.q_norm.eps if self.q_norm is not None else 0.0, kept_zero, self.num_heads,
                self.num_kv_heads, self.head_dim, self.scale, self.window)
            self.o_proj(out, x, accumulate=accumulate)
            return
        kernels.qk_norm_rope_store(
            proj, q, view.k if call.writes_cache else None,
            view.v if call.writes_cache else None, view.page_stride, view.block_table,
            ctx.row_slot, ctx.row_pos,
            self.q_norm.weight if self.q_norm is not None else None,
            self.k_norm.weight if self.k_norm is not None else None,
            inv_freq, attn_factor, self.num_heads, self.num_kv_heads, self.head_dim, rot_dim,
            view.page_size, self.q_norm.eps if self.q_norm is not None else 0.0, angles,
            clear_proj=kept_zero, values_are_keys=self.values_are_keys)
        driver.attention(ctx, q, out, view, self.num_heads, self.num_kv_heads, self.head_dim,
                         self.scale, self.mask)
        if self.gate_col is not None:
            kernels.head_gate(out, proj[:, self.gate_col:self.gate_col + self.num_heads],
                              self.num_heads, self.head_dim, clear=kept_zero)
        self.o_proj(out, x, accumulate=accumulate)


register_part("mixer", "attention", Attention, replace=True)
