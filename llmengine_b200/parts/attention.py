"""Grouped-query attention over the paged cache, with optional per-head QK norm and a
position encoding chosen by the configuration."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..config.spec import PartSpec
from ..engine.plan import Plan
from dataclasses import dataclass

from .base import (PagedAndStateSpec, PagedAndStateView, PagedKVSpec, Part, Runtime, StatesSpec, WeightSpec, build_part,
                   register_part, run_alone)


@register_part("mixer", "gqa_attention")
class GQAttention(Part):
    """q, k, v projections (no bias) -> per-head RMS norm of q and k with one gain vector each and
    `qk_norm_eps` (None = no QK norm) -> position encoding -> keys and values stored in the cache
    -> causal attention, query head h reading key/value head h // (num_heads // num_kv_heads),
    scores scaled by 1/sqrt(head_dim) -> output projection.
    (src/model/transformer_graph_builder.cpp:214-248; attention arithmetic in
    src/runtime/kernels/cpu_kernels.cpp:338-420.)

    `window` = 0 attends to every earlier key; W > 0 to the last W keys (the query's own
    included), which the reference does not have.

    The three projections are stored as one matrix [q | k | v] so that one product serves them.
    """

    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int,
                 head_dim: int, qk_norm_eps: Optional[float], position_encoding: PartSpec, window: int = 0):
        super().__init__(rt, prefix)
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} key/value heads")
        self.hidden, self.nh, self.nkv, self.hd = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.window = int(window)
        self.q_size, self.kv_size = self.nh * self.hd, self.nkv * self.hd
        self.scale = 1.0 / math.sqrt(self.hd)
        self.position = build_part("position", position_encoding, rt, prefix)
        self.w_qkv = self.w_o = self.q_gain = self.k_gain = None

    # ------------------------------------------------------------------ weights
    def weight_specs(self) -> Dict[str, WeightSpec]:
        s = {
            self.name("q_proj.weight"): WeightSpec((self.q_size, self.hidden)),
            self.name("k_proj.weight"): WeightSpec((self.kv_size, self.hidden)),
            self.name("v_proj.weight"): WeightSpec((self.kv_size, self.hidden)),
            self.name("o_proj.weight"): WeightSpec((self.hidden, self.q_size)),
        }
        if self.eps is not None:
            s[self.name("q_norm.weight")] = WeightSpec((self.hd,), role="vector", init="gain")
            s[self.name("k_norm.weight")] = WeightSpec((self.hd,), role="vector", init="gain")
        return s

    def load_weights(self, t: Dict[str, torch.Tensor]) -> None:
        self.w_qkv = torch.cat([t[self.name("q_proj.weight")], t[self.name("k_proj.weight")],
                                t[self.name("v_proj.weight")]], dim=0).contiguous()
        self.w_o = t[self.name("o_proj.weight")].contiguous()
        if self.eps is not None:
            qg, kg = t[self.name("q_norm.weight")], t[self.name("k_norm.weight")]
            if qg.dtype != kg.dtype:          # one kernel launch takes one gain type
                qg, kg = qg.float(), kg.float()
            self.q_gain, self.k_gain = qg.contiguous(), kg.contiguous()

    def cache_spec(self) -> PagedKVSpec:
        return PagedKVSpec(self.nkv, self.hd, self.window)

    # ------------------------------------------------------------------ compute
    def emit(self, plan: Plan, h: torch.Tensor, cache) -> torch.Tensor:
        """q|k|v product -> norm, position encoding, cache write, attention -> output product.  Which kernels serve
        a step (one that norms, rotates, stores and attends in one launch for steps of single tokens; the tensor-core
        kernels for prompt portions; the plain kernel) is the executor's choice, step by step."""
        rt = self.rt
        qs, kvs = self.q_size, self.kv_size
        writes = cache.writes
        width = qs + 2 * kvs if writes else qs
        qkv = rt.workspace("qkv", width, rt.dtype)
        plan.linear(h, self.w_qkv[:width], qkv)
        q = rt.workspace("q", qs, rt.dtype)
        out = rt.workspace("attn_out", qs, rt.dtype)
        scratch = rt.attention_scratch(self.nh, self.nkv, self.hd)
        common = dict(cache=cache.kv, group=cache.group, num_heads=self.nh, num_kv_heads=self.nkv, head_dim=self.hd)
        norm = dict(q_gain=self.q_gain, k_gain=self.k_gain, eps=self.eps or 0.0)
        table = self.position.rotary_table()
        if table is not None or not getattr(self.position, "needs_apply", True):
            plan.attention(qkv=qkv, q=q, out=out, writes=writes, window=self.window, scale=self.scale, cos_sin=table,
                           scratch=scratch, **common, **norm)
        else:
            # a position encoding without a rotary table: norm, then the part's own `apply`, then the write
            k = rt.workspace("k", kvs, rt.dtype) if writes else None
            plan.qkv_post(q_in=qkv[:, :qs], k_in=qkv[:, qs:qs + kvs] if writes else None, v_in=None, q_out=q, k_out=k,
                          num_heads=self.nh, num_kv_heads=self.nkv, head_dim=self.hd, **norm)
            plan.call(lambda batch: self.position.apply(rt.rows(q), rt.rows(k), batch.positions, self.nh, self.nkv),
                      f"position encoding of {self.prefix}")
            if writes:
                plan.qkv_post(q_in=None, k_in=k, v_in=qkv[:, qs + kvs:], **common)
            plan.attend(q=q, out=out, window=self.window, scale=self.scale, scratch=scratch, **common)
        delta = rt.workspace("mixer_out", self.hidden, torch.float32)
        plan.linear(out, self.w_o, delta)
        return delta

    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        plan = Plan()
        delta = self.emit(plan, h, cache)
        run_alone(self.rt, plan, batch)
        return delta[: h.shape[0]]


@dataclass
class SplitKVView:
    """The cache a run of `WindowSinkAttention` works on."""

    kv: torch.Tensor                # [pages, kv_heads * page_size * (k_dim + v_dim)]
    group: int
    writes: bool


@dataclass(frozen=True)
class SplitKVSpec:
    """Keys and values of different widths in pages: a page holds the keys of its tokens, [kv_heads, page_size, k_dim],
    and behind them the values, [kv_heads, page_size, v_dim].  `window` W > 0: only the last W positions are needed,
    and beside them the first `keep_first` positions of the request, whose pages are never given back."""

    num_kv_heads: int
    k_dim: int
    v_dim: int
    window: int = 0
    keep_first: int = 0
    paged = True

    def allocate(self, count: int, page_size: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        return torch.zeros(count, self.num_kv_heads * page_size * (self.k_dim + self.v_dim), dtype=dtype, device=device)

    def bytes_per_token(self, dtype: torch.dtype) -> int:
        return self.num_kv_heads * (self.k_dim + self.v_dim) * torch.empty((), dtype=dtype).element_size()

    def view(self, tensor: torch.Tensor, group: Optional[int], writes: bool) -> SplitKVView:
        return SplitKVView(tensor, group, writes)


@register_part("mixer", "gqa_window_sink")
class WindowSinkAttention(Part):
    """Grouped-query attention with the options of several recent designs, each a parameter:

    * query/key size `qk_dim` and value size `v_dim` per head may differ;
    * with `norm_eps`, q and k are RMS-normed over the whole projection (all heads at once) with gain vectors of that
      size, before the rotation;
    * `position_encoding`: a part that offers `frequencies()`, `dims` and `amplitude` (rotate-half pairs over the first
      `dims` coordinates of every head), or None;
    * scores are scaled by `scale`;
    * query i sees key j if j <= i and (i - j < window or j < keep_first); window 0: every earlier key;
    * with `sink`, one learned logit per head takes part in the softmax's normalisation only: p_j = exp(s_j) /
      (exp(sink_h) + sum over visible keys of exp(s_j')); nothing is attended to through it and `scale` does not apply to it;
    * `own_kv` False: the layer has no key and value projections and reads the cache of the run that the layer order
      names (keys as stored there, normed and rotated); `retain_window` / `retain_first` then say what that cache
      keeps (the widest needs among the layers that read it), which may be more than this layer's own mask.

    * `head_norm`: the norm of q and k is taken per head over its qk_dim coordinates, with gain vectors of that size
      shared by the heads, instead of over the whole projection;
    * `biases`: the q and k projections (and v, where there is one) have biases (<tensor>.b), added in the projection;
    * `values_are_keys`: there is no value projection; a token's values are its keys as projected (with the bias,
      before norm and rotation), so v_dim = qk_dim;
    * `gate` "sigmoid": the concatenated heads are multiplied by sigmoid(W_g h) (tensor g) before the output product;
      W_g reads the same input as the other projections and is stored with them as one matrix; "sigmoid_head": W_g has one
      row per head, and head a's output is multiplied by the one number sigmoid((W_g h)_a);
    * `conv_taps` K > 0: q, k and v each pass a short causal convolution per channel right behind the projection
      (tensors q.conv, k.conv, v.conv [channels, K], no bias, no activation: y_t = sum_j w[:, j] u_(t - K + 1 + j), zeros
      before the request's start); the request's last K - 1 projected values are a state beside the pages;
    * `softcap` c > 0: a score s becomes c tanh(s / c) behind the scale;
    * `unit_sink`: the softmax's denominator holds one more term of one (a sink whose logit is zero);
    * a position part with `interleaved` pairs coordinate 2i with 2i + 1.

    Tensors: q, k, v, o; q.norm, k.norm; sink; g; q.b, k.b, v.b; q.conv, k.conv, v.conv.

    Beside `emit` the part has the pieces a mixer of several branches puts together itself: `w_in` (all projections of the
    input as one matrix), `emit_heads` (from that product to the gated heads, times a constant, into a place of the
    caller's) and `w_o`."""

    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, qk_dim: int,
                 v_dim: int, scale: float, norm_eps: Optional[float] = None, position_encoding: Optional[PartSpec] = None,
                 window: int = 0, keep_first: int = 0, sink: bool = False, own_kv: bool = True,
                 retain_window: Optional[int] = None, retain_first: Optional[int] = None, head_norm: bool = False,
                 biases: bool = False, values_are_keys: bool = False, gate: Optional[str] = None, conv_taps: int = 0,
                 softcap: float = 0.0, unit_sink: bool = False):
        super().__init__(rt, prefix)
        self.taps, self.softcap, self.unit_sink = int(conv_taps), float(softcap), bool(unit_sink)
        if self.unit_sink and sink:
            raise ValueError(f"{prefix}: a learned sink and a sink of one exclude each other")
        if self.taps and (not own_kv or values_are_keys or biases or norm_eps is not None):
            raise ValueError(f"{prefix}: the convolution stands behind plain q, k and v projections of the layer's own")
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} key/value heads")
        self.hidden, self.nh, self.nkv = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dk, self.dv, self.scale = int(qk_dim), int(v_dim), float(scale)
        self.eps = None if norm_eps is None else float(norm_eps)
        self.window, self.keep_first = int(window), int(keep_first)
        self.retain_window = self.window if retain_window is None else int(retain_window)
        self.retain_first = self.keep_first if retain_first is None else int(retain_first)
        if self.retain_window and (not self.window or self.window > self.retain_window or self.keep_first > self.retain_first):
            raise ValueError(f"{prefix}: the cache keeps less than the layer's mask needs")
        self.has_sink, self.own_kv = bool(sink), bool(own_kv)
        self.head_norm, self.biases, self.values_are_keys = bool(head_norm), bool(biases), bool(values_are_keys)
        if gate not in (None, "sigmoid", "sigmoid_head"):
            raise ValueError(f"{prefix}: unknown output gate {gate!r}; known: sigmoid, sigmoid_head")
        self.gate = gate
        if self.values_are_keys and self.dv != self.dk:
            raise ValueError(f"{prefix}: values that are the keys have the keys' size, not {self.dv} against {self.dk}")
        if self.values_are_keys and not self.own_kv:
            raise ValueError(f"{prefix}: values_are_keys describes a layer with a key projection of its own")
        self.position = build_part("position", position_encoding, rt, prefix) if position_encoding is not None else None
        if self.position is not None and self.position.dims > self.dk:
            raise ValueError(f"{prefix}: {self.position.dims} rotated coordinates do not fit a head of {self.dk}")
        self.q_size, self.k_size, self.v_size = self.nh * self.dk, self.nkv * self.dk, self.nkv * self.dv
        self.o_size = self.nh * self.dv
        self.heads_size = self.o_size
        self.has_v = self.own_kv and not self.values_are_keys
        self.w_in = self.w_o = self.q_gain = self.k_gain = self.sink = None
        self.q_bias = self.k_bias = self.v_bias = self.conv_w = None
        self.gate_size = 0 if gate is None else (self.nh if gate == "sigmoid_head" else self.o_size)
        self.conv_channels = self.q_size + self.k_size + self.v_size

    def weight_specs(self) -> Dict[str, WeightSpec]:
        s = {self.name("q"): WeightSpec((self.q_size, self.hidden)), self.name("o"): WeightSpec((self.hidden, self.o_size))}
        if self.own_kv:
            s[self.name("k")] = WeightSpec((self.k_size, self.hidden))
        if self.has_v:
            s[self.name("v")] = WeightSpec((self.v_size, self.hidden))
        if self.gate is not None:
            s[self.name("g")] = WeightSpec((self.gate_size, self.hidden))
        if self.taps:
            for n, c in (("q", self.q_size), ("k", self.k_size), ("v", self.v_size)):
                s[self.name(n + ".conv")] = WeightSpec((c, self.taps), role="vector", init="unit")
        if self.eps is not None:
            s[self.name("q.norm")] = WeightSpec((self.dk if self.head_norm else self.q_size,), role="vector", init="gain")
            if self.own_kv:
                s[self.name("k.norm")] = WeightSpec((self.dk if self.head_norm else self.k_size,), role="vector", init="gain")
        if self.has_sink:
            s[self.name("sink")] = WeightSpec((self.nh,), role="vector", init="unit")
        if self.biases:
            s[self.name("q.b")] = WeightSpec((self.q_size,), role="vector")
            if self.own_kv:
                s[self.name("k.b")] = WeightSpec((self.k_size,), role="vector")
            if self.has_v:
                s[self.name("v.b")] = WeightSpec((self.v_size,), role="vector")
        return s

    def load_weights(self, t: Dict[str, torch.Tensor]) -> None:
        parts = [t[self.name("q")]] + ([t[self.name("k")]] if self.own_kv else []) + ([t[self.name("v")]] if self.has_v else [])
        if self.gate is not None:
            parts.append(t[self.name("g")])
        self.w_in = torch.cat(parts, dim=0).contiguous()
        self.w_o = t[self.name("o")].contiguous()
        if self.eps is not None:
            self.q_gain = t[self.name("q.norm")].float().contiguous()
            self.k_gain = t[self.name("k.norm")].float().contiguous() if self.own_kv else None
        self.sink = t[self.name("sink")].float().contiguous() if self.has_sink else None
        if self.unit_sink:
            self.sink = torch.zeros(self.nh, dtype=torch.float32, device=self.w_in.device)
        if self.taps:
            self.conv_w = torch.cat([t[self.name(n + ".conv")].float() for n in ("q", "k", "v")], 0).contiguous()
        if self.biases:
            self.q_bias = t[self.name("q.b")].float().contiguous()
            self.k_bias = t[self.name("k.b")].float().contiguous() if self.own_kv else None
            self.v_bias = t[self.name("v.b")].float().contiguous() if self.has_v else (self.k_bias if self.values_are_keys else None)

    @property
    def in_size(self) -> int:
        """Rows of `w_in`: the width of the product that holds every projection of the mixer's input."""
        return self.q_size + (self.k_size if self.own_kv else 0) + (self.v_size if self.has_v else 0) + self.gate_size

    def cache_spec(self):
        pages = SplitKVSpec(self.nkv, self.dk, self.dv, self.retain_window, self.retain_first)
        if not self.taps:
            return pages
        return PagedAndStateSpec(pages, StatesSpec((("conv", (max(self.taps - 1, 1), self.conv_channels)),)))

    def emit_heads(self, plan: Plan, proj: torch.Tensor, cache, out: torch.Tensor, scale: float = 1.0) -> None:
        """From `proj` = h w_in^T [T, in_size] to the heads [T, num_heads v_dim] (gated, where the layer has a gate), times
        `scale`, written to `out` (any row stride)."""
        rt = self.rt
        states = None
        if isinstance(cache, PagedAndStateView):
            cache, states = cache.paged, cache.state
        if cache.writes != self.own_kv:
            raise ValueError(f"{self.prefix}: a layer with key and value projections keeps a cache of its own, one "
                             f"without reads another layer's")
        qs, ks = self.q_size, self.k_size
        q = rt.workspace("q", qs, rt.dtype)
        src = proj
        if self.taps:
            # the convolution's results stay 32-bit up to the rotation; the finished queries and the cached keys and
            # values then take the type of the products
            if states is None:
                raise ValueError(f"{self.prefix}: the convolution needs its state beside the pages")
            src = rt.workspace("qkv_conv", self.conv_channels, torch.float32)
            plan.short_conv(x=proj[:, :self.conv_channels], w=self.conv_w, bias=None, state=states.states["conv"], out=src, act=None)
        k_in = src[:, qs:qs + ks] if self.own_kv else None
        v_in = (k_in if self.values_are_keys else src[:, qs + ks:qs + ks + self.v_size]) if self.own_kv else None
        gated = self.gate is not None
        heads = rt.workspace("attn_out", self.o_size, rt.dtype) if (gated or scale != 1.0 or not out.is_contiguous()) else out
        pos = self.position
        plan.window_attention(
            q_in=src[:, :qs], k_in=k_in, v_in=v_in,
            q_gain=self.q_gain, k_gain=self.k_gain, eps=self.eps or 0.0,
            inv_freq=pos.frequencies() if pos is not None else None, rot_dims=pos.dims if pos is not None else 0,
            amplitude=pos.amplitude if pos is not None else 1.0, q=q, out=heads, cache=cache.kv, group=cache.group,
            num_heads=self.nh, num_kv_heads=self.nkv, qk_dim=self.dk, v_dim=self.dv, window=self.window,
            keep_first=self.keep_first, scale=self.scale, sink=self.sink,
            q_bias=self.q_bias, k_bias=self.k_bias, v_bias=self.v_bias, head_norm=self.head_norm, softcap=self.softcap,
            interleaved=bool(pos is not None and getattr(pos, "interleaved", False)),
            # up to 8 key ranges per decoded token: a maximum, a sum and an output row per range and head
            scratch=(rt.buffer("window_attention_scratch", 1, rt.max_requests * self.nh * 8 * (self.dv + 2), torch.float32,
                               exact=True).view(-1) if rt.dtype == torch.bfloat16 else None))
        if gated:
            g0 = self.in_size - self.gate_size
            plan.pointwise("sigmoid_mul", heads, proj[:, g0:g0 + self.gate_size], out, scale=scale,
                           group=self.dv if self.gate == "sigmoid_head" else 1)
        elif heads is not out:
            raise ValueError(f"{self.prefix}: heads without a gate go to a dense place of their own, unscaled")

    def emit(self, plan: Plan, h: torch.Tensor, cache) -> torch.Tensor:
        rt = self.rt
        proj = rt.workspace("qkv", self.w_in.shape[0], rt.dtype)
        plan.linear(h, self.w_in, proj)
        out = rt.workspace("attn_gated" if self.gate is not None else "attn_out", self.o_size, rt.dtype)
        self.emit_heads(plan, proj, cache, out)
        delta = rt.workspace("mixer_out", self.hidden, torch.float32)
        plan.linear(out, self.w_o, delta)
        return delta

    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        plan = Plan()
        delta = self.emit(plan, h, cache)
        run_alone(self.rt, plan, batch)
        return delta[: h.shape[0]]
