"""Mixers that carry a state of fixed size per request, and the mixer that runs several mixers side by side.

* `StateSpaceMixer` (kind `state_space`): a selective state space.  One product gives [z | x | B | C | dt]; x, B and C
  pass a short causal convolution per channel and silu; d_t = softplus(dt_t + dt_bias); per head a (whose B and C are
  those of group a // (heads / groups)):  S_t = exp(-exp(A_log_a) d_t) S_(t-1) + d_t B_t x_t^T,  y_t = S_t^T C_t + D_a x_t;
  y silu(z) is RMS-normed in `norm_groups` equal parts, times a weight vector, and projected.  State per request: the
  matrices S (32-bit) and the convolution's last taps - 1 inputs.
* `Retention` (kind `retention`): linear attention with a fixed decay per head, no softmax and no denominator.
  q, k, v and a gate come from one product; q and k are rotated by position, k then times qk_dim^(-1/2);
  S_t = decay_a S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t;  every head's o is divided by its root mean square, the heads are
  multiplied by silu(gate) and projected.  State per request: the matrices S (32-bit).
* `MatrixMemory` (kind `matrix_memory`): a matrix memory with exponential input and forget gates, kept in range by a running
  maximum of the gates' logarithms.  Per head: q = W_q h / sqrt(d), k = W_k h, v = W_v h; log gates a_t = cap tanh((W_i h +
  b_i) / cap) and b_t = logsigmoid(cap tanh((W_f h + b_f) / cap)); M_t = max(b_t + M_(t-1), a_t), M_0 = 0;
  S_t = exp(b_t + M_(t-1) - M_t) S_(t-1) + exp(a_t - M_t) k_t v_t^T and n_t the same with k_t alone;
  o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-M_t)) + 1e-6); every head's o is divided by its root mean square, the heads are
  multiplied by a weight vector and by sigmoid(W_g h), and projected.  State per request: S and n (n is one more column of
  S, whose v is one) and M, all 32-bit.
* `ParallelMixer` (kind `parallel`): branches that read the same input; the result is sum_b scale_b branch_b(h).  The
  branches' input projections are ONE product, and so are their output projections: every branch writes its gated heads,
  times its scale, into its columns of one row, and the output matrices stand side by side.

Everything that enters a recurrence is 32-bit in both precisions: rotated q and k, the convolution's outputs, step sizes and
decays, the state, the outputs and their norms.  The products and the gates take the engine's product type.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence, Tuple

import torch

from ..config.spec import PartSpec
from ..engine.plan import Plan
from .base import (PagedAndStateSpec, PagedAndStateView, Part, Runtime, StatesSpec, StatesView, WeightSpec, build_part,
                   register_part, run_alone)


@register_part("mixer", "state_space")
class StateSpaceMixer(Part):
    """Tensors: in [2 inner + 2 groups state + heads, hidden] with inner = heads head_dim; conv [inner + 2 groups state, taps]
    and conv.b; dt_bias, A_log, D [heads]; norm [inner]; o [hidden, inner].  The last column of `conv` meets the present
    token, the one before it the token before, and so on; before a request's start the inputs are zero."""

    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, num_heads: int, head_dim: int, state_size: int, groups: int,
                 taps: int, norm_groups: int, norm_eps: float):
        super().__init__(rt, prefix)
        self.hidden, self.nh, self.p, self.n = int(hidden_size), int(num_heads), int(head_dim), int(state_size)
        self.groups, self.taps, self.norm_groups, self.eps = int(groups), int(taps), int(norm_groups), float(norm_eps)
        if self.nh % self.groups:
            raise ValueError(f"{prefix}: {self.nh} heads are not a multiple of {self.groups} groups")
        self.inner = self.nh * self.p
        if self.inner % self.norm_groups:
            raise ValueError(f"{prefix}: {self.norm_groups} norm groups do not divide {self.inner} channels")
        if self.taps < 1:
            raise ValueError(f"{prefix}: a convolution needs at least one tap")
        self.bc = self.groups * self.n
        self.conv_channels = self.inner + 2 * self.bc
        self.in_size = 2 * self.inner + 2 * self.bc + self.nh
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.skip = self.norm_w = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        v = lambda n, init="normal": WeightSpec((n,), role="vector", init=init)
        return {self.name("in"): WeightSpec((self.in_size, self.hidden)), self.name("o"): WeightSpec((self.hidden, self.inner)),
                self.name("conv"): WeightSpec((self.conv_channels, self.taps), role="vector", init="unit"),
                self.name("conv.b"): v(self.conv_channels), self.name("dt_bias"): v(self.nh, "unit"),
                self.name("A_log"): v(self.nh, "unit"), self.name("D"): v(self.nh, "gain"), self.name("norm"): v(self.inner, "gain")}

    def load_weights(self, t: Dict[str, torch.Tensor]) -> None:
        f = lambda n: t[self.name(n)].float().contiguous()
        self.w_in, self.w_o = t[self.name("in")].contiguous(), t[self.name("o")].contiguous()
        self.conv_w, self.conv_b, self.dt_bias, self.a_log, self.skip, self.norm_w = (f("conv"), f("conv.b"), f("dt_bias"), f("A_log"),
                                                                                     f("D"), f("norm"))

    def cache_spec(self) -> StatesSpec:
        return StatesSpec((("conv", (max(self.taps - 1, 1), self.conv_channels)), ("state", (self.nh, self.p, self.n))))

    def emit(self, plan: Plan, h: torch.Tensor, cache: StatesView) -> torch.Tensor:
        rt, inner, bc = self.rt, self.inner, self.bc
        proj = rt.workspace("ssm_in", self.in_size, rt.dtype)
        plan.linear(h, self.w_in, proj)
        xbc = rt.workspace("ssm_conv", self.conv_channels, torch.float32)
        plan.short_conv(x=proj[:, inner:inner + self.conv_channels], w=self.conv_w, bias=self.conv_b, state=cache.states["conv"],
                        out=xbc, act="silu")
        y = rt.workspace("ssm_y", inner, torch.float32)
        plan.recurrence(q=xbc[:, inner + bc:], k=xbc[:, inner:inner + bc], v=xbc[:, :inner], state=cache.states["state"], out=y,
                        heads=self.nh, n=self.n, p=self.p, qk_groups=self.groups, dt=proj[:, inner + self.conv_channels:],
                        dt_bias=self.dt_bias, a_log=self.a_log, skip=self.skip,
                        scratch=rt.recurrence_scratch(self.nh, self.p, self.n))
        gated = rt.workspace("ssm_gated", inner, rt.dtype)
        plan.gated_norm(y=y, gate=proj[:, :inner], weight=self.norm_w, out=gated, group=inner // self.norm_groups, gate_first=True,
                        eps=self.eps)
        delta = rt.workspace("mixer_out", self.hidden, torch.float32)
        plan.linear(gated, self.w_o, delta)
        return delta

    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        plan = Plan()
        buf = self.rt.workspace("normed", self.hidden, self.rt.dtype)
        buf[: h.shape[0]].copy_(h)
        delta = self.emit(plan, buf, cache)
        run_alone(self.rt, plan, batch)
        return delta[: h.shape[0]]


@register_part("mixer", "retention")
class Retention(Part):
    """Tensors: q, k [heads qk_dim, hidden]; v, g [heads v_dim, hidden]; o [hidden, heads v_dim]; no biases.  `decay` lists
    one number per head.  Beside `emit` the part has the pieces a mixer of several branches puts together itself: `w_in`,
    `emit_heads` and `w_o`."""

    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, num_heads: int, qk_dim: int, v_dim: int, decay: Sequence[float],
                 norm_eps: float, position_encoding: Optional[PartSpec] = None):
        super().__init__(rt, prefix)
        self.hidden, self.nh, self.dk, self.dv, self.eps = int(hidden_size), int(num_heads), int(qk_dim), int(v_dim), float(norm_eps)
        if len(decay) != self.nh:
            raise ValueError(f"{prefix}: {len(decay)} decays for {self.nh} heads")
        self.decay_values = tuple(float(d) for d in decay)
        self.position = build_part("position", position_encoding, rt, prefix) if position_encoding is not None else None
        if self.position is not None and self.position.dims > self.dk:
            raise ValueError(f"{prefix}: {self.position.dims} rotated coordinates do not fit a head of {self.dk}")
        self.qk_size, self.heads_size = self.nh * self.dk, self.nh * self.dv
        self.in_size = 2 * self.qk_size + 2 * self.heads_size
        self.w_in = self.w_o = self.decay = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.name("q"): WeightSpec((self.qk_size, self.hidden)), self.name("k"): WeightSpec((self.qk_size, self.hidden)),
                self.name("v"): WeightSpec((self.heads_size, self.hidden)), self.name("g"): WeightSpec((self.heads_size, self.hidden)),
                self.name("o"): WeightSpec((self.hidden, self.heads_size))}

    def load_weights(self, t: Dict[str, torch.Tensor]) -> None:
        self.w_in = torch.cat([t[self.name(n)] for n in ("q", "k", "v", "g")], 0).contiguous()
        self.w_o = t[self.name("o")].contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.w_in.device)

    def cache_spec(self) -> StatesSpec:
        return StatesSpec((("state", (self.nh, self.dv, self.dk)),))

    def emit_heads(self, plan: Plan, proj: torch.Tensor, cache: StatesView, out: torch.Tensor, scale: float = 1.0) -> None:
        """From `proj` = h w_in^T [T, in_size] to the normed and gated heads [T, heads v_dim], times `scale`, into `out`."""
        rt, qs, hs = self.rt, self.qk_size, self.heads_size
        q32 = rt.workspace("retention_q", qs, torch.float32)
        k32 = rt.workspace("retention_k", qs, torch.float32)
        pos = self.position
        plan.rotate(x=(proj[:, :qs], proj[:, qs:2 * qs]), out=(q32, k32), heads=(self.nh, self.nh), scale=(1.0, float(self.dk) ** -0.5),
                    dim=self.dk, rot_dims=pos.dims if pos is not None else 0, inv_freq=pos.frequencies() if pos is not None else None)
        o = rt.workspace("retention_o", hs, torch.float32)
        plan.recurrence(q=q32, k=k32, v=proj[:, 2 * qs:2 * qs + hs], state=cache.states["state"], out=o, heads=self.nh, n=self.dk,
                        p=self.dv, qk_groups=self.nh, decay=self.decay, scratch=rt.recurrence_scratch(self.nh, self.dv, self.dk))
        plan.gated_norm(y=o, gate=proj[:, 2 * qs + hs:2 * qs + 2 * hs], weight=None, out=out, group=self.dv, gate_first=False,
                        eps=self.eps, scale=scale)

    def emit(self, plan: Plan, h: torch.Tensor, cache: StatesView) -> torch.Tensor:
        rt = self.rt
        proj = rt.workspace("retention_in", self.in_size, rt.dtype)
        plan.linear(h, self.w_in, proj)
        heads = rt.workspace("retention_heads", self.heads_size, rt.dtype)
        self.emit_heads(plan, proj, cache, heads)
        delta = rt.workspace("mixer_out", self.hidden, torch.float32)
        plan.linear(heads, self.w_o, delta)
        return delta

    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        plan = Plan()
        buf = self.rt.workspace("normed", self.hidden, self.rt.dtype)
        buf[: h.shape[0]].copy_(h)
        delta = self.emit(plan, buf, cache)
        run_alone(self.rt, plan, batch)
        return delta[: h.shape[0]]


@register_part("mixer", "matrix_memory")
class MatrixMemory(Part):
    """Tensors: q, k [heads qk_dim, hidden]; v, g [heads v_dim, hidden]; i, f [heads, hidden] with biases i.b, f.b; norm
    [heads v_dim]; o [hidden, heads v_dim].  `gate_cap` 0: the gates' pre-activations are not capped.  q, k, v and g are one
    product in the type of the products; the gates' pre-activations are a second, small one whose result is 32-bit."""

    DEN_EPS = 1e-6                       # what the design adds to the denominator max(|n . q|, exp(-M))

    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, num_heads: int, qk_dim: int, v_dim: int, gate_cap: float,
                 norm_eps: float):
        super().__init__(rt, prefix)
        self.hidden, self.nh, self.dk, self.dv = int(hidden_size), int(num_heads), int(qk_dim), int(v_dim)
        self.cap, self.eps = float(gate_cap), float(norm_eps)
        self.qk_size, self.heads_size = self.nh * self.dk, self.nh * self.dv
        self.in_size = 2 * self.qk_size + 2 * self.heads_size
        self.w_in = self.w_gates = self.b_gates = self.w_o = self.norm_w = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        v = lambda n, init="normal": WeightSpec((n,), role="vector", init=init)
        return {self.name("q"): WeightSpec((self.qk_size, self.hidden)), self.name("k"): WeightSpec((self.qk_size, self.hidden)),
                self.name("v"): WeightSpec((self.heads_size, self.hidden)), self.name("g"): WeightSpec((self.heads_size, self.hidden)),
                self.name("o"): WeightSpec((self.hidden, self.heads_size)), self.name("norm"): v(self.heads_size, "gain"),
                self.name("i"): WeightSpec((self.nh, self.hidden)), self.name("i.b"): v(self.nh, "unit"),
                self.name("f"): WeightSpec((self.nh, self.hidden)), self.name("f.b"): v(self.nh, "unit")}

    def load_weights(self, t: Dict[str, torch.Tensor]) -> None:
        self.w_in = torch.cat([t[self.name(n)] for n in ("q", "k", "v", "g")], 0).contiguous()
        self.w_gates = torch.cat([t[self.name("i")], t[self.name("f")]], 0).contiguous()
        self.b_gates = torch.cat([t[self.name("i.b")].float(), t[self.name("f.b")].float()]).contiguous()
        self.w_o = t[self.name("o")].contiguous()
        self.norm_w = t[self.name("norm")].float().contiguous()

    def cache_spec(self) -> StatesSpec:
        return StatesSpec((("state", (self.nh, self.dv + 1, self.dk)), ("max", (self.nh,))))

    def emit(self, plan: Plan, h: torch.Tensor, cache: StatesView) -> torch.Tensor:
        rt, H, qs, hs = self.rt, self.nh, self.qk_size, self.heads_size
        proj = rt.workspace("memory_in", self.in_size, rt.dtype)
        plan.linear(h, self.w_in, proj)
        pre = rt.workspace("memory_gates_in", 2 * H, torch.float32)
        plan.linear(h, self.w_gates, pre, bias=self.b_gates)
        gates = rt.workspace("memory_gates", 3 * H, torch.float32)          # [keep | take | floor]
        plan.exp_gates(i_pre=pre[:, :H], f_pre=pre[:, H:], cap=self.cap, state=cache.states["max"], keep=gates[:, :H],
                       take=gates[:, H:2 * H], floor=gates[:, 2 * H:])
        q32 = rt.workspace("memory_q", qs, torch.float32)
        k32 = rt.workspace("memory_k", qs, torch.float32)
        plan.rotate(x=(proj[:, :qs], proj[:, qs:2 * qs]), out=(q32, k32), heads=(H, H), scale=(float(self.dk) ** -0.5, 1.0),
                    dim=self.dk, rot_dims=0, inv_freq=None)
        o = rt.workspace("memory_o", H * (self.dv + 1), torch.float32)
        plan.recurrence(q=q32, k=k32, v=proj[:, 2 * qs:2 * qs + hs], state=cache.states["state"], out=o, heads=H, n=self.dk,
                        p=self.dv + 1, qk_groups=H, keep=gates[:, :H], take=gates[:, H:2 * H], unit_column=True,
                        scratch=rt.recurrence_scratch(H, self.dv + 1, self.dk))
        heads = rt.workspace("memory_heads", hs, rt.dtype)
        plan.gated_norm(y=o, gate=proj[:, 2 * qs + hs:], weight=self.norm_w, out=heads, group=self.dv, gate_first=False,
                        eps=self.eps, gate_act="sigmoid", floor=gates[:, 2 * H:], den_eps=self.DEN_EPS)
        delta = rt.workspace("mixer_out", self.hidden, torch.float32)
        plan.linear(heads, self.w_o, delta)
        return delta

    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        plan = Plan()
        buf = self.rt.workspace("normed", self.hidden, self.rt.dtype)
        buf[: h.shape[0]].copy_(h)
        delta = self.emit(plan, buf, cache)
        run_alone(self.rt, plan, batch)
        return delta[: h.shape[0]]


@register_part("mixer", "parallel")
class ParallelMixer(Part):
    """`branches`: (name, PartSpec of a mixer, scale) triples; branch b's tensors lie under `<prefix>.<name>`.  A branch is
    any mixer that offers `w_in` / `in_size` (all its projections of the input as one matrix), `heads_size`, `w_o` and
    `emit_heads(plan, proj, cache, out, scale)`.  At most one branch keeps pages; the branches with states share the
    run's state row."""

    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, branches: Sequence[Tuple[str, PartSpec, float]]):
        super().__init__(rt, prefix)
        self.hidden = int(hidden_size)
        if not branches:
            raise ValueError(f"{prefix}: a parallel mixer needs a branch")
        self.names = tuple(str(b[0]) for b in branches)
        self.scales = tuple(float(b[2]) for b in branches)
        self.branches = tuple(build_part("mixer", b[1], rt, self.name(b[0])) for b in branches)
        for n, b in zip(self.names, self.branches):
            if not all(hasattr(b, a) for a in ("in_size", "heads_size", "emit_heads")):
                raise ValueError(f"{prefix}: the mixer of branch {n!r} cannot stand beside others (no emit_heads)")
        self._specs = [b.cache_spec() for b in self.branches]
        if sum(1 for s in self._specs if s is not None and getattr(s, "paged", False)) > 1:
            raise ValueError(f"{prefix}: more than one branch keeps pages")
        for s in self._specs:
            if s is not None and not getattr(s, "paged", False) and not isinstance(s, StatesSpec):
                raise ValueError(f"{prefix}: a branch with a state describes it as named states")
        self.w_in = self.w_o = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        out: Dict[str, WeightSpec] = {}
        for b in self.branches:
            out.update(b.weight_specs())
        return out

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for b in self.branches:
            b.load_weights({n: tensors[n] for n in b.weight_specs()})
        self.w_in = torch.cat([b.w_in for b in self.branches], 0).contiguous()
        self.w_o = torch.cat([b.w_o for b in self.branches], 1).contiguous()
        at_in = at_out = 0
        for b in self.branches:                         # the branches keep views of the joint matrices, not copies
            b.w_in, b.w_o = self.w_in[at_in:at_in + b.in_size], self.w_o[:, at_out:at_out + b.heads_size]
            at_in, at_out = at_in + b.in_size, at_out + b.heads_size

    def cache_spec(self):
        paged = [s for s in self._specs if s is not None and getattr(s, "paged", False)]
        states = tuple((f"{n}.{name}", shape) for n, s in zip(self.names, self._specs) if isinstance(s, StatesSpec)
                       for name, shape in s.parts)
        state = StatesSpec(states) if states else None
        if paged and state is not None:
            return PagedAndStateSpec(paged[0], state)
        return paged[0] if paged else state

    def _branch_caches(self, cache):
        """What each branch is handed: the pages for the branch that keeps pages, its own states (under their own names)
        for a branch with states."""
        paged = cache.paged if isinstance(cache, PagedAndStateView) else (None if isinstance(cache, StatesView) else cache)
        states = cache.state if isinstance(cache, PagedAndStateView) else (cache if isinstance(cache, StatesView) else None)
        out = []
        for n, s in zip(self.names, self._specs):
            if s is None:
                out.append(None)
            elif getattr(s, "paged", False):
                out.append(paged)
            else:
                out.append(StatesView({name: states.states[f"{n}.{name}"] for name, _ in s.parts}))
        return out

    def emit(self, plan: Plan, h: torch.Tensor, cache) -> torch.Tensor:
        rt = self.rt
        proj = rt.workspace("parallel_in", self.w_in.shape[0], rt.dtype)
        plan.linear(h, self.w_in, proj)
        heads = rt.workspace("parallel_heads", self.w_o.shape[1], rt.dtype)
        at_in = at_out = 0
        for b, c, scale in zip(self.branches, self._branch_caches(cache), self.scales):
            b.emit_heads(plan, proj[:, at_in:at_in + b.in_size], c, heads[:, at_out:at_out + b.heads_size], scale)
            at_in, at_out = at_in + b.in_size, at_out + b.heads_size
        delta = rt.workspace("mixer_out", self.hidden, torch.float32)
        plan.linear(heads, self.w_o, delta)
        return delta

    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        plan = Plan()
        buf = self.rt.workspace("normed", self.hidden, self.rt.dtype)
        buf[: h.shape[0]].copy_(h)
        delta = self.emit(plan, buf, cache)
        run_alone(self.rt, plan, batch)
        return delta[: h.shape[0]]
