"""Feed-forward parts."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..engine.plan import Plan
from .base import Part, Runtime, WeightSpec, register_part, run_alone


@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    """down( silu(gate(h)) * up(h) ), no biases; silu(g) = g / (1 + exp(-g))
    (src/model/transformer_graph_builder.cpp:261-274; src/runtime/kernels/cpu_kernels.cpp:848-859).
    The gate and up matrices are stored as one [gate | up] matrix so that one product serves both; where a
    kernel carries the activation in its epilogue the [T, 2 * intermediate] product never exists in memory."""

    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, intermediate_size: int):
        super().__init__(rt, prefix)
        self.hidden, self.inter = int(hidden_size), int(intermediate_size)
        self.w_gate_up = self.w_down = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {
            self.name("gate_proj.weight"): WeightSpec((self.inter, self.hidden)),
            self.name("up_proj.weight"): WeightSpec((self.inter, self.hidden)),
            self.name("down_proj.weight"): WeightSpec((self.hidden, self.inter)),
        }

    def load_weights(self, t: Dict[str, torch.Tensor]) -> None:
        self.w_gate_up = torch.cat([t[self.name("gate_proj.weight")], t[self.name("up_proj.weight")]], 0).contiguous()
        self.w_down = t[self.name("down_proj.weight")].contiguous()

    def emit(self, plan: Plan, h: torch.Tensor) -> torch.Tensor:
        rt = self.rt
        act = rt.workspace("act", self.inter, rt.dtype)
        gate_up = rt.workspace("gate_up", 2 * self.inter, rt.dtype)
        plan.linear_swiglu(h, self.w_gate_up, gate_up, act)
        delta = rt.workspace("ffn_out", self.hidden, torch.float32)
        plan.linear(act, self.w_down, delta)
        return delta

    def forward(self, h: torch.Tensor, batch=None) -> torch.Tensor:
        from ..engine.batch import StepBatch
        plan = Plan()
        delta = self.emit(plan, h)
        run_alone(self.rt, plan, batch if batch is not None else StepBatch.bare(h.shape[0], h.device))
        return delta[: h.shape[0]]


def _softplus32(v: torch.Tensor) -> float:
    v = v.detach().to("cpu", torch.float32)
    return float(torch.log1p(torch.exp(-v.abs())) + torch.clamp(v, min=0))


@register_part("feed_forward", "dense_xielu")
class DenseXIELU(Part):
    """down( act(up(h)) ), no biases, with the activation xIELU and its two learned numbers (p, q):
    z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2.
    The two coefficients are formed once in 32-bit when the weights are loaded and travel as constants."""

    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, intermediate_size: int):
        super().__init__(rt, prefix)
        self.hidden, self.inter = int(hidden_size), int(intermediate_size)
        self.w_up = self.w_down = None
        self.a_pos = self.a_neg = 0.0

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {
            self.name("up"): WeightSpec((self.inter, self.hidden)),
            self.name("down"): WeightSpec((self.hidden, self.inter)),
            self.name("act"): WeightSpec((2,), role="vector", init="unit"),
        }

    def load_weights(self, t: Dict[str, torch.Tensor]) -> None:
        self.w_up = t[self.name("up")].contiguous()
        self.w_down = t[self.name("down")].contiguous()
        pq = t[self.name("act")]
        self.a_pos = _softplus32(pq[0])
        self.a_neg = float(torch.tensor(0.5, dtype=torch.float32) + torch.tensor(_softplus32(pq[1]), dtype=torch.float32))

    def emit(self, plan: Plan, h: torch.Tensor) -> torch.Tensor:
        rt = self.rt
        up = rt.workspace("ffn_up", self.inter, rt.dtype)
        act = rt.workspace("act", self.inter, rt.dtype)
        plan.linear_act(h, self.w_up, up, act, "xielu", (self.a_pos, self.a_neg))
        delta = rt.workspace("ffn_out", self.hidden, torch.float32)
        plan.linear(act, self.w_down, delta)
        return delta

    def forward(self, h: torch.Tensor, batch=None) -> torch.Tensor:
        from ..engine.batch import StepBatch
        plan = Plan()
        delta = self.emit(plan, h)
        run_alone(self.rt, plan, batch if batch is not None else StepBatch.bare(h.shape[0], h.device))
        return delta[: h.shape[0]]


GATED_ACTIVATIONS = ("silu", "clamped_swish", "gelu_tanh")


@register_part("feed_forward", "gated_dense")
class GatedDense(Part):
    """down( act(gate(h), up(h)) ), tensors gate / up / down (with `biases`: every projection has one, <tensor>.b, added
    in 32-bit to the product before the activation and behind the last product), the activation a parameter:
    "silu": g sigmoid(g) u;  "clamped_swish" with `limit` (and `slope`, 1.702 unless given): g' = min(g, limit),
    u' = clamp(u, -limit, limit), g' sigmoid(slope g') (u' + 1);  "gelu_tanh": gelu(g) u with the tanh form of gelu.  The gate and up matrices are stored as one matrix so
    that one product serves both, with the activation in its epilogue where a kernel has it."""

    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, intermediate_size: int, activation: str = "silu",
                 limit: Optional[float] = None, slope: float = 1.702, biases: bool = False):
        super().__init__(rt, prefix)
        self.hidden, self.inter = int(hidden_size), int(intermediate_size)
        self.biases = bool(biases)
        self.b_gate_up = self.b_down = None
        if activation not in GATED_ACTIVATIONS:
            raise ValueError(f"{prefix}: unknown gated activation {activation!r}; known: {', '.join(GATED_ACTIVATIONS)}")
        if activation == "clamped_swish" and limit is None:
            raise ValueError(f"{prefix}: the clamped activation needs its limit")
        self.act = activation
        self.params = (float(limit), float(slope)) if activation == "clamped_swish" else ()
        self.w_gate_up = self.w_down = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        s = {self.name("gate"): WeightSpec((self.inter, self.hidden)), self.name("up"): WeightSpec((self.inter, self.hidden)),
             self.name("down"): WeightSpec((self.hidden, self.inter))}
        if self.biases:
            s[self.name("gate.b")] = WeightSpec((self.inter,), role="vector")
            s[self.name("up.b")] = WeightSpec((self.inter,), role="vector")
            s[self.name("down.b")] = WeightSpec((self.hidden,), role="vector")
        return s

    def load_weights(self, t: Dict[str, torch.Tensor]) -> None:
        self.w_gate_up = torch.cat([t[self.name("gate")], t[self.name("up")]], 0).contiguous()
        self.w_down = t[self.name("down")].contiguous()
        if self.biases:
            self.b_gate_up = torch.cat([t[self.name("gate.b")].float(), t[self.name("up.b")].float()]).contiguous()
            self.b_down = t[self.name("down.b")].float().contiguous()

    def emit(self, plan: Plan, h: torch.Tensor, out_name: str = "ffn_out") -> torch.Tensor:
        rt = self.rt
        act = rt.workspace("act", self.inter, rt.dtype)
        gate_up = rt.workspace("gate_up", 2 * self.inter, rt.dtype)
        plan.linear_swiglu(h, self.w_gate_up, gate_up, act, act=self.act, params=self.params, bias=self.b_gate_up)
        delta = rt.workspace(out_name, self.hidden, torch.float32)
        plan.linear(act, self.w_down, delta, bias=self.b_down)
        return delta

    def forward(self, h: torch.Tensor, batch=None) -> torch.Tensor:
        from ..engine.batch import StepBatch
        plan = Plan()
        delta = self.emit(plan, h)
        run_alone(self.rt, plan, batch if batch is not None else StepBatch.bare(h.shape[0], h.device))
        return delta[: h.shape[0]]


@register_part("feed_forward", "routed_experts")
class RoutedExperts(Part):
    """A mixture of `num_experts` small feed-forwards down(silu(gate h) * (up h)) of which every token uses `top_k`:
    z = W_router h (+ a bias with `router_bias`) in 32-bit.  `routing` "sigmoid": s = sigmoid(z), C = the `top_k` experts of
    largest s, w_e = route_scale * s_e / (sum over C of s + 1e-20); "softmax_chosen": C = the experts of largest z and w_e =
    route_scale * softmax over the chosen logits alone.  Output = sum over C of w_e expert_e(h), plus, with `shared_size` > 0,
    one more expert of that size that takes every token, with weight one or, with `shared_gate`, with weight
    sigmoid(W_sg h), one number a token.  Tensors: router (router.b); e<i>.gate / up / down; shared.gate / up / down
    (shared.sg [1, hidden]).

    The experts' matrices are stacked ([E, 2 ff, D] and [E, D, ff]) and run as two grouped products over the
    (token, choice) pairs listed expert by expert; the pairs' outputs are combined per token in the order of the
    choices, so a token's result does not depend on what else is in the step.  The shared expert's gate is one more row
    of the router's matrix, so one product gives both."""

    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, num_experts: int, top_k: int, expert_size: int,
                 route_scale: float = 1.0, shared_size: int = 0, routing: str = "sigmoid", router_bias: bool = False,
                 shared_gate: bool = False):
        super().__init__(rt, prefix)
        self.hidden, self.E, self.top, self.ff = int(hidden_size), int(num_experts), int(top_k), int(expert_size)
        if not 0 < self.top <= self.E:
            raise ValueError(f"{prefix}: {self.top} of {self.E} experts cannot be chosen")
        if routing not in ("sigmoid", "softmax_chosen"):
            raise ValueError(f"{prefix}: unknown routing {routing!r}; known: sigmoid, softmax_chosen")
        self.route_scale, self.routing, self.router_bias = float(route_scale), routing, bool(router_bias)
        self.shared = (GatedDense(rt, self.name("shared"), hidden_size, int(shared_size)) if shared_size else None)
        self.shared_gate = bool(shared_gate)
        if self.shared_gate and self.shared is None:
            raise ValueError(f"{prefix}: a gate on the shared expert needs a shared expert")
        self.w_router = self.w_gate_up = self.w_down = self.b_router = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        s = {self.name("router"): WeightSpec((self.E, self.hidden))}
        if self.router_bias:
            s[self.name("router.b")] = WeightSpec((self.E,), role="vector")
        for e in range(self.E):
            s[self.name(f"e{e}.gate")] = WeightSpec((self.ff, self.hidden))
            s[self.name(f"e{e}.up")] = WeightSpec((self.ff, self.hidden))
            s[self.name(f"e{e}.down")] = WeightSpec((self.hidden, self.ff))
        if self.shared is not None:
            s.update(self.shared.weight_specs())
        if self.shared_gate:
            s[self.name("shared.sg")] = WeightSpec((1, self.hidden))
        return s

    def load_weights(self, t: Dict[str, torch.Tensor]) -> None:
        rows = [t[self.name("router")]] + ([t[self.name("shared.sg")]] if self.shared_gate else [])
        used = sum(r.shape[0] for r in rows)
        pad = -used % 8                 # rows of zeros up to a multiple of 8: the product's 32-bit output rows then start on 32 bytes
        if pad:
            rows.append(rows[0].new_zeros(pad, self.hidden))
        self.w_router = torch.cat(rows, 0).contiguous()
        if self.router_bias:
            b = t[self.name("router.b")].float()
            self.b_router = torch.cat([b, b.new_zeros(self.w_router.shape[0] - self.E)]).contiguous()
        self.w_gate_up = torch.stack([torch.cat([t[self.name(f"e{e}.gate")], t[self.name(f"e{e}.up")]], 0)
                                      for e in range(self.E)]).contiguous()
        self.w_down = torch.stack([t[self.name(f"e{e}.down")] for e in range(self.E)]).contiguous()
        if self.shared is not None:
            self.shared.load_weights({n: t[n] for n in self.shared.weight_specs()})

    def emit(self, plan: Plan, h: torch.Tensor) -> torch.Tensor:
        rt = self.rt
        T, E, top = rt.max_tokens, self.E, self.top
        wide = rt.workspace("router_logits", self.w_router.shape[0], torch.float32)    # [logits | gate of the shared expert]
        plan.linear(h, self.w_router, wide, bias=self.b_router)
        logits = wide[:, :E]
        experts = rt.workspace("route_experts", top, torch.int32)
        weights = rt.workspace("route_weights", top, torch.float32)
        offsets = rt.buffer("route_offsets", 1, E + 1, torch.int32, exact=True, zero=True).view(-1)
        counts = rt.buffer("route_counts", 1, E, torch.int32, exact=True, zero=True).view(-1)
        order = rt.buffer("route_order", T * top, 1, torch.int32).view(-1)
        plan.moe_route(logits=logits, top_k=top, scale=self.route_scale, experts=experts, weights=weights,
                       offsets=offsets, order=order, counts=counts, mode=self.routing)
        act = rt.buffer("expert_act", T * top, self.ff, rt.dtype)
        mid = rt.buffer("expert_gate_up", T * top, 2 * self.ff, rt.dtype)
        plan.grouped_linear(x=h, w=self.w_gate_up, out=act, offsets=offsets, order=order, top_k=top, gather=True,
                            scatter=False, mid=mid, act="silu")
        y = rt.buffer("expert_out", T * top, self.hidden, torch.float32)
        plan.grouped_linear(x=act, w=self.w_down, out=y, offsets=offsets, order=order, top_k=top, gather=False, scatter=True)
        base = self.shared.emit(plan, h, out_name="shared_out") if self.shared is not None else None
        delta = rt.workspace("ffn_out", self.hidden, torch.float32)
        plan.moe_combine(y=y, weights=weights, base=base, out=delta, base_gate=wide[:, E:E + 1] if self.shared_gate else None)
        return delta

    def forward(self, h: torch.Tensor, batch=None) -> torch.Tensor:
        from ..engine.batch import StepBatch
        plan = Plan()
        delta = self.emit(plan, h)
        run_alone(self.rt, plan, batch if batch is not None else StepBatch.bare(h.shape[0], h.device))
        return delta[: h.shape[0]]
