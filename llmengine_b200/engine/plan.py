"""A model's launch sequence as data: the operation records that the parts emit when a model is loaded.

A `Plan` is a list of records; each record names an operation and holds the tensors it works on: weights, and
workspace buffers made for the step's token budget (a step uses their first rows).  Nothing in a record
depends on a step: how many tokens, which requests decode and where their pages lie comes with the step.  The
kernel set compiles a plan once (`ops.compile(plan)`): on the GPU into the native executor's records
(include/llmengine_b200/executor.h), which are walked in C++ for every step; in the host tests into a list that a
CPU stand-in interprets.  Either way the parts emit their operations once, in one place.

The reference walks a graph of nodes in topological order and looks the kernel of every node up per run
(src/runtime/executor.cpp:112-142); a plan is that order fixed at load time.

A part written outside this package needs no record kind of its own: `Plan.call(fn)` makes a record that calls
`fn(batch)` in its turn, on the same stream, with the step's batch.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional

import torch

ROWS_TOKENS, ROWS_LOGITS = "tokens", "logits"


@dataclass
class Op:
    kind: str
    a: Dict[str, Any] = field(default_factory=dict)


class Plan:
    def __init__(self) -> None:
        self.ops: List[Op] = []
        self._copies: Dict[int, torch.Tensor] = {}     # address of a 32-bit tensor -> its present copy in the product type

    # A part whose sublayers read the residual stream itself needs it in the type of the matrix products.  The record
    # that last changed the stream may have written that copy in the same pass; it says so here, and a record that
    # changes the stream without doing so withdraws it.
    def note_copy(self, x: torch.Tensor, copy: Optional[torch.Tensor]) -> None:
        if copy is None:
            self._copies.pop(x.data_ptr(), None)
        else:
            self._copies[x.data_ptr()] = copy

    def copy_of(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        return self._copies.get(x.data_ptr())

    def _add(self, kind: str, **a: Any) -> None:
        self.ops.append(Op(kind, a))

    def embedding(self, table: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
        """out[t] = table[token_ids[t]] * scale as 32-bit, for the step's tokens."""
        self._add("embedding", table=table, out=out, scale=float(scale))

    def rmsnorm(self, x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor,
                delta: Optional[torch.Tensor] = None, rows: str = ROWS_TOKENS, gain2: Optional[torch.Tensor] = None,
                out2: Optional[torch.Tensor] = None) -> None:
        """x += delta (if given), out = rmsnorm(x) * gain; `rows` = "logits": only the step's wanted rows,
        gathered into the first rows of `out`.  With `gain2` and `out2` (the types of `gain` and `out`) the same normed
        rows also go, times the second gain, to the second place: two norms of the same x in one pass."""
        self._add("rmsnorm", x=x, gain=gain, eps=float(eps), out=out, delta=delta, rows=rows, gain2=gain2, out2=out2)
        if delta is not None:
            self.note_copy(x, None)

    def linear(self, x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor], rows: str = ROWS_TOKENS,
               bias: Optional[torch.Tensor] = None) -> None:
        """out = x w^T (+ bias, a 32-bit vector) for the step's tokens (or its wanted rows); `out` None: the step's logits."""
        self._add("linear", x=x, w=w, out=out, rows=rows, bias=bias)

    def linear_swiglu(self, x: torch.Tensor, w_gate_up: torch.Tensor, gate_up: torch.Tensor, out: torch.Tensor,
                      act: str = "silu", params: tuple = (), bias: Optional[torch.Tensor] = None) -> None:
        """out = act(x Wg^T + bg, x Wu^T + bu) with w_gate_up = [Wg | Wu] by rows (`bias` = [bg | bu], 32-bit, or None); `gate_up` is the workspace of the form
        that runs the product and the activation as two kernels.  Gated activations of (g, u):
        "silu": g sigmoid(g) u;  "clamped_swish" with params (limit, slope): g' = min(g, limit),
        u' = clamp(u, -limit, limit), g' sigmoid(slope g') (u' + 1)."""
        self._add("linear_swiglu", x=x, w_gate_up=w_gate_up, gate_up=gate_up, out=out, act=act,
                  params=tuple(float(p) for p in params), bias=bias)

    def qkv_post(self, *, q_in, k_in, v_in, num_heads: int, num_kv_heads: int, head_dim: int, q_gain=None, k_gain=None,
                 eps: float = 0.0, cos_sin=None, q_out=None, k_out=None, cache=None, group: int = 0) -> None:
        """Per-head norm (with gains), rotation (with a table) and cache write (with a cache) of what is given."""
        self._add("qkv_post", q_in=q_in, k_in=k_in, v_in=v_in, num_heads=num_heads, num_kv_heads=num_kv_heads,
                  head_dim=head_dim, q_gain=q_gain, k_gain=k_gain, eps=float(eps), cos_sin=cos_sin, q_out=q_out,
                  k_out=k_out, cache=cache, group=group)

    def attend(self, *, q, out, cache, group: int, num_heads: int, num_kv_heads: int, head_dim: int, window: int,
               scale: float, scratch=None) -> None:
        """Attention of every token of the step over its request's cache; queries finished."""
        self._add("attend", q=q, out=out, cache=cache, group=group, num_heads=num_heads, num_kv_heads=num_kv_heads,
                  head_dim=head_dim, window=window, scale=float(scale), scratch=scratch)

    def attention(self, *, qkv, q, out, cache, writes: bool, group: int, num_heads: int, num_kv_heads: int, head_dim: int,
                  window: int, scale: float, q_gain=None, k_gain=None, eps: float = 0.0, cos_sin=None, scratch=None) -> None:
        """From the raw q|k|v projections to the attention output: norm, rotation (cos_sin None: none), cache write
        (if `writes`) and attention; the executor fuses them where a kernel does all of it."""
        self._add("attention", qkv=qkv, q=q, out=out, cache=cache, writes=bool(writes), group=group, num_heads=num_heads,
                  num_kv_heads=num_kv_heads, head_dim=head_dim, window=window, scale=float(scale), q_gain=q_gain,
                  k_gain=k_gain, eps=float(eps), cos_sin=cos_sin, scratch=scratch)

    def call(self, fn: Callable[[Any], None], what: str = "") -> None:
        """`fn(batch)` is called in its turn with the step's `StepBatch`, on the step's stream."""
        self._add("call", fn=fn, what=what)

    def linear_act(self, x: torch.Tensor, w: torch.Tensor, mid: torch.Tensor, out: torch.Tensor, act: str,
                   params: tuple = ()) -> None:
        """out = act(x w^T), elementwise; `mid` is the workspace of the form that runs product and activation as two
        kernels.  Activations: "xielu" with params (a_pos, a_neg): z > 0: a_pos z^2 + z/2, else a_neg (exp(z) - 1 - z) + z/2."""
        self._add("linear_act", x=x, w=w, mid=mid, out=out, act=act, params=tuple(float(p) for p in params))

    def pointwise(self, kind: str, a: torch.Tensor, b: Optional[torch.Tensor], out: torch.Tensor, scale: float = 1.0,
                  group: int = 1) -> None:
        """Elementwise over the step's rows (row strides free).  "sigmoid_mul": out = a * sigmoid(b) * scale; with
        `group` > 1, b has one value for every `group` neighbouring columns of a (a gate per head)."""
        self._add("pointwise", what=kind, a=a, b=b, out=out, scale=float(scale), group=int(group))

    def batched_linear(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
        """out[t, b, :] = w[b] x[t, b, :] for every batch member b (one small matrix per head): x [T, B, k] and
        out [T, B, n] are views with free row and member strides, w is [B, n, k]."""
        self._add("batched_linear", x=x, w=w, out=out)

    def residual_add(self, x: torch.Tensor, a: torch.Tensor, b: Optional[torch.Tensor] = None,
                     a_scale: Optional[torch.Tensor] = None, b_scale: Optional[torch.Tensor] = None) -> None:
        """x += a (+ b) in 32-bit: contributions that no following norm adds.  With `a_scale` / `b_scale` (32-bit vectors
        of the stream's width) each contribution is multiplied by its vector, column by column, before the sum."""
        self._add("residual_add", x=x, a=a, b=b, a_scale=a_scale, b_scale=b_scale)
        self.note_copy(x, None)

    def latent_attention(self, *, q_rot, kv_in, c_gain, eps: float, inv_freq, rot_dims: int, q, out, cache, group: int,
                         num_heads: int, kv_rank: int, rot_dim: int, scale: float, sink=None, scratch=None, window: int = 0,
                         interleaved: bool = False) -> None:
        """Attention over a cache of latents, one row [c | rotated key part] per token, shared by all heads.
        `kv_in` [T, kv_rank + rot_dim] is the raw down-projection: its first kv_rank values are RMS-normed with
        `c_gain`, the rest rotated by the token's position (`inv_freq`: rot_dims / 2 frequencies; none: no positions),
        and the row is stored.  `q` [T, H, kv_rank + rot_dim] holds each head's query against the latent already;
        its last rot_dim values are filled here from `q_rot` [T, H, rot_dim] (a strided view), rotated.  Then
        score = (q . row) * scale, causal (with `window` W > 0 query i sees key j only if i - j < W), softmax (with `sink`
        [H]: the denominator also holds exp(sink_h)), and out[t, h, :] = sum_j w_j c_j  [T, H, kv_rank].  `interleaved`:
        the rotation pairs coordinate 2i with 2i + 1 instead of i with i + rot_dims / 2."""
        self._add("latent_attention", q_rot=q_rot, kv_in=kv_in, c_gain=c_gain, eps=float(eps), inv_freq=inv_freq,
                  rot_dims=int(rot_dims), q=q, out=out, cache=cache, group=group, num_heads=num_heads, kv_rank=kv_rank,
                  rot_dim=rot_dim, scale=float(scale), sink=sink, scratch=scratch, window=int(window), interleaved=bool(interleaved))

    def token_side(self, *, x, a, b, table, offset: int, dim: int, w_gate, w_proj, gain, eps: float, xb, g, y) -> None:
        """x += a (+ b); e = table[token][offset : offset + dim]; g = gelu_tanh(w_gate x) * e; y = w_proj g;
        x += y / sqrt(mean(y^2) + eps) * gain.  `xb` [T, D], `g` [T, dim] and `y` [T, D] (32-bit) are the workspace of
        the form that runs this as single kernels."""
        self._add("token_side", x=x, a=a, b=b, table=table, offset=int(offset), dim=int(dim), w_gate=w_gate, w_proj=w_proj,
                  gain=gain, eps=float(eps), xb=xb, g=g, y=y)
        self.note_copy(x, None)

    def postnorm(self, x: torch.Tensor, y: Optional[torch.Tensor], gain: Optional[torch.Tensor], eps: float,
                 accumulate: bool = True, copy: Optional[torch.Tensor] = None) -> None:
        """The norm on a sublayer's output: x += y / sqrt(mean(y^2) + eps) * gain in 32-bit (`accumulate` False:
        x = ...; y may then be x itself), and `copy`, if given, receives the new x in its own type.  Without y only
        the copy is made."""
        self._add("postnorm", x=x, y=y, gain=gain, eps=float(eps), accumulate=bool(accumulate), copy=copy)
        self.note_copy(x, copy)

    def window_attention(self, *, q_in, k_in, v_in, q_gain, k_gain, eps: float, inv_freq, rot_dims: int, amplitude: float,
                         q, out, cache, group: int, num_heads: int, num_kv_heads: int, qk_dim: int, v_dim: int,
                         window: int, keep_first: int, scale: float, sink=None, scratch=None, q_bias=None, k_bias=None,
                         v_bias=None, head_norm: bool = False, softcap: float = 0.0, interleaved: bool = False) -> None:
        """Grouped-query attention over a cache whose keys are `qk_dim` and whose values are `v_dim` wide, from the raw
        projections: q_in [T, H qk_dim] and, for a layer that stores, k_in [T, G qk_dim] and v_in [T, G v_dim] (column
        ranges of one product).  With gains, queries and keys are RMS-normed over the WHOLE projection (all heads at
        once, gain vectors of that size); the first `rot_dims` coordinates of every head are rotated in rotate-half
        pairs by position * inv_freq[i], cosine and sine times `amplitude` (inv_freq None: no rotation); keys and
        values are stored.  Then query i sees key j if j <= i and (i - j < window or j < keep_first) (window 0: every
        earlier key); s_ij = scale (q_i . k_j); p_ij = exp(s_ij) / (sum_j' exp(s_ij') [+ exp(sink_h) with `sink` [H]]);
        out [T, H v_dim].  `q` [T, H qk_dim] is the workspace of the finished queries; `scratch` (32-bit) is where the
        parts of single tokens meet whose keys a kernel cuts into ranges.  Options: `q_bias`, `k_bias`, `v_bias` (32-bit
        vectors) are added to the projections first; with `head_norm` every head is normed by itself over its qk_dim
        coordinates and the gains are [qk_dim], shared by the heads; `v_in` may be `k_in` itself (the values are then the
        keys as projected, before norm and rotation); `softcap` c > 0: s_ij <- c tanh(s_ij / c) behind the scale;
        `interleaved`: the rotation pairs coordinate 2i with 2i + 1 instead of i with i + rot_dims / 2.  The projections may
        be 32-bit where everything else has the type of the products (they then come from a convolution, not a product)."""
        self._add("window_attention", q_bias=q_bias, k_bias=k_bias, v_bias=v_bias, head_norm=bool(head_norm), q_in=q_in, k_in=k_in, v_in=v_in, q_gain=q_gain, k_gain=k_gain, eps=float(eps),
                  inv_freq=inv_freq, rot_dims=int(rot_dims), amplitude=float(amplitude), q=q, out=out, cache=cache, group=group,
                  num_heads=num_heads, num_kv_heads=num_kv_heads, qk_dim=qk_dim, v_dim=v_dim, window=int(window),
                  keep_first=int(keep_first), scale=float(scale), sink=sink, scratch=scratch, softcap=float(softcap),
                  interleaved=bool(interleaved))

    def moe_route(self, *, logits, top_k: int, scale: float, experts, weights, offsets, order, counts,
                  mode: str = "sigmoid") -> None:
        """Routing of every token of the step from its router `logits` [T, E] (32-bit, any row stride): s = sigmoid(logits);
        C = the `top_k` experts of largest s (`experts` [T, top_k] int32, best first); `weights` [T, top_k]: w_e = scale *
        s_e / (sum over C of s + 1e-20).  `mode` "softmax_chosen": C = the experts of largest logits and w_e = scale *
        exp(z_e) / sum over C of exp(z).  The (token, choice) pairs are then listed expert by expert:
        `offsets` [E + 1] int32 with the pairs of expert e at order[offsets[e] : offsets[e + 1]], a pair being
        token * top_k + choice.  `counts` [E] int32 is scratch that is zero between launches."""
        if mode not in ("sigmoid", "softmax_chosen"):
            raise ValueError(f"moe_route: unknown mode {mode!r}")
        self._add("moe_route", logits=logits, top_k=int(top_k), scale=float(scale), experts=experts, weights=weights,
                  offsets=offsets, order=order, counts=counts, mode=mode)

    def grouped_linear(self, *, x, w, out, offsets, order, top_k: int, gather: bool, scatter: bool, mid=None,
                       act: Optional[str] = None) -> None:
        """One product per expert over the rows that were routed to it: for place r of expert e's range of `order`,
        out_row = w[e] x_row, with x_row = x[order[r] // top_k] if `gather` (the token's row) else x[r], and written
        to out[order[r]] if `scatter` (the pair's row) else out[r].  w is [E, n, k].  With `act` ("silu"), w[e] is
        [gate | up] by rows and the row written is silu(gate) * up, half as wide (`mid` [pairs, n]: workspace of the
        form that runs product and activation apart)."""
        self._add("grouped_linear", x=x, w=w, out=out, offsets=offsets, order=order, top_k=int(top_k), gather=bool(gather),
                  scatter=bool(scatter), mid=mid, act=act)

    def moe_combine(self, *, y, weights, base, out, base_gate=None) -> None:
        """out[t] = base[t] (if given) + sum_k weights[t, k] * y[t * top_k + k], the choices added in their order,
        in 32-bit.  With `base_gate` [T, 1] (32-bit, any row stride) base[t] is first multiplied by sigmoid(base_gate[t])."""
        self._add("moe_combine", y=y, weights=weights, base=base, out=out, base_gate=base_gate)

    def short_conv(self, *, x, w, bias, state, out, act: Optional[str] = "silu") -> None:
        """Causal convolution per channel over each request's tokens: y_t = bias + sum_j w[:, K-1-j] x_(t-j) with zeros
        before the request's start, then `act` ("silu" or None).  x [T, C] (any row stride), w [C, K] and bias [C] 32-bit,
        out [T, C] 32-bit.  `state` [slots, K - 1, C] 32-bit holds each request's last K - 1 inputs between steps."""
        self._add("short_conv", x=x, w=w, bias=bias, state=state, out=out, act=act)

    def rotate(self, *, x, out, heads, scale, dim: int, rot_dims: int, inv_freq) -> None:
        """Rotation by position into 32-bit: for each of up to two tensors x[i] [T, heads[i] * dim] the first `rot_dims`
        coordinates of every head turn in rotate-half pairs by position * inv_freq[j]; the rest pass; then times scale[i]."""
        self._add("rotate", x=tuple(x), out=tuple(out), heads=tuple(heads), scale=tuple(scale), dim=int(dim), rot_dims=int(rot_dims),
                  inv_freq=inv_freq)

    def recurrence(self, *, q, k, v, state, out, heads: int, n: int, p: int, qk_groups: int, decay=None, dt=None, dt_bias=None,
                   a_log=None, skip=None, scratch=None, keep=None, take=None, unit_column: bool = False) -> None:
        """Per request and head, over the request's tokens in order: S_t = a_t S_(t-1) + s_t k_t v_t^T (S is n x p),
        y_t = S_t^T q_t + skip_h v_t.  With `decay` [H]: a_t = decay_h, s_t = 1.  With `dt` [T, H], `dt_bias` and `a_log`
        [H]: d = softplus(dt + dt_bias), a_t = exp(-exp(a_log_h) d), s_t = d.  q, k [T, qk_groups * n] and out [T, H p] are
        32-bit; head h reads group h // (H / qk_groups).  `state` [slots, H, p, n] 32-bit goes from step to step.  With `scratch`
        (32-bit, a few states large) a long portion is cut into pieces that run side by side.  With `keep` and `take` [T, H]
        (32-bit): a_t = keep[t, h], s_t = take[t, h], both made by an earlier record.  `unit_column`: the last of the p columns
        has no v behind it, its v_t is one (that column of S sums s_t k_t alone, and that column of y is its product with q);
        v is then [T, H (p - 1)]."""
        self._add("recurrence", q=q, k=k, v=v, state=state, out=out, heads=int(heads), n=int(n), p=int(p), qk_groups=int(qk_groups),
                  decay=decay, dt=dt, dt_bias=dt_bias, a_log=a_log, skip=skip, scratch=scratch, keep=keep, take=take,
                  unit_column=bool(unit_column))

    def gated_norm(self, *, y, gate, weight, out, group: int, gate_first: bool, eps: float, scale: float = 1.0,
                   gate_act: str = "silu", floor=None, den_eps: float = 0.0) -> None:
        """RMS norm of y [T, C] (32-bit) in groups of `group` columns, with g = silu(gate) (`gate_act` "sigmoid": sigmoid(gate)):
        `gate_first`: u = y g, out = u / rms(u) * weight; else out = y / rms(y) * weight * g; then times `scale`.  `weight` [C]
        32-bit or None.  With `floor` [T, C / group] (32-bit) every group of y is one column wider than its group of the gate
        and of out: the extra value d stands behind the group's own, and the group is divided by max(|d|, floor) + den_eps
        before anything else."""
        if gate_act not in ("silu", "sigmoid"):
            raise ValueError(f"gated_norm: unknown gate {gate_act!r}")
        self._add("gated_norm", y=y, gate=gate, weight=weight, out=out, group=int(group), gate_first=bool(gate_first),
                  eps=float(eps), scale=float(scale), gate_act=gate_act, floor=floor, den_eps=float(den_eps))

    def row_norm(self, *, x, gain, eps: float, out) -> None:
        """out = x / sqrt(mean(x^2) + eps) * gain over the rows of x [T, C]: a norm on (a column range of) a product, in
        and out of any type and row stride; the arithmetic is 32-bit."""
        self._add("row_norm", x=x, gain=gain, eps=float(eps), out=out)

    def exp_gates(self, *, i_pre, f_pre, cap: float, state, keep, take, floor) -> None:
        """The gates of a matrix memory with exponential gating, per request and head over the request's tokens in order,
        all 32-bit.  From the pre-activations i_pre, f_pre [T, H]: a_t = cap tanh(i_pre / cap), b_t = logsigmoid(cap
        tanh(f_pre / cap)) (cap 0: no cap); the running maximum M_t = max(b_t + M_(t-1), a_t), kept in `state` [slots, H]
        (zero when a request starts); keep[t] = exp(b_t + M_(t-1) - M_t), take[t] = exp(a_t - M_t), floor[t] = exp(-M_t)."""
        self._add("exp_gates", i_pre=i_pre, f_pre=f_pre, cap=float(cap), state=state, keep=keep, take=take, floor=floor)
