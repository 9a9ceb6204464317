"""Attention over a cached low-rank latent: per token one row [c | rotated key part] serves every head.

Per head the design defines key = W_uk c and value = W_uv c.  Neither is ever formed: the head's query is carried
into the latent space (q' = W_uk_h^T q_h, one small matrix per head), scores are q' . c (+ q_rot . k_rot), the
weighted sum runs over c itself and W_uv_h is applied to that sum.  The same arithmetic up to the order of the
sums; the cache holds kv_rank + rot_dim numbers per token and layer instead of heads * (dim + vdim), and the
attention kernels read one shared key/value row per token for all heads.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import numpy as np
import torch

from ..config.spec import PartSpec
from ..engine.plan import Plan
from .base import Part, Runtime, WeightSpec, build_part, register_part, run_alone


@dataclass
class LatentCacheView:
    """The cache a latent mixer run works on."""

    kv: torch.Tensor                # [pages, page_size, kv_rank + rot_dim]
    group: int
    writes: bool


@dataclass(frozen=True)
class LatentKVSpec:
    """A mixer that keeps one row of `width` numbers per earlier token, in pages."""

    width: int
    window: int = 0
    paged = True

    def allocate(self, count: int, page_size: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        return torch.zeros(count, page_size, self.width, dtype=dtype, device=device)

    def bytes_per_token(self, dtype: torch.dtype) -> int:
        return self.width * torch.empty((), dtype=dtype).element_size()

    def view(self, tensor: torch.Tensor, group: Optional[int], writes: bool) -> LatentCacheView:
        return LatentCacheView(tensor, group, writes)


@register_part("position", "rotary_partial")
class PartialRotaryEncoding(Part):
    """Rotate-half rotary encoding of the first `dims` coordinates of a vector; what lies beyond them passes
    unchanged.  Coordinate i pairs with i + dims/2; at position p the pair is turned by the angle p * f_i with
    f_i = base^(-2i/dims).  The frequencies are formed once on the host in 32-bit; the kernels form the 32-bit angle
    and its cosine and sine from the token's position, so there is no table of positions and no longest position.

    `scaling` = {factor, original, fast, slow} stretches the encoding to sequences `factor` times longer than the
    `original` length it was made for: with turns(t) = dims ln(original / (2 pi t)) / (2 ln base) the coordinate that
    makes t turns over the original length, lo = max(floor(turns(fast)), 0), hi = min(ceil(turns(slow)), dims - 1) and
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency becomes f_i / factor * r_i + f_i (1 - r_i) (fast
    coordinates keep their frequency, slow ones are slowed), and cosine and sine are multiplied by
    `amplitude` = 0.1 ln(factor) + 1.

    `interleaved`: coordinate 2i pairs with 2i + 1 instead (same frequencies, same turn): (u, v) -> (u cos - v sin,
    v cos + u sin)."""

    needs_apply = True

    def __init__(self, rt: Runtime, prefix: str, dims: int, base: float, scaling: Optional[dict] = None,
                 interleaved: bool = False):
        super().__init__(rt, prefix)
        if dims <= 0 or dims % 2:
            raise ValueError(f"rotary encoding needs an even number of rotated coordinates, got {dims}")
        self.dims, self.base, self.interleaved = int(dims), float(base), bool(interleaved)
        self.scaling = None if not scaling else tuple(float(scaling[k]) for k in ("factor", "original", "fast", "slow"))
        self.amplitude = 1.0 if self.scaling is None else float(np.float32(0.1 * np.log(self.scaling[0]) + 1.0))

    @staticmethod
    def build_frequencies(dims: int, base: float, scaling: Optional[tuple] = None) -> torch.Tensor:
        i = np.arange(dims // 2, dtype=np.float32)
        expo = (np.float32(-2.0) * i) / np.float32(dims)
        f = np.power(np.float64(np.float32(base)), expo.astype(np.float64))
        if scaling is not None:
            factor, original, fast, slow = scaling

            def turns(t: float) -> float:
                return dims * np.log(original / (2.0 * np.pi * t)) / (2.0 * np.log(base))
            lo = max(int(np.floor(turns(fast))), 0)
            hi = min(int(np.ceil(turns(slow))), dims - 1)
            ramp = np.clip((i.astype(np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            f = f / factor * ramp + f * (1.0 - ramp)
        return torch.from_numpy(f.astype(np.float32))

    def frequencies(self) -> torch.Tensor:
        return self.rt.shared_table(("rotary_partial", self.dims, self.base, self.scaling),
                                    lambda: self.build_frequencies(self.dims, self.base, self.scaling))

    def rotary_table(self) -> Optional[torch.Tensor]:
        return None


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    """q = W_q h, per head [nope_dim unrotated | rot_dim rotated]; W_dkv h = [kv_rank | rot_dim]: the first part,
    RMS-normed with a weight vector, is the latent c, the second one rotated key part for all heads; per head
    key = [W_uk c | rotated part], value = W_uv c; score = q . key * scale, causal; softmax, with `sink` a learned
    number per head whose exponential joins the denominator; with `output_gate` the concatenated heads are
    multiplied by sigmoid(W_g h); then W_o.  `rot_dim` = 0 with no position encoding: no rotated part at all.
    With `q_rank` > 0 the queries come through a latent of their own: c_q = rmsnorm(W_dq h) with a weight vector
    (dq.norm), q = W_uq c_q (tensors dq, dq.norm, uq instead of q).  With `window` W > 0 a query sees only the last W
    keys, its own included, and the cache gives pages back as the window passes them.

    Stored as: one matrix [W_q or W_dq | W_dkv | W_g] (one product serves the three), W_uk transposed per head
    [H, kv_rank, nope_dim] (it carries queries into the latent space), W_uv per head [H, v_dim, kv_rank].
    """

    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, num_heads: int, nope_dim: int, rot_dim: int,
                 v_dim: int, kv_rank: int, scale: float, norm_eps: float, position_encoding: Optional[PartSpec] = None,
                 sink: bool = False, output_gate: bool = False, q_rank: int = 0, window: int = 0):
        super().__init__(rt, prefix)
        self.hidden, self.nh, self.dn, self.dr = int(hidden_size), int(num_heads), int(nope_dim), int(rot_dim)
        self.dv, self.rank, self.scale, self.eps = int(v_dim), int(kv_rank), float(scale), float(norm_eps)
        self.has_sink, self.has_gate = bool(sink), bool(output_gate)
        self.q_rank, self.window = int(q_rank), int(window)
        if (self.dr > 0) != (position_encoding is not None):
            raise ValueError(f"{prefix}: a rotated part needs a position encoding, and a position encoding a rotated part")
        self.position = build_part("position", position_encoding, rt, prefix) if position_encoding is not None else None
        if self.position is not None and self.position.dims > self.dr:
            raise ValueError(f"{prefix}: {self.position.dims} rotated coordinates do not fit rot_dim = {self.dr}")
        self.q_size = self.nh * (self.dn + self.dr)
        self.kv_size = self.rank + self.dr
        self.o_size = self.nh * self.dv
        self.w_in = self.w_uk_t = self.w_uv = self.w_o = self.c_gain = self.sink = self.w_uq = self.q_gain = None

    # ------------------------------------------------------------------ weights
    def weight_specs(self) -> Dict[str, WeightSpec]:
        s = {
            self.name("dkv"): WeightSpec((self.kv_size, self.hidden)),
            self.name("dkv.norm"): WeightSpec((self.rank,), role="vector", init="gain"),
            self.name("uk"): WeightSpec((self.nh * self.dn, self.rank)),
            self.name("uv"): WeightSpec((self.o_size, self.rank)),
            self.name("o"): WeightSpec((self.hidden, self.o_size)),
        }
        if self.q_rank:
            s[self.name("dq")] = WeightSpec((self.q_rank, self.hidden))
            s[self.name("dq.norm")] = WeightSpec((self.q_rank,), role="vector", init="gain")
            s[self.name("uq")] = WeightSpec((self.q_size, self.q_rank))
        else:
            s[self.name("q")] = WeightSpec((self.q_size, self.hidden))
        if self.has_sink:
            s[self.name("sink")] = WeightSpec((self.nh,), role="vector", init="unit")
        if self.has_gate:
            s[self.name("g")] = WeightSpec((self.o_size, self.hidden))
        return s

    def load_weights(self, t: Dict[str, torch.Tensor]) -> None:
        parts = [t[self.name("dq" if self.q_rank else "q")], t[self.name("dkv")]] + ([t[self.name("g")]] if self.has_gate else [])
        self.w_in = torch.cat(parts, dim=0).contiguous()
        if self.q_rank:
            self.w_uq = t[self.name("uq")].contiguous()
            self.q_gain = t[self.name("dq.norm")].contiguous()
        self.w_uk_t = t[self.name("uk")].view(self.nh, self.dn, self.rank).transpose(1, 2).contiguous()
        self.w_uv = t[self.name("uv")].view(self.nh, self.dv, self.rank).contiguous()
        self.w_o = t[self.name("o")].contiguous()
        self.c_gain = t[self.name("dkv.norm")].contiguous()
        self.sink = t[self.name("sink")].float().contiguous() if self.has_sink else None

    def cache_spec(self) -> LatentKVSpec:
        return LatentKVSpec(self.kv_size, self.window)

    # ------------------------------------------------------------------ compute
    def emit(self, plan: Plan, h: torch.Tensor, cache) -> torch.Tensor:
        rt = self.rt
        if not cache.writes:
            raise ValueError(f"{self.prefix}: a latent mixer keeps a cache of its own")
        H, dn, dr, dv, r = self.nh, self.dn, self.dr, self.dv, self.rank
        T = rt.max_tokens
        width = self.w_in.shape[0]
        proj = rt.workspace("latent_in", width, rt.dtype)
        plan.linear(h, self.w_in, proj)
        first = self.q_rank or self.q_size                       # columns of the product that belong to the queries
        if self.q_rank:
            cq = rt.workspace("latent_cq", self.q_rank, rt.dtype)
            plan.row_norm(x=proj[:, :first], gain=self.q_gain, eps=self.eps, out=cq)
            q_full = rt.workspace("latent_q_heads", self.q_size, rt.dtype)
            plan.linear(cq, self.w_uq, q_full)
            q_heads = q_full.view(T, H, dn + dr)
        else:
            q_heads = proj[:, :first].view(T, H, dn + dr)
        kv_in = proj[:, first:first + self.kv_size]
        q = rt.workspace("latent_q", H * (r + dr), rt.dtype)
        q3 = q.view(T, H, r + dr)
        plan.batched_linear(q_heads[:, :, :dn], self.w_uk_t, q3[:, :, :r])
        out = rt.workspace("latent_out", H * r, rt.dtype)
        plan.latent_attention(q_rot=q_heads[:, :, dn:] if dr else None, kv_in=kv_in, c_gain=self.c_gain, eps=self.eps,
                              inv_freq=self.position.frequencies() if self.position is not None else None,
                              rot_dims=self.position.dims if self.position is not None else 0, q=q, out=out,
                              cache=cache.kv, group=cache.group, num_heads=H, kv_rank=r, rot_dim=dr, scale=self.scale,
                              sink=self.sink, scratch=rt.latent_scratch(H, r), window=self.window,
                              interleaved=bool(self.position is not None and self.position.interleaved))
        heads = rt.workspace("latent_heads", self.o_size, rt.dtype)
        plan.batched_linear(out.view(T, H, r), self.w_uv, heads.view(T, H, dv))
        if self.has_gate:
            plan.pointwise("sigmoid_mul", heads, proj[:, first + self.kv_size:], heads)
        delta = rt.workspace("mixer_out", self.hidden, torch.float32)
        plan.linear(heads, self.w_o, delta)
        return delta

    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        plan = Plan()
        delta = self.emit(plan, h, cache)
        run_alone(self.rt, plan, batch)
        return delta[: h.shape[0]]
