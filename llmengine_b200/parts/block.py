"""How a layer arranges its mixer, feed-forward and norms."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..config.spec import LayerSpec
from ..engine.plan import Plan
from .base import (Part, Runtime, WeightSpec, build_part, emit_feed_forward, emit_mixer, emit_norm, register_part,
                   run_alone)


@register_part("block", "prenorm_residual")
class PreNormResidualBlock(Part):
    """x = x + mixer(norm1(x));  x = x + feed_forward(norm2(x))
    (src/model/transformer_graph_builder.cpp:207-274: the un-normed x is the residual).

    The residual stream `x` stays 32-bit.  A contribution is not added where it is produced:
    it travels as `delta` to the next norm, whose kernel adds it to `x` and normalises in one
    pass.  The block reads the parts "mixer", "mixer_norm", "feed_forward" and "feed_forward_norm" of its
    layer; the names under which their tensors are stored come with the spec.
    """

    def __init__(self, rt: Runtime, prefix: str, layer: LayerSpec, mixer_name: str = "mixer",
                 feed_forward_name: str = "feed_forward", mixer_norm_name: str = "mixer_norm",
                 feed_forward_norm_name: str = "feed_forward_norm"):
        super().__init__(rt, prefix)
        need = ("mixer", "mixer_norm", "feed_forward", "feed_forward_norm")
        missing = [n for n in need if n not in layer.parts]
        if missing:
            raise ValueError(f"layer {prefix!r}: a prenorm_residual block needs the parts {', '.join(missing)}")
        self.mixer_norm = build_part("norm", layer.parts["mixer_norm"], rt, self.name(mixer_norm_name))
        self.mixer = build_part("mixer", layer.parts["mixer"], rt, self.name(mixer_name))
        self.ffn_norm = build_part("norm", layer.parts["feed_forward_norm"], rt, self.name(feed_forward_norm_name))
        self.ffn = build_part("feed_forward", layer.parts["feed_forward"], rt, self.name(feed_forward_name))
        self.parts = (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)
        self.capture_safe = all(p.capture_safe and hasattr(p, "emit") for p in self.parts)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        out: Dict[str, WeightSpec] = {}
        for p in self.parts:
            out.update(p.weight_specs())
        return out

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts:
            p.load_weights({n: tensors[n] for n in p.weight_specs()})

    def cache_spec(self):
        return self.mixer.cache_spec()

    def emit(self, plan: Plan, x: torch.Tensor, delta: Optional[torch.Tensor], cache) -> Tuple[torch.Tensor, torch.Tensor]:
        hidden = x.shape[1]
        h = emit_norm(plan, self.mixer_norm, x, delta=delta)
        a = emit_mixer(plan, self.mixer, h, cache, hidden)
        h = emit_norm(plan, self.ffn_norm, x, delta=a)
        return x, emit_feed_forward(plan, self.ffn, h, hidden)

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor], batch, cache) -> Tuple[torch.Tensor, torch.Tensor]:
        plan = Plan()
        x, out = self.emit(plan, x, delta, cache)
        run_alone(self.rt, plan, batch)
        return x, out[: x.shape[0]]


@register_part("block", "parallel_residual")
class ParallelResidualBlock(Part):
    """h = norm(x);  x = x + (mixer(h) + feed_forward(h)): one norm, both sublayers read its output.  A layer may
    have no feed-forward.  With a "token_side" part, that part follows on the updated x (and does the addition of
    the sublayers' contributions itself, in the same pass).

    Options of other designs: with a part "feed_forward_norm" the feed-forward reads a norm of its own of the same x
    (x = x + mixer(norm(x)) + feed_forward(feed_forward_norm(x))); with `mixer_scale_name` / `feed_forward_scale_name`
    each sublayer's result is multiplied, column by column, by a learned vector of the stream's width (tensors of those
    names below the layer's prefix) before the sum.

    The block reads the parts "norm", "mixer" and, where the layer has them, "feed_forward", "feed_forward_norm" and
    "token_side".
    """

    def __init__(self, rt: Runtime, prefix: str, layer: LayerSpec, norm_name: str = "norm", mixer_name: str = "mixer",
                 feed_forward_name: str = "feed_forward", token_side_name: str = "token_side",
                 feed_forward_norm_name: str = "feed_forward_norm", mixer_scale_name: Optional[str] = None,
                 feed_forward_scale_name: Optional[str] = None, hidden_size: Optional[int] = None):
        super().__init__(rt, prefix)
        missing = [n for n in ("norm", "mixer") if n not in layer.parts]
        if missing:
            raise ValueError(f"layer {prefix!r}: a parallel_residual block needs the parts {', '.join(missing)}")
        self.norm = build_part("norm", layer.parts["norm"], rt, self.name(norm_name))
        self.mixer = build_part("mixer", layer.parts["mixer"], rt, self.name(mixer_name))
        self.ffn = (build_part("feed_forward", layer.parts["feed_forward"], rt, self.name(feed_forward_name))
                    if "feed_forward" in layer.parts else None)
        self.ffn_norm = (build_part("norm", layer.parts["feed_forward_norm"], rt, self.name(feed_forward_norm_name))
                         if self.ffn is not None and "feed_forward_norm" in layer.parts else None)
        self.side = (build_part("token_side", layer.parts["token_side"], rt, self.name(token_side_name))
                     if "token_side" in layer.parts else None)
        self.scale_names = (mixer_scale_name, feed_forward_scale_name if self.ffn is not None else None)
        if any(self.scale_names) and (hidden_size is None or self.side is not None):
            raise ValueError(f"layer {prefix!r}: scale vectors need the stream's width and a block without a token side input")
        self.hidden = None if hidden_size is None else int(hidden_size)
        self.scales = [None, None]
        self.parts = tuple(p for p in (self.norm, self.mixer, self.ffn_norm, self.ffn, self.side) if p is not None)
        self.capture_safe = all(p.capture_safe and hasattr(p, "emit") for p in self.parts)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        out: Dict[str, WeightSpec] = {}
        for p in self.parts:
            out.update(p.weight_specs())
        for n in self.scale_names:
            if n:
                out[self.name(n)] = WeightSpec((self.hidden,), role="vector", init="gain")
        return out

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts:
            p.load_weights({n: tensors[n] for n in p.weight_specs()})
        self.scales = [tensors[self.name(n)].float().contiguous() if n else None for n in self.scale_names]

    def tied_tensors(self) -> Dict[str, str]:
        out: Dict[str, str] = {}
        for p in self.parts:
            out.update(p.tied_tensors())
        return out

    def receive_tied(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts:
            own = p.tied_tensors()
            if own:
                p.receive_tied({n: tensors[n] for n in own})

    def cache_spec(self):
        return self.mixer.cache_spec()

    def emit(self, plan: Plan, x: torch.Tensor, delta: Optional[torch.Tensor], cache):
        hidden = x.shape[1]
        h2 = None
        if self.ffn_norm is not None and hasattr(self.norm, "pairs_with") and self.norm.pairs_with(self.ffn_norm):
            h, h2 = self.norm.emit_pair(plan, self.ffn_norm, x, delta=delta)      # both norms of the same x in one pass
        else:
            h = emit_norm(plan, self.norm, x, delta=delta)
        a = emit_mixer(plan, self.mixer, h, cache, hidden)
        b = None
        if self.ffn is not None:
            # a second norm of the same x goes to a workspace of its own: the mixer's input may still be needed
            if h2 is not None:
                pass
            elif self.ffn_norm is None:
                h2 = h
            elif hasattr(self.ffn_norm, "emit"):
                h2 = self.ffn_norm.emit(plan, x, out_name="normed_second")
            else:
                h2 = emit_norm(plan, self.ffn_norm, x)
            b = emit_feed_forward(plan, self.ffn, h2, hidden)
        if self.side is not None:
            self.side.emit(plan, x, a, b)
            return x, None
        if b is None and self.scales[0] is None:
            return x, a                       # the next norm adds it
        plan.residual_add(x, a, b, a_scale=self.scales[0], b_scale=self.scales[1] if b is not None else None)
        return x, None

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor], batch, cache):
        plan = Plan()
        x, out = self.emit(plan, x, delta, cache)
        run_alone(self.rt, plan, batch)
        return x, None if out is None else out[: x.shape[0]]


@register_part("block", "postnorm_residual")
class PostNormResidualBlock(Part):
    """x = x + norm1(mixer(x));  x = x + norm2(feed_forward(x)): the norms stand on the sublayers' OUTPUTS, and the
    sublayers read the residual stream itself.  A layer may have no feed-forward (and then no second norm).

    The stream is 32-bit.  Where the matrix products take another type, the kernel that adds a normed contribution
    also writes the new stream in that type, which is what the next sublayer reads.  The block reads the parts
    "mixer", "mixer_norm" and, where the layer has them, "feed_forward" and "feed_forward_norm" (norm parts with a
    gain vector and an eps)."""

    def __init__(self, rt: Runtime, prefix: str, layer: LayerSpec, mixer_name: str = "mixer",
                 feed_forward_name: str = "feed_forward", mixer_norm_name: str = "mixer_norm",
                 feed_forward_norm_name: str = "feed_forward_norm"):
        super().__init__(rt, prefix)
        missing = [n for n in ("mixer", "mixer_norm") if n not in layer.parts]
        if "feed_forward" in layer.parts and "feed_forward_norm" not in layer.parts:
            missing.append("feed_forward_norm")
        if missing:
            raise ValueError(f"layer {prefix!r}: a postnorm_residual block needs the parts {', '.join(missing)}")
        self.mixer = build_part("mixer", layer.parts["mixer"], rt, self.name(mixer_name))
        self.mixer_norm = build_part("norm", layer.parts["mixer_norm"], rt, self.name(mixer_norm_name))
        has_ffn = "feed_forward" in layer.parts
        self.ffn = build_part("feed_forward", layer.parts["feed_forward"], rt, self.name(feed_forward_name)) if has_ffn else None
        self.ffn_norm = build_part("norm", layer.parts["feed_forward_norm"], rt, self.name(feed_forward_norm_name)) if has_ffn else None
        self.parts = tuple(p for p in (self.mixer, self.mixer_norm, self.ffn, self.ffn_norm) if p is not None)
        for n in (self.mixer_norm, self.ffn_norm):
            if n is not None and not (hasattr(n, "gain") and hasattr(n, "eps")):
                raise ValueError(f"layer {prefix!r}: the norm on a sublayer's output needs a gain vector and an eps")
        self.capture_safe = all(p.capture_safe and hasattr(p, "emit") for p in (self.mixer, self.ffn) if p is not None)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        out: Dict[str, WeightSpec] = {}
        for p in self.parts:
            out.update(p.weight_specs())
        return out

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts:
            p.load_weights({n: tensors[n] for n in p.weight_specs()})

    def cache_spec(self):
        return self.mixer.cache_spec()

    def _input(self, plan: Plan, x: torch.Tensor) -> torch.Tensor:
        """The stream as a sublayer reads it: itself in the 32-bit engine, else its copy in the product type."""
        rt = self.rt
        if rt.dtype == torch.float32:
            return x
        h = plan.copy_of(x)
        if h is None:
            h = rt.workspace("stream_copy", x.shape[1], rt.dtype)
            plan.postnorm(x, None, None, 0.0, copy=h)
        return h

    def emit(self, plan: Plan, x: torch.Tensor, delta: Optional[torch.Tensor], cache):
        rt = self.rt
        hidden = x.shape[1]
        if delta is not None:
            plan.residual_add(x, delta)
        copy = None if rt.dtype == torch.float32 else rt.workspace("stream_copy", hidden, rt.dtype)
        a = emit_mixer(plan, self.mixer, self._input(plan, x), cache, hidden)
        plan.postnorm(x, a, self.mixer_norm.gain, self.mixer_norm.eps, copy=copy)
        if self.ffn is not None:
            b = emit_feed_forward(plan, self.ffn, self._input(plan, x), hidden)
            plan.postnorm(x, b, self.ffn_norm.gain, self.ffn_norm.eps, copy=copy)
        return x, None

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor], batch, cache):
        plan = Plan()
        x, _ = self.emit(plan, x, delta, cache)
        run_alone(self.rt, plan, batch)
        return x, None


@register_part("block", "sandwich_residual")
class SandwichResidualBlock(Part):
    """x = x + norm1b(mixer(norm1(x)));  x = x + norm2b(feed_forward(norm2(x))): a norm before AND after each sublayer.
    A layer may have no feed-forward (and then neither of its norms).

    The stream is 32-bit.  The norm before a sublayer writes its input in the type of the products; the norm behind it
    is the kernel that norms a sublayer's output and adds it to the stream in one pass.  The block reads the parts
    "mixer", "mixer_norm", "mixer_out_norm" and, where the layer has a feed-forward, "feed_forward", "feed_forward_norm"
    and "feed_forward_out_norm"."""

    def __init__(self, rt: Runtime, prefix: str, layer: LayerSpec, mixer_name: str = "mixer", feed_forward_name: str = "feed_forward",
                 mixer_norm_name: str = "mixer_norm", mixer_out_norm_name: str = "mixer_out_norm",
                 feed_forward_norm_name: str = "feed_forward_norm", feed_forward_out_norm_name: str = "feed_forward_out_norm"):
        super().__init__(rt, prefix)
        has_ffn = "feed_forward" in layer.parts
        need = ["mixer", "mixer_norm", "mixer_out_norm"] + (["feed_forward_norm", "feed_forward_out_norm"] if has_ffn else [])
        missing = [n for n in need if n not in layer.parts]
        if missing:
            raise ValueError(f"layer {prefix!r}: a sandwich_residual block needs the parts {', '.join(missing)}")
        self.mixer_norm = build_part("norm", layer.parts["mixer_norm"], rt, self.name(mixer_norm_name))
        self.mixer = build_part("mixer", layer.parts["mixer"], rt, self.name(mixer_name))
        self.mixer_out_norm = build_part("norm", layer.parts["mixer_out_norm"], rt, self.name(mixer_out_norm_name))
        self.ffn = self.ffn_norm = self.ffn_out_norm = None
        if has_ffn:
            self.ffn_norm = build_part("norm", layer.parts["feed_forward_norm"], rt, self.name(feed_forward_norm_name))
            self.ffn = build_part("feed_forward", layer.parts["feed_forward"], rt, self.name(feed_forward_name))
            self.ffn_out_norm = build_part("norm", layer.parts["feed_forward_out_norm"], rt, self.name(feed_forward_out_norm_name))
        self.parts = tuple(p for p in (self.mixer_norm, self.mixer, self.mixer_out_norm, self.ffn_norm, self.ffn, self.ffn_out_norm)
                           if p is not None)
        for n in (self.mixer_out_norm, self.ffn_out_norm):
            if n is not None and not (hasattr(n, "gain") and hasattr(n, "eps")):
                raise ValueError(f"layer {prefix!r}: the norm on a sublayer's output needs a gain vector and an eps")
        self.capture_safe = all(p.capture_safe and hasattr(p, "emit") for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)
                                if p is not None)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        out: Dict[str, WeightSpec] = {}
        for p in self.parts:
            out.update(p.weight_specs())
        return out

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts:
            p.load_weights({n: tensors[n] for n in p.weight_specs()})

    def cache_spec(self):
        return self.mixer.cache_spec()

    def emit(self, plan: Plan, x: torch.Tensor, delta: Optional[torch.Tensor], cache):
        hidden = x.shape[1]
        h = emit_norm(plan, self.mixer_norm, x, delta=delta)
        a = emit_mixer(plan, self.mixer, h, cache, hidden)
        plan.postnorm(x, a, self.mixer_out_norm.gain, self.mixer_out_norm.eps)
        if self.ffn is not None:
            h = emit_norm(plan, self.ffn_norm, x)
            b = emit_feed_forward(plan, self.ffn, h, hidden)
            plan.postnorm(x, b, self.ffn_out_norm.gain, self.ffn_out_norm.eps)
        return x, None

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor], batch, cache):
        plan = Plan()
        x, _ = self.emit(plan, x, delta, cache)
        run_alone(self.rt, plan, batch)
        return x, None
