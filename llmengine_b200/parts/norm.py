"""RMS norm over the residual stream, fused with the pending residual add."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..engine.plan import ROWS_LOGITS, ROWS_TOKENS, Plan
from .base import Part, Runtime, WeightSpec, register_part, run_alone


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    """y = (x * 1/sqrt(mean(x^2) + eps)) * gain, eps inside the root, gain used as stored
    (src/runtime/kernels/cpu_kernels.cpp:225-256).  The reference adds the residual with a
    separate Add node before the norm (src/model/transformer_graph_builder.cpp:251-257); here
    the norm kernel takes the not-yet-added contribution `delta` and does both."""

    def __init__(self, rt: Runtime, prefix: str, size: int, eps: float, leaf: str = "weight"):
        super().__init__(rt, prefix)
        self.size = int(size)
        self.eps = float(eps)
        self.leaf = leaf
        self.gain: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.name(self.leaf): WeightSpec((self.size,), role="vector", init="gain")}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.gain = tensors[self.name(self.leaf)]

    def emit(self, plan: Plan, x: torch.Tensor, delta: Optional[torch.Tensor] = None, rows: str = ROWS_TOKENS,
             out_name: Optional[str] = None) -> torch.Tensor:
        out = self.rt.workspace(out_name or ("normed" if rows == ROWS_TOKENS else "normed_rows"), self.size, self.rt.dtype)
        plan.rmsnorm(x, self.gain, self.eps, out, delta=delta, rows=rows)
        return out

    def pairs_with(self, other) -> bool:
        """Whether `other` norms the same rows in the same way but for its gain, so that one pass can serve both."""
        return (isinstance(other, RMSNorm) and other.size == self.size and other.eps == self.eps and self.gain is not None
                and other.gain is not None and other.gain.dtype == self.gain.dtype)

    def emit_pair(self, plan: Plan, other: "RMSNorm", x: torch.Tensor, delta: Optional[torch.Tensor] = None,
                  other_name: str = "normed_second"):
        """Both norms of the same x (this one's and `other`'s) as one record; returns the two outputs."""
        out = self.rt.workspace("normed", self.size, self.rt.dtype)
        out2 = self.rt.workspace(other_name, self.size, self.rt.dtype)
        plan.rmsnorm(x, self.gain, self.eps, out, delta=delta, gain2=other.gain, out2=out2)
        return out, out2

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor] = None,
                out_rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        from ..engine.batch import StepBatch
        plan = Plan()
        out = self.emit(plan, x, delta=delta, rows=ROWS_TOKENS if out_rows is None else ROWS_LOGITS)
        run_alone(self.rt, plan, StepBatch.bare(x.shape[0], x.device, logit_rows=out_rows))
        return out[: x.shape[0] if out_rows is None else out_rows.numel()]


@register_part("norm", "rmsnorm_scalar")
class ScalarGainRMSNorm(RMSNorm):
    """y = x / sqrt(mean(x^2) + eps) * g with ONE learned number g for all coordinates (a tensor without
    dimensions).  The kernels are those of the norm with a gain vector: the number is spread over a vector when
    the weights are loaded, so the fused residual add and the row gather of the final norm serve it too."""

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.name(self.leaf): WeightSpec((), role="vector", init="gain")}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.gain = tensors[self.name(self.leaf)].reshape(1).expand(self.size).contiguous()


@register_part("norm", "rmsnorm_one_plus")
class OnePlusRMSNorm(RMSNorm):
    """y = x / sqrt(mean(x^2) + eps) * (1 + w): the stored vector w lies around zero.  1 + w is formed once in 32-bit when
    the weights are loaded; the kernels are those of the norm with a gain vector (as a pre-norm, and as the norm on a
    sublayer's output, which reads `gain` and `eps`)."""

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.name(self.leaf): WeightSpec((self.size,), role="vector", init="normal")}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.gain = (1.0 + tensors[self.name(self.leaf)].float()).contiguous()
