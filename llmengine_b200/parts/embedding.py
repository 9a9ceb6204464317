"""Token embedding and the output head."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..engine.plan import ROWS_LOGITS, Plan
from .base import Part, Runtime, WeightSpec, register_part, run_alone


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    """x[t,:] = E[ids[t],:] as 32-bit (src/runtime/kernels/cpu_kernels.cpp:262-274), times the constant `scale` where a
    design has one (the product is formed in 32-bit).

    `leaf` is the table's name below the prefix ("" = the prefix itself).  `extra_tables` (full tensor name ->
    width) are further per-token tables [vocab, width] that the part only stores: other parts of the model take
    them as shared tensors and gather from them by the step's token ids."""

    def __init__(self, rt: Runtime, prefix: str, vocab_size: int, hidden_size: int, leaf: str = "weight",
                 extra_tables: Optional[Dict[str, int]] = None, norm_leaf: Optional[str] = None,
                 norm_eps: Optional[float] = None, scale: float = 1.0):
        super().__init__(rt, prefix)
        self.vocab, self.hidden = int(vocab_size), int(hidden_size)
        self.leaf = leaf
        self.scale = float(scale)
        # with `norm_leaf`, the gathered rows are RMS-normed with that gain vector before they enter the stream
        self.norm_leaf, self.norm_eps = norm_leaf, None if norm_eps is None else float(norm_eps)
        if (norm_leaf is None) != (norm_eps is None):
            raise ValueError(f"{prefix}: a norm on the embedding needs both its tensor name and its eps")
        self.norm_gain: Optional[torch.Tensor] = None
        self.extra_widths = {n: int(w) for n, w in dict(extra_tables or {}).items()}
        self.table: Optional[torch.Tensor] = None
        self.extra: Dict[str, torch.Tensor] = {}

    def weight_specs(self) -> Dict[str, WeightSpec]:
        s = {self.name(self.leaf): WeightSpec((self.vocab, self.hidden))}
        for n, w in self.extra_widths.items():
            s[n] = WeightSpec((self.vocab, w), init="unit")
        if self.norm_leaf is not None:
            s[self.name(self.norm_leaf)] = WeightSpec((self.hidden,), role="vector", init="gain")
        return s

    def load_weights(self, t: Dict[str, torch.Tensor]) -> None:
        self.table = t[self.name(self.leaf)].contiguous()
        self.extra = {n: t[n].contiguous() for n in self.extra_widths}
        if self.norm_leaf is not None:
            self.norm_gain = t[self.name(self.norm_leaf)].contiguous()

    def shared_tensor(self, name: str) -> Optional[torch.Tensor]:
        if name in self.extra:
            return self.extra[name]
        return self.table if name == self.name(self.leaf) else None

    def emit(self, plan: Plan) -> torch.Tensor:
        x = self.rt.workspace("residual", self.hidden, torch.float32)
        plan.embedding(self.table, x, scale=self.scale)
        if self.norm_leaf is not None:
            # the stream in the type of the products too: a block whose sublayers read the stream itself finds it there
            copy = None if self.rt.dtype == torch.float32 else self.rt.workspace("stream_copy", self.hidden, self.rt.dtype)
            plan.postnorm(x, x, self.norm_gain, self.norm_eps, accumulate=False, copy=copy)
        return x

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        from ..engine.batch import StepBatch
        plan = Plan()
        x = self.emit(plan)
        run_alone(self.rt, plan, StepBatch.bare(token_ids.numel(), token_ids.device, token_ids=token_ids))
        return x[: token_ids.numel()]


@register_part("head", "lm_head")
class LMHead(Part):
    """logits = h W^T in 32-bit, no bias, no scaling (src/model/transformer_graph_builder.cpp:287).
    With `tied_to` (the name of the embedding's tensor), W is that table: stored once, used twice
    (src/io/gguf_weight_loader.cpp:46-50)."""

    def __init__(self, rt: Runtime, prefix: str, vocab_size: int, hidden_size: int, tied_to: Optional[str] = None,
                 tied: bool = False, leaf: str = "weight"):
        super().__init__(rt, prefix)
        self.vocab, self.hidden = int(vocab_size), int(hidden_size)
        self.leaf = leaf
        self.tied_to = tied_to
        self.tied = bool(tied) or tied_to is not None
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {} if self.tied else {self.name(self.leaf): WeightSpec((self.vocab, self.hidden))}

    def tied_tensors(self) -> Dict[str, str]:
        return {self.name(self.leaf): self.tied_to} if self.tied_to is not None else {}

    def receive_tied(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.tie(tensors[self.name(self.leaf)])

    def load_weights(self, t: Dict[str, torch.Tensor]) -> None:
        if not self.tied:
            self.weight = t[self.name(self.leaf)].contiguous()

    def tie(self, table: torch.Tensor) -> None:
        if tuple(table.shape) != (self.vocab, self.hidden):
            raise ValueError(f"{self.prefix}: a table of shape {tuple(table.shape)} cannot serve a head of "
                             f"{(self.vocab, self.hidden)}")
        self.weight = table

    def emit(self, plan: Plan, h: torch.Tensor) -> None:
        plan.linear(h, self.weight, None, rows=ROWS_LOGITS)      # into the step's logits

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        from ..engine.batch import StepBatch
        logits = self.rt.buffer("logits", h.shape[0], self.vocab, torch.float32)
        plan = Plan()
        self.emit(plan, h)
        rows = torch.arange(h.shape[0], dtype=torch.int32, device=h.device)
        run_alone(self.rt, plan, StepBatch.bare(h.shape[0], h.device, logit_rows=rows, logits=logits))
        return logits
