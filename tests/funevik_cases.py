"""Shared equipment of the Funevik tests: the schedules a set of requests is replayed under and the comparison with the
plain implementation."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from helpers import compare, engine_for, max_live_tokens, random_ids, replay
from plain_funevik import PlainFunevik
from torisun_cases import schedules, variant_dir          # noqa: F401  (the same four schedules; the same way to vary a config)

TOL_F32 = 3e-4          # for logits of order one to ten (only the order of sums differs); it grows with larger ones


def keep_away_from_close_calls(model: PlainFunevik, reqs: Dict[str, List[int]], margin: float) -> None:
    """Changes the requests IN PLACE until the model makes no close call on them: where the last chosen expert's logit lies
    less than `margin` above the first one not chosen, rounding decides which expert a token uses, and where a memory's
    query is nearly orthogonal to what the memory holds (its first token; a token behind a forget gate that emptied it),
    rounding decides the direction of that head's output; no comparison can rest on either.  The token at the first such position is exchanged for the next one of the vocabulary
    (positions before it are not affected: the model is causal)."""
    vocab = model.cfg["vocab"]
    for r, ids in reqs.items():
        for _ in range(40 * len(ids)):
            model.logits(ids)
            close = (model.gaps < margin).nonzero()
            if not close.numel():
                break
            p = int(close[0])
            ids[p] = (ids[p] + 1) % vocab
        else:
            raise AssertionError(f"request {r}: no way around the routers' close calls")


def reference_logits(model_dir: str, reqs: Dict[str, List[int]], dtype: str):
    """(reference, tolerance).  32-bit engine: the plain implementation in 32-bit.  bfloat16 engine: the plain implementation
    rounding to bfloat16 where the engine stores bfloat16; it is the reference because a mixture of experts is not
    continuous, and only a run that rounds where the engine rounds takes the same choices.  The yardstick of the tolerance is
    the model's own sensitivity to rounding (the distance between the rounded and the unrounded plain run): the engine must
    stay within two yardsticks of the rounded run (the models here have up to six layers, three kinds of mixer and routers in
    most layers, and the engine also rounds the attention's probabilities and the queries carried into the latent space)."""
    plain = PlainFunevik(model_dir)
    rounded = PlainFunevik(model_dir, round_to=torch.bfloat16)
    keep_away_from_close_calls(rounded if dtype == "bfloat16" else plain, reqs, 0.25 if dtype == "bfloat16" else 2e-4)
    ref = {r: plain.logits(ids) for r, ids in reqs.items()}
    if dtype != "bfloat16":
        return ref, TOL_F32 * max(1.0, max(float(v.abs().max()) for v in ref.values()) / 10.0)
    ref16 = {r: rounded.logits(ids) for r, ids in reqs.items()}
    inherent = max(float((ref16[r] - ref[r]).abs().max()) for r in ref)
    return ref16, max(5e-3, 2.0 * inherent)


def replay_all_schedules(model_dir: str, cfg: dict, dtype: str, lens: Sequence[int], page: int, ops, device: str,
                         kernels="fast", only: Optional[Sequence[str]] = None, seed: int = 100, tail: int = 32) -> Dict[str, float]:
    """Every schedule against the plain implementation, free pages poisoned before every step; in the mixed schedule at
    most four requests are live, so that pages and state slots are handed to a second request."""
    reqs = {f"r{i}": random_ids(n, cfg["vocab"], seed + i) for i, n in enumerate(lens)}
    ref, tol = reference_logits(model_dir, reqs, dtype)
    worst = {}
    for what, steps in schedules(reqs, tail).items():
        if only is not None and what not in only:
            continue
        pool = max_live_tokens(steps, 64)
        eng = engine_for(model_dir, dtype, pool, page_size=page, ops=ops, device=device, kernels=kernels, max_requests=4,
                         max_model_len=max(len(v) for v in reqs.values()) + 64)
        slots = set()
        got = replay(eng, steps, poison=True, tamper=lambda e, i: slots.update((r, st.slot) for r, st in e.cache.requests.items()))
        worst[what] = compare(got, ref, tol, f"{dtype}/{what}") / tol
        eng.cache.check_invariants()
        assert not eng.cache.requests, "every request was ended, nothing may be held"
        assert all(g.pool.free_count == g.pool.num_pages for g in eng.cache.groups)
        if what == "mixed" and len(reqs) > 4:
            by_slot: Dict[int, set] = {}
            for r, s in slots:
                by_slot.setdefault(s, set()).add(r)
            assert any(len(v) > 1 for v in by_slot.values()), "no state slot was handed to a second request"
    return worst


def greedy_by_the_plain_model(plain: PlainFunevik, prompt: Sequence[int], n: int) -> List[int]:
    ids, out = list(prompt), []
    for _ in range(n):
        t = int(torch.argmax(plain.logits(ids)[-1]))
        out.append(t)
        ids.append(t)
    return out
