"""Shared equipment of the Vifelix tests: the schedules a set of requests is replayed under and the comparison with the
plain implementation."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from helpers import (compare, engine_for, max_live_tokens, random_ids, replay, trace_bulk_then_single, trace_mixed,
                     trace_portions, trace_whole)
from plain_vifelix import PlainVifelix

TOL_F32 = 3e-4          # for logits of order one to ten (only the order of sums differs); it grows with larger ones


def reference_logits(model_dir: str, reqs: Dict[str, List[int]], dtype: str):
    """(reference, tolerance).  32-bit engine: the plain implementation in 32-bit.  bfloat16 engine: the plain
    implementation rounding to bfloat16 where the engine stores bfloat16; the yardstick of the tolerance is the model's
    own sensitivity to rounding (the distance between the rounded and the unrounded plain run): the engine must stay
    within one and a half yardsticks of the rounded run."""
    plain = PlainVifelix(model_dir)
    ref = {r: plain.logits(ids) for r, ids in reqs.items()}
    if dtype != "bfloat16":
        return ref, TOL_F32 * max(1.0, max(float(v.abs().max()) for v in ref.values()) / 10.0)
    rounded = PlainVifelix(model_dir, round_to=torch.bfloat16)
    ref16 = {r: rounded.logits(ids) for r, ids in reqs.items()}
    inherent = max(float((ref16[r] - ref[r]).abs().max()) for r in ref)
    return ref16, max(5e-3, 1.5 * inherent)


def schedules(reqs: Dict[str, List[int]], tail: int = 32):
    prompt = {r: max(1, len(ids) - 12) for r, ids in reqs.items()}
    return {
        "whole": trace_whole(reqs),
        "bulk_then_single": trace_bulk_then_single(reqs, tail),
        "portions": trace_portions(reqs),
        "mixed": trace_mixed(reqs, prompt, max_live=4, seed=3),
    }


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


def greedy_by_the_plain_model(plain: PlainVifelix, prompt: Sequence[int], n: int) -> List[int]:
    ids, out = list(prompt), []
    for _ in range(n):
        t = int(torch.argmax(plain.logits(ids)[-1]))
        out.append(t)
        ids.append(t)
    return out
