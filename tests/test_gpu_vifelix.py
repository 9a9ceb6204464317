"""The Vifelix design on the GPU against the plain implementation: single kernels, each mixer in a model of its own, every
schedule in both precisions and with both kernel sets, constants that are one off (negative controls on the plain
implementation, then the engine with the right ones), a key that stands out at a window's edge, a token far back that
only the states remember, decoding from the first token on through captured steps, generation through the scheduler,
the trace program."""
import json
import math
import os
import subprocess

import numpy as np
import pytest
import torch

from helpers import compare, engine_for, max_live_tokens, random_ids, replay, trace_bulk_then_single, trace_portions, trace_whole
from plain_vifelix import PlainVifelix, causal_conv, rotate_partial, silu, softplus, unit_rms
from tiny_vifelix import (ONLY_PARALLEL, ONLY_STATE, TINY_A, TINY_B, layer, left, make_vifelix_dir, model, parallel, right, ssm)
from torisun_cases import variant_dir
from vifelix_cases import greedy_by_the_plain_model, reference_logits, replay_all_schedules, schedules

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = "cuda:0"


def _ops(kernels="fast"):
    from llmengine_b200.kernels.ops import CudaOps
    ops = CudaOps(torch.device(DEV))
    ops.choose_kernels(kernels)
    return ops


def _run(ops, record, batch):
    from llmengine_b200.engine.plan import Plan
    plan = Plan()
    record(plan)
    ops.compile(plan).run(batch)
    torch.cuda.synchronize()


def _batch(q_lens, slots, positions=None):
    """A step of requests with `q_lens` tokens each in state slots `slots` (no pages)."""
    from llmengine_b200.engine.batch import StepBatch
    i32 = lambda v: torch.tensor(list(v), dtype=torch.int32, device=DEV)
    T = sum(q_lens)
    pos = positions if positions is not None else [p for n in q_lens for p in range(n)]
    req = [r for r, n in enumerate(q_lens) for _ in range(n)]
    return StepBatch(num_tokens=T, num_requests=len(q_lens), q_lens=list(q_lens), start_positions=[0] * len(q_lens), token_ids=i32([0] * T),
                     positions=i32(pos), token_request=i32(req), cu_q_lens=i32([0] + list(np.cumsum(q_lens))), ctx_lens=i32(q_lens),
                     state_slots=i32(slots), first_portion=i32([1] * len(q_lens)), logit_rows=i32([]),
                     decode_rows=i32([i for i, q in enumerate(q_lens) if q == 1]), portion_rows=i32([i for i, q in enumerate(q_lens) if q != 1]),
                     groups=[])


# ----------------------------------------------------------------------------- single kernels
@pytest.mark.parametrize("C,K", [(40, 4), (7, 1), (300, 5), (64, 2), (50, 3), (1100, 4)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_short_convolution_kernel(dtype, C, K):
    """Three requests of unequal length in slots that are not in order, cut into two steps at places of their own (one
    request brings a single token in the second step, one nothing in the first): the state carries the last K - 1 inputs."""
    _check_short_convolution(dtype, C, K, [9, 1, 6], [4, 0, 5], 3)


@pytest.mark.parametrize("C,K", [(64, 4), (40, 3), (520, 2), (36, 5)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_short_convolution_over_long_portions(dtype, C, K):
    """Steps of more than a hundred tokens, rows that start on 16 bytes: the kernel in which a thread walks over 16 tokens
    with four channels; requests begin and end inside a walk, one brings a single token, one continues from its state."""
    _check_short_convolution(dtype, C, K, [150, 1, 37, 203], [90, 0, 36, 47], 4)


def _check_short_convolution(dtype, C, K, lens, cuts, pad):
    ops = _ops()
    g = torch.Generator().manual_seed(C + K)
    slots = [3, 0, 2, 4][:len(lens)]
    xs = [torch.randn(n, C, generator=g).to(dtype) for n in lens]
    w, b = torch.randn(C, K, generator=g), torch.randn(C, generator=g)
    state = torch.zeros(6, max(K - 1, 1), C, device=DEV)
    state[1] = float("nan")                                        # a slot nobody uses is never touched
    got = [[] for _ in lens]
    for step in range(2):
        spans = [(r, 0, cuts[r]) if step == 0 else (r, cuts[r], lens[r]) for r in range(len(lens))]
        spans = [s for s in spans if s[2] > s[1]]
        wide = torch.cat([torch.zeros(sum(b_ - a for _, a, b_ in spans), pad, dtype=dtype), torch.cat([xs[r][a:b_] for r, a, b_ in spans])], 1).to(DEV)
        out = torch.zeros(wide.shape[0] + 1, C, device=DEV)
        _run(ops, lambda p: p.short_conv(x=wide[:, pad:], w=w.to(DEV), bias=b.to(DEV), state=state, out=out, act="silu"),
             _batch([b_ - a for _, a, b_ in spans], [slots[r] for r, _, _ in spans]))
        assert float(out[-1].abs().max()) == 0.0
        at = 0
        for r, a, b_ in spans:
            got[r].append(out[at:at + b_ - a].cpu())
            at += b_ - a
    for r in range(len(lens)):
        want = silu(causal_conv(xs[r].float(), w, b))
        assert float((torch.cat(got[r]) - want).abs().max()) < 1e-5
    assert torch.isnan(state[1]).all() and torch.isfinite(state[[0, 2, 3, 4, 5]]).all()
    if K > 1:
        assert torch.equal(state[3][-1].cpu(), xs[0][-1].float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotation_kernel(dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(5)
    T, dim, dims = 6, 20, 12
    a, b = torch.randn(T, 3 * dim, generator=g).to(dtype), torch.randn(T, 2 * dim, generator=g).to(dtype)
    pos = [0, 1, 7, 100, 5000, 31]
    f = torch.tensor([77.0 ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64).float()
    oa, ob = torch.zeros(T, 3 * dim, device=DEV), torch.zeros(T, 2 * dim, device=DEV)
    _run(ops, lambda p: p.rotate(x=(a.to(DEV), b.to(DEV)), out=(oa, ob), heads=(3, 2), scale=(1.0, 0.25), dim=dim, rot_dims=dims,
                                 inv_freq=f.to(DEV)), _batch([T], [0], positions=pos))
    wa = rotate_partial(a.float().view(T, 3, dim), torch.tensor(pos), 77.0, dims).reshape(T, -1)
    wb = rotate_partial(b.float().view(T, 2, dim), torch.tensor(pos), 77.0, dims).reshape(T, -1) * 0.25
    assert float((oa.cpu() - wa).abs().max()) < 2e-4 and float((ob.cpu() - wb).abs().max()) < 2e-4   # the angle 5000 f is 32-bit
    assert torch.equal(oa.cpu()[0], a.float()[0])                  # position 0 turns nothing


def _recurrence_plain(q, k, v, decay, step, skip, S):
    """S_t = decay_t S_(t-1) + step_t k_t v_t^T; y_t = S_t^T q_t + skip v_t for one head: q, k [T, n], v [T, p]."""
    ys = []
    for t in range(q.shape[0]):
        S = decay[t] * S + step[t] * k[t][:, None] * v[t][None, :]
        ys.append(S.t() @ q[t] + skip * v[t])
    return torch.stack(ys), S


@pytest.mark.parametrize("H,G,n,p", [(4, 2, 8, 16), (3, 3, 6, 5), (2, 1, 40, 3), (2, 2, 128, 64), (1, 1, 200, 9)])
@pytest.mark.parametrize("gated", [False, True])
def test_recurrence_kernel(gated, H, G, n, p):
    """Both forms of the recurrence (a fixed decay per head; decay and step from every token's dt), requests of unequal
    length in two steps, a request that starts from a state left by the step before, heads sharing q and k by groups."""
    _check_recurrence(gated, H, G, n, p, [37, 1, 12], [30, 0, 11], [1, 3, 0], 0, 2e-5)


@pytest.mark.parametrize("H,G,n,p,room", [(2, 1, 8, 16, 64), (3, 3, 6, 5, 7), (2, 2, 128, 64, 20), (1, 1, 40, 9, 4), (1, 1, 200, 9, 30), (2, 1, 300, 12, 8)])
@pytest.mark.parametrize("gated", [False, True])
def test_recurrence_in_pieces(gated, H, G, n, p, room):
    """Long portions cut into pieces that run side by side: requests of one piece, of exactly one and two pieces, one token
    more and one fewer, beside single tokens; the second step starts every request from the state the first one left.  With
    little room the pieces grow longer than the shortest the kernel cuts (64 tokens)."""
    _check_recurrence(gated, H, G, n, p, [431, 1, 128, 65, 140, 64, 2], [300, 0, 64, 0, 11, 63, 1], [1, 3, 0, 5, 2, 6, 4],
                      room * H * (p * n + 1), 1e-4)


def _check_recurrence(gated, H, G, n, p, lens, cuts, slots, scratch_floats, tol):
    ops = _ops()
    g = torch.Generator().manual_seed(n + p)
    scratch = torch.full((scratch_floats,), float("nan"), device=DEV) if scratch_floats else None
    mk = lambda *s: torch.randn(*s, generator=g)
    q, k, v = [mk(L, G * n) for L in lens], [mk(L, G * n) / math.sqrt(n) for L in lens], [mk(L, H * p) for L in lens]
    dt = [mk(L, H).to(torch.bfloat16) for L in lens]
    dt_bias, a_log, skip = mk(H) - 1, mk(H) * 0.5, mk(H)
    decay = torch.rand(H, generator=g) * 0.3 + 0.7
    state = torch.zeros(max(slots) + 2, H, p, n, device=DEV)
    got = [[] for _ in lens]
    for step in range(2):
        spans = [(r, 0, cuts[r]) if step == 0 else (r, cuts[r], lens[r]) for r in range(len(lens))]
        spans = [s for s in spans if s[2] > s[1]]
        cat = lambda xs: torch.cat([xs[r][a:b] for r, a, b in spans]).to(DEV)
        out = torch.zeros(sum(b - a for _, a, b in spans), H * p, device=DEV)
        kw = dict(dt=cat(dt), dt_bias=dt_bias.to(DEV), a_log=a_log.to(DEV), skip=skip.to(DEV)) if gated else dict(decay=decay.to(DEV))
        _run(ops, lambda pl: pl.recurrence(q=cat(q), k=cat(k), v=cat(v), state=state, out=out, heads=H, n=n, p=p, qk_groups=G, scratch=scratch, **kw),
             _batch([b - a for _, a, b in spans], [slots[r] for r, _, _ in spans]))
        at = 0
        for r, a, b in spans:
            got[r].append(out[at:at + b - a].cpu())
            at += b - a
    for r, L in enumerate(lens):
        y = torch.cat(got[r])
        for h in range(H):
            gq = h // (H // G)
            if gated:
                st = softplus(dt[r][:, h].float() + dt_bias[h])
                dc = torch.exp(-torch.exp(a_log[h]) * st)
            else:
                st, dc = torch.ones(L), decay[h].expand(L)
            want, S = _recurrence_plain(q[r][:, gq * n:(gq + 1) * n], k[r][:, gq * n:(gq + 1) * n], v[r][:, h * p:(h + 1) * p], dc, st,
                                        skip[h] if gated else 0.0, torch.zeros(n, p))
            scale = max(1.0, float(want.abs().max()))
            assert float((y[:, h * p:(h + 1) * p] - want).abs().max()) < tol * scale, (r, h)
            assert float((state[slots[r], h].cpu() - S.t()).abs().max()) < tol * max(1.0, float(S.abs().max()))
    assert float(state[max(slots) + 1].abs().max()) == 0.0


@pytest.mark.parametrize("cols,group", [(64, 16), (30, 30), (36, 6), (512, 128), (1024, 512), (600, 300), (2048, 1024), (1300, 1300)])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_gated_group_norm_kernel(dtype, tol, cols, group):
    """The gate before the norm (the norm sees y silu(g)) and behind it (the norm sees y): the two orders differ."""
    ops = _ops()
    g = torch.Generator().manual_seed(cols)
    T = 5
    y, gate, w = torch.randn(T, cols, generator=g) * 3, torch.randn(T, cols, generator=g).to(dtype), 1 + 0.2 * torch.randn(cols, generator=g)
    res = {}
    for first in (True, False):
        out = torch.zeros(T + 1, cols, dtype=dtype, device=DEV)
        _run(ops, lambda p: p.gated_norm(y=y.to(DEV), gate=gate.to(DEV), weight=w.to(DEV) if first else None, out=out, group=group,
                                         gate_first=first, eps=1e-5, scale=1.0 if first else 1.5), _batch([T], [0]))
        sg = silu(gate.float())
        want = (unit_rms((y * sg).view(T, -1, group), 1e-5).reshape(T, cols) * w) if first else unit_rms(y.view(T, -1, group), 1e-5).reshape(T, cols) * sg * 1.5
        assert float((out[:T].float().cpu() - want).abs().max()) < tol * max(1.0, float(want.abs().max()))
        assert float(out[T].abs().max()) == 0.0
        res[first] = want
    assert float((res[True] - res[False]).abs().max()) > 0.1


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
def test_biases_and_scales_of_the_shared_records(dtype, tol):
    """What the design adds to records other designs use: a scaled embedding, a product with a bias, a gated activation
    whose gate and up rows have biases, a sigmoid gate times a constant into a strided place."""
    ops = _ops()
    g = torch.Generator().manual_seed(3)
    T, K, N = 6, 40, 24
    x, w, b = torch.randn(T, K, generator=g).to(dtype), (torch.randn(N, K, generator=g) / 6).to(dtype), torch.randn(N, generator=g)
    out = torch.zeros(T, N, device=DEV)
    _run(ops, lambda p: p.linear(x.to(DEV), w.to(DEV), out, bias=b.to(DEV)), _batch([T], [0]))
    assert float((out.cpu() - (x.float() @ w.float().t() + b)).abs().max()) < tol
    gu, act = torch.zeros(T, N, dtype=dtype, device=DEV), torch.zeros(T, N // 2, dtype=dtype, device=DEV)
    _run(ops, lambda p: p.linear_swiglu(x.to(DEV), w.to(DEV), gu, act, bias=b.to(DEV)), _batch([T], [0]))
    z = (x.float() @ w.float().t()).to(dtype).float() + b
    want = silu(z[:, :N // 2].to(dtype).float()) * z[:, N // 2:].to(dtype).float()
    assert float((act.float().cpu() - want).abs().max()) < tol * 2
    assert float((want - silu(z[:, :N // 2] - b[:N // 2]) * (z[:, N // 2:] - b[N // 2:])).abs().max()) > 0.1
    table = torch.randn(11, K, generator=g).to(dtype)
    emb = torch.zeros(T, K, device=DEV)
    bt = _batch([T], [0])
    bt.token_ids.copy_(torch.tensor([3, 0, 10, 3, 7, 1], dtype=torch.int32))
    _run(ops, lambda p: p.embedding(table.to(DEV), emb, scale=5.5), bt)
    assert torch.equal(emb.cpu(), table[[3, 0, 10, 3, 7, 1]].float() * 5.5)
    a, s = torch.randn(T, 16, generator=g).to(dtype), torch.randn(T, 16, generator=g).to(dtype)
    place = torch.zeros(T, 40, dtype=dtype, device=DEV)
    _run(ops, lambda p: p.pointwise("sigmoid_mul", a.to(DEV), s.to(DEV), place[:, 8:24], scale=1.3), _batch([T], [0]))
    assert float((place[:, 8:24].float().cpu() - a.float() * torch.sigmoid(s.float()) * 1.3).abs().max()) < tol
    assert float(place[:, :8].abs().max()) == 0.0 and float(place[:, 24:].abs().max()) == 0.0


# ----------------------------------------------------------------------------- each mixer in a model of its own
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg", [("state", ONLY_STATE), ("parallel", ONLY_PARALLEL)])
def test_each_mixer_alone(tmp_path, name, cfg, dtype):
    d = make_vifelix_dir(str(tmp_path / name), cfg, seed=9)
    replay_all_schedules(d, cfg, dtype, [70, 5, 130, 1, 2], 16, None, DEV, only=("whole", "bulk_then_single", "portions"))


# ----------------------------------------------------------------------------- every schedule
BIG = model(131, 128, 1e-6, 11.0, [
    layer("mamba2", ssm(4, 32, 64, 2, 4, 2)),
    layer("parallel", parallel(left(4, 2, 64, 0.125, 70, base=5000.0, dims=32), right(2, 64, 32, (0.97, 0.995), base=700.0), 1.1, 0.9), 192),
    layer("parallel", parallel(left(2, 1, 128, 0.09, 33, base=5000.0), right(4, 32, 64, (0.9, 0.99, 1.0, 0.95), dims=16), 0.8, 1.2), None),
    layer("mamba2", ssm(8, 16, 128, 1, 3, 1), 160),
])


@pytest.mark.parametrize("kernels", ["fast", "plain"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg,page,lens", [
    ("A", TINY_A, 16, [70, 33, 100, 1, 19, 45, 64]),
    ("B", TINY_B, 8, [2, 5, 64, 130, 200, 48]),
    ("S", ONLY_STATE, 64, [150, 3, 40, 64, 7]),
    ("BIG", BIG, 64, [300, 129, 40, 420, 128, 17]),
    ("BIG16", BIG, 16, [260, 3, 141, 64]),
])
def test_replay_gpu(tmp_path, name, cfg, page, lens, dtype, kernels):
    d = make_vifelix_dir(str(tmp_path / name), cfg, seed=11)
    worst = replay_all_schedules(d, cfg, dtype, lens, page, None, DEV, kernels=kernels)
    print(f"replay {name} {dtype} {kernels}: share of the tolerance: " + ", ".join(f"{k} {v:.2f}" for k, v in worst.items()))


# ----------------------------------------------------------------------------- constants that are one off
EDGE = model(50, 64, 1e-5, 6.0, [
    layer("parallel", parallel(left(4, 2, 32, 0.5, 21, base=1000.0, dims=16), right(2, 16, 32, (0.93, 0.99), base=200.0, dims=8), 1.0, 0.6), None),
    layer("mamba2", ssm(4, 16, 8, 2, 3, 2)),
])


def _sharpen(w):
    w["l0.mix.left.q.norm"] = (w["l0.mix.left.q.norm"].float() * 3).to(torch.bfloat16)     # attention far from uniform


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_constants_that_are_one_off(tmp_path, dtype):
    """A window one key wider or narrower, other rotated coordinates, the decays of two heads exchanged, another number of
    norm groups or of groups, taps in the other order, the gate behind the norm: each moves the plain implementation's
    logits far beyond the tolerance.  The engine, with the right constants, stays within it at every position, in prompts and
    decoded, with page edges (4, 16, 64) inside and outside the window."""
    d = make_vifelix_dir(str(tmp_path / "edge"), EDGE, seed=31, change=_sharpen)
    reqs = {"a": random_ids(150, 50, 1), "b": random_ids(23, 50, 2), "c": random_ids(5, 50, 3)}
    ref, tol = reference_logits(d, reqs, dtype)
    changes = {
        "window + 1": lambda c: c["layers"][0]["mixer"]["left"]["mask"].__setitem__("size", 22),
        "window - 1": lambda c: c["layers"][0]["mixer"]["left"]["mask"].__setitem__("size", 20),
        "all coordinates rotated": lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 32),
        "retention rotated otherwise": lambda c: c["layers"][0]["mixer"]["right"]["rot"].__setitem__("dims", 16),
        "decays exchanged": lambda c: c["layers"][0]["mixer"]["right"].__setitem__("decay", [0.99, 0.93]),
        "branch scales exchanged": lambda c: (c["layers"][0]["mixer"].__setitem__("left_scale", 0.6), c["layers"][0]["mixer"].__setitem__("right_scale", 1.0)),
        "one norm group": lambda c: c["layers"][1]["mixer"].__setitem__("norm_groups", 1),
        "embedding not scaled": lambda c: c["embedding"].__setitem__("scale", 1.0),
    }
    for what, change in changes.items():
        other = PlainVifelix(variant_dir(d, str(tmp_path / what.replace(" ", "_")), change))
        moved = float((other.logits(reqs["a"]) - ref["a"]).abs().max())
        assert moved > 3 * tol, f"{what} moves the logits by {moved:.3g} only (tolerance {tol:.3g})"
    for page in (4, 16, 64):
        for what, steps in (("whole", trace_whole(reqs)), ("decoded", trace_bulk_then_single(reqs, 60)), ("portions", trace_portions(reqs))):
            eng = engine_for(d, dtype, 320, page_size=page, max_requests=2, max_model_len=256)
            compare(replay(eng, steps, poison=True), ref, tol, f"{dtype}/page {page}/{what}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_key_that_stands_out_at_the_window_s_edge(tmp_path, dtype):
    """One token of the vocabulary gets a key that stands out: the key projection's last row (a coordinate that is not
    rotated) points along that token's normed embedding, and the query bias on that coordinate is large, so wherever the
    token still lies inside a query's window it takes most of the attention.  The logits jump at the position where it
    leaves the window, by more than twenty tolerances, and the engine has the jump where the plain implementation has it:
    for prompts and for decoded tokens, at page sizes that put the token's page inside and outside the window."""
    cfg = model(40, 32, 1e-5, 4.0, [layer("parallel", parallel(left(2, 1, 16, 0.6, 13, base=100.0, dims=8), right(1, 8, 8, (0.5,)), 1.5, 0.2), None)])

    def change(w):
        h7 = unit_rms(w["embed"][7].float() * 4.0, 1e-5) * (1 + w["l0.norm1"].float())
        k, kb, qb = w["l0.mix.left.k"].float(), w["l0.mix.left.k.b"].float(), w["l0.mix.left.q.b"].float()
        k[15] = 3.0 * h7 / (h7 @ h7)                   # token 7: 3 on the last coordinate; others about 3 / sqrt(width)
        kb[15] = 0.0
        qb[15] = qb[31] = 4.0                          # both query heads look for it
        w["l0.mix.left.k"], w["l0.mix.left.k.b"], w["l0.mix.left.q.b"] = k.to(torch.bfloat16), kb.to(torch.bfloat16), qb.to(torch.bfloat16)
    d = make_vifelix_dir(str(tmp_path / "m"), cfg, seed=2, change=change)
    ids = [t if t != 7 else 8 for t in random_ids(60, 40, 4)]
    ids[20] = 7                                                    # seen by queries 20 .. 32, not by 33
    reqs = {"a": ids}
    ref, tol = reference_logits(d, reqs, dtype)
    without = list(ids)
    without[20] = 9
    plain = PlainVifelix(d)
    seen = (plain.logits(ids) - plain.logits(without)).abs().amax(-1)
    assert float(seen[32]) > 20 * tol and float(seen[33:].max()) < tol, "the token shows exactly while it is inside the window"
    for page in (4, 16):
        for what, steps in (("whole", trace_whole(reqs)), ("decoded", trace_bulk_then_single(reqs, 35)), ("portions", trace_portions(reqs, (19, 2, 11, 1, 2, 3)))):
            eng = engine_for(d, dtype, 128, page_size=page, max_requests=2, max_model_len=128)
            compare(replay(eng, steps, poison=True), ref, tol, f"{dtype}/page {page}/{what}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_token_far_back_that_only_the_states_remember(tmp_path, dtype):
    """A model whose window is 4 tokens, whose retention never forgets (decay 1) and whose state space forgets slowly: changing
    the FIRST token of a prompt of 300 still moves the last logits far beyond the 32-bit tolerance, so a state that is lost,
    zeroed or taken from another slot on the way (portions, single tokens, slots used again) would show there; the bfloat16
    run replays the same schedules."""
    cfg = model(45, 48, 1e-5, 5.0, [
        layer("parallel", parallel(left(2, 1, 16, 0.3, 4, base=100.0), right(2, 16, 16, (1.0, 0.999), base=1e6), 0.3, 1.5), None),
        layer("mamba2", ssm(3, 16, 16, 1, 2, 3)),
    ])

    def change(w):
        w["l1.mix.A_log"] = torch.full((3,), -6.0).to(torch.bfloat16)     # decay exp(-exp(-6) dt): close to one
    d = make_vifelix_dir(str(tmp_path / "m"), cfg, seed=6, change=change)
    reqs = {f"r{i}": random_ids(n, 45, 70 + i) for i, n in enumerate([300, 40, 170, 9, 260])}
    ref, tol = reference_logits(d, reqs, dtype)
    plain = PlainVifelix(d)
    other = list(reqs["r0"])
    other[0] = (other[0] + 1) % 45
    if dtype == "float32":      # bfloat16 rounding of 300 tokens' sums moves these logits more than the first token does
        assert float((plain.logits(other)[-1] - ref["r0"][-1]).abs().max()) > 5 * tol
    for what, steps in schedules(reqs, tail=40).items():
        eng = engine_for(d, dtype, max_live_tokens(steps, 64), page_size=16, max_requests=4, max_model_len=512)
        compare(replay(eng, steps, poison=True), ref, tol, f"far/{dtype}/{what}")


# ----------------------------------------------------------------------------- from the first token on, for long
@pytest.mark.parametrize("cfg_name", ["A", "S"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_from_the_first_token_through_captured_steps(tmp_path, dtype, cfg_name):
    """Three requests decoded token by token from position 0 on, far past every window and over several pages, with the
    steps captured in CUDA graphs: the same logits as whole prompts.  Also for a model that keeps no pages at all."""
    from llmengine_b200.engine.engine import StepEntry
    cfg = TINY_A if cfg_name == "A" else ONLY_STATE
    d = make_vifelix_dir(str(tmp_path / "m"), cfg, seed=13)
    n = 150
    reqs = {f"r{i}": random_ids(n, cfg["vocab"], 50 + i) for i in range(3)}
    ref, tol = reference_logits(d, reqs, dtype)
    eng = engine_for(d, dtype, 3 * 192, page_size=16, max_requests=4, use_cuda_graphs=True, max_model_len=192)
    rows = {r: [] for r in reqs}
    for i in range(n):
        out = eng.step([StepEntry(r, [ids[i]], [0]) for r, ids in reqs.items()], list(reqs) if i == n - 1 else [])
        for k, r in enumerate(reqs):
            rows[r].append(out[k].float().cpu().clone())
    assert eng.graphs_enabled and eng._graphs, "the parts of this design can be captured"
    compare({r: torch.stack(v) for r, v in rows.items()}, ref, tol, f"captured decode {dtype}")
    eng.cache.check_invariants()
    assert all(g.pool.free_count == g.pool.num_pages for g in eng.cache.groups)


def test_greedy_generation_through_the_scheduler(tmp_path):
    from llmengine_b200 import LLM, SamplingParams
    d = make_vifelix_dir(str(tmp_path / "m"), TINY_A, seed=5)
    llm = LLM(d, dtype="float32", page_size=16, max_cached_tokens=512, max_num_seqs=4, max_num_batched_tokens=64,
              prefill_chunk=40, max_model_len=256)
    prompts = [random_ids(n, TINY_A["vocab"], i) for i, n in enumerate([1, 5, 64, 90, 33, 7])]
    outs = llm.generate(prompts, SamplingParams(greedy=True), max_tokens=12, eos_token_id=None)
    plain = PlainVifelix(d)
    for p, o in zip(prompts, outs):
        assert o.token_ids == greedy_by_the_plain_model(plain, p, 12)
    llm.engine.cache.check_invariants()
    assert not llm.engine.cache.requests and llm.scheduler.all_done()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path, dtype):
    cfg = TINY_A
    d = make_vifelix_dir(str(tmp_path / "m"), cfg, seed=17)
    reqs = {f"r{i}": random_ids(n, cfg["vocab"], 200 + i) for i, n in enumerate([70, 33, 100, 1, 19, 45])}
    ref, tol = reference_logits(d, reqs, dtype)
    steps = schedules(reqs)["mixed"]
    out = tmp_path / "out"
    lines = [json.dumps({"step": i, "entries": [{"id": r, "tokens": t, "want": w} for r, t, w in e], "end": end})
             for i, (e, end) in enumerate(steps)]
    p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out),
                        "--max-tokens", str(max_live_tokens(steps, 64))],
                       input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    rows = {}
    for i, (e, _) in enumerate(steps):
        arr = torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"]))
        k = 0
        for r, t, w in e:
            rows.setdefault(r, []).append(arr[k:k + len(w)])
            k += len(w)
        assert k == arr.shape[0]
    compare({r: torch.cat(v) for r, v in rows.items()}, ref, tol, f"trace_run/{dtype}")
