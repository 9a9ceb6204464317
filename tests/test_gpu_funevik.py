"""The Funevik design on the GPU against the plain implementation: single kernels, each mixer in a model of its own, every
schedule in both precisions and with both kernel sets, constants that are one off (negative controls on the plain
implementation, then the engine with the right ones), a key that stands out at a window's edge and one far back, a first
token that only the memory remembers, decoding from the first token on through captured steps, generation through the
scheduler, the trace program."""
import json
import math
import os
import subprocess

import numpy as np
import pytest
import torch

from funevik_cases import greedy_by_the_plain_model, reference_logits, replay_all_schedules, schedules, variant_dir
from helpers import compare, engine_for, max_live_tokens, random_ids, replay, trace_bulk_then_single, trace_portions, trace_whole
from plain_funevik import PlainFunevik, log_sigmoid, rms_norm, unit_rms
from test_gpu_vifelix import _batch, _ops, _run
from tiny_funevik import (ONLY_ATTENTION, ONLY_LATENT, ONLY_MEMORY, TINY_A, TINY_B, attention, dense, latent, layer, make_funevik_dir,
                          memory, model, moe)

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = "cuda:0"


# ----------------------------------------------------------------------------- single kernels
def _plain_gates(i_pre, f_pre, cap, M):
    """keep, take, floor [T] and the last maximum for one head, token by token."""
    keep, take, floor = [], [], []
    for t in range(i_pre.shape[0]):
        a, b = i_pre[t], f_pre[t]
        if cap > 0:
            a, b = cap * torch.tanh(a / cap), cap * torch.tanh(b / cap)
        b = log_sigmoid(b)
        new = torch.maximum(b + M, a)
        keep.append(torch.exp(b + M - new)); take.append(torch.exp(a - new)); floor.append(torch.exp(-new))
        M = new
    return torch.stack(keep), torch.stack(take), torch.stack(floor), M


@pytest.mark.parametrize("H,cap", [(1, 0.0), (3, 15.0), (6, 2.0)])
def test_exponential_gates_kernel(H, cap):
    """Requests of unequal length (one of a hundred tokens, one of a single token) in slots that are not in order, cut into two
    steps: the running maximum goes from step to step in the request's slot; gates of +-30 are capped (or not)."""
    ops = _ops()
    g = torch.Generator().manual_seed(H)
    lens, cuts, slots = [100, 1, 37, 33], [64, 0, 36, 1], [2, 0, 3, 5]
    pre = [torch.randn(L, 2 * H, generator=g) * 6 for L in lens]
    state = torch.zeros(7, H, device=DEV)
    state[1] = float("nan")
    got = [[] for _ in lens]
    for step in range(2):
        spans = [(r, 0, cuts[r]) if step == 0 else (r, cuts[r], lens[r]) for r in range(len(lens))]
        spans = [s for s in spans if s[2] > s[1]]
        x = torch.cat([pre[r][a:b] for r, a, b in spans]).to(DEV)
        out = torch.zeros(x.shape[0], 3 * H, device=DEV)
        _run(ops, lambda p: p.exp_gates(i_pre=x[:, :H], f_pre=x[:, H:], cap=cap, state=state, keep=out[:, :H], take=out[:, H:2 * H],
                                        floor=out[:, 2 * H:]), _batch([b - a for _, a, b in spans], [slots[r] for r, _, _ in spans]))
        at = 0
        for r, a, b in spans:
            got[r].append(out[at:at + b - a].cpu())
            at += b - a
    for r, L in enumerate(lens):
        y = torch.cat(got[r])
        for h in range(H):
            keep, take, floor, M = _plain_gates(pre[r][:, h], pre[r][:, H + h], cap, torch.tensor(0.0))
            for i, want in enumerate((keep, take, floor)):
                assert float(((y[:, i * H + h] - want).abs() / (want.abs() + 1e-3)).max()) < 1e-4, (r, h, i)
            assert abs(float(state[slots[r], h]) - float(M)) < 1e-4
    assert torch.isnan(state[1]).all()


@pytest.mark.parametrize("H,n,p,room", [(2, 8, 16, 0), (3, 6, 5, 0), (2, 32, 48, 40), (1, 200, 9, 30), (2, 64, 33, 8), (1, 40, 3, 4)])
def test_recurrence_with_given_gates_and_a_unit_column(H, n, p, room):
    """S_t = keep_t S + take_t k v^T with a last column whose v is one (the normaliser), single tokens beside portions and long
    portions cut into pieces; the second step starts every request from the state the first one left."""
    ops = _ops()
    g = torch.Generator().manual_seed(n + p)
    lens, cuts, slots = [431, 1, 128, 65, 2], [300, 0, 64, 0, 1], [1, 3, 0, 5, 2]
    P = p + 1
    scratch = torch.full((room * H * (P * n + 1),), float("nan"), device=DEV) if room else None
    mk = lambda *s: torch.randn(*s, generator=g)
    q, k, v = [mk(L, H * n) for L in lens], [mk(L, H * n) / math.sqrt(n) for L in lens], [mk(L, H * p).to(torch.bfloat16) for L in lens]
    keep, take = [torch.rand(L, H, generator=g) * 0.5 + 0.5 for L in lens], [torch.rand(L, H, generator=g) for L in lens]
    state = torch.zeros(max(slots) + 2, H, P, n, device=DEV)
    got = [[] for _ in lens]
    for step in range(2):
        spans = [(r, 0, cuts[r]) if step == 0 else (r, cuts[r], lens[r]) for r in range(len(lens))]
        spans = [s for s in spans if s[2] > s[1]]
        cat = lambda xs: torch.cat([xs[r][a:b] for r, a, b in spans]).to(DEV)
        gates = torch.cat([cat(keep), cat(take)], 1)
        out = torch.zeros(gates.shape[0], H * P, device=DEV)
        _run(ops, lambda pl: pl.recurrence(q=cat(q), k=cat(k), v=cat(v), state=state, out=out, heads=H, n=n, p=P, qk_groups=H, scratch=scratch,
                                           keep=gates[:, :H], take=gates[:, H:], unit_column=True),
             _batch([b - a for _, a, b in spans], [slots[r] for r, _, _ in spans]))
        at = 0
        for r, a, b in spans:
            got[r].append(out[at:at + b - a].cpu())
            at += b - a
    for r, L in enumerate(lens):
        y = torch.cat(got[r]).view(L, H, P)
        for h in range(H):
            S, want = torch.zeros(n, P), []
            for t in range(L):
                vv = torch.cat([v[r][t, h * p:(h + 1) * p].float(), torch.ones(1)])
                S = keep[r][t, h] * S + take[r][t, h] * k[r][t, h * n:(h + 1) * n][:, None] * vv[None, :]
                want.append(S.t() @ q[r][t, h * n:(h + 1) * n])
            want = torch.stack(want)
            assert float((y[:, h] - want).abs().max()) < 1e-4 * max(1.0, float(want.abs().max())), (r, h)
            assert float((state[slots[r], h].cpu() - S.t()).abs().max()) < 1e-4 * max(1.0, float(S.abs().max()))
    assert float(state[max(slots) + 1].abs().max()) == 0.0


@pytest.mark.parametrize("groups,group", [(4, 16), (3, 5), (2, 48), (2, 300)])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_normalised_gated_norm_kernel(dtype, tol, groups, group):
    """Groups of y that carry their normaliser behind them: divided by max(|d|, floor) + 1e-6, RMS-normed, times a weight and a
    sigmoid gate.  Both branches of the maximum occur."""
    ops = _ops()
    g = torch.Generator().manual_seed(group)
    T, cols = 7, groups * group
    y = torch.randn(T, groups, group + 1, generator=g) * 3
    floor = torch.rand(T, groups, generator=g) * 2
    gate, w = torch.randn(T, cols, generator=g).to(dtype), 1 + 0.2 * torch.randn(cols, generator=g)
    out = torch.zeros(T + 1, cols, dtype=dtype, device=DEV)
    _run(ops, lambda p: p.gated_norm(y=y.reshape(T, -1).to(DEV), gate=gate.to(DEV), weight=w.to(DEV), out=out, group=group, gate_first=False,
                                     eps=1e-5, gate_act="sigmoid", floor=floor.to(DEV), den_eps=1e-6), _batch([T], [0]))
    den = torch.maximum(y[..., -1].abs(), floor) + 1e-6
    assert bool((y[..., -1].abs() > floor).any()) and bool((y[..., -1].abs() < floor).any())
    want = unit_rms(y[..., :-1] / den[..., None], 1e-5).reshape(T, cols) * w * torch.sigmoid(gate.float())
    assert float((out[:T].float().cpu() - want).abs().max()) < tol * max(1.0, float(want.abs().max()))
    assert float(out[T].abs().max()) == 0.0


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
def test_small_records_of_the_design(dtype, tol):
    """A norm on a column range of a product (narrow and wider than a warp's share); two norms of the same rows as one record;
    a sigmoid gate with one value per head;
    contributions times scale vectors in the residual add; the gated activation with gelu in its tanh form."""
    ops = _ops()
    g = torch.Generator().manual_seed(4)
    T = 6
    for C in (12, 48, 1500):
        wide = torch.randn(T, C + 9, generator=g).to(dtype)
        gain = (1 + 0.2 * torch.randn(C, generator=g)).to(dtype)
        out = torch.zeros(T + 1, C + 3, dtype=dtype, device=DEV)
        xs = wide.to(DEV)
        _run(ops, lambda p: p.row_norm(x=xs[:, 5:5 + C], gain=gain.to(DEV), eps=1e-5, out=out[:, 2:2 + C]), _batch([T], [0]))
        want = rms_norm(wide[:, 5:5 + C].float(), gain.float(), 1e-5)
        assert float((out[:T, 2:2 + C].float().cpu() - want).abs().max()) < tol * 3 and float(out[T].abs().max()) == 0.0
        assert float(out[:, :2].abs().max()) == 0.0 and float(out[:, 2 + C:].abs().max()) == 0.0
    for D in (20, 64, 1100, 4096):              # two norms of the same rows in one pass (scalar and 16-byte forms), with the pending add
        x, delta = torch.randn(T, D, generator=g), torch.randn(T, D, generator=g).to(dtype)
        g1, g2 = 1 + 0.2 * torch.randn(D, generator=g), 1 + 0.2 * torch.randn(D, generator=g)
        xd, o1, o2 = x.to(DEV), torch.zeros(T, D, dtype=dtype, device=DEV), torch.zeros(T, D, dtype=dtype, device=DEV)
        _run(ops, lambda p: p.rmsnorm(xd, g1.to(DEV), 1e-5, o1, delta=delta.to(DEV), gain2=g2.to(DEV), out2=o2), _batch([T], [0]))
        summed = x + delta.float()
        assert float((xd.cpu() - summed).abs().max()) < 1e-6
        for got, gain in ((o1, g1), (o2, g2)):
            assert float((got.float().cpu() - rms_norm(summed, gain, 1e-5)).abs().max()) < tol * 3
    H, dv = 3, 10
    a, s = torch.randn(T, H * dv, generator=g).to(dtype), torch.randn(T, H + 2, generator=g).to(dtype)
    place, sd = torch.zeros(T, H * dv, dtype=dtype, device=DEV), s.to(DEV)
    _run(ops, lambda p: p.pointwise("sigmoid_mul", a.to(DEV), sd[:, 1:1 + H], place, group=dv), _batch([T], [0]))
    want = a.float() * torch.sigmoid(s[:, 1:1 + H].float()).repeat_interleave(dv, 1)
    assert float((place.float().cpu() - want).abs().max()) < tol
    D = 20
    x, u, v = torch.randn(T, D, generator=g), torch.randn(T, D, generator=g), torch.randn(T, D, generator=g)
    su, sv = torch.randn(D, generator=g), torch.randn(D, generator=g)
    xd = x.to(DEV)
    _run(ops, lambda p: p.residual_add(xd, u.to(DEV), v.to(DEV), a_scale=su.to(DEV), b_scale=sv.to(DEV)), _batch([T], [0]))
    assert float((xd.cpu() - (x + u * su + v * sv)).abs().max()) < 1e-5
    xd = x.to(DEV)
    _run(ops, lambda p: p.residual_add(xd, u.to(DEV), None, a_scale=su.to(DEV)), _batch([T], [0]))
    assert float((xd.cpu() - (x + u * su)).abs().max()) < 1e-5
    K, N = 40, 24
    xx, w = torch.randn(T, K, generator=g).to(dtype), (torch.randn(N, K, generator=g) / 3).to(dtype)
    gu, act = torch.zeros(T, N, dtype=dtype, device=DEV), torch.zeros(T, N // 2, dtype=dtype, device=DEV)
    _run(ops, lambda p: p.linear_swiglu(xx.to(DEV), w.to(DEV), gu, act, act="gelu_tanh"), _batch([T], [0]))
    z = (xx.float() @ w.float().t()).to(dtype).float()
    gz = z[:, :N // 2]
    want = 0.5 * gz * (1 + torch.tanh(math.sqrt(2 / math.pi) * (gz + 0.044715 * gz ** 3))) * z[:, N // 2:]
    assert float((act.float().cpu() - want).abs().max()) < tol * 2


@pytest.mark.parametrize("E,top", [(5, 1), (6, 2), (16, 4), (3, 3), (40, 9)])
def test_routing_by_the_softmax_over_the_chosen_logits(E, top):
    """The largest logits are chosen (read from a column range of a wider row), the weights are the softmax over the chosen
    alone, the pairs are listed expert by expert; the shared part enters the sum through a sigmoid gate of its own."""
    ops = _ops()
    g = torch.Generator().manual_seed(E)
    T, D = 9, 12
    wide = (torch.randn(T, E + 1, generator=g) * 3).to(DEV)
    experts, weights = torch.zeros(T, top, dtype=torch.int32, device=DEV), torch.zeros(T, top, device=DEV)
    offsets, counts = torch.zeros(E + 1, dtype=torch.int32, device=DEV), torch.zeros(E, dtype=torch.int32, device=DEV)
    order = torch.zeros(T * top, dtype=torch.int32, device=DEV)
    y, base, out = torch.randn(T * top, D, generator=g).to(DEV), torch.randn(T, D, generator=g).to(DEV), torch.zeros(T, D, device=DEV)

    def records(p):
        p.moe_route(logits=wide[:, :E], top_k=top, scale=1.0, experts=experts, weights=weights, offsets=offsets, order=order, counts=counts,
                    mode="softmax_chosen")
        p.moe_combine(y=y, weights=weights, base=base, out=out, base_gate=wide[:, E:E + 1])
    _run(ops, records, _batch([T], [0]))
    val, idx = torch.topk(wide[:, :E].cpu(), top, dim=-1)
    assert torch.equal(experts.cpu().long(), idx)
    wt = torch.softmax(val, -1)
    assert float((weights.cpu() - wt).abs().max()) < 1e-6
    off, od = offsets.cpu().tolist(), order.cpu().tolist()
    for e in range(E):
        assert sorted(od[off[e]:off[e + 1]]) == sorted(i for i in range(T * top) if int(idx.reshape(-1)[i]) == e)
    want = base.cpu() * torch.sigmoid(wide[:, E:E + 1].cpu()) + (wt[:, :, None] * y.cpu().view(T, top, D)).sum(1)
    assert float((out.cpu() - want).abs().max()) < 1e-5 and float(counts.abs().max()) == 0


# ----------------------------------------------------------------------------- each mixer in a model of its own
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg", [("memory", ONLY_MEMORY), ("latent", ONLY_LATENT), ("attention", ONLY_ATTENTION)])
def test_each_mixer_alone(tmp_path, name, cfg, dtype):
    d = make_funevik_dir(str(tmp_path / name), cfg, seed=9)
    replay_all_schedules(d, cfg, dtype, [70, 5, 130, 1, 2], 16, None, DEV, only=("whole", "bulk_then_single", "portions"))


# ----------------------------------------------------------------------------- every schedule
# sizes the tensor-core kernels take (a latent of 128 with a window that is no multiple of a key tile; keys of 64 with values of
# 32), memories of 64 and 128 rows, windows that end inside pages
BIG = model(131, 128, 1e-6, 11.0, [
    layer("latent_attention", latent(4, 32, 32, 32, 128, 96, 0.125, size=70, base=5000.0, dims=16), moe(8, 2, 64, shared=96)),
    layer("mlstm", memory(4, 64, 32, cap=15.0), dense(192)),
    layer("attention", attention(4, 2, 64, 32, 0.11, 4, base=5000.0, dims=32, softcap=20.0), dense(96)),
    layer("mlstm", memory(2, 128, 64, cap=15.0)),
    layer("latent_attention", latent(8, 16, 16, 16, 64, 64, 0.2, base=700.0)),
    layer("attention", attention(2, 1, 128, 128, 0.09, 2, base=100.0, dims=64, size=33), dense(160)),
])


@pytest.mark.parametrize("kernels", ["fast", "plain"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg,page,lens", [
    ("A", TINY_A, 16, [70, 33, 100, 1, 19, 45, 64]),
    ("B", TINY_B, 8, [2, 5, 64, 130, 200, 48]),
    ("M", ONLY_MEMORY, 64, [150, 3, 40, 64, 7]),
    ("BIG", BIG, 64, [200, 129, 40, 260, 128, 17]),
    ("BIG16", BIG, 16, [260, 3, 141, 64]),
])
def test_replay_gpu(tmp_path, name, cfg, page, lens, dtype, kernels):
    d = make_funevik_dir(str(tmp_path / name), cfg, seed=11)
    worst = replay_all_schedules(d, cfg, dtype, lens, page, None, DEV, kernels=kernels)
    print(f"replay {name} {dtype} {kernels}: share of the tolerance: " + ", ".join(f"{k} {v:.2f}" for k, v in worst.items()))


# ----------------------------------------------------------------------------- constants that are one off
EDGE = model(50, 64, 1e-5, 6.0, [
    layer("latent_attention", latent(4, 16, 8, 16, 32, 24, 0.5, size=21, base=1000.0, dims=4)),
    layer("attention", attention(4, 2, 32, 16, 0.4, 3, base=200.0, dims=8, softcap=4.0), moe(4, 2, 32, shared=16)),
    layer("mlstm", memory(2, 16, 16, cap=3.0), dense(48)),
])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_constants_that_are_one_off(tmp_path, dtype):
    """A window one key wider or narrower, other rotated coordinates, another cap on the scores or on the gates, another
    scale, one expert fewer: each moves the plain implementation's logits far beyond the tolerance.  The engine, with the
    right constants, stays within it at every position, in prompts and decoded, with page edges (4, 16, 64) inside and
    outside the window."""
    d = make_funevik_dir(str(tmp_path / "edge"), EDGE, seed=31)
    reqs = {"a": random_ids(150, 50, 1), "b": random_ids(23, 50, 2), "c": random_ids(5, 50, 3)}
    ref, tol = reference_logits(d, reqs, dtype)
    changes = {
        "window + 1": lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 22),
        "window - 1": lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 20),
        "no window": lambda c: c["layers"][0]["mixer"].pop("mask"),
        "more of the shared key part rotated": lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 8),
        "attention rotated otherwise": lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 16),
        "another cap on the scores": lambda c: c["layers"][1]["mixer"].__setitem__("softcap", 8.0),
        "no cap on the scores": lambda c: c["layers"][1]["mixer"].pop("softcap"),
        "a window on the attention": lambda c: c["layers"][1]["mixer"].__setitem__("mask", {"size": 40}),
        "another cap on the gates": lambda c: c["layers"][2]["mixer"].__setitem__("gate_cap", 6.0),
        "one expert per token": lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 1),
        "embedding not scaled": lambda c: c["embedding"].__setitem__("scale", 1.0),
    }
    for what, change in changes.items():
        other = PlainFunevik(variant_dir(d, str(tmp_path / what.replace(" ", "_")), change))
        moved = float((other.logits(reqs["a"]) - ref["a"]).abs().max())
        assert moved > 3 * tol, f"{what} moves the logits by {moved:.3g} only (tolerance {tol:.3g})"
    for page in (4, 16, 64):
        for what, steps in (("whole", trace_whole(reqs)), ("decoded", trace_bulk_then_single(reqs, 60)), ("portions", trace_portions(reqs))):
            eng = engine_for(d, dtype, 320, page_size=page, max_requests=2, max_model_len=256)
            compare(replay(eng, steps, poison=True), ref, tol, f"{dtype}/page {page}/{what}")


def _constant_first_coordinate(w, scale, norm="l0.norm1"):
    """Every token's embedding gets the same first coordinate, so that the first layer's input has a part that does not depend
    on the token: a query built on it looks for the same key from every position."""
    e = w["embed"].float()
    e[:, 0] = 2.0 / scale
    w["embed"] = e.to(torch.bfloat16)
    n = w[norm].float()
    n[0] = 1.0
    w[norm] = n.to(torch.bfloat16)


def _first_layer_input(w, token, scale, eps, norm="l0.norm1"):
    return unit_rms(w["embed"][token].float() * scale, eps) * w[norm].float()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_key_that_stands_out_at_the_latent_window_s_edge(tmp_path, dtype):
    """One token of the vocabulary gets a key that stands out: the last coordinate of the shared key part (not rotated, not
    normed) points along that token's input, and every head's query has a large constant there.  Wherever the token still
    lies inside a query's window it takes most of the attention: the logits jump where it leaves the window, and the engine
    has the jump where the plain implementation has it, for prompts and decoded tokens, at page sizes that put the token's
    page inside and outside the window."""
    H, d, r, R, Q, W = 2, 8, 4, 16, 8, 13
    cfg = model(40, 32, 1e-5, 4.0, [layer("latent_attention", latent(H, d, r, 8, R, Q, 0.6, size=W, base=100.0, dims=2))])

    def change(w):
        _constant_first_coordinate(w, 4.0)
        h7 = _first_layer_input(w, 7, 4.0, 1e-5)
        h7[0] = 0.0
        dkv = w["l0.mix.dkv"].float()
        dkv[R + r - 1] = 3.0 * h7 / (h7 @ h7)          # token 7: 3 on the last coordinate; the others about 3 / sqrt(width)
        dq = w["l0.mix.dq"].float()
        dq[0] = 0.0
        dq[0, 0] = 1.0                                 # the query latent's first coordinate: the constant part of the input
        uq = w["l0.mix.uq"].float()
        for a in range(H):
            uq[a * (d + r) + d + r - 1] = 0.0
            uq[a * (d + r) + d + r - 1, 0] = 4.0       # every head looks for it
        gain = w["l0.mix.dq.norm"].float()
        gain[0] = 1.0
        w.update({"l0.mix.dkv": dkv.to(torch.bfloat16), "l0.mix.dq": dq.to(torch.bfloat16), "l0.mix.uq": uq.to(torch.bfloat16),
                  "l0.mix.dq.norm": gain.to(torch.bfloat16), "l0.mix.sink": torch.zeros(H).to(torch.bfloat16)})
    d_ = make_funevik_dir(str(tmp_path / "m"), cfg, seed=2, change=change)
    ids = [t if t != 7 else 8 for t in random_ids(60, 40, 4)]
    ids[20] = 7                                                    # seen by queries 20 .. 32, not by 33
    reqs = {"a": ids}
    ref, tol = reference_logits(d_, reqs, dtype)
    without = list(ids)
    without[20] = 9
    plain = PlainFunevik(d_)
    seen = (plain.logits(ids) - plain.logits(without)).abs().amax(-1)
    assert float(seen[20 + W - 1]) > 20 * tol and float(seen[20 + W:].max()) < tol, "the token shows exactly while it is inside the window"
    for page in (4, 16):
        for what, steps in (("whole", trace_whole(reqs)), ("decoded", trace_bulk_then_single(reqs, 35)), ("portions", trace_portions(reqs, (19, 2, 11, 1, 2, 3)))):
            eng = engine_for(d_, dtype, 128, page_size=page, max_requests=2, max_model_len=128)
            compare(replay(eng, steps, poison=True), ref, tol, f"{dtype}/page {page}/{what}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_key_far_back_among_hundreds(tmp_path, dtype):
    """The attention without a window: one token's key stands out on a coordinate that is not rotated and that the convolution
    passes unchanged (taps 0, 0, 1), and every query looks for it.  Put at position 3 of 400 it still takes most of the
    attention at the end, over page borders: exchanging it moves the last logits by many tolerances, in the plain
    implementation and, within the tolerance of it, in the engine; the sink of one takes part (without the key the weights
    do not add up to one)."""
    H, G, dk = 2, 1, 16
    cfg = model(40, 32, 1e-5, 4.0, [layer("attention", attention(H, G, dk, 8, 0.5, 3, base=100.0, dims=8, softcap=9.0))])

    def change(w):
        _constant_first_coordinate(w, 4.0)
        h7 = _first_layer_input(w, 7, 4.0, 1e-5)
        h7[0] = 0.0
        k, q = w["l0.mix.k"].float(), w["l0.mix.q"].float()
        k[dk - 1] = 3.0 * h7 / (h7 @ h7)
        kc, qc = w["l0.mix.k.conv"].float(), w["l0.mix.q.conv"].float()
        kc[dk - 1] = torch.tensor([0.0, 0.0, 1.0])
        for a in range(H):
            q[a * dk + dk - 1] = 0.0
            q[a * dk + dk - 1, 0] = 3.0
            qc[a * dk + dk - 1] = torch.tensor([0.0, 0.0, 1.0])
        w.update({"l0.mix.k": k.to(torch.bfloat16), "l0.mix.q": q.to(torch.bfloat16), "l0.mix.k.conv": kc.to(torch.bfloat16),
                  "l0.mix.q.conv": qc.to(torch.bfloat16)})
    d_ = make_funevik_dir(str(tmp_path / "m"), cfg, seed=3, change=change)
    ids = [t if t != 7 else 8 for t in random_ids(400, 40, 5)]
    ids[3] = 7
    reqs = {"a": ids, "b": ids[:70]}
    ref, tol = reference_logits(d_, reqs, dtype)
    without = list(ids)
    without[3] = 9
    plain = PlainFunevik(d_)
    assert float((plain.logits(ids)[-1] - plain.logits(without)[-1]).abs().max()) > 20 * tol
    for page in (16, 64):
        for what, steps in (("whole", trace_whole(reqs)), ("decoded", trace_bulk_then_single(reqs, 40)), ("portions", trace_portions(reqs))):
            eng = engine_for(d_, dtype, 512, page_size=page, max_requests=2, max_model_len=512)
            compare(replay(eng, steps, poison=True), ref, tol, f"{dtype}/page {page}/{what}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_first_token_that_only_the_memory_remembers(tmp_path, dtype):
    """A model whose latent window is 4 tokens and whose memories rarely forget (forget gates near one): changing the FIRST token
    of a prompt of 300 still moves the last logits beyond the 32-bit tolerance, so a state that is lost, zeroed or taken from
    another slot on the way (portions, single tokens, slots used again) would show there."""
    cfg = model(45, 48, 1e-5, 5.0, [
        layer("mlstm", memory(2, 16, 16, cap=15.0)),
        layer("latent_attention", latent(2, 8, 4, 8, 16, 12, 0.3, size=4, base=100.0), dense(40)),
        layer("mlstm", memory(3, 8, 16, cap=15.0), dense(40)),
    ])

    def change(w):
        for i in (0, 2):
            w[f"l{i}.mix.f.b"] = torch.full_like(w[f"l{i}.mix.f.b"], 9.0)        # log forget gates about -1e-4
            w[f"l{i}.mix.i.b"] = torch.full_like(w[f"l{i}.mix.i.b"], -1.0)
    d = make_funevik_dir(str(tmp_path / "m"), cfg, seed=6, change=change)
    reqs = {f"r{i}": random_ids(n, 45, 70 + i) for i, n in enumerate([300, 40, 170, 9, 260])}
    ref, tol = reference_logits(d, reqs, dtype)
    plain = PlainFunevik(d)
    other = list(reqs["r0"])
    other[0] = (other[0] + 1) % 45
    if dtype == "float32":      # bfloat16 rounding of 300 tokens' sums moves these logits more than the first token does
        assert float((plain.logits(other)[-1] - ref["r0"][-1]).abs().max()) > 5 * tol
    for what, steps in schedules(reqs, tail=40).items():
        eng = engine_for(d, dtype, max_live_tokens(steps, 64), page_size=16, max_requests=4, max_model_len=512)
        compare(replay(eng, steps, poison=True), ref, tol, f"far/{dtype}/{what}")


# ----------------------------------------------------------------------------- from the first token on, for long
@pytest.mark.parametrize("cfg_name", ["A", "M"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_from_the_first_token_through_captured_steps(tmp_path, dtype, cfg_name):
    """Three requests decoded token by token from position 0 on, far past every window and over several pages, with the
    steps captured in CUDA graphs: the same logits as whole prompts.  Also for a model that keeps no pages at all."""
    from llmengine_b200.engine.engine import StepEntry
    cfg = TINY_A if cfg_name == "A" else ONLY_MEMORY
    d = make_funevik_dir(str(tmp_path / "m"), cfg, seed=13)
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
    d = make_funevik_dir(str(tmp_path / "m"), TINY_A, seed=5)
    llm = LLM(d, dtype="float32", page_size=16, max_cached_tokens=512, max_num_seqs=4, max_num_batched_tokens=64,
              prefill_chunk=40, max_model_len=256)
    prompts = [random_ids(n, TINY_A["vocab"], i) for i, n in enumerate([1, 5, 64, 90, 33, 7])]
    outs = llm.generate(prompts, SamplingParams(greedy=True), max_tokens=12, eos_token_id=None)
    plain = PlainFunevik(d)
    for p, o in zip(prompts, outs):
        assert o.token_ids == greedy_by_the_plain_model(plain, p, 12)
    llm.engine.cache.check_invariants()
    assert not llm.engine.cache.requests and llm.scheduler.all_done()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path, dtype):
    cfg = TINY_A
    d = make_funevik_dir(str(tmp_path / "m"), cfg, seed=17)
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
