"""The Funevik design on the host: configuration, tensor names, the cache a layer asks for, the plain implementation's
mechanisms on inputs whose result can be written down, and the engine's own logic (batch metadata, pages, state slots,
scheduling) with a CPU stand-in for the kernels, against the plain implementation."""
import copy
import math

import pytest
import torch

from funevik_cases import greedy_by_the_plain_model, replay_all_schedules
from helpers import random_ids
from host_ops import HostOps
from llmengine_b200 import LLM, SamplingParams
from llmengine_b200.config import ConfigError, FunevikConfig, config_from_dict
from llmengine_b200.engine.model import Model
from llmengine_b200.parts import Runtime
from llmengine_b200.parts.base import PagedAndStateSpec, StatesSpec
from plain_funevik import (PlainFunevik, causal_conv, causal_mask, conv_attention, gelu_tanh, latent_attention, log_sigmoid,
                           matrix_memory, rotate_interleaved, routed_ff, softmax_with_sink, unit_rms)
from tiny_funevik import ONLY_ATTENTION, ONLY_LATENT, ONLY_MEMORY, TINY_A, TINY_B, make_funevik_dir, tensor_shapes

ALL = [("A", TINY_A), ("B", TINY_B), ("M", ONLY_MEMORY), ("L", ONLY_LATENT), ("T", ONLY_ATTENTION)]


def test_every_size_and_constant_comes_from_the_file():
    c = config_from_dict(TINY_A)
    assert isinstance(c, FunevikConfig) and (c.hidden_size, c.vocab_size, c.norm_eps, c.embedding_scale) == (64, 101, 1e-5, 8.0)
    m, l, a = c.mixers[0], c.mixers[1], c.mixers[2]
    assert (m.heads, m.dim, m.vdim, m.gate_cap) == (2, 16, 32, 15.0)
    assert (l.heads, l.dim, l.rot_dim, l.vdim, l.kv_rank, l.q_rank, l.scale, l.rot_base, l.rot_dims, l.window) == (4, 16, 16, 32, 64, 48, 0.18, 500.0, 16, 11)
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.taps, a.rot_base, a.rot_dims, a.softcap, a.window) == (4, 2, 32, 16, 0.2, 4, 300.0, 16, 30.0, 0)
    f = c.mlps
    assert (f[0].kind, f[0].ff) == ("dense", 96) and (f[1].kind, f[1].ff, f[1].experts, f[1].top, f[1].shared_ff) == ("moe", 24, 6, 2, 40)
    assert f[2].shared_ff == 0 and f[3] is None
    b = config_from_dict(TINY_B)
    assert b.mixers[0].window == 9 and b.mixers[0].softcap == 0.0 and b.mixers[1].window == 0 and b.mixers[1].rot_dims == 4 and b.mixers[2].gate_cap == 0.0
    for cfg in (TINY_A, TINY_B):
        assert config_from_dict(config_from_dict(cfg).to_dict()) == config_from_dict(cfg)
    for path in (["width"], ["norm"], ["embedding", "scale"], ["layers", 0, "mixer", "vdim"], ["layers", 1, "mixer", "kv_rank"],
                 ["layers", 1, "mixer", "q_rank"], ["layers", 1, "mixer", "rot", "base"], ["layers", 1, "mixer", "scale"],
                 ["layers", 1, "mixer", "rot_dim"], ["layers", 2, "mixer", "kv_heads"], ["layers", 2, "mixer", "conv"],
                 ["layers", 2, "mixer", "rot", "dims"], ["layers", 1, "mlp", "router", "top"], ["layers", 1, "mlp", "expert"],
                 ["layers", 0, "mlp", "ff"], ["layers", 2, "type"]):
        d = copy.deepcopy(TINY_A)
        at = d
        for k in path[:-1]:
            at = at[k]
        del at[path[-1]]
        with pytest.raises(ConfigError, match=str(path[-1])):
            config_from_dict(d)
    for edit, word in ((lambda d: d["layers"][2]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
                       (lambda d: d["layers"][1]["mixer"]["rot"].__setitem__("dims", 18), "rot.dims"),
                       (lambda d: d["layers"][1]["mlp"]["router"].__setitem__("top", 7), "top"),
                       (lambda d: d["layers"][0].__setitem__("type", "something_else"), "something_else"),
                       (lambda d: d["layers"][0]["mlp"].__setitem__("kind", "sparse"), "sparse")):
        d = copy.deepcopy(TINY_A)
        edit(d)
        with pytest.raises(ConfigError, match=word):
            config_from_dict(d)


@pytest.mark.parametrize("name,cfg", ALL)
def test_the_model_declares_the_design_s_tensors(name, cfg):
    model = Model(config_from_dict(cfg).model_spec(), Runtime(None, torch.device("cpu"), torch.float32, 1))
    assert {n: tuple(s.shape) for n, s in model.weight_specs().items()} == tensor_shapes(cfg)


def test_what_each_layer_keeps_between_steps():
    """A matrix memory keeps its matrix (with the normaliser as one more column) and the running maximum; a latent layer pages
    of one row per token, given back as its window passes; an attention layer pages AND the convolution's last inputs."""
    model = Model(config_from_dict(TINY_A).model_spec(), Runtime(None, torch.device("cpu"), torch.float32, 1))
    specs = [b.cache_spec() for b in model.blocks]
    assert isinstance(specs[0], StatesSpec) and dict(specs[0].parts) == {"state": (2, 33, 16), "max": (2,)}
    assert specs[1].paged and specs[1].window == 11 and specs[1].width == 64 + 16
    assert isinstance(specs[2], PagedAndStateSpec) and specs[2].window == 0 and dict(specs[2].state.parts) == {"conv": (3, 4 * 32 + 2 * 32 + 2 * 16)}
    b = [blk.cache_spec() for blk in Model(config_from_dict(TINY_B).model_spec(), Runtime(None, torch.device("cpu"), torch.float32, 1)).blocks]
    assert b[0].window == 9 and b[1].window == 0 and dict(b[3].state.parts)["conv"] == (4, 2 * 20 + 2 * 20 + 2 * 6)


# ----------------------------------------------------------------------------- the plain implementation against itself
def test_plain_mechanisms_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    assert torch.allclose(unit_rms(x, 0.0), x / (12.5 ** 0.5))
    assert causal_mask(4, 2).tolist() == [[True, False, False, False], [True, True, False, False], [False, True, True, False], [False, False, True, True]]
    assert causal_mask(3, None).tolist() == [[True, False, False], [True, True, False], [True, True, True]]
    # the last column of the taps meets the present token; zeros before the start
    y = causal_conv(torch.tensor([[1.0], [10.0], [100.0]]), torch.tensor([[2.0, 3.0, 5.0]]))
    assert y.view(-1).tolist() == [5 * 1, 5 * 10 + 3 * 1, 5 * 100 + 3 * 10 + 2 * 1]
    # rotation: position 0 changes nothing; coordinates from `dims` on pass; neighbours pair; pair 0 has frequency 1
    v = torch.arange(12.0).view(1, 2, 6)
    assert torch.equal(rotate_interleaved(v, torch.tensor([0]), 100.0, 4), v)
    r = rotate_interleaved(v.expand(3, 2, 6), torch.tensor([0, 1, 7]), 100.0, 4)
    assert torch.equal(r[..., 4:], v.expand(3, 2, 6)[..., 4:])
    c, s = math.cos(7.0), math.sin(7.0)
    assert abs(float(r[2, 0, 0]) - (0 * c - 1 * s)) < 1e-5 and abs(float(r[2, 0, 1]) - (1 * c + 0 * s)) < 1e-5
    c, s = math.cos(7.0 * 100.0 ** -0.5), math.sin(7.0 * 100.0 ** -0.5)
    assert abs(float(r[2, 1, 2]) - (8 * c - 9 * s)) < 1e-5 and abs(float(r[2, 1, 3]) - (9 * c + 8 * s)) < 1e-5
    # a sink only joins the denominator; with a sink of zero that is one
    p = softmax_with_sink(torch.zeros(1, 2, 2), causal_mask(2, None), torch.tensor([0.0]))
    assert torch.allclose(p[0], torch.tensor([[0.5, 0.0], [1 / 3, 1 / 3]]))
    p = softmax_with_sink(torch.zeros(1, 1, 1), causal_mask(1, None), torch.tensor([math.log(3.0)]))
    assert abs(float(p) - 0.25) < 1e-6
    assert abs(float(gelu_tanh(torch.tensor(1.0))) - 0.841192) < 1e-5 and abs(float(log_sigmoid(torch.tensor(0.0))) + math.log(2.0)) < 1e-6


def test_the_matrix_memory_is_what_its_sums_say():
    """The recurrence with its running maximum against the explicit sums over earlier tokens in 64-bit: with A_t = sum of the
    log forget gates up to t, the unstabilised memory is C_t = sum_s exp(A_t - A_s + a_s) k_s v_s^T, M_t = max(A_t, max_s (A_t - A_s
    + a_s)) (M_0 = 0), and the stored state is C_t exp(-M_t)."""
    g = torch.Generator().manual_seed(0)
    T, H, d, P = 7, 2, 4, 3
    D = 2 * H * d + 2 * H * P + 2 * H
    h = torch.randn(T, D, generator=g, dtype=torch.float64)
    eye = torch.eye(D, dtype=torch.float64)
    at = [0, H * d, 2 * H * d, 2 * H * d + H * P, 2 * H * d + 2 * H * P, D - H, D]
    w = {"p." + n: eye[at[i]:at[i + 1]] for i, n in enumerate(("q", "k", "v", "g", "i", "f"))}
    w.update({"p.i.b": torch.tensor([0.3, -0.2], dtype=torch.float64), "p.f.b": torch.tensor([1.0, 2.0], dtype=torch.float64),
              "p.norm": torch.ones(H * P, dtype=torch.float64)})
    cap = 2.0
    got, (S, n, M) = matrix_memory(h, w, "p.", {"heads": H, "dim": d, "vdim": P, "gate_cap": cap}, 1e-6, None)
    q, k = h[:, :H * d].view(T, H, d) * d ** -0.5, h[:, H * d:2 * H * d].view(T, H, d)
    v, gate = h[:, 2 * H * d:2 * H * d + H * P].view(T, H, P), torch.sigmoid(h[:, at[3]:at[4]])
    a = cap * torch.tanh((h[:, at[4]:at[5]] + w["p.i.b"]) / cap)
    b = log_sigmoid(cap * torch.tanh((h[:, at[5]:] + w["p.f.b"]) / cap))
    A = torch.cumsum(b, 0)
    for t in range(T):
        for x in range(H):
            logs = torch.stack([A[t, x] - A[s, x] + a[s, x] for s in range(t + 1)])
            Mt = torch.maximum(A[t, x], logs.max())
            num = sum(torch.exp(logs[s] - Mt) * float(q[t, x] @ k[s, x]) * v[s, x] for s in range(t + 1))
            nq = sum(torch.exp(logs[s] - Mt) * float(q[t, x] @ k[s, x]) for s in range(t + 1))
            o = num / (max(abs(float(nq)), float(torch.exp(-Mt))) + 1e-6)
            o = o / torch.sqrt((o * o).mean() + 1e-6) * gate[t, x * P:(x + 1) * P]
            assert torch.allclose(got[t, x * P:(x + 1) * P], o, atol=1e-9)
            if t == T - 1:
                assert abs(float(M[x] - Mt)) < 1e-12
    # cut in two with the carry handed on: the same
    first, carry = matrix_memory(h[:3], w, "p.", {"heads": H, "dim": d, "vdim": P, "gate_cap": cap}, 1e-6, None)
    second, _ = matrix_memory(h[3:], w, "p.", {"heads": H, "dim": d, "vdim": P, "gate_cap": cap}, 1e-6, None, carry)
    assert torch.allclose(torch.cat([first, second]), got, atol=1e-12)


def test_latent_attention_is_attention_over_per_head_keys_and_values():
    """The latent mixer against ordinary attention written out per head and token, with keys [W_uk c | rotated part] and
    values W_uv c formed explicitly, a window of 3 and the sink in the denominator."""
    g = torch.Generator().manual_seed(1)
    T, D, H, d, r, P, R, Q = 6, 10, 2, 4, 2, 3, 5, 6
    m = {"heads": H, "dim": d, "rot_dim": r, "vdim": P, "kv_rank": R, "q_rank": Q, "scale": 0.4, "rot": {"base": 50.0, "dims": 2}, "mask": {"size": 3}}
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    w = {"p.dq": rnd(Q, D), "p.dq.norm": 1 + 0.1 * rnd(Q), "p.uq": rnd(H * (d + r), Q), "p.dkv": rnd(R + r, D), "p.dkv.norm": 1 + 0.1 * rnd(R),
         "p.uk": rnd(H * d, R), "p.uv": rnd(H * P, R), "p.sink": rnd(H)}
    h, pos = rnd(T, D), torch.arange(T)
    got = latent_attention(h, w, "p.", m, 1e-5, pos, None)
    cq = unit_rms(h @ w["p.dq"].t(), 1e-5) * w["p.dq.norm"]
    q = (cq @ w["p.uq"].t()).view(T, H, d + r)
    kv = h @ w["p.dkv"].t()
    c = unit_rms(kv[:, :R], 1e-5) * w["p.dkv.norm"]
    kr = rotate_interleaved(kv[:, None, R:], pos, 50.0, 2)[:, 0]
    qr = rotate_interleaved(q[..., d:], pos, 50.0, 2)
    for i in range(T):
        for a in range(H):
            js = [j for j in range(i + 1) if i - j < 3]
            key = lambda j: torch.cat([w["p.uk"][a * d:(a + 1) * d] @ c[j], kr[j]])
            s = torch.stack([torch.cat([q[i, a, :d], qr[i, a]]) @ key(j) * 0.4 for j in js])
            e = torch.exp(s)
            o = sum(e[n] * (w["p.uv"][a * P:(a + 1) * P] @ c[j]) for n, j in enumerate(js)) / (e.sum() + torch.exp(w["p.sink"][a]))
            assert torch.allclose(got[i, a * P:(a + 1) * P], o, atol=1e-9)


def test_routing_takes_the_largest_logits_and_weighs_by_their_softmax():
    g = torch.Generator().manual_seed(2)
    D, E = 6, 4
    w = {"p.router": torch.eye(E, D), "p.router.b": torch.tensor([0.0, 0.0, 0.0, 5.0]), "p.shared.sg": torch.zeros(1, D)}
    for e in range(E):                         # expert e answers with e + 1 in every coordinate when its gate sees one and up sees one
        w.update({f"p.e{e}.gate": torch.zeros(1, D), f"p.e{e}.up": torch.zeros(1, D), f"p.e{e}.down": torch.full((D, 1), float(e + 1))})
        w[f"p.e{e}.gate"][0, 5] = w[f"p.e{e}.up"][0, 5] = 1.0
    w.update({"p.shared.gate": torch.zeros(1, D), "p.shared.up": torch.zeros(1, D), "p.shared.down": torch.full((D, 1), 100.0)})
    w["p.shared.gate"][0, 5] = w["p.shared.up"][0, 5] = 1.0
    h = torch.tensor([[1.0, 3.0, 2.0, 0.0, 0.0, 1.0]])       # logits 1, 3, 2, 5 (the bias): experts 3 and 1 are chosen
    unit = float(torch.nn.functional.silu(torch.tensor(1.0)))
    got = routed_ff(h, w, "p.", {"router": {"experts": E, "top": 2}, "shared": {"ff": 1}}, None)
    wt = torch.softmax(torch.tensor([5.0, 3.0]), 0)
    want = unit * (float(wt[0]) * 4 + float(wt[1]) * 2) + unit * 100.0 * 0.5     # the shared expert's gate is sigmoid(0)
    assert torch.allclose(got, torch.full((1, D), want), atol=1e-5)


# ----------------------------------------------------------------------------- the engine's host logic
@pytest.mark.parametrize("name,cfg,page", [("A", TINY_A, 16), ("B", TINY_B, 8), ("M", ONLY_MEMORY, 32), ("L", ONLY_LATENT, 4), ("T", ONLY_ATTENTION, 16)])
def test_host_logic_replay_cpu(tmp_path, name, cfg, page):
    d = make_funevik_dir(str(tmp_path / name), cfg, seed=3)
    replay_all_schedules(d, cfg, "float32", [40, 23, 57, 1, 9, 30], page, HostOps(), "cpu", tail=12)


def test_greedy_generation_through_the_scheduler(tmp_path):
    d = make_funevik_dir(str(tmp_path / "m"), TINY_A, seed=5)
    llm = LLM(d, dtype="float32", page_size=16, max_cached_tokens=512, max_num_seqs=4, max_num_batched_tokens=64,
              prefill_chunk=40, max_model_len=256, device="cpu", ops=HostOps(), use_cuda_graphs=False)
    prompts = [random_ids(n, TINY_A["vocab"], i) for i, n in enumerate([1, 5, 50, 33, 7])]
    outs = llm.generate(prompts, SamplingParams(greedy=True), max_tokens=4, eos_token_id=None)
    plain = PlainFunevik(d)
    for p, o in zip(prompts, outs):
        assert o.token_ids == greedy_by_the_plain_model(plain, p, 4)
    llm.engine.cache.check_invariants()
    assert not llm.engine.cache.requests and llm.scheduler.all_done()


def test_a_weight_file_that_does_not_fit_is_refused(tmp_path):
    from llmengine_b200.config import EngineConfig
    from llmengine_b200.engine.engine import Engine
    from llmengine_b200.weights import WeightError

    def damage(t):
        del t["l0.mix.f.b"]
        t["l1.mix.uq"] = t["l1.mix.uq"][:, :-1].contiguous()
        t["l2.mix.q.b"] = torch.zeros(4, dtype=torch.bfloat16)          # this attention has no biases: no such tensor
        t["l3.norm2"] = torch.zeros(64, dtype=torch.bfloat16)           # a norm for a feed-forward the layer lacks: ignored
    d = make_funevik_dir(str(tmp_path / "m"), TINY_A, seed=1, change=damage)
    ec = EngineConfig(dtype="float32", max_cached_tokens=64, max_num_seqs=2, max_num_batched_tokens=64, max_model_len=64, device="cpu")
    with pytest.raises(WeightError, match="l0.mix.f.b") as e:
        Engine(d, engine_config=ec, ops=HostOps())
    assert "l1.mix.uq" in str(e.value) and "l2.mix.q.b" in str(e.value) and "l3.norm2" not in str(e.value)
