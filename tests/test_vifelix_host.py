"""The Vifelix design on the host: configuration, tensor names, the cache a layer asks for, and the engine's own logic (batch
metadata, pages, state slots, scheduling) with a CPU stand-in for the kernels, against the plain implementation."""
import copy

import pytest
import torch

from helpers import random_ids
from host_ops import HostOps
from llmengine_b200 import LLM, SamplingParams
from llmengine_b200.config import ConfigError, VifelixConfig, config_from_dict
from llmengine_b200.engine.model import Model
from llmengine_b200.parts import Runtime
from llmengine_b200.parts.base import PagedAndStateSpec, StatesSpec
from plain_vifelix import PlainVifelix, causal_conv, one_plus_norm, retention, rotate_partial, state_space, unit_rms, window_mask
from tiny_vifelix import ONLY_PARALLEL, ONLY_STATE, TINY_A, TINY_B, make_vifelix_dir, tensor_shapes
from vifelix_cases import greedy_by_the_plain_model, replay_all_schedules


def test_every_size_and_constant_comes_from_the_file():
    c = config_from_dict(TINY_A)
    assert isinstance(c, VifelixConfig) and (c.hidden_size, c.vocab_size, c.norm_eps, c.embedding_scale) == (64, 101, 1e-5, 8.0)
    p = c.mixers[0]
    assert (p.left.heads, p.left.kv_heads, p.left.dim, p.left.scale, p.left.window, p.left.rot_base, p.left.rot_dims) == \
        (4, 2, 32, 0.2, 11, 500.0, 16)
    assert (p.right.heads, p.right.dim, p.right.vdim, p.right.decay, p.right.rot_base, p.right.rot_dims) == (2, 16, 32, (0.9, 0.97), 300.0, 8)
    assert (p.left_scale, p.right_scale) == (0.7, 1.4)
    s = c.mixers[1]
    assert (s.heads, s.vdim, s.state, s.groups, s.taps, s.norm_groups) == (4, 16, 8, 2, 4, 2)
    assert c.mlps[0].ff == 72 and c.mlps[1] is None and c.mlps[3].ff == 40
    assert config_from_dict(c.to_dict()) == c
    for path in (["width"], ["norm"], ["embedding", "scale"], ["layers", 0, "mixer", "left", "kv_heads"], ["layers", 0, "mixer", "left", "rot", "base"],
                 ["layers", 0, "mixer", "left", "mask", "size"], ["layers", 0, "mixer", "left", "scale"], ["layers", 0, "mixer", "right", "decay"],
                 ["layers", 0, "mixer", "right_scale"], ["layers", 0, "mixer", "right", "rot", "dims"], ["layers", 1, "mixer", "state"],
                 ["layers", 1, "mixer", "conv"], ["layers", 1, "mixer", "norm_groups"], ["layers", 1, "mixer", "groups"],
                 ["layers", 0, "mlp", "ff"], ["layers", 2, "type"]):
        d = copy.deepcopy(TINY_A)
        at = d
        for k in path[:-1]:
            at = at[k]
        del at[path[-1]]
        with pytest.raises(ConfigError, match=str(path[-1])):
            config_from_dict(d)
    for edit, word in ((lambda d: d["layers"][0]["mixer"]["right"].__setitem__("decay", [0.5]), "decay"),
                       (lambda d: d["layers"][0]["mixer"]["left"].__setitem__("vdim", 16), "values are the keys"),
                       (lambda d: d["layers"][1]["mixer"].__setitem__("groups", 3), "groups"),
                       (lambda d: d["layers"][1]["mixer"].__setitem__("norm_groups", 7), "norm_groups"),
                       (lambda d: d["layers"][0].__setitem__("type", "something_else"), "something_else"),
                       (lambda d: d["layers"][0]["mlp"].__setitem__("kind", "sparse"), "sparse")):
        d = copy.deepcopy(TINY_A)
        edit(d)
        with pytest.raises(ConfigError, match=word):
            config_from_dict(d)


@pytest.mark.parametrize("cfg", [TINY_A, TINY_B, ONLY_STATE, ONLY_PARALLEL])
def test_the_model_declares_the_design_s_tensors(cfg):
    model = Model(config_from_dict(cfg).model_spec(), Runtime(None, torch.device("cpu"), torch.float32, 1))
    declared = {n: tuple(s.shape) for n, s in model.weight_specs().items()}
    assert declared == tensor_shapes(cfg)


def test_what_each_layer_keeps_between_steps():
    """A parallel layer keeps pages (keys and values of its window) AND a state; a state-space layer two states."""
    model = Model(config_from_dict(TINY_A).model_spec(), Runtime(None, torch.device("cpu"), torch.float32, 1))
    specs = [b.cache_spec() for b in model.blocks]
    assert isinstance(specs[0], PagedAndStateSpec) and specs[0].paged and specs[0].window == 11
    assert dict(specs[0].state.parts) == {"right.state": (2, 32, 16)}
    assert isinstance(specs[1], StatesSpec) and dict(specs[1].parts) == {"conv": (3, 4 * 16 + 2 * 2 * 8), "state": (4, 16, 8)}
    assert specs[2].window == 40 and dict(specs[2].state.parts) == {"right.state": (3, 16, 32)}
    one_tap = Model(config_from_dict(TINY_B).model_spec(), Runtime(None, torch.device("cpu"), torch.float32, 1)).blocks[1].cache_spec()
    assert dict(one_tap.parts)["conv"][1] == 6 * 5 + 2 * 2 * 12


# ----------------------------------------------------------------------------- the plain implementation against itself
def test_plain_mechanisms_by_hand():
    """Each function of the plain implementation on inputs whose result can be written down."""
    x = torch.tensor([[3.0, 4.0]])
    assert torch.allclose(unit_rms(x, 0.0), x / (12.5 ** 0.5))
    assert torch.allclose(one_plus_norm(x, torch.tensor([0.0, 1.0]), 0.0), x / (12.5 ** 0.5) * torch.tensor([1.0, 2.0]))
    m = window_mask(5, 2)
    assert m.tolist() == [[True, False, False, False, False], [True, True, False, False, False], [False, True, True, False, False],
                          [False, False, True, True, False], [False, False, False, True, True]]
    # the last column of the taps meets the present token; zeros before the start
    y = causal_conv(torch.tensor([[1.0], [10.0], [100.0]]), torch.tensor([[2.0, 3.0, 5.0]]), torch.tensor([0.5]))
    assert y.view(-1).tolist() == [0.5 + 5 * 1, 0.5 + 5 * 10 + 3 * 1, 0.5 + 5 * 100 + 3 * 10 + 2 * 1]
    # rotation: position 0 changes nothing; coordinates from `dims` on pass; a quarter turn swaps a pair
    v = torch.arange(12.0).view(1, 2, 6)
    assert torch.equal(rotate_partial(v, torch.tensor([0]), 100.0, 4), v)
    r = rotate_partial(v.expand(3, 2, 6), torch.tensor([0, 1, 7]), 100.0, 4)
    assert torch.equal(r[..., 4:], v.expand(3, 2, 6)[..., 4:]) and not torch.allclose(r[1, :, :4], v[0, :, :4])
    import math
    c, s = math.cos(7.0), math.sin(7.0)       # pair (0, 2) has frequency 1
    assert abs(float(r[2, 0, 0]) - (0 * c - 2 * s)) < 1e-5 and abs(float(r[2, 0, 2]) - (2 * c + 0 * s)) < 1e-5


def test_plain_recurrences_are_what_their_sums_say():
    """Retention and the state-space recurrence written as explicit sums over earlier tokens, against the token-by-token
    form of the plain implementation (through weights that make the projections identities)."""
    g = torch.Generator().manual_seed(0)
    T, H, d, P = 6, 2, 4, 3
    D = 2 * H * d + 2 * H * P
    h = torch.randn(T, D, generator=g)
    eye = torch.eye(D)
    w = {"p.q": eye[:H * d], "p.k": eye[H * d:2 * H * d], "p.v": eye[2 * H * d:2 * H * d + H * P], "p.g": eye[2 * H * d + H * P:]}
    m = {"heads": H, "dim": d, "vdim": P, "decay": [0.5, 0.9], "rot": {"base": 10.0, "dims": 2}}
    got = retention(h, w, "p.", m, 1e-6, torch.arange(T), None)
    q = rotate_partial(h[:, :H * d].view(T, H, d), torch.arange(T), 10.0, 2)
    k = rotate_partial(h[:, H * d:2 * H * d].view(T, H, d), torch.arange(T), 10.0, 2) * d ** -0.5
    v = h[:, 2 * H * d:2 * H * d + H * P].view(T, H, P)
    gate = h[:, 2 * H * d + H * P:]
    for t in range(T):
        for a in range(H):
            o = sum(m["decay"][a] ** (t - s) * float(q[t, a] @ k[s, a]) * v[s, a] for s in range(t + 1))
            o = o / torch.sqrt((o * o).mean() + 1e-6) * (gate[t, a * P:(a + 1) * P] * torch.sigmoid(gate[t, a * P:(a + 1) * P]))
            assert torch.allclose(got[t, a * P:(a + 1) * P], o, atol=1e-5)


# ----------------------------------------------------------------------------- the engine's host logic
@pytest.mark.parametrize("name,cfg,page", [("A", TINY_A, 16), ("B", TINY_B, 8), ("S", ONLY_STATE, 32), ("P", ONLY_PARALLEL, 4)])
def test_host_logic_replay_cpu(tmp_path, name, cfg, page):
    d = make_vifelix_dir(str(tmp_path / name), cfg, seed=3)
    replay_all_schedules(d, cfg, "float32", [70, 33, 100, 1, 19, 45], page, HostOps(), "cpu", tail=20)


def test_greedy_generation_through_the_scheduler(tmp_path):
    d = make_vifelix_dir(str(tmp_path / "m"), TINY_A, seed=5)
    llm = LLM(d, dtype="float32", page_size=16, max_cached_tokens=512, max_num_seqs=4, max_num_batched_tokens=64,
              prefill_chunk=40, max_model_len=256, device="cpu", ops=HostOps(), use_cuda_graphs=False)
    prompts = [random_ids(n, TINY_A["vocab"], i) for i, n in enumerate([1, 5, 64, 90, 33, 7])]
    outs = llm.generate(prompts, SamplingParams(greedy=True), max_tokens=5, eos_token_id=None)
    plain = PlainVifelix(d)
    for p, o in zip(prompts, outs):
        assert o.token_ids == greedy_by_the_plain_model(plain, p, 5)
    llm.engine.cache.check_invariants()
    assert not llm.engine.cache.requests and llm.scheduler.all_done()


def test_a_weight_file_that_does_not_fit_is_refused(tmp_path):
    from llmengine_b200.config import EngineConfig
    from llmengine_b200.engine.engine import Engine
    from llmengine_b200.weights import WeightError

    def damage(t):
        del t["l1.mix.A_log"]
        t["l0.mix.right.g"] = t["l0.mix.right.g"][:, :-1].contiguous()
        t["l0.mix.left.v"] = torch.zeros(4, 4, dtype=torch.bfloat16)     # the values are the keys: there is no such tensor
        t["l1.norm2"] = torch.zeros(64, dtype=torch.bfloat16)            # a norm for a feed-forward the layer lacks: ignored
    d = make_vifelix_dir(str(tmp_path / "m"), TINY_A, seed=1, change=damage)
    ec = EngineConfig(dtype="float32", max_cached_tokens=64, max_num_seqs=2, max_num_batched_tokens=64, max_model_len=64,
                      device="cpu")
    with pytest.raises(WeightError, match="l1.mix.A_log") as e:
        Engine(d, engine_config=ec, ops=HostOps())
    assert "l0.mix.right.g" in str(e.value) and "l0.mix.left.v" in str(e.value) and "l1.norm2" not in str(e.value)
