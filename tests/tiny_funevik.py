"""Tiny Funevik configurations and weights for the tests.

The configurations differ from one another in every size, in the order of the layers and in what a layer has: models that
start with each of the three mixers, a model without any attention (no pages at all), layers without a feed-forward, dense
and routed feed-forwards with and without a shared expert, one expert of one and all experts chosen, grouped query heads and
one query head per key/value head, query/key and value sizes that differ, fewer rotated coordinates than a head (or the
rotated part) is wide, one tap and five, windows of one token, shorter and longer than the sequences and none at all, with and
without a cap on the scores and on the gates, sizes that are no multiples of 8 or 16.

Weights are drawn so that activations stay of order one through the layers (matrices with variance 1 / inputs).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, Optional

import torch

from llmengine_b200.weights import write_safetensors


def memory(heads, dim, vdim, cap=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim}
    if cap is not None:
        m["gate_cap"] = cap
    return m


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, size=None, base=10000.0, dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    if size is not None:
        m["mask"] = {"size": size}
    return m


def attention(heads, kv_heads, dim, vdim, scale, conv, base=10000.0, dims=None, softcap=None, size=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "conv": conv,
         "rot": {"base": base, "dims": dim if dims is None else dims}}
    if softcap is not None:
        m["softcap"] = softcap
    if size is not None:
        m["mask"] = {"size": size}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def model(vocab, width, eps, scale, layers):
    return {"architecture": "Funevik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
            "layers": layers}


# sizes the tensor-core kernels take; starts with a matrix memory; windows shorter than the prompts
TINY_A = model(101, 64, 1e-5, 8.0, [
    layer("mlstm", memory(2, 16, 32, cap=15.0), dense(96)),
    layer("latent_attention", latent(4, 16, 16, 32, 64, 48, 0.18, size=11, base=500.0), moe(6, 2, 24, shared=40)),
    layer("attention", attention(4, 2, 32, 16, 0.2, 4, base=300.0, dims=16, softcap=30.0), moe(5, 1, 32)),
    layer("mlstm", memory(4, 32, 16, cap=8.0)),
])

# sizes that are no multiples of 8: the plain kernels everywhere; starts with an attention of one tap and a window; a latent
# attention without a window whose rotated part is wider than what is rotated; a memory without a cap; all experts chosen
TINY_B = model(67, 52, 1e-6, 3.0, [
    layer("attention", attention(3, 1, 12, 10, 0.3, 1, base=40.0, dims=6, size=9), dense(44)),
    layer("latent_attention", latent(3, 10, 6, 14, 20, 12, 0.25, base=1000.0, dims=4)),
    layer("mlstm", memory(3, 6, 5), moe(3, 3, 20, shared=12)),
    layer("attention", attention(2, 2, 20, 6, 0.2, 5, base=2000.0, dims=20, softcap=5.0), moe(4, 2, 12)),
])

# no attention at all: the engine then has states and no pages
ONLY_MEMORY = model(83, 48, 1e-5, 2.0, [
    layer("mlstm", memory(4, 8, 16, cap=10.0), dense(64)),
    layer("mlstm", memory(2, 40, 9, cap=3.0)),
])

# one latent layer by itself; a window of 7; starts the model
ONLY_LATENT = model(59, 32, 1e-5, 4.0, [
    layer("latent_attention", latent(2, 8, 8, 12, 24, 16, 0.3, size=7, base=100.0, dims=4), dense(48)),
])

# one attention layer by itself
ONLY_ATTENTION = model(61, 40, 1e-5, 5.0, [
    layer("attention", attention(4, 1, 16, 8, 0.35, 3, base=100.0, dims=8, softcap=12.0), moe(4, 2, 16, shared=24)),
])


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    """Every tensor of a model of this configuration, by the design's naming."""
    D, V = cfg["width"], cfg["vocab"]
    s: Dict[str, tuple] = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        s[p + "norm1"] = s[p + "ls1"] = (D,)
        H = m["heads"]
        if L["type"] == "mlstm":
            s.update({p + "mix.q": (H * m["dim"], D), p + "mix.k": (H * m["dim"], D), p + "mix.v": (H * m["vdim"], D),
                      p + "mix.g": (H * m["vdim"], D), p + "mix.o": (D, H * m["vdim"]), p + "mix.norm": (H * m["vdim"],),
                      p + "mix.i": (H, D), p + "mix.i.b": (H,), p + "mix.f": (H, D), p + "mix.f.b": (H,)})
        elif L["type"] == "latent_attention":
            s.update({p + "mix.dq": (m["q_rank"], D), p + "mix.dq.norm": (m["q_rank"],), p + "mix.uq": (H * (m["dim"] + m["rot_dim"]), m["q_rank"]),
                      p + "mix.dkv": (m["kv_rank"] + m["rot_dim"], D), p + "mix.dkv.norm": (m["kv_rank"],),
                      p + "mix.uk": (H * m["dim"], m["kv_rank"]), p + "mix.uv": (H * m["vdim"], m["kv_rank"]), p + "mix.sink": (H,),
                      p + "mix.o": (D, H * m["vdim"])})
        else:
            G = m["kv_heads"]
            s.update({p + "mix.q": (H * m["dim"], D), p + "mix.k": (G * m["dim"], D), p + "mix.v": (G * m["vdim"], D),
                      p + "mix.q.conv": (H * m["dim"], m["conv"]), p + "mix.k.conv": (G * m["dim"], m["conv"]),
                      p + "mix.v.conv": (G * m["vdim"], m["conv"]), p + "mix.g": (H, D), p + "mix.o": (D, H * m["vdim"])})
        mlp = L["mlp"]
        if mlp is None:
            continue
        s[p + "norm2"] = s[p + "ls2"] = (D,)
        if mlp["kind"] == "dense":
            s.update({p + "mlp.gate": (mlp["ff"], D), p + "mlp.up": (mlp["ff"], D), p + "mlp.down": (D, mlp["ff"])})
        else:
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            s.update({p + "mlp.router": (E, D), p + "mlp.router.b": (E,)})
            for e in range(E):
                s.update({p + f"mlp.e{e}.gate": (ff, D), p + f"mlp.e{e}.up": (ff, D), p + f"mlp.e{e}.down": (D, ff)})
            if mlp.get("shared") is not None:
                sf = mlp["shared"]["ff"]
                s.update({p + "mlp.shared.gate": (sf, D), p + "mlp.shared.up": (sf, D), p + "mlp.shared.down": (D, sf),
                          p + "mlp.shared.sg": (1, D)})
    return s


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2", "norm", "ls1", "ls2") or name == "final.norm":
            t = 1.0 + 0.3 * torch.randn(shape, generator=g)              # gains and scale vectors, used as stored
        elif leaf == "conv":
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
        elif name.endswith("mix.f.b"):
            t = 2.0 + torch.randn(shape, generator=g)                     # forget gates that mostly keep
        elif leaf == "b" or leaf == "sink":
            t = torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g) / cfg["embedding"]["scale"]
        elif leaf == "router":
            t = 2.0 * torch.randn(shape, generator=g) / math.sqrt(shape[-1])      # routers that decide
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16)
    return out


def make_funevik_dir(path: str, cfg: dict, seed: int, change=None) -> str:
    """A model folder with random weights; `change(weights)` may edit them (tests that make one key stand out)."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    w = make_weights(cfg, seed)
    if change is not None:
        change(w)
    write_safetensors(os.path.join(path, "model.safetensors"), w)
    return path
