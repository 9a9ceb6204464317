"""Tiny Vifelix configurations and weights for the tests.

The configurations differ from one another in every size, in the order of the layers and in what a layer has: a model
that starts with a parallel layer and one that starts with a state-space layer, a model without any attention (no
pages at all), a state-space layer WITH a feed-forward and a parallel layer WITHOUT one, one group and one norm group as
well as several, one tap and five, grouped query heads and one head per key/value head, fewer rotated coordinates than
a head is wide, windows of one token, shorter and longer than the sequences, retention heads whose key and value sizes
differ, decays of one (nothing forgotten) and far below, scales that differ between the branches, sizes that are no
multiples of 8 or 16.

Weights are drawn so that activations stay of order one through the layers (matrices with variance 1 / inputs).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict

import torch

from llmengine_b200.weights import write_safetensors


def ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def left(heads, kv_heads, dim, scale, size, base=10000.0, dims=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "mask": {"size": size},
            "rot": {"base": base, "dims": dim if dims is None else dims}}


def right(heads, dim, vdim, decay, base=10000.0, dims=None):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay), "rot": {"base": base, "dims": dim if dims is None else dims}}


def parallel(l, r, left_scale, right_scale):
    return {"left": l, "right": r, "left_scale": left_scale, "right_scale": right_scale}


def layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def model(vocab, width, eps, scale, layers):
    return {"architecture": "Vifelix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
            "layers": layers}


# sizes the tensor-core kernels take; starts with a parallel layer; a window shorter than the prompts
TINY_A = model(101, 64, 1e-5, 8.0, [
    layer("parallel", parallel(left(4, 2, 32, 0.2, 11, base=500.0, dims=16), right(2, 16, 32, (0.9, 0.97), base=300.0, dims=8), 0.7, 1.4), 72),
    layer("mamba2", ssm(4, 16, 8, 2, 4, 2)),
    layer("parallel", parallel(left(2, 2, 16, 0.3, 40, base=90.0), right(3, 32, 16, (1.0, 0.5, 0.99)), 1.0, 0.5), None),
    layer("mamba2", ssm(2, 24, 16, 1, 2, 1), 40),
])

# sizes that are no multiples of 8: the plain kernels everywhere; a window of one token; one tap; five taps
TINY_B = model(67, 52, 1e-6, 3.0, [
    layer("mamba2", ssm(3, 10, 6, 3, 5, 3)),
    layer("mamba2", ssm(6, 5, 12, 2, 1, 5), 36),
    layer("parallel", parallel(left(3, 1, 12, 0.4, 1, base=40.0, dims=6), right(1, 10, 14, (0.8,), base=1000.0, dims=4), 1.3, 0.9), 44),
    layer("parallel", parallel(left(2, 1, 20, 0.25, 300, base=2000.0, dims=20), right(2, 6, 6, (0.95, 0.999), dims=6), 0.6, 1.1), None),
])

# no attention at all: the engine then has states and no pages
ONLY_STATE = model(83, 48, 1e-5, 2.0, [
    layer("mamba2", ssm(4, 8, 16, 4, 3, 4), 64),
    layer("mamba2", ssm(2, 16, 8, 1, 4, 2)),
])

# one parallel layer by itself; window 7
ONLY_PARALLEL = model(59, 32, 1e-5, 4.0, [
    layer("parallel", parallel(left(4, 2, 16, 0.35, 7, base=100.0, dims=8), right(2, 16, 16, (0.96, 0.9), base=50.0), 1.2, 0.8), 48),
])


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    """Every tensor of a model of this configuration, by the design's naming."""
    D, V = cfg["width"], cfg["vocab"]
    s: Dict[str, tuple] = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        s[p + "norm1"] = s[p + "norm1b"] = (D,)
        if L["type"] == "mamba2":
            inner, bc = m["heads"] * m["vdim"], m["groups"] * m["state"]
            s.update({p + "mix.in": (2 * inner + 2 * bc + m["heads"], D), p + "mix.conv": (inner + 2 * bc, m["conv"]),
                      p + "mix.conv.b": (inner + 2 * bc,), p + "mix.dt_bias": (m["heads"],), p + "mix.A_log": (m["heads"],),
                      p + "mix.D": (m["heads"],), p + "mix.norm": (inner,), p + "mix.o": (D, inner)})
        else:
            l, r = m["left"], m["right"]
            q, kv = l["heads"] * l["dim"], l["kv_heads"] * l["dim"]
            s.update({p + "mix.left.q": (q, D), p + "mix.left.q.b": (q,), p + "mix.left.k": (kv, D), p + "mix.left.k.b": (kv,),
                      p + "mix.left.q.norm": (l["dim"],), p + "mix.left.k.norm": (l["dim"],), p + "mix.left.g": (q, D),
                      p + "mix.left.o": (D, q)})
            rq, rv = r["heads"] * r["dim"], r["heads"] * r["vdim"]
            s.update({p + "mix.right.q": (rq, D), p + "mix.right.k": (rq, D), p + "mix.right.v": (rv, D), p + "mix.right.g": (rv, D),
                      p + "mix.right.o": (D, rv)})
        if L["mlp"] is not None:
            ff = L["mlp"]["ff"]
            s[p + "norm2"] = s[p + "norm2b"] = (D,)
            s.update({p + "mlp.gate": (ff, D), p + "mlp.gate.b": (ff,), p + "mlp.up": (ff, D), p + "mlp.up.b": (ff,),
                      p + "mlp.down": (D, ff), p + "mlp.down.b": (D,)})
    return s


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if name.endswith(".q.norm") or name.endswith(".k.norm"):
            t = 1.0 + 0.3 * torch.randn(shape, generator=g)              # plain gains
        elif name.endswith("mix.norm"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif leaf in ("norm1", "norm2", "norm1b", "norm2b") or name == "final.norm":
            t = 0.2 * torch.randn(shape, generator=g)                    # stored around zero
        elif name.endswith(".b"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif name.endswith("mix.conv"):
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
        elif leaf == "dt_bias":
            t = torch.randn(shape, generator=g) - 1.0                    # steps around softplus(-1): both small and large ones
        elif leaf == "A_log":
            t = torch.randn(shape, generator=g) * 0.7
        elif leaf == "D":
            t = 1.0 + 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g) / cfg["embedding"]["scale"]
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16)
    return out


def make_vifelix_dir(path: str, cfg: dict, seed: int, change=None) -> str:
    """A model folder with random weights; `change(weights)` may edit them (tests that make one key stand out)."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    w = make_weights(cfg, seed)
    if change is not None:
        change(w)
    write_safetensors(os.path.join(path, "model.safetensors"), w)
    return path
