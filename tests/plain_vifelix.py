"""The plain implementation of the Vifelix design: whole sequences, no cache, no chunks, one function per
mechanism, elementary tensor arithmetic on the CPU; recurrences run token by token.

It shares no code with the engine: it reads config.json and model.safetensors itself.  `round_to` rounds to
bfloat16 where the engine's bfloat16 path stores bfloat16 (weights, the inputs of the matrix products, cached keys);
the arithmetic itself is always 32-bit.

Notation: D width, T tokens, H heads, G key/value heads (or groups of a state-space mixer), d query/key size per head,
P value size per head, N state size, K taps of the short convolution.
"""
from __future__ import annotations

import json
import math
import os
from typing import List, Optional, Sequence

import torch

from plain_bepuzen import read_safetensors

F32 = torch.float32


def _r(x: torch.Tensor, round_to: Optional[torch.dtype]) -> torch.Tensor:
    return x if round_to is None else x.to(round_to).to(F32)


# --------------------------------------------------------------------- mechanisms
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def one_plus_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layer norms of the design store their weight around zero: unit_rms(x) * (1 + w)."""
    return unit_rms(x, eps) * (1.0 + w.to(F32))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.clamp(z, min=0) + torch.log1p(torch.exp(-z.abs()))


def rotate_partial(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [T, heads, d]: coordinate i < dims/2 of every head pairs with i + dims/2 and the pair turns by the angle
    position * base^(-2i/dims); coordinates from `dims` on pass unchanged."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64).to(F32)
    ang = positions.to(F32)[:, None] * f[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def window_mask(T: int, size: int) -> torch.Tensor:
    """[T, T] bool: query i sees key j if 0 <= i - j < size."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i - j < size)


def window_attention(h, w, pre, m, eps, positions, round_to):
    """The softmax mixer: grouped heads, the values are the keys as projected (before norm and rotation), biases on the
    query and key projections, per-head RMS norm of q and k with one weight vector each, partial rotation, a sliding
    window, and a sigmoid gate on the concatenated heads.  Returns the gated heads [T, H d] (before the output product)."""
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    q = _r(h @ w[pre + "q"].t() + w[pre + "q.b"], round_to).view(T, H, d)
    k = _r(h @ w[pre + "k"].t() + w[pre + "k.b"], round_to).view(T, G, d)
    v = k                                                              # no value projection
    q = unit_rms(q, eps) * w[pre + "q.norm"]
    kn = unit_rms(k, eps) * w[pre + "k.norm"]
    q = _r(rotate_partial(q, positions, m["rot"]["base"], m["rot"]["dims"]), round_to)
    kn = _r(rotate_partial(kn, positions, m["rot"]["base"], m["rot"]["dims"]), round_to)
    rep = H // G
    kh, vh = kn.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)  # query head a reads key/value head a // rep
    s = torch.einsum("iad,jad->aij", q, kh) * m["scale"]
    s = s.masked_fill(~window_mask(T, m["mask"]["size"])[None], float("-inf"))
    p = torch.softmax(s, -1)
    o = torch.einsum("aij,jad->iad", p, vh).reshape(T, H * d)
    gate = torch.sigmoid(_r(h @ w[pre + "g"].t(), round_to))
    return o * gate


def retention(h, w, pre, m, eps, positions, round_to, state=None):
    """Linear attention with a fixed decay per head: S_t = decay_a S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, no softmax and
    no denominator; k carries d^(-1/2) after the rotation.  Each head's o is divided by its root mean square, the heads
    are multiplied by silu(W_g h).  Returns the gated heads [T, H P]."""
    H, d, P = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = _r(h @ w[pre + "q"].t(), round_to).view(T, H, d)
    k = _r(h @ w[pre + "k"].t(), round_to).view(T, H, d)
    v = _r(h @ w[pre + "v"].t(), round_to).view(T, H, P)
    q = rotate_partial(q, positions, m["rot"]["base"], m["rot"]["dims"])
    k = rotate_partial(k, positions, m["rot"]["base"], m["rot"]["dims"]) * (d ** -0.5)
    decay = torch.tensor(m["decay"], dtype=F32)
    S = torch.zeros(H, d, P) if state is None else state
    o = torch.empty(T, H, P)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("adp,ad->ap", S, q[t])
    o = unit_rms(o, eps).reshape(T, H * P)
    return o * silu(_r(h @ w[pre + "g"].t(), round_to))


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, K]: y_t = bias + sum_j taps[:, K-1-j] x_(t-j), zeros before the start (the last column is the
    present token's)."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C), x], 0)
    y = bias.to(F32).expand(T, C).clone()
    for j in range(K):
        y = y + padded[K - 1 - j: K - 1 - j + T] * taps[:, K - 1 - j]
    return y


def state_space(h, w, pre, m, eps, round_to):
    """The state-space mixer.  W_in h = [z | x | B | C | dt]; x, B, C pass the short convolution and silu;
    dt = softplus(dt + dt_bias); per head a (group a // (H / G)): S_t = exp(-exp(A_log_a) dt) S_(t-1) + dt B_t x_t^T,
    y_t = S_t^T C_t + D_a x_t; y silu(z) is RMS-normed in `norm_groups` equal parts, times a weight.  Returns [T, H P]."""
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    T = h.shape[0]
    proj = _r(h @ w[pre + "in"].t(), round_to)
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[pre + "conv"], w[pre + "conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N).repeat_interleave(H // G, 1)
    C = xbc[:, inner + G * N:].view(T, G, N).repeat_interleave(H // G, 1)
    dt = softplus(dt + w[pre + "dt_bias"])                            # [T, H]
    decay = torch.exp(-torch.exp(w[pre + "A_log"].to(F32)) * dt)
    S = torch.zeros(H, N, P)
    y = torch.empty(T, H, P)
    for t in range(T):
        S = decay[t][:, None, None] * S + dt[t][:, None, None] * B[t][:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("anp,an->ap", S, C[t]) + w[pre + "D"][:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[pre + "norm"]
    return y


def dense_ff(h, w, pre, round_to):
    g = _r(h @ w[pre + "gate"].t() + w[pre + "gate.b"], round_to)
    u = _r(h @ w[pre + "up"].t() + w[pre + "up.b"], round_to)
    return _r(silu(g) * u, round_to) @ w[pre + "down"].t() + w[pre + "down.b"]


# --------------------------------------------------------------------- the model
class PlainVifelix:
    def __init__(self, model_dir: str, round_to: Optional[torch.dtype] = None):
        with open(os.path.join(model_dir, "config.json")) as f:
            self.cfg = json.load(f)
        self.w = {n: t.to(F32) for n, t in read_safetensors(os.path.join(model_dir, "model.safetensors")).items()}
        self.round_to = round_to

    def mixer(self, i: int, L: dict, h: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        w, rt, eps = self.w, self.round_to, self.cfg["norm"]["eps"]
        m, pre = L["mixer"], f"l{i}.mix."
        if L["type"] == "mamba2":
            return _r(state_space(h, w, pre, m, eps, rt), rt) @ w[pre + "o"].t()
        if L["type"] == "parallel":
            left = _r(window_attention(h, w, pre + "left.", m["left"], eps, pos, rt), rt) @ w[pre + "left.o"].t()
            right = _r(retention(h, w, pre + "right.", m["right"], eps, pos, rt), rt) @ w[pre + "right.o"].t()
            return m["left_scale"] * left + m["right_scale"] * right
        raise ValueError(L["type"])

    def forward(self, ids: Sequence[int], layers_out: Optional[list] = None) -> torch.Tensor:
        cfg, w, rt = self.cfg, self.w, self.round_to
        eps = cfg["norm"]["eps"]
        T = len(ids)
        pos = torch.arange(T)
        x = w["embed"][torch.tensor(list(ids), dtype=torch.long)] * float(cfg["embedding"]["scale"])
        for i, L in enumerate(cfg["layers"]):
            p = f"l{i}."
            h = _r(one_plus_norm(x, w[p + "norm1"], eps), rt)
            x = x + one_plus_norm(self.mixer(i, L, h, pos), w[p + "norm1b"], eps)
            if L.get("mlp") is not None:
                if L["mlp"]["kind"] != "dense":
                    raise ValueError(L["mlp"]["kind"])
                h = _r(one_plus_norm(x, w[p + "norm2"], eps), rt)
                x = x + one_plus_norm(dense_ff(h, w, p + "mlp.", rt), w[p + "norm2b"], eps)
            if layers_out is not None:
                layers_out.append(x.clone())
        return _r(one_plus_norm(x, w["final.norm"], eps), rt) @ w["head"].t()

    def logits(self, ids: Sequence[int]) -> torch.Tensor:
        return self.forward(ids)
