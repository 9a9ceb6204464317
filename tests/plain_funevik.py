"""The plain implementation of the Funevik design: whole sequences, no cache, no chunks, one function per mechanism,
elementary tensor arithmetic on the CPU; the recurrence runs token by token.

It shares no code with the engine: it reads config.json and model.safetensors itself.  `round_to` rounds to bfloat16
where the engine's bfloat16 path stores bfloat16 (weights, the inputs of the matrix products, projections, cached
rows); the arithmetic itself is 32-bit (or 64-bit with `wide`).

Notation: D width, T tokens, H heads, G key/value heads, d query/key size per head, P value size per head, R the
latent's size, r the rotated size of the latent mixer, K taps of the short convolution, E experts.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, Optional, Sequence

import torch

from plain_bepuzen import read_safetensors


def _r(x: torch.Tensor, round_to: Optional[torch.dtype]) -> torch.Tensor:
    return x if round_to is None else x.to(round_to).to(x.dtype)


# --------------------------------------------------------------------- small pieces
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z * z * z)))


def log_sigmoid(z: torch.Tensor) -> torch.Tensor:
    return torch.clamp(z, max=0) - torch.log1p(torch.exp(-z.abs()))


def rotate_interleaved(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [T, heads, d]: among the first `dims` coordinates of every head, coordinate 2i pairs with 2i + 1 and the pair
    (u, v) turns by the angle a = position * base^(-2i/dims): (u cos a - v sin a, v cos a + u sin a).  The rest pass."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64).to(torch.float32).to(x.dtype)
    ang = positions.to(x.dtype)[:, None] * f[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    turned = torch.stack([u * c - v * s, v * c + u * s], -1).flatten(-2)
    return torch.cat([turned, x[..., dims:]], -1)


def causal_mask(T: int, size: Optional[int]) -> torch.Tensor:
    """[T, T] bool: query i sees key j if j <= i and, with a window, i - j < size."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    return m if not size else m & (i - j < size)


def softmax_with_sink(s: torch.Tensor, mask: torch.Tensor, sink: torch.Tensor) -> torch.Tensor:
    """s [H, T, T] scores, sink [H]: p_ij = exp(s_ij) / (exp(sink_h) + sum over visible j' of exp(s_ij'))."""
    s = s.masked_fill(~mask[None], float("-inf"))
    top = torch.maximum(s.max(-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(s - top)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - top))


def causal_conv(u: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """u [T, C], taps [C, K]: y_t = sum_j taps[:, j] u_(t - K + 1 + j), zeros before the start (the last column meets
    the present token)."""
    T, C = u.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=u.dtype), u], 0)
    y = torch.zeros(T, C, dtype=u.dtype)
    for j in range(K):
        y = y + padded[j:j + T] * taps[:, j]
    return y


# --------------------------------------------------------------------- mixers
def matrix_memory(h, w, pre, m, eps, round_to, carry=None, calls=None):
    """The matrix memory with exponential gates.  Per head: q = W_q h / sqrt(d), k = W_k h, v = W_v h; log gates
    a = cap tanh((W_i h + b_i) / cap) (input) and b = logsigmoid(cap tanh((W_f h + b_f) / cap)) (forget); a running
    maximum M that starts at 0: M_t = max(b + M_(t-1), a);  S_t = exp(b + M_(t-1) - M_t) S_(t-1) + exp(a - M_t) k v^T and
    n_t the same with k alone;  o_t = S_t^T q / (max(|n_t . q|, exp(-M_t)) + 1e-6).  Every head's o is divided by its root
    mean square; the heads, side by side, are multiplied by a weight and by sigmoid(W_g h).  Returns [T, H P] and the carry.

    After the division by its root mean square only the direction of S_t^T q_t is left of a head's output.  Where q_t is nearly
    orthogonal to what the memory holds, that direction is decided by rounding: at a request's first token, and wherever the
    forget gate has just emptied the memory, S_t is one term k v^T and the output is v / rms(v) times the SIGN of k . q_t, a step
    function of the input.  `calls` (a list) receives, per token, how far the model is from such a point: 2.5 sqrt(d) |S_t^T q_t| /
    (|S_t| |q_t|) (Frobenius and Euclidean norms; for a memory of one term that is 2.5 sqrt(d) |cos(q, k)|, about 2.5 for a
    query in general position), the least over the heads, in the units of the routers' margins, so that one threshold serves
    both kinds of close call: a margin of 0.25 keeps a query twenty-five times farther from orthogonal than rounding moves it."""
    H, d, P, cap = m["heads"], m["dim"], m["vdim"], m.get("gate_cap")
    T = h.shape[0]
    q = _r(h @ w[pre + "q"].t(), round_to).view(T, H, d) * (d ** -0.5)
    k = _r(h @ w[pre + "k"].t(), round_to).view(T, H, d)
    v = _r(h @ w[pre + "v"].t(), round_to).view(T, H, P)
    a, b = h @ w[pre + "i"].t() + w[pre + "i.b"], h @ w[pre + "f"].t() + w[pre + "f.b"]
    if cap:                                                       # (a model without a cap has uncapped gates)
        a, b = cap * torch.tanh(a / cap), cap * torch.tanh(b / cap)
    b = log_sigmoid(b)
    away = torch.full((T,), float("inf"))
    if carry is None:
        S, n, M = torch.zeros(H, d, P, dtype=h.dtype), torch.zeros(H, d, dtype=h.dtype), torch.zeros(H, dtype=h.dtype)
    else:
        S, n, M = carry
    o = torch.empty(T, H, P, dtype=h.dtype)
    for t in range(T):
        M_new = torch.maximum(b[t] + M, a[t])
        keep, take = torch.exp(b[t] + M - M_new), torch.exp(a[t] - M_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        M = M_new
        num = torch.einsum("adp,ad->ap", S, q[t])
        if calls is not None:
            hold = S.flatten(1).norm(dim=-1) * q[t].norm(dim=-1)
            away[t] = 2.5 * math.sqrt(d) * float((num.norm(dim=-1) / hold.clamp_min(1e-30)).min())
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-M)) + 1e-6
        o[t] = num / den[:, None]
    if calls is not None:
        calls.append(away)
    o = unit_rms(o, eps).reshape(T, H * P) * w[pre + "norm"]
    return o * torch.sigmoid(_r(h @ w[pre + "g"].t(), round_to)), (S, n, M)


def latent_attention(h, w, pre, m, eps, positions, round_to):
    """Attention whose queries, keys and values come through low-rank latents.  c_q = rms_norm(W_dq h); q = W_uq c_q, per head
    [d unrotated | r rotated]; W_dkv h = [R | r]: c = rms_norm(first R), the last r are one rotated key part for all heads;
    key_a = [W_uk c | rotated part], value_a = W_uv c; score = q . key * scale inside a sliding window; the softmax's
    denominator also holds exp(sink_a).  Returns the heads [T, H P] (before the output product)."""
    H, d, r, P, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    cq = _r(rms_norm(_r(h @ w[pre + "dq"].t(), round_to), w[pre + "dq.norm"], eps), round_to)
    q = _r(cq @ w[pre + "uq"].t(), round_to).view(T, H, d + r)
    kv = _r(h @ w[pre + "dkv"].t(), round_to)
    c = _r(rms_norm(kv[:, :R], w[pre + "dkv.norm"], eps), round_to)
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    k_rot = _r(rotate_interleaved(kv[:, None, R:], positions, base, dims), round_to)           # [T, 1, r]
    q_rot = _r(rotate_interleaved(q[..., d:], positions, base, dims), round_to)
    k_nope = (c @ w[pre + "uk"].t()).view(T, H, d)
    v = (c @ w[pre + "uv"].t()).view(T, H, P)
    s = torch.einsum("iad,jad->aij", q[..., :d], k_nope) + torch.einsum("iad,jd->aij", q_rot, k_rot[:, 0])
    size = (m.get("mask") or {}).get("size")
    p = softmax_with_sink(s * m["scale"], causal_mask(T, size), w[pre + "sink"])
    return torch.einsum("aij,jad->iad", p, v).reshape(T, H * P)


def conv_attention(h, w, pre, m, positions, round_to):
    """Grouped-query attention whose q, k and v each pass a short causal convolution per channel right behind the
    projection; then the first rot.dims coordinates of every q and k head are rotated (interleaved pairs);
    s = scale q . k, then s <- softcap tanh(s / softcap); causal; p_j = exp(s_j) / (1 + sum exp(s_j')); head a's output is
    multiplied by sigmoid((W_g h)_a), one number per head.  Returns the gated heads [T, H P]."""
    H, G, d, P = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = causal_conv(_r(h @ w[pre + "q"].t(), round_to), w[pre + "q.conv"]).view(T, H, d)
    k = causal_conv(_r(h @ w[pre + "k"].t(), round_to), w[pre + "k.conv"]).view(T, G, d)
    v = _r(causal_conv(_r(h @ w[pre + "v"].t(), round_to), w[pre + "v.conv"]), round_to).view(T, G, P)
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    q = _r(rotate_interleaved(q, positions, base, dims), round_to)
    k = _r(rotate_interleaved(k, positions, base, dims), round_to)
    rep = H // G
    kh, vh = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)          # query head a reads key/value head a // rep
    s = torch.einsum("iad,jad->aij", q, kh) * m["scale"]
    cap = m.get("softcap")
    if cap:
        s = cap * torch.tanh(s / cap)
    size = (m.get("mask") or {}).get("size")
    p = softmax_with_sink(s, causal_mask(T, size), torch.zeros(H, dtype=h.dtype))
    o = torch.einsum("aij,jad->iad", p, vh)
    gate = torch.sigmoid(_r(h @ w[pre + "g"].t(), round_to))                  # [T, H]
    return (o * gate[:, :, None]).reshape(T, H * P)


# --------------------------------------------------------------------- feed-forwards
def gated_ff(h, w, pre, act, round_to):
    g = _r(h @ w[pre + "gate"].t(), round_to)
    u = _r(h @ w[pre + "up"].t(), round_to)
    return _r(act(g) * u, round_to) @ w[pre + "down"].t()


def routed_ff(h, w, pre, mlp, round_to, gaps=None):
    """z = W_router h + b; the `top` largest logits choose the experts, whose weights are the softmax over the chosen
    logits alone; output = sum of weight_e expert_e(h), plus the shared expert times sigmoid(W_sg h) (one number a token).
    `gaps` (a list) receives, per token, how far the last chosen logit lies above the first one not chosen."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ w[pre + "router"].t() + w[pre + "router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    if gaps is not None and top < E:
        both = torch.topk(z, top + 1, dim=-1).values
        gaps.append((both[:, top - 1] - both[:, top]).to(torch.float32))
    wt = torch.softmax(val, -1)
    out = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=h.dtype)
    for c in range(top):                                   # a token's choices are added in their order
        for e in idx[:, c].unique().tolist():
            rows = idx[:, c] == e
            out[rows] += wt[rows, c, None] * gated_ff(h[rows], w, f"{pre}e{e}.", silu, round_to)
    if mlp.get("shared") is not None:
        out = out + gated_ff(h, w, pre + "shared.", silu, round_to) * torch.sigmoid(h @ w[pre + "shared.sg"].t())
    return out


# --------------------------------------------------------------------- the model
class PlainFunevik:
    def __init__(self, model_dir: str, round_to: Optional[torch.dtype] = None, wide: bool = False):
        with open(os.path.join(model_dir, "config.json")) as f:
            self.cfg = json.load(f)
        self.ft = torch.float64 if wide else torch.float32
        self.w: Dict[str, torch.Tensor] = {n: t.to(self.ft) for n, t in
                                           read_safetensors(os.path.join(model_dir, "model.safetensors")).items()}
        self.round_to = round_to
        self._gaps: list = []
        self.gaps = torch.zeros(0)

    def mixer(self, i: int, L: dict, h: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        w, rt, eps = self.w, self.round_to, self.cfg["norm"]["eps"]
        m, pre = L["mixer"], f"l{i}.mix."
        if L["type"] == "mlstm":
            heads = matrix_memory(h, w, pre, m, eps, rt, calls=self._gaps)[0]
        elif L["type"] == "latent_attention":
            heads = latent_attention(h, w, pre, m, eps, pos, rt)
        elif L["type"] == "attention":
            heads = conv_attention(h, w, pre, m, pos, rt)
        else:
            raise ValueError(L["type"])
        return _r(heads, rt) @ w[pre + "o"].t()

    def feed_forward(self, i: int, mlp: dict, h: torch.Tensor) -> torch.Tensor:
        pre = f"l{i}.mlp."
        if mlp["kind"] == "dense":
            return gated_ff(h, self.w, pre, gelu_tanh, self.round_to)
        if mlp["kind"] == "moe":
            return routed_ff(h, self.w, pre, mlp, self.round_to, self._gaps)
        raise ValueError(mlp["kind"])

    def forward(self, ids: Sequence[int], layers_out: Optional[list] = None) -> torch.Tensor:
        cfg, w, rt = self.cfg, self.w, self.round_to
        eps = cfg["norm"]["eps"]
        pos = torch.arange(len(ids))
        self._gaps = []
        x = w["embed"][torch.tensor(list(ids), dtype=torch.long)] * float(cfg["embedding"]["scale"])
        for i, L in enumerate(cfg["layers"]):
            p = f"l{i}."
            # both sublayers read the same x, each through a norm of its own; each result times its layer scale
            y = self.mixer(i, L, _r(rms_norm(x, w[p + "norm1"], eps), rt), pos) * w[p + "ls1"]
            if L.get("mlp") is not None:
                y = y + self.feed_forward(i, L["mlp"], _r(rms_norm(x, w[p + "norm2"], eps), rt)) * w[p + "ls2"]
            x = x + y
            if layers_out is not None:
                layers_out.append(x.clone())
        # per position, the closest call any router or memory of the model made on it
        self.gaps = torch.stack(self._gaps).amin(0) if self._gaps else torch.full((len(ids),), float("inf"))
        return _r(rms_norm(x, w["final.norm"], eps), rt) @ w["head"].t()

    def logits(self, ids: Sequence[int]) -> torch.Tensor:
        return self.forward(ids).to(torch.float32)
