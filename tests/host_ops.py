"""A stand-in for the CUDA kernel set, for tests of the engine's HOST logic on a machine
without a GPU (batch metadata, cache bookkeeping, scheduling).  It follows the kernels'
calling conventions and cache layout with elementary torch arithmetic on the CPU.  It is
test equipment: the package never imports it, and the `-m gpu` tests never use it.
"""
from __future__ import annotations

import math

import torch


class HostOps:
    def __init__(self):
        self.launches = 0

    def require(self, *names):
        return None

    def choose_kernels(self, kernels):
        return None

    def compile(self, plan):
        return HostPlan(self, plan)

    def embedding(self, ids, table, out, scale=1.0):
        out.copy_(table[ids.long()].float() * scale)
        return out

    def rmsnorm(self, x, gain, eps, out, delta=None, rows=None, gain2=None, out2=None):
        if delta is not None:
            if rows is None:
                x += delta.float()
            else:
                x[rows.long()] += delta.float()[rows.long()]
        src = x if rows is None else x[rows.long()]
        ms = (src * src).sum(-1, keepdim=True) / src.shape[-1]
        out.copy_(((src * (1.0 / torch.sqrt(ms + eps))) * gain.float()).to(out.dtype))
        if out2 is not None:
            out2.copy_(((src * (1.0 / torch.sqrt(ms + eps))) * gain2.float()).to(out2.dtype))
        return out

    def qkv_post(self, *, q_in, k_in, v_in, num_heads, num_kv_heads, head_dim, q_gain=None, k_gain=None, eps=0.0,
                 cos_sin=None, positions=None, q_out=None, k_out=None, cache=None, slot_mapping=None, page_size=0):
        hd, half = head_dim, head_dim // 2

        def post(x, heads, gain):
            x = x.float().reshape(x.shape[0], heads, hd)
            if gain is not None:
                ms = (x * x).sum(-1, keepdim=True) / hd
                x = (x * (1.0 / torch.sqrt(ms + eps))) * gain.float()
            if cos_sin is not None:
                cs = cos_sin[positions.long()]
                c, s = cs[:, None, :half], cs[:, None, half:]
                a, b = x[..., :half], x[..., half:]
                x = torch.cat([a * c - b * s, a * s + b * c], -1)
            return x

        def store(which, x):  # x [T, nkv, hd] -> cache[page, which, kvh, off, :]
            for t in range(x.shape[0]):
                slot = int(slot_mapping[t])
                if slot < 0:
                    continue
                cache[slot // page_size, which, :, slot % page_size, :] = x[t].to(cache.dtype)

        if q_in is not None:
            q = post(q_in, num_heads, q_gain)
            if q_out is not None:
                q_out.copy_(q.reshape(q.shape[0], -1).to(q_out.dtype))
        if k_in is not None:
            k = post(k_in, num_kv_heads, k_gain)
            if k_out is not None:
                k_out.copy_(k.reshape(k.shape[0], -1).to(k_out.dtype))
            if cache is not None:
                store(0, k)
        if v_in is not None and cache is not None:
            store(1, v_in.float().reshape(v_in.shape[0], num_kv_heads, hd))

    def attention_plain(self, *, q, cache, out, positions, token_request, block_tables, num_heads, num_kv_heads,
                        head_dim, page_size, window, scale):
        T = q.shape[0]
        g = num_heads // num_kv_heads
        qf = q.float().reshape(T, num_heads, head_dim)
        for t in range(T):
            p = int(positions[t])
            lo = max(0, p - window + 1) if window > 0 else 0
            bt = block_tables[int(token_request[t])]
            js = torch.arange(lo, p + 1)
            pages = bt[(js // page_size).long()].long()
            assert (pages >= 0).all(), "attention would read a page that is not held"
            k = cache[pages, 0, :, (js % page_size).long(), :].float()      # [n, nkv, hd]
            v = cache[pages, 1, :, (js % page_size).long(), :].float()
            for h in range(num_heads):
                s = (k[:, h // g] @ qf[t, h]) * scale
                w = torch.softmax(s, 0)
                out[t, h * head_dim:(h + 1) * head_dim] = (w @ v[:, h // g]).to(out.dtype)
        return out

    # the fast kernels share the plain one's semantics
    attention = attention_plain

    def swiglu(self, gate_up, out, bias=None):
        inter = out.shape[1]
        g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
        if bias is not None:
            g, u = (g + bias[:inter]).to(out.dtype).float(), (u + bias[inter:]).to(out.dtype).float()
        out.copy_(((g / (1.0 + torch.exp(-g))) * u).to(out.dtype))
        return out

    def linear(self, x, w, out, bias=None):
        y = x.float() @ w.float().t()
        out.copy_((y if bias is None else y.to(out.dtype).float() + bias).to(out.dtype))
        return out

    def activation(self, act, params, x, out):
        assert act == "xielu"
        z = x.float()
        ap, an = params
        out.copy_(torch.where(z > 0, ap * z * z + 0.5 * z, an * (torch.expm1(torch.clamp(z, max=0)) - z) + 0.5 * z).to(out.dtype))

    def pointwise(self, kind, a, b, out, scale=1.0, group=1):
        assert kind == "sigmoid_mul"
        g = torch.sigmoid(b.float())
        if group > 1:
            g = g.repeat_interleave(group, 1)
        out.copy_((a.float() * g * scale).to(out.dtype))

    # ---- layers with a state of fixed size per request
    @staticmethod
    def _requests(batch):
        cu = batch.cu_q_lens.tolist()
        return [(cu[r], cu[r + 1], int(batch.state_slots[r])) for r in range(len(cu) - 1)]

    def short_conv(self, a, batch):
        w, K = a["w"], a["w"].shape[1]
        for lo, hi, slot in self._requests(batch):
            if hi == lo:
                continue
            x = a["x"][lo:hi].float()
            past = a["state"][slot][: K - 1] if K > 1 else x[:0]
            full = torch.cat([past, x], 0)
            y = a["bias"].float().expand(hi - lo, -1).clone() if a["bias"] is not None else torch.zeros_like(x)
            for j in range(K):
                y += full[K - 1 - j: K - 1 - j + (hi - lo)] * w[:, K - 1 - j]
            a["out"][lo:hi] = y * torch.sigmoid(y) if a["act"] == "silu" else y
            if K > 1:
                a["state"][slot][: K - 1] = full[-(K - 1):]

    def rotate(self, a, T, positions):
        for x, out, heads, scale in zip(a["x"], a["out"], a["heads"], a["scale"]):
            if x is None:
                continue
            v = x[:T].float().view(T, heads, a["dim"])
            if a["rot_dims"]:
                half = a["rot_dims"] // 2
                ang = positions.float()[:, None] * a["inv_freq"][None, :]
                c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
                u, w = v[..., :half], v[..., half:2 * half]
                v = torch.cat([u * c - w * s, w * c + u * s, v[..., 2 * half:]], -1)
            out[:T] = v.reshape(T, -1) * scale

    def recurrence(self, a, batch):
        H, n, p, G = a["heads"], a["n"], a["p"], a["qk_groups"]
        rep = H // G
        for lo, hi, slot in self._requests(batch):
            S = a["state"][slot]                                           # [H, p, n]
            for t in range(lo, hi):
                q = a["q"][t].view(G, n).repeat_interleave(rep, 0)
                k = a["k"][t].view(G, n).repeat_interleave(rep, 0)
                if a.get("unit_column"):
                    v = torch.cat([a["v"][t].float().view(H, p - 1), torch.ones(H, 1)], 1)
                else:
                    v = a["v"][t].float().view(H, p)
                if a.get("keep") is not None:
                    decay, step = a["keep"][t], a["take"][t]
                elif a["dt"] is None:
                    decay, step = a["decay"], torch.ones(H)
                else:
                    z = a["dt"][t].float() + (a["dt_bias"] if a["dt_bias"] is not None else 0.0)
                    step = torch.clamp(z, min=0) + torch.log1p(torch.exp(-z.abs()))
                    decay = torch.exp(-torch.exp(a["a_log"]) * step)
                S.mul_(decay[:, None, None]).add_((step[:, None] * v)[:, :, None] * k[:, None, :])
                y = torch.einsum("hpn,hn->hp", S, q)
                if a["skip"] is not None:
                    y = y + a["skip"][:, None] * v
                a["out"][t] = y.reshape(-1)

    def gated_norm(self, a, T):
        y, g = a["y"][:T], a["gate"][:T].float()
        gate = torch.sigmoid(g) if a.get("gate_act", "silu") == "sigmoid" else g * torch.sigmoid(g)
        if a.get("floor") is not None:
            wide = y.reshape(T, -1, a["group"] + 1)
            den = torch.maximum(wide[..., -1].abs(), a["floor"][:T]) + a["den_eps"]
            y = (wide[..., :-1] / den[..., None]).reshape(T, -1)
        u = y * gate if a["gate_first"] else y
        parts = u.view(T, -1, a["group"])
        u = (parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + a["eps"])).reshape(T, -1)
        if a["weight"] is not None:
            u = u * a["weight"]
        if not a["gate_first"]:
            u = u * gate
        a["out"][:T] = (u * a["scale"]).to(a["out"].dtype)

    def row_norm(self, a, T):
        x = a["x"][:T].float()
        a["out"][:T] = (x * (1.0 / torch.sqrt((x * x).mean(-1, keepdim=True) + a["eps"])) * a["gain"].float()).to(a["out"].dtype)

    def exp_gates(self, a, batch):
        cap = a["cap"]
        for lo, hi, slot in self._requests(batch):
            M = a["state"][slot]
            for t in range(lo, hi):
                i, f = a["i_pre"][t].float(), a["f_pre"][t].float()
                if cap > 0:
                    i, f = cap * torch.tanh(i / cap), cap * torch.tanh(f / cap)
                f = torch.clamp(f, max=0) - torch.log1p(torch.exp(-f.abs()))
                new = torch.maximum(f + M, i)
                a["keep"][t] = torch.exp(f + M - new)
                a["take"][t] = torch.exp(i - new)
                a["floor"][t] = torch.exp(-new)
                M.copy_(new)

    def batched_linear(self, x, w, out):
        out.copy_(torch.einsum("tbk,bnk->tbn", x.float(), w.float()).to(out.dtype))

    @staticmethod
    def _rotate(x, positions, inv_freq, dims, interleaved=False, amplitude=1.0):
        half = dims // 2
        ang = positions.float()[:, None] * inv_freq.float()[None, :]
        shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
        c, s = (torch.cos(ang) * amplitude).reshape(shape), (torch.sin(ang) * amplitude).reshape(shape)
        if interleaved:
            u, v = x[..., 0:dims:2], x[..., 1:dims:2]
            return torch.cat([torch.stack([u * c - v * s, v * c + u * s], -1).flatten(-2), x[..., dims:]], -1)
        u, v = x[..., :half], x[..., half:dims]
        return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)

    def latent_attention(self, a, T, positions, token_request, block_tables, slot_mapping, page_size):
        H, r, dr = a["num_heads"], a["kv_rank"], a["rot_dim"]
        cache, q, out = a["cache"], a["q"][:T].view(T, H, r + dr), a["out"][:T].view(T, H, r)
        kv = a["kv_in"][:T].float()
        c = kv[:, :r]
        c = c * (1.0 / torch.sqrt((c * c).mean(-1, keepdim=True) + a["eps"])) * a["c_gain"].float()
        row = c
        if dr:
            il = bool(a.get("interleaved"))
            row = torch.cat([c, self._rotate(kv[:, r:], positions, a["inv_freq"], a["rot_dims"], il)], -1)
            q[:, :, r:] = self._rotate(a["q_rot"][:T].float(), positions, a["inv_freq"], a["rot_dims"], il).to(q.dtype)
        flat = cache.view(-1, r + dr)
        for t in range(T):
            if int(slot_mapping[t]) >= 0:
                flat[int(slot_mapping[t])] = row[t].to(cache.dtype)
        for t in range(T):
            p = int(positions[t])
            bt = block_tables[int(token_request[t])]
            W = a.get("window", 0)
            js = torch.arange(max(0, p - W + 1) if W > 0 else 0, p + 1)
            pages = bt[(js // page_size).long()].long()
            assert (pages >= 0).all(), "attention would read a page that is not held"
            rows = flat[pages * page_size + (js % page_size)].float()            # [n, r + dr]
            s = (q[t].float() @ rows.t()) * a["scale"]                           # [H, n]
            if a["sink"] is not None:
                s = torch.cat([s, a["sink"].float()[:, None]], -1)
            w = torch.softmax(s, -1)[:, : js.numel()]
            out[t] = (w @ rows[:, :r]).to(out.dtype)

    def gated_act(self, act, params, gate_up, out):
        inter = out.shape[1]
        if act == "gelu_tanh":
            g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
            out.copy_((0.5 * g * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (g + 0.044715 * g ** 3))) * u).to(out.dtype))
            return
        assert act == "clamped_swish"
        limit, slope = params
        g = torch.clamp(gate_up[:, :inter].float(), max=limit)
        u = torch.clamp(gate_up[:, inter:].float(), -limit, limit)
        out.copy_((g * torch.sigmoid(slope * g) * (u + 1.0)).to(out.dtype))

    def postnorm(self, x, y, gain, eps, accumulate, copy):
        if y is not None:
            yf = y.float()
            n = yf * (1.0 / torch.sqrt((yf * yf).mean(-1, keepdim=True) + eps)) * gain.float()
            if accumulate:
                x += n
            else:
                x.copy_(n)
        if copy is not None:
            copy.copy_(x.to(copy.dtype))

    def window_attention(self, a, T, positions, token_request, block_tables, slot_mapping, page_size):
        H, G, dk, dv = a["num_heads"], a["num_kv_heads"], a["qk_dim"], a["v_dim"]
        cache, ps = a["cache"], page_size
        pages = cache.view(cache.shape[0], -1)
        keys = pages[:, :G * ps * dk].view(-1, G, ps, dk)
        vals = pages[:, G * ps * dk:].view(-1, G, ps, dv)

        def biased(x, bias):
            return x[:T] if bias is None else (x[:T].float() + bias).to(x.dtype)

        def finish(x, heads, gain, bias=None):
            x = biased(x, bias).float()
            if gain is not None and a.get("head_norm"):
                x = x.view(T, heads, dk)
                x = (x * (1.0 / torch.sqrt((x * x).mean(-1, keepdim=True) + a["eps"])) * gain).reshape(T, -1)
            elif gain is not None:
                x = x * (1.0 / torch.sqrt((x * x).mean(-1, keepdim=True) + a["eps"])) * gain
            x = x.view(T, heads, dk)
            if a["inv_freq"] is not None:
                x = self._rotate(x, positions, a["inv_freq"], a["rot_dims"], bool(a.get("interleaved")), a["amplitude"])
            return x
        q = finish(a["q_in"], H, a["q_gain"], a.get("q_bias")).to(cache.dtype)
        a["q"][:T] = q.reshape(T, -1)
        if a["k_in"] is not None:
            k = finish(a["k_in"], G, a["k_gain"], a.get("k_bias")).to(cache.dtype)
            v = biased(a["v_in"], a.get("v_bias")).reshape(T, G, dv).to(cache.dtype)
            for t in range(T):
                slot = int(slot_mapping[t])
                if slot >= 0:
                    keys[slot // ps, :, slot % ps] = k[t]
                    vals[slot // ps, :, slot % ps] = v[t]
        rep = H // G
        W, first = a["window"], a["keep_first"]
        for t in range(T):
            p = int(positions[t])
            lo = max(0, p - W + 1) if W > 0 else 0
            js = torch.tensor([j for j in range(p + 1) if j >= lo or j < first])
            bt = block_tables[int(token_request[t])]
            pg = bt[(js // ps).long()].long()
            assert (pg >= 0).all(), "attention would read a page that is not held"
            kk = keys[pg, :, (js % ps).long()].float()            # [n, G, dk]
            vv = vals[pg, :, (js % ps).long()].float()
            for h in range(H):
                s = (kk[:, h // rep] @ q[t, h].float()) * a["scale"]
                if a.get("softcap"):
                    s = a["softcap"] * torch.tanh(s / a["softcap"])
                if a["sink"] is not None:
                    s = torch.cat([s, a["sink"][h:h + 1]])
                w = torch.softmax(s, 0)[: js.numel()]
                a["out"][t, h * dv:(h + 1) * dv] = (w @ vv[:, h // rep]).to(a["out"].dtype)

    def moe_route(self, a, T):
        top, E = a["top_k"], a["logits"].shape[1]
        if a.get("mode", "sigmoid") == "softmax_chosen":
            val, idx = torch.topk(a["logits"][:T].float(), top, dim=-1)
            wt = torch.softmax(val, -1) * a["scale"]
        else:
            s = torch.sigmoid(a["logits"][:T].float())
            val, idx = torch.topk(s, top, dim=-1)
            wt = val / (val.sum(-1, keepdim=True) + 1e-20) * a["scale"]
        a["experts"][:T] = idx.to(torch.int32)
        a["weights"][:T] = wt
        flat = idx.reshape(-1)
        order = torch.argsort(flat, stable=True)
        a["order"][:T * top] = order.to(torch.int32)
        counts = torch.bincount(flat, minlength=E)
        a["offsets"][1:] = torch.cumsum(counts, 0).to(torch.int32)
        a["offsets"][0] = 0

    def grouped_linear(self, a, T):
        top, w = a["top_k"], a["w"]
        off, order = a["offsets"].tolist(), a["order"]
        for e in range(w.shape[0]):
            for r in range(off[e], off[e + 1]):
                pair = int(order[r])
                row = a["x"][pair // top if a["gather"] else r].float()
                y = w[e].float() @ row
                if a["act"]:
                    n = y.numel() // 2
                    g, u = y[:n].to(a["x"].dtype).float(), y[n:].to(a["x"].dtype).float()
                    y = g * torch.sigmoid(g) * u
                a["out"][pair if a["scatter"] else r] = y.to(a["out"].dtype)

    def token_side(self, a, T, token_ids):
        x = a["x"][:T]
        x += a["a"][:T].float() + (a["b"][:T].float() if a["b"] is not None else 0.0)
        e = a["table"][token_ids.long()][:, a["offset"]:a["offset"] + a["dim"]].float()
        z = x @ a["w_gate"].float().t()
        g = 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3))) * e
        y = g @ a["w_proj"].float().t()
        x += y * (1.0 / torch.sqrt((y * y).mean(-1, keepdim=True) + a["eps"])) * a["gain"].float()

    def repetition_penalty(self, logits, rows, tokens, counts, penalty):
        for r, t, c in zip(rows.tolist(), tokens.tolist(), counts.tolist()):
            p = float(penalty[r])
            for _ in range(c):
                logits[r, t] = logits[r, t] / p if logits[r, t] > 0 else logits[r, t] * p

    def sample(self, logits, *, greedy, temperature, top_k, top_p, u, out):
        from plain_model import plain_sample
        for r in range(logits.shape[0]):
            out[r] = plain_sample(logits[r], greedy=bool(greedy[r]), temperature=float(temperature[r]),
                                  top_k=int(top_k[r]), top_p=float(top_p[r]), u=float(u[r]))
        return out


class HostPlan:
    """A plan interpreted on the CPU: every record runs on the first rows of its buffers, as the native
    executor runs it on the device."""

    def __init__(self, ops, plan):
        self.ops, self.plan = ops, plan

    def run(self, batch, first=0, count=-1):
        o = self.ops
        T, NL = batch.num_tokens, batch.logit_rows.numel()
        last = len(self.plan.ops) if count < 0 else first + count

        def n_rows(kind):
            return NL if kind == "logits" else T

        def cut(t, n=T):
            return None if t is None else t[:n]
        for op in self.plan.ops[first:last]:
            a, k = op.a, op.kind
            if k == "embedding":
                o.embedding(batch.token_ids, a["table"], a["out"][:T], a.get("scale", 1.0))
            elif k == "rmsnorm":
                some = a["rows"] == "logits"
                o.rmsnorm(a["x"][:T], a["gain"], a["eps"], a["out"][:n_rows(a["rows"])], delta=cut(a["delta"]),
                          rows=batch.logit_rows if some else None, gain2=a.get("gain2"),
                          out2=a["out2"][:n_rows(a["rows"])] if a.get("out2") is not None else None)
            elif k == "linear":
                n = n_rows(a["rows"])
                if n:
                    o.linear(a["x"][:n], a["w"], batch.logits if a["out"] is None else a["out"][:n], a.get("bias"))
            elif k == "short_conv":
                o.short_conv(a, batch)
            elif k == "rotate":
                o.rotate(a, T, batch.positions)
            elif k == "recurrence":
                o.recurrence(a, batch)
            elif k == "gated_norm":
                o.gated_norm(a, T)
            elif k == "row_norm":
                o.row_norm(a, T)
            elif k == "exp_gates":
                o.exp_gates(a, batch)
            elif k == "linear_swiglu":
                o.linear(a["x"][:T], a["w_gate_up"], a["gate_up"][:T])
                if a.get("act", "silu") == "silu":
                    o.swiglu(a["gate_up"][:T], a["out"][:T], a.get("bias"))
                else:
                    assert a.get("bias") is None
                    o.gated_act(a["act"], a["params"], a["gate_up"][:T], a["out"][:T])
            elif k == "postnorm":
                o.postnorm(a["x"][:T], cut(a["y"]), a["gain"], a["eps"], a["accumulate"], cut(a["copy"]))
            elif k == "window_attention":
                g = batch.groups[a["group"]]
                o.window_attention(a, T, batch.positions, batch.token_request, g.block_tables, g.slot_mapping, g.page_size)
            elif k == "moe_route":
                o.moe_route(a, T)
            elif k == "grouped_linear":
                o.grouped_linear(a, T)
            elif k == "moe_combine":
                top = a["weights"].shape[1]
                y = a["y"][:T * top].view(T, top, -1)
                v = (a["weights"][:T, :, None] * y).sum(1)
                base = a["base"][:T] if a["base"] is not None else None
                if base is not None and a.get("base_gate") is not None:
                    base = base * torch.sigmoid(a["base_gate"][:T])
                a["out"][:T] = v if base is None else base + v
            elif k == "qkv_post":
                self._qkv_post(a, batch, T)
            elif k == "attend":
                self._attend(a, batch, T)
            elif k == "attention":
                nh, nkv, hd = a["num_heads"], a["num_kv_heads"], a["head_dim"]
                qs, kvs = nh * hd, nkv * hd
                qkv, w = a["qkv"], a["writes"]
                self._qkv_post(dict(a, q_in=qkv[:, :qs], k_in=qkv[:, qs:qs + kvs] if w else None,
                                    v_in=qkv[:, qs + kvs:] if w else None, q_out=a["q"], k_out=None,
                                    cache=a["cache"] if w else None), batch, T)
                self._attend(a, batch, T)
            elif k == "linear_act":
                o.linear(a["x"][:T], a["w"], a["mid"][:T])
                o.activation(a["act"], a["params"], a["mid"][:T], a["out"][:T])
            elif k == "pointwise":
                o.pointwise(a["what"], a["a"][:T], cut(a["b"]), a["out"][:T], a.get("scale", 1.0), a.get("group", 1))
            elif k == "batched_linear":
                o.batched_linear(a["x"][:T], a["w"], a["out"][:T])
            elif k == "residual_add":
                u = a["a"][:T].float() * (a["a_scale"] if a.get("a_scale") is not None else 1.0)
                if a["b"] is not None:
                    u = u + a["b"][:T].float() * (a["b_scale"] if a.get("b_scale") is not None else 1.0)
                a["x"][:T] += u
            elif k == "latent_attention":
                g = batch.groups[a["group"]]
                o.latent_attention(a, T, batch.positions, batch.token_request, g.block_tables, g.slot_mapping, g.page_size)
            elif k == "token_side":
                o.token_side(a, T, batch.token_ids)
            elif k == "call":
                a["fn"](batch)
            else:
                raise ValueError(k)

    def _qkv_post(self, a, batch, T):
        cut = lambda t: None if t is None else t[:T]
        g = batch.groups[a["group"]] if a.get("cache") is not None else None
        self.ops.qkv_post(q_in=cut(a.get("q_in")), k_in=cut(a.get("k_in")), v_in=cut(a.get("v_in")), num_heads=a["num_heads"],
                          num_kv_heads=a["num_kv_heads"], head_dim=a["head_dim"], q_gain=a.get("q_gain"), k_gain=a.get("k_gain"),
                          eps=a.get("eps", 0.0), cos_sin=a.get("cos_sin"), positions=batch.positions, q_out=cut(a.get("q_out")),
                          k_out=cut(a.get("k_out")), cache=a.get("cache"), slot_mapping=g.slot_mapping if g else None,
                          page_size=g.page_size if g else 0)

    def _attend(self, a, batch, T):
        g = batch.groups[a["group"]]
        self.ops.attention_plain(q=a["q"][:T], cache=a["cache"], out=a["out"][:T], positions=batch.positions,
                                 token_request=batch.token_request, block_tables=g.block_tables, num_heads=a["num_heads"],
                                 num_kv_heads=a["num_kv_heads"], head_dim=a["head_dim"], page_size=g.page_size,
                                 window=a["window"], scale=a["scale"])
