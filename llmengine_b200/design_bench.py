"""A design beside its closest existing model at equal size (`python bench.py --design bepuzen | torisun | vifelix | funevik`).

For each size: prefill of one 2,048-token prompt and decode at batch 1 / 8 / 64 over 2,048 cached tokens, tokens/s,
for the design and for the grouped-query model of the same width, depth and (active) weight count per layer;
and the time of every record of one layer of each (the model's own plan, record by record inside a CUDA graph, each
layer's own weights, CUDA events) with the record's roofline: the larger of its algorithmic bytes over the copy
bandwidth and its floating-point operations over the product peak, divided by the time measured.
"""
from __future__ import annotations

import json
import statistics
from typing import Any, Dict, List

L1, L2 = "latent_attention", "latent_attention_2"
# a 32-bit operation outside the tensor cores counts as this many operations of the bf16 product peak that the tables divide
# by (set by `run` from the measured peak), so that `ideal` is its time at the 32-bit ceiling
FP32_SHARE = 1.0


def bepuzen_shape(layers: int, width: int, heads: int, ff: int, kv_rank: int = 512, dim: int = 128, rot: int = 64,
                  vdim: int = 128, side: int = 256, vocab: int = 32768) -> Dict[str, Any]:
    """Layers of the two mixers in turn (every third with the rotated part, sink and gate)."""
    out = []
    for i in range(layers):
        if i % 3 == 0:
            m = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": kv_rank, "scale": (dim + rot) ** -0.5,
                 "rot": {"base": 10000.0, "dims": rot}}
            out.append({"type": L1, "mixer": m, "mlp": {"kind": "dense", "ff": ff}})
        else:
            m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": dim ** -0.5}
            out.append({"type": L2, "mixer": m, "mlp": {"kind": "dense", "ff": ff}})
    return {"architecture": "Bepuzen", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "token_side": {"dim": side},
            "layers": out}


def gqa_shape(layers: int, width: int, heads: int, inter: int, vocab: int = 32768) -> Dict[str, Any]:
    return {"architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": layers, "hidden_size": width,
            "num_attention_heads": heads, "num_key_value_heads": max(1, heads // 4), "head_dim": 128, "intermediate_size": inter,
            "vocab_size": vocab, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
            "max_position_embeddings": 40960, "hidden_act": "silu"}


def torisun_shape(layers: int, width: int, heads: int, kv_heads: int, ff: int, experts: int, top: int, expert_ff: int,
                  window: int = 1024, keep_first: int = 4, dim: int = 128, vocab: int = 32768) -> Dict[str, Any]:
    """Layers in pairs: one with keys and values of its own and the dense feed-forward, then one that reads the first
    one's keys and values (with a narrower window) and has the mixture of experts with a shared expert."""
    rot = {"base": 1000000.0, "dims": dim // 2, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    out = []
    for i in range(layers):
        m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
             "mask": {"size": window if i % 2 == 0 else window // 2, "keep_first": keep_first}, "rot": rot}
        if i % 2 == 0:
            mlp = {"kind": "dense", "ff": ff, "limit": 7.0}
        else:
            m["kv_from"] = i - 1
            mlp = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top, "scale": 2.5},
                   "shared": {"ff": expert_ff}}
        out.append({"type": "attention", "mixer": m, "mlp": mlp})
    return {"architecture": "Torisun", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": out}


def vifelix_shape(width: int, heads: int, kv_heads: int, ff: int, ssm_heads: int, retention_heads: int, window: int = 1024,
                  dim: int = 128, state: int = 128, vocab: int = 32768) -> Dict[str, Any]:
    """Six layers: four state-space layers without feed-forward and two parallel layers (window attention beside retention)
    with one.  The state-space mixer is twice the width inside, in heads of 64."""
    mamba = {"type": "mamba2", "mlp": None,
             "mixer": {"heads": ssm_heads, "vdim": 64, "state": state, "groups": 8, "conv": 4, "norm_groups": 8}}
    par = {"type": "parallel", "mlp": {"kind": "dense", "ff": ff}, "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "mask": {"size": window},
                 "rot": {"base": 10000.0, "dims": dim // 2}},
        "right": {"heads": retention_heads, "dim": dim, "vdim": dim, "decay": [1.0 - 0.04 / (1 + i) for i in range(retention_heads)],
                  "rot": {"base": 100000.0, "dims": dim}},
        "left_scale": 0.9, "right_scale": 0.7}}
    return {"architecture": "Vifelix", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": width ** 0.5},
            "layers": [mamba, mamba, par, mamba, mamba, par]}


def funevik_shape(width: int, heads: int, kv_heads: int, ff: int, experts: int, top: int, expert_ff: int, memory_heads: int,
                  window: int = 1024, dim: int = 128, vocab: int = 32768) -> Dict[str, Any]:
    """Six layers, every layer with two norms and two scale vectors: three matrix memories (heads of 128 x 256), two latent
    attentions (queries through a latent of 1,536, keys and values through one of 512, a shared rotated part of 64, a window)
    and one grouped-query attention with short convolutions and capped scores; dense and routed feed-forwards in turn."""
    mem = {"heads": memory_heads, "dim": 128, "vdim": 256, "gate_cap": 15.0}
    lat = {"heads": heads, "dim": dim, "rot_dim": 64, "vdim": dim, "kv_rank": 512, "q_rank": 1536, "scale": (dim + 64) ** -0.5,
           "rot": {"base": 10000.0, "dims": 64}, "mask": {"size": window}}
    att = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "conv": 4, "softcap": 50.0,
           "rot": {"base": 10000.0, "dims": dim // 2}}
    dense = {"kind": "dense", "ff": ff}
    routed = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top}, "shared": {"ff": expert_ff}}
    kinds = [("mlstm", mem, dense), ("latent_attention", lat, routed), ("mlstm", mem, dense), ("attention", att, routed),
             ("mlstm", mem, None), ("latent_attention", lat, dense)]
    return {"architecture": "Funevik", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": width ** 0.5},
            "layers": [{"type": t, "mixer": m, "mlp": f} for t, m, f in kinds]}


# 32-bit multiply-adds outside the tensor cores: 148 SMs x 128 lanes x 2 x 1.965 GHz (nominal), the compute ceiling of a
# recurrence whose state and inputs are 32-bit
FP32_TFLOPS = 74.4

# name -> (layers timed, the design's shape, the grouped-query model of the same width and feed-forward weight count)
TORISUN_SIZES = {
    "2048": (6, torisun_shape(6, 2048, 16, 4, 5504, 32, 4, 1024), gqa_shape(6, 2048, 16, 5504)),
    "4096": (6, torisun_shape(6, 4096, 32, 8, 10944, 64, 4, 2048), gqa_shape(6, 4096, 32, 10944)),
}
SIZES = {
    "2048": (6, bepuzen_shape(6, 2048, 16, 8192), gqa_shape(6, 2048, 16, 5504)),
    "4096": (6, bepuzen_shape(6, 4096, 32, 16384), gqa_shape(6, 4096, 32, 10944)),
}
VIFELIX_SIZES = {
    "2048": (6, vifelix_shape(2048, 16, 4, 5504, 64, 8), gqa_shape(6, 2048, 16, 5504)),
    "4096": (6, vifelix_shape(4096, 32, 8, 10944, 128, 16), gqa_shape(6, 4096, 32, 10944)),
}
FUNEVIK_SIZES = {
    "2048": (6, funevik_shape(2048, 16, 4, 5504, 32, 4, 1024, 8), gqa_shape(6, 2048, 16, 5504)),
    "4096": (6, funevik_shape(4096, 32, 8, 10944, 64, 4, 2048, 16), gqa_shape(6, 4096, 32, 10944)),
}
CACHED, PROMPT = 2048, 2048


def _vocab(cfg) -> int:
    return cfg.get("vocab", cfg.get("vocab_size"))


def _bytes(t) -> int:
    return 0 if t is None else t.numel() * t.element_size()


def record_cost(op, T: int, keys_per_row: float, cache_rows: float):
    """(label, floating-point operations, algorithmic bytes) of one record for a step of T tokens.  `keys_per_row`: mean
    number of keys a token attends to; `cache_rows`: cache rows the step's requests hold together (each read once)."""
    a, k = op.a, op.kind
    el = 2

    def rows(t, n=T):
        return 0 if t is None else n * t.shape[-1] * t.element_size() if t.dim() == 2 else n * t[0].numel() * t.element_size()
    if k in ("linear", "linear_act", "linear_swiglu"):
        w = a["w_gate_up"] if k == "linear_swiglu" else a["w"]
        out = a["out"]
        n_out = out.shape[1] if out is not None else w.shape[0]
        return f"{k} {w.shape[0]}x{w.shape[1]}", 2.0 * T * w.numel(), _bytes(w) + T * (w.shape[1] * el + n_out * (out.element_size() if out is not None else 4))
    if k == "batched_linear":
        w = a["w"]
        return f"batched_linear {w.shape[0]}x{w.shape[1]}x{w.shape[2]}", 2.0 * T * w.numel(), _bytes(w) + T * w.shape[0] * (w.shape[1] + w.shape[2]) * el
    if k == "latent_attention":
        H, r, dr, W = a["num_heads"], a["kv_rank"], a["rot_dim"], a.get("window", 0)
        keys, rows_read = keys_per_row, cache_rows
        if W and T > cache_rows / 2:                                     # a prompt: the mean over positions 0 .. ctx - 1
            n = int(2 * keys_per_row - 1)
            keys = sum(min(i + 1, W) for i in range(n)) / n
        elif W:
            keys = min(keys_per_row, W)
            rows_read = cache_rows * keys / keys_per_row
        return (f"latent attention {H} heads, rows of {r}+{dr}" + (f", window {W}" if W else ""), 2.0 * T * H * keys * (2 * r + dr),
                rows_read * (r + dr) * el + T * H * (2 * r + dr) * el)
    if k in ("attention", "attend"):
        nh, nkv, hd = a["num_heads"], a["num_kv_heads"], a["head_dim"]
        return (f"attention {nh}/{nkv} heads of {hd}", 4.0 * T * nh * hd * keys_per_row, cache_rows * 2 * nkv * hd * el + 2 * T * nh * hd * el)
    if k == "window_attention":
        H, G, dk, dv, W, first = a["num_heads"], a["num_kv_heads"], a["qk_dim"], a["v_dim"], a["window"], a["keep_first"]
        keys, rows_read = keys_per_row, cache_rows
        if W:
            ctx = 2 * keys_per_row - 1 if T > cache_rows / 2 else keys_per_row       # a prompt's mean is over positions 0..ctx-1
            if T > cache_rows / 2:
                n = int(ctx)
                keys = (sum(min(i + 1, W) for i in range(n)) / n) + min(first, max(0, n - W))
            else:
                keys = min(keys_per_row, W + first)
                rows_read = cache_rows * keys / keys_per_row
        proj = a["q_in"].shape[1] + (a["k_in"].shape[1] + a["v_in"].shape[1] if a["k_in"] is not None else 0)
        return (f"window attention {H}/{G} heads of {dk}/{dv}, window {W}+{first}" + ("" if a["k_in"] is not None else ", reads another layer's keys"),
                2.0 * T * H * keys * (dk + dv), rows_read * G * (dk + dv) * el + T * (proj + 2 * H * dk + H * dv) * el)
    if k == "postnorm":
        D = a["x"].shape[1]
        return "norm of a sublayer's output + residual add", 0.0, T * D * (4 + 4 + 4 + el)
    if k == "moe_route":
        E = a["logits"].shape[1]
        return f"routing {a['top_k']} of {E}", 0.0, T * E * 4 + T * a["top_k"] * 12
    if k == "grouped_linear":
        w, top = a["w"], a["top_k"]
        E, n, kk = w.shape
        used = E * (1.0 - (1.0 - top / E) ** T)                       # experts that some token of the step uses, in the mean
        n_out = n // 2 if a["act"] else n
        return (f"grouped {'gate|up + silu' if a['act'] else 'down'} {E}x{n}x{kk}", 2.0 * T * top * n * kk,
                used * n * kk * el + T * top * (kk * el + n_out * a["out"].element_size()))
    if k == "moe_combine":
        D, top = a["out"].shape[1], a["weights"].shape[1]
        return "weighted sum of the chosen experts", 0.0, T * D * (top * 4 + (4 if a["base"] is not None else 0) + 4)
    if k == "rmsnorm":
        return "rmsnorm + residual add", 0.0, T * a["x"].shape[1] * (4 + 4 + 4 + el)
    if k == "token_side":
        D, dim = a["x"].shape[1], a["dim"]
        return f"token side input (dim {dim})", 4.0 * T * D * dim, T * D * (4 * 4) + 2 * D * dim * el
    if k == "pointwise":
        return f"pointwise {a['what']}", 0.0, 3 * T * a["out"].shape[1] * el
    if k == "residual_add":
        return "residual add" + (" with scale vectors" if a.get("a_scale") is not None else ""), 0.0, T * a["x"].shape[1] * 16
    if k == "row_norm":
        return f"norm on a product's columns ({a['x'].shape[1]})", 0.0, T * a["x"].shape[1] * 2 * el
    if k == "exp_gates":
        return f"exponential gates, {a['i_pre'].shape[1]} heads", 0.0, T * a["i_pre"].shape[1] * 5 * 4
    requests = T if T <= cache_rows / 2 else 1                            # a decode step has one token a request
    if k == "short_conv":
        C, K = a["w"].shape
        return (f"short convolution {C}x{K}", 2.0 * T * C * K * FP32_SHARE,
                T * C * (a["x"].element_size() + 4) + C * (K + 1) * 4 + requests * 2 * (K - 1) * C * 4)
    if k == "rotate":
        cols = sum(h for x_, h in zip(a["x"], a["heads"]) if x_ is not None) * a["dim"]
        return f"rotation into 32-bit, {cols} columns", 0.0, T * cols * (el + 4)
    if k == "recurrence":
        H, n, p, G = a["heads"], a["n"], a["p"], a["qk_groups"]
        return (f"recurrence {H} heads, state {n}x{p}" + (", decay per token" if a.get("dt") is not None else
                                                          ", given gates" if a.get("keep") is not None else ", fixed decay"),
                4.0 * T * H * n * p * FP32_SHARE, requests * 2 * H * n * p * 4 + T * (2 * G * n * 4 + H * p * (a["v"].element_size() + 4)))
    if k == "gated_norm":
        cols = a["y"].shape[1]
        return f"gate + norm in groups of {a['group']}" + (", normalised" if a.get("floor") is not None else ""), 0.0, T * cols * (4 + 2 * el)
    return k, 0.0, 0.0


def layer_table(cfg, layers: int, batch: int, page: int, pk) -> Dict[str, List[Dict[str, Any]]]:
    """Per record of one layer: microseconds and the share of its roofline, for a decode step and for a prompt."""
    import torch

    from .config import EngineConfig
    from .engine.engine import Engine, StepEntry

    T = PROMPT
    ec = EngineConfig(dtype="bfloat16", page_size=page, max_cached_tokens=batch * (CACHED + page) + T + page, max_num_seqs=batch + 1,
                      max_num_batched_tokens=T, max_model_len=max(CACHED + page, T), use_cuda_graphs=False)
    eng = Engine(config=cfg, random_seed=0, engine_config=ec)
    gen = torch.Generator().manual_seed(0)
    V = _vocab(cfg)
    names = [f"r{i}" for i in range(batch)]
    for n in names:
        eng.step([StepEntry(n, torch.randint(0, V, (CACHED,), generator=gen).tolist(), [])])
        eng.cache.reserve(n, CACHED + 1)
    plan = eng.model.plan(eng._caches)
    compiled = eng.ops.compile(plan)
    # which records belong to which layer: every block emits once more into a plan of its own, and is counted
    from .engine.plan import Plan
    from .parts.base import emit_block, emit_embedding
    scratch = Plan()
    x = emit_embedding(scratch, eng.model.embedding, eng.spec.hidden_size)
    per_layer, delta = [], None
    for i, run_ in enumerate(eng.model.order):
        at = len(scratch.ops)
        x, delta = emit_block(scratch, eng.model.blocks[run_.layer], x, delta, eng._caches[i])
        per_layer.append(list(range(at, len(scratch.ops))))
    assert len(scratch.ops) + 2 == len(plan.ops), "the plan is not embedding, layers, final norm, head"
    assert all(a.kind == b.kind for a, b in zip(scratch.ops, plan.ops))

    def measure(indices, batch_obj, reps=10):
        eng.rt.batch = batch_obj

        def run_all():
            for i in indices:
                compiled.run(batch_obj, i, 1)
        run_all()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            run_all()
        g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps / len(indices) * 1000.0

    def table(batch_obj, tokens, keys_per_row, cache_rows):
        out = []
        # the same record of different layers is timed together; layers may differ in kind (two mixers in turn)
        members: Dict[tuple, List[int]] = {}
        for idx in per_layer:
            seen: Dict[str, int] = {}
            for i in idx:
                label, _, _ = record_cost(plan.ops[i], tokens, keys_per_row, cache_rows)
                seen[label] = seen.get(label, 0) + 1
                members.setdefault((label, seen[label]), []).append(i)
        for (label, _), which in members.items():
            _, fl, by = record_cost(plan.ops[which[0]], tokens, keys_per_row, cache_rows)
            us = measure(which, batch_obj)
            ideal = max(fl / (pk["bf16_tflops"] * 1e12), by / (pk["hbm_gbs"] * 1e9)) * 1e6
            out.append({"record": label, "us": round(us, 2), "ideal_us": round(ideal, 2),
                        "of_roofline": round(ideal / us, 3) if us > 0 else None, "layers": len(which)})
        return out

    dec = eng._build_batch([StepEntry(n, [5], [0]) for n in names], [CACHED] * batch)
    eng.cache.flush()
    result = {"decode": table(dec, batch, CACHED + 1, batch * (CACHED + 1))}
    eng.cache.add_request("prefill")
    eng.cache.reserve("prefill", T)
    pre = eng._build_batch([StepEntry("prefill", torch.randint(0, V, (T,), generator=gen).tolist(), [T - 1])], [0])
    eng.cache.flush()
    result["prefill"] = table(pre, T, (T + 1) / 2, T)
    eng.check_kernels()
    return result


def throughput(cfg, batches, page: int, steps: int, warmup: int) -> Dict[str, Any]:
    import torch

    from . import LLM, SamplingParams
    from .config import EngineConfig
    from .engine.engine import StepEntry

    context = CACHED + 256
    ec = EngineConfig(dtype="bfloat16", page_size=page, max_cached_tokens=max(batches) * context, max_num_seqs=max(batches),
                      max_num_batched_tokens=PROMPT, prefill_chunk=PROMPT, max_model_len=context, use_cuda_graphs=True)
    llm = LLM(config=cfg, random_seed=0, engine_config=ec)
    eng = llm.engine
    gen = torch.Generator().manual_seed(0)
    V = _vocab(cfg)
    greedy = SamplingParams(greedy=True)
    out: Dict[str, Any] = {}
    prompt = torch.randint(0, V, (PROMPT,), generator=gen).tolist()
    times = []
    for i in range(3 + 10):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.step([StepEntry(f"p{i}", prompt, [PROMPT - 1])], end=[f"p{i}"])
        b.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append(a.elapsed_time(b))
    ms = statistics.median(times)
    out["prefill"] = {"tokens": PROMPT, "ms": round(ms, 3), "tokens_per_s": round(PROMPT * 1000.0 / ms, 1)}
    for batch in batches:
        names = [f"d{batch}_{i}" for i in range(batch)]
        for n in names:
            eng.step([StepEntry(n, torch.randint(0, V, (CACHED,), generator=gen).tolist(), [])])

        def one():
            logits = eng.step([StepEntry(n, [7], [0]) for n in names])
            llm.sampler.sample(logits, [greedy] * batch, [0] * batch)
        for _ in range(warmup):
            one()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            one()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / steps
        out[f"decode_b{batch}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(batch * 1000.0 / ms, 1)}
        for n in names:
            eng.free(n)
    eng.check_kernels()
    return out


def run(args, pk) -> int:
    import gc

    import torch
    design_name = getattr(args, "design", None) or "bepuzen"
    table_of_sizes = {"bepuzen": SIZES, "torisun": TORISUN_SIZES, "vifelix": VIFELIX_SIZES, "funevik": FUNEVIK_SIZES}[design_name]
    global FP32_SHARE
    FP32_SHARE = pk["bf16_tflops"] / FP32_TFLOPS
    sizes = [args.size] if getattr(args, "size", None) else list(table_of_sizes)
    rec: Dict[str, Any] = {"metric": f"{design_name.capitalize()} beside the grouped-query model of equal size, bf16: tokens/s and per-record rooflines",
                           "unit": "tokens/s", "n_gpus": 1, "dtype": "bf16", "data": "synthetic token ids, random weights",
                           "peaks": pk["source"], "page_size": args.page_size, "cached_tokens": CACHED, "sizes": {}}
    for name in sizes:
        layers, design, closest = table_of_sizes[name]
        entry: Dict[str, Any] = {"layers": layers}
        for label, cfg in ((design_name, design), ("gqa", closest)):
            entry[label] = throughput(cfg, [1, 8, 64], args.page_size, min(args.steps, 32), max(3, args.warmup))
            gc.collect()
            torch.cuda.empty_cache()
            entry[label]["records"] = layer_table(cfg, layers, args.batch, args.page_size, pk)
            gc.collect()
            torch.cuda.empty_cache()
        rec["sizes"][name] = entry
    first = rec["sizes"][sizes[0]]
    rec["value"] = first[design_name][f"decode_b{8}"]["tokens_per_s"]
    print(json.dumps(rec))
    return 0
