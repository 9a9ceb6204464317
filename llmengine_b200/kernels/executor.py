"""Python face of the native step executor (include/llmengine_b200/executor.h): the ctypes mirror of its records
and the compilation of a `Plan` (engine/plan.py) into them."""
from __future__ import annotations

import ctypes
from ctypes import CFUNCTYPE, POINTER, Structure, byref, c_char_p, c_float, c_int, c_longlong, c_size_t, c_void_p
from typing import Any, Callable, Dict, List, Optional

import torch

MAX_GROUPS = 32
F32, BF16 = 0, 1
ROWS = {"tokens": 0, "logits": 1}
(OP_EMBEDDING, OP_RMSNORM, OP_LINEAR, OP_LINEAR_SWIGLU, OP_QKV_POST, OP_ATTEND, OP_ATTENTION, OP_CALL, OP_LINEAR_ACT,
 OP_POINTWISE, OP_BATCHED_LINEAR, OP_RESIDUAL_ADD, OP_LATENT_ATTENTION, OP_TOKEN_SIDE, OP_POSTNORM, OP_WINDOW_ATTENTION,
 OP_MOE_ROUTE, OP_GROUPED_LINEAR, OP_MOE_COMBINE, OP_SHORT_CONV, OP_ROTATE, OP_RECURRENCE, OP_GATED_NORM, OP_ROW_NORM,
 OP_EXP_GATES) = range(1, 26)
GATES = {"silu": 0, "clamped_swish": 1, "gelu_tanh": 2}
ROUTING = {"sigmoid": 0, "softmax_chosen": 1}
ACTIVATIONS = {"xielu": 1}
POINTWISE = {"sigmoid_mul": 1}


def code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise TypeError(f"kernels take float32 or bfloat16 tensors, got {dt}")


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class StepGroup(Structure):
    _fields_ = [("block_tables", c_void_p), ("slot_mapping", c_void_p), ("max_blocks", c_int), ("page_size", c_int),
                ("window", c_int)]


class Step(Structure):
    _fields_ = [
        ("num_tokens", c_int), ("num_requests", c_int), ("num_logit_rows", c_int), ("num_decode", c_int),
        ("num_portion", c_int), ("max_portion_len", c_int), ("max_decode_ctx", c_int),
        ("token_ids", c_void_p), ("positions", c_void_p), ("token_request", c_void_p), ("cu_q_lens", c_void_p),
        ("ctx_lens", c_void_p), ("state_slots", c_void_p), ("first_portion", c_void_p), ("logit_rows", c_void_p),
        ("decode_rows", c_void_p), ("portion_rows", c_void_p), ("logits", c_void_p), ("blas", c_void_p),
        ("num_groups", c_int), ("groups", StepGroup * MAX_GROUPS),
    ]


CallFn = CFUNCTYPE(c_int, c_void_p, POINTER(Step), c_void_p)


class EmbeddingOp(Structure):
    _fields_ = [("table", c_void_p), ("table_dtype", c_int), ("vocab", c_int), ("hidden", c_int), ("out", c_void_p),
                ("scale", c_float)]


class RmsNormOp(Structure):
    _fields_ = [("x", c_void_p), ("delta", c_void_p), ("delta_dtype", c_int), ("gain", c_void_p), ("gain_dtype", c_int),
                ("out", c_void_p), ("out_dtype", c_int), ("size", c_int), ("eps", c_float), ("rows", c_int), ("gain2", c_void_p),
                ("out2", c_void_p)]


class LinearOp(Structure):
    _fields_ = [("x", c_void_p), ("ldx", c_longlong), ("x_dtype", c_int), ("w", c_void_p), ("ldw", c_longlong),
                ("w_dtype", c_int), ("out", c_void_p), ("ldo", c_longlong), ("out_dtype", c_int), ("n", c_int), ("k", c_int),
                ("rows", c_int), ("bias", c_void_p)]


class LinearSwigluOp(Structure):
    _fields_ = [("x", c_void_p), ("ldx", c_longlong), ("dtype", c_int), ("w_gate_up", c_void_p), ("ldw", c_longlong),
                ("gate_up", c_void_p), ("out", c_void_p), ("ldo", c_longlong), ("inter", c_int), ("k", c_int),
                ("act", c_int), ("p0", c_float), ("p1", c_float), ("bias", c_void_p)]


class QkvPostOp(Structure):
    _fields_ = [("q_in", c_void_p), ("k_in", c_void_p), ("v_in", c_void_p), ("q_stride", c_longlong), ("k_stride", c_longlong),
                ("v_stride", c_longlong), ("in_dtype", c_int), ("q_gain", c_void_p), ("k_gain", c_void_p), ("gain_dtype", c_int),
                ("eps", c_float), ("cos_sin", c_void_p), ("max_positions", c_int), ("q_out", c_void_p), ("k_out", c_void_p),
                ("out_dtype", c_int), ("cache", c_void_p), ("group", c_int), ("nh", c_int), ("nkv", c_int), ("hd", c_int)]


class AttendOp(Structure):
    _fields_ = [("q", c_void_p), ("out", c_void_p), ("dtype", c_int), ("cache", c_void_p), ("cache_rows", c_longlong),
                ("group", c_int), ("nh", c_int), ("nkv", c_int), ("hd", c_int), ("window", c_int), ("scale", c_float),
                ("scratch", c_void_p), ("scratch_floats", c_longlong)]


class AttentionOp(Structure):
    _fields_ = [("post", QkvPostOp), ("attend", AttendOp), ("qkv", c_void_p), ("qkv_stride", c_longlong), ("rotary", c_int)]


class CallOp(Structure):
    _fields_ = [("fn", CallFn), ("user", c_void_p)]


class LinearActOp(Structure):
    _fields_ = [("product", LinearOp), ("out", c_void_p), ("ldo", c_longlong), ("act", c_int), ("p0", c_float), ("p1", c_float)]


class PointwiseOp(Structure):
    _fields_ = [("what", c_int), ("dtype", c_int), ("cols", c_int), ("a", c_void_p), ("lda", c_longlong), ("b", c_void_p),
                ("ldb", c_longlong), ("out", c_void_p), ("ldo", c_longlong), ("scale", c_float), ("group", c_int)]


class BatchedLinearOp(Structure):
    _fields_ = [("x", c_void_p), ("ldx", c_longlong), ("x_member", c_longlong), ("x_dtype", c_int),
                ("w", c_void_p), ("ldw", c_longlong), ("w_member", c_longlong), ("w_dtype", c_int),
                ("out", c_void_p), ("ldo", c_longlong), ("out_member", c_longlong), ("out_dtype", c_int),
                ("batch", c_int), ("n", c_int), ("k", c_int)]


class ResidualAddOp(Structure):
    _fields_ = [("x", c_void_p), ("a", c_void_p), ("b", c_void_p), ("dtype", c_int), ("size", c_int), ("a_scale", c_void_p),
                ("b_scale", c_void_p)]


class LatentAttentionOp(Structure):
    _fields_ = [("kv_in", c_void_p), ("kv_stride", c_longlong), ("q_rot", c_void_p), ("q_rot_stride", c_longlong),
                ("q_rot_head_stride", c_longlong), ("c_gain", c_void_p), ("gain_dtype", c_int), ("eps", c_float),
                ("inv_freq", c_void_p), ("rot_dims", c_int), ("q", c_void_p), ("out", c_void_p), ("dtype", c_int),
                ("cache", c_void_p), ("cache_rows", c_longlong), ("group", c_int), ("nh", c_int), ("rank", c_int), ("rot", c_int),
                ("scale", c_float), ("sink", c_void_p), ("scratch", c_void_p), ("scratch_floats", c_longlong), ("window", c_int),
                ("interleaved", c_int)]


class TokenSideOp(Structure):
    _fields_ = [("x", c_void_p), ("a", c_void_p), ("b", c_void_p), ("ab_dtype", c_int), ("size", c_int),
                ("table", c_void_p), ("table_dtype", c_int), ("ld_table", c_longlong), ("offset", c_int), ("dim", c_int),
                ("vocab", c_int), ("w_gate", c_void_p), ("w_proj", c_void_p), ("w_dtype", c_int), ("gain", c_void_p),
                ("gain_dtype", c_int), ("eps", c_float), ("xb", c_void_p), ("g", c_void_p), ("act_dtype", c_int), ("y", c_void_p)]


class PostNormOp(Structure):
    _fields_ = [("x", c_void_p), ("y", c_void_p), ("y_dtype", c_int), ("gain", c_void_p), ("gain_dtype", c_int), ("eps", c_float),
                ("copy", c_void_p), ("copy_dtype", c_int), ("size", c_int), ("accumulate", c_int)]


class WindowAttentionOp(Structure):
    _fields_ = [("q_in", c_void_p), ("k_in", c_void_p), ("v_in", c_void_p), ("q_stride", c_longlong), ("k_stride", c_longlong),
                ("v_stride", c_longlong), ("dtype", c_int), ("q_gain", c_void_p), ("k_gain", c_void_p), ("eps", c_float),
                ("inv_freq", c_void_p), ("rot_dims", c_int), ("amplitude", c_float), ("q", c_void_p), ("out", c_void_p),
                ("cache", c_void_p), ("group", c_int), ("nh", c_int), ("nkv", c_int), ("dk", c_int), ("dv", c_int),
                ("window", c_int), ("keep_first", c_int), ("scale", c_float), ("sink", c_void_p), ("scratch", c_void_p),
                ("scratch_floats", c_longlong), ("q_bias", c_void_p), ("k_bias", c_void_p), ("v_bias", c_void_p),
                ("head_norm", c_int), ("softcap", c_float), ("interleaved", c_int), ("in_f32", c_int)]


class MoeRouteOp(Structure):
    _fields_ = [("logits", c_void_p), ("ld", c_longlong), ("num_experts", c_int), ("top_k", c_int), ("scale", c_float),
                ("experts", c_void_p), ("weights", c_void_p), ("offsets", c_void_p), ("order", c_void_p), ("counts", c_void_p),
                ("mode", c_int)]


class GroupedLinearOp(Structure):
    _fields_ = [("x", c_void_p), ("ldx", c_longlong), ("x_dtype", c_int), ("w", c_void_p), ("ldw", c_longlong),
                ("w_expert", c_longlong), ("w_dtype", c_int), ("out", c_void_p), ("ldo", c_longlong), ("out_dtype", c_int),
                ("mid", c_void_p), ("ld_mid", c_longlong), ("offsets", c_void_p), ("order", c_void_p), ("num_experts", c_int),
                ("top_k", c_int), ("n", c_int), ("k", c_int), ("gather", c_int), ("scatter", c_int), ("act", c_int)]


class MoeCombineOp(Structure):
    _fields_ = [("y", c_void_p), ("ldy", c_longlong), ("weights", c_void_p), ("base", c_void_p), ("out", c_void_p),
                ("top_k", c_int), ("size", c_int), ("base_gate", c_void_p), ("ld_gate", c_longlong)]


class ShortConvOp(Structure):
    _fields_ = [("x", c_void_p), ("ldx", c_longlong), ("x_dtype", c_int), ("w", c_void_p), ("bias", c_void_p),
                ("state", c_void_p), ("state_stride", c_longlong), ("out", c_void_p), ("ldo", c_longlong),
                ("channels", c_int), ("taps", c_int), ("act", c_int)]


class RotateOp(Structure):
    _fields_ = [("x", c_void_p * 2), ("ldx", c_longlong * 2), ("out", c_void_p * 2), ("ldo", c_longlong * 2), ("heads", c_int * 2),
                ("scale", c_float * 2), ("dtype", c_int), ("dim", c_int), ("rot_dims", c_int), ("inv_freq", c_void_p)]


class RecurrenceOp(Structure):
    _fields_ = [("q", c_void_p), ("k", c_void_p), ("ldq", c_longlong), ("ldk", c_longlong), ("qk_groups", c_int),
                ("v", c_void_p), ("ldv", c_longlong), ("v_dtype", c_int), ("gate", c_int), ("decay", c_void_p),
                ("dt", c_void_p), ("lddt", c_longlong), ("dt_dtype", c_int), ("dt_bias", c_void_p), ("a_log", c_void_p),
                ("skip", c_void_p), ("state", c_void_p), ("state_stride", c_longlong), ("out", c_void_p), ("ldo", c_longlong),
                ("heads", c_int), ("n", c_int), ("p", c_int), ("scratch", c_void_p), ("scratch_floats", c_longlong),
                ("keep", c_void_p), ("take", c_void_p), ("ld_gates", c_longlong), ("unit_column", c_int)]


class GatedNormOp(Structure):
    _fields_ = [("y", c_void_p), ("ldy", c_longlong), ("gate", c_void_p), ("ldg", c_longlong), ("weight", c_void_p),
                ("out", c_void_p), ("ldo", c_longlong), ("dtype", c_int), ("cols", c_int), ("group", c_int),
                ("gate_first", c_int), ("eps", c_float), ("scale", c_float), ("gate_act", c_int), ("floor", c_void_p),
                ("ld_floor", c_longlong), ("den_eps", c_float)]


class RowNormOp(Structure):
    _fields_ = [("x", c_void_p), ("ldx", c_longlong), ("x_dtype", c_int), ("gain", c_void_p), ("gain_dtype", c_int),
                ("out", c_void_p), ("ldo", c_longlong), ("out_dtype", c_int), ("cols", c_int), ("eps", c_float)]


class ExpGatesOp(Structure):
    _fields_ = [("i_pre", c_void_p), ("f_pre", c_void_p), ("ld_pre", c_longlong), ("cap", c_float), ("state", c_void_p),
                ("state_stride", c_longlong), ("keep", c_void_p), ("take", c_void_p), ("floor", c_void_p), ("ld_out", c_longlong),
                ("heads", c_int)]


def _f32(t, n=None) -> bool:
    return t is None or (t.dtype == torch.float32 and t.is_contiguous() and (n is None or t.numel() == n))


def _state(t) -> bool:
    """A 32-bit state [slots, ...]: every slot's part is dense; the slots may lie apart (several states share a row)."""
    return t.dtype == torch.float32 and t[0].is_contiguous()


def declare(lib: ctypes.CDLL) -> None:
    lib.llme_executor_create.restype = c_void_p
    lib.llme_executor_create.argtypes = [c_int]
    lib.llme_executor_destroy.argtypes = [c_void_p]
    lib.llme_executor_register.argtypes = [c_void_p, c_char_p, c_void_p]
    lib.llme_executor_choose.argtypes = [c_void_p, c_char_p, c_char_p]
    lib.llme_executor_chosen.restype = c_char_p
    lib.llme_executor_chosen.argtypes = [c_void_p, c_char_p]
    lib.llme_executor_error.restype = c_char_p
    lib.llme_executor_error.argtypes = [c_void_p]
    lib.llme_executor_launches.restype = c_longlong
    lib.llme_executor_launches.argtypes = [c_void_p]
    lib.llme_attention_scratch_floats.restype = c_longlong
    lib.llme_attention_scratch_floats.argtypes = [c_void_p, c_int, c_int, c_int, c_int]
    lib.llme_latent_scratch_floats.restype = c_longlong
    lib.llme_latent_scratch_floats.argtypes = [c_void_p, c_int, c_int]
    lib.llme_decode_splits.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int]
    lib.llme_plan_create.restype = c_void_p
    lib.llme_plan_create.argtypes = [c_void_p]
    lib.llme_plan_destroy.argtypes = [c_void_p]
    lib.llme_plan_add.argtypes = [c_void_p, c_int, c_void_p, c_size_t]
    lib.llme_plan_size.argtypes = [c_void_p]
    lib.llme_plan_run.argtypes = [c_void_p, POINTER(Step), c_int, c_int, c_void_p]


def _qkv_post_record(a: Dict[str, Any]) -> QkvPostOp:
    q_in, k_in, v_in = a.get("q_in"), a.get("k_in"), a.get("v_in")
    ref = q_in if q_in is not None else (k_in if k_in is not None else v_in)
    outs = [t for t in (a.get("q_out"), a.get("k_out"), a.get("cache")) if t is not None]
    if ref is None or not outs:
        raise ValueError("qkv_post: nothing to read or nothing to write")
    for t in (q_in, k_in, v_in):
        assert t is None or (t.dtype == ref.dtype and t.stride(-1) == 1)
    assert all(t.dtype == outs[0].dtype for t in outs)
    gains = [g for g in (a.get("q_gain"), a.get("k_gain")) if g is not None]
    assert all(g.dtype == gains[0].dtype for g in gains)
    cs = a.get("cos_sin")
    return QkvPostOp(ptr(q_in), ptr(k_in), ptr(v_in), q_in.stride(0) if q_in is not None else 0,
                     k_in.stride(0) if k_in is not None else 0, v_in.stride(0) if v_in is not None else 0, code(ref.dtype),
                     ptr(a.get("q_gain")), ptr(a.get("k_gain")), code(gains[0].dtype) if gains else 0, a.get("eps", 0.0),
                     ptr(cs), cs.shape[0] if cs is not None else 0, ptr(a.get("q_out")), ptr(a.get("k_out")),
                     code(outs[0].dtype), ptr(a.get("cache")), a.get("group") or 0, a["num_heads"], a["num_kv_heads"],
                     a["head_dim"])


def _attend_record(a: Dict[str, Any]) -> AttendOp:
    q, out, cache = a["q"], a["out"], a["cache"]
    assert q.dtype == cache.dtype == out.dtype and q.is_contiguous() and out.is_contiguous() and cache.is_contiguous()
    scratch = a.get("scratch")
    rows = 1
    for d in cache.shape[:-1]:
        rows *= int(d)
    return AttendOp(q.data_ptr(), out.data_ptr(), code(q.dtype), cache.data_ptr(), rows, a["group"], a["num_heads"],
                    a["num_kv_heads"], a["head_dim"], a["window"], a["scale"], ptr(scratch),
                    scratch.numel() if scratch is not None else 0)


def records(op, keep: List[Any]):
    """(kind, ctypes record) of one plan operation; `keep` collects what must stay alive with the plan."""
    a = op.a
    keep.extend(v for v in a.values() if isinstance(v, torch.Tensor))
    k = op.kind
    if k == "embedding":
        t, out = a["table"], a["out"]
        assert out.dtype == torch.float32 and t.is_contiguous() and out.is_contiguous()
        return OP_EMBEDDING, EmbeddingOp(t.data_ptr(), code(t.dtype), t.shape[0], t.shape[1], out.data_ptr(), float(a.get("scale", 1.0)))
    if k == "rmsnorm":
        x, d, g, out = a["x"], a["delta"], a["gain"], a["out"]
        assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and (d is None or d.is_contiguous())
        g2, out2 = a.get("gain2"), a.get("out2")
        assert (g2 is None) == (out2 is None) and (g2 is None or (g2.dtype == g.dtype and g2.is_contiguous() and g2.numel() == g.numel()
                                                                  and out2.dtype == out.dtype and out2.is_contiguous() and out2.shape == out.shape))
        return OP_RMSNORM, RmsNormOp(x.data_ptr(), ptr(d), code(d.dtype) if d is not None else 0, g.data_ptr(), code(g.dtype),
                                     out.data_ptr(), code(out.dtype), x.shape[1], a["eps"], ROWS[a["rows"]], ptr(g2), ptr(out2))
    if k == "linear":
        x, w, out = a["x"], a["w"], a["out"]
        assert x.stride(1) == 1 and w.stride(1) == 1 and w.shape[1] == x.shape[1] and (out is None or out.stride(1) == 1)
        assert out is None or out.shape[1] == w.shape[0]
        assert _f32(a.get("bias"), w.shape[0])
        return OP_LINEAR, LinearOp(x.data_ptr(), x.stride(0), code(x.dtype), w.data_ptr(), w.stride(0), code(w.dtype), ptr(out),
                                   out.stride(0) if out is not None else 0, code(out.dtype) if out is not None else F32,
                                   w.shape[0], w.shape[1], ROWS[a["rows"]], ptr(a.get("bias")))
    if k == "linear_swiglu":
        x, w, gu, out = a["x"], a["w_gate_up"], a["gate_up"], a["out"]
        assert x.dtype == w.dtype == out.dtype and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
        assert w.shape[0] == 2 * out.shape[1] and w.shape[1] == x.shape[1]
        p = a.get("params", ())
        assert _f32(a.get("bias"), w.shape[0])
        return OP_LINEAR_SWIGLU, LinearSwigluOp(x.data_ptr(), x.stride(0), code(x.dtype), w.data_ptr(), w.stride(0), ptr(gu),
                                                out.data_ptr(), out.stride(0), out.shape[1], x.shape[1], GATES[a.get("act", "silu")],
                                                p[0] if p else 0.0, p[1] if len(p) > 1 else 0.0, ptr(a.get("bias")))
    if k == "qkv_post":
        return OP_QKV_POST, _qkv_post_record(a)
    if k == "attend":
        return OP_ATTEND, _attend_record(a)
    if k == "attention":
        qkv, nh, nkv, hd = a["qkv"], a["num_heads"], a["num_kv_heads"], a["head_dim"]
        qs, kvs = nh * hd, nkv * hd
        writes = a["writes"]
        assert qkv.stride(1) == 1 and qkv.shape[1] == (qs + 2 * kvs if writes else qs)
        post = _qkv_post_record(dict(q_in=qkv[:, :qs], k_in=qkv[:, qs:qs + kvs] if writes else None,
                                     v_in=qkv[:, qs + kvs:] if writes else None, q_gain=a.get("q_gain"), k_gain=a.get("k_gain"),
                                     eps=a.get("eps", 0.0), cos_sin=a.get("cos_sin"), q_out=a["q"],
                                     cache=a["cache"] if writes else None, group=a["group"], num_heads=nh, num_kv_heads=nkv,
                                     head_dim=hd))
        return OP_ATTENTION, AttentionOp(post, _attend_record(a), qkv.data_ptr(), qkv.stride(0),
                                         1 if a.get("cos_sin") is not None else 0)
    if k == "linear_act":
        x, w, mid, out = a["x"], a["w"], a["mid"], a["out"]
        assert x.stride(1) == 1 and w.stride(1) == 1 and mid.stride(1) == 1 and out.stride(1) == 1 and w.shape[1] == x.shape[1]
        assert mid.shape[1] == out.shape[1] == w.shape[0] and mid.dtype == out.dtype
        p = a["params"]
        lin = LinearOp(x.data_ptr(), x.stride(0), code(x.dtype), w.data_ptr(), w.stride(0), code(w.dtype), mid.data_ptr(),
                       mid.stride(0), code(mid.dtype), w.shape[0], w.shape[1], ROWS["tokens"])
        return OP_LINEAR_ACT, LinearActOp(lin, out.data_ptr(), out.stride(0), ACTIVATIONS[a["act"]], p[0] if p else 0.0,
                                          p[1] if len(p) > 1 else 0.0)
    if k == "pointwise":
        x, b, out = a["a"], a["b"], a["out"]
        assert x.stride(1) == 1 and out.stride(1) == 1 and (b is None or (b.stride(1) == 1 and b.dtype == x.dtype)) and out.dtype == x.dtype
        group = int(a.get("group", 1))
        assert group >= 1 and out.shape[1] % group == 0 and (b is None or b.shape[1] * group == out.shape[1])
        return OP_POINTWISE, PointwiseOp(POINTWISE[a["what"]], code(x.dtype), out.shape[1], x.data_ptr(), x.stride(0), ptr(b),
                                         b.stride(0) if b is not None else 0, out.data_ptr(), out.stride(0), float(a.get("scale", 1.0)), group)
    if k == "batched_linear":
        x, w, out = a["x"], a["w"], a["out"]
        assert x.dim() == 3 and w.dim() == 3 and out.dim() == 3 and x.stride(2) == 1 and out.stride(2) == 1 and w.is_contiguous()
        assert x.shape[1] == w.shape[0] == out.shape[1] and x.shape[2] == w.shape[2] and out.shape[2] == w.shape[1]
        return OP_BATCHED_LINEAR, BatchedLinearOp(x.data_ptr(), x.stride(0), x.stride(1), code(x.dtype), w.data_ptr(), w.stride(1),
                                                  w.stride(0), code(w.dtype), out.data_ptr(), out.stride(0), out.stride(1),
                                                  code(out.dtype), w.shape[0], w.shape[1], w.shape[2])
    if k == "residual_add":
        x, u, v = a["x"], a["a"], a["b"]
        assert x.dtype == torch.float32 and x.is_contiguous() and u.is_contiguous() and u.shape == x.shape
        assert v is None or (v.is_contiguous() and v.dtype == u.dtype and v.shape == x.shape)
        assert _f32(a.get("a_scale"), x.shape[1]) and _f32(a.get("b_scale"), x.shape[1])
        return OP_RESIDUAL_ADD, ResidualAddOp(x.data_ptr(), u.data_ptr(), ptr(v), code(u.dtype), x.shape[1], ptr(a.get("a_scale")),
                                              ptr(a.get("b_scale")))
    if k == "latent_attention":
        q, out, cache, kv, qr, gain = a["q"], a["out"], a["cache"], a["kv_in"], a["q_rot"], a["c_gain"]
        H, r, dr = a["num_heads"], a["kv_rank"], a["rot_dim"]
        assert q.dtype == out.dtype == cache.dtype == kv.dtype and q.is_contiguous() and out.is_contiguous() and cache.is_contiguous()
        assert q.shape[1] == H * (r + dr) and out.shape[1] == H * r and cache.shape[-1] == r + dr and kv.stride(1) == 1
        assert (qr is None) == (dr == 0) and (qr is None or (qr.dtype == q.dtype and qr.stride(2) == 1 and tuple(qr.shape[1:]) == (H, dr)))
        freq, sink, scratch = a["inv_freq"], a["sink"], a.get("scratch")
        assert freq is None or (freq.dtype == torch.float32 and freq.numel() * 2 == a["rot_dims"])
        assert sink is None or (sink.dtype == torch.float32 and sink.numel() == H)
        return OP_LATENT_ATTENTION, LatentAttentionOp(
            kv.data_ptr(), kv.stride(0), ptr(qr), qr.stride(0) if qr is not None else 0, qr.stride(1) if qr is not None else 0,
            gain.data_ptr(), code(gain.dtype), a["eps"], ptr(freq), a["rot_dims"], q.data_ptr(), out.data_ptr(), code(q.dtype),
            cache.data_ptr(), cache.shape[0] * cache.shape[1], a["group"], H, r, dr, a["scale"], ptr(sink), ptr(scratch),
            scratch.numel() if scratch is not None else 0, int(a.get("window", 0)), 1 if a.get("interleaved") else 0)
    if k == "token_side":
        x, u, v, table, wg, wp, gain, xb, g, y = (a[n] for n in ("x", "a", "b", "table", "w_gate", "w_proj", "gain", "xb", "g", "y"))
        D, dim = x.shape[1], a["dim"]
        assert x.dtype == y.dtype == torch.float32 and all(t.is_contiguous() for t in (x, u, table, wg, wp, gain, xb, g, y))
        assert v is None or (v.is_contiguous() and v.dtype == u.dtype)
        assert tuple(wg.shape) == (dim, D) and tuple(wp.shape) == (D, dim) and wg.dtype == wp.dtype and xb.dtype == g.dtype == table.dtype
        assert xb.shape[1] == D and g.shape[1] == dim and y.shape[1] == D and gain.numel() == D
        return OP_TOKEN_SIDE, TokenSideOp(x.data_ptr(), u.data_ptr(), ptr(v), code(u.dtype), D, table.data_ptr(), code(table.dtype),
                                          table.stride(0), a["offset"], dim, table.shape[0], wg.data_ptr(), wp.data_ptr(),
                                          code(wg.dtype), gain.data_ptr(), code(gain.dtype), a["eps"], xb.data_ptr(), g.data_ptr(),
                                          code(g.dtype), y.data_ptr())
    if k == "postnorm":
        x, y, g, c = a["x"], a["y"], a["gain"], a["copy"]
        assert x.dtype == torch.float32 and x.is_contiguous() and (y is None or (y.is_contiguous() and y.shape[1] == x.shape[1]))
        assert (y is None) == (g is None) and (c is None or (c.is_contiguous() and c.shape[1] == x.shape[1])) and (y is not None or c is not None)
        return OP_POSTNORM, PostNormOp(x.data_ptr(), ptr(y), code(y.dtype) if y is not None else 0, ptr(g),
                                       code(g.dtype) if g is not None else 0, a["eps"], ptr(c), code(c.dtype) if c is not None else 0,
                                       x.shape[1], 1 if a["accumulate"] else 0)
    if k == "window_attention":
        qi, ki, vi, q, out, cache = a["q_in"], a["k_in"], a["v_in"], a["q"], a["out"], a["cache"]
        H, G, dk, dv = a["num_heads"], a["num_kv_heads"], a["qk_dim"], a["v_dim"]
        wide = qi.dtype == torch.float32 and q.dtype != torch.float32       # 32-bit projections (from a convolution)
        assert q.dtype == out.dtype == cache.dtype and (wide or qi.dtype == q.dtype) and qi.stride(1) == 1 and q.is_contiguous() and out.is_contiguous()
        assert cache.is_contiguous() and qi.shape[1] == q.shape[1] == H * dk and out.shape[1] == H * dv and cache.shape[1] % (G * (dk + dv)) == 0
        assert (ki is None) == (vi is None) and (ki is None or (ki.dtype == vi.dtype == qi.dtype and ki.stride(1) == vi.stride(1) == 1
                                                              and ki.shape[1] == G * dk and vi.shape[1] == G * dv))
        per_head = bool(a.get("head_norm"))
        for t, n in ((a["q_gain"], dk if per_head else H * dk), (a["k_gain"], dk if per_head else G * dk), (a["sink"], H),
                     (a["inv_freq"], a["rot_dims"] // 2), (a.get("q_bias"), H * dk), (a.get("k_bias"), G * dk), (a.get("v_bias"), G * dv)):
            assert t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == n)
        return OP_WINDOW_ATTENTION, WindowAttentionOp(
            qi.data_ptr(), ptr(ki), ptr(vi), qi.stride(0), ki.stride(0) if ki is not None else 0, vi.stride(0) if vi is not None else 0,
            code(q.dtype), ptr(a["q_gain"]), ptr(a["k_gain"]), a["eps"], ptr(a["inv_freq"]), a["rot_dims"], a["amplitude"],
            q.data_ptr(), out.data_ptr(), cache.data_ptr(), a["group"], H, G, dk, dv, a["window"], a["keep_first"], a["scale"],
            ptr(a["sink"]), ptr(a.get("scratch")), a["scratch"].numel() if a.get("scratch") is not None else 0,
            ptr(a.get("q_bias")), ptr(a.get("k_bias")), ptr(a.get("v_bias")), 1 if a.get("head_norm") else 0,
            float(a.get("softcap", 0.0)), 1 if a.get("interleaved") else 0, 1 if wide else 0)
    if k == "moe_route":
        z, ex_, wt, off, order, counts = a["logits"], a["experts"], a["weights"], a["offsets"], a["order"], a["counts"]
        assert z.dtype == wt.dtype == torch.float32 and z.stride(1) == 1 and ex_.is_contiguous() and wt.is_contiguous()
        assert all(t.dtype == torch.int32 and t.is_contiguous() for t in (ex_, off, order, counts))
        E, top = z.shape[1], a["top_k"]
        assert ex_.shape[1] == wt.shape[1] == top and off.numel() == E + 1 and counts.numel() == E and order.numel() >= ex_.shape[0] * top
        return OP_MOE_ROUTE, MoeRouteOp(z.data_ptr(), z.stride(0), E, top, a["scale"], ex_.data_ptr(), wt.data_ptr(), off.data_ptr(),
                                        order.data_ptr(), counts.data_ptr(), ROUTING[a.get("mode", "sigmoid")])
    if k == "grouped_linear":
        x, w, out, mid = a["x"], a["w"], a["out"], a["mid"]
        act = 1 if a["act"] else 0
        assert a["act"] in (None, "silu") and w.dim() == 3 and w.is_contiguous() and x.stride(1) == 1 and out.stride(1) == 1
        assert w.shape[2] == x.shape[1] and out.shape[1] == (w.shape[1] // 2 if act else w.shape[1]) and x.dtype == w.dtype
        return OP_GROUPED_LINEAR, GroupedLinearOp(
            x.data_ptr(), x.stride(0), code(x.dtype), w.data_ptr(), w.stride(1), w.stride(0), code(w.dtype), out.data_ptr(), out.stride(0),
            code(out.dtype), ptr(mid), mid.stride(0) if mid is not None else 0, a["offsets"].data_ptr(), a["order"].data_ptr(), w.shape[0],
            a["top_k"], w.shape[1], w.shape[2], 1 if a["gather"] else 0, 1 if a["scatter"] else 0, act)
    if k == "moe_combine":
        y, wt, base, out = a["y"], a["weights"], a["base"], a["out"]
        assert y.dtype == wt.dtype == out.dtype == torch.float32 and y.stride(1) == 1 and wt.is_contiguous() and out.is_contiguous()
        assert base is None or (base.dtype == torch.float32 and base.is_contiguous() and base.shape[1] == out.shape[1])
        bg = a.get("base_gate")
        assert bg is None or (base is not None and bg.dtype == torch.float32 and bg.dim() == 2 and bg.shape[1] == 1)
        return OP_MOE_COMBINE, MoeCombineOp(y.data_ptr(), y.stride(0), wt.data_ptr(), ptr(base), out.data_ptr(), wt.shape[1], out.shape[1],
                                            ptr(bg), bg.stride(0) if bg is not None else 0)
    if k == "short_conv":
        x, w, b, st, out = a["x"], a["w"], a["bias"], a["state"], a["out"]
        C, K = w.shape
        assert x.stride(1) == 1 and x.shape[1] == C and out.dtype == torch.float32 and out.stride(1) == 1 and out.shape[1] == C
        assert _f32(w) and _f32(b, C) and _state(st) and st.dim() == 3 and tuple(st.shape[1:]) == (max(K - 1, 1), C)
        return OP_SHORT_CONV, ShortConvOp(x.data_ptr(), x.stride(0), code(x.dtype), w.data_ptr(), ptr(b), st.data_ptr(), st.stride(0),
                                          out.data_ptr(), out.stride(0), C, K, 1 if a["act"] == "silu" else 0)
    if k == "rotate":
        xs, outs, heads, scales = a["x"], a["out"], a["heads"], a["scale"]
        ref = next(t for t in xs if t is not None)
        for t, o, h in zip(xs, outs, heads):
            assert t is None or (t.dtype == ref.dtype and t.stride(1) == 1 and o.dtype == torch.float32 and o.stride(1) == 1
                                 and t.shape[1] == o.shape[1] == h * a["dim"])
        assert _f32(a["inv_freq"], a["rot_dims"] // 2)
        A = lambda ty, v: (ty * 2)(*v)
        return OP_ROTATE, RotateOp(A(c_void_p, [ptr(t) for t in xs]), A(c_longlong, [t.stride(0) if t is not None else 0 for t in xs]),
                                   A(c_void_p, [ptr(t) for t in outs]), A(c_longlong, [t.stride(0) if t is not None else 0 for t in outs]),
                                   A(c_int, [int(h) for h in heads]), A(c_float, [float(v) for v in scales]), code(ref.dtype),
                                   a["dim"], a["rot_dims"], ptr(a["inv_freq"]))
    if k == "recurrence":
        q, kk, v, st, out = a["q"], a["k"], a["v"], a["state"], a["out"]
        H, n, p, G = a["heads"], a["n"], a["p"], a["qk_groups"]
        assert q.dtype == kk.dtype == out.dtype == torch.float32 and q.stride(1) == kk.stride(1) == v.stride(1) == out.stride(1) == 1
        unit = bool(a.get("unit_column"))
        assert q.shape[1] == kk.shape[1] == G * n and out.shape[1] == H * p and v.shape[1] == H * (p - 1 if unit else p) and H % G == 0
        keep, take = a.get("keep"), a.get("take")
        assert (keep is None) == (take is None) and (keep is None or a.get("dt") is None)
        for t in (keep, take):
            assert t is None or (t.dtype == torch.float32 and t.stride(1) == 1 and t.shape[1] == H and t.stride(0) == keep.stride(0))
        assert _state(st) and tuple(st.shape[1:]) == (H, p, n)
        dt, scratch = a.get("dt"), a.get("scratch")
        assert scratch is None or (scratch.dtype == torch.float32 and scratch.is_contiguous())
        assert dt is None or (dt.stride(1) == 1 and dt.shape[1] == H)
        for t in ("decay", "dt_bias", "a_log", "skip"):
            assert _f32(a.get(t), H)
        return OP_RECURRENCE, RecurrenceOp(q.data_ptr(), kk.data_ptr(), q.stride(0), kk.stride(0), G, v.data_ptr(), v.stride(0), code(v.dtype),
                                           2 if keep is not None else (0 if dt is None else 1), ptr(a.get("decay")), ptr(dt), dt.stride(0) if dt is not None else 0,
                                           code(dt.dtype) if dt is not None else 0, ptr(a.get("dt_bias")), ptr(a.get("a_log")),
                                           ptr(a.get("skip")), st.data_ptr(), st.stride(0), out.data_ptr(), out.stride(0), H, n, p,
                                           ptr(scratch), scratch.numel() if scratch is not None else 0, ptr(keep), ptr(take),
                                           keep.stride(0) if keep is not None else 0, 1 if unit else 0)
    if k == "gated_norm":
        y, g, w, out = a["y"], a["gate"], a["weight"], a["out"]
        cols, floor = out.shape[1], a.get("floor")
        assert y.dtype == torch.float32 and y.stride(1) == g.stride(1) == out.stride(1) == 1 and g.dtype == out.dtype
        assert g.shape[1] == cols and cols % a["group"] == 0 and _f32(w, cols)
        groups = cols // a["group"]
        assert y.shape[1] == (cols + groups if floor is not None else cols)
        assert floor is None or (floor.dtype == torch.float32 and floor.stride(1) == 1 and floor.shape[1] == groups)
        return OP_GATED_NORM, GatedNormOp(y.data_ptr(), y.stride(0), g.data_ptr(), g.stride(0), ptr(w), out.data_ptr(), out.stride(0),
                                          code(out.dtype), cols, a["group"], 1 if a["gate_first"] else 0, a["eps"], a["scale"],
                                          1 if a.get("gate_act", "silu") == "sigmoid" else 0, ptr(floor),
                                          floor.stride(0) if floor is not None else 0, float(a.get("den_eps", 0.0)))
    if k == "row_norm":
        x, g, out = a["x"], a["gain"], a["out"]
        assert x.stride(1) == 1 and out.stride(1) == 1 and x.shape[1] == out.shape[1] == g.numel() and g.is_contiguous()
        return OP_ROW_NORM, RowNormOp(x.data_ptr(), x.stride(0), code(x.dtype), g.data_ptr(), code(g.dtype), out.data_ptr(), out.stride(0),
                                      code(out.dtype), x.shape[1], a["eps"])
    if k == "exp_gates":
        ip, fp, st, keep, take, floor = a["i_pre"], a["f_pre"], a["state"], a["keep"], a["take"], a["floor"]
        H = ip.shape[1]
        for t in (ip, fp, keep, take, floor):
            assert t.dtype == torch.float32 and t.stride(1) == 1 and t.shape[1] == H
        assert ip.stride(0) == fp.stride(0) and keep.stride(0) == take.stride(0) == floor.stride(0)
        assert _state(st) and tuple(st.shape[1:]) == (H,)
        return OP_EXP_GATES, ExpGatesOp(ip.data_ptr(), fp.data_ptr(), ip.stride(0), a["cap"], st.data_ptr(), st.stride(0), keep.data_ptr(),
                                        take.data_ptr(), floor.data_ptr(), keep.stride(0), H)
    raise ValueError(f"the executor has no record for the operation {k!r}")
