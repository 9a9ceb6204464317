"""Typed configuration of the Funevik design, read from config.json.

The file lists the layers one by one: each entry names its mixer (`type`), the mixer's sizes and constants (`mixer`)
and its feed-forward (`mlp`, or null).  Nothing is assumed about their order, and no size or constant has a stand-in
in code: what a layer needs and the file lacks is an error that names the key.

    architecture     "Funevik"
    vocab, width     vocabulary and residual width
    norm.eps         eps of every RMS norm
    embedding.scale  the constant every embedded row is multiplied by
    layers[i].type   "mlstm" | "latent_attention" | "attention"
    layers[i].mixer  mlstm:            heads, dim, vdim, gate_cap
                     latent_attention: heads, dim (unrotated), rot_dim (rotated), vdim, kv_rank, q_rank, scale,
                                       rot.base, rot.dims, mask.size (may be absent: every earlier key)
                     attention:        heads, kv_heads, dim, vdim, scale, conv (taps), rot.base, rot.dims,
                                       softcap (may be absent), mask.size (may be absent)
    layers[i].mlp    null; kind "dense" with ff; kind "moe" with expert.ff, router.{experts, top} and optionally
                     shared.ff

A layer is x <- x + ls1 * mixer(norm1(x)) + ls2 * mlp(norm2(x)): both sublayers read the same x, each through a norm of
its own, and each result is multiplied by a learned vector.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple, Union

from .bepuzen import MAX_POSITIONS, _need, _pos_float, _pos_int
from .qwen3 import ConfigError
from .spec import LayerRun, LayerSpec, ModelSpec, PartSpec
from .vifelix import _number


@dataclass(frozen=True)
class MatrixMemoryConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class LatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    window: int                 # 0: every earlier key


@dataclass(frozen=True)
class ConvAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    taps: int
    rot_base: float
    rot_dims: int
    softcap: float              # 0: none
    window: int                 # 0: every earlier key


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                   # "dense" | "moe"
    ff: int                     # dense: its size; moe: the size of one expert
    experts: int = 0
    top: int = 0
    shared_ff: int = 0          # 0: no shared expert


MixerConfig = Union[MatrixMemoryConfig, LatentConfig, ConvAttentionConfig]


def _window(m: Mapping[str, Any], at: str) -> int:
    mask = m.get("mask")
    return 0 if mask is None else _pos_int(mask, "size", at + "mask.")


def _rot(m: Mapping[str, Any], at: str, most: int) -> Tuple[float, int]:
    rot = _need(m, "rot", at)
    base, dims = _pos_float(rot, "base", at + "rot."), _pos_int(rot, "dims", at + "rot.")
    if dims % 2 or dims > most:
        raise ConfigError(f"{at}rot.dims={dims} must be even and at most {most}")
    return base, dims


@dataclass(frozen=True)
class FunevikConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    embedding_scale: float
    mixers: Tuple[MixerConfig, ...]
    mlps: Tuple[Optional[FeedForwardConfig], ...]
    eos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    ARCHITECTURE = "Funevik"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "FunevikConfig":
        layers = _need(d, "layers", "")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config key 'layers' must be a non-empty list")
        eps = _pos_float(_need(d, "norm", ""), "eps", "norm.")
        mixers, mlps = [], []
        for i, L in enumerate(layers):
            at = f"layers[{i}]."
            kind = _need(L, "type", at)
            m = _need(L, "mixer", at)
            if kind == "mlstm":
                mixers.append(cls._memory(m, at + "mixer."))
            elif kind == "latent_attention":
                mixers.append(cls._latent(m, at + "mixer."))
            elif kind == "attention":
                mixers.append(cls._attention(m, at + "mixer."))
            else:
                raise ConfigError(f"{at}type={kind!r} is not a mixer of this design (mlstm, latent_attention, attention)")
            mlps.append(cls._mlp(L.get("mlp"), at + "mlp."))
        eos = d.get("eos_token_id")
        return cls(architecture=cls.ARCHITECTURE, vocab_size=_pos_int(d, "vocab", ""), hidden_size=_pos_int(d, "width", ""),
                   norm_eps=eps, embedding_scale=_number(_need(d, "embedding", ""), "scale", "embedding."),
                   mixers=tuple(mixers), mlps=tuple(mlps), eos_token_id=eos if isinstance(eos, int) else None,
                   torch_dtype=str(d.get("torch_dtype", "bfloat16")))

    @staticmethod
    def _memory(m: Mapping[str, Any], at: str) -> MatrixMemoryConfig:
        cap = _number(m, "gate_cap", at) if m.get("gate_cap") is not None else 0.0
        if cap < 0:
            raise ConfigError(f"{at}gate_cap={cap} must not be negative")
        return MatrixMemoryConfig(heads=_pos_int(m, "heads", at), dim=_pos_int(m, "dim", at), vdim=_pos_int(m, "vdim", at), gate_cap=cap)

    @staticmethod
    def _latent(m: Mapping[str, Any], at: str) -> LatentConfig:
        rot_dim = _pos_int(m, "rot_dim", at)
        base, dims = _rot(m, at, rot_dim)
        return LatentConfig(heads=_pos_int(m, "heads", at), dim=_pos_int(m, "dim", at), rot_dim=rot_dim, vdim=_pos_int(m, "vdim", at),
                            kv_rank=_pos_int(m, "kv_rank", at), q_rank=_pos_int(m, "q_rank", at), scale=_pos_float(m, "scale", at),
                            rot_base=base, rot_dims=dims, window=_window(m, at))

    @staticmethod
    def _attention(m: Mapping[str, Any], at: str) -> ConvAttentionConfig:
        dim = _pos_int(m, "dim", at)
        base, dims = _rot(m, at, dim)
        c = ConvAttentionConfig(heads=_pos_int(m, "heads", at), kv_heads=_pos_int(m, "kv_heads", at), dim=dim, vdim=_pos_int(m, "vdim", at),
                                scale=_pos_float(m, "scale", at), taps=_pos_int(m, "conv", at), rot_base=base, rot_dims=dims,
                                softcap=_pos_float(m, "softcap", at) if m.get("softcap") is not None else 0.0, window=_window(m, at))
        if c.heads % c.kv_heads:
            raise ConfigError(f"{at}heads={c.heads} must be a multiple of kv_heads={c.kv_heads}")
        return c

    @staticmethod
    def _mlp(mlp: Optional[Mapping[str, Any]], at: str) -> Optional[FeedForwardConfig]:
        if mlp is None:
            return None
        kind = _need(mlp, "kind", at)
        if kind == "dense":
            return FeedForwardConfig("dense", _pos_int(mlp, "ff", at))
        if kind == "moe":
            router = _need(mlp, "router", at)
            sh = mlp.get("shared")
            c = FeedForwardConfig("moe", _pos_int(_need(mlp, "expert", at), "ff", at + "expert."),
                                  experts=_pos_int(router, "experts", at + "router."), top=_pos_int(router, "top", at + "router."),
                                  shared_ff=_pos_int(sh, "ff", at + "shared.") if sh is not None else 0)
            if c.top > c.experts:
                raise ConfigError(f"{at}router.top={c.top} exceeds router.experts={c.experts}")
            return c
        raise ConfigError(f"{at}kind={kind!r} is not a feed-forward of this design (dense, moe)")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for m, f in zip(self.mixers, self.mlps):
            if isinstance(m, MatrixMemoryConfig):
                kind, mixer = "mlstm", {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "gate_cap": m.gate_cap}
            elif isinstance(m, LatentConfig):
                kind = "latent_attention"
                mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank, "q_rank": m.q_rank,
                         "scale": m.scale, "rot": {"base": m.rot_base, "dims": m.rot_dims}}
                if m.window:
                    mixer["mask"] = {"size": m.window}
            else:
                kind = "attention"
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale, "conv": m.taps,
                         "rot": {"base": m.rot_base, "dims": m.rot_dims}}
                if m.softcap:
                    mixer["softcap"] = m.softcap
                if m.window:
                    mixer["mask"] = {"size": m.window}
            if f is None:
                mlp = None
            elif f.kind == "dense":
                mlp = {"kind": "dense", "ff": f.ff}
            else:
                mlp = {"kind": "moe", "expert": {"ff": f.ff}, "router": {"experts": f.experts, "top": f.top}}
                if f.shared_ff:
                    mlp["shared"] = {"ff": f.shared_ff}
            layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                             "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale}, "layers": layers}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    # ------------------------------------------------------------------ the model as parts
    @property
    def num_hidden_layers(self) -> int:
        return len(self.mixers)

    def model_spec(self) -> ModelSpec:
        D, eps = self.hidden_size, self.norm_eps
        norm = PartSpec("rmsnorm", {"size": D, "eps": eps, "leaf": ""})
        block = PartSpec("parallel_residual", {
            "norm_name": "norm1", "feed_forward_norm_name": "norm2", "mixer_name": "mix", "feed_forward_name": "mlp",
            "mixer_scale_name": "ls1", "feed_forward_scale_name": "ls2", "hidden_size": D})
        layers = []
        for i, (m, f) in enumerate(zip(self.mixers, self.mlps)):
            if isinstance(m, MatrixMemoryConfig):
                mixer = PartSpec("matrix_memory", {"hidden_size": D, "num_heads": m.heads, "qk_dim": m.dim, "v_dim": m.vdim,
                                                   "gate_cap": m.gate_cap, "norm_eps": eps})
            elif isinstance(m, LatentConfig):
                mixer = PartSpec("latent_attention", {
                    "hidden_size": D, "num_heads": m.heads, "nope_dim": m.dim, "rot_dim": m.rot_dim, "v_dim": m.vdim,
                    "kv_rank": m.kv_rank, "q_rank": m.q_rank, "scale": m.scale, "norm_eps": eps, "sink": True, "window": m.window,
                    "position_encoding": PartSpec("rotary_partial", {"dims": m.rot_dims, "base": m.rot_base, "interleaved": True})})
            else:
                mixer = PartSpec("gqa_window_sink", {
                    "hidden_size": D, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "qk_dim": m.dim, "v_dim": m.vdim,
                    "scale": m.scale, "window": m.window, "conv_taps": m.taps, "softcap": m.softcap, "unit_sink": True,
                    "gate": "sigmoid_head",
                    "position_encoding": PartSpec("rotary_partial", {"dims": m.rot_dims, "base": m.rot_base, "interleaved": True})})
            parts = {"mixer": mixer, "norm": norm}
            if f is not None:
                parts["feed_forward_norm"] = norm
                if f.kind == "dense":
                    parts["feed_forward"] = PartSpec("gated_dense", {"hidden_size": D, "intermediate_size": f.ff, "activation": "gelu_tanh"})
                else:
                    parts["feed_forward"] = PartSpec("routed_experts", {
                        "hidden_size": D, "num_experts": f.experts, "top_k": f.top, "expert_size": f.ff, "shared_size": f.shared_ff,
                        "routing": "softmax_chosen", "router_bias": True, "shared_gate": bool(f.shared_ff)})
            layers.append(LayerSpec(prefix=f"l{i}", block=block, parts=parts))
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=D, vocab_size=self.vocab_size, max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": D, "leaf": "",
                                                   "scale": self.embedding_scale}),
            layers=tuple(layers), order=tuple(LayerRun(i) for i in range(len(layers))), final_norm=norm,
            lm_head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": D, "leaf": ""}),
            embedding_prefix="embed", final_norm_prefix="final.norm", lm_head_prefix="head")
        spec.validate()
        return spec

    @staticmethod
    def canonical_tensor_name(name: str) -> str:
        return name

    def ignorable_tensor(self, name: str) -> bool:
        """The norm and the scale vector stored for a feed-forward that the layer does not have."""
        return any(f is None and name in (f"l{i}.norm2", f"l{i}.ls2") for i, f in enumerate(self.mlps))
