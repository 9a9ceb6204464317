"""Typed configuration of the Vifelix design, read from config.json.

The file lists the layers one by one: each entry names its mixer (`type`), the mixer's sizes and constants
(`mixer`) and its feed-forward (`mlp`, or null).  Nothing is assumed about their order, and no size or
constant has a stand-in in code: what a layer needs and the file lacks is an error that names the key.

    architecture     "Vifelix"
    vocab, width     vocabulary and residual width
    norm.eps         eps of every RMS norm
    embedding.scale  the constant every embedded row is multiplied by
    layers[i].type   "mamba2" | "parallel"
    layers[i].mixer  mamba2:   heads, vdim (value size per head), state, groups, conv (taps), norm_groups
                     parallel: left_scale, right_scale, and
                       left  (softmax attention in a window): heads, kv_heads, dim, vdim, scale, mask.size,
                             rot.base, rot.dims
                       right (linear attention with a fixed decay per head): heads, dim, vdim, decay [heads],
                             rot.base, rot.dims
    layers[i].mlp    null; or kind "dense" with ff
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple, Union

from .bepuzen import MAX_POSITIONS, _need, _pos_float, _pos_int
from .qwen3 import ConfigError
from .spec import LayerRun, LayerSpec, ModelSpec, PartSpec


def _number(d: Mapping[str, Any], key: str, where: str) -> float:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config key '{where}{key}' must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    taps: int
    norm_groups: int


@dataclass(frozen=True)
class WindowBranchConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    rot_base: float
    rot_dims: int


@dataclass(frozen=True)
class RetentionBranchConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot_base: float
    rot_dims: int


@dataclass(frozen=True)
class ParallelConfig:
    left: WindowBranchConfig
    right: RetentionBranchConfig
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class DenseConfig:
    ff: int


MixerConfig = Union[StateSpaceConfig, ParallelConfig]


@dataclass(frozen=True)
class VifelixConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    embedding_scale: float
    mixers: Tuple[MixerConfig, ...]
    mlps: Tuple[Optional[DenseConfig], ...]
    eos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    ARCHITECTURE = "Vifelix"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "VifelixConfig":
        layers = _need(d, "layers", "")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config key 'layers' must be a non-empty list")
        eps = _pos_float(_need(d, "norm", ""), "eps", "norm.")
        mixers, mlps = [], []
        for i, L in enumerate(layers):
            at = f"layers[{i}]."
            kind = _need(L, "type", at)
            m = _need(L, "mixer", at)
            if kind == "mamba2":
                mixers.append(cls._state_space(m, at + "mixer."))
            elif kind == "parallel":
                mixers.append(cls._parallel(m, at + "mixer."))
            else:
                raise ConfigError(f"{at}type={kind!r} is not a mixer of this design (mamba2, parallel)")
            mlps.append(cls._mlp(L.get("mlp"), at + "mlp."))
        eos = d.get("eos_token_id")
        return cls(architecture=cls.ARCHITECTURE, vocab_size=_pos_int(d, "vocab", ""), hidden_size=_pos_int(d, "width", ""),
                   norm_eps=eps, embedding_scale=_number(_need(d, "embedding", ""), "scale", "embedding."),
                   mixers=tuple(mixers), mlps=tuple(mlps), eos_token_id=eos if isinstance(eos, int) else None,
                   torch_dtype=str(d.get("torch_dtype", "bfloat16")))

    @staticmethod
    def _state_space(m: Mapping[str, Any], at: str) -> StateSpaceConfig:
        c = StateSpaceConfig(heads=_pos_int(m, "heads", at), vdim=_pos_int(m, "vdim", at), state=_pos_int(m, "state", at),
                             groups=_pos_int(m, "groups", at), taps=_pos_int(m, "conv", at),
                             norm_groups=_pos_int(m, "norm_groups", at))
        if c.heads % c.groups:
            raise ConfigError(f"{at}heads={c.heads} must be a multiple of groups={c.groups}")
        if (c.heads * c.vdim) % c.norm_groups:
            raise ConfigError(f"{at}norm_groups={c.norm_groups} must divide heads * vdim = {c.heads * c.vdim}")
        return c

    @staticmethod
    def _rot(m: Mapping[str, Any], at: str, dim: int) -> Tuple[float, int]:
        rot = _need(m, "rot", at)
        base, dims = _pos_float(rot, "base", at + "rot."), _pos_int(rot, "dims", at + "rot.")
        if dims % 2 or dims > dim:
            raise ConfigError(f"{at}rot.dims={dims} must be even and at most dim={dim}")
        return base, dims

    @classmethod
    def _parallel(cls, m: Mapping[str, Any], at: str) -> ParallelConfig:
        lm, rm = _need(m, "left", at), _need(m, "right", at)
        la, ra = at + "left.", at + "right."
        dim = _pos_int(lm, "dim", la)
        base, dims = cls._rot(lm, la, dim)
        left = WindowBranchConfig(heads=_pos_int(lm, "heads", la), kv_heads=_pos_int(lm, "kv_heads", la), dim=dim,
                                  vdim=_pos_int(lm, "vdim", la), scale=_pos_float(lm, "scale", la),
                                  window=_pos_int(_need(lm, "mask", la), "size", la + "mask."), rot_base=base, rot_dims=dims)
        if left.heads % left.kv_heads:
            raise ConfigError(f"{la}heads={left.heads} must be a multiple of kv_heads={left.kv_heads}")
        if left.vdim != left.dim:
            raise ConfigError(f"{la}vdim={left.vdim} must equal dim={left.dim}: the values are the keys")
        rdim = _pos_int(rm, "dim", ra)
        base, dims = cls._rot(rm, ra, rdim)
        decay = _need(rm, "decay", ra)
        heads = _pos_int(rm, "heads", ra)
        if not isinstance(decay, list) or len(decay) != heads or any(isinstance(v, bool) or not isinstance(v, (int, float)) for v in decay):
            raise ConfigError(f"{ra}decay must list one number per head ({heads})")
        right = RetentionBranchConfig(heads=heads, dim=rdim, vdim=_pos_int(rm, "vdim", ra), decay=tuple(float(v) for v in decay),
                                      rot_base=base, rot_dims=dims)
        return ParallelConfig(left, right, _number(m, "left_scale", at), _number(m, "right_scale", at))

    @staticmethod
    def _mlp(mlp: Optional[Mapping[str, Any]], at: str) -> Optional[DenseConfig]:
        if mlp is None:
            return None
        kind = _need(mlp, "kind", at)
        if kind != "dense":
            raise ConfigError(f"{at}kind={kind!r} is not a feed-forward of this design (dense)")
        return DenseConfig(_pos_int(mlp, "ff", at))

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for m, f in zip(self.mixers, self.mlps):
            if isinstance(m, StateSpaceConfig):
                kind = "mamba2"
                mixer: Dict[str, Any] = {"heads": m.heads, "vdim": m.vdim, "state": m.state, "groups": m.groups, "conv": m.taps,
                                         "norm_groups": m.norm_groups}
            else:
                kind = "parallel"
                l, r = m.left, m.right
                mixer = {"left": {"heads": l.heads, "kv_heads": l.kv_heads, "dim": l.dim, "vdim": l.vdim, "scale": l.scale,
                                  "mask": {"size": l.window}, "rot": {"base": l.rot_base, "dims": l.rot_dims}},
                         "right": {"heads": r.heads, "dim": r.dim, "vdim": r.vdim, "decay": list(r.decay),
                                   "rot": {"base": r.rot_base, "dims": r.rot_dims}},
                         "left_scale": m.left_scale, "right_scale": m.right_scale}
            layers.append({"type": kind, "mixer": mixer, "mlp": None if f is None else {"kind": "dense", "ff": f.ff}})
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
        norm = PartSpec("rmsnorm_one_plus", {"size": D, "eps": eps, "leaf": ""})
        block = PartSpec("sandwich_residual", {
            "mixer_name": "mix", "feed_forward_name": "mlp", "mixer_norm_name": "norm1", "mixer_out_norm_name": "norm1b",
            "feed_forward_norm_name": "norm2", "feed_forward_out_norm_name": "norm2b"})
        layers = []
        for i, (m, f) in enumerate(zip(self.mixers, self.mlps)):
            if isinstance(m, StateSpaceConfig):
                mixer = PartSpec("state_space", {
                    "hidden_size": D, "num_heads": m.heads, "head_dim": m.vdim, "state_size": m.state, "groups": m.groups,
                    "taps": m.taps, "norm_groups": m.norm_groups, "norm_eps": eps})
            else:
                l, r = m.left, m.right
                left = PartSpec("gqa_window_sink", {
                    "hidden_size": D, "num_heads": l.heads, "num_kv_heads": l.kv_heads, "qk_dim": l.dim, "v_dim": l.vdim,
                    "scale": l.scale, "norm_eps": eps, "window": l.window, "head_norm": True, "biases": True,
                    "values_are_keys": True, "gate": "sigmoid",
                    "position_encoding": PartSpec("rotary_partial", {"dims": l.rot_dims, "base": l.rot_base})})
                right = PartSpec("retention", {
                    "hidden_size": D, "num_heads": r.heads, "qk_dim": r.dim, "v_dim": r.vdim, "decay": tuple(r.decay),
                    "norm_eps": eps, "position_encoding": PartSpec("rotary_partial", {"dims": r.rot_dims, "base": r.rot_base})})
                mixer = PartSpec("parallel", {"hidden_size": D, "branches": (("left", left, m.left_scale),
                                                                             ("right", right, m.right_scale))})
            parts = {"mixer": mixer, "mixer_norm": norm, "mixer_out_norm": norm}
            if f is not None:
                parts["feed_forward"] = PartSpec("gated_dense", {"hidden_size": D, "intermediate_size": f.ff,
                                                                 "activation": "silu", "biases": True})
                parts["feed_forward_norm"] = norm
                parts["feed_forward_out_norm"] = norm
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
        """Norm weights stored for a feed-forward that the layer does not have."""
        return any(f is None and name in (f"l{i}.norm2", f"l{i}.norm2b") for i, f in enumerate(self.mlps))
