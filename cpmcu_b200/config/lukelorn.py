"""Typed configuration of the Lukelorn architecture: a decoder of parallel layers (one norm; the mixer and the
feed-forward both read its output and their sum, times one constant, is added to the residual) whose mixer is softmax
attention with a window that keeps a sequence's first tokens, capped scores, a learned sink per head and an output gate;
or a gated delta rule with a decay per key channel; or attention over a cached latent with a rotated key part; and whose
feed-forward is dense or a mixture of experts.  A layer may run on another layer's tensors with a cache of its own.

``config.json`` is nested; every size and constant is read from it:

    architecture, vocab, width, residual_mult, norm.eps,
    layers[i] = {type: "attention" | "channel_delta" | "latent_attention", mixer: {...}, mlp: {...} | null, weights_of: j}
    attention:        mixer = {heads, kv_heads, dim, vdim, scale, softcap, mask: {size, keep_first},
                               rot: {dims, base, scaling: {factor, low, high, original}}}
    channel_delta:    mixer = {heads, kv_heads, dim, vdim, conv}   (the ranks of the decay's and the gate's first projections
                               are sizes of the checkpoint's tensors; ``decay_rank`` / ``gate_rank`` may state them)
    latent_attention: mixer = {heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, mask: {size}, rot: {dims, base}}
    mlp = {kind: "dense", ff, act: "silu" (default) | "gelu_tanh"} | {kind: "moe", router: {experts, top}, expert: {ff}}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple, Union

from .base import ConfigError, FieldReader

NAME = "Lukelorn"


@dataclass(frozen=True)
class Rotation:
    dims: int                        # 0: no rotation
    base: float = 10000.0
    factor: Optional[float] = None   # None: frequencies as they are; else stretched by wavelength
    low: float = 1.0
    high: float = 4.0
    original: int = 8192

    def to_json(self) -> Optional[Dict[str, Any]]:
        if not self.dims:
            return None
        out: Dict[str, Any] = {"dims": self.dims, "base": self.base}
        if self.factor is not None:
            out["scaling"] = {"factor": self.factor, "low": self.low, "high": self.high, "original": self.original}
        return out


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float                   # 0: scores are not capped
    window: Optional[int]            # mask.size; None: every earlier token is seen
    keep_first: int                  # mask.keep_first: first tokens a window keeps
    rot: Rotation

    def to_json(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale}
        if self.softcap:
            out["softcap"] = self.softcap
        if self.window is not None:
            out["mask"] = {"size": self.window}
            if self.keep_first:
                out["mask"]["keep_first"] = self.keep_first
        if self.rot.dims:
            out["rot"] = self.rot.to_json()
        return out


@dataclass(frozen=True)
class DeltaMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: int = 0              # 0: left to the checkpoint's tensors
    gate_rank: int = 0

    def to_json(self) -> Dict[str, Any]:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}
        if self.decay_rank:
            out["decay_rank"] = self.decay_rank
        if self.gate_rank:
            out["gate_rank"] = self.gate_rank
        return out


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: Optional[int]
    rot: Rotation

    def to_json(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                               "q_rank": self.q_rank, "kv_rank": self.kv_rank, "scale": self.scale}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.rot.dims:
            out["rot"] = self.rot.to_json()
        return out


@dataclass(frozen=True)
class DenseMlp:
    ff: int
    act: str = "silu"                # the gate's activation: "silu" or "gelu_tanh"

    def to_json(self) -> Dict[str, Any]:
        out = {"kind": "dense", "ff": self.ff}
        if self.act != "silu":
            out["act"] = self.act
        return out


@dataclass(frozen=True)
class MoeMlp:
    experts: int
    top: int
    expert_ff: int

    def to_json(self) -> Dict[str, Any]:
        return {"kind": "moe", "expert": {"ff": self.expert_ff}, "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class LukelornLayer:
    type: str
    mixer: Union[AttentionMixer, DeltaMixer, LatentMixer]
    mlp: Union[DenseMlp, MoeMlp, None]
    weights_of: Optional[int] = None         # the layer whose tensors this one runs on; None: its own

    def to_json(self) -> Dict[str, Any]:
        out = {"type": self.type, "mixer": self.mixer.to_json(), "mlp": self.mlp.to_json() if self.mlp else None}
        if self.weights_of is not None:
            out["weights_of"] = self.weights_of
        return out


def _rotation(mr: FieldReader, default_dims: Optional[int] = None) -> Rotation:
    rot = mr.child("rot")
    if rot is None:
        return Rotation(0)
    dims = rot.integer("dims", default_dims if default_dims is not None else 0, minimum=0) or 0
    base = rot.number("base", 10000.0, positive=True) or 10000.0
    out = Rotation(dims, base)
    sc = rot.child("scaling")
    if sc is not None:
        out = Rotation(dims, base, sc.number("factor", positive=True), sc.number("low", 1.0, positive=True),
                       sc.number("high", 4.0, positive=True), sc.integer("original", minimum=1))
        if None not in (out.low, out.high):
            sc.check(out.high > out.low, "'high' must be larger than 'low'")
    rot.absorb(sc)
    mr.absorb(rot)
    return out


def _window(mr: FieldReader) -> Tuple[Optional[int], int]:
    mask = mr.child("mask")
    if mask is None:
        return None, 0
    size = mask.integer("size", None, minimum=1)
    keep = mask.integer("keep_first", 0, minimum=0) or 0
    mr.absorb(mask)
    return size, keep


@dataclass(frozen=True)
class LukelornConfig:
    vocab: int
    width: int
    residual_mult: float
    norm_eps: float
    layers: Tuple[LukelornLayer, ...]
    architecture: str = NAME

    MIXER_TYPES = ("attention", "channel_delta", "latent_attention")

    @staticmethod
    def _attention(mr: FieldReader) -> AttentionMixer:
        heads, kv = mr.integer("heads", minimum=1), mr.integer("kv_heads", None, minimum=1)
        dim = mr.integer("dim", minimum=1)
        vdim = mr.integer("vdim", dim, minimum=1)
        scale = mr.number("scale", positive=True)
        softcap = mr.number("softcap", 0.0) or 0.0
        window, keep = _window(mr)
        rot = _rotation(mr)
        m = AttentionMixer(heads, kv if kv is not None else heads, dim, vdim, scale, float(softcap), window, keep, rot)
        if None not in (m.heads, m.kv_heads, m.dim):
            mr.check(m.heads % m.kv_heads == 0, f"'heads' {m.heads} must be a multiple of 'kv_heads' {m.kv_heads}")
            mr.check(rot.dims % 2 == 0 and rot.dims <= m.dim, f"'rot.dims' must be even and at most 'dim' {m.dim}")
        mr.check(m.softcap >= 0, "'softcap' must not be negative")
        return m

    @staticmethod
    def _delta(mr: FieldReader) -> DeltaMixer:
        heads, kv = mr.integer("heads", minimum=1), mr.integer("kv_heads", None, minimum=1)
        dim = mr.integer("dim", minimum=1)
        m = DeltaMixer(heads, kv if kv is not None else heads, dim, mr.integer("vdim", dim, minimum=1),
                       mr.integer("conv", 1, minimum=1), mr.integer("decay_rank", 0, minimum=0) or 0,
                       mr.integer("gate_rank", 0, minimum=0) or 0)
        if None not in (m.heads, m.kv_heads):
            mr.check(m.heads % m.kv_heads == 0, f"'heads' {m.heads} must be a multiple of 'kv_heads' {m.kv_heads}")
        if m.conv is not None:
            mr.check(m.conv <= 8, "'conv' must be at most 8 taps")
        return m

    @staticmethod
    def _latent(mr: FieldReader) -> LatentMixer:
        heads, dim = mr.integer("heads", minimum=1), mr.integer("dim", minimum=1)
        rot_dim = mr.integer("rot_dim", 0, minimum=0) or 0
        window, _ = _window(mr)
        rot = _rotation(mr, default_dims=rot_dim)
        m = LatentMixer(heads, dim, rot_dim, mr.integer("vdim", dim, minimum=1), mr.integer("q_rank", minimum=1),
                        mr.integer("kv_rank", minimum=1), mr.number("scale", positive=True), window, rot)
        mr.check(rot_dim % 2 == 0, "'rot_dim' must be even")
        mr.check(rot.dims == rot_dim, f"'rot.dims' {rot.dims} must equal 'rot_dim' {rot_dim}")
        return m

    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "LukelornConfig":
        r = FieldReader(data)
        vocab = r.integer("vocab", minimum=1)
        width = r.integer("width", minimum=1)
        mult = r.number("residual_mult", 1.0)
        norm = r.child("norm")
        eps = norm.number("eps", positive=True) if norm is not None else None
        if norm is None:
            r.check(False, "required key 'norm' is missing")
        r.absorb(norm)
        raw_layers = data.get("layers")
        layers: List[LukelornLayer] = []
        if not isinstance(raw_layers, list) or not raw_layers:
            r.check(False, "'layers' must be a non-empty list")
            raw_layers = []
        for i, raw in enumerate(raw_layers):
            lr = FieldReader(raw, f"config.json:layers[{i}]") if isinstance(raw, dict) else None
            if lr is None:
                r.check(False, f"layers[{i}] must be an object")
                continue
            kind = lr.string("type", choices=cls.MIXER_TYPES)
            mr = lr.child("mixer")
            mixer = None
            if mr is None:
                lr.check(False, "required key 'mixer' is missing")
            elif kind == "attention":
                mixer = cls._attention(mr)
            elif kind == "channel_delta":
                mixer = cls._delta(mr)
            elif kind == "latent_attention":
                mixer = cls._latent(mr)
            lr.absorb(mr)
            pr = lr.child("mlp")
            mlp = None
            if pr is not None:
                what = pr.string("kind", choices=("dense", "moe"))
                if what == "dense":
                    mlp = DenseMlp(pr.integer("ff", minimum=1), pr.string("act", "silu", choices=("silu", "gelu_tanh")) or "silu")
                elif what == "moe":
                    router, expert = pr.child("router"), pr.child("expert")
                    if router is None or expert is None:
                        pr.check(False, "a mixture of experts needs 'router' and 'expert'")
                    else:
                        mlp = MoeMlp(router.integer("experts", minimum=1), router.integer("top", minimum=1),
                                     expert.integer("ff", minimum=1))
                        if None not in (mlp.experts, mlp.top):
                            router.check(mlp.top <= mlp.experts, f"'top' {mlp.top} exceeds the {mlp.experts} experts")
                    pr.absorb(router)
                    pr.absorb(expert)
            lr.absorb(pr)
            weights_of = lr.integer("weights_of", None, minimum=0)
            r.problems.extend(lr.problems)
            if not lr.problems and mixer is not None:
                layers.append(LukelornLayer(kind, mixer, mlp, weights_of))
        # a layer that runs on another's tensors: that layer has tensors of its own and the same entry otherwise
        if len(layers) == len(raw_layers):
            for i, layer in enumerate(layers):
                j = layer.weights_of
                if j is None:
                    continue
                where = f"layers[{i}].weights_of"
                if j >= len(layers) or j == i or layers[j].weights_of is not None:
                    r.check(False, f"{where} must name another layer that has tensors of its own")
                    continue
                src = layers[j]
                r.check((src.type, src.mixer, src.mlp) == (layer.type, layer.mixer, layer.mlp),
                        f"{where}: layer {j} differs in type, mixer or feed-forward")
        r.finish()
        return cls(vocab, width, float(mult), float(eps), tuple(layers))

    @classmethod
    def from_json(cls, path: str) -> "LukelornConfig":
        from .base import read_config_json
        return cls.from_dict(read_config_json(path))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "residual_mult": self.residual_mult, "norm": {"eps": self.norm_eps},
                "layers": [layer.to_json() for layer in self.layers]}
