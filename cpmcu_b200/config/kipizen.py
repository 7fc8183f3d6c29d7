"""Typed configuration of the Kipizen architecture: a decoder whose layers carry either softmax attention with a
sliding window, capped scores and a sink (some layers reading another layer's keys and values), or lightning
attention (a linear recurrence with one fixed decay per head), each followed by a mixture of experts.

``config.json`` is nested; every size and constant is read from it:

    architecture, vocab, width, embedding.scale, norm.eps,
    layers[i] = {type: "attention" | "lightning", mixer: {...}, mlp: {...} | null}
    attention: mixer = {heads, kv_heads, dim, vdim, scale, softcap, mask: {size}, kv_from (absent: own keys and values),
                        rot: {dims, base, scaling: {factor}}}
    lightning: mixer = {heads, dim, vdim, decay: [one number per head]}
    mlp = {kind: "moe", router: {experts, top}, expert: {ff}}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple, Union

from .base import ConfigError, FieldReader

NAME = "Kipizen"


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float                   # 0: scores are not capped
    window: Optional[int]            # mask.size; None: every earlier token is seen
    rot_dims: int                    # 0: no rotation
    rot_base: float
    rot_factor: float                # every frequency is divided by it
    kv_from: Optional[int]           # the layer whose cached keys and values this one reads; None: its own

    def to_json(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale}
        if self.softcap:
            out["softcap"] = self.softcap
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.rot_dims:
            out["rot"] = {"dims": self.rot_dims, "base": self.rot_base}
            if self.rot_factor != 1.0:
                out["rot"]["scaling"] = {"factor": self.rot_factor}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class LightningMixer:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    def to_json(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class MoeMlp:
    experts: int
    top: int
    expert_ff: int

    def to_json(self) -> Dict[str, Any]:
        return {"kind": "moe", "expert": {"ff": self.expert_ff}, "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class KipizenLayer:
    type: str
    mixer: Union[AttentionMixer, LightningMixer]
    mlp: Optional[MoeMlp]

    def to_json(self) -> Dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_json(), "mlp": self.mlp.to_json() if self.mlp else None}


@dataclass(frozen=True)
class KipizenConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[KipizenLayer, ...]
    architecture: str = NAME

    MIXER_TYPES = ("attention", "lightning")

    @staticmethod
    def _attention(mr: FieldReader) -> AttentionMixer:
        heads, kv = mr.integer("heads", minimum=1), mr.integer("kv_heads", None, minimum=1)
        dim = mr.integer("dim", minimum=1)
        vdim = mr.integer("vdim", dim, minimum=1)
        scale = mr.number("scale", positive=True)
        softcap = mr.number("softcap", 0.0)
        mask = mr.child("mask")
        window = mask.integer("size", minimum=1) if mask is not None else None
        mr.absorb(mask)
        rot = mr.child("rot")
        dims, base, factor = 0, 10000.0, 1.0
        if rot is not None:
            dims = rot.integer("dims", minimum=0) or 0
            base = rot.number("base", positive=True) or 10000.0
            scaling = rot.child("scaling")
            if scaling is not None:
                factor = scaling.number("factor", 1.0, positive=True) or 1.0
            rot.absorb(scaling)
        mr.absorb(rot)
        kv_from = mr.integer("kv_from", None, minimum=0)
        m = AttentionMixer(heads, kv if kv is not None else heads, dim, vdim, scale, float(softcap or 0.0), window, dims, base,
                           factor, kv_from)
        if None not in (m.heads, m.kv_heads, m.dim):
            mr.check(m.heads % m.kv_heads == 0, f"'heads' {m.heads} must be a multiple of 'kv_heads' {m.kv_heads}")
            mr.check(m.rot_dims % 2 == 0 and m.rot_dims <= m.dim, f"'rot.dims' must be even and at most 'dim' {m.dim}")
        mr.check(m.softcap >= 0, "'softcap' must not be negative")
        return m

    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "KipizenConfig":
        r = FieldReader(data)
        vocab = r.integer("vocab", minimum=1)
        width = r.integer("width", minimum=1)
        emb = r.child("embedding")
        emb_scale = emb.number("scale", 1.0) if emb is not None else 1.0
        r.absorb(emb)
        norm = r.child("norm")
        eps = norm.number("eps", positive=True) if norm is not None else None
        if norm is None:
            r.check(False, "required key 'norm' is missing")
        r.absorb(norm)
        raw_layers = data.get("layers")
        layers: List[KipizenLayer] = []
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
            elif kind == "lightning":
                heads = mr.integer("heads", minimum=1)
                dim = mr.integer("dim", minimum=1)
                decay = mr.numbers("decay")
                mixer = LightningMixer(heads, dim, mr.integer("vdim", dim, minimum=1), tuple(decay or ()))
                if heads is not None and decay is not None:
                    mr.check(len(decay) == heads, f"'decay' must hold one number per head ({heads}), got {len(decay)}")
            lr.absorb(mr)
            pr = lr.child("mlp")
            mlp = None
            if pr is not None:
                pr.string("kind", "moe", choices=("moe",))
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
            r.problems.extend(lr.problems)
            if not lr.problems and mixer is not None:
                layers.append(KipizenLayer(kind, mixer, mlp))
        # a layer that reads another's keys and values: that layer is an earlier attention layer with projections of its
        # own and the same head counts, head sizes and rotation
        if len(layers) == len(raw_layers):
            for i, layer in enumerate(layers):
                m = layer.mixer
                if not isinstance(m, AttentionMixer) or m.kv_from is None:
                    continue
                src = layers[m.kv_from].mixer if m.kv_from < i else None
                where = f"layers[{i}].mixer.kv_from"
                if not isinstance(src, AttentionMixer) or src.kv_from is not None:
                    r.check(False, f"{where} must name an earlier attention layer that has keys and values of its own")
                    continue
                same = (src.kv_heads, src.dim, src.vdim, src.rot_dims, src.rot_base, src.rot_factor) == \
                       (m.kv_heads, m.dim, m.vdim, m.rot_dims, m.rot_base, m.rot_factor)
                r.check(same, f"{where}: layer {m.kv_from} differs in key-value heads, head sizes or rotation")
        r.finish()
        return cls(vocab, width, float(emb_scale), float(eps), tuple(layers))

    @classmethod
    def from_json(cls, path: str) -> "KipizenConfig":
        from .base import read_config_json
        return cls.from_dict(read_config_json(path))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                "layers": [layer.to_json() for layer in self.layers]}
