"""Kipizen as data: which parts, with which constants, under which tensor names.

Tensor names: ``embed``, ``head``, ``final.norm``, and per layer ``l<i>.``: ``norm1``, ``norm2``, ``mix.*`` (q, k, v, o
with biases ``.b`` on q, k, v for attention; q, k, v, g, o, norm for lightning attention) and ``mlp.*`` (router,
router.b, e<j>.gate / .up / .down).  A layer that reads another layer's keys and values has no k and v tensors and runs
on that layer's cache lane without writing it; every other layer has a lane of its own.
"""
from __future__ import annotations

from ..config.kipizen import AttentionMixer, KipizenConfig, LightningMixer
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

LAYER_NAMES = {"mixer_norm": "norm1", "feed_forward_norm": "norm2", "mixer": "mix.", "feed_forward": "mlp."}


def model_spec(cfg: KipizenConfig) -> ModelSpec:
    norm = PartSpec("rms_norm", {"hidden_size": cfg.width, "eps": cfg.norm_eps, "weight_name": ""})
    block = PartSpec("pre_norm_residual", {})
    layers, schedule, lane_of = [], [], {}
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if isinstance(m, AttentionMixer):
            position = PartSpec("scaled_rope", {"head_dim": m.dim, "theta": m.rot_base, "rot_dim": m.rot_dims,
                                                "factor": m.rot_factor}) if m.rot_dims else PartSpec("none", {})
            own = m.kv_from is None
            mixer = PartSpec("sink_window_attention", {
                "hidden_size": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
                "softmax_scale": m.scale, "position": position, "eps": cfg.norm_eps, "window": m.window, "softcap": m.softcap,
                "sink": True, "unit_rms": True, "biases": ("q", "k", "v"), "own_kv": own})
        elif isinstance(m, LightningMixer):
            own = True
            mixer = PartSpec("lightning_attention", {
                "hidden_size": cfg.width, "n_heads": m.heads, "head_dim": m.dim, "value_dim": m.vdim, "decay": tuple(m.decay),
                "eps": cfg.norm_eps, "q_scale": 1.0, "norm_heads": "all", "gate": "sigmoid"})
        else:
            raise ValueError(f"layer {i}: unknown mixer {type(m).__name__}")
        if own:
            lane_of[i] = len(lane_of)
            schedule.append(ScheduleEntry(layer=i, lane=lane_of[i], writes_cache=True))
        else:
            if m.kv_from not in lane_of:
                raise ValueError(f"layer {i} reads the keys and values of layer {m.kv_from}, which has none of its own before it")
            schedule.append(ScheduleEntry(layer=i, lane=lane_of[m.kv_from], writes_cache=False))
        ffn = None
        if layer.mlp is not None:
            p = layer.mlp
            ffn = PartSpec("routed_experts", {"hidden_size": cfg.width, "n_experts": p.experts, "top": p.top,
                                              "expert_size": p.expert_ff, "scoring": "top_first", "router_bias": True})
        layers.append(LayerSpec(block=block, mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                feed_forward_norm=norm if ffn is not None else None, prefix=f"l{i}.", names=LAYER_NAMES))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("scaled_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "scale": cfg.embedding_scale,
                                                "weight_name": "embed"}),
        layers=layers, schedule=schedule, final_norm=norm,
        head=PartSpec("scaled_lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "scale": 1.0, "weight_name": "head"}),
        embedding_name="", final_norm_name="final.norm", head_name="", max_positions=0)
