"""Lukelorn as data: which parts, with which constants, under which tensor names.

Tensor names: ``embed``, ``head``, ``final.norm``, and per layer with tensors of its own ``l<i>.``: ``norm1`` (stored
around zero: the norm multiplies by 1 + w; so does ``final.norm``), ``mix.*`` and ``mlp.*`` (gate, up, down of a dense
feed-forward; router and e<j>.up / .down of a mixture of experts).  A layer that names another with ``weights_of`` runs
that layer's parts on a cache lane of its own: the schedule lists the other layer with a new lane.
"""
from __future__ import annotations

from dataclasses import replace

from ..config.lukelorn import AttentionMixer, DeltaMixer, DenseMlp, LatentMixer, LukelornConfig, MoeMlp, Rotation
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

LAYER_NAMES = {"mixer_norm": "norm1", "mixer": "mix.", "feed_forward": "mlp."}
DEFAULT_RANK = 32          # of the decay's and the gate's first projections when neither the configuration nor a checkpoint gives it


def fit_config_to_checkpoint(cfg: LukelornConfig, shapes) -> LukelornConfig:
    """The ranks of the delta rule's two-step projections are sizes only their tensors give: ``l<i>.mix.a1`` and
    ``l<i>.mix.g1`` are [rank, width]."""
    layers = list(cfg.layers)
    for i, layer in enumerate(layers):
        m = layer.mixer
        if not isinstance(m, DeltaMixer):
            continue
        src = i if layer.weights_of is None else layer.weights_of
        a1, g1 = shapes.get(f"l{src}.mix.a1"), shapes.get(f"l{src}.mix.g1")
        if not m.decay_rank and a1 is not None and len(a1) == 2:
            m = replace(m, decay_rank=int(a1[0]))
        if not m.gate_rank and g1 is not None and len(g1) == 2:
            m = replace(m, gate_rank=int(g1[0]))
        layers[i] = replace(layer, mixer=m)
    return replace(cfg, layers=tuple(layers))


def _position(rot: Rotation, head_dim: int) -> PartSpec:
    if not rot.dims:
        return PartSpec("none", {})
    params = {"head_dim": head_dim, "theta": rot.base, "rot_dim": rot.dims, "adjacent": True}
    if rot.factor is not None:
        params.update({"factor": rot.factor, "low": rot.low, "high": rot.high, "original": rot.original})
    return PartSpec("wavelength_scaled_rope", params)


def _mixer(cfg: LukelornConfig, m) -> PartSpec:
    if isinstance(m, AttentionMixer):
        return PartSpec("sink_window_attention", {
            "hidden_size": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
            "softmax_scale": m.scale, "position": _position(m.rot, m.dim), "eps": cfg.norm_eps, "window": m.window,
            "keep_first": m.keep_first, "softcap": m.softcap, "sink": "learned", "unit_rms": False, "biases": (), "gate": True})
    if isinstance(m, DeltaMixer):
        return PartSpec("gated_delta_rule", {
            "hidden_size": cfg.width, "n_heads": m.heads, "n_qk_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
            "conv_taps": m.conv, "eps": cfg.norm_eps, "decay_rank": m.decay_rank or DEFAULT_RANK,
            "gate_rank": m.gate_rank or DEFAULT_RANK, "gate": "sigmoid"})
    if isinstance(m, LatentMixer):
        names = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv",
                 "o": "o", "gate": "g"}
        return PartSpec("latent_attention", {
            "hidden_size": cfg.width, "n_heads": m.heads, "head_dim": m.dim, "value_dim": m.vdim, "q_rank": m.q_rank,
            "kv_rank": m.kv_rank, "softmax_scale": m.scale, "eps": cfg.norm_eps, "window": m.window, "rot_dim": m.rot_dim,
            "position": _position(m.rot, m.rot_dim) if m.rot_dim else None, "gate": True, "names": names})
    raise ValueError(f"unknown mixer {type(m).__name__}")


def _feed_forward(cfg: LukelornConfig, p):
    if p is None:
        return None
    if isinstance(p, DenseMlp):
        return PartSpec("gated_ffn", {"hidden_size": cfg.width, "intermediate_size": p.ff, "activation": p.act,
                                      "names": {"gate": "gate", "up": "up", "down": "down"}})
    if isinstance(p, MoeMlp):
        return PartSpec("routed_experts", {"hidden_size": cfg.width, "n_experts": p.experts, "top": p.top, "expert_size": p.expert_ff,
                                           "scoring": "sigmoid", "expert_form": "up_relu2", "weight_on": "input"})
    raise ValueError(f"unknown feed-forward {type(p).__name__}")


def model_spec(cfg: LukelornConfig) -> ModelSpec:
    norm = PartSpec("rms_norm", {"hidden_size": cfg.width, "eps": cfg.norm_eps, "weight_name": "", "offset": 1.0})
    block = PartSpec("parallel_residual", {"residual_scale": cfg.residual_mult})
    layers, schedule, spec_of = [], [], {}
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        spec_of[i] = len(layers)
        layers.append(LayerSpec(block=block, mixer=_mixer(cfg, layer.mixer), feed_forward=_feed_forward(cfg, layer.mlp),
                                mixer_norm=norm, feed_forward_norm=None, prefix=f"l{i}.", names=LAYER_NAMES))
    for i, layer in enumerate(cfg.layers):            # every layer of the configuration is a run with a lane of its own
        src = i if layer.weights_of is None else layer.weights_of
        if src not in spec_of:
            raise ValueError(f"layer {i} runs on the tensors of layer {src}, which has none of its own")
        schedule.append(ScheduleEntry(layer=spec_of[src], lane=i, writes_cache=True))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("scaled_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "scale": 1.0,
                                                "weight_name": "embed"}),
        layers=layers, schedule=schedule, final_norm=norm,
        head=PartSpec("scaled_lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "scale": 1.0, "weight_name": "head"}),
        embedding_name="", final_norm_name="final.norm", head_name="", max_positions=0)
