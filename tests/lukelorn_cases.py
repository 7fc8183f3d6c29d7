"""Small Lukelorn configurations and random weights for the tests, and an error measure.

The configurations differ from one another in every size, in the order of the layers and in what is left out (the
window, the kept first tokens, the cap on the scores, the rotation and its stretching, a layer's feed-forward, layers
that run on another layer's tensors).  Values that a given checkpoint might happen to make equal (key and value sizes of
a head, head counts of the mixers, the ranks of the two-step projections) or 1 are unequal here, or 1 where a checkpoint
would have more.  Weights are rounded to bfloat16 so that both precisions read the same values.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import torch

NAME = "Lukelorn"


def _attn(heads, kv, dim, vdim, scale, window=None, keep=0, cap=None, rot=None, scaling=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
        if keep:
            m["mask"]["keep_first"] = keep
    if cap:
        m["softcap"] = cap
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
        if scaling:
            m["rot"]["scaling"] = {"factor": scaling[0], "low": scaling[1], "high": scaling[2], "original": scaling[3]}
    return {"type": "attention", "mixer": m}


def _delta(heads, kv, dim, vdim, conv, ranks=(12, 8)):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv},
            "_ranks": ranks}


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, window=None, base=1000.0):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if rot_dim:
        m["rot"] = {"dims": rot_dim, "base": base}
    return {"type": "latent_attention", "mixer": m}


def _moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def _dense(ff, act=None):
    return {"kind": "dense", "ff": ff, "act": act} if act else {"kind": "dense", "ff": ff}


def _layer(mixer: dict, mlp: Optional[dict], weights_of: Optional[int] = None) -> dict:
    out = dict(mixer, mlp=mlp)
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def config_a() -> dict:
    """All three mixers, grouped heads, a window that ends inside a page with a few kept first tokens, a rotation of part
    of a head with stretched long waves, two layers that run on earlier layers' tensors (an attention layer and a delta
    layer, each with a cache or state of its own), dense and routed feed-forwards."""
    attn = _attn(4, 2, 24, 40, 0.4, window=20, keep=5, cap=5.0, rot=(16, 5000.0), scaling=(4.0, 1.0, 4.0, 64))
    delta = _delta(4, 2, 20, 24, 4)
    return {"architecture": NAME, "vocab": 211, "width": 96, "residual_mult": 0.7, "norm": {"eps": 1e-5},
            "layers": [
                _layer(attn, _moe(8, 2, 40)),
                _layer(delta, _dense(64)),
                _layer(_latent(3, 16, 8, 24, 40, 24, 0.3, window=37), _moe(6, 3, 32)),
                _layer(attn, _moe(8, 2, 40), weights_of=0),
                _layer(delta, _dense(64), weights_of=1),
            ]}


def config_b() -> dict:
    """One head everywhere; no window, no cap, no stretching, no residual constant; a latent layer without a window and
    one whose window is a single token; a convolution of one tap; a layer without a feed-forward first; ``top`` of one
    and of all experts; a layer that names a later layer's tensors."""
    lat = _latent(1, 40, 4, 72, 24, 56, 0.2)
    return {"architecture": NAME, "vocab": 130, "width": 64, "norm": {"eps": 1e-3},
            "layers": [
                _layer(lat, None, weights_of=2),
                _layer(_attn(1, 1, 32, 16, 0.3, rot=(32, 100.0)), _moe(4, 1, 24)),
                _layer(lat, None),
                _layer(_delta(1, 1, 40, 72, 1, ranks=(1, 5)), _moe(3, 3, 8)),
                _layer(_latent(2, 8, 2, 8, 8, 16, 1.1, window=1), _dense(40, "gelu_tanh")),
                _layer(_attn(3, 3, 8, 8, 1.1, window=1, keep=3, cap=2.0), None),
            ]}


def config_c() -> dict:
    """Sizes that fit no kernel's favourite multiple: a width of 100, five heads of 12 with values of 36, a rotation of
    six dimensions, windows of exactly one page (keeping exactly one page) and of a page and one token (keeping one
    token), a latent row of 26 values, nine experts, feed-forwards of 20, a convolution of two taps, seven value heads
    on one key head."""
    return {"architecture": NAME, "vocab": 77, "width": 100, "residual_mult": 1.5, "norm": {"eps": 1e-4},
            "layers": [
                _layer(_delta(7, 1, 36, 12, 2, ranks=(5, 9)), _moe(9, 4, 20)),
                _layer(_attn(5, 5, 12, 36, 0.5, window=64, keep=64, cap=8.0, rot=(6, 777.0), scaling=(1.5, 2.0, 3.0, 10)),
                       _moe(9, 2, 20)),
                _layer(_latent(5, 12, 6, 36, 28, 20, 0.25, window=65, base=50.0), _moe(2, 1, 12)),
                _layer(_attn(10, 5, 12, 36, 0.5, window=65, keep=1, rot=(12, 30.0)), _dense(20)),
                _layer(_attn(2, 1, 20, 20, 0.3, window=3, keep=100), None),
            ]}


def config_d() -> dict:
    """Head sizes the tensor-core kernels take (64 and 128, equal key and value sizes, even groups; a latent row of 64):
    windows that end inside the third page with kept tokens beyond the first page, and a window beyond the test's
    sequences; a delta rule of 64 x 64 states."""
    attn = _attn(4, 2, 64, 64, 0.3, window=150, keep=70, cap=10.0, rot=(32, 20000.0), scaling=(8.0, 1.0, 4.0, 128))
    return {"architecture": NAME, "vocab": 150, "width": 128, "residual_mult": 0.5, "norm": {"eps": 1e-6},
            "layers": [
                _layer(attn, _moe(4, 2, 32)),
                _layer(_delta(4, 4, 64, 64, 3, ranks=(16, 24)), _moe(4, 2, 32)),
                _layer(_attn(8, 2, 128, 128, 0.2, window=1000, keep=130, cap=15.0, rot=(128, 1e6)), _moe(6, 3, 24)),
                _layer(_latent(4, 32, 16, 32, 64, 48, 0.35, window=70), _dense(96)),
                _layer(attn, _moe(4, 2, 32), weights_of=0),
                _layer(_attn(2, 1, 32, 32, 0.4, window=40, keep=33), _moe(4, 2, 32)),
            ]}


def only(kind: str) -> dict:
    """Three layers of one kind of mixer and no feed-forward: the mechanism alone."""
    mixers = {
        "attention": [_attn(6, 3, 16, 24, 0.35, window=30, keep=7, cap=6.0, rot=(8, 900.0), scaling=(3.0, 1.0, 2.0, 32)),
                      _attn(2, 2, 40, 8, 0.2, rot=(40, 50.0)), _attn(4, 1, 32, 32, 0.3, window=70, keep=2)],
        "channel_delta": [_delta(3, 3, 16, 40, 3, ranks=(7, 4)), _delta(6, 2, 40, 8, 5, ranks=(3, 11)), _delta(2, 1, 70, 20, 2)],
        "latent_attention": [_latent(3, 8, 8, 16, 20, 32, 0.4, window=30), _latent(2, 24, 0, 8, 12, 16, 0.3),
                             _latent(5, 4, 12, 4, 16, 8, 0.5, window=66, base=20.0)],
    }[kind]
    return {"architecture": NAME, "vocab": 90, "width": 80, "residual_mult": 0.8, "norm": {"eps": 1e-5},
            "layers": [_layer(m, None) for m in mixers]}


CONFIGS = {"a": config_a, "b": config_b, "c": config_c, "d": config_d,
           "attention": lambda: only("attention"), "channel_delta": lambda: only("channel_delta"),
           "latent_attention": lambda: only("latent_attention")}


def clean(cfg: dict) -> dict:
    """The configuration as a file holds it: without the test's private notes on tensor sizes."""
    out = dict(cfg, layers=[{k: v for k, v in layer.items() if not k.startswith("_")} for layer in cfg["layers"]])
    return out


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    W, out = cfg["width"], {}
    out["embed"] = (cfg["vocab"], W)
    out["head"] = (cfg["vocab"], W)
    out["final.norm"] = (W,)
    for i, layer in enumerate(cfg["layers"]):
        if "weights_of" in layer:
            continue
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (W,)
        if layer["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * d, W), p + "mix.k": (G * d, W), p + "mix.v": (G * dv, W), p + "mix.sink": (H,),
                        p + "mix.g": (H, W), p + "mix.o": (W, H * dv)})
        elif layer["type"] == "channel_delta":
            H, G, d, dv, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            ra, rg = layer.get("_ranks", (12, 8))
            out.update({p + "mix.q": (G * d, W), p + "mix.q.conv": (G * d, K), p + "mix.k": (G * d, W), p + "mix.k.conv": (G * d, K),
                        p + "mix.v": (H * dv, W), p + "mix.v.conv": (H * dv, K), p + "mix.b": (H, W), p + "mix.A_log": (H,),
                        p + "mix.norm": (dv,), p + "mix.a1": (ra, W), p + "mix.a2": (H * d, ra), p + "mix.dt_bias": (H * d,),
                        p + "mix.g1": (rg, W), p + "mix.g2": (H * dv, rg), p + "mix.o": (W, H * dv)})
        else:
            H, d, dr, dv, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out.update({p + "mix.dq": (Q, W), p + "mix.dq.norm": (Q,), p + "mix.uq": (H * (d + dr), Q), p + "mix.dkv": (R + dr, W),
                        p + "mix.dkv.norm": (R,), p + "mix.uk": (H * d, R), p + "mix.uv": (H * dv, R), p + "mix.g": (H, W),
                        p + "mix.o": (W, H * dv)})
        mlp = layer["mlp"]
        if mlp and mlp["kind"] == "dense":
            out.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
        elif mlp:
            ff, E = mlp["expert"]["ff"], mlp["router"]["experts"]
            for e in range(E):
                out.update({f"{p}mlp.e{e}.up": (ff, W), f"{p}mlp.e{e}.down": (W, ff)})
            out[p + "mlp.router"] = (E, W)
    return out


def random_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if name == "embed":
            t = torch.randn(shape, generator=g)
        elif last == "router":
            t = torch.randn(shape, generator=g) * (2.5 / shape[1] ** 0.5)
        elif last == "sink":
            t = torch.randn(shape, generator=g) * 1.5
        elif last == "A_log":
            t = torch.randn(shape, generator=g) * 0.7 - 1.0
        elif last == "dt_bias":
            t = torch.randn(shape, generator=g) * 1.0 - 0.5
        elif last == "conv":
            t = torch.randn(shape, generator=g) * 0.6
        elif name.endswith("mix.norm") or name.endswith("dq.norm") or name.endswith("dkv.norm"):
            t = 1.0 + 0.25 * torch.randn(shape, generator=g)           # plain norm weights
        elif len(shape) == 2:
            t = torch.randn(shape, generator=g) * (1.4 / shape[1] ** 0.5)
        else:
            t = 0.3 * torch.randn(shape, generator=g)                  # norm weights stored around zero
        out[name] = t.to(torch.bfloat16)
    return out


def write_folder(cfg: dict, weights: Dict[str, torch.Tensor], out_dir: str) -> str:
    from cpmcu_b200.weights.safetensors_io import save_file

    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(clean(cfg), f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(out_dir, "model.safetensors"))
    return out_dir


def random_ids(vocab: int, n: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def moe_runs(cfg: dict) -> int:
    return sum(1 for layer in cfg["layers"] if layer["mlp"] and layer["mlp"]["kind"] == "moe")


# Largest allowed root mean square of (engine - plain) over the vocabulary, the mean difference taken off, relative to
# the root mean square of the plain logits, for the worst row and for the median row.  float32: summation order only.
# bfloat16: activations between the kernels and the cached keys and values are rounded to bfloat16 in the engine; single
# rows react strongly to that rounding (sharp routers, expert inputs squared), so the worst row has a loose bound and the
# median a tight one, and float32 carries the exact comparison.
TOL = {"float32": 5e-4, "bfloat16": 0.6}
MEDIAN_TOL = {"float32": 2e-5, "bfloat16": 5e-2}
# A token's choice of experts may fall the other way where two scores nearly tie; the plain implementation uses the
# engine's choice, whose lowest score must lie this close to the rule's cut-off (scores lie in [0, 1])
CHOICE_SLACK = {"float32": 1e-5, "bfloat16": 4e-2}


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
