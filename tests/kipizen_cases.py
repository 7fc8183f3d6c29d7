"""Small Kipizen configurations and random weights for the tests, and an error measure.

The configurations differ from one another in every size, in the order of the layers and in what is left out (the
window, the cap on the scores, the rotation and its scaling, a layer's feed-forward).  Values that a given checkpoint
might happen to make equal (key and value sizes of a head, the head counts and sizes of the two kinds of mixer, the
windows of a layer and of the layer whose keys it reads) or 1 are unequal here, or 1 where a checkpoint would have
more.  Weights are rounded to bfloat16 so that both precisions read the same values.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import torch

NAME = "Kipizen"


def _attn(heads, kv, dim, vdim, scale, window=None, cap=None, rot=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if cap:
        m["softcap"] = cap
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
        if len(rot) > 2:
            m["rot"]["scaling"] = {"factor": rot[2]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def _lightning(heads, dim, vdim, decay):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def _moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def _layer(mixer: dict, mlp: Optional[dict]) -> dict:
    return dict(mixer, mlp=mlp)


def config_a() -> dict:
    """Attention first; a reader of its keys two layers on that looks further back than the writer and has no cap;
    grouped heads; a rotation of part of a head with stretched positions; a window that ends inside a page."""
    rot = (16, 5000.0, 4.0)
    return {"architecture": NAME, "vocab": 211, "width": 96, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
            "layers": [
                _layer(_attn(4, 2, 24, 40, 0.4, window=20, cap=5.0, rot=rot), _moe(8, 2, 40)),
                _layer(_lightning(3, 20, 24, (0.5, 0.9, 1.0)), _moe(6, 3, 32)),
                _layer(_attn(4, 2, 24, 40, 0.7, window=37, rot=rot, kv_from=0), None),
                _layer(_lightning(2, 8, 40, (0.97, 0.3)), _moe(5, 5, 16)),
            ]}


def config_b() -> dict:
    """Lightning first; one head everywhere; no window, no cap; a whole head rotated without scaling; a window of one
    token (a token sees itself and the sink); ``top`` of one; a layer without a feed-forward first."""
    return {"architecture": NAME, "vocab": 130, "width": 64, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-3},
            "layers": [
                _layer(_lightning(1, 40, 72, (0.8,)), None),
                _layer(_attn(1, 1, 32, 16, 0.3, rot=(32, 100.0)), _moe(4, 1, 24)),
                _layer(_attn(3, 3, 8, 8, 1.1, window=1, cap=2.0), _moe(3, 2, 8)),
                _layer(_attn(1, 1, 32, 16, 0.2, window=70, cap=30.0, rot=(32, 100.0), kv_from=1), _moe(4, 4, 8)),
            ]}


def config_c() -> dict:
    """Sizes that fit no kernel's favourite multiple: a width of 100, five heads of 12 with values of 36, a rotation of
    six dimensions, windows of exactly one page and of a page and one token, nine experts, feed-forwards of 20."""
    rot = (6, 777.0, 1.5)
    return {"architecture": NAME, "vocab": 77, "width": 100, "embedding": {"scale": 10.0}, "norm": {"eps": 1e-4},
            "layers": [
                _layer(_lightning(5, 36, 12, (0.999, 0.6, 0.9, 0.95, 0.7)), _moe(9, 4, 20)),
                _layer(_attn(5, 5, 12, 36, 0.5, window=64, cap=8.0, rot=rot), _moe(9, 2, 20)),
                _layer(_attn(5, 5, 12, 36, 0.25, window=65, cap=50.0, rot=rot, kv_from=1), _moe(2, 1, 12)),
                _layer(_attn(10, 5, 12, 36, 0.5, window=3, rot=rot, kv_from=1), None),
            ]}


def config_d() -> dict:
    """Head sizes the tensor-core kernels take (64 and 128, equal key and value sizes, even groups): windows that end
    inside the third page and beyond the test's sequences, a reader with a smaller window than the writer."""
    return {"architecture": NAME, "vocab": 150, "width": 128, "embedding": {"scale": 5.0}, "norm": {"eps": 1e-6},
            "layers": [
                _layer(_attn(4, 2, 64, 64, 0.3, window=150, cap=10.0, rot=(32, 20000.0, 2.0)), _moe(4, 2, 32)),
                _layer(_lightning(4, 16, 32, (0.9, 0.95, 0.99, 0.8)), _moe(4, 2, 32)),
                _layer(_attn(8, 2, 128, 128, 0.2, window=1000, cap=15.0, rot=(128, 1e6)), _moe(6, 3, 24)),
                _layer(_attn(4, 2, 64, 64, 0.35, window=70, cap=4.0, rot=(32, 20000.0, 2.0), kv_from=0), _moe(4, 2, 32)),
                _layer(_attn(2, 1, 32, 32, 0.4), _moe(4, 2, 32)),
            ]}


CONFIGS = {"a": config_a, "b": config_b, "c": config_c, "d": config_d}


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    W, out = cfg["width"], {}
    out["embed"] = (cfg["vocab"], W)
    out["head"] = (cfg["vocab"], W)
    out["final.norm"] = (W,)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (W,)
        if layer["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * d, W), p + "mix.q.b": (H * d,), p + "mix.o": (W, H * dv)})
            if "kv_from" not in m:
                out.update({p + "mix.k": (G * d, W), p + "mix.k.b": (G * d,), p + "mix.v": (G * dv, W), p + "mix.v.b": (G * dv,)})
        else:
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * d, W), p + "mix.k": (H * d, W), p + "mix.v": (H * dv, W), p + "mix.g": (H * dv, W),
                        p + "mix.o": (W, H * dv), p + "mix.norm": (H * dv,)})
        if layer["mlp"]:
            out[p + "norm2"] = (W,)
            mlp = layer["mlp"]
            ff, E = mlp["expert"]["ff"], mlp["router"]["experts"]
            for e in range(E):
                out.update({f"{p}mlp.e{e}.gate": (ff, W), f"{p}mlp.e{e}.up": (ff, W), f"{p}mlp.e{e}.down": (W, ff)})
            out.update({p + "mlp.router": (E, W), p + "mlp.router.b": (E,)})
    return out


def random_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if name in ("embed",):
            t = torch.randn(shape, generator=g) / cfg["embedding"]["scale"]
        elif last == "router":
            t = torch.randn(shape, generator=g) * (2.5 / shape[1] ** 0.5)
        elif name.endswith("router.b"):
            t = torch.randn(shape, generator=g) * 0.5 - 1.0            # logits are often all negative
        elif last == "b":
            t = torch.randn(shape, generator=g) * 0.5                  # biases of q, k, v
        elif len(shape) == 2:
            t = torch.randn(shape, generator=g) * (1.4 / shape[1] ** 0.5)
        else:
            t = 1.0 + 0.25 * torch.randn(shape, generator=g)           # norm weights
        out[name] = t.to(torch.bfloat16)
    return out


def write_folder(cfg: dict, weights: Dict[str, torch.Tensor], out_dir: str) -> str:
    from cpmcu_b200.weights.safetensors_io import save_file

    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(out_dir, "model.safetensors"))
    return out_dir


def random_ids(vocab: int, n: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def moe_layers(cfg: dict) -> int:
    return sum(1 for layer in cfg["layers"] if layer["mlp"])


# Largest allowed root mean square of (engine - plain) over the vocabulary, the mean difference taken off, relative to
# the root mean square of the plain logits, for the worst row and for the median row.  float32: summation order only.
# bfloat16: activations between the kernels and the cached keys and values are rounded to bfloat16 in the engine; single
# rows react strongly to that rounding (sharp routers), so the worst row has a loose bound and the median a tight one,
# and float32 carries the exact comparison.
TOL = {"float32": 5e-4, "bfloat16": 0.6}
MEDIAN_TOL = {"float32": 2e-5, "bfloat16": 4e-2}
# A token's choice of experts may fall the other way where two logits nearly tie; the plain implementation uses the
# engine's choice, whose lowest logit must lie this close to the rule's cut-off
CHOICE_SLACK = {"float32": 1e-4, "bfloat16": 0.25}


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
