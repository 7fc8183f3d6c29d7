"""A plain, slow implementation of the Kipizen architecture on whole sequences: no cache, no state carried between
calls (except where a caller hands one in), one function per mechanism, float64 by default.  It shares no code with the
package; it reads the raw configuration dictionary and the tensors by their names in the checkpoint.

Notation: T tokens, W the model's width; x [T, W].  ``first`` is the position of the first row where rows are a later
piece of a sequence.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

DT = torch.float64


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rotate_half(x: torch.Tensor, dims: int, base: float, factor: float, first: int = 0) -> torch.Tensor:
    """x [T, heads, d]: column i < dims/2 is paired with column i + dims/2 and the pair turned by the angle
    p * base^(-2i/dims) / factor; columns from ``dims`` on pass unchanged."""
    if not dims:
        return x
    T, half = x.shape[0], dims // 2
    p = torch.arange(first, first + T, dtype=DT)
    f = torch.pow(torch.tensor(float(base), dtype=DT), -2.0 * torch.arange(half, dtype=DT) / dims) / factor
    a = p[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def attention_keys_values(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    """What an attention layer keeps of its input: keys after rotation and unit root mean square, and values."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    rot = m.get("rot") or {}
    k = rotate_half(k, rot.get("dims", 0), rot.get("base", 1.0), (rot.get("scaling") or {}).get("factor", 1.0))
    return rms_norm(k, None, eps), v


def sink_softmax(s: torch.Tensor, visible: torch.Tensor) -> torch.Tensor:
    """Rows of s: exp(s_j) / (1 + sum over the visible j of exp(s_j)): one more, valueless key of score 0."""
    s = s.masked_fill(~visible, float("-inf"))
    m = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - m)
    return e / (torch.exp(-m) + e.sum(-1, keepdim=True))


def window_attention_core(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, cap: float,
                          window: Optional[int], sink: bool = True) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv] of one whole sequence -> [T, H, dv]: scores times ``scale``, capped by
    cap * tanh(s / cap) (``cap`` 0: not capped), key j visible to query i when 0 <= i - j < window (None: j <= i),
    softmax with a sink (or plain)."""
    T, H, G = q.shape[0], q.shape[1], k.shape[1]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    visible = (j <= i) if window is None else (j <= i) & (i - j < window)
    out = []
    for g in range(H):
        s = (q[:, g] @ k[:, g // (H // G)].T) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        if sink:
            pr = sink_softmax(s, visible)
        else:
            pr = torch.softmax(s.masked_fill(~visible, float("-inf")), dim=-1)
        out.append(pr @ v[:, g // (H // G)])
    return torch.stack(out, dim=1)


def window_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, kv=None) -> torch.Tensor:
    """Grouped-query attention with biased projections, a rotation of part of each head, unit-rms queries and keys,
    capped scores, a sliding window and a sink.  ``kv``: another layer's (keys, values) used instead of own ones."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    rot = m.get("rot") or {}
    q = rotate_half(q, rot.get("dims", 0), rot.get("base", 1.0), (rot.get("scaling") or {}).get("factor", 1.0))
    q = rms_norm(q, None, eps)
    k, v = kv if kv is not None else attention_keys_values(h, w, p, m, eps)
    o = window_attention_core(q, k, v, m["scale"], m.get("softcap", 0.0), (m.get("mask") or {}).get("size"))
    return o.reshape(T, H * dv) @ w[p + "o"].T


def lightning_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor,
                         state: Optional[torch.Tensor] = None):
    """q, k [T, H, d], v [T, H, dv], decay [H]: S <- decay S + k v^T, o = S^T q token by token.  Returns (o, last S)."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[-1], dtype=q.dtype) if state is None else state.clone()
    out = torch.empty(T, H, v.shape[-1], dtype=q.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hcv,hc->hv", S, q[t])
    return out, S


def lightning_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).view(T, H, d)
    k = silu(h @ w[p + "k"].T).view(T, H, d)
    v = silu(h @ w[p + "v"].T).view(T, H, dv)
    o, _ = lightning_recurrence(q, k, v, torch.tensor(m["decay"], dtype=h.dtype))
    o = rms_norm(o.reshape(T, H * dv), w[p + "norm"], eps)            # all heads of a token normed together
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def route(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict):
    """(logits [T, E], chosen [T, top], weights [T, top]): the largest logits, softmax over the chosen only."""
    z = h @ w[p + "router"].T + w[p + "router.b"]
    val, idx = torch.topk(z, m["router"]["top"], dim=-1)
    return z, idx, torch.softmax(val, dim=-1)


def expert(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def mixture_of_experts(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, chosen: Optional[torch.Tensor] = None,
                       slack: Optional[list] = None):
    """Returns (output, logits, chosen).  ``chosen`` [T, top]: use these experts instead of the rule's (their weights
    are still the softmax over their own logits); ``slack`` then receives, per token, how far the lowest chosen logit
    lies below the rule's cut-off (0 when the choice is the rule's)."""
    z, idx, wt = route(h, w, p, m)
    if chosen is not None:
        cut = torch.gather(z, 1, idx).min(-1).values
        idx = chosen.long()
        picked = torch.gather(z, 1, idx)
        if slack is not None:
            slack.extend((cut - picked.min(-1).values).clamp_min(0).tolist())
        wt = torch.softmax(picked, dim=-1)
    out = torch.zeros_like(h)
    for e in range(m["router"]["experts"]):
        hit = idx == e
        rows = hit.any(-1)
        if rows.any():
            out[rows] += expert(h[rows], w, f"{p}e{e}.") * (wt * hit)[rows].sum(-1, keepdim=True)
    return out, z, idx


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, chosen: Optional[List[torch.Tensor]] = None, taps: Optional[dict] = None,
            slack: Optional[list] = None):
    """Logits [T, vocab] of a whole sequence.  ``chosen``: per layer with a feed-forward, the experts to use (``slack``:
    see ``mixture_of_experts``).  ``taps``: receives "streams" (x after every layer), "logits" and "chosen" of the routers."""
    w = {k: v.to(DT) if v.is_floating_point() else v for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    kept = {}
    n_ff = 0
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = attention_keys_values(h, w, p + "mix.", m, eps)
            x = x + window_attention(h, w, p + "mix.", m, eps, kv=kept[i if src is None else src])
        elif layer["type"] == "lightning":
            x = x + lightning_attention(h, w, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            h2 = rms_norm(x, w[p + "norm2"], eps)
            f, z, idx = mixture_of_experts(h2, w, p + "mlp.", layer["mlp"], None if chosen is None else chosen[n_ff], slack)
            n_ff += 1
            if taps is not None:
                taps.setdefault("logits", []).append(z)
                taps.setdefault("chosen", []).append(idx)
            x = x + f
        if taps is not None:
            taps.setdefault("streams", []).append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt, n_new: int):
    """(the n_new tokens greedy decoding appends, the gap between the two best logits at every choice)."""
    ids, out, gaps = list(prompt), [], []
    for _ in range(n_new):
        top = torch.topk(forward(cfg, w, ids)[-1], 2)
        out.append(int(top.indices[0]))
        gaps.append(float(top.values[0] - top.values[1]))
        ids.append(out[-1])
    return out, gaps
