"""A plain, slow implementation of the Lukelorn architecture on whole sequences: no cache, no state carried between
calls, one function per mechanism, float64 by default.  It shares no code with the package; it reads the raw
configuration dictionary and the tensors by their names in the checkpoint.

Notation: T tokens, W the model's width; x [T, W]; positions are 0 .. T-1.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

DT = torch.float64
UNIT_EPS = 1e-6


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float, offset: float = 0.0) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * (offset + weight)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * (weight + offset)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def frequencies(rot: dict) -> torch.Tensor:
    """base^(-2i/dims) for i < dims/2, then (with ``scaling``) stretched by wavelength: short waves stay, long waves are
    divided by ``factor``, those between are blended."""
    dims = rot["dims"]
    f = torch.pow(torch.tensor(float(rot["base"]), dtype=DT), -2.0 * torch.arange(dims // 2, dtype=DT) / dims)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        wave = 2.0 * math.pi / f
        blend = (orig / wave - low) / (high - low)
        mid = (1.0 - blend) * f / factor + blend * f
        f = torch.where(wave < orig / high, f, torch.where(wave > orig / low, f / factor, mid))
    return f


def rotate_pairs(x: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """x [T, heads, d]: columns 2i and 2i+1 (i < dims/2) are a pair turned by the angle p * f_i; the rest passes."""
    if not rot or not rot.get("dims"):
        return x
    T, dims = x.shape[0], rot["dims"]
    a = torch.arange(T, dtype=DT)[:, None] * frequencies(rot)[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    turned = torch.stack([u * c - v * s, v * c + u * s], dim=-1).reshape(*x.shape[:-1], dims)
    return torch.cat([turned, x[..., dims:]], dim=-1)


def visible_keys(T: int, window: Optional[int], keep_first: int = 0) -> torch.Tensor:
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & ((i - j < window) | (j < keep_first))
    return seen


def softmax_with_sink(s: torch.Tensor, visible: torch.Tensor, sink: Optional[float]) -> torch.Tensor:
    """Rows of s: exp(s_j) / (exp(sink) + sum over the visible j of exp(s_j)); ``sink`` None: the plain softmax."""
    s = s.masked_fill(~visible, float("-inf"))
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.clamp(m, min=float(sink))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(float(sink) - m)
    return e / den


def attention_core(q, k, v, scale: float, cap: float, window: Optional[int], keep_first: int, sinks) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]."""
    T, H, G = q.shape[0], q.shape[1], k.shape[1]
    seen = visible_keys(T, window, keep_first)
    out = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        out.append(softmax_with_sink(s, seen, None if sinks is None else float(sinks[h])) @ v[:, g])
    return torch.stack(out, dim=1)


def attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rotate_pairs((h @ w[p + "q"].T).view(T, H, d), m.get("rot"))
    k = rotate_pairs((h @ w[p + "k"].T).view(T, G, d), m.get("rot"))
    v = (h @ w[p + "v"].T).view(T, G, dv)
    mask = m.get("mask") or {}
    o = attention_core(q, k, v, m["scale"], m.get("softcap") or 0.0, mask.get("size"), mask.get("keep_first") or 0, w[p + "sink"])
    o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w[p + "o"].T


def short_convolution(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, K] (the last column is the current token's): y_t = sum_j taps[:, K-1-j] x_(t-j)."""
    T, K = x.shape[0], taps.shape[1]
    y = torch.zeros_like(x)
    for j in range(K):
        y[j:] += x[:T - j] * taps[:, K - 1 - j]
    return y


def unit_vectors(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + UNIT_EPS)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def delta_recurrence(q, k, v, beta, g, state: Optional[torch.Tensor] = None):
    """q, k, g [T, H, d], v [T, H, dv], beta [T, H]: S <- g S (rows); u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, H, d = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, d, dv, dtype=q.dtype) if state is None else state.clone()
    out = torch.empty(T, H, dv, dtype=q.dtype)
    for t in range(T):
        S = g[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hcv,hc->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hcv,hc->hv", S, q[t])
    return out, S


def channel_delta(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_convolution(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, d)
    k = silu(short_convolution(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, d)
    v = silu(short_convolution(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
    q = unit_vectors(q) * d ** -0.5
    k = unit_vectors(k)
    rep = H // G
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    dt = softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).view(T, H, d)
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * dt)
    o, _ = delta_recurrence(q, k, v, beta, g)
    o = rms_norm(o, w[p + "norm"], eps)
    o = o * torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, H, dv)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = dict(m.get("rot") or {}, dims=dr) if dr else None
    c_q = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (c_q @ w[p + "uq"].T).view(T, H, d + dr)
    q_plain, q_turn = q[..., :d], rotate_pairs(q[..., d:], rot)
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :R], w[p + "dkv.norm"], eps)
    k_turn = rotate_pairs(down[:, R:].view(T, 1, dr), rot)[:, 0]
    k_plain = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    seen = visible_keys(T, (m.get("mask") or {}).get("size"))
    gate = torch.sigmoid(h @ w[p + "g"].T)
    out = []
    for i in range(H):
        s = (q_plain[:, i] @ k_plain[:, i].T + q_turn[:, i] @ k_turn.T) * m["scale"]
        out.append(softmax_with_sink(s, seen, None) @ v[:, i] * gate[:, i:i + 1])
    return torch.stack(out, dim=1).reshape(T, H * dv) @ w[p + "o"].T


def dense_feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, act: str = "silu") -> torch.Tensor:
    gate = {"silu": silu, "gelu_tanh": gelu_tanh}[act]
    return (gate(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict):
    """(scores [T, E], chosen [T, top], weights [T, top]): sigmoid scores, the largest chosen, used as they are."""
    s = torch.sigmoid(h @ w[p + "router"].T)
    val, idx = torch.topk(s, m["router"]["top"], dim=-1)
    return s, idx, val


def expert(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (torch.relu(h @ w[p + "up"].T) ** 2) @ w[p + "down"].T


def mixture_of_experts(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, chosen: Optional[torch.Tensor] = None,
                       slack: Optional[list] = None):
    """Returns (output, scores, chosen): sum over the chosen experts e of expert_e(s_e * h).  ``chosen`` [T, top]: use
    these experts instead of the rule's; ``slack`` then receives, per token, how far the lowest chosen score lies below
    the rule's cut-off."""
    s, idx, wt = route(h, w, p, m)
    if chosen is not None:
        cut = wt.min(-1).values
        idx = chosen.long()
        wt = torch.gather(s, 1, idx)
        if slack is not None:
            slack.extend((cut - wt.min(-1).values).clamp_min(0).tolist())
    out = torch.zeros_like(h)
    for e in range(m["router"]["experts"]):
        hit = idx == e
        rows = hit.any(-1)
        if rows.any():
            scale = (wt * hit)[rows].sum(-1, keepdim=True)
            out[rows] += expert(h[rows] * scale, w, f"{p}e{e}.")
    return out, s, idx


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, chosen: Optional[List[torch.Tensor]] = None, taps: Optional[dict] = None,
            slack: Optional[list] = None):
    """Logits [T, vocab] of a whole sequence.  ``chosen``: per run of a layer with experts, the experts to use.
    ``taps``: receives "streams" (x after every layer), "scores" and "chosen" of the routers."""
    w = {k: v.to(DT) if v.is_floating_point() else v for k, v in w.items()}
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    n_moe = 0
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', i)}."
        m = layer["mixer"]
        h = rms_norm(x, w[p + "norm1"], eps, offset=1.0)
        if layer["type"] == "attention":
            a = attention(h, w, p + "mix.", m)
        elif layer["type"] == "channel_delta":
            a = channel_delta(h, w, p + "mix.", m, eps)
        elif layer["type"] == "latent_attention":
            a = latent_attention(h, w, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None and mlp["kind"] == "dense":
            a = a + dense_feed_forward(h, w, p + "mlp.", mlp.get("act", "silu"))
        elif mlp is not None:
            f, s, idx = mixture_of_experts(h, w, p + "mlp.", mlp, None if chosen is None else chosen[n_moe], slack)
            n_moe += 1
            if taps is not None:
                taps.setdefault("scores", []).append(s)
                taps.setdefault("chosen", []).append(idx)
            a = a + f
        x = x + mult * a
        if taps is not None:
            taps.setdefault("streams", []).append(x.clone())
    return rms_norm(x, w["final.norm"], eps, offset=1.0) @ w["head"].T


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt, n_new: int):
    """(the n_new tokens greedy decoding appends, the gap between the two best logits at every choice)."""
    ids, out, gaps = list(prompt), [], []
    for _ in range(n_new):
        top = torch.topk(forward(cfg, w, ids)[-1], 2)
        out.append(int(top.indices[0]))
        gaps.append(float(top.values[0] - top.values[1]))
        ids.append(out[-1])
    return out, gaps
