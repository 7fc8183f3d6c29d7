"""Mixers whose memory is a matrix per head that every token decays and adds to (a linear recurrence), instead of
cached keys.  Per head S is [d, dv], 32-bit, zero at a sequence's start, kept per sequence by the cache manager:

    S <- diag(a_t) S;   u = v_t  or  beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t

The projections come from one product with 32-bit results; everything after them (convolution, activations, unit
lengths, gates, decays, the recurrence, the per-head norm) is 32-bit; the gated, normed read-out enters the output
projection in the compute dtype.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import MIXERS, CacheNeeds, Mixer, WeightSpec


class _MatrixStateMixer(Mixer):
    recordable_prompt = True

    def _keep32(self, t: torch.Tensor) -> torch.Tensor:
        return self.ops.keep(t.float().contiguous())

    def cache_bytes_read(self, kv_len: int) -> int:
        return 4 * self.heads * self.d * self.dv


@MIXERS.register("gated_linear_attention")
class GatedLinearAttention(_MatrixStateMixer):
    """Linear attention with a decay per key channel:

        q = Wq h * d^(-1/2),  k = Wk h,  v = Wv h,  a = sigmoid(Wa2 (Wa1 h) + ba2)^(1/tau)      (a: heads x d)
        S_t = diag(a_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t
        out = Wo ( rms_norm_dv(o) * w_norm * silu(Wg h) )                                        (norm per head)

    ``names``: tensors below the part's prefix by "q", "k", "v", "g", "o", "norm", "a1", "a2", "a2_bias".
    """

    DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "a1": "a1", "a2": "a2", "a2_bias": "a2.b"}

    def __init__(self, ops, hidden_size: int, n_heads: int, head_dim: int, value_dim: int, decay_rank: int, tau: float,
                 eps: float, names=None):
        super().__init__(ops)
        self.hidden_size, self.heads, self.d, self.dv = int(hidden_size), int(n_heads), int(head_dim), int(value_dim)
        self.rank, self.tau, self.eps = int(decay_rank), float(tau), float(eps)
        self.names = dict(self.DEFAULT_NAMES, **(dict(names) if names else {}))

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n, W, H, d, dv, r = self.names, self.hidden_size, self.heads, self.d, self.dv, self.rank
        return {n["q"]: WeightSpec((H * d, W)), n["k"]: WeightSpec((H * d, W)), n["v"]: WeightSpec((H * dv, W)),
                n["g"]: WeightSpec((H * dv, W)), n["o"]: WeightSpec((W, H * dv)), n["norm"]: WeightSpec((dv,), "vector"),
                n["a1"]: WeightSpec((r, W)), n["a2"]: WeightSpec((H * d, r)), n["a2_bias"]: WeightSpec((H * d,), "vector")}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        self.w_in = self.ops.keep(torch.cat([tensors[n[x]] for x in ("q", "k", "v", "g")], dim=0).contiguous())
        self.w_a1 = self.ops.keep(tensors[n["a1"]].contiguous())
        self.w_a2 = self.ops.keep(tensors[n["a2"]].contiguous())
        self.w_o = self.ops.keep(tensors[n["o"]].contiguous())
        self.b_a2 = self._keep32(tensors[n["a2_bias"]])
        self.w_norm = self._keep32(tensors[n["norm"]])

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_a1, self.w_a2, self.w_o, self.b_a2, self.w_norm))

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(state={"matrix_state": ((self.heads, self.d, self.dv), torch.float32)})

    def forward(self, ctx, y: torch.Tensor, lane, writes_cache: bool) -> torch.Tensor:
        ops, H, d, dv = self.ops, self.heads, self.d, self.dv
        proj = ops.linear(y, self.w_in, out_f32=True)                       # [q | k | v | g]
        z = ops.linear(ops.linear(y, self.w_a1), self.w_a2, out_f32=True)
        decay = ops.sigmoid_power(z, self.b_a2, self.tau)
        q, k = proj[:, :H * d], proj[:, H * d:2 * H * d]
        v, g = proj[:, 2 * H * d:2 * H * d + H * dv], proj[:, 2 * H * d + H * dv:]
        o = ops.linear_recurrence(ctx, q, k, v, decay, None, lane.state["matrix_state"], H, H, d, dv, d ** -0.5,
                                  vector_decay=True)
        return ops.linear(ops.gated_head_norm(o, g, self.w_norm, self.eps), self.w_o)


@MIXERS.register("gated_delta_rule")
class GatedDeltaRule(_MatrixStateMixer):
    """The gated delta rule with short convolutions:

        q, k, v = silu(conv(Wq h)), silu(conv(Wk h)), silu(conv(Wv h))      conv: causal over time, per channel, K taps
        q, k <- unit length per head (x / sqrt(sum x^2 + 1e-6));  q <- q * d^(-1/2)
        beta = sigmoid(Wb h);   g = exp(-exp(A_log) * softplus(Wa h + dt_bias))                  (one per head)
        S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
        out = Wo ( rms_norm_dv(o) * w_norm * silu(Wg h) )

    q and k have ``n_qk_heads`` heads; value head h uses q/k head h / (heads / qk_heads).  Besides S the last K-1
    inputs of the convolutions are per-sequence state.  ``names``: "q", "k", "v" (their taps under ``<name>.conv``),
    "b", "a", "A_log", "dt_bias", "g", "o", "norm".

    With ``decay_rank`` the decay is one number per head and key channel, acting on the rows of S, through two projections:
    g = exp(-exp(A_log_h) * softplus(Wa2 (Wa1 h) + dt_bias)), laid out heads x d (Wa1 [rank, hidden] ``names["a1"]``, Wa2
    [heads * d, rank] ``names["a2"]``, dt_bias [heads * d]).  With ``gate_rank`` the output gate is gate(Wg2 (Wg1 h))
    (``names["g1"]``, ``names["g2"]``) instead of gate(Wg h); ``gate``: "silu" or "sigmoid".
    """

    DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "conv": ".conv", "b": "b", "a": "a", "A_log": "A_log", "dt_bias": "dt_bias",
                     "g": "g", "o": "o", "norm": "norm", "a1": "a1", "a2": "a2", "g1": "g1", "g2": "g2"}
    UNIT_EPS = 1e-6

    def __init__(self, ops, hidden_size: int, n_heads: int, n_qk_heads: int, head_dim: int, value_dim: int, conv_taps: int,
                 eps: float, names=None, decay_rank: int = 0, gate_rank: int = 0, gate: str = "silu"):
        super().__init__(ops)
        self.decay_rank, self.gate_rank, self.gate = int(decay_rank or 0), int(gate_rank or 0), str(gate)
        if self.gate not in ("silu", "sigmoid"):
            raise ValueError(f"gated_delta_rule: the gate is 'silu' or 'sigmoid', not '{gate}'")
        self.hidden_size, self.heads, self.qk_heads = int(hidden_size), int(n_heads), int(n_qk_heads)
        self.d, self.dv, self.taps, self.eps = int(head_dim), int(value_dim), int(conv_taps), float(eps)
        if self.heads % self.qk_heads:
            raise ValueError(f"{self.heads} value heads cannot be grouped over {self.qk_heads} query/key heads")
        if not 1 <= self.taps <= 8:
            raise ValueError(f"gated_delta_rule: the convolution kernel takes 1 to 8 taps, got {self.taps}")
        self.names = dict(self.DEFAULT_NAMES, **(dict(names) if names else {}))
        self.channels = 2 * self.qk_heads * self.d + self.heads * self.dv

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n, W, H, G, d, dv, K = self.names, self.hidden_size, self.heads, self.qk_heads, self.d, self.dv, self.taps
        out = {n["q"]: WeightSpec((G * d, W)), n["q"] + n["conv"]: WeightSpec((G * d, K), "vector"),
               n["k"]: WeightSpec((G * d, W)), n["k"] + n["conv"]: WeightSpec((G * d, K), "vector"),
               n["v"]: WeightSpec((H * dv, W)), n["v"] + n["conv"]: WeightSpec((H * dv, K), "vector"),
               n["b"]: WeightSpec((H, W)), n["A_log"]: WeightSpec((H,), "vector"), n["o"]: WeightSpec((W, H * dv)),
               n["norm"]: WeightSpec((dv,), "vector")}
        if self.decay_rank:
            out.update({n["a1"]: WeightSpec((self.decay_rank, W)), n["a2"]: WeightSpec((H * d, self.decay_rank)),
                        n["dt_bias"]: WeightSpec((H * d,), "vector")})
        else:
            out.update({n["a"]: WeightSpec((H, W)), n["dt_bias"]: WeightSpec((H,), "vector")})
        if self.gate_rank:
            out.update({n["g1"]: WeightSpec((self.gate_rank, W)), n["g2"]: WeightSpec((H * dv, self.gate_rank))})
        else:
            out[n["g"]] = WeightSpec((H * dv, W))
        return out

    def _fused(self):
        """What the one product of the layer's input gives, in the order of its columns: (name, columns)."""
        H, G, d, dv = self.heads, self.qk_heads, self.d, self.dv
        cols = [("q", G * d), ("k", G * d), ("v", H * dv)]
        if not self.gate_rank:
            cols.append(("g", H * dv))
        cols.append(("b", H))
        if not self.decay_rank:
            cols.append(("a", H))
        if self.gate_rank:
            cols.append(("g1", self.gate_rank))
        if self.decay_rank:
            cols.append(("a1", self.decay_rank))
        return cols

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        self.w_in = self.ops.keep(torch.cat([tensors[n[x]] for x, _ in self._fused()], dim=0).contiguous())
        self.col = {}
        at = 0
        for x, width in self._fused():
            self.col[x] = at
            at += width
        self.w_a2 = self.ops.keep(tensors[n["a2"]].contiguous()) if self.decay_rank else None
        self.w_g2 = self.ops.keep(tensors[n["g2"]].contiguous()) if self.gate_rank else None
        self.w_o = self.ops.keep(tensors[n["o"]].contiguous())
        self.w_taps = self._keep32(torch.cat([tensors[n[x] + n["conv"]].float() for x in ("q", "k", "v")], dim=0))
        self.a_log = self._keep32(tensors[n["A_log"]])
        self.dt_bias = self._keep32(tensors[n["dt_bias"]])
        self.w_norm = self._keep32(tensors[n["norm"]])

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o, self.w_taps, self.a_log, self.dt_bias, self.w_norm,
                                                          self.w_a2, self.w_g2) if t is not None)

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(state={"matrix_state": ((self.heads, self.d, self.dv), torch.float32),
                                 "conv_inputs": ((max(self.taps - 1, 1), self.channels), torch.float32)})

    def cache_bytes_read(self, kv_len: int) -> int:
        return super().cache_bytes_read(kv_len) + 4 * max(self.taps - 1, 1) * self.channels

    def forward(self, ctx, y: torch.Tensor, lane, writes_cache: bool) -> torch.Tensor:
        ops, H, G, d, dv = self.ops, self.heads, self.qk_heads, self.d, self.dv
        col = self.col
        proj = ops.linear(y, self.w_in, out_f32=True)                       # [q | k | v | (g) | b | (a) | (g1) | (a1)]
        q, k, v, beta, decay = ops.conv_prepare(ctx, proj, self.w_taps, lane.state["conv_inputs"], self.a_log, self.dt_bias,
                                                col["b"], col.get("a", 0), H, G, d, dv, self.UNIT_EPS,
                                                head_decay=not self.decay_rank)
        if self.decay_rank:
            # the second projection takes the first's result in the compute dtype; its own result, the softplus, the
            # exponentials and the decay are 32-bit
            low = self._narrow(proj, col["a1"], self.decay_rank)
            decay = ops.channel_decay(ops.linear(low, self.w_a2, out_f32=True), self.a_log, self.dt_bias, H, d)
        o = ops.linear_recurrence(ctx, q, k, v, decay, beta, lane.state["matrix_state"], H, G, d, dv, d ** -0.5,
                                  vector_decay=bool(self.decay_rank))
        if self.gate_rank:
            gate = ops.linear(self._narrow(proj, col["g1"], self.gate_rank), self.w_g2, out_f32=True)
        else:
            gate = proj[:, col["g"]:col["g"] + H * dv]
        return ops.linear(ops.gated_head_norm(o, gate, self.w_norm, self.eps, self.gate), self.w_o)

    def _narrow(self, proj: torch.Tensor, first: int, width: int) -> torch.Tensor:
        """Columns of the fused product as a contiguous operand of the next product (compute dtype)."""
        out = self.ops.empty(proj.shape[0], width)
        out.copy_(proj[:, first:first + width])
        return out


@MIXERS.register("lightning_attention")
class LightningAttention(_MatrixStateMixer):
    """Linear attention with one fixed decay per head:

        q = silu(Wq h),  k = silu(Wk h)   (heads x d),   v = silu(Wv h)   (heads x dv)
        S_t = decay_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t * q_scale
        out = Wo ( rms_norm(o) * w_norm * gate(Wg h) )

    ``norm_heads``: how many heads the norm takes together ("all": the token's heads as one vector with a weight of
    heads * dv numbers; 1: every head alone with a weight of dv numbers).  ``gate``: "sigmoid" or "silu".  The state
    [heads, d, dv] is 32-bit per sequence; activations, decay, recurrence, norm and gate are 32-bit.
    ``names``: "q", "k", "v", "g", "o", "norm".
    """

    DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}

    def __init__(self, ops, hidden_size: int, n_heads: int, head_dim: int, value_dim: int, decay, eps: float,
                 q_scale: float = 1.0, norm_heads="all", gate: str = "sigmoid", names=None):
        super().__init__(ops)
        self.hidden_size, self.heads, self.d, self.dv = int(hidden_size), int(n_heads), int(head_dim), int(value_dim)
        self.decay_values = [float(a) for a in decay]
        if len(self.decay_values) != self.heads:
            raise ValueError(f"lightning_attention: {self.heads} heads need {self.heads} decays, got {len(self.decay_values)}")
        self.eps, self.q_scale, self.gate = float(eps), float(q_scale), str(gate)
        self.group = self.heads if norm_heads == "all" else int(norm_heads)
        if self.heads % self.group:
            raise ValueError(f"lightning_attention: {self.heads} heads cannot be normed in groups of {self.group}")
        self.names = dict(self.DEFAULT_NAMES, **(dict(names) if names else {}))
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=ops.device) if ops is not None else None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n, W, H, d, dv = self.names, self.hidden_size, self.heads, self.d, self.dv
        return {n["q"]: WeightSpec((H * d, W)), n["k"]: WeightSpec((H * d, W)), n["v"]: WeightSpec((H * dv, W)),
                n["g"]: WeightSpec((H * dv, W)), n["o"]: WeightSpec((W, H * dv)), n["norm"]: WeightSpec((self.group * dv,), "vector")}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        self.w_in = self.ops.keep(torch.cat([tensors[n[x]] for x in ("q", "k", "v", "g")], dim=0).contiguous())
        self.w_o = self.ops.keep(tensors[n["o"]].contiguous())
        self.w_norm = self._keep32(tensors[n["norm"]])
        self.decay = self.ops.keep(torch.tensor(self.decay_values, dtype=torch.float32, device=self.w_norm.device))

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o, self.w_norm))

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(state={"matrix_state": ((self.heads, self.d, self.dv), torch.float32)})

    def forward(self, ctx, y: torch.Tensor, lane, writes_cache: bool) -> torch.Tensor:
        ops, H, d, dv = self.ops, self.heads, self.d, self.dv
        proj = ops.linear(y, self.w_in, out_f32=True)                       # [q | k | v | g]
        ops.silu_columns(proj, 2 * H * d + H * dv)
        q, k = proj[:, :H * d], proj[:, H * d:2 * H * d]
        v, g = proj[:, 2 * H * d:2 * H * d + H * dv], proj[:, 2 * H * d + H * dv:]
        decay = self.decay.unsqueeze(0).expand(ctx.n_tokens, H)             # the same row for every token (stride 0)
        o = ops.linear_recurrence(ctx, q, k, v, decay, None, lane.state["matrix_state"], H, H, d, dv, self.q_scale)
        return ops.linear(ops.gated_group_norm(o, g, self.w_norm, self.eps, self.group, self.gate), self.w_o)
