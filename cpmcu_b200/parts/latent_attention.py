"""Attention whose keys and values are linear maps of one cached latent per token."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import MIXERS, POSITIONS, CacheNeeds, Mixer, PartSpec, WeightSpec, build_part


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """Queries go through a latent, c_q = rms(Wdq h) * g_q and q = Wuq c_q; keys and values come from a second latent,
    c = rms(Wdkv h) * g_kv (``kv_rank`` values), as k = Wuk c and v = Wuv c, head by head.  No position enters.
    score = (q . k) * scale; a query at position i sees the keys j with 0 <= i - j < window (window None: all
    j <= i); softmax; the heads' outputs go through Wo.

    Only c is cached: one row of ``kv_rank`` values per token, whatever the number of heads.  The attention runs on
    the cached latents themselves, with Wuk moved to the query side (q'_h = Wuk_h^T q_h, so q'_h . c = q_h . k_h) and
    Wuv applied to the weighted sum of latents (Wuv_h sum_j p_j c_j = sum_j p_j v_j): the same arithmetic serves a
    prompt, a portion of one and a single decoded token, and nothing is decompressed.  Norms, scores, softmax and the
    weighted sum are 32-bit, and so are q' and the weighted latents between the kernels.  ``names``: the tensors'
    names below the part's prefix, by "dq", "dq_norm", "uq", "dkv", "dkv_norm", "uk", "uv", "o", "gate".

    With ``rot_dim`` > 0 every query head has ``rot_dim`` further channels behind its ``head_dim`` plain ones (Wuq has
    heads * (head_dim + rot_dim) rows) and Wdkv ``rot_dim`` further rows behind the latent's: one key part per token,
    shared by all heads and not normed.  Both are turned by ``position`` (a rotation of pairs over all ``rot_dim``
    channels) and the score is (q_plain . k_plain + q_turned . k_turned) * scale.  The cached row of a token is then
    [c | turned key part], the query in latent space [Wuk_h^T q_plain | q_turned], and the turned part's columns of the
    weighted sum of rows are dropped by the value map (zero rows in its matrix): still one row per token, nothing
    decompressed.  With ``gate`` head h's output is multiplied by sigmoid(Wg h)_h before Wo.
    """

    recordable_prompt = True

    DEFAULT_NAMES = {"dq": "dq.weight", "dq_norm": "dq_norm.weight", "uq": "uq.weight", "dkv": "dkv.weight",
                     "dkv_norm": "dkv_norm.weight", "uk": "uk.weight", "uv": "uv.weight", "o": "o.weight", "gate": "g"}

    def __init__(self, ops, hidden_size: int, n_heads: int, head_dim: int, value_dim: int, q_rank: int, kv_rank: int,
                 softmax_scale: float, eps: float, window: Optional[int] = None, names=None, rot_dim: int = 0,
                 position: Optional[PartSpec] = None, gate: bool = False):
        super().__init__(ops)
        self.hidden_size, self.n_heads, self.d, self.vd = int(hidden_size), int(n_heads), int(head_dim), int(value_dim)
        self.q_rank, self.kv_rank = int(q_rank), int(kv_rank)
        self.scale, self.eps = float(softmax_scale), float(eps)
        self.window = int(window) if window else 0
        self.rot_dim, self.gate = int(rot_dim or 0), bool(gate)
        self.row = self.kv_rank + self.rot_dim                    # what the cache keeps of a token
        if self.row > 1024:
            raise ValueError(f"latent_attention: a cached row of {self.row} values is beyond the 1,024 the attention kernels keep per head")
        self.inv_freq, self.adjacent = None, False
        if self.rot_dim:
            if position is None:
                raise ValueError("latent_attention: a rotated part needs a position encoding")
            enc = build_part(POSITIONS, position, ops)
            rot = enc.rotary()
            if rot is None or rot[1] != 1.0 or rot[2] != self.rot_dim:
                raise ValueError("latent_attention: the position encoding must be a rotation of pairs over all rot_dim channels")
            self.inv_freq, self.adjacent = rot[0], bool(getattr(enc, "adjacent", False))
        self.names = dict(self.DEFAULT_NAMES, **(dict(names) if names else {}))
        self.w_down = self.w_uq = self.w_uk = self.w_uv = self.w_o = self.g_q = self.g_kv = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n, H, h = self.names, self.n_heads, self.hidden_size
        out = {n["dq"]: WeightSpec((self.q_rank, h)), n["dq_norm"]: WeightSpec((self.q_rank,), "vector"),
               n["uq"]: WeightSpec((H * (self.d + self.rot_dim), self.q_rank)), n["dkv"]: WeightSpec((self.row, h)),
               n["dkv_norm"]: WeightSpec((self.kv_rank,), "vector"), n["uk"]: WeightSpec((H * self.d, self.kv_rank)),
               n["uv"]: WeightSpec((H * self.vd, self.kv_rank)), n["o"]: WeightSpec((h, H * self.vd))}
        if self.gate:
            out[n["gate"]] = WeightSpec((H, h))
        return out

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        n, H, keep = self.names, self.n_heads, self.ops.keep
        down = [tensors[n["dq"]], tensors[n["dkv"]]] + ([tensors[n["gate"]]] if self.gate else [])
        self.w_down = keep(torch.cat(down, dim=0).contiguous())      # one product for both latents (and the gates' logits)
        self.w_uq = keep(tensors[n["uq"]].contiguous())
        # per head [k][n] matrices for in[t, h, :] @ w[h]: Wuk_h is [dim, rank] as stored; Wuv_h [vdim, rank] is transposed
        uk = tensors[n["uk"]].view(H, self.d, self.kv_rank)
        uv = tensors[n["uv"]].view(H, self.vd, self.kv_rank).transpose(1, 2)
        if self.rot_dim:
            # the turned channels pass from the query into latent space as they are (an identity block), and the value map
            # has zero rows for the turned part of a weighted sum of cached rows
            r = self.rot_dim
            wide = torch.zeros(H, self.d + r, self.row, dtype=uk.dtype, device=uk.device)
            wide[:, :self.d, :self.kv_rank] = uk
            wide[:, self.d:, self.kv_rank:] = torch.eye(r, dtype=uk.dtype, device=uk.device)
            tall = torch.zeros(H, self.row, self.vd, dtype=uv.dtype, device=uv.device)
            tall[:, :self.kv_rank] = uv
            uk, uv = wide, tall
        self.w_uk = keep(uk.contiguous())
        self.w_uv = keep(uv.contiguous())
        self.w_o = keep(tensors[n["o"]].contiguous())
        self.g_q = keep(tensors[n["dq_norm"]].float().contiguous())
        self.g_kv = keep(tensors[n["dkv_norm"]].float().contiguous())

    def weight_bytes(self) -> int:
        mats = (self.w_down, self.w_uq, self.w_uk, self.w_uv, self.w_o)
        return sum(m.numel() for m in mats) * self.w_o.element_size() + 4 * (self.q_rank + self.kv_rank)

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(kv_heads=1, head_dim=self.row, window=self.window or None, values=False)

    def cache_bytes_read(self, kv_len: int) -> int:
        keys = min(kv_len, self.window) if self.window else kv_len
        return keys * self.row * self.ops.element_size

    def forward(self, ctx, y: torch.Tensor, lane, writes_cache: bool) -> torch.Tensor:
        ops = self.ops
        ops.set_page_limit(lane.k.shape[0])
        H = self.n_heads
        down = ops.linear(y, self.w_down, out_f32=True)                 # [tokens, q_rank + kv_rank (+ rot_dim) (+ heads)], 32-bit
        c_q = ops.latent_norm_store(ctx, down, self.g_q, self.g_kv, lane, self.q_rank, self.kv_rank, self.eps, writes_cache,
                                    rot_dim=self.rot_dim, inv_freq=self.inv_freq, adjacent=self.adjacent)
        if self.rot_dim:
            q = ops.rotate_heads(ctx, ops.linear(c_q, self.w_uq, out_f32=True), H, self.d, self.rot_dim, self.inv_freq,
                                 self.adjacent)                                          # [tokens, heads * (dim + rot_dim)]
        else:
            q = ops.linear(c_q, self.w_uq)                                               # [tokens, heads * dim]
        q_lat = ops.head_project(q, self.w_uk, H, out_f32=True)                          # [tokens, heads, row], 32-bit
        # [tokens, heads, row]: 32-bit, unless the map that follows is a library product of many tokens, which takes bf16
        narrow = ops.head_project_by_library(ctx.n_tokens) and ops.latent_attention_on_tensor_cores(self.row)
        o_lat = ops.latent_attention(ctx, q_lat, lane, self.scale, self.window, out_compute_dtype=narrow)
        o = ops.head_project(o_lat, self.w_uv, H, out_f32=False).view(ctx.n_tokens, H * self.vd)
        if self.gate:
            ops.head_gate(o, down[:, down.shape[1] - H:], H)
        return ops.linear(o, self.w_o)
