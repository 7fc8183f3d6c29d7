"""Arrangements of a layer's parts around the residual stream."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import BLOCKS, Block, CacheNeeds, ResidualStream, WeightSpec, NORMS, build_part, PartSpec


@BLOCKS.register("pre_norm_residual")
class PreNormResidualBlock(Block):
    """x += s * mixer(norm1(x)); x += s * feed_forward(norm2(x)), with one residual scale s.

    The reference scales each part's output by ``scale_depth / sqrt(layers)`` and adds
    it inside the next norm kernel (src/model/layer.cuh:47-67, src/model/norm.cuh:53-99).
    The scale is a parameter of the block; the block does not know where it comes from.
    """

    recordable_prompt = True

    def __init__(self, ops, mixer, feed_forward, mixer_norm, feed_forward_norm, names,
                 residual_scale: float = 1.0):
        super().__init__(ops, mixer, feed_forward, mixer_norm, feed_forward_norm, names)
        self.residual_scale = float(residual_scale)

    def forward(self, ctx, stream: ResidualStream, lane, writes_cache: bool) -> None:
        y = stream.normed(self.mixer_norm)
        a = self.mixer.forward(ctx, y, lane, writes_cache)
        stream.add(a, self.residual_scale)
        if self.feed_forward is None:
            return                                   # a layer of a mixer alone
        y2 = stream.normed(self.feed_forward_norm)
        f = self.feed_forward.forward(ctx, y2)
        stream.add(f, self.residual_scale)


@BLOCKS.register("parallel_residual")
class ParallelResidualBlock(Block):
    """x += s * (mixer(h) + feed_forward(h)) with h = norm(x): one norm, and both sublayers read its output.  The layer
    has no second norm (``feed_forward_norm`` is None); without a feed-forward it is x += s * mixer(norm(x)).  The two
    outputs are added to the 32-bit stream one after the other inside the next layer's norm kernel."""

    recordable_prompt = True

    def __init__(self, ops, mixer, feed_forward, mixer_norm, feed_forward_norm, names, residual_scale: float = 1.0):
        if feed_forward_norm is not None:
            raise ValueError("parallel_residual: the layer has one norm; its feed-forward reads the mixer's input")
        super().__init__(ops, mixer, feed_forward, mixer_norm, None, names)
        self.residual_scale = float(residual_scale)

    def forward(self, ctx, stream: ResidualStream, lane, writes_cache: bool) -> None:
        h = stream.normed(self.mixer_norm)
        a = self.mixer.forward(ctx, h, lane, writes_cache)
        f = self.feed_forward.forward(ctx, h) if self.feed_forward is not None else None
        stream.add(a, self.residual_scale, second=f)


@BLOCKS.register("sandwich_norm_shift")
class SandwichNormShiftBlock(Block):
    """x += post1(mixer(shift(pre1(x)))); x += post2(feed_forward(pre2(x))): a norm before and after each sublayer,
    and a token shift in front of the mixer.

    The shift blends what the mixer reads with the previous token's: h_t <- h_t + (h_{t-1} - h_t) * mix, element by
    element, h = pre1(x) as it was before the blend and zeros before a sequence's first token.  The previous h is
    per-sequence state of every run of the layer (``shift_prev`` [hidden], 32-bit).  The norms after the sublayers
    (``post_mixer_norm``, ``post_feed_forward_norm``) are parts of this block; their tensors are named by
    ``names["post_mixer_norm"]`` and ``names["post_feed_forward_norm"]``, the blend's vector by ``names["shift"]``.
    The residual sum, the norms and the blend are 32-bit; a sublayer's output is added in the kernel that norms it,
    and where a feed-forward follows, that kernel also forms the feed-forward's input.
    """

    recordable_prompt = True

    def __init__(self, ops, mixer, feed_forward, mixer_norm, feed_forward_norm, names, hidden_size: int,
                 post_norm: PartSpec = None):
        super().__init__(ops, mixer, feed_forward, mixer_norm, feed_forward_norm, names)
        self.hidden_size = int(hidden_size)
        if post_norm is None:
            raise ValueError("sandwich_norm_shift needs the specification of its norms after the sublayers")
        self.post_mixer_norm = build_part(NORMS, post_norm, ops)
        self.post_feed_forward_norm = build_part(NORMS, post_norm, ops) if feed_forward is not None else None
        for n in (mixer_norm, feed_forward_norm, self.post_mixer_norm, self.post_feed_forward_norm):
            if n is not None and not (hasattr(n, "shift_forward") and hasattr(n, "add_normed")):
                raise ValueError("sandwich_norm_shift needs norms that offer shift_forward and add_normed (layer_norm)")
        self.mix: Optional[torch.Tensor] = None

    def sub_parts(self):
        parts = super().sub_parts()
        parts.append((self.names.get("post_mixer_norm", "post_mixer_norm."), self.post_mixer_norm))
        if self.post_feed_forward_norm is not None:
            parts.append((self.names.get("post_feed_forward_norm", "post_feed_forward_norm."), self.post_feed_forward_norm))
        return parts

    def weight_specs(self) -> Dict[str, WeightSpec]:
        out = super().weight_specs()
        out[self.names.get("shift", "shift")] = WeightSpec((self.hidden_size,), "vector")
        return out

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        super().load_weights(tensors)
        self.mix = self.ops.keep(tensors[self.names.get("shift", "shift")].float().contiguous())

    def weight_bytes(self) -> int:
        return super().weight_bytes() + 4 * self.hidden_size

    def cache_needs(self) -> CacheNeeds:
        return self.mixer.cache_needs().with_state({"shift_prev": ((self.hidden_size,), torch.float32)})

    def forward(self, ctx, stream: ResidualStream, lane, writes_cache: bool) -> None:
        x = stream.flush()
        h = self.mixer_norm.shift_forward(ctx, x, self.mix, lane.state["shift_prev"])
        a = self.mixer.forward(ctx, h, lane, writes_cache)
        if self.feed_forward is None:
            self.post_mixer_norm.add_normed(x, a)
            return
        y = self.post_mixer_norm.add_normed(x, a, then=self.feed_forward_norm)
        f = self.feed_forward.forward(ctx, y)
        self.post_feed_forward_norm.add_normed(x, f)


@BLOCKS.register("hyper_connections")
class HyperConnectionsBlock(Block):
    """A layer over several residual streams per token.  Sublayer q (1: mixer, 2: feed-forward) reads one blend of the
    streams and writes into all of them:

        u = sum_s in_q[s] x_s;   y = sublayer_q(norm_q(u));   x_r <- sum_s mix_q[s][r] x_s + out_q[r] y   (all r at once)

    with the layer's tensors ``<names["hyper1"]>in`` [S], ``...out`` [S], ``...mix`` [S, S] (indexed [from][to]), and the
    same under ``names["hyper2"]``.  The norms are RMS norms with one number (``scalar_rms_norm``); the streams and
    everything here are 32-bit.  A sublayer's write is done by the kernel of the next read (of this layer's second
    sublayer, or of the next layer's first), which also norms; the model's output norm sees the sum of the streams.
    """

    recordable_prompt = True

    def __init__(self, ops, mixer, feed_forward, mixer_norm, feed_forward_norm, names, n_streams: int):
        super().__init__(ops, mixer, feed_forward, mixer_norm, feed_forward_norm, names)
        self.n_streams = int(n_streams)
        for n in (mixer_norm, feed_forward_norm):
            if n is not None and not hasattr(n, "gain"):
                raise ValueError("hyper_connections needs norms with one gain (scalar_rms_norm)")
        self.hyper = {}

    def _subs(self):
        return ["hyper1"] + (["hyper2"] if self.feed_forward is not None else [])

    def weight_specs(self) -> Dict[str, WeightSpec]:
        out = super().weight_specs()
        S = self.n_streams
        for sub in self._subs():
            p = self.names.get(sub, sub + ".")
            out[p + "in"] = WeightSpec((S,), "vector")
            out[p + "out"] = WeightSpec((S,), "vector")
            out[p + "mix"] = WeightSpec((S, S), "vector")
        return out

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        super().load_weights(tensors)
        for sub in self._subs():
            p = self.names.get(sub, sub + ".")
            self.hyper[sub] = tuple(self.ops.keep(tensors[p + k].float().contiguous()) for k in ("in", "out", "mix"))

    def weight_bytes(self) -> int:
        return super().weight_bytes() + len(self._subs()) * 4 * (2 * self.n_streams + self.n_streams ** 2)

    def forward(self, ctx, stream: ResidualStream, lane, writes_cache: bool) -> None:
        X = stream.copies
        if X is None or X.shape[1] != self.n_streams:
            raise ValueError(f"hyper_connections: the model carries no {self.n_streams} residual streams (ModelSpec.streams)")
        ops = self.ops
        in1, out1, mix1 = self.hyper["hyper1"]
        h = ops.hyper_step(X, write=stream.pending_write, read=(in1, self.mixer_norm.gain), eps=self.mixer_norm.eps)
        a = self.mixer.forward(ctx, h, lane, writes_cache)
        stream.pending_write = (a, mix1, out1)
        if self.feed_forward is None:
            return
        in2, out2, mix2 = self.hyper["hyper2"]
        h2 = ops.hyper_step(X, write=stream.pending_write, read=(in2, self.feed_forward_norm.gain), eps=self.feed_forward_norm.eps)
        f = self.feed_forward.forward(ctx, h2)
        stream.pending_write = (f, mix2, out2)
