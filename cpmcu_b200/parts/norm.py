"""Norms of the residual stream.

RMS norm (src/model/norm.cuh:7-51): y = x * rsqrt(mean(x^2) + eps) * weight, the weight
used as it is stored (not 1 + weight) unless the part is given an ``offset``.  Layer norm: y = (x - mean) / sqrt(var + eps) * weight + bias with var
the mean of the squared deviations; the reference has none."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import NORMS, Norm, WeightSpec


@NORMS.register("rms_norm")
class RMSNorm(Norm):
    recordable_prompt = True
    takes_two_addends = True        # ``add_forward(..., second=)`` adds two deferred outputs in the norm's own pass

    def __init__(self, ops, hidden_size: int, eps: float, weight_name: str = "weight", offset: float = 0.0):
        """``weight_name``: the tensor's name below the part's prefix.  ``offset``: a constant added to the stored weight
        (1 for a weight that is stored around zero: y = x / rms * (1 + w)); the sum is formed once, in 32-bit."""
        super().__init__(ops)
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)
        self.weight_name = str(weight_name)
        self.offset = float(offset)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.hidden_size,), "vector")}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = tensors[self.weight_name]
        if self.offset:
            w = w.float() + self.offset
        self.weight = self.ops.keep(w.contiguous())

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.ops.add_rmsnorm(x, None, 0.0, self.weight, self.eps, rows)

    def add_forward(self, x: torch.Tensor, delta: torch.Tensor, scale: float,
                    rows: Optional[torch.Tensor] = None, second: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.ops.add_rmsnorm(x, delta, scale, self.weight, self.eps, rows, delta2=second)


@NORMS.register("layer_norm")
class LayerNorm(Norm):
    """Layer norm with weight and bias, computed in 32-bit.  ``weight_name`` / ``bias_name`` are the tensors' names
    below the part's prefix.  Besides the plain forms it offers the two joins that a layer with a norm on both
    sides of each sublayer uses: ``shift_forward`` (norm, then a blend of every token with the token before it)
    and ``add_normed`` (the stream takes the norm of a sublayer's output, and another norm's output of the new
    stream is formed in the same pass)."""

    recordable_prompt = True

    def __init__(self, ops, hidden_size: int, eps: float, weight_name: str = "weight", bias_name: str = "bias"):
        super().__init__(ops)
        self.hidden_size, self.eps = int(hidden_size), float(eps)
        self.weight_name, self.bias_name = str(weight_name), str(bias_name)
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.hidden_size,), "vector"),
                self.bias_name: WeightSpec((self.hidden_size,), "vector")}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = self.ops.keep(tensors[self.weight_name].float().contiguous())
        self.bias = self.ops.keep(tensors[self.bias_name].float().contiguous())

    def weight_bytes(self) -> int:
        return 8 * self.hidden_size

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.ops.layernorm(x, self.weight, self.bias, self.eps, rows)

    def add_forward(self, x: torch.Tensor, delta: torch.Tensor, scale: float,
                    rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if rows is None:
            self.ops.residual_add(x, delta, scale)
            return self.forward(x)
        raise NotImplementedError("layer_norm: a deferred addition cannot be joined with a norm of listed rows")

    def shift_forward(self, ctx, x: torch.Tensor, mix: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
        """h = norm(x); returns h_t + (h_{t-1} - h_t) * mix per token, h_{t-1} of a sequence's first token of the
        step taken from ``state`` [slots, hidden] (zeros at position 0), which then receives the h of the
        sequence's last token."""
        return self.ops.layernorm_shift(ctx, x, self.weight, self.bias, self.eps, mix, state)

    def add_normed(self, x: torch.Tensor, a: torch.Tensor, then: Optional["LayerNorm"] = None) -> Optional[torch.Tensor]:
        """x += norm(a) in place; with ``then``, also returns then(x)."""
        return self.ops.post_norm_add(x, a, self.weight, self.bias, self.eps,
                                      None if then is None else (then.weight, then.bias))


@NORMS.register("scalar_rms_norm")
class ScalarRMSNorm(Norm):
    """RMS norm with one number for all coordinates: y = x / sqrt(mean(x^2) + eps) * g.  The tensor ``weight_name``
    below the part's prefix holds g (no axes).  The plain forms run on the RMS-norm kernel with g spread over the
    width; ``gain`` (one 32-bit float on the device) is what a kernel that norms as part of a larger pass takes."""

    recordable_prompt = True

    def __init__(self, ops, hidden_size: int, eps: float, weight_name: str = "weight"):
        super().__init__(ops)
        self.hidden_size, self.eps = int(hidden_size), float(eps)
        self.weight_name = str(weight_name)
        self.gain: Optional[torch.Tensor] = None
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((), "vector")}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        g = tensors[self.weight_name].float().reshape(1)
        self.gain = self.ops.keep(g.contiguous())
        self.weight = self.ops.keep(g.expand(self.hidden_size).contiguous())

    def weight_bytes(self) -> int:
        return 4

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.ops.add_rmsnorm(x, None, 0.0, self.weight, self.eps, rows)

    def add_forward(self, x: torch.Tensor, delta: torch.Tensor, scale: float,
                    rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.ops.add_rmsnorm(x, delta, scale, self.weight, self.eps, rows)
