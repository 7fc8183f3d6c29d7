"""Gated feed-forward: down( act(gate(y)) * up(y) ) (src/model/ffn.cuh:18-89).

gate and up are kept as one [2*inter, hidden] matrix so that one product gives both
(src/model/ffn.cuh:47-48 keeps them as [gate | up]; here their rows are interleaved in
blocks of 8 when the size allows); the activation is SiLU in fp32
(src/model/activation.cuh:6-18)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import FEED_FORWARDS, FeedForward, WeightSpec

ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}      # the codes of the activation kernels (csrc/activation.cu)


@FEED_FORWARDS.register("gated_ffn")
class GatedFeedForward(FeedForward):
    recordable_prompt = True

    def __init__(self, ops, hidden_size: int, intermediate_size: int, activation: str = "silu", names=None):
        """``activation``: "silu", or "gelu_tanh" (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))).  ``names``: the three
        matrices' names below the part's prefix, by "gate", "up" and "down" (default: the reference's)."""
        super().__init__(ops)
        if activation not in ACTIVATIONS:
            raise ValueError(f"gated_ffn: activation '{activation}' is not built; known: {sorted(ACTIVATIONS)}")
        self.activation = ACTIVATIONS[activation]
        self.names = dict(names) if names else {}
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.interleave = 0
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        i, h = self.intermediate_size, self.hidden_size
        return {
            self._name("gate"): WeightSpec((i, h)),
            self._name("up"): WeightSpec((i, h)),
            self._name("down"): WeightSpec((h, i)),
        }

    def _name(self, which: str) -> str:
        return self.names.get(which, which + "_proj.weight")

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        gate, up = tensors[self._name("gate")], tensors[self._name("up")]
        i, h = self.intermediate_size, self.hidden_size
        if i % 8 == 0:
            # blocks of 8 gate rows followed by the 8 up rows of the same features: gate and up of a
            # feature then fall into one tile of the product, which can apply the activation itself
            self.interleave = 8
            self.w_gate_up = torch.stack([gate.view(i // 8, 8, h), up.view(i // 8, 8, h)], dim=1).reshape(2 * i, h).contiguous()
        else:
            self.interleave = 0
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_gate_up = self.ops.keep(self.w_gate_up)
        self.w_down = self.ops.keep(tensors[self._name("down")].contiguous())

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_gate_up.element_size()

    def forward(self, ctx, y: torch.Tensor) -> torch.Tensor:
        h = self.ops.gated_linear(y, self.w_gate_up, self.interleave, self.activation)
        return self.ops.linear(h, self.w_down)


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    """A mixture of gated feed-forward experts, of which every token uses ``top``:

        s = softmax(W_router y)  (32-bit);  choice scores c = s + correction
        experts form ``n_groups`` equal groups of neighbours; a group's score is its largest c; only experts of the
        ``keep_groups`` best groups can be chosen; the ``top`` largest c among them are chosen
        out = sum over the chosen e of s_e * down_e( act(gate_e y) * up_e y )            (s_e not renormalised)
            + sigmoid(w_sg . y) * shared(y)                                              (when ``shared_size`` > 0)

    ``scoring`` "top_first" is another rule: the choice scores are the router's logits plus a bias
    (``names["router_bias"]``, [experts]; ``router_bias`` False: none), the ``top`` largest are chosen, and the weights are
    the softmax over the chosen logits only; it has no correction tensor and no groups.

    ``scoring`` "sigmoid": the scores are the sigmoids of the router's logits, the ``top`` largest are chosen and are the
    weights as they are; no correction, bias or groups.  ``expert_form`` "up_relu2": an expert is down_e(relu(up_e x)^2)
    with no gate matrix.  ``weight_on`` "input": out = sum over the chosen e of expert_e(s_e * y), the weight on what the
    expert reads instead of on what it gives (it is applied to the up product's result, which is linear in its input).

    Expert e's matrices are ``<names["expert"]><e>.gate`` / ``.up`` / ``.down``; the shared expert's lie under
    ``names["shared"]`` with its gate vector ``names["shared_gate"]`` [1, hidden].  The router's product (with the
    shared gate's row appended) has 32-bit results; the experts' products run over the (token, expert) pairs grouped
    by expert, on the device, with no host read.
    """

    recordable_prompt = True
    DEFAULT_NAMES = {"router": "router", "correction": "correction", "expert": "e", "gate": ".gate", "up": ".up", "down": ".down",
                     "shared": "shared.", "shared_gate": "shared.sg", "router_bias": "router.b"}
    SCORINGS = ("softmax_first", "top_first", "sigmoid")
    EXPERT_FORMS = ("gated_silu", "up_relu2")

    def __init__(self, ops, hidden_size: int, n_experts: int, top: int, expert_size: int, n_groups: int = 1, keep_groups: int = 1,
                 shared_size: int = 0, names=None, scoring: str = "softmax_first", router_bias: bool = True,
                 expert_form: str = "gated_silu", weight_on: str = "output"):
        super().__init__(ops)
        if scoring not in self.SCORINGS:
            raise ValueError(f"routed_experts: scoring '{scoring}' is not built; known: {list(self.SCORINGS)}")
        if expert_form not in self.EXPERT_FORMS or weight_on not in ("output", "input"):
            raise ValueError(f"routed_experts: expert_form is one of {list(self.EXPERT_FORMS)}, weight_on 'output' or 'input'")
        self.gated = expert_form == "gated_silu"
        self.weight_on_input = weight_on == "input"
        if self.weight_on_input and self.gated:
            raise ValueError("routed_experts: the weight on an expert's input is built for experts without a gate matrix")
        self.sigmoid = scoring == "sigmoid"
        self.top_first = scoring == "top_first"
        self.has_router_bias = self.top_first and bool(router_bias)
        if (self.top_first or self.sigmoid) and int(n_groups) != 1:
            raise ValueError("routed_experts: this choice rule has no groups of experts")
        self.hidden_size, self.E, self.top, self.ff = int(hidden_size), int(n_experts), int(top), int(expert_size)
        self.n_groups, self.keep = int(n_groups), int(keep_groups)
        if self.E % self.n_groups or not 1 <= self.keep <= self.n_groups:
            raise ValueError(f"routed_experts: {self.E} experts do not form {self.n_groups} equal groups of which {self.keep} are kept")
        if not 1 <= self.top <= self.keep * (self.E // self.n_groups):
            raise ValueError(f"routed_experts: top {self.top} exceeds the experts of the kept groups")
        if self.E > 512:
            raise ValueError("routed_experts: the routing kernel takes up to 512 experts")
        self.names = dict(self.DEFAULT_NAMES, **(dict(names) if names else {}))
        self.shared = None
        if shared_size:
            self.shared = GatedFeedForward(ops, hidden_size, shared_size, "silu",
                                           {"gate": "gate", "up": "up", "down": "down"})

    def _expert(self, e: int, which: str) -> str:
        return f"{self.names['expert']}{e}{self.names[which]}"

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n, W, ff = self.names, self.hidden_size, self.ff
        out = {n["router"]: WeightSpec((self.E, W))}
        if not (self.top_first or self.sigmoid):
            out[n["correction"]] = WeightSpec((self.E,), "vector")
        if self.has_router_bias:
            out[n["router_bias"]] = WeightSpec((self.E,), "vector")
        for e in range(self.E):
            if self.gated:
                out[self._expert(e, "gate")] = WeightSpec((ff, W))
            out[self._expert(e, "up")] = WeightSpec((ff, W))
            out[self._expert(e, "down")] = WeightSpec((W, ff))
        if self.shared is not None:
            for name, spec in self.shared.weight_specs().items():
                out[n["shared"] + name] = spec
            out[n["shared_gate"]] = WeightSpec((1, W))
        return out

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        rows = [tensors[n["router"]]] + ([tensors[n["shared_gate"]]] if self.shared is not None else [])
        self.w_router = self.ops.keep(torch.cat(rows, dim=0).contiguous())
        self.correction = self.ops.keep(tensors[n["correction"]].float().contiguous()) if n["correction"] in tensors else None
        self.router_bias = self.ops.keep(tensors[n["router_bias"]].float().contiguous()) if self.has_router_bias else None
        self.w_gate = self.ops.keep(torch.stack([tensors[self._expert(e, "gate")] for e in range(self.E)]).contiguous()) \
            if self.gated else None
        self.w_up = self.ops.keep(torch.stack([tensors[self._expert(e, "up")] for e in range(self.E)]).contiguous())
        self.w_down = self.ops.keep(torch.stack([tensors[self._expert(e, "down")] for e in range(self.E)]).contiguous())
        if self.shared is not None:
            self.shared.load_weights({name: tensors[n["shared"] + name] for name in self.shared.weight_specs()})

    def weight_bytes(self) -> int:
        """What a decode step of one token reads: the router, ``top`` experts, the shared expert."""
        per_expert = (3 if self.gated else 2) * self.ff * self.hidden_size * self.w_up.element_size()
        total = self.w_router.numel() * self.w_router.element_size() + self.top * per_expert
        return total + (self.shared.weight_bytes() if self.shared is not None else 0)

    def forward(self, ctx, y: torch.Tensor) -> torch.Tensor:
        ops = self.ops
        logits = ops.linear(y, self.w_router, out_f32=True)
        chosen, weights, gate = ops.moe_route(logits, self.correction, self.E, self.top, self.n_groups, self.keep,
                                              gate_col=self.E if self.shared is not None else -1, bias=self.router_bias,
                                              top_first=self.top_first, sigmoid=self.sigmoid)
        taps = ctx.extras.get("taps")
        if taps is not None and not ctx.captured and taps.get("experts") is not None:
            taps["experts"].append(chosen.clone())          # a caller that wants to see the choice (tests do)
        pairs = ops.moe_experts(y, chosen, self.w_gate, self.w_up, self.w_down,
                                input_scale=weights if self.weight_on_input else None)
        shared = self.shared.forward(ctx, y) if self.shared is not None else None
        return ops.moe_combine(pairs, None if self.weight_on_input else weights, shared, gate, top=self.top)
