"""Gated feed-forward layers with unquantised weights: ``down(act(gate x) * (up x))``.

``GatedMLP`` is the dense form (gate and up stacked into one product, the activation fused with the gating product in
one launch); ``TopKRouter`` + ``MixtureOfExperts`` the sparse one: router logits in fp32, the ``top`` largest chosen,
weights either a softmax over the chosen logits or each chosen logit's sigmoid as it is, the chosen experts' outputs
summed with those weights (or, ``weight_on="input"``, each expert run on its weight times the token), optionally plus
a shared expert that every token takes.  Experts are gated or, without ``w_gate``, plain ``down(act(up x))``.  The expert products are grouped GEMMs of the blocks library over a device-built
list of (token, choice) pairs sorted by expert: no host synchronisation, and a token's result does not depend on the
rest of the batch."""

from __future__ import annotations

import torch

from .basics import linear, linear_wide

ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "relu_squared": 2, "clamped_swish": 3}
SCORINGS = {"softmax": 0, "sigmoid": 1, "softmax_all": 2}


class DenseMLP:
    """The ungated feed-forward ``down(act(up x))``; the down projection hands its fp32 accumulator on."""

    def __init__(self, w_up: torch.Tensor, w_down: torch.Tensor, act: str):
        self.w_up, self.w_down, self.act = w_up.contiguous(), w_down.contiguous(), ACTIVATIONS[act]

    def __call__(self, h: torch.Tensor) -> torch.Tensor:
        from extensions_b200.tiny_llm_ext_b200 import blocks

        return linear_wide(blocks.act_rows(linear(h, self.w_up), self.act), self.w_down)


class GatedMLP:
    """``act="clamped_swish"`` (with ``limit`` and ``slope``): ``g = min(gate x, limit)``, ``u = clamp(up x, -limit, limit)``,
    ``down(g sigmoid(slope g) (u + 1))``.  ``b_gate`` / ``b_up`` are added by the first product; ``b_down`` is kept for the
    caller (``down_bias``), who adds it where the residual sum is made."""

    def __init__(self, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, act: str, b_gate=None, b_up=None, b_down=None,
                 limit: float = 0.0, slope: float = 1.0):
        self.w_gate_up = torch.cat([w_gate, w_up], dim=0).contiguous()  # [2 ff, D]: one product for both
        self.w_down = w_down.contiguous()
        self.act = ACTIVATIONS[act]
        if (b_gate is None) != (b_up is None):
            raise ValueError("gated feed-forward: biases on both first projections or on neither")
        self.b_gate_up = None if b_gate is None else torch.cat([b_gate, b_up]).contiguous()
        self.down_bias = None if b_down is None else b_down.contiguous()
        self.limit, self.slope = float(limit), float(slope)
        if act == "clamped_swish" and not self.limit > 0:
            raise ValueError("gated feed-forward: the clamped activation needs a positive limit")

    def __call__(self, h: torch.Tensor, wide: bool = False) -> torch.Tensor:
        """``wide``: hand the down projection's fp32 accumulator back unrounded (when a norm reads it next)."""
        from extensions_b200.tiny_llm_ext_b200 import blocks

        first = linear(h, self.w_gate_up) if self.b_gate_up is None else torch.addmm(self.b_gate_up, h, self.w_gate_up.t())
        return (linear_wide if wide else linear)(blocks.gated_act(first, self.act, self.limit, self.slope), self.w_down)


class TopKRouter:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None, top: int, scoring: str = "softmax", choice_bias: torch.Tensor | None = None,
                 weight_scale: float = 1.0):
        """``scoring="softmax_all"``: scores are a softmax over ALL router outputs, the ``top`` are chosen by score +
        ``choice_bias`` (which the weights do not see), the chosen scores are renormalised and times ``weight_scale``."""
        self.weight, self.bias, self.top = weight.contiguous(), None if bias is None else bias.contiguous(), int(top)
        self.scoring = SCORINGS[scoring]
        self.choice_bias, self.weight_scale = None if choice_bias is None else choice_bias.contiguous(), float(weight_scale)
        if (choice_bias is not None or self.weight_scale != 1.0) and scoring != "softmax_all":
            raise ValueError("router: a choice bias and a weight scale go with scoring='softmax_all'")
        if not 0 < self.top <= weight.shape[0]:
            raise ValueError(f"router: top={top} of {weight.shape[0]} experts")

    def __call__(self, h: torch.Tensor):
        """-> (expert ids int32 [T, top], weights fp32 [T, top])."""
        from extensions_b200.tiny_llm_ext_b200 import blocks

        return blocks.moe_route(h, self.weight, self.bias, self.top, self.scoring, self.choice_bias, self.weight_scale)


class MixtureOfExperts:
    def __init__(self, router: TopKRouter, w_gate: torch.Tensor | None, w_up: torch.Tensor, w_down: torch.Tensor, act: str,
                 shared: GatedMLP | None = None, weight_on: str = "output", identity: int = 0):
        """``w_gate, w_up [E, ff, D]``, ``w_down [E, D, ff]`` (the experts stacked); ``w_gate`` None = experts without a gate.
        ``identity``: the router's last ``identity`` outputs are experts without weights whose output is their input."""
        if weight_on not in ("output", "input"):
            raise ValueError(f"weight_on={weight_on!r}")
        self.identity = int(identity)
        if self.identity < 0 or router.weight.shape[0] != w_up.shape[0] + self.identity:
            raise ValueError(f"router outputs ({router.weight.shape[0]}) != experts ({w_up.shape[0]}) + identity experts ({identity})")
        if self.identity and weight_on == "input":
            raise ValueError("identity experts take the router's weight on their output")
        self.router, self.shared, self.scale_input = router, shared, weight_on == "input"
        self.w_gate, self.w_up, self.w_down = None if w_gate is None else w_gate.contiguous(), w_up.contiguous(), w_down.contiguous()
        self.act = ACTIVATIONS[act]

    def __call__(self, h: torch.Tensor) -> torch.Tensor:
        """-> fp32 [T, D]."""
        from extensions_b200.tiny_llm_ext_b200 import blocks

        idx, gate = self.router(h)
        shared = None if self.shared is None else self.shared(h)
        return blocks.moe_experts(h, idx, gate, self.w_gate, self.w_up, self.w_down, self.act, shared, scale_input=self.scale_input, identity=self.identity > 0)
