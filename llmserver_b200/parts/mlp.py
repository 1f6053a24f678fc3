"""Dense feed-forwards: SwiGLU, a gated layer with clamped values, and a layer without a gate."""
from __future__ import annotations

import functools

import torch

from .. import ops
from ..weights.declare import WeightDecl
from .base import FeedForward
from .registry import FEED_FORWARDS


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """down(silu(gate(x)) * up(x)) without biases (utils/layers.py:182-218).  gate and up are
    concatenated once at load into one [2 I, H] matrix, gate rows first, as the reference's
    ``fuse_projections`` (utils/layers.py:194-203).  Parameters: ``hidden``, ``intermediate``; ``bias`` must be off
    and ``activation``, if given, "silu"."""

    KNOWN_PARAMS = ("hidden", "intermediate", "bias", "activation")

    @classmethod
    def check_params(cls, params):
        super().check_params(params)
        if params.get("bias"):
            raise ValueError("swiglu has no biases (bias must be absent or false)")
        if params.get("activation", "silu") != "silu":
            raise ValueError(f"swiglu gates with SiLU, not {params['activation']!r}")

    @classmethod
    def declare_weights(cls, params):
        hidden, intermediate = params["hidden"], params["intermediate"]
        return {"gate_proj.weight": WeightDecl((intermediate, hidden)),
                "up_proj.weight": WeightDecl((intermediate, hidden)),
                "down_proj.weight": WeightDecl((hidden, intermediate))}

    def __init__(self, params, weights, runtime):
        super().__init__(params, weights, runtime)
        gate, up = weights["gate_proj.weight"], weights["up_proj.weight"]
        # bfloat16: gate and up rows interleaved in groups of 64, the layout in which the product kernel for few rows
        # can apply the gate itself; the 32-bit path keeps gate rows first
        self.group = ops.GATE_UP_GROUP if gate.dtype == torch.bfloat16 and gate.shape[0] % ops.GATE_UP_GROUP == 0 else 0
        self.gate_up = ops.interleave_gate_up(gate, up) if self.group else torch.cat([gate, up], dim=0).contiguous()
        self.down = weights["down_proj.weight"].contiguous()

    feeds_stream = True

    @functools.cached_property
    def takes_unscaled(self):
        return ops.unscaled_rows_supported(self.gate_up)

    def forward(self, x, sink=None):
        return ops.linear(ops.gate_up_silu(x, self.gate_up, self.group), self.down, sink=sink)


@FEED_FORWARDS.register("clamped_glu")
class ClampedGLU(FeedForward):
    """A dense gated feed-forward whose gate and up values are clamped:

        g = min(W_gate x, limit),  u = clamp(W_up x, -limit, limit),  y = W_down (g * sigmoid(alpha * g) * (u + 1))

    the form the experts of ``routed_experts`` have, as one dense layer.  Parameters: ``hidden``, ``intermediate``,
    ``limit``; ``alpha`` (default 1.702); ``names``: pairs (role, tensor name behind the prefix) for the roles gate, up
    and down.  gate and up are one [2 I, H] matrix, gate rows first; the activation is formed in 32-bit."""

    KNOWN_PARAMS = ("hidden", "intermediate", "limit", "alpha", "names")
    NAMES = {"gate": "gate", "up": "up", "down": "down"}

    @classmethod
    def names(cls, params) -> dict:
        return {**cls.NAMES, **dict(params.get("names") or ())}

    @classmethod
    def declare_weights(cls, params):
        hidden, intermediate = int(params["hidden"]), int(params["intermediate"])
        name = cls.names(params)
        return {name["gate"]: WeightDecl((intermediate, hidden)), name["up"]: WeightDecl((intermediate, hidden)),
                name["down"]: WeightDecl((hidden, intermediate))}

    def __init__(self, params, weights, runtime):
        super().__init__(params, weights, runtime)
        name = self.names(params)
        self.gate_up = torch.cat([weights[name["gate"]], weights[name["up"]]], dim=0).contiguous()
        self.down = weights[name["down"]].contiguous()
        self.limit, self.alpha = float(params["limit"]), float(params.get("alpha", 1.702))

    def forward(self, x):
        return ops.linear(ops.clamped_glu(ops.linear(x, self.gate_up), self.limit, self.alpha), self.down)


@FEED_FORWARDS.register("squared_relu")
class SquaredReLU(FeedForward):
    """A feed-forward without a gate: y = W_down (max(W_up x, 0)^2), no biases.  Parameters: ``hidden``, ``intermediate``;
    ``names``: pairs (role, tensor name behind the prefix) for the roles up and down.  The activation is formed in 32-bit
    from the product's result and rounded once."""

    KNOWN_PARAMS = ("hidden", "intermediate", "names")
    NAMES = {"up": "up", "down": "down"}

    @classmethod
    def names(cls, params) -> dict:
        return {**cls.NAMES, **dict(params.get("names") or ())}

    @classmethod
    def declare_weights(cls, params):
        hidden, intermediate = int(params["hidden"]), int(params["intermediate"])
        name = cls.names(params)
        return {name["up"]: WeightDecl((intermediate, hidden)), name["down"]: WeightDecl((hidden, intermediate))}

    def __init__(self, params, weights, runtime):
        super().__init__(params, weights, runtime)
        name = self.names(params)
        self.up = weights[name["up"]].contiguous()
        self.down = weights[name["down"]].contiguous()

    def forward(self, x):
        return ops.linear(ops.relu_squared(ops.linear(x, self.up)), self.down)
