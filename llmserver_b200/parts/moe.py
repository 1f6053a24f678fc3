"""A routed feed-forward: many small gated experts of which each token uses a few, and an optional shared one."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.declare import WIDE, WeightDecl
from .base import FeedForward
from .registry import FEED_FORWARDS


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    """y = sum over the chosen experts e of w_e * expert_e(x)  (+ shared(x)).

    Router: z = W_r x in 32-bit, s = sigmoid(z).  The ``top`` experts with the largest s + correction are chosen (the
    correction, a learned number per expert, only steers the choice; ties go to the lower index); their weights are
    s * ``route_scale``, not renormalised.  An expert is a gated feed-forward without biases:

        g = min(W_gate x, limit),  u = clamp(W_up x, -limit, limit),  expert(x) = W_down (g * sigmoid(alpha * g) * (u + 1))

    and the shared expert, which every token uses with weight 1, has the same form with sizes and a limit of its own.
    With ``activation`` "silu" an expert is the plain gated layer expert(x) = W_down (silu(W_gate x) * (W_up x)), nothing
    clamped (``limit`` and ``alpha`` are then not given).  With ``weight_on`` "input" a routing weight multiplies what goes
    into its expert instead of what comes out, y = sum_e expert_e(w_e * x): the pair's row is scaled as the first product
    reads it, and the experts' outputs are summed as they are.

    Parameters: ``hidden``, ``experts``, ``top``, ``intermediate``, ``limit``, ``route_scale``; ``alpha`` (default
    1.702); ``correction`` (default True: the router has one); ``shared_intermediate`` and ``shared_limit`` (absent: no
    shared expert).  Tensors behind the part's prefix: ``e<i>.gate``, ``e<i>.up`` [intermediate, hidden], ``e<i>.down``
    [hidden, intermediate], ``router`` [experts, hidden], ``correction`` [experts], ``shared.gate`` / ``.up`` /
    ``.down``.  Router and correction are held in float32 in either path."""

    KNOWN_PARAMS = ("hidden", "experts", "top", "intermediate", "limit", "route_scale", "alpha", "correction",
                    "shared_intermediate", "shared_limit", "activation", "weight_on")
    ACTIVATIONS = ("clamped_swish", "silu")

    @classmethod
    def check_params(cls, params):
        super().check_params(params)
        if not 0 < int(params["top"]) <= int(params["experts"]):
            raise ValueError(f"routed_experts: top {params['top']} must lie in 1..experts ({params['experts']})")
        activation = params.get("activation", "clamped_swish")
        if activation not in cls.ACTIVATIONS:
            raise ValueError(f"routed_experts: unknown activation {activation!r} (known: {', '.join(cls.ACTIVATIONS)})")
        if activation == "silu" and (params.get("limit") is not None or params.get("alpha") is not None or params.get("shared_intermediate")):
            raise ValueError("routed_experts: the plain silu activation takes no limit or alpha, and has no shared expert")
        if activation != "silu" and params.get("limit") is None:
            raise ValueError("routed_experts: the clamped activation needs its limit")
        if params.get("weight_on", "output") not in ("output", "input"):
            raise ValueError(f"routed_experts: weight_on is 'output' or 'input', not {params.get('weight_on')!r}")

    @classmethod
    def declare_weights(cls, params):
        hidden, inter = int(params["hidden"]), int(params["intermediate"])
        wanted = {}
        for e in range(int(params["experts"])):
            wanted[f"e{e}.gate"] = WeightDecl((inter, hidden))
            wanted[f"e{e}.up"] = WeightDecl((inter, hidden))
            wanted[f"e{e}.down"] = WeightDecl((hidden, inter))
        wanted["router"] = WeightDecl((int(params["experts"]), hidden), WIDE)
        if params.get("correction", True):
            wanted["correction"] = WeightDecl((int(params["experts"]),), WIDE)
        if params.get("shared_intermediate"):
            shared = int(params["shared_intermediate"])
            wanted["shared.gate"] = WeightDecl((shared, hidden))
            wanted["shared.up"] = WeightDecl((shared, hidden))
            wanted["shared.down"] = WeightDecl((hidden, shared))
        return wanted

    def __init__(self, params, weights, runtime):
        super().__init__(params, weights, runtime)
        self.experts, self.top = int(params["experts"]), int(params["top"])
        if params.get("activation", "clamped_swish") == "silu":
            # the gated epilogues compute min(g, limit) * sigmoid(alpha * min(g, limit)) * (clamp(u) + shift)
            self.limit, self.alpha, self.gate = float("inf"), 1.0, (float("inf"), 1.0, 0.0)
        else:
            self.limit, self.alpha = float(params["limit"]), float(params.get("alpha", 1.702))
            self.gate = (self.limit, self.alpha)
        self.route_scale = float(params.get("route_scale", 1.0))
        self.weight_on_input = params.get("weight_on", "output") == "input"
        # one tensor per kind of matrix: [E, 2 I, H] with an expert's gate rows in front of its up rows, and [E, H, I]
        self.gate_up = torch.stack([torch.cat([weights[f"e{e}.gate"], weights[f"e{e}.up"]], dim=0)
                                    for e in range(self.experts)]).contiguous()
        self.down = torch.stack([weights[f"e{e}.down"] for e in range(self.experts)]).contiguous()
        self.router = weights["router"].to(torch.float32).contiguous()
        # A router whose weights are bfloat16 numbers (what a bfloat16 checkpoint holds) can be multiplied on the tensor
        # cores without leaving 32-bit arithmetic: products of two bfloat16 numbers are exact in 32-bit, and the sums
        # are 32-bit.  Any other router, and the 32-bit path, use the FMA kernel that makes the choice as well.
        narrow = self.router.to(torch.bfloat16)
        self.router_narrow = narrow.contiguous() if runtime.dtype == torch.bfloat16 and bool((narrow.float() == self.router).all()) else None
        self.correction = weights["correction"].to(torch.float32).contiguous() if params.get("correction", True) else None
        self.shared_gate_up = self.shared_down = None
        if params.get("shared_intermediate"):
            self.shared_gate_up = torch.cat([weights["shared.gate"], weights["shared.up"]], dim=0).contiguous()
            self.shared_down = weights["shared.down"].contiguous()
            self.shared_limit = float(params.get("shared_limit", self.limit))

        # bfloat16 steps of more than a few tokens sort their (token, expert) pairs by expert and run one tiled product
        # over all experts; the 32-bit path and steps of few tokens multiply pair by pair, reading each pair's matrices
        self.grouped = (runtime.dtype == torch.bfloat16 and ops.moe_grouped_supported(self.gate_up, True)
                        and ops.moe_grouped_supported(self.down, False) and self.down.shape[1] % 4 == 0
                        and self.gate_up.shape[2] % 64 == 0 and self.down.shape[2] % 64 == 0)

    GROUPED_FROM = 16     # tokens from which pairs are sorted and multiplied tile by tile

    def forward(self, x):
        tokens = x.shape[0]
        if self.router_narrow is not None:
            logits = ops.linear_wide(x, self.router_narrow)
            chosen, weights = ops.moe_select(logits, self.correction, self.top, self.route_scale)
        else:
            chosen, weights = ops.moe_route(x, self.router, self.correction, self.top, self.route_scale)
        shared = None
        if self.shared_gate_up is not None:
            shared = ops.linear(ops.clamped_glu(ops.linear(x, self.shared_gate_up), self.shared_limit, self.alpha),
                                self.shared_down)
        on_input = weights.view(-1) if self.weight_on_input else None
        if self.weight_on_input:
            weights = self._ones(weights)       # the weights act on the way in; on the way out the outputs are summed
        if self.grouped and tokens >= self.GROUPED_FROM:
            plan = ops.moe_plan(chosen, self.experts)
            hidden = ops.moe_grouped(x, self.gate_up, plan, gather_div=self.top, gated=self.gate, pair_scale=on_input)
            down = ops.moe_grouped(hidden, self.down, plan)
            return ops.moe_combine_rows(down, plan, weights, shared, self.runtime.dtype)
        pairs = tokens * self.top
        index = chosen.view(-1)
        hidden = ops.indexed_linear(x, self.gate_up, index, pairs, in_div=self.top, gated=self.gate, in_scale=on_input)
        down = ops.indexed_linear(hidden, self.down, index, pairs, out_dtype=torch.float32)
        return ops.moe_combine(down, weights, shared, self.runtime.dtype)

    def _ones(self, like):
        """Unit weights of ``like``'s shape (kept: a step's shapes repeat, and a captured step must not allocate anew)."""
        kept = getattr(self, "_unit_weights", None)
        if kept is None or kept.numel() < like.numel():
            kept = self._unit_weights = torch.ones(max(like.numel(), 4096), dtype=torch.float32, device=like.device)
        return kept[:like.numel()].view(like.shape)
