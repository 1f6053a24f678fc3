"""The gated delta rule: a matrix-valued state per head that forgets by one decay per head and is corrected, token by
token, towards the value its key should read out."""
from __future__ import annotations

import torch

from .. import ops
from ..cache.manager import StateNeed
from ..weights.declare import NORM, WIDE, WeightDecl
from .base import Mixer
from .registry import MIXERS


@MIXERS.register("gated_delta_rule")
class GatedDeltaRule(Mixer):
    """Per head, with S in R^(dim x value_dim) starting at zero for every request (the recurrence of Yang, Kautz and
    Hatamizadeh, "Gated Delta Networks: Improving Mamba2 with Delta Rule"):

        q, k, v = silu(conv(W_q x)), silu(conv(W_k x)), silu(conv(W_v x))      a short causal convolution per channel
        q <- q / sqrt(sum(q^2) + 1e-6) * dim^(-1/2),  k <- k / sqrt(sum(k^2) + 1e-6)        per head
        beta = sigmoid(W_b x),  g = exp(-exp(A) * softplus(W_a x + dt))         one of each per head
        S <- g S;  d = beta (v - S^T k);  S <- S + k d^T;  o = S^T q
        y = W_o (concat_h(o_h / rms(o_h) * norm) * silu(W_g x))                 norm of value_dim, shared by the heads

    There are ``qk_heads`` query/key heads of ``dim`` and ``heads`` value heads of ``value_dim``; head h reads query/key
    head h // (heads / qk_heads).  Per request the mixer keeps the state, float32 [heads, dim, value_dim], and the last
    ``conv`` - 1 inputs of the convolutions, float32 [conv - 1, channels].  Unit norms, beta, g (from the 32-bit sums of
    their projections on), the recurrence and the head norm are 32-bit in either path.  Parameters: ``hidden``, ``heads``,
    ``qk_heads``, ``dim``, ``value_dim``, ``conv`` (taps), ``eps``; ``names``: pairs (role, tensor name behind the prefix)
    for q, k, v, g, o, b, a, A, dt, norm (a convolution's weights are its projection's name with ".conv" added)."""

    KNOWN_PARAMS = ("hidden", "heads", "qk_heads", "dim", "value_dim", "conv", "eps", "names")
    NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "b": "b", "a": "a", "A": "A_log", "dt": "dt_bias", "norm": "norm"}
    UNIT_EPS = 1e-6

    @classmethod
    def names(cls, params) -> dict:
        given = dict(params.get("names") or ())
        unknown = sorted(set(given) - set(cls.NAMES))
        if unknown:
            raise ValueError(f"gated_delta_rule has no tensor in the role(s) {', '.join(unknown)}")
        return {**cls.NAMES, **given}

    @classmethod
    def check_params(cls, params):
        super().check_params(params)
        if int(params["heads"]) % int(params["qk_heads"]):
            raise ValueError(f"gated_delta_rule: {params['heads']} heads are no multiple of {params['qk_heads']} query/key heads")
        if int(params["conv"]) < 1:
            raise ValueError("gated_delta_rule: the convolution needs at least one tap")

    @classmethod
    def sizes(cls, params):
        heads, qk_heads = int(params["heads"]), int(params["qk_heads"])
        return heads, qk_heads, qk_heads * int(params["dim"]), heads * int(params["value_dim"])

    @classmethod
    def declare_weights(cls, params):
        hidden, taps = int(params["hidden"]), int(params["conv"])
        heads, _, keys, values = cls.sizes(params)
        name = cls.names(params)
        return {name["q"]: WeightDecl((keys, hidden)), name["q"] + ".conv": WeightDecl((keys, taps), WIDE),
                name["k"]: WeightDecl((keys, hidden)), name["k"] + ".conv": WeightDecl((keys, taps), WIDE),
                name["v"]: WeightDecl((values, hidden)), name["v"] + ".conv": WeightDecl((values, taps), WIDE),
                name["b"]: WeightDecl((heads, hidden)), name["a"]: WeightDecl((heads, hidden)),
                name["A"]: WeightDecl((heads,), WIDE), name["dt"]: WeightDecl((heads,), WIDE),
                name["norm"]: WeightDecl((int(params["value_dim"]),), NORM), name["g"]: WeightDecl((values, hidden)),
                name["o"]: WeightDecl((hidden, values))}

    @classmethod
    def cache_need(cls, params):
        heads, _, keys, values = cls.sizes(params)
        return (StateNeed((heads, int(params["dim"]), int(params["value_dim"])), "float32"),
                StateNeed((max(int(params["conv"]) - 1, 1), 2 * keys + values), "float32"))

    def __init__(self, params, weights, runtime):
        super().__init__(params, weights, runtime)
        self.heads, self.qk_heads, self.keys, self.values = self.sizes(params)
        self.dim, self.value_dim, self.eps = int(params["dim"]), int(params["value_dim"]), float(params["eps"])
        if not ops.matrix_recurrence_supported(self.dim, self.value_dim):
            raise ValueError(f"gated_delta_rule: no kernel for heads of {self.dim} key and {self.value_dim} value channels")
        name = self.names(params)
        self.fused = torch.cat([weights[name[role]] for role in ("q", "k", "v", "g")], dim=0).contiguous()
        self.taps = torch.cat([weights[name[role] + ".conv"].to(torch.float32) for role in ("q", "k", "v")], dim=0).contiguous()
        self.steps = torch.cat([weights[name["b"]], weights[name["a"]]], dim=0).contiguous()       # beta's and g's projections
        self.a_log = weights[name["A"]].to(torch.float32).contiguous()
        self.dt_bias = weights[name["dt"]].to(torch.float32).contiguous()
        self.norm = weights[name["norm"]].contiguous()
        self.out = weights[name["o"]].contiguous()

    def forward(self, x, batch, cache):
        state, history = cache.parts[0].state, cache.parts[1].state
        proj = ops.linear(x, self.fused)
        wide = ops.linear_wide(x, self.steps)       # 32-bit sums: what becomes a decay or a step size is never rounded to 16 bits
        pre = ops.short_conv_units(proj, 0, self.taps, history, batch, 2 * self.qk_heads, self.dim, self.qk_heads, self.heads,
                                   self.value_dim, self.UNIT_EPS, self.dim ** -0.5)
        mixed = ops.delta_rule_recurrent(proj, 2 * self.keys + self.values, pre, wide, self.a_log, self.dt_bias, self.norm, state,
                                         batch, self.heads, self.qk_heads, self.dim, self.value_dim, self.eps)
        return ops.linear(mixed, self.out)
