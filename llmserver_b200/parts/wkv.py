"""Time mixing with a per-channel decay: every projection reads its own mix of a token with the one before it, and a
matrix-valued state per head carries the past."""
from __future__ import annotations

import torch

from .. import ops
from ..cache.manager import StateNeed
from ..weights.declare import NORM, WIDE, WeightDecl
from .base import Mixer
from .registry import MIXERS


@MIXERS.register("wkv_time_mix")
class WKVTimeMix(Mixer):
    """With h' the input row of the token before (zeros at a sequence's start) and S in R^(dim x dim) per head, starting
    at zero for every request (the time mixing of Peng et al., "Eagle and Finch: RWKV with Matrix-Valued States and
    Dynamic Recurrence", in the form whose mixing vectors are fixed):

        x_s = h + (h' - h) * mu_s                                    s in r, k, v, g, w
        r, k, v = W_r x_r, W_k x_k, W_v x_v;   gate = silu(W_g x_g)
        w = exp(-exp(W_w2 tanh(W_w1 x_w) + w0))                      one decay per head and key channel
        o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t;   S_t = diag(w_t) S_(t-1) + k_t v_t^T
        y = W_o (concat_h(o_h / rms(o_h)) * norm * gate)             norm of heads * dim

    Per request the mixer keeps two things: the state, float32 [heads, dim, dim], and the last input row, float32
    [hidden].  The decay (from the 32-bit sums of its second projection on), the bonus u and the recurrence are 32-bit in
    either path; the projections and the mixes run in the activation type.  Parameters: ``hidden``, ``heads``, ``dim``,
    ``decay_rank`` (rows of W_w1; None: the tensor's shape says), ``eps``; ``names``: pairs (role, tensor name behind the
    prefix) for r, k, v, g, o, w1, w2, w0, u, norm and mu (the mixing vectors are mu's name with ".r", ".k" ... added)."""

    KNOWN_PARAMS = ("hidden", "heads", "dim", "decay_rank", "eps", "names")
    NAMES = {"r": "r", "k": "k", "v": "v", "g": "g", "o": "o", "w1": "w1", "w2": "w2", "w0": "w0", "u": "u", "norm": "norm", "mu": "mu"}
    MIXES = ("r", "k", "v", "g", "w")

    @classmethod
    def names(cls, params) -> dict:
        given = dict(params.get("names") or ())
        unknown = sorted(set(given) - set(cls.NAMES))
        if unknown:
            raise ValueError(f"wkv_time_mix has no tensor in the role(s) {', '.join(unknown)}")
        return {**cls.NAMES, **given}

    @classmethod
    def declare_weights(cls, params):
        hidden, inner = int(params["hidden"]), int(params["heads"]) * int(params["dim"])
        rank = int(params["decay_rank"]) if params.get("decay_rank") else -1      # -1: whatever the checkpoint holds
        name = cls.names(params)
        wanted = {f"{name['mu']}.{mix}": WeightDecl((hidden,), WIDE) for mix in cls.MIXES}
        wanted.update({name[role]: WeightDecl((inner, hidden)) for role in ("r", "k", "v", "g")})
        wanted.update({name["w1"]: WeightDecl((rank, hidden)), name["w2"]: WeightDecl((inner, rank)),
                       name["w0"]: WeightDecl((inner,), WIDE), name["u"]: WeightDecl((int(params["heads"]), int(params["dim"])), WIDE),
                       name["norm"]: WeightDecl((inner,), NORM), name["o"]: WeightDecl((hidden, inner))})
        return wanted

    @classmethod
    def cache_need(cls, params):
        heads, dim = int(params["heads"]), int(params["dim"])
        return (StateNeed((heads, dim, dim), "float32"), StateNeed((int(params["hidden"]),), "float32"))

    def __init__(self, params, weights, runtime):
        super().__init__(params, weights, runtime)
        self.heads, self.dim, self.eps = int(params["heads"]), int(params["dim"]), float(params["eps"])
        if not ops.matrix_recurrence_supported(self.dim, self.dim):
            raise ValueError(f"wkv_time_mix: no kernel for heads of {self.dim} channels")
        name = self.names(params)
        self.mu = torch.stack([weights[f"{name['mu']}.{mix}"].to(torch.float32) for mix in self.MIXES]).contiguous()
        self.projections = [weights[name[role]].contiguous() for role in ("r", "k", "v", "g")]
        self.decay_in, self.decay_out = weights[name["w1"]].contiguous(), weights[name["w2"]].contiguous()
        self.decay_offset = weights[name["w0"]].to(torch.float32).contiguous()
        self.bonus = weights[name["u"]].to(torch.float32).contiguous()
        self.norm = weights[name["norm"]].contiguous()
        self.out = weights[name["o"]].contiguous()

    def forward(self, x, batch, cache):
        state, shift = cache.parts[0].state, cache.parts[1].state
        mixes = ops.token_shift_mix(x, shift, batch, self.mu)
        inner = self.heads * self.dim
        rkvg = torch.empty((4, x.shape[0], inner), dtype=x.dtype, device=x.device)
        for index, weight in enumerate(self.projections):
            ops.linear(mixes[index], weight, out=rkvg[index])
        # the decay's pre-activation keeps its 32-bit sums; tanh is formed on the first projection's 32-bit sums
        z = ops.linear_wide(ops.tanh_narrow(ops.linear_wide(mixes[4], self.decay_in), x.dtype), self.decay_out)
        mixed = ops.wkv_recurrent(rkvg, z, self.decay_offset, self.bonus, self.norm, state, batch, self.heads, self.dim, self.eps,
                                  h=x, shift_state=shift)
        return ops.linear(mixed, self.out)
