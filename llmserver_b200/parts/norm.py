"""RMSNorm over the residual stream."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..weights.declare import NORM, OFFSET, WeightDecl
from .base import Norm
from .registry import NORMS


@dataclass
class NormedDelta:
    """A sub-layer's output that still has to pass a norm of its own before it joins the stream: the block hands this
    to the next norm's ``add_norm`` in place of a plain delta, and one kernel normalises it, adds it (with ``extra``,
    a second 32-bit stream, when given) and normalises the stream for the next sub-layer.  ``bias``: the bias of the
    projection that made ``delta`` (float32 [width]), which that kernel adds in 32-bit before it normalises."""
    delta: Optional[torch.Tensor]
    norm: Optional["RMSNorm"] = None
    extra: Optional[torch.Tensor] = None
    bias: Optional[torch.Tensor] = None


@dataclass
class ScaledDelta:
    """The outputs of sub-layers that read the same normalised stream and join it together, each through a learned scale
    per channel (float32 [width]): ``parts`` is a list of (output, scale).  The next norm's kernel multiplies, adds all of
    them to the 32-bit stream and normalises it in one pass."""
    parts: list


def add_and_read(residual: torch.Tensor, delta, act_dtype: torch.dtype) -> torch.Tensor:
    """Adds what is pending (a ``NormedDelta`` or nothing) to the 32-bit stream and returns the stream itself in the
    activation type: the input of a sub-layer that reads the stream without a norm in front."""
    if delta is None:
        return ops.normed_add_rmsnorm(residual, None, None, 0.0, None, 0.0, act_dtype=act_dtype)
    if not isinstance(delta, NormedDelta):
        raise TypeError(f"a block that reads the stream as it is takes a NormedDelta or nothing, not {type(delta).__name__}")
    post = delta.norm
    return ops.normed_add_rmsnorm(residual, delta.delta, post.weight, post.eps, None, 0.0, extra=delta.extra,
                                  act_dtype=act_dtype, delta_bias=delta.bias)


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """y = weight * x / sqrt(mean(x^2) + eps) (utils/layers.py:123-138): weight multiplies, it is not
    (1 + weight); no bias.  Parameters: ``width``, ``eps``; ``tensor``: the weight's name behind the part's prefix
    (default "weight"; "" when the prefix is the whole name); ``one_plus`` (default False): the tensor holds the weight's
    distance from one, y = (1 + w) * x / rms: the sum is made once, in 32-bit, when the model is built (in bfloat16 it
    would round the small w away), and the kernels read that 32-bit weight.  Fused with the residual add that precedes
    it, as the reference's add_rms_norm (utils/fused_ops.py:145-155)."""

    KNOWN_PARAMS = ("width", "eps", "tensor", "one_plus")

    @classmethod
    def declare_weights(cls, params):
        return {params.get("tensor", "weight"): WeightDecl((params["width"],), OFFSET if params.get("one_plus") else NORM)}

    def __init__(self, params, weights, runtime):
        super().__init__(params, weights, runtime)
        self.weight = weights[params.get("tensor", "weight")].contiguous()
        if params.get("one_plus"):
            self.weight = (self.weight.to(torch.float32) + 1.0).contiguous()
        self.eps = float(params["eps"])

    def add_norm(self, residual, delta, rows=None, unscaled=False):
        if isinstance(delta, NormedDelta):
            post = delta.norm
            return ops.normed_add_rmsnorm(residual, delta.delta, post.weight if post is not None else None,
                                          post.eps if post is not None else 0.0, self.weight, self.eps,
                                          extra=delta.extra, rows=rows, act_dtype=self.runtime.dtype, delta_bias=delta.bias)
        if isinstance(delta, ScaledDelta):
            (first, first_scale), second = delta.parts[0], (delta.parts[1] if len(delta.parts) > 1 else (None, None))
            for extra, extra_scale in delta.parts[2:]:      # more than two sub-layers: the others join the stream first
                ops.scaled_add_rmsnorm(residual, extra, extra_scale, None, None, None, 0.0, act_dtype=self.runtime.dtype,
                                       want_output=False)
            return ops.scaled_add_rmsnorm(residual, first, first_scale, second[0], second[1], self.weight, self.eps, rows=rows,
                                          act_dtype=self.runtime.dtype)
        if isinstance(delta, ops.StreamSink):
            # the part in front added its result to the stream itself and, if asked, prepared this norm's input
            if delta.owner is not self or not delta.added:
                raise RuntimeError("a stream sink reached a norm that did not make it, or was never used")
            if delta.scaled is not None and rows is None:
                return delta.scaled
            delta = None
        unscaled = unscaled and rows is None and self._few_rows(residual)
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, rows=rows, act_dtype=self.runtime.dtype,
                               unscaled=unscaled)

    def _few_rows(self, residual) -> bool:
        return self.runtime.dtype == torch.bfloat16 and residual.shape[0] <= ops.STREAM_ROWS

    def sink(self, residual, consumer):
        if not self._few_rows(residual) or (consumer is not None and not getattr(consumer, "takes_unscaled", False)):
            return None
        if consumer is None:
            return ops.StreamSink(residual, owner=self)
        return ops.StreamSink(residual, self.weight, self.eps, owner=self)

    def norm(self, x):
        return ops.rmsnorm(x, self.weight, self.eps)
