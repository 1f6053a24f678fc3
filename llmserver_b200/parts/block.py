"""Block arrangements: how norms, mixer and feed-forward sit around the residual stream."""
from __future__ import annotations

from .base import Block
import torch

from ..weights.declare import NORM, WeightDecl
from .norm import NormedDelta, ScaledDelta, add_and_read
from .registry import BLOCKS


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    """h += mixer(norm1(h)); h += feed_forward(norm2(h))  (utils/model.py:16-35).

    Each add is fused with the norm that follows it, as the reference's fused dataflow does
    (utils/model.py:87-96): the block receives the stream and the previous sub-layer's output that has
    not been added yet, and returns the stream and its feed-forward's output, still to be added.
    Parameters: the tensor-name prefixes of its four parts (``mixer_prefix`` ...)."""

    KNOWN_PARAMS = ("mixer_prefix", "feed_forward_prefix", "mixer_norm_prefix", "feed_forward_norm_prefix")

    passes_stream = True

    def entry(self):
        return self.mixer_norm, self.mixer

    def forward(self, residual, delta, batch, cache, after=None):
        # With few rows, parts that can do so add their results to the stream themselves and prepare the next norm's
        # input (``sink``), and take a norm's output before its division (``unscaled``); see ``ops.stream``.  Parts
        # and norms that cannot are called as ever.
        normed = _add_norm(self.mixer_norm, residual, delta, self.mixer)
        sink = self.feed_forward_norm.sink(residual, self.feed_forward) if self.mixer.feeds_stream else None
        mixed = self.mixer.forward(normed, batch, cache, sink=sink) if sink is not None else self.mixer.forward(normed, batch, cache)
        normed = _add_norm(self.feed_forward_norm, residual, sink if sink is not None and sink.added else mixed, self.feed_forward)
        sink = after[0].sink(residual, after[1]) if after is not None and self.feed_forward.feeds_stream else None
        out = self.feed_forward.forward(normed, sink=sink) if sink is not None else self.feed_forward.forward(normed)
        return residual, (sink if sink is not None and sink.added else out)


def _add_norm(norm, residual, delta, consumer):
    if getattr(consumer, "takes_unscaled", False) and norm.sink(residual, consumer) is not None:
        return norm.add_norm(residual, delta, unscaled=True)
    return norm.add_norm(residual, delta)


@BLOCKS.register("sandwich_norm")
class SandwichNormBlock(Block):
    """A norm in front of and behind each sub-layer:

        h += mixer_out_norm(mixer(mixer_norm(h)));  h += feed_forward_out_norm(feed_forward(feed_forward_norm(h)))

    A sub-layer's output is not added by itself: it travels on as a ``NormedDelta`` and the next norm's kernel
    normalises it, adds it to the 32-bit stream and normalises the stream in one pass (the model's final norm does the
    same for the last layer).  Parameters: ``feed_forward`` (default True; False: the layer is its mixer alone) and
    the tensor-name prefixes of its parts (``mixer_prefix``, ``mixer_norm_prefix``, ``mixer_out_norm_prefix`` ...)."""

    KNOWN_PARAMS = ("feed_forward", "mixer_prefix", "feed_forward_prefix", "mixer_norm_prefix", "mixer_out_norm_prefix",
                    "feed_forward_norm_prefix", "feed_forward_out_norm_prefix")

    @classmethod
    def roles(cls, params):
        roles = {"mixer": "mixer", "mixer_norm": "norm", "mixer_out_norm": "norm"}
        if params.get("feed_forward", True):
            roles.update({"feed_forward": "feed_forward", "feed_forward_norm": "norm", "feed_forward_out_norm": "norm"})
        return roles

    def forward(self, residual, delta, batch, cache):
        mixed = self.mixer.forward(self.mixer_norm.add_norm(residual, delta), batch, cache)
        pending = NormedDelta(mixed, self.mixer_out_norm)
        if not self.params.get("feed_forward", True):
            return residual, pending
        out = self.feed_forward.forward(self.feed_forward_norm.add_norm(residual, pending))
        return residual, NormedDelta(out, self.feed_forward_out_norm)


@BLOCKS.register("output_norm")
class OutputNormBlock(Block):
    """A norm on each sub-layer's output only; the sub-layers read the stream as it is:

        h += mixer_out_norm(mixer(h));  h += feed_forward_out_norm(feed_forward(h))

    A sub-layer's output travels on as a ``NormedDelta``: the kernel that hands the next sub-layer its input normalises
    it, adds it to the 32-bit stream and returns the updated stream in the activation type (the model's final norm does
    the same for the last layer, followed by its own normalisation).  A mixer that says ``output_bias`` has the bias of
    its last projection added by that kernel, in 32-bit.  Parameters: ``feed_forward`` (default True; False: the layer
    is its mixer alone) and the tensor-name prefixes of its parts."""

    KNOWN_PARAMS = ("feed_forward", "mixer_prefix", "feed_forward_prefix", "mixer_out_norm_prefix", "feed_forward_out_norm_prefix")

    @classmethod
    def roles(cls, params):
        roles = {"mixer": "mixer", "mixer_out_norm": "norm"}
        if params.get("feed_forward", True):
            roles.update({"feed_forward": "feed_forward", "feed_forward_out_norm": "norm"})
        return roles

    def forward(self, residual, delta, batch, cache):
        act = self.mixer.runtime.dtype
        mixed = self.mixer.forward(add_and_read(residual, delta, act), batch, cache)
        pending = NormedDelta(mixed, self.mixer_out_norm, bias=getattr(self.mixer, "output_bias", None))
        if not self.params.get("feed_forward", True):
            return residual, pending
        out = self.feed_forward.forward(add_and_read(residual, pending, act))
        return residual, NormedDelta(out, self.feed_forward_out_norm, bias=getattr(self.feed_forward, "output_bias", None))


@BLOCKS.register("parallel_residual")
class ParallelResidualBlock(Block):
    """One norm whose output both sub-layers read, and one sum:

        n = mixer_norm(h);  h += s1 * mixer(n) + s2 * feed_forward(n)

    with a learned scale per channel on each sub-layer's output (``layer_scale``; without it s1 = s2 = 1).  Nothing is
    added here: both outputs travel on as a ``ScaledDelta`` and the next norm's kernel (the next block's, or the model's
    final norm) multiplies, adds them to the 32-bit stream and normalises it.  Parameters: ``width``; ``feed_forward``
    (default True; False: the layer is its mixer alone); ``layer_scale`` (default False); the tensor-name prefixes of its
    parts (``mixer_prefix``, ``feed_forward_prefix``, ``mixer_norm_prefix``) and, behind the layer's prefix, the names of
    the two scales (``mixer_scale``, ``feed_forward_scale``)."""

    KNOWN_PARAMS = ("width", "feed_forward", "layer_scale", "mixer_prefix", "feed_forward_prefix", "mixer_norm_prefix",
                    "mixer_scale", "feed_forward_scale")

    @classmethod
    def roles(cls, params):
        roles = {"mixer": "mixer", "mixer_norm": "norm"}
        if params.get("feed_forward", True):
            roles["feed_forward"] = "feed_forward"
        return roles

    @classmethod
    def declare_weights(cls, params):
        if not params.get("layer_scale"):
            return {}
        wanted = {params.get("mixer_scale", "mixer_scale"): WeightDecl((int(params["width"]),), NORM)}
        if params.get("feed_forward", True):
            wanted[params.get("feed_forward_scale", "feed_forward_scale")] = WeightDecl((int(params["width"]),), NORM)
        return wanted

    def __init__(self, params, parts, weights=None):
        super().__init__(params, parts)
        device = self.mixer.runtime.device

        def scale(name):
            if params.get("layer_scale"):
                return weights[params.get(name, name)].to(torch.float32).contiguous()
            return torch.ones(int(params["width"]), dtype=torch.float32, device=device)

        self.mixer_scale = scale("mixer_scale")
        self.feed_forward_scale = scale("feed_forward_scale") if params.get("feed_forward", True) else None

    def forward(self, residual, delta, batch, cache):
        normed = self.mixer_norm.add_norm(residual, delta)
        pending = [(self.mixer.forward(normed, batch, cache), self.mixer_scale)]
        if self.params.get("feed_forward", True):
            pending.append((self.feed_forward.forward(normed), self.feed_forward_scale))
        return residual, ScaledDelta(pending)
