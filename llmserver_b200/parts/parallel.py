"""Several mixers side by side on the same input, their outputs joined as a weighted sum."""
from __future__ import annotations

from .. import ops
from ..config.spec import PartSpec
from .base import Mixer
from .registry import MIXERS


@MIXERS.register("parallel_mixers")
class ParallelMixers(Mixer):
    """y = sum_b scale_b * mixer_b(x): every branch is a mixer of this registry with its own parameters, tensors (under
    ``<branch name>.``) and cache (pages, state, or both: the part's cache need is the tuple of its branches' needs, and
    branch b works on ``cache.parts[b]``).  Parameters: ``branches``, a tuple of (name, mixer specification, scale, takes
    the layer's position encoding).  The sum is formed in 32-bit from the branches' outputs and rounded once."""

    KNOWN_PARAMS = ("branches",)

    @classmethod
    def branches(cls, params):
        found = []
        for name, spec, scale, positioned in params["branches"]:
            if not isinstance(spec, PartSpec):
                raise ValueError(f"parallel_mixers: branch {name!r} is no mixer specification")
            found.append((str(name), spec, MIXERS.get(spec.kind), float(scale), bool(positioned)))
        if len(found) < 2:
            raise ValueError("parallel_mixers joins at least two branches")
        return found

    @classmethod
    def check_params(cls, params):
        super().check_params(params)
        for _, spec, mixer_cls, _, _ in cls.branches(params):
            mixer_cls.check_params(spec.as_dict())

    @classmethod
    def declare_weights(cls, params):
        wanted = {}
        for name, spec, mixer_cls, _, _ in cls.branches(params):
            for local, declaration in mixer_cls.declare_weights(spec.as_dict()).items():
                wanted[f"{name}.{local}"] = declaration
        return wanted

    @classmethod
    def cache_need(cls, params):
        return tuple(mixer_cls.cache_need(spec.as_dict()) for _, spec, mixer_cls, _, _ in cls.branches(params))

    def __init__(self, params, weights, runtime):
        super().__init__(params, weights, runtime)
        self.mixers, self.scales, self.positioned = [], [], []
        for name, spec, mixer_cls, scale, positioned in self.branches(params):
            own = {local: weights[f"{name}.{local}"] for local in mixer_cls.declare_weights(spec.as_dict())}
            self.mixers.append(mixer_cls(spec.as_dict(), own, runtime))
            self.scales.append(scale)
            self.positioned.append(positioned)
        self.capturable = all(getattr(mixer, "capturable", True) for mixer in self.mixers)

    def attach(self, position):
        for mixer, positioned in zip(self.mixers, self.positioned):
            mixer.attach(position if positioned else None)

    def forward(self, x, batch, cache):
        outputs = [mixer.forward(x, batch, part) for mixer, part in zip(self.mixers, cache.parts)]
        joined = ops.scaled_sum(outputs[0], self.scales[0], outputs[1], self.scales[1])
        for output, scale in zip(outputs[2:], self.scales[2:]):
            joined = ops.scaled_sum(joined, 1.0, output, scale)
        return joined
