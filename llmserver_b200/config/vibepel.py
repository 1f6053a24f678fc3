"""Typed configuration of the Vibepel decoder, read from its own config.json keys.

Vibepel lists its layers one by one.  A layer's mixer is either time mixing with a matrix-valued state ("wkv") or two
mixers side by side whose outputs are joined as a weighted sum ("parallel": attention over a sliding window on the left,
the gated delta rule on the right); its feed-forward, where it has one, is a dense layer without a gate.  Nothing is
assumed equal between layers.

    vocab, width, norm.eps, embedding.scale, logit_softcap
    layers[i].type       "wkv" | "parallel"
    layers[i].mixer      wkv:       heads, dim   (w_rank: optional, else the tensor's shape says)
                         parallel:  left_scale, right_scale,
                                    left:  heads, kv_heads, dim, vdim, scale, mask: {size} | null,
                                           rot: {base, dims, scaling: {factor, low, high, original} | null} | null
                                    right: heads, kv_heads, dim, vdim, conv
    layers[i].mlp        null | {kind: "dense", ff}
"""
from __future__ import annotations

import copy
import json
import os
from dataclasses import dataclass, field
from typing import Optional, Tuple

from .errors import UnsupportedModelError

LAYER_TYPES = ("wkv", "parallel")
FEED_FORWARD_KINDS = ("dense",)


def _need(where: str, raw, *keys):
    if not isinstance(raw, dict):
        raise UnsupportedModelError(f"Vibepel config: {where} must be an object")
    missing = [key for key in keys if raw.get(key) is None]
    if missing:
        raise UnsupportedModelError(f"Vibepel config: {where} lacks {', '.join(missing)}")


def _positive(where: str, raw: dict, *keys):
    for key in keys:
        if int(raw[key]) <= 0:
            raise UnsupportedModelError(f"Vibepel config: {where}.{key} must be positive")


@dataclass(frozen=True)
class VibepelLayer:
    type: str
    mixer: dict
    mlp: Optional[dict]


@dataclass(frozen=True)
class VibepelConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_softcap: float
    layers: Tuple[VibepelLayer, ...]
    eos_token_id: Tuple[int, ...] = ()
    architecture: str = "Vibepel"
    extra: dict = field(default_factory=dict, compare=False)

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    # ---------------------------------------------------------------- parsing
    @classmethod
    def from_dict(cls, raw: dict) -> "VibepelConfig":
        _need("config.json", raw, "vocab", "width", "layers", "norm")
        _need("norm", raw["norm"], "eps")
        _positive("config.json", raw, "vocab", "width")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise UnsupportedModelError("Vibepel config: layers must be a non-empty list")
        layers = []
        for index, entry in enumerate(raw["layers"]):
            where = f"layers[{index}]"
            _need(where, entry, "type", "mixer")
            kind = entry["type"]
            if kind not in LAYER_TYPES:
                raise UnsupportedModelError(f"Vibepel config: {where} has the unknown mixer type {kind!r} "
                                            f"(known: {', '.join(LAYER_TYPES)})")
            mixer = entry["mixer"]
            if kind == "wkv":
                _need(where + ".mixer", mixer, "heads", "dim")
                _positive(where + ".mixer", mixer, "heads", "dim")
            else:
                _need(where + ".mixer", mixer, "left", "right", "left_scale", "right_scale")
                left, right = mixer["left"], mixer["right"]
                _need(where + ".mixer.left", left, "heads", "kv_heads", "dim", "vdim", "scale")
                _need(where + ".mixer.right", right, "heads", "kv_heads", "dim", "vdim", "conv")
                _positive(where + ".mixer.left", left, "heads", "kv_heads", "dim", "vdim")
                _positive(where + ".mixer.right", right, "heads", "kv_heads", "dim", "vdim", "conv")
                for side, part in (("left", left), ("right", right)):
                    if int(part["heads"]) % int(part["kv_heads"]):
                        raise UnsupportedModelError(f"Vibepel config: {where}.mixer.{side}: {part['heads']} heads are no multiple "
                                                    f"of {part['kv_heads']} kv_heads")
                rot = left.get("rot")
                if rot:
                    _need(where + ".mixer.left.rot", rot, "base", "dims")
                    if int(rot["dims"]) % 2 or not 0 < int(rot["dims"]) <= int(left["dim"]):
                        raise UnsupportedModelError(f"Vibepel config: {where}: rot.dims must be even and at most dim")
                    if rot.get("scaling"):
                        _need(where + ".mixer.left.rot.scaling", rot["scaling"], "factor", "low", "high", "original")
                mask = left.get("mask")
                if mask:
                    _need(where + ".mixer.left.mask", mask, "size")
                    _positive(where + ".mixer.left.mask", mask, "size")
            mlp = entry.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "dense") not in FEED_FORWARD_KINDS:
                    raise UnsupportedModelError(f"Vibepel config: {where}.mlp has the unknown kind {mlp.get('kind')!r} "
                                                f"(known: {', '.join(FEED_FORWARD_KINDS)})")
                _need(where + ".mlp", mlp, "ff")
                _positive(where + ".mlp", mlp, "ff")
            layers.append(VibepelLayer(kind, copy.deepcopy(mixer), copy.deepcopy(mlp)))
        embedding = raw.get("embedding") or {}
        softcap = float(raw.get("logit_softcap") or 0.0)
        if softcap < 0:
            raise UnsupportedModelError("Vibepel config: logit_softcap must not be negative")
        eos = raw.get("eos_token_id")
        eos = () if eos is None else ((int(eos),) if isinstance(eos, int) else tuple(int(e) for e in eos))
        known = {"architecture", "architectures", "vocab", "width", "norm", "layers", "embedding", "logit_softcap", "eos_token_id"}
        return cls(vocab=int(raw["vocab"]), width=int(raw["width"]), norm_eps=float(raw["norm"]["eps"]),
                   embedding_scale=float(embedding.get("scale", 1.0)), logit_softcap=softcap, layers=tuple(layers),
                   eos_token_id=eos, extra={key: value for key, value in raw.items() if key not in known})

    @classmethod
    def from_json_file(cls, path: str) -> "VibepelConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as handle:
            return cls.from_dict(json.load(handle))

    def to_dict(self) -> dict:
        """config.json form (round-trips through ``from_dict``)."""
        layers = [{"type": layer.type, "mixer": copy.deepcopy(layer.mixer), "mlp": copy.deepcopy(layer.mlp)} for layer in self.layers]
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "embedding": {"scale": self.embedding_scale}, "logit_softcap": self.logit_softcap, "layers": layers}
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out
