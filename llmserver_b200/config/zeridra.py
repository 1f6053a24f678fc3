"""Typed configuration of the Zeridra decoder, read from its own config.json keys.

Zeridra describes itself layer by layer.  A layer has one norm, a mixer and, optionally, a routed feed-forward that both
read that norm's output; its mixer is grouped-query attention whose keys are also its values, or attention through
low-rank latents with a rotating key part, a sliding window and a learned term in the softmax denominator.  A latent
layer may name an earlier latent layer whose cached rows it reads (``kv_from``) instead of making its own.  Nothing is
assumed equal between layers.

    vocab, width, norm.eps, embedding.scale, logit_scale, logit_softcap
    layers[i].type            "attention" | "latent_attention"
    layers[i].mixer           attention:         heads, kv_heads, dim, vdim, scale, q_temp: {coef, every} | null
                              latent_attention:  heads, dim, rot_dim, vdim, q_rank, kv_rank, scale,
                                                 mask: {size} | null, rot: {base, dims} | null, kv_from: absent | index
    layers[i].mlp             null | {kind: "moe", router: {experts, top}, expert: {ff}}
"""
from __future__ import annotations

import copy
import json
import os
from dataclasses import dataclass, field
from typing import Optional, Tuple

from .errors import UnsupportedModelError

MIXER_KEYS = {
    "attention": ("heads", "kv_heads", "dim", "scale"),
    "latent_attention": ("heads", "dim", "vdim", "q_rank", "kv_rank", "scale"),
}
FEED_FORWARD_KINDS = ("moe",)


def _need(where: str, raw, *keys):
    if not isinstance(raw, dict):
        raise UnsupportedModelError(f"Zeridra config: {where} must be an object")
    missing = [key for key in keys if raw.get(key) is None]
    if missing:
        raise UnsupportedModelError(f"Zeridra config: {where} lacks {', '.join(missing)}")


@dataclass(frozen=True)
class ZeridraLayer:
    type: str
    mixer: dict
    mlp: Optional[dict]

    @property
    def kv_from(self) -> Optional[int]:
        named = self.mixer.get("kv_from")
        return None if named is None else int(named)

    @property
    def window(self) -> Optional[int]:
        size = (self.mixer.get("mask") or {}).get("size")
        return int(size) if size else None


@dataclass(frozen=True)
class ZeridraConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    logit_softcap: float
    layers: Tuple[ZeridraLayer, ...]
    eos_token_id: Tuple[int, ...] = ()
    architecture: str = "Zeridra"
    extra: dict = field(default_factory=dict, compare=False)

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    def readers_of(self, index: int):
        """The layers that read the rows layer ``index`` caches (itself not counted)."""
        return [other for other, layer in enumerate(self.layers) if layer.kv_from == index]

    # ---------------------------------------------------------------- parsing
    @classmethod
    def from_dict(cls, raw: dict) -> "ZeridraConfig":
        _need("config.json", raw, "vocab", "width", "layers", "norm")
        _need("norm", raw["norm"], "eps")
        if int(raw["vocab"]) <= 0 or int(raw["width"]) <= 0:
            raise UnsupportedModelError("Zeridra config: vocab and width must be positive")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise UnsupportedModelError("Zeridra config: layers must be a non-empty list")
        layers = []
        for index, entry in enumerate(raw["layers"]):
            where = f"layers[{index}]"
            _need(where, entry, "type", "mixer")
            kind = entry["type"]
            if kind not in MIXER_KEYS:
                raise UnsupportedModelError(f"Zeridra config: {where} has the unknown mixer type {kind!r} "
                                            f"(known: {', '.join(sorted(MIXER_KEYS))})")
            mixer = entry["mixer"]
            _need(where + ".mixer", mixer, *MIXER_KEYS[kind])
            for key in ("heads", "dim"):
                if int(mixer[key]) <= 0:
                    raise UnsupportedModelError(f"Zeridra config: {where}.mixer.{key} must be positive")
            if kind == "attention":
                heads, kv_heads = int(mixer["heads"]), int(mixer["kv_heads"])
                if kv_heads <= 0 or heads % kv_heads:
                    raise UnsupportedModelError(f"Zeridra config: {where}: {heads} heads are no multiple of {kv_heads} kv_heads")
                if mixer.get("vdim") is not None and int(mixer["vdim"]) != int(mixer["dim"]):
                    raise UnsupportedModelError(f"Zeridra config: {where}: the values are the keys, so vdim must equal dim")
                temperature = mixer.get("q_temp")
                if temperature:
                    _need(where + ".mixer.q_temp", temperature, "coef", "every")
                    if int(temperature["every"]) <= 0:
                        raise UnsupportedModelError(f"Zeridra config: {where}: q_temp.every must be positive")
                for key in ("mask", "rot", "kv_from"):
                    if mixer.get(key) is not None:
                        raise UnsupportedModelError(f"Zeridra config: {where}: an attention layer has no {key}")
            else:
                rot_dim = int(mixer.get("rot_dim") or 0)
                if int(mixer["q_rank"]) <= 0 or int(mixer["kv_rank"]) <= 0 or int(mixer["vdim"]) <= 0 or rot_dim < 0:
                    raise UnsupportedModelError(f"Zeridra config: {where}: q_rank, kv_rank and vdim must be positive")
                rot = mixer.get("rot")
                if rot:
                    _need(where + ".mixer.rot", rot, "base", "dims")
                    if int(rot["dims"]) % 2 or not 0 < int(rot["dims"]) <= rot_dim:
                        raise UnsupportedModelError(f"Zeridra config: {where}: rot.dims must be even and at most rot_dim")
                mask = mixer.get("mask")
                if mask:
                    _need(where + ".mixer.mask", mask, "size")
                    if int(mask["size"]) <= 0:
                        raise UnsupportedModelError(f"Zeridra config: {where}: mask.size must be positive")
            mlp = entry.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "moe") not in FEED_FORWARD_KINDS:
                    raise UnsupportedModelError(f"Zeridra config: {where}.mlp has the unknown kind {mlp.get('kind')!r} "
                                                f"(known: {', '.join(FEED_FORWARD_KINDS)})")
                _need(where + ".mlp", mlp, "router", "expert")
                _need(where + ".mlp.router", mlp["router"], "experts", "top")
                _need(where + ".mlp.expert", mlp["expert"], "ff")
                if not 0 < int(mlp["router"]["top"]) <= int(mlp["router"]["experts"]):
                    raise UnsupportedModelError(f"Zeridra config: {where}.mlp: top must lie in 1..experts")
            layers.append(ZeridraLayer(kind, copy.deepcopy(mixer), copy.deepcopy(mlp)))
        for index, layer in enumerate(layers):
            named = layer.kv_from
            if named is None:
                continue
            if not 0 <= named < index:
                raise UnsupportedModelError(f"Zeridra config: layers[{index}].mixer.kv_from names layer {named}, which does not run before it")
            owner = layers[named]
            if owner.type != "latent_attention" or owner.kv_from is not None:
                raise UnsupportedModelError(f"Zeridra config: layers[{index}] reads the cache of layer {named}, which keeps no latents of its own")
            for key in ("kv_rank", "rot_dim"):
                if int(owner.mixer.get(key) or 0) != int(layer.mixer.get(key) or 0):
                    raise UnsupportedModelError(f"Zeridra config: layers[{index}] reads the cache of layer {named}, whose {key} differs")
            if (owner.mixer.get("rot") or None) != (layer.mixer.get("rot") or None):
                raise UnsupportedModelError(f"Zeridra config: layers[{index}] reads the cache of layer {named}, which turns its key part otherwise")
        embedding = raw.get("embedding") or {}
        eos = raw.get("eos_token_id")
        eos = () if eos is None else ((int(eos),) if isinstance(eos, int) else tuple(int(e) for e in eos))
        known = {"architecture", "architectures", "vocab", "width", "norm", "layers", "embedding", "eos_token_id", "logit_scale",
                 "logit_softcap"}
        return cls(vocab=int(raw["vocab"]), width=int(raw["width"]), norm_eps=float(raw["norm"]["eps"]),
                   embedding_scale=float(embedding.get("scale", 1.0)), logit_scale=float(raw.get("logit_scale") or 1.0),
                   logit_softcap=float(raw.get("logit_softcap") or 0.0), layers=tuple(layers), eos_token_id=eos,
                   extra={key: value for key, value in raw.items() if key not in known})

    @classmethod
    def from_json_file(cls, path: str) -> "ZeridraConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as handle:
            return cls.from_dict(json.load(handle))

    def to_dict(self) -> dict:
        """config.json form (round-trips through ``from_dict``)."""
        layers = [{"type": layer.type, "mixer": copy.deepcopy(layer.mixer), "mlp": copy.deepcopy(layer.mlp)} for layer in self.layers]
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale, "layers": layers}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out
