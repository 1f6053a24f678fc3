"""Vibepel: from its typed configuration to the architecture-neutral model specification.

This is the only place that knows how Vibepel arranges its parts and names its tensors.  Every layer normalises the
output of each sub-layer, with norm weights stored as their distance from one, and lets the sub-layers read the stream as
it is (``output_norm``); its mixer is time mixing with a matrix-valued state (``wkv_time_mix``) or two mixers side by
side (``parallel_mixers``): grouped-query attention over a sliding window with per-head Q/K norms and partly rotated
heads (``gqa_attention``) and the gated delta rule (``gated_delta_rule``); its feed-forward, where it has one, is a
dense layer without a gate (``squared_relu``).  The embedded tokens are scaled as they enter the stream; the head is
the embedding table itself and the logits are capped.

Tensors: ``embed``, ``final.norm``; layer i: ``l<i>.norm1`` (behind the mixer), ``l<i>.norm2`` (behind the
feed-forward), ``l<i>.mix.*`` (a parallel layer's under ``.left.`` and ``.right.``), ``l<i>.mlp.up`` / ``.down``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..config.vibepel import VibepelConfig

ATTENTION_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("q_norm", "q.norm"), ("k_norm", "k.norm"))


def _position_of(left: dict, positions: dict):
    """Name of the position encoding the attention uses (made on first use; equal constants share one)."""
    rot = left.get("rot")
    if not rot:
        return None
    scaling = rot.get("scaling")
    if scaling:
        part = PartSpec.of("banded_rotary", head_dim=int(left["dim"]), theta=float(rot["base"]), rotary_dim=int(rot["dims"]),
                           factor=float(scaling["factor"]), low=float(scaling["low"]), high=float(scaling["high"]),
                           original=float(scaling["original"]))
    else:
        part = PartSpec.of("rotary", head_dim=int(left["dim"]), theta=float(rot["base"]), rotary_dim=int(rot["dims"]))
    for name, known in positions.items():
        if known == part:
            return name
    name = f"rot{len(positions)}"
    positions[name] = part
    return name


def _mixer_of(kind: str, mixer: dict, config: VibepelConfig) -> PartSpec:
    if kind == "wkv":
        # the rank of the decay's first projection is given by its tensor's shape; a configuration may name it
        # ("w_rank") for models whose weights are made rather than read
        rank = mixer.get("w_rank")
        return PartSpec.of("wkv_time_mix", hidden=config.width, heads=int(mixer["heads"]), dim=int(mixer["dim"]),
                           decay_rank=int(rank) if rank else None, eps=config.norm_eps)
    left, right = mixer["left"], mixer["right"]
    mask = left.get("mask") or {}
    attention = PartSpec.of("gqa_attention", hidden=config.width, heads=int(left["heads"]), kv_heads=int(left["kv_heads"]),
                            head_dim=int(left["dim"]), value_dim=int(left["vdim"]), scale=float(left["scale"]), qk_norm=True,
                            eps=config.norm_eps, window=int(mask["size"]) if mask.get("size") else None,
                            precise_weights=True, names=ATTENTION_NAMES)
    delta = PartSpec.of("gated_delta_rule", hidden=config.width, heads=int(right["heads"]), qk_heads=int(right["kv_heads"]),
                        dim=int(right["dim"]), value_dim=int(right["vdim"]), conv=int(right["conv"]), eps=config.norm_eps)
    return PartSpec.of("parallel_mixers", branches=(("left", attention, float(mixer["left_scale"]), True),
                                                    ("right", delta, float(mixer["right_scale"]), False)))


def vibepel_spec(config: VibepelConfig) -> ModelSpec:
    def norm():
        return PartSpec.of("rmsnorm", width=config.width, eps=config.norm_eps, tensor="", one_plus=True)

    positions, layers = {}, []
    for index, layer in enumerate(config.layers):
        feed_forward = None
        if layer.mlp is not None:
            feed_forward = PartSpec.of("squared_relu", hidden=config.width, intermediate=int(layer.mlp["ff"]))
        block = PartSpec.of("output_norm", feed_forward=feed_forward is not None, mixer_prefix="mix.", feed_forward_prefix="mlp.",
                            mixer_out_norm_prefix="norm1", feed_forward_out_norm_prefix="norm2")
        extra = (("mixer_out_norm", norm()),) + ((("feed_forward_out_norm", norm()),) if feed_forward is not None else ())
        layers.append(LayerSpec(prefix=f"l{index}.", block=block, mixer=_mixer_of(layer.type, layer.mixer, config),
                                feed_forward=feed_forward,
                                position=_position_of(layer.mixer["left"], positions) if layer.type == "parallel" else None,
                                extra=extra))
    schedule = [ScheduleEntry(index) for index in range(len(layers))]
    return ModelSpec(architecture=config.architecture, vocab_size=config.vocab, hidden_size=config.width, layers=layers,
                     schedule=schedule, positions=positions, final_norm=norm(), embedding_name="embed",
                     final_norm_prefix="final.norm", head_name="head", tie_head=True, embedding_scale=config.embedding_scale,
                     logit_softcap=config.logit_softcap, eos_token_ids=config.eos_token_id)


register_architecture("Vibepel", VibepelConfig, vibepel_spec)
