"""Zeridra: from its typed configuration to the architecture-neutral model specification.

This is the only place that knows how Zeridra arranges its parts and names its tensors.  Every layer is a
``parallel_residual`` block with a scale per channel on each sub-layer's output; its mixer is ``gqa_attention`` in the form
without a value projection (keys are values, a unit sink, a query temperature) or ``latent_attention`` with a rotating
key part, a window and learned sinks; its feed-forward, where it has one, is ``routed_experts`` with plain silu experts
whose routing weight acts on the expert's input.  A latent layer that names another one's cache becomes a schedule entry
that reads that entry's pages.  The embedded tokens are scaled as they enter the stream; the logits are scaled and capped.

Tensors: ``embed``, ``head``, ``final.norm``; layer i: ``l<i>.norm1``, ``l<i>.ls1`` / ``l<i>.ls2`` (the scales),
``l<i>.mix.*``, ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.gate`` / ``.up`` / ``.down``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..config.zeridra import ZeridraConfig


def _position_of(mixer: dict, positions: dict):
    """Name of the position encoding this mixer uses (made on first use; equal constants share one)."""
    rot = mixer.get("rot")
    if not rot:
        return None
    part = PartSpec.of("rotary", head_dim=int(mixer["rot_dim"]), theta=float(rot["base"]), rotary_dim=int(rot["dims"]),
                       pairing="interleaved")
    for name, known in positions.items():
        if known == part:
            return name
    name = f"rot{len(positions)}"
    positions[name] = part
    return name


def _cache_window(config: ZeridraConfig, index: int):
    """The window layer ``index``'s cache has to keep: the widest among itself and the layers that read its rows, or
    None when one of them reads every earlier key."""
    windows = [config.layers[reader].window for reader in [index] + config.readers_of(index)]
    return None if any(window is None for window in windows) else max(windows)


def _mixer_of(config: ZeridraConfig, index: int) -> PartSpec:
    layer = config.layers[index]
    mixer = layer.mixer
    if layer.type == "attention":
        temperature = mixer.get("q_temp")
        return PartSpec.of("gqa_attention", hidden=config.width, heads=int(mixer["heads"]), kv_heads=int(mixer["kv_heads"]),
                           head_dim=int(mixer["dim"]), scale=float(mixer["scale"]), values_are_keys=True, unit_sink=True,
                           precise_weights=True,
                           query_temperature=(float(temperature["coef"]), int(temperature["every"])) if temperature else None,
                           names=(("q", "q"), ("k", "k"), ("o", "o")))
    shared = layer.kv_from is not None
    return PartSpec.of("latent_attention", hidden=config.width, heads=int(mixer["heads"]), dim=int(mixer["dim"]),
                       rot_dim=int(mixer.get("rot_dim") or 0), value_dim=int(mixer["vdim"]), q_rank=int(mixer["q_rank"]),
                       kv_rank=int(mixer["kv_rank"]), scale=float(mixer["scale"]), eps=config.norm_eps, window=layer.window,
                       cache_window=layer.window if shared else _cache_window(config, index), sinks=True, shared_kv=shared)


def zeridra_spec(config: ZeridraConfig) -> ModelSpec:
    def norm():
        return PartSpec.of("rmsnorm", width=config.width, eps=config.norm_eps, tensor="")

    positions, layers, schedule = {}, [], []
    for index, layer in enumerate(config.layers):
        feed_forward = None
        if layer.mlp is not None:
            feed_forward = PartSpec.of("routed_experts", hidden=config.width, experts=int(layer.mlp["router"]["experts"]),
                                       top=int(layer.mlp["router"]["top"]), intermediate=int(layer.mlp["expert"]["ff"]),
                                       activation="silu", weight_on="input", correction=False, route_scale=1.0)
        block = PartSpec.of("parallel_residual", width=config.width, feed_forward=feed_forward is not None, layer_scale=True,
                            mixer_prefix="mix.", feed_forward_prefix="mlp.", mixer_norm_prefix="norm1", mixer_scale="ls1",
                            feed_forward_scale="ls2")
        layers.append(LayerSpec(prefix=f"l{index}.", block=block, mixer=_mixer_of(config, index), feed_forward=feed_forward,
                                mixer_norm=norm(), position=_position_of(layer.mixer, positions) if layer.type == "latent_attention" else None))
        schedule.append(ScheduleEntry(index, cache_from=layer.kv_from))
    return ModelSpec(architecture=config.architecture, vocab_size=config.vocab, hidden_size=config.width, layers=layers,
                     schedule=schedule, positions=positions, final_norm=norm(), embedding_name="embed",
                     final_norm_prefix="final.norm", head_name="head", tie_head=False, embedding_scale=config.embedding_scale,
                     logit_scale=config.logit_scale, logit_softcap=config.logit_softcap, eos_token_ids=config.eos_token_id)


register_architecture("Zeridra", ZeridraConfig, zeridra_spec)
