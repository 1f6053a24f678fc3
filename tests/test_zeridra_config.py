"""Zeridra without a GPU: the configuration, the specification it becomes, cache needs, declared tensors, and properties
of the plain implementation the GPU tests compare with."""
import copy

import pytest
import torch

import plain_zeridra as plain
from zeridra_configs import ALL_KINDS, ATTENTION_ONLY, LATENT_ONLY, TENSOR_CORE_SIZES, ZERIDRA

import llmserver_b200.models  # noqa: F401  registers the architectures
from llmserver_b200.cache.manager import CacheManager, KVPagesNeed
from llmserver_b200.config import UnsupportedModelError, ZeridraConfig, architecture_of
from llmserver_b200.parts import BLOCKS, FEED_FORWARDS, MIXERS
from llmserver_b200.weights import RandomSource
from llmserver_b200.weights.declare import declared_weights


def spec_of(raw):
    return architecture_of(raw).build_spec(ZeridraConfig.from_dict(raw))


@pytest.mark.parametrize("name", sorted(ZERIDRA))
def test_configuration_round_trip(name):
    raw = ZERIDRA[name][0]
    config = ZeridraConfig.from_dict(raw)
    assert ZeridraConfig.from_dict(config.to_dict()) == config
    assert config.vocab_size == raw["vocab"] and config.hidden_size == raw["width"]
    assert architecture_of(raw).name == "Zeridra"


def test_absent_constants_do_not_exist():
    raw = copy.deepcopy(ATTENTION_ONLY)
    del raw["embedding"], raw["logit_scale"]
    config = ZeridraConfig.from_dict(raw)
    assert config.embedding_scale == 1.0 and config.logit_scale == 1.0 and config.logit_softcap == 0.0
    spec = spec_of(raw)
    assert spec.logit_softcap == 0.0 and spec.logit_scale == 1.0


@pytest.mark.parametrize("change,message", [
    (lambda raw: raw["layers"][0].update(type="conv"), "unknown mixer type"),
    (lambda raw: raw["layers"][1]["mixer"].update(kv_heads=4), "no multiple"),
    (lambda raw: raw["layers"][0]["mixer"].update(vdim=20), "vdim must equal dim"),
    (lambda raw: raw["layers"][0]["mixer"]["q_temp"].update(every=0), "every must be positive"),
    (lambda raw: raw["layers"][1]["mlp"]["router"].update(top=9), "top must lie"),
    (lambda raw: raw["layers"][1]["mlp"].update(kind="dense"), "unknown kind"),
    (lambda raw: raw.pop("norm"), "lacks norm"),
])
def test_refusals_of_attention_layers(change, message):
    raw = copy.deepcopy(ATTENTION_ONLY)
    change(raw)
    with pytest.raises(UnsupportedModelError, match=message):
        ZeridraConfig.from_dict(raw)


@pytest.mark.parametrize("change,message", [
    (lambda raw: raw["layers"][2]["mixer"].update(kv_from=2), "does not run before"),
    (lambda raw: raw["layers"][2]["mixer"].update(kv_from=3), "does not run before"),
    (lambda raw: raw["layers"][3]["mixer"].update(kv_from=2), "keeps no latents of its own"),
    (lambda raw: raw["layers"][2]["mixer"].update(kv_rank=24), "kv_rank differs"),
    (lambda raw: raw["layers"][2]["mixer"]["rot"].update(base=7.0), "turns its key part otherwise"),
    (lambda raw: raw["layers"][0]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda raw: raw["layers"][0]["mixer"]["mask"].update(size=0), "lacks size|must be positive"),
])
def test_refusals_of_latent_layers(change, message):
    raw = copy.deepcopy(LATENT_ONLY)
    change(raw)
    with pytest.raises(UnsupportedModelError, match=message):
        ZeridraConfig.from_dict(raw)


def test_specification_parts_and_constants():
    spec = spec_of(ALL_KINDS)
    assert [layer.block.kind for layer in spec.layers] == ["parallel_residual"] * 7
    assert [layer.mixer.kind for layer in spec.layers] == ["latent_attention", "gqa_attention", "latent_attention", "gqa_attention",
                                                          "latent_attention", "latent_attention", "latent_attention"]
    assert [entry.cache_from for entry in spec.schedule] == [None, None, 0, None, None, 4, 4]
    assert spec.embedding_scale == 0.7 and spec.logit_scale == 2.0 and spec.logit_softcap == 25.0
    attention = spec.layers[1].mixer.as_dict()
    assert attention["values_are_keys"] and attention["unit_sink"] and attention["query_temperature"] == (0.4, 16)
    assert spec.layers[3].mixer.as_dict()["query_temperature"] is None
    experts = spec.layers[0].feed_forward.as_dict()
    assert (experts["activation"], experts["weight_on"], experts["correction"], experts["top"]) == ("silu", "input", False, 2)
    assert spec.layers[2].feed_forward is None and not spec.layers[2].block.get("feed_forward")
    # equal rotation constants share one encoding; every encoding pairs neighbours
    assert spec.layers[0].position == spec.layers[2].position and spec.layers[4].position != spec.layers[0].position
    assert all(part.get("pairing") == "interleaved" for part in spec.positions.values())
    # a layer that reads another's cache has no down projection of its own
    reader = spec.layers[2].mixer.as_dict()
    assert reader["shared_kv"] and reader["window"] == 61


def test_cache_keeps_the_widest_window_among_its_readers():
    spec = spec_of(ALL_KINDS)
    needs = [MIXERS.get(layer.mixer.kind).cache_need(layer.mixer.as_dict()) for layer in spec.layers]
    assert needs[0] == KVPagesNeed(1, 56 + 16, 61, None, keys_only=True)        # its own window is 23, its reader's 61
    assert needs[4] == KVPagesNeed(1, 32 + 8, None, None, keys_only=True)       # one reader sees every key
    assert needs[1] == KVPagesNeed(2, 24, None, None, keys_only=True) and needs[3] == KVPagesNeed(6, 16, None, None, keys_only=True)
    from llmserver_b200.models.decoder import DecoderModel
    owned = [None if entry.cache_from is not None else needs[entry.layer] for entry in spec.schedule]
    manager = CacheManager(owned, page_size=8, num_pages=32, num_slots=4, prefix_sharing=True)
    assert len(manager.groups) == 4 and not manager.prefix_sharing       # a windowed group: prompts are recomputed
    manager.admit("a")
    manager.ensure("a", 100)
    manager.advance("a", 100)
    windowed = [group for group in manager.groups if group.window == 61][0]
    assert windowed.tables["a"][:5] == [-1] * 5 and windowed.tables["a"][5] >= 0       # (100 - 61 + 1) // 8 pages have passed
    manager.free("a")
    manager.check_invariants()
    assert DecoderModel is not None


@pytest.mark.parametrize("name", sorted(ZERIDRA))
def test_declared_tensors(name):
    raw = ZERIDRA[name][0]
    wanted = declared_weights(spec_of(raw))
    expected = {"embed", "head", "final.norm"}
    for index, layer in enumerate(raw["layers"]):
        expected |= {f"l{index}.norm1", f"l{index}.ls1", f"l{index}.mix.o"}
        mixer = layer["mixer"]
        if layer["type"] == "attention":
            expected |= {f"l{index}.mix.q", f"l{index}.mix.k"}
            assert wanted[f"l{index}.mix.k"].shape == (mixer["kv_heads"] * mixer["dim"], raw["width"])
        else:
            expected |= {f"l{index}.mix.{t}" for t in ("dq", "dq.norm", "uq", "uk", "uv", "sink")}
            if mixer.get("kv_from") is None:
                expected |= {f"l{index}.mix.dkv", f"l{index}.mix.dkv.norm"}
                assert wanted[f"l{index}.mix.dkv"].shape == (mixer["kv_rank"] + mixer["rot_dim"], raw["width"])
            assert wanted[f"l{index}.mix.uq"].shape == (mixer["heads"] * (mixer["dim"] + mixer["rot_dim"]), mixer["q_rank"])
            assert wanted[f"l{index}.mix.sink"].shape == (mixer["heads"],)
        if layer["mlp"] is not None:
            expected |= {f"l{index}.ls2", f"l{index}.mlp.router"}
            for e in range(layer["mlp"]["router"]["experts"]):
                expected |= {f"l{index}.mlp.e{e}.{t}" for t in ("gate", "up", "down")}
    assert set(wanted) == expected


def test_parts_refuse_what_they_have_no_code_for():
    with pytest.raises(ValueError, match="values that are the keys"):
        MIXERS.get("gqa_attention").check_params({"hidden": 8, "heads": 2, "kv_heads": 1, "head_dim": 4, "scale": 1.0,
                                                  "values_are_keys": True, "value_dim": 8})
    with pytest.raises(ValueError, match="not both"):
        MIXERS.get("gqa_attention").check_params({"hidden": 8, "heads": 2, "kv_heads": 1, "head_dim": 4, "scale": 1.0,
                                                  "sinks": True, "unit_sink": True})
    with pytest.raises(ValueError, match="unknown activation"):
        FEED_FORWARDS.get("routed_experts").check_params({"hidden": 8, "experts": 2, "top": 1, "intermediate": 4, "activation": "gelu"})
    with pytest.raises(ValueError, match="takes no limit"):
        FEED_FORWARDS.get("routed_experts").check_params({"hidden": 8, "experts": 2, "top": 1, "intermediate": 4, "activation": "silu", "limit": 7.0})
    with pytest.raises(ValueError, match="weight_on"):
        FEED_FORWARDS.get("routed_experts").check_params({"hidden": 8, "experts": 2, "top": 1, "intermediate": 4, "limit": 7.0, "weight_on": "both"})
    with pytest.raises(ValueError, match="does not know"):
        BLOCKS.get("parallel_residual").check_params({"width": 8, "dropout": 0.1})


# ------------------------------------------------------------------------------------------------ the plain implementation
def _random_model(raw, seed):
    source = RandomSource(spec_of(raw), seed, torch.float32, "cpu")
    weights = {name: source.get(name).to(torch.float64) for name in source.wanted}
    generator = torch.Generator().manual_seed(seed)
    for name in weights:
        if name.endswith((".mix.q", ".mix.k", ".mix.dq", ".mix.dkv", ".mix.uq", ".mix.uk", ".router")):
            weights[name] = torch.randn(weights[name].shape, generator=generator, dtype=torch.float64) * 2.0 / weights[name].shape[1] ** 0.5
        elif name.endswith((".mix.uv", ".mix.o", ".gate", ".up", ".down", "head")):
            weights[name] = torch.randn(weights[name].shape, generator=generator, dtype=torch.float64) / weights[name].shape[1] ** 0.5
        elif name.endswith(".sink"):
            weights[name] = torch.linspace(-2.0, 3.0, weights[name].shape[0], dtype=torch.float64)
        elif name == "embed":
            weights[name] = torch.randn(weights[name].shape, generator=generator, dtype=torch.float64)
    return weights


def test_turning_pairs_neighbours_and_leaves_the_rest():
    x = torch.arange(1.0, 13.0, dtype=torch.float64).view(1, 1, 12).repeat(3, 2, 1)
    rot = {"base": 100.0, "dims": 4}
    out = plain.turn_pairs(x, torch.tensor([0, 1, 5]), rot)
    assert torch.equal(out[0], x[0]) and torch.equal(out[..., 4:], x[..., 4:])
    angle = 5 * 100.0 ** (-2 / 4)
    u, v = 3.0, 4.0
    assert torch.allclose(out[2, 0, 2:4], torch.tensor([u * torch.cos(torch.tensor(angle)) - v * torch.sin(torch.tensor(angle)),
                                                       v * torch.cos(torch.tensor(angle)) + u * torch.sin(torch.tensor(angle))], dtype=torch.float64))


def test_query_temperature_steps():
    factor = plain.query_temperature(torch.arange(0, 40), {"coef": 0.5, "every": 16})
    assert torch.all(factor[:15] == 1.0) and factor[15] == factor[30] and factor[31] > factor[30]
    assert torch.isclose(factor[15], torch.tensor(1.0 + 0.5 * 0.6931471805599453, dtype=torch.float64))


def test_denominator_terms_and_window_edges_show():
    """A model without its extra denominator terms, or with windows one token longer or shorter, is far from the model."""
    for raw, seed in (ZERIDRA["latent_only"], ZERIDRA["all_kinds"], ZERIDRA["attention_only"]):
        weights = _random_model(raw, seed)
        tokens = torch.randint(0, raw["vocab"], (90,), generator=torch.Generator().manual_seed(1)).tolist()
        want = plain.forward(raw, weights, tokens)
        scale = want.abs().max(-1).values
        for wrong in ({"drop_sinks": True}, {"window_shift": 1}, {"window_shift": -1}):
            if raw is ATTENTION_ONLY and "window_shift" in wrong:
                continue
            got = plain.forward(raw, weights, tokens, **wrong)
            assert ((got - want).abs().max(-1).values / scale).max() > 0.1, wrong


def test_a_cache_reader_sees_its_owners_rows_not_its_own():
    raw = copy.deepcopy(LATENT_ONLY)
    weights = _random_model(raw, 5)
    tokens = list(range(40))
    want = plain.forward(raw, weights, tokens)
    # the same model with layer 2 making rows of its own (from weights that the reader does not have) is another model
    own = copy.deepcopy(raw)
    del own["layers"][2]["mixer"]["kv_from"]
    more = dict(weights)
    more["l2.mix.dkv"], more["l2.mix.dkv.norm"] = weights["l0.mix.dkv"], weights["l0.mix.dkv.norm"]
    other = plain.forward(own, more, tokens)
    assert (other - want).abs().max() > 1e-3


def test_attention_over_the_cached_rows_alone_equals_attention_over_keys_and_values():
    """q_h . (W_uk,h c) = (W_uk,h^T q_h) . c and sum_j p_j W_uv,h c_j = W_uv,h sum_j p_j c_j: what the engine computes."""
    mixer = LATENT_ONLY["layers"][0]["mixer"]
    weights = _random_model(LATENT_ONLY, 9)
    T, heads, dim, rot_dim, vdim, rank = 30, mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"], mixer["kv_rank"]
    h = torch.randn((T, LATENT_ONLY["width"]), generator=torch.Generator().manual_seed(2), dtype=torch.float64)
    positions = torch.arange(T)
    kv = plain.latent_kv(h, positions, mixer, weights, "l0.mix.", 1e-6)
    want = plain.latent_mixer(h, positions, mixer, weights, "l0.mix.", 1e-6, kv)
    c, r = kv
    c_q = plain.rms_norm(h @ weights["l0.mix.dq"].T, weights["l0.mix.dq.norm"], 1e-6)
    q = (c_q @ weights["l0.mix.uq"].T).view(T, heads, dim + rot_dim)
    up_k = weights["l0.mix.uk"].view(heads, dim, rank)
    carried = torch.cat([torch.einsum("thd,hdr->thr", q[..., :dim], up_k), plain.turn_pairs(q[..., dim:], positions, mixer["rot"])], dim=-1)
    rows = torch.cat([c, r], dim=-1)
    scores = torch.einsum("ihr,jr->hij", carried, rows) * mixer["scale"]
    p = plain.softmax_with_extra(scores, plain.visible(positions, mixer["mask"]["size"]), weights["l0.mix.sink"])
    attended = torch.einsum("hij,jr->ihr", p, c)
    out = torch.einsum("ihr,hvr->ihv", attended, weights["l0.mix.uv"].view(heads, vdim, rank)).reshape(T, heads * vdim)
    assert torch.allclose(out @ weights["l0.mix.o"].T, want, atol=1e-10)


def test_weights_on_the_input_are_not_weights_on_the_output():
    mlp = {"router": {"experts": 4, "top": 2}, "expert": {"ff": 8}}
    generator = torch.Generator().manual_seed(3)
    weights = {"m.router": torch.randn((4, 16), generator=generator, dtype=torch.float64)}
    for e in range(4):
        weights[f"m.e{e}.gate"] = torch.randn((8, 16), generator=generator, dtype=torch.float64)
        weights[f"m.e{e}.up"] = torch.randn((8, 16), generator=generator, dtype=torch.float64)
        weights[f"m.e{e}.down"] = torch.randn((16, 8), generator=generator, dtype=torch.float64)
    h = torch.randn((6, 16), generator=generator, dtype=torch.float64)
    got = plain.feed_forward(h, mlp, weights, "m.")
    chosen, scores = plain.route(h, mlp, weights, "m.")
    assert chosen.shape == (6, 2) and bool((scores[:, 0] >= scores[:, 1]).all()) and bool((scores < 1).all())
    on_output = torch.stack([sum(scores[t, j] * plain.expert(h[t], weights, f"m.e{int(chosen[t, j])}.") for j in range(2)) for t in range(6)])
    on_input = torch.stack([sum(plain.expert(scores[t, j] * h[t], weights, f"m.e{int(chosen[t, j])}.") for j in range(2)) for t in range(6)])
    assert torch.allclose(got, on_input) and (got - on_output).abs().max() > 1e-2
    margins = plain.route_margin(h, mlp, weights, "m.")
    assert margins.shape == (6,) and bool((margins >= 0).all())


def test_tensor_core_configuration_has_the_sizes_it_is_named_for():
    for layer in TENSOR_CORE_SIZES["layers"]:
        mixer = layer["mixer"]
        if layer["type"] == "attention":
            assert mixer["dim"] in (64, 128)
        else:
            assert mixer["kv_rank"] + mixer["rot_dim"] in (64, 128)
