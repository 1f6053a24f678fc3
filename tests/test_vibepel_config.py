"""Vibepel without a GPU: configuration, refusals, cache needs that are tuples, declared tensors, and properties of the
plain implementation that the GPU tests lean on."""
import copy
import math

import pytest
import torch

import plain_vibepel as plain
from vibepel_configs import BOTH_KINDS, PARALLEL_ONLY, VIBEPEL, WKV_ONLY

F64 = torch.float64


def _spec(raw):
    import llmserver_b200.models  # noqa: F401
    from llmserver_b200.config import VibepelConfig
    from llmserver_b200.config.registry import architecture_of
    config = VibepelConfig.from_dict(raw)
    return config, architecture_of(raw).build_spec(config)


def _needs(spec):
    from llmserver_b200.parts import BLOCKS, MIXERS
    needs = []
    for entry in spec.schedule:
        layer = spec.layers[entry.layer]
        mixer = layer.part(BLOCKS.get(layer.block.kind).mixer_role(layer.block.as_dict()))
        needs.append(MIXERS.get(mixer.kind).cache_need(mixer.as_dict()))
    return needs


@pytest.mark.parametrize("name", sorted(VIBEPEL))
def test_configuration_round_trips(name):
    from llmserver_b200.config import VibepelConfig
    raw = VIBEPEL[name][0]
    config = VibepelConfig.from_dict(raw)
    assert VibepelConfig.from_dict(config.to_dict()) == config
    assert config.vocab_size == raw["vocab"] and config.hidden_size == raw["width"]
    assert config.logit_softcap == raw["logit_softcap"] and config.embedding_scale == raw["embedding"]["scale"]


def test_refusals():
    from llmserver_b200.config import UnsupportedModelError, VibepelConfig

    def broken(change):
        raw = copy.deepcopy(BOTH_KINDS)
        change(raw)
        with pytest.raises(UnsupportedModelError):
            VibepelConfig.from_dict(raw)
    broken(lambda raw: raw["layers"][1].update(type="attention"))
    broken(lambda raw: raw["layers"][1]["mixer"]["left"].update(kv_heads=3))
    broken(lambda raw: raw["layers"][1]["mixer"]["right"].update(kv_heads=3))
    broken(lambda raw: raw["layers"][1]["mixer"]["left"]["rot"].update(dims=18))
    broken(lambda raw: raw["layers"][1]["mixer"]["left"]["rot"]["scaling"].pop("low"))
    broken(lambda raw: raw["layers"][1]["mixer"].pop("right_scale"))
    broken(lambda raw: raw["layers"][1]["mixer"]["right"].pop("conv"))
    broken(lambda raw: raw["layers"][0]["mixer"].update(dim=0))
    broken(lambda raw: raw["layers"][0]["mlp"].update(kind="moe"))
    broken(lambda raw: raw.update(logit_softcap=-1.0))
    broken(lambda raw: raw.pop("norm"))


def test_specification_parts_and_constants():
    config, spec = _spec(BOTH_KINDS)
    assert [layer.mixer.kind for layer in spec.layers] == ["wkv_time_mix", "parallel_mixers", "wkv_time_mix", "parallel_mixers", "parallel_mixers"]
    assert spec.tie_head and spec.logit_softcap == 25.0 and spec.embedding_scale == 2.5
    assert spec.final_norm.get("one_plus") and all(dict(layer.extra)["mixer_out_norm"].get("one_plus") for layer in spec.layers)
    # equal rotary constants share one position part; scaled and unscaled frequencies do not
    assert len(spec.positions) == 3 and spec.layers[0].position is None
    assert {spec.positions[layer.position].kind for layer in spec.layers if layer.position} == {"banded_rotary", "rotary"}
    branches = spec.layers[1].mixer.get("branches")
    assert [(name, scale) for name, _, scale, _ in branches] == [("left", 0.62), ("right", 0.48)]
    assert branches[0][1].get("window") == 23 and branches[0][1].get("qk_norm") and branches[1][1].get("conv") == 4


def test_cache_needs_are_tuples_and_declared_tensors():
    from llmserver_b200.cache import CacheManager, KVPagesNeed, StateNeed
    from llmserver_b200.weights.declare import declared_weights
    config, spec = _spec(BOTH_KINDS)
    needs = _needs(spec)
    assert needs[0] == (StateNeed((3, 16, 16), "float32"), StateNeed((96,), "float32"))
    assert needs[1] == (KVPagesNeed(2, 16, 23, None), (StateNeed((4, 16, 24), "float32"), StateNeed((3, 2 * 32 + 96), "float32")))
    assert needs[3] == (KVPagesNeed(1, 32, 9, 48), (StateNeed((2, 32, 16), "float32"), StateNeed((2, 2 * 64 + 32), "float32")))
    cache = CacheManager(needs, 8, 10, num_slots=2, prefix_sharing=True)
    assert len(cache.groups) == 2 and [len(group.entries) for group in cache.groups] == [2, 1]
    assert sorted(cache.group_of_entry) == [(1, 0), (3, 0), (4, 0)]
    assert sorted(cache.state_entries) == [(0, 0), (0, 1), (1, 1, 0), (1, 1, 1), (2, 0), (2, 1), (3, 1, 0), (3, 1, 1), (4, 1, 0), (4, 1, 1)]
    assert not cache.prefix_sharing       # a window and a state both rule shared prefixes out
    # a request's slot serves every state tensor, and is given back with its pages
    cache.admit("a")
    cache.ensure("a", 20)
    assert cache.slot_of("a") == 0 and [len(cache.table("a", group)) for group in range(2)] == [3, 3]
    cache.free("a")
    cache.check_invariants()
    names = declared_weights(spec)
    assert "head" not in names and names["embed"].shape == (300, 96) and names["final.norm"].shape == (96,)
    assert names["l0.mix.mu.w"].shape == (96,) and names["l0.mix.w1"].shape == (12, 96) and names["l0.mix.u"].shape == (3, 16)
    assert names["l1.mix.left.q"].shape == (64, 96) and names["l1.mix.left.k.norm"].shape == (16,)
    assert names["l1.mix.right.v.conv"].shape == (96, 4) and names["l1.mix.right.A_log"].shape == (4,)
    assert names["l1.mix.right.k"].shape == (32, 96) and names["l1.mix.right.norm"].shape == (24,)
    assert "l2.norm2" not in names and "l1.norm2" in names and "l2.mlp.up" not in names and names["l1.mlp.up"].shape == (80, 96)


def test_a_decay_rank_the_configuration_does_not_name_is_taken_from_the_tensor():
    from llmserver_b200.weights.declare import declared_weights
    from llmserver_b200.weights.loader import shape_fits
    raw = copy.deepcopy(WKV_ONLY)
    for layer in raw["layers"]:
        del layer["mixer"]["w_rank"]
    _, spec = _spec(raw)
    names = declared_weights(spec)
    assert names["l0.mix.w1"].shape == (-1, 40) and names["l0.mix.w2"].shape == (48, -1)
    assert shape_fits((7, 40), names["l0.mix.w1"].shape) and not shape_fits((7, 41), names["l0.mix.w1"].shape)


def test_banded_rotary_table():
    from llmserver_b200.parts import POSITION_ENCODINGS, Runtime
    scaling = {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 48}
    rot = {"base": 500.0, "dims": 12, "scaling": scaling}
    part = POSITION_ENCODINGS.get("banded_rotary")({"head_dim": 16, "theta": 500.0, "rotary_dim": 12, "factor": 4.0, "low": 1.0,
                                                    "high": 3.0, "original": 48}, {}, Runtime(torch.float32, torch.device("cpu")))
    want = plain.rotary_frequencies(rot)
    assert torch.allclose(part.inv_freq.double(), want, rtol=1e-6) and part.rotary_dim == 12
    unscaled = plain.rotary_frequencies({"base": 500.0, "dims": 12})
    ratio = (want / unscaled).tolist()
    assert ratio[0] == 1.0 and ratio[-1] == 0.25 and any(0.25 < value < 1.0 for value in ratio)     # all three bands occur


# ------------------------------------------------------------------------------------------------ the plain implementation
def _random_weights(raw, seed):
    from llmserver_b200.weights.declare import declared_weights
    from llmserver_b200.weights.random_init import random_tensor
    _, spec = _spec(raw)
    return {name: random_tensor(name, declaration, seed).to(F64) for name, declaration in declared_weights(spec).items()}


def test_plain_recurrent_state_carries_over_portions():
    weights = _random_weights(BOTH_KINDS, 1)
    generator = torch.Generator().manual_seed(2)
    h = torch.randn((19, BOTH_KINDS["width"]), dtype=F64, generator=generator)
    mixer = BOTH_KINDS["layers"][0]["mixer"]
    whole, (last_S, last_row) = plain.time_mix(h, weights, "l0.mix.", mixer, 1e-6)
    first, state = plain.time_mix(h[:7], weights, "l0.mix.", mixer, 1e-6)
    second, (end_S, end_row) = plain.time_mix(h[7:], weights, "l0.mix.", mixer, 1e-6, state=state)
    assert torch.allclose(torch.cat([first, second]), whole, atol=1e-12) and torch.allclose(end_S, last_S, atol=1e-12)
    assert torch.equal(end_row, h[-1]) and torch.equal(last_row, h[-1])
    right = BOTH_KINDS["layers"][1]["mixer"]["right"]
    whole, (last_S, _) = plain.gated_delta_rule(h, weights, "l1.mix.right.", right, 1e-6)
    out, state = [], None
    for begin, end in ((0, 1), (1, 3), (3, 4), (4, 12), (12, 19)):      # portions shorter than the convolution too
        piece, state = plain.gated_delta_rule(h[begin:end], weights, "l1.mix.right.", right, 1e-6, state=state)
        out.append(piece)
    assert torch.allclose(torch.cat(out), whole, atol=1e-12) and torch.allclose(state[0], last_S, atol=1e-12)


def test_plain_scans_against_their_unrolled_sums():
    generator = torch.Generator().manual_seed(5)
    T, D, V = 6, 4, 3
    r, k, w = (torch.rand((T, D), dtype=F64, generator=generator) for _ in range(3))
    v = torch.randn((T, V), dtype=F64, generator=generator)
    u = torch.randn(D, dtype=F64, generator=generator)
    out, _ = plain.wkv_scan(r, k, v, w, u, torch.zeros((D, V), dtype=F64))
    for t in range(T):      # o_t = sum_(s<t) (r_t . (prod_(s<j<t) w_j) k_s) v_s + (r_t . u k_t) v_t
        want = (r[t] * u * k[t]).sum() * v[t]
        for s in range(t):
            decay = torch.ones(D, dtype=F64)
            for j in range(s + 1, t):
                decay = decay * w[j]
            want = want + (r[t] * decay * k[s]).sum() * v[s]
        assert torch.allclose(out[t], want, atol=1e-12)
    # the delta rule with beta = 1 and g = 1 and orthonormal keys stores each value exactly, and reads it back
    keys = torch.eye(D, dtype=F64)
    values = torch.randn((D, V), dtype=F64, generator=generator)
    out, S = plain.delta_rule_scan(keys, keys, values, torch.ones(D, dtype=F64), torch.ones(D, dtype=F64), torch.zeros((D, V), dtype=F64))
    assert torch.allclose(out, values, atol=1e-12) and torch.allclose(S, values, atol=1e-12)
    # writing a key a second time with another value replaces the first; with g < 1 older content fades
    again, S = plain.delta_rule_scan(keys[:1], keys[:1], values[1:2], torch.ones(1, dtype=F64), torch.tensor([0.5], dtype=F64), S)
    assert torch.allclose(again[0], values[1], atol=1e-12) and torch.allclose(S[2], 0.5 * values[2], atol=1e-12)


def test_plain_window_edges_and_short_convolution():
    raw = PARALLEL_ONLY
    weights = _random_weights(raw, 3)
    h = torch.randn((12, raw["width"]), dtype=F64, generator=torch.Generator().manual_seed(4))
    left = raw["layers"][0]["mixer"]["left"]          # a window of five tokens
    _, kept = plain.window_attention(h, weights, "l0.mix.left.", left, 1e-6, want_probabilities=True)
    row = kept[0][9]
    assert bool((row[:5] == 0).all()) and bool((row[5:10] > 0).all()) and bool((row[10:] == 0).all()) and abs(float(row.sum()) - 1) < 1e-12
    alone = raw["layers"][2]["mixer"]["left"]         # a window of one: every token sees itself only
    _, kept = plain.window_attention(h, weights, "l2.mix.left.", alone, 1e-6, want_probabilities=True)
    assert torch.allclose(kept[1], torch.eye(12, dtype=F64))
    # positions matter only through differences: a portion that starts later gives the same rows
    shifted = plain.window_attention(h, weights, "l0.mix.left.", left, 1e-6, first_position=37)
    assert torch.allclose(shifted, plain.window_attention(h, weights, "l0.mix.left.", left, 1e-6), atol=1e-9)
    x = torch.randn((7, 3), dtype=F64, generator=torch.Generator().manual_seed(6))
    taps_w = torch.randn((3, 4), dtype=F64, generator=torch.Generator().manual_seed(7))
    y, history = plain.short_convolution(x, taps_w)
    assert torch.allclose(y[0], x[0] * taps_w[:, 3]) and torch.allclose(y[2], x[2] * taps_w[:, 3] + x[1] * taps_w[:, 2] + x[0] * taps_w[:, 1])
    assert torch.equal(history, x[4:])
    tail, _ = plain.short_convolution(x[5:], taps_w, history=x[2:5])
    assert torch.allclose(tail, y[5:], atol=1e-12)


def test_plain_forward_runs_every_configuration():
    for name, (raw, seed) in VIBEPEL.items():
        weights = _random_weights(raw, seed)
        tokens = [(7 * i + 3) % raw["vocab"] for i in range(13)]
        streams = []
        logits = plain.forward(raw, weights, tokens, streams=streams)
        assert logits.shape == (13, raw["vocab"]) and len(streams) == len(raw["layers"])
        assert bool(torch.isfinite(logits).all())
        cap = raw["logit_softcap"]
        assert not cap or float(logits.abs().max()) < cap
        # causal: a later token changes no earlier row
        changed = plain.forward(raw, weights, tokens[:-1] + [(tokens[-1] + 1) % raw["vocab"]])
        assert torch.allclose(changed[:-1], logits[:-1], atol=1e-12) and not torch.allclose(changed[-1], logits[-1], atol=1e-9)


def test_segments_of_long_portions_are_chosen_by_length_type_and_scratch():
    """The recurrences walk a long bfloat16 portion by segments of at least 64 tokens, at most 64 of them, within a bound
    on the scratch (a state and a transition per sequence, segment and head); short steps, 32-bit steps and steps whose
    scratch would not hold two segments run in one pass; a given segment length is taken as it is."""
    from types import SimpleNamespace

    from llmserver_b200 import ops

    def choose(n_seqs, longest, dtype, segment=None, heads=2, dim=16, vdim=16, move=16):
        batch = SimpleNamespace(n_seqs=n_seqs, max_q_len=longest, scratch={})
        chosen = ops._recurrence_segments(batch, torch.empty((1,), dtype=dtype), segment, heads, dim, vdim, move)
        return chosen, batch

    (segment, segments, state, move), batch = choose(1, 2048, torch.bfloat16)
    assert (segment, segments) == (64, 32) and state.shape == (1, 32, 2, 16, 16) and move.shape == (1, 32, 2, 16, 16)
    assert len(batch.scratch) == 1
    assert choose(1, 2048, torch.float32)[0] == (0, 0, None, None)
    assert choose(3, 127, torch.bfloat16)[0] == (0, 0, None, None)
    assert choose(3, 128, torch.bfloat16)[0][:2] == (64, 2)
    assert choose(1, 64 * 64 + 1, torch.bfloat16)[0][:2] == (65, 64)            # no more than 64 segments
    assert choose(2, 100, torch.bfloat16, segment=7)[0][:2] == (7, 15)
    assert choose(2, 100, torch.float32, segment=7)[0][:2] == (7, 15)
    # a diagonal transition takes one value per key channel
    assert choose(1, 300, torch.bfloat16, move=1)[0][3].shape == (1, 5, 2, 16, 1)
    # heads of 128 x 128 with full transitions: 128 KiB per (sequence, segment, head); 16 heads and 100 sequences leave
    # room for 5 segments of a 2048-token portion, 600 sequences for none
    many = choose(100, 2048, torch.bfloat16, heads=16, dim=128, vdim=128, move=128)[0]
    assert many[:2] == (410, 5) and many[2].numel() * 4 + many[3].numel() * 4 <= ops.REC_SCRATCH_BYTES
    assert choose(600, 2048, torch.bfloat16, heads=16, dim=128, vdim=128, move=128)[0] == (0, 0, None, None)
