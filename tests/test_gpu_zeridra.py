"""Zeridra on the GPU against the plain implementation in plain_zeridra.py: each mechanism alone, then whole models
through the step function, the cache and the scheduler, cut and batched in different ways, in 32-bit and bfloat16."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_zeridra as plain
import traces
from helpers import tokens_for
from zeridra_configs import ZERIDRA

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"
DTYPES = ["float32", "bfloat16"]
NAMES = sorted(ZERIDRA)
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F64 = torch.float64
# Largest allowed |engine - plain| as a fraction of the row's largest |plain value|.  bfloat16: activations are rounded
# to 8 significant bits between kernels, and the weights here are drawn for peaked attention.
ALLOWED = {"float32": 2e-5, "bfloat16": 5e-2}
MARGIN = 0.03       # bfloat16 rows are compared where every routing decision of the token is at least this clear


def redraw(tensors, seed):
    """Weights under which a fault shows: query and key projections large enough for peaked attention, routers whose
    scores spread, sinks from -2 to 3, scales on the sub-layers' outputs far from one."""
    generator = torch.Generator().manual_seed(seed)
    for key in sorted(tensors):
        shape = tensors[key].shape

        def draw(deviation):
            return (torch.randn(shape, generator=generator) * deviation).to(torch.bfloat16)
        if key.endswith((".mix.dq", ".mix.dkv", ".router")):
            tensors[key] = draw(2.0 / math.sqrt(shape[1]))
        elif key.endswith((".mix.q", ".mix.k", ".mix.uq", ".mix.uk")):      # scores a few units apart: peaked, yet not an argmax
            tensors[key] = draw(1.2 / math.sqrt(shape[1]))
        elif key.endswith((".mix.uv", ".mix.o", ".gate", ".up", ".down", "head")):
            tensors[key] = draw(1.0 / math.sqrt(shape[1]))
        elif key.endswith(".sink"):
            tensors[key] = torch.linspace(-2.0, 3.0, shape[0]).to(torch.bfloat16)
        elif key.endswith((".ls1", ".ls2")):
            tensors[key] = (0.3 + torch.rand(shape, generator=generator)).to(torch.bfloat16)
        elif key == "embed":
            tensors[key] = draw(1.0)
    return tensors


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from safetensors.torch import load_file, save_file

    import llmserver_b200.models  # noqa: F401
    from llmserver_b200.config import ZeridraConfig
    from llmserver_b200.weights import write_model_folder

    import copy
    root = tmp_path_factory.mktemp("zeridra")
    made = {}
    for name, (raw, seed) in ZERIDRA.items():
        # "<name>": the configuration as it is; "<name>+all": the same with routers that choose all of their experts, so
        # that no routing decision can go the other way once activations are rounded
        every = copy.deepcopy(raw)
        for layer in every["layers"]:
            if layer["mlp"] is not None:
                layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
        for key, config in ((name, raw), (name + "+all", every)):
            folder = write_model_folder(ZeridraConfig.from_dict(config), str(root / key), seed, torch.bfloat16)
            path = os.path.join(folder, "model.safetensors")
            save_file(redraw(load_file(path), seed), path)
            made[key] = folder
    return made


def variants(name, dtype):
    """The model folders a test runs in this type: in bfloat16 also the form whose routers choose every expert."""
    return [name] if dtype == "float32" else [name, name + "+all"]


_PLAIN, _LOGITS = {}, {}


def plain_model_of(folder):
    if folder not in _PLAIN:
        from safetensors.torch import load_file
        with open(os.path.join(folder, "config.json")) as handle:
            config = json.load(handle)
        _PLAIN[folder] = (config, {key: value.to(F64) for key, value in load_file(os.path.join(folder, "model.safetensors")).items()})
    return _PLAIN[folder]


def plain_logits(folder, tokens):
    """(logits [T, V], smallest routing margin of each token [T])"""
    key = (folder, tuple(tokens))
    if key not in _LOGITS:
        config, weights = plain_model_of(folder)
        margins = []
        logits = plain.forward(config, weights, list(tokens), margins=margins).numpy()
        _LOGITS[key] = (logits, margins[0].numpy() if margins else np.full(len(tokens), np.inf))
    return _LOGITS[key]


def run_in_process(folder, dtype, records, max_tokens, page_size=16):
    from llmserver_b200.engine.replay import TraceReplayer

    replayer = TraceReplayer(folder, dtype, max_tokens, page_size)
    out = {}
    for record in records:
        logits = replayer.run_step(record)
        if logits is not None:
            out[record["step"]] = logits
    replayer.cache.check_invariants()
    assert not replayer.cache.requests, "requests left in the cache after the trace ended"
    for group in replayer.cache.groups:
        assert group.pool.num_available == group.pool.num_pages, "pages were lost"
    return out, replayer


def compare(got, records, requests, folder, dtype, what):
    """32-bit: every row within the allowance.  bfloat16: a token whose two best experts are a hair apart goes either way
    once activations are rounded, and later tokens that attend to it follow.  So a model whose routers choose among
    their experts is compared where every routing decision of the token itself is clear in the plain implementation (at
    least a third of the rows must be such), and of those rows one in three may lie outside the allowance while the middle
    row lies inside (a model with five routed layers takes a few such turns per prompt); the same model with routers that
    choose all of their experts is compared row by row like a 32-bit one, and so is every routed layer by itself
    (``test_experts_that_see_their_token_times_its_score``)."""
    want = traces.expected_rows(records, requests, lambda name: plain_logits(folder, requests[name])[0])
    clear = traces.expected_rows(records, requests, lambda name: plain_logits(folder, requests[name])[1][:, None])
    assert set(got) == set(want), f"{what}: steps with logits differ"
    errors, skipped = [], 0
    for step in sorted(want):
        assert got[step].shape == want[step].shape and np.isfinite(got[step]).all(), f"{what} step {step}"
        scale = np.abs(want[step]).max(axis=-1)
        for row, error in enumerate(np.abs(got[step] - want[step]).max(axis=-1) / scale):
            if dtype == "bfloat16" and clear[step][row, 0] < MARGIN:
                skipped += 1
            else:
                errors.append((float(error), step, row))
    assert len(errors) >= (len(errors) + skipped) / 3, f"{what}: only {len(errors)} rows of {len(errors) + skipped} have clear routing"
    worst, step, row = max(errors)
    if dtype == "bfloat16" and skipped:
        over = sum(1 for error, _, _ in errors if error > ALLOWED[dtype])
        middle = sorted(error for error, _, _ in errors)[len(errors) // 2]
        assert over <= len(errors) / 3 and middle <= ALLOWED[dtype], \
            f"{what}: {over} of {len(errors)} rows differ by more than {ALLOWED[dtype]:.1e}, the middle row by {middle:.3e}"
        return
    assert worst <= ALLOWED[dtype], f"{what} step {step}: row {row} differs by {worst:.3e} of its largest logit, allowed {ALLOWED[dtype]:.1e}"


def close(got, want, dtype, what, rows=None):
    got, want = got.detach().cpu().to(F64), want.to(F64)
    assert got.shape == want.shape and bool(torch.isfinite(got).all()), what
    error = (got - want).abs().amax(-1) / want.abs().amax(-1).clamp_min(1e-30)
    if rows is not None:
        error = error[rows]
    assert float(error.max()) <= ALLOWED[dtype], f"{what}: row {int(error.argmax())} differs by {float(error.max()):.3e}"


def torch_type(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [40, 96, 1000])
def test_two_scaled_outputs_join_the_stream_in_front_of_the_norm(dtype, width):
    from llmserver_b200 import ops
    act = torch_type(dtype)
    generator = torch.Generator().manual_seed(width)
    rows = 7
    stream = torch.randn((rows, width), generator=generator) * 3
    a, b = (torch.randn((rows, width), generator=generator).to(act) for _ in range(2))
    scale_a, scale_b = torch.rand(width, generator=generator) + 0.2, torch.rand(width, generator=generator) * 2
    weight = (1 + 0.1 * torch.randn(width, generator=generator)).to(act)
    for second in (True, False):
        residual = stream.clone().to(DEVICE)
        out = ops.scaled_add_rmsnorm(residual, a.to(DEVICE), scale_a.to(DEVICE), b.to(DEVICE) if second else None,
                                     scale_b.to(DEVICE) if second else None, weight.to(DEVICE), 1e-5, act_dtype=act)
        summed = stream.double() + a.double() * scale_a.double() + (b.double() * scale_b.double() if second else 0)
        assert torch.allclose(residual.cpu().double(), summed, atol=1e-5, rtol=1e-6)       # the stream itself stays 32-bit
        close(out, plain.rms_norm(summed, weight, 1e-5), dtype, f"width {width}")
        # chosen rows: the stream is left as it was
        residual = stream.clone().to(DEVICE)
        picked = torch.tensor([5, 0, 5], dtype=torch.int32)
        out = ops.scaled_add_rmsnorm(residual, a.to(DEVICE), scale_a.to(DEVICE), b.to(DEVICE) if second else None,
                                     scale_b.to(DEVICE) if second else None, weight.to(DEVICE), 1e-5, rows=picked.to(DEVICE), act_dtype=act)
        assert torch.equal(residual.cpu(), stream)
        close(out, plain.rms_norm(summed[picked.long()], weight, 1e-5), dtype, f"width {width}, chosen rows")


@pytest.mark.parametrize("dtype", DTYPES)
def test_scaled_and_capped_logits(dtype):
    from llmserver_b200 import ops
    logits = torch.randn((5, 77), generator=torch.Generator().manual_seed(1)) * 40
    for cap, scale in ((30.0, 0.25), (12.0, 1.0), (0.0, 2.0), (0.0, 1.0)):
        got = ops.softcap_(logits.clone().to(DEVICE), cap, scale).cpu().double()
        want = logits.double() * scale
        want = cap * torch.tanh(want / cap) if cap else want
        assert torch.allclose(got, want, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_rank,kv_rank,rot_dim,dims,page_size", [(24, 40, 8, 8, 4), (72, 16, 12, 6, 8), (64, 96, 32, 32, 16), (16, 33, 6, 2, 3)])
def test_latent_and_turning_part_into_the_cache(dtype, q_rank, kv_rank, rot_dim, dims, page_size):
    """One unit whose first part is normalised and whose last part turns, pair by pair, written across page borders into
    pages that are not in order; the query latent normalised into a packed buffer."""
    from llmserver_b200 import ops
    from llmserver_b200.engine.batch import SequenceSlice, build_batch
    act = torch_type(dtype)
    generator = torch.Generator().manual_seed(kv_rank)
    lengths = [(0, 13), (9, 1), (5, 10)]       # (tokens before, tokens now)
    tables = [[6, 2, 9, 4, 12], [1, 8, 3, 0, 13], [5, 7, 10, 11, 14]]
    row = kv_rank + rot_dim
    pages = torch.zeros((15, 1, page_size, row), dtype=act, device=DEVICE)
    batch = build_batch([SequenceSlice(f"r{s}", [0] * now, before, [], [tables[s]], 0) for s, (before, now) in enumerate(lengths)], 1, DEVICE)
    tokens = sum(now for _, now in lengths)
    down = torch.randn((tokens, q_rank + row + 3), generator=generator).to(act)      # three more columns that stay as they are
    q_weight, k_weight = ((1 + 0.2 * torch.randn(n, generator=generator)).to(act) for n in (q_rank, kv_rank))
    inv_freq = torch.tensor([50.0 ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float32)
    c_q = torch.empty((tokens, q_rank), dtype=act, device=DEVICE)
    on_device = down.clone().to(DEVICE)
    ops.norm_rope_units(on_device, batch.positions, batch.seq_of_token, batch.block_tables[0], pages, None, 1, 1, 1, q_rank, row, 0,
                        batch.error_flag, q_weight=q_weight.to(DEVICE), k_weight=k_weight.to(DEVICE), eps=1e-6, inv_freq=inv_freq.to(DEVICE),
                        rotary_dim=dims, q_out=c_q, k_norm_dim=kv_rank, q_rot_start=-1, k_rot_start=kv_rank, interleaved=True)
    assert int(batch.error_flag.item()) == 0 and torch.equal(on_device.cpu(), down)      # the projection itself is not touched
    positions = torch.cat([torch.arange(before, before + now) for before, now in lengths])
    close(c_q, plain.rms_norm(down[:, :q_rank].double(), q_weight, 1e-6), dtype, "query latent")
    want = torch.cat([plain.rms_norm(down[:, q_rank:q_rank + kv_rank].double(), k_weight, 1e-6),
                      plain.turn_pairs(down[:, q_rank + kv_rank:q_rank + row].double(), positions, {"base": 50.0, "dims": dims})], dim=-1)
    at = 0
    for s, (before, now) in enumerate(lengths):
        for position in range(before, before + now):
            stored = pages[tables[s][position // page_size], 0, position % page_size]
            close(stored[None], want[at][None], dtype, f"sequence {s} position {position}")
            at += 1
    written = {(tables[s][p // page_size], p % page_size) for s, (before, now) in enumerate(lengths) for p in range(before, before + now)}
    for page in range(15):
        for slot in range(page_size):
            assert (page, slot) in written or not bool(pages[page, 0, slot].any()), "a slot nobody owns was written"


@pytest.mark.parametrize("dtype", DTYPES)
def test_queries_alone_turn_behind_their_still_part_and_warm_up_with_the_position(dtype):
    from llmserver_b200 import ops
    from llmserver_b200.engine.batch import SequenceSlice, build_batch
    act = torch_type(dtype)
    generator = torch.Generator().manual_seed(4)
    heads, dim, rot_dim, dims = 3, 10, 8, 6
    positions = torch.tensor([0, 1, 2, 700, 31, 32], dtype=torch.int32)
    q = torch.randn((6, heads * (dim + rot_dim) + 5), generator=generator).to(act)
    inv_freq = torch.tensor([1e4 ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float32)
    turned = q.clone().to(DEVICE)
    ops.rotate_units(turned, positions.to(DEVICE), heads, dim + rot_dim, inv_freq.to(DEVICE), dims, rot_start=dim, interleaved=True)
    heads_of = q[:, :heads * (dim + rot_dim)].double().view(6, heads, dim + rot_dim)
    want = torch.cat([heads_of[..., :dim], plain.turn_pairs(heads_of[..., dim:], positions.long(), {"base": 1e4, "dims": dims})], dim=-1)
    close(turned[:, :heads * (dim + rot_dim)], want.view(6, -1), dtype, "turned queries")
    assert torch.equal(turned[:, heads * (dim + rot_dim):].cpu(), q[:, heads * (dim + rot_dim):])
    # the temperature: query units alone grow with the position; key units are cached as projected
    kv_heads, head = 2, 12
    lengths = [(0, 3), (30, 3)]
    batch = build_batch([SequenceSlice(f"r{s}", [0] * now, before, [], [[s * 5 + i for i in range(5)]], 0) for s, (before, now) in enumerate(lengths)], 1, DEVICE)
    pages = torch.zeros((10, kv_heads, 8, head), dtype=act, device=DEVICE)
    qk = torch.randn((6, (heads + kv_heads) * head), generator=generator).to(act)
    warmed = qk.clone().to(DEVICE)
    ops.norm_rope_units(warmed, batch.positions, batch.seq_of_token, batch.block_tables[0], pages, None, heads, kv_heads, 1, head, head, 0,
                        batch.error_flag, q_temp=(0.5, 16))
    factor = plain.query_temperature(torch.tensor([0, 1, 2, 30, 31, 32]), {"coef": 0.5, "every": 16})
    assert factor[0] == 1 and factor[4] > factor[3] > 1
    close(warmed[:, :heads * head], qk[:, :heads * head].double() * factor[:, None], dtype, "warmed queries")
    assert torch.equal(warmed[:, heads * head:].cpu(), qk[:, heads * head:])
    assert torch.equal(pages[8, :, 7].cpu().view(-1), qk[4, heads * head:])       # position 31 of the second sequence


def _experts(width, experts, ff, seed, act):
    generator = torch.Generator().manual_seed(seed)
    weights = {"router": (torch.randn((experts, width), generator=generator) * 2 / math.sqrt(width)).to(torch.bfloat16).float()}
    for e in range(experts):
        weights[f"e{e}.gate"] = (torch.randn((ff, width), generator=generator) / math.sqrt(width)).to(torch.bfloat16)
        weights[f"e{e}.up"] = (torch.randn((ff, width), generator=generator) / math.sqrt(width)).to(torch.bfloat16)
        weights[f"e{e}.down"] = (torch.randn((width, ff), generator=generator) / math.sqrt(ff)).to(torch.bfloat16)
    return weights


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,experts,top,ff,tokens", [(48, 5, 2, 24, 9), (48, 3, 3, 40, 40), (192, 8, 2, 128, 5), (192, 8, 2, 128, 150),
                                                         (128, 6, 1, 64, 70), (64, 12, 4, 64, 33)])
def test_experts_that_see_their_token_times_its_score(dtype, width, experts, top, ff, tokens):
    """Few tokens multiply pair by pair, many go through the sorted, tiled product (bfloat16, sizes in 64s); in both the
    routing weight acts on the expert's input and the outputs are summed as they are."""
    from llmserver_b200.parts import FEED_FORWARDS, Runtime
    act = torch_type(dtype)
    weights = _experts(width, experts, ff, width + tokens, act)
    params = {"hidden": width, "experts": experts, "top": top, "intermediate": ff, "activation": "silu", "weight_on": "input",
              "correction": False, "route_scale": 1.0}
    part = FEED_FORWARDS.get("routed_experts")(params, {k: (v if k == "router" else v.to(act)).to(DEVICE) for k, v in weights.items()},
                                               Runtime(act, torch.device(DEVICE)))
    h = torch.randn((tokens, width), generator=torch.Generator().manual_seed(3)).to(act)
    got = part.forward(h.to(DEVICE))
    mlp = {"router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    named = {"m." + k: v.double() for k, v in weights.items()}
    want = plain.feed_forward(h.double(), mlp, named, "m.")
    clear = plain.route_margin(h.double(), mlp, named, "m.") >= (MARGIN if dtype == "bfloat16" else 1e-6)
    assert int(clear.sum()) >= tokens // 3
    close(got, want, dtype, "experts", rows=clear)


def _mixer_alone(kind, params, weights, position, xs, steps, dtype, page_size):
    """Runs a mixer part by itself over hand-made inputs.  ``xs``: per sequence its rows [T, hidden] (float64);
    ``steps``: a list of steps, each a list of (sequence, tokens now).  Returns per sequence the outputs [T, out]."""
    from llmserver_b200.cache import CacheManager
    from llmserver_b200.engine.batch import SequenceSlice, build_batch
    from llmserver_b200.parts import MIXERS, POSITION_ENCODINGS, EntryCache, Runtime
    act = torch_type(dtype)
    runtime = Runtime(act, torch.device(DEVICE))
    cls = MIXERS.get(kind)
    part = cls(params, {k: (v.float() if k.endswith("sink") else v.to(act)).to(DEVICE) for k, v in weights.items()}, runtime)
    if position is not None:
        part.attach(POSITION_ENCODINGS.get(position.kind)(position.as_dict(), {}, runtime))
    cache = CacheManager([cls.cache_need(params)], page_size, 160, num_slots=8, prefix_sharing=False)
    cache.materialize(runtime.device, act)
    # leave the pool out of order: pages handed out and given back in another order
    cache.admit("warm")
    cache.ensure("warm", 9 * page_size)
    cache.free("warm")
    k_pages, v_pages, group = cache.pages_of_entry(0)
    view = EntryCache(k_pages=k_pages, v_pages=v_pages, group=group, writes=True)
    done = [0] * len(xs)
    outs = [[] for _ in xs]
    for s in range(len(xs)):
        cache.admit(s)
    for step in steps:
        slices, rows = [], []
        for s, now in step:
            cache.ensure(s, done[s] + now)
            slices.append(SequenceSlice(s, [0] * now, done[s], [], [cache.table(s, 0)], cache.slot_of(s)))
            rows.append(xs[s][done[s]:done[s] + now])
        batch = build_batch(slices, 1, DEVICE)
        out = part.forward(torch.cat(rows).to(act).to(DEVICE), batch, view)
        assert int(batch.error_flag.item()) == 0
        at = 0
        for s, now in step:
            outs[s].append(out[at:at + now].cpu())
            at += now
            done[s] += now
            cache.advance(s, done[s])
    return [torch.cat(parts) for parts in outs]


def _spiked(length, width, seed, spikes, act):
    """Rows of unit size of which a few are several times larger: as keys (and queries) they carry whole softmax rows.
    (Eight times in 32-bit; three in bfloat16, where a score's rounding error grows with the score.)"""
    x = torch.randn((length, width), generator=torch.Generator().manual_seed(seed), dtype=F64)
    for place in spikes:
        x[place] *= 8.0 if act == torch.float32 else 3.0
    return x.to(act).double()


def _steps(lengths, sizes):
    """Steps in which sequence s brings sizes[s][i] tokens to step i (0: it sits the step out) while it has tokens left;
    a sequence's last size takes all that is left."""
    left, steps = list(lengths), []
    for turn in range(max(len(row) for row in sizes)):
        step = []
        for s, row in enumerate(sizes):
            size = row[turn] if turn < len(row) else 0
            size = left[s] if turn == len(row) - 1 else min(size, left[s])
            if size > 0:
                step.append((s, size))
                left[s] -= size
        if step:
            steps.append(step)
    assert left == [0] * len(lengths)
    return steps


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,temperature,page_size", [(4, 2, 16, (0.5, 7), 4), (6, 1, 24, None, 8), (3, 3, 40, (0.3, 64), 16),
                                                                      (4, 2, 64, (0.3, 16), 16), (2, 1, 128, None, 8)])
def test_attention_whose_values_are_its_keys(dtype, heads, kv_heads, dim, temperature, page_size):
    """A far key among hundreds, at a page's last slot and at its first, carries some rows; prompts and single tokens."""
    width, length = 48, 300
    act = torch_type(dtype)
    generator = torch.Generator().manual_seed(dim)
    weights = {"q": torch.randn((heads * dim, width), generator=generator) * 1.2 / math.sqrt(width),
               "k": torch.randn((kv_heads * dim, width), generator=generator) * 1.2 / math.sqrt(width),
               "o": torch.randn((width, heads * dim), generator=generator) / math.sqrt(heads * dim)}
    weights = {k: v.to(torch.bfloat16) for k, v in weights.items()}
    params = {"hidden": width, "heads": heads, "kv_heads": kv_heads, "head_dim": dim, "scale": 1.0 / math.sqrt(dim), "values_are_keys": True,
              "unit_sink": True, "precise_weights": True, "query_temperature": temperature, "names": (("q", "q"), ("k", "k"), ("o", "o"))}
    spikes = [2, page_size - 1, page_size, 5 * page_size - 1, 149]
    xs = [_spiked(length, width, 1, spikes, act), _spiked(70, width, 2, [0, 33], act)]
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "scale": params["scale"],
             "q_temp": {"coef": temperature[0], "every": temperature[1]} if temperature else None}
    named = {"m." + k: v.double() for k, v in weights.items()}
    want = [plain.attention_mixer(x, torch.arange(x.shape[0]), mixer, named, "m.") for x in xs]
    without = plain.attention_mixer(xs[0], torch.arange(length), mixer, named, "m.", one_more=False)
    assert ((without - want[0]).abs().amax(-1) / want[0].abs().amax(-1)).max() > 3 * ALLOWED[dtype], "the one in the denominator does not show"
    cuts = _steps([length, 70], [[200, 1, 60, 2] + [1] * 30 + [length], [2, 1, 1, 40, 0, 0, 0, 70]])
    for steps in ([[(0, length), (1, 70)]], cuts):
        got = _mixer_alone("gqa_attention", params, weights, None, xs, steps, dtype, page_size)
        for s in range(2):
            close(got[s], want[s], dtype, f"sequence {s} in {len(steps)} steps")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,rot_dim,vdim,q_rank,kv_rank,window,dims,page_size", [
    (3, 16, 8, 8, 24, 40, 5, 8, 4), (5, 8, 12, 24, 72, 16, 0, 6, 8), (2, 24, 8, 40, 16, 40, 1, 8, 4), (4, 32, 32, 64, 64, 96, 70, 32, 16),
    (8, 64, 16, 32, 128, 48, 150, 16, 8), (2, 16, 0, 16, 32, 64, 33, 0, 16), (20, 8, 8, 8, 32, 56, 40, 8, 16)])
def test_latent_attention_with_a_turning_key_part(dtype, heads, dim, rot_dim, vdim, q_rank, kv_rank, window, dims, page_size):
    """Spiked rows give keys whose turned part carries whole softmax rows while they are in the window, and drops out of
    them one token later: the key that has just come in, the one that has just left, keys at page borders and near the
    start, for prompt rows and for single tokens; sinks from -2 to 3."""
    from llmserver_b200.config.spec import PartSpec
    width, length = 64, 260
    act = torch_type(dtype)
    generator = torch.Generator().manual_seed(kv_rank + heads)

    def draw(rows, columns, gain=1.0):
        return (torch.randn((rows, columns), generator=generator) * gain / math.sqrt(columns)).to(torch.bfloat16)
    weights = {"dq": draw(q_rank, width, 2.0), "dq.norm": (1 + 0.1 * torch.randn(q_rank, generator=generator)).to(torch.bfloat16),
               "uq": draw(heads * (dim + rot_dim), q_rank, 1.5), "dkv": draw(kv_rank + rot_dim, width, 2.0),
               "dkv.norm": (1 + 0.1 * torch.randn(kv_rank, generator=generator)).to(torch.bfloat16), "uk": draw(heads * dim, kv_rank, 1.5),
               "uv": draw(heads * vdim, kv_rank), "o": draw(width, heads * vdim), "sink": torch.linspace(-2.0, 3.0, heads)}
    params = {"hidden": width, "heads": heads, "dim": dim, "rot_dim": rot_dim, "value_dim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
              "scale": 1.0 / math.sqrt(dim + rot_dim), "eps": 1e-6, "window": window or None, "sinks": True}
    position = PartSpec.of("rotary", head_dim=rot_dim, theta=1e4, rotary_dim=dims, pairing="interleaved") if dims else None
    spikes = [1, page_size - 1, page_size, 100, 101, 199]
    xs = [_spiked(length, width, 3, spikes, act), _spiked(90, width, 4, [0, 50], act)]
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": params["scale"],
             "mask": {"size": window} if window else None, "rot": {"base": 1e4, "dims": dims} if dims else None}
    named = {"m." + k: v.double() for k, v in weights.items()}

    def plain_out(x, shift=0, sinks=True):
        local = dict(named)
        if not sinks:
            local["m.sink"] = torch.full((heads,), -1e30, dtype=F64)
        positions = torch.arange(x.shape[0])
        return plain.latent_mixer(x, positions, mixer, local, "m.", 1e-6, plain.latent_kv(x, positions, mixer, local, "m.", 1e-6), shift)
    want = [plain_out(x) for x in xs]
    wrong = [plain_out(xs[0], sinks=False)] + ([plain_out(xs[0], shift=1), plain_out(xs[0], shift=-1)] if window > 1 else [])
    for other in wrong:
        assert ((other - want[0]).abs().amax(-1) / want[0].abs().amax(-1)).max() > 3 * ALLOWED[dtype], "a fault would not show"
    # single tokens from just before the spiked rows at 100 and 101 leave the window to well past it, portions down to two
    # tokens, and single tokens again
    head = min(100 + max(window, 2) - 3, length - 40)
    cuts = _steps([length, 90], [[head] + [1] * 6 + [2, 31, 3] + [1] * 20 + [length], [3] + [1] * 6 + [0, 50, 2] + [0] * 20 + [90]])
    for steps in ([[(0, length), (1, 90)]], cuts):
        got = _mixer_alone("latent_attention", params, weights, position, xs, steps, dtype, page_size)
        for s in range(2):
            close(got[s], want[s], dtype, f"sequence {s} in {len(steps)} steps")


# ------------------------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompt_and_token_by_token(folders, name, dtype):
    vocab = ZERIDRA[name][0]["vocab"]
    tokens = tokens_for(vocab, 203, 7)
    for name in variants(name, dtype):
        records = traces.whole("r", tokens)
        got, _ = run_in_process(folders[name], dtype, records, traces.rounded(len(tokens)))
        compare(got, records, {"r": tokens}, folders[name], dtype, f"{name} whole")
        records = traces.tail_decoded("r", tokens, 90)      # the windows of these models pass over decoded tokens
        got, _ = run_in_process(folders[name], dtype, records, traces.rounded(len(tokens)), page_size=8)
        compare(got, records, {"r": tokens}, folders[name], dtype, f"{name} tail decoded")
        short = tokens[:30]                                 # and from the very first token on, one by one
        records = traces.tail_decoded("r", short, 29)
        got, _ = run_in_process(folders[name], dtype, records, traces.rounded(len(short)), page_size=4)
        compare(got, records, {"r": short}, folders[name], dtype, f"{name} decoded from the start")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_down_to_two_tokens(folders, name, dtype):
    vocab = ZERIDRA[name][0]["vocab"]
    tokens = tokens_for(vocab, 181, 11)
    records = traces.portions("r", tokens, [7, 2, 5, 3, 2, 16, 33, 2, 64, 1, 17])
    for name in variants(name, dtype):
        got, _ = run_in_process(folders[name], dtype, records, traces.rounded(len(tokens)), page_size=8)
        compare(got, records, {"r": tokens}, folders[name], dtype, f"{name} portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_mixed_batches_reuse_pages_and_slots(folders, name, dtype):
    vocab = ZERIDRA[name][0]["vocab"]
    lengths = {"r0": 110, "r1": 67, "r2": 40, "r3": 131, "r4": 64, "r5": 18, "r6": 99}
    requests = {key: tokens_for(vocab, length, 31 + index) for index, (key, length) in enumerate(lengths.items())}
    records, peak = traces.mixed(requests, seed=5)
    for name in variants(name, dtype):
        got, replayer = run_in_process(folders[name], dtype, records, peak)
        compare(got, records, requests, folders[name], dtype, f"{name} mixed")
        for group in replayer.cache.groups:
            if group.window is None:
                assert group.pool.allocations > group.pool.num_pages, "the trace was meant to reuse pages"
        assert replayer.cache.slots.num_slots == 4 and len(replayer.cache.slots.free) == 4


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(folders, dtype):
    name = "all_kinds"
    vocab = ZERIDRA[name][0]["vocab"]
    tokens = tokens_for(vocab, 330, 3)
    records = traces.tail_decoded("r", tokens, tail=322)
    for name in variants(name, dtype):
        got, _ = run_in_process(folders[name], dtype, records, traces.rounded(len(tokens)))
        compare(got, records, {"r": tokens}, folders[name], dtype, f"{name} long decoding")


def test_a_window_one_token_off_or_a_missing_sink_would_show(folders):
    for name in ("latent_only", "all_kinds", "tensor_core_sizes"):
        config, weights = plain_model_of(folders[name])
        tokens = tokens_for(config["vocab"], 120, 13)
        want = plain_logits(folders[name], tokens)[0]
        scale = np.abs(want).max(axis=-1)
        for wrong in ({"window_shift": 1}, {"window_shift": -1}, {"drop_sinks": True}):
            off = plain.forward(config, weights, tokens, **wrong).numpy()
            assert (np.abs(off - want).max(axis=-1) / scale).max() > 2 * ALLOWED["bfloat16"], (name, wrong)


def test_float32_logits_do_not_depend_on_the_cut(folders):
    name = "all_kinds"
    vocab = ZERIDRA[name][0]["vocab"]
    tokens = tokens_for(vocab, 120, 19)
    other = tokens_for(vocab, 75, 20)
    whole, _ = run_in_process(folders[name], "float32", traces.whole("r", tokens), 128)
    pieces, _ = run_in_process(folders[name], "float32", traces.portions("r", tokens, [3, 2, 40, 1, 1, 9]), 128, page_size=4)
    assert np.array_equal(np.concatenate([pieces[step] for step in sorted(pieces)]), whole[0])
    records, peak = traces.mixed({"r": tokens, "o": other}, seed=2)
    mixed, _ = run_in_process(folders[name], "float32", records, peak)
    fed = 0
    for record in records:
        row = 0
        for entry in record["entries"]:
            for place in entry["want"]:
                if entry["id"] == "r":
                    assert np.array_equal(mixed[record["step"]][row], whole[0][fed + place])
                row += 1
            if entry["id"] == "r":
                fed += len(entry["tokens"])


def test_bfloat16_rows_do_not_depend_on_their_batch(folders):
    name = "tensor_core_sizes+all"
    vocab = ZERIDRA["tensor_core_sizes"][0]["vocab"]
    requests = {"r": tokens_for(vocab, 170, 19), "o": tokens_for(vocab, 45, 20), "p": tokens_for(vocab, 90, 21)}
    clear = plain_logits(folders[name], requests["r"])[1]
    alone, _ = run_in_process(folders[name], "bfloat16", traces.whole("r", requests["r"]), 192)
    records, peak = traces.mixed(requests, seed=4)
    mixed, _ = run_in_process(folders[name], "bfloat16", records, peak)
    fed, seen = 0, 0
    for record in records:
        row = 0
        for entry in record["entries"]:
            for place in entry["want"]:
                if entry["id"] == "r" and clear[fed + place] >= MARGIN:
                    want = alone[0][fed + place]
                    assert np.abs(mixed[record["step"]][row] - want).max() <= ALLOWED["bfloat16"] * np.abs(want).max()
                    seen += 1
                row += 1
            if entry["id"] == "r":
                fed += len(entry["tokens"])
    assert seen > 20


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_engine(folders, name, dtype):
    """Requests of unequal length through the engine's own scheduler (portions, continuous batching, a pool so small
    that pages come back and are used again): every generated token maximises the plain logits of its own prefix."""
    from llmserver_b200 import Engine
    vocab = ZERIDRA[name][0]["vocab"]
    prompts = [tokens_for(vocab, length, 50 + length) for length in (5, 23, 41, 9, 30)]
    engine = Engine(folders[name], max_new_tokens=10, max_batch_size=3, max_num_batched_tokens=32, prefill_chunk_size=12,
                    kv_cache_num_blocks=40, kv_cache_block_size=4, ignore_eos=True, dtype=dtype)
    if name == "tensor_core_sizes":
        engine.warmup()      # products tuned and decode graphs captured ahead of the first request
    generated = engine.generate(prompts)
    assert all(len(tokens) == 10 for tokens in generated)
    for prompt, tokens in zip(prompts, generated):
        logits, clear = plain_logits(folders[name], list(prompt) + list(tokens))
        for index, token in enumerate(tokens):
            row = logits[len(prompt) - 1 + index]
            if dtype == "bfloat16" and clear[:len(prompt) + index].min() < MARGIN:
                break       # a close routing call somewhere in the prefix: the continuation may differ legitimately
            assert row[token] >= row.max() - 2 * ALLOWED[dtype] * np.abs(row).max(), f"token {index} of a prompt of {len(prompt)}"
    engine.cache.check_invariants()
    assert engine.cache.available() == engine.cache.capacity()


def test_trace_run_program(folders, tmp_path):
    name, dtype = "all_kinds", "float32"
    vocab = ZERIDRA[name][0]["vocab"]
    requests = {"x": tokens_for(vocab, 90, 1), "y": tokens_for(vocab, 33, 2), "z": tokens_for(vocab, 130, 3)}
    records, peak = traces.mixed(requests, seed=9, max_live=2)
    out_dir = tmp_path / "out"
    process = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders[name],
                              "--dtype", dtype, "--out", str(out_dir), "--max-tokens", str(peak)],
                             input="\n".join(json.dumps(record) for record in records) + "\n",
                             capture_output=True, text=True, timeout=600)
    assert process.returncode == 0, process.stderr[-2000:]
    assert [line for line in process.stdout.splitlines() if line.startswith("done ")] == [f"done {r['step']}" for r in records]
    got = {}
    for record in records:
        wanted = sum(len(entry["want"]) for entry in record["entries"])
        if wanted:
            got[record["step"]] = np.fromfile(out_dir / f"{record['step']}.f32", dtype="<f4").reshape(wanted, vocab)
    compare(got, records, requests, folders[name], dtype, f"trace_run {name}")


def test_generate_command(folders):
    """The command line a user generates with: ids in, ids out, the model chosen by its config.json."""
    name = "all_kinds"
    vocab = ZERIDRA[name][0]["vocab"]
    prompts = [tokens_for(vocab, 19, 71), tokens_for(vocab, 3, 72)]
    command = [sys.executable, "-m", "llmserver_b200.cli.generate", "--model", folders[name], "--dtype", "float32",
               "--max-new-tokens", "6", "--ignore-eos", "--block-size", "8", "--json"]
    for prompt in prompts:
        command += ["--prompt-ids", ",".join(str(token) for token in prompt)]
    process = subprocess.run(command, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert process.returncode == 0, process.stderr[-2000:]
    generated = json.loads(process.stdout.strip().splitlines()[-1])["generated"]
    for prompt, tokens in zip(prompts, generated):
        assert len(tokens) == 6
        logits = plain_logits(folders[name], list(prompt) + list(tokens))[0]
        assert tokens == [int(logits[len(prompt) - 1 + index].argmax()) for index in range(6)]
