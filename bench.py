#!/usr/bin/env python3
"""Headline benchmark: decode tokens per second of the Qwen3-8B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B]

One "step" is one decode step of the whole batch.  The default run builds the 8B shape (36 layers,
width 4096, 32/8 heads of 128, intermediate 12288, vocabulary 151936) with seeded random bfloat16
weights, puts ``--batch`` requests (default 8) at a context whose mean over the timed steps is 3072
(2048-token prompts decoded to 4096), and times K decode steps with CUDA events after W warm-up steps.
It prints ONE JSON line: ``value`` is decoded tokens per second on the device, ``e2e`` the same through
``llmserver_b200.Engine`` with host token ids in and sampled ids out, ``prefill`` a 2048-token prompt
in one step, ``roofline`` the decode step's bytes over its time against the measured copy bandwidth,
``points`` decode at batch 1 and 64.  Inputs larger than L2: every step streams all weights (16 GB).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from llmserver_b200.cli.harness import (CONTEXT, MEAN_DECODE_CONTEXT, PAGE_SIZE, PROMPT, QWEN3_8B, ClockSampler,  # noqa: E402
                                        Harness, decode_bytes, prefill_flops, read_peaks)


def reference_arm(args) -> int:
    """Runs the unmodified reference (a copy of its files under baseline/_ref) on the same metric and configuration, in
    a process of its own that imports nothing of this package: ``baseline/reference_arm.py`` drives the reference's
    ``model_loader`` and ``Engine`` over a model folder with seeded random weights of the benchmark's shape, which is
    written here first.  Whatever stops it is printed as ``unavailable`` in its own words."""
    import shutil
    import subprocess
    import tempfile

    line = {"impl": "reference", "metric": "decode tok/s (Qwen3-8B shape, batch 8, context 4096)", "unit": "tokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic: seeded random weights N(0,0.02), uniform random token ids"}

    def unavailable(why: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": " ".join(why.split())[:700]}))
        return 0

    reference = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isfile(os.path.join(reference, "utils", "engine.py")):
        return unavailable("baseline/_ref does not hold the reference's files: pip cannot install AshvinSehgal/LLMServer (it has "
                           "neither setup.py nor pyproject.toml), so it runs from a plain copy of its files, which is missing here")
    if args.gpus != 1:
        return unavailable("the reference's engine is measured on one GPU, like this one")
    import torch
    import llmserver_b200.models  # noqa: F401  (registers the architecture)
    from llmserver_b200.config import Qwen3Config
    from llmserver_b200.weights import write_model_folder
    if not torch.cuda.is_available():
        return unavailable("no CUDA device is visible")
    raw = dict(QWEN3_8B, num_hidden_layers=args.layers, bos_token_id=1, eos_token_id=2, pad_token_id=0)
    free = {path: shutil.disk_usage(path).free for path in ("/dev/shm", tempfile.gettempdir()) if os.path.isdir(path)}
    need = 2.2 * (args.layers * 0.2e9 + 1.3e9) + (1 << 30)
    places = [path for path, room in free.items() if room > need]
    if not places:
        return unavailable(f"no room for the {need / 1e9:.0f} GB model folder the reference's loader reads: free space {free}")
    folder = tempfile.mkdtemp(prefix="llmserver_b200_ref_", dir=places[0])
    try:
        write_model_folder(Qwen3Config.from_dict(raw), folder, 0, torch.bfloat16, device="cuda:0")
        with open(os.path.join(folder, "config.json")) as handle:
            config_json = json.load(handle)
        config_json.update(bos_token_id=1, eos_token_id=2, pad_token_id=0, torch_dtype="bfloat16")
        with open(os.path.join(folder, "config.json"), "w") as handle:
            json.dump(config_json, handle)
        with open(os.path.join(folder, "generation_config.json"), "w") as handle:
            json.dump({"bos_token_id": 1, "eos_token_id": 2, "pad_token_id": 0}, handle)
        torch.cuda.empty_cache()
        command = [sys.executable, os.path.join(ROOT, "baseline", "reference_arm.py"), "--model", folder, "--batch", str(args.batch),
                   "--steps", str(args.steps), "--warmup", str(max(args.warmup, 3)), "--context-mean", str(MEAN_DECODE_CONTEXT),
                   "--context", str(CONTEXT), "--block-size", str(PAGE_SIZE)]
        environment = dict(os.environ, HF_HUB_OFFLINE="1", TRANSFORMERS_OFFLINE="1", PYTHONPATH=reference)
        try:
            done = subprocess.run(command, capture_output=True, text=True, timeout=1500, env=environment, cwd=reference)
        except subprocess.TimeoutExpired:
            return unavailable("the reference did not finish within 1500 s")
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    result = None
    for text in reversed(done.stdout.strip().splitlines()):
        try:
            result = json.loads(text)
            break
        except ValueError:
            continue
    if result is None:
        tail = (done.stderr or done.stdout).strip().splitlines()[-3:]
        return unavailable(f"the reference's process ended with code {done.returncode}: " + " | ".join(tail))
    if "unavailable" in result:
        return unavailable("the reference failed on this box: " + result["unavailable"])
    config = Qwen3Config.from_dict(raw)
    line.update(value=round(result["value"], 1), ms_per_step=round(result["ms_per_step"], 4),
                e2e={key: (round(value, 1) if isinstance(value, float) else value) for key, value in result["e2e"].items()},
                config={"model": "Qwen3-8B shape", "layers": args.layers, "layers_full": QWEN3_8B["num_hidden_layers"],
                        "hidden": config.hidden_size, "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
                        "head_dim": config.head_dim, "intermediate": config.intermediate_size, "vocab": config.vocab_size,
                        "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT,
                        "decode_context_mean": round(result["mean_context"]), "page_size": PAGE_SIZE, "parallelism": "none (1 GPU)",
                        "path": "utils.model_loader + utils.engine.Engine, paged decode, CUDA graphs"},
                reference={key: result[key] for key in ("load_s", "prefill_s", "graphs", "paged_decode") if key in result})
    print(json.dumps(line))
    return 0


def design_comparison(args) -> int:
    """Gefarax beside the Qwen3 decoder of equal size: a 2048-token prompt in one step and decode steps at batch 1, 8
    and 64 (contexts averaging 3072), device-timed like the headline run; bytes and FLOPs counted per step, fractions of
    the measured peaks.  Random bfloat16 weights, a few layers of each size."""
    import torch
    from llmserver_b200.cli.harness import (GEFARAX_SIZES, dense_step_cost, dense_twin_config, gefarax_config,
                                            gefarax_step_cost)
    import llmserver_b200.models  # noqa: F401

    os.environ["PATH"] = os.path.dirname(sys.executable) + os.pathsep + os.environ.get("PATH", "")
    layers = args.layers if "--layers" in " ".join(sys.argv) else 4
    peaks, peak_source = read_peaks()
    wanted = args.sizes.split(",") if args.sizes else list(GEFARAX_SIZES)
    steps, warmup = min(args.steps, 32), max(3, min(args.warmup, 4))
    results = {}
    with ClockSampler() as clocks:
        for name in wanted:
            size = GEFARAX_SIZES[name]
            results[name] = {"size": size}
            for label, config, cost in (("gefarax", gefarax_config(size, layers), gefarax_step_cost),
                                        ("dense", dense_twin_config(size, layers), dense_step_cost)):
                harness = Harness(layers, 64, config=config)
                row = {}
                prefill_ms = harness.time_prefill(PROMPT)
                _, flops = cost(size, layers, PROMPT, 0, PROMPT * (PROMPT + 1) / 2)
                row["prefill"] = {"ms": round(prefill_ms, 3), "tokens_per_s": round(PROMPT / prefill_ms * 1e3),
                                  "tflops": round(flops / prefill_ms / 1e9, 1),
                                  "frac_of_bf16_burst": round(flops / prefill_ms / 1e9 / peaks["bf16_tflops"], 3)}
                for batch in (1, 8, 64):
                    harness.time_decode(batch, 4, 3)
                    run = harness.time_decode(batch, steps, warmup)
                    bytes_, _ = cost(size, layers, batch, batch * run["mean_context"], batch * run["mean_context"])
                    gbs = bytes_ / run["ms_per_step"] / 1e6
                    row[f"decode_b{batch}"] = {"ms": round(run["ms_per_step"], 4), "tokens_per_s": round(run["tokens_per_s"], 1),
                                               "gb_per_step": round(bytes_ / 1e9, 3), "gbs": round(gbs, 1),
                                               "frac_of_copy": round(gbs / peaks["hbm_gbs"], 3)}
                results[name][label] = row
                harness.close()
    print(json.dumps({"design": "gefarax", "beside": "Qwen3 dense of equal width, heads and active feed-forward", "layers": layers,
                      "prompt": PROMPT, "decode_context_mean": MEAN_DECODE_CONTEXT, "dtype": "bf16",
                      "data": "synthetic: seeded random weights, uniform random token ids", "peaks": {**peaks, "source": peak_source},
                      "clocks": clocks.summary(), "sizes": results}))
    return 0


def dikusun_comparison(args) -> int:
    """Dikusun beside the Qwen3 decoder of equal width, heads and feed-forward: a 2048-token prompt in one step and decode
    steps at batch 1, 8 and 64 (contexts averaging 3072), device-timed like the headline run; bytes and FLOPs counted per
    step, fractions of the measured peaks.  Random bfloat16 weights; four layers of one kind of mixer, or a mix."""
    from llmserver_b200.cli.harness import (DIKUSUN_SIZES, dikusun_config, dikusun_dense_cost, dikusun_dense_twin,
                                            dikusun_step_cost)
    import llmserver_b200.models  # noqa: F401

    os.environ["PATH"] = os.path.dirname(sys.executable) + os.pathsep + os.environ.get("PATH", "")
    layers = args.layers if "--layers" in " ".join(sys.argv) else 4
    peaks, peak_source = read_peaks()
    wanted = args.sizes.split(",") if args.sizes else list(DIKUSUN_SIZES)
    steps, warmup = min(args.steps, 32), max(3, min(args.warmup, 4))
    results, dense_done = {}, {}
    with ClockSampler() as clocks:
        for name in wanted:
            size = DIKUSUN_SIZES[name]
            results[name] = {"kinds": list(size["kinds"])}
            arms = [("dikusun", dikusun_config(size, layers), dikusun_step_cost)]
            if size["width"] not in dense_done:
                arms.append(("dense", dikusun_dense_twin(size, layers), dikusun_dense_cost))
            for label, config, cost in arms:
                harness = Harness(layers, 64, config=config)
                row = {}
                prefill_ms = harness.time_prefill(PROMPT)
                _, flops = cost(size, layers, PROMPT, 1, 0)
                row["prefill"] = {"ms": round(prefill_ms, 3), "tokens_per_s": round(PROMPT / prefill_ms * 1e3),
                                  "tflops": round(flops / prefill_ms / 1e9, 1),
                                  "frac_of_bf16_burst": round(flops / prefill_ms / 1e9 / peaks["bf16_tflops"], 3)}
                for batch in (1, 8, 64):
                    harness.time_decode(batch, 4, 3)
                    run = harness.time_decode(batch, steps, warmup)
                    bytes_, _ = cost(size, layers, batch, batch, run["mean_context"])
                    gbs = bytes_ / run["ms_per_step"] / 1e6
                    row[f"decode_b{batch}"] = {"ms": round(run["ms_per_step"], 4), "tokens_per_s": round(run["tokens_per_s"], 1),
                                               "gb_per_step": round(bytes_ / 1e9, 3), "gbs": round(gbs, 1),
                                               "frac_of_copy": round(gbs / peaks["hbm_gbs"], 3),
                                               "graph_steps": harness.step_function.graph_steps}
                if label == "dense":
                    dense_done[size["width"]] = row
                else:
                    results[name][label] = row
                harness.close()
            results[name]["dense"] = dense_done[size["width"]]
    print(json.dumps({"design": "dikusun", "beside": "Qwen3 dense of equal width, heads and feed-forward", "layers": layers,
                      "prompt": PROMPT, "decode_context_mean": MEAN_DECODE_CONTEXT, "dtype": "bf16",
                      "data": "synthetic: seeded random weights, uniform random token ids", "peaks": {**peaks, "source": peak_source},
                      "clocks": clocks.summary(), "sizes": results}))
    return 0


def vibepel_comparison(args) -> int:
    """Vibepel beside the Dikusun model of equal size (differential attention over the same window for a parallel layer,
    gated linear attention for time mixing) and beside the Qwen3 decoder of equal width, heads and feed-forward width: a
    2048-token prompt in one step and decode steps at batch 1, 8 and 64 (contexts averaging 3072), device-timed like the
    headline run; bytes and FLOPs counted per step, fractions of the measured peaks.  Random bfloat16 weights."""
    from llmserver_b200.cli.harness import (VIBEPEL_SIZES, dikusun_dense_cost, dikusun_dense_twin, dikusun_step_cost,
                                            vibepel_config, vibepel_dikusun_twin, vibepel_step_cost)
    import llmserver_b200.models  # noqa: F401

    os.environ["PATH"] = os.path.dirname(sys.executable) + os.pathsep + os.environ.get("PATH", "")
    layers = args.layers if "--layers" in " ".join(sys.argv) else 4
    peaks, peak_source = read_peaks()
    wanted = args.sizes.split(",") if args.sizes else list(VIBEPEL_SIZES)
    steps, warmup = min(args.steps, 32), max(3, min(args.warmup, 4))
    results, dense_done = {}, {}
    with ClockSampler() as clocks:
        for name in wanted:
            size = VIBEPEL_SIZES[name]
            results[name] = {"kinds": list(size["kinds"])}
            twin, twin_config = vibepel_dikusun_twin(size, layers)
            arms = [("vibepel", size, vibepel_config(size, layers), vibepel_step_cost), ("dikusun", twin, twin_config, dikusun_step_cost)]
            if size["width"] not in dense_done:
                arms.append(("dense", twin, dikusun_dense_twin(twin, layers), dikusun_dense_cost))
            for label, sizes, config, cost in arms:
                harness = Harness(layers, 64, config=config)
                row = {}
                prefill_ms = harness.time_prefill(PROMPT)
                _, flops = cost(sizes, layers, PROMPT, 1, 0)
                row["prefill"] = {"ms": round(prefill_ms, 3), "tokens_per_s": round(PROMPT / prefill_ms * 1e3),
                                  "tflops": round(flops / prefill_ms / 1e9, 1),
                                  "frac_of_bf16_burst": round(flops / prefill_ms / 1e9 / peaks["bf16_tflops"], 3)}
                for batch in (1, 8, 64):
                    harness.time_decode(batch, 4, 3)
                    run = harness.time_decode(batch, steps, warmup)
                    bytes_, _ = cost(sizes, layers, batch, batch, run["mean_context"])
                    gbs = bytes_ / run["ms_per_step"] / 1e6
                    row[f"decode_b{batch}"] = {"ms": round(run["ms_per_step"], 4), "tokens_per_s": round(run["tokens_per_s"], 1),
                                               "gb_per_step": round(bytes_ / 1e9, 3), "gbs": round(gbs, 1),
                                               "frac_of_copy": round(gbs / peaks["hbm_gbs"], 3),
                                               "graph_steps": harness.step_function.graph_steps}
                if label == "dense":
                    dense_done[size["width"]] = row
                else:
                    results[name][label] = row
                harness.close()
            results[name]["dense"] = dense_done[size["width"]]
    print(json.dumps({"design": "vibepel", "beside": "Dikusun of equal size (attention for parallel, gla for wkv); Qwen3 dense of equal width, heads and feed-forward width",
                      "layers": layers, "prompt": PROMPT, "decode_context_mean": MEAN_DECODE_CONTEXT, "dtype": "bf16",
                      "data": "synthetic: seeded random weights, uniform random token ids", "peaks": {**peaks, "source": peak_source},
                      "clocks": clocks.summary(), "sizes": results}))
    return 0


def zeridra_comparison(args) -> int:
    """Zeridra beside the Gefarax model of equal size (grouped attention with keys and values of 128 and the same routed
    experts): a 2048-token prompt in one step and decode steps at batch 1, 8 and 64 (contexts averaging 3072),
    device-timed like the headline run; bytes and FLOPs counted per step, fractions of the measured peaks.  Random
    bfloat16 weights; four layers of one kind of mixer, or a mix with a layer that reads another layer's cache."""
    from llmserver_b200.cli.harness import (ZERIDRA_SIZES, zeridra_config, zeridra_gefarax_twin, zeridra_step_cost, zeridra_twin_cost)
    import llmserver_b200.models  # noqa: F401

    os.environ["PATH"] = os.path.dirname(sys.executable) + os.pathsep + os.environ.get("PATH", "")
    layers = args.layers if "--layers" in " ".join(sys.argv) else 4
    peaks, peak_source = read_peaks()
    wanted = args.sizes.split(",") if args.sizes else list(ZERIDRA_SIZES)
    steps, warmup = min(args.steps, 32), max(3, min(args.warmup, 4))
    results, twin_done = {}, {}
    with ClockSampler() as clocks:
        for name in wanted:
            size = ZERIDRA_SIZES[name]
            results[name] = {"kinds": list(size["kinds"])}
            arms = [("zeridra", size, zeridra_config(size, layers), zeridra_step_cost)]
            if size["width"] not in twin_done:
                twin, twin_config = zeridra_gefarax_twin(size, layers)
                arms.append(("gefarax", twin, twin_config, zeridra_twin_cost))
            for label, sizes, config, cost in arms:
                harness = Harness(layers, 64, config=config)
                row = {}
                prefill_ms = harness.time_prefill(PROMPT)
                _, flops = cost(sizes, layers, PROMPT, 1, 0)
                row["prefill"] = {"ms": round(prefill_ms, 3), "tokens_per_s": round(PROMPT / prefill_ms * 1e3),
                                  "tflops": round(flops / prefill_ms / 1e9, 1),
                                  "frac_of_bf16_burst": round(flops / prefill_ms / 1e9 / peaks["bf16_tflops"], 3)}
                for batch in (1, 8, 64):
                    harness.time_decode(batch, 4, 3)
                    run = harness.time_decode(batch, steps, warmup)
                    bytes_, _ = cost(sizes, layers, batch, batch, run["mean_context"])
                    gbs = bytes_ / run["ms_per_step"] / 1e6
                    row[f"decode_b{batch}"] = {"ms": round(run["ms_per_step"], 4), "tokens_per_s": round(run["tokens_per_s"], 1),
                                               "gb_per_step": round(bytes_ / 1e9, 3), "gbs": round(gbs, 1),
                                               "frac_of_copy": round(gbs / peaks["hbm_gbs"], 3),
                                               "graph_steps": harness.step_function.graph_steps}
                if label == "gefarax":
                    twin_done[size["width"]] = row
                else:
                    results[name][label] = row
                harness.close()
            results[name]["gefarax"] = twin_done[size["width"]]
    print(json.dumps({"design": "zeridra", "beside": "Gefarax of equal width, heads (keys and values of 128) and routed experts",
                      "layers": layers, "prompt": PROMPT, "decode_context_mean": MEAN_DECODE_CONTEXT, "dtype": "bf16",
                      "data": "synthetic: seeded random weights, uniform random token ids", "peaks": {**peaks, "source": peak_source},
                      "clocks": clocks.summary(), "sizes": results}))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--layers", type=int, default=QWEN3_8B["num_hidden_layers"],
                        help="fewer layers than the 8B shape's 36 (layer sizes stay); the record names both numbers")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--skip-points", action="store_true", help="skip the batch-1 and batch-64 points")
    parser.add_argument("--design", default=None, choices=["gefarax", "dikusun", "vibepel", "zeridra"],
                        help="instead of the headline run: prefill and decode of this design at a few layer sizes, beside the "
                             "dense decoder of equal size (one JSON line; --layers defaults to 4 here)")
    parser.add_argument("--sizes", default=None, help="with --design: comma-separated names of the sizes to run (default: all)")
    args = parser.parse_args()
    if args.design == "gefarax":
        return design_comparison(args)
    if args.design == "dikusun":
        return dikusun_comparison(args)
    if args.design == "zeridra":
        return zeridra_comparison(args)
    if args.design == "vibepel":
        return vibepel_comparison(args)
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported (the engine has no multi-GPU path)")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    import torch

    os.environ["PATH"] = os.path.dirname(sys.executable) + os.pathsep + os.environ.get("PATH", "")
    peaks, peak_source = read_peaks()
    harness = Harness(args.layers, max(args.batch, 1 if args.skip_points else 64))
    config = harness.config
    harness.time_decode(args.batch, 4, 3)      # untimed: lets the library choose its kernels
    with ClockSampler() as clocks:
        main_run = harness.time_decode(args.batch, args.steps, args.warmup)
    points = {}
    if not args.skip_points:
        for batch in (1, 64):
            if batch == args.batch:
                points[f"decode_b{batch}"] = round(main_run["tokens_per_s"], 1)
                continue
            points[f"decode_b{batch}"] = round(harness.time_decode(batch, min(args.steps, 32), 3)["tokens_per_s"], 1)
    prefill_ms = harness.time_prefill(PROMPT)
    flops = prefill_flops(config, args.layers, PROMPT)
    e2e = harness.time_e2e(args.batch, args.steps, args.warmup)
    bytes_per_step = decode_bytes(config, args.layers, args.batch, main_run["mean_context"])
    achieved = bytes_per_step / (main_run["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": "decode tok/s (Qwen3-8B shape, batch 8, context 4096)", "value": round(main_run["tokens_per_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: seeded random weights N(0,0.02), uniform random token ids",
        "config": {"model": "Qwen3-8B shape", "layers": args.layers, "layers_full": QWEN3_8B["num_hidden_layers"],
                   "hidden": config.hidden_size, "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
                   "head_dim": config.head_dim, "intermediate": config.intermediate_size, "vocab": config.vocab_size,
                   "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT,
                   "decode_context_mean": round(main_run["mean_context"]), "page_size": PAGE_SIZE, "parallelism": "none (1 GPU)",
                   "l2": "inputs larger than L2: each step streams all weights", "peaks": peak_source},
        "clocks": clocks.summary(),
        "e2e": {key: (round(value, 1) if isinstance(value, float) else value) for key, value in e2e.items()},
        "gpu_launches": main_run["launches"],
        "prefill": {"value": round(PROMPT / (prefill_ms / 1e3), 1), "tokens": PROMPT, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
