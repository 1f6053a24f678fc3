"""What the benchmarks share: the model shapes of the published configurations, the measured peaks, a clock
sampler, the bytes and FLOPs of a step, and a harness that holds a model, a cache and a step function on the device.

``bench.py`` at the root of the repository (the headline line), ``cli/benchmark.py`` (the reference's own method and
the serving scenarios) and ``cli/microbench.py`` (single kernels and steps for the profiler) all build on this module.
"""
from __future__ import annotations

import json
import os
import threading
import time

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

def _qwen3(layers: int, hidden: int, heads: int, intermediate: int) -> dict:
    return dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=hidden,
                intermediate_size=intermediate, num_hidden_layers=layers, num_attention_heads=heads, num_key_value_heads=8,
                head_dim=128, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                max_position_embeddings=40960, hidden_act="silu", attention_bias=False, use_sliding_window=False)


# the dense Qwen3 sizes the reference publishes numbers for (docs/results.md); random weights stand in for checkpoints
SHAPES = {"8b": _qwen3(36, 4096, 32, 12288), "14b": _qwen3(40, 5120, 40, 17408), "32b": _qwen3(64, 5120, 64, 25600)}
QWEN3_8B = SHAPES["8b"]
CONTEXT = 4096          # prompts of 2048 tokens decoded to 4096
PROMPT = 2048
MEAN_DECODE_CONTEXT = (CONTEXT + PROMPT) // 2
PAGE_SIZE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as handle:
                raw = json.load(handle)
            peaks = {key: float(raw[key]) for key in FALLBACK_PEAKS if key in raw}
            if "hbm_gbs" in peaks and "bf16_tflops" in peaks:
                peaks.setdefault("bf16_tflops_sustained", peaks["bf16_tflops"])
                return peaks, "measured"
        except (OSError, ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML while the timed region runs (reads only)."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int = 0, period: float = 0.1):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.period, self.index = period, index
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:  # NVML missing: report nothing rather than fail the benchmark
            self.nvml = None

    def _loop(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self.nvml.nvmlDeviceGetClockInfo(self.handle, self.nvml.NVML_CLOCK_SM))
                mask = self.nvml.nvmlDeviceGetCurrentClocksEventReasons(self.handle) if hasattr(
                    self.nvml, "nvmlDeviceGetCurrentClocksEventReasons") else self.nvml.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nvml is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        ordered = sorted(self.samples)
        return {"sm_mhz": ordered[len(ordered) // 2] if ordered else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons)}


def weight_bytes(config, layers: int) -> float:
    """Bytes of every weight a step reads (the embedding table, of which a step reads a few rows, left out)."""
    hidden, inter, dim = config.hidden_size, config.intermediate_size, config.head_dim
    heads, kv_heads = config.num_attention_heads, config.num_key_value_heads
    per_layer = ((heads + 2 * kv_heads) * dim * hidden + hidden * heads * dim + 3 * hidden * inter + 2 * hidden + 2 * dim) * 2
    return layers * per_layer + config.vocab_size * hidden * 2 + hidden * 2


def cache_bytes_per_token(config, layers: int) -> float:
    """Bytes of keys and values one cached token holds over all layers."""
    return 2 * config.num_key_value_heads * config.head_dim * 2 * layers


def decode_bytes(config, layers: int, batch: int, context: int) -> float:
    """Bytes one decode step has to read: every weight it uses once, and the cache of the live requests."""
    return weight_bytes(config, layers) + cache_bytes_per_token(config, layers) * batch * context


def linear_flops_per_token(config, layers: int) -> float:
    hidden, inter, dim = config.hidden_size, config.intermediate_size, config.head_dim
    heads, kv_heads = config.num_attention_heads, config.num_key_value_heads
    return 2 * layers * ((heads + 2 * kv_heads) * dim * hidden + hidden * heads * dim + 3 * hidden * inter)


def attention_flops(config, layers: int, query_key_pairs: float) -> float:
    """QK^T and PV for ``query_key_pairs`` (query token, visible key) pairs, all heads and layers."""
    return 2 * 2 * config.num_attention_heads * config.head_dim * query_key_pairs * layers


def prefill_flops(config, layers: int, tokens: int) -> float:
    hidden, inter, dim = config.hidden_size, config.intermediate_size, config.head_dim
    heads, kv_heads = config.num_attention_heads, config.num_key_value_heads
    linear = 2 * tokens * ((heads + 2 * kv_heads) * dim * hidden + hidden * heads * dim + 3 * hidden * inter)
    attention = 2 * 2 * heads * dim * tokens * (tokens + 1) / 2      # QK^T and PV over the causal half
    return layers * (linear + attention) + 2 * config.vocab_size * hidden   # logits of the last token only


class Harness:
    """Model, cache and step function sized for the largest batch, reused by every measurement."""

    def __init__(self, layers: int, max_batch: int, seed: int = 0, shape: str = "8b", config=None):
        """``config``: a typed configuration of any registered architecture (then ``layers`` and ``shape`` only label the
        run); default: the Qwen3 ``shape`` with ``layers`` layers."""
        import torch
        from llmserver_b200.cache import CacheManager
        from llmserver_b200.config import Qwen3Config
        from llmserver_b200.engine.step import StepFunction
        from llmserver_b200.models import random_model

        self.torch = torch
        if config is None:
            config = Qwen3Config.from_dict(dict(SHAPES[shape], num_hidden_layers=layers))
        self.config = config
        self.layers = layers
        self.model = random_model(self.config, seed, "bfloat16", "cuda:0")
        pages = max_batch * (CONTEXT // PAGE_SIZE) + 8     # the reference benchmark's sizing rule
        self.cache = CacheManager(self.model.cache_needs(), PAGE_SIZE, pages, num_slots=max_batch, prefix_sharing=False)
        self.cache.materialize(self.model.runtime.device, self.model.runtime.dtype)
        for group in self.cache.groups:     # contents do not change the timing; avoid an all-zero cache anyway
            group.key_storage.normal_(0.0, 0.5)
            group.value_storage.normal_(0.0, 0.5)
        self.step_function = StepFunction(self.model, self.cache)
        self.generator = torch.Generator().manual_seed(seed)

    def close(self):
        """Gives the device memory back (for runs that measure several models one after the other)."""
        self.step_function = self.cache = self.model = None
        import gc
        gc.collect()
        self.torch.cuda.empty_cache()

    def tokens(self, count: int):
        return self.torch.randint(0, self.config.vocab_size, (count,), generator=self.generator).tolist()

    def place(self, batch: int, context: int):
        """Puts ``batch`` requests at ``context`` cached tokens each (pages allocated, contents as they are)."""
        for request_id in list(self.step_function.computed):
            self.step_function.release(request_id)
        ids = [f"b{index}" for index in range(batch)]
        for request_id in ids:
            self.step_function.admit(request_id)
            self.cache.ensure(request_id, context)
            self.step_function.computed[request_id] = context
        return ids

    def time_decode(self, batch: int, steps: int, warmup: int):
        torch = self.torch
        from llmserver_b200 import ops
        start_context = max(1, MEAN_DECODE_CONTEXT - steps // 2 - warmup)
        ids = self.place(batch, start_context)
        from llmserver_b200.sampling import SamplingRow
        if self.step_function.graphs is None:
            self.step_function.enable_graphs(CONTEXT, 64)
        tokens = self.tokens(batch)
        events = []
        launches_before = None
        rows = [SamplingRow() for _ in ids]
        for step in range(warmup + steps):
            if step == warmup:
                torch.cuda.synchronize()
                launches_before = ops.launch_count()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            # one decode step: batch in (one copy), forward, sampling, tokens out (one copy)
            tokens = self.step_function.run_and_sample([(request_id, [token], [0]) for request_id, token in zip(ids, tokens)], rows)
            end.record()
            if step >= warmup:
                events.append((begin, end))
        torch.cuda.synchronize()
        launches = ops.launch_count() - launches_before
        if self.step_function.graph_steps:      # replayed steps launch the captured kernels: count them per step
            launches = steps * self.launches_per_step(batch)
        self.step_function.check_errors()
        times = [begin.elapsed_time(end) for begin, end in events]
        total_ms = sum(times)
        mean_context = start_context + warmup + (steps + 1) / 2
        return {"ms_per_step": total_ms / steps, "tokens_per_s": batch * steps / (total_ms / 1e3),
                "launches": launches, "mean_context": mean_context}

    def launches_per_step(self, batch: int) -> int:
        """Kernels of this package in one decode step, counted on an eager step of the same shape."""
        from llmserver_b200 import ops
        ids = list(self.step_function.computed)[:batch]
        graphs, self.step_function.graphs = self.step_function.graphs, None
        before = ops.launch_count()
        self.step_function.run([(request_id, [0], [0]) for request_id in ids])
        count = ops.launch_count() - before + 1     # + the sampling kernel
        self.step_function.graphs = graphs
        return count

    def time_prefill(self, tokens: int, repeats: int = 3):
        torch = self.torch
        best = None
        for _ in range(repeats + 1):     # the first run warms up
            for request_id in list(self.step_function.computed):
                self.step_function.release(request_id)
            self.step_function.admit("p")
            prompt = self.tokens(tokens)
            torch.cuda.synchronize()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            self.step_function.run([("p", prompt, [tokens - 1])])
            end.record()
            torch.cuda.synchronize()
            elapsed = begin.elapsed_time(end)
            best = elapsed if best is None else min(best, elapsed)
        self.step_function.release("p")
        return best

    def time_e2e(self, batch: int, steps: int, warmup: int):
        """The same decode through the public entry point: host token ids in, sampled ids out; every
        step copies its batch from pinned host memory and reads the sampled tokens back."""
        torch = self.torch
        from llmserver_b200.engine.engine import Engine
        from llmserver_b200.engine.request import RequestStatus

        for request_id in list(self.step_function.computed):
            self.step_function.release(request_id)
        prompt_len = max(1, MEAN_DECODE_CONTEXT - steps // 2 - warmup)
        # the engine shares the model and the cache that are already on the device
        # requests that finish their prompt first decode while the others still prefill: leave room for that
        prefill_steps = -(-batch * prompt_len // max(8192, batch)) + 2
        engine = Engine(self.model, max_new_tokens=warmup + steps + prefill_steps + 8, max_batch_size=batch,
                        max_num_batched_tokens=max(8192, batch), ignore_eos=True, cache=self.cache,
                        step_function=self.step_function)
        requests = [engine.add_request(prompt_token_ids=self.tokens(prompt_len)) for _ in range(batch)]
        while any(request.status != RequestStatus.DECODING for request in requests):
            engine.step()
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        before = sum(len(request.generated_token_ids) for request in requests)
        stats_before = dict(engine.stats)
        started = time.perf_counter()
        for _ in range(steps):
            engine.step()
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - started
        generated = sum(len(request.generated_token_ids) for request in requests) - before
        if generated != batch * steps:
            raise RuntimeError(f"the timed steps produced {generated} tokens, not {batch} x {steps}")
        h2d = engine.step_function.last_batch_bytes
        for request in requests:
            engine.cancel_request(request.request_id)
        # where a step's host time goes (mean over the engine's steps; read_back is the wait for the device)
        phases = {name: 1e3 * (engine.stats[name + "_s"] - stats_before[name + "_s"]) / steps
                  for name in ("schedule", "pack_copy", "launch", "read_back", "accept")}
        return {"value": batch * steps / elapsed, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": batch * 4, "ms_per_step": elapsed * 1e3 / steps,
                "host_phases_ms": ", ".join(f"{name} {phases[name]:.3f}" for name in ("schedule", "pack_copy", "launch", "read_back", "accept"))}




# ---------------------------------------------------------------------------------------------------------------------
# Gefarax beside the dense decoder at equal size
# ---------------------------------------------------------------------------------------------------------------------
def _gefarax_size(width, heads, kv_heads, dim, vdim, experts, top, ff, shared_ff):
    return dict(width=width, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, experts=experts, top=top, ff=ff, shared_ff=shared_ff)


# Layer sizes that resemble served models: a small one with heads of 64, one whose active feed-forward and attention
# equal the Qwen3-8B shape's, and one with many small experts and value heads half the size of its key heads.
GEFARAX_SIZES = {
    "w2048-h64": _gefarax_size(2048, 32, 8, 64, 64, 32, 4, 768, 768),
    "w4096-h128": _gefarax_size(4096, 32, 8, 128, 128, 64, 6, 1792, 1536),
    "w4096-v64": _gefarax_size(4096, 64, 8, 128, 64, 128, 4, 1024, 2048),
}
COMPARE_VOCAB = 151936


def gefarax_config(size: dict, layers: int):
    """A Gefarax configuration of ``layers`` equal layers of the given sizes (no loop), with the constants of a model
    stretched from 4096 to 32768 positions."""
    from llmserver_b200.config import GefaraxConfig
    layer = {"type": "attention",
             "mixer": {"heads": size["heads"], "kv_heads": size["kv_heads"], "dim": size["dim"], "vdim": size["vdim"],
                       "scale": size["dim"] ** -0.5,
                       "rot": {"base": 150000.0, "dims": size["dim"],
                               "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}},
             "mlp": {"kind": "moe", "router": {"experts": size["experts"], "top": size["top"], "scale": 1.0},
                     "expert": {"ff": size["ff"], "limit": 7.0}, "shared": {"ff": size["shared_ff"], "limit": 7.0}}}
    return GefaraxConfig.from_dict({"architecture": "Gefarax", "vocab": COMPARE_VOCAB, "width": size["width"], "norm": {"eps": 1e-6},
                                    "layers": [layer] * layers, "loop": None})


def dense_twin_config(size: dict, layers: int):
    """The dense decoder of equal size: the same width, heads and key size, and a feed-forward as wide as the experts a
    token uses plus the shared one."""
    from llmserver_b200.config import Qwen3Config
    raw = dict(_qwen3(layers, size["width"], size["heads"], size["top"] * size["ff"] + size["shared_ff"]),
               num_key_value_heads=size["kv_heads"], head_dim=size["dim"], vocab_size=COMPARE_VOCAB)
    return Qwen3Config.from_dict(raw)


def gefarax_step_cost(size: dict, layers: int, tokens: int, cached_tokens: float, pairs: float):
    """(bytes, FLOPs) of one step of ``tokens`` new tokens: bytes = every weight the step touches once (of the routed
    experts the expected number of distinct ones its tokens choose) + ``cached_tokens`` keys and values;
    FLOPs = the products of its tokens + attention over ``pairs`` (query, key) pairs + logits of one row per sequence
    (left out: they are the same in both models)."""
    width, heads, kv_heads, dim, vdim = size["width"], size["heads"], size["kv_heads"], size["dim"], size["vdim"]
    experts, top, ff, shared_ff = size["experts"], size["top"], size["ff"], size["shared_ff"]
    attention_weights = (heads * dim + kv_heads * dim + kv_heads * vdim) * width + width * heads * vdim
    distinct = experts * (1.0 - (1.0 - top / experts) ** tokens)
    weight_bytes = 2 * layers * (attention_weights + 3 * width * (distinct * ff + shared_ff)) + 4 * layers * experts * width
    cache_bytes = 2 * layers * kv_heads * (dim + vdim) * cached_tokens
    linear = 2 * tokens * layers * (attention_weights + 3 * width * (top * ff + shared_ff) + experts * width)
    attention = 2 * layers * heads * (dim + vdim) * pairs
    return weight_bytes + cache_bytes + COMPARE_VOCAB * width * 2, linear + attention


def dense_step_cost(size: dict, layers: int, tokens: int, cached_tokens: float, pairs: float):
    width, heads, kv_heads, dim = size["width"], size["heads"], size["kv_heads"], size["dim"]
    inter = size["top"] * size["ff"] + size["shared_ff"]
    weights = (heads + 2 * kv_heads) * dim * width + width * heads * dim + 3 * width * inter
    return (2 * layers * weights + 2 * layers * kv_heads * 2 * dim * cached_tokens + COMPARE_VOCAB * width * 2,
            2 * tokens * layers * weights + 2 * layers * heads * 2 * dim * pairs)


# ---------------------------------------------------------------------------------------------------------------------
# Dikusun beside the dense decoder at equal size
# ---------------------------------------------------------------------------------------------------------------------
def _dikusun_size(width, ff, attention, latent, gla, kinds):
    return dict(width=width, ff=ff, attention=attention, latent=latent, gla=gla, kinds=kinds)


def _dikusun_mixers(width, heads, kv_heads):
    """Mixers of one width: differential attention whose two maps together are as wide as a dense head, a window of
    1024 tokens; latent attention with a latent of 128 (the widest head the tensor-core attention kernels take);
    gated linear attention with keys half and values as wide as the stream."""
    return (dict(heads=heads, kv_heads=kv_heads, dim=64, vdim=128, scale=0.125, diff=0.2, softcap=30.0, mask={"size": 1024},
                 rot={"base": 500000.0, "dims": 64}),
            dict(heads=16, dim=128, vdim=128, q_rank=width // 4, kv_rank=128, scale=128 ** -0.5),
            dict(heads=width // 128, dim=64, vdim=128, tau=8.0, a_rank=32))


# Layer sizes that resemble served models, each as four layers of one kind of mixer and as a mix of the three; every
# layer has a feed-forward three times as wide as the stream.
DIKUSUN_SIZES = {}
for _width, _heads, _kv in ((2048, 16, 4), (4096, 32, 8)):
    _a, _l, _g = _dikusun_mixers(_width, _heads, _kv)
    for _label, _kinds in (("attention", ("attention",) * 4), ("latent", ("latent_attention",) * 4), ("gla", ("gla",) * 4),
                           ("mixed", ("attention", "gla", "latent_attention", "attention"))):
        DIKUSUN_SIZES[f"w{_width}-{_label}"] = _dikusun_size(_width, 3 * _width, _a, _l, _g, _kinds)


def dikusun_config(size: dict, layers: int = None):
    from llmserver_b200.config import DikusunConfig
    mixer_of = {"attention": size["attention"], "latent_attention": size["latent"], "gla": size["gla"]}
    kinds = size["kinds"] if layers is None else [size["kinds"][index % len(size["kinds"])] for index in range(layers)]
    return DikusunConfig.from_dict({"architecture": "Dikusun", "vocab": COMPARE_VOCAB, "width": size["width"], "norm": {"eps": 1e-6},
                                    "embedding": {"scale": 1.0},
                                    "layers": [{"type": kind, "mixer": mixer_of[kind], "mlp": {"kind": "dense", "ff": size["ff"], "limit": 7.0}}
                                               for kind in kinds]})


def dikusun_dense_twin(size: dict, layers: int):
    """The dense decoder of equal size: the same width, the attention layers' head count with heads of 128, the same
    feed-forward."""
    from llmserver_b200.config import Qwen3Config
    raw = dict(_qwen3(layers, size["width"], size["attention"]["heads"], size["ff"]),
               num_key_value_heads=size["attention"]["kv_heads"], head_dim=128, vocab_size=COMPARE_VOCAB)
    return Qwen3Config.from_dict(raw)


def dikusun_step_cost(size: dict, layers: int, tokens: int, sequences: int, context: float):
    """(bytes, FLOPs) of one step in which each of ``sequences`` requests brings tokens / sequences new tokens behind
    ``context`` cached ones: bytes = every weight once + what the mixers read of cache and state; FLOPs = the products
    of the tokens + what the mixers do per (query, key) pair or per token of a recurrence."""
    width, ff = size["width"], size["ff"]
    per_sequence = tokens / sequences
    total_bytes = COMPARE_VOCAB * width * 2.0
    flops = 0.0
    kinds = [size["kinds"][index % len(size["kinds"])] for index in range(layers)]
    for kind in kinds:
        weights = 3.0 * width * ff
        if kind == "attention":
            m = size["attention"]
            heads, kv, dim, vdim, window = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["mask"]["size"]
            weights += (heads * 2 * dim + kv * 2 * dim + kv * vdim + heads) * width + width * heads * vdim
            seen = min(context + per_sequence, window)
            total_bytes += sequences * seen * kv * (2 * dim + vdim) * 2.0
            pairs = sequences * sum(min(context + i + 1, window) for i in range(int(per_sequence)))
            flops += 2.0 * heads * (2 * dim + 2 * vdim) * pairs
        elif kind == "latent_attention":
            m = size["latent"]
            heads, dim, vdim, q_rank, kv_rank = m["heads"], m["dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            weights += (q_rank + kv_rank) * width + heads * dim * (q_rank + kv_rank) + heads * vdim * kv_rank + width * heads * vdim
            total_bytes += sequences * (context + per_sequence) * kv_rank * 2.0
            pairs = sequences * (per_sequence * context + per_sequence * (per_sequence + 1) / 2)
            flops += 2.0 * heads * 2 * kv_rank * pairs
        else:
            m = size["gla"]
            heads, dim, vdim, rank = m["heads"], m["dim"], m["vdim"], m["a_rank"]
            weights += (2 * heads * dim + 2 * heads * vdim + rank) * width + heads * dim * rank + width * heads * vdim
            total_bytes += sequences * heads * dim * vdim * 4.0 * 2          # the state, read and written
            flops += tokens * heads * dim * vdim * 5.0
        total_bytes += 2.0 * weights
        flops += 2.0 * tokens * weights
    return total_bytes, flops


def dikusun_dense_cost(size: dict, layers: int, tokens: int, sequences: int, context: float):
    width, heads, kv, dim, inter = size["width"], size["attention"]["heads"], size["attention"]["kv_heads"], 128, size["ff"]
    weights = (heads + 2 * kv) * dim * width + width * heads * dim + 3 * width * inter
    per_sequence = tokens / sequences
    pairs = sequences * (per_sequence * context + per_sequence * (per_sequence + 1) / 2)
    return (2.0 * layers * weights + 2.0 * layers * kv * 2 * dim * sequences * (context + per_sequence) + COMPARE_VOCAB * width * 2.0,
            2.0 * tokens * layers * weights + 2.0 * layers * heads * 2 * dim * pairs)


# ---------------------------------------------------------------------------------------------------------------------
# Vibepel beside Dikusun (the closest design: the same block, windowed attention, a recurrence with a matrix state) and
# beside the dense decoder, at equal size
# ---------------------------------------------------------------------------------------------------------------------
def _vibepel_mixers(width, heads, kv_heads):
    """Mixers of one width: attention with heads of 128 over a window of 1024 tokens, half of each head rotating, beside a
    gated delta rule with half as many heads of 128 x 128; time mixing with heads of 64 channels across the stream."""
    left = dict(heads=heads, kv_heads=kv_heads, dim=128, vdim=128, scale=128 ** -0.5, mask={"size": 1024},
                rot={"base": 500000.0, "dims": 64, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 8192}})
    right = dict(heads=heads // 2, kv_heads=kv_heads, dim=128, vdim=128, conv=4)
    return (dict(left=left, right=right, left_scale=0.7, right_scale=0.4), dict(heads=width // 64, dim=64, w_rank=64))


# Layer sizes that resemble served models: four layers of one kind of mixer, or parallel, time mixing, parallel,
# parallel; every layer has a feed-forward three times as wide as the stream.
VIBEPEL_SIZES = {}
for _width, _heads, _kv in ((2048, 16, 4), (4096, 32, 8)):
    _p, _w = _vibepel_mixers(_width, _heads, _kv)
    for _label, _kinds in (("parallel", ("parallel",) * 4), ("wkv", ("wkv",) * 4), ("mixed", ("parallel", "wkv", "parallel", "parallel"))):
        VIBEPEL_SIZES[f"w{_width}-{_label}"] = dict(width=_width, ff=3 * _width, parallel=_p, wkv=_w, kinds=_kinds)


def vibepel_config(size: dict, layers: int = None):
    from llmserver_b200.config import VibepelConfig
    kinds = size["kinds"] if layers is None else [size["kinds"][index % len(size["kinds"])] for index in range(layers)]
    return VibepelConfig.from_dict({"architecture": "Vibepel", "vocab": COMPARE_VOCAB, "width": size["width"], "norm": {"eps": 1e-6},
                                    "embedding": {"scale": 8.0}, "logit_softcap": 30.0,
                                    "layers": [{"type": kind, "mixer": size[kind], "mlp": {"kind": "dense", "ff": size["ff"]}}
                                               for kind in kinds]})


def vibepel_dikusun_twin(size: dict, layers: int):
    """The Dikusun model of equal size: differential attention over the same window where Vibepel has a parallel layer,
    gated linear attention where it has time mixing, the same width and feed-forward width."""
    attention, _, gla = _dikusun_mixers(size["width"], size["parallel"]["left"]["heads"], size["parallel"]["left"]["kv_heads"])
    kinds = tuple("attention" if kind == "parallel" else "gla" for kind in size["kinds"])
    twin = _dikusun_size(size["width"], size["ff"], attention, None, gla, kinds)
    return twin, dikusun_config(twin, layers)


def vibepel_step_cost(size: dict, layers: int, tokens: int, sequences: int, context: float):
    """(bytes, FLOPs) of one step in which each of ``sequences`` requests brings tokens / sequences new tokens behind
    ``context`` cached ones: bytes = every weight once + what the mixers read of cache and state (states are read and
    written); FLOPs = the products of the tokens + attention per (query, key) pair + the recurrences' multiply-adds."""
    width, ff = size["width"], size["ff"]
    per_sequence = tokens / sequences
    total_bytes = COMPARE_VOCAB * width * 2.0
    flops = 0.0
    kinds = [size["kinds"][index % len(size["kinds"])] for index in range(layers)]
    for kind in kinds:
        weights = 2.0 * width * ff
        if kind == "parallel":
            left, right = size["parallel"]["left"], size["parallel"]["right"]
            heads, kv, dim, vdim, window = left["heads"], left["kv_heads"], left["dim"], left["vdim"], left["mask"]["size"]
            weights += (heads * dim + kv * dim + kv * vdim) * width + width * heads * vdim
            seen = min(context + per_sequence, window)
            total_bytes += sequences * seen * kv * (dim + vdim) * 2.0
            pairs = sequences * sum(min(context + i + 1, window) for i in range(int(per_sequence)))
            flops += 2.0 * heads * (dim + vdim) * pairs
            r_heads, r_kv, r_dim, r_vdim = right["heads"], right["kv_heads"], right["dim"], right["vdim"]
            weights += (2 * r_kv * r_dim + 2 * r_heads * r_vdim + 2 * r_heads) * width + width * r_heads * r_vdim
            total_bytes += sequences * r_heads * r_dim * r_vdim * 4.0 * 2
            flops += tokens * r_heads * r_dim * r_vdim * 8.0          # four multiply-adds per cell of the state
        else:
            m = size["wkv"]
            heads, dim, rank = m["heads"], m["dim"], m["w_rank"]
            weights += 5 * heads * dim * width + rank * width + heads * dim * rank
            total_bytes += sequences * heads * dim * dim * 4.0 * 2
            flops += tokens * heads * dim * dim * 6.0                 # three multiply-adds per cell of the state
        total_bytes += 2.0 * weights
        flops += 2.0 * tokens * weights
    return total_bytes, flops


# ---------------------------------------------------------------------------------------------------------------------
# Zeridra beside Gefarax (the closest design: grouped attention with a term of its own in the denominator, routed gated
# experts under a sigmoid router) at equal size
# ---------------------------------------------------------------------------------------------------------------------
def _zeridra_mixers(width, heads, kv_heads):
    """Mixers of one width: attention with heads of 128 whose keys are its values, warmed-up queries; latent attention
    with 16 heads of 64 still and 32 turning elements through a query latent of a quarter of the width and a cached row
    of 96 + 32 (the widest the tensor-core attention kernels take), values of 128, a window of 1024."""
    return (dict(heads=heads, kv_heads=kv_heads, dim=128, vdim=128, scale=128 ** -0.5, q_temp={"coef": 0.1, "every": 1024}),
            dict(heads=16, dim=64, rot_dim=32, vdim=128, q_rank=width // 4, kv_rank=96, scale=96 ** -0.5, mask={"size": 1024},
                 rot={"base": 500000.0, "dims": 32}))


# Layer sizes that resemble served models: four layers of one kind of mixer, or attention, latent, attention and a latent
# layer that reads the second layer's cache; every layer has routed experts (the sizes of Gefarax's comparison).
ZERIDRA_SIZES = {}
for _width, _heads, _kv, _experts, _top, _ff in ((2048, 16, 4, 32, 4, 768), (4096, 32, 8, 64, 6, 1792)):
    _a, _l = _zeridra_mixers(_width, _heads, _kv)
    for _label, _kinds in (("attention", ("attention",) * 4), ("latent", ("latent_attention",) * 4),
                           ("mixed", ("attention", "latent_attention", "attention", "shared_latent"))):
        ZERIDRA_SIZES[f"w{_width}-{_label}"] = dict(width=_width, attention=_a, latent=_l, experts=_experts, top=_top, ff=_ff, kinds=_kinds)


def _zeridra_kinds(size: dict, layers: int):
    return [size["kinds"][index % len(size["kinds"])] for index in range(layers)]


def zeridra_config(size: dict, layers: int = None):
    from llmserver_b200.config import ZeridraConfig
    kinds = _zeridra_kinds(size, layers or len(size["kinds"]))
    made, owner = [], None
    for index, kind in enumerate(kinds):
        if kind == "attention":
            mixer = dict(size["attention"])
        else:
            mixer = dict(size["latent"])
            if kind == "shared_latent" and owner is not None:
                mixer["kv_from"] = owner
            else:
                owner = index
        made.append({"type": "attention" if kind == "attention" else "latent_attention", "mixer": mixer,
                     "mlp": {"kind": "moe", "router": {"experts": size["experts"], "top": size["top"]}, "expert": {"ff": size["ff"]}}})
    return ZeridraConfig.from_dict({"architecture": "Zeridra", "vocab": COMPARE_VOCAB, "width": size["width"], "norm": {"eps": 1e-6},
                                    "embedding": {"scale": size["width"] ** 0.5}, "logit_scale": 0.5, "logit_softcap": 50.0,
                                    "layers": made})


def zeridra_gefarax_twin(size: dict, layers: int):
    """The Gefarax model of equal size: the same width, the attention layers' heads (keys and values of 128, all of a key
    rotating), the same experts, no shared expert."""
    a = size["attention"]
    twin = _gefarax_size(size["width"], a["heads"], a["kv_heads"], a["dim"], a["vdim"], size["experts"], size["top"], size["ff"], 0)
    raw = gefarax_config(dict(twin, shared_ff=8), layers).to_dict()
    for layer in raw["layers"]:
        layer["mlp"]["shared"] = None
    from llmserver_b200.config import GefaraxConfig
    return twin, GefaraxConfig.from_dict(raw)


def zeridra_twin_cost(size: dict, layers: int, tokens: int, sequences: int, context: float):
    per_sequence = tokens / sequences
    pairs = sequences * (per_sequence * context + per_sequence * (per_sequence + 1) / 2)
    return gefarax_step_cost(size, layers, tokens, sequences * (context + per_sequence), pairs)


def zeridra_step_cost(size: dict, layers: int, tokens: int, sequences: int, context: float):
    """(bytes, FLOPs) of one step in which each of ``sequences`` requests brings tokens / sequences new tokens behind
    ``context`` cached ones: bytes = every weight the step touches once (of the routed experts the expected number of
    distinct ones its tokens choose) + the cached rows its mixers read (a key that is its own value counts once);
    FLOPs = the products of the tokens + attention per (query, key) pair as the design defines it (latent layers: keys of
    dim + rot_dim and values of vdim per head)."""
    width, experts, top, ff = size["width"], size["experts"], size["top"], size["ff"]
    per_sequence = tokens / sequences
    total_bytes = COMPARE_VOCAB * width * 2.0
    flops = 0.0
    distinct = experts * (1.0 - (1.0 - top / experts) ** tokens)
    for kind in _zeridra_kinds(size, layers):
        total_bytes += 2.0 * 3 * width * distinct * ff + 4.0 * experts * width
        flops += 2.0 * tokens * (3 * width * top * ff + experts * width)
        if kind == "attention":
            m = size["attention"]
            heads, kv, dim = m["heads"], m["kv_heads"], m["dim"]
            weights = (heads + kv) * dim * width + width * heads * dim
            total_bytes += sequences * (context + per_sequence) * kv * dim * 2.0
            pairs = sequences * (per_sequence * context + per_sequence * (per_sequence + 1) / 2)
            flops += 2.0 * heads * 2 * dim * pairs
        else:
            m = size["latent"]
            heads, dim, rot, vdim, q_rank, kv_rank, window = (m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"],
                                                             m["mask"]["size"])
            weights = q_rank * width + heads * (dim + rot) * q_rank + heads * dim * kv_rank + heads * vdim * kv_rank + width * heads * vdim
            if kind != "shared_latent":
                weights += (kv_rank + rot) * width
            total_bytes += sequences * min(context + per_sequence, window) * (kv_rank + rot) * 2.0
            pairs = sequences * sum(min(context + i + 1, window) for i in range(int(per_sequence)))
            flops += 2.0 * heads * (dim + rot + vdim) * pairs
        total_bytes += 2.0 * weights
        flops += 2.0 * tokens * weights
    return total_bytes, flops
