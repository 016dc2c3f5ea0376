"""Throughput measurement: decode tokens per second and prefill tokens per second.

The workload is the reference's headline one scaled to this engine: a Qwen3-8B-shaped
model with seeded random bfloat16 weights, prompts of uniform random token ids, decode
from 2,048-token contexts.  The reference's own ``leone bench`` measures batch 1 only,
prompt ``[1; P]``, one warm-up run then repetitions (crates/leone-cli/src/main.rs:2098-2157),
and relates the decode rate to memory bandwidth (crates/leone-cli/src/main.rs:4762).  Rates
are defined as there: decode rate = decoded tokens / decode time including reading the
sampled ids back (crates/leone/src/runtime.rs:419-427).

Timing: CUDA events on the launching stream around exactly ``steps`` decode steps, after
``warmup`` untimed steps.  Every decode step reads all weights (≈15 GB), far more than the
126 MB L2, so consecutive timed steps cannot serve each other from cache.
"""
from __future__ import annotations

import json
import os
import statistics
import subprocess
import threading
import time
from typing import Dict, List, Optional

import torch

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=36, hidden_size=4096,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6,
                max_position_embeddings=40960, tie_word_embeddings=False)   # positions as the checkpoints' config.json has them

QWEN3_1_7B = dict(QWEN3_8B, num_hidden_layers=28, hidden_size=2048, num_attention_heads=16,
                  intermediate_size=6144, tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64,
                 intermediate_size=25600)
# name -> (config, decode context, batch sizes measured beside the headline batch)
SHAPES = {"qwen3-8b": (QWEN3_8B, 2048, (1, 64)), "qwen3-1.7b": (QWEN3_1_7B, 2048, (1, 64)),
          "qwen3-32b": (QWEN3_32B, 8192, (1, 32))}

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def measured_peaks() -> Dict[str, float]:
    """Measured copy bandwidth and bf16 GEMM rate of this pool's GPUs, if the file is there."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as fh:
            raw = json.load(fh)
        return dict(hbm_gbs=float(raw["hbm_gbs"]), bf16_tflops=float(raw["bf16_tflops"]),
                    bf16_tflops_sustained=float(raw.get("bf16_tflops_sustained", raw["bf16_tflops"])),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines: List[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                max_clock = float(parts[1])
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks)}


def _random_prompts(vocab: int, batch: int, length: int, seed: int) -> List[List[int]]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (batch, length), generator=gen).tolist()


def prefill_all(engine, rids, prompts, chunk: int) -> List[int]:
    """Run the prompts through the step function in portions; returns each request's first
    sampled token (greedy)."""
    from .sampling.sampler import SamplingParams
    firsts = []
    for rid, prompt in zip(rids, prompts):
        pos = 0
        logits = None
        while pos < len(prompt):
            n = min(chunk, len(prompt) - pos)
            last = pos + n == len(prompt)
            logits = engine.step([(rid, prompt[pos:pos + n], [n - 1] if last else [])])
            pos += n
        firsts.append(engine.sample(logits, [SamplingParams()], [len(prompt) - 1])[0])
    return firsts


def time_decode(engine, batch: int, context: int, steps: int, warmup: int, seed: int = 0, reps: int = 5):
    """Device-timed decode through ``Engine.decode_steps``: ``reps`` runs of exactly ``steps``
    decode steps each (captured steps replayed in quanta of up to 64 with the sampled ids fed
    back on the device, and read back once per quantum), CUDA events around each run; the
    median run is reported."""
    from .sampling.sampler import SamplingParams
    vocab = engine.spec.vocab_size
    rids = [f"bench{batch}_{i}" for i in range(batch)]
    prompts = _random_prompts(vocab, batch, context, seed + batch)
    firsts = prefill_all(engine, rids, prompts, engine.max_batch_tokens)
    params = [SamplingParams() for _ in rids]
    last = firsts
    last = engine.decode_steps(rids, last, params, max(warmup, 1))[-1]
    times = []
    mid = []
    for _ in range(reps):
        # every run starts from the same context length: the tokens of the run before are dropped
        engine.drop_lookahead()
        for r in rids:
            engine.cache.truncate(r, context + max(warmup, 1))
        mid.append(engine.cache.length(rids[0]) + steps / 2.0)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        done, feed = 0, last
        while done < steps:
            q = min(64, steps - done)
            feed = engine.decode_steps(rids, feed, params, q)[-1]
            done += q
        stop.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(stop))
    ms = statistics.median(times)
    graph = engine._decode_graphs[batch]
    for r in rids:
        engine.close(r)
    return dict(ms_per_step=ms / steps, tokens_per_s=batch * steps / (ms / 1e3), mid_context=mid[0],
                launches=graph.launches_per_step * steps, runs_ms=[round(t, 3) for t in times])


def time_prefill(engine, tokens: int, reps: int = 5, seed: int = 99):
    """Median device time of one prompt of ``tokens`` tokens.  The repetitions are a quarter of
    a second apart: back to back they run into the power cap and measure the sustained rate,
    while the peak they are divided by is a burst figure (both fractions are reported)."""
    vocab = engine.spec.vocab_size
    times = []
    for rep in range(reps + 1):
        prompt = _random_prompts(vocab, 1, tokens, seed + rep)[0]
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        pos = 0
        while pos < tokens:
            n = min(engine.max_batch_tokens, tokens - pos)
            engine.step([("prefill_bench", prompt[pos:pos + n], [n - 1] if pos + n == tokens else [])],
                        check=False)
            pos += n
        stop.record()
        torch.cuda.synchronize()
        engine.check_status()
        engine.close("prefill_bench")
        time.sleep(0.25)
        if rep > 0:                      # the first run is the warm-up
            times.append(start.elapsed_time(stop))
    return statistics.median(times)


def model_flops_prefill(cfg: dict, layers: int, tokens: int) -> float:
    h, d = cfg["hidden_size"], cfg["head_dim"]
    n_q, n_kv, inter = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["intermediate_size"]
    linear = 2.0 * tokens * (h * (n_q + 2 * n_kv) * d + n_q * d * h + 3 * h * inter)
    attention = 2.0 * n_q * d * tokens * tokens          # causal half of 4 n_q d T^2
    return layers * (linear + attention) + 2.0 * cfg["vocab_size"] * h


def kv_bytes_per_token(cfg: dict, layers: int, itemsize: int = 2) -> int:
    return 2 * layers * cfg["num_key_value_heads"] * cfg["head_dim"] * itemsize


def serving(shape: str = "qwen3-1.7b", requests: int = 64, min_prompt: int = 64, max_prompt: int = 2048,
            new_tokens: int = 128, max_batch_tokens: int = 2048, prefill_chunk: int = 1024,
            layers: Optional[int] = None, seed: int = 0) -> int:
    """Continuous batching through the scheduler: ``requests`` requests arrive at once with prompt
    lengths uniform in [min_prompt, max_prompt]; prompt portions run beside the decode tokens of
    the requests already past their prompt; each generates ``new_tokens``.  The workload runs
    twice (the first run builds the decode graphs) and the second is reported: generated tokens
    per second of wall clock, time to first token per request, and where the steps' time went."""
    from .config.qwen3 import Qwen3Config
    from .engine.engine import Engine
    from .engine.scheduler import Scheduler, SchedulerConfig
    from .sampling.sampler import SamplingParams
    cfg = dict(SHAPES[shape][0])
    full_layers = cfg["num_hidden_layers"]
    if layers:
        cfg["num_hidden_layers"] = layers
    config = Qwen3Config.from_dict(cfg)
    gen = torch.Generator().manual_seed(seed)
    lengths = torch.randint(min_prompt, max_prompt + 1, (requests,), generator=gen).tolist()
    prompts = [torch.randint(0, config.vocab_size, (n,), generator=gen).tolist() for n in lengths]
    pool_tokens = sum(-(-(n + new_tokens) // 64) * 64 for n in lengths)
    engine = Engine.from_config(config, seed=0, dtype="bfloat16", page_tokens=16, max_tokens=pool_tokens,
                                max_requests=requests, max_batch_tokens=max_batch_tokens)
    report = None
    for rep in range(2):
        sched = Scheduler(engine, SchedulerConfig(max_running=requests, max_batch_tokens=max_batch_tokens,
                                                  prefill_chunk_tokens=prefill_chunk, prefill_first=False))
        for i, p in enumerate(prompts):
            sched.add_request(i, p, new_tokens, SamplingParams(0.0, seed + i), -1)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        first: Dict[int, float] = {}
        kinds = {"mixed": [], "decode": []}
        while sched.has_work():
            before_prefill = sched.stats["prefill_tokens"]
            t = time.perf_counter()
            outs = sched.step()
            now = time.perf_counter()
            kinds["mixed" if sched.stats["prefill_tokens"] > before_prefill else "decode"].append(now - t)
            for o in outs:
                first.setdefault(o.rid, now - t0)
        wall = time.perf_counter() - t0
        generated = sum(len(sched.requests[i].generated) for i in range(requests))
        ttft = sorted(first.values())
        report = {
            "metric": "generated tokens/s, continuous batching of chunked prefill with decode",
            "value": generated / wall, "unit": "tokens/s", "wall_s": wall,
            "prompt_tokens": sum(lengths), "generated_tokens": generated,
            "all_tokens_per_s": (sum(lengths) + generated) / wall,
            "ttft_s": {"p50": ttft[len(ttft) // 2], "p90": ttft[int(len(ttft) * 0.9)], "max": ttft[-1]},
            "steps": {k: {"count": len(v), "total_s": sum(v), "mean_ms": 1e3 * sum(v) / max(len(v), 1)}
                      for k, v in kinds.items()},
            "config": {"model": shape, "layers": cfg["num_hidden_layers"], "layers_of_model": full_layers,
                       "requests": requests, "prompt_lengths": f"uniform {min_prompt}-{max_prompt}",
                       "new_tokens": new_tokens, "max_batch_tokens": max_batch_tokens,
                       "prefill_chunk": prefill_chunk, "page_tokens": 16},
            "dtype": "bf16", "data": "synthetic: uniform random token ids, seeded random weights N(0,0.02)",
        }
    print(json.dumps(report))
    return 0


def run(gpus: int, steps: int, warmup: int, impl: str, layers: Optional[int] = None, batch: int = 8,
        context: Optional[int] = None, prefill_tokens: int = 2048, points: bool = True,
        shape: str = "qwen3-8b") -> int:
    if impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace (maturin bin wheel); no cargo/rustc in this "
                          "image and its CUDA kernels target sm_89 GGUF Q4_K only"}))
        return 0
    if gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {gpus} is not supported")
        return 2
    from .config.qwen3 import Qwen3Config
    from .engine.engine import Engine
    from .engine.generate import generate

    cfg, shape_context, other_batches = SHAPES[shape]
    cfg = dict(cfg)
    context = context or shape_context
    full_layers = cfg["num_hidden_layers"]
    if layers:
        cfg["num_hidden_layers"] = layers
    layers = cfg["num_hidden_layers"]
    config = Qwen3Config.from_dict(cfg)
    peaks = measured_peaks()
    page_tokens = 16
    big = max(other_batches + (batch,)) if points else batch
    pool_tokens = big * (context + steps + warmup + 128)
    t_build = time.time()
    engine = Engine.from_config(config, seed=0, dtype="bfloat16", page_tokens=page_tokens,
                                max_tokens=pool_tokens, max_requests=max(big, batch),
                                max_batch_tokens=max(prefill_tokens, 2048))
    build_s = time.time() - t_build

    # prefill
    prefill_ms = time_prefill(engine, prefill_tokens)
    flops = model_flops_prefill(cfg, layers, prefill_tokens)
    prefill = {"value": prefill_tokens / (prefill_ms / 1e3), "tokens": prefill_tokens, "ms": prefill_ms,
               "frac": flops / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12),
               "tflops": flops / (prefill_ms / 1e3) / 1e12, "peak_tflops": peaks["bf16_tflops"],
               "frac_of_sustained": flops / (prefill_ms / 1e3) / (peaks["bf16_tflops_sustained"] * 1e12)}

    # the headline decode batch, with clocks sampled during the timed region
    sampler = ClockSampler()
    sampler.start()
    main = time_decode(engine, batch, context, steps, warmup)
    clocks = sampler.stop()
    weight_bytes = engine.model.decode_weight_bytes()
    step_bytes = weight_bytes + batch * main["mid_context"] * kv_bytes_per_token(cfg, layers)
    achieved = step_bytes / (main["ms_per_step"] / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "peaks": peaks["source"]}

    extra = {}
    if points:
        for b in other_batches:
            r = time_decode(engine, b, context, steps, warmup)
            extra[f"decode_b{b}"] = r["tokens_per_s"]

    # end to end through the Python entry point: host token ids in, host token ids out
    prompts = _random_prompts(config.vocab_size, batch, context, 4242)
    new_tokens = steps + 1
    generate(engine, _random_prompts(config.vocab_size, batch, 64, 17), 4, eos_token_id=-1,
             max_running=batch)                      # warm-up of the entry point itself
    torch.cuda.synchronize()
    results, stats = generate(engine, prompts, new_tokens, temperature=0.0, return_stats=True,
                              eos_token_id=-1, prefill_chunk=engine.max_batch_tokens,
                              max_batch_tokens=engine.max_batch_tokens, max_running=batch)
    graph = engine._decode_graphs[batch]
    e2e = {"value": stats.decode_tokens_per_second, "unit": "tokens/s",
           # a step launched ahead gets the host's positions and lengths (2 x 4 bytes a request) and
           # new block-table entries; the first step of a run gets the whole metadata buffer
           "h2d_bytes_per_step": int(8 * batch + 4) if engine.lookahead else
           int(graph.size * 4 + batch * 64),
           "d2h_bytes_per_step": int(batch * 4 + 16),
           "prefill_tokens_per_s": stats.prefill_tokens_per_second}

    line = {
        "metric": f"decode tok/s at batch {batch} ({shape} bf16, {context}-token contexts); prefill and batch "
                  f"{'/'.join(map(str, other_batches))} alongside",
        "value": main["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: uniform random token ids, seeded random weights N(0,0.02)",
        "config": {"model": {"qwen3-8b": "Qwen3-8B shape"}.get(shape, shape + " shape"), "layers": layers, "layers_of_model": full_layers,
                   "hidden_size": cfg["hidden_size"], "num_heads": cfg["num_attention_heads"],
                   "num_kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate_size": cfg["intermediate_size"], "vocab_size": cfg["vocab_size"],
                   "tied_head": bool(cfg["tie_word_embeddings"]), "global_batch": batch, "seq_len": context,
                   "max_context": cfg["max_position_embeddings"], "page_tokens": page_tokens,
                   "prefill_tokens": prefill_tokens, "parallelism": "1 gpu",
                   "cache_between_steps": "each step reads all weights (GBs), far beyond the 126 MB L2",
                   "decode": "Engine.decode_steps: captured step replayed, sampled ids fed back on device, "
                             "read back per quantum of 64; median of 5 runs of `steps` steps"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": main["launches"], "prefill": prefill,
        "roofline": roofline, "points": extra, "impl": "leone_b200", "build_seconds": round(build_s, 1),
    }
    print(json.dumps(line))
    return 0
