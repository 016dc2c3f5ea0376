"""The Python entry point: token ids in, token ids out.

The reference has no Python API (README.md:61-62); its entry point is
``leone generate -m <model> -p <prompt> -n <tokens>`` (crates/leone-cli/src/main.rs:1073-1233)
with ``--temp`` and ``--seed`` (crates/leone-cli/src/main.rs:418-446).  The same names and
meanings are used here; prompts are token ids because no tokenizer is built.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Optional, Sequence, Union

from ..sampling.sampler import SamplingParams
from .engine import Engine
from .scheduler import Scheduler, SchedulerConfig


@dataclass
class GenerationStats:
    """Rates as the reference defines them (crates/leone/src/runtime.rs:419-427): prefill rate =
    prompt tokens / time to the first token; decode rate = (emitted - 1) / decode time."""
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    steps: int = 0
    preemptions: int = 0

    @property
    def prefill_tokens_per_second(self) -> float:
        return self.prompt_tokens / self.prefill_seconds if self.prefill_seconds > 0 else 0.0

    first_tokens: int = 0

    @property
    def decode_tokens_per_second(self) -> float:
        n = self.generated_tokens - self.first_tokens
        return n / self.decode_seconds if self.decode_seconds > 0 else 0.0


def load_config(source):
    """A typed configuration from a model folder, a ``config.json`` path, a dict or itself."""
    import json
    import os
    from ..config.base import ModelConfig
    from ..registry import config_from_dict, config_from_folder
    if isinstance(source, ModelConfig):
        return source
    if isinstance(source, dict):
        return config_from_dict(source)
    if isinstance(source, str) and os.path.isfile(source):
        with open(source) as fh:
            return config_from_dict(json.load(fh))
    return config_from_folder(source)


def generate(model: Union[str, Engine], prompts: Sequence[Sequence[int]], max_new_tokens: int,
             temperature: float = 0.0, seed: int = 0, dtype: str = "bfloat16",
             eos_token_id=None, page_tokens: int = 16,
             num_pages: Optional[int] = None, prefill_chunk: int = 2048,
             max_batch_tokens: int = 2048, max_running: int = 64, policy: str = "reserve",
             device: str = "cuda:0", return_stats: bool = False, decode_quantum: int = 1,
             use_graphs: bool = True, prefill_first: bool = True, truncations=(), penalties=None, mirostat=None,
             random_weights: bool = False, weights_seed: Optional[int] = None):
    """Generate ``max_new_tokens`` tokens for each prompt (a list of token ids).

    ``model`` is a model folder (config.json + model.safetensors) or an :class:`Engine`.
    With ``random_weights`` no tensor file is read: ``model`` is a folder with a ``config.json``,
    the path of such a file, its contents as a dict, or a typed configuration, and the weights
    are drawn on the device from ``weights_seed`` (default: ``seed``) as
    ``leone_b200.weights.random_init`` defines them, the same values as a folder written by
    ``write_random_model`` for that configuration and seed holds.
    ``temperature`` 0 is greedy; otherwise each request ``i`` draws with seed ``seed + i`` so
    its stream does not depend on what it is batched with.  ``prefill_first`` (default) runs
    all prompts before decoding starts, so the requests decode as one batch; ``False`` mixes
    prompt portions with decode tokens of earlier requests, as a server would.  Returns the
    generated ids per prompt (and a :class:`GenerationStats` if ``return_stats``).
    ``truncations``: ``(stage, value)`` pairs applied in order after the temperature (top_k,
    top_p, min_p, top_a, tfs, typical, epsilon, eta, min_k, top_n_sigma: the reference's
    ``--top-k`` .. ``--top-n-sigma``, crates/leone-cli/src/main.rs:836-845); such requests' decode
    steps run from the captured graph one at a time and are sampled outside it.  ``penalties``: a
    :class:`leone_b200.sampling.sampler.Penalties` applied to the logits from each request's own
    history before sampling (greedy included).  ``mirostat``: ``(target surprise, learning rate)``
    for Mirostat v2, which keeps a maximum surprise per request.
    """
    prompts = [list(map(int, p)) for p in prompts]
    if isinstance(model, Engine):
        engine = model
    else:
        longest = max((len(p) for p in prompts), default=0) + max_new_tokens
        if num_pages is None:
            per_request = -(-longest // page_tokens) + 1
            num_pages = per_request * min(len(prompts), max_running)
        kw = dict(dtype=dtype, device=device, page_tokens=page_tokens, num_pages=num_pages,
                  max_requests=max_running, max_batch_tokens=max_batch_tokens)
        if random_weights:
            engine = Engine.from_config(load_config(model), seed if weights_seed is None else weights_seed, **kw)
        else:
            engine = Engine.from_folder(model, **kw)
    if eos_token_id is None:
        eos_token_id = engine.spec.stop_ids() or None
    sched = Scheduler(engine, SchedulerConfig(max_running=min(max_running, engine.max_requests),
                                              max_batch_tokens=min(max_batch_tokens, engine.max_batch_tokens),
                                              prefill_chunk_tokens=prefill_chunk, policy=policy,
                                              decode_quantum=decode_quantum, use_graphs=use_graphs,
                                              prefill_first=prefill_first))
    for i, p in enumerate(prompts):
        sched.add_request(i, p, max_new_tokens, SamplingParams(temperature, seed + i, tuple(truncations), penalties, mirostat),
                          eos_token_id)
    stats = GenerationStats(prompt_tokens=sum(len(p) for p in prompts))
    t0 = time.perf_counter()
    first_done = None
    seen_first = set()
    while sched.has_work():
        outs = sched.step()
        for o in outs:
            seen_first.add(o.rid)
        if first_done is None and len(seen_first) == len(prompts):
            first_done = time.perf_counter()
    t1 = time.perf_counter()
    results = [sched.requests[i].generated for i in range(len(prompts))]
    if return_stats:
        stats.generated_tokens = sum(len(r) for r in results)
        stats.first_tokens = len(prompts)
        stats.prefill_seconds = (first_done or t1) - t0
        stats.decode_seconds = t1 - (first_done or t1)
        stats.steps = sched.stats["steps"]
        stats.preemptions = sched.stats["preemptions"]
        return results, stats
    return results
