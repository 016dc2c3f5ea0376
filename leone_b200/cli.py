"""The ``leone`` command line: ``generate``, ``doctor``, ``replay``, ``bench``, ``random-model``.

Option names and meanings follow the reference's CLI where it has them
(crates/leone-cli/src/main.rs:418-446 and 1073-1233): ``generate -m <model> -n <tokens>``
with ``--temp``, ``--seed``, ``--eager-decode``, ``--kv``, ``--debug-tokens``,
``--debug-logits``; ``doctor [-m <model>] [--probe]`` (crates/leone-cli/src/doctor.rs:32-132).
The model is a folder (``config.json`` + ``model.safetensors``) instead of a GGUF file, and
because no tokenizer is built, prompts are token ids (``-t``); ``-p`` text is refused with a
message that says so.
"""
from __future__ import annotations

import argparse
import json
import os
import struct
import sys
import time
from typing import List, Optional


def parse_token_ids(text: str) -> List[int]:
    """``"1,2,3"`` or ``@file`` (little-endian u32 ids, the reference's ``eval --tokens``
    format, crates/leone-cli/src/token_io.rs:5-17; a ``.json`` file holds a JSON list)."""
    if text.startswith("@"):
        path = text[1:]
        if path.endswith(".json"):
            with open(path) as fh:
                return [int(t) for t in json.load(fh)]
        with open(path, "rb") as fh:
            raw = fh.read()
        if len(raw) % 4:
            raise ValueError(f"{path}: length is not a multiple of 4 bytes")
        return list(struct.unpack(f"<{len(raw) // 4}I", raw))
    return [int(t) for t in text.replace(" ", ",").split(",") if t != ""]


def cmd_generate(args) -> int:
    if args.prompt is not None:
        print("leone generate: -p/--prompt needs a tokenizer, which this engine does not have; "
              "give token ids with -t/--prompt-tokens (\"1,2,3\" or @file)", file=sys.stderr)
        return 2
    if not args.prompt_tokens:
        print("generate requires -t <token ids>", file=sys.stderr)
        return 2
    if args.kv is not None:
        want = {"bfloat16": "bf16", "float32": "f32"}[args.dtype]
        if args.kv != want:
            print(f"leone generate: --kv {args.kv} is not available; the cache is stored in the run "
                  f"dtype ({want}); quantized and f16 caches are not built", file=sys.stderr)
            return 2
    from .engine.engine import Engine
    from .engine.generate import generate
    from .sampling.sampler import Penalties
    penalties = Penalties(args.repeat_penalty, args.presence_penalty, args.frequency_penalty, args.penalty_window,
                          args.dry_multiplier, args.dry_base, args.dry_allowed_length, args.dry_window)
    prompts = [parse_token_ids(t) for t in args.prompt_tokens]
    longest = max(len(p) for p in prompts) + args.tokens
    pages = args.num_pages or (-(-longest // args.page_tokens) + 1) * len(prompts)
    kw = dict(dtype=args.dtype, page_tokens=args.page_tokens, num_pages=pages, max_requests=max(len(prompts), 1),
              max_batch_tokens=args.max_batch_tokens)
    if args.random_weights:
        from .engine.generate import load_config
        engine = Engine.from_config(load_config(args.model),
                                    args.seed if args.weights_seed is None else args.weights_seed, **kw)
    else:
        engine = Engine.from_folder(args.model, **kw)
    debug_rows = []
    if args.debug_logits:
        _wrap_sampling_for_debug(engine, debug_rows)
    out, stats = generate(engine, prompts, args.tokens, temperature=args.temp or 0.0, seed=args.seed,
                          eos_token_id=args.eos, prefill_chunk=args.prefill_chunk,
                          max_batch_tokens=args.max_batch_tokens, return_stats=True,
                          use_graphs=not args.eager_decode and not args.debug_logits,
                          decode_quantum=args.decode_quantum, truncations=tuple(args.truncations or ()),
                          penalties=penalties if penalties.active else None)
    for toks in out:
        print(",".join(str(t) for t in toks))
    if args.debug_tokens:
        with open(args.debug_tokens, "w") as fh:
            json.dump(out if len(out) > 1 else out[0], fh)
    if args.debug_logits:
        with open(args.debug_logits, "w") as fh:
            json.dump(debug_rows, fh, indent=1)
    print(f"prefill: {stats.prompt_tokens} tokens, {stats.prefill_tokens_per_second:.1f} tok/s; "
          f"decode: {stats.generated_tokens} tokens, {stats.decode_tokens_per_second:.1f} tok/s; "
          f"{stats.steps} steps", file=sys.stderr)
    return 0


def _wrap_sampling_for_debug(engine, rows) -> None:
    """Record the top five logits of every sampled row, with their float bits, as the
    reference's ``--debug-logits`` does (crates/leone-cli/src/main.rs:2997-3022)."""
    import torch
    inner = engine.sample

    def sample(logits, params, positions, **kw):
        top = torch.topk(logits.float(), k=min(5, logits.shape[1]), dim=1)
        for r in range(logits.shape[0]):
            rows.append({"position": int(positions[r]), "top": [
                {"token": int(i), "logit": float(v),
                 "bits": f"{struct.unpack('<I', struct.pack('<f', float(v)))[0]:08x}"}
                for v, i in zip(top.values[r].tolist(), top.indices[r].tolist())]})
        return inner(logits, params, positions, **kw)

    engine.sample = sample


def cmd_doctor(args) -> int:
    import platform
    print(f"platform: {platform.system()} {platform.machine()}, python {platform.python_version()}")
    try:
        import torch
        print(f"torch: {torch.__version__}, cuda runtime {torch.version.cuda}")
        if torch.cuda.is_available():
            props = torch.cuda.get_device_properties(0)
            free, total = torch.cuda.mem_get_info(0)
            print(f"gpu 0: {props.name}, sm_{props.major}{props.minor}, {props.multi_processor_count} SMs, "
                  f"{free / 2**30:.1f} of {total / 2**30:.1f} GiB free")
            ok = props.major == 10
            print("backend cuda (sm_100a): " + ("ready" if ok else "not usable: kernels are built for sm_100a"))
        else:
            ok = False
            print("backend cuda (sm_100a): no CUDA device visible")
    except Exception as err:  # a broken install is a finding, not a crash
        ok = False
        print(f"torch: unavailable ({err})")
    from .csrc.build import find_nvcc, BuildError
    try:
        print(f"nvcc: {find_nvcc()}")
    except BuildError as err:
        print(f"nvcc: {err}")
    if args.model:
        from .config.base import ConfigError
        from .engine.model import Model
        from .parts.base import Runtime
        from .registry import ARCHITECTURES, config_from_folder, spec_from_config
        from .weights.loader import WeightError, check_names_and_shapes
        from .weights.safetensors import Checkpoint, SafetensorsError
        import torch
        try:
            config = config_from_folder(args.model)
        except ConfigError as err:
            print(f"model metadata: {err}")
            print(f"known architectures: {', '.join(ARCHITECTURES.names())}")
            return 1
        print(f"architecture: {config.architecture}")
        for key, value in config.to_json_dict().items():
            if key != "architectures":
                print(f"  {key}: {value}")
        print(f"context limit: {config.max_position_embeddings} tokens")
        spec = spec_from_config(config)
        model = Model(spec, Runtime("cpu", torch.float32, None, 0))
        try:
            ckpt = Checkpoint(args.model)
            check_names_and_shapes(model.weight_specs(), ckpt.entries, model.load_notes(set(ckpt.names())))
            total = sum(e.nbytes for e in ckpt.entries.values())
            print(f"checkpoint: {len(ckpt.entries)} tensors, {total / 2**20:.1f} MiB, names and shapes match")
            ckpt.close()
        except (WeightError, SafetensorsError) as err:
            print(str(err))
            return 1
        print("model metadata: ready")
        if args.probe:
            if not ok:
                print("probe: skipped, no usable GPU")
                return 1
            from .engine.engine import Engine
            t0 = time.time()
            engine = Engine.from_folder(args.model, dtype=args.dtype, max_tokens=64, max_requests=1,
                                        max_batch_tokens=16)
            logits = engine.step([("probe", [0], [0])])
            engine.close("probe")
            print(f"probe: loaded and ran one token in {time.time() - t0:.1f} s, "
                  f"logits finite: {bool(logits.isfinite().all())}")
    return 0


def cmd_random_model(args) -> int:
    import torch
    from .registry import config_from_dict
    from .weights.random_init import write_random_model
    with open(args.config) as fh:
        config = config_from_dict(json.load(fh))
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[args.store_dtype]
    write_random_model(config, args.out, args.seed, dtype)
    print(f"wrote {args.out}/config.json and model.safetensors (seed {args.seed}, {args.store_dtype})")
    return 0


def cmd_replay(args, rest) -> int:
    import runpy
    script = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "trace_run")
    sys.argv = [script] + rest
    runpy.run_path(script, run_name="__main__")
    return 0


def cmd_bench(args) -> int:
    from .benchmark import run, serving
    if args.workload == "serving":
        return serving(args.shape or "qwen3-1.7b", requests=args.requests, new_tokens=args.new_tokens,
                       prefill_chunk=args.prefill_chunk, layers=args.layers)
    return run(1, args.steps, max(3, args.warmup), "leone_b200", layers=args.layers, batch=args.batch,
               context=args.context, points=not args.no_points, shape=args.shape or "qwen3-8b")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="leone", description="leone_b200 command line")
    sub = ap.add_subparsers(dest="command")
    g = sub.add_parser("generate", help="generate -m <dir> -t <token ids> -n <tokens> [options]")
    g.add_argument("-m", "--model", required=True,
                   help="model folder (config.json + model.safetensors; with --random-weights config.json alone)")
    g.add_argument("-p", "--prompt", help="prompt text (refused: no tokenizer is built)")
    g.add_argument("-t", "--prompt-tokens", action="append",
                   help='prompt token ids: "1,2,3" or @file (u32le or .json); repeat for a batch')
    g.add_argument("-n", "--tokens", type=int, required=True, help="tokens to generate per prompt")
    g.add_argument("--temp", type=float, default=None, help="scale logits by 1/t (default: greedy)")
    g.add_argument("--seed", type=int, default=0, help="seed the sampler. Default: 0")

    class Stage(argparse.Action):
        """Truncation stages apply in the order their flags are given
        (crates/leone-cli/src/main.rs:1378-1430)."""

        def __call__(self, parser, namespace, value, option_string=None):
            stages = list(getattr(namespace, "truncations", None) or [])
            stages.append((self.dest, value))
            namespace.truncations = stages

    for flag, dest, kind, text in (
            ("--top-k", "top_k", int, "Keep the n highest-probability tokens"),
            ("--top-p", "top_p", float, "Keep the shortest prefix whose mass reaches p"),
            ("--min-p", "min_p", float, "Keep tokens above m times the highest"),
            ("--top-a", "top_a", float, "Keep tokens above a times the highest squared"),
            ("--tfs", "tfs", float, "Tail-free sampling on the second derivative"),
            ("--typical", "typical", float, "Locally typical sampling to mass p"),
            ("--epsilon", "epsilon", float, "Keep tokens with probability at least e"),
            ("--eta", "eta", float, "Entropy-relaxed probability floor"),
            ("--min-k", "min_k", float, "Keep the top k raw logits at the sharpest drop"),
            ("--top-n-sigma", "top_n_sigma", float, "Keep raw logits within n deviations of the peak")):
        g.add_argument(flag, dest=dest, type=kind, action=Stage, help=text)
    g.set_defaults(truncations=None)
    # crates/leone-cli/src/main.rs:850-857
    g.add_argument("--repeat-penalty", type=float, default=1.0, help="Apply sign-aware scaling to seen logits. 1.0 is off")
    g.add_argument("--presence-penalty", type=float, default=0.0, help="Subtract once from any seen token")
    g.add_argument("--frequency-penalty", type=float, default=0.0, help="Subtract once per earlier occurrence")
    g.add_argument("--penalty-window", type=int, default=64, help="Tokens considered. Zero disables. Default: 64")
    g.add_argument("--dry-multiplier", type=float, default=0.0, help="Enable the repeated-suffix penalty. 0.0 is off")
    g.add_argument("--dry-base", type=float, default=1.75, help="Growth per token of match. Default: 1.75")
    g.add_argument("--dry-allowed-length", type=int, default=2, help="Free match length. Default: 2")
    g.add_argument("--dry-window", type=int, default=64, help="Tokens of history searched. Default: 64")
    g.add_argument("--random-weights", action="store_true",
                   help="read no tensor file: -m names a folder with config.json (or that file) and the "
                        "weights are drawn from --weights-seed")
    g.add_argument("--weights-seed", type=int, default=None, help="seed of --random-weights. Default: --seed")
    g.add_argument("--eager-decode", action="store_true", help="disable decode graph replay")
    g.add_argument("--kv", choices=["q8", "f16", "f32", "bf16"], default=None,
                   help="KV cache storage; only the run dtype is available")
    g.add_argument("--debug-tokens", help="write generated token ids as JSON")
    g.add_argument("--debug-logits", help="write the top five logits for each token")
    g.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    g.add_argument("--eos", type=int, default=None, help="stop token id (default: the model's)")
    g.add_argument("--page-tokens", type=int, default=16)
    g.add_argument("--num-pages", type=int, default=None)
    g.add_argument("--prefill-chunk", type=int, default=2048)
    g.add_argument("--max-batch-tokens", type=int, default=2048)
    g.add_argument("--decode-quantum", type=int, default=1)
    d = sub.add_parser("doctor", help="doctor [-m <dir>] [--probe]")
    d.add_argument("-m", "--model")
    d.add_argument("--probe", action="store_true", help="load the weights and run one token")
    d.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    r = sub.add_parser("random-model", help="write a model folder with seeded random weights")
    r.add_argument("--config", required=True, help="a config.json to take the sizes from")
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--store-dtype", choices=["float32", "bfloat16"], default="bfloat16")
    sub.add_parser("replay", help="same options as bin/trace_run", add_help=False)
    b = sub.add_parser("bench", help="decode/prefill throughput of a Qwen3-8B-shaped model")
    b.add_argument("--steps", type=int, default=256)
    b.add_argument("--warmup", type=int, default=3)
    b.add_argument("--layers", type=int, default=None)
    b.add_argument("--batch", type=int, default=8)
    b.add_argument("--context", type=int, default=None, help="decode context (default: the shape's)")
    b.add_argument("--no-points", action="store_true")
    b.add_argument("--shape", choices=["qwen3-8b", "qwen3-1.7b", "qwen3-32b"], default=None)
    b.add_argument("--workload", choices=["decode", "serving"], default="decode",
                   help="decode: device-timed decode and prefill; serving: many requests through the scheduler")
    b.add_argument("--requests", type=int, default=64)
    b.add_argument("--new-tokens", type=int, default=128)
    b.add_argument("--prefill-chunk", type=int, default=1024)
    return ap


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "replay":
        return cmd_replay(None, argv[1:])
    ap = build_parser()
    args = ap.parse_args(argv)
    if args.command == "generate":
        return cmd_generate(args)
    if args.command == "doctor":
        return cmd_doctor(args)
    if args.command == "random-model":
        return cmd_random_model(args)
    if args.command == "bench":
        return cmd_bench(args)
    ap.print_help()
    return 2


if __name__ == "__main__":
    sys.exit(main())
