#!/usr/bin/env python3
"""Decode and prefill throughput of a Qwen3-8B-shaped model on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl leone_b200|reference]

Prints one JSON line.  ``--gpus N`` with N > 1 prints one line saying that this engine runs
on one GPU and exits with 2.  ``--impl reference`` prints why the reference cannot run here.
``--shape qwen3-32b | qwen3-1.7b``, ``--batch``, ``--context`` measure the other baseline
configurations; ``--workload serving`` runs many requests through the scheduler.
"""
import argparse
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256, help="decode steps timed (the baseline workload decodes 256)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="leone_b200", choices=["leone_b200", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=None, help="decode context (default: the shape's)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--shape", default=None, choices=["qwen3-8b", "qwen3-1.7b", "qwen3-32b"],
                    help="layer sizes (default: the headline Qwen3-8B shape; for --workload serving the 1.7B shape)")
    ap.add_argument("--workload", default="decode", choices=["decode", "serving"],
                    help="serving: many requests with mixed prompt lengths through the scheduler (its own JSON line)")
    ap.add_argument("--requests", type=int, default=64, help="serving: concurrent requests")
    args = ap.parse_args()
    if args.impl != "reference" and args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.workload == "serving" and args.impl != "reference":
        from leone_b200.benchmark import serving
        return serving(args.shape or "qwen3-1.7b", requests=args.requests, layers=args.layers)
    from leone_b200.benchmark import run
    return run(args.gpus, args.steps, max(args.warmup, 3), args.impl, layers=args.layers,
               batch=args.batch, context=args.context, points=not args.no_points, shape=args.shape or "qwen3-8b")


if __name__ == "__main__":
    sys.exit(main())
