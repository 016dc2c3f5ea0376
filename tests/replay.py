"""Building replay traces and checking replayed logits against the plain implementation."""
import json
import os
import random
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def random_tokens(vocab, n, seed):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


# -- traces: lists of {"step", "entries", "end"} -----------------------------------------------
def trace_whole(requests):
    """Each request alone and whole, all positions wanted."""
    steps = []
    for i, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def trace_decode_tail(requests, tail=32):
    """Most of a request in one step, the last ``tail`` tokens one by one."""
    steps, n = [], 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}],
                      "end": []})
        n += 1
        for p in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
            n += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(requests, sizes=(7, 2, 5, 3, 2, 11, 1, 2, 16, 2, 33)):
    steps, n = [], 0
    for rid, toks in requests.items():
        pos, k = 0, 0
        while pos < len(toks):
            s = min(sizes[k % len(sizes)], len(toks) - pos)
            k += 1
            last = pos + s == len(toks)
            steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[pos:pos + s],
                                                   "want": list(range(s))}], "end": [rid] if last else []})
            pos += s
            n += 1
    return steps


def trace_mixed(requests, seed=0, max_live=4, decode_from=0.6):
    """Up to ``max_live`` requests at a time; each is first fed in portions of changing size,
    then token by token, while others are at other stages; finished ones end and their pages
    go to the next arrivals.  Some requests sit out some steps."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live = {}
    steps, n = [], 0
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.7):
            rid, toks = waiting.pop(0)
            live[rid] = dict(toks=toks, pos=0, switch=max(1, int(len(toks) * decode_from)))
        entries, end = [], []
        for rid, st in list(live.items()):
            if len(live) > 1 and rng.random() < 0.2:
                continue                                  # left out of this step
            left = len(st["toks"]) - st["pos"]
            if st["pos"] >= st["switch"]:
                s = 1
            else:
                s = min(rng.choice([2, 3, 5, 8, 13, 2]), st["switch"] - st["pos"], left)
            toks = st["toks"][st["pos"]:st["pos"] + s]
            entries.append({"id": rid, "tokens": toks, "want": list(range(s))})
            st["pos"] += s
            if st["pos"] == len(st["toks"]):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append({"step": n, "entries": entries, "end": end})
            n += 1
    return steps


def max_live_tokens(steps, unit=64):
    """Most tokens held by live requests at any time, each rounded up to ``unit``."""
    held, peak = {}, 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-v // unit) * unit for v in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


# -- running -------------------------------------------------------------------------------------
def run_trace_program(folder, dtype, steps, out_dir, max_tokens, extra=()):
    """Drive bin/trace_run as a user would: a child process, steps over stdin."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens), *extra]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for st in steps:
            proc.stdin.write(json.dumps(st) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {st['step']}", f"expected 'done {st['step']}', got {line!r}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    return read_outputs(steps, out_dir)


def run_trace_engine(engine, steps):
    """The same trace through an engine in this process."""
    outputs = {}
    for st in steps:
        entries = [(e["id"], e["tokens"], e["want"]) for e in st["entries"]]
        logits = engine.step(entries)
        if logits is not None:
            outputs[st["step"]] = logits.detach().float().cpu().numpy()
        for rid in st["end"]:
            engine.close(rid)
        engine.cache.check_invariants()
    return outputs


def read_outputs(steps, out_dir):
    outputs = {}
    for st in steps:
        path = os.path.join(out_dir, f"{st['step']}.f32")
        if any(e["want"] for e in st["entries"]):
            outputs[st["step"]] = np.fromfile(path, dtype="<f4")
    return outputs


def compare(steps, outputs, plain, requests, rtol, atol_scale, what):
    """Every written row against the plain model's logits at (request, position)."""
    pos = {rid: 0 for rid in requests}
    worst = 0.0
    for st in steps:
        rows = []
        for e in st["entries"]:
            full = plain.logits(requests[e["id"]])
            for w in e["want"]:
                rows.append(full[pos[e["id"]] + w])
            pos[e["id"]] += len(e["tokens"])
        if not rows:
            continue
        want = torch.stack(rows).double().numpy()
        got = np.asarray(outputs[st["step"]], dtype=np.float64).reshape(want.shape)
        scale = np.abs(want).max()
        err = np.abs(got - want)
        bound = atol_scale * scale + rtol * np.abs(want)
        if (err > bound).any():
            r, c = np.unravel_index(np.argmax(err - bound), err.shape)
            raise AssertionError(
                f"{what}: step {st['step']} row {r} (entries {[(e['id'], len(e['tokens'])) for e in st['entries']]}) "
                f"col {c}: got {got[r, c]:.6g}, want {want[r, c]:.6g}, err {err[r, c]:.3g} > {bound[r, c]:.3g}")
        worst = max(worst, float((err / scale).max()))
    return worst


# -- tolerances ------------------------------------------------------------------------------------
# fp32: only summation order differs from the float64 plain implementation.
FP32_TOL = (2e-5, 2e-5)
# bfloat16: weights are the same bf16 values on both sides; the engine rounds activations to
# bf16 (8 significant bits, relative step 2^-8) at about six places per layer.  This blanket
# bound only catches gross faults; `check_worst` holds each case to what a clean run showed.
BF16_TOL = (3e-2, 3e-2)


def tolerance(dtype):
    """(rtol, atol_scale) for :func:`compare`."""
    return FP32_TOL if dtype == "float32" else BF16_TOL


def check_worst(key, worst):
    """Hold a case to twice the worst error (relative to the largest logit) that a clean run of
    it showed (``tests/recorded_worst.py``), so that a defect small enough to hide under the
    blanket tolerance (a misplaced key among forty, a dropped split) still fails."""
    from tests.recorded_worst import RECORDED
    print(f"worst {key!r}: {worst:.4e}")
    log = os.environ.get("LEONE_WORST_LOG")         # a clean run's figures, to put into recorded_worst.py
    if log:
        with open(log, "a") as fh:
            fh.write(f"    {key!r}: {worst:.3e},\n")
    if key in RECORDED:
        assert worst <= 2.0 * RECORDED[key], f"{key}: worst error {worst:.3e} is more than twice the recorded {RECORDED[key]:.3e}"
