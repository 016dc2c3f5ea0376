#!/usr/bin/env python3
"""Writes tests/golden/attention_oracle.json from the reference's own attention oracle.

The only model code of the reference that can run here is its pure-Python float64 attention
oracle, research/prefix_attention/common_oracle.py (``make_inputs`` :139-153, ``oracle_values``
:156-192): one query row per request over ``tokens`` keys with grouped heads, which is a decode
step.  This script runs it on small cases and stores inputs (queries as floats, keys and values as float16 bit patterns) and outputs; the
tests compare the plain implementation and the GPU kernels with the stored outputs.

    python tests/golden/make_attention_golden.py [path to research/prefix_attention]
"""
import json
import os
import sys

CASES = [
    dict(tokens=21, query_rows=2, query_heads=4, kv_heads=2, head_dim=16, seed=11, shared_prefix=False),
    dict(tokens=33, query_rows=1, query_heads=6, kv_heads=3, head_dim=32, seed=12, shared_prefix=False),
    dict(tokens=19, query_rows=3, query_heads=5, kv_heads=1, head_dim=48, seed=13, shared_prefix=True),
]


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_attention_golden.py <the reference checkout's research/prefix_attention folder>")
    ref = sys.argv[1]
    sys.path.insert(0, ref)
    import common_oracle as oracle
    out = []
    for case in CASES:
        full = {field: case.get(field, 0) for field in oracle.CASE_FIELDS}
        full.update(case)
        queries, keys, values = oracle.make_inputs(full)
        outputs = oracle.oracle_values(full, queries, keys, values)
        out.append({"case": case, "queries": [float(q) for q in queries],
                    "keys_f16_bits": list(keys), "values_f16_bits": list(values),
                    "outputs": outputs})
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "attention_oracle.json")
    with open(path, "w") as fh:
        json.dump(out, fh)
    print(f"wrote {path} ({os.path.getsize(path)} bytes)")


if __name__ == "__main__":
    main()
