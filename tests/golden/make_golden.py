"""Writes tests/golden/matvec_cases.npz: small seeded inputs with the CPU oracle's outputs.

The oracle (oracle/synapse_oracle.c) restates the reference's CPU kernels; it was pinned to the reference
tests' known-answer vectors by tests/test_oracle_pins.py before these vectors were produced. Re-run with
`python tests/golden/make_golden.py` from the repository root; the output is deterministic.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from synapse_b200 import synth  # noqa: E402

CASES = [  # name, type, rows, columns, tokens
    ("q8_0_a", synth.Q8_0, 37, 896, 1),
    ("q8_0_b", synth.Q8_0, 10, 224, 3),
    ("q4_k_a", synth.Q4_K, 24, 512, 3),
    ("q4_k_b", synth.Q4_K, 7, 1792, 1),
    ("q6_k_a", synth.Q6_K, 24, 512, 3),
    ("q6_k_b", synth.Q6_K, 5, 1280, 2),
]


def main():
    oracle.build()
    out = {}
    for index, (name, ggml_type, rows, columns, tokens) in enumerate(CASES):
        weights = synth.matrix(ggml_type, rows, columns, seed=1000 + index, name=name)
        x = synth.activations(tokens, columns, seed=2000 + index, name=name)
        codes, scales = oracle.quantize(x)
        out[f"{name}.meta"] = np.array([ggml_type, rows, columns, tokens], np.int64)
        out[f"{name}.weights"] = weights
        out[f"{name}.x"] = x
        out[f"{name}.codes"] = codes
        out[f"{name}.scales"] = scales
        out[f"{name}.y_xq8"] = oracle.kq_q8_matmul(ggml_type, weights, rows, columns, codes, scales)
        out[f"{name}.y_xf32"] = oracle.f32_matmul(ggml_type, weights, rows, columns, x)
        out[f"{name}.dots"] = oracle.int_dots(ggml_type, weights, rows, columns, codes)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "matvec_cases.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
