"""Parity gates shared by the GPU tests.

FP32 results must satisfy |a - b| <= 1e-5 + 1e-3 * |b| against the matching-contract oracle. A dot product of
K random-sign terms can cancel to almost nothing, and there no FP32 summation order (the oracle's included)
is accurate to 1e-3 of the result, so an element also passes when it is within 8 * eps32 * sum|term| of the
oracle -- 40 times tighter than the reference's own kernel tolerance of 2e-5 * sum|term|
(native/synapse-kernels/tests/Features/CpuKernels/q8_0_tests.rs:116). Every element must in any case be
within that reference tolerance of the FP64 value.
"""
import numpy as np

EPS32 = float(np.finfo(np.float32).eps)


def assert_parity(got, want, exact, magnitude, label=""):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    difference = np.abs(got - want)
    gate = difference <= 1e-5 + 1e-3 * np.abs(want)
    reorder = difference <= 8 * EPS32 * magnitude
    bad = ~(gate | reorder)
    assert not bad.any(), (
        f"{label}: {int(bad.sum())} of {bad.size} outputs miss both gates; worst |a-b|={difference[bad].max():.3e}, "
        f"want={want[bad][np.argmax(difference[bad])]:.6e}")
    reference_form = np.abs(got - exact) <= 2e-5 * magnitude + 1e-12
    assert reference_form.all(), f"{label}: {int((~reference_form).sum())} outputs exceed 2e-5 * sum|term| of the FP64 value"
    return {"outside_rel_gate": int((~gate).sum()), "count": int(gate.size),
            "max_normalised": float(np.max(difference / np.maximum(magnitude, 1e-30)))}


def rows_in_parallel(function, ggml_type, weights, rows, columns, *operands, threads=None):
    """Runs an oracle product `function(ggml_type, weights, rows, columns, *operands)` over row chunks on all host
    threads (every output row is independent, so chunking changes no value) and joins the [tokens, rows] results.
    Functions that return (value, magnitude) pairs are joined element-wise."""
    import concurrent.futures
    import os

    threads = threads or os.cpu_count() or 1
    row_bytes = weights.size // rows
    chunk = max(1, -(-rows // (threads * 4)))
    spans = [(first, min(chunk, rows - first)) for first in range(0, rows, chunk)]

    def run(span):
        first, count = span
        return function(ggml_type, weights[first * row_bytes:(first + count) * row_bytes], count, columns, *operands)

    with concurrent.futures.ThreadPoolExecutor(max_workers=threads) as pool:
        parts = list(pool.map(run, spans))
    if isinstance(parts[0], tuple):
        return tuple(np.concatenate([p[i] for p in parts], axis=1) for i in range(len(parts[0])))
    return np.concatenate(parts, axis=1)
