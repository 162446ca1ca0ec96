"""Oracle parity on the very shapes and kernel variants the benchmark reports.

The decode matrix-vector kernel picks its CTA shape from the matrix size: eight consumer warps with two rows each up to
96 MB, sixteen warps with one row each beyond that (the vocabulary projections), and a CTA walks its ring of weight
stages several times on the large matrices. The small shapes of test_matvec_gpu.py reach neither the sixteen-warp
variant nor a ring that wraps, so every benchmark shape is compared here with the quantised-activation oracle (O6 for
Q4_K / Q6_K, the reference's scalar kernel order O2 for Q8_0) at one and at eight tokens, with the exact integer
sub-block dots of a row slice beside it. Form follows native/synapse-kernels/tests/Features/CpuKernels/q8_0_tests.rs:110-166
(seeded inputs, FP64 evaluation, error against sum|term|).
"""
import numpy as np
import pytest

import synapse_b200 as sb
from synapse_b200 import synth
from parity import assert_parity, rows_in_parallel

pytestmark = pytest.mark.gpu

BENCH_SHAPES = [  # type, rows, columns
    (sb.Q4_K, 18944, 3584),    # ffn_gate / ffn_up of the 7B set: the roofline kernel of the benchmark
    (sb.Q4_K, 152064, 3584),   # vocabulary projection (sixteen-warp CTAs)
    (sb.Q6_K, 3584, 18944),    # ffn_down
    (sb.Q6_K, 152064, 3584),   # vocabulary projection as Q6_K
    (sb.Q8_0, 151936, 896),    # vocabulary projection of the 0.5B model
    (sb.Q8_0, 18944, 3584),
    (sb.Q4_K, 28672, 8192),    # the row-sharded sweep's matrices
    (sb.Q4_K, 8192, 28672),
]


@pytest.mark.parametrize("ggml_type,rows,columns", BENCH_SHAPES)
def test_benchmark_shapes_against_the_oracle(oracle, ggml_type, rows, columns):
    weights = synth.matrix(ggml_type, rows, columns, seed=301)
    x = synth.activations(8, columns, seed=302)
    codes, scales = oracle.quantize(x)
    want = rows_in_parallel(oracle.kq_q8_matmul, ggml_type, weights, rows, columns, codes, scales)
    exact, magnitude = rows_in_parallel(oracle.kq_q8_exact, ggml_type, weights, rows, columns, codes, scales)
    counts = {}
    with sb.QuantizedMatrix(weights, ggml_type, rows, columns) as matrix:
        one = matrix.matvec(x[:1], sb.MODE_XQ8)
        counts[1] = assert_parity(one, want[:1], exact[:1], magnitude[:1], "one token")
        eight = matrix.matvec(x, sb.MODE_XQ8)
        counts[8] = assert_parity(eight, want, exact, magnitude, "eight tokens")
        assert eight[:1].tobytes() == one.tobytes(), "a token's result depends on how many tokens share the launch"
        # exact integer sub-block dots of a row slice in the middle of the matrix and of its last rows
        row_bytes = weights.size // rows
        for first in (rows // 2, rows - 48):
            got = matrix.block_dots(codes[:1], row_start=first, row_count=48)
            assert np.array_equal(got, oracle.int_dots(ggml_type, weights[first * row_bytes:(first + 48) * row_bytes], 48, columns, codes[:1]))
        assert sb.library().device_faults() == 0
    print(f"type {ggml_type} {rows}x{columns}: outputs outside the relative gate (passed on the summation-order gate) "
          f"{counts[1]['outside_rel_gate']}/{counts[1]['count']} at one token, {counts[8]['outside_rel_gate']}/{counts[8]['count']} at eight")


@pytest.mark.parametrize("ggml_type,rows,columns", [(sb.Q4_K, 18944, 3584), (sb.Q6_K, 3584, 18944), (sb.Q8_0, 4864, 896)])
@pytest.mark.parametrize("tokens", [3, 4])
def test_fp32_activation_contract_at_three_and_four_tokens(oracle, ggml_type, rows, columns, tokens):
    """The `reference` backend's contract (FP32 activations, the only one the reference defines for K-quants) on the token
    counts that still run on the matrix-vector kernels (step/projection.rs:51-72: prompt runs of up to four tokens)."""
    weights = synth.matrix(ggml_type, rows, columns, seed=311)
    x = synth.activations(tokens, columns, seed=312)
    with sb.QuantizedMatrix(weights, ggml_type, rows, columns) as matrix:
        y = matrix.matvec(x, sb.MODE_XF32)
    want = oracle.f32_matmul_threads(ggml_type, weights, rows, columns, x, 16)
    exact, magnitude = rows_in_parallel(oracle.f32_exact, ggml_type, weights, rows, columns, x)
    assert_parity(y, want, exact, magnitude, f"xf32 {tokens} tokens")
