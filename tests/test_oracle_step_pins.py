"""Pins of the decode-step pieces of the oracle (O8) against the reference's own operator vectors that need no model file.

The whole-step tests of the reference run on the downloaded Qwen2.5 GGUF (OptimizedQwen2Tests.cs) and cannot be replayed
here; its operator tests can: RMSNorm and SiLU against an FP64 formula, the stable softmax, the NeoX rotation at known
coordinates, and the rotary table formula.
"""
import math

import numpy as np

from synapse_b200 import decoder as dec


def within(actual, expected, absolute=1e-5, relative=1e-4):
    """NumericalPolicy.Fp32 (GraphExecution/Reference/NumericalPolicy.cs:9,18-21)."""
    return abs(float(actual) - expected) <= absolute + relative * abs(expected)


def test_rms_norm_and_silu_match_the_fp64_formula(oracle):
    """ReferenceOperatorsTests.cs:105-125."""
    x = np.array([0.25, -2.0, 3.5, 0.0], np.float32)
    weights = np.array([1.0, 0.5, -1.25, 2.0], np.float32)
    normalized = oracle.rms_norm(x, weights, 1e-5)
    activated = oracle.swiglu(x, np.ones(4, np.float32))
    scale = 1.0 / math.sqrt(sum(float(v) * float(v) for v in x) / 4 + float(np.float32(1e-5)))
    for i in range(4):
        assert within(normalized[i], float(x[i]) * scale * float(weights[i]))
        assert within(activated[i], float(x[i]) / (1 + math.exp(-float(x[i]))))


def test_softmax_is_stable(oracle):
    """ReferenceOperatorsTests.cs:127-141."""
    out = oracle.softmax(np.array([1000.0, 1001.0, -1000.0], np.float32))
    assert within(out[0], 1 / (1 + math.e)) and within(out[1], math.e / (1 + math.e))
    assert out[2] == 0.0 and 0.99999 <= float(out.sum()) <= 1.00001


def test_neox_rotation_at_known_coordinates(oracle):
    """ReferenceOperatorsTests.cs:143-164: head of four values, position 1, theta 10000; first element cos 1 - 3 sin 1 and
    the rotation keeps the norm."""
    cosines, sines = dec.rope_tables(4, 2, theta=10_000.0)
    x = np.array([1.0, 2.0, 3.0, 4.0], np.float32)
    rotated = oracle.rotate_neox(x, cosines[1], sines[1])
    assert within(rotated[0], math.cos(1) - 3 * math.sin(1))
    assert within(float((rotated.astype(np.float64) ** 2).sum()), 30.0)


def test_rotary_tables_follow_the_unscaled_formula():
    """RopeFrequenciesTests.cs:13-34: angle = position / theta^(2i/d) in FP32, then cos and sin of that FP32 angle."""
    head_dim, theta = 128, 1_000_000.0
    positions = [0, 1, 17, 4095, 32767]
    cosines, sines = dec.rope_tables(head_dim, max(positions) + 1, theta)
    for position in positions:
        for index in range(head_dim // 2):
            angle = np.float32(position) / np.float32(np.power(np.float32(theta), np.float32(2.0 * index / head_dim)))
            # one FP32 step of slack: the C# test compares MathF with MathF, numpy and libm may round the last bit differently
            assert abs(float(cosines[position, index]) - math.cos(float(angle))) <= 2 ** -23
            assert abs(float(sines[position, index]) - math.sin(float(angle))) <= 2 ** -23
